// Permutation of (token, k) pairs into per-expert row segments padded to 128-row tiles.
//
// Replaces the reference's `exclusive_scan_kernel`, `dispatch_place_kernel`,
// `fused_dispatch_single_block_kernel` (solution/python/moe_fused.cu:888-1051) and
// `fused_gather_hidden_scales_kernel` (moe_fused.cu:736-768).  Unlike the reference's
// atomic cursor, placement is stable by token id, so the packed order (and every later
// intermediate) is identical from run to run.
//
//   scan   : per-expert totals from the per-chunk histogram, 128-padded segment starts,
//            the M-tile -> expert table, per-chunk bases, padding rows marked -1
//   place  : one block per 256-token chunk; a warp walks an expert's tokens in order
//   place  also records, per (token, k), the packed row it went to (-1: expert not local)
//   gather : one warp per packed row copies the e4m3 row and its 1x128 scales
#include "common.cuh"
#include "kernels.cuh"

namespace b200moe {

namespace {

__global__ void __launch_bounds__(256)
scan_kernel(Workspace ws, int e_local, int n_chunks, int pad_rows) {
  __shared__ int s_scan[256];
  const int e = threadIdx.x;
  chain_wait();
  chain_release();
  int* chunk_counts = ws.at<int>(ws.L.chunk_counts);
  int* chunk_base = ws.at<int>(ws.L.chunk_base);
  int total = 0;
  if (e < e_local) {
    // eight independent loads in flight per round instead of one load per chunk in a chain
    for (int c0 = 0; c0 < n_chunks; c0 += 8) {
      int cnt[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) cnt[j] = c0 + j < n_chunks ? chunk_counts[(c0 + j) * e_local + e] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (c0 + j < n_chunks) chunk_base[(c0 + j) * e_local + e] = total;
        total += cnt[j];
      }
    }
  }
  int padded = (total + pad_rows - 1) / pad_rows * pad_rows;   // whole M tiles
  s_scan[e] = padded;
  __syncthreads();
  // inclusive Hillis-Steele scan over 256 entries
  for (int off = 1; off < 256; off <<= 1) {
    int v = e >= off ? s_scan[e - off] : 0;
    __syncthreads();
    s_scan[e] += v;
    __syncthreads();
  }
  int row0 = s_scan[e] - padded;
  __syncthreads();
  const int padded_total_all = s_scan[255];
  int* expert_row0 = ws.at<int>(ws.L.expert_row0);
  int* expert_count = ws.at<int>(ws.L.expert_count);
  int* tile_expert = ws.at<int>(ws.L.tile_expert);
  int* row_token = ws.at<int>(ws.L.row_token);
  if (e < e_local) {
    expert_row0[e] = row0;
    expert_count[e] = total;
    for (int t = row0 / kTileM; t < (row0 + padded) / kTileM; ++t) tile_expert[t] = e;
    for (int r = row0 + total; r < row0 + padded; ++r) row_token[r] = -1;
  }
  // totals: rows with a local expert (for reporting) and padded rows
  __shared__ int s_rows;
  if (e == 0) s_rows = 0;
  __syncthreads();
  if (e < e_local && total) atomicAdd(&s_rows, total);
  __syncthreads();
  if (e == 0) {
    int padded_total = padded_total_all;
    expert_row0[e_local] = padded_total;
    int* meta = ws.at<int>(ws.L.meta);
    meta[0] = padded_total / kTileM;
    meta[1] = padded_total;
    meta[2] = s_rows;
    meta[3] = pad_rows;
  }
}

__global__ void __launch_bounds__(1024)
place_kernel(Workspace ws, const int32_t* __restrict__ ids, long long ids_stride,
             const float* __restrict__ w, long long w_stride, int T, int local_off, int e_local,
             const int* __restrict__ n_rows_dev) {
  __shared__ int s_ids[kTopK][kChunkTokens];   // [k][token]: conflict-free when lanes walk tokens
  chain_wait();
  chain_release();
  if (n_rows_dev) T = min(T, *n_rows_dev);   // T was the capacity; rows past the count hold nothing
  const int c = blockIdx.x;
  const int t0 = c * kChunkTokens;
  for (int i = threadIdx.x; i < kChunkTokens * kTopK; i += blockDim.x) {
    int tl = i / kTopK, k = i % kTopK;
    int t = t0 + tl;
    s_ids[k][tl] = t < T ? ids[(size_t)t * ids_stride + k] : -1;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int* chunk_counts = ws.at<int>(ws.L.chunk_counts);
  const int* chunk_base = ws.at<int>(ws.L.chunk_base);
  const int* expert_row0 = ws.at<int>(ws.L.expert_row0);
  int* row_token = ws.at<int>(ws.L.row_token);
  float* row_weight = ws.at<float>(ws.L.row_weight);
  int* tok_rows = ws.at<int>(ws.L.tok_rows);
  // every (token, k) of the chunk starts as "not local"; local ones are overwritten below
  for (int i = threadIdx.x; i < kChunkTokens * kTopK; i += blockDim.x) {
    int t = t0 + i / kTopK;
    if (t < T) tok_rows[(size_t)t * kTopK + i % kTopK] = -1;
  }
  __syncthreads();
  for (int e = warp; e < e_local; e += nwarps) {
    if (chunk_counts[c * e_local + e] == 0) continue;
    int pos = expert_row0[e] + chunk_base[c * e_local + e];
    const int want = e + local_off;
    for (int sub = 0; sub < kChunkTokens / 32; ++sub) {
      int tl = sub * 32 + lane;
      int kf = -1;
#pragma unroll
      for (int k = 0; k < kTopK; ++k)
        if (s_ids[k][tl] == want) kf = k;
      uint32_t hit = __ballot_sync(0xffffffffu, kf >= 0);
      if (kf >= 0) {
        int r = pos + __popc(hit & ((1u << lane) - 1u));
        int t = t0 + tl;
        row_token[r] = t;
        row_weight[r] = w[(size_t)t * w_stride + kf];
        tok_rows[(size_t)t * kTopK + kf] = r;
      }
      pos += __popc(hit);
    }
  }
}

__global__ void __launch_bounds__(256)
gather_kernel(Workspace ws, const uint8_t* __restrict__ hidden, long long hidden_row_stride,
              const float* __restrict__ hscale, long long sstride_t, long long sstride_kb, int hidden_dim,
              RowSegments segs, __nv_bfloat16* __restrict__ out, long long out_stride, int T,
              const RowSegments* __restrict__ segs_dev, const int* __restrict__ n_rows_dev) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  chain_wait();
  chain_release();
  if (segs_dev) segs = *segs_dev;            // the table was built on the device (see launch_ep_segments_pull)
  if (n_rows_dev) T = min(T, *n_rows_dev);
  // The layer's output starts as zeros: GEMM2's epilogue adds every packed row into its token's row, and a
  // token that no local expert took stays exactly 0.  Zeroed here, by all blocks, instead of by a memset
  // of its own (one launch boundary less; this kernel runs before the GEMMs in every call).
  {
    const int vec_per_row = hidden_dim / 8;   // 8 bf16 = 16 bytes
    const long long total = (long long)T * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const long long t = i / vec_per_row;
      reinterpret_cast<uint4*>(out + t * out_stride)[i - t * vec_per_row] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  const int rows = ws.at<int>(ws.L.meta)[1];
  const int* row_token = ws.at<int>(ws.L.row_token);
  uint8_t* a_packed = ws.at<uint8_t>(ws.L.a_packed);
  float* a_scale = ws.at<float>(ws.L.a_scale);
  unsigned* row_amax = ws.at<unsigned>(ws.L.row_amax);
  const int m_cap = ws.L.m_cap;
  const int vecs = hidden_dim / 16;
  const int kblocks = hidden_dim / kBlockK;
  for (int m = blockIdx.x * warps_per_block + (threadIdx.x >> 5); m < rows; m += gridDim.x * warps_per_block) {
    int t = row_token[m];
    if (t < 0) continue;
    if (lane == 0) row_amax[m] = 0u;   // GEMM1's epilogue takes the running maximum with atomicMax
    uint4* dst = reinterpret_cast<uint4*>(a_packed + (size_t)m * hidden_dim);
    if (segs.n > 0) {
      // the row is a send row of some rank of the group (payload, then its scales), read where it was packed:
      // plain loads from this GPU's or a peer's memory, so the dispatch and the gather are one pass
      const uint8_t* row = segs.row(t);
      const uint4* src = reinterpret_cast<const uint4*>(row);
      for (int v = lane; v < vecs; v += 32) dst[v] = src[v];
      const float* sc = reinterpret_cast<const float*>(row + hidden_dim);
      for (int kb = lane; kb < kblocks; kb += 32) a_scale[(size_t)kb * m_cap + m] = sc[kb];
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * hidden_row_stride);
    for (int v = lane; v < vecs; v += 32) dst[v] = __ldg(src + v);
    for (int kb = lane; kb < kblocks; kb += 32)
      a_scale[(size_t)kb * m_cap + m] = hscale[(size_t)t * sstride_t + (size_t)kb * sstride_kb];
  }
}

}  // namespace

cudaError_t launch_permute(const Workspace& ws, const int32_t* ids, long long ids_stride, const float* w,
                           long long w_stride, const uint8_t* hidden, long long hidden_row_stride,
                           const float* hscale, long long sstride_t, long long sstride_kb, int T, int e_local,
                           int local_off, int hidden_dim, int pad_rows, int num_sms, cudaStream_t stream,
                           bool placed, const RowSegments* segs, void* out_bf16, long long out_row_stride,
                           const RowSegments* segs_dev, const int* n_rows_dev) {
  const int n_chunks = (T + kChunkTokens - 1) / kChunkTokens;
  cudaError_t err = cudaSuccess;
  if (!placed) {
    err = launch_chained(scan_kernel, dim3(1), dim3(256), 0, stream, ws, e_local, n_chunks, pad_rows);
    if (err != cudaSuccess) return err;
  }
  if (n_chunks > 0) {
    if (!placed) {
      // 32 warps per chunk: a call has few chunks, and a warp's walk over its experts is a chain of small loads
      err = launch_chained(place_kernel, dim3(n_chunks), dim3(1024), 0, stream, ws, ids, ids_stride, w, w_stride, T,
                           local_off, e_local, n_rows_dev);
      if (err != cudaSuccess) return err;
    }
    // padded rows of this call: at most 8 T pairs plus 127 rows of padding per expert that has any
    const long long pairs = (long long)T * kTopK;
    long long cap_rows = pairs + (long long)(kTileM - 1) * (pairs < e_local ? pairs : e_local);
    if (cap_rows > ws.L.m_cap) cap_rows = ws.L.m_cap;
    int blocks = (int)((cap_rows + 7) / 8);
    int cap = num_sms * 8;
    if (blocks > cap) blocks = cap;
    RowSegments none;
    none.n = 0;
    err = launch_chained(gather_kernel, dim3(blocks), dim3(256), 0, stream, ws, hidden, hidden_row_stride, hscale,
                         sstride_t, sstride_kb, hidden_dim, segs ? *segs : none,
                         reinterpret_cast<__nv_bfloat16*>(out_bf16), out_row_stride, T, segs_dev, n_rows_dev);
  }
  return err;
}

}  // namespace b200moe
