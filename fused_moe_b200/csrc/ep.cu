// Expert-parallel helpers: build per-destination send rows, and sum the partial outputs
// that come back.  The reference has no multi-GPU path (it only consumes
// `local_expert_offset`, solution/python/kernel.py:591); rows travel between these two
// kernels by NCCL all-to-all into the receiving GPU's own memory, or - when the ranks' send and
// partial buffers are mapped into each other's address space - are read in place by the
// gather (permute.cu) and by ep_combine_peers_kernel with plain loads: no multicast anywhere.
//
// A token is sent at most once to each rank that owns one of its 8 experts; the send row
// carries the e4m3 payload, its 1x128 scales and all 8 (id, weight) pairs, so the receiver
// runs the ordinary local pipeline on the rows it gets.
#include "common.cuh"
#include "kernels.cuh"

namespace b200moe {

namespace {

constexpr int kMaxWorld = 8;

// One block; threads walk tokens in order so that slots are ascending in token id.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int32_t* __restrict__ ids, int T, int world, int32_t* __restrict__ dest_counts,
               int32_t* __restrict__ send_slot) {
  __shared__ int s_warp[32][kMaxWorld];
  __shared__ int s_base[kMaxWorld];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int experts_per_rank = kNumExperts / world;
  if (threadIdx.x < kMaxWorld) s_base[threadIdx.x] = 0;
  __syncthreads();
  for (int t0 = 0; t0 < T; t0 += blockDim.x) {
    const int t = t0 + threadIdx.x;
    uint32_t mask = 0;
    if (t < T) {
#pragma unroll
      for (int k = 0; k < kTopK; ++k) {
        int id = ids[(size_t)t * kTopK + k];
        if (id >= 0 && id < kNumExperts) mask |= 1u << (id / experts_per_rank);
      }
    }
    int my_rank_in_warp[kMaxWorld];
#pragma unroll
    for (int d = 0; d < kMaxWorld; ++d) {
      uint32_t b = __ballot_sync(0xffffffffu, (mask >> d) & 1u);
      my_rank_in_warp[d] = __popc(b & ((1u << lane) - 1u));
      if (lane == 0) s_warp[warp][d] = __popc(b);
    }
    __syncthreads();
    // exclusive scan over the 32 warps, one destination per thread
    if (threadIdx.x < kMaxWorld) {
      int run = s_base[threadIdx.x];
      for (int wv = 0; wv < 32; ++wv) {
        int c = s_warp[wv][threadIdx.x];
        s_warp[wv][threadIdx.x] = run;
        run += c;
      }
      s_base[threadIdx.x] = run;
    }
    __syncthreads();
    if (t < T) {
#pragma unroll
      for (int d = 0; d < kMaxWorld; ++d) {
        if (d < world)
          send_slot[(size_t)t * world + d] = ((mask >> d) & 1u) ? s_warp[warp][d] + my_rank_in_warp[d] : -1;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x < world) dest_counts[threadIdx.x] = s_base[threadIdx.x];
}

__global__ void __launch_bounds__(256)
ep_copy_kernel(const int32_t* __restrict__ ids, const float* __restrict__ w, const uint8_t* __restrict__ hidden,
               long long hidden_row_stride, const float* __restrict__ hscale, long long sstride_t,
               long long sstride_kb, int T, int hidden_dim, int world, const int32_t* __restrict__ send_slot,
               const int32_t* __restrict__ dest_counts, uint8_t* __restrict__ send_rows) {
  int seg_base[kMaxWorld];   // segments are compact: destination d starts after all rows of d' < d
  {
    int run = 0;
#pragma unroll
    for (int d = 0; d < kMaxWorld; ++d) {
      seg_base[d] = run;
      if (d < world) run += dest_counts[d];
    }
  }
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int kblocks = hidden_dim / kBlockK;
  const size_t row_bytes = (size_t)hidden_dim + 4 * (size_t)kblocks + 64;
  const long long n = (long long)T * world;
  for (long long i = blockIdx.x * (long long)wpb + (threadIdx.x >> 5); i < n; i += (long long)gridDim.x * wpb) {
    const int t = (int)(i / world), d = (int)(i % world);
    const int slot = send_slot[i];
    if (slot < 0) continue;
    int base = 0;
#pragma unroll
    for (int dd = 0; dd < kMaxWorld; ++dd)
      if (dd == d) base = seg_base[dd];
    uint8_t* dst = send_rows + ((size_t)base + slot) * row_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * hidden_row_stride);
    for (int v = lane; v < hidden_dim / 16; v += 32) reinterpret_cast<uint4*>(dst)[v] = __ldg(src + v);
    float* sdst = reinterpret_cast<float*>(dst + hidden_dim);
    for (int kb = lane; kb < kblocks; kb += 32) sdst[kb] = hscale[(size_t)t * sstride_t + (size_t)kb * sstride_kb];
    if (lane < kTopK) {
      reinterpret_cast<int32_t*>(dst + hidden_dim + 4 * kblocks)[lane] = ids[(size_t)t * kTopK + lane];
      reinterpret_cast<float*>(dst + hidden_dim + 4 * kblocks + 32)[lane] = w[(size_t)t * kTopK + lane];
    }
  }
}

__global__ void __launch_bounds__(256)
ep_combine_kernel(const __nv_bfloat16* __restrict__ returned, const int32_t* __restrict__ send_slot,
                  const int32_t* __restrict__ dest_counts, int T, int hidden_dim, int world,
                  __nv_bfloat16* __restrict__ out) {
  int seg_base[kMaxWorld];
  {
    int run = 0;
#pragma unroll
    for (int d = 0; d < kMaxWorld; ++d) {
      seg_base[d] = run;
      if (d < world) run += dest_counts[d];
    }
  }
  const int vec_per_row = hidden_dim / 8;   // 8 bf16 = 16 bytes
  const long long n = (long long)T * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec_per_row), v = (int)(i % vec_per_row);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int d = 0; d < kMaxWorld; ++d) {
      if (d >= world) break;
      const int slot = send_slot[(size_t)t * world + d];
      if (slot < 0) continue;
      const uint4 raw = reinterpret_cast<const uint4*>(returned + ((size_t)seg_base[d] + slot) * hidden_dim)[v];
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(p2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 pk;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<uint4*>(out + (size_t)t * hidden_dim)[v] = pk;
  }
}

// Builds the segment table of this step from the (count, offset) pairs the sources sent (one thread).
__global__ void ep_segments_kernel(PeerBases send_base, const int32_t* __restrict__ from_peers, int n,
                                   long long row_bytes, int cap_rows, RowSegments* __restrict__ segs_out,
                                   int* __restrict__ n_rows_out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  RowSegments sg;
  sg.n = n;
  sg.row_bytes = row_bytes;
  int run = 0;
  for (int s = 0; s < 8; ++s) {
    int cnt = 0, off = 0;
    if (s < n) {
      cnt = from_peers[3 * s];
      off = from_peers[3 * s + 1];
      if (cnt < 0) cnt = 0;
      if (cnt > cap_rows - run) cnt = cap_rows - run;   // never past the capacity the workspace was sized for
    }
    sg.start[s] = run;
    sg.base[s] = s < n ? send_base.base[s] + (size_t)off * row_bytes : nullptr;
    run += cnt;
  }
  sg.start[8] = run;
  for (int s = n; s < 8; ++s) sg.start[s] = run;
  *segs_out = sg;
  *n_rows_out = run;
}

// ids + weights of every send row addressed to this rank, read where the sender packed them
__global__ void __launch_bounds__(256)
ep_pull_ids_kernel(const RowSegments* __restrict__ segs_dev, const int* __restrict__ n_rows_dev, int hidden_dim,
                   int32_t* __restrict__ ids_out, float* __restrict__ w_out) {
  const RowSegments segs = *segs_dev;
  const int rows = *n_rows_dev;
  const int trailer = hidden_dim + 4 * (hidden_dim / kBlockK);   // byte offset of ids[8] | weights[8]
  const long long n = (long long)rows * 16;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i >> 4), j = (int)(i & 15);
    const uint32_t v = reinterpret_cast<const uint32_t*>(segs.row(r) + trailer)[j];
    if (j < 8) ids_out[(size_t)r * 8 + j] = (int32_t)v;
    else w_out[(size_t)r * 8 + (j - 8)] = __uint_as_float(v);
  }
}

// ep_combine_kernel with the return exchange folded in: each partial row is read from the
// memory of the rank that produced it (plain loads over NVLink for a peer).
__global__ void __launch_bounds__(256)
ep_combine_peers_kernel(PeerPartials peers, const int32_t* __restrict__ row_start,
                        const int32_t* __restrict__ send_slot, int T, int hidden_dim, int world,
                        __nv_bfloat16* __restrict__ out) {
  int start[kMaxWorld];
#pragma unroll
  for (int d = 0; d < kMaxWorld; ++d) start[d] = d < world ? row_start[d] : 0;
  const int vec_per_row = hidden_dim / 8;   // 8 bf16 = 16 bytes
  const long long n = (long long)T * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec_per_row), v = (int)(i % vec_per_row);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int d = 0; d < kMaxWorld; ++d) {
      if (d >= world) break;
      const int slot = send_slot[(size_t)t * world + d];
      if (slot < 0) continue;
      const __nv_bfloat16* rows = reinterpret_cast<const __nv_bfloat16*>(peers.partial[d]);
      const uint4 raw = reinterpret_cast<const uint4*>(rows + ((size_t)start[d] + slot) * hidden_dim)[v];
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(p2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 pk;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<uint4*>(out + (size_t)t * hidden_dim)[v] = pk;
  }
}

}  // namespace

cudaError_t launch_ep_segments_pull(const PeerBases& send_base, const int32_t* from_peers, int n, long long row_bytes,
                                    int cap_rows, int hidden_dim, RowSegments* segs_out, int* n_rows_out,
                                    int32_t* ids_out, float* w_out, int num_sms, cudaStream_t stream) {
  ep_segments_kernel<<<1, 32, 0, stream>>>(send_base, from_peers, n, row_bytes, cap_rows, segs_out, n_rows_out);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess || cap_rows <= 0) return err;
  long long work = (long long)cap_rows * 16;
  int blocks = (int)((work + 255) / 256);
  int cap = num_sms * 8;
  if (blocks > cap) blocks = cap;
  ep_pull_ids_kernel<<<blocks, 256, 0, stream>>>(segs_out, n_rows_out, hidden_dim, ids_out, w_out);
  return cudaGetLastError();
}

cudaError_t launch_ep_combine_peers(const PeerPartials& peers, const int32_t* row_start, const int32_t* send_slot,
                                    int T, int hidden_dim, int world, void* out_bf16, int num_sms,
                                    cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  long long n = (long long)T * (hidden_dim / 8);
  int blocks = (int)((n + 255) / 256);
  int cap = num_sms * 16;
  if (blocks > cap) blocks = cap;
  ep_combine_peers_kernel<<<blocks, 256, 0, stream>>>(peers, row_start, send_slot, T, hidden_dim, world,
                                                      reinterpret_cast<__nv_bfloat16*>(out_bf16));
  return cudaGetLastError();
}

cudaError_t launch_ep_pack(const int32_t* ids, const float* w, const uint8_t* hidden, long long hidden_row_stride,
                           const float* hscale, long long sstride_t, long long sstride_kb, int T, int hidden_dim,
                           int world, uint8_t* send_rows, int32_t* dest_counts, int32_t* send_slot, int num_sms,
                           cudaStream_t stream) {
  ep_plan_kernel<<<1, 1024, 0, stream>>>(ids, T, world, dest_counts, send_slot);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess || T <= 0) return err;
  long long n = (long long)T * world;
  int blocks = (int)((n + 7) / 8);
  int cap = num_sms * 8;
  if (blocks > cap) blocks = cap;
  ep_copy_kernel<<<blocks, 256, 0, stream>>>(ids, w, hidden, hidden_row_stride, hscale, sstride_t, sstride_kb, T,
                                             hidden_dim, world, send_slot, dest_counts, send_rows);
  return cudaGetLastError();
}

cudaError_t launch_ep_combine(const void* returned_bf16, const int32_t* send_slot, const int32_t* dest_counts, int T,
                              int hidden_dim, int world, void* out_bf16, int num_sms, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  long long n = (long long)T * (hidden_dim / 8);
  int blocks = (int)((n + 255) / 256);
  int cap = num_sms * 16;
  if (blocks > cap) blocks = cap;
  ep_combine_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(returned_bf16), send_slot,
                                                dest_counts, T, hidden_dim, world,
                                                reinterpret_cast<__nv_bfloat16*>(out_bf16));
  return cudaGetLastError();
}

}  // namespace b200moe
