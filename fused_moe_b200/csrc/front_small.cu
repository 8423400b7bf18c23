// Routing, scan and placement of a decode-size call (at most 32 tokens) in ONE block.
//
// At these sizes the three kernels it stands for (route.cu, and scan + place of permute.cu,
// which replace the reference's `fused_route_topk_kernel`, `exclusive_scan_kernel` and
// `dispatch_place_kernel`, solution/python/moe_fused.cu:568-698, 888-1051) do a few
// microseconds of work between them and two launch boundaries; the reference folds scan and
// placement into `fused_dispatch_single_block_kernel` for the same reason.  Results are
// identical to the separate kernels: same routing arithmetic (route_core.cuh), segments padded
// to `pad_rows`, placement stable by token id.
#include "common.cuh"
#include "kernels.cuh"
#include "route_core.cuh"

namespace b200moe {

namespace {

constexpr int kFrontWarps = kFrontSmallMaxTokens;   // one warp per token

__global__ void __launch_bounds__(kFrontWarps * 32, 1)
route_place_small_kernel(Workspace ws, const void* __restrict__ logits, int logits_dtype,
                         const void* __restrict__ bias, int bias_dtype, int T, float rsf, int local_off, int e_local,
                         int pad_rows) {
  __shared__ int s_ids[kTopK][kFrontSmallMaxTokens];     // [k][token]
  __shared__ float s_w[kTopK][kFrontSmallMaxTokens];
  __shared__ int s_scan[kNumExperts];
  __shared__ int s_row0[kNumExperts];
  __shared__ int s_cnt[kNumExperts];
  __shared__ int s_rows;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  chain_release();   // launched in plain stream order itself (the first kernel of a call)
  // The call's counters (status word, meta, split-K and slab arrival counts): cleared here instead of by a
  // memset of its own, one launch boundary less.  Nothing of them is read before the barriers below.
  {
    uint32_t* z = ws.at<uint32_t>(ws.L.status);
    const int n = (int)((ws.L.chunk_counts - ws.L.status) / 4);
    for (int i = threadIdx.x; i < n; i += blockDim.x) z[i] = 0u;
  }

  int32_t* topk_ids = ws.at<int32_t>(ws.L.topk_ids);
  float* topk_w = ws.at<float>(ws.L.topk_w);
  int* tok_rows = ws.at<int>(ws.L.tok_rows);
  unsigned* row_amax = ws.at<unsigned>(ws.L.row_amax);

  // ---- route: warp t routes token t
  if (warp < T) {
    float b[kNumGroups];
#pragma unroll
    for (int g = 0; g < kNumGroups; ++g) b[g] = load_as_float(bias, bias_dtype, g * 32 + lane);
    int my_id;
    float my_w;
    route_one_token(logits, logits_dtype, warp, b, rsf, lane, my_id, my_w);
    if (lane < kTopK) {
      topk_ids[(size_t)warp * kTopK + lane] = my_id;
      topk_w[(size_t)warp * kTopK + lane] = my_w;
      tok_rows[(size_t)warp * kTopK + lane] = -1;   // local pairs are overwritten below
      s_ids[lane][warp] = my_id;
      s_w[lane][warp] = my_w;
    }
  } else if (lane < kTopK) {
    s_ids[lane][warp] = -1;
  }
  if (threadIdx.x == 0) s_rows = 0;
  __syncthreads();

  // ---- scan: thread e counts the pairs of local expert e, pads, prefix-sums
  const int e = threadIdx.x;
  int total = 0, padded = 0;
  if (e < kNumExperts) {
    if (e < e_local) {
      const int want = e + local_off;
      for (int t = 0; t < T; ++t) {
#pragma unroll
        for (int k = 0; k < kTopK; ++k) total += (s_ids[k][t] == want) ? 1 : 0;
      }
    }
    padded = (total + pad_rows - 1) / pad_rows * pad_rows;
    s_scan[e] = padded;
  }
  __syncthreads();
  for (int off = 1; off < kNumExperts; off <<= 1) {
    int v = 0;
    if (e < kNumExperts && e >= off) v = s_scan[e - off];
    __syncthreads();
    if (e < kNumExperts) s_scan[e] += v;
    __syncthreads();
  }
  int* expert_row0 = ws.at<int>(ws.L.expert_row0);
  int* expert_count = ws.at<int>(ws.L.expert_count);
  int* tile_expert = ws.at<int>(ws.L.tile_expert);
  int* row_token = ws.at<int>(ws.L.row_token);
  float* row_weight = ws.at<float>(ws.L.row_weight);
  if (e < kNumExperts) {
    const int row0 = s_scan[e] - padded;
    s_row0[e] = row0;
    s_cnt[e] = total;
    if (e < e_local) {
      expert_row0[e] = row0;
      expert_count[e] = total;
      for (int t = row0 / kTileM; t < (row0 + padded) / kTileM; ++t) tile_expert[t] = e;
      for (int r = row0 + total; r < row0 + padded; ++r) row_token[r] = -1;
      if (total) atomicAdd(&s_rows, total);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int padded_total = s_scan[kNumExperts - 1];
    expert_row0[e_local] = padded_total;
    int* meta = ws.at<int>(ws.L.meta);
    meta[0] = padded_total / kTileM;
    meta[1] = padded_total;
    meta[2] = s_rows;
    meta[3] = pad_rows;
  }

  // ---- place: a warp walks an expert's tokens in token order (lane = token)
  for (int le = warp; le < e_local; le += kFrontWarps) {
    if (s_cnt[le] == 0) continue;
    const int want = le + local_off;
    int kf = -1;
#pragma unroll
    for (int k = 0; k < kTopK; ++k)
      if (s_ids[k][lane] == want) kf = k;
    const uint32_t hit = __ballot_sync(0xffffffffu, kf >= 0);
    if (kf >= 0) {
      const int r = s_row0[le] + __popc(hit & ((1u << lane) - 1u));
      row_token[r] = lane;
      row_weight[r] = s_w[kf][lane];
      row_amax[r] = 0u;   // GEMM1's epilogue takes the running maximum with atomicMax
      tok_rows[(size_t)lane * kTopK + kf] = r;
    }
  }
}

}  // namespace

cudaError_t launch_route_place_small(const Workspace& ws, const void* logits, int logits_dtype, const void* bias,
                                     int bias_dtype, int T, float rsf, int local_off, int e_local, int pad_rows,
                                     cudaStream_t stream) {
  if (T <= 0 || T > kFrontSmallMaxTokens) return cudaErrorInvalidValue;
  route_place_small_kernel<<<1, kFrontWarps * 32, 0, stream>>>(ws, logits, logits_dtype, bias, bias_dtype, T, rsf,
                                                               local_off, e_local, pad_rows);
  return cudaGetLastError();
}

}  // namespace b200moe
