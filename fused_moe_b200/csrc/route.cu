// Routing (DeepSeek-V3 no-aux) and the per-chunk histogram of local experts.
//
// Replaces the reference's `fused_route_topk_kernel` (solution/python/moe_fused.cu:568-698)
// and `dispatch_count_kernel` (moe_fused.cu:866-881).  Semantics follow the reference's
// torch check (experiments/fast_bench/correctness_bench.py:47-61): fp32 logits are used as
// given, group scores count equal values with multiplicity, and every selection breaks ties
// toward the lowest index.
#include "common.cuh"
#include "kernels.cuh"
#include "route_core.cuh"

namespace b200moe {

namespace {

constexpr int kRouteWarps = 8;

__global__ void __launch_bounds__(kRouteWarps * 32)
route_kernel(const void* __restrict__ logits, int logits_dtype, const void* __restrict__ bias, int bias_dtype,
             int T, float rsf, int local_off, int e_local,
             int32_t* __restrict__ topk_ids, float* __restrict__ topk_w, int* __restrict__ chunk_counts) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  chain_release();   // launched in plain stream order itself; the kernel after it may become resident early
  // Lane L owns expert g*32+L of every group g, so a group reduction is a warp reduction.
  float b[kNumGroups];
#pragma unroll
  for (int g = 0; g < kNumGroups; ++g) b[g] = load_as_float(bias, bias_dtype, g * 32 + lane);

  for (int t = blockIdx.x * kRouteWarps + warp; t < T; t += gridDim.x * kRouteWarps) {
    int my_id;
    float my_w;
    route_one_token(logits, logits_dtype, t, b, rsf, lane, my_id, my_w);
    if (lane < kTopK) {
      topk_ids[(size_t)t * kTopK + lane] = my_id;
      topk_w[(size_t)t * kTopK + lane] = my_w;
      int le = my_id - local_off;
      if (le >= 0 && le < e_local) atomicAdd(&chunk_counts[(t / kChunkTokens) * e_local + le], 1);
    }
  }
}

__global__ void __launch_bounds__(256)
count_kernel(const int32_t* __restrict__ ids, long long row_stride, int T, int local_off, int e_local,
             int* __restrict__ chunk_counts, const int* __restrict__ n_rows_dev) {
  chain_release();
  if (n_rows_dev) T = min(T, *n_rows_dev);
  long long n = (long long)T * kTopK;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    int t = (int)(i / kTopK), k = (int)(i % kTopK);
    int le = ids[(size_t)t * row_stride + k] - local_off;
    if (le >= 0 && le < e_local) atomicAdd(&chunk_counts[(t / kChunkTokens) * e_local + le], 1);
  }
}

}  // namespace

cudaError_t launch_route(const void* logits, int logits_dtype, const void* bias, int bias_dtype, int T, float rsf,
                         int local_off, int e_local, int32_t* ids, float* w, int* chunk_counts, int num_sms,
                         cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  int blocks = (T + kRouteWarps - 1) / kRouteWarps;
  int cap = num_sms * 8;
  if (blocks > cap) blocks = cap;
  route_kernel<<<blocks, kRouteWarps * 32, 0, stream>>>(logits, logits_dtype, bias, bias_dtype, T, rsf, local_off,
                                                       e_local, ids, w, chunk_counts);
  return cudaGetLastError();
}

cudaError_t launch_count(const int32_t* ids, long long row_stride, int T, int local_off, int e_local,
                         int* chunk_counts, int num_sms, cudaStream_t stream, const int* n_rows_dev) {
  if (T <= 0) return cudaSuccess;
  long long n = (long long)T * kTopK;
  int blocks = (int)((n + 255) / 256);
  int cap = num_sms * 8;
  if (blocks > cap) blocks = cap;
  count_kernel<<<blocks, 256, 0, stream>>>(ids, row_stride, T, local_off, e_local, chunk_counts, n_rows_dev);
  return cudaGetLastError();
}

}  // namespace b200moe
