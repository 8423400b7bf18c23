// Routing for callers that must not allocate device memory.
//
// Some hosts of this library run inside a callback that forbids allocation: an inference
// engine's plugin "enqueue" hook, a serving loop with a frozen memory budget, or any code
// that must not trigger the implicit device synchronisation of cudaMalloc/cudaFree.  They
// cannot size and allocate the workspace that b200moe_route wants for its histogram.  This
// entry point does the same routing with its scratch (the per-chunk expert histogram) in a
// fixed array that lives in the library image, so the caller brings only inputs and outputs.
//
// Trade-offs, all documented at the declaration: the array has a fixed capacity (64 Ki
// tokens), every GPU that loads the library carries its 256 KiB until the process exits,
// all calls on a device share it (two calls that overlap on the GPU race), and the first
// call on each device looks up the array's device address, which is a set-up step that
// belongs before any stream capture.
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr int kStaticMaxTokens = 65536;
constexpr int kStaticMaxChunks = kStaticMaxTokens / kChunkTokens;            // 256
constexpr int kStaticScratchInts = kStaticMaxChunks * kNumExperts;           // 65536 ints = 256 KiB

// Scratch of b200moe_route_static.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address and must never be passed to a kernel.
static __device__ __align__(256) int g_route_scratch[kStaticScratchInts];

std::mutex g_static_mutex;
int* g_scratch_dev_ptr[64] = {nullptr};   // per device: address of g_route_scratch on that device
int g_static_sms[64] = {0};
thread_local char g_static_error[192] = "";

// counts[e] = sum over chunks of hist[c][e]
__global__ void __launch_bounds__(256)
sum_chunks_kernel(const int* __restrict__ hist, int n_chunks, int e_local, int32_t* __restrict__ counts) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= e_local) return;
  int total = 0;
  for (int c = 0; c < n_chunks; ++c) total += hist[c * e_local + e];
  counts[e] = total;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

const char* b200moe_route_static_error(void) { return g_static_error; }

int b200moe_route_static_max_tokens(void) { return kStaticMaxTokens; }

int b200moe_route_static(const void* logits, int logits_dtype, const void* bias, int bias_dtype, int T,
                         float routed_scaling_factor, int local_expert_offset, int e_local, int32_t* topk_ids,
                         float* topk_w, int32_t* expert_counts, void* stream) {
  g_static_error[0] = 0;
  if (T < 0 || e_local < 1 || e_local > kNumExperts || local_expert_offset < 0 ||
      local_expert_offset + e_local > kNumExperts)
    return B200MOE_ERR_INVALID_ARGUMENT;
  if ((logits_dtype != B200MOE_F32 && logits_dtype != B200MOE_BF16) ||
      (bias_dtype != B200MOE_F32 && bias_dtype != B200MOE_BF16) || !expert_counts)
    return B200MOE_ERR_INVALID_ARGUMENT;
  if (T > 0 && (!logits || !bias || !topk_ids || !topk_w)) return B200MOE_ERR_INVALID_ARGUMENT;
  if (T > kStaticMaxTokens) {
    snprintf(g_static_error, sizeof(g_static_error),
             "b200moe_route_static handles at most %d tokens per call (got %d): its scratch is a fixed "
             "array; use b200moe_route with a workspace for larger batches",
             kStaticMaxTokens, T);
    return B200MOE_ERR_UNSUPPORTED_SHAPE;
  }
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= 64) return B200MOE_ERR_CUDA;
  int* scratch = nullptr;
  int num_sms = 0;
  {
    // First call on this device (with it current): resolve the device address of the array.
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_scratch_dev_ptr[dev]) {
      void* p = nullptr;
      err = cudaGetSymbolAddress(&p, g_route_scratch);
      if (err != cudaSuccess || !p) {
        snprintf(g_static_error, sizeof(g_static_error), "cudaGetSymbolAddress(g_route_scratch): %s",
                 cudaGetErrorString(err));
        return B200MOE_ERR_CUDA;
      }
      int sms = 0;
      err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (err != cudaSuccess || sms <= 0) {
        snprintf(g_static_error, sizeof(g_static_error), "cudaDeviceGetAttribute: %s", cudaGetErrorString(err));
        return B200MOE_ERR_CUDA;
      }
      g_static_sms[dev] = sms;
      g_scratch_dev_ptr[dev] = reinterpret_cast<int*>(p);
    }
    scratch = g_scratch_dev_ptr[dev];
    num_sms = g_static_sms[dev];
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int n_chunks = T > 0 ? (T + kChunkTokens - 1) / kChunkTokens : 1;
  // The array keeps whatever the previous call left: the histogram must start at zero.
  err = cudaMemsetAsync(scratch, 0, (size_t)n_chunks * e_local * sizeof(int), st);
  if (err == cudaSuccess)
    err = launch_route(logits, logits_dtype, bias, bias_dtype, T, routed_scaling_factor, local_expert_offset,
                       e_local, topk_ids, topk_w, scratch, num_sms, st);
  if (err == cudaSuccess) {
    sum_chunks_kernel<<<(e_local + 255) / 256, 256, 0, st>>>(scratch, n_chunks, e_local, expert_counts);
    err = cudaGetLastError();
  }
  if (err != cudaSuccess) {
    snprintf(g_static_error, sizeof(g_static_error), "launch: %s", cudaGetErrorString(err));
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}

}  // extern "C"
