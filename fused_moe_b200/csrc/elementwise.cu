// Row-wise e4m3 requantisation of the SwiGLU output and the bf16 finalisation of the output.
//
// requant replaces the back half of the reference's `swiglu_fp8_requant_kernel`
// (solution/python/moe_fused.cu:175-195): one scale per row, scale = max(amax/448, 1e-8),
// values rounded to nearest even.  The row maximum comes from GEMM1's epilogue, so the
// fp32 activations are read exactly once here.
// finalize replaces the bf16 write of `reduce_scatter_from_2d_perm_kernel`
// (moe_fused.cu:346-393): the fp32 sums of GEMM2's epilogue are rounded once to bf16.
#include "common.cuh"
#include "kernels.cuh"

namespace b200moe {

namespace {

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  // two RNE, saturating conversions of float pairs; byte order = element order
  uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

__global__ void __launch_bounds__(256)
requant_kernel(Workspace ws, int inter) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int rows = ws.at<int>(ws.L.meta)[1];
  const int* row_token = ws.at<int>(ws.L.row_token);
  const float* act = ws.at<float>(ws.L.act);
  const unsigned* row_amax = ws.at<unsigned>(ws.L.row_amax);
  uint8_t* act_q = ws.at<uint8_t>(ws.L.act_q);
  float* row_scale = ws.at<float>(ws.L.row_scale);
  for (int m = blockIdx.x * wpb + (threadIdx.x >> 5); m < rows; m += gridDim.x * wpb) {
    if (row_token[m] < 0) continue;
    float amax = fmaxf(__uint_as_float(row_amax[m]), 1e-8f);
    float scale = fmaxf(amax / 448.0f, 1e-8f);
    if (lane == 0) row_scale[m] = scale;
    const float4* src = reinterpret_cast<const float4*>(act + (size_t)m * inter);
    uint32_t* dst = reinterpret_cast<uint32_t*>(act_q + (size_t)m * inter);
    for (int v = lane; v < inter / 4; v += 32) {
      float4 x = src[v];
      dst[v] = pack4_e4m3(x.x / scale, x.y / scale, x.z / scale, x.w / scale);
    }
  }
}

__global__ void __launch_bounds__(256)
finalize_kernel(const float* __restrict__ acc, int T, int hidden, __nv_bfloat16* __restrict__ out, long long stride) {
  const int vec_per_row = hidden / 4;
  const long long n = (long long)T * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    int t = (int)(i / vec_per_row), v = (int)(i % vec_per_row);
    float4 x = reinterpret_cast<const float4*>(acc)[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(x.z, x.w);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + (size_t)t * stride + 4 * v) = pk;
  }
}

}  // namespace

cudaError_t launch_requant(const Workspace& ws, int inter, int num_sms, cudaStream_t stream) {
  long long cap_rows = ws.L.m_cap;
  int blocks = (int)((cap_rows + 7) / 8);
  int cap = num_sms * 8;
  if (blocks > cap) blocks = cap;
  requant_kernel<<<blocks, 256, 0, stream>>>(ws, inter);
  return cudaGetLastError();
}

cudaError_t launch_finalize(const float* out_acc, int T, int hidden, void* out_bf16, long long out_row_stride,
                            int num_sms, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  long long n = (long long)T * (hidden / 4);
  int blocks = (int)((n + 255) / 256);
  int cap = num_sms * 16;
  if (blocks > cap) blocks = cap;
  finalize_kernel<<<blocks, 256, 0, stream>>>(out_acc, T, hidden, reinterpret_cast<__nv_bfloat16*>(out_bf16),
                                              out_row_stride);
  return cudaGetLastError();
}

}  // namespace b200moe
