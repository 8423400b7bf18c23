// Row-wise e4m3 requantisation of the SwiGLU output.
//
// requant replaces the back half of the reference's `swiglu_fp8_requant_kernel`
// (solution/python/moe_fused.cu:175-195): one scale per row, scale = max(amax/448, 1e-8),
// values rounded to nearest even.  The row maximum comes from GEMM1's epilogue, so the
// fp16 activations are read exactly once here.
// The reference's `reduce_scatter_from_2d_perm_kernel` / `weighted_scatter_kernel`
// (moe_fused.cu:346-393, 490-517) have no counterpart here: the weighted sum over a token's rows
// happens in GEMM2's epilogue.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.cuh"

namespace b200moe {

namespace {

// One block per group of four packed rows (grid-stride): a row is 2-8 KB, so one warp walking
// it alone would be a chain of dependent global loads; 256 threads fetch a row in one or two
// rounds, and four rows' loads are in flight together.
constexpr int kRequantRows = 4;

__global__ void __launch_bounds__(256)
requant_kernel(Workspace ws, int inter) {
  chain_wait();
  chain_release();
  const int rows = ws.at<int>(ws.L.meta)[1];
  const int* row_token = ws.at<int>(ws.L.row_token);
  const __half* act = ws.at<__half>(ws.L.act);
  const unsigned* row_amax = ws.at<unsigned>(ws.L.row_amax);
  uint8_t* act_q = ws.at<uint8_t>(ws.L.act_q);
  float* row_scale = ws.at<float>(ws.L.row_scale);
  const int vecs = inter / 8;   // 8 halves = 16 bytes
  for (int m0 = blockIdx.x * kRequantRows; m0 < rows; m0 += gridDim.x * kRequantRows) {
    float scale[kRequantRows];
    bool live[kRequantRows];
#pragma unroll
    for (int r = 0; r < kRequantRows; ++r) {
      const int m = m0 + r;
      live[r] = m < rows && row_token[m] >= 0;
      const float amax = live[r] ? fmaxf(__uint_as_float(row_amax[m]), 1e-8f) : 1.f;
      scale[r] = fmaxf(amax / 448.0f, 1e-8f);
      if (live[r] && threadIdx.x == 0) row_scale[m] = scale[r];
    }
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      uint4 raw[kRequantRows];
#pragma unroll
      for (int r = 0; r < kRequantRows; ++r)
        if (live[r]) raw[r] = reinterpret_cast<const uint4*>(act + (size_t)(m0 + r) * inter)[v];
#pragma unroll
      for (int r = 0; r < kRequantRows; ++r) {
        if (!live[r]) continue;
        const float sc = scale[r];
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw[r].x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw[r].y));
        const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&raw[r].z));
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&raw[r].w));
        uint2 pk;
        pk.x = pack4_e4m3(a.x / sc, a.y / sc, b.x / sc, b.y / sc);
        pk.y = pack4_e4m3(c.x / sc, c.y / sc, d.x / sc, d.y / sc);
        reinterpret_cast<uint2*>(act_q + (size_t)(m0 + r) * inter)[v] = pk;
      }
    }
  }
}

// Self-test of the bounded wait: one thread waits on a barrier that nothing ever arrives on,
// with a budget of about a millisecond, and must come back with the timeout code recorded.
__global__ void wait_timeout_selftest_kernel(int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait_budget(smem_u32(&bar), 0u, &abort_flag, status, 99, 2000000LL);
    status[2] = ok ? 1 : 0;
    status[3] = abort_flag;
  }
}

}  // namespace

cudaError_t launch_wait_timeout_selftest(int* status, cudaStream_t stream) {
  wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(status);
  return cudaGetLastError();
}

cudaError_t launch_requant(const Workspace& ws, int inter, int num_sms, cudaStream_t stream) {
  long long groups = (ws.L.m_cap + kRequantRows - 1) / kRequantRows;
  int blocks = (int)(groups < (long long)num_sms * 8 ? groups : (long long)num_sms * 8);
  if (blocks < 1) blocks = 1;
  return launch_chained(requant_kernel, dim3(blocks), dim3(256), 0, stream, ws, inter);
}

}  // namespace b200moe
