// Row-wise e4m3 requantisation of the SwiGLU output and the per-token combine of the output.
//
// requant replaces the back half of the reference's `swiglu_fp8_requant_kernel`
// (solution/python/moe_fused.cu:175-195): one scale per row, scale = max(amax/448, 1e-8),
// values rounded to nearest even.  The row maximum comes from GEMM1's epilogue, so the
// fp16 activations are read exactly once here.
// combine replaces `reduce_scatter_from_2d_perm_kernel` / `weighted_scatter_kernel`
// (moe_fused.cu:346-393, 490-517): a gather per token over its rows instead of atomics,
// so the output is bit-reproducible.
#include <cuda_fp16.h>

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

// out[t,:] = sum of the token's rows, taken in ascending packed-row order (= ascending
// expert) and rounded to bf16 after every addition: the arithmetic of the reference's
// `out[t] += bf16(G2 * w)` loop (experiments/fast_bench/correctness_bench.py:107-111).
__global__ void __launch_bounds__(256)
combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ tok_rows, int T, int hidden,
               __nv_bfloat16* __restrict__ out, long long stride, int splits) {
  chain_wait();
  chain_release();
  const int vec_per_row = hidden / 8;   // 8 bf16 = 16 bytes
  // One block per token (block-stride): the token's eight row numbers are sorted once per
  // thread and then reused for all of the thread's 16-byte column groups.  Small batches cut a
  // token's columns into `splits` parts on as many blocks, so that a thread has one group.
  const int part_len = (vec_per_row + splits - 1) / splits;
  for (int item = blockIdx.x; item < T * splits; item += gridDim.x) {
    const int t = item / splits;
    const int v_begin = (item % splits) * part_len;
    const int v_end = min(vec_per_row, v_begin + part_len);
    int rows[kTopK];
    {
      const int4 a = reinterpret_cast<const int4*>(tok_rows + (size_t)t * kTopK)[0];
      const int4 b = reinterpret_cast<const int4*>(tok_rows + (size_t)t * kTopK)[1];
      rows[0] = a.x; rows[1] = a.y; rows[2] = a.z; rows[3] = a.w;
      rows[4] = b.x; rows[5] = b.y; rows[6] = b.z; rows[7] = b.w;
    }
    // ascending order with -1 (not local) last: 8-element insertion sort on unsigned keys
#pragma unroll
    for (int a = 1; a < kTopK; ++a) {
#pragma unroll
      for (int b = a; b > 0; --b) {
        unsigned x = (unsigned)rows[b - 1], z = (unsigned)rows[b];
        if (z < x) { rows[b - 1] = (int)z; rows[b] = (int)x; }
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * stride);
    if (rows[0] < 0) {   // no local expert took this token
      for (int v = v_begin + threadIdx.x; v < v_end; v += blockDim.x) dst[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    for (int v = v_begin + threadIdx.x; v < v_end; v += blockDim.x) {
      uint4 raw[kTopK];
#pragma unroll
      for (int k = 0; k < kTopK; ++k)
        if (rows[k] >= 0) raw[k] = reinterpret_cast<const uint4*>(y + (size_t)rows[k] * hidden)[v];
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int k = 0; k < kTopK; ++k) {
        if (rows[k] < 0) break;
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw[k]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(p2[j]);
          // bf16 + bf16 in fp32 is exact before the rounding, so this equals a bf16 addition
          acc[2 * j] = __bfloat162float(__float2bfloat16_rn(acc[2 * j] + f.x));
          acc[2 * j + 1] = __bfloat162float(__float2bfloat16_rn(acc[2 * j + 1] + f.y));
        }
      }
      uint4 pk;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
      for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      dst[v] = pk;
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

cudaError_t launch_combine(const Workspace& ws, int T, int hidden, void* out_bf16, long long out_row_stride,
                           int num_sms, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  const int splits = T < 2 * num_sms ? 4 : 1;
  int blocks = T * splits;
  const int cap = num_sms * 8;   // 8 blocks of 256 threads are resident per SM
  if (blocks > cap) blocks = cap;
  return launch_chained(combine_kernel, dim3(blocks), dim3(256), 0, stream,
                        (const __nv_bfloat16*)ws.at<__nv_bfloat16>(ws.L.y), (const int*)ws.at<int>(ws.L.tok_rows), T,
                        hidden, reinterpret_cast<__nv_bfloat16*>(out_bf16), out_row_stride, splits);
}

}  // namespace b200moe
