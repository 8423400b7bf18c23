// Grouped FP8 GEMMs on CTA pairs: tcgen05.mma.cta_group::2 over a thread-block cluster of two.
//
// Same arithmetic, roles and epilogues as the one-CTA kernel in gemm.cu (which replaces the
// reference's `moe_blockwise_grouped_mm_v2`, solution/python/moe_gemm.cu:527-654); the tile is
// 256 packed rows x 256 weight rows per pair.  Each CTA loads its own 128 rows of A and only
// HALF of the B tile (128 weight rows) - plain TMA loads, no multicast - and one MMA issued by
// the leader CTA reads both CTAs' shared memory and writes both CTAs' tensor memory.  Per
// 128-wide K block a CTA therefore pulls 32 KB through L2 instead of 48 KB, six stages fit,
// and an expert with up to 256 rows has its weights fetched exactly once.
//
// Barriers.  In the leader CTA: full[s] (count 2: one arrive.expect_tx per CTA's producer, TMA
// bytes of both CTAs) and tempty[b] (count 16: the eight promotion warps of each CTA).  In
// each CTA: empty[s] and tfull[b], signalled for both CTAs at once by the leader's
// tcgen05.commit (barrier-arrive multicast, not a data multicast).  GEMM1: the leader holds
// the gate rows, its peer the matching up rows, so D's columns [0,128) are gate and [128,256)
// up in both CTAs, exactly as in the one-CTA kernel.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.cuh"

namespace b200moe {

namespace {

constexpr int kCtrlWarps = 4;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 32 * (kCtrlWarps + kEpiWarps);   // 384
constexpr int kCtrlRegs = 56;
constexpr int kEpiRegs = 224;
constexpr int BN = 256;                       // weight rows per pair tile
constexpr int kABytes = kTileM * kBlockK;     // 16 KiB: this CTA's 128 rows of A
constexpr int kBBytes = (BN / 2) * kBlockK;   // 16 KiB: this CTA's half of B
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int S = 6;
constexpr int kTmemCols = 2 * BN;
constexpr int kSmemBytes = S * kStageBytes + 256 + 1024;
constexpr int kScalePrefetchDist = 6;
constexpr int CPT = BN / 2;                   // accumulator columns per promotion thread

__device__ __forceinline__ float silu_mul(float g, float u) {
  float sig = __fdividef(1.0f, 1.0f + __expf(-u));   // approximate reciprocal: 2 ulp, far below e4m3 resolution
  return g * (u * sig);
}

__device__ __forceinline__ void fma_chunk(float2* acc, const uint32_t (&r)[32], float sc) {
  const float2 s2 = make_float2(sc, sc);
#pragma unroll
  for (int j = 0; j < 16; ++j)
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), s2, acc[j]);
}

template <int MODE>
__device__ __forceinline__ uint32_t chunk_col(int c, int h) {
  if (MODE == 1) {
    const bool up = c >= 2;
    return (up ? BN / 2 : 0) + h * (BN / 4) + (up ? c - 2 : c) * 32;
  }
  return h * (BN / 2) + c * 32;
}

template <int MODE, bool PROF>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * kStageBytes);
  const uint32_t bar_full = smem_u32(bars);              // used in the leader only
  const uint32_t bar_empty = bar_full + 8 * S;           // per CTA
  const uint32_t bar_tfull = bar_empty + 8 * S;          // per CTA
  const uint32_t bar_tempty = bar_tfull + 16;            // used in the leader only
  const uint32_t bar_drain = bar_tempty + 16;            // leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();               // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 2);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 2 * kEpiWarps);
    }
    mbar_init(bar_drain, 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmap_a);
    tma_prefetch_desc(&p.tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before anyone signals the peer's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int m_pairs = p.meta[0] >> 1;   // segments are padded to 256 rows in this mode
  const int total_items = m_pairs * p.n_tiles;
  const int kblocks = p.kblocks;

  if (warp < kCtrlWarps) {
    reg_dealloc<kCtrlRegs>();
    if (warp == 0 && lane == 0) {
      // ------------------------------ TMA producer (both CTAs) ------------------------------
      uint32_t it = 0;
      bool alive = true;
      for (int w = pair_id; w < total_items && alive; w += num_pairs) {
        const int m_pair = w / p.n_tiles, n_tile = w % p.n_tiles;
        const int m_tile = 2 * m_pair + (int)rank;
        const int e = p.tile_expert[2 * m_pair];
        int brow;
        if (MODE == 1) brow = e * p.n_per_expert + n_tile * (BN / 2) + (rank ? p.inter : 0);
        else brow = e * p.n_per_expert + n_tile * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % S, ph = (it / S) & 1u;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status, 11)) { alive = false; break; }
          const uint32_t full = map_to_cta(bar_full + 8 * s, 0);
          const uint32_t a_dst = smem_base + s * kStageBytes;
          mbar_arrive_expect_tx_cluster(full, kStageBytes);
          tma_load_2d_pair(a_dst, &p.tmap_a, kb * kBlockK, m_tile * kTileM, full);
          tma_load_2d_pair(a_dst + kABytes, &p.tmap_b, kb * kBlockK, brow, full);
        }
      }
      // This CTA's copies are all consumed once the last stages' "empty" arrives came back
      // (an MMA that read a stage completed after its copies landed).
      const uint32_t first = it > (uint32_t)S ? it - S : 0u;
      for (uint32_t j = first; j < it; ++j)
        (void)mbar_wait(bar_empty + 8 * (j % S), (j / S) & 1u, abort_flag + 1, p.status, 16);
    } else if (warp == 1 && lane == 0 && rank == 0) {
      // ------------------------------ MMA issuer (leader only) ------------------------------
      constexpr uint32_t idesc = make_idesc_e4m3(2 * kTileM, BN);
      uint32_t it = 0;
      bool alive = true;
      long long wait_epi = 0, wait_tma = 0;
      for (int w = pair_id; w < total_items && alive; w += num_pairs) {
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % S, ph = (it / S) & 1u;
          const uint32_t b = it & 1u, bph = (it >> 1) & 1u;
          const long long m0 = PROF ? clock64() : 0;
          if (!mbar_wait_cluster(bar_tempty + 8 * b, bph ^ 1u, abort_flag, p.status, 12)) { alive = false; break; }
          const long long m1 = PROF ? clock64() : 0;
          if (!mbar_wait_cluster(bar_full + 8 * s, ph, abort_flag, p.status, 13)) { alive = false; break; }
          if (PROF) {
            wait_epi += m1 - m0;
            wait_tma += clock64() - m1;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * kStageBytes;
          const uint32_t b_addr = a_addr + kABytes;
          const uint32_t d_addr = tmem_base + b * BN;
#pragma unroll
          for (int k4 = 0; k4 < kBlockK / 32; ++k4) {
            tc_mma_f8_pair(d_addr, make_kmajor_sw128_desc(a_addr + k4 * 32), make_kmajor_sw128_desc(b_addr + k4 * 32),
                           idesc, k4 > 0 ? 1u : 0u);
          }
          tc_commit_pair(bar_empty + 8 * s, (uint16_t)3);
          tc_commit_pair(bar_tfull + 8 * b, (uint16_t)3);
        }
      }
      tc_commit_pair_local(bar_drain);
      (void)mbar_wait(bar_drain, 0u, abort_flag + 1, p.status, 15);
      if (PROF && p.prof && blockIdx.x == 0) {
        p.prof[7] = (unsigned long long)wait_epi;
        p.prof[8] = (unsigned long long)wait_tma;
      }
    }
  } else {
    // ------------------------------ promotion + epilogue (both CTAs) ------------------------------
    reg_alloc<kEpiRegs>();
    const int ew = warp - kCtrlWarps;
    const int q = warp & 3;
    const int h = ew >> 2;
    uint32_t it = 0;
    bool alive = true;
    const bool prof_me = PROF && p.prof && blockIdx.x == 0 && ew == 0 && lane == 0;
    const long long t_begin = PROF ? clock64() : 0;
    long long t_wait = 0, t_promote = 0, t_epi = 0;
    const int nblk_per_expert = p.n_per_expert / kBlockK;
    const uint32_t tempty_leader = map_to_cta(bar_tempty, 0);
    for (int w = pair_id; w < total_items && alive; w += num_pairs) {
      const int m_pair = w / p.n_tiles, n_tile = w % p.n_tiles;
      const int m_tile = 2 * m_pair + (int)rank;
      const int e = p.tile_expert[2 * m_pair];
      const int row = m_tile * kTileM + q * 32 + lane;
      const int tok = p.row_token[row];
      float2 acc[CPT / 2];
#pragma unroll
      for (int j = 0; j < CPT / 2; ++j) acc[j] = make_float2(0.f, 0.f);

      const float* sa_ptr = nullptr;
      const float* sb0_ptr;
      const float* sb1_ptr = nullptr;
      if (MODE == 1) {
        sa_ptr = p.a_scale + row;
        const int gcol0 = n_tile * (BN / 2) + h * (BN / 4);
        sb0_ptr = p.b_scale + ((size_t)e * nblk_per_expert + gcol0 / kBlockK) * kblocks;
        sb1_ptr = p.b_scale + ((size_t)e * nblk_per_expert + (p.inter + gcol0) / kBlockK) * kblocks;
#pragma unroll 1
        for (int kb = 1; kb < kScalePrefetchDist && kb < kblocks; ++kb) prefetch_l2(sa_ptr + (size_t)kb * p.m_cap);
      } else {
        const int col0 = n_tile * BN + h * (BN / 2);
        sb0_ptr = p.b_scale + ((size_t)e * nblk_per_expert + col0 / kBlockK) * kblocks;
      }
      float sa_n = MODE == 1 ? sa_ptr[0] : 1.f;
      float sb0_n = sb0_ptr[0];
      float sb1_n = MODE == 1 ? sb1_ptr[0] : 0.f;

      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const uint32_t b = it & 1u, bph = (it >> 1) & 1u;
        const float sc0 = sa_n * sb0_n;
        const float sc1 = sa_n * sb1_n;
        if (kb + 1 < kblocks) {
          if (MODE == 1) {
            sa_n = sa_ptr[(size_t)(kb + 1) * p.m_cap];
            sb1_n = sb1_ptr[kb + 1];
            if (kb + kScalePrefetchDist < kblocks) prefetch_l2(sa_ptr + (size_t)(kb + kScalePrefetchDist) * p.m_cap);
          }
          sb0_n = sb0_ptr[kb + 1];
        }
        const long long c0 = PROF ? clock64() : 0;
        bool ok = mbar_wait(bar_tfull + 8 * b, bph, abort_flag, p.status, 14);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
        const long long c1 = PROF ? clock64() : 0;
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + b * BN;
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(t_row + chunk_col<MODE>(0, h), ra);
        tmem_ld_32x32(t_row + chunk_col<MODE>(1, h), rb);
        tmem_ld_wait_on(ra, rb);
        fma_chunk(acc, ra, sc0);
        tmem_ld_32x32(t_row + chunk_col<MODE>(2, h), ra);
        fma_chunk(acc + 16, rb, sc0);
        tmem_ld_32x32(t_row + chunk_col<MODE>(3, h), rb);
        tmem_ld_wait_on(ra, rb);
        fma_chunk(acc + 32, ra, MODE == 1 ? sc1 : sc0);
        fma_chunk(acc + 48, rb, MODE == 1 ? sc1 : sc0);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(tempty_leader + 8 * b);
        if (PROF) {
          t_wait += c1 - c0;
          t_promote += clock64() - c1;
        }
      }
      if (!alive) break;
      const long long te0 = PROF ? clock64() : 0;

      if (tok >= 0) {
        if (MODE == 1) {
          constexpr int HP = CPT / 4;
          // fp16 keeps 11 significant bits, three more than the e4m3 codes made from it need;
          // the row maximum is taken over the rounded values so that it is attained exactly.
          __half* dst = p.act + (size_t)row * p.inter + n_tile * (BN / 2) + h * (BN / 4);
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < HP; j += 4) {
            uint4 pk;
            uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              __half2 hh = __floats2half2_rn(silu_mul(acc[j + t].x, acc[HP + j + t].x),
                                             silu_mul(acc[j + t].y, acc[HP + j + t].y));
              float2 back = __half22float2(hh);
              amax = fmaxf(amax, fmaxf(fabsf(back.x), fabsf(back.y)));
              w[t] = *reinterpret_cast<uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(dst + 2 * j) = pk;
          }
          atomicMax(p.row_amax + row, __float_as_uint(amax));
        } else {
          const float rs = p.row_scale[row] * p.row_weight[row];
          __nv_bfloat16* dst = p.y + (size_t)row * p.hidden + n_tile * BN + h * (BN / 2);
#pragma unroll
          for (int j = 0; j < CPT / 2; j += 4) {
            uint4 pk;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(acc[j].x * rs, acc[j].y * rs);
            __nv_bfloat162 t1 = __floats2bfloat162_rn(acc[j + 1].x * rs, acc[j + 1].y * rs);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[j + 2].x * rs, acc[j + 2].y * rs);
            __nv_bfloat162 t3 = __floats2bfloat162_rn(acc[j + 3].x * rs, acc[j + 3].y * rs);
            pk.x = *reinterpret_cast<uint32_t*>(&t0);
            pk.y = *reinterpret_cast<uint32_t*>(&t1);
            pk.z = *reinterpret_cast<uint32_t*>(&t2);
            pk.w = *reinterpret_cast<uint32_t*>(&t3);
            *reinterpret_cast<uint4*>(dst + 2 * j) = pk;
          }
        }
      }
      if (PROF) t_epi += clock64() - te0;
    }
    if (prof_me) {
      p.prof[0] = (unsigned long long)t_wait;
      p.prof[1] = (unsigned long long)t_promote;
      p.prof[3] = (unsigned long long)it;
      p.prof[4] = (unsigned long long)(clock64() - t_begin);
      p.prof[5] = (unsigned long long)t_epi;
    }
  }

  // Neither CTA may leave (or free tensor memory) while its peer can still signal its
  // barriers or the leader's MMAs can still touch its shared or tensor memory.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
}

template <int MODE>
cudaError_t launch_one(const GemmParams& p, int num_sms, cudaStream_t stream) {
  const int grid = num_sms & ~1;
  if (p.prof)
    grouped_gemm_pair_kernel<MODE, true><<<grid, kThreads, kSmemBytes, stream>>>(p);
  else
    grouped_gemm_pair_kernel<MODE, false><<<grid, kThreads, kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

template <int MODE>
cudaError_t configure_one() {
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_pair_kernel<MODE, true>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(grouped_gemm_pair_kernel<MODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              kSmemBytes);
}

}  // namespace

cudaError_t configure_grouped_gemm_pair() {
  cudaError_t e;
  if ((e = configure_one<1>()) != cudaSuccess) return e;
  return configure_one<2>();
}

cudaError_t launch_grouped_gemm_pair(int mode, const GemmParams& p, int num_sms, cudaStream_t stream) {
  return mode == 1 ? launch_one<1>(p, num_sms, stream) : launch_one<2>(p, num_sms, stream);
}

}  // namespace b200moe
