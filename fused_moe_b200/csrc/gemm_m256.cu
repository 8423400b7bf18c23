// Grouped FP8 GEMMs with 256-row tiles on one CTA: two M tiles of an expert share every B box.
// Opt-in variant (B200MOE_M256=1); the default is gemm.cu, which measured faster (see the end of this comment).
//
// Same arithmetic, roles and epilogues as gemm.cu (which replaces the reference's
// `moe_blockwise_grouped_mm_v2`, solution/python/moe_gemm.cu:527-654); what changes is the
// shape of a work item: (PAIR of consecutive 128-row M tiles of one expert, 128 weight rows)
// instead of (one M tile, 256 weight rows).  Per 128-wide K block the CTA still moves 48 KB
// (A: 256 rows x 128 B in one box, B: 128 rows x 128 B) and runs 512 cycles of MMA, but only
// 16 KB of that is weights, and an expert with up to 256 rows has every weight byte fetched
// by exactly one SM.  The idea it tests: where the layer is a stream of weights out of HBM,
// one SM draws ~50 GB/s from HBM at most (~27 B/clk), and with 128-row items the two M tiles
// of a 130-250-row expert run on two SMs that both pull the same 32 KB of weights per K block
// at miss latency - close to that limit at the ~1250 cycles per K block measured there.
//
// Tensor memory: accumulator (m, b) = M tile m of the pair, K-block parity b, 128 columns each
// (all 512 columns).  Issuer m (warp 1 + m) owns M tile m: four MMAs M=128, N=128 per K block
// into accumulator (m, kb & 1).  Promotion warps 4-7 serve M tile 0, warps 8-11 M tile 1; a
// thread owns one row and all 128 columns of the tile (GEMM1: 64 gate + the 64 matching up).
// When the pair's second tile belongs to another expert (odd tile count), M tile 1 is skipped:
// its issuer only releases the stage, its promotion warps sit the item out.
//
// Measured: bit-identical results, but 3.58 ms against 3.04 ms per call on the 256-expert layer at
// 4096 tokens and equal time on the compute-bound Zipf case.  The two M tiles are two
// accumulator hand-off chains of N = 128 MMAs, and a chain advances one K block per ~1000
// cycles whatever its MMA size, so two half-size chains do what one full-size chain does, and
// an expert with a single M tile gets half a chain's work per step.  The per-SM HBM draw is
// therefore not what bounds the 128-row items in the weight-streaming regime.
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
constexpr int BN = 128;                              // weight rows (GEMM1: 64 gate + 64 up) per item
constexpr int kABytes = 2 * kTileM * kBlockK;        // 32 KiB: both M tiles of the pair
constexpr int kBBytes = BN * kBlockK;                // 16 KiB
constexpr int kStageBytes = kABytes + kBBytes;       // 48 KiB
constexpr int S = 4;
constexpr int kTmemCols = 512;
constexpr int kSmemBytes = S * kStageBytes + 256 + 1024;
constexpr int kScalePrefetchDist = 6;
constexpr int CPT = BN;                              // accumulator columns per promotion thread

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
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_m256_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * kStageBytes);
  const uint32_t bar_full = smem_u32(bars);              // S: stage filled by TMA
  const uint32_t bar_empty = bar_full + 8 * S;           // S: stage released by both issuers
  const uint32_t bar_tfull = bar_empty + 8 * S;          // 4 [m][b]: accumulator written
  const uint32_t bar_tempty = bar_tfull + 32;            // 4 [m][b]: accumulator read back
  const uint32_t bar_drain = bar_tempty + 32;            // 2: each issuer's MMAs retired (teardown)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 2);
    }
    for (int b = 0; b < 4; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, kEpiWarps / 2);
    }
    mbar_init(bar_drain, 1);
    mbar_init(bar_drain + 8, 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;   // never set by others: the teardown waits ignore an abort
    fence_mbar_init();
    tma_prefetch_desc(&p.tmap_a);
    tma_prefetch_desc(&p.tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Everything above touched only this CTA's own state; global memory written by earlier
  // kernels is read from here on.
  chain_wait();
  chain_release();
  const int m_tiles = p.meta[0];
  const int n_pairs = p.meta[4];
  const int total_items = n_pairs * p.n_tiles;
  const int kblocks = p.kblocks;

  if (warp < kCtrlWarps) {
    reg_dealloc<kCtrlRegs>();
    if ((warp == 0 || warp == 3) && lane == 0) {
      // ------------------------------ TMA producers (alternate K blocks) ------------------------------
      const uint32_t pme = warp == 0 ? 0u : 1u;
      uint32_t it = 0;
      bool alive = true;
      for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
        const int m_tile0 = p.pair_tile[w / p.n_tiles], n_tile = w % p.n_tiles;
        const int e = p.tile_expert[m_tile0];
        // GEMM1: first row inside the gate (and up) plane of expert e; GEMM2: row of [e_local*hidden][inter]
        const int brow = MODE == 1 ? n_tile * (BN / 2) : e * p.n_per_expert + n_tile * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if ((it & 1u) != pme) continue;
          const uint32_t s = it % S, ph = (it / S) & 1u;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status, 41)) { alive = false; break; }
          const uint32_t full = bar_full + 8 * s;
          const uint32_t a_dst = smem_base + s * kStageBytes;
          mbar_arrive_expect_tx(full, kStageBytes);
          // 256 packed rows in one box (when the pair's second tile is another expert's, its rows are loaded and ignored)
          tma_load_2d(a_dst, &p.tmap_a, kb * kBlockK, m_tile0 * kTileM, full);
          if (MODE == 1) tma_load_3d(a_dst + kABytes, &p.tmap_b, kb * kBlockK, brow, 2 * e, full);
          else tma_load_2d(a_dst + kABytes, &p.tmap_b, kb * kBlockK, brow, full);
        }
      }
      // Copies still in flight must land before the CTA's shared memory is released.
      const uint32_t first = it > (uint32_t)S ? it - S : 0u;
      for (uint32_t j = first; j < it; ++j)
        if ((j & 1u) == pme) (void)mbar_wait(bar_full + 8 * (j % S), (j / S) & 1u, abort_flag + 1, p.status, 46);
    } else if ((warp == 1 || warp == 2) && lane == 0) {
      // ------------------------------ MMA issuers (one per M tile of the pair) ------------------------------
      constexpr uint32_t idesc = make_idesc_e4m3(kTileM, BN);
      const uint32_t m = (uint32_t)(warp - 1);
      uint32_t it = 0;      // K blocks of the CTA (stage ring)
      uint32_t jt = 0;      // K blocks this M tile really ran (accumulator ring)
      bool alive = true;
      for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
        const int m_tile0 = p.pair_tile[w / p.n_tiles];
        const bool valid = m == 0 || (m_tile0 + 1 < m_tiles && p.tile_expert[m_tile0 + 1] == p.tile_expert[m_tile0]);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % S, ph = (it / S) & 1u;
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 43)) { alive = false; break; }
          if (!valid) {
            mbar_arrive(bar_empty + 8 * s);   // nothing of this thread reads the stage
            continue;
          }
          const uint32_t b = jt & 1u, bph = (jt >> 1) & 1u;
          if (!mbar_wait(bar_tempty + 8 * (2 * m + b), bph ^ 1u, abort_flag, p.status, 42)) { alive = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * kStageBytes;
          tc_mma_f8_kblock(tmem_base + b * 256 + m * BN, kmajor_sw128_desc_lo(a_addr + m * (kTileM * kBlockK)),
                           kmajor_sw128_desc_lo(a_addr + kABytes), kKmajorSw128DescHi, idesc);
          tc_commit(bar_empty + 8 * s);
          tc_commit(bar_tfull + 8 * (2 * m + b));
          ++jt;
        }
      }
      // All MMAs must retire before TMEM is freed.
      tc_commit(bar_drain + 8 * m);
      (void)mbar_wait(bar_drain + 8 * m, 0u, abort_flag + 1, p.status, 45);
    }
  } else {
    // ------------------------------ promotion + epilogue ------------------------------
    reg_alloc<kEpiRegs>();
    const int ew = warp - kCtrlWarps;
    const int q = warp & 3;        // TMEM lane quarter this warp may read
    const int m = ew >> 2;         // which M tile of the pair
    uint32_t jt = 0;
    bool alive = true;
    const int nblk_per_expert = p.n_per_expert / kBlockK;
    for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
      const int m_tile0 = p.pair_tile[w / p.n_tiles], n_tile = w % p.n_tiles;
      const int e = p.tile_expert[m_tile0];
      if (m == 1 && !(m_tile0 + 1 < m_tiles && p.tile_expert[m_tile0 + 1] == e)) continue;
      const int row = (m_tile0 + m) * kTileM + q * 32 + lane;
      const int tok = p.row_token[row];
      float2 acc[CPT / 2];
#pragma unroll
      for (int j = 0; j < CPT / 2; ++j) acc[j] = make_float2(0.f, 0.f);

      const float* sa_ptr = nullptr;
      const float* sb0_ptr;
      const float* sb1_ptr = nullptr;
      if (MODE == 1) {
        sa_ptr = p.a_scale + row;
        const int gcol0 = n_tile * (BN / 2);          // first gate row of this tile
        sb0_ptr = p.b_scale + ((size_t)e * nblk_per_expert + gcol0 / kBlockK) * kblocks;
        sb1_ptr = p.b_scale + ((size_t)e * nblk_per_expert + (p.inter + gcol0) / kBlockK) * kblocks;
#pragma unroll 1
        for (int kb = 4; kb < 4 + kScalePrefetchDist && kb < kblocks; ++kb) prefetch_l2(sa_ptr + (size_t)kb * p.m_cap);
      } else {
        sb0_ptr = p.b_scale + ((size_t)e * nblk_per_expert + (n_tile * BN) / kBlockK) * kblocks;
      }
      constexpr int kScaleAhead = 3;
      float sa_r[kScaleAhead + 1], sb0_r[kScaleAhead + 1], sb1_r[kScaleAhead + 1];
#pragma unroll
      for (int i = 0; i <= kScaleAhead; ++i) {
        const bool in = i < kblocks;
        sa_r[i] = (MODE == 1 && in) ? sa_ptr[(size_t)i * p.m_cap] : 1.f;
        sb0_r[i] = in ? sb0_ptr[i] : 0.f;
        sb1_r[i] = (MODE == 1 && in) ? sb1_ptr[i] : 0.f;
      }

      for (int kb = 0; kb < kblocks; ++kb, ++jt) {
        const uint32_t b = jt & 1u, bph = (jt >> 1) & 1u;
        const uint32_t mb = 2 * m + b;
        const float sc0 = sa_r[0] * sb0_r[0];
        const float sc1 = sa_r[0] * sb1_r[0];
#pragma unroll
        for (int i = 0; i < kScaleAhead; ++i) {
          sa_r[i] = sa_r[i + 1];
          sb0_r[i] = sb0_r[i + 1];
          sb1_r[i] = sb1_r[i + 1];
        }
        {
          const int nk = kb + kScaleAhead + 1;
          if (nk < kblocks) {
            if (MODE == 1) {
              sa_r[kScaleAhead] = sa_ptr[(size_t)nk * p.m_cap];
              sb1_r[kScaleAhead] = sb1_ptr[nk];
              if (nk + kScalePrefetchDist < kblocks) prefetch_l2(sa_ptr + (size_t)(nk + kScalePrefetchDist) * p.m_cap);
            }
            sb0_r[kScaleAhead] = sb0_ptr[nk];
          }
        }
        bool ok = mbar_wait(bar_tfull + 8 * mb, bph, abort_flag, p.status, 44);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + b * 256 + m * BN;
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(t_row, ra);
        tmem_ld_32x32(t_row + 32, rb);
        tmem_ld_wait_on(ra, rb);
        fma_chunk(acc, ra, sc0);
        tmem_ld_32x32(t_row + 64, ra);
        fma_chunk(acc + 16, rb, sc0);
        tmem_ld_32x32(t_row + 96, rb);
        tmem_ld_wait_on(ra, rb);
        // The accumulator is free as soon as its last column sits in registers.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * mb);
        fma_chunk(acc + 32, ra, MODE == 1 ? sc1 : sc0);
        fma_chunk(acc + 48, rb, MODE == 1 ? sc1 : sc0);
      }
      if (!alive) break;

      if (tok >= 0) {
        if (MODE == 1) {
          // acc pairs [0 .. CPT/4) = gate columns, [CPT/4 .. CPT/2) = matching up columns
          constexpr int HP = CPT / 4;
          __half* dst = p.act + (size_t)row * p.inter + n_tile * (BN / 2);
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < HP; j += 8) {
            uint32_t wv[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              __half2 hh = __floats2half2_rn(silu_mul(acc[j + t].x, acc[HP + j + t].x),
                                             silu_mul(acc[j + t].y, acc[HP + j + t].y));
              float2 back = __half22float2(hh);
              amax = fmaxf(amax, fmaxf(fabsf(back.x), fabsf(back.y)));
              wv[t] = *reinterpret_cast<uint32_t*>(&hh);
            }
            st_global_v8(dst + 2 * j, wv);
          }
          atomicMax(p.row_amax + row, __float_as_uint(amax));
        } else {
          const float rs = p.row_scale[row] * p.row_weight[row];
          __nv_bfloat16* dst = p.y + (size_t)row * p.hidden + n_tile * BN;
#pragma unroll
          for (int j = 0; j < CPT / 2; j += 8) {
            uint32_t wv[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              __nv_bfloat162 v = __floats2bfloat162_rn(acc[j + t].x * rs, acc[j + t].y * rs);
              wv[t] = *reinterpret_cast<uint32_t*>(&v);
            }
            st_global_v8(dst + 2 * j, wv);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

template <int MODE>
cudaError_t launch_one(const GemmParams& p, int num_sms, cudaStream_t stream) {
  return launch_chained(grouped_gemm_m256_kernel<MODE>, dim3(num_sms), dim3(kThreads), kSmemBytes, stream, p);
}

}  // namespace

cudaError_t configure_grouped_gemm_m256() {
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_m256_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(grouped_gemm_m256_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

cudaError_t launch_grouped_gemm_m256(int mode, const GemmParams& p, int num_sms, cudaStream_t stream) {
  return mode == 1 ? launch_one<1>(p, num_sms, stream) : launch_one<2>(p, num_sms, stream);
}

}  // namespace b200moe
