// Persistent grouped FP8 GEMMs on tcgen05 tensor cores with exact fp32 block scales.
//
// Replaces the reference's CUTLASS grouped GEMM `moe_blockwise_grouped_mm_v2`
// (solution/python/moe_gemm.cu:310-340, 418-654) plus, in the epilogues, the front half
// of its `swiglu_fp8_requant_kernel` (solution/python/moe_fused.cu:131-196) and the
// per-row scaling of its combine kernels (moe_fused.cu:346-393, 490-517).
//
// One CTA per SM walks work items (M tile of 128 packed rows, N tile of BN weight rows).
// Per 128-wide K block (= one fp32 scale block, = one 128-byte swizzled TMA row):
//   warps 0, 3  TMA producers (one lane each, alternate K blocks): A box 128x128 B and one B box BNx128 B into a smem ring
//   warps 1, 2  (one lane each, alternate K blocks) issue 4 tcgen05.mma (K=32 each) into one of two TMEM accumulators, starting
//               from zero, so each accumulator holds the raw e4m3 dot product of one K block
//   warps 4-11  read that accumulator back (tcgen05.ld, two loads in flight) and fold it into
//               fp32 registers with packed FMAs: acc += (a_scale * b_scale) * partial.  The
//               block scales are arbitrary fp32 numbers, so they cannot ride on the MMA.
// The control warpgroup (warps 0-3) gives registers back (setmaxnreg) so that the eight
// promotion warps can hold a 128x256 fp32 tile (128 accumulators per thread) without spills.
// GEMM1 pairs gate rows [n, n+BN/2) with up rows [inter+n, ...) in one tile, so the epilogue
// computes g*silu(u) in registers, stores fp16 activations and the row maximum.
// GEMM2's epilogue multiplies by (row requant scale * routing weight) and stores the row as
// bf16; the combine kernel sums a token's rows.
//
// Every wait is bounded (see mbar_wait); on a timeout the CTA drains and frees its TMEM.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.cuh"

namespace b200moe {

namespace {

constexpr int kCtrlWarps = 4;
constexpr int kEpiWarps = 8;
constexpr int kGemmThreads = 32 * (kCtrlWarps + kEpiWarps);   // 384: three warpgroups
constexpr int kCtrlRegs = 56;
constexpr int kEpiRegs = 224;   // 128*56 + 256*224 = 64512 = 384 threads * 168 registers at launch
constexpr int kABytes = kTileM * kBlockK;   // 16 KiB
constexpr int kScalePrefetchDist = 6;       // K blocks ahead for the activation-scale L2 prefetch

template <int BN> struct TileCfg {
  static constexpr int kBBytes = BN * kBlockK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;   // + alignment slack
  static constexpr int kColsPerThread = BN / 2;
  static constexpr int kChunks = kColsPerThread / 32;
};

__device__ __forceinline__ float silu_mul(float g, float u) {
  float sig = __fdividef(1.0f, 1.0f + __expf(-u));   // approximate reciprocal: 2 ulp, far below e4m3 resolution
  return g * (u * sig);
}

// acc[16 pairs] += scale * r[32] with packed fp32 FMAs
__device__ __forceinline__ void fma_chunk(float2* acc, const uint32_t (&r)[32], float sc) {
  const float2 s2 = make_float2(sc, sc);
#pragma unroll
  for (int j = 0; j < 16; ++j)
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), s2, acc[j]);
}

// First TMEM column (inside the tile) and scale selector of chunk c of a thread in column half h.
template <int MODE, int BN>
__device__ __forceinline__ uint32_t chunk_col(int c, int h) {
  constexpr int CH = TileCfg<BN>::kChunks;
  if (MODE == 1) {
    const bool up = c >= CH / 2;
    return (up ? BN / 2 : 0) + h * (BN / 4) + (up ? c - CH / 2 : c) * 32;
  }
  return h * (BN / 2) + c * 32;
}

template <int MODE, int BN, bool PROF>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = TileCfg<BN>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes);
  const uint32_t bar_full = smem_u32(bars);              // S barriers: stage filled by TMA
  const uint32_t bar_empty = bar_full + 8 * S;           // S barriers: stage consumed by the MMAs
  const uint32_t bar_tfull = bar_empty + 8 * S;          // 2 barriers: accumulator written
  const uint32_t bar_tempty = bar_tfull + 16;            // 2 barriers: accumulator read back
  const uint32_t bar_drain = bar_tempty + 16;            // 2 barriers: each issuer's MMAs retired (teardown)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, kEpiWarps);
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
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
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
  const int total_items = m_tiles * p.n_tiles;
  const int kblocks = p.kblocks;

  if (warp < kCtrlWarps) {
    reg_dealloc<kCtrlRegs>();
    if ((warp == 0 || warp == 3) && lane == 0) {
      // ------------------------------ TMA producers (alternate K blocks) ------------------------------
      const uint32_t pme = warp == 0 ? 0u : 1u;
      uint32_t it = 0;
      bool alive = true;
      for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
        const int m_tile = w / p.n_tiles, n_tile = w % p.n_tiles;
        const int e = p.tile_expert[m_tile];
        // GEMM1: first row inside the gate (and up) plane of expert e; GEMM2: row of [e_local*hidden][inter]
        const int brow = MODE == 1 ? n_tile * (BN / 2) : e * p.n_per_expert + n_tile * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if ((it & 1u) != pme) continue;
          const uint32_t s = it % S, ph = (it / S) & 1u;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status, 1)) { alive = false; break; }
          const uint32_t full = bar_full + 8 * s;
          const uint32_t a_dst = smem_base + s * Cfg::kStageBytes;
          mbar_arrive_expect_tx(full, Cfg::kStageBytes);
          tma_load_2d(a_dst, &p.tmap_a, kb * kBlockK, m_tile * kTileM, full);
          // the whole B tile in one operation: BN/2 gate rows + BN/2 up rows (3D box over the two planes), or BN rows
          if (MODE == 1) tma_load_3d(a_dst + kABytes, &p.tmap_b, kb * kBlockK, brow, 2 * e, full);
          else tma_load_2d(a_dst + kABytes, &p.tmap_b, kb * kBlockK, brow, full);
        }
      }
      // Copies still in flight must land before the CTA's shared memory is released.
      const uint32_t first = it > (uint32_t)S ? it - S : 0u;
      for (uint32_t j = first; j < it; ++j)
        if ((j & 1u) == pme) (void)mbar_wait(bar_full + 8 * (j % S), (j / S) & 1u, abort_flag + 1, p.status, 6);
    } else if ((warp == 1 || warp == 2) && lane == 0) {
      // ------------------------------ MMA issuers ------------------------------
      // Two threads (on different SM sub-partitions) take alternate K blocks.  Issuing the
      // four MMAs and two commits of a K block costs one thread ~300 cycles whatever the
      // tile size, and its waits for operands and for a free accumulator add to that; with
      // two issuers one waits while the other issues.  Issuer i always writes accumulator i.
      constexpr uint32_t idesc = make_idesc_e4m3(kTileM, BN);
      const uint32_t me = (uint32_t)(warp - 1);
      uint32_t it = 0;
      bool alive = true;
      long long wait_epi = 0, wait_tma = 0, t_issue = 0;
      for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if ((it & 1u) != me) continue;
          const uint32_t s = it % S, ph = (it / S) & 1u;
          const uint32_t b = me, bph = (it >> 1) & 1u;
          const long long m0 = PROF ? clock64() : 0;
          // Operands first: they usually landed long ago, so only one wake-up (the free
          // accumulator) is left on the critical path.
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 3)) { alive = false; break; }
          const long long m1 = PROF ? clock64() : 0;
          if (!mbar_wait(bar_tempty + 8 * b, bph ^ 1u, abort_flag, p.status, 2)) { alive = false; break; }
          const long long m2 = PROF ? clock64() : 0;
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * Cfg::kStageBytes;
          tc_mma_f8_kblock(tmem_base + b * BN, kmajor_sw128_desc_lo(a_addr), kmajor_sw128_desc_lo(a_addr + kABytes),
                           kKmajorSw128DescHi, idesc);
          tc_commit(bar_empty + 8 * s);
          tc_commit(bar_tfull + 8 * b);
          if (PROF) {
            const long long m3 = clock64();
            wait_tma += m1 - m0;
            wait_epi += m2 - m1;
            t_issue += m3 - m2;
            if (p.trace && blockIdx.x == 0 && it < 64) {
              p.trace[it * 8 + 0] = (unsigned long long)m0;   // issuer starts waiting for operands
              p.trace[it * 8 + 1] = (unsigned long long)m1;   // operands landed seen
              p.trace[it * 8 + 2] = (unsigned long long)m2;   // accumulator free seen
              p.trace[it * 8 + 3] = (unsigned long long)m3;   // MMAs and commits issued
            }
          }
        }
      }
      // All MMAs must retire before TMEM is freed.
      tc_commit(bar_drain + 8 * me);
      (void)mbar_wait(bar_drain + 8 * me, 0u, abort_flag + 1, p.status, 5);
      if (PROF && p.prof && blockIdx.x == 0 && me == 0) {
        p.prof[7] = (unsigned long long)wait_epi;   // issuer 0 waiting for the promotion warps
        p.prof[8] = (unsigned long long)wait_tma;   // issuer 0 waiting for TMA data
        p.prof[2] = (unsigned long long)t_issue;    // issuer 0 issuing MMAs and commits
      }
    }
  } else {
    // ------------------------------ promotion + epilogue ------------------------------
    reg_alloc<kEpiRegs>();
    const int ew = warp - kCtrlWarps;
    const int q = warp & 3;        // TMEM lane quarter this warp may read
    const int h = ew >> 2;         // which half of the tile's columns
    constexpr int CPT = Cfg::kColsPerThread;
    constexpr int CH = Cfg::kChunks;
    static_assert(CH == 2 || CH == 4, "two or four 32-column chunks per thread");
    uint32_t it = 0;
    bool alive = true;
    const bool prof_me = PROF && p.prof && blockIdx.x == 0 && ew == 0 && lane == 0;
    const long long t_begin = PROF ? clock64() : 0;
    long long t_wait = 0, t_promote = 0, t_epi = 0;
    const int nblk_per_expert = p.n_per_expert / kBlockK;
    for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
      const int m_tile = w / p.n_tiles, n_tile = w % p.n_tiles;
      const int e = p.tile_expert[m_tile];
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
        const int gcol0 = n_tile * (BN / 2) + h * (BN / 4);          // first gate row of this thread
        sb0_ptr = p.b_scale + ((size_t)e * nblk_per_expert + gcol0 / kBlockK) * kblocks;
        sb1_ptr = p.b_scale + ((size_t)e * nblk_per_expert + (p.inter + gcol0) / kBlockK) * kblocks;
#pragma unroll 1
        for (int kb = 4; kb < 4 + kScalePrefetchDist && kb < kblocks; ++kb) prefetch_l2(sa_ptr + (size_t)kb * p.m_cap);
      } else {
        const int col0 = n_tile * BN + h * (BN / 2);
        sb0_ptr = p.b_scale + ((size_t)e * nblk_per_expert + col0 / kBlockK) * kblocks;
      }
      // Scales of K blocks kb .. kb+3 ride in registers: a load issued only one K block ahead
      // is still in flight when it is needed (L2 under the weight stream answers in ~1 us).
      constexpr int kScaleAhead = 3;
      float sa_r[kScaleAhead + 1], sb0_r[kScaleAhead + 1], sb1_r[kScaleAhead + 1];
#pragma unroll
      for (int i = 0; i <= kScaleAhead; ++i) {
        const bool in = i < kblocks;
        sa_r[i] = (MODE == 1 && in) ? sa_ptr[(size_t)i * p.m_cap] : 1.f;
        sb0_r[i] = in ? sb0_ptr[i] : 0.f;
        sb1_r[i] = (MODE == 1 && in) ? sb1_ptr[i] : 0.f;
      }

      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const uint32_t b = it & 1u, bph = (it >> 1) & 1u;
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
        const long long c0 = PROF ? clock64() : 0;
        bool ok = mbar_wait(bar_tfull + 8 * b, bph, abort_flag, p.status, 4);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
        const long long c1 = PROF ? clock64() : 0;
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + b * BN;
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(t_row + chunk_col<MODE, BN>(0, h), ra);
        tmem_ld_32x32(t_row + chunk_col<MODE, BN>(1, h), rb);
        tmem_ld_wait_on(ra, rb);
        const long long c1a = PROF ? clock64() : 0;
        // The accumulator is free as soon as its last column sits in registers: signal the MMA
        // thread before the remaining FMAs, which then overlap the next K block's MMAs.
        long long c1b = c1a;
        if constexpr (CH == 2) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
          fma_chunk(acc, ra, sc0);
          fma_chunk(acc + 16, rb, MODE == 1 ? sc1 : sc0);
        } else {
          fma_chunk(acc, ra, sc0);
          tmem_ld_32x32(t_row + chunk_col<MODE, BN>(2, h), ra);
          fma_chunk(acc + 16, rb, sc0);
          tmem_ld_32x32(t_row + chunk_col<MODE, BN>(3, h), rb);
          tmem_ld_wait_on(ra, rb);
          c1b = PROF ? clock64() : 0;
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
          fma_chunk(acc + 32, ra, MODE == 1 ? sc1 : sc0);
          fma_chunk(acc + 48, rb, MODE == 1 ? sc1 : sc0);
        }
        if (PROF) {
          const long long c2 = clock64();
          t_wait += c1 - c0;
          t_promote += c2 - c1;
          if (prof_me && p.trace && it < 64) {
            p.trace[it * 8 + 4] = (unsigned long long)c1;    // accumulator ready seen by promotion warp 0
            p.trace[it * 8 + 5] = (unsigned long long)c1a;   // first two chunks in registers
            p.trace[it * 8 + 6] = (unsigned long long)c1b;   // last chunk in registers: accumulator released
            p.trace[it * 8 + 7] = (unsigned long long)c2;    // promotion of this K block done
          }
        }
      }
      if (!alive) break;
      const long long te0 = PROF ? clock64() : 0;

      if (tok >= 0) {
        if (MODE == 1) {
          // acc pairs [0 .. CPT/4) = gate columns, [CPT/4 .. CPT/2) = matching up columns
          constexpr int HP = CPT / 4;
          // fp16 keeps 11 significant bits, three more than the e4m3 codes made from it need;
          // the row maximum is taken over the rounded values so that it is attained exactly.
          __half* dst = p.act + (size_t)row * p.inter + n_tile * (BN / 2) + h * (BN / 4);
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < HP; j += 8) {
            uint32_t w[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              __half2 hh = __floats2half2_rn(silu_mul(acc[j + t].x, acc[HP + j + t].x),
                                             silu_mul(acc[j + t].y, acc[HP + j + t].y));
              float2 back = __half22float2(hh);
              amax = fmaxf(amax, fmaxf(fabsf(back.x), fabsf(back.y)));
              w[t] = *reinterpret_cast<uint32_t*>(&hh);
            }
            st_global_v8(dst + 2 * j, w);
          }
          atomicMax(p.row_amax + row, __float_as_uint(amax));
        } else {
          const float rs = p.row_scale[row] * p.row_weight[row];
          __nv_bfloat16* dst = p.y + (size_t)row * p.hidden + n_tile * BN + h * (BN / 2);
#pragma unroll
          for (int j = 0; j < CPT / 2; j += 8) {
            uint32_t w[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              __nv_bfloat162 v = __floats2bfloat162_rn(acc[j + t].x * rs, acc[j + t].y * rs);
              w[t] = *reinterpret_cast<uint32_t*>(&v);
            }
            st_global_v8(dst + 2 * j, w);
          }
        }
      }
      if (PROF) t_epi += clock64() - te0;
    }
    if (prof_me) {
      p.prof[0] = (unsigned long long)t_wait;                  // waiting for an accumulator
      p.prof[1] = (unsigned long long)t_promote;               // TMEM read-back + FMAs
      p.prof[3] = (unsigned long long)it;                      // K blocks
      p.prof[4] = (unsigned long long)(clock64() - t_begin);   // whole role
      p.prof[5] = (unsigned long long)t_epi;                   // per-tile epilogues
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int MODE, int BN>
cudaError_t launch_one(const GemmParams& p, int num_sms, cudaStream_t stream) {
  if (p.prof)
    return launch_chained(grouped_gemm_kernel<MODE, BN, true>, dim3(num_sms), dim3(kGemmThreads),
                          TileCfg<BN>::kSmemBytes, stream, p);
  else
    return launch_chained(grouped_gemm_kernel<MODE, BN, false>, dim3(num_sms), dim3(kGemmThreads),
                          TileCfg<BN>::kSmemBytes, stream, p);
}

template <int MODE, int BN>
cudaError_t configure_one() {
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<MODE, BN, true>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, TileCfg<BN>::kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(grouped_gemm_kernel<MODE, BN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              TileCfg<BN>::kSmemBytes);
}

}  // namespace

cudaError_t configure_grouped_gemm() {
  cudaError_t e;
  if ((e = configure_one<1, 128>()) != cudaSuccess) return e;
  if ((e = configure_one<1, 256>()) != cudaSuccess) return e;
  if ((e = configure_one<2, 128>()) != cudaSuccess) return e;
  if ((e = configure_one<2, 256>()) != cudaSuccess) return e;
  return cudaSuccess;
}

cudaError_t launch_grouped_gemm(int mode, int bn, const GemmParams& p, int num_sms, cudaStream_t stream) {
  if (mode == 1) return bn == 128 ? launch_one<1, 128>(p, num_sms, stream) : launch_one<1, 256>(p, num_sms, stream);
  return bn == 128 ? launch_one<2, 128>(p, num_sms, stream) : launch_one<2, 256>(p, num_sms, stream);
}

}  // namespace b200moe
