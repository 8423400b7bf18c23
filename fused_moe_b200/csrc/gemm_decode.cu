// Decode-size grouped FP8 GEMMs (at most 64 tokens per call): operands swapped.
//
// With a handful of rows per expert the layer is a stream of expert weights through the SMs
// (44 MB per active expert), so the tile is turned around: the 128 MMA rows (TMEM lanes) are
// 128 WEIGHT rows and the MMA's N dimension is the expert's token rows (16 or 64, all of
// them, since an expert cannot hold more rows than the call has tokens).  Per 128-wide K
// block a CTA then moves 16 KB of weights and only NT x 128 B of activations, the MMA and the
// read-back are a few dozen cycles, four small accumulators rotate in tensor memory, and
// 8-10 stages of weights are in flight per SM.  Arithmetic is the one of gemm.cu (which
// replaces the reference's `moe_blockwise_grouped_mm_v2`, solution/python/moe_gemm.cu:527-654,
// whose own small-batch configuration also swaps A and B, moe_gemm.cu:614-648): raw e4m3 dot
// product per K block, promoted in fp32 registers with the fp32 block scales.
//
// Weights arrive as ONE TMA box per K block (GEMM1: a 3D box over the expert's gate and up
// planes), issued by four producer threads in turn: a box costs its issuing thread a few hundred
// cycles whatever its size.  When a call has fewer (expert tile, slab) items than half the SMs,
// the K range of an item is split over 2 or 4 CTAs (one SM draws ~50 GB/s from HBM at most):
// every piece leaves fp32 partial sums in scratch and the CTA that arrives last adds them in
// piece order and runs the epilogue, so results stay run-to-run identical.
//
// Work item = (expert tile, slab of 128 weight rows).  GEMM1's slab is 64 gate rows plus the
// 64 matching up rows, so lanes 0-63 hold g and lanes 64-127 hold u of the same columns; the
// up warps hand u over through shared memory and the gate warps write g*silu(u) (fp16) and
// the row maxima.  GEMM2's slab is 128 output columns; its epilogue writes bf16(acc * row
// scale * routing weight).  Stores are token-major: a warp writes 32 consecutive columns of
// one token row per instruction.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.cuh"

namespace b200moe {

namespace {

constexpr int kThreads = 320;            // warps 0-3 control (0 and 3: TMA, 1 and 2: MMA), warps 4-7 promotion, warps 8-9: TMA
constexpr int kProducers = 4;            // a TMA box costs its issuing thread a few hundred cycles: four threads take turns
constexpr int kSlabRows = 128;
constexpr int kWBytes = kSlabRows * kBlockK;   // 16 KiB of weights per stage
constexpr int kRing = 4;                 // accumulators in tensor memory

template <int NT> struct DCfg {
  static constexpr int kTokBytes = NT * kBlockK;
  static constexpr int kStageBytes = kWBytes + kTokBytes;
  static constexpr int kStages = (NT <= 16) ? 9 : 6;
  static constexpr int kTmemCols = (kRing * NT < 32) ? 32 : kRing * NT;
  static constexpr int kXchBytes = 64 * NT * 4;                 // u values of 64 up rows
  static constexpr int kMaxKBlocks = 56;                        // hidden <= 7168 for the scale panels
  static constexpr int kPanelBytes = kMaxKBlocks * NT * 4 + 256;   // one promotion warp's copy of the token scales + weight scales
  static constexpr int kSmemBytes = kStages * kStageBytes + kXchBytes + 4 * kPanelBytes + 512 + 1024;
};

__device__ __forceinline__ float silu_mul_d(float g, float u) {
  float sig = __fdividef(1.0f, 1.0f + __expf(-u));
  // The activations are stored as fp16: a product beyond its range saturates (the row then requantises to
  // the largest e4m3 code) instead of becoming inf and, through an infinite row scale, NaN.
  return fminf(fmaxf(g * (u * sig), -65504.0f), 65504.0f);
}

// 32 lanes x 16 consecutive fp32 columns
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait_on16(uint32_t (&a)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : B200MOE_RW8(a, 0), B200MOE_RW8(a, 8) : : "memory");
}

template <int MODE, int NT, bool PROF>
__global__ void __launch_bounds__(kThreads, 1)
decode_gemm_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = DCfg<NT>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  float* xch = reinterpret_cast<float*>(smem + S * Cfg::kStageBytes);               // [64][NT]
  float* panels = reinterpret_cast<float*>(smem + S * Cfg::kStageBytes + Cfg::kXchBytes);   // [4 warps][kblocks][NT]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes + Cfg::kXchBytes + 4 * Cfg::kPanelBytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * S;
  const uint32_t bar_tfull = bar_empty + 8 * S;
  const uint32_t bar_tempty = bar_tfull + 8 * kRing;
  const uint32_t bar_drain = bar_tempty + 8 * kRing;
  const uint32_t bar_xready = bar_drain + 16;    // 2 barriers: u of an up warp is in shared memory
  const uint32_t bar_xfree = bar_xready + 16;    // 2 barriers: its gate warp has read it
  const uint32_t bar_split = bar_xfree + 16;     // 2 barriers (split K): partial sums written; arrival order known
  const uint32_t bar_rq = bar_split + 16;        // 2 barriers (GEMM1): this item's activations stored; outcome of the arrival count known
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 2 * kRing + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* split_flag = reinterpret_cast<volatile int*>(tmem_slot + 3);
  volatile int* rq_flag = reinterpret_cast<volatile int*>(tmem_slot + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < kRing; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 4);
    }
    mbar_init(bar_drain, 1);
    mbar_init(bar_drain + 8, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_xready + 8 * i, 1);
      mbar_init(bar_xfree + 8 * i, 1);
    }
    mbar_init(bar_split, 4);
    mbar_init(bar_split + 8, 1);
    mbar_init(bar_rq, 4);
    mbar_init(bar_rq + 8, 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;
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
  if (MODE == 1 && p.zero_tokens > 0) {
    // no gather pass ran: the output rows that GEMM2 adds into are zeroed here, a few stores per CTA
    const int vec_per_row = p.hidden / 8;   // 8 bf16 = 16 bytes
    const long long total = (long long)p.zero_tokens * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const long long t = i / vec_per_row;
      reinterpret_cast<uint4*>(p.out + t * p.out_stride)[i - t * vec_per_row] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  const int m_tiles = p.meta[0];
  const int tiles = m_tiles * p.n_tiles;
  const int kblocks = p.kblocks;
  // Split K: with few active experts fewer (expert tile, slab) items exist than SMs, and one SM
  // pulls at most ~50 GB/s from HBM, so the K range of an item is cut into KS pieces on KS CTAs.
  // Each piece leaves its fp32 partial sums in scratch; the CTA that arrives last on the item's
  // counter adds the pieces in piece order (deterministic) and runs the epilogue.
  int KS = 1;
  if (NT == 16 && p.splitk_scratch != nullptr && tiles > 0 && tiles <= kSplitKSlots) {
    const int want = (int)gridDim.x / tiles;
    if (want >= 4 && kblocks % 4 == 0 && kblocks / 4 >= 8) KS = 4;
    else if (want >= 2 && kblocks % 2 == 0 && kblocks / 2 >= 8) KS = 2;
  }
  const int kbs = kblocks / KS;          // K blocks per piece
  const int total_items = tiles * KS;    // item w = (tile w / KS, piece w % KS)

  if (warp == 0 || warp == 3 || warp >= 8) {
    if (lane == 0) {
      // ------------------------------ TMA producers (every fourth K block each) ------------------------------
      const uint32_t pme = warp == 0 ? 0u : (warp == 3 ? 1u : (uint32_t)(warp - 6));
      uint32_t it = 0;
      bool alive = true;
      long long pw = 0, pi = 0;
      const long long pbegin = PROF ? clock64() : 0;
      for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
        const int tile = w / KS, ks = w % KS;
        const int m_tile = tile / p.n_tiles, slab = tile % p.n_tiles;
        const int e = p.tile_expert[m_tile];
        // GEMM1: 64 gate rows + the matching 64 up rows of expert e, one 3D box over its two planes;
        // GEMM2: 128 consecutive rows of [e_local*hidden][inter]
        const int wrow = MODE == 1 ? slab * 64 : e * p.n_per_expert + slab * kSlabRows;
        // Without a gather pass (GEMM1 of a call that was routed and placed by the one-block front kernel) the
        // expert's token rows are fetched where the caller keeps them: one one-row box per row and K block (an
        // expert has one or two rows at these sizes); rows past the expert's count keep whatever the stage held,
        // as padding rows do, and their columns are never stored.
        const bool direct = MODE == 1 && NT == 16 && p.direct_a != 0;
        int cnt = 0;
        int toks[16];
        if (direct) {
          cnt = min(p.expert_count[e], 16);
#pragma unroll
          for (int j = 0; j < 16; ++j) toks[j] = j < cnt ? p.row_token[m_tile * kTileM + j] : 0;
        }
        for (int kb = ks * kbs; kb < (ks + 1) * kbs; ++kb, ++it) {
          if ((it % kProducers) != pme) continue;
          const uint32_t s = it % S, ph = (it / S) & 1u;
          const long long q0 = PROF ? clock64() : 0;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status, 21)) { alive = false; break; }
          const long long q1 = PROF ? clock64() : 0;
          const uint32_t full = bar_full + 8 * s;
          const uint32_t w_dst = smem_base + s * Cfg::kStageBytes;
          mbar_arrive_expect_tx(full, direct ? kWBytes + cnt * kBlockK : Cfg::kStageBytes);
          if (MODE == 1) tma_load_3d(w_dst, &p.tmap_b, kb * kBlockK, wrow, 2 * e, full);
          else tma_load_2d(w_dst, &p.tmap_b, kb * kBlockK, wrow, full);
          if (direct) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < cnt) tma_load_2d(w_dst + kWBytes + j * kBlockK, &p.tmap_a, kb * kBlockK, toks[j], full);
          } else {
            tma_load_2d(w_dst + kWBytes, &p.tmap_a, kb * kBlockK, m_tile * kTileM, full);
          }
          if (PROF) { pw += q1 - q0; pi += clock64() - q1; }
        }
      }
      if (PROF && p.prof && blockIdx.x == 0 && pme == 0) {
        p.prof[0] = (unsigned long long)pw;                     // producer 0: waiting for a free stage
        p.prof[1] = (unsigned long long)pi;                     // producer 0: expect_tx + two TMA issues
        p.prof[2] = (unsigned long long)(clock64() - pbegin);   // producer 0: whole loop
        p.prof[3] = (unsigned long long)it;                     // K blocks of CTA 0
      }
      const uint32_t first = it > (uint32_t)S ? it - S : 0u;
      for (uint32_t j = first; j < it; ++j)
        if ((j % kProducers) == pme) (void)mbar_wait(bar_full + 8 * (j % S), (j / S) & 1u, abort_flag + 1, p.status, 26);
    }
  } else if (warp == 1 || warp == 2) {
    if (lane == 0) {
      // ------------------------------ MMA issuers (alternate K blocks) ------------------------------
      constexpr uint32_t idesc = make_idesc_e4m3(kSlabRows, NT);
      const uint32_t me = (uint32_t)(warp - 1);
      uint32_t it = 0;
      bool alive = true;
      long long iw0 = 0, iw1 = 0, ii = 0;
      for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
        for (int kb = 0; kb < kbs; ++kb, ++it) {
          if ((it & 1u) != me) continue;
          const uint32_t s = it % S, ph = (it / S) & 1u;
          const uint32_t b = it % kRing, bph = (it / kRing) & 1u;
          const long long q0 = PROF ? clock64() : 0;
          if (!mbar_wait(bar_tempty + 8 * b, bph ^ 1u, abort_flag, p.status, 22)) { alive = false; break; }
          const long long q1 = PROF ? clock64() : 0;
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 23)) { alive = false; break; }
          const long long q2 = PROF ? clock64() : 0;
          tc_fence_after();
          const uint32_t w_addr = smem_base + s * Cfg::kStageBytes;
          tc_mma_f8_kblock(tmem_base + b * NT, kmajor_sw128_desc_lo(w_addr), kmajor_sw128_desc_lo(w_addr + kWBytes),
                           kKmajorSw128DescHi, idesc);
          tc_commit(bar_empty + 8 * s);
          tc_commit(bar_tfull + 8 * b);
          if (PROF) { iw0 += q1 - q0; iw1 += q2 - q1; ii += clock64() - q2; }
        }
      }
      tc_commit(bar_drain + 8 * me);
      (void)mbar_wait(bar_drain + 8 * me, 0u, abort_flag + 1, p.status, 25);
      if (PROF && p.prof && blockIdx.x == 0 && me == 0) {
        p.prof[4] = (unsigned long long)iw0;   // issuer 0: waiting for a free accumulator
        p.prof[5] = (unsigned long long)iw1;   // issuer 0: waiting for operands
        p.prof[6] = (unsigned long long)ii;    // issuer 0: MMAs + commits
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------ promotion + epilogue ------------------------------
    const int q = warp & 3;                 // TMEM lane quarter: weight rows 32q .. 32q+31 of the slab
    uint32_t it = 0, xi = 0, si = 0, ri = 0;
    bool alive = true;
    long long ew_wait = 0;
    const long long ebegin = PROF ? clock64() : 0;
    const int nblk_per_expert = p.n_per_expert / kBlockK;
    for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
      const int tile = w / KS, ks = w % KS;
      const int m_tile = tile / p.n_tiles, slab = tile % p.n_tiles;
      const int e = p.tile_expert[m_tile];
      const int row0 = m_tile * kTileM;     // the expert's first packed row; its rows are row0 .. row0+cnt-1
      float acc[NT];
#pragma unroll
      for (int j = 0; j < NT; ++j) acc[j] = 0.f;

      // weight-scale block of this warp's rows
      int wblock;
      if (MODE == 1) wblock = (q < 2) ? (slab * 64) / kBlockK : (p.inter + slab * 64) / kBlockK;
      else wblock = slab;
      const float* sb_ptr = p.b_scale + ((size_t)e * nblk_per_expert + wblock) * kblocks;
      const float* sa_ptr = MODE == 1 ? p.a_scale + row0 : nullptr;   // [kb][m_cap], NT consecutive rows
      // GEMM1: the token scales of the whole item ([kblocks][NT] floats) are copied once into
      // this warp's own panel in shared memory; per K block they are then a broadcast read
      // instead of a global load whose latency would bound every iteration.
      float* panel = panels + (size_t)(warp - 4) * (Cfg::kPanelBytes / 4);
      float* panel_sb = panel + Cfg::kMaxKBlocks * NT;     // this warp's weight scales, one per K block
      __syncwarp();
      for (int i = lane; i < kblocks; i += 32) panel_sb[i] = sb_ptr[i];
      if (MODE == 1 && NT == 16 && p.direct_a) {
        // the token scales where the caller keeps them: lane j < 16 knows row j's token
        const int n_rows = min(p.expert_count[e], NT);
        const int my_tok = lane < n_rows ? p.row_token[row0 + lane] : -1;
        const int tj = __shfl_sync(0xffffffffu, my_tok, lane & (NT - 1));   // entry i belongs to row i % 16 = lane % 16
        for (int i = lane; i < kblocks * NT; i += 32) {
          const int kb = i / NT;
          panel[i] = tj >= 0 ? p.hscale[(size_t)tj * p.hs_stride_t + (size_t)kb * p.hs_stride_kb] : 0.f;
        }
      } else if (MODE == 1) {
        for (int i = lane; i < kblocks * (NT / 4); i += 32) {
          const int kb = i / (NT / 4), v = i % (NT / 4);
          reinterpret_cast<float4*>(panel)[i] = reinterpret_cast<const float4*>(sa_ptr + (size_t)kb * p.m_cap)[v];
        }
      }
      __syncwarp();

      for (int kb = ks * kbs; kb < (ks + 1) * kbs; ++kb, ++it) {
        const uint32_t b = it % kRing, bph = (it / kRing) & 1u;
        float4 sa_c[NT / 4];
        if (MODE == 1) {
#pragma unroll
          for (int j = 0; j < NT / 4; ++j) sa_c[j] = reinterpret_cast<const float4*>(panel + kb * NT)[j];
        }
        const float sb_cur = panel_sb[kb];
        const long long e0 = PROF ? clock64() : 0;
        bool ok = mbar_wait(bar_tfull + 8 * b, bph, abort_flag, p.status, 24);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
        if (PROF) ew_wait += clock64() - e0;
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + b * NT;
        if constexpr (NT == 16) {
          uint32_t r[16];
          tmem_ld_32x16(t_row, r);
          tmem_ld_wait_on16(r);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float sc = MODE == 1 ? reinterpret_cast<const float*>(sa_c)[j] * sb_cur : sb_cur;
            acc[j] = fmaf(__uint_as_float(r[j]), sc, acc[j]);
          }
        } else {
          uint32_t ra[32], rb[32];
          tmem_ld_32x32(t_row, ra);
          tmem_ld_32x32(t_row + 32, rb);
          tmem_ld_wait_on(ra, rb);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float s0 = MODE == 1 ? reinterpret_cast<const float*>(sa_c)[j] * sb_cur : sb_cur;
            const float s1 = MODE == 1 ? reinterpret_cast<const float*>(sa_c)[32 + j] * sb_cur : sb_cur;
            acc[j] = fmaf(__uint_as_float(ra[j]), s0, acc[j]);
            acc[32 + j] = fmaf(__uint_as_float(rb[j]), s1, acc[32 + j]);
          }
        }
      }
      if (!alive) break;

      if (KS > 1) {
        float* scr_tile = p.splitk_scratch + (size_t)tile * KS * NT * kSlabRows;
        float* scr = scr_tile + (size_t)ks * NT * kSlabRows + q * 32 + lane;
#pragma unroll
        for (int j = 0; j < NT; ++j) scr[j * kSlabRows] = acc[j];
        __threadfence();
        __syncwarp();
        const uint32_t sph = si & 1u;
        ++si;
        if (lane == 0) mbar_arrive(bar_split);          // all four promotion warps have published their pieces
        bool oks = mbar_wait(bar_split, sph, abort_flag, p.status, 29);
        oks = __all_sync(0xffffffffu, oks);
        if (!oks) { alive = false; break; }
        if (warp == 4 && lane == 0) {
          __threadfence();   // the other warps' pieces (ordered before this point by the barrier) before the count
          const int prev = atomicAdd(p.splitk_count + tile, 1);
          if (prev == KS - 1) p.splitk_count[tile] = 0;   // every piece has arrived: leave the counter clean
          *split_flag = prev;
          mbar_arrive(bar_split + 8);
        }
        oks = mbar_wait(bar_split + 8, sph, abort_flag, p.status, 30);
        oks = __all_sync(0xffffffffu, oks);
        if (!oks) { alive = false; break; }
        if (*split_flag != KS - 1) continue;              // another CTA finishes this item
        __threadfence();
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j] = 0.f;
        for (int k = 0; k < KS; ++k) {
          const float* src = scr_tile + (size_t)k * NT * kSlabRows + q * 32 + lane;
#pragma unroll
          for (int j = 0; j < NT; ++j) acc[j] += __ldcg(src + j * kSlabRows);
        }
      }

      const int cnt = min(p.expert_count[e], NT);   // real rows of this expert
      if (MODE == 1) {
        // up warp q (2, 3) hands its u values to gate warp q-2 through shared memory
        // ([token][row] so that lanes hit consecutive banks); bounded mbarrier waits, no bar.sync.
        const int pr = q & 1;
        const uint32_t xph = xi & 1u;
        if (q >= 2) {
          bool okx = mbar_wait(bar_xfree + 8 * pr, xph ^ 1u, abort_flag, p.status, 27);
          okx = __all_sync(0xffffffffu, okx);
          if (!okx) { alive = false; break; }
#pragma unroll
          for (int j = 0; j < NT; ++j) xch[j * 64 + pr * 32 + lane] = acc[j];
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_xready + 8 * pr);
        } else {
          bool okx = mbar_wait(bar_xready + 8 * pr, xph, abort_flag, p.status, 28);
          okx = __all_sync(0xffffffffu, okx);
          if (!okx) { alive = false; break; }
          const int col = slab * 64 + q * 32 + lane;         // activation column of this lane
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            if (j < cnt) {
              const float u = xch[j * 64 + pr * 32 + lane];
              const __half hv = __float2half_rn(silu_mul_d(acc[j], u));
              p.act[(size_t)(row0 + j) * p.inter + col] = hv;
              const uint32_t mx = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(__half2float(hv))));
              if (lane == 0) atomicMax(p.row_amax + row0 + j, mx);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_xfree + 8 * pr);
        }
        ++xi;
        if (p.tile_done) {
          // Requantisation inside this kernel: an expert's 32 weight slabs count their arrivals, and the CTA
          // that stores the last one finds all of the expert's (at most NT) activation rows and their
          // final maxima in L2 and turns them into e4m3 codes with one scale per row (max|act| / 448,
          // solution/python/moe_fused.cu:175-195 of the reference).  A CTA runs one or two items at these
          // sizes, so the round trip of the counting atomic is paid once or twice.
          const uint32_t rph = ri & 1u;
          ++ri;
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_rq);            // this warp's stores and row maxima are issued
          if (warp == 4) {
            bool okr = mbar_wait(bar_rq, rph, abort_flag, p.status, 31);
            okr = __all_sync(0xffffffffu, okr);
            if (!okr) { alive = false; break; }
            if (lane == 0) {
              __threadfence();   // the four warps' stores (ordered before this point by the barrier) before the count
              const int prev = atomicAdd(p.tile_done + m_tile, 1);
              *rq_flag = prev == p.n_tiles - 1 ? 1 : 0;
              mbar_arrive(bar_rq + 8);
            }
          }
          bool okq = mbar_wait(bar_rq + 8, rph, abort_flag, p.status, 32);
          okq = __all_sync(0xffffffffu, okq);
          if (!okq) { alive = false; break; }
          if (*rq_flag) {
            __threadfence();
            const int tid = (warp - 4) * 32 + lane;
            const int vecs = p.inter / 8;              // 8 halves = 16 bytes in, 8 bytes out
            for (int j = 0; j < cnt; ++j) {
              const int m = row0 + j;
              const float amax = fmaxf(__uint_as_float(__ldcg(p.row_amax + m)), 1e-8f);
              const float sc = fmaxf(amax / 448.0f, 1e-8f);
              if (tid == 0) p.row_scale_out[m] = sc;
              const uint4* src = reinterpret_cast<const uint4*>(p.act + (size_t)m * p.inter);
              uint2* dstq = reinterpret_cast<uint2*>(p.act_q_out + (size_t)m * p.inter);
              for (int v = tid; v < vecs; v += 128) {
                const uint4 raw = __ldcg(src + v);
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 b2 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&raw.z));
                const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&raw.w));
                uint2 pk;
                pk.x = pack4_e4m3(a.x / sc, a.y / sc, b2.x / sc, b2.y / sc);
                pk.y = pack4_e4m3(c.x / sc, c.y / sc, d.x / sc, d.y / sc);
                dstq[v] = pk;
              }
            }
          }
        }
      } else {
        const int col = slab * kSlabRows + q * 32 + lane;    // output column of this lane
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          if (j < cnt) {
            const float rs = p.row_scale[row0 + j] * p.row_weight[row0 + j];
            atomicAdd(p.out + (size_t)p.row_token[row0 + j] * p.out_stride + col, __float2bfloat16_rn(acc[j] * rs));
          }
        }
      }
    }
    if (PROF && p.prof && blockIdx.x == 0 && warp == 4 && lane == 0) {
      p.prof[7] = (unsigned long long)ew_wait;                  // promotion warp 0: waiting for an accumulator
      p.prof[8] = (unsigned long long)(clock64() - ebegin);     // promotion warp 0: whole role
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
  if (threadIdx.x == 0 && abort_flag[0] && p.status_mirror) {
    // a wait of this CTA ran out: let the host see the status word without a copy of its own
    p.status_mirror[1] = p.status[kStatusDetail];
    p.status_mirror[0] = p.status[kStatusCode];
    __threadfence_system();
  }
}

template <int MODE, int NT>
cudaError_t launch_one(const GemmParams& p, int num_sms, cudaStream_t stream) {
  if (p.prof)
    return launch_chained(decode_gemm_kernel<MODE, NT, true>, dim3(num_sms), dim3(kThreads), DCfg<NT>::kSmemBytes,
                          stream, p);
  return launch_chained(decode_gemm_kernel<MODE, NT, false>, dim3(num_sms), dim3(kThreads), DCfg<NT>::kSmemBytes,
                        stream, p);
}

template <int MODE, int NT>
cudaError_t configure_one() {
  cudaError_t e = cudaFuncSetAttribute(decode_gemm_kernel<MODE, NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       DCfg<NT>::kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(decode_gemm_kernel<MODE, NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              DCfg<NT>::kSmemBytes);
}

}  // namespace

cudaError_t configure_decode_gemm() {
  cudaError_t e;
  if ((e = configure_one<1, 16>()) != cudaSuccess) return e;
  if ((e = configure_one<1, 64>()) != cudaSuccess) return e;
  if ((e = configure_one<2, 16>()) != cudaSuccess) return e;
  return configure_one<2, 64>();
}

int decode_gemm_max_kblocks() { return DCfg<16>::kMaxKBlocks; }

cudaError_t launch_decode_gemm(int mode, int nt, const GemmParams& p, int num_sms, cudaStream_t stream) {
  // the per-warp scale panels hold kMaxKBlocks entries: a longer K range would write past them
  if (p.kblocks > DCfg<16>::kMaxKBlocks) return cudaErrorInvalidValue;
  if (mode == 1) return nt == 16 ? launch_one<1, 16>(p, num_sms, stream) : launch_one<1, 64>(p, num_sms, stream);
  return nt == 16 ? launch_one<2, 16>(p, num_sms, stream) : launch_one<2, 64>(p, num_sms, stream);
}

}  // namespace b200moe
