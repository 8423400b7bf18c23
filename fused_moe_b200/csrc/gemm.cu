// Persistent grouped FP8 GEMMs on tcgen05 tensor cores with exact fp32 block scales.
//
// Replaces the reference's CUTLASS grouped GEMM `moe_blockwise_grouped_mm_v2`
// (solution/python/moe_gemm.cu:310-340, 418-654) plus, in the epilogues, the front half
// of its `swiglu_fp8_requant_kernel` (solution/python/moe_fused.cu:131-196) and the
// per-row scaling of its combine kernels (moe_fused.cu:346-393, 490-517).
//
// One CTA of 12 warps per SM walks work items (M tile of 128 packed rows, N tile of 256
// weight rows).  Per 128-wide K block (= one fp32 scale block, = one 128-byte swizzled row):
//   warps 0, 3   TMA producers (one lane each, alternate K blocks): A box 128x128 B, one B box
//                256x128 B and (GEMM1) the 128 activation scales of the K block into a smem ring
//   warps 1, 2   MMA issuers (one lane each, alternate K blocks, issuer i always writes TMEM
//                accumulator i): 4 tcgen05.mma (K=32 each) starting from zero, so an accumulator
//                holds the raw e4m3 dot product of ONE K block
//   warps 4-11   promotion: two warps per TMEM lane quarter, 128 accumulator columns each; they
//                read the K block's partial sums back (tcgen05.ld, two loads in flight) and fold
//                them into fp32 registers with packed FMAs: acc += (a_scale * b_scale) * partial.
//                The block scales are arbitrary (signed) fp32 numbers, so they cannot ride on the
//                MMA.  (Sixteen warps with 64 columns each fit only 112 registers per thread and
//                measured slower.)
// What shaped the hand-offs (measured with one-off probes on this GPU): an mbarrier wait costs ~180
// cycles of latency even when the phase is already complete; a single thread needs ~360 cycles to
// issue a K block's four MMAs and commits, two threads taking turns reach the MMA rate (513 cycles
// per 128x256x128 block) with the TMA copies running; the promotion warps' read-back plus FMAs take
// ~500-600 cycles per K block whatever is done about the waits, and a K block's MMAs complete
// ~700 cycles after their issue ends (390 in isolation).  Therefore
//   * a promotion warp looks at the NEXT K block's "accumulator written" barrier (non-blocking) before
//     the last FMAs of the current one, so the look's latency hides under the FMAs;
//   * "accumulator read back" is a shared-memory counter the promotion warps add to and the
//     issuer polls with plain acquire loads (~30 cycles) instead of a second mbarrier;
//   * activation scales arrive in shared memory with the operands (same barrier); the weight scales of an
//     item and its rows' token / output factors are copied into a per-warp panel while the item BEFORE it
//     is in its K loop (cp.async), so neither the K loop nor an item's start waits on global memory.
// Also measured, and slower or no faster (cycles per 128x256x128 K block, this kernel: ~940):
//   * handing the accumulator over in two 128-column halves (N = 128 MMAs, four barriers): ~1000 - an
//     N = 128 MMA of one CTA takes ~90 cycles instead of 64 (it re-reads A from shared memory twice as often,
//     and shared memory is already ~80 % busy with TMA writes and operand reads), so the tensor pipe alone
//     needs ~720;
//   * rings of their own for the two operands (three A slots, five B slots): no faster, and with rings of odd
//     length the two issuing threads alternate on a slot, so a parity wait can take the phase before last
//     for the current one - each issuer then has to publish which K blocks it has seen landed;
//   * CTA pairs on 256 x 128 tiles with four 128-column accumulators, a thread's 64 columns read in one go
//     and the next K block's read-back in flight during the FMAs: ~1000 per half-sized step - a step has
//     the same four or five dependent shared-memory round trips (~110 cycles each under this load) as a K
//     block here, for half of the FMAs;
//   * zeros instead of stale bytes in the padding rows of an expert's last tile, and a bare hand-off loop for
//     promotion warps whose 32 rows are all padding: no change of the step time under the board's power limit
//     (a sustained run settles near 1.5-1.6 GHz), and the extra loop cost the main one ~4 %.
// GEMM1 pairs gate rows [n, n+128) with up rows [inter+n, ...) in one tile, so the epilogue
// computes g*silu(u) in registers, stores fp16 activations and the row maximum.  (Requantising
// inside this kernel - the CTA that completes the last N tile of an M tile turning the tile's rows
// into e4m3 - was built and measured: read back at once it costs every item an atomic round trip,
// read back one item later the rows have left L2 and the lone CTA waits on HBM latency, 2.5 ms per
// step at 256 experts; the row scale needs all 16 N tiles, so the requantisation stays a kernel.)
// GEMM2's epilogue multiplies by (row requant scale * routing weight) and adds the bf16 row into its
// token's row of the output (red.global.add.noftz.v4.bf16x2): no second pass over the rows.
//
// Every wait is bounded (see mbar_wait); on a timeout the CTA drains and frees its TMEM.
#include <cuda_fp16.h>
#include <stdlib.h>

#include "common.cuh"
#include "kernels.cuh"

namespace b200moe {

namespace {

constexpr int kCtrlWarps = 4;
constexpr int kPromoWarps = 8;
constexpr int kGemmThreads = 32 * (kCtrlWarps + kPromoWarps);   // 384: three warpgroups
// Register budget: the CTA owns what it was launched with, 384 threads x 168 registers, and
// setmaxnreg only moves registers inside that pool (an increase that the pool cannot serve blocks
// for ever): 128 control threads give up 168 - 56 each, 256 promotion threads take 224 - 168 each.
constexpr int kLaunchRegs = 168;
constexpr int kCtrlRegs = 56;
constexpr int kPromoRegs = 224;
static_assert(32 * kCtrlWarps * (kLaunchRegs - kCtrlRegs) >= 32 * kPromoWarps * (kPromoRegs - kLaunchRegs),
              "setmaxnreg.inc would wait for registers that nobody releases");
static_assert(kGemmThreads * kLaunchRegs <= 65536 && kGemmThreads * (kLaunchRegs + 8) > 65536,
              "kLaunchRegs must be what 384 threads per SM are launched with");
constexpr int kBN = 256;
constexpr int kABytes = kTileM * kBlockK;   // 16 KiB
constexpr int kBBytes = kBN * kBlockK;      // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStages = 4;
constexpr int kRing = 8;                    // activation-scale slots; see the reuse argument at the producer
constexpr int kRingBytes = kRing * kTileM * 4;
// Per promotion warp and work item, staged one item ahead (two buffers): two runs of up to 64 weight
// scales, then per lane the row's token, requantisation scale and routing weight.
constexpr int kPanelFloats = 128;
constexpr int kItemFloats = kPanelFloats + 3 * 32;
constexpr int kPanelBytes = kPromoWarps * 2 * kItemFloats * 4;
constexpr int kMaxKBlocks = 64;
constexpr int kBarBytes = 256;
constexpr int kSmemBytes = kStages * kStageBytes + kRingBytes + kPanelBytes + kBarBytes + 1024;   // + alignment slack
constexpr int kTmemCols = 2 * kBN;

__device__ __forceinline__ float silu_mul(float g, float u) {
  float sig = __fdividef(1.0f, 1.0f + __expf(-u));   // approximate reciprocal: 2 ulp, far below e4m3 resolution
  // The activations are stored as fp16: a product beyond its range saturates (the row then requantises to
  // the largest e4m3 code) instead of becoming inf and, through an infinite row scale, NaN.
  return fminf(fmaxf(g * (u * sig), -65504.0f), 65504.0f);
}

// acc[16 pairs] += scale * r[32] with packed fp32 FMAs (scalar FMAs measured the same)
__device__ __forceinline__ void fma_chunk(float2* acc, const uint32_t (&r)[32], float sc) {
  const float2 s2 = make_float2(sc, sc);
#pragma unroll
  for (int j = 0; j < 16; ++j)
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), s2, acc[j]);
}

// untiled bulk copy global -> shared (16-byte aligned, size a multiple of 16), counted on an mbarrier
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Relaxed: what the counter publishes ("these TMEM columns sit in my registers") was completed by
// tcgen05.wait::ld before this instruction; the tcgen05 fences on both sides order the tensor-memory accesses.
__device__ __forceinline__ void red_add_smem(uint32_t addr, uint32_t v) {
  asm volatile("red.relaxed.cta.shared::cta.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_smem(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float ld_smem_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cta.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// 4-byte asynchronous copy global -> shared (no register holds the value while it is in flight)
__device__ __forceinline__ void copy4_async(uint32_t smem_dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_dst), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ uint32_t ld_smem_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// Bounded poll of a monotonic shared-memory counter (wrap-safe comparison).
__device__ __forceinline__ bool counter_wait(uint32_t addr, uint32_t target, volatile int* abort_flag, int* status,
                                             int where) {
  long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if ((int32_t)(ld_acquire_smem(addr) - target) >= 0) return true;
    if (++spins >= 256u) {
      spins = 0;
      if (*abort_flag) return false;
      long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > kWaitBudgetCycles) {
        *abort_flag = 1;
        if (atomicCAS(status + kStatusCode, 0, (int)B200MOE_ERR_DEVICE_TIMEOUT) == 0)
          status[kStatusDetail] = where;
        return false;
      }
    }
  }
}

template <int MODE, bool PROF>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
  constexpr int S = kStages;
  constexpr int CH = 4;                // 32-column chunks per promotion thread: 256 columns / 2 warps per lane quarter / 32
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t ring_base = smem_base + S * kStageBytes;          // [kRing][128] activation scales
  const uint32_t panel_base = ring_base + kRingBytes;              // [8 warps][2 buffers][kItemFloats] staged per-item values
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * kStageBytes + kRingBytes + kPanelBytes);
  const uint32_t bar_full = smem_u32(bars);              // S barriers: stage filled by TMA
  const uint32_t bar_empty = bar_full + 8 * S;           // S barriers: stage consumed by the MMAs
  const uint32_t bar_tfull = bar_empty + 8 * S;          // 2 barriers: accumulator written
  const uint32_t bar_drain = bar_tfull + 16;             // 2 barriers: each issuer's MMAs retired (teardown)
  uint32_t* words = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  const uint32_t cnt_read = smem_u32(words);             // 2 counters: promotion warps that read accumulator b back
  uint32_t* tmem_slot = words + 2;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(words + 3);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tfull + 8, 1);
    mbar_init(bar_drain, 1);
    mbar_init(bar_drain + 8, 1);
    words[0] = 0;
    words[1] = 0;
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
  const int total_items = m_tiles * p.n_tiles;
  const int kblocks = p.kblocks;

  if (warp < kCtrlWarps) {
    reg_dealloc<kCtrlRegs>();
    if ((warp == 0 || warp == 3) && lane == 0) {
      // ------------------------------ TMA producers (alternate K blocks) ------------------------------
      // Ring of activation scales: slot it % 8 is rewritten for K block it once the MMAs of K block
      // it - 4 have completed (the stage's "empty" barrier).  Its last readers, the promotion warps of
      // K block it - 8, read their scale before they released that accumulator, i.e. before the MMAs
      // of K block it - 6 could start.
      // (Pulling weight boxes into L2 ahead of their copy - by the TMA unit or by prefetch.global.L2 from
      // spare lanes, 2 to 24 K blocks ahead - and L2 eviction hints on the copies were all measured: every
      // form of look-ahead made the streaming case slower, the hints changed nothing.)
      const uint32_t pme = warp == 0 ? 0u : 1u;
      uint32_t it = 0;
      bool alive = true;
      for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
        const int m_tile = w / p.n_tiles, n_tile = w % p.n_tiles;
        const int e = p.tile_expert[m_tile];
        // GEMM1: first row inside the gate (and up) plane of expert e; GEMM2: row of [e_local*hidden][inter]
        const int brow = MODE == 1 ? n_tile * (kBN / 2) : e * p.n_per_expert + n_tile * kBN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if ((it & 1u) != pme) continue;
          const uint32_t s = it % S, ph = (it / S) & 1u;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status, 1)) { alive = false; break; }
          const uint32_t full = bar_full + 8 * s;
          const uint32_t a_dst = smem_base + s * kStageBytes;
          mbar_arrive_expect_tx(full, kStageBytes + (MODE == 1 ? kTileM * 4 : 0));
          // the whole B tile in one operation: 128 gate rows + 128 up rows (3D box over the two planes), or 256
          // rows; first, because it is the part that comes from HBM
          if (MODE == 1) tma_load_3d(a_dst + kABytes, &p.tmap_b, kb * kBlockK, brow, 2 * e, full);
          else tma_load_2d(a_dst + kABytes, &p.tmap_b, kb * kBlockK, brow, full);
          tma_load_2d(a_dst, &p.tmap_a, kb * kBlockK, m_tile * kTileM, full);
          if (MODE == 1)
            bulk_load(ring_base + (it % kRing) * (kTileM * 4),
                      p.a_scale + (size_t)kb * p.m_cap + (size_t)m_tile * kTileM, kTileM * 4, full);
        }
      }
      // Copies still in flight must land before the CTA's shared memory is released.
      const uint32_t first = it > (uint32_t)S ? it - S : 0u;
      for (uint32_t j = first; j < it; ++j)
        if ((j & 1u) == pme) (void)mbar_wait(bar_full + 8 * (j % S), (j / S) & 1u, abort_flag + 1, p.status, 6);
    } else if ((warp == 1 || warp == 2) && lane == 0) {
      // ------------------------------ MMA issuers ------------------------------
      // Two threads (on different SM sub-partitions) take alternate K blocks: issuing the four
      // MMAs and two commits of a K block costs one thread ~360 cycles whatever the tile size.
      // Issuer i always writes accumulator i.
      constexpr uint32_t idesc = make_idesc_e4m3(kTileM, kBN);
      const uint32_t me = (uint32_t)(warp - 1);
      uint32_t it = 0;
      bool alive = true;
      long long wait_epi = 0, wait_tma = 0, t_issue = 0;
      for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x) {
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if ((it & 1u) != me) continue;
          const uint32_t s = it % S, ph = (it / S) & 1u;
          const long long m0 = PROF ? clock64() : 0;
          // Operands first: they usually landed long ago, so only the accumulator hand-off is
          // left on the critical path.
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 3)) { alive = false; break; }
          const long long m1 = PROF ? clock64() : 0;
          // use number it/2 of accumulator `me`: all promotion warps have read the previous one
          if (!counter_wait(cnt_read + 4 * me, (uint32_t)kPromoWarps * (it >> 1), abort_flag, p.status, 2)) {
            alive = false;
            break;
          }
          const long long m2 = PROF ? clock64() : 0;
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * kStageBytes;
          tc_mma_f8_kblock(tmem_base + me * kBN, kmajor_sw128_desc_lo(a_addr), kmajor_sw128_desc_lo(a_addr + kABytes),
                           kKmajorSw128DescHi, idesc);
          tc_commit(bar_empty + 8 * s);
          tc_commit(bar_tfull + 8 * me);
          if (PROF) {
            const long long m3 = clock64();
            wait_tma += m1 - m0;
            wait_epi += m2 - m1;
            t_issue += m3 - m2;
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
    reg_alloc<kPromoRegs>();
    const int pw = warp - kCtrlWarps;
    const int q = pw & 3;          // TMEM lane quarter this warp may read (= warp % 4)
    const int cg = pw >> 2;        // which half of the tile's 256 accumulator columns
    constexpr int HC = CH / 2;     // chunks per half (GEMM1: gate half, up half)
    // GEMM1: HC x 32 gate columns and the matching up columns; GEMM2: CH x 32 consecutive columns.
    // chunk c < HC sits at col_lo + 32 c, chunk c >= HC at col_hi + 32 (c - HC)
    const uint32_t col_lo = MODE == 1 ? cg * (HC * 32) : cg * (CH * 32);
    const uint32_t col_hi = MODE == 1 ? kBN / 2 + cg * (HC * 32) : cg * (CH * 32) + HC * 32;
    const uint32_t stage_me = panel_base + pw * (2 * kItemFloats * 4);
    const uint32_t ring_me = ring_base + (q * 32 + lane) * 4;
    uint32_t it = 0;
    bool alive = true;
    const bool prof_me = PROF && p.prof && blockIdx.x == 0 && pw == 0 && lane == 0;
    const long long t_begin = PROF ? clock64() : 0;
    long long t_wait = 0, t_promote = 0, t_epi = 0;
    const int nblk_per_expert = p.n_per_expert / kBlockK;
    uint32_t peek = 0;   // "accumulator written" of the coming K block already seen complete
    // What an item needs besides its operands - the weight scales of its (expert, N tile) and, per row, the
    // token and the two output factors - is copied into shared memory while the item BEFORE it is in its K
    // loop: fetched at the item's start, the chain tile_expert -> scales (two dependent loads under the weight
    // stream) cost ~5000 cycles per item during which the MMAs ran dry.
    auto stage_item = [&](int w, int e, uint32_t dst) {
      const int m_tile = w / p.n_tiles, n_tile = w % p.n_tiles;
      const float* run0;
      const float* run1;
      if (MODE == 1) {
        run0 = p.b_scale + ((size_t)e * nblk_per_expert + n_tile) * kblocks;                       // gate block
        run1 = p.b_scale + ((size_t)e * nblk_per_expert + p.inter / kBlockK + n_tile) * kblocks;   // up block
      } else {
        run0 = p.b_scale + ((size_t)e * nblk_per_expert + 2 * n_tile + (cg * (CH * 32)) / kBlockK) * kblocks;
        run1 = run0;
      }
      if (lane < kblocks) {
        copy4_async(dst + lane * 4, run0 + lane);
        if (MODE == 1) copy4_async(dst + (64 + lane) * 4, run1 + lane);
      }
      if (lane + 32 < kblocks) {
        copy4_async(dst + (32 + lane) * 4, run0 + lane + 32);
        if (MODE == 1) copy4_async(dst + (96 + lane) * 4, run1 + lane + 32);
      }
      const int row = m_tile * kTileM + q * 32 + lane;
      copy4_async(dst + (kPanelFloats + lane) * 4, p.row_token + row);
      if (MODE == 2) {
        copy4_async(dst + (kPanelFloats + 32 + lane) * 4, p.row_scale + row);
        copy4_async(dst + (kPanelFloats + 64 + lane) * 4, p.row_weight + row);
      }
    };
    const int kb_stage = kblocks > 4 ? kblocks - 4 : 0;   // the K block during which the next item is staged
    uint32_t pb = 0;
    if ((int)blockIdx.x < total_items) stage_item(blockIdx.x, p.tile_expert[blockIdx.x / p.n_tiles], stage_me);
    for (int w = blockIdx.x; w < total_items && alive; w += gridDim.x, pb ^= 1u) {
      const int m_tile = w / p.n_tiles, n_tile = w % p.n_tiles;
      const int row = m_tile * kTileM + q * 32 + lane;
      const uint32_t panel = stage_me + pb * (kItemFloats * 4);
      const int w_next = w + gridDim.x;
      // read now, used at K block kb_stage: the expert of the next item
      const int e_next = w_next < total_items ? p.tile_expert[w_next / p.n_tiles] : 0;
      float2 acc[CH * 16];
#pragma unroll
      for (int j = 0; j < CH * 16; ++j) acc[j] = make_float2(0.f, 0.f);
      copy_async_wait_all();   // this item's staged values (copied during the previous item's K loop)
      __syncwarp();

      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const uint32_t b = it & 1u, bph = (it >> 1) & 1u;
        const long long c0 = PROF ? clock64() : 0;
        if (!peek) {
          bool ok = mbar_wait(bar_tfull + 8 * b, bph, abort_flag, p.status, 4);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) { alive = false; break; }
        }
        tc_fence_after();
        const long long c1 = PROF ? clock64() : 0;
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + b * kBN;
        const uint32_t nit = it + 1;
        float sc0, sc1;
        auto load_scales = [&]() {   // issued behind the first TMEM loads so that the latencies overlap
          sc0 = ld_smem_f32(panel + kb * 4);
          sc1 = MODE == 1 ? ld_smem_f32(panel + (64 + kb) * 4) : sc0;
          if (MODE == 1) {
            const float sa = ld_smem_f32(ring_me + (it % kRing) * (kTileM * 4));
            sc0 *= sa;
            sc1 *= sa;
          }
        };
        // The accumulator is free as soon as its last column sits in registers: the MMA thread is told
        // before the remaining FMAs, which then overlap the next K block's MMAs.  Right behind that the
        // other accumulator's barrier is looked at (non-blocking) for the next K block; the answer is
        // picked up after the last FMAs, so its latency costs nothing, and when it says "written" the
        // next iteration starts without a wait.  (Past the CTA's last K block nothing consumes it.)
        uint32_t pk;
        {
          uint32_t ra[32], rb[32];
          tmem_ld_32x32(t_row + col_lo, ra);
          tmem_ld_32x32(t_row + col_lo + 32, rb);
          load_scales();
          tmem_ld_wait_on(ra, rb);
          fma_chunk(acc, ra, sc0);
          tmem_ld_32x32(t_row + col_hi, ra);
          fma_chunk(acc + 16, rb, sc0);
          tmem_ld_32x32(t_row + col_hi + 32, rb);
          tmem_ld_wait_on(ra, rb);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) red_add_smem(cnt_read + 4 * b, 1u);
          pk = mbar_test_wait(bar_tfull + 8 * (nit & 1u), (nit >> 1) & 1u);
          fma_chunk(acc + 32, ra, sc1);
          fma_chunk(acc + 48, rb, sc1);
        }
        peek = __all_sync(0xffffffffu, pk != 0u) ? 1u : 0u;
        if (kb == kb_stage && w_next < total_items) stage_item(w_next, e_next, stage_me + (pb ^ 1u) * (kItemFloats * 4));
        if (PROF) {
          const long long c2 = clock64();
          t_wait += c1 - c0;
          t_promote += c2 - c1;
        }
      }
      if (!alive) break;
      const long long te0 = PROF ? clock64() : 0;

      const int tok = (int)ld_smem_u32(panel + (kPanelFloats + lane) * 4);
      if (tok >= 0) {
        if (MODE == 1) {
          // acc[0 .. HC*16) = gate columns (pairs), acc[HC*16 ..) = the matching up columns.
          // fp16 keeps 11 significant bits, three more than the e4m3 codes made from it need;
          // the row maximum is taken over the rounded values so that it is attained exactly.
          constexpr int HP = HC * 16;
          __half* dst = p.act + (size_t)row * p.inter + n_tile * (kBN / 2) + cg * (HC * 32);
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
          // the routing-weighted unpermute/reduce: bf16(G2 * w) of this row is added straight into its
          // token's output row (zeroed at call start), eight bf16 sums per 16-byte red.global.add - the
          // arithmetic of the reference's `out[t] += bf16(G2 * w)` on a bf16 tensor
          // (experiments/fast_bench/correctness_bench.py:107-111), in the order the tiles finish
          const float rs = ld_smem_f32(panel + (kPanelFloats + 32 + lane) * 4) * ld_smem_f32(panel + (kPanelFloats + 64 + lane) * 4);
          __nv_bfloat16* dst = p.out + (size_t)tok * p.out_stride + n_tile * kBN + cg * (CH * 32);
#pragma unroll
          for (int j = 0; j < CH * 16; j += 4) {
            uint32_t wv[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              __nv_bfloat162 v = __floats2bfloat162_rn(acc[j + t].x * rs, acc[j + t].y * rs);
              wv[t] = *reinterpret_cast<uint32_t*>(&v);
            }
            red_add_bf16x8(dst + 2 * j, wv[0], wv[1], wv[2], wv[3]);
          }
        }
      }
      if (PROF) t_epi += clock64() - te0;
    }
    copy_async_wait_all();   // (an aborted item loop may leave copies of the next item's values in flight)
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
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && abort_flag[0] && p.status_mirror) {
    // a wait of this CTA ran out: let the host see the status word without a copy of its own
    p.status_mirror[1] = p.status[kStatusDetail];
    p.status_mirror[0] = p.status[kStatusCode];
    __threadfence_system();
  }
}

template <int MODE>
cudaError_t launch_one(const GemmParams& p, int num_sms, cudaStream_t stream) {
  if (p.prof)
    return launch_chained(grouped_gemm_kernel<MODE, true>, dim3(num_sms), dim3(kGemmThreads), kSmemBytes, stream, p);
  else
    return launch_chained(grouped_gemm_kernel<MODE, false>, dim3(num_sms), dim3(kGemmThreads), kSmemBytes, stream, p);
}

template <int MODE>
cudaError_t configure_one() {
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<MODE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(grouped_gemm_kernel<MODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              kSmemBytes);
}

}  // namespace

cudaError_t configure_grouped_gemm() {
  cudaError_t e;
  if ((e = configure_one<1>()) != cudaSuccess) return e;
  return configure_one<2>();
}

int grouped_gemm_max_kblocks() { return kMaxKBlocks; }

cudaError_t launch_grouped_gemm(int mode, const GemmParams& p, int num_sms, cudaStream_t stream) {
  return mode == 1 ? launch_one<1>(p, num_sms, stream) : launch_one<2>(p, num_sms, stream);
}

}  // namespace b200moe
