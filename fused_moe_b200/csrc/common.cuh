// Shared device helpers: PTX wrappers for mbarrier, TMA, tcgen05 (sm_100a), bounded waits.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdlib.h>
#include <utility>

#include "../../include/b200moe.h"

namespace b200moe {

constexpr int kNumExperts = 256;
constexpr int kNumGroups = 8;
constexpr int kGroupSize = 32;
constexpr int kTopKGroups = 4;
constexpr int kTopK = 8;
constexpr int kBlockK = 128;       // one scale block along K = one 128-byte swizzle row of e4m3
constexpr int kTileM = 128;        // packed rows per M tile (= TMEM lanes)
constexpr int kChunkTokens = 256;  // tokens per placement chunk

// Status word indices inside the workspace status array.
constexpr int kStatusCode = 0;
constexpr int kStatusDetail = 1;

// Device-side wait budget: about 0.2 s at 2 GHz.  Legitimate waits in these kernels are
// microseconds long; a wait that exceeds the budget means a protocol bug, and the kernel
// records B200MOE_ERR_DEVICE_TIMEOUT and leaves instead of hanging the GPU.
constexpr long long kWaitBudgetCycles = 400000000LL;

// Workspace carve-up shared by host code and tests (see b200moe_ws_layout).
struct Workspace {
  b200moe_ws_layout L;
  uint8_t* base;
  template <typename T> __host__ __device__ T* at(uint64_t off) const { return reinterpret_cast<T*>(base + off); }
};

// ---------------------------------------------------------------------------------------
// small PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Non-blocking look at a phase (try_wait may suspend the thread for a while when the phase is still open).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Bounded wait on an mbarrier phase.  Returns false when the CTA is aborting (another
// thread gave up) or when this wait ran out of budget; in the latter case the status word
// in global memory receives the timeout code and `where` for diagnosis.
__device__ __forceinline__ bool mbar_wait_budget(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                 int* status, int where, long long budget_cycles) {
  long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (++spins >= 128u) {
      spins = 0;
      if (*abort_flag) return false;
      long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > budget_cycles) {
        *abort_flag = 1;
        if (atomicCAS(status + kStatusCode, 0, (int)B200MOE_ERR_DEVICE_TIMEOUT) == 0)
          status[kStatusDetail] = where;
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int where) {
  return mbar_wait_budget(bar, parity, abort_flag, status, where, kWaitBudgetCycles);
}
// TMA: 2D tiled load global -> shared, completion counted on an mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tcgen05 / tensor memory ----
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result_addr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrive on an mbarrier once every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, e4m3 x e4m3 -> fp32, issued by one thread.
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Four MMAs (K = 4 x 32) of one 128-wide K block in a single instruction sequence: the first
// overwrites the accumulator, the others add.  The issuing thread runs alone, so every
// instruction it spends is on the critical path; descriptors are therefore passed as
// prebuilt 32-bit halves (low word = start address >> 4 plus constants, see
// make_kmajor_sw128_desc) and advanced by 32 bytes (2 units) in place.
__device__ __forceinline__ void tc_mma_f8_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                                 uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred pf, pt;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, pf;\n\t"
      "add.u32 al, %1, 2;\n\t"
      "add.u32 bl, %2, 2;\n\t"
      "mov.b64 da, {al, %3};\n\t"
      "mov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, pt;\n\t"
      "add.u32 al, %1, 4;\n\t"
      "add.u32 bl, %2, 4;\n\t"
      "mov.b64 da, {al, %3};\n\t"
      "mov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, pt;\n\t"
      "add.u32 al, %1, 6;\n\t"
      "add.u32 bl, %2, 6;\n\t"
      "mov.b64 da, {al, %3};\n\t"
      "mov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, pt;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc)
      : "memory");
}
// Halves of make_kmajor_sw128_desc(smem_addr): low word for an address, and the constant high word.
__device__ __forceinline__ uint32_t kmajor_sw128_desc_lo(uint32_t smem_addr) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
}
constexpr uint32_t kKmajorSw128DescHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes
// with the 128-byte swizzle (what a TMA box with a 128-byte inner extent produces):
// 8-row groups are 1024 bytes apart (stride byte offset), leading byte offset unused (1).
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                         // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset
  d |= (uint64_t)1 << 46;                         // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                         // layout: 128-byte swizzle
  return d;
}

// Instruction descriptor: e4m3 A and B (both K-major), fp32 accumulator, M x N tile.
__host__ __device__ constexpr uint32_t make_idesc_e4m3(int m, int n) {
  return (1u << 4)                       // accumulator format: f32
         | (0u << 7) | (0u << 10)        // A, B format: e4m3
         | (0u << 15) | (0u << 16)       // A, B K-major
         | ((uint32_t)(n >> 3) << 17)    // N / 8
         | ((uint32_t)(m >> 4) << 24);   // M / 16
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp reads lane (base+i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// tcgen05.wait::ld that also names the loaded registers as read-write operands, so that no
// use of them can be scheduled ahead of the wait by the compiler.
#define B200MOE_RW8(r, o) "+r"(r[o]), "+r"(r[o + 1]), "+r"(r[o + 2]), "+r"(r[o + 3]), "+r"(r[o + 4]), "+r"(r[o + 5]), "+r"(r[o + 6]), "+r"(r[o + 7])
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&a)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : B200MOE_RW8(a, 0), B200MOE_RW8(a, 8), B200MOE_RW8(a, 16), B200MOE_RW8(a, 24)
               :
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&a)[32], uint32_t (&b)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : B200MOE_RW8(a, 0), B200MOE_RW8(a, 8), B200MOE_RW8(a, 16), B200MOE_RW8(a, 24),
                 B200MOE_RW8(b, 0), B200MOE_RW8(b, 8), B200MOE_RW8(b, 16), B200MOE_RW8(b, 24)
               :
               : "memory");
}

// Register budget moves between warpgroups (all four warps of a warpgroup must execute it).
template <int N> __device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

__device__ __forceinline__ void prefetch_l1(const void* p) {
  asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// 32-byte store (one full sector per lane); address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* addr, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// four floats -> four e4m3 bytes (round to nearest even, saturating); byte order = element order
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Eight bf16 additions to global memory in one 16-byte operation (each sum rounded to bf16, as an
// `out += bf16(x)` on a bf16 tensor is); addr must be 16-byte aligned.
__device__ __forceinline__ void red_add_bf16x8(void* addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ float load_as_float(const void* p, int dtype, size_t i) {
  return dtype == B200MOE_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                               : reinterpret_cast<const float*>(p)[i];
}

// ---- programmatic dependent launch ----
// A kernel launched with `launch_chained` may become resident while the kernel before it on
// the stream is still running, so that its prologue (barrier init, tensor-memory allocation,
// descriptor fetch) overlaps that kernel's tail.  It must call chain_wait() before it reads
// or writes anything in global memory: the call returns once the previous kernel has
// completed and its writes are visible.  chain_release() lets the NEXT kernel on the stream
// become resident; every kernel calls it right after its own wait, so completion still
// propagates down the chain in order.  Both are no-ops for a plain launch.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// B200MOE_PDL=0 falls back to plain stream order.
inline bool chained_launch_enabled() {
  static const bool on = [] {
    const char* v = getenv("B200MOE_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

}  // namespace b200moe
