// C ABI of the library (declared in include/b200moe.h): argument checks, workspace
// carve-up, TMA descriptors, and the launch sequence of one layer call.
//
// Launch sequence of b200moe_run (all on the caller's stream, nothing allocated):
//   memset counters | route (+histogram) | scan | place | gather | GEMM1(+SwiGLU,+row max)
//   | requant | GEMM2(+row scale * routing weight, each row added into its token's zeroed bf16 output row)
// It replaces the two Python pipelines of the reference
// (solution/python/kernel.py:381-429 and 432-572), which need a host synchronisation
// above 2048 tokens (kernel.py:196); here tile counts stay on the device.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "kernels.cuh"

using namespace b200moe;

namespace {

thread_local char g_cuda_error[256] = "";

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", what, cudaGetErrorString(e));
  return B200MOE_ERR_CUDA;
}

#define CUDA_TRY(expr)                                  \
  do {                                                  \
    cudaError_t _e = (expr);                            \
    if (_e != cudaSuccess) return cuda_fail(_e, #expr); \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceInfo {
  bool ready = false;
  int num_sms = 0;
};

// Optional cudaEvent_t pair recorded around the GEMM1 launch of this thread's next
// b200moe_experts call (then forgotten); lets a benchmark time the dominant kernel in place.
thread_local cudaEvent_t g_prof_start = nullptr;
thread_local cudaEvent_t g_prof_stop = nullptr;

// Optional host-mapped int32[4] of this thread's calls: a kernel that gives up on a bounded wait copies the
// status word there, so a host can notice without a device-to-host copy per call.
thread_local int* g_status_mirror = nullptr;

std::mutex g_mutex;
EncodeTiledFn g_encode = nullptr;
DeviceInfo g_dev[64];

// Once per process: the driver entry point for tensor-map encoding; once per device: the
// SM count and the opt-in shared memory sizes of the GEMM kernels.
int ensure_device(int* num_sms) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200MOE_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !fn) {
      snprintf(g_cuda_error, sizeof(g_cuda_error), "cuTensorMapEncodeTiled not available from this driver");
      return B200MOE_ERR_CUDA;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  if (!g_dev[dev].ready) {
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10) {
      snprintf(g_cuda_error, sizeof(g_cuda_error), "device %d is sm_%d%d; this library is built for sm_100a only",
               dev, prop.major, prop.minor);
      return B200MOE_ERR_CUDA;
    }
    g_dev[dev].num_sms = prop.multiProcessorCount;
    CUDA_TRY(configure_grouped_gemm());
    CUDA_TRY(configure_decode_gemm());
    g_dev[dev].ready = true;
  }
  *num_sms = g_dev[dev].num_sms;
  return B200MOE_OK;
}

// rows x K e4m3 matrix, row pitch `pitch` bytes; box = box_rows x 128 bytes, 128-byte swizzle.
int make_tmap(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k, uint64_t pitch, uint32_t box_rows) {
  cuuint64_t dims[2] = {k, rows};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_error, sizeof(g_cuda_error), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}

// GEMM1 weights [e_local][2*inter][k] seen as planes: plane 2e holds expert e's gate rows, plane
// 2e+1 its up rows.  One box = the same `box_rows` rows of two consecutive planes (gate rows,
// then the matching up rows), 128 bytes of K wide, 128-byte swizzle: one TMA operation
// instead of two per K block (a box costs the issuing thread and the TMA unit a few hundred
// cycles whatever its size).
int make_tmap_gate_up(CUtensorMap* map, const void* base, uint64_t e_local, uint64_t inter, uint64_t k,
                      uint32_t box_rows) {
  cuuint64_t dims[3] = {k, inter, 2 * e_local};
  cuuint64_t strides[2] = {k, inter * k};
  cuuint32_t box[3] = {(cuuint32_t)kBlockK, box_rows, 2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_error, sizeof(g_cuda_error), "cuTensorMapEncodeTiled (3D) failed with CUresult %d", (int)r);
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}

uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

constexpr int kDirectRowsMaxTokens = 8;   // largest call whose decode GEMM1 reads the caller's rows in place

// Decode-size calls (up to 16 tokens) take the swapped-operand kernels (B200MOE_DECODE=0 turns them off;
// B200MOE_DECODE=64 extends them to 64 tokens, where the 128-row tiles currently measure faster).  Their
// per-warp scale panels hold a bounded number of K blocks; larger shapes take the grouped kernels.
// Returns the token tile of the decode kernels, or 0 for the grouped kernels.
int decode_tile(int T, int hidden, int inter) {
  static const bool decode_on = [] {
    const char* v = getenv("B200MOE_DECODE");
    return !(v && v[0] == '0');
  }();
  static const int decode_max_t = [] {
    const char* v = getenv("B200MOE_DECODE");
    return (v && v[0] == '6') ? 64 : 16;
  }();
  const bool fits = hidden / kBlockK <= decode_gemm_max_kblocks() && inter / kBlockK <= decode_gemm_max_kblocks();
  return (decode_on && fits && T <= decode_max_t) ? (T <= 16 ? 16 : 64) : 0;
}

int shape_ok(int T, int e_local, int hidden, int inter) {
  if (T < 0 || e_local < 1) return B200MOE_ERR_INVALID_ARGUMENT;
  if (e_local > kNumExperts || hidden < 256 || hidden % 256 != 0 || inter < 128 || inter % 128 != 0)
    return B200MOE_ERR_UNSUPPORTED_SHAPE;
  if ((long long)T * kTopK > (1ll << 30)) return B200MOE_ERR_UNSUPPORTED_SHAPE;
  // the GEMMs keep one weight scale per K block of an item in shared-memory panels
  if (hidden / kBlockK > grouped_gemm_max_kblocks() || inter / kBlockK > grouped_gemm_max_kblocks())
    return B200MOE_ERR_UNSUPPORTED_SHAPE;
  return B200MOE_OK;
}

void compute_layout(int T, int e_local, int hidden, int inter, b200moe_ws_layout* L) {
  memset(L, 0, sizeof(*L));
  const int n_chunks = T > 0 ? (T + kChunkTokens - 1) / kChunkTokens : 1;
  const long long pairs = (long long)T * (e_local < kTopK ? e_local : kTopK);
  // every expert segment is padded to a whole 128-row M tile; m_cap stays a multiple of 256
  const long long m_cap = (long long)align_up((uint64_t)pairs, 2 * kTileM) + (long long)2 * kTileM * e_local;
  L->m_cap = (int32_t)m_cap;
  L->max_tiles = (int32_t)(m_cap / kTileM);
  L->n_chunks = n_chunks;
  L->chunk_tokens = kChunkTokens;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) { uint64_t o = off; off = align_up(off + bytes, 256); return o; };
  L->status = take(16 * 4);
  L->meta = take(8 * 4);
  L->splitk_count = take(2 * kSplitKSlots * 4);   // inside the range that clear_counters() zeroes
  L->tile_done = take((uint64_t)L->max_tiles * 4);   // likewise
  L->chunk_counts = take((uint64_t)n_chunks * e_local * 4);
  L->chunk_base = take((uint64_t)n_chunks * e_local * 4);
  L->expert_count = take((uint64_t)e_local * 4);
  L->expert_row0 = take((uint64_t)(e_local + 1) * 4);
  L->tile_expert = take((uint64_t)L->max_tiles * 4);
  L->row_token = take((uint64_t)m_cap * 4);
  L->row_weight = take((uint64_t)m_cap * 4);
  L->a_packed = take((uint64_t)m_cap * hidden);
  L->a_scale = take((uint64_t)(hidden / kBlockK) * m_cap * 4);
  L->act = take((uint64_t)m_cap * inter * 2);
  L->row_amax = take((uint64_t)m_cap * 4);
  L->act_q = take((uint64_t)m_cap * inter);
  L->row_scale = take((uint64_t)m_cap * 4);
  L->tok_rows = take((uint64_t)(T > 0 ? T : 1) * kTopK * 4);
  L->topk_ids = take((uint64_t)(T > 0 ? T : 1) * kTopK * 4);
  L->topk_w = take((uint64_t)(T > 0 ? T : 1) * kTopK * 4);
  L->trace = take(2 * 8 * 64 * 8);   // B200MOE_PROF: absolute cycle stamps of CTA 0's first 64 K blocks
  L->splitk_scratch = take((uint64_t)kSplitKSlots * kSplitKMax * 16 * 128 * 4);   // 2 MiB
  L->ep_segments = take(256);   // RowSegments at +0, int32 row count at +192 (b200moe_ep_local_experts)
  L->total_bytes = off;
}

int bind_workspace(int T, int e_local, int hidden, int inter, void* workspace, size_t bytes, Workspace* ws) {
  int rc = shape_ok(T, e_local, hidden, inter);
  if (rc != B200MOE_OK) return rc;
  if (!workspace) return B200MOE_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return B200MOE_ERR_MISALIGNED;
  compute_layout(T, e_local, hidden, inter, &ws->L);
  if (bytes < ws->L.total_bytes) return B200MOE_ERR_WORKSPACE_TOO_SMALL;
  ws->base = reinterpret_cast<uint8_t*>(workspace);
  return B200MOE_OK;
}

// Clears the status word and the histogram (start of a layer call).
int clear_counters(const Workspace& ws, int e_local, cudaStream_t stream) {
  // status, meta, splitk_count, tile_done, chunk_counts are adjacent: one memset covers them
  size_t bytes = (size_t)(ws.L.chunk_counts - ws.L.status) + (size_t)ws.L.n_chunks * e_local * 4;
  CUDA_TRY(cudaMemsetAsync(ws.base + ws.L.status, 0, bytes, stream));
  return B200MOE_OK;
}

}  // namespace

extern "C" {

int b200moe_version(void) { return 1; }

const char* b200moe_status_string(int status) {
  switch (status) {
    case B200MOE_OK: return "ok";
    case B200MOE_ERR_INVALID_ARGUMENT: return "invalid argument";
    case B200MOE_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
    case B200MOE_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case B200MOE_ERR_CUDA: return "CUDA call failed";
    case B200MOE_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait timed out";
    case B200MOE_ERR_MISALIGNED: return "misaligned pointer or stride";
    default: return "unknown status";
  }
}

const char* b200moe_last_cuda_error(void) { return g_cuda_error; }

int b200moe_workspace_layout(int T, int e_local, int hidden, int inter, b200moe_ws_layout* layout) {
  int rc = shape_ok(T, e_local, hidden, inter);
  if (rc != B200MOE_OK) return rc;
  b200moe_ws_layout L;
  compute_layout(T, e_local, hidden, inter, &L);
  if (layout) *layout = L;
  return B200MOE_OK;
}

int b200moe_set_status_mirror(void* host_mapped_int4) {
  g_status_mirror = reinterpret_cast<int*>(host_mapped_int4);
  return B200MOE_OK;
}

int b200moe_profile_next_gemm1(void* start_event, void* stop_event) {
  g_prof_start = reinterpret_cast<cudaEvent_t>(start_event);
  g_prof_stop = reinterpret_cast<cudaEvent_t>(stop_event);
  return B200MOE_OK;
}

int b200moe_launches_per_run(int T, int e_local) {
  (void)e_local;
  if (T <= 0) return 0;
  const char* front = getenv("B200MOE_FRONT");
  const bool fused_front = T <= kFrontSmallMaxTokens && !(front && front[0] == '0');
  // route, scan, place, gather, gemm1, requant, gemm2 (+ weighted unpermute / reduce into the output); calls of at
  // most 32 tokens fuse the first three, the decode GEMM1 (at most 16 tokens) also requantises
  static const bool decode_on = [] {
    const char* v = getenv("B200MOE_DECODE");
    return !(v && v[0] == '0');
  }();
  static const int decode_max_t = [] {
    const char* v = getenv("B200MOE_DECODE");
    return (v && v[0] == '6') ? 64 : 16;
  }();
  const int requant = (decode_on && T <= decode_max_t) ? 0 : 1;   // decode GEMM1 requantises by itself
  // ... and, behind the fused front kernel, fetches the token rows itself: no gather pass (three launches)
  const int gather = (fused_front && decode_on && T <= kDirectRowsMaxTokens) ? 0 : 1;
  return (fused_front ? 3 : 5) + gather + requant;
}

int b200moe_route(const void* logits, int logits_dtype, const void* bias, int bias_dtype, int T,
                  float routed_scaling_factor, int local_expert_offset, int e_local, int hidden, int inter,
                  int32_t* topk_ids, float* topk_w, void* workspace, size_t workspace_bytes, void* stream) {
  if (!logits || !bias || !topk_ids || !topk_w) return B200MOE_ERR_INVALID_ARGUMENT;
  if ((logits_dtype != B200MOE_F32 && logits_dtype != B200MOE_BF16) ||
      (bias_dtype != B200MOE_F32 && bias_dtype != B200MOE_BF16))
    return B200MOE_ERR_INVALID_ARGUMENT;
  if (local_expert_offset < 0 || local_expert_offset + e_local > kNumExperts) return B200MOE_ERR_INVALID_ARGUMENT;
  Workspace ws;
  int rc = bind_workspace(T, e_local, hidden, inter, workspace, workspace_bytes, &ws);
  if (rc != B200MOE_OK) return rc;
  int num_sms = 0;
  if ((rc = ensure_device(&num_sms)) != B200MOE_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if ((rc = clear_counters(ws, e_local, st)) != B200MOE_OK) return rc;
  CUDA_TRY(launch_route(logits, logits_dtype, bias, bias_dtype, T, routed_scaling_factor, local_expert_offset, e_local,
                        topk_ids, topk_w, ws.at<int>(ws.L.chunk_counts), num_sms, st));
  return B200MOE_OK;
}

int b200moe_count(const int32_t* topk_ids, int64_t ids_row_stride, int T, int local_expert_offset, int e_local,
                  int hidden, int inter, void* workspace, size_t workspace_bytes, void* stream) {
  if (!topk_ids || ids_row_stride < kTopK) return B200MOE_ERR_INVALID_ARGUMENT;
  if (local_expert_offset < 0 || local_expert_offset + e_local > kNumExperts) return B200MOE_ERR_INVALID_ARGUMENT;
  Workspace ws;
  int rc = bind_workspace(T, e_local, hidden, inter, workspace, workspace_bytes, &ws);
  if (rc != B200MOE_OK) return rc;
  int num_sms = 0;
  if ((rc = ensure_device(&num_sms)) != B200MOE_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if ((rc = clear_counters(ws, e_local, st)) != B200MOE_OK) return rc;
  CUDA_TRY(launch_count(topk_ids, ids_row_stride, T, local_expert_offset, e_local, ws.at<int>(ws.L.chunk_counts),
                        num_sms, st));
  return B200MOE_OK;
}

// `placed`: routing, scan and placement of this call already ran as one kernel (front_small.cu).
static int experts_impl(const int32_t* topk_ids, int64_t ids_row_stride, const float* topk_w, int64_t w_row_stride,
                        const uint8_t* hidden_states, int64_t hidden_row_stride, const float* hidden_scale,
                        int64_t scale_stride_t, int64_t scale_stride_kb, const uint8_t* w1, const float* w1_scale,
                        const uint8_t* w2, const float* w2_scale, int T, int e_local, int local_expert_offset,
                        int hidden, int inter, void* workspace, size_t workspace_bytes, void* out_bf16,
                        int64_t out_row_stride, void* stream, bool placed, const RowSegments* segs = nullptr,
                        const RowSegments* segs_dev = nullptr, const int* n_rows_dev = nullptr) {
  // The event pair armed by b200moe_profile_next_gemm1 is for this call only: forget it on every
  // way out (the GEMM1 launch below consumes it first when the call gets that far).
  struct DisarmProfile {
    ~DisarmProfile() { g_prof_start = g_prof_stop = nullptr; }
  } disarm_profile;
  if (!topk_ids || !topk_w || !w1 || !w1_scale || !w2 || !w2_scale) return B200MOE_ERR_INVALID_ARGUMENT;
  if (T > 0 && ((!segs && !segs_dev && (!hidden_states || !hidden_scale)) || !out_bf16))
    return B200MOE_ERR_INVALID_ARGUMENT;
  if (segs || segs_dev) {   // rows are read from the segments: no separate payload / scale arrays
    hidden_row_stride = hidden;
    hidden_states = nullptr;
  }
  if (ids_row_stride < kTopK || w_row_stride < kTopK) return B200MOE_ERR_INVALID_ARGUMENT;
  if (local_expert_offset < 0 || local_expert_offset + e_local > kNumExperts) return B200MOE_ERR_INVALID_ARGUMENT;
  Workspace ws;
  int rc = bind_workspace(T, e_local, hidden, inter, workspace, workspace_bytes, &ws);
  if (rc != B200MOE_OK) return rc;
  if (hidden_row_stride < hidden || hidden_row_stride % 16 != 0 ||
      reinterpret_cast<uintptr_t>(hidden_states) % 16 != 0 || reinterpret_cast<uintptr_t>(w1) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(w2) % 16 != 0 || reinterpret_cast<uintptr_t>(out_bf16) % 16 != 0 ||
      out_row_stride < hidden || out_row_stride % 8 != 0)
    return B200MOE_ERR_MISALIGNED;
  if (T == 0) return B200MOE_OK;
  int num_sms = 0;
  if ((rc = ensure_device(&num_sms)) != B200MOE_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  const int nt = decode_tile(T, hidden, inter);
  // A call of at most 8 tokens that the one-block front kernel routed and placed runs no gather pass: its GEMM1
  // fetches the token rows and their scales where the caller keeps them (and zeroes the output rows).  Measured
  // with inputs cold in HBM: -4 us at 1 token, -2 at 4, but +2..4 at 16 tokens with 4 rows (56 separate 128-byte
  // pieces per row instead of one coalesced pass), hence the limit.
  const bool direct_a = placed && nt == 16 && T <= kDirectRowsMaxTokens && !segs && !segs_dev;
  // (the gather kernel also zeroes the output rows, which GEMM2's epilogue adds into)
  if (!direct_a)
    CUDA_TRY(launch_permute(ws, topk_ids, ids_row_stride, topk_w, w_row_stride, hidden_states, hidden_row_stride,
                            hidden_scale, scale_stride_t, scale_stride_kb, T, e_local, local_expert_offset, hidden,
                            kTileM, num_sms, st, placed, segs, out_bf16, out_row_stride, segs_dev, n_rows_dev));

  GemmParams g1;
  memset(&g1, 0, sizeof(g1));
  if (direct_a) {   // the caller's rows, one row per box
    if ((rc = make_tmap(&g1.tmap_a, hidden_states, (uint64_t)T, (uint64_t)hidden, (uint64_t)hidden_row_stride, 1)) !=
        B200MOE_OK)
      return rc;
  } else if ((rc = make_tmap(&g1.tmap_a, ws.base + ws.L.a_packed, (uint64_t)ws.L.m_cap, (uint64_t)hidden,
                             (uint64_t)hidden, nt ? nt : kTileM)) != B200MOE_OK) {
    return rc;
  }
  // one box = 128 gate rows + the matching 128 up rows (decode kernels: 64 + 64)
  if ((rc = make_tmap_gate_up(&g1.tmap_b, w1, (uint64_t)e_local, (uint64_t)inter, (uint64_t)hidden, nt ? 64 : 128)) !=
      B200MOE_OK)
    return rc;
  g1.meta = ws.at<int>(ws.L.meta);
  g1.tile_expert = ws.at<int>(ws.L.tile_expert);
  g1.row_token = ws.at<int>(ws.L.row_token);
  g1.a_scale = ws.at<float>(ws.L.a_scale);
  g1.b_scale = w1_scale;
  g1.m_cap = ws.L.m_cap;
  g1.n_per_expert = 2 * inter;
  g1.kblocks = hidden / kBlockK;
  g1.n_tiles = nt ? inter / 64 : inter / 128;
  g1.expert_count = ws.at<int>(ws.L.expert_count);
  g1.inter = inter;
  g1.hidden = hidden;
  g1.act = ws.at<__half>(ws.L.act);
  g1.row_amax = ws.at<unsigned>(ws.L.row_amax);
  g1.tile_done = ws.at<int>(ws.L.tile_done);
  g1.act_q_out = ws.at<uint8_t>(ws.L.act_q);
  g1.row_scale_out = ws.at<float>(ws.L.row_scale);
  g1.direct_a = direct_a ? 1 : 0;
  g1.zero_tokens = direct_a ? T : 0;   // no gather pass: GEMM1's CTAs zero the output rows that GEMM2 adds into
  g1.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  g1.out_stride = out_row_stride;
  g1.hscale = hidden_scale;
  g1.hs_stride_t = scale_stride_t;
  g1.hs_stride_kb = scale_stride_kb;
  g1.status = ws.at<int>(ws.L.status);
  g1.status_mirror = g_status_mirror;
  g1.splitk_scratch = ws.at<float>(ws.L.splitk_scratch);
  g1.splitk_count = ws.at<int>(ws.L.splitk_count);
  // B200MOE_PROF=1: CTA 0 adds cycle counters into the padding after `meta`
  // (GEMM1: 9 x u64 at meta+32, GEMM2: at meta+136); cleared with the counters each call.
  static const bool prof_on = getenv("B200MOE_PROF") != nullptr;
  g1.prof = prof_on ? ws.at<unsigned long long>(ws.L.meta + 32) : nullptr;
  g1.trace = prof_on ? ws.at<unsigned long long>(ws.L.trace) : nullptr;
  if (g_prof_start) CUDA_TRY(cudaEventRecord(g_prof_start, st));
  {
    cudaError_t le = nt ? launch_decode_gemm(1, nt, g1, num_sms, st) : launch_grouped_gemm(1, g1, num_sms, st);
    cudaEvent_t stop = g_prof_stop;
    g_prof_start = g_prof_stop = nullptr;   // one shot, whatever happens next
    if (le != cudaSuccess) return cuda_fail(le, "GEMM1 launch");
    if (stop) CUDA_TRY(cudaEventRecord(stop, st));
  }

  // decode sizes requantise inside GEMM1 (the CTA that stores an expert's last weight slab); the 128-row tiles
  // need a pass of their own (see gemm.cu)
  if (!nt) CUDA_TRY(launch_requant(ws, inter, num_sms, st));

  GemmParams g2;
  memset(&g2, 0, sizeof(g2));
  if ((rc = make_tmap(&g2.tmap_a, ws.base + ws.L.act_q, (uint64_t)ws.L.m_cap, (uint64_t)inter, (uint64_t)inter,
                      nt ? nt : kTileM)) != B200MOE_OK)
    return rc;
  if ((rc = make_tmap(&g2.tmap_b, w2, (uint64_t)e_local * hidden, (uint64_t)inter, (uint64_t)inter,
                      nt ? 128 : 256)) != B200MOE_OK)   // the whole B tile (decode: the 128-row slab) in one box
    return rc;
  g2.meta = g1.meta;
  g2.tile_expert = g1.tile_expert;
  g2.row_token = g1.row_token;
  g2.b_scale = w2_scale;
  g2.m_cap = ws.L.m_cap;
  g2.n_per_expert = hidden;
  g2.kblocks = inter / kBlockK;
  g2.n_tiles = nt ? hidden / 128 : hidden / 256;
  g2.expert_count = g1.expert_count;
  g2.inter = inter;
  g2.hidden = hidden;
  g2.row_scale = ws.at<float>(ws.L.row_scale);
  g2.row_weight = ws.at<float>(ws.L.row_weight);
  g2.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  g2.out_stride = out_row_stride;
  g2.status = g1.status;
  g2.status_mirror = g1.status_mirror;
  g2.splitk_scratch = g1.splitk_scratch;
  g2.splitk_count = g1.splitk_count + kSplitKSlots;
  g2.prof = prof_on ? ws.at<unsigned long long>(ws.L.meta + 136) : nullptr;
  g2.trace = prof_on ? ws.at<unsigned long long>(ws.L.trace) + 8 * 64 : nullptr;
  if (nt) CUDA_TRY(launch_decode_gemm(2, nt, g2, num_sms, st));
  else CUDA_TRY(launch_grouped_gemm(2, g2, num_sms, st));

  // nothing follows GEMM2: its epilogue added every packed row into its token's output row
  return B200MOE_OK;
}

int b200moe_experts(const int32_t* topk_ids, int64_t ids_row_stride, const float* topk_w, int64_t w_row_stride,
                    const uint8_t* hidden_states, int64_t hidden_row_stride, const float* hidden_scale,
                    int64_t scale_stride_t, int64_t scale_stride_kb, const uint8_t* w1, const float* w1_scale,
                    const uint8_t* w2, const float* w2_scale, int T, int e_local, int local_expert_offset,
                    int hidden, int inter, void* workspace, size_t workspace_bytes, void* out_bf16,
                    int64_t out_row_stride, void* stream) {
  return experts_impl(topk_ids, ids_row_stride, topk_w, w_row_stride, hidden_states, hidden_row_stride, hidden_scale,
                      scale_stride_t, scale_stride_kb, w1, w1_scale, w2, w2_scale, T, e_local, local_expert_offset,
                      hidden, inter, workspace, workspace_bytes, out_bf16, out_row_stride, stream, false);
}

int b200moe_run(const void* logits, int logits_dtype, const void* bias, int bias_dtype, const uint8_t* hidden_states,
                int64_t hidden_row_stride, const float* hidden_scale, int64_t scale_stride_t,
                int64_t scale_stride_kb, const uint8_t* w1, const float* w1_scale, const uint8_t* w2,
                const float* w2_scale, int T, int e_local, int local_expert_offset, float routed_scaling_factor,
                int hidden, int inter, void* workspace, size_t workspace_bytes, void* out_bf16,
                int64_t out_row_stride, void* stream) {
  Workspace ws;
  int rc = bind_workspace(T, e_local, hidden, inter, workspace, workspace_bytes, &ws);
  if (rc != B200MOE_OK) return rc;
  if (T == 0) return B200MOE_OK;
  int32_t* ids = ws.at<int32_t>(ws.L.topk_ids);
  float* w = ws.at<float>(ws.L.topk_w);
  // Decode-size calls: routing, scan and placement in one block (B200MOE_FRONT=0: the separate kernels).
  static const bool front_on = [] {
    const char* v = getenv("B200MOE_FRONT");
    return !(v && v[0] == '0');
  }();
  if (front_on && T <= kFrontSmallMaxTokens) {
    if (!logits || !bias) return B200MOE_ERR_INVALID_ARGUMENT;
    if ((logits_dtype != B200MOE_F32 && logits_dtype != B200MOE_BF16) ||
        (bias_dtype != B200MOE_F32 && bias_dtype != B200MOE_BF16))
      return B200MOE_ERR_INVALID_ARGUMENT;
    if (local_expert_offset < 0 || local_expert_offset + e_local > kNumExperts) return B200MOE_ERR_INVALID_ARGUMENT;
    int num_sms = 0;
    if ((rc = ensure_device(&num_sms)) != B200MOE_OK) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // (no memset: this kernel clears the call's counters itself)
    CUDA_TRY(launch_route_place_small(ws, logits, logits_dtype, bias, bias_dtype, T, routed_scaling_factor,
                                      local_expert_offset, e_local, kTileM, st));
    return experts_impl(ids, kTopK, w, kTopK, hidden_states, hidden_row_stride, hidden_scale, scale_stride_t,
                        scale_stride_kb, w1, w1_scale, w2, w2_scale, T, e_local, local_expert_offset, hidden, inter,
                        workspace, workspace_bytes, out_bf16, out_row_stride, stream, true);
  }
  rc = b200moe_route(logits, logits_dtype, bias, bias_dtype, T, routed_scaling_factor, local_expert_offset, e_local,
                     hidden, inter, ids, w, workspace, workspace_bytes, stream);
  if (rc != B200MOE_OK) return rc;
  return b200moe_experts(ids, kTopK, w, kTopK, hidden_states, hidden_row_stride, hidden_scale, scale_stride_t,
                         scale_stride_kb, w1, w1_scale, w2, w2_scale, T, e_local, local_expert_offset, hidden, inter,
                         workspace, workspace_bytes, out_bf16, out_row_stride, stream);
}

int b200moe_read_status(const void* workspace, void* stream, int32_t* detail) {
  if (!workspace) return B200MOE_ERR_INVALID_ARGUMENT;
  int32_t host[4] = {0, 0, 0, 0};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CUDA_TRY(cudaMemcpyAsync(host, workspace, sizeof(host), cudaMemcpyDeviceToHost, st));
  CUDA_TRY(cudaStreamSynchronize(st));
  if (detail) memcpy(detail, host, sizeof(host));
  return host[kStatusCode];
}

int b200moe_selftest_wait_timeout(void* status_int4, void* stream) {
  if (!status_int4) return B200MOE_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CUDA_TRY(cudaMemsetAsync(status_int4, 0, 16, st));
  CUDA_TRY(launch_wait_timeout_selftest(reinterpret_cast<int*>(status_int4), st));
  return B200MOE_OK;
}

int b200moe_ep_pack(const int32_t* topk_ids, const float* topk_w, const uint8_t* hidden_states,
                    int64_t hidden_row_stride, const float* hidden_scale, int64_t scale_stride_t,
                    int64_t scale_stride_kb, int T, int hidden, int world, uint8_t* send_rows, int32_t* dest_counts,
                    int32_t* send_slot, void* stream) {
  if (!dest_counts || T < 0) return B200MOE_ERR_INVALID_ARGUMENT;
  if (T > 0 && (!topk_ids || !topk_w || !send_rows || !send_slot || !hidden_states || !hidden_scale))
    return B200MOE_ERR_INVALID_ARGUMENT;   // an empty batch may come with null (zero-sized) buffers
  if (world != 1 && world != 2 && world != 4 && world != 8) return B200MOE_ERR_UNSUPPORTED_SHAPE;
  if (hidden < 512 || hidden % 512 != 0) return B200MOE_ERR_UNSUPPORTED_SHAPE;   // keeps send rows 16-byte aligned
  if (hidden_row_stride % 16 != 0 || reinterpret_cast<uintptr_t>(hidden_states) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(send_rows) % 16 != 0)
    return B200MOE_ERR_MISALIGNED;
  int num_sms = 0;
  int rc = ensure_device(&num_sms);
  if (rc != B200MOE_OK) return rc;
  CUDA_TRY(launch_ep_pack(topk_ids, topk_w, hidden_states, hidden_row_stride, hidden_scale, scale_stride_t,
                          scale_stride_kb, T, hidden, world, send_rows, dest_counts, send_slot, num_sms,
                          reinterpret_cast<cudaStream_t>(stream)));
  return B200MOE_OK;
}

int b200moe_ep_local_experts(const void* const* send_base, const int32_t* from_peers, int world, int cap_rows,
                             int64_t row_bytes, const uint8_t* w1, const float* w1_scale, const uint8_t* w2,
                             const float* w2_scale, int e_local, int local_expert_offset, int hidden, int inter,
                             void* workspace, size_t workspace_bytes, void* out_bf16, int64_t out_row_stride,
                             void* stream) {
  if (!send_base || !from_peers || cap_rows < 0) return B200MOE_ERR_INVALID_ARGUMENT;
  if (world != 1 && world != 2 && world != 4 && world != 8) return B200MOE_ERR_UNSUPPORTED_SHAPE;
  if (row_bytes < hidden + 4 * (hidden / kBlockK) + 64 || row_bytes % 16 != 0) return B200MOE_ERR_MISALIGNED;
  if (local_expert_offset < 0 || local_expert_offset + e_local > kNumExperts) return B200MOE_ERR_INVALID_ARGUMENT;
  PeerBases bases;
  memset(&bases, 0, sizeof(bases));
  for (int s = 0; s < world; ++s) {
    if (!send_base[s]) return B200MOE_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(send_base[s]) % 16 != 0) return B200MOE_ERR_MISALIGNED;
    bases.base[s] = reinterpret_cast<const uint8_t*>(send_base[s]);
  }
  Workspace ws;
  int rc = bind_workspace(cap_rows, e_local, hidden, inter, workspace, workspace_bytes, &ws);
  if (rc != B200MOE_OK) return rc;
  if (cap_rows == 0) return B200MOE_OK;
  int num_sms = 0;
  if ((rc = ensure_device(&num_sms)) != B200MOE_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if ((rc = clear_counters(ws, e_local, st)) != B200MOE_OK) return rc;
  RowSegments* segs_dev = ws.at<RowSegments>(ws.L.ep_segments);
  int* n_rows_dev = ws.at<int>(ws.L.ep_segments + 192);
  static_assert(sizeof(RowSegments) <= 192, "the segment table and the row count share 256 bytes");
  int32_t* ids = ws.at<int32_t>(ws.L.topk_ids);
  float* w = ws.at<float>(ws.L.topk_w);
  CUDA_TRY(launch_ep_segments_pull(bases, from_peers, world, row_bytes, cap_rows, hidden, segs_dev, n_rows_dev, ids, w,
                                   num_sms, st));
  CUDA_TRY(launch_count(ids, kTopK, cap_rows, local_expert_offset, e_local, ws.at<int>(ws.L.chunk_counts), num_sms, st,
                        n_rows_dev));
  return experts_impl(ids, kTopK, w, kTopK, nullptr, hidden, nullptr, 0, 0, w1, w1_scale, w2, w2_scale, cap_rows,
                      e_local, local_expert_offset, hidden, inter, workspace, workspace_bytes, out_bf16, out_row_stride,
                      stream, false, nullptr, segs_dev, n_rows_dev);
}

int b200moe_ep_combine_peers(const void* const* partial_bf16, const int32_t* row_start, const int32_t* send_slot,
                             int T, int hidden, int world, void* out_bf16, void* stream) {
  if (T < 0) return B200MOE_ERR_INVALID_ARGUMENT;
  if (T == 0) return B200MOE_OK;
  if (!partial_bf16 || !row_start || !send_slot || !out_bf16) return B200MOE_ERR_INVALID_ARGUMENT;
  if (world != 1 && world != 2 && world != 4 && world != 8) return B200MOE_ERR_UNSUPPORTED_SHAPE;
  if (hidden < 8 || hidden % 8 != 0) return B200MOE_ERR_UNSUPPORTED_SHAPE;
  PeerPartials peers;
  memset(&peers, 0, sizeof(peers));
  for (int d = 0; d < world; ++d) {
    if (!partial_bf16[d] || reinterpret_cast<uintptr_t>(partial_bf16[d]) % 16 != 0) return B200MOE_ERR_MISALIGNED;
    peers.partial[d] = partial_bf16[d];
  }
  if (reinterpret_cast<uintptr_t>(out_bf16) % 16 != 0) return B200MOE_ERR_MISALIGNED;
  int num_sms = 0;
  int rc = ensure_device(&num_sms);
  if (rc != B200MOE_OK) return rc;
  CUDA_TRY(launch_ep_combine_peers(peers, row_start, send_slot, T, hidden, world, out_bf16, num_sms,
                                   reinterpret_cast<cudaStream_t>(stream)));
  return B200MOE_OK;
}

int b200moe_ep_combine(const void* returned_bf16, const int32_t* send_slot, const int32_t* dest_counts, int T,
                       int hidden, int world, void* out_bf16, void* stream) {
  if (T < 0) return B200MOE_ERR_INVALID_ARGUMENT;
  if (T == 0) return B200MOE_OK;
  if (!returned_bf16 || !send_slot || !dest_counts || !out_bf16) return B200MOE_ERR_INVALID_ARGUMENT;
  if (world != 1 && world != 2 && world != 4 && world != 8) return B200MOE_ERR_UNSUPPORTED_SHAPE;
  if (hidden < 8 || hidden % 8 != 0) return B200MOE_ERR_UNSUPPORTED_SHAPE;
  if (reinterpret_cast<uintptr_t>(returned_bf16) % 16 != 0 || reinterpret_cast<uintptr_t>(out_bf16) % 16 != 0)
    return B200MOE_ERR_MISALIGNED;
  int num_sms = 0;
  int rc = ensure_device(&num_sms);
  if (rc != B200MOE_OK) return rc;
  CUDA_TRY(launch_ep_combine(returned_bf16, send_slot, dest_counts, T, hidden, world, out_bf16, num_sms,
                             reinterpret_cast<cudaStream_t>(stream)));
  return B200MOE_OK;
}

}  // extern "C"
