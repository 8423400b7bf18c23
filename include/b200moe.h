/*
 * b200moe — C ABI of the B200-native FP8 block-scale fused-MoE layer.
 *
 * The library replaces the device side of the reference project's entry point
 *   run(routing_logits, routing_bias, hidden_states, hidden_states_scale,
 *       gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale,
 *       local_expert_offset, routed_scaling_factor) -> bf16 [T, hidden]
 * (solution/python/kernel.py:575-648) and the pybind module that entry point
 * drives (solution/python/moe_fused.cu:1152-1184, solution/python/moe_gemm.cu).
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless its comment says "host";
 *  - `stream` is a cudaStream_t passed as void* (0 = legacy default stream);
 *    every call is asynchronous on that stream and allocates nothing: all
 *    scratch lives in the caller-provided workspace;
 *  - every function returns a b200moe_status (0 = ok, negative = error) and
 *    writes nothing on an argument error;
 *  - device-side waits are bounded; a kernel that gives up records a negative
 *    code in the workspace status word, read back by b200moe_read_status.
 *
 * Fixed routing constants (DeepSeek-V3 no-aux routing): 256 experts in 8 groups
 * of 32, top-4 groups, top-8 experts.  `hidden` must be a multiple of 256 and
 * `inter` a multiple of 128; the benchmark shape is hidden 7168, inter 2048.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200MOE_API __attribute__((visibility("default")))
#else
#define B200MOE_API
#endif

#define B200MOE_NUM_EXPERTS 256
#define B200MOE_TOP_K 8

typedef enum b200moe_status {
  B200MOE_OK = 0,
  B200MOE_ERR_INVALID_ARGUMENT = -1,   /* null pointer, negative extent, bad dtype tag */
  B200MOE_ERR_UNSUPPORTED_SHAPE = -2,  /* hidden % 256, inter % 128, e_local not in 1..256, ... */
  B200MOE_ERR_WORKSPACE_TOO_SMALL = -3,
  B200MOE_ERR_CUDA = -4,               /* a CUDA runtime/driver call failed (see b200moe_last_cuda_error) */
  B200MOE_ERR_DEVICE_TIMEOUT = -5,     /* a bounded device-side wait gave up */
  B200MOE_ERR_MISALIGNED = -6          /* pointer or stride not aligned as documented */
} b200moe_status;

typedef enum b200moe_dtype {
  B200MOE_F32 = 0,
  B200MOE_BF16 = 1
} b200moe_dtype;

/* Byte offsets of the intermediates inside a workspace, for tests and tools.
 * Replaces the reference's dict of preallocated tensors
 * (solution/python/kernel.py:208-329, `_get_workspace`). */
typedef struct b200moe_ws_layout {
  uint64_t total_bytes;
  uint64_t status;        /* int32[16]: [0] status code, [1] detail, [2..] debug */
  uint64_t meta;          /* int32[8]: [0] m_tiles, [1] padded rows, [2] rows with a local expert, [3] pad granularity */
  uint64_t splitk_count;  /* int32[2][64]: arrivals per (GEMM, weight slab) when a decode GEMM splits K; cleared per call */
  uint64_t tile_done;     /* int32[max_tiles]: decode GEMM1, weight slabs of each expert tile already stored; cleared per call */
  uint64_t chunk_counts;  /* int32[n_chunks][e_local] */
  uint64_t chunk_base;    /* int32[n_chunks][e_local] */
  uint64_t expert_count;  /* int32[e_local] */
  uint64_t expert_row0;   /* int32[e_local+1]: first (128-padded) row of each expert */
  uint64_t tile_expert;   /* int32[max_tiles] */
  uint64_t row_token;     /* int32[m_cap]: token of each packed row, -1 for padding */
  uint64_t row_weight;    /* float[m_cap] */
  uint64_t a_packed;      /* uint8[m_cap][hidden] e4m3 rows in expert order */
  uint64_t a_scale;       /* float[hidden/128][m_cap] */
  uint64_t act;           /* fp16[m_cap][inter] SwiGLU output */
  uint64_t row_amax;      /* uint32[m_cap]: bits of max|act| per row */
  uint64_t act_q;         /* uint8[m_cap][inter] e4m3 */
  uint64_t row_scale;     /* float[m_cap] */
  uint64_t tok_rows;      /* int32[T][8]: packed row of (token,k), -1 if the expert is not local */
  uint64_t topk_ids;      /* int32[T][8]  (used by b200moe_run) */
  uint64_t topk_w;        /* float[T][8]  (used by b200moe_run) */
  uint64_t trace;         /* uint64[2][64][8]: cycle stamps written when B200MOE_PROF is set */
  uint64_t splitk_scratch; /* float[64][4][16][128]: partial sums of a decode GEMM whose K range is split over CTAs */
  uint64_t ep_segments;    /* 256 bytes: segment table and row count of b200moe_ep_local_experts (device-written) */
  int32_t m_cap;          /* capacity in packed rows (multiple of 128) */
  int32_t max_tiles;
  int32_t n_chunks;
  int32_t chunk_tokens;
} b200moe_ws_layout;

/* Library ABI version (bumped on any signature change). */
B200MOE_API int b200moe_version(void);

/* Text for a status code; never NULL.  Host pointer, static storage. */
B200MOE_API const char* b200moe_status_string(int status);

/* Text of the last CUDA error seen by this thread inside the library (host pointer). */
B200MOE_API const char* b200moe_last_cuda_error(void);

/* Workspace size and layout for up to T tokens and e_local local experts.
 * Replaces kernel.py:208-329.  `layout` may be NULL. */
B200MOE_API int b200moe_workspace_layout(int T, int e_local, int hidden, int inter,
                             b200moe_ws_layout* layout /* host */);

/* Routing: replaces `fused_route_topk` (solution/python/moe_fused.cu:568-725) and the
 * count pass of `fused_dispatch` (moe_fused.cu:866-881).
 * logits [T,256] (fp32 or bf16, row-major), bias [256] (bf16 or fp32).
 * Writes topk_ids int32 [T,8] (global ids, descending score, lowest id first on ties),
 * topk_w float [T,8], and adds the per-chunk histogram of local experts into the
 * workspace (which this call first clears). */
B200MOE_API int b200moe_route(const void* logits, int logits_dtype, const void* bias, int bias_dtype,
                  int T, float routed_scaling_factor, int local_expert_offset, int e_local,
                  int hidden, int inter,
                  int32_t* topk_ids, float* topk_w,
                  void* workspace, size_t workspace_bytes, void* stream);

/* Routing without a workspace, for callers that are not allowed to allocate device memory
 * (an engine plugin's enqueue hook, a serving loop with a frozen memory budget, code that
 * must avoid the device-wide synchronisation of cudaMalloc).  No counterpart in the
 * reference, whose host code allocates freely (solution/python/kernel.py:208-329).
 * Same routing and outputs as b200moe_route (topk_ids int32 [T,8], topk_w float [T,8]);
 * in addition expert_counts int32[e_local] receives the number of (token,k) pairs per local
 * expert.  The scratch this needs (a per-chunk histogram) is a fixed 256 KiB array inside
 * the library image, which every GPU that loads the library holds until the process exits.
 *  - at most b200moe_route_static_max_tokens() = 65536 tokens per call; larger T returns
 *    B200MOE_ERR_UNSUPPORTED_SHAPE (text in b200moe_route_static_error) and launches nothing;
 *  - calls nothing that allocates (no cudaMalloc/cudaFree, no torch);
 *  - the first call on each device resolves the array's device address
 *    (cudaGetSymbolAddress, with that device current): make that first call before any
 *    stream capture begins;
 *  - all calls on a device share the array: calls that can overlap on the GPU (different
 *    streams without ordering) race on it and give wrong counts. */
B200MOE_API int b200moe_route_static(const void* logits, int logits_dtype, const void* bias, int bias_dtype,
                         int T, float routed_scaling_factor, int local_expert_offset, int e_local,
                         int32_t* topk_ids, float* topk_w, int32_t* expert_counts, void* stream);
B200MOE_API int b200moe_route_static_max_tokens(void);
B200MOE_API const char* b200moe_route_static_error(void);

/* Histogram of local experts for routing that was computed elsewhere (the
 * expert-parallel path, where rows arrive with their ids).  Clears and fills the same
 * workspace counters as b200moe_route.  ids_row_stride in int32 elements. */
B200MOE_API int b200moe_count(const int32_t* topk_ids, int64_t ids_row_stride, int T,
                  int local_expert_offset, int e_local, int hidden, int inter,
                  void* workspace, size_t workspace_bytes, void* stream);

/* Expert MLPs + routing-weighted reduce for given routing; the counters in the workspace must have been
 * filled by b200moe_route or b200moe_count for the same ids on the same stream.  The call zeroes the T
 * output rows itself and GEMM2's epilogue adds every (token, expert) row into its token's row in bf16
 * (no combine pass; the sum order follows tile completion, so two runs agree to a few bf16 steps).
 * Replaces `fused_dispatch`, `fused_gather_hidden_scales`, `moe_blockwise_grouped_mm_v2`
 * (x2), `swiglu_fp8_requant*`, `weighted_scatter` / `reduce_scatter_unweighted_fused`
 * (moe_fused.cu:131-542, 736-1150; moe_gemm.cu:527-654).
 *  hidden_states  e4m3 [T,hidden], row stride `hidden_row_stride` bytes (multiple of 16)
 *  hidden_scale   fp32, element (t,kb) at hidden_scale[t*scale_stride_t + kb*scale_stride_kb]
 *  w1 e4m3 [e_local,2*inter,hidden], w1_scale fp32 [e_local,2*inter/128,hidden/128]
 *  w2 e4m3 [e_local,hidden,inter],   w2_scale fp32 [e_local,hidden/128,inter/128]
 *  out bf16 [T,hidden], row stride `out_row_stride` elements. */
B200MOE_API int b200moe_experts(const int32_t* topk_ids, int64_t ids_row_stride,
                    const float* topk_w, int64_t w_row_stride,
                    const uint8_t* hidden_states, int64_t hidden_row_stride,
                    const float* hidden_scale, int64_t scale_stride_t, int64_t scale_stride_kb,
                    const uint8_t* w1, const float* w1_scale,
                    const uint8_t* w2, const float* w2_scale,
                    int T, int e_local, int local_expert_offset, int hidden, int inter,
                    void* workspace, size_t workspace_bytes,
                    void* out_bf16, int64_t out_row_stride, void* stream);

/* The whole layer: b200moe_route followed by b200moe_experts, ids/weights kept in the
 * workspace.  This is what the reference's `run` does per call (kernel.py:575-636). */
B200MOE_API int b200moe_run(const void* logits, int logits_dtype, const void* bias, int bias_dtype,
                const uint8_t* hidden_states, int64_t hidden_row_stride,
                const float* hidden_scale, int64_t scale_stride_t, int64_t scale_stride_kb,
                const uint8_t* w1, const float* w1_scale,
                const uint8_t* w2, const float* w2_scale,
                int T, int e_local, int local_expert_offset, float routed_scaling_factor,
                int hidden, int inter,
                void* workspace, size_t workspace_bytes,
                void* out_bf16, int64_t out_row_stride, void* stream);

/* Synchronises `stream` and reads the workspace status word: returns B200MOE_OK or the
 * code a kernel recorded; `detail` (host, may be NULL) receives int32[4] of context. */
B200MOE_API int b200moe_read_status(const void* workspace, void* stream, int32_t* detail /* host */);

/* Asynchronous failure reporting (the reference's calls cannot fail on the device: it has no
 * device-side waits, solution/python/kernel.py:575-639 checks nothing after its launches): the
 * calling thread's following b200moe_run / b200moe_experts* calls hand `host_mapped_int4` to their
 * GEMM kernels, and a CTA that gives up on a bounded wait copies the status word (code, detail)
 * there besides recording it in the workspace.  The pointer must be device-accessible host memory
 * (pinned, on a unified-addressing system) of at least four int32 and stay valid while such calls
 * are in flight; NULL switches the mirror off.  The host looks at it whenever it likes, no copy or
 * synchronisation per call. */
B200MOE_API int b200moe_set_status_mirror(void* host_mapped_int4);

/* Measurement hook (no counterpart in the reference, whose per-stage timing replays the
 * pipeline stage by stage from Python, experiments/fast_bench/bench_server.py:470-632):
 * the calling thread's next b200moe_experts / b200moe_run records `start_event` before and
 * `stop_event` after its GEMM1 launch (cudaEvent_t as void*, either may be NULL), once. */
B200MOE_API int b200moe_profile_next_gemm1(void* start_event, void* stop_event);

/* Failure-detection self-test (the reference has no device-side waits of its own; its
 * errors are CUTLASS status checks, moe_gemm.cu:296-306): launches a one-block kernel whose
 * thread waits ~1 ms on a barrier that nothing signals.  status_int4 (device, int32[4],
 * cleared first) receives [0] = B200MOE_ERR_DEVICE_TIMEOUT, [1] = 99 (where), [2] = 0 (the
 * wait returned false), [3] = 1 (abort flag set).  The context stays usable. */
B200MOE_API int b200moe_selftest_wait_timeout(void* status_int4, void* stream);

/* Number of kernels b200moe_run launches for this problem (memsets not counted). */
B200MOE_API int b200moe_launches_per_run(int T, int e_local);

/* ---- expert parallelism (no counterpart in the reference, which only consumes
 * local_expert_offset, kernel.py:591; rows travel by NCCL all-to-all between these) ---- */

/* For every destination rank d (experts [d*256/world, (d+1)*256/world)), the tokens that
 * chose an expert of d, in ascending token order: one send row per (token, d).
 * send_rows: [rows][row_bytes] with row_bytes = hidden + 4*hidden/128 + 64:
 *   e4m3 payload | fp32 scales | int32 ids[8] | fp32 weights[8];
 * destination segments are compact and in rank order (segment d starts at row
 * dest_counts[0] + ... + dest_counts[d-1]); capacity needed: T * min(4, world) rows.
 * dest_counts int32[world] (filled); send_slot int32[T][world] = row index of (token,d)
 * inside d's segment, or -1.  hidden must be a multiple of 512. */
B200MOE_API int b200moe_ep_pack(const int32_t* topk_ids, const float* topk_w,
                    const uint8_t* hidden_states, int64_t hidden_row_stride,
                    const float* hidden_scale, int64_t scale_stride_t, int64_t scale_stride_kb,
                    int T, int hidden, int world,
                    uint8_t* send_rows, int32_t* dest_counts, int32_t* send_slot, void* stream);

/* out[t,:] = bf16( sum over d with send_slot[t][d] >= 0 of fp32(partial_d[row]) ), ascending d.
 * returned: bf16 rows in the send-buffer order of b200moe_ep_pack (same dest_counts). */
B200MOE_API int b200moe_ep_combine(const void* returned_bf16, const int32_t* send_slot,
                       const int32_t* dest_counts, int T, int hidden, int world,
                       void* out_bf16, void* stream);

/* ---- the same exchange over mapped peer memory (NVLink loads inside the kernels instead of
 * NCCL all-to-all; no counterpart in the reference) ----
 * The local expert pipeline of one expert-parallel step, reading its rows where the ranks packed them
 * (dispatch and gather in one pass) and with every row count staying on the device.
 *   send_base   HOST array of `world` pointers: rank s's send buffer (b200moe_ep_pack layout) as mapped
 *               into this process (this GPU's own memory for s == this rank).
 *   from_peers  DEVICE int32[world][3], what the small all-to-all between the ranks delivered: row s =
 *               (rows rank s has for this rank, index of their first row in rank s's send buffer, unused).
 *   cap_rows    the largest total the ranks can send here (world x the exchange's token capacity); the
 *               workspace is sized for it: b200moe_workspace_layout(cap_rows, ...).
 * Builds the segment table on the device (virtual row order: rank 0's rows, then rank 1's, ...), copies
 * the rows' (ids, weights) trailers, counts, places, gathers and runs both GEMMs; out row r belongs to
 * virtual row r.  Nothing is read back by the host.  The caller orders the kernels between ranks: the
 * senders' pack kernels must have completed (the exchange that delivers from_peers runs after them), and
 * a sender must not repack before the readers are done. */
B200MOE_API int b200moe_ep_local_experts(const void* const* send_base, const int32_t* from_peers, int world,
                        int cap_rows, int64_t row_bytes,
                        const uint8_t* w1, const float* w1_scale, const uint8_t* w2, const float* w2_scale,
                        int e_local, int local_expert_offset, int hidden, int inter,
                        void* workspace, size_t workspace_bytes,
                        void* out_bf16, int64_t out_row_stride, void* stream);

/* b200moe_ep_combine with the return exchange folded in: partial_bf16[d] (HOST array of `world`
 * pointers) is rank d's output buffer of b200moe_ep_local_experts as mapped here, row_start[d]
 * (DEVICE int32[world]) the first row of this rank's segment inside it.  The caller makes sure
 * every rank's expert kernels have completed (e.g. the exchange that delivers row_start runs
 * after them). */
B200MOE_API int b200moe_ep_combine_peers(const void* const* partial_bf16, const int32_t* row_start,
                        const int32_t* send_slot, int T, int hidden, int world,
                        void* out_bf16, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* B200MOE_H_ */
