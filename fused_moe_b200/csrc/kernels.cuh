// Launchers of the device kernels (one translation unit each), called from capi.cu.
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"

namespace b200moe {

cudaError_t launch_route(const void* logits, int logits_dtype, const void* bias, int bias_dtype, int T, float rsf,
                         int local_off, int e_local, int32_t* ids, float* w, int* chunk_counts, int num_sms,
                         cudaStream_t stream);

// `n_rows_dev` (optional, device): the number of rows actually present, when the host only knows the
// capacity T (expert-parallel calls whose row counts never leave the device).
cudaError_t launch_count(const int32_t* ids, long long row_stride, int T, int local_off, int e_local,
                         int* chunk_counts, int num_sms, cudaStream_t stream, const int* n_rows_dev = nullptr);

// Rows that live in up to eight separate buffers (the send buffers of the ranks of an
// expert-parallel group, this GPU's own or its peers' mapped memory): row r of the virtual
// concatenation belongs to segment s with start[s] <= r < start[s+1] and sits at
// base[s] + (r - start[s]) * row_bytes.  n == 0: not used.
struct RowSegments {
  int n;
  int start[9];
  const uint8_t* base[8];
  long long row_bytes;
  __host__ __device__ const uint8_t* row(int r) const {
    int s = 0;
#pragma unroll
    for (int i = 1; i < 8; ++i)
      if (i < n && r >= start[i]) s = i;
    return base[s] + (size_t)(r - start[s]) * row_bytes;
  }
};

// `placed`: scan and place already ran (launch_route_place_small); only the gather is launched.
cudaError_t launch_permute(const Workspace& ws, const int32_t* ids, long long ids_stride, const float* w,
                           long long w_stride, const uint8_t* hidden, long long hidden_row_stride,
                           const float* hscale, long long sstride_t, long long sstride_kb, int T, int e_local,
                           int local_off, int hidden_dim, int pad_rows, int num_sms, cudaStream_t stream,
                           bool placed, const RowSegments* segs, void* out_bf16, long long out_row_stride,
                           const RowSegments* segs_dev = nullptr, const int* n_rows_dev = nullptr);

// Routing + scan + placement of at most kFrontSmallMaxTokens tokens in one block (front_small.cu);
// writes the workspace's own topk_ids / topk_w.
constexpr int kFrontSmallMaxTokens = 32;
cudaError_t launch_route_place_small(const Workspace& ws, const void* logits, int logits_dtype, const void* bias,
                                     int bias_dtype, int T, float rsf, int local_off, int e_local, int pad_rows,
                                     cudaStream_t stream);

// Decode GEMMs split the K range of a weight slab over up to kSplitKMax CTAs when a call has at
// most kSplitKSlots (expert tile, slab) items, i.e. fewer than half of the SMs would stream weights.
constexpr int kSplitKSlots = 64;
constexpr int kSplitKMax = 4;

// Arguments of the two grouped GEMMs.  `tmap_a` covers the packed rows [m_cap][K],
// `tmap_b` the weights viewed as [e_local * N][K]; both e4m3, 128-byte swizzled boxes.
struct GemmParams {
  CUtensorMap tmap_a;
  CUtensorMap tmap_b;
  const int* meta;          // [0] = number of 128-row M tiles
  const int* tile_expert;   // expert of each M tile
  const int* row_token;     // token of each packed row, -1 for padding
  const int* expert_count;  // rows per local expert (decode kernel)
  const float* a_scale;     // GEMM1: [K/128][m_cap] activation scales
  const float* b_scale;     // [e_local][N/128][K/128] weight scales
  int m_cap;
  int n_per_expert;         // weight rows per expert (GEMM1: 2*inter, GEMM2: hidden)
  int kblocks;              // K / 128
  int n_tiles;              // N tiles per M tile
  int inter;
  int hidden;
  __half* act;              // GEMM1 out: [m_cap][inter] fp16
  unsigned* row_amax;       // GEMM1 out: bits of max |act| per row
  int* tile_done;           // decode GEMM1: slabs of each expert tile whose activations are stored (zero at call start)
  uint8_t* act_q_out;       // decode GEMM1 out (the CTA that stores an expert's last slab): [m_cap][inter] e4m3
  float* row_scale_out;     // decode GEMM1 out (same CTA): requantisation scale per row
  const float* row_scale;   // GEMM2 in: requantisation scale per row
  const float* row_weight;  // GEMM2 in: routing weight per row
  __nv_bfloat16* out;       // GEMM2 out: the layer's output rows [T][out_stride], zeroed at call start; every packed
  long long out_stride;     //            row is added into its token's row (bf16 red.global.add)
  // decode GEMM1 without a gather pass: tmap_a covers the caller's hidden states [T][K] with one-row boxes, a row's
  // 1x128 scales are read at hscale[token * hs_stride_t + kb * hs_stride_kb]
  int direct_a;
  int zero_tokens;          // ... and this many rows of `out` are zeroed by GEMM1's CTAs (GEMM2 adds into them)
  const float* hscale;
  long long hs_stride_t, hs_stride_kb;
  int* status;
  int* status_mirror;       // optional host-mapped int32[4]: receives the status word when a CTA gives up on a wait
  float* splitk_scratch;    // decode GEMMs: [kSplitKSlots][kSplitKMax][16][128] partial sums
  int* splitk_count;        // decode GEMMs: arrivals per weight slab, zero at kernel start and end
  unsigned long long* prof;   // optional cycle counters of CTA 0 (null: off)
  unsigned long long* trace;  // optional [64][8] absolute cycle stamps of CTA 0's first K blocks
};

// mode 1: GEMM1 + SwiGLU + row amax; mode 2: GEMM2 + weighted combine.  Tiles of 128 rows x 256 weight rows.
cudaError_t launch_grouped_gemm(int mode, const GemmParams& p, int num_sms, cudaStream_t stream);
cudaError_t configure_grouped_gemm();   // opt-in shared memory sizes, once per process and device
int grouped_gemm_max_kblocks();         // largest K / 128 the kernels' scale panels hold

// Decode sizes (T <= nt, nt 16 or 64): operands swapped, weights on the MMA's M side (gemm_decode.cu).
cudaError_t launch_decode_gemm(int mode, int nt, const GemmParams& p, int num_sms, cudaStream_t stream);
cudaError_t configure_decode_gemm();
int decode_gemm_max_kblocks();          // largest K / 128 its per-warp scale panels hold

cudaError_t launch_wait_timeout_selftest(int* status, cudaStream_t stream);

cudaError_t launch_requant(const Workspace& ws, int inter, int num_sms, cudaStream_t stream);


cudaError_t launch_ep_pack(const int32_t* ids, const float* w, const uint8_t* hidden, long long hidden_row_stride,
                           const float* hscale, long long sstride_t, long long sstride_kb, int T, int hidden_dim,
                           int world, uint8_t* send_rows, int32_t* dest_counts, int32_t* send_slot, int num_sms,
                           cudaStream_t stream);
// ids + weights (the 64-byte trailer) of every row of `segs` into compact local arrays [rows][8]
// The segment table of an expert-parallel step built ON THE DEVICE from what the small all-to-all delivered:
// `from_peers` [n][3] int32 = (rows source s has for this rank, their first row in s's send buffer, unused),
// `send_base[s]` = source s's (mapped) send buffer.  Writes the table and the total row count (clamped to
// `cap_rows`) to `segs_out` / `n_rows_out`, then copies the (ids, weights) trailer of every row.
struct PeerBases {
  const uint8_t* base[8];
};
cudaError_t launch_ep_segments_pull(const PeerBases& send_base, const int32_t* from_peers, int n, long long row_bytes,
                                    int cap_rows, int hidden_dim, RowSegments* segs_out, int* n_rows_out,
                                    int32_t* ids_out, float* w_out, int num_sms, cudaStream_t stream);
// ep_combine reading each destination's partial rows where they were produced: partial[d] is rank d's
// (mapped) output buffer, row_start[d] (device) the first row of this rank's segment inside it
struct PeerPartials {
  const void* partial[8];
};
cudaError_t launch_ep_combine_peers(const PeerPartials& peers, const int32_t* row_start, const int32_t* send_slot,
                                    int T, int hidden_dim, int world, void* out_bf16, int num_sms,
                                    cudaStream_t stream);
cudaError_t launch_ep_combine(const void* returned_bf16, const int32_t* send_slot, const int32_t* dest_counts, int T,
                              int hidden_dim, int world, void* out_bf16, int num_sms, cudaStream_t stream);

}  // namespace b200moe
