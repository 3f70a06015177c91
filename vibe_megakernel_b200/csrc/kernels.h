// Host-callable launchers of the layer's kernels (internal to the library).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moe_b200.h"

#include <utility>

#include "common.cuh"

namespace moe {

// Records how many kernels the entry point that just ran on this thread launched (moe_last_launch_count).
void note_launches(int n);

// Launch with programmatic stream serialization: the kernel may start while the previous kernel of
// the stream drains; it must call dependent_wait() before reading what that kernel wrote.
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Byte ranges the logits kernel asks the L2 to fetch while it runs (extra blocks, fire and forget):
// the shared expert's weights do not depend on the routing, so they can be on their way while HBM
// is otherwise nearly idle. Addresses and sizes are multiples of 16.
struct L2Warm {
  const uint8_t* ptr[3];
  uint64_t bytes[3];
  int32_t* stamp;      // status words for the optional timeline (-DMOE_TIMELINE), else unused
};

cudaError_t launch_router(const moe_config_t& cfg, const __nv_bfloat16* x, const float* router, const float* bias,
                          int tokens, float* logits, int32_t* ids32, float* weights, int64_t* ids64,
                          float* weights_out, cudaStream_t stream, int* launches, const L2Warm* warm = nullptr);

cudaError_t launch_router_logits(const __nv_bfloat16* x, const float* router, int tokens, int experts, int hidden,
                                 float* logits, cudaStream_t stream, const L2Warm* warm = nullptr);

struct GroupArgs {
  const int32_t* ids32;   // one of ids32 / ids64 is set
  const int64_t* ids64;
  int n;                  // routed rows
  int id_base, n_local;   // ids in [id_base, id_base + n_local) are kept
  int topk;               // row r belongs to token r / topk
  int shared_rows;        // rows of the shared expert appended as expert n_local (0 = none)
  int tile;               // rows per chunk
  int max_chunks;
  int32_t* counts;        // [n_local + 1]
  int32_t* offsets;       // [n_local + 2]
  int32_t* n_chunks;
  Chunk* chunks;
  int32_t* row_token;     // optional
  int32_t* row_dest;      // optional
  int64_t* order;         // optional, [n]
  int32_t* slot_pos;      // optional, [n]: the grouped row a kept routed row went to (rows not kept are not written)
  int32_t* status;        // optional
  int zero_status;        // the kernel clears the 8 status words itself (it is the call's first that may report)
  const int32_t* seg_counts;  // optional: rows come in segments of seg_cap, segment s holds seg_counts[s] rows
  int seg_cap;
  int32_t* progress;          // optional: counters of the GEMMs, zeroed here (see GemmArgs, WorkListLayout)
  int progress_len;
  FlagWait wait;              // expert parallel: the rows and ids were stored by peers; wait for their flags first
};
cudaError_t launch_group_rows(const GroupArgs& a, cudaStream_t stream, int* launches);

// Small batches: logits, then ONE kernel for selection + permutation + work list + quantiser of the
// grouped rows (bf16 tokens, every expert local). `fused_route_fits` says whether the shape allows it.
bool fused_route_fits(const moe_config_t& cfg, int tokens);
cudaError_t launch_router_fused(const moe_config_t& cfg, const __nv_bfloat16* x, const float* router, const float* bias,
                                int tokens, float* logits, int32_t* ids32, float* weights, int64_t* ids64,
                                float* weights_out, const GroupArgs& g, uint8_t* xq, float* xs, cudaStream_t stream,
                                int* launches, const L2Warm* warm = nullptr);

cudaError_t launch_quantize(const void* x, int dtype, int rows, int width, const int32_t* gather, uint8_t* q,
                            float* scales, cudaStream_t stream, int* launches);

// e4m3 payload with one power-of-two scale (biased exponent, uint8) per `block` = 32 or 128 channels
// The same rows from the token side, for large batches in which every routed row is kept: a token's
// groups are quantised once and stored to each of its `topk` grouped rows slot_pos[token * topk + k]
// and, with `shared_base` >= 0, to row shared_base + token (bf16 rows of whole groups only).
bool quantize_scatter_fits(int tokens, int width, const void* x);
cudaError_t launch_quantize_scatter(const __nv_bfloat16* x, int tokens, int width, int topk, const int32_t* slot_pos,
                                    int shared_base, uint8_t* q, float* scales, cudaStream_t stream, int* launches);
cudaError_t launch_quantize_ue8m0(const void* x, int dtype, int rows, int width, int block, uint8_t* q, uint8_t* scales,
                                  cudaStream_t stream);

// residual (optional, bf16 [tokens, hidden]): y = bf16(residual + bf16(sum)) instead of bf16(sum)
cudaError_t launch_combine(const __nv_bfloat16* slots, const float* weights, int tokens, int topk, int hidden,
                           int shared, __nv_bfloat16* y, cudaStream_t stream, int* launches,
                           const __nv_bfloat16* residual = nullptr, const FlagWait* wait = nullptr);

// RMSNorm of bf16 rows with a bf16 weight (megabench/tasks/common.py:13-21), both roundings of the reference.
cudaError_t launch_rmsnorm(const __nv_bfloat16* x, const __nv_bfloat16* weight, float eps, int weight_in_fp32, int tokens,
                           int hidden, __nv_bfloat16* out, cudaStream_t stream, int* launches);

// Copy rows that arrived in any order (and the home rows of the shared expert) into expert order.
struct GatherArgs {
  const int32_t* row_source;   // grouped position -> arrival index (routed) or home token (shared)
  const int32_t* offsets;      // offsets[n_local] = routed rows kept; shared rows follow
  int n_local, shared_rows, hidden;
  const uint8_t* recv_q;       // arrivals: e4m3 [*, H] and fp32 scales [*, H/128]
  const float* recv_s;
  const uint8_t* xq_home;      // rows of the shared expert
  const float* xs_home;
  uint8_t* xq;                 // grouped output
  float* xs;
};
cudaError_t launch_gather_rows(const GatherArgs& a, int row_blocks, cudaStream_t stream, int* launches);

// Tokens per MMA tile (the N extent: 16, 32 or 64), from the rows a routed expert can expect.
// A tile wider than the chunks it meets costs shared memory per pipeline stage and epilogue
// registers for columns that are never used; a narrower one only splits the few large chunks
// (the shared expert, hot experts), whose weight tiles are then re-read from the L2.
// With widest = 128 (callers whose GEMM arm has the kernel for it): 128-row tiles with the tokens on
// the MMA's M side once an expert can expect more than `wide_above` rows (measured on the Mixtral
// shape: 64 rows per expert 418 -> 375 us with them; at 32 and fewer rows per expert, there and on
// the Qwen and Kimi shapes, the 16..64-token tiles are as fast or faster).
inline int pick_token_tile(long long routed_rows, int experts, int widest = 64, int wide_above = 32) {
  const long long expected = (routed_rows + experts - 1) / (experts > 0 ? experts : 1);
  if (widest >= 128 && expected > wide_above) return 128;
  return expected <= 8 ? 16 : expected <= 16 ? 32 : 64;
}

// MegaMoE-native GEMMs: expected rows per expert above which the 128-row kernel is taken (its MMAs cost
// the same whether a tile's 128 rows are all there or not, the 64-token kernel's grow with the rows)
constexpr int kMxWideAbove = 32;

// Parts the down projection's contraction is cut in, from the geometry alone (never from the
// batch, so that a token's result does not depend on what else is in flight): contractions
// longer than 64 K blocks are cut in parts of at most 32.
inline int down_ksplit(int inter) {
  const int kblocks = inter / 128;
  return kblocks > 64 ? (kblocks + 31) / 32 : 1;
}

// The work list's region of a workspace: the chunks, then the int32 counters the permutation
// kernel zeroes (per-chunk gate/up progress, 4 spare words of which the first is the down GEMM's
// dispenser, and with a split contraction one counter per down tile), then the fp32 partial tiles.
// Small batches of the one-GPU layer: the combine is done by the down GEMM itself. Its CTAs meet
// at the kernel's end (one counter, bounded wait) and then share out the sum of the slot rows, in
// slot order, exactly as the combine kernel would (same bits: the sum is a function of the stored
// bf16 rows). Saves a launch where a layer call is a few tens of microseconds.
constexpr int kFoldMaxTokens = 16;

struct WorkListLayout {
  uint64_t counters, parts_done, fold_count, partial, bytes;   // byte offsets from the first chunk
  int counters_len;
};
inline WorkListLayout work_list_layout(int max_chunks, int hidden, int inter, int tile, int fold_tokens = 0) {
  const int ksplit = down_ksplit(inter);
  const int tiles_down = hidden / 128;
  WorkListLayout w;
  w.counters = 16ull * max_chunks;
  const int parts_len = ksplit > 1 ? max_chunks * tiles_down : 0;
  w.counters_len = max_chunks + 4 + parts_len + (fold_tokens > 0 ? 4 : 0);
  w.parts_done = w.counters + 4ull * (max_chunks + 4);
  w.fold_count = w.parts_done + 4ull * parts_len;
  uint64_t off = w.counters + 4ull * w.counters_len;
  off = (off + 255) / 256 * 256;
  w.partial = off;
  if (ksplit > 1 && tile < 128) off += 4ull * max_chunks * tiles_down * ksplit * tile * 128;   // 128-row tiles sum their parts in registers
  w.bytes = off;
  return w;
}

// The two optional steps of the MegaMoE form of SwiGLU (megabench/tasks/megamoe.py:116-122):
// gate clamped to at most `limit` and up to +-limit on the bf16 GEMM outputs (limit > 0), and the
// fp32 product multiplied by the row's routing weight before requantisation (slot_weight != null;
// a routed row's slot is row_dest[row] < routed_rows, the shared expert's rows keep weight 1).
struct SwigluMode {
  float limit = 0.f;
  const float* slot_weight = nullptr;
  const int32_t* row_dest = nullptr;
  int routed_rows = 0;
};

// The combine folded into the down GEMM (see kFoldMaxTokens).
struct FoldCombine {
  __nv_bfloat16* y = nullptr;            // [tokens, hidden]; NULL = off
  const float* weights = nullptr;        // [tokens*topk], NULL = the rows carry their weight already
  const __nv_bfloat16* residual = nullptr;   // optional [tokens, hidden]: y = bf16(residual + bf16(sum))
  int32_t* count = nullptr;              // one counter of the CTAs that have stored their rows, zero on entry
  int tokens = 0, topk = 0, shared = 0;
};

// Down GEMM of an expert-parallel call: finished rows go straight into their sources' slot buffers
// (peer stores from the epilogue) instead of a local buffer that a copy kernel would read again, and
// the kernel's last CTA raises the return flags. base[0] == NULL: off.
struct PeerReturn {
  uint8_t* base[8];           // every rank's exchange buffer
  const int32_t* row_source;  // grouped position -> arrival index (routed) or home token (shared expert)
  const int32_t* recv_slot;   // arrival index -> slot at its source
  const int32_t* offsets;     // offsets[n_local] = routed rows kept
  int n_local, cap, world, rank, home_tokens, topk;
  uint64_t off_slots, off_flags;
  int32_t* done;              // counter of CTAs that are through: zero on entry, left at zero
  uint64_t epoch;
};

struct GemmArgs {
  bool dual;                 // true: gate+up with SwiGLU + requantisation; false: down projection
  int tile;                  // tokens per MMA tile: 16, 32 or 64
  int k;                     // contraction length (H for gate/up, I for down)
  int m;                     // output channels per expert (I for gate/up, H for down)
  int n_local;               // routed experts held here; chunk.expert == n_local is the shared expert
  int total_rows;            // rows of the activation buffer
  int max_units;             // upper bound of chunks * (m / 128)
  const Chunk* chunks;
  const int32_t* n_chunks;
  const uint8_t* act;        // e4m3 [total_rows, k]
  const float* act_scale;    // [total_rows, k/128]
  const uint8_t* w_a;        // gate or down, [n_local, m, k]
  const float* w_a_scale;
  const uint8_t* w_b;        // up (dual only)
  const float* w_b_scale;
  const uint8_t* s_a;        // shared expert counterparts (may be NULL when there is none)
  const float* s_a_scale;
  const uint8_t* s_b;
  const float* s_b_scale;
  uint8_t* aq;               // dual: e4m3 [total_rows, m]
  float* as;                 // dual: [total_rows, m/128]
  __nv_bfloat16* out;        // single: bf16 rows [*, m] addressed through row_dest
  const int32_t* row_dest;
  int32_t* status;
  // Hand-over between the two GEMMs of a layer call without a kernel boundary: progress[c] counts
  // the gate/up tiles of work item c that are finished and visible; progress[max_chunks] is the
  // down GEMM's work-item dispenser. The gate/up GEMM increments, the down GEMM (which may be
  // scheduled on SMs the gate/up GEMM has already left) waits per work item and takes items
  // dynamically. NULL = plain kernel-boundary ordering and a static walk.
  int32_t* progress;
  int max_chunks;
  int tiles_before;          // down GEMM: gate/up tiles per work item that must be finished
  // Down GEMM with a long contraction: cut in `ksplit` parts (work items of their own); fp32
  // partial tiles [chunk * tiles + tile][part][token column][128] and one zeroed counter per tile.
  int ksplit;
  float* partial;
  int32_t* parts_done;
  SwigluMode swiglu;         // dual only
  FoldCombine fold;          // down GEMM only: the combine done by the last tile of every token (y == NULL: off)
  int max_stages;            // > 0: cap of the shared-memory ring, so that the CTAs of the call's two GEMMs fit on an SM together
  bool bf16_operands;        // CUDA-core arm only: operands dequantised and rounded to bf16 first (MOE_GEMM_SIMT_BF16)
  PeerReturn ret;            // down GEMM of the weights-on-M tensor-core kernel only (tile <= 64)
};
cudaError_t launch_gemm_tc(const GemmArgs& a, cudaStream_t stream, int* launches, int* driver_error);
// tile == 128: tokens on the MMA's M side (gemm_wide.cu); no hand-over, no folded combine
cudaError_t launch_gemm_wide(const GemmArgs& a, cudaStream_t stream, int* launches, int* driver_error);

// Grouped GEMM in the MegaMoE-native formats (MXFP4 weights, E4M3 rows, E8M0 scales per 32 channels
// on both sides), block-scaled tensor-core MMA. dual: linear1 ([E, 2m, k]: gate rows then up rows) with
// clamped SwiGLU, routing weight and requantisation; else linear2 ([E, m, k]) into bf16 slot rows.
struct MxGemmArgs {
  bool dual;
  int tile;                   // tokens per MMA tile: 16, 32 or 64 (weights on M), or 128 (tokens on M)
  int k, m;                   // contraction length; output channels per expert (I for linear1, H for linear2)
  int n_experts;
  int total_rows;             // rows of the activation buffer
  int max_units;              // upper bound of chunks * (m / 128)
  const Chunk* chunks;
  const int32_t* n_chunks;
  const uint8_t* act;         // e4m3 [total_rows, k], grouped by expert
  const uint8_t* act_scales;  // E8M0 [total_rows, k/32]
  const uint8_t* w_blocks;    // packed E2M1, [n_experts * rows, k/2] bytes
  const uint8_t* w_scales;    // E8M0 [n_experts * rows, k/32]
  uint8_t* aq;                // dual: e4m3 [total_rows, m]
  uint8_t* as;                // dual: E8M0 [total_rows, m/32]
  __nv_bfloat16* out;         // single: bf16 rows [*, m] addressed through row_dest
  const int32_t* row_dest;
  const float* slot_weight;   // dual: routing weight of slot row_dest[row]; NULL = 1
  float limit;                // dual: clamp of gate/up, 0 = none
  int32_t* status;
  // dual, optional: the up rows live in a tensor of their own ([n_experts * m, k/2] bytes and scales) instead of
  // following the gate rows inside w_blocks / w_scales (megabench/tasks/kimi_layer.py:113-120 stores them apart)
  const uint8_t* w_blocks_b;
  const uint8_t* w_scales_b;
  int activation;             // dual: 0 = clamped SwiGLU (megabench/tasks/megamoe.py:116-122), 1 = situ (megabench/tasks/kimi.py:134-135)
  // Rows come in (hi, lo) pairs, the two E4M3 pieces of one bf16 row (grouped rows 2p and 2p+1): the
  // epilogue adds a pair's two results. dual: the activation's bf16 value is split again into two
  // rows of aq / as; single: one bf16 row per pair at out[row_dest[2p] / 2].
  bool pairs;
};
cudaError_t launch_gemm_mx(const MxGemmArgs& a, cudaStream_t stream, int* launches, int* driver_error);
// tile == 128: tokens on the MMA's M side (gemm_mx_wide.cu); plain rows, gate and up rows in one tensor, m % 256 == 0 for linear2
cudaError_t launch_gemm_mx_wide(const MxGemmArgs& a, cudaStream_t stream, int* launches, int* driver_error);
// Grouped row r < *kept <- row row_token[r] of e4m3 [tokens, hidden] with its hidden/32 scale bytes.
cudaError_t launch_gather_mx_rows(const uint8_t* x, const uint8_t* x_scales, const int32_t* row_token, const int32_t* kept,
                                  int rows, int tokens, int hidden, uint8_t* xg, uint8_t* xgs, cudaStream_t stream,
                                  int* launches);
cudaError_t launch_gemm_simt(const GemmArgs& a, cudaStream_t stream, int* launches);
// The arm `impl` (MOE_GEMM_*) asks for.
inline cudaError_t launch_gemm(int impl, GemmArgs& a, cudaStream_t stream, int* launches, int* driver_error) {
  if (impl == MOE_GEMM_TCGEN05 && a.tile == 128) return launch_gemm_wide(a, stream, launches, driver_error);
  if (impl == MOE_GEMM_TCGEN05) return launch_gemm_tc(a, stream, launches, driver_error);
  a.bf16_operands = impl == MOE_GEMM_SIMT_BF16;
  return launch_gemm_simt(a, stream, launches);
}

// Dense bf16 projection y = f(x W^T) on tensor cores (dense_tc.cu; the Kimi latent block above eight
// tokens). mode 0: bf16(sum); 1: situ(bf16(sum over w), bf16(sum over w2)); 2: bf16(bf16(sum) + other).
// n % 128 == 0, k % 64 == 0, 16-byte aligned pointers. The contraction is cut in plan.ksplit parts that
// meet in `partial` (plan.partial_bytes) and `parts_done` (plan.tiles counters, zero on entry, left at zero).
struct DenseTcPlan {
  int tiles, ksplit;
  uint64_t partial_bytes;
};
DenseTcPlan dense_tc_plan(int tokens, int n, int k);
cudaError_t launch_dense_tc(int mode, const __nv_bfloat16* w, const __nv_bfloat16* w2, const __nv_bfloat16* x, int tokens, int n,
                            int k, const __nv_bfloat16* other, __nv_bfloat16* y, float* partial, int32_t* parts_done,
                            int32_t* status, cudaStream_t stream, int* launches, int* driver_error);

}  // namespace moe
