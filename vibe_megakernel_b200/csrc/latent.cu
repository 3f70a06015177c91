// The Kimi-K3 latent MoE block: kernels that the FP8 layer does not have, and its C ABI entry.
//
// Reference: megabench/tasks/kimi_layer.py:189-230 (`moe`, serial form) with the experts of :175-186
// and the activation of megabench/tasks/kimi.py:134-135:
//   per token: sigmoid top-k routing (scaling 1, no groups); latent = latent_down @ token (bf16);
//   per routed slot: situ(latent @ gate^T, latent @ up^T) @ down^T with MXFP4 weights dequantised to
//   bf16 and bf16 activations; fp32 slot-order weighted sum, rounded to bf16, RMSNorm (latent_norm),
//   latent_up; plus shared_down @ situ(shared_gate @ token, shared_up @ token); the two are added.
//
// The routed experts multiply bf16 rows with 4-bit weights. The block-scaled tensor-core MMA wants
// 8-bit (or narrower) operands on both sides, so every bf16 row travels as TWO E4M3 rows with E8M0
// scales per 32 channels: hi = the value rounded to E4M3 under its block's scale, lo = the
// remainder under the remainder's own block scale. A bf16 number has 8 significant bits and an
// E4M3 number 4, so hi + lo is the bf16 value exactly (for elements more than 2^15 below their
// block's largest the error is below 2^-23 of that largest: under the fp32 accumulation's own
// rounding). The weights keep streaming as 4 bits per value and W x = W hi + W lo is what the
// reference computes: exact products of the dequantised weights and the bf16 row, summed in fp32.
#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "kernels.h"
#include "split_e4m3.cuh"

namespace moe {

// Grouped pair p (rows 2p and 2p+1 of the split buffers) <- bf16 row row_token[2p] of x. One block
// per pair, a warp takes 128 channels (4 per lane: 8 lanes share a scale block).
__global__ void __launch_bounds__(256) split_rows_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ row_token,
                                                         const int32_t* __restrict__ kept, int tokens, int width,
                                                         uint8_t* __restrict__ q, uint8_t* __restrict__ scales) {
  dependent_wait();
  dependents_may_launch();
  const int pos = 2 * blockIdx.x;
  if (pos >= *kept) return;
  const int token = row_token[pos];
  if (token < 0 || token >= tokens) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* in = x + static_cast<size_t>(token) * width;
  const int blocks = width / 32;
  for (int k0 = warp * 128; k0 < width; k0 += 8 * 128) {
    const int k = k0 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(in + k);
    float v[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                  __uint_as_float(raw.y & 0xffff0000u)};
    uint8_t hi[4], lo[4];
    int e_hi, e_lo;
    split_e4m3(v, 8, hi, lo, e_hi, e_lo);
    *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(pos) * width + k) = hi[0] | (hi[1] << 8) | (hi[2] << 16) | (hi[3] << 24);
    *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(pos + 1) * width + k) = lo[0] | (lo[1] << 8) | (lo[2] << 16) | (lo[3] << 24);
    if ((lane & 7) == 0) {
      scales[static_cast<size_t>(pos) * blocks + k / 32] = static_cast<uint8_t>(e_hi);
      scales[static_cast<size_t>(pos + 1) * blocks + k / 32] = static_cast<uint8_t>(e_lo);
    }
  }
}

// ids2[2r] = ids2[2r+1] = ids[r]: the two pieces of a routed row go to the same expert, side by side.
__global__ void duplicate_ids_kernel(const int32_t* __restrict__ ids, int n, int32_t* __restrict__ ids2) {
  dependent_wait();
  dependents_may_launch();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < 2 * n) ids2[i] = ids[i >> 1];
}

}  // namespace moe

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
namespace {

inline uint64_t up256(uint64_t v) { return (v + 255) / 256 * 256; }
inline int cuda_rc(cudaError_t e) { return e == cudaSuccess ? MOE_OK : static_cast<int>(e); }

struct LatentLayout {
  uint64_t status, dense_parts, logits, ids32, weights, ids2, counts, offsets, n_chunks, chunks, row_token, row_dest, latent, xq,
      xs, aq, as, slots, sum, normed, act, shared, dense_partial, total;
  int dense_parts_len;
  int rows2, tile, max_chunks;
};

int latent_layout(const moe_latent_config_t* c, int tokens, LatentLayout* L) {
  if (!c) return MOE_ERR_BAD_ARG;
  if (c->hidden < 128 || c->latent < 128 || c->inter < 128 || c->n_experts < 1 || c->topk < 1 || c->topk > c->n_experts ||
      c->n_shared < 1 || tokens < 1 || !(c->latent_eps >= 0.f))
    return MOE_ERR_BAD_ARG;
  if (c->hidden % 128 || c->latent % 128 || c->inter % 128 || c->n_experts > MOE_MAX_EXPERTS || c->topk > MOE_MAX_TOPK ||
      2ll * tokens * c->topk > 32768)
    return MOE_ERR_UNSUPPORTED;
  const uint64_t H = c->hidden, LH = c->latent, I = c->inter, E = c->n_experts;
  const int rows = tokens * c->topk, rows2 = 2 * rows;
  LatentLayout l;
  l.rows2 = rows2;
  l.tile = moe::pick_token_tile(rows2, c->n_experts);
  l.max_chunks = std::min(rows2, c->n_experts) + rows2 / l.tile + 1;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) { const uint64_t at = off; off = up256(off + bytes); return at; };
  l.status = take(32);
  // the dense projections: the two counters of their grid meeting and the fp32 partial tiles of a split
  // contraction, shared by the four projections (they run one after another)
  const moe::DenseTcPlan plans[4] = {moe::dense_tc_plan(tokens, c->latent, c->hidden),
                                     moe::dense_tc_plan(tokens, c->n_shared * c->inter, c->hidden),
                                     moe::dense_tc_plan(tokens, c->hidden, c->n_shared * c->inter),
                                     moe::dense_tc_plan(tokens, c->hidden, c->latent)};
  int most_tiles = 1;
  uint64_t most_partial = 0;
  for (const moe::DenseTcPlan& plan : plans) {
    most_tiles = std::max(most_tiles, plan.tiles);
    most_partial = std::max(most_partial, plan.partial_bytes);
  }
  l.dense_parts_len = most_tiles;
  l.dense_parts = take(4ull * most_tiles);
  l.logits = take(4ull * tokens * E);
  l.ids32 = take(4ull * rows);
  l.weights = take(4ull * rows);
  l.ids2 = take(4ull * rows2);
  l.counts = take(4ull * (E + 1));
  l.offsets = take(4ull * (E + 2));
  l.n_chunks = take(4);
  l.chunks = take(16ull * l.max_chunks);
  l.row_token = take(4ull * rows2);
  l.row_dest = take(4ull * rows2);
  l.latent = take(2ull * tokens * LH);
  l.xq = take(static_cast<uint64_t>(rows2) * LH);
  l.xs = take(static_cast<uint64_t>(rows2) * (LH / 32));
  l.aq = take(static_cast<uint64_t>(rows2) * I);
  l.as = take(static_cast<uint64_t>(rows2) * (I / 32));
  l.slots = take(2ull * rows * LH);
  l.sum = take(2ull * tokens * LH);
  l.normed = take(2ull * tokens * LH);
  l.act = take(2ull * tokens * c->n_shared * I);
  l.shared = take(2ull * tokens * H);
  l.dense_partial = take(most_partial);
  l.total = off;
  *L = l;
  return MOE_OK;
}

}  // namespace

extern "C" {

int moe_latent_workspace(const moe_latent_config_t* cfg, int32_t tokens, uint64_t* bytes) {
  LatentLayout L;
  const int rc = latent_layout(cfg, tokens, &L);
  if (rc) return rc;
  if (bytes) *bytes = L.total;
  return MOE_OK;
}

int moe_latent_forward(const moe_latent_config_t* cfg, const moe_latent_weights_t* w, const void* x_bf16, int32_t tokens,
                       void* y_bf16, int64_t* expert_ids, float* topk_weights, void* workspace, size_t workspace_bytes,
                       void* stream_) {
  LatentLayout L;
  const int rc = latent_layout(cfg, tokens, &L);
  if (rc) return rc;
  if (!w || !x_bf16 || !y_bf16 || !workspace) return MOE_ERR_BAD_ARG;
  const void* need[] = {w->router, w->latent_down, w->latent_up, w->latent_norm, w->gate_blocks, w->gate_scales, w->up_blocks,
                        w->up_scales, w->down_blocks, w->down_scales, w->shared_gate, w->shared_up, w->shared_down};
  for (const void* ptr : need)
    if (!ptr) return MOE_ERR_BAD_ARG;
  if (workspace_bytes < L.total) return MOE_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return MOE_ERR_BAD_ARG;
  // the weight tiles move by TMA as packed 4-bit values (32-byte aligned base), the scale rows by 16-byte copies
  if ((reinterpret_cast<uintptr_t>(w->gate_blocks) | reinterpret_cast<uintptr_t>(w->up_blocks) |
       reinterpret_cast<uintptr_t>(w->down_blocks)) & 31 ||
      (reinterpret_cast<uintptr_t>(w->gate_scales) | reinterpret_cast<uintptr_t>(w->up_scales) |
       reinterpret_cast<uintptr_t>(w->down_scales)) & 15)
    return MOE_ERR_BAD_ARG;
  using bf16 = __nv_bfloat16;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(ws + L.status);
  int32_t* ids32 = reinterpret_cast<int32_t*>(ws + L.ids32);
  float* tw = reinterpret_cast<float*>(ws + L.weights);
  int32_t* ids2 = reinterpret_cast<int32_t*>(ws + L.ids2);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + L.offsets);
  int32_t* row_token = reinterpret_cast<int32_t*>(ws + L.row_token);
  int32_t* row_dest = reinterpret_cast<int32_t*>(ws + L.row_dest);
  bf16* latent = reinterpret_cast<bf16*>(ws + L.latent);
  bf16* slots = reinterpret_cast<bf16*>(ws + L.slots);
  bf16* sum = reinterpret_cast<bf16*>(ws + L.sum);
  bf16* normed = reinterpret_cast<bf16*>(ws + L.normed);
  bf16* act = reinterpret_cast<bf16*>(ws + L.act);
  bf16* shared = reinterpret_cast<bf16*>(ws + L.shared);
  const bf16* x = static_cast<const bf16*>(x_bf16);
  const int H = cfg->hidden, LH = cfg->latent, I = cfg->inter, E = cfg->n_experts, K = cfg->topk;
  const int rows = tokens * K;
  int launches = 0;
  // status word, and the dense projections' part counters behind it (left at zero by the kernels, but the
  // workspace arrives uninitialised)
  cudaError_t e = cudaMemsetAsync(status, 0, L.dense_parts + 4ull * L.dense_parts_len, stream);
  if (e != cudaSuccess) return cuda_rc(e);
  int driver_error = 0;
  float* dense_partial = reinterpret_cast<float*>(ws + L.dense_partial);
  int32_t* dense_parts = reinterpret_cast<int32_t*>(ws + L.dense_parts);
  // a dense bf16 projection (dense_tc.cu): every width of this block is a multiple of 128
  auto dense = [&](int mode, const void* wm, const void* wm2, const bf16* in, int n, int k, const bf16* other, bf16* out) {
    return moe::launch_dense_tc(mode, static_cast<const bf16*>(wm), static_cast<const bf16*>(wm2), in, tokens, n, k, other, out,
                                dense_partial, dense_parts, status, stream, &launches, &driver_error);
  };

  // 1. router: sigmoid scores plus selection bias, no groups, weights normalised with scaling 1
  //    (megabench/tasks/kimi_layer.py:200-201)
  moe_config_t rc_cfg;
  std::memset(&rc_cfg, 0, sizeof(rc_cfg));
  rc_cfg.hidden = H; rc_cfg.inter = I; rc_cfg.n_experts = E; rc_cfg.topk = K; rc_cfg.scoring = MOE_SCORING_SIGMOID;
  rc_cfg.n_group = 1; rc_cfg.topk_group = 1; rc_cfg.routed_scaling = 1.f; rc_cfg.ep_world = 1;
  e = moe::launch_router(rc_cfg, x, w->router, w->router_bias, tokens, reinterpret_cast<float*>(ws + L.logits), ids32, tw,
                         expert_ids, topk_weights, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);

  // 2. latent rows (megabench/tasks/kimi_layer.py:203)
  e = dense(0, w->latent_down, nullptr, x, LH, H, nullptr, latent);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);

  // 3. every routed row becomes a pair of E4M3 rows; the pairs are grouped by expert
  moe::launch_dependent(moe::duplicate_ids_kernel, dim3((2 * rows + 255) / 256), dim3(256), 0, stream,
                        static_cast<const int32_t*>(ids32), rows, ids2);
  ++launches;
  moe::GroupArgs g;
  std::memset(&g, 0, sizeof(g));
  g.ids32 = ids2;
  g.n = L.rows2;
  g.n_local = E;
  g.topk = 2 * K;                  // split row r belongs to token r / (2 topk)
  g.tile = L.tile;
  g.max_chunks = L.max_chunks;
  g.counts = reinterpret_cast<int32_t*>(ws + L.counts);
  g.offsets = offsets;
  g.n_chunks = reinterpret_cast<int32_t*>(ws + L.n_chunks);
  g.chunks = reinterpret_cast<moe::Chunk*>(ws + L.chunks);
  g.row_token = row_token;
  g.row_dest = row_dest;
  g.status = status;
  e = moe::launch_group_rows(g, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);
  uint8_t* xq = ws + L.xq;
  uint8_t* xs = ws + L.xs;
  moe::launch_dependent(moe::split_rows_kernel, dim3(rows), dim3(256), 0, stream, static_cast<const bf16*>(latent),
                        static_cast<const int32_t*>(row_token), static_cast<const int32_t*>(offsets + E), tokens, LH, xq, xs);
  ++launches;

  // 4. gate/up with situ, split again; down into slot rows (megabench/tasks/kimi_layer.py:175-186)
  moe::MxGemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.tile = L.tile;
  a.n_experts = E;
  a.total_rows = L.rows2;
  a.chunks = g.chunks;
  a.n_chunks = g.n_chunks;
  a.status = status;
  a.pairs = true;
  a.dual = true;
  a.k = LH; a.m = I;
  a.max_units = L.max_chunks * (I / 128);
  a.act = xq; a.act_scales = xs;
  a.w_blocks = w->gate_blocks; a.w_scales = w->gate_scales;
  a.w_blocks_b = w->up_blocks; a.w_scales_b = w->up_scales;
  a.aq = ws + L.aq; a.as = ws + L.as;
  a.row_dest = row_dest;
  a.activation = 1;
  e = moe::launch_gemm_mx(a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);
  a.dual = false;
  a.k = I; a.m = LH;
  a.max_units = L.max_chunks * (LH / 128);
  a.act = ws + L.aq; a.act_scales = ws + L.as;
  a.w_blocks = w->down_blocks; a.w_scales = w->down_scales;
  a.w_blocks_b = nullptr; a.w_scales_b = nullptr;
  a.aq = nullptr; a.as = nullptr;
  a.out = slots;
  e = moe::launch_gemm_mx(a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);

  // 5. fp32 slot-order weighted sum rounded to bf16, latent RMSNorm (megabench/tasks/kimi_layer.py:222-227)
  e = moe::launch_combine(slots, tw, tokens, K, LH, 0, sum, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);
  e = moe::launch_rmsnorm(sum, static_cast<const bf16*>(w->latent_norm), cfg->latent_eps, 0, tokens, LH, normed, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);

  // 6. shared experts on the full-width token (megabench/tasks/kimi_layer.py:228), then latent_up + shared
  e = dense(1, w->shared_gate, w->shared_up, x, cfg->n_shared * I, H, nullptr, act);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);
  e = dense(0, w->shared_down, nullptr, act, H, cfg->n_shared * I, nullptr, shared);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);
  e = dense(2, w->latent_up, nullptr, normed, H, LH, shared, static_cast<bf16*>(y_bf16));
  if (driver_error) return MOE_ERR_DRIVER;
  moe::note_launches(launches);
  return cuda_rc(e);
}

}  // extern "C"
