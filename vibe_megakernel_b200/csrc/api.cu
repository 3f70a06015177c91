// C ABI: argument checks, workspace layout and the launch sequence of one layer call.
#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace {

thread_local int g_last_launches = 0;

// Optional stage timing: events recorded on the launching stream around each stage.
constexpr int kStages = 6;   // router, permutation, quantiser, gate/up GEMM, down GEMM, combine
thread_local bool g_profile = false;
thread_local cudaEvent_t g_events[kStages + 1] = {};
thread_local bool g_events_ready = false;

void mark(int i, cudaStream_t stream) {
  if (!g_profile) return;
  if (!g_events_ready) {
    for (auto& ev : g_events) cudaEventCreate(&ev);
    g_events_ready = true;
  }
  cudaEventRecord(g_events[i], stream);
}

inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

int check_config(const moe_config_t* c) {
  if (!c) return MOE_ERR_BAD_ARG;
  if (c->hidden <= 0 || c->inter <= 0 || c->n_experts <= 0 || c->topk <= 0) return MOE_ERR_BAD_ARG;
  if (c->hidden % 128 || c->inter % 128) return MOE_ERR_UNSUPPORTED;
  if (c->n_experts > MOE_MAX_EXPERTS || c->topk > MOE_MAX_TOPK || c->topk > c->n_experts) return MOE_ERR_UNSUPPORTED;
  if (c->n_shared < 0 || c->n_shared > 1) return MOE_ERR_UNSUPPORTED;
  if (c->scoring < MOE_SCORING_SOFTMAX || c->scoring > MOE_SCORING_SOFTMAX_BIASED) return MOE_ERR_BAD_ARG;
  if (c->n_group < 1 || c->n_group > 32 || c->n_experts % c->n_group) return MOE_ERR_BAD_ARG;
  if (c->topk_group < 1 || c->topk_group > c->n_group) return MOE_ERR_BAD_ARG;
  if (c->ep_world < 1 || c->ep_rank < 0 || c->ep_rank >= c->ep_world || c->n_experts % c->ep_world) return MOE_ERR_BAD_ARG;
  if (c->gemm_impl < MOE_GEMM_TCGEN05 || c->gemm_impl > MOE_GEMM_SIMT_BF16) return MOE_ERR_BAD_ARG;
  if (c->hidden / 128 > 112 || c->inter / 128 > 112) return MOE_ERR_UNSUPPORTED;
  if (!(c->swiglu_limit >= 0.f) || (c->weight_before_requant != 0 && c->weight_before_requant != 1)) return MOE_ERR_BAD_ARG;
  if (c->weight_before_requant && c->ep_world != 1) return MOE_ERR_UNSUPPORTED;
  return MOE_OK;
}


// Tokens whose combine the down GEMM does itself (0: the combine kernel runs): small batches on one GPU.
inline int fold_tokens(const moe_config_t* c, int tokens) {
  return (c->ep_world == 1 && tokens <= moe::kFoldMaxTokens) ? tokens : 0;
}

int layout_of(const moe_config_t* c, int tokens, moe_workspace_layout_t* L) {
  const int rc = check_config(c);
  if (rc) return rc;
  if (tokens < 1 || static_cast<int64_t>(tokens) * c->topk > 32768) return MOE_ERR_UNSUPPORTED;
  const int n_local = c->n_experts / c->ep_world;
  const int routed = tokens * c->topk;
  const int rows = routed + tokens * c->n_shared;
  const int tile = moe::pick_token_tile(routed, n_local, c->gemm_impl == MOE_GEMM_TCGEN05 && c->ep_world == 1 ? 128 : 64);
  const int max_chunks = std::min(routed, n_local) + routed / tile + (tokens + tile - 1) / tile + 1;
  const uint64_t H = c->hidden, I = c->inter;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) { const uint64_t at = off; off = align_up(off + bytes, 256); return at; };
  moe_workspace_layout_t l;
  std::memset(&l, 0, sizeof(l));
  l.status = take(8 * 4);
  l.logits = take(4ull * tokens * c->n_experts);
  l.topk_ids = take(4ull * routed);
  l.topk_weights = take(4ull * routed);
  l.counts = take(4ull * (n_local + 1));
  l.offsets = take(4ull * (n_local + 2));
  l.n_chunks = take(4);
  l.chunks = take(moe::work_list_layout(max_chunks, c->hidden, c->inter, tile, fold_tokens(c, tokens)).bytes);   // work items, counters, partial tiles
  l.row_token = take(4ull * rows);
  l.row_dest = take(4ull * rows);
  l.xq = take(static_cast<uint64_t>(rows) * H);
  l.xs = take(4ull * rows * (H / 128));
  l.aq = take(static_cast<uint64_t>(rows) * I);
  l.as = take(4ull * rows * (I / 128));
  l.slots = take(2ull * rows * H);
  take(2ull * tokens * H);               // normalised token rows of moe_block_forward (see norm_offset)
  take(4ull * routed);                   // grouped row of every routed row (see slot_pos_offset)
  l.total_bytes = off;
  l.rows = rows;
  l.max_chunks = max_chunks;
  l.token_tile = tile;
  if (L) *L = l;
  return MOE_OK;
}

// bf16 [T, H] behind the slot rows: the RMSNorm output when the call covers the whole block
inline uint64_t norm_offset(const moe_workspace_layout_t& L, int hidden) {
  return align_up(L.slots + 2ull * L.rows * hidden, 256);
}

// int32 [T * topk] behind those: where the permutation put each routed row (large batches quantise from the token side)
inline uint64_t slot_pos_offset(const moe_workspace_layout_t& L, int hidden, int tokens) {
  return align_up(norm_offset(L, hidden) + 2ull * tokens * hidden, 256);
}

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

inline int from_cuda(cudaError_t e) { return e == cudaSuccess ? MOE_OK : static_cast<int>(e); }

}  // namespace

namespace moe {
void note_launches(int n) { g_last_launches = n; }
}  // namespace moe

extern "C" {

int moe_workspace_layout(const moe_config_t* cfg, int32_t tokens, moe_workspace_layout_t* layout) {
  return layout_of(cfg, tokens, layout);
}

int moe_route(const moe_config_t* cfg, const void* x_bf16, const float* router, const float* router_bias,
              int32_t tokens, int64_t* expert_ids, float* weights, void* workspace, size_t workspace_bytes,
              void* stream) {
  moe_workspace_layout_t L;
  const int rc = layout_of(cfg, tokens, &L);
  if (rc) return rc;
  if (!x_bf16 || !router || !workspace) return MOE_ERR_BAD_ARG;
  if (workspace_bytes < L.total_bytes) return MOE_ERR_WORKSPACE;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int launches = 0;
  return from_cuda(moe::launch_router(*cfg, static_cast<const __nv_bfloat16*>(x_bf16), router, router_bias, tokens,
                                      reinterpret_cast<float*>(ws + L.logits),
                                      reinterpret_cast<int32_t*>(ws + L.topk_ids),
                                      reinterpret_cast<float*>(ws + L.topk_weights), expert_ids, weights,
                                      static_cast<cudaStream_t>(stream), &launches));
}

int moe_quantize_rows(const void* x, int32_t dtype, int32_t rows, int32_t width, const int32_t* gather, uint8_t* q,
                      float* scales, void* stream) {
  if (!x || !q || !scales || rows < 0 || width < 1 || (dtype != 0 && dtype != 1)) return MOE_ERR_BAD_ARG;
  int launches = 0;
  return from_cuda(moe::launch_quantize(x, dtype, rows, width, gather, q, scales, static_cast<cudaStream_t>(stream),
                                        &launches));
}

int moe_quantize_rows_ue8m0(const void* x, int32_t dtype, int32_t rows, int32_t width, int32_t block, uint8_t* q,
                            uint8_t* scales, void* stream) {
  if (!x || !q || !scales || rows < 0 || width < 1 || (dtype != 0 && dtype != 1)) return MOE_ERR_BAD_ARG;
  if (block != 32 && block != 128) return MOE_ERR_UNSUPPORTED;
  return from_cuda(moe::launch_quantize_ue8m0(x, dtype, rows, width, block, q, scales, static_cast<cudaStream_t>(stream)));
}

int moe_group_rows(const int64_t* ids, int32_t n, int32_t id_base, int32_t n_local, int64_t* order, int32_t* counts,
                   void* stream) {
  if (!ids || !order || !counts || n < 0 || n_local < 1 || n_local > MOE_MAX_EXPERTS || n > 32768) return MOE_ERR_BAD_ARG;
  moe::GroupArgs a;
  std::memset(&a, 0, sizeof(a));
  a.ids64 = ids;
  a.n = n;
  a.id_base = id_base;
  a.n_local = n_local;
  a.topk = 1;
  a.tile = 1;
  a.counts = counts;
  a.order = order;
  int launches = 0;
  return from_cuda(moe::launch_group_rows(a, static_cast<cudaStream_t>(stream), &launches));
}

int moe_combine(const void* rows_bf16, const float* weights, int32_t tokens, int32_t topk, int32_t hidden, int32_t shared,
                void* y_bf16, void* stream) {
  if (!rows_bf16 || !weights || !y_bf16 || tokens < 1 || topk < 1 || hidden < 8 || hidden % 8) return MOE_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(rows_bf16) | reinterpret_cast<uintptr_t>(y_bf16)) & 15) return MOE_ERR_BAD_ARG;
  int launches = 0;
  return from_cuda(moe::launch_combine(static_cast<const __nv_bfloat16*>(rows_bf16), weights, tokens, topk, hidden,
                                       shared ? 1 : 0, static_cast<__nv_bfloat16*>(y_bf16),
                                       static_cast<cudaStream_t>(stream), &launches));
}

// One layer call; with `norm_weight` the whole block: RMSNorm in front, residual add behind.
static int layer_forward_impl(const moe_config_t* cfg, const moe_weights_t* w, const void* x_in, int32_t tokens,
                              void* y_bf16, int64_t* expert_ids, float* topk_weights, int64_t* order, void* workspace,
                              size_t workspace_bytes, void* stream_, const void* norm_weight, float eps,
                              int weight_in_fp32) {
  moe_workspace_layout_t L;
  const int rc = layout_of(cfg, tokens, &L);
  if (rc) return rc;
  if (cfg->ep_world != 1) return MOE_ERR_UNSUPPORTED;
  const void* x_bf16 = x_in;
  if (!w || !x_bf16 || !y_bf16 || !workspace) return MOE_ERR_BAD_ARG;
  if (!w->router || !w->gate || !w->gate_scale || !w->up || !w->up_scale || !w->down || !w->down_scale) return MOE_ERR_BAD_ARG;
  if (cfg->n_shared && (!w->shared_gate || !w->shared_gate_scale || !w->shared_up || !w->shared_up_scale ||
                        !w->shared_down || !w->shared_down_scale))
    return MOE_ERR_BAD_ARG;
  if (workspace_bytes < L.total_bytes) return MOE_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return MOE_ERR_BAD_ARG;

  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(ws + L.status);
  float* logits = reinterpret_cast<float*>(ws + L.logits);
  int32_t* ids32 = reinterpret_cast<int32_t*>(ws + L.topk_ids);
  float* tw = reinterpret_cast<float*>(ws + L.topk_weights);
  moe::Chunk* chunks = reinterpret_cast<moe::Chunk*>(ws + L.chunks);
  int32_t* n_chunks = reinterpret_cast<int32_t*>(ws + L.n_chunks);
  int32_t* row_token = reinterpret_cast<int32_t*>(ws + L.row_token);
  int32_t* row_dest = reinterpret_cast<int32_t*>(ws + L.row_dest);
  uint8_t* xq = ws + L.xq;
  float* xs = reinterpret_cast<float*>(ws + L.xs);
  uint8_t* aq = ws + L.aq;
  float* as = reinterpret_cast<float*>(ws + L.as);
  __nv_bfloat16* slots = reinterpret_cast<__nv_bfloat16*>(ws + L.slots);

  const int n_local = cfg->n_experts;
  const int routed = tokens * cfg->topk;
  int launches = 0;
  cudaError_t e = cudaSuccess;      // the status words are cleared by the permutation kernel (see zero_status)

  const __nv_bfloat16* residual = nullptr;
  if (norm_weight) {
    // the normalised rows live behind the last scratch array of the layout (counted in total_bytes)
    __nv_bfloat16* normalised = reinterpret_cast<__nv_bfloat16*>(ws + norm_offset(L, cfg->hidden));
    e = moe::launch_rmsnorm(static_cast<const __nv_bfloat16*>(x_in), static_cast<const __nv_bfloat16*>(norm_weight), eps,
                            weight_in_fp32, tokens, cfg->hidden, normalised, stream, &launches);
    if (e != cudaSuccess) return from_cuda(e);
    residual = static_cast<const __nv_bfloat16*>(x_in);
    x_bf16 = normalised;
  }

  moe::GroupArgs g;
  std::memset(&g, 0, sizeof(g));
  g.ids32 = ids32;
  g.n = routed;
  g.id_base = 0;
  g.n_local = n_local;
  g.topk = cfg->topk;
  g.shared_rows = cfg->n_shared ? tokens : 0;
  g.tile = L.token_tile;
  g.max_chunks = L.max_chunks;
  g.counts = reinterpret_cast<int32_t*>(ws + L.counts);
  g.offsets = reinterpret_cast<int32_t*>(ws + L.offsets);
  g.n_chunks = n_chunks;
  g.chunks = chunks;
  g.row_token = row_token;
  g.row_dest = row_dest;
  g.order = order;
  g.status = status;
  g.zero_status = 1;       // no kernel before the permutation reports, so no memset node in front of the call
  const moe::WorkListLayout W = moe::work_list_layout(L.max_chunks, cfg->hidden, cfg->inter, L.token_tile,
                                                      fold_tokens(cfg, tokens));
  g.progress = reinterpret_cast<int32_t*>(ws + L.chunks + W.counters);
  g.progress_len = W.counters_len;

  // The shared expert's weights are needed whatever the router decides: the logits kernel asks
  // the L2 for them while HBM has little else to do.
  moe::L2Warm warm = {};
  warm.stamp = status;
  if (cfg->n_shared) {
    const uint64_t bytes = static_cast<uint64_t>(cfg->inter) * cfg->hidden;
    warm.ptr[0] = w->shared_gate; warm.bytes[0] = bytes;
    warm.ptr[1] = w->shared_up; warm.bytes[1] = bytes;
    warm.ptr[2] = w->shared_down; warm.bytes[2] = bytes;
  }

  // Large batches quantise from the token side (every routed row is kept here: all experts are local).
  const bool fused_route = !g_profile && moe::fused_route_fits(*cfg, tokens);
  const bool scatter = !fused_route && cfg->topk <= 16 && moe::quantize_scatter_fits(tokens, cfg->hidden, x_bf16);
  if (scatter) g.slot_pos = reinterpret_cast<int32_t*>(ws + slot_pos_offset(L, cfg->hidden, tokens));

  mark(0, stream);
  if (fused_route) {
    // small batch: logits, then selection + permutation + quantiser in one launch (steps 1-3 below)
    e = moe::launch_router_fused(*cfg, static_cast<const __nv_bfloat16*>(x_bf16), w->router, w->router_bias, tokens,
                                 logits, ids32, tw, expert_ids, topk_weights, g, xq, xs, stream, &launches, &warm);
    if (e != cudaSuccess) return from_cuda(e);
  } else {
    // 1. router
    e = moe::launch_router(*cfg, static_cast<const __nv_bfloat16*>(x_bf16), w->router, w->router_bias, tokens, logits,
                           ids32, tw, expert_ids, topk_weights, stream, &launches, g_profile ? nullptr : &warm);
    if (e != cudaSuccess) return from_cuda(e);

    // 2. token -> expert permutation and the work list of the GEMMs
    mark(1, stream);
    e = moe::launch_group_rows(g, stream, &launches);
    if (e != cudaSuccess) return from_cuda(e);

    // 3. activation quantiser, gathering each grouped row from its token
    mark(2, stream);
    if (scatter)
      e = moe::launch_quantize_scatter(static_cast<const __nv_bfloat16*>(x_bf16), tokens, cfg->hidden, cfg->topk,
                                       g.slot_pos, cfg->n_shared ? routed : -1, xq, xs, stream, &launches);
    else
      e = moe::launch_quantize(x_bf16, 0, L.rows, cfg->hidden, row_token, xq, xs, stream, &launches);
    if (e != cudaSuccess) return from_cuda(e);
  }

  // 4. gate/up GEMM + SwiGLU + requantisation; 5. down GEMM into slot rows
  mark(3, stream);
  moe::GemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.tile = L.token_tile;
  a.n_local = n_local;
  a.total_rows = L.rows;
  a.chunks = chunks;
  a.n_chunks = n_chunks;
  a.status = status;
  // per-stage timing wants the two GEMMs apart; 128-row tiles run them one after the other as well
  a.progress = g_profile || L.token_tile == 128 ? nullptr : g.progress;
  a.max_chunks = L.max_chunks;
  a.tiles_before = cfg->inter / 128;
  int driver_error = 0;

  // One tile of rows in all (batch 1) and a partial last wave of gate/up items: the CTAs of the two GEMMs
  // are sized to be resident on an SM together (rings of 3 and 2 steps), so that down items run beside the
  // last gate/up items.
  // (Only when the gate/up items make more than one wave: a single full wave streams at the HBM rate
  // and would only lose its deeper ring. Measured at batch 1: Mixtral shape 101 -> 90 us with, DeepSeek
  // shape 110 -> 114 us with.)
  const bool together = a.progress != nullptr && L.rows <= 16 &&
                        static_cast<long long>(std::min(L.rows, n_local + cfg->n_shared)) * (cfg->inter / 128) > sm_count();
  a.dual = true;
  a.max_stages = together ? 3 : 0;
  a.k = cfg->hidden;
  a.m = cfg->inter;
  a.max_units = L.max_chunks * (cfg->inter / 128);
  a.act = xq;
  a.act_scale = xs;
  a.w_a = w->gate; a.w_a_scale = w->gate_scale;
  a.w_b = w->up; a.w_b_scale = w->up_scale;
  a.s_a = w->shared_gate; a.s_a_scale = w->shared_gate_scale;
  a.s_b = w->shared_up; a.s_b_scale = w->shared_up_scale;
  a.aq = aq;
  a.as = as;
  // The clamp acts on bf16 values and gives a bf16 value (`gate.clamp(max=bound)` on the bf16 GEMM
  // output, megabench/tasks/megamoe.py:119-121), so the bound counts rounded to bf16.
  a.swiglu.limit = __bfloat162float(__float2bfloat16_rn(cfg->swiglu_limit));
  if (cfg->weight_before_requant) {
    a.swiglu.slot_weight = tw;
    a.swiglu.row_dest = row_dest;
    a.swiglu.routed_rows = tokens * cfg->topk;
  }
  e = moe::launch_gemm(cfg->gemm_impl, a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return from_cuda(e);

  mark(4, stream);
  a.dual = false;
  a.max_stages = together ? 2 : 0;
  a.k = cfg->inter;
  a.m = cfg->hidden;
  a.max_units = L.max_chunks * (cfg->hidden / 128);
  a.ksplit = moe::down_ksplit(cfg->inter);
  a.partial = reinterpret_cast<float*>(ws + L.chunks + W.partial);
  a.parts_done = reinterpret_cast<int32_t*>(ws + L.chunks + W.parts_done);
  a.act = aq;
  a.act_scale = as;
  a.w_a = w->down; a.w_a_scale = w->down_scale;
  a.w_b = nullptr; a.w_b_scale = nullptr;
  a.s_a = w->shared_down; a.s_a_scale = w->shared_down_scale;
  a.s_b = nullptr; a.s_b_scale = nullptr;
  a.aq = nullptr;
  a.as = nullptr;
  a.out = slots;
  a.row_dest = row_dest;
  a.swiglu = moe::SwigluMode{};
  // Small batches: the CTA that stores a token's last slot row of a channel tile adds the rows up
  // itself (the combine kernel's arithmetic on the same stored rows), which saves the launch.
  const bool fold = !g_profile && cfg->gemm_impl == MOE_GEMM_TCGEN05 && fold_tokens(cfg, tokens) > 0;
  if (fold) {
    a.fold.y = static_cast<__nv_bfloat16*>(y_bf16);
    a.fold.weights = cfg->weight_before_requant ? nullptr : tw;
    a.fold.residual = residual;
    a.fold.count = reinterpret_cast<int32_t*>(ws + L.chunks + W.fold_count);
    a.fold.tokens = tokens;
    a.fold.topk = cfg->topk;
    a.fold.shared = cfg->n_shared;
  }
  e = moe::launch_gemm(cfg->gemm_impl, a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return from_cuda(e);

  // 6. weighted combine in slot order, plus the shared expert's row
  mark(5, stream);
  if (!fold)
    e = moe::launch_combine(slots, cfg->weight_before_requant ? nullptr : tw, tokens, cfg->topk, cfg->hidden, cfg->n_shared,
                            static_cast<__nv_bfloat16*>(y_bf16), stream, &launches, residual);
  mark(6, stream);
  g_last_launches = launches;
  return from_cuda(e);
}

int moe_layer_forward(const moe_config_t* cfg, const moe_weights_t* w, const void* x_bf16, int32_t tokens,
                      void* y_bf16, int64_t* expert_ids, float* topk_weights, int64_t* order, void* workspace,
                      size_t workspace_bytes, void* stream) {
  return layer_forward_impl(cfg, w, x_bf16, tokens, y_bf16, expert_ids, topk_weights, order, workspace, workspace_bytes,
                            stream, nullptr, 0.f, 0);
}

int moe_block_forward(const moe_config_t* cfg, const moe_weights_t* w, const void* x_bf16, const void* norm_weight_bf16,
                      float eps, int32_t weight_in_fp32, int32_t tokens, void* x_out_bf16, int64_t* expert_ids,
                      float* topk_weights, int64_t* order, void* workspace, size_t workspace_bytes, void* stream) {
  if (!norm_weight_bf16 || !(eps >= 0.f)) return MOE_ERR_BAD_ARG;
  return layer_forward_impl(cfg, w, x_bf16, tokens, x_out_bf16, expert_ids, topk_weights, order, workspace,
                            workspace_bytes, stream, norm_weight_bf16, eps, weight_in_fp32 ? 1 : 0);
}

int moe_profile_enable(int32_t on) {
  g_profile = on != 0;
  return MOE_OK;
}

int moe_profile_read(float* stage_ms, int32_t n) {
  if (!stage_ms || n < kStages) return MOE_ERR_BAD_ARG;
  if (!g_events_ready) return MOE_ERR_BAD_ARG;
  cudaError_t e = cudaEventSynchronize(g_events[kStages]);
  for (int i = 0; i < kStages && e == cudaSuccess; ++i) e = cudaEventElapsedTime(stage_ms + i, g_events[i], g_events[i + 1]);
  return from_cuda(e);
}

int moe_device_status(const void* workspace, void* stream, int32_t* detail) {
  if (!workspace) return MOE_ERR_BAD_ARG;
  int32_t host[2] = {0, 0};
  cudaError_t e = cudaMemcpyAsync(host, workspace, sizeof(host), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  if (detail) *detail = host[1];
  return host[0];
}

int moe_last_launch_count(void) { return g_last_launches; }

}  // extern "C"
