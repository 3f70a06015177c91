// moe_experts_forward: the local experts applied to rows that are already quantised and carry
// their expert id, result rows in the input order.
//
// Reference boundary: `experts(case, values, rows, scales, local_ids, ...)` of
// megabench/tasks/megamoe.py:131-150 (rows grouped per expert by a stable sort, one GEMM pair per
// expert, `output[selected] = ...`) with the FP8 block-scaled weight format of
// megabench/tasks/quantization.py:119-131 and the unweighted SwiGLU of megabench/tasks/frontier.py:337.
// It is the piece a host-driven expert-parallel loop (NCCL all-to-all around the experts, as the
// reference runs it) needs from this library; the layer entry points use the same kernels.
#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace {

struct ExpertsLayout {
  uint64_t status, counts, offsets, n_chunks, chunks, row_source, row_dest, xq, xs, aq, as, total;
  int rows, max_chunks, tile;
};

inline uint64_t up256(uint64_t v) { return (v + 255) / 256 * 256; }

int experts_layout(const moe_config_t* c, int n_rows, ExpertsLayout* L) {
  const int rc = moe_workspace_layout(c, 1, nullptr);     // geometry checks
  if (rc != MOE_OK) return rc;
  if (n_rows < 1 || n_rows > 32768) return MOE_ERR_UNSUPPORTED;
  const int n_local = c->n_experts / c->ep_world;
  const uint64_t H = c->hidden, I = c->inter;
  const int tile = moe::pick_token_tile(n_rows, n_local);
  // sized for the narrowest tile: a call for the shared expert alone picks its own (all rows are one expert's)
  const int max_chunks = std::min(n_rows, n_local) + n_rows / 16 + (n_rows + 15) / 16 + 1;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) { const uint64_t at = off; off = up256(off + bytes); return at; };
  L->status = take(32);
  L->counts = take(4ull * (n_local + 1));
  L->offsets = take(4ull * (n_local + 2));
  L->n_chunks = take(4);
  L->chunks = take(moe::work_list_layout(max_chunks, c->hidden, c->inter, 64).bytes);   // work items, counters, partial tiles
  L->row_source = take(4ull * n_rows);
  L->row_dest = take(4ull * n_rows);
  L->xq = take(static_cast<uint64_t>(n_rows) * H);
  L->xs = take(4ull * n_rows * (H / 128));
  L->aq = take(static_cast<uint64_t>(n_rows) * I);
  L->as = take(4ull * n_rows * (I / 128));
  L->total = off;
  L->rows = n_rows;
  L->max_chunks = max_chunks;
  L->tile = tile;
  return MOE_OK;
}

inline int cuda_rc(cudaError_t e) { return e == cudaSuccess ? MOE_OK : static_cast<int>(e); }

}  // namespace

extern "C" {

int moe_experts_workspace(const moe_config_t* cfg, int32_t n_rows, uint64_t* bytes) {
  ExpertsLayout L;
  const int rc = experts_layout(cfg, n_rows, &L);
  if (rc) return rc;
  if (bytes) *bytes = L.total;
  return MOE_OK;
}

int moe_experts_forward(const moe_config_t* cfg, const moe_weights_t* w, const uint8_t* rows_q, const float* rows_scale,
                        const int32_t* local_ids, int32_t n_rows, void* out_bf16, void* workspace, size_t workspace_bytes,
                        void* stream_) {
  ExpertsLayout L;
  const int rc = experts_layout(cfg, n_rows, &L);
  if (rc) return rc;
  if (cfg->weight_before_requant) return MOE_ERR_UNSUPPORTED;   // the rows' routing weights are not known here
  if (!w || !rows_q || !rows_scale || !out_bf16 || !workspace) return MOE_ERR_BAD_ARG;
  const bool shared = local_ids == nullptr;
  if (shared ? (!cfg->n_shared || !w->shared_gate || !w->shared_gate_scale || !w->shared_up || !w->shared_up_scale ||
                !w->shared_down || !w->shared_down_scale)
             : (!w->gate || !w->gate_scale || !w->up || !w->up_scale || !w->down || !w->down_scale))
    return MOE_ERR_BAD_ARG;
  if (workspace_bytes < L.total) return MOE_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return MOE_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(ws + L.status);
  const int n_local = cfg->n_experts / cfg->ep_world;
  int launches = 0;
  cudaError_t e = cudaMemsetAsync(status, 0, 32, stream);
  if (e != cudaSuccess) return cuda_rc(e);

  moe::GroupArgs g;
  std::memset(&g, 0, sizeof(g));
  g.ids32 = local_ids;                 // unused when n == 0
  g.n = shared ? 0 : n_rows;
  g.n_local = n_local;
  g.topk = 1;
  g.shared_rows = shared ? n_rows : 0;
  const int tile = shared ? moe::pick_token_tile(n_rows, 1) : L.tile;
  g.tile = tile;
  g.max_chunks = L.max_chunks;
  g.counts = reinterpret_cast<int32_t*>(ws + L.counts);
  g.offsets = reinterpret_cast<int32_t*>(ws + L.offsets);
  g.n_chunks = reinterpret_cast<int32_t*>(ws + L.n_chunks);
  g.chunks = reinterpret_cast<moe::Chunk*>(ws + L.chunks);
  g.row_token = reinterpret_cast<int32_t*>(ws + L.row_source);
  g.row_dest = reinterpret_cast<int32_t*>(ws + L.row_dest);
  g.status = status;
  const moe::WorkListLayout W = moe::work_list_layout(L.max_chunks, cfg->hidden, cfg->inter, 64);
  g.progress = reinterpret_cast<int32_t*>(ws + L.chunks + W.counters);
  g.progress_len = W.counters_len;
  e = moe::launch_group_rows(g, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);

  moe::GatherArgs ga;
  ga.row_source = g.row_token;
  ga.offsets = g.offsets;
  ga.n_local = n_local;
  ga.shared_rows = g.shared_rows;
  ga.hidden = cfg->hidden;
  ga.recv_q = rows_q; ga.recv_s = rows_scale;
  ga.xq_home = rows_q; ga.xs_home = rows_scale;
  ga.xq = ws + L.xq;
  ga.xs = reinterpret_cast<float*>(ws + L.xs);
  e = moe::launch_gather_rows(ga, n_rows, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);

  moe::GemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.tile = tile;
  a.n_local = n_local;
  a.total_rows = n_rows;
  a.chunks = g.chunks;
  a.n_chunks = g.n_chunks;
  a.status = status;
  a.progress = g.progress;
  a.max_chunks = L.max_chunks;
  a.tiles_before = cfg->inter / 128;
  int driver_error = 0;
  a.dual = true;
  a.k = cfg->hidden; a.m = cfg->inter;
  a.max_units = L.max_chunks * (cfg->inter / 128);
  a.act = ga.xq; a.act_scale = ga.xs;
  a.w_a = w->gate; a.w_a_scale = w->gate_scale; a.w_b = w->up; a.w_b_scale = w->up_scale;
  a.s_a = w->shared_gate; a.s_a_scale = w->shared_gate_scale; a.s_b = w->shared_up; a.s_b_scale = w->shared_up_scale;
  if (shared) { a.n_local = 0; a.w_a = nullptr; a.w_b = nullptr; }
  a.aq = ws + L.aq; a.as = reinterpret_cast<float*>(ws + L.as);
  a.swiglu.limit = __bfloat162float(__float2bfloat16_rn(cfg->swiglu_limit));   // the clamp gives bf16 values
  e = moe::launch_gemm(cfg->gemm_impl, a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);
  a.dual = false;
  a.k = cfg->inter; a.m = cfg->hidden;
  a.max_units = L.max_chunks * (cfg->hidden / 128);
  a.ksplit = moe::down_ksplit(cfg->inter);
  a.partial = reinterpret_cast<float*>(ws + L.chunks + W.partial);
  a.parts_done = reinterpret_cast<int32_t*>(ws + L.chunks + W.parts_done);
  a.act = ws + L.aq; a.act_scale = reinterpret_cast<const float*>(ws + L.as);
  a.w_a = shared ? nullptr : w->down; a.w_a_scale = w->down_scale; a.w_b = nullptr; a.w_b_scale = nullptr;
  a.s_a = w->shared_down; a.s_a_scale = w->shared_down_scale; a.s_b = nullptr; a.s_b_scale = nullptr;
  a.aq = nullptr; a.as = nullptr;
  a.swiglu = moe::SwigluMode{};
  a.out = static_cast<__nv_bfloat16*>(out_bf16);
  a.row_dest = g.row_dest;
  e = moe::launch_gemm(cfg->gemm_impl, a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  moe::note_launches(launches);
  return cuda_rc(e);
}

}  // extern "C"
