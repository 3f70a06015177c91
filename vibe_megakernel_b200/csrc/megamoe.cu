// The routed experts in the MegaMoE-native formats behind the C ABI: permutation of the routed
// rows (routing is an input), gather of the E4M3 rows with their E8M0 scales into expert order,
// linear1 + clamped SwiGLU + requantisation, linear2 into slot rows, plain slot-order sum.
// Reference: megabench/tasks/megamoe.py:131-182 with serial=True.
#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace moe {

// One block per grouped row: 16-byte pieces of the payload, then the scale bytes. Only the first
// *kept rows exist: a routed row whose expert id is out of range was dropped by the grouping and
// the tail of row_token is not written.
__global__ void __launch_bounds__(128) gather_mx_rows_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ x_scales,
                                                             const int32_t* __restrict__ row_token,
                                                             const int32_t* __restrict__ kept, int tokens, int hidden,
                                                             uint8_t* __restrict__ xg, uint8_t* __restrict__ xgs) {
  dependent_wait();
  dependents_may_launch();
  const size_t row = blockIdx.x;
  if (static_cast<int>(blockIdx.x) >= *kept) return;
  const int token = row_token[row];
  if (token < 0 || token >= tokens) return;
  const size_t src = static_cast<size_t>(token);
  const uint4* in = reinterpret_cast<const uint4*>(x + src * hidden);
  uint4* out = reinterpret_cast<uint4*>(xg + row * hidden);
  for (int i = threadIdx.x; i < hidden / 16; i += blockDim.x) out[i] = in[i];
  const int ks = hidden / 32;
  for (int i = threadIdx.x; i < ks; i += blockDim.x) xgs[row * ks + i] = x_scales[src * ks + i];
}

cudaError_t launch_gather_mx_rows(const uint8_t* x, const uint8_t* x_scales, const int32_t* row_token, const int32_t* kept,
                                  int rows, int tokens, int hidden, uint8_t* xg, uint8_t* xgs, cudaStream_t stream,
                                  int* launches) {
  if (rows <= 0) return cudaSuccess;
  launch_dependent(gather_mx_rows_kernel, dim3(rows), dim3(128), 0, stream, x, x_scales, row_token, kept, tokens, hidden, xg,
                   xgs);
  if (launches) *launches += 1;
  return cudaGetLastError();
}

}  // namespace moe

namespace {

inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

struct MxLayout {
  uint64_t status, counts, offsets, n_chunks, chunks, row_token, row_dest, xg, xgs, aq, as, slots, total;
  int rows, tile, max_chunks;
};

int mx_layout(const moe_config_t* c, int tokens, MxLayout* L) {
  if (!c) return MOE_ERR_BAD_ARG;
  if (c->hidden < 128 || c->inter < 128 || c->n_experts < 1 || c->topk < 1 || c->topk > c->n_experts || tokens < 1 ||
      !(c->swiglu_limit >= 0.f))
    return MOE_ERR_BAD_ARG;
  if (c->hidden % 128 || c->inter % 128 || c->n_experts > MOE_MAX_EXPERTS || c->n_shared != 0 || c->ep_world != 1 ||
      static_cast<int64_t>(tokens) * c->topk > 32768)
    return MOE_ERR_UNSUPPORTED;
  const int rows = tokens * c->topk;
  const uint64_t H = c->hidden, I = c->inter;
  MxLayout l;
  l.rows = rows;
  l.tile = moe::pick_token_tile(rows, c->n_experts, c->hidden % 256 == 0 ? 128 : 64, moe::kMxWideAbove);
  l.max_chunks = std::min(rows, c->n_experts) + rows / l.tile + 1;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) { const uint64_t at = off; off = align_up(off + bytes, 256); return at; };
  l.status = take(8 * 4);
  l.counts = take(4ull * (c->n_experts + 1));
  l.offsets = take(4ull * (c->n_experts + 2));
  l.n_chunks = take(4);
  l.chunks = take(16ull * l.max_chunks);
  l.row_token = take(4ull * rows);
  l.row_dest = take(4ull * rows);
  l.xg = take(rows * H);
  l.xgs = take(rows * (H / 32));
  l.aq = take(rows * I);
  l.as = take(rows * (I / 32));
  l.slots = take(2ull * rows * H);
  l.total = off;
  *L = l;
  return MOE_OK;
}

inline int from_cuda(cudaError_t e) { return e == cudaSuccess ? MOE_OK : static_cast<int>(e); }

}  // namespace

extern "C" {

int moe_mx_workspace(const moe_config_t* cfg, int32_t tokens, uint64_t* bytes) {
  MxLayout L;
  const int rc = mx_layout(cfg, tokens, &L);
  if (rc) return rc;
  if (bytes) *bytes = L.total;
  return MOE_OK;
}

int moe_mx_forward(const moe_config_t* cfg, const moe_mx_weights_t* w, const uint8_t* x_q, const uint8_t* x_scales,
                   const int64_t* topk_idx, const float* topk_weights, int32_t tokens, void* y_bf16, int64_t* order,
                   void* workspace, size_t workspace_bytes, void* stream_) {
  MxLayout L;
  const int rc = mx_layout(cfg, tokens, &L);
  if (rc) return rc;
  if (!w || !w->l1_blocks || !w->l1_scales || !w->l2_blocks || !w->l2_scales || !x_q || !x_scales || !topk_idx ||
      !topk_weights || !y_bf16 || !workspace)
    return MOE_ERR_BAD_ARG;
  if (workspace_bytes < L.total) return MOE_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255 || reinterpret_cast<uintptr_t>(x_q) & 15) return MOE_ERR_BAD_ARG;
  // the weight tiles move by TMA as packed 4-bit values (32-byte aligned base), the scale rows by 16-byte copies
  if (reinterpret_cast<uintptr_t>(w->l1_blocks) & 31 || reinterpret_cast<uintptr_t>(w->l2_blocks) & 31 ||
      reinterpret_cast<uintptr_t>(w->l1_scales) & 15 || reinterpret_cast<uintptr_t>(w->l2_scales) & 15)
    return MOE_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(ws + L.status);
  int launches = 0;

  // 1. token -> expert permutation and the work list
  moe::GroupArgs g;
  std::memset(&g, 0, sizeof(g));
  g.ids64 = topk_idx;
  g.n = L.rows;
  g.id_base = 0;
  g.n_local = cfg->n_experts;
  g.topk = cfg->topk;
  g.shared_rows = 0;
  g.tile = L.tile;
  g.max_chunks = L.max_chunks;
  g.counts = reinterpret_cast<int32_t*>(ws + L.counts);
  g.offsets = reinterpret_cast<int32_t*>(ws + L.offsets);
  g.n_chunks = reinterpret_cast<int32_t*>(ws + L.n_chunks);
  g.chunks = reinterpret_cast<moe::Chunk*>(ws + L.chunks);
  g.row_token = reinterpret_cast<int32_t*>(ws + L.row_token);
  g.row_dest = reinterpret_cast<int32_t*>(ws + L.row_dest);
  g.order = order;
  g.status = status;
  g.zero_status = 1;
  cudaError_t e = moe::launch_group_rows(g, stream, &launches);
  if (e != cudaSuccess) return from_cuda(e);

  // 2. rows into expert order
  uint8_t* xg = ws + L.xg;
  uint8_t* xgs = ws + L.xgs;
  e = moe::launch_gather_mx_rows(x_q, x_scales, g.row_token, g.offsets + cfg->n_experts, L.rows, tokens, cfg->hidden, xg, xgs,
                                 stream, &launches);
  if (e != cudaSuccess) return from_cuda(e);

  // 3. linear1 + SwiGLU + requantisation; 4. linear2 into slot rows
  moe::MxGemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.tile = L.tile;
  a.n_experts = cfg->n_experts;
  a.total_rows = L.rows;
  a.chunks = g.chunks;
  a.n_chunks = g.n_chunks;
  a.status = status;
  int driver_error = 0;

  a.dual = true;
  a.k = cfg->hidden;
  a.m = cfg->inter;
  a.max_units = L.max_chunks * (cfg->inter / 128);
  a.act = xg;
  a.act_scales = xgs;
  a.w_blocks = w->l1_blocks;
  a.w_scales = w->l1_scales;
  a.aq = ws + L.aq;
  a.as = ws + L.as;
  a.row_dest = g.row_dest;
  a.slot_weight = topk_weights;
  // the clamp acts on bf16 values (megabench/tasks/megamoe.py:119-121): the bound counts rounded to bf16
  a.limit = __bfloat162float(__float2bfloat16_rn(cfg->swiglu_limit));
  e = moe::launch_gemm_mx(a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return from_cuda(e);

  a.dual = false;
  a.k = cfg->inter;
  a.m = cfg->hidden;
  a.max_units = L.max_chunks * (cfg->hidden / 128);
  a.act = ws + L.aq;
  a.act_scales = ws + L.as;
  a.w_blocks = w->l2_blocks;
  a.w_scales = w->l2_scales;
  a.aq = nullptr;
  a.as = nullptr;
  a.out = reinterpret_cast<__nv_bfloat16*>(ws + L.slots);
  a.slot_weight = nullptr;
  a.limit = 0.f;
  e = moe::launch_gemm_mx(a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return from_cuda(e);

  // 5. fp32 sum over the slots in slot order, one bf16 rounding (megabench/tasks/megamoe.py:176-182)
  e = moe::launch_combine(reinterpret_cast<const __nv_bfloat16*>(ws + L.slots), nullptr, tokens, cfg->topk, cfg->hidden, 0,
                          static_cast<__nv_bfloat16*>(y_bf16), stream, &launches);
  moe::note_launches(launches);
  return from_cuda(e);
}

}  // extern "C"
