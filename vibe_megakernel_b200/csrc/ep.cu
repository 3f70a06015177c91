// Expert-parallel layer: dispatch and return of routed rows as peer stores from inside the kernels.
//
// Reference: megabench/tasks/megamoe.py:153-182 (owner order, all-to-all dispatch, local experts,
// all-to-all back, slot-order combine) with megabench/tasks/parallel.py:52-68 as the collective.
// Here the source rank's quantiser kernel writes each routed row (e4m3 payload, fp32 group scales,
// local expert id, slot row to return to) directly into the owner's receive buffer at a position
// that depends only on (source rank, token, slot) order; the last block to finish publishes the
// row counts and raises one flag per destination. The owner polls the flags of all sources with a
// bounded wait, groups the arrivals by expert (same stable counting sort as on one GPU), runs the
// grouped GEMMs, and a return kernel stores every finished row into its source's slot buffer and
// raises the return flags; the source combines once all owners have reported.
//
// A row's result does not depend on the other rows multiplied with it (every token is its own MMA
// column with a fixed K order), so expert-parallel results equal single-GPU results bit for bit
// whatever the arrival order.
//
// Waits give up after 2 s and report MOE_ERR_DEVICE_TIMEOUT; nothing spins forever.
#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "kernels.h"
#include "quant_group.cuh"

namespace moe {

struct EpLocal {       // offsets inside the private scratch
  uint64_t status, counters, logits, topk_ids, topk_weights, xq_home, xs_home, counts, offsets, n_chunks, chunks,
      row_source, xq, xs, aq, as, out, total;
};

static inline uint64_t up256(uint64_t v) { return (v + 255) / 256 * 256; }

static void ep_layouts(const moe_config_t& c, int max_tokens, moe_ep_layout_t* L, EpLocal* P) {
  const int world = c.ep_world;
  const int n_local = c.n_experts / world;
  const uint64_t H = c.hidden, I = c.inter;
  const int cap = max_tokens * c.topk;
  const int rows = world * cap + max_tokens;
  const int tile = moe::pick_token_tile(static_cast<long long>(world) * cap, c.n_experts, c.gemm_impl == MOE_GEMM_TCGEN05 ? 128 : 64);
  const int max_chunks = std::min(world * cap, n_local) + world * cap / tile + (max_tokens + tile - 1) / tile + 1;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) { const uint64_t at = off; off = up256(off + bytes); return at; };
  std::memset(L, 0, sizeof(*L));
  L->flags_dispatch = take(8ull * world);
  L->flags_return = take(8ull * world);
  L->recv_count = take(4ull * world);
  L->recv_expert = take(4ull * world * cap);
  L->recv_slot = take(4ull * world * cap);
  L->recv_weight = take(4ull * world * cap);
  L->recv_q = take(static_cast<uint64_t>(world) * cap * H);
  L->recv_s = take(4ull * world * cap * (H / 128));
  L->slots = take(2ull * (cap + max_tokens) * H);
  L->exchange_bytes = off;
  L->cap = cap;
  L->rows = rows;
  L->max_chunks = max_chunks;
  L->token_tile = tile;
  off = 0;
  P->status = take(32);
  P->counters = take(32);
  P->logits = take(4ull * max_tokens * c.n_experts);
  P->topk_ids = take(4ull * cap);
  P->topk_weights = take(4ull * cap);
  P->xq_home = take(static_cast<uint64_t>(max_tokens) * H);
  P->xs_home = take(4ull * max_tokens * (H / 128));
  P->counts = take(4ull * (n_local + 1));
  P->offsets = take(4ull * (n_local + 2));
  P->n_chunks = take(4);
  P->chunks = take(moe::work_list_layout(max_chunks, c.hidden, c.inter, tile).bytes);   // work items, counters, partial tiles
  P->row_source = take(4ull * rows);
  P->xq = take(static_cast<uint64_t>(rows) * H);
  P->xs = take(4ull * rows * (H / 128));
  P->aq = take(static_cast<uint64_t>(rows) * I);
  P->as = take(4ull * rows * (I / 128));
  P->out = take(2ull * rows * H);
  P->total = off;
  L->local_bytes = off;
}

struct Peers {
  uint8_t* base[8];
};

// ---- dispatch: quantise each routed row and store it into its owner's receive buffer -----------
struct DispatchArgs {
  const __nv_bfloat16* x;
  const int32_t* ids;        // [tokens*topk] global expert ids, (token, slot) order
  int tokens, hidden, topk, world, rank, n_local, cap;
  Peers peers;
  uint64_t off_count, off_expert, off_slot, off_q, off_s, off_flags;
  uint8_t* xq_home;          // local copy for the shared expert: [tokens, H]
  float* xs_home;
  int32_t* done;
  uint64_t epoch;
  int64_t* order;            // optional [tokens*topk]: the stable order of the routed rows by owning rank
};

__global__ void __launch_bounds__(256) ep_dispatch_kernel(DispatchArgs a) {
  __shared__ int s_part[8];
  __shared__ int s_lower[8];
  __shared__ int s_counts[8];
  __shared__ int s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int routed = a.tokens * a.topk;
  const int r = blockIdx.x;
  const int H = a.hidden, G = H / kGroup;
  dependent_wait();             // the picks come from the kernel before
  dependents_may_launch();
  int t;
  uint8_t* dst_q;
  float* dst_s;
  if (r < routed) {
    t = r / a.topk;
    const int e = a.ids[r];
    const int d = e / a.n_local;
    int before = 0;                      // earlier rows of this rank bound for the same owner
    int lower = 0;                       // rows bound for owners of lower rank (only counted when the order is wanted)
    for (int q = tid; q < r; q += 256) before += (a.ids[q] / a.n_local == d);
    if (a.order)
      for (int q = tid; q < routed; q += 256) lower += (a.ids[q] / a.n_local < d);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      before += __shfl_xor_sync(0xffffffffu, before, off);
      lower += __shfl_xor_sync(0xffffffffu, lower, off);
    }
    if (lane == 0) { s_part[warp] = before; s_lower[warp] = lower; }
    __syncthreads();
    int j = 0, below = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) { j += s_part[w]; below += s_lower[w]; }
    // position of row r in `torch.sort(owner, stable=True)` (megabench/tasks/megamoe.py:161-164)
    if (a.order && tid == 0) a.order[below + j] = r;
    const size_t row = static_cast<size_t>(a.rank) * a.cap + j;
    uint8_t* peer = a.peers.base[d];
    dst_q = peer + a.off_q + row * H;
    dst_s = reinterpret_cast<float*>(peer + a.off_s) + row * G;
    if (tid == 0) {
      reinterpret_cast<int32_t*>(peer + a.off_expert)[row] = e - d * a.n_local;
      reinterpret_cast<int32_t*>(peer + a.off_slot)[row] = r;
    }
  } else {
    t = r - routed;
    dst_q = a.xq_home + static_cast<size_t>(t) * H;
    dst_s = a.xs_home + static_cast<size_t>(t) * G;
  }
  // per-row, per-128-channel e4m3 quantiser (megabench/tasks/quantization.py:87-109), one warp per group
  const __nv_bfloat16* in = a.x + static_cast<size_t>(t) * H;
  constexpr int kAhead = 4;       // groups whose loads a warp issues before it uses the first
  for (int g0 = warp; g0 < G; g0 += 8 * kAhead) {
    float v[kAhead][4];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) load_group<__nv_bfloat16>(in, min(g0 + 8 * u, G - 1), H, lane, v[u]);
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int g = g0 + 8 * u;
      if (g < G) {
        const float scale = quantize_loaded(v[u], dst_q, g, H, lane);
        if (lane == 0) dst_s[g] = scale;
      }
    }
  }
  // the last block to finish publishes the counts and raises one flag per owner
  __threadfence_system();
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(a.done, 1) == static_cast<int>(gridDim.x) - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (tid < 8) s_counts[tid] = 0;
  __syncthreads();
  for (int q = tid; q < routed; q += 256) atomicAdd(&s_counts[a.ids[q] / a.n_local], 1);
  __syncthreads();
  if (tid < a.world) {
    uint8_t* peer = a.peers.base[tid];
    reinterpret_cast<int32_t*>(peer + a.off_count)[a.rank] = s_counts[tid];
    __threadfence_system();
    store_release_sys(reinterpret_cast<uint64_t*>(peer + a.off_flags) + a.rank, a.epoch);
  }
  if (tid == 0) *a.done = 0;
}

// ---- bounded wait for `world` flags to reach `epoch` --------------------------------------------
__global__ void ep_wait_kernel(const uint64_t* flags, int world, uint64_t epoch, int32_t* status, int detail,
                               uint64_t timeout_ns) {
  const int tid = threadIdx.x;
  dependent_wait();             // under a dependent launch: polling starts when the predecessor is done
  dependents_may_launch();
  if (tid >= world) return;
  const uint64_t t0 = globaltimer();
  while (load_acquire_sys(flags + tid) < epoch) {
    if (globaltimer() - t0 > timeout_ns) {
      report(status, MOE_ERR_DEVICE_TIMEOUT, detail + tid);
      break;
    }
    __nanosleep(64);
  }
}

// ---- owner side: bring arrivals (and the home rows of the shared expert) into expert order ------
__global__ void __launch_bounds__(128) ep_gather_kernel(GatherArgs a) {
  dependent_wait();
  dependents_may_launch();
  const int kept = a.offsets[a.n_local];
  const int pos = blockIdx.x;
  if (pos >= kept + a.shared_rows) return;
  const int H = a.hidden, G = H / kGroup;
  const int src = a.row_source[pos];
  const uint8_t* q = (pos < kept ? a.recv_q : a.xq_home) + static_cast<size_t>(src) * H;
  const float* s = (pos < kept ? a.recv_s : a.xs_home) + static_cast<size_t>(src) * G;
  uint4* dq = reinterpret_cast<uint4*>(a.xq + static_cast<size_t>(pos) * H);
  for (int i = threadIdx.x; i < H / 16; i += 128) dq[i] = reinterpret_cast<const uint4*>(q)[i];
  for (int i = threadIdx.x; i < G; i += 128) a.xs[static_cast<size_t>(pos) * G + i] = s[i];
}

cudaError_t launch_gather_rows(const GatherArgs& a, int row_blocks, cudaStream_t stream, int* launches) {
  launch_dependent(ep_gather_kernel, dim3(row_blocks > 0 ? row_blocks : 1), dim3(128), 0, stream, a);
  if (launches) *launches += 1;
  return cudaGetLastError();
}

// ---- return: store every finished row into its source's slot buffer, then raise the flags --------
struct ReturnArgs {
  const __nv_bfloat16* out;    // [rows, H] grouped order
  const int32_t* row_source;
  const int32_t* offsets;
  const int32_t* recv_slot;
  int n_local, shared_rows, hidden, cap, world, rank, home_tokens, topk;
  Peers peers;
  uint64_t off_slots, off_flags;
  int32_t* done;
  uint64_t epoch;
};

__global__ void __launch_bounds__(128) ep_return_kernel(ReturnArgs a) {
  __shared__ int s_last;
  dependent_wait();
  dependents_may_launch();
  const int kept = a.offsets[a.n_local];
  const int pos = blockIdx.x;
  const int H = a.hidden;
  if (pos < kept + a.shared_rows) {
    const int src = a.row_source[pos];
    uint8_t* peer;
    size_t slot;
    if (pos < kept) {
      peer = a.peers.base[src / a.cap];
      slot = static_cast<size_t>(a.recv_slot[src]);
    } else {
      peer = a.peers.base[a.rank];
      slot = static_cast<size_t>(a.home_tokens) * a.topk + src;
    }
    uint4* d = reinterpret_cast<uint4*>(peer + a.off_slots + slot * H * 2);
    const uint4* s = reinterpret_cast<const uint4*>(a.out + static_cast<size_t>(pos) * H);
    for (int i = threadIdx.x; i < H / 8; i += 128) d[i] = s[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(a.done, 1) == static_cast<int>(gridDim.x) - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x < a.world)
    store_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.off_flags) + a.rank, a.epoch);
  if (threadIdx.x == 0) *a.done = 0;
}

// =============================================================================================
// The same exchange for the routed experts in the MegaMoE-native formats (MXFP4 weights, E4M3 rows
// with one E8M0 scale per 32 channels): the expert-parallel form of megabench/tasks/megamoe.py:153-182.
// Routing is an input and the rows arrive quantised, so the dispatching kernel only copies: payload,
// scale bytes, local expert id, slot to return to, and the fp32 routing weight (the four dispatched
// tensors of megabench/tasks/megamoe.py:167-173). The owner multiplies the weight into the SwiGLU
// output before requantisation, so the source's combine is a plain slot-order sum.
// =============================================================================================
struct MxEpLocal {
  uint64_t status, counters, counts, offsets, n_chunks, chunks, row_source, xq, xs, aq, as, out, total;
};

static void mx_ep_layouts(const moe_config_t& c, int max_tokens, moe_ep_layout_t* L, MxEpLocal* P) {
  const int world = c.ep_world;
  const int n_local = c.n_experts / world;
  const uint64_t H = c.hidden, I = c.inter;
  const int cap = max_tokens * c.topk;
  const int rows = world * cap;
  const int tile = moe::pick_token_tile(rows, c.n_experts, c.hidden % 256 == 0 ? 128 : 64, moe::kMxWideAbove);
  const int max_chunks = std::min(rows, n_local) + rows / tile + 1;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) { const uint64_t at = off; off = up256(off + bytes); return at; };
  std::memset(L, 0, sizeof(*L));
  L->flags_dispatch = take(8ull * world);
  L->flags_return = take(8ull * world);
  L->recv_count = take(4ull * world);
  L->recv_expert = take(4ull * rows);
  L->recv_slot = take(4ull * rows);
  L->recv_weight = take(4ull * rows);
  L->recv_q = take(static_cast<uint64_t>(rows) * H);
  L->recv_s = take(static_cast<uint64_t>(rows) * (H / 32));
  L->slots = take(2ull * cap * H);
  L->exchange_bytes = off;
  L->cap = cap;
  L->rows = rows;
  L->max_chunks = max_chunks;
  L->token_tile = tile;
  off = 0;
  P->status = take(32);
  P->counters = take(32);
  P->counts = take(4ull * (n_local + 1));
  P->offsets = take(4ull * (n_local + 2));
  P->n_chunks = take(4);
  P->chunks = take(16ull * max_chunks);
  P->row_source = take(4ull * rows);
  P->xq = take(static_cast<uint64_t>(rows) * H);
  P->xs = take(static_cast<uint64_t>(rows) * (H / 32));
  P->aq = take(static_cast<uint64_t>(rows) * I);
  P->as = take(static_cast<uint64_t>(rows) * (I / 32));
  P->out = take(2ull * rows * H);
  P->total = off;
  L->local_bytes = off;
}

struct MxDispatchArgs {
  const uint8_t* x;          // e4m3 [tokens, H]
  const uint8_t* x_scales;   // E8M0 [tokens, H/32]
  const int64_t* ids;        // [tokens*topk] global expert ids, (token, slot) order
  const float* weights;      // [tokens*topk]
  int tokens, hidden, topk, world, rank, n_local, cap;
  Peers peers;
  uint64_t off_count, off_expert, off_slot, off_weight, off_q, off_s, off_flags;
  int32_t* done;
  uint64_t epoch;
  int64_t* order;            // optional: stable order of the routed rows by owning rank (rows without an owner last)
};

// owner of a routed row, -1 when its expert id is out of range (such a row is not sent)
__device__ __forceinline__ int mx_owner(long long id, int n_local, int world) {
  return (id >= 0 && id < static_cast<long long>(n_local) * world) ? static_cast<int>(id / n_local) : -1;
}

constexpr int kMxDispatchRows = 8;      // routed rows per block of the dispatch kernel: one per warp

// Every block stages the owner of every routed row in shared memory once (a byte each); a warp then
// finds its row's place among the rows of the same owner and in the owner order by counting over
// that array, and copies the row to the owner. (One block per row, each counting over the ids in
// global memory, took 59 us for 3,072 rows.)
__global__ void __launch_bounds__(256) mx_ep_dispatch_kernel(MxDispatchArgs a) {
  extern __shared__ int8_t s_owner[];      // [routed]
  __shared__ int s_counts[8];
  __shared__ int s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int routed = a.tokens * a.topk;
  const int H = a.hidden;
  dependent_wait();
  dependents_may_launch();
  for (int q = tid; q < routed; q += 256) s_owner[q] = static_cast<int8_t>(mx_owner(a.ids[q], a.n_local, a.world));
  __syncthreads();
  const int r = blockIdx.x * kMxDispatchRows + warp;
  if (r < routed) {
    const int d = s_owner[r];
    int before = 0, lower = 0;
    for (int q = lane; q < routed; q += 32) {
      const int o = s_owner[q];
      before += (q < r && o == d);
      lower += d >= 0 ? (o >= 0 && o < d) : (o >= 0);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      before += __shfl_xor_sync(0xffffffffu, before, off);
      lower += __shfl_xor_sync(0xffffffffu, lower, off);
    }
    if (a.order && lane == 0) a.order[lower + before] = r;       // megabench/tasks/megamoe.py:161-164
    if (d >= 0) {
      const int t = r / a.topk;
      const size_t row = static_cast<size_t>(a.rank) * a.cap + before;
      uint8_t* peer = a.peers.base[d];
      uint4* dq = reinterpret_cast<uint4*>(peer + a.off_q + row * H);
      const uint4* sq = reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(t) * H);
      for (int i = lane; i < H / 16; i += 32) dq[i] = sq[i];
      uint32_t* ds = reinterpret_cast<uint32_t*>(peer + a.off_s + row * (H / 32));
      const uint32_t* ss = reinterpret_cast<const uint32_t*>(a.x_scales + static_cast<size_t>(t) * (H / 32));
      for (int i = lane; i < H / 128; i += 32) ds[i] = ss[i];
      if (lane == 0) {
        reinterpret_cast<int32_t*>(peer + a.off_expert)[row] =
            static_cast<int>(a.ids[r] - static_cast<long long>(d) * a.n_local);
        reinterpret_cast<int32_t*>(peer + a.off_slot)[row] = r;
        reinterpret_cast<float*>(peer + a.off_weight)[row] = a.weights[r];
      }
    }
  }
  // the last block to finish publishes the counts and raises one flag per owner
  __threadfence_system();
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(a.done, 1) == static_cast<int>(gridDim.x) - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (tid < 8) s_counts[tid] = 0;
  __syncthreads();
  for (int q = tid; q < routed; q += 256) {
    const int o = s_owner[q];
    if (o >= 0) atomicAdd(&s_counts[o], 1);
  }
  __syncthreads();
  if (tid < a.world) {
    uint8_t* peer = a.peers.base[tid];
    reinterpret_cast<int32_t*>(peer + a.off_count)[a.rank] = s_counts[tid];
    __threadfence_system();
    store_release_sys(reinterpret_cast<uint64_t*>(peer + a.off_flags) + a.rank, a.epoch);
  }
  if (tid == 0) *a.done = 0;
}

}  // namespace moe

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
namespace {

int ep_check(const moe_config_t* c, int max_tokens) {
  if (!c) return MOE_ERR_BAD_ARG;
  const int rc = moe_workspace_layout(c, 1, nullptr);      // geometry checks shared with the one-GPU path
  if (rc != MOE_OK) return rc;
  if (c->ep_world > 8 || c->weight_before_requant) return MOE_ERR_UNSUPPORTED;
  if (max_tokens < 1) return MOE_ERR_BAD_ARG;
  if (static_cast<int64_t>(c->ep_world) * max_tokens * c->topk > 32768) return MOE_ERR_UNSUPPORTED;
  return MOE_OK;
}

inline int cuda_rc(cudaError_t e) { return e == cudaSuccess ? MOE_OK : static_cast<int>(e); }

}  // namespace

extern "C" {

int moe_ep_layout(const moe_config_t* cfg, int32_t max_tokens, moe_ep_layout_t* layout) {
  const int rc = ep_check(cfg, max_tokens);
  if (rc) return rc;
  moe_ep_layout_t L;
  moe::EpLocal P;
  moe::ep_layouts(*cfg, max_tokens, &L, &P);
  if (layout) *layout = L;
  return MOE_OK;
}

int moe_ep_forward(const moe_config_t* cfg, const moe_weights_t* w, const void* x_bf16, int32_t tokens,
                   int32_t max_tokens, void* y_bf16, int64_t* expert_ids, float* topk_weights, int64_t* order,
                   void* const* exchange, void* local, size_t local_bytes, uint64_t epoch, void* stream_) {
  const int rc = ep_check(cfg, max_tokens);
  if (rc) return rc;
  if (!w || !x_bf16 || !y_bf16 || !exchange || !local || tokens < 1 || tokens > max_tokens || epoch == 0)
    return MOE_ERR_BAD_ARG;
  if (!w->router || !w->gate || !w->gate_scale || !w->up || !w->up_scale || !w->down || !w->down_scale) return MOE_ERR_BAD_ARG;
  if (cfg->n_shared && (!w->shared_gate || !w->shared_gate_scale || !w->shared_up || !w->shared_up_scale ||
                        !w->shared_down || !w->shared_down_scale))
    return MOE_ERR_BAD_ARG;
  moe_ep_layout_t L;
  moe::EpLocal P;
  moe::ep_layouts(*cfg, max_tokens, &L, &P);
  if (local_bytes < L.local_bytes) return MOE_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(local) & 255) return MOE_ERR_BAD_ARG;
  const int world = cfg->ep_world, rank = cfg->ep_rank;
  moe::Peers peers;
  for (int i = 0; i < 8; ++i) peers.base[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    if (!exchange[i] || (reinterpret_cast<uintptr_t>(exchange[i]) & 255)) return MOE_ERR_BAD_ARG;
    peers.base[i] = static_cast<uint8_t*>(exchange[i]);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(local);
  uint8_t* mine = peers.base[rank];
  int32_t* status = reinterpret_cast<int32_t*>(ws + P.status);
  int32_t* counters = reinterpret_cast<int32_t*>(ws + P.counters);
  int32_t* ids32 = reinterpret_cast<int32_t*>(ws + P.topk_ids);
  float* tw = reinterpret_cast<float*>(ws + P.topk_weights);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + P.offsets);
  int32_t* row_source = reinterpret_cast<int32_t*>(ws + P.row_source);
  const int n_local = cfg->n_experts / world;
  const int H = cfg->hidden;
  int launches = 0;

  // counters are only ever left at zero by the kernels; the status word is cleared per call
  cudaError_t e = cudaMemsetAsync(status, 0, epoch == 1 ? 64 + 256 : 32, stream);
  if (e != cudaSuccess) return cuda_rc(e);

  // 1. router on the home tokens
  moe::L2Warm warm = {};      // the shared expert's weights are needed whatever the router decides
  if (cfg->n_shared) {
    const uint64_t bytes = static_cast<uint64_t>(cfg->inter) * cfg->hidden;
    warm.ptr[0] = w->shared_gate; warm.bytes[0] = bytes;
    warm.ptr[1] = w->shared_up; warm.bytes[1] = bytes;
    warm.ptr[2] = w->shared_down; warm.bytes[2] = bytes;
  }
  e = moe::launch_router(*cfg, static_cast<const __nv_bfloat16*>(x_bf16), w->router, w->router_bias, tokens,
                         reinterpret_cast<float*>(ws + P.logits), ids32, tw, expert_ids, topk_weights, stream, &launches,
                         &warm);
  if (e != cudaSuccess) return cuda_rc(e);

  // 2. quantise + dispatch (peer stores), counts and flags published by the last block
  moe::DispatchArgs d;
  d.x = static_cast<const __nv_bfloat16*>(x_bf16);
  d.ids = ids32;
  d.tokens = tokens; d.hidden = H; d.topk = cfg->topk; d.world = world; d.rank = rank; d.n_local = n_local; d.cap = L.cap;
  d.peers = peers;
  d.off_count = L.recv_count; d.off_expert = L.recv_expert; d.off_slot = L.recv_slot; d.off_q = L.recv_q;
  d.off_s = L.recv_s; d.off_flags = L.flags_dispatch;
  d.xq_home = ws + P.xq_home;
  d.xs_home = reinterpret_cast<float*>(ws + P.xs_home);
  d.done = counters;
  d.epoch = epoch;
  d.order = order;
  moe::launch_dependent(moe::ep_dispatch_kernel, dim3(tokens * cfg->topk + tokens), dim3(256), 0, stream, d);
  ++launches;

  // 3. the grouping kernel waits for every source (bounded), then groups the arrivals by expert
  moe::GroupArgs g;
  std::memset(&g, 0, sizeof(g));
  g.wait = moe::FlagWait{reinterpret_cast<const uint64_t*>(mine + L.flags_dispatch), world, epoch, moe::kWaitNs, status, 200};
  g.ids32 = reinterpret_cast<const int32_t*>(mine + L.recv_expert);
  g.n = world * L.cap;
  g.id_base = 0;
  g.n_local = n_local;
  g.topk = 1;
  g.shared_rows = cfg->n_shared ? tokens : 0;
  g.tile = L.token_tile;
  g.max_chunks = L.max_chunks;
  g.counts = reinterpret_cast<int32_t*>(ws + P.counts);
  g.offsets = offsets;
  g.n_chunks = reinterpret_cast<int32_t*>(ws + P.n_chunks);
  g.chunks = reinterpret_cast<moe::Chunk*>(ws + P.chunks);
  g.row_token = row_source;
  g.status = status;
  g.seg_counts = reinterpret_cast<const int32_t*>(mine + L.recv_count);
  g.seg_cap = L.cap;
  const moe::WorkListLayout W = moe::work_list_layout(L.max_chunks, cfg->hidden, cfg->inter, L.token_tile);
  g.progress = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(g.chunks) + W.counters);
  g.progress_len = W.counters_len;
  e = moe::launch_group_rows(g, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);

  moe::GatherArgs ga;
  ga.row_source = row_source; ga.offsets = offsets; ga.n_local = n_local; ga.shared_rows = g.shared_rows; ga.hidden = H;
  ga.recv_q = mine + L.recv_q;
  ga.recv_s = reinterpret_cast<const float*>(mine + L.recv_s);
  ga.xq_home = ws + P.xq_home;
  ga.xs_home = reinterpret_cast<const float*>(ws + P.xs_home);
  ga.xq = ws + P.xq;
  ga.xs = reinterpret_cast<float*>(ws + P.xs);
  const int row_blocks = world * L.cap + g.shared_rows;
  e = moe::launch_gather_rows(ga, row_blocks, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);

  // 4. grouped GEMMs on the local experts (and the shared expert for the home tokens)
  moe::GemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.tile = L.token_tile;
  a.n_local = n_local;
  a.total_rows = L.rows;
  a.chunks = g.chunks;
  a.n_chunks = g.n_chunks;
  a.status = status;
  a.progress = L.token_tile == 128 ? nullptr : g.progress;      // 128-row tiles run the two GEMMs one after the other
  a.max_chunks = L.max_chunks;
  a.tiles_before = cfg->inter / 128;
  int driver_error = 0;
  a.dual = true;
  a.k = H; a.m = cfg->inter;
  a.max_units = L.max_chunks * (cfg->inter / 128);
  a.act = ws + P.xq; a.act_scale = reinterpret_cast<const float*>(ws + P.xs);
  a.w_a = w->gate; a.w_a_scale = w->gate_scale; a.w_b = w->up; a.w_b_scale = w->up_scale;
  a.s_a = w->shared_gate; a.s_a_scale = w->shared_gate_scale; a.s_b = w->shared_up; a.s_b_scale = w->shared_up_scale;
  a.aq = ws + P.aq; a.as = reinterpret_cast<float*>(ws + P.as);
  a.swiglu.limit = __bfloat162float(__float2bfloat16_rn(cfg->swiglu_limit));   // the clamp gives bf16 values
  e = moe::launch_gemm(cfg->gemm_impl, a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);
  a.dual = false;
  a.k = cfg->inter; a.m = H;
  a.max_units = L.max_chunks * (H / 128);
  a.ksplit = moe::down_ksplit(cfg->inter);
  a.partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(g.chunks) + W.partial);
  a.parts_done = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(g.chunks) + W.parts_done);
  a.act = ws + P.aq; a.act_scale = reinterpret_cast<const float*>(ws + P.as);
  a.w_a = w->down; a.w_a_scale = w->down_scale; a.w_b = nullptr; a.w_b_scale = nullptr;
  a.s_a = w->shared_down; a.s_a_scale = w->shared_down_scale; a.s_b = nullptr; a.s_b_scale = nullptr;
  a.aq = nullptr; a.as = nullptr;
  a.swiglu = moe::SwigluMode{};
  a.out = reinterpret_cast<__nv_bfloat16*>(ws + P.out);
  a.row_dest = nullptr;
  // 5. rows go home as peer stores, flags raised when all are on their way: from the down GEMM's own
  // epilogue and last CTA (the weights-on-M tensor-core kernel), else by a copy kernel behind it
  const bool fold_return = cfg->gemm_impl == MOE_GEMM_TCGEN05 && L.token_tile != 128;
  if (fold_return) {
    for (int r = 0; r < 8; ++r) a.ret.base[r] = r < world ? peers.base[r] : nullptr;
    a.ret.row_source = row_source;
    a.ret.recv_slot = reinterpret_cast<const int32_t*>(mine + L.recv_slot);
    a.ret.offsets = offsets;
    a.ret.n_local = n_local; a.ret.cap = L.cap; a.ret.world = world; a.ret.rank = rank;
    a.ret.home_tokens = tokens; a.ret.topk = cfg->topk;
    a.ret.off_slots = L.slots; a.ret.off_flags = L.flags_return;
    a.ret.done = counters + 1;
    a.ret.epoch = epoch;
  }
  e = moe::launch_gemm(cfg->gemm_impl, a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);

  if (!fold_return) {
    moe::ReturnArgs r;
    r.out = a.out; r.row_source = row_source; r.offsets = offsets;
    r.recv_slot = reinterpret_cast<const int32_t*>(mine + L.recv_slot);
    r.n_local = n_local; r.shared_rows = g.shared_rows; r.hidden = H; r.cap = L.cap; r.world = world; r.rank = rank;
    r.home_tokens = tokens; r.topk = cfg->topk;
    r.peers = peers;
    r.off_slots = L.slots; r.off_flags = L.flags_return;
    r.done = counters + 1;
    r.epoch = epoch;
    moe::launch_dependent(moe::ep_return_kernel, dim3(row_blocks), dim3(128), 0, stream, r);
    ++launches;
  }
  // 6. wait for all owners, combine
  const moe::FlagWait home{reinterpret_cast<const uint64_t*>(mine + L.flags_return), world, epoch, moe::kWaitNs, status, 300};
  e = moe::launch_combine(reinterpret_cast<const __nv_bfloat16*>(mine + L.slots), tw, tokens, cfg->topk, H, cfg->n_shared,
                          static_cast<__nv_bfloat16*>(y_bf16), stream, &launches, nullptr, &home);
  moe::note_launches(launches);
  return cuda_rc(e);
}

static int mx_ep_check(const moe_config_t* c, int max_tokens) {
  if (!c) return MOE_ERR_BAD_ARG;
  if (c->hidden < 128 || c->inter < 128 || c->n_experts < 1 || c->topk < 1 || c->topk > c->n_experts || max_tokens < 1 ||
      !(c->swiglu_limit >= 0.f) || c->ep_world < 1 || c->ep_rank < 0 || c->ep_rank >= c->ep_world)
    return MOE_ERR_BAD_ARG;
  if (c->hidden % 128 || c->inter % 128 || c->n_experts > MOE_MAX_EXPERTS || c->n_shared != 0 || c->ep_world > 8 ||
      c->n_experts % c->ep_world || static_cast<int64_t>(c->ep_world) * max_tokens * c->topk > 32768)
    return MOE_ERR_UNSUPPORTED;
  return MOE_OK;
}

int moe_mx_ep_layout(const moe_config_t* cfg, int32_t max_tokens, moe_ep_layout_t* layout) {
  const int rc = mx_ep_check(cfg, max_tokens);
  if (rc) return rc;
  moe_ep_layout_t L;
  moe::MxEpLocal P;
  moe::mx_ep_layouts(*cfg, max_tokens, &L, &P);
  if (layout) *layout = L;
  return MOE_OK;
}

int moe_mx_ep_forward(const moe_config_t* cfg, const moe_mx_weights_t* w, const uint8_t* x_q, const uint8_t* x_scales,
                      const int64_t* topk_idx, const float* topk_weights, int32_t tokens, int32_t max_tokens, void* y_bf16,
                      int64_t* order, void* const* exchange, void* local, size_t local_bytes, uint64_t epoch,
                      void* stream_) {
  const int rc = mx_ep_check(cfg, max_tokens);
  if (rc) return rc;
  if (!w || !w->l1_blocks || !w->l1_scales || !w->l2_blocks || !w->l2_scales || !x_q || !x_scales || !topk_idx ||
      !topk_weights || !y_bf16 || !exchange || !local || tokens < 1 || tokens > max_tokens || epoch == 0)
    return MOE_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(w->l1_blocks) & 31 || reinterpret_cast<uintptr_t>(w->l2_blocks) & 31 ||
      reinterpret_cast<uintptr_t>(w->l1_scales) & 15 || reinterpret_cast<uintptr_t>(w->l2_scales) & 15 ||
      reinterpret_cast<uintptr_t>(x_q) & 15 || reinterpret_cast<uintptr_t>(x_scales) & 3)
    return MOE_ERR_BAD_ARG;
  moe_ep_layout_t L;
  moe::MxEpLocal P;
  moe::mx_ep_layouts(*cfg, max_tokens, &L, &P);
  if (local_bytes < L.local_bytes) return MOE_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(local) & 255) return MOE_ERR_BAD_ARG;
  const int world = cfg->ep_world, rank = cfg->ep_rank;
  moe::Peers peers;
  for (int i = 0; i < 8; ++i) peers.base[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    if (!exchange[i] || (reinterpret_cast<uintptr_t>(exchange[i]) & 255)) return MOE_ERR_BAD_ARG;
    peers.base[i] = static_cast<uint8_t*>(exchange[i]);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(local);
  uint8_t* mine = peers.base[rank];
  int32_t* status = reinterpret_cast<int32_t*>(ws + P.status);
  int32_t* counters = reinterpret_cast<int32_t*>(ws + P.counters);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + P.offsets);
  int32_t* row_source = reinterpret_cast<int32_t*>(ws + P.row_source);
  const int n_local = cfg->n_experts / world;
  const int H = cfg->hidden;
  int launches = 0;
  cudaError_t e = cudaMemsetAsync(status, 0, epoch == 1 ? 64 + 256 : 32, stream);
  if (e != cudaSuccess) return cuda_rc(e);

  // 1. dispatch (peer stores): payload, scale bytes, local expert id, slot, routing weight
  moe::MxDispatchArgs d;
  d.x = x_q; d.x_scales = x_scales; d.ids = topk_idx; d.weights = topk_weights;
  d.tokens = tokens; d.hidden = H; d.topk = cfg->topk; d.world = world; d.rank = rank; d.n_local = n_local; d.cap = L.cap;
  d.peers = peers;
  d.off_count = L.recv_count; d.off_expert = L.recv_expert; d.off_slot = L.recv_slot; d.off_weight = L.recv_weight;
  d.off_q = L.recv_q; d.off_s = L.recv_s; d.off_flags = L.flags_dispatch;
  d.done = counters;
  d.epoch = epoch;
  d.order = order;
  moe::launch_dependent(moe::mx_ep_dispatch_kernel, dim3((tokens * cfg->topk + moe::kMxDispatchRows - 1) / moe::kMxDispatchRows),
                        dim3(256), static_cast<size_t>(tokens) * cfg->topk, stream, d);
  ++launches;

  // 2. wait for every source (bounded), group the arrivals by local expert
  moe::GroupArgs g;
  std::memset(&g, 0, sizeof(g));
  g.wait = moe::FlagWait{reinterpret_cast<const uint64_t*>(mine + L.flags_dispatch), world, epoch, moe::kWaitNs, status, 200};
  g.ids32 = reinterpret_cast<const int32_t*>(mine + L.recv_expert);
  g.n = world * L.cap;
  g.id_base = 0;
  g.n_local = n_local;
  g.topk = 1;
  g.shared_rows = 0;
  g.tile = L.token_tile;
  g.max_chunks = L.max_chunks;
  g.counts = reinterpret_cast<int32_t*>(ws + P.counts);
  g.offsets = offsets;
  g.n_chunks = reinterpret_cast<int32_t*>(ws + P.n_chunks);
  g.chunks = reinterpret_cast<moe::Chunk*>(ws + P.chunks);
  g.row_token = row_source;
  g.status = status;
  g.seg_counts = reinterpret_cast<const int32_t*>(mine + L.recv_count);
  g.seg_cap = L.cap;
  e = moe::launch_group_rows(g, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);

  // 3. arrivals into expert order
  uint8_t* xg = ws + P.xq;
  uint8_t* xgs = ws + P.xs;
  e = moe::launch_gather_mx_rows(mine + L.recv_q, mine + L.recv_s, row_source, offsets + n_local, world * L.cap,
                                 world * L.cap, H, xg, xgs, stream, &launches);
  if (e != cudaSuccess) return cuda_rc(e);

  // 4. linear1 + clamped SwiGLU * routing weight + requantisation; linear2
  moe::MxGemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.tile = L.token_tile;
  a.n_experts = n_local;
  a.total_rows = L.rows;
  a.chunks = g.chunks;
  a.n_chunks = g.n_chunks;
  a.status = status;
  int driver_error = 0;
  a.dual = true;
  a.k = H; a.m = cfg->inter;
  a.max_units = L.max_chunks * (cfg->inter / 128);
  a.act = xg; a.act_scales = xgs;
  a.w_blocks = w->l1_blocks; a.w_scales = w->l1_scales;
  a.aq = ws + P.aq; a.as = ws + P.as;
  a.row_dest = row_source;                                               // grouped row -> arrival index ...
  a.slot_weight = reinterpret_cast<const float*>(mine + L.recv_weight);  // ... whose routing weight travelled with it
  a.limit = __bfloat162float(__float2bfloat16_rn(cfg->swiglu_limit));
  e = moe::launch_gemm_mx(a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);
  a.dual = false;
  a.k = cfg->inter; a.m = H;
  a.max_units = L.max_chunks * (H / 128);
  a.act = ws + P.aq; a.act_scales = ws + P.as;
  a.w_blocks = w->l2_blocks; a.w_scales = w->l2_scales;
  a.aq = nullptr; a.as = nullptr;
  a.out = reinterpret_cast<__nv_bfloat16*>(ws + P.out);
  a.row_dest = nullptr;
  a.slot_weight = nullptr;
  a.limit = 0.f;
  e = moe::launch_gemm_mx(a, stream, &launches, &driver_error);
  if (driver_error) return MOE_ERR_DRIVER;
  if (e != cudaSuccess) return cuda_rc(e);

  // 5. rows go home; 6. wait for all owners, plain slot-order sum
  moe::ReturnArgs r;
  r.out = a.out; r.row_source = row_source; r.offsets = offsets;
  r.recv_slot = reinterpret_cast<const int32_t*>(mine + L.recv_slot);
  r.n_local = n_local; r.shared_rows = 0; r.hidden = H; r.cap = L.cap; r.world = world; r.rank = rank;
  r.home_tokens = tokens; r.topk = cfg->topk;
  r.peers = peers;
  r.off_slots = L.slots; r.off_flags = L.flags_return;
  r.done = counters + 1;
  r.epoch = epoch;
  moe::launch_dependent(moe::ep_return_kernel, dim3(world * L.cap), dim3(128), 0, stream, r);
  ++launches;
  const moe::FlagWait home{reinterpret_cast<const uint64_t*>(mine + L.flags_return), world, epoch, moe::kWaitNs, status, 300};
  e = moe::launch_combine(reinterpret_cast<const __nv_bfloat16*>(mine + L.slots), nullptr, tokens, cfg->topk, H, 0,
                          static_cast<__nv_bfloat16*>(y_bf16), stream, &launches, nullptr, &home);
  moe::note_launches(launches);
  return cuda_rc(e);
}

int moe_ep_wait_flags(const uint64_t* flags, int32_t world, uint64_t epoch, uint64_t timeout_ns, void* status_words,
                      void* stream) {
  if (!flags || !status_words || world < 1 || world > 8 || timeout_ns == 0 || timeout_ns > moe::kWaitNs)
    return MOE_ERR_BAD_ARG;
  moe::ep_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, world, epoch,
                                                                      static_cast<int32_t*>(status_words), 200, timeout_ns);
  return cuda_rc(cudaGetLastError());
}

int moe_ep_buffer_alloc(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes == 0) return MOE_ERR_BAD_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(*ptr, 0, bytes);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), *ptr);
  if (e != cudaSuccess) {
    cudaFree(*ptr);
    *ptr = nullptr;
  }
  return cuda_rc(e);
}

int moe_ep_buffer_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return MOE_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  return cuda_rc(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

int moe_ep_buffer_close(void* ptr) { return ptr ? cuda_rc(cudaIpcCloseMemHandle(ptr)) : MOE_ERR_BAD_ARG; }

int moe_ep_buffer_free(void* ptr) { return ptr ? cuda_rc(cudaFree(ptr)) : MOE_ERR_BAD_ARG; }

}  // extern "C"
