// Router, second half: per-token expert selection by one warp from the fp32 logits.
//
// Selection rules reproduced (reference: megabench/tasks/frontier.py:229-242 for the sigmoid
// group-limited router; megabench/tasks/distributed.py:174-176 for the stable softmax top-k):
//   sigmoid: p = sigmoid(s), c = p + bias; group score = sum of the group's two largest c; keep the
//            topk_group best groups (ties to the lower group), others -> -inf; ids = first topk of a
//            stable descending sort of c; w = p[ids] / (sum + 1e-20) * scaling.
//   softmax: ids = first topk of a stable descending sort of s; w = softmax(s[ids]).
// Two more scorings ride on the same two shapes (see score_of): sqrt-softplus scores with the
// sigmoid rule's selection bias and normalisation (megabench/tasks/dsv41.py:622-626), and a softmax
// over logits that carry the router's linear bias (megabench/tasks/gptoss.py:106-109).
#include "common.cuh"
#include "group_tables.cuh"
#include "kernels.h"
#include "quant_group.cuh"

namespace moe {

struct RouteArgs {
  const float* logits;
  const float* bias;
  int tokens, experts, topk, scoring, n_group, topk_group;
  float scaling;
  int32_t* ids32;
  float* weights;
  int64_t* ids64;     // optional
  float* weights_out; // optional
};

constexpr int kRouteWarps = 4;

// Score p (what the weights are made of) and selection value c of one logit.
//   sigmoid:        p = sigmoid(s), c = p + bias                (megabench/tasks/frontier.py:229-231)
//   sqrt-softplus:  p = sqrt(softplus(s)), c = p + bias         (megabench/tasks/dsv41.py:623-624; softplus with
//                   torch's threshold: s itself above 20)
//   softmax:        p = c = s
//   biased softmax: p = c = s + bias                            (megabench/tasks/gptoss.py:106)
__device__ __forceinline__ void score_of(int scoring, float s, float bias, float& p, float& c) {
  if (scoring == MOE_SCORING_SIGMOID) {
    p = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-s)));
    c = __fadd_rn(p, bias);
  } else if (scoring == MOE_SCORING_SQRT_SOFTPLUS) {
    p = __fsqrt_rn(s > 20.f ? s : log1pf(expf(s)));
    c = __fadd_rn(p, bias);
  } else if (scoring == MOE_SCORING_SOFTMAX_BIASED) {
    p = __fadd_rn(s, bias);
    c = p;
  } else {
    p = s;
    c = s;
  }
}
// The rules whose weights are p / (sum of the picked p) * scaling and which know router groups;
// the others take a softmax over the picked values.
__device__ __forceinline__ bool normalised_scoring(int scoring) {
  return scoring == MOE_SCORING_SIGMOID || scoring == MOE_SCORING_SQRT_SOFTPLUS;
}

__global__ void __launch_bounds__(kRouteWarps * 32) route_select_kernel(RouteArgs a) {
  __shared__ float s_choice[kRouteWarps][MOE_MAX_EXPERTS];
  __shared__ float s_prob[kRouteWarps][MOE_MAX_EXPERTS];
  __shared__ int s_pick[kRouteWarps][MOE_MAX_TOPK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  dependent_wait();
  dependents_may_launch();
  if (t >= a.tokens) return;
  float* c = s_choice[warp];
  float* p = s_prob[warp];
  const int E = a.experts;
  const float ninf = __int_as_float(0xff800000);

  const bool normalised = normalised_scoring(a.scoring);
  for (int e = lane; e < E; e += 32)
    score_of(a.scoring, a.logits[static_cast<size_t>(t) * E + e], a.bias ? a.bias[e] : 0.f, p[e], c[e]);
  __syncwarp();

  if (normalised && a.n_group > 1) {
    const int gsz = E / a.n_group;
    float score = ninf;
    if (lane < a.n_group) {
      float m1 = ninf, m2 = ninf;
      for (int j0 = 0; j0 < gsz; ++j0) {
        int j = j0 + lane;                  // rotated start: lanes hit different banks
        if (j >= gsz) j -= gsz * (j / gsz);
        const float v = c[lane * gsz + j];
        if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
      }
      score = gsz >= 2 ? __fadd_rn(m1, m2) : m1;
    }
    int rank = 0;
    for (int g = 0; g < a.n_group; ++g) {
      const float other = __shfl_sync(0xffffffffu, score, g);
      if (other > score || (other == score && g < lane)) ++rank;
    }
    const unsigned alive = __ballot_sync(0xffffffffu, lane < a.n_group && rank < a.topk_group);
    for (int e = lane; e < E; e += 32)
      if (!((alive >> (e / gsz)) & 1u)) c[e] = ninf;
    __syncwarp();
  }

  unsigned taken = 0;  // bit i: expert lane + 32*i already picked
  for (int j = 0; j < a.topk; ++j) {
    float bv = ninf;
    int be = -1;
    for (int i = 0; lane + 32 * i < E; ++i) {
      if ((taken >> i) & 1u) continue;
      const int e = lane + 32 * i;
      const float v = c[e];
      if (be < 0 || v > bv) { bv = v; be = e; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oe = __shfl_xor_sync(0xffffffffu, be, off);
      if (oe >= 0 && (be < 0 || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; }
    }
    if (be >= 0 && (be & 31) == lane) taken |= 1u << (be >> 5);
    if (lane == 0) s_pick[warp][j] = be;
  }
  __syncwarp();

  if (lane == 0) {
    float w[MOE_MAX_TOPK];
    if (normalised) {
      float sum = 0.f;
      for (int j = 0; j < a.topk; ++j) { w[j] = p[s_pick[warp][j]]; sum = __fadd_rn(sum, w[j]); }
      const float den = __fadd_rn(sum, 1e-20f);
      for (int j = 0; j < a.topk; ++j) w[j] = __fmul_rn(__fdiv_rn(w[j], den), a.scaling);
    } else {
      const float m = p[s_pick[warp][0]];
      float sum = 0.f;
      for (int j = 0; j < a.topk; ++j) { w[j] = expf(__fsub_rn(p[s_pick[warp][j]], m)); sum = __fadd_rn(sum, w[j]); }
      for (int j = 0; j < a.topk; ++j) w[j] = __fdiv_rn(w[j], sum);
    }
    for (int j = 0; j < a.topk; ++j) {
      const size_t o = static_cast<size_t>(t) * a.topk + j;
      a.ids32[o] = s_pick[warp][j];
      a.weights[o] = w[j];
      if (a.ids64) a.ids64[o] = s_pick[warp][j];
      if (a.weights_out) a.weights_out[o] = w[j];
    }
  }
}

// Register-resident variant for the common shapes: lane l holds experts [l*EPL, (l+1)*EPL) (EPL =
// E/32 values, loaded as one contiguous run), a router group is a whole number of lanes, and every
// step is shuffles over registers instead of shared-memory sweeps. Same rules, same tie order
// (larger value first, lower expert index on equal values).
// One warp selects for token t; lane j < topk returns choice j and its weight.
// `bias_regs` (optional): this lane's EPL bias values, loaded by the caller ahead of time.
template <int EPL>
__device__ __forceinline__ void select_in_registers(const RouteArgs& a, int t, int lane, int& pick, float& weight,
                                                    const float* bias_regs = nullptr) {
  const int E = a.experts;
  const float ninf = __int_as_float(0xff800000);
  const bool sigmoid = normalised_scoring(a.scoring);    // sigmoid-like: grouped, normalised weights
  const int e0 = lane * EPL;
  float p[EPL], c[EPL], s[EPL], b[EPL];
  // E == 32 * EPL here, so every lane's run is in range: plain loads, all issued before first use
#pragma unroll
  for (int i = 0; i < EPL; ++i) s[i] = __ldg(a.logits + static_cast<size_t>(t) * E + e0 + i);
  const bool biased = a.scoring != MOE_SCORING_SOFTMAX && a.bias != nullptr;
#pragma unroll
  for (int i = 0; i < EPL; ++i) b[i] = !biased ? 0.f : bias_regs ? bias_regs[i] : __ldg(a.bias + e0 + i);
#pragma unroll
  for (int i = 0; i < EPL; ++i) score_of(a.scoring, s[i], b[i], p[i], c[i]);
  if (sigmoid && a.n_group > 1) {
    const int gsz = E / a.n_group;
    const int lanes_per_group = gsz / EPL;             // power of two (checked by the launcher)
    float m1 = ninf, m2 = ninf;                         // two largest of this lane, then of its group
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      if (c[i] > m1) { m2 = m1; m1 = c[i]; } else if (c[i] > m2) { m2 = c[i]; }
    }
    for (int off = 1; off < lanes_per_group; off <<= 1) {
      const float o1 = __shfl_xor_sync(0xffffffffu, m1, off);
      const float o2 = __shfl_xor_sync(0xffffffffu, m2, off);
      const float hi = fmaxf(m1, o1);
      const float lo = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
      m1 = hi;
      m2 = lo;
    }
    const float score = gsz >= 2 ? __fadd_rn(m1, m2) : m1;
    const int g = lane / lanes_per_group;               // this lane's group (lanes past E idle)
    const bool live_lane = e0 < E;
    int rank = 0;
    for (int o = 0; o < a.n_group; ++o) {
      const float other = __shfl_sync(0xffffffffu, score, o * lanes_per_group);
      if (other > score || (other == score && o < g)) ++rank;
    }
    if (!live_lane || rank >= a.topk_group) {
#pragma unroll
      for (int i = 0; i < EPL; ++i) c[i] = ninf;
    }
  }
  unsigned taken = 0;
  int my_pick = -1;
  float my_prob = 0.f;
  for (int j = 0; j < a.topk; ++j) {
    float bv = ninf;
    int be = -1;
    float bp = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = e0 + i;
      if (e < E && !((taken >> i) & 1u) && (be < 0 || c[i] > bv)) { bv = c[i]; be = e; bp = p[i]; }
    }
    // Across the warp with two integer reductions: the largest value (floats mapped to unsigned
    // keys of the same order; -0 counts as +0 as in a float comparison), then the lowest expert
    // index among the lanes holding it.
    const unsigned bits = __float_as_uint(bv + 0.f);
    const unsigned key = be < 0 ? 0u : ((bits & 0x80000000u) ? ~bits : (bits | 0x80000000u));
    const unsigned top = __reduce_max_sync(0xffffffffu, key);
    const unsigned lowest =
        __reduce_min_sync(0xffffffffu, (be >= 0 && key == top) ? static_cast<unsigned>(be) : 0xffffffffu);
    const int chosen = static_cast<int>(lowest);            // -1 when nothing was left
    const float chosen_p = __shfl_sync(0xffffffffu, bp, max(chosen, 0) / EPL);
    if (chosen >= 0 && chosen / EPL == lane) taken |= 1u << (chosen - e0);
    if (lane == j) { my_pick = chosen; my_prob = chosen_p; }      // lane j keeps pick j
  }
  // weights: slot-order sum as the scalar reference code, then one division per slot
  float w = 0.f;
  if (sigmoid) {
    float sum = 0.f;
    for (int j = 0; j < a.topk; ++j) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, my_prob, j));
    w = __fmul_rn(__fdiv_rn(my_prob, __fadd_rn(sum, 1e-20f)), a.scaling);
  } else {
    const float m = __shfl_sync(0xffffffffu, my_prob, 0);
    const float ex = expf(__fsub_rn(my_prob, m));
    float sum = 0.f;
    for (int j = 0; j < a.topk; ++j) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, ex, j));
    w = __fdiv_rn(ex, sum);
  }
  pick = my_pick;
  weight = w;
}

template <int EPL>
__global__ void __launch_bounds__(kRouteWarps * 32) route_select_regs_kernel(RouteArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  dependent_wait();
  dependents_may_launch();
  if (t >= a.tokens) return;
  int pick;
  float w;
  select_in_registers<EPL>(a, t, lane, pick, w);
  if (lane < a.topk) {
    const size_t o = static_cast<size_t>(t) * a.topk + lane;
    a.ids32[o] = pick;
    a.weights[o] = w;
    if (a.ids64) a.ids64[o] = pick;
    if (a.weights_out) a.weights_out[o] = w;
  }
}

// Small batches, one launch for everything between the logits and the expert GEMMs: every block
// repeats the selection of all tokens (a warp per token) and the stable grouping of the
// tokens * topk rows (a few hundred comparisons per thread), then quantises the one grouped row
// it is responsible for; block 0 instead publishes ids, weights, permutation and the work list. The
// three separate kernels cost more in launch hand-overs than in work at these sizes. Same device
// functions as the separate kernels, so the bytes are the same.
constexpr int kFusedMaxRows = 512;     // tokens * topk
constexpr int kFusedMaxTokens = 32;    // at 64 the repeated selections cost 80-100 us: three kernels are faster there

struct FusedArgs {
  RouteArgs r;
  GroupArgs g;               // ids32 / n / topk / id_base = 0 / n_local = experts as for the permutation kernel
  const __nv_bfloat16* x;    // [tokens, hidden]
  int hidden;
  uint8_t* xq;               // grouped rows, then the shared expert's rows
  float* xs;
};

template <int EPL, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) route_group_quant_kernel(FusedArgs a) {
  __shared__ int16_t s_id[kFusedMaxRows];
  __shared__ int16_t s_pos[kFusedMaxRows];
  __shared__ float s_w[kFusedMaxRows];
  __shared__ int s_count[MOE_MAX_EXPERTS + 1];
  __shared__ int s_offset[MOE_MAX_EXPERTS + 2];
  __shared__ int s_chunk0[MOE_MAX_EXPERTS + 2];
  __shared__ int s_src;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = a.r.tokens, K = a.r.topk, R = T * K, E = a.r.experts;
  const bool publisher = blockIdx.x == 0;      // block 0 publishes the tables, block 1 + i quantises grouped row i
  const int my_row = static_cast<int>(blockIdx.x) - 1;
  // The selection bias is a weight, not a result of the logits kernel: it is fetched while this
  // kernel still waits for that one (from HBM when the L2 does not hold it, two microseconds).
  float bias_regs[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i)
    bias_regs[i] = (a.r.bias && a.r.scoring != MOE_SCORING_SOFTMAX) ? __ldg(a.r.bias + lane * EPL + i) : 0.f;
  dependent_wait();
  dependents_may_launch();
#ifdef MOE_TIMELINE
  if (tid == 0) MOE_STAMP_LAST(a.g.status, 3);
  if (a.g.zero_status && a.g.status && publisher && tid < 2) a.g.status[tid] = 0;
#else
  if (a.g.zero_status && a.g.status && publisher && tid < 8) a.g.status[tid] = 0;
#endif

  for (int t = warp; t < T; t += WARPS) {       // a warp per token, two rounds beyond 32 tokens
    int pick;
    float w;
    select_in_registers<EPL>(a.r, t, lane, pick, w, bias_regs);
    if (lane < K) {
      s_id[t * K + lane] = static_cast<int16_t>(pick);
      s_w[t * K + lane] = w;
    }
  }
  for (int i = tid; i <= E; i += WARPS * 32) s_count[i] = 0;
  if (tid == 0) s_src = 0;
  __syncthreads();
#if defined(MOE_TIMELINE) && MOE_TIMELINE == 2
  if (tid == 0) MOE_STAMP_LAST(a.g.status, 5);      // selection done
#endif

  // Stable position of every row: rows of lower experts first, then earlier rows of the same one.
  for (int r = tid; r < R; r += WARPS * 32) {
    const int e = s_id[r];
    int pos = 0;
    for (int o = 0; o < R; ++o) {
      const int eo = s_id[o];
      pos += (eo < e || (eo == e && o < r)) ? 1 : 0;
    }
    s_pos[r] = static_cast<int16_t>(pos);
    if (pos == my_row) s_src = r / K;
    if (publisher) atomicAdd(&s_count[e], 1);
  }
  if (my_row >= R && tid == 0) s_src = my_row - R;   // a row of the shared expert
  if (publisher && tid == 0) s_count[E] = a.g.shared_rows;
  __syncthreads();
#if defined(MOE_TIMELINE) && MOE_TIMELINE == 2
  if (tid == 0) MOE_STAMP_LAST(a.g.status, 6);      // positions known
#endif

  if (!publisher) {   // this block's row
    const int groups = (a.hidden + kGroup - 1) / kGroup;
    const __nv_bfloat16* in = a.x + static_cast<size_t>(s_src) * a.hidden;
    uint8_t* out = a.xq + static_cast<size_t>(my_row) * a.hidden;
    constexpr int kAhead = 4;     // groups whose loads a warp issues before it uses the first
    for (int g0 = warp; g0 < groups; g0 += WARPS * kAhead) {
      float v[kAhead][4];
#pragma unroll
      for (int u = 0; u < kAhead; ++u) load_group<__nv_bfloat16>(in, min(g0 + u * WARPS, groups - 1), a.hidden, lane, v[u]);
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int g = g0 + u * WARPS;
        if (g < groups) {
          const float scale = quantize_loaded(v[u], out, g, a.hidden, lane);
          if (lane == 0) a.xs[static_cast<size_t>(my_row) * groups + g] = scale;
        }
      }
    }
  } else {
    if (warp == 0) group_prefix(s_count, s_offset, s_chunk0, E + 1, a.g.tile, lane);
    for (int r = tid; r < R; r += WARPS * 32) {
      const int pos = s_pos[r], id = s_id[r];
      const float w = s_w[r];
      a.r.ids32[r] = id;
      a.r.weights[r] = w;
      if (a.r.ids64) a.r.ids64[r] = id;
      if (a.r.weights_out) a.r.weights_out[r] = w;
      if (a.g.order) a.g.order[pos] = r;
      if (a.g.row_token) a.g.row_token[pos] = r / K;
      if (a.g.row_dest) a.g.row_dest[pos] = r;
    }
    __syncthreads();
#if defined(MOE_TIMELINE) && MOE_TIMELINE == 2
    if (tid == 0) MOE_STAMP_LAST(a.g.status, 7);    // publisher: prefix and per-row outputs written
#endif
    group_publish(a.g, s_count, s_offset, s_chunk0, tid, WARPS * 32);
  }
#ifdef MOE_TIMELINE
  __syncthreads();
  if (tid == 0) MOE_STAMP_LAST(a.g.status, 4);

#endif
}

// True when the register variant applies: E fills whole lanes and groups are whole power-of-two
// runs of lanes.
static bool regs_variant_fits(const moe_config_t& cfg, int epl) {
  if (cfg.n_experts != 32 * epl || cfg.topk > 32) return false;
  if ((cfg.scoring == MOE_SCORING_SIGMOID || cfg.scoring == MOE_SCORING_SQRT_SOFTPLUS) && cfg.n_group > 1) {
    const int gsz = cfg.n_experts / cfg.n_group;
    if (gsz % epl) return false;
    const int lpg = gsz / epl;
    if (lpg & (lpg - 1)) return false;
  }
  return true;
}

static int regs_variant_of(const moe_config_t& cfg) {
  for (int epl : {1, 2, 4, 8, 12, 16, 28})
    if (regs_variant_fits(cfg, epl)) return epl;
  return 0;
}

bool fused_route_fits(const moe_config_t& cfg, int tokens) {
  const int epl = regs_variant_of(cfg);       // (28 values per lane leave the 1024-thread kernel no registers)
  return tokens >= 1 && tokens <= kFusedMaxTokens && tokens * cfg.topk <= kFusedMaxRows && epl != 0 && epl <= 16;
}

template <int EPL>
static void launch_fused_typed(const FusedArgs& a, int blocks, cudaStream_t stream) {
  if (a.r.tokens <= 16)
    launch_dependent(route_group_quant_kernel<EPL, 16>, dim3(blocks), dim3(16 * 32), 0, stream, a);
  else
    launch_dependent(route_group_quant_kernel<EPL, 32>, dim3(blocks), dim3(32 * 32), 0, stream, a);
}

cudaError_t launch_router_fused(const moe_config_t& cfg, const __nv_bfloat16* x, const float* router, const float* bias,
                                int tokens, float* logits, int32_t* ids32, float* weights, int64_t* ids64,
                                float* weights_out, const GroupArgs& g, uint8_t* xq, float* xs, cudaStream_t stream,
                                int* launches, const L2Warm* warm) {
  if (!fused_route_fits(cfg, tokens) || g.n_local != cfg.n_experts || g.id_base != 0 || g.n != tokens * cfg.topk)
    return cudaErrorInvalidValue;
  cudaError_t e = launch_router_logits(x, router, tokens, cfg.n_experts, cfg.hidden, logits, stream, warm);
  if (e != cudaSuccess) return e;
  FusedArgs a;
  a.r = RouteArgs{logits, bias, tokens, cfg.n_experts, cfg.topk, cfg.scoring, cfg.n_group, cfg.topk_group,
                  cfg.routed_scaling, ids32, weights, ids64, weights_out};
  a.g = g;
  a.x = x;
  a.hidden = cfg.hidden;
  a.xq = xq;
  a.xs = xs;
  const int blocks = 1 + g.n + g.shared_rows;
  switch (regs_variant_of(cfg)) {
    case 1: launch_fused_typed<1>(a, blocks, stream); break;
    case 2: launch_fused_typed<2>(a, blocks, stream); break;
    case 4: launch_fused_typed<4>(a, blocks, stream); break;
    case 8: launch_fused_typed<8>(a, blocks, stream); break;
    case 12: launch_fused_typed<12>(a, blocks, stream); break;
    default: launch_fused_typed<16>(a, blocks, stream); break;
  }
  if (launches) *launches += 2;
  return cudaGetLastError();
}

cudaError_t launch_router(const moe_config_t& cfg, const __nv_bfloat16* x, const float* router, const float* bias,
                          int tokens, float* logits, int32_t* ids32, float* weights, int64_t* ids64,
                          float* weights_out, cudaStream_t stream, int* launches, const L2Warm* warm) {
  cudaError_t e = launch_router_logits(x, router, tokens, cfg.n_experts, cfg.hidden, logits, stream, warm);
  if (e != cudaSuccess) return e;
  RouteArgs a{logits, bias, tokens, cfg.n_experts, cfg.topk, cfg.scoring, cfg.n_group, cfg.topk_group,
              cfg.routed_scaling, ids32, weights, ids64, weights_out};
  const int blocks = (tokens + kRouteWarps - 1) / kRouteWarps;
  const int threads = kRouteWarps * 32;
  void (*kernel)(RouteArgs) = route_select_kernel;
  if (regs_variant_fits(cfg, 1)) kernel = route_select_regs_kernel<1>;
  else if (regs_variant_fits(cfg, 2)) kernel = route_select_regs_kernel<2>;
  else if (regs_variant_fits(cfg, 4)) kernel = route_select_regs_kernel<4>;
  else if (regs_variant_fits(cfg, 8)) kernel = route_select_regs_kernel<8>;
  else if (regs_variant_fits(cfg, 12)) kernel = route_select_regs_kernel<12>;
  else if (regs_variant_fits(cfg, 16)) kernel = route_select_regs_kernel<16>;
  else if (regs_variant_fits(cfg, 28)) kernel = route_select_regs_kernel<28>;      // 896 experts
  launch_dependent(kernel, dim3(blocks), dim3(threads), 0, stream, a);
  if (launches) *launches += 2;
  return cudaGetLastError();
}

}  // namespace moe
