// Router: fp32 logits with fp64 accumulation, then per-token expert selection by one warp.
//
// Selection rules reproduced (reference: megabench/tasks/frontier.py:229-242 for the sigmoid
// group-limited router; megabench/tasks/distributed.py:174-176 for the stable softmax top-k):
//   sigmoid: p = sigmoid(s), c = p + bias; group score = sum of the group's two largest c; keep the
//            topk_group best groups (ties to the lower group), others -> -inf; ids = first topk of a
//            stable descending sort of c; w = p[ids] / (sum + 1e-20) * scaling.
//   softmax: ids = first topk of a stable descending sort of s; w = softmax(s[ids]).
#include "common.cuh"
#include "kernels.h"

namespace moe {

constexpr int kLogitWarps = 8;
constexpr int kLogitTokens = 8;    // tokens per block

// logits[t][e] = sum_k router[e][k] * x[t][k], products and sums in fp64, one rounding to fp32.
// fp64 keeps the result within half an fp32 ulp of the exact value whatever the summation
// order, which is what makes expert ids reproducible against a host fp32 GEMV on inputs whose
// decision margins are audited.
//   SPLITK = false: warp w of block b owns expert b*8+w, its lanes sweep the whole row.
//   SPLITK = true : block b owns expert b, the 128-channel pieces of the row are dealt round-robin
//                   to the warps (small batches: more blocks in flight for the same bytes).
template <bool SPLITK>
__global__ void __launch_bounds__(kLogitWarps * 32) router_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                                         const float* __restrict__ router, int tokens,
                                                                         int experts, int hidden,
                                                                         float* __restrict__ logits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = SPLITK ? blockIdx.x : blockIdx.x * kLogitWarps + warp;
  const int t0 = blockIdx.y * kLogitTokens;
  const int tcount = min(kLogitTokens, tokens - t0);
  double acc[kLogitTokens];
#pragma unroll
  for (int t = 0; t < kLogitTokens; ++t) acc[t] = 0.0;
  if (e < experts) {
    const float* row = router + static_cast<size_t>(e) * hidden;
    const int pieces = hidden / 128;
    for (int c = SPLITK ? warp : 0; c < pieces; c += SPLITK ? kLogitWarps : 1) {
      const int k = c * 128 + lane * 4;
      const float4 r = *reinterpret_cast<const float4*>(row + k);
      const double r0 = r.x, r1 = r.y, r2 = r.z, r3 = r.w;
#pragma unroll
      for (int t = 0; t < kLogitTokens; ++t) {
        if (t < tcount) {
          const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(t0 + t) * hidden + k);
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          double a = acc[t];
          a = fma(r0, static_cast<double>(__bfloat162float(lo.x)), a);
          a = fma(r1, static_cast<double>(__bfloat162float(lo.y)), a);
          a = fma(r2, static_cast<double>(__bfloat162float(hi.x)), a);
          a = fma(r3, static_cast<double>(__bfloat162float(hi.y)), a);
          acc[t] = a;
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kLogitTokens; ++t) {
    if (t < tcount) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], off);
    }
  }
  if (SPLITK) {
    __shared__ double part[kLogitWarps][kLogitTokens];
    if (lane == 0) {
#pragma unroll
      for (int t = 0; t < kLogitTokens; ++t) part[warp][t] = acc[t];
    }
    __syncthreads();
    if (threadIdx.x < tcount && e < experts) {
      double v = 0.0;
#pragma unroll
      for (int w = 0; w < kLogitWarps; ++w) v += part[w][threadIdx.x];
      logits[static_cast<size_t>(t0 + threadIdx.x) * experts + e] = static_cast<float>(v);
    }
  } else if (lane == 0 && e < experts) {
#pragma unroll
    for (int t = 0; t < kLogitTokens; ++t)
      if (t < tcount) logits[static_cast<size_t>(t0 + t) * experts + e] = static_cast<float>(acc[t]);
  }
}

// Larger batches: a block keeps 8 token rows in shared memory and streams 16 router rows (two per
// warp) against them, so x is read from L2 once per block and the inner loop is bound by the
// fp64 units. Same arithmetic as above: every lane sums its channels in order, lanes are
// combined by a shuffle tree.
constexpr int kTiledExpertsPerWarp = 2;
constexpr int kTiledExperts = kLogitWarps * kTiledExpertsPerWarp;

__global__ void __launch_bounds__(kLogitWarps * 32) router_logits_tiled_kernel(const __nv_bfloat16* __restrict__ x,
                                                                               const float* __restrict__ router,
                                                                               int tokens, int experts, int hidden,
                                                                               float* __restrict__ logits) {
  extern __shared__ uint2 s_x[];                       // [8][hidden / 4], four bf16 per entry
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quads = hidden / 4;
  const int t0 = blockIdx.y * kLogitTokens;
  const int tcount = min(kLogitTokens, tokens - t0);
  for (int i = threadIdx.x; i < kLogitTokens * quads; i += blockDim.x) {
    const int t = i / quads, c = i - t * quads;
    s_x[i] = t < tcount ? *reinterpret_cast<const uint2*>(x + static_cast<size_t>(t0 + t) * hidden + 4 * c)
                        : make_uint2(0u, 0u);
  }
  __syncthreads();
  const int e0 = blockIdx.x * kTiledExperts + warp * kTiledExpertsPerWarp;
  double acc[kTiledExpertsPerWarp][kLogitTokens];
#pragma unroll
  for (int j = 0; j < kTiledExpertsPerWarp; ++j)
#pragma unroll
    for (int t = 0; t < kLogitTokens; ++t) acc[j][t] = 0.0;
  for (int q = lane; q < quads; q += 32) {
    float4 r[kTiledExpertsPerWarp];
#pragma unroll
    for (int j = 0; j < kTiledExpertsPerWarp; ++j)
      r[j] = e0 + j < experts ? *reinterpret_cast<const float4*>(router + static_cast<size_t>(e0 + j) * hidden + 4 * q)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < kLogitTokens; ++t) {
      const uint2 raw = s_x[t * quads + q];
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      const double x0 = __bfloat162float(lo.x), x1 = __bfloat162float(lo.y);
      const double x2 = __bfloat162float(hi.x), x3 = __bfloat162float(hi.y);
#pragma unroll
      for (int j = 0; j < kTiledExpertsPerWarp; ++j) {
        double a = acc[j][t];
        a = fma(static_cast<double>(r[j].x), x0, a);
        a = fma(static_cast<double>(r[j].y), x1, a);
        a = fma(static_cast<double>(r[j].z), x2, a);
        a = fma(static_cast<double>(r[j].w), x3, a);
        acc[j][t] = a;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kTiledExpertsPerWarp; ++j)
#pragma unroll
    for (int t = 0; t < kLogitTokens; ++t) {
      double v = acc[j][t];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == 0 && t < tcount && e0 + j < experts)
        logits[static_cast<size_t>(t0 + t) * experts + e0 + j] = static_cast<float>(v);
    }
}

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

__global__ void __launch_bounds__(kRouteWarps * 32) route_select_kernel(RouteArgs a) {
  __shared__ float s_choice[kRouteWarps][MOE_MAX_EXPERTS];
  __shared__ float s_prob[kRouteWarps][MOE_MAX_EXPERTS];
  __shared__ int s_pick[kRouteWarps][MOE_MAX_TOPK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= a.tokens) return;
  float* c = s_choice[warp];
  float* p = s_prob[warp];
  const int E = a.experts;
  const float ninf = __int_as_float(0xff800000);

  for (int e = lane; e < E; e += 32) {
    const float s = a.logits[static_cast<size_t>(t) * E + e];
    if (a.scoring == MOE_SCORING_SIGMOID) {
      const float pr = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-s)));
      p[e] = pr;
      c[e] = __fadd_rn(pr, a.bias ? a.bias[e] : 0.f);
    } else {
      p[e] = s;
      c[e] = s;
    }
  }
  __syncwarp();

  if (a.scoring == MOE_SCORING_SIGMOID && a.n_group > 1) {
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
    if (a.scoring == MOE_SCORING_SIGMOID) {
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

cudaError_t launch_router(const moe_config_t& cfg, const __nv_bfloat16* x, const float* router, const float* bias,
                          int tokens, float* logits, int32_t* ids32, float* weights, int64_t* ids64,
                          float* weights_out, cudaStream_t stream, int* launches) {
  const int token_tiles = (tokens + kLogitTokens - 1) / kLogitTokens;
  const size_t tile_smem = static_cast<size_t>(kLogitTokens) * cfg.hidden * sizeof(__nv_bfloat16);
  if (token_tiles == 1) {          // up to 8 tokens: one block per expert keeps every SM reading
    dim3 grid(cfg.n_experts, 1);
    router_logits_kernel<true><<<grid, kLogitWarps * 32, 0, stream>>>(x, router, tokens, cfg.n_experts, cfg.hidden, logits);
  } else if (tile_smem <= 200 * 1024) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(router_logits_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           200 * 1024);
      if (e != cudaSuccess) return e;
      configured = true;
    }
    dim3 grid((cfg.n_experts + kTiledExperts - 1) / kTiledExperts, token_tiles);
    router_logits_tiled_kernel<<<grid, kLogitWarps * 32, tile_smem, stream>>>(x, router, tokens, cfg.n_experts,
                                                                               cfg.hidden, logits);
  } else {
    dim3 grid((cfg.n_experts + kLogitWarps - 1) / kLogitWarps, token_tiles);
    router_logits_kernel<false><<<grid, kLogitWarps * 32, 0, stream>>>(x, router, tokens, cfg.n_experts, cfg.hidden, logits);
  }
  RouteArgs a{logits, bias, tokens, cfg.n_experts, cfg.topk, cfg.scoring, cfg.n_group, cfg.topk_group,
              cfg.routed_scaling, ids32, weights, ids64, weights_out};
  route_select_kernel<<<(tokens + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, 0, stream>>>(a);
  if (launches) *launches += 2;
  return cudaGetLastError();
}

}  // namespace moe
