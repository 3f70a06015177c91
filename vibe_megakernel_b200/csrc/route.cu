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

constexpr int kLogitExperts = 2;   // experts per block
constexpr int kLogitTokens = 16;   // tokens per block

// logits[t][e] = sum_k router[e][k] * x[t][k], products and sums in fp64, one rounding to fp32.
// fp64 keeps the result within half an fp32 ulp of the exact value whatever the summation
// order, which is what makes expert ids reproducible against a host fp32 GEMV on inputs whose
// decision margins are audited.
__global__ void __launch_bounds__(256) router_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const float* __restrict__ router, int tokens,
                                                            int experts, int hidden, float* __restrict__ logits) {
  const int e0 = blockIdx.x * kLogitExperts;
  const int t0 = blockIdx.y * kLogitTokens;
  const int tcount = min(kLogitTokens, tokens - t0);
  double acc[kLogitExperts][kLogitTokens];
#pragma unroll
  for (int e = 0; e < kLogitExperts; ++e)
#pragma unroll
    for (int t = 0; t < kLogitTokens; ++t) acc[e][t] = 0.0;

  for (int k = threadIdx.x * 4; k < hidden; k += 256 * 4) {
    float4 r[kLogitExperts];
#pragma unroll
    for (int e = 0; e < kLogitExperts; ++e) {
      r[e] = (e0 + e < experts) ? *reinterpret_cast<const float4*>(router + static_cast<size_t>(e0 + e) * hidden + k)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int t = 0; t < kLogitTokens; ++t) {
      if (t < tcount) {
        const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(t0 + t) * hidden + k);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        const double x0 = __bfloat162float(lo.x), x1 = __bfloat162float(lo.y);
        const double x2 = __bfloat162float(hi.x), x3 = __bfloat162float(hi.y);
#pragma unroll
        for (int e = 0; e < kLogitExperts; ++e) {
          double a = acc[e][t];
          a = fma(static_cast<double>(r[e].x), x0, a);
          a = fma(static_cast<double>(r[e].y), x1, a);
          a = fma(static_cast<double>(r[e].z), x2, a);
          a = fma(static_cast<double>(r[e].w), x3, a);
          acc[e][t] = a;
        }
      }
    }
  }
  __shared__ double part[8][kLogitExperts * kLogitTokens];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int e = 0; e < kLogitExperts; ++e)
#pragma unroll
    for (int t = 0; t < kLogitTokens; ++t) {
      double v = acc[e][t];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == 0) part[warp][e * kLogitTokens + t] = v;
    }
  __syncthreads();
  if (threadIdx.x < kLogitExperts * kLogitTokens) {
    const int e = threadIdx.x / kLogitTokens, t = threadIdx.x % kLogitTokens;
    if (e0 + e < experts && t < tcount) {
      double v = 0.0;
#pragma unroll
      for (int w = 0; w < 8; ++w) v += part[w][threadIdx.x];
      logits[static_cast<size_t>(t0 + t) * experts + e0 + e] = static_cast<float>(v);
    }
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
      for (int j = 0; j < gsz; ++j) {
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
  dim3 grid((cfg.n_experts + kLogitExperts - 1) / kLogitExperts, (tokens + kLogitTokens - 1) / kLogitTokens);
  router_logits_kernel<<<grid, 256, 0, stream>>>(x, router, tokens, cfg.n_experts, cfg.hidden, logits);
  RouteArgs a{logits, bias, tokens, cfg.n_experts, cfg.topk, cfg.scoring, cfg.n_group, cfg.topk_group,
              cfg.routed_scaling, ids32, weights, ids64, weights_out};
  route_select_kernel<<<(tokens + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, 0, stream>>>(a);
  if (launches) *launches += 2;
  return cudaGetLastError();
}

}  // namespace moe
