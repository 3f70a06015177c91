// Router logits: logits[t][e] = sum_k router[e][k] * x[t][k]  (fp32 router, bf16 tokens).
// Reference: `router.float() @ x.float()` per token, megabench/tasks/frontier.py:343.
//
// Arithmetic, the same in both kernels so that a token's logits do not depend on the batch it
// came in: one warp owns one (expert, token) sum; lane l adds channels 4q..4q+3 for
// q = l, l+32, l+64, ... in that order with fp32 FMAs; the 32 lane partials are combined by a
// butterfly of error-free two-float (hi + lo) sums and rounded once. Only the short per-lane
// chains round: an absolute error of about 1e-7 on a logit at the magnitudes of this layer, two
// orders below the decision margin the input audit enforces. (fp64 accumulation would be simpler
// but runs at a few FMAs per clock per SM on this GPU and made the router the slowest small stage.)
#include "common.cuh"
#include "kernels.h"

namespace moe {

constexpr int kLogitTokens = 8;    // tokens per block of the tiled kernel

struct Sum2 {
  float hi, lo;
};
__device__ __forceinline__ float fma4(const float4& r, const uint2& raw, float acc) {
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  acc = fmaf(r.x, __bfloat162float(lo.x), acc);
  acc = fmaf(r.y, __bfloat162float(lo.y), acc);
  acc = fmaf(r.z, __bfloat162float(hi.x), acc);
  acc = fmaf(r.w, __bfloat162float(hi.y), acc);
  return acc;
}
// a + b in two-float arithmetic; symmetric in its arguments, so a butterfly leaves the same bits
// in every lane.
__device__ __forceinline__ Sum2 sum2_merge(const Sum2& a, const Sum2& b) {
  const float t = __fadd_rn(a.hi, b.hi);
  const float bb = __fsub_rn(t, a.hi);
  const float err = __fadd_rn(__fsub_rn(a.hi, __fsub_rn(t, bb)), __fsub_rn(b.hi, bb));
  return Sum2{t, __fadd_rn(__fadd_rn(a.lo, b.lo), err)};
}
__device__ __forceinline__ float warp_total(float lane_sum) {
  Sum2 s{lane_sum, 0.f};
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    Sum2 o;
    o.hi = __shfl_xor_sync(0xffffffffu, s.hi, off);
    o.lo = __shfl_xor_sync(0xffffffffu, s.lo, off);
    s = sum2_merge(s, o);
  }
  return __fadd_rn(s.hi, s.lo);
}

// Blocks past the logits grid (index `block` of `blocks`) ask the L2 to fetch the given ranges,
// 4 KB per request, and return without waiting for the data.
constexpr int kWarmBlocks = 32;
constexpr uint32_t kWarmPiece = 4096;
__device__ __forceinline__ void warm_l2(const L2Warm& w, int block, int blocks) {
  const uint64_t first = static_cast<uint64_t>(block) * blockDim.x + threadIdx.x;
  const uint64_t stride = static_cast<uint64_t>(blocks) * blockDim.x;
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    const uint64_t pieces = w.bytes[r] / kWarmPiece;     // a ragged tail is left to the GEMM's own loads
    for (uint64_t i = first; i < pieces; i += stride)
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(w.ptr[r] + i * kWarmPiece), "r"(kWarmPiece) : "memory");
  }
}

// Small batches (TT tokens at most): two warps per block, one expert row per warp, so that a
// 256-expert router still spreads over 128 blocks; each trip issues the loads of kRowsAhead pieces
// of 128 channels before the first use (14 KB of the router row per warp for a single token: with
// two warps per SM the kernel is bound by memory round trips, so fewer and larger trips win).
constexpr int kRowsWarps = 2;
template <int TT>
struct RowsAhead {
  static constexpr int value = TT == 1 ? 28 : TT <= 4 ? 14 : 8;
};

template <int TT>
__global__ void __launch_bounds__(kRowsWarps * 32) router_logits_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                                              const float* __restrict__ router,
                                                                              int tokens, int experts, int hidden,
                                                                              float* __restrict__ logits,
                                                                              const L2Warm warm, int logit_blocks) {
  if (static_cast<int>(blockIdx.x) >= logit_blocks) {   // weights do not change: no need to wait for anything
    if (blockIdx.y == 0) warm_l2(warm, blockIdx.x - logit_blocks, gridDim.x - logit_blocks);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.x * kRowsWarps + warp;
  const int t0 = blockIdx.y * TT;
  const int tcount = min(TT, tokens - t0);
  dependent_wait();
  dependents_may_launch();
  if (e >= experts) return;
  float acc[TT];
#pragma unroll
  for (int t = 0; t < TT; ++t) acc[t] = 0.f;
  const float* row = router + static_cast<size_t>(e) * hidden;
  const int quads = hidden / 4;
  constexpr int kRowsAhead = RowsAhead<TT>::value;
  for (int q0 = lane; q0 < quads; q0 += 32 * kRowsAhead) {
    float4 r[kRowsAhead];
    uint2 xv[kRowsAhead][TT];
#pragma unroll
    for (int u = 0; u < kRowsAhead; ++u) {
      // unconditional loads from clamped addresses: the compiler can then issue all of a trip's
      // loads back to back (values loaded past the row or the batch are never used)
      const int q = min(q0 + 32 * u, quads - 1);
      r[u] = __ldg(reinterpret_cast<const float4*>(row + 4 * q));
#pragma unroll
      for (int t = 0; t < TT; ++t)
        xv[u][t] = __ldg(reinterpret_cast<const uint2*>(x + static_cast<size_t>(t0 + min(t, tcount - 1)) * hidden + 4 * q));
    }
#pragma unroll
    for (int u = 0; u < kRowsAhead; ++u) {
      if (q0 + 32 * u < quads) {
#pragma unroll
        for (int t = 0; t < TT; ++t) acc[t] = fma4(r[u], xv[u][t], acc[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    if (t < tcount) {
      const float v = warp_total(acc[t]);
      if (lane == 0) logits[static_cast<size_t>(t0 + t) * experts + e] = v;
    }
  }
}

// Larger batches: a block keeps 8 token rows in shared memory and streams 16 router rows (two per
// warp) against them, so x is read from L2 once per block.
constexpr int kTiledWarps = 8;
constexpr int kTiledExpertsPerWarp = 2;
constexpr int kTiledExperts = kTiledWarps * kTiledExpertsPerWarp;

__global__ void __launch_bounds__(kTiledWarps * 32) router_logits_tiled_kernel(const __nv_bfloat16* __restrict__ x,
                                                                               const float* __restrict__ router,
                                                                               int tokens, int experts, int hidden,
                                                                               float* __restrict__ logits,
                                                                               const L2Warm warm, int logit_blocks) {
  extern __shared__ __align__(128) uint2 s_x[];        // [8][hidden / 4], four bf16 per entry
  if (static_cast<int>(blockIdx.x) >= logit_blocks) {
    if (blockIdx.y == 0) warm_l2(warm, blockIdx.x - logit_blocks, gridDim.x - logit_blocks);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quads = hidden / 4;
  const int t0 = blockIdx.y * kLogitTokens;
  const int tcount = min(kLogitTokens, tokens - t0);
  // Token rows arrive by bulk async copies (one per row, 16-byte aligned by the launcher's check);
  // rows past the batch are zero-filled by the threads.
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  dependent_wait();
  dependents_may_launch();
  if (threadIdx.x == 0) {
    const uint32_t row_bytes = static_cast<uint32_t>(hidden) * 2u;
    mbar_expect_tx(&bar, row_bytes * tcount);
    for (int t = 0; t < tcount; ++t)
      bulk_copy_g2s(s_x + static_cast<size_t>(t) * quads, x + static_cast<size_t>(t0 + t) * hidden, row_bytes, &bar);
  }
  for (int i = tcount * quads + threadIdx.x; i < kLogitTokens * quads; i += blockDim.x) s_x[i] = make_uint2(0u, 0u);
  mbar_wait(&bar, 0);           // bounded; a copy that never lands leaves wrong logits, not a hang
  __syncthreads();
  const int e0 = blockIdx.x * kTiledExperts + warp * kTiledExpertsPerWarp;
  float acc[kTiledExpertsPerWarp][kLogitTokens];
#pragma unroll
  for (int j = 0; j < kTiledExpertsPerWarp; ++j)
#pragma unroll
    for (int t = 0; t < kLogitTokens; ++t) acc[j][t] = 0.f;
  // Four pieces per trip: all router loads of a trip are issued before the first use, so a warp
  // keeps 4 KB in flight instead of waiting out one L2 round trip per piece.
  constexpr int kAhead = 4;
  for (int q0 = lane; q0 < quads; q0 += 32 * kAhead) {
    float4 r[kAhead][kTiledExpertsPerWarp];
#pragma unroll
    for (int u = 0; u < kAhead; ++u)
#pragma unroll
      for (int j = 0; j < kTiledExpertsPerWarp; ++j) {
        const int q = min(q0 + 32 * u, quads - 1);       // clamped, unconditional (see the rows kernel)
        const int e = min(e0 + j, experts - 1);
        r[u][j] = __ldg(reinterpret_cast<const float4*>(router + static_cast<size_t>(e) * hidden + 4 * q));
      }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int q = q0 + 32 * u;
      if (q < quads) {
#pragma unroll
        for (int t = 0; t < kLogitTokens; ++t) {
          const uint2 raw = s_x[t * quads + q];
#pragma unroll
          for (int j = 0; j < kTiledExpertsPerWarp; ++j) acc[j][t] = fma4(r[u][j], raw, acc[j][t]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kTiledExpertsPerWarp; ++j)
#pragma unroll
    for (int t = 0; t < kLogitTokens; ++t) {
      if (t < tcount) {
        const float v = warp_total(acc[j][t]);
        if (lane == 0 && e0 + j < experts) logits[static_cast<size_t>(t0 + t) * experts + e0 + j] = v;
      }
    }
}

cudaError_t launch_router_logits(const __nv_bfloat16* x, const float* router, int tokens, int experts, int hidden,
                                 float* logits, cudaStream_t stream, const L2Warm* warm_request) {
  const size_t tile_smem = static_cast<size_t>(kLogitTokens) * hidden * sizeof(__nv_bfloat16);
  const int row_blocks = (experts + kRowsWarps - 1) / kRowsWarps;
  const bool tiled_ok = tile_smem <= 200 * 1024 && !(reinterpret_cast<uintptr_t>(x) & 15) && hidden % 8 == 0;
  const dim3 rows_block(kRowsWarps * 32);
  L2Warm warm = {};
  int extra = 0;
  if (warm_request) {
    for (int r = 0; r < 3; ++r) {
      if (warm_request->ptr[r] && !(reinterpret_cast<uintptr_t>(warm_request->ptr[r]) & 15)) {
        warm.ptr[r] = warm_request->ptr[r];
        warm.bytes[r] = warm_request->bytes[r];
        extra = kWarmBlocks;
      }
    }
  }
  if (tokens == 1) {
    launch_dependent(router_logits_rows_kernel<1>, dim3(row_blocks + extra, 1), rows_block, 0, stream, x, router, tokens,
                     experts, hidden, logits, warm, row_blocks);
  } else if (tokens <= 4) {
    launch_dependent(router_logits_rows_kernel<4>, dim3(row_blocks + extra, 1), rows_block, 0, stream, x, router, tokens,
                     experts, hidden, logits, warm, row_blocks);
  } else if (tokens <= 8 || !tiled_ok) {
    launch_dependent(router_logits_rows_kernel<8>, dim3(row_blocks + extra, (tokens + 7) / 8), rows_block, 0, stream, x,
                     router, tokens, experts, hidden, logits, warm, row_blocks);
  } else {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(router_logits_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           200 * 1024);
      if (e != cudaSuccess) return e;
      configured = true;
    }
    const int tiled_blocks = (experts + kTiledExperts - 1) / kTiledExperts;
    dim3 grid(tiled_blocks + extra, (tokens + kLogitTokens - 1) / kLogitTokens);
    launch_dependent(router_logits_tiled_kernel, grid, dim3(kTiledWarps * 32), tile_smem, stream, x, router, tokens,
                     experts, hidden, logits, warm, tiled_blocks);
  }
  return cudaGetLastError();
}

}  // namespace moe
