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

constexpr size_t kLogitsSmemLimit = 200 * 1024;   // dynamic shared memory the logits kernels may ask for

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
// 256-expert router still spreads over 128 blocks. The router rows (weights: requested before the
// wait on the previous kernel) and the token rows arrive in shared memory by bulk async copies, one
// request per row: everything a block needs is in flight at once, which loads through registers
// did not achieve (the compiler kept a handful in flight and the kernel was bound by round trips).
constexpr int kRowsWarps = 2;

template <int TT>
__global__ void __launch_bounds__(kRowsWarps * 32) router_logits_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                                              const float* __restrict__ router,
                                                                              int tokens, int experts, int hidden,
                                                                              float* __restrict__ logits,
                                                                              const L2Warm warm, int logit_blocks) {
  extern __shared__ __align__(128) uint8_t s_rows_raw[];
  if (threadIdx.x == 0) MOE_STAMP_FIRST(warm.stamp, 2);
  if (static_cast<int>(blockIdx.x) >= logit_blocks) {   // weights do not change: no need to wait for anything
    if (blockIdx.y == 0) warm_l2(warm, blockIdx.x - logit_blocks, gridDim.x - logit_blocks);
    return;
  }
  __shared__ uint64_t bar;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.x * kRowsWarps + warp;
  const int e_first = blockIdx.x * kRowsWarps;
  const int t0 = blockIdx.y * TT;
  const int tcount = min(TT, tokens - t0);
  const int quads = hidden / 4;
  float4* s_router = reinterpret_cast<float4*>(s_rows_raw);                       // [kRowsWarps][quads]
  uint2* s_x = reinterpret_cast<uint2*>(s_router + kRowsWarps * quads);           // [TT][quads], four bf16 per entry
  const int rows_here = min(kRowsWarps, experts - e_first);
  const uint32_t router_bytes = static_cast<uint32_t>(hidden) * 4u, x_bytes = static_cast<uint32_t>(hidden) * 2u;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(&bar, router_bytes * rows_here + x_bytes * tcount);
    for (int w = 0; w < rows_here; ++w)
      bulk_copy_g2s(s_router + static_cast<size_t>(w) * quads, router + static_cast<size_t>(e_first + w) * hidden,
                    router_bytes, &bar);
  }
  dependent_wait();
  dependents_may_launch();
  if (threadIdx.x == 0) {
    for (int t = 0; t < tcount; ++t)
      bulk_copy_g2s(s_x + static_cast<size_t>(t) * quads, x + static_cast<size_t>(t0 + t) * hidden, x_bytes, &bar);
  }
  __syncthreads();              // the barrier is initialised before anyone polls it
  mbar_wait(&bar, 0);           // bounded; a copy that never lands leaves wrong logits, not a hang
  if (e >= experts) return;
  float acc[TT];
#pragma unroll
  for (int t = 0; t < TT; ++t) acc[t] = 0.f;
  const float4* row = s_router + static_cast<size_t>(warp) * quads;
  for (int q = lane; q < quads; q += 32) {
    const float4 r = row[q];
#pragma unroll
    for (int t = 0; t < TT; ++t)
      if (t < tcount) acc[t] = fma4(r, s_x[static_cast<size_t>(t) * quads + q], acc[t]);
  }
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    if (t < tcount) {
      const float v = warp_total(acc[t]);
      if (lane == 0) logits[static_cast<size_t>(t0 + t) * experts + e] = v;
    }
  }
}

// Four bf16 values of a token row as fp32 (a bf16 is the upper half of an fp32).
__device__ __forceinline__ void unpack4(const uint2& raw, float (&v)[4]) {
  v[0] = __uint_as_float(raw.x << 16);
  v[1] = __uint_as_float(raw.x & 0xffff0000u);
  v[2] = __uint_as_float(raw.y << 16);
  v[3] = __uint_as_float(raw.y & 0xffff0000u);
}

// Larger batches: a block keeps TOK token rows in shared memory and streams the router rows of
// 8 * kTiledExpertsPerWarp experts against them, so x is read from L2 once per block. Four experts
// per warp halve the instructions per FMA (the token values are unpacked once for all of them);
// two give twice the blocks, which wins while the grid would not fill the SMs.
constexpr int kTiledWarps = 8;

template <int TOK, int kTiledExpertsPerWarp>
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
  const int t0 = blockIdx.y * TOK;
  const int tcount = min(TOK, tokens - t0);
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
  for (int i = tcount * quads + threadIdx.x; i < TOK * quads; i += blockDim.x) s_x[i] = make_uint2(0u, 0u);
  mbar_wait(&bar, 0);           // bounded; a copy that never lands leaves wrong logits, not a hang
  __syncthreads();
  const int e0 = (blockIdx.x * kTiledWarps + warp) * kTiledExpertsPerWarp;
  float acc[kTiledExpertsPerWarp][TOK];
#pragma unroll
  for (int j = 0; j < kTiledExpertsPerWarp; ++j)
#pragma unroll
    for (int t = 0; t < TOK; ++t) acc[j][t] = 0.f;
  // Several pieces per trip: all router loads of a trip (8 x 16 bytes per lane) are issued before the
  // first use. The token values are converted once per piece and shared by the warp's four
  // experts; two tokens go through every packed FMA (each half is the scalar chain of fma4).
  // (with one or two experts per warp more pieces per trip keep as many bytes in flight as four experts do)
  constexpr int kAhead = kTiledExpertsPerWarp >= 4 ? 2 : 8 / kTiledExpertsPerWarp;
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
        for (int t = 0; t < TOK; t += 2) {
          float xa[4], xb[4];
          unpack4(s_x[t * quads + q], xa);
          unpack4(s_x[(t + 1) * quads + q], xb);
#pragma unroll
          for (int j = 0; j < kTiledExpertsPerWarp; ++j) {
            const float4 w = r[u][j];
            fma2(w.x, w.x, xa[0], xb[0], acc[j][t], acc[j][t + 1]);
            fma2(w.y, w.y, xa[1], xb[1], acc[j][t], acc[j][t + 1]);
            fma2(w.z, w.z, xa[2], xb[2], acc[j][t], acc[j][t + 1]);
            fma2(w.w, w.w, xa[3], xb[3], acc[j][t], acc[j][t + 1]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kTiledExpertsPerWarp; ++j)
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      if (t < tcount) {
        const float v = warp_total(acc[j][t]);
        if (lane == 0 && e0 + j < experts) logits[static_cast<size_t>(t0 + t) * experts + e0 + j] = v;
      }
    }
}

cudaError_t launch_router_logits(const __nv_bfloat16* x, const float* router, int tokens, int experts, int hidden,
                                 float* logits, cudaStream_t stream, const L2Warm* warm_request) {
  auto tile_smem = [&](int tok) { return static_cast<size_t>(tok) * hidden * sizeof(__nv_bfloat16); };
  const int row_blocks = (experts + kRowsWarps - 1) / kRowsWarps;
  const bool tiled_ok = tile_smem(8) <= kLogitsSmemLimit && hidden % 8 == 0;
  const dim3 rows_block(kRowsWarps * 32);
  L2Warm warm = {};
  int extra = 0;
  if (warm_request) warm.stamp = warm_request->stamp;
  if (warm_request) {
    for (int r = 0; r < 3; ++r) {
      if (warm_request->ptr[r] && !(reinterpret_cast<uintptr_t>(warm_request->ptr[r]) & 15)) {
        warm.ptr[r] = warm_request->ptr[r];
        warm.bytes[r] = warm_request->bytes[r];
        extra = kWarmBlocks;
      }
    }
  }
  // bulk copies need 16-byte aligned rows (hidden is a multiple of 128, so only the bases matter)
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(router)) & 15) return cudaErrorMisalignedAddress;
  const size_t router_smem = static_cast<size_t>(kRowsWarps) * hidden * sizeof(float);
  auto rows_smem = [&](int tt) { return router_smem + static_cast<size_t>(tt) * hidden * sizeof(__nv_bfloat16); };
  auto launch_rows = [&](auto kernel, int tt) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    return launch_dependent(kernel, dim3(row_blocks + extra, (tokens + tt - 1) / tt), rows_block, rows_smem(tt), stream, x,
                            router, tokens, experts, hidden, logits, warm, row_blocks);
  };
  const size_t smem_limit = 200 * 1024;
  if (rows_smem(1) > smem_limit) return cudaErrorInvalidValue;
  if (tokens == 1 || rows_smem(4) > smem_limit) {
    cudaError_t e = launch_rows(router_logits_rows_kernel<1>, 1);
    if (e != cudaSuccess) return e;
  } else if (tokens <= 4 || rows_smem(8) > smem_limit) {
    cudaError_t e = launch_rows(router_logits_rows_kernel<4>, 4);
    if (e != cudaSuccess) return e;
  } else if ((tokens <= 8 && row_blocks <= 2 * 148) || !tiled_ok) {
    // (with many hundreds of experts the rows kernel's blocks, each holding the 8 token rows and two
    // router rows, run in several waves: the tiled kernel below streams the router rows instead)
    cudaError_t e = launch_rows(router_logits_rows_kernel<8>, 8);
    if (e != cudaSuccess) return e;
  } else {
    auto launch_tiled = [&](auto kernel, int tok, int experts_per_block) -> cudaError_t {
      const int tiled_blocks = (experts + experts_per_block - 1) / experts_per_block;
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(kLogitsSmemLimit));
      if (e != cudaSuccess) return e;
      return launch_dependent(kernel, dim3(tiled_blocks + extra, (tokens + tok - 1) / tok), dim3(kTiledWarps * 32),
                              tile_smem(tok), stream, x, router, tokens, experts, hidden, logits, warm, tiled_blocks);
    };
    // 8 token rows per block: 12 (the most that fit at H = 7168) measured 15-25 % slower, the extra
    // accumulators costing more than the saved passes over the router rows
    const long long wide_grid = static_cast<long long>((experts + 31) / 32) * ((tokens + 7) / 8);
    // experts per warp: as many as still leave about a hundred blocks
    const long long mid_grid = static_cast<long long>((experts + 15) / 16) * ((tokens + 7) / 8);
    cudaError_t e = wide_grid >= 148 ? launch_tiled(router_logits_tiled_kernel<8, 4>, 8, 32)
                  : mid_grid >= 100  ? launch_tiled(router_logits_tiled_kernel<8, 2>, 8, 16)
                                     : launch_tiled(router_logits_tiled_kernel<8, 1>, 8, 8);
    if (e != cudaSuccess) return e;
  }
  return cudaGetLastError();
}

}  // namespace moe
