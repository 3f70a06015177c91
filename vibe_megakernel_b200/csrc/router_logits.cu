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

// The totals of N per-lane sums (N a power of two, at most 32), by the same tree as warp_total
// (partners 16, 8, 4, 2, 1 lanes apart, the symmetric two-float merge at every node, so the bits
// are those of warp_total), but as a reduce-scatter: at every level a lane keeps half of its values
// and hands the other half to its partner: about 2 N shuffles instead of 10 N. Lane l returns the
// total of value l * N / 32.
template <int N>
__device__ __forceinline__ float warp_totals(const float (&v)[N], int lane) {
  static_assert(N >= 1 && N <= 32 && (N & (N - 1)) == 0, "a power of two up to the warp size");
  float hi[N], lo[N];
#pragma unroll
  for (int i = 0; i < N; ++i) hi[i] = v[i], lo[i] = 0.f;
  int off = 16;
#pragma unroll
  for (int count = N; count > 1; count >>= 1) {
    const int half = count >> 1;
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const Sum2 mine{upper ? hi[i + half] : hi[i], upper ? lo[i + half] : lo[i]};
      const float send_hi = upper ? hi[i] : hi[i + half], send_lo = upper ? lo[i] : lo[i + half];
      Sum2 other;
      other.hi = __shfl_xor_sync(0xffffffffu, send_hi, off);
      other.lo = count == N ? 0.f : __shfl_xor_sync(0xffffffffu, send_lo, off);   // the lane sums have no low part yet
      const Sum2 m = sum2_merge(mine, other);
      hi[i] = m.hi, lo[i] = m.lo;
    }
    off >>= 1;
  }
  Sum2 s{hi[0], lo[0]};
#pragma unroll
  for (int o = 16 / N; o > 0; o >>= 1) {      // the levels left when N < 32: every partner holds the same value index
    Sum2 other;
    other.hi = __shfl_xor_sync(0xffffffffu, s.hi, o);
    other.lo = __shfl_xor_sync(0xffffffffu, s.lo, o);
    s = sum2_merge(s, other);
  }
  return __fadd_rn(s.hi, s.lo);
}

// Larger batches: a block takes TOK token rows against the router rows of 8 * EPW experts. The token
// rows pass through shared memory in pieces of 1,024 channels, two pieces in flight (a piece is
// requested as soon as all warps have left its buffer), so a block holds 32 KB instead of whole rows
// and several blocks share an SM; the router rows stream through registers, the loads of a trip
// issued one trip ahead of their use (with them issued at the top of the trip that uses them, the
// two warps a scheduler had spent most of their time waiting for the L2). Four experts per warp halve
// the instructions per FMA (the token values are unpacked once for all of them); fewer give more
// blocks, which wins while the grid would not fill the SMs. The order of a lane's additions is that
// of the rows kernel whatever the piece size.
constexpr int kTiledWarps = 8;
constexpr int kPieceQuads = 256;                      // four channels per quad

template <int TOK, int EPW>
__global__ void __launch_bounds__(kTiledWarps * 32) router_logits_tiled_kernel(const __nv_bfloat16* __restrict__ x,
                                                                               const float* __restrict__ router,
                                                                               int tokens, int experts, int hidden,
                                                                               float* __restrict__ logits,
                                                                               const L2Warm warm, int logit_blocks) {
  extern __shared__ __align__(128) uint2 s_x[];        // [2][TOK][kPieceQuads], four bf16 per entry
  if (static_cast<int>(blockIdx.x) >= logit_blocks) {
    if (blockIdx.y == 0) warm_l2(warm, blockIdx.x - logit_blocks, gridDim.x - logit_blocks);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quads = hidden / 4;
  const int pieces = (quads + kPieceQuads - 1) / kPieceQuads;
  const int t0 = blockIdx.y * TOK;
  const int tcount = min(TOK, tokens - t0);
  // Bulk async copies, one per row and piece (16-byte aligned: the launcher checks the base, and
  // hidden is a multiple of 8); rows past the batch are zero-filled by the threads, once.
  __shared__ uint64_t bar[2];
  auto request = [&](int piece) {
    const int first = piece * kPieceQuads;
    const uint32_t bytes = static_cast<uint32_t>(min(kPieceQuads, quads - first)) * 8u;
    uint64_t* b = &bar[piece & 1];
    mbar_expect_tx(b, bytes * tcount);
    for (int t = 0; t < tcount; ++t)
      bulk_copy_g2s(s_x + static_cast<size_t>((piece & 1) * TOK + t) * kPieceQuads,
                    x + static_cast<size_t>(t0 + t) * hidden + 4 * first, bytes, b);
  };
  if (threadIdx.x == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int e0 = (blockIdx.x * kTiledWarps + warp) * EPW;
  // Several quads per trip: all router loads of a trip (8 x 16 bytes per lane) are in flight together.
  // The token values are converted once per quad and shared by the warp's experts; two tokens
  // go through every packed FMA (each half is the scalar chain of fma4).
  constexpr int kAhead = EPW >= 4 ? 2 : 4 / EPW;      // (two register sets are in flight)
  static_assert(kPieceQuads % (64 * kAhead) == 0, "a round of two trips never straddles two pieces");
  const float4* row[EPW];                                // this warp's router rows (clamped: see the rows kernel)
#pragma unroll
  for (int j = 0; j < EPW; ++j)
    row[j] = reinterpret_cast<const float4*>(router + static_cast<size_t>(min(e0 + j, experts - 1)) * hidden);
  auto fetch = [&](int q0, float4 (&r)[kAhead][EPW]) {
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int q = min(q0 + 32 * u, quads - 1);         // clamped, unconditional
#pragma unroll
      for (int j = 0; j < EPW; ++j) r[u][j] = __ldg(row[j] + q);
    }
  };
  float4 r[kAhead][EPW], r_odd[kAhead][EPW];
  fetch(lane, r);                                        // weights: nothing to wait for
  dependent_wait();
  dependents_may_launch();
  if (threadIdx.x == 0) {
    request(0);
    if (pieces > 1) request(1);
  }
  for (int i = threadIdx.x; i < 2 * (TOK - tcount) * kPieceQuads; i += blockDim.x) {
    const int row = tcount + (i / kPieceQuads) % (TOK - tcount), buf = i / ((TOK - tcount) * kPieceQuads);
    s_x[static_cast<size_t>(buf * TOK + row) * kPieceQuads + i % kPieceQuads] = make_uint2(0u, 0u);
  }
  __syncthreads();
  float acc[EPW * TOK];
#pragma unroll
  for (int i = 0; i < EPW * TOK; ++i) acc[i] = 0.f;
  for (int piece = 0; piece < pieces; ++piece) {
    mbar_wait(&bar[piece & 1], (piece >> 1) & 1);   // bounded; a copy that never lands leaves wrong logits, not a hang
    const uint2* xs = s_x + static_cast<size_t>(piece & 1) * TOK * kPieceQuads;
    const int first = piece * kPieceQuads, end = min(first + kPieceQuads, quads);
    auto trip = [&](int q0, const float4 (&w4)[kAhead][EPW]) {
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int q = q0 + 32 * u;
        if (q < end) {
#pragma unroll
          for (int t = 0; t < TOK; t += 2) {
            float xa[4], xb[4];
            unpack4(xs[t * kPieceQuads + q - first], xa);
            unpack4(xs[(t + 1) * kPieceQuads + q - first], xb);
#pragma unroll
            for (int j = 0; j < EPW; ++j) {
              const float4 w = w4[u][j];
              fma2(w.x, w.x, xa[0], xb[0], acc[j * TOK + t], acc[j * TOK + t + 1]);
              fma2(w.y, w.y, xa[1], xb[1], acc[j * TOK + t], acc[j * TOK + t + 1]);
              fma2(w.z, w.z, xa[2], xb[2], acc[j * TOK + t], acc[j * TOK + t + 1]);
              fma2(w.w, w.w, xa[3], xb[3], acc[j * TOK + t], acc[j * TOK + t + 1]);
            }
          }
        }
      }
    };
    // two trips per round, the two register sets taking turns (no copies from the set that was fetched
    // ahead into the set that is used)
    for (int q0 = first + lane; q0 < end; q0 += 64 * kAhead) {
      fetch(q0 + 32 * kAhead, r_odd);
      trip(q0, r);
      fetch(q0 + 64 * kAhead, r);
      trip(q0 + 32 * kAhead, r_odd);
    }
    __syncthreads();                                  // every warp has left this piece's buffer
    if (threadIdx.x == 0 && piece + 2 < pieces) request(piece + 2);
  }
  const float total = warp_totals<EPW * TOK>(acc, lane);
  constexpr int kLanesPerValue = 32 / (EPW * TOK);
  const int value = lane / kLanesPerValue, j = value / TOK, t = value % TOK;
  if (lane % kLanesPerValue == 0 && t < tcount && e0 + j < experts)
    logits[static_cast<size_t>(t0 + t) * experts + e0 + j] = total;
}

cudaError_t launch_router_logits(const __nv_bfloat16* x, const float* router, int tokens, int experts, int hidden,
                                 float* logits, cudaStream_t stream, const L2Warm* warm_request) {
  auto tile_smem = [&](int tok) { return static_cast<size_t>(2) * tok * kPieceQuads * sizeof(uint2); };
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
    // (and never more experts per block than there are: Mixtral's 8 take one per warp)
    cudaError_t e = wide_grid >= 148 && experts > 16 ? launch_tiled(router_logits_tiled_kernel<8, 4>, 8, 32)
                  : mid_grid >= 100 && experts > 8   ? launch_tiled(router_logits_tiled_kernel<8, 2>, 8, 16)
                                                     : launch_tiled(router_logits_tiled_kernel<8, 1>, 8, 8);
    if (e != cudaSuccess) return e;
  }
  return cudaGetLastError();
}

}  // namespace moe
