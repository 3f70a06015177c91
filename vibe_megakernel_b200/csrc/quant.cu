// Per-row, per-128-channel dynamic e4m3 quantiser (one warp per group of 128 channels).
//
// Reference: pack_fp8_activation(value, power_of_two=False, block=128, scale_format="float"),
// megabench/tasks/quantization.py:87-109 with fp8_scale (:57-59): scale = max(amax, 1e-4) / 448,
// payload = RNE_e4m3(clamp(x / scale, +-448)) using a true fp32 division; a ragged last group is
// padded with zeros for the amax and the padding is not stored.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"
#include "quant_group.cuh"

namespace moe {

// GPW groups per warp: 1 for few rows (most warps, least latency), 4 for many (four loads in
// flight per lane instead of one: with one, a full batch moved at 1.9 TB/s, bound by round trips).
template <typename T, int GPW>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const T* __restrict__ x, int rows, int width,
                                                            const int32_t* __restrict__ gather,
                                                            uint8_t* __restrict__ q, float* __restrict__ scales) {
  dependent_wait();
  dependents_may_launch();
  const int groups = (width + kGroup - 1) / kGroup;
  const int runs = (groups + GPW - 1) / GPW;                              // runs of GPW groups per row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * 8 + warp;   // (row, run) pair
  if (item >= static_cast<long long>(rows) * runs) return;
  const int row = static_cast<int>(item / runs), g0 = static_cast<int>(item % runs) * GPW;
  const int src = gather ? gather[row] : row;
  const T* in = x + static_cast<size_t>(src) * width;
  uint8_t* out = q + static_cast<size_t>(row) * width;
  float v[GPW][4];
#pragma unroll
  for (int u = 0; u < GPW; ++u) load_group<T>(in, min(g0 + u, groups - 1), width, lane, v[u]);
#pragma unroll
  for (int u = 0; u < GPW; ++u) {
    if (g0 + u < groups) {
      const float scale = quantize_loaded(v[u], out, g0 + u, width, lane);
      if (lane == 0) scales[static_cast<size_t>(row) * groups + g0 + u] = scale;
    }
  }
}

// Large batches of bf16 rows (whole groups, 8-byte aligned): a fixed number of warps walks the (row,
// run of four groups) items with a stride, each lane reading its four channels of a group as one
// 8-byte load, and the loads of a warp's next item (row index first, when rows are gathered) are
// issued before the current one is quantised. One short-lived block per eight items, four 2-byte
// loads per lane and group, moved 2.4 TB/s at 9,216 rows of 7,168 channels.
constexpr int kStreamGroups = 4;

__global__ void __launch_bounds__(256) quantize_rows_stream_kernel(const __nv_bfloat16* __restrict__ x, int rows, int width,
                                                                   const int32_t* __restrict__ gather,
                                                                   uint8_t* __restrict__ q, float* __restrict__ scales) {
  dependent_wait();
  dependents_may_launch();
  const int groups = width / kGroup;
  const int runs = (groups + kStreamGroups - 1) / kStreamGroups;
  const long long items = static_cast<long long>(rows) * runs;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long stride = static_cast<long long>(gridDim.x) * 8;
  auto fetch = [&](long long item, uint2 (&raw)[kStreamGroups]) {
    const int row = static_cast<int>(item / runs), g0 = static_cast<int>(item % runs) * kStreamGroups;
    const int src = gather ? __ldg(gather + row) : row;
    const uint2* in = reinterpret_cast<const uint2*>(x + static_cast<size_t>(src) * width);
#pragma unroll
    for (int u = 0; u < kStreamGroups; ++u) raw[u] = __ldg(in + min(g0 + u, groups - 1) * 32 + lane);
  };
  long long item = static_cast<long long>(blockIdx.x) * 8 + warp;
  uint2 cur[kStreamGroups], nxt[kStreamGroups];
  if (item < items) fetch(item, cur);
  for (; item < items; item += stride) {
    if (item + stride < items) fetch(item + stride, nxt);
    const int row = static_cast<int>(item / runs), g0 = static_cast<int>(item % runs) * kStreamGroups;
    uint8_t* out = q + static_cast<size_t>(row) * width;
#pragma unroll
    for (int u = 0; u < kStreamGroups; ++u) {
      if (g0 + u < groups) {
        const float v[4] = {__uint_as_float(cur[u].x << 16), __uint_as_float(cur[u].x & 0xffff0000u),
                            __uint_as_float(cur[u].y << 16), __uint_as_float(cur[u].y & 0xffff0000u)};
        const float scale = quantize_loaded(v, out, g0 + u, width, lane);
        if (lane == 0) scales[static_cast<size_t>(row) * groups + g0 + u] = scale;
      }
    }
#pragma unroll
    for (int u = 0; u < kStreamGroups; ++u) cur[u] = nxt[u];
  }
}

// The token side of the same work, when every routed row is kept: each (token, run of four groups)
// is loaded and quantised once and its bytes and scales are stored to the token's topk grouped rows
// (and its shared-expert row). The gathering kernel above re-reads and re-quantises a token once per
// grouped row: nine times the loads and the arithmetic for the same 66 MB of stores at 1,024 tokens of
// 7,168 channels, top-8 and a shared expert.
constexpr int kScatterMaxTopk = 16;

__global__ void __launch_bounds__(256) quantize_scatter_kernel(const __nv_bfloat16* __restrict__ x, int tokens, int width,
                                                               int topk, const int32_t* __restrict__ slot_pos,
                                                               int shared_base, int rows, uint8_t* __restrict__ q,
                                                               float* __restrict__ scales) {
  dependent_wait();
  dependents_may_launch();
  const int groups = width / kGroup;
  const int runs = (groups + kStreamGroups - 1) / kStreamGroups;
  const long long items = static_cast<long long>(tokens) * runs;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long stride = static_cast<long long>(gridDim.x) * 8;
  const int dests = topk + (shared_base >= 0 ? 1 : 0);
  auto fetch = [&](long long item, uint2 (&raw)[kStreamGroups], int& dest) {
    const int token = static_cast<int>(item / runs), g0 = static_cast<int>(item % runs) * kStreamGroups;
    // lane k < topk holds the token's k-th grouped row, lane topk the shared expert's
    dest = lane < topk ? __ldg(slot_pos + static_cast<size_t>(token) * topk + lane) : shared_base + token;
    const uint2* in = reinterpret_cast<const uint2*>(x + static_cast<size_t>(token) * width);
#pragma unroll
    for (int u = 0; u < kStreamGroups; ++u) raw[u] = __ldg(in + min(g0 + u, groups - 1) * 32 + lane);
  };
  long long item = static_cast<long long>(blockIdx.x) * 8 + warp;
  uint2 cur[kStreamGroups], nxt[kStreamGroups];
  int dest = 0, dest_next = 0;
  if (item < items) fetch(item, cur, dest);
  for (; item < items; item += stride) {
    if (item + stride < items) fetch(item + stride, nxt, dest_next);
    const int g0 = static_cast<int>(item % runs) * kStreamGroups;
    uint32_t bytes[kStreamGroups];
    float scale[kStreamGroups];
#pragma unroll
    for (int u = 0; u < kStreamGroups; ++u) {
      const float v[4] = {__uint_as_float(cur[u].x << 16), __uint_as_float(cur[u].x & 0xffff0000u),
                          __uint_as_float(cur[u].y << 16), __uint_as_float(cur[u].y & 0xffff0000u)};
      scale[u] = quantize_values(v, bytes[u]);
    }
    for (int k = 0; k < dests; ++k) {
      const int to = __shfl_sync(0xffffffffu, dest, k);
      if (to < 0 || to >= rows) continue;      // (every routed row is kept by contract; a position outside the buffers is never written)
      const size_t row = static_cast<size_t>(to);
      uint32_t* out = reinterpret_cast<uint32_t*>(q + row * width);
#pragma unroll
      for (int u = 0; u < kStreamGroups; ++u)
        if (g0 + u < groups) out[(g0 + u) * 32 + lane] = bytes[u];
      if (lane < kStreamGroups && g0 + lane < groups) {
        float mine = scale[0];
#pragma unroll
        for (int u = 1; u < kStreamGroups; ++u) mine = lane == u ? scale[u] : mine;
        scales[row * groups + g0 + lane] = mine;
      }
    }
#pragma unroll
    for (int u = 0; u < kStreamGroups; ++u) cur[u] = nxt[u];
    dest = dest_next;
  }
}

bool quantize_scatter_fits(int tokens, int width, const void* x) {
  // (below this size the gathering kernels' many short blocks are as fast, and small batches take the fused routing kernel)
  return width % kGroup == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0 &&
         static_cast<long long>(tokens) * (width / kGroup) >= 8192;
}

cudaError_t launch_quantize_scatter(const __nv_bfloat16* x, int tokens, int width, int topk, const int32_t* slot_pos,
                                    int shared_base, uint8_t* q, float* scales, cudaStream_t stream, int* launches) {
  if (tokens <= 0) return cudaSuccess;
  if (topk < 1 || topk > kScatterMaxTopk || !quantize_scatter_fits(tokens, width, x)) return cudaErrorInvalidValue;
  const int groups = width / kGroup;
  const long long items = static_cast<long long>(tokens) * ((groups + kStreamGroups - 1) / kStreamGroups);
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const long long blocks = std::min((items + 7) / 8, static_cast<long long>(sms) * 8);
  const int rows = tokens * topk + (shared_base >= 0 ? tokens : 0);
  launch_dependent(quantize_scatter_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, x, tokens, width,
                   topk, slot_pos, shared_base, rows, q, scales);
  if (launches) *launches += 1;
  return cudaGetLastError();
}

template <typename T>
static void launch_quantize_typed(const T* x, int rows, int width, const int32_t* gather, uint8_t* q, float* scales,
                                  cudaStream_t stream) {
  const int groups = (width + kGroup - 1) / kGroup;
  if (static_cast<long long>(rows) * groups >= 32768) {
    const long long items = static_cast<long long>(rows) * ((groups + 3) / 4);
    launch_dependent(quantize_rows_kernel<T, 4>, dim3(static_cast<unsigned>((items + 7) / 8)), dim3(256), 0, stream, x,
                     rows, width, gather, q, scales);
  } else {
    const long long items = static_cast<long long>(rows) * groups;
    launch_dependent(quantize_rows_kernel<T, 1>, dim3(static_cast<unsigned>((items + 7) / 8)), dim3(256), 0, stream, x,
                     rows, width, gather, q, scales);
  }
}

cudaError_t launch_quantize(const void* x, int dtype, int rows, int width, const int32_t* gather, uint8_t* q,
                            float* scales, cudaStream_t stream, int* launches) {
  if (rows <= 0) return cudaSuccess;
  const int groups = (width + kGroup - 1) / kGroup;
  if (dtype == 0 && width % kGroup == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0 &&
      static_cast<long long>(rows) * groups >= 32768) {
    const long long items = static_cast<long long>(rows) * ((groups + kStreamGroups - 1) / kStreamGroups);
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long blocks = std::min((items + 7) / 8, static_cast<long long>(sms) * 8);
    launch_dependent(quantize_rows_stream_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream,
                     static_cast<const __nv_bfloat16*>(x), rows, width, gather, q, scales);
  } else if (dtype == 0)
    launch_quantize_typed(static_cast<const __nv_bfloat16*>(x), rows, width, gather, q, scales, stream);
  else
    launch_quantize_typed(static_cast<const float*>(x), rows, width, gather, q, scales, stream);
  if (launches) *launches += 1;
  return cudaGetLastError();
}

}  // namespace moe

// ---------------------------------------------------------------------------------------------
// Power-of-two (UE8M0) scales per `block` channels: the activation format of the MXFP4 MegaMoE layer.
//
// Reference: pack_fp8_activation(value, block=32, scale_format="e8m0"),
// megabench/tasks/quantization.py:62-84,87-109: the scale is a biased exponent taken from the fp32
// bits of the block maximum with integer arithmetic (the exponent rises by one when the mantissa
// exceeds that of 448 = 1.75 * 2^8, 448's exponent is removed, floor at the exponent of the 1e-4
// clamp), the payload is RNE_e4m3(x * 2^-(e-127)), an exact multiplication. A ragged last block is
// padded with zeros for the maximum and the padding is not stored.
// ---------------------------------------------------------------------------------------------
namespace moe {

template <typename T>
__global__ void __launch_bounds__(256) quantize_rows_ue8m0_kernel(const T* __restrict__ x, int rows, int width,
                                                                  int block, uint8_t* __restrict__ q,
                                                                  uint8_t* __restrict__ scales) {
  dependent_wait();
  dependents_may_launch();
  const int pieces = (width + 127) / 128;                 // a warp takes 128 channels: 4 per lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * 8 + warp;
  if (item >= static_cast<long long>(rows) * pieces) return;
  const int row = static_cast<int>(item / pieces), piece = static_cast<int>(item % pieces);
  const int k0 = piece * 128 + lane * 4;
  const T* in = x + static_cast<size_t>(row) * width;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = (k0 + j < width) ? load_as_float<T>(in + k0 + j) : 0.f;
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  const int lanes = block / 4;                            // lanes that share a scale: 8 (block 32) or 32 (block 128)
  for (int off = 1; off < lanes; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const int bits = __float_as_int(amax);
  const int exponent = max((bits + (0x7FFFFF - 0x600000)) >> 23, 105 + 8) - 8;       // biased, as uint8
  const float inverse = __int_as_float((254 - exponent) << 23);                        // exact 2^-(e-127)
  uint8_t* out = q + static_cast<size_t>(row) * width;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (k0 + j < width)
      out[k0 + j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(__fmul_rn(v[j], inverse), __NV_SATFINITE, __NV_E4M3));
  const int blocks_per_row = (width + block - 1) / block;
  const int b = k0 / block;
  if ((lane % lanes) == 0 && b < blocks_per_row)
    scales[static_cast<size_t>(row) * blocks_per_row + b] = static_cast<uint8_t>(exponent);
}

cudaError_t launch_quantize_ue8m0(const void* x, int dtype, int rows, int width, int block, uint8_t* q, uint8_t* scales,
                                  cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  const long long items = static_cast<long long>(rows) * ((width + 127) / 128);
  const unsigned blocks = static_cast<unsigned>((items + 7) / 8);
  if (dtype == 0)
    launch_dependent(quantize_rows_ue8m0_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                     static_cast<const __nv_bfloat16*>(x), rows, width, block, q, scales);
  else
    launch_dependent(quantize_rows_ue8m0_kernel<float>, dim3(blocks), dim3(256), 0, stream, static_cast<const float*>(x),
                     rows, width, block, q, scales);
  return cudaGetLastError();
}

}  // namespace moe
