// Per-row, per-128-channel dynamic e4m3 quantiser (one warp per group of 128 channels).
//
// Reference: pack_fp8_activation(value, power_of_two=False, block=128, scale_format="float"),
// megabench/tasks/quantization.py:87-109 with fp8_scale (:57-59): scale = max(amax, 1e-4) / 448,
// payload = RNE_e4m3(clamp(x / scale, +-448)) using a true fp32 division; a ragged last group is
// padded with zeros for the amax and the padding is not stored.
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
  if (dtype == 0)
    launch_quantize_typed(static_cast<const __nv_bfloat16*>(x), rows, width, gather, q, scales, stream);
  else
    launch_quantize_typed(static_cast<const float*>(x), rows, width, gather, q, scales, stream);
  if (launches) *launches += 1;
  return cudaGetLastError();
}

}  // namespace moe
