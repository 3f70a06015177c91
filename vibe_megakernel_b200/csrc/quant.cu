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

template <typename T>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const T* __restrict__ x, int rows, int width,
                                                            const int32_t* __restrict__ gather,
                                                            uint8_t* __restrict__ q, float* __restrict__ scales) {
  dependent_wait();
  dependents_may_launch();
  const int groups = (width + kGroup - 1) / kGroup;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * 8 + warp;   // (row, group) pair
  if (item >= static_cast<long long>(rows) * groups) return;
  const int row = static_cast<int>(item / groups), g = static_cast<int>(item % groups);
  const int src = gather ? gather[row] : row;
  const float scale = quantize_group<T>(x + static_cast<size_t>(src) * width, q + static_cast<size_t>(row) * width, g,
                                        width, lane);
  if (lane == 0) scales[static_cast<size_t>(row) * groups + g] = scale;
}

cudaError_t launch_quantize(const void* x, int dtype, int rows, int width, const int32_t* gather, uint8_t* q,
                            float* scales, cudaStream_t stream, int* launches) {
  if (rows <= 0) return cudaSuccess;
  const long long items = static_cast<long long>(rows) * ((width + kGroup - 1) / kGroup);
  const unsigned blocks = static_cast<unsigned>((items + 7) / 8);
  if (dtype == 0)
    launch_dependent(quantize_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                     static_cast<const __nv_bfloat16*>(x), rows, width, gather, q, scales);
  else
    launch_dependent(quantize_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, static_cast<const float*>(x),
                     rows, width, gather, q, scales);
  if (launches) *launches += 1;
  return cudaGetLastError();
}

}  // namespace moe
