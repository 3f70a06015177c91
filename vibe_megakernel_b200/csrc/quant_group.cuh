// One warp quantises one group of 128 channels of one row to e4m3 with a dynamic fp32 scale.
// Reference: pack_fp8_activation(value, power_of_two=False, block=128, scale_format="float"),
// megabench/tasks/quantization.py:87-109 with fp8_scale (:57-59).
#pragma once

#include "common.cuh"

namespace moe {

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// in/out: the row's first element; g: group index; width: row length (a ragged last group is padded
// with zeros for the amax and the padding is not stored). Returns the scale (same in all lanes).
template <typename T>
__device__ __forceinline__ void load_group(const T* in, int g, int width, int lane, float (&v)[4]) {
  const int k0 = g * kGroup + lane * 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = (k0 + j < width) ? load_as_float<T>(in + k0 + j) : 0.f;
}

// Second half, on values already loaded (so a caller can have several groups' loads in flight).
__device__ __forceinline__ float quantize_loaded(const float (&v)[4], uint8_t* out, int g, int width, int lane) {
  const int k0 = g * kGroup + lane * 4;
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float scale = group_scale(amax);
  if (k0 + 3 < width && (width & 3) == 0) {
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) packed |= static_cast<uint32_t>(to_e4m3(v[j], scale)) << (8 * j);
    *reinterpret_cast<uint32_t*>(out + k0) = packed;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (k0 + j < width) out[k0 + j] = to_e4m3(v[j], scale);
  }
  return scale;
}

// The same arithmetic for a whole group whose bytes the caller stores itself (to several rows):
// the lane's four e4m3 bytes in `packed`, the scale returned.
__device__ __forceinline__ float quantize_values(const float (&v)[4], uint32_t& packed) {
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float scale = group_scale(amax);
  packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) packed |= static_cast<uint32_t>(to_e4m3(v[j], scale)) << (8 * j);
  return scale;
}

template <typename T>
__device__ __forceinline__ float quantize_group(const T* in, uint8_t* out, int g, int width, int lane) {
  float v[4];
  load_group<T>(in, g, width, lane, v);
  return quantize_loaded(v, out, g, width, lane);
}

}  // namespace moe
