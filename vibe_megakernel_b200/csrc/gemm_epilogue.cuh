// Epilogues shared by the tensor-core grouped GEMM and the CUDA-core check arm. Both run with
// 128 threads, thread m owning output channel (tile*128 + m) for every token of the chunk.
#pragma once

#include "common.cuh"

namespace moe {

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier over the 128 epilogue threads that also returns the OR of `pred`, so that every
// thread takes the same exit decision.
__device__ __forceinline__ bool epilogue_any(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.or.pred q, 1, 128, p;\nselp.u32 %0, 1, 0, q;\n}\n"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}

// SwiGLU on the bf16-rounded gate/up GEMM outputs, fp32 g/(1+exp(-g))*u, then per-token
// requantisation of this tile's 128 channels (exactly one quantisation group).
// Reference: megabench/tasks/megamoe.py:116-128 (without clamp and routing weight) and
// megabench/tasks/quantization.py:87-109.
//   s_amax: shared float[4][NT] scratch; m: 0..127 (thread's channel inside the tile).
template <int NT>
__device__ __forceinline__ void epilogue_swiglu_requant(float (&gate)[NT], const float (&up)[NT], int m, int rows,
                                                        int row0, int tile_m, int inter, float* s_amax,
                                                        uint8_t* __restrict__ aq, float* __restrict__ as) {
  const int quarter = m >> 5, lane = m & 31;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const float g = bf16_round(gate[n]);
    const float u = bf16_round(up[n]);
    const float a = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.f, expf(-g))), u);
    gate[n] = a;
    const unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(a)));
    if (lane == 0) s_amax[quarter * NT + n] = __uint_as_float(bits);
  }
  epilogue_sync();
  const int groups = inter / kGroup;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    if (n < rows) {
      const float amax = fmaxf(fmaxf(s_amax[n], s_amax[NT + n]), fmaxf(s_amax[2 * NT + n], s_amax[3 * NT + n]));
      const float scale = group_scale(amax);
      const size_t row = static_cast<size_t>(row0 + n);
      aq[row * inter + tile_m * kGroup + m] = to_e4m3(gate[n], scale);
      if (m == 0) as[row * groups + tile_m] = scale;
    }
  }
  epilogue_sync();   // s_amax may be reused by the next work item
}

// Down projection: one bf16 rounding of the fp32 accumulator, stored at the row's slot.
// Reference: megabench/tasks/megamoe.py:149 (`@ w2.T` with a bf16 result).
template <int NT>
__device__ __forceinline__ void epilogue_store_rows(const float (&acc)[NT], int m, int rows, int row0, int tile_m,
                                                    int hidden, const int32_t* __restrict__ row_dest,
                                                    __nv_bfloat16* __restrict__ out) {
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    if (n < rows) {
      const size_t dest = static_cast<size_t>(row_dest[row0 + n]);
      out[dest * hidden + tile_m * kGroup + m] = __float2bfloat16_rn(acc[n]);
    }
  }
}

}  // namespace moe
