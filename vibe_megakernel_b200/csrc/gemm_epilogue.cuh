// Epilogues shared by the tensor-core grouped GEMM and the CUDA-core check arm. A thread owns
// output channel (tile*128 + m) for CPT consecutive tokens of the chunk starting at column col0;
// THREADS epilogue threads cooperate (128 per group of token columns).
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace moe {

template <int THREADS>
__device__ __forceinline__ void epilogue_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}
// Barrier over the epilogue threads that also returns the OR of `pred`, so that every thread
// takes the same exit decision.
template <int THREADS>
__device__ __forceinline__ bool epilogue_any(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.or.pred q, 1, %2, p;\nselp.u32 %0, 1, 0, q;\n}\n"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred)), "n"(THREADS)
      : "memory");
  return r != 0;
}

// SwiGLU on the bf16-rounded gate/up GEMM outputs, fp32 g/(1+exp(-g))*u, then per-token
// requantisation of this tile's 128 channels (exactly one quantisation group).
// Reference: megabench/tasks/megamoe.py:116-128 (clamp and routing weight only when `mode` asks)
// and megabench/tasks/quantization.py:87-109.
//   s_amax: shared float[4][nt] scratch (one row per 32-channel quarter of the tile);
//   m: 0..127, the thread's channel inside the tile; rows: valid tokens of the chunk.
template <int CPT, int THREADS>
__device__ __forceinline__ void epilogue_swiglu_requant(float (&gate)[CPT], const float (&up)[CPT], int m, int col0,
                                                        int nt, int rows, int row0, int tile_m, int inter,
                                                        float* s_amax, uint8_t* __restrict__ aq,
                                                        float* __restrict__ as, const SwigluMode& mode) {
  const int quarter = m >> 5, lane = m & 31;
#pragma unroll
  for (int n = 0; n < CPT; ++n) {
    if (col0 + n < rows) {      // uniform across the warp
      float g = bf16_round(gate[n]);
      float u = bf16_round(up[n]);
      if (mode.limit > 0.f) {
        g = fminf(g, mode.limit);
        u = fminf(fmaxf(u, -mode.limit), mode.limit);
      }
      float a = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.f, expf(-g))), u);
      if (mode.slot_weight) {
        const int dest = mode.row_dest[row0 + col0 + n];
        if (dest < mode.routed_rows) a = __fmul_rn(a, mode.slot_weight[dest]);
      }
      gate[n] = a;
      const unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(a)));
      if (lane == 0) s_amax[quarter * nt + col0 + n] = __uint_as_float(bits);
    }
  }
  epilogue_sync<THREADS>();
  const int groups = inter / kGroup;
#pragma unroll
  for (int n = 0; n < CPT; ++n) {
    const int c = col0 + n;
    if (c < rows) {
      const float amax = fmaxf(fmaxf(s_amax[c], s_amax[nt + c]), fmaxf(s_amax[2 * nt + c], s_amax[3 * nt + c]));
      const float scale = group_scale(amax);
      const size_t row = static_cast<size_t>(row0 + c);
      aq[row * inter + tile_m * kGroup + m] = to_e4m3(gate[n], scale);
      if (m == 0) as[row * groups + tile_m] = scale;
    }
  }
  // The stores above are made visible device-wide (to plain loads and to TMA reads) before the
  // barrier, so one thread may announce the tile right after it.
  __threadfence();
  fence_async_global();
  epilogue_sync<THREADS>();   // s_amax may be reused by the next work item
}

// Down projection: one bf16 rounding of the fp32 accumulator, stored at the row's slot.
// Reference: megabench/tasks/megamoe.py:149 (`@ w2.T` with a bf16 result).
template <int CPT>
__device__ __forceinline__ void epilogue_store_rows(const float (&acc)[CPT], int m, int col0, int rows, int row0,
                                                    int tile_m, int hidden, const int32_t* __restrict__ row_dest,
                                                    __nv_bfloat16* __restrict__ out) {
#pragma unroll
  for (int n = 0; n < CPT; ++n) {
    const int c = col0 + n;
    if (c < rows) {
      const size_t dest = static_cast<size_t>(row_dest ? row_dest[row0 + c] : row0 + c);   // null = in place
      out[dest * hidden + tile_m * kGroup + m] = __float2bfloat16_rn(acc[n]);
    }
  }
}

}  // namespace moe
