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

// The same arithmetic for the tensor-core kernel, laid out for a persistent CTA whose epilogue warps
// also fold the next item's K blocks, so every cycle here delays the tensor pipe:
//   * the activations of a thread's columns are computed first, independent chains the scheduler can
//     interleave (a warp reduction per column in the same loop serialised them);
//   * one thread per token computes the scale (a division) instead of all 128 of the column;
//   * the e4m3 bytes are collected in shared memory as [token][128 channels] and leave as whole rows,
//     16 bytes per thread, instead of one byte per thread and token;
//   * the divisions (SwiGLU, quantisation) take the forms without range check and slow path
//     (common.cuh), the quantisation's with the reciprocal of the token's scale computed once;
//   * no thread fences: whoever announces the tile does, after the closing barrier.
//   tid: 0..THREADS-1; rend: end of this thread's valid columns; rows: the chunk's rows;
//   s_amax: float[4][nt]; s_scale: float[2][nt] (scales, then their reciprocals);
//   s_tile: uint8_t[nt][128], 16-byte aligned.
template <int CPT, int THREADS>
__device__ __forceinline__ void epilogue_swiglu_requant_tile(float (&gate)[CPT], const float (&up)[CPT], int tid, int m,
                                                             int col0, int nt, int rend, int rows, int row0, int tile_m,
                                                             int inter, float* s_amax, float* s_scale, uint8_t* s_tile,
                                                             uint8_t* __restrict__ aq, float* __restrict__ as,
                                                             const SwigluMode& mode) {
  const int quarter = m >> 5, lane = m & 31;
#pragma unroll
  for (int n = 0; n < CPT; ++n) {
    if (col0 + n < rend) {      // uniform across the warp
      float g = bf16_round(gate[n]);
      float u = bf16_round(up[n]);
      if (mode.limit > 0.f) {
        g = fminf(g, mode.limit);
        u = fminf(fmaxf(u, -mode.limit), mode.limit);
      }
      float a = silu_times(g, u);
      if (mode.slot_weight) {
        const int dest = mode.row_dest[row0 + col0 + n];
        if (dest < mode.routed_rows) a = __fmul_rn(a, mode.slot_weight[dest]);
      }
      gate[n] = a;
    }
  }
#pragma unroll
  for (int n = 0; n < CPT; ++n) {
    if (col0 + n < rend) {
      const unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(gate[n])));
      if (lane == 0) s_amax[quarter * nt + col0 + n] = __uint_as_float(bits);
    }
  }
  epilogue_sync<THREADS>();
  const int groups = inter / kGroup;
  for (int c = tid; c < rows; c += THREADS) {
    const float amax = fmaxf(fmaxf(s_amax[c], s_amax[nt + c]), fmaxf(s_amax[2 * nt + c], s_amax[3 * nt + c]));
    const float scale = group_scale(amax);
    s_scale[c] = scale;
    s_scale[nt + c] = __frcp_rn(scale);
    as[static_cast<size_t>(row0 + c) * groups + tile_m] = scale;
  }
  epilogue_sync<THREADS>();
#pragma unroll
  for (int n = 0; n < CPT; ++n) {
    const int c = col0 + n;
    if (c < rend) s_tile[c * kGroup + m] = to_e4m3_near(gate[n], s_scale[c], s_scale[nt + c]);
  }
  epilogue_sync<THREADS>();
  for (int i = tid; i < rows * (kGroup / 16); i += THREADS) {
    const int r = i >> 3, part = i & 7;
    *reinterpret_cast<uint4*>(aq + static_cast<size_t>(row0 + r) * inter + tile_m * kGroup + part * 16) =
        *reinterpret_cast<const uint4*>(s_tile + r * kGroup + part * 16);
  }
  epilogue_sync<THREADS>();   // every row is on its way: the tile may be announced, the scratch reused
}

// Down projection in the tensor-core kernel: the bf16 roundings of a work item collected in shared
// memory as [token][128 channels] and stored as whole 256-byte row pieces, 16 bytes per thread.
//   dest: shared int[nt], destination row of every token column; s_tile: bf16 [nt][128].
// The caller's next barrier over the epilogue threads protects the tile against reuse.
//   row_ptr (optional, shared uint64[nt]): the address of every token column's output row instead of
//   dest/out (rows that live in other GPUs' memory).
template <int CPT, int THREADS>
__device__ __forceinline__ void epilogue_store_tile(const float (&sum)[CPT], int tid, int m, int col0, int rend, int rows,
                                                    int tile_m, int hidden, const int* dest, __nv_bfloat16* s_tile,
                                                    __nv_bfloat16* __restrict__ out,
                                                    const unsigned long long* row_ptr = nullptr) {
#pragma unroll
  for (int n = 0; n < CPT; ++n) {
    const int c = col0 + n;
    if (c < rend) s_tile[c * kGroup + m] = __float2bfloat16_rn(sum[n]);
  }
  epilogue_sync<THREADS>();
  for (int i = tid; i < rows * (kGroup / 8); i += THREADS) {
    const int r = i >> 4, part = i & 15;
    __nv_bfloat16* row = row_ptr ? reinterpret_cast<__nv_bfloat16*>(row_ptr[r]) : out + static_cast<size_t>(dest[r]) * hidden;
    *reinterpret_cast<uint4*>(row + tile_m * kGroup + part * 8) = *reinterpret_cast<const uint4*>(s_tile + r * kGroup + part * 8);
  }
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
