// Device helpers shared by the Kimi latent-MoE kernels and the MXFP4 GEMM's pair epilogues: the
// (hi, lo) E4M3 split of a bf16 value and the situ activation.
#pragma once

#include "common.cuh"

namespace moe {

// ---- bf16 value -> (hi, lo) E4M3 pieces under per-32-channel E8M0 scales --------------------------
// `lanes` lanes (a power of two, consecutive) hold the block's 32 channels between them.
// megabench/tasks/quantization.py:62-84 gives the scale rule (biased exponent from the block maximum).
__device__ __forceinline__ int ue8m0_of(float amax) {
  return max((__float_as_int(amax) + (0x7FFFFF - 0x600000)) >> 23, 105 + 8) - 8;
}
__device__ __forceinline__ float block_max(float v, int lanes) {
  for (int off = 1; off < lanes; off <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}
template <int N>
__device__ __forceinline__ void split_e4m3(const float (&v)[N], int lanes, uint8_t (&hi)[N], uint8_t (&lo)[N], int& e_hi,
                                           int& e_lo) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < N; ++i) amax = fmaxf(amax, fabsf(v[i]));
  e_hi = ue8m0_of(block_max(amax, lanes));
  const float inv_hi = __int_as_float((254 - e_hi) << 23), scale_hi = __int_as_float(e_hi << 23);
  float r[N], rmax = 0.f;
#pragma unroll
  for (int i = 0; i < N; ++i) {
    hi[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(__fmul_rn(v[i], inv_hi), __NV_SATFINITE, __NV_E4M3));
    r[i] = __fsub_rn(v[i], __fmul_rn(e4m3_to_float(hi[i]), scale_hi));     // exact: both have few bits
    rmax = fmaxf(rmax, fabsf(r[i]));
  }
  e_lo = ue8m0_of(block_max(rmax, lanes));
  const float inv_lo = __int_as_float((254 - e_lo) << 23);
#pragma unroll
  for (int i = 0; i < N; ++i)
    lo[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(__fmul_rn(r[i], inv_lo), __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float situ_f32(float g, float u) {
  // 4 tanh(g/4) * sigmoid(g) * 25 tanh(u/25), in the reference's order (megabench/tasks/kimi.py:134-135)
  const float a = __fmul_rn(4.f, tanhf(__fdiv_rn(g, 4.f)));
  const float s = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-g)));
  const float b = __fmul_rn(25.f, tanhf(__fdiv_rn(u, 25.f)));
  return __fmul_rn(__fmul_rn(a, s), b);
}

}  // namespace moe
