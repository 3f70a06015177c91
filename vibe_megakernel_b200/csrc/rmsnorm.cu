// RMSNorm of the residual stream in front of the MoE block, one block of threads per token.
//
// Reference: `rms` of megabench/tasks/common.py:13-21 as called for the MoE block at
// megabench/tasks/frontier.py:260,335:
//   n = x.float() * rsqrt(mean(x.float()^2) + eps)
//   weight_in_fp32 (DeepSeek family): out = bf16(n * weight.float())
//   otherwise (Llama / Qwen / GLM):   out = bf16(n) * weight       (a bf16 product: one more rounding)
// The mean is an fp32 sum in a fixed order (per-thread runs, warp butterflies, then the warps in
// order), so a row's result does not depend on the batch.
#include "common.cuh"
#include "kernels.h"

namespace moe {

constexpr int kNormThreads = 256;

__global__ void __launch_bounds__(kNormThreads) rmsnorm_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                                    const __nv_bfloat16* __restrict__ weight, float eps,
                                                                    int weight_in_fp32, int hidden,
                                                                    __nv_bfloat16* __restrict__ out) {
  __shared__ float s_part[kNormThreads / 32];
  __shared__ float s_scale;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const __nv_bfloat16* row = x + static_cast<size_t>(blockIdx.x) * hidden;
  dependent_wait();
  dependents_may_launch();
  float sum = 0.f;
  for (int k = tid * 8; k < hidden; k += kNormThreads * 8) {     // hidden is a multiple of 8 (checked by the launcher)
    const uint4 raw = *reinterpret_cast<const uint4*>(row + k);
    const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = __bfloat162float(v[i]);
      sum = fmaf(f, f, sum);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, off));
  if (lane == 0) s_part[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
    for (int w = 0; w < kNormThreads / 32; ++w) total = __fadd_rn(total, s_part[w]);
    s_scale = __frsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(hidden)), eps));
  }
  __syncthreads();
  const float scale = s_scale;
  __nv_bfloat16* dst = out + static_cast<size_t>(blockIdx.x) * hidden;
  for (int k = tid * 8; k < hidden; k += kNormThreads * 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + k);
    const uint4 wraw = *reinterpret_cast<const uint4*>(weight + k);
    const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
    const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&wraw);
    uint4 packed;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float n = __fmul_rn(__bfloat162float(v[i]), scale);
      const float gw = __bfloat162float(g[i]);
      o[i] = weight_in_fp32 ? __float2bfloat16_rn(__fmul_rn(n, gw))
                            : __float2bfloat16_rn(__fmul_rn(__bfloat162float(__float2bfloat16_rn(n)), gw));
    }
    *reinterpret_cast<uint4*>(dst + k) = packed;
  }
}

cudaError_t launch_rmsnorm(const __nv_bfloat16* x, const __nv_bfloat16* weight, float eps, int weight_in_fp32, int tokens,
                           int hidden, __nv_bfloat16* out, cudaStream_t stream, int* launches) {
  if (hidden % 8 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) |
                      reinterpret_cast<uintptr_t>(out)) & 15))
    return cudaErrorInvalidValue;
  launch_dependent(rmsnorm_rows_kernel, dim3(tokens), dim3(kNormThreads), 0, stream, x, weight, eps, weight_in_fp32,
                   hidden, out);
  if (launches) *launches += 1;
  return cudaGetLastError();
}

}  // namespace moe
