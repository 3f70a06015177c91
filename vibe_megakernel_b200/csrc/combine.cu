// Weighted combine / un-permute: y[t] = bf16( sum over slots, in slot order, of row*weight, then
// the shared expert's row ), all in fp32 with a separate multiply and add per slot.
//
// Reference: megabench/tasks/frontier.py:349-354 (`output + down.float()*weights[slot]`, then the
// shared expert) and the slot-order fp32 sum with one bf16 rounding of
// megabench/tasks/megamoe.py:176-182 (there the routing weight was applied before the down
// projection: weights == NULL gives that plain sum). The down-projection rows are already stored in slot order
// (row token*topk+slot), which is the reference's `slots[order] = output` un-permutation.
// With a residual stream the block's output is x + bf16(sum), itself rounded to bf16
// (`x = x + output.to(x.dtype)`, megabench/tasks/frontier.py:354).
#include "common.cuh"
#include "kernels.h"

namespace moe {

__global__ void __launch_bounds__(256) combine_kernel(const __nv_bfloat16* __restrict__ slots,
                                                      const float* __restrict__ weights, int tokens, int topk,
                                                      int hidden, int shared, __nv_bfloat16* __restrict__ y,
                                                      const __nv_bfloat16* __restrict__ residual, const FlagWait wait) {
  dependent_wait();
  wait_for_peers(wait);         // expert parallel: the slot rows come from the experts' owners
  const int t = blockIdx.y;
  const int c = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c >= hidden) return;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  // eight slots at a time: their loads are issued before the first addition (a load per addition made
  // the sum a chain of topk memory latencies); the additions keep the slot order
  for (int s0 = 0; s0 < topk; s0 += 8) {
    uint4 raw[8];
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const size_t row = static_cast<size_t>(t) * topk + min(s0 + j, topk - 1);
      w[j] = weights ? weights[row] : 1.f;   // null: the rows carry their weight already
      raw[j] = *reinterpret_cast<const uint4*>(slots + row * hidden + c);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (s0 + j < topk) {
        const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(__bfloat162float(v[i]), w[j]));
      }
    }
  }
  if (shared) {
    const size_t row = static_cast<size_t>(tokens) * topk + t;
    const uint4 raw = *reinterpret_cast<const uint4*>(slots + row * hidden + c);
    const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __bfloat162float(v[i]));
  }
  uint4 packed;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(acc[i]);
  if (residual) {
    const uint4 raw = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * hidden + c);
    const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(__fadd_rn(__bfloat162float(v[i]), __bfloat162float(o[i])));
  }
  *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * hidden + c) = packed;
}

cudaError_t launch_combine(const __nv_bfloat16* slots, const float* weights, int tokens, int topk, int hidden,
                           int shared, __nv_bfloat16* y, cudaStream_t stream, int* launches,
                           const __nv_bfloat16* residual, const FlagWait* wait) {
  dim3 grid((hidden / 8 + 255) / 256, tokens);
  launch_dependent(combine_kernel, grid, dim3(256), 0, stream, slots, weights, tokens, topk, hidden, shared, y,
                   residual, wait ? *wait : FlagWait{});
  if (launches) *launches += 1;
  return cudaGetLastError();
}

}  // namespace moe
