// Device-side self-check of the divisions the tensor-core epilogues use in place of the library's
// (common.cuh: quotient_rn, silu_times, to_e4m3_pair): every value pair is run through both forms and
// the disagreements are counted. Test infrastructure behind moe_selfcheck_divisions; nothing else
// calls it.
#include "common.cuh"
#include "kernels.h"

namespace moe {

// counts[0]: SwiGLU values whose bits differ from the plain expression; counts[1]: e4m3 codes that
// differ from to_e4m3; counts[2]: pairs checked.
__global__ void selfcheck_divisions_kernel(const float* g, const float* u, const float* scale, int n, int* counts) {
  int bad_act = 0, bad_code = 0, seen = 0;
  for (int pair = blockIdx.x * blockDim.x + threadIdx.x; 2 * pair + 1 < n; pair += gridDim.x * blockDim.x) {
    const int i = 2 * pair, j = i + 1;      // two neighbours per step: the pair form packs two codes
    const float a0 = __fmul_rn(__fdiv_rn(g[i], __fadd_rn(1.f, expf(-g[i]))), u[i]);
    const float a1 = __fmul_rn(__fdiv_rn(g[j], __fadd_rn(1.f, expf(-g[j]))), u[j]);
    const float b0 = silu_times(g[i], u[i]);
    const float b1 = silu_times(g[j], u[j]);
    bad_act += (__float_as_uint(a0) != __float_as_uint(b0)) + (__float_as_uint(a1) != __float_as_uint(b1));
    const float s = scale[pair];
    const float r = __frcp_rn(s);
    const uint32_t want = static_cast<uint32_t>(to_e4m3(a0, s)) | static_cast<uint32_t>(to_e4m3(a1, s)) << 8;
    bad_code += (to_e4m3_pair(b0, b1, s, r) != want);
    seen += 1;
  }
  atomicAdd(counts + 0, bad_act);
  atomicAdd(counts + 1, bad_code);
  atomicAdd(counts + 2, seen);
}

}  // namespace moe

extern "C" int moe_selfcheck_divisions(const float* gate, const float* up, const float* scales, int32_t n, int32_t* counts,
                                       void* stream) {
  if (!gate || !up || !scales || !counts || n < 2 || (n & 1)) return MOE_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(counts, 0, 3 * sizeof(int32_t), st);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int threads = 256;
  const int blocks = (n / 2 + threads - 1) / threads;
  moe::selfcheck_divisions_kernel<<<blocks, threads, 0, st>>>(gate, up, scales, n, counts);
  e = cudaGetLastError();
  return e == cudaSuccess ? MOE_OK : static_cast<int>(e);
}
