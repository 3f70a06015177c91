// CUDA-core check arms of the grouped FP8 GEMMs. Same work decomposition and epilogues as the
// tensor-core kernel. They exist for the tests; neither is tuned and the layer never selects one
// unless the caller asks for it.
//   MOE_GEMM_SIMT       the tensor-core arithmetic on CUDA cores: exact e4m3 products summed per
//                       128-deep block by plain FMAs, then acc += block * (w_scale * x_scale). Tells
//                       a tensor-core/TMA fault from a pipeline fault.
//   MOE_GEMM_SIMT_BF16  the reference's "dequantize-then-bf16" schedule, megabench/tasks/megamoe.py:146-149:
//                       w = bf16(e4m3 * block scale), x = bf16(e4m3 * group scale) (the fp32 product
//                       rounded once more to bf16, as `unpack_*(...).to(bfloat16)` does), products
//                       of two bf16 values are exact in fp32 and are summed in fp32 over the whole
//                       contraction in channel order; the epilogues round that sum once to bf16.
//                       What separates this arm from the reference's CPU GEMM is only the order
//                       of the fp32 additions.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "kernels.h"

namespace moe {

struct SimtDev {
  const Chunk* chunks;
  const int32_t* n_chunks;
  int tiles_m, kblocks, m, k, n_local;
  const uint8_t* act;
  const float* act_scale;
  const uint8_t* w_a; const float* w_a_scale;
  const uint8_t* w_b; const float* w_b_scale;
  const uint8_t* s_a; const float* s_a_scale;
  const uint8_t* s_b; const float* s_b_scale;
  uint8_t* aq; float* as;
  __nv_bfloat16* out; const int32_t* row_dest;
  SwigluMode swiglu;
};

__device__ __forceinline__ void unpack16(const uint4& v, float* f) {
  const uint8_t* b = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
  for (int i = 0; i < 16; ++i) f[i] = e4m3_to_float(b[i]);
}

// 16 e4m3 values times `scale`, each product rounded to bf16 (kept as fp32)
__device__ __forceinline__ void unpack16_bf16(const uint4& v, float scale, float* f) {
  const uint8_t* b = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
  for (int i = 0; i < 16; ++i) f[i] = bf16_round(__fmul_rn(e4m3_to_float(b[i]), scale));
}

// The reference's rounding schedule (see the head of the file). One thread per output channel,
// token rows of the current K block dequantised once into shared memory.
template <int NT, bool DUAL>
__global__ void __launch_bounds__(128) grouped_gemm_bf16ops_kernel(const SimtDev p) {
  __shared__ float s_amax[4 * NT];
  __shared__ __align__(16) float s_x[NT * 128];
  const int n_units = *p.n_chunks * p.tiles_m;
  const int u = blockIdx.x;
  if (u >= n_units) return;
  const Chunk ch = p.chunks[u / p.tiles_m];
  const int mt = u % p.tiles_m;
  const bool shared_e = ch.expert >= p.n_local;
  const int m = threadIdx.x;
  const int KB = p.kblocks;
  const size_t wrow = (shared_e ? 0 : static_cast<size_t>(ch.expert) * p.m) + mt * 128 + m;
  const uint8_t* wa = (shared_e ? p.s_a : p.w_a) + wrow * p.k;
  const uint8_t* wb = DUAL ? (shared_e ? p.s_b : p.w_b) + wrow * p.k : nullptr;
  const float* sa = (shared_e ? p.s_a_scale : p.w_a_scale + static_cast<size_t>(ch.expert) * p.tiles_m * KB) +
                    static_cast<size_t>(mt) * KB;
  const float* sb = DUAL ? (shared_e ? p.s_b_scale : p.w_b_scale + static_cast<size_t>(ch.expert) * p.tiles_m * KB) +
                               static_cast<size_t>(mt) * KB
                         : nullptr;
  float acc_a[NT], acc_b[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) { acc_a[n] = 0.f; acc_b[n] = 0.f; }
  for (int kb = 0; kb < KB; ++kb) {
    __syncthreads();
    for (int i = threadIdx.x; i < NT * 8; i += 128) {   // 16 channels of a token row's K block
      const int n = i >> 3, c = i & 7;
      float f[16];
      if (n < ch.rows) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.act + static_cast<size_t>(ch.row0 + n) * p.k + kb * 128 + c * 16);
        unpack16_bf16(v, p.act_scale[static_cast<size_t>(ch.row0 + n) * KB + kb], f);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) s_x[n * 128 + c * 16 + j] = f[j];
    }
    __syncthreads();
    const float wsa = sa[kb];
    const float wsb = DUAL ? sb[kb] : 0.f;
    for (int c = 0; c < 8; ++c) {
      float fa[16], fb[16];
      unpack16_bf16(*reinterpret_cast<const uint4*>(wa + kb * 128 + c * 16), wsa, fa);
      if (DUAL) unpack16_bf16(*reinterpret_cast<const uint4*>(wb + kb * 128 + c * 16), wsb, fb);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const float* fx = s_x + n * 128 + c * 16;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          acc_a[n] = fmaf(fa[j], fx[j], acc_a[n]);
          if (DUAL) acc_b[n] = fmaf(fb[j], fx[j], acc_b[n]);
        }
      }
    }
  }
  if constexpr (DUAL) {
    epilogue_swiglu_requant<NT, 128>(acc_a, acc_b, m, 0, NT, ch.rows, ch.row0, mt, p.m, s_amax, p.aq, p.as, p.swiglu);
  } else {
    epilogue_store_rows<NT>(acc_a, m, 0, ch.rows, ch.row0, mt, p.m, p.row_dest, p.out);
  }
}

template <int NT, bool DUAL>
__global__ void __launch_bounds__(128) grouped_gemm_simt_kernel(const SimtDev p) {
  __shared__ float s_amax[4 * NT];
  __shared__ __align__(16) uint8_t s_x[NT * 128];
  const int n_units = *p.n_chunks * p.tiles_m;
  const int u = blockIdx.x;
  if (u >= n_units) return;
  const Chunk ch = p.chunks[u / p.tiles_m];
  const int mt = u % p.tiles_m;
  const bool shared_e = ch.expert >= p.n_local;
  const int m = threadIdx.x;
  const int KB = p.kblocks;
  const size_t wrow = (shared_e ? 0 : static_cast<size_t>(ch.expert) * p.m) + mt * 128 + m;
  const uint8_t* wa = (shared_e ? p.s_a : p.w_a) + wrow * p.k;
  const uint8_t* wb = DUAL ? (shared_e ? p.s_b : p.w_b) + wrow * p.k : nullptr;
  const float* sa = (shared_e ? p.s_a_scale : p.w_a_scale + static_cast<size_t>(ch.expert) * p.tiles_m * KB) +
                    static_cast<size_t>(mt) * KB;
  const float* sb = DUAL ? (shared_e ? p.s_b_scale : p.w_b_scale + static_cast<size_t>(ch.expert) * p.tiles_m * KB) +
                               static_cast<size_t>(mt) * KB
                         : nullptr;
  float acc_a[NT], acc_b[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) { acc_a[n] = 0.f; acc_b[n] = 0.f; }

  for (int kb = 0; kb < KB; ++kb) {
    __syncthreads();
    for (int i = threadIdx.x; i < NT * 8; i += 128) {   // 16-byte pieces of the token rows' K block
      const int n = i >> 3, c = i & 7;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (n < ch.rows) v = *reinterpret_cast<const uint4*>(p.act + static_cast<size_t>(ch.row0 + n) * p.k + kb * 128 + c * 16);
      *reinterpret_cast<uint4*>(s_x + n * 128 + c * 16) = v;
    }
    __syncthreads();
    float pa[NT], pb[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) { pa[n] = 0.f; pb[n] = 0.f; }
    for (int c = 0; c < 8; ++c) {
      float fa[16], fb[16];
      unpack16(*reinterpret_cast<const uint4*>(wa + kb * 128 + c * 16), fa);
      if (DUAL) unpack16(*reinterpret_cast<const uint4*>(wb + kb * 128 + c * 16), fb);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        float fx[16];
        unpack16(*reinterpret_cast<const uint4*>(s_x + n * 128 + c * 16), fx);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          pa[n] = fmaf(fa[j], fx[j], pa[n]);
          if (DUAL) pb[n] = fmaf(fb[j], fx[j], pb[n]);
        }
      }
    }
    const float wsa = sa[kb];
    const float wsb = DUAL ? sb[kb] : 0.f;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const float xs = n < ch.rows ? p.act_scale[static_cast<size_t>(ch.row0 + n) * KB + kb] : 0.f;
      acc_a[n] = fmaf(pa[n], __fmul_rn(wsa, xs), acc_a[n]);
      if (DUAL) acc_b[n] = fmaf(pb[n], __fmul_rn(wsb, xs), acc_b[n]);
    }
  }
  if constexpr (DUAL) {
    epilogue_swiglu_requant<NT, 128>(acc_a, acc_b, m, 0, NT, ch.rows, ch.row0, mt, p.m, s_amax, p.aq, p.as, p.swiglu);
  } else {
    epilogue_store_rows<NT>(acc_a, m, 0, ch.rows, ch.row0, mt, p.m, p.row_dest, p.out);
  }
}

cudaError_t launch_gemm_simt(const GemmArgs& a, cudaStream_t stream, int* launches) {
  if (a.k % 128 || a.m % 128) return cudaErrorInvalidValue;
  SimtDev d{a.chunks, a.n_chunks, a.m / 128, a.k / 128, a.m, a.k, a.n_local, a.act, a.act_scale, a.w_a, a.w_a_scale,
            a.w_b, a.w_b_scale, a.s_a, a.s_a_scale, a.s_b, a.s_b_scale, a.aq, a.as, a.out, a.row_dest, a.swiglu};
  const int grid = a.max_units > 0 ? a.max_units : 1;
#define MOE_SIMT(NT, DUAL)                                                              \
  do {                                                                                  \
    if (a.bf16_operands) grouped_gemm_bf16ops_kernel<NT, DUAL><<<grid, 128, 0, stream>>>(d); \
    else grouped_gemm_simt_kernel<NT, DUAL><<<grid, 128, 0, stream>>>(d);               \
  } while (0)
  if (a.dual) {
    if (a.tile == 16) MOE_SIMT(16, true); else if (a.tile == 32) MOE_SIMT(32, true); else MOE_SIMT(64, true);
  } else {
    if (a.tile == 16) MOE_SIMT(16, false); else if (a.tile == 32) MOE_SIMT(32, false); else MOE_SIMT(64, false);
  }
#undef MOE_SIMT
  if (launches) *launches += 1;
  return cudaGetLastError();
}

}  // namespace moe
