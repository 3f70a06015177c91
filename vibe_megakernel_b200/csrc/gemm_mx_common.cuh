// What the two MegaMoE-native GEMM kernels (gemm_mx.cu: weights on the MMA's M side; gemm_mx_wide.cu:
// tokens on it) share: the block-scaled MMA and its descriptors, the TMEM stores of the scale
// factors, the asynchronous copies of scale bytes, the walk over the work list, the tensor maps.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace moe {

constexpr int kMxSmem = 232448;       // 227 KiB per CTA
constexpr int kMxSfCols = 16;         // TMEM columns of scale factors per K block of 128
constexpr int kMxSfGroup = 4;         // K blocks whose scale factors are written and released together (16 bytes per row)
constexpr int kMxSfSlots = 4;         // groups that fit in TMEM at a time
constexpr int kMxSfAhead = 2;         // groups whose scale bytes are on their way to shared memory
constexpr int kMxSfRing = kMxSfAhead + 2;   // + the group being read + the one a faster thread may already refill

__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ void tmem_st2(uint32_t taddr, uint32_t a, uint32_t b) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, int32_t x, int32_t y, int32_t z, uint64_t* bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3, %4}], [%5], %6;"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
// Instruction descriptor, kind::mxf8f6f4 with block scales: A = E2M1, B = E4M3, both K-major,
// E8M0 scales, M = 128; `sf` picks the byte (32-wide K block) of the scale columns for both sides.
__device__ __forceinline__ uint32_t idesc_mx(int n, uint32_t sf) {
  return (sf << 4) | (5u << 7) | (0u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) |
         (static_cast<uint32_t>(128 >> 4) << 24) | (sf << 29);
}
__device__ __forceinline__ void mma_mx(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}

// Scale bytes of K blocks [4g, 4g+4) of one row, asynchronously into 16 bytes of shared memory:
// one 16-byte copy when the row length allows, else up to four 4-byte copies (a 128-wide K block
// always has its four bytes); K blocks past the end read as zero.
__device__ __forceinline__ void copy_scale_group(uint8_t* dst, const uint8_t* row, int g, int kblocks, bool vec) {
  if (vec) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(row + 16 * g) : "memory");
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (4 * g + j < kblocks)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst + 4 * j)), "l"(row + 4 * (4 * g + j)) : "memory");
      else
        *reinterpret_cast<uint32_t*>(dst + 4 * j) = 0u;
    }
  }
}
// Barrier over the 128 scale-writer threads that also returns the OR of `pred`: one exit decision
// for all of them, and what each wrote to shared memory before it is visible to the others after.
__device__ __forceinline__ bool scale_writers_any(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.or.pred q, 1, 128, p;\nselp.u32 %0, 1, 0, q;\n}\n"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}

// The chunk of walk position u, or an empty one past the end: every role fetches the chunk of its
// next item while it works on the current one, so that the load's latency is not paid per item.
__device__ __forceinline__ Chunk chunk_at(const Chunk* chunks, int u, int tiles_m, int n_units) {
  Chunk c{0, 0, 0, 0};
  if (u < n_units) {
    const int4 v = __ldg(reinterpret_cast<const int4*>(chunks + u / tiles_m));
    c.expert = v.x; c.row0 = v.y; c.rows = v.z; c.pad = v.w;
  }
  return c;
}

// ---------------------------------------------------------------------------------------
// Host side: tensor maps
// ---------------------------------------------------------------------------------------
typedef CUresult (*MxEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline MxEncodeFn mx_encode_fn() {
  static MxEncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<MxEncodeFn>(sym);
  }
  return fn;
}

// [rows, k] values; packed 4-bit codes (k/2 bytes per row, box 128 x 128 values, expanded to one
// byte per value in shared memory) or bytes (box 128 bytes x box_rows); 128-byte swizzle.
static inline int mx_make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t k, bool four_bit, uint32_t box_rows) {
  MxEncodeFn fn = mx_encode_fn();
  if (!fn) return -1;
  const uint64_t row_bytes = four_bit ? k / 2 : k;
  if (reinterpret_cast<uintptr_t>(ptr) & 31 || k % 128 || row_bytes % 32) return -2;
  cuuint64_t dims[2] = {k, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, four_bit ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// linear1 weights [experts, 2 halves (gate, up), m rows, k values] as a 3-D map whose box takes the
// same 128-row tile of both halves: one request of 16 KB instead of two of 8 KB (the number of
// requests a CTA has in flight, not their size, limits what it can keep on its way from HBM).
static inline int mx_make_pair_map(CUtensorMap* map, const void* ptr, uint64_t experts, uint64_t m, uint64_t k) {
  MxEncodeFn fn = mx_encode_fn();
  if (!fn) return -1;
  if (reinterpret_cast<uintptr_t>(ptr) & 31 || k % 128 || (k / 2) % 32) return -2;
  cuuint64_t dims[3] = {k, m, 2 * experts};
  cuuint64_t strides[2] = {k / 2, m * (k / 2)};
  cuuint32_t box[3] = {128, 128, 2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace moe
