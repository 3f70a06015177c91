// What the tensor-core grouped GEMM kernels share: the walk over the work list, the queue that hands
// the CTA's work items from the producer warp to the other roles, and the host side's tensor maps.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace moe {

// Optional probe (compile with -DMOE_GEMM_PROBE): cycles each role spends waiting, summed over the
// CTAs into the spare status words in units of 256 cycles: [2] producer for a free stage, [3] MMA
// for a free accumulator, [4] MMA for data, [5] epilogue for an accumulator, [6] epilogue for
// scales, [7] lifetime of the CTA. MOE_GEMM_PROBE=1 records the gate/up GEMM, =2 the down GEMM.
// With -DMOE_GEMM_PROBE_EPI besides, words [2], [3], [4] and [6] hold the first epilogue thread's
// cycles instead: reading the accumulators, releasing them, folding them, and the item's closing
// epilogue (activation, requantisation, stores). Off by default: the words stay zero.
#ifdef MOE_GEMM_PROBE
#define PROBE_DECL(name) long long name = 0
#define PROBE_START(t) const long long t = clock64()
#define PROBE_ADD(name, t) name += clock64() - t
#define PROBE_FLUSH(status, slot, name) \
  if (DUAL == (MOE_GEMM_PROBE == 1)) atomicAdd((status) + (slot), static_cast<int>((name) >> 8))
#ifdef MOE_GEMM_PROBE_EPI
#define PROBE_FLUSH_ROLE(status, slot, name)
#define PROBE_FLUSH_EPI(status, slot, name) PROBE_FLUSH(status, slot, name)
#else
#define PROBE_FLUSH_ROLE(status, slot, name) PROBE_FLUSH(status, slot, name)
#define PROBE_FLUSH_EPI(status, slot, name)
#endif
#else
#define PROBE_DECL(name)
#define PROBE_START(t)
#define PROBE_ADD(name, t)
#define PROBE_FLUSH(status, slot, name)
#define PROBE_FLUSH_ROLE(status, slot, name)
#define PROBE_FLUSH_EPI(status, slot, name)
#endif

constexpr int kQueue = 4;             // work items the producer may run ahead of the slowest role

// Position u of the walk -> work item. The walk goes expert by expert; inside an expert with
// several row chunks it goes channel tile by channel tile with the chunks innermost, so that the
// CTAs running at the same time read the same weight tile (once from HBM, then from L2) instead
// of returning to it one pass over the expert's weights later. Returns the chunk and rewrites u
// to chunk_index * tiles_m + channel_tile; u < 0 gives an empty chunk.
__device__ __forceinline__ Chunk load_chunk(const Chunk* chunks, int& u, int tiles_m) {
  Chunk c{0, 0, 0, 0};
  if (u >= 0) {
    const int at = u / tiles_m;
    int4 v = __ldg(reinterpret_cast<const int4*>(chunks + at));
    const int nc = v.w >> 16;
    if (nc > 1) {
      const int first = at - (v.w & 0xffff);
      const int local = u - first * tiles_m;
      const int mt = local / nc, which = first + local % nc;
      v = __ldg(reinterpret_cast<const int4*>(chunks + which));
      u = which * tiles_m + mt;
    }
    c.expert = v.x; c.row0 = v.y; c.rows = v.z; c.pad = v.w;
  }
  return c;
}

// The CTA's i-th work item as published by the producer warp: {u, expert, row0, rows}, u < 0 after
// the last one. Every consumer thread takes every item and arrives on the slot's empty barrier.
__device__ __forceinline__ bool take_item(const int4* queue, uint64_t* bar_qfull, uint64_t* bar_qempty, uint32_t i,
                                          const volatile int* abort, int& u, Chunk& ch) {
  const uint32_t q = i % kQueue;
  if (!mbar_wait(bar_qfull + q, (i / kQueue) & 1u, abort)) return false;
  const int4 v = queue[q];
  u = v.x; ch.expert = v.y; ch.row0 = v.z; ch.rows = v.w & 0xff; ch.pad = v.w >> 8;   // pad: part of a split contraction
  mbar_arrive(bar_qempty + q);
  return true;
}

// K blocks [lo, hi) of part `part` when the contraction of `kblocks` blocks is cut in `parts`.
__device__ __forceinline__ void k_range(int kblocks, int parts, int part, int& lo, int& hi) {
  const int per = (kblocks + parts - 1) / parts;
  lo = part * per;
  hi = min(kblocks, lo + per);
}

// K blocks of the step that starts at `kb` in an item covering [.., hi): two for the down
// projection unless the item ends or a part of a split contraction ends after the first.
template <bool DUAL>
__device__ __forceinline__ int step_blocks(int kb, int hi, int part_len) {
  if constexpr (DUAL) return 1;
  return (kb + 1 < hi && (kb + 1) % part_len != 0) ? 2 : 1;
}

// ---------------------------------------------------------------------------------------
// Host side: tensor maps.
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D byte matrix [rows, cols], box = [box_rows, 128 bytes], 128-byte swizzle, zero fill outside.
static inline int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  if (reinterpret_cast<uintptr_t>(ptr) & 15 || cols % 16) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

static inline int gemm_sm_count() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

}  // namespace moe
