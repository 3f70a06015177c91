// Dense bf16 projections of the Kimi-K3 latent block on tcgen05 tensor cores:
//
//   y[t][n] = f( sum_k W[n][k] x[t][k] )        W bf16 [N, K] row-major, x bf16 [T, K], fp32 accumulation
//
// Orientation as in the decode GEMMs: 128 weight rows are the MMA's M side, up to 64 tokens the N side
// (`tcgen05.mma.kind::f16`, bf16 x bf16 -> fp32 in TMEM, K = 16 per instruction), so the weights stream
// once per tile of 64 tokens. There are no scales: a work item accumulates its whole K range in one TMEM
// accumulator (two for the gate/up pair) and the epilogue reads it once. A projection has only
// N / 128 = 28..56 weight tiles, too few for 148 SMs, so the contraction is cut in parts that are work
// items of their own: fp32 partial tiles in global memory; at the kernel's end the grid meets (one
// counter, bounded wait) and all CTAs share out the sums, every element's parts added in part order,
// and apply f.
//
//   mode 0: y = bf16(sum)
//   mode 1: y = situ(bf16(sum over W), bf16(sum over W2))     (gate and up rows of the shared experts)
//   mode 2: y = bf16(bf16(sum) + other[t][n])                 (routed + shared)
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 = epilogue (a thread owns
// an output channel). Every wait is bounded as in the other GEMM kernels.
// Reference: `W @ token` of megabench/tasks/kimi_layer.py:203,227-228 (bf16 linear, fp32 accumulation).
#include <algorithm>

#include "common.cuh"
#include "kernels.h"
#include "split_e4m3.cuh"

namespace moe {

constexpr int kDtThreads = 192;
constexpr int kDtTokens = 64;                 // token columns of a tile
constexpr int kDtWTile = 128 * 128;           // 128 rows x 64 bf16
constexpr int kDtXTile = kDtTokens * 128;
constexpr int kDtMaxStages = 8;
constexpr int kDtSmem = 232448;
constexpr int kDtTail = (2 * kDtMaxStages + 4) * 8 + 64;

template <bool DUAL>
struct DtCfg {
  static constexpr int kStageBytes = (DUAL ? 2 : 1) * kDtWTile + kDtXTile;
  static constexpr int kFit = (kDtSmem - 1024 - kDtTail) / kStageBytes;
  static constexpr int kStages = kFit < kDtMaxStages ? kFit : kDtMaxStages;
  static constexpr int kAccCols = (DUAL ? 2 : 1) * kDtTokens;
};

struct DtDev {
  int tiles_m, token_tiles, kblocks, ksplit, n, tokens, mode;
  const __nv_bfloat16* other;
  __nv_bfloat16* y;
  float* partial;          // ksplit > 1: [tile][part][matrix][token column][128 channels]
  int32_t* parts_done;     // ksplit > 1: two counters (CTAs whose parts are stored, CTAs that have left), zero on entry, left at zero
  int32_t* status;
};

// Instruction descriptor, kind::f16: bf16 x bf16 -> fp32, both operands K-major.
__device__ __forceinline__ uint32_t idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One output element from its complete fp32 sums (a: the projection, b: the up projection of the pair).
template <bool DUAL>
__device__ __forceinline__ __nv_bfloat16 dense_value(float a, float b, float other, int mode) {
  float v = bf16_round(a);
  if constexpr (DUAL) v = bf16_round(situ_f32(v, bf16_round(b)));
  else if (mode == 2) v = bf16_round(__fadd_rn(v, other));
  return __float2bfloat16_rn(v);
}

template <bool DUAL>
__global__ void __launch_bounds__(kDtThreads, 1)
dense_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_w2,
                const __grid_constant__ CUtensorMap tm_x, const DtDev p) {
  using C = DtCfg<DUAL>;
  constexpr int S = C::kStages;
  constexpr int MATS = DUAL ? 2 : 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stages = base;
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(base + S * C::kStageBytes);
  uint64_t* bar_empty = bar_full + kDtMaxStages;
  uint64_t* bar_tfull = bar_empty + kDtMaxStages;
  uint64_t* bar_tempty = bar_tfull + 2;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bar_tempty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile uint32_t* s_issued = reinterpret_cast<volatile uint32_t*>(s_tmem + 2);
  volatile uint32_t* s_consumed = reinterpret_cast<volatile uint32_t*>(s_tmem + 3);
  volatile uint32_t* s_committed = reinterpret_cast<volatile uint32_t*>(s_tmem + 4);
  volatile uint32_t* s_drained = reinterpret_cast<volatile uint32_t*>(s_tmem + 5);
  volatile int* s_last = reinterpret_cast<volatile int*>(s_tmem + 6);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(bar_full + s, 1); mbar_init(bar_empty + s, 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(bar_tfull + s, 1); mbar_init(bar_tempty + s, 128); }
    *s_abort = 0; *s_issued = 0; *s_consumed = 0; *s_committed = 0; *s_drained = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tm_w); prefetch_tmap(&tm_x);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  dependent_wait();
  dependents_may_launch();
  // work item u -> (weight tile, token tile, part of the contraction); the parts of a tile are neighbours
  const int n_units = p.tiles_m * p.token_tiles * p.ksplit;
  const int per = (p.kblocks + p.ksplit - 1) / p.ksplit;
  const int first = blockIdx.x, stride = gridDim.x;
  auto k_lo = [&](int part) { return part * per; };
  auto k_hi = [&](int part) { return min(p.kblocks, (part + 1) * per); };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    const uint64_t pol_w = policy_evict_first();
    const uint64_t pol_x = policy_evict_last();
    uint32_t it = 0, s = 0, ph = 0;
    bool ok = true;
    for (int u = first; ok && u < n_units; u += stride) {
      const int part = u % p.ksplit, tile = u / p.ksplit;
      const int tt = tile % p.token_tiles, mt = tile / p.token_tiles;
      const int cols = min(kDtTokens, p.tokens - tt * kDtTokens);
      const int n16 = (cols + 15) >> 4;
      const uint32_t bytes = MATS * kDtWTile + n16 * 2048;
      for (int kb = k_lo(part); kb < k_hi(part); ++kb, ++it) {
        if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + s, ph ^ 1u, s_abort))) {
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 41); *s_abort = 1; }
          ok = false;
          break;
        }
        if (elect_one()) {
          mbar_expect_tx(bar_full + s, bytes);
          uint8_t* st = stages + s * C::kStageBytes;
          tma_load_2d(st, &tm_w, kb * 64, mt * 128, bar_full + s, pol_w);
          if constexpr (DUAL) tma_load_2d(st + kDtWTile, &tm_w2, kb * 64, mt * 128, bar_full + s, pol_w);
          uint8_t* sx = st + MATS * kDtWTile;
          for (int j = 0; j < n16; ++j) tma_load_2d(sx + j * 2048, &tm_x, kb * 64, tt * kDtTokens + j * 16, bar_full + s, pol_x);
          *s_issued = it + 1;
        }
        __syncwarp();
        if (++s == S) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    uint32_t s = 0, ph = 0, item = 0, it = 0;
    bool ok = true;
    for (int u = first; ok && u < n_units; u += stride, ++item) {
      const int part = u % p.ksplit, tile = u / p.ksplit;
      const int tt = tile % p.token_tiles;
      const int cols = min(kDtTokens, p.tokens - tt * kDtTokens);
      const uint32_t idesc = idesc_bf16(128, ((cols + 15) >> 4) * 16);
      const uint32_t ab = item & 1u, aph = (item >> 1) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty + ab, aph ^ 1u, s_abort))) {
        if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 42); *s_abort = 1; }
        break;
      }
      const int lo = k_lo(part), hi = k_hi(part);
      for (int kb = lo; kb < hi; ++kb, ++it) {
        if (!__all_sync(0xffffffffu, mbar_wait(bar_full + s, ph, s_abort))) {
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 43); *s_abort = 1; }
          ok = false;
          break;
        }
        tc_fence_after();
        if (elect_one()) {
          *s_consumed = it + 1;
          const uint64_t desc0 = smem_desc_sw128(smem_u32(stages + s * C::kStageBytes));
          const uint32_t d0 = tmem + ab * C::kAccCols;
#pragma unroll
          for (uint32_t k4 = 0; k4 < 4; ++k4) {
            const uint32_t acc = (kb > lo || k4 > 0) ? 1u : 0u;    // the item's first MMA overwrites
            const uint64_t ad = desc0 + ((k4 * 32) >> 4);
            const uint64_t xd = ad + ((MATS * kDtWTile) >> 4);
            mma_bf16(d0, ad, xd, idesc, acc);
            if constexpr (DUAL) mma_bf16(d0 + kDtTokens, ad + (kDtWTile >> 4), xd, idesc, acc);
          }
          mma_commit(bar_empty + s);
          if (kb + 1 == hi) { mma_commit(bar_tfull + ab); *s_committed = item + 1; }
        }
        __syncwarp();
        if (++s == S) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue -----------------------------------
    const uint32_t quarter = warp & 3u;
    const int m = static_cast<int>(quarter) * 32 + lane;      // channel inside the tile
    const int tid = static_cast<int>(threadIdx.x) - 64;
    uint32_t item = 0;
    for (int u = first; u < n_units; u += stride, ++item) {
      const int part = u % p.ksplit, tile = u / p.ksplit;
      const int tt = tile % p.token_tiles, mt = tile / p.token_tiles;
      const int cols = min(kDtTokens, p.tokens - tt * kDtTokens);
      const int n16 = (cols + 15) >> 4;
      const uint32_t ab = item & 1u, aph = (item >> 1) & 1u;
      if (!mbar_wait(bar_tfull + ab, aph, s_abort)) {
        if (!*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 45); *s_abort = 1; }
        break;
      }
      tc_fence_after();
      const uint32_t t = tmem + ((quarter * 32u) << 16) + ab * C::kAccCols;
      float* mine = p.partial + (static_cast<size_t>(tile) * p.ksplit + part) * (MATS * kDtTokens * 128);
      const int channel = mt * 128 + m;
      auto finish = [&](int col, float a, float b) {      // one output element from its complete fp32 sums
        const size_t at = static_cast<size_t>(tt * kDtTokens + col) * p.n + channel;
        p.y[at] = dense_value<DUAL>(a, b, p.mode == 2 ? __bfloat162float(p.other[at]) : 0.f, p.mode);
      };
      for (int j = 0; j < n16; ++j) {
        uint32_t g[16], v[16];
        tmem_ld16(t + j * 16, g);
        if constexpr (DUAL) tmem_ld16(t + kDtTokens + j * 16, v);
        tmem_wait_ld();
        if (j == n16 - 1) {                        // every column of this accumulator is in registers
          tc_fence_before();
          mbar_arrive(bar_tempty + ab);
          if (tid == 0) *s_drained = item + 1;
        }
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const int col = j * 16 + c;
          if (col >= cols) break;                  // uniform across the CTA
          if (p.ksplit == 1) {
            finish(col, __uint_as_float(g[c]), DUAL ? __uint_as_float(v[c]) : 0.f);
          } else {
            __stcg(mine + col * 128 + m, __uint_as_float(g[c]));
            if constexpr (DUAL) __stcg(mine + (kDtTokens + col) * 128 + m, __uint_as_float(v[c]));
          }
        }
      }
    }
  }

  // ------------------------------ common exit ---------------------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*s_abort && threadIdx.x == 0) {
    for (uint32_t it = *s_consumed; it < *s_issued; ++it) mbar_wait(bar_full + it % S, (it / S) & 1u);
    for (uint32_t it = *s_drained; it < *s_committed; ++it) mbar_wait(bar_tfull + (it & 1u), (it >> 1) & 1u);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
  }
  if (p.ksplit > 1) {
    // The parts meet. Every CTA of this grid is resident (at most one per SM, and nothing it waits for
    // depends on a CTA that is not), so the grid can meet here: each CTA announces that its partial
    // tiles are stored, waits (bounded) for all the others, and then adds up its share of the outputs,
    // every element's parts in part order. (One CTA per tile adding 64 columns x 8 parts on its own took
    // longer than streaming the weights.)
    if (threadIdx.x == 0) {
      __threadfence();
      atomicAdd(p.parts_done, 1);
      if (!wait_counter(p.parts_done, static_cast<int>(gridDim.x))) report(p.status, MOE_ERR_DEVICE_TIMEOUT, 46);
      __threadfence();
    }
    __syncthreads();
    constexpr int kTileFloats = MATS * kDtTokens * 128;
    const long long elements = static_cast<long long>(p.tiles_m) * p.token_tiles * kDtTokens * 128;
    for (long long e = static_cast<long long>(blockIdx.x) * kDtThreads + threadIdx.x; e < elements;
         e += static_cast<long long>(gridDim.x) * kDtThreads) {
      const int m = static_cast<int>(e & 127), col = static_cast<int>((e >> 7) & (kDtTokens - 1));
      const int tile = static_cast<int>(e >> 13);          // 128 channels x 64 columns per tile
      const int tt = tile % p.token_tiles, mt = tile / p.token_tiles;
      const int token = tt * kDtTokens + col;
      if (token >= p.tokens) continue;
      const float* parts = p.partial + static_cast<size_t>(tile) * p.ksplit * kTileFloats + col * 128 + m;
      const size_t at = static_cast<size_t>(token) * p.n + mt * 128 + m;
      constexpr int kMaxParts = 8;
      float va[kMaxParts], vb[kMaxParts];
#pragma unroll
      for (int q = 0; q < kMaxParts; ++q) {      // all loads first, then the sums in part order
        const float* src = parts + static_cast<size_t>(q < p.ksplit ? q : 0) * kTileFloats;
        va[q] = __ldcg(src);
        vb[q] = DUAL ? __ldcg(src + kDtTokens * 128) : 0.f;
      }
      const float other = p.mode == 2 ? __bfloat162float(p.other[at]) : 0.f;
      float a = 0.f, b = 0.f;
#pragma unroll
      for (int q = 0; q < kMaxParts; ++q) {
        if (q < p.ksplit) {
          a = __fadd_rn(a, va[q]);
          if constexpr (DUAL) b = __fadd_rn(b, vb[q]);
        }
      }
      p.y[at] = dense_value<DUAL>(a, b, other, p.mode);
    }
    // the last CTA to leave puts the two counters back to zero for the next launch
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(p.parts_done + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      p.parts_done[0] = 0;
      p.parts_done[1] = 0;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*DtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// bf16 matrix [rows, k], box = [box_rows, 64 values = 128 bytes], 128-byte swizzle, zero fill outside.
static int dt_make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t k, uint32_t box_rows) {
  static DtEncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<DtEncodeFn>(sym);
  }
  if (!fn) return -1;
  if (reinterpret_cast<uintptr_t>(ptr) & 15 || k % 64) return -2;
  cuuint64_t dims[2] = {k, rows};
  cuuint64_t strides[1] = {k * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

DenseTcPlan dense_tc_plan(int tokens, int n, int k) {
  DenseTcPlan plan{};
  if (tokens < 1 || n % 128 || k % 64) return plan;
  plan.tiles = (n / 128) * ((tokens + kDtTokens - 1) / kDtTokens);
  const int kblocks = k / 64;
  // enough parts for two work items per SM at one tile of tokens, each at least eight K blocks deep, at
  // most eight; from the matrix alone, never from the batch, so that a token's sums are added in the same
  // order whatever else is in flight
  int ksplit = (2 * 148 + n / 128 - 1) / (n / 128);
  ksplit = std::max(1, std::min({ksplit, 8, kblocks / 8}));
  const int per = (kblocks + ksplit - 1) / ksplit;
  ksplit = (kblocks + per - 1) / per;                 // no empty part
  plan.ksplit = ksplit;
  plan.partial_bytes = ksplit > 1 ? static_cast<uint64_t>(plan.tiles) * ksplit * 2 * kDtTokens * 128 * 4 : 0;
  return plan;
}

template <bool DUAL>
static cudaError_t dt_launch(const DtDev& dev, const CUtensorMap* maps, int grid, cudaStream_t stream) {
  using C = DtCfg<DUAL>;
  static_assert(C::kStages >= 3, "shared memory of one CTA");
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    cudaError_t e = cudaFuncSetAttribute(dense_tc_kernel<DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDtSmem);
    if (e != cudaSuccess) return e;
    if (device >= 0 && device < 64) configured[device] = true;
  }
  constexpr int smem = 1024 + C::kStages * C::kStageBytes + kDtTail;
  return launch_dependent(dense_tc_kernel<DUAL>, dim3(grid), dim3(kDtThreads), smem, stream, maps[0], maps[1], maps[2], dev);
}

cudaError_t launch_dense_tc(int mode, const __nv_bfloat16* w, const __nv_bfloat16* w2, const __nv_bfloat16* x, int tokens, int n,
                            int k, const __nv_bfloat16* other, __nv_bfloat16* y, float* partial, int32_t* parts_done,
                            int32_t* status, cudaStream_t stream, int* launches, int* driver_error) {
  const DenseTcPlan plan = dense_tc_plan(tokens, n, k);
  if (plan.tiles == 0 || mode < 0 || mode > 2 || (mode == 1) != (w2 != nullptr) || (mode == 2) != (other != nullptr) ||
      (plan.ksplit > 1 && (!partial || !parts_done)))
    return cudaErrorInvalidValue;
  CUtensorMap maps[3];
  int rc = dt_make_map(&maps[0], w, n, k, 128);
  rc = rc ? rc : dt_make_map(&maps[1], mode == 1 ? w2 : w, n, k, 128);
  rc = rc ? rc : dt_make_map(&maps[2], x, tokens, k, 16);        // token rows move in boxes of 16; rows past the batch read as zero
  if (rc) {
    if (driver_error) *driver_error = rc;
    return cudaErrorUnknown;
  }
  DtDev dev{n / 128, (tokens + kDtTokens - 1) / kDtTokens, k / 64, plan.ksplit, n, tokens, mode, other, y, partial, parts_done, status};
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int grid = std::max(1, std::min(sms, plan.tiles * plan.ksplit));
  const cudaError_t e = mode == 1 ? dt_launch<true>(dev, maps, grid, stream) : dt_launch<false>(dev, maps, grid, stream);
  if (launches) *launches += 1;
  return e;
}

}  // namespace moe
