// Grouped GEMM in the MegaMoE-native formats for experts with many rows: the tokens are the MMA's M side.
//
//   D[t, n] = sum over 32-wide K blocks b of  2^(sx[t,b]-127) * 2^(sw[n,b]-127) * sum_k X[t,k] * W[n,k]
//
// gemm_mx.cu puts 128 weight rows on M and at most 64 tokens on N; the reference's own MegaMoE cases
// bring 64 to 512 rows per expert (megabench/cases.py:380-388), where a 64-wide N leaves the tensor
// pipe reading operands most of the time and every weight tile is fetched from the L2 once per 64
// rows. Here a tile is 128 token rows (M) x 256 weight rows (N): the gate and the up rows of a
// 128-channel tile of linear1, or 256 channels of linear2; `tcgen05.mma.kind::mxf8f6f4.block_scale`
// with A = E4M3, B = E2M1, the whole contraction in one TMEM accumulator of 256 columns.
//
// TMEM: columns 0..255 the accumulator, 256..511 the scale factors (four groups of four K blocks,
// 16 columns per K block: 8 for the 256 weight rows, 4 for the 128 token rows; row r in lane r % 32 of
// every lane quarter, column r / 32, byte = 32-wide K block inside the 128-wide one). One accumulator
// means the MMAs of an item wait until the epilogue has read the previous one; an item is 56 K blocks
// of 512 tensor-pipe cycles, the read a few thousand.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 = scale writers (as in
// gemm_mx.cu), warps 6-13 = epilogue: a thread owns a token row and 64 (linear1: gate and up) or 128
// (linear2) of the tile's columns. A thread's 32 consecutive channels are exactly one E8M0 scale
// block, so the requantisation needs no exchange between threads, and a row's bytes leave as 16-byte
// stores. Every wait is bounded, as in gemm_mx.cu.
//
// Arithmetic: that of gemm_mx.cu, element by element (the MMA sums the same products in the same K
// order whichever operand sits on M; tests/test_gpu_megamoe.py compares the two kernels bit for bit).
// Reference: megabench/tasks/megamoe.py:131-150, :116-128, megabench/tasks/quantization.py:62-84.
#include <algorithm>

#include "common.cuh"
#include "gemm_mx_common.cuh"
#include "kernels.h"

namespace moe {

constexpr int kMxwThreads = 448;
constexpr int kMxwEpiThreads = 256;
constexpr int kMxwTile = 16384;                      // 128 rows x 128 bytes in shared memory
constexpr int kMxwStageBytes = 3 * kMxwTile;         // token tile, two weight tiles of one K block
constexpr int kMxwSfSlotBytes = 3 * 2048;            // a group's scale bytes: 16 per row of the two weight tiles, then of the tokens
constexpr int kMxwMaxStages = 4;
constexpr int kMxwTailBytes = (2 * kMxwMaxStages + 2 + 2 * kMxSfSlots) * 8 + 64;
constexpr int kMxwStages = (kMxSmem - 1024 - kMxwTailBytes - kMxSfRing * kMxwSfSlotBytes) / kMxwStageBytes < kMxwMaxStages
                               ? (kMxSmem - 1024 - kMxwTailBytes - kMxSfRing * kMxwSfSlotBytes) / kMxwStageBytes
                               : kMxwMaxStages;
constexpr int kMxwSfBase = 256;                      // TMEM column of the first scale factor
static_assert(kMxwSfBase + kMxSfSlots * kMxSfGroup * kMxSfCols <= 512, "TMEM columns");
static_assert(kMxwStages >= 3, "shared memory of one CTA");

struct MxWideDev {
  const Chunk* chunks;
  const int32_t* n_chunks;
  int tiles, kblocks, m;      // tiles: m / 128 (linear1) or m / 256 (linear2)
  int rows_per_expert;        // rows of the weight matrix one expert owns (2I for linear1, H for linear2)
  int second_offset;          // rows between a row of the first weight tile and its partner in the second (I, or 128)
  const uint8_t* w_scales;    // [experts * rows_per_expert, K/32]
  const uint8_t* x_scales;    // [rows, K/32]
  uint8_t* aq;                // linear1: e4m3 [rows, m]
  uint8_t* as;                // linear1: E8M0 [rows, m/32]
  __nv_bfloat16* out;         // linear2: bf16 rows [*, m] at row_dest
  const int32_t* row_dest;
  const float* slot_weight;   // linear1: routing weight of slot row_dest[row] (NULL = 1)
  float limit;                // linear1: clamp, 0 = none
  int32_t* status;
};

// Instruction descriptor, kind::mxf8f6f4 with block scales: A = E4M3, B = E2M1, both K-major, E8M0
// scales, M = 128, N = 256; `sf` picks the byte (32-wide K block) of the scale columns for both sides.
__device__ __forceinline__ uint32_t idesc_mx_wide(uint32_t sf) {
  return (sf << 4) | (0u << 7) | (5u << 10) | (static_cast<uint32_t>(256 >> 3) << 17) | (1u << 23) |
         (static_cast<uint32_t>(128 >> 4) << 24) | (sf << 29);
}

__device__ __forceinline__ void tmem_ld32_mx(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

template <bool DUAL>
__global__ void __launch_bounds__(kMxwThreads, 1)
mx_gemm_wide_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    const __grid_constant__ CUtensorMap tm_xw, const MxWideDev p) {
  constexpr int S = kMxwStages;
  extern __shared__ uint8_t smem_raw[];
  const int KB = p.kblocks;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stages = base;
  uint8_t* sf_ring = base + S * kMxwStageBytes;                      // [kMxSfRing][kMxwSfSlotBytes]
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(sf_ring + kMxSfRing * kMxwSfSlotBytes);
  uint64_t* bar_empty = bar_full + kMxwMaxStages;
  uint64_t* bar_tfull = bar_empty + kMxwMaxStages;
  uint64_t* bar_tempty = bar_tfull + 1;
  uint64_t* bar_sffull = bar_tempty + 1;           // a group's scale factors are in TMEM
  uint64_t* bar_sfempty = bar_sffull + kMxSfSlots; // the MMAs that read a group are done
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bar_sfempty + kMxSfSlots);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile uint32_t* s_issued = reinterpret_cast<volatile uint32_t*>(s_tmem + 2);    // K blocks whose TMA was issued
  volatile uint32_t* s_consumed = reinterpret_cast<volatile uint32_t*>(s_tmem + 3);  // K blocks whose data arrived
  volatile uint32_t* s_committed = reinterpret_cast<volatile uint32_t*>(s_tmem + 4); // accumulators committed
  volatile uint32_t* s_drained = reinterpret_cast<volatile uint32_t*>(s_tmem + 5);   // accumulators read

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(bar_full + s, 1); mbar_init(bar_empty + s, 1); }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tempty, kMxwEpiThreads);
    for (int s = 0; s < kMxSfSlots; ++s) { mbar_init(bar_sffull + s, 4); mbar_init(bar_sfempty + s, 1); }   // four scale warps
    *s_abort = 0; *s_issued = 0; *s_consumed = 0; *s_committed = 0; *s_drained = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tm_w); prefetch_tmap(&tm_x); prefetch_tmap(&tm_xw);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  dependent_wait();
  dependents_may_launch();
  const int n_units = *p.n_chunks * p.tiles;
  const int first = blockIdx.x, stride = gridDim.x;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    const uint64_t pol_w = policy_evict_normal();      // read again within microseconds by the CTAs of the expert's other chunks
    const uint64_t pol_x = policy_evict_last();
    uint32_t it = 0, s = 0, ph = 0;
    bool ok = true;
    Chunk ahead = chunk_at(p.chunks, first, p.tiles, n_units);
    for (int u = first; ok && u < n_units; u += stride) {
      const Chunk ch = ahead;
      ahead = chunk_at(p.chunks, u + stride, p.tiles, n_units);
      const int tile = u % p.tiles;
      const int n16 = (ch.rows + 15) >> 4;
      const uint32_t bytes = 2 * 8192 + n16 * 2048;      // the weight tiles count their packed bytes
      for (int kb = 0; kb < KB; ++kb, ++it) {
        if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + s, ph ^ 1u, s_abort))) {
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 31); *s_abort = 1; }
          ok = false;
          break;
        }
        if (elect_one()) {
          mbar_expect_tx(bar_full + s, bytes);
          uint8_t* st = stages + s * kMxwStageBytes;
          const int kx = kb * 128;
          if constexpr (DUAL)       // the gate tile, then the up tile of the same rows: one request
            tma_load_3d(st + kMxwTile, &tm_w, kx, tile * 128, 2 * ch.expert, bar_full + s, pol_w);
          else                      // 256 consecutive rows
            tma_load_2d(st + kMxwTile, &tm_w, kx, ch.expert * p.rows_per_expert + tile * 256, bar_full + s, pol_w);
          if (n16 == 8) tma_load_2d(st, &tm_xw, kx, ch.row0, bar_full + s, pol_x);      // a full tile: one request
          else for (int j = 0; j < n16; ++j) tma_load_2d(st + j * 2048, &tm_x, kx, ch.row0 + j * 16, bar_full + s, pol_x);
          *s_issued = it + 1;
        }
        __syncwarp();
        if (++s == S) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    uint32_t s = 0, ph = 0, item = 0, it = 0, gi = 0;      // gi: scale-factor groups so far
    bool ok = true;
    const uint32_t idesc4[4] = {idesc_mx_wide(0), idesc_mx_wide(1), idesc_mx_wide(2), idesc_mx_wide(3)};
    for (int u = first; ok && u < n_units; u += stride, ++item) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty, (item & 1u) ^ 1u, s_abort))) {
        if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 32); *s_abort = 1; }
        break;
      }
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const uint32_t slot = gi % kMxSfSlots, in_group = kb % kMxSfGroup;
        bool got = mbar_wait(bar_full + s, ph, s_abort);
        if (in_group == 0) got = got && mbar_wait(bar_sffull + slot, (gi / kMxSfSlots) & 1u, s_abort);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 33); *s_abort = 1; }
          ok = false;
          break;
        }
        tc_fence_after();
        const bool last = kb + 1 == KB;
        const bool group_done = in_group + 1 == kMxSfGroup || last;
        if (elect_one()) {
          *s_consumed = it + 1;
          const uint64_t desc0 = smem_desc_sw128(smem_u32(stages + s * kMxwStageBytes));     // the token tile
          const uint32_t sf = tmem + kMxwSfBase + (slot * kMxSfGroup + in_group) * kMxSfCols;
#pragma unroll
          for (uint32_t k4 = 0; k4 < 4; ++k4) {
            const uint32_t acc = (kb > 0 || k4 > 0) ? 1u : 0u;   // the item's first MMA overwrites
            const uint64_t ad = desc0 + ((k4 * 32) >> 4);
            mma_mx(tmem, ad, ad + (kMxwTile >> 4), idesc4[k4], sf + 8, sf, acc);      // scales: tokens at +8, weights at +0..7
          }
          mma_commit(bar_empty + s);                 // the stage may be refilled once these MMAs are done
          if (group_done) mma_commit(bar_sfempty + slot);   // and the group's scale columns rewritten
          if (last) { mma_commit(bar_tfull); *s_committed = item + 1; }
        }
        __syncwarp();
        if (group_done) ++gi;
        if (++s == S) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------ scale writers ------------------------------
    // As in gemm_mx.cu: a group = four K blocks = 16 scale bytes per row; thread t copies the bytes of
    // row t of the first weight tile, of the second, and of token row t into a ring in shared memory
    // (cp.async, kMxSfAhead groups ahead across work items); then warp w fills lane quarter w % 4 of the
    // group's TMEM columns.
    const int t = static_cast<int>(threadIdx.x) - 64;      // 0..127
    const uint32_t quarter = warp & 3u;
    const int KS = KB * 4;                         // scale bytes per row
    const bool vec = (KS % 16) == 0;
    const int groups = (KB + 3) / 4;
    int iu = first, ig = 0;
    uint32_t issued = 0;
    Chunk ich = iu < n_units ? p.chunks[iu / p.tiles] : Chunk{0, 0, 0, 0};
    auto issue = [&]() {
      if (iu < n_units) {
        uint8_t* slot = sf_ring + (issued % kMxSfRing) * kMxwSfSlotBytes;
        const size_t wrow = static_cast<size_t>(ich.expert) * p.rows_per_expert + (iu % p.tiles) * (DUAL ? 128 : 256) + t;
        copy_scale_group(slot + t * 16, p.w_scales + wrow * KS, ig, KB, vec);
        copy_scale_group(slot + 2048 + t * 16, p.w_scales + (wrow + p.second_offset) * KS, ig, KB, vec);
        uint8_t* dst = slot + 4096 + t * 16;
        if (t < ich.rows) copy_scale_group(dst, p.x_scales + static_cast<size_t>(ich.row0 + t) * KS, ig, KB, vec);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);   // past the chunk: scale 1, results unused
        if (++ig == groups) {
          ig = 0;
          iu += stride;
          if (iu < n_units) ich = p.chunks[iu / p.tiles];
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");   // an empty group past the end keeps the count uniform
      ++issued;
    };
    for (int i = 0; i < kMxSfAhead; ++i) issue();
    uint32_t gi = 0;                               // groups stored so far
    bool ok = true;
    for (int u = first; ok && u < n_units; u += stride) {
      for (int g = 0; g < groups; ++g, ++gi) {
        issue();
        asm volatile("cp.async.wait_group %0;" ::"n"(kMxSfAhead) : "memory");   // this thread's copies of group gi have landed
        const uint32_t slot = gi % kMxSfSlots;
        const bool late = !mbar_wait(bar_sfempty + slot, ((gi / kMxSfSlots) & 1u) ^ 1u, s_abort);
        if (scale_writers_any(late)) {
          if (t == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 34); *s_abort = 1; }
          ok = false;
          break;
        }
        tc_fence_after();
        const uint8_t* src = sf_ring + (gi % kMxSfRing) * kMxwSfSlotBytes;
        uint4 a[4], b[4], x[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          a[c] = *reinterpret_cast<const uint4*>(src + (32 * c + lane) * 16);
          b[c] = *reinterpret_cast<const uint4*>(src + 2048 + (32 * c + lane) * 16);
          x[c] = *reinterpret_cast<const uint4*>(src + 4096 + (32 * c + lane) * 16);
        }
        const uint32_t t0 = tmem + ((quarter * 32u) << 16) + kMxwSfBase + slot * kMxSfGroup * kMxSfCols;
#define MX_WORD(v, j) ((j) == 0 ? (v).x : (j) == 1 ? (v).y : (j) == 2 ? (v).z : (v).w)
#pragma unroll
        for (int j = 0; j < 4; ++j) {              // a ragged last group stores spare columns nobody reads
          const uint32_t tj = t0 + j * kMxSfCols;
          tmem_st4(tj, MX_WORD(a[0], j), MX_WORD(a[1], j), MX_WORD(a[2], j), MX_WORD(a[3], j));
          tmem_st4(tj + 4, MX_WORD(b[0], j), MX_WORD(b[1], j), MX_WORD(b[2], j), MX_WORD(b[3], j));
          tmem_st4(tj + 8, MX_WORD(x[0], j), MX_WORD(x[1], j), MX_WORD(x[2], j), MX_WORD(x[3], j));
        }
#undef MX_WORD
        tmem_wait_st();
        tc_fence_before();
        if (lane == 0) mbar_arrive(bar_sffull + slot);
        __syncwarp();
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else {
    // ------------------------------ epilogue -----------------------------------
    const uint32_t quarter = warp & 3u;
    const int half = (warp - 6) >> 2;
    const int t = static_cast<int>(quarter) * 32 + lane;      // token row inside the tile
    uint32_t item = 0;
    Chunk ahead = chunk_at(p.chunks, first, p.tiles, n_units);
    for (int u = first; u < n_units; u += stride, ++item) {
      const Chunk ch = ahead;
      ahead = chunk_at(p.chunks, u + stride, p.tiles, n_units);
      const int tile = u % p.tiles;
      const bool valid = t < ch.rows;
      const size_t row = static_cast<size_t>(ch.row0 + (valid ? t : 0));
      // destination slot and routing weight of this thread's row, fetched while the MMAs still run
      const int dest = valid ? (p.row_dest ? p.row_dest[row] : static_cast<int>(row)) : 0;
      const float weight = (DUAL && p.slot_weight && valid) ? p.slot_weight[dest] : 1.f;
      if (!mbar_wait(bar_tfull, item & 1u, s_abort)) {
        if (!*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 35); *s_abort = 1; }
        break;
      }
      tc_fence_after();
      const uint32_t tl = tmem + ((quarter * 32u) << 16);
      if constexpr (DUAL) {
        // gate columns [64 half, +64) and the up columns of the same channels, 32 (= one scale block) at a time
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t g[32], v[32];
          tmem_ld32_mx(tl + half * 64 + c * 32, g);
          tmem_ld32_mx(tl + 128 + half * 64 + c * 32, v);
          tmem_wait_ld();
          if (c == 1) {                            // every column this thread reads is in registers
            tc_fence_before();
            mbar_arrive(bar_tempty);
            if (threadIdx.x == 6 * 32) *s_drained = item + 1;
          }
          if (valid) {
            // megabench/tasks/megamoe.py:116-122: bf16 GEMM outputs, clamp, fp32 SwiGLU, routing weight
            float act[32];
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float gate = bf16_round(__uint_as_float(g[i]));
              float up = bf16_round(__uint_as_float(v[i]));
              if (p.limit > 0.f) {
                gate = fminf(gate, p.limit);
                up = fminf(fmaxf(up, -p.limit), p.limit);
              }
              float a = silu_times(gate, up);
              if (p.slot_weight) a = __fmul_rn(a, weight);
              act[i] = a;
              amax = fmaxf(amax, fabsf(a));
            }
            // megabench/tasks/quantization.py:62-84: one power-of-two scale for the 32 channels
            const int exponent = max((__float_as_int(amax) + (0x7FFFFF - 0x600000)) >> 23, 105 + 8) - 8;
            const float inverse = __int_as_float((254 - exponent) << 23);
            const int ch0 = tile * 128 + half * 64 + c * 32;
            uint8_t* dst = p.aq + row * p.m + ch0;
#pragma unroll
            for (int i = 0; i < 32; i += 16) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(act[i + 4 * j], inverse), __fmul_rn(act[i + 4 * j + 1], inverse)), __NV_SATFINITE, __NV_E4M3);
                const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(act[i + 4 * j + 2], inverse), __fmul_rn(act[i + 4 * j + 3], inverse)), __NV_SATFINITE, __NV_E4M3);
                w[j] = lo | hi << 16;
              }
              *reinterpret_cast<uint4*>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            p.as[row * (p.m / 32) + ch0 / 32] = static_cast<uint8_t>(exponent);
          }
        }
      } else {
        // columns [128 half, +128): one bf16 rounding of the fp32 sum (megabench/tasks/megamoe.py:149)
        __nv_bfloat16* dst = p.out + static_cast<size_t>(dest) * p.m + tile * 256 + half * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32];
          tmem_ld32_mx(tl + half * 128 + c * 32, g);
          tmem_wait_ld();
          if (c == 3) {
            tc_fence_before();
            mbar_arrive(bar_tempty);
            if (threadIdx.x == 6 * 32) *s_drained = item + 1;
          }
          if (valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(g[i + 2 * j]), __uint_as_float(g[i + 2 * j + 1]));
                w[j] = *reinterpret_cast<const uint32_t*>(&pair);
              }
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = make_uint4(w[0], w[1], w[2], w[3]);
            }
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
    // Give copies and MMAs that were issued but never consumed a bounded chance to land.
    for (uint32_t it = *s_consumed; it < *s_issued; ++it) mbar_wait(bar_full + it % S, (it / S) & 1u);
    for (uint32_t it = *s_drained; it < *s_committed; ++it) mbar_wait(bar_tfull, it & 1u);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
template <bool DUAL>
static cudaError_t mx_wide_launch_typed(const MxWideDev& dev, const CUtensorMap* maps, int grid, cudaStream_t stream) {
  static bool configured[64] = {};      // the attribute belongs to the device the call runs on
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    cudaError_t e = cudaFuncSetAttribute(mx_gemm_wide_kernel<DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMxSmem);
    if (e != cudaSuccess) return e;
    if (device >= 0 && device < 64) configured[device] = true;
  }
  constexpr int smem = 1024 + kMxwStages * kMxwStageBytes + kMxSfRing * kMxwSfSlotBytes + kMxwTailBytes;
  static_assert(smem <= kMxSmem, "shared memory of one CTA");
  return launch_dependent(mx_gemm_wide_kernel<DUAL>, dim3(grid), dim3(kMxwThreads), smem, stream, maps[0], maps[1], maps[2], dev);
}

cudaError_t launch_gemm_mx_wide(const MxGemmArgs& a, cudaStream_t stream, int* launches, int* driver_error) {
  // gate and up rows in one tensor, plain rows (no (hi, lo) pairs), whole 256-channel tiles of linear2
  if (a.tile != 128 || a.k % 128 || a.m % 128 || a.n_experts < 1 || a.w_blocks_b || a.w_scales_b || a.pairs || a.activation != 0 ||
      (!a.dual && a.m % 256))
    return cudaErrorInvalidValue;
  const int rows_per_expert = a.dual ? 2 * a.m : a.m;
  CUtensorMap maps[3];
  int rc = a.dual ? mx_make_pair_map(&maps[0], a.w_blocks, a.n_experts, a.m, a.k)
                  : mx_make_map(&maps[0], a.w_blocks, static_cast<uint64_t>(a.n_experts) * rows_per_expert, a.k, true, 256);
  rc = rc ? rc : mx_make_map(&maps[1], a.act, a.total_rows, a.k, false, 16);      // token rows of a ragged chunk move in boxes of 16,
  rc = rc ? rc : mx_make_map(&maps[2], a.act, a.total_rows, a.k, false, 128);     // a full tile's in one of 128
  if (rc) {
    if (driver_error) *driver_error = rc;
    return cudaErrorUnknown;
  }
  const int tiles = a.dual ? a.m / 128 : a.m / 256;
  MxWideDev dev{a.chunks, a.n_chunks, tiles, a.k / 128, a.m, rows_per_expert, a.dual ? a.m : 128, a.w_scales, a.act_scales,
                a.aq, a.as, a.out, a.row_dest, a.slot_weight, a.limit, a.status};
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  // max_units counts chunks * (m / 128)
  const long long units = a.dual ? a.max_units : (static_cast<long long>(a.max_units) + 1) / 2;
  const int grid = static_cast<int>(std::max(1ll, std::min(static_cast<long long>(sms), units)));
  const cudaError_t e = a.dual ? mx_wide_launch_typed<true>(dev, maps, grid, stream) : mx_wide_launch_typed<false>(dev, maps, grid, stream);
  if (launches) *launches += 1;
  return e;
}

}  // namespace moe
