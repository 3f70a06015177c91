// Grouped FP8 GEMM for experts with many rows: the tokens are the MMA's M side.
//
// The decode kernel (gemm_tc.cu) puts the weights on M and 16 to 64 tokens on N, so that a small
// batch streams every weight byte once. With a hundred and more rows per expert that orientation
// pays three times over: an epilogue thread owns a channel and needs the scale of every token column
// of every K block (broadcast loads that saturate the shared-memory pipe), a 64-wide N leaves the
// tensor pipe reading operands most of the time, and the results leave transposed. Here a tile is
//
//   128 token rows (M)  x  128 gate + 128 up channels (N = 256, one MMA)       gate/up GEMM
//   128 token rows (M)  x  128 channels, two K blocks per step (2 x N = 128)    down GEMM
//
// so an epilogue thread owns one token row: one token scale and one or two weight scales per K block,
// read from global memory a step ahead, no scale table at all; the row's 128 channels make exactly
// one requantisation group, and a thread stores 64 consecutive output channels of its row.
//
//   D[t, n] = sum_k X[t, k] * W[n, k]        e4m3 x e4m3 -> fp32 in TMEM, kind::f8f6f4
//
// Arithmetic: identical to the decode kernel, element by element: every 128-deep K block is
// accumulated into a fresh TMEM accumulator and folded as acc += D * (w_scale * x_scale) in K order,
// a long down contraction is summed in the same parts (down_ksplit), so a token's result does not
// depend on which of the two kernels its expert's rows meet.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-3 idle (they complete the
// warp group that gives its registers away), warps 4-11 = epilogue: warp w reads TMEM lanes
// 32*(w%4).., the first four warps take columns 0-63 of each 128-column accumulator, the last four
// columns 64-127. An epilogue thread keeps 128 fp32 sums, which is why the epilogue warp groups raise
// their register allowance (setmaxnreg) from what the other warp groups release. The gate/up kernel has
// a fourth warp group, warps 12-15, that closes the work items (SwiGLU + requantisation) from a tile of
// bf16 (gate, up) pairs the epilogue warps leave in shared memory, so that those go straight on to the
// next item's K blocks and the accumulators keep coming back to the MMAs.
//
// Every wait is bounded, as in the decode kernel: on expiry the role records
// MOE_ERR_DEVICE_TIMEOUT, raises the CTA's abort flag, and all roles fall through to the common exit.
//
// Reference arithmetic: megabench/tasks/megamoe.py:146-149 (grouped expert GEMMs), :116-128
// (SwiGLU + requantisation), megabench/tasks/frontier.py:180-186 (FP8 linear).
#include <algorithm>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_items.cuh"
#include "kernels.h"

namespace moe {

constexpr int kWideThreads = 384;
constexpr int kWideEpiThreads = 256;
#ifndef MOE_WIDE_CLOSERS
#define MOE_WIDE_CLOSERS 1               // gate/up: warps 2-3 close the work items (SwiGLU + requantisation), see below
#endif
constexpr int kWideServiceRegs = 40;     // registers per thread the first warp group keeps
constexpr int kWideEpiRegs = 232;        // ... and the epilogue warp groups rise to: 128*40 + 256*232 = 384*168
// gate/up with a fourth warp group that closes the items: 128*40 + 256*200 + 128*72 = 512*128
constexpr int kWideCloserRegs = 72;
constexpr int kWideEpiRegsWithClosers = 200;
constexpr int kWideCloseTile = 128 * 128 * 4;                    // a work item's bf16 (gate, up) pairs, [row][channel]
constexpr int kWideLaunchRegs = 168;     // what the kernel must have been given per thread for that to add up
constexpr int kWideSmem = 232448;
constexpr int kWideAcc = 2;              // accumulator stages of 256 TMEM columns
constexpr int kWideMaxStages = 4;
constexpr int kWideTile = 16384;         // 128 rows x 128 bytes

template <bool DUAL>
struct WideCfg {
  // gate/up: tokens, gate tile, up tile of one K block; down: tokens and weights of two K blocks
  static constexpr int kStageBytes = (DUAL ? 3 : 4) * kWideTile;
  // after the ring: barriers, the item queue, amax exchange [2 items][2 halves][128], flags
  static constexpr int kTailBytes = (2 * kWideMaxStages + 2 * kWideAcc + 2 * kQueue + 2) * 8 + kQueue * 16 + 2 * 2 * 128 * 4 + 64 + 16;
  // gate/up with closing warps: the tile the epilogue hands them sits between the ring and the tail
  static constexpr bool kClosers = DUAL && MOE_WIDE_CLOSERS;
  static constexpr int kCloseBytes = kClosers ? kWideCloseTile : 0;
  static constexpr int kThreads = kClosers ? 512 : kWideThreads;
  static constexpr int kEpiRegs = kClosers ? kWideEpiRegsWithClosers : kWideEpiRegs;
  static constexpr int kLaunchRegs = kClosers ? 128 : kWideLaunchRegs;
  static constexpr int kRegsNeeded = 128 * kWideServiceRegs + kWideEpiThreads * kEpiRegs + (kClosers ? 128 * kWideCloserRegs : 0);
  static constexpr int kStages = (kWideSmem - 1024 - kTailBytes - kCloseBytes) / kStageBytes < kWideMaxStages
                                     ? (kWideSmem - 1024 - kTailBytes - kCloseBytes) / kStageBytes
                                     : kWideMaxStages;
};

struct WideDev {
  const Chunk* chunks;
  const int32_t* n_chunks;
  int tiles_m, kblocks, m, n_local;
  const float* act_scale;
  const float* w_a_scale;
  const float* w_b_scale;
  const float* s_a_scale;
  const float* s_b_scale;
  uint8_t* aq;
  float* as;
  __nv_bfloat16* out;
  const int32_t* row_dest;
  int32_t* status;
  int ksplit;              // down GEMM: parts the contraction is summed in (1 = whole)
  SwigluMode swiglu;
};

// 32 consecutive fp32 columns of this thread's TMEM lane (issue only; tmem_wait_ld() before use).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
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

// acc[0..32) += d[0..32) * s, two columns per instruction (each half an ordinary fused multiply-add)
__device__ __forceinline__ void fold32(const uint32_t* d, float s, float* acc) {
#pragma unroll
  for (int j = 0; j < 32; j += 2) fma2(__uint_as_float(d[j]), __uint_as_float(d[j + 1]), s, s, acc[j], acc[j + 1]);
}

template <bool DUAL>
__global__ void __launch_bounds__(WideCfg<DUAL>::kThreads, 1)
grouped_gemm_wide_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         const __grid_constant__ CUtensorMap tm_sa, const __grid_constant__ CUtensorMap tm_sb,
                         const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_xw,
                         const WideDev p) {
  using C = WideCfg<DUAL>;
  constexpr int S = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  const int KB = p.kblocks;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stages = base;
  uint4* s_close = reinterpret_cast<uint4*>(base + S * C::kStageBytes);      // [128 rows][32 chunks of four (gate, up) pairs], swizzled
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(base + S * C::kStageBytes + C::kCloseBytes);
  uint64_t* bar_empty = bar_full + kWideMaxStages;
  uint64_t* bar_tfull = bar_empty + kWideMaxStages;
  uint64_t* bar_tempty = bar_tfull + kWideAcc;
  uint64_t* bar_qfull = bar_tempty + kWideAcc;
  uint64_t* bar_qempty = bar_qfull + kQueue;
  uint64_t* bar_cfull = bar_qempty + kQueue;       // the closing warps' tile is written / has been read
  uint64_t* bar_cempty = bar_cfull + 1;
  int4* s_queue = reinterpret_cast<int4*>(bar_cempty + 1);
  float* s_amax = reinterpret_cast<float*>(s_queue + kQueue);            // [2][2][128]
  int4* s_close_item = reinterpret_cast<int4*>(s_amax + 2 * 2 * 128);      // {channel tile, first row, rows, 1 = no more items}
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_close_item + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile uint32_t* s_issued = reinterpret_cast<volatile uint32_t*>(s_tmem + 2);    // steps whose TMA was issued
  volatile uint32_t* s_consumed = reinterpret_cast<volatile uint32_t*>(s_tmem + 3);  // steps whose data arrived
  volatile uint32_t* s_committed = reinterpret_cast<volatile uint32_t*>(s_tmem + 4); // accumulators committed
  volatile uint32_t* s_drained = reinterpret_cast<volatile uint32_t*>(s_tmem + 5);   // accumulators read

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(bar_full + s, 1); mbar_init(bar_empty + s, 1); }
    for (int s = 0; s < kWideAcc; ++s) { mbar_init(bar_tfull + s, 1); mbar_init(bar_tempty + s, kWideEpiThreads); }
    for (int s = 0; s < kQueue; ++s) { mbar_init(bar_qfull + s, 1); mbar_init(bar_qempty + s, 32 + kWideEpiThreads); }
    mbar_init(bar_cfull, kWideEpiThreads);
    mbar_init(bar_cempty, 128);
    *s_abort = 0; *s_issued = 0; *s_consumed = 0; *s_committed = 0; *s_drained = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tm_a); prefetch_tmap(&tm_x); prefetch_tmap(&tm_xw);
    if (DUAL) prefetch_tmap(&tm_b);
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

  // Everything above touched only shared memory, TMEM and kernel parameters: under a dependent
  // launch it overlaps the tail of the previous kernel. From here on its results are needed.
  dependent_wait();
  dependents_may_launch();
  const int n_units = *p.n_chunks * p.tiles_m;
  const int ksplit = DUAL ? 1 : p.ksplit;
  const int part_len = (KB + ksplit - 1) / ksplit;     // K blocks per part (the whole contraction when it is not split)

  // The first warp group gives registers away, the two epilogue warp groups take them (the host
  // checked that the kernel was given enough per thread for the sums to work out).
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kWideServiceRegs));
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // weight tiles are read again within microseconds by the CTAs that hold the expert's other row
    // chunks, token tiles by every channel tile of the GEMM
    const uint64_t pol_w = policy_evict_normal();
    const uint64_t pol_x = policy_evict_last();
    uint32_t it = 0, s = 0, ph = 0, item = 0;
    bool ok = true;
    PROBE_DECL(probe_stage);
    int u_next = static_cast<int>(blockIdx.x) < n_units ? static_cast<int>(blockIdx.x) : -1;
    Chunk next = load_chunk(p.chunks, u_next, p.tiles_m);
    for (; ok; ++item) {
      const int u = u_next;
      const Chunk ch = next;
      {   // publish the item (or the end mark) to the other roles
        const uint32_t q = item % kQueue;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_qempty + q, ((item / kQueue) & 1u) ^ 1u, s_abort))) {
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 26); *s_abort = 1; }
          break;
        }
        if (lane == 0) {
          s_queue[q] = make_int4(u, ch.expert, ch.row0, ch.rows);
          mbar_arrive(bar_qfull + q);
        }
        __syncwarp();
      }
      if (u < 0) {
        if (lane == 0) { PROBE_FLUSH_ROLE(p.status, 2, probe_stage); }
        break;
      }
      {
        const long long at = static_cast<long long>(blockIdx.x) + static_cast<long long>(item + 1) * gridDim.x;
        u_next = at < n_units ? static_cast<int>(at) : -1;
        next = load_chunk(p.chunks, u_next, p.tiles_m);
      }
      const int mt = u % p.tiles_m;
      const bool shared_e = ch.expert >= p.n_local;
      const CUtensorMap* ma = shared_e ? &tm_sa : &tm_a;
      const CUtensorMap* mb = shared_e ? &tm_sb : &tm_b;
      const int wrow = (shared_e ? 0 : ch.expert * p.m) + mt * 128;
      const int n16 = (ch.rows + 15) >> 4;            // token rows move in boxes of 16; rows past them keep what
                                                      // the stage held before (their TMEM lanes are never read out)
      for (int kb = 0; kb < KB; ++it) {
        const int len = step_blocks<DUAL>(kb, KB, part_len);
        const uint32_t bytes = DUAL ? n16 * 2048 + 2 * kWideTile : len * (n16 * 2048 + kWideTile);
        PROBE_START(t_stage);
        if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + s, ph ^ 1u, s_abort))) {
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 21); *s_abort = 1; }
          ok = false;
          break;
        }
        PROBE_ADD(probe_stage, t_stage);
        uint8_t* st = stages + s * C::kStageBytes;
        if (elect_one()) {
          mbar_expect_tx(bar_full + s, bytes);
          if constexpr (DUAL) {
            tma_load_2d(st + kWideTile, ma, kb * 128, wrow, bar_full + s, pol_w);
            tma_load_2d(st + 2 * kWideTile, mb, kb * 128, wrow, bar_full + s, pol_w);
            if (n16 == 8) tma_load_2d(st, &tm_xw, kb * 128, ch.row0, bar_full + s, pol_x);     // a full tile: one request
            else for (int j = 0; j < n16; ++j) tma_load_2d(st + j * 2048, &tm_x, kb * 128, ch.row0 + j * 16, bar_full + s, pol_x);
          } else {
            for (int l = 0; l < len; ++l) {
              tma_load_2d(st + (2 + l) * kWideTile, ma, (kb + l) * 128, wrow, bar_full + s, pol_w);
              if (n16 == 8) tma_load_2d(st + l * kWideTile, &tm_xw, (kb + l) * 128, ch.row0, bar_full + s, pol_x);
              else for (int j = 0; j < n16; ++j)
                tma_load_2d(st + l * kWideTile + j * 2048, &tm_x, (kb + l) * 128, ch.row0 + j * 16, bar_full + s, pol_x);
            }
          }
          *s_issued = it + 1;
        }
        __syncwarp();
        if (++s == static_cast<uint32_t>(S)) { s = 0; ph ^= 1u; }
        kb += len;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    // The whole warp runs the loop with warp-uniform values and one elected lane issues.
    uint32_t it = 0, s = 0, ph = 0;
    bool ok = true;
    const uint32_t idesc = idesc_e4m3(128, DUAL ? 256 : 128);
    PROBE_DECL(probe_acc);
    PROBE_DECL(probe_data);
    for (uint32_t item = 0; ok; ++item) {
      int u = -1;
      Chunk ch;
      if (!__all_sync(0xffffffffu, take_item(s_queue, bar_qfull, bar_qempty, item, s_abort, u, ch))) {
        if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 28); *s_abort = 1; }
        break;
      }
      if (u < 0) {
        if (lane == 0) { PROBE_FLUSH_ROLE(p.status, 3, probe_acc); PROBE_FLUSH_ROLE(p.status, 4, probe_data); }
        break;
      }
      for (int kb = 0; kb < KB; ++it) {
        const int len = step_blocks<DUAL>(kb, KB, part_len);
        const uint32_t as = it % kWideAcc, aph = (it / kWideAcc) & 1u;
        PROBE_START(t_acc);
        bool got = mbar_wait(bar_tempty + as, aph ^ 1u, s_abort);
        PROBE_ADD(probe_acc, t_acc);
        PROBE_START(t_data);
        got = got && mbar_wait(bar_full + s, ph, s_abort);
        PROBE_ADD(probe_data, t_data);
        if (!__all_sync(0xffffffffu, got)) {      // one decision for the warp
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 22); *s_abort = 1; }
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(stages + s * C::kStageBytes);
        const uint32_t d0 = tmem + as * 256;
        if (elect_one()) {
          *s_consumed = it + 1;
          const uint64_t desc0 = smem_desc_sw128(sa);      // the token tile; every other operand is this plus a constant
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const uint64_t ad = desc0 + ((k4 * 32) >> 4);
            if constexpr (DUAL) {
              mma_f8(d0, ad, ad + (kWideTile >> 4), idesc, k4 > 0 ? 1u : 0u);      // gate rows, then up rows: N = 256
            } else {
              mma_f8(d0, ad, ad + ((2 * kWideTile) >> 4), idesc, k4 > 0 ? 1u : 0u);
              if (len == 2)    // the next K block: its own token tile, weight tile and accumulator
                mma_f8(d0 + 128, ad + (kWideTile >> 4), ad + ((3 * kWideTile) >> 4), idesc, k4 > 0 ? 1u : 0u);
            }
          }
          mma_commit(bar_empty + s);     // the stage may be refilled once these MMAs have read it
          mma_commit(bar_tfull + as);    // the accumulators are complete
          *s_committed = it + 1;
        }
        __syncwarp();
        if (++s == static_cast<uint32_t>(S)) { s = 0; ph ^= 1u; }
        kb += len;
      }
    }
    __syncwarp();
  }
  } else if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kWideCloserRegs));
    // ------------------------------ closing warps (gate/up) -------------------
    // SwiGLU on the bf16-rounded GEMM outputs and requantisation of each row's 128 channels of the tile
    // (megabench/tasks/megamoe.py:116-128, megabench/tasks/quantization.py:87-109), off the epilogue
    // warps: those hand over a finished item as bf16 (gate, up) pairs in shared memory and go on folding
    // the next item's K blocks, so the accumulators keep coming back while an item is closed (with the
    // epilogue threads closing their own rows the MMAs stood still for most of the 11,000 cycles it
    // took: TMEM holds two accumulators). Warps 12-15: a warp takes a row at a time, a lane four channels.
    const SwigluMode& mode = p.swiglu;
    for (uint32_t k = 0;; ++k) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_cfull, k & 1u, s_abort))) {
        if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 35); *s_abort = 1; }
        break;
      }
      const int4 item = *s_close_item;
      if (item.w) break;                                   // the CTA's last item is behind us
      const int mt = item.x, row0 = item.y, rows = item.z;
      for (int r = warp - 12; r < rows; r += 4) {
        const uint4 v = s_close[r * 32 + (lane ^ (r & 31))];
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
        float weight = 1.f;
        bool weighted = false;
        if (mode.slot_weight) {
          const int dest = mode.row_dest[row0 + r];
          if (dest < mode.routed_rows) { weight = mode.slot_weight[dest]; weighted = true; }
        }
        float a[4];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float g = __uint_as_float(w4[j] << 16);            // a bf16 is the upper half of an fp32
          float u = __uint_as_float(w4[j] & 0xffff0000u);
          if (mode.limit > 0.f) {
            g = fminf(g, mode.limit);
            u = fminf(fmaxf(u, -mode.limit), mode.limit);
          }
          a[j] = silu_times(g, u);
          if (weighted) a[j] = __fmul_rn(a[j], weight);
          amax = fmaxf(amax, fabsf(a[j]));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float scale = group_scale(amax);
        const float rcp = __frcp_rn(scale);
        const uint32_t bytes = to_e4m3_pair(a[0], a[1], scale, rcp) | to_e4m3_pair(a[2], a[3], scale, rcp) << 16;
        *reinterpret_cast<uint32_t*>(p.aq + static_cast<size_t>(row0 + r) * p.m + mt * kGroup + 4 * lane) = bytes;
        if (lane == 0) p.as[static_cast<size_t>(row0 + r) * (p.m / kGroup) + mt] = scale;
      }
      mbar_arrive(bar_cempty);                             // this thread has read what it needed of the tile
    }
    __syncwarp();
    __syncwarp();
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::kEpiRegs));
    // ------------------------------ epilogue ----------------------------------
    const int tid = static_cast<int>(threadIdx.x) - 128;
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
    const int half = (warp - 4) >> 2;             // which 64 columns of each 128-column accumulator
    const int t = quarter * 32 + lane;            // token row inside the tile
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + half * 64;
    uint32_t it = 0;
    bool failed = false;
    PROBE_DECL(probe_tfull);
    PROBE_DECL(probe_read);
    PROBE_DECL(probe_fold);
    PROBE_DECL(probe_close);
    PROBE_DECL(probe_cta);
    PROBE_START(t_cta);
    for (uint32_t un = 0;; ++un) {
      int u = -1;
      Chunk ch;
      if (!take_item(s_queue, bar_qfull, bar_qempty, un, s_abort, u, ch)) {
        if (!*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 29); *s_abort = 1; }
        failed = true;
      }
      // one decision for all epilogue threads (the item is the same for all of them unless one failed)
      const bool any_failed = epilogue_any<kWideEpiThreads>(failed);
      if (any_failed || u < 0) {
        if constexpr (DUAL && MOE_WIDE_CLOSERS) {
          if (!any_failed) {      // tell the closing warps that nothing follows (they have a bounded wait otherwise)
            mbar_wait(bar_cempty, (un & 1u) ^ 1u, s_abort);
            if (tid == 0) *s_close_item = make_int4(0, 0, 0, 1);
            mbar_arrive(bar_cfull);
          }
        }
        if (tid == 0) {
          PROBE_ADD(probe_cta, t_cta);
          PROBE_FLUSH(p.status, 5, probe_tfull);
          PROBE_FLUSH_EPI(p.status, 2, probe_read);
          PROBE_FLUSH_EPI(p.status, 4, probe_fold);
          PROBE_FLUSH_EPI(p.status, 6, probe_close);
          PROBE_FLUSH(p.status, 7, probe_cta);
        }
        break;
      }
      const int mt = u % p.tiles_m;
      const bool shared_e = ch.expert >= p.n_local;
      const bool valid = t < ch.rows;
      const int row = ch.row0 + (valid ? t : 0);       // rows past the chunk fold a neighbour's scales into lanes nobody stores
      const float* xs = p.act_scale + static_cast<size_t>(row) * KB;
      const float* wa = (shared_e ? p.s_a_scale : p.w_a_scale + static_cast<size_t>(ch.expert) * p.tiles_m * KB) +
                        static_cast<size_t>(mt) * KB;
      const float* wb = wa;
      if constexpr (DUAL)
        wb = (shared_e ? p.s_b_scale : p.w_b_scale + static_cast<size_t>(ch.expert) * p.tiles_m * KB) +
             static_cast<size_t>(mt) * KB;
      float acc_a[64], acc_b[64];
#pragma unroll
      for (int n = 0; n < 64; ++n) { acc_a[n] = 0.f; acc_b[n] = 0.f; }
      // The scales of a step are read one step ahead (token scales at L2: the kernel before wrote them).
      // A thread's token scales are KB consecutive floats of its own row, so each 4-byte load is a
      // 32-byte sector of its own from the L2: where the rows are 16-byte aligned (KB a multiple of 4)
      // they come four K blocks per load, one group ahead (a quarter of the requests; with a load per
      // K block the scale reads were a sixth of the SM's L2 traffic beside the operand tiles).
      const bool by_four = (KB & 3) == 0 && (reinterpret_cast<uintptr_t>(p.act_scale) & 15) == 0;
      float4 x_now = make_float4(0.f, 0.f, 0.f, 0.f), x_ahead = x_now;
      int x_group = 0;
      if (by_four) {
        x_now = __ldcg(reinterpret_cast<const float4*>(xs));
        x_ahead = KB > 4 ? __ldcg(reinterpret_cast<const float4*>(xs) + 1) : x_now;
      }
      auto token_scale = [&](int k) -> float {      // k never decreases and advances by at most two
        if (!by_four) return __ldcg(xs + k);
        if ((k >> 2) != x_group) {
          x_group = k >> 2;
          x_now = x_ahead;
          if (4 * (x_group + 1) < KB) x_ahead = __ldcg(reinterpret_cast<const float4*>(xs) + x_group + 1);
        }
        const int i = k & 3;
        return i == 0 ? x_now.x : i == 1 ? x_now.y : i == 2 ? x_now.z : x_now.w;
      };
      float x0 = token_scale(0), w0 = __ldg(wa);
      float x1 = DUAL ? x0 : (KB > 1 ? token_scale(1) : 0.f);
      float w1 = DUAL ? __ldg(wb) : (KB > 1 ? __ldg(wa + 1) : 0.f);
      for (int kb = 0; kb < KB; ++it) {
        const int len = step_blocks<DUAL>(kb, KB, part_len);
        const bool second = DUAL || len == 2;          // the step's second accumulator holds something
        const float s0 = __fmul_rn(w0, x0), s1 = __fmul_rn(w1, x1);
        {
          const int nb = kb + len;                     // first K block of the next step
          if (nb < KB) {
            x0 = token_scale(nb); w0 = __ldg(wa + nb);
            if constexpr (DUAL) { x1 = x0; w1 = __ldg(wb + nb); }
            else if (nb + 1 < KB) { x1 = token_scale(nb + 1); w1 = __ldg(wa + nb + 1); }
          }
        }
        const uint32_t as = it % kWideAcc, aph = (it / kWideAcc) & 1u;
        PROBE_START(t_tfull);
        if (!failed && !mbar_wait(bar_tfull + as, aph, s_abort)) {
          if (!*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 23); *s_abort = 1; }
          failed = true;
        }
        PROBE_ADD(probe_tfull, t_tfull);
        PROBE_START(t_read);
        if (failed) { kb += len; continue; }   // keep in step with the other epilogue threads up to the item's end
        tc_fence_after();
        const uint32_t t0 = lane_base + as * 256;
        // 32 columns at a time through two register buffers: the next read is on its way while the
        // last one is folded (tcgen05.wait::ld waits for every read issued so far)
        uint32_t ra[32], rb[32];
        tmem_ld32(t0, ra);
        tmem_wait_ld();
        tmem_ld32(t0 + 32, rb);
        fold32(ra, s0, acc_a);
        tmem_wait_ld();
        if (second) tmem_ld32(t0 + 128, ra);
        fold32(rb, s0, acc_a + 32);
        if (second) {
          // gate/up: the up half of K block kb; down: K block kb + 1, into the same sums after kb
          tmem_wait_ld();
          tmem_ld32(t0 + 128 + 32, rb);
          fold32(ra, s1, DUAL ? acc_b : acc_a);
          tmem_wait_ld();
        }
        // The last values are in registers: hand the accumulators back before folding them.
        tc_fence_before();
        mbar_arrive(bar_tempty + as);
        if (tid == 0) *s_drained = it + 1;
        if (second) fold32(rb, s1, (DUAL ? acc_b : acc_a) + 32);
        PROBE_ADD(probe_read, t_read);
        kb += len;
        if constexpr (!DUAL) {
          if (ksplit > 1 && (kb % part_len == 0 || kb == KB)) {   // a part ends here: parts are summed in part order
#pragma unroll
            for (int n = 0; n < 64; ++n) {
              acc_b[n] = __fadd_rn(acc_b[n], acc_a[n]);
              acc_a[n] = 0.f;
            }
          }
        }
      }
      PROBE_START(t_close);
      // One decision for all epilogue threads: nobody may be left alone at a later barrier.
      if (epilogue_any<kWideEpiThreads>(failed || *s_abort)) break;
      if constexpr (DUAL && MOE_WIDE_CLOSERS) {
        // The item goes to the closing warps as bf16 (gate, up) pairs, four channels per 16-byte chunk,
        // chunk c of row t at position c ^ (t & 31) of the row: the lanes of a warp (32 rows, the same
        // chunk) and the lanes of a closing warp (one row, 32 chunks) both touch every bank once.
        const bool late = !mbar_wait(bar_cempty, (un & 1u) ^ 1u, s_abort);     // the previous item's tile has been read
        if (epilogue_any<kWideEpiThreads>(late)) {
          if (tid == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 36); *s_abort = 1; }
          break;
        }
#pragma unroll
        for (int n = 0; n < 64; n += 4) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            w[j] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(acc_a[n + j]))) |
                   static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(acc_b[n + j]))) << 16;
          s_close[t * 32 + ((half * 16 + (n >> 2)) ^ (t & 31))] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        if (tid == 0) *s_close_item = make_int4(mt, ch.row0, ch.rows, 0);
        mbar_arrive(bar_cfull);                    // (release: the stores above are visible to who waits on it)
      } else if constexpr (DUAL) {
        // SwiGLU on the bf16-rounded GEMM outputs and requantisation of the row's 128 channels of this
        // tile (megabench/tasks/megamoe.py:116-128, megabench/tasks/quantization.py:87-109); the row's
        // two threads exchange their maxima through shared memory (a buffer per item parity, so one
        // barrier per item is enough).
        const SwigluMode& mode = p.swiglu;
        float weight = 1.f;
        bool weighted = false;
        if (mode.slot_weight && valid) {
          const int dest = mode.row_dest[ch.row0 + t];
          if (dest < mode.routed_rows) { weight = mode.slot_weight[dest]; weighted = true; }
        }
        float amax = 0.f;
        if (valid) {      // (the lanes of rows past the chunk hold whatever the stage held before)
#pragma unroll
          for (int n = 0; n < 64; ++n) {
            float g = bf16_round(acc_a[n]);
            float v = bf16_round(acc_b[n]);
            if (mode.limit > 0.f) {
              g = fminf(g, mode.limit);
              v = fminf(fmaxf(v, -mode.limit), mode.limit);
            }
            float a = silu_times(g, v);
            if (weighted) a = __fmul_rn(a, weight);
            acc_a[n] = a;
            amax = fmaxf(amax, fabsf(a));
          }
        }
        float* mine = s_amax + (un & 1u) * 256;
        mine[half * 128 + t] = amax;
        epilogue_sync<kWideEpiThreads>();
        if (valid) {
          const float scale = group_scale(fmaxf(mine[t], mine[128 + t]));
          const float r = __frcp_rn(scale);
          uint8_t* dst = p.aq + static_cast<size_t>(ch.row0 + t) * p.m + mt * kGroup + half * 64;
#pragma unroll
          for (int n = 0; n < 64; n += 16) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              w[j] = to_e4m3_pair(acc_a[n + 4 * j], acc_a[n + 4 * j + 1], scale, r) |
                     to_e4m3_pair(acc_a[n + 4 * j + 2], acc_a[n + 4 * j + 3], scale, r) << 16;
            *reinterpret_cast<uint4*>(dst + n) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          if (half == 0) p.as[static_cast<size_t>(ch.row0 + t) * (p.m / kGroup) + mt] = scale;
        }
      } else if (valid) {
        // one bf16 rounding of the fp32 sum (megabench/tasks/megamoe.py:149), 64 channels of the row's slot
        const size_t dest = static_cast<size_t>(p.row_dest ? p.row_dest[ch.row0 + t] : ch.row0 + t);
        __nv_bfloat16* dst = p.out + dest * p.m + mt * kGroup + half * 64;
#pragma unroll
        for (int n = 0; n < 64; n += 8) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float lo = ksplit > 1 ? acc_b[n + 2 * j] : acc_a[n + 2 * j];
            const float hi = ksplit > 1 ? acc_b[n + 2 * j + 1] : acc_a[n + 2 * j + 1];
            const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
            w[j] = *reinterpret_cast<const uint32_t*>(&pair);
          }
          *reinterpret_cast<uint4*>(dst + n) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      PROBE_ADD(probe_close, t_close);
    }
  }

  // ------------------------------ common exit ---------------------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*s_abort && threadIdx.x == 0) {
    // Give copies and MMAs that were issued but never consumed a bounded chance to land.
    for (uint32_t it = *s_consumed; it < *s_issued; ++it) mbar_wait(bar_full + it % S, (it / S) & 1u);
    for (uint32_t it = *s_drained; it < *s_committed; ++it) mbar_wait(bar_tfull + it % kWideAcc, (it / kWideAcc) & 1u);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// Host side.
// ---------------------------------------------------------------------------------------
template <bool DUAL>
static cudaError_t launch_wide_typed(const WideDev& dev, const CUtensorMap* maps, int grid, cudaStream_t stream) {
  using C = WideCfg<DUAL>;
  static_assert(C::kStages >= 2, "the ring needs two stages");
  static int configured[64] = {};       // 1 = ready, -1 = unusable; the attribute belongs to the device the call runs on
  int device = 0;
  cudaGetDevice(&device);
  const bool cached = device >= 0 && device < 64;
  if (!cached || !configured[device]) {
    // The epilogue warp groups' setmaxnreg would wait for ever for registers the CTA was never given:
    // the kernel is launched only if the compiler sized it as the constants above assume.
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, grouped_gemm_wide_kernel<DUAL>);
    if (e != cudaSuccess) return e;
    const bool fits = attr.numRegs * C::kThreads >= C::kRegsNeeded && attr.numRegs >= C::kLaunchRegs;
    if (fits) e = cudaFuncSetAttribute(grouped_gemm_wide_kernel<DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, kWideSmem);
    if (e != cudaSuccess) return e;
    if (cached) configured[device] = fits ? 1 : -1;
    if (!fits) return cudaErrorInvalidConfiguration;
  }
  if (cached && configured[device] < 0) return cudaErrorInvalidConfiguration;
  const int smem = 1024 + C::kStages * C::kStageBytes + C::kCloseBytes + C::kTailBytes;
  return launch_dependent(grouped_gemm_wide_kernel<DUAL>, dim3(grid), dim3(C::kThreads), smem, stream, maps[0], maps[1],
                          maps[2], maps[3], maps[4], maps[5], dev);
}

cudaError_t launch_gemm_wide(const GemmArgs& a, cudaStream_t stream, int* launches, int* driver_error) {
  if (a.tile != 128 || a.k % 128 || a.m % 128 || a.k / 128 > 112 || a.progress || a.fold.y) return cudaErrorInvalidValue;
  CUtensorMap maps[6];
  int rc = 0;
  const uint64_t wrows = static_cast<uint64_t>(a.n_local) * a.m;
  // With no routed experts on this rank the routed maps alias the shared ones (never dereferenced).
  const uint8_t* wa = a.n_local > 0 ? a.w_a : a.s_a;
  const uint8_t* wb = a.n_local > 0 ? a.w_b : a.s_b;
  rc |= make_map(&maps[0], wa, a.n_local > 0 ? wrows : a.m, a.k, 128);
  rc |= make_map(&maps[1], a.dual ? wb : wa, a.n_local > 0 ? wrows : a.m, a.k, 128);
  const uint8_t* sa = a.s_a ? a.s_a : wa;
  const uint8_t* sb = a.dual ? (a.s_b ? a.s_b : wb) : sa;
  rc |= make_map(&maps[2], sa, a.s_a ? a.m : wrows, a.k, 128);
  rc |= make_map(&maps[3], sb, a.s_a ? a.m : wrows, a.k, 128);
  rc |= make_map(&maps[4], a.act, a.total_rows, a.k, 16);      // token rows of a ragged chunk move in boxes of 16,
  rc |= make_map(&maps[5], a.act, a.total_rows, a.k, 128);     // a full tile's in one of 128 (a tenth of the requests per K block)
  if (rc) {
    if (driver_error) *driver_error = rc;
    return cudaErrorUnknown;
  }
  const int ksplit = a.dual || a.ksplit < 1 ? 1 : a.ksplit;
  if (ksplit > 1 && (ksplit - 1) * ((a.k / 128 + ksplit - 1) / ksplit) >= a.k / 128) return cudaErrorInvalidValue;
  WideDev dev{a.chunks, a.n_chunks, a.m / 128, a.k / 128, a.m, a.n_local, a.act_scale, a.w_a_scale, a.w_b_scale,
              a.s_a_scale, a.s_b_scale, a.aq, a.as, a.out, a.row_dest, a.status, ksplit, a.swiglu};
  const int grid = std::max(1, std::min(gemm_sm_count(), a.max_units));
  const cudaError_t e = a.dual ? launch_wide_typed<true>(dev, maps, grid, stream) : launch_wide_typed<false>(dev, maps, grid, stream);
  if (launches) *launches += 1;
  return e;
}

}  // namespace moe
