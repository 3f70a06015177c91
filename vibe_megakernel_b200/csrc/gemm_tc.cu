// Persistent grouped FP8 GEMM for the expert MLPs on tcgen05 tensor cores.
//
// Orientation: the weights are the MMA's M side (128 output channels per tile) and the tokens
// of one expert are the N side (16 to 64 per tile, in steps of 16), so a decode batch streams
// every weight byte exactly once through TMA while the token rows stay L2-resident.
//
//   D[m, n] = sum_k W[m, k] * X[n, k]       e4m3 x e4m3 -> fp32 in TMEM, kind::f8f6f4
//
// Block scales: W has one fp32 scale per 128x128 block, X one per token per 128 channels
// (megabench/tasks/quantization.py:87-131). They are not powers of two, so each 128-deep K block
// is accumulated into a fresh TMEM accumulator and the epilogue warps fold it into fp32
// registers as acc += D * (w_scale * x_scale[n]); four to eight TMEM accumulators let the MMAs
// of the next K blocks run meanwhile.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warp 2 = scale loader (stages
// the next work item's scales in shared memory while the current one is computed), warps 3.. =
// epilogue (a thread owns one TMEM lane = one output channel, for a run of token columns).
// Work items (expert, row chunk, channel tile) are walked by a persistent grid; their list is
// produced on the device by the permutation kernel, so no host synchronisation is needed between
// routing and the GEMMs. A chunk with r rows only moves and multiplies ceil(r/16)*16 token
// columns. The producer warp decides the CTA's next item and passes it to the other roles through
// a small queue in shared memory.
//
// Hand-over between the two GEMMs of a layer: the gate/up GEMM counts finished tiles per chunk in
// global memory; the down GEMM does not wait for the gate/up kernel as a whole but, per item, for
// that chunk's counter, and takes its items from a global dispenser instead of a fixed stride.
// Its CTAs therefore start on SMs the gate/up GEMM has already left and stream down-projection
// weights while the last gate/up tiles finish elsewhere. All gate/up CTAs are resident before the
// first down CTA can be scheduled (the grid is at most one CTA per SM and the dependent launch is
// released only after every gate/up CTA has started), so the waits cannot starve their producers.
//
// Every wait is bounded: on expiry the role records MOE_ERR_DEVICE_TIMEOUT, raises the CTA's
// abort flag, and all roles fall through to the common exit, which waits (bounded) for copies
// still in flight and frees TMEM.
//
// Reference arithmetic: megabench/tasks/megamoe.py:146-149 (grouped expert GEMMs),
// :116-128 (SwiGLU + requantisation), megabench/tasks/frontier.py:180-186 (FP8 linear).
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_items.cuh"
#include "kernels.h"

namespace moe {

// TMEM accumulators in flight (per configuration: as many as fit in the 512 columns, at most 8).
// One K block's round trip MMA -> commit -> epilogue wake-up -> tcgen05.ld -> release -> MMA takes
// about a microsecond, so the number of accumulators bounds the K blocks a CTA retires per
// microsecond: 4 of them capped a down-projection CTA (16 KB of weights per K block) near
// 40 GB/s, which showed wherever fewer CTAs than SMs had work.
constexpr int kMaxAccStages = 8;
constexpr int kMaxStages = 12;
constexpr int kMaxSmem = 232448;      // 227 KiB per CTA
constexpr int kMaxKBlocks = 112;      // K <= 14336

template <int NT, bool DUAL>
struct GemmCfg {
  static constexpr int kEpiWarps = NT >= 32 ? 8 : 4;
  static constexpr int kEpiThreads = kEpiWarps * 32;
  static constexpr int kThreads = 96 + kEpiThreads;
  static constexpr int kCpt = NT / (kEpiWarps / 4);   // token columns per epilogue thread
  // A pipeline step carries two weight tiles and feeds two accumulators: gate and up of one K block
  // (DUAL), or two consecutive K blocks of the down projection with their token tiles. The fixed cost
  // of a step in the MMA warp (waits, election, commits: 500-600 cycles) is the same either way; with
  // one 16 KB tile per step it, not HBM, set the pace of a down-projection CTA at small batches.
  static constexpr int kABytes = 128 * 128;
  static constexpr int kBBytes = NT * 128;
  static constexpr int kStageBytes = 2 * kABytes + (DUAL ? 1 : 2) * kBBytes;
  static constexpr int kAccCols = 2 * NT;
  static constexpr int kAcc = 512 / kAccCols < kMaxAccStages ? 512 / kAccCols : kMaxAccStages;
  static constexpr int kTmemCols = kAcc * kAccCols < 32 ? 32 : kAcc * kAccCols;   // a power of two
  // Shared memory after the stage ring, for a contraction of kb K blocks:
  //   the output tile [NT][128] (e4m3 for gate/up, bf16 for down) the epilogue collects an item's
  //   results in, 2 buffers of { scale table [kb][NT], gate/up: weight scales [2][kb], destination
  //   rows [NT] }, amax scratch [4][NT], the token scales and their reciprocals [2][NT],
  //   barriers (2*kMaxStages + 2*kMaxAccStages + 2 + 2 + 2*kQueue), the item queue, 8 words of flags.
  // (every part a multiple of four floats, so the token scales can be read 16 bytes at a time)
  // Down GEMM: the table holds the products w_scale * x_scale (computed once by the scale loader
  // instead of by each of the 128 threads that own a channel of the column). Gate/up: the token
  // scales, with the two weight scales of every K block behind them (two product tables would
  // double the broadcast loads of the fold, which the shared-memory pipe, not the FP pipe, limits).
  static constexpr int weight_scale_floats(int kb) { return DUAL ? (2 * kb + 3) & ~3 : 0; }
  static constexpr int scale_floats(int kb) { return kb * NT + weight_scale_floats(kb) + NT + (DUAL ? 0 : 2 * NT); }   // + destination rows [NT], down: + row addresses [NT] x 8 bytes
  static constexpr int kTileBytes = NT * 128 * (DUAL ? 1 : 2);
  static constexpr int tail_bytes(int kb) {
    return kTileBytes + 2 * scale_floats(kb) * 4 + 6 * NT * 4 + (2 * kMaxStages + 2 * kMaxAccStages + 4 + 2 * kQueue) * 8 + kQueue * 16 + 64;
  }
  static constexpr int stages_for(int kb) {
    const int s = (kMaxSmem - 1024 - tail_bytes(kb)) / kStageBytes;
    return s > kMaxStages ? kMaxStages : s;
  }
};

struct GemmDev {
  const Chunk* chunks;
  const int32_t* n_chunks;
  int tiles_m, kblocks, m, n_local, stages;
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
  int32_t* progress;       // see GemmArgs; NULL = kernel-boundary ordering, fixed-stride walk
  int max_chunks, tiles_before;
  int ksplit;              // down GEMM: parts the contraction is cut in (1 = whole)
  float* partial;          // ksplit > 1: fp32 [tile index][part][NT columns][128 channels]
  int32_t* parts_done;     // ksplit > 1: per (chunk, channel tile) count of finished parts, zero on entry
  SwigluMode swiglu;       // DUAL: clamp and routing weight of the MegaMoE form, off by default
  FoldCombine fold;        // !DUAL: the combine, done by whoever stores a token's last slot row of a channel tile
  PeerReturn ret;          // !DUAL: rows stored into their sources' slot buffers, flags raised by the last CTA
};

template <int NT, bool DUAL>
__global__ void __launch_bounds__(GemmCfg<NT, DUAL>::kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_sa, const __grid_constant__ CUtensorMap tm_sb,
                    const __grid_constant__ CUtensorMap tm_x, const GemmDev p) {
  using C = GemmCfg<NT, DUAL>;
  extern __shared__ uint8_t smem_raw[];
  const int KB = p.kblocks;
  const int S = p.stages;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stages = base;
  uint8_t* s_tile = base + S * C::kStageBytes;                               // [NT][128] e4m3 or bf16
  float* s_scales = reinterpret_cast<float*>(s_tile + C::kTileBytes);        // [2][scale_floats(KB)]
  const int sf = C::scale_floats(KB);
  float* s_amax = s_scales + 2 * sf;                                         // [4][NT], then scales and reciprocals [2][NT]
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(s_amax + 6 * NT);
  uint64_t* bar_empty = bar_full + kMaxStages;
  uint64_t* bar_tfull = bar_empty + kMaxStages;
  uint64_t* bar_tempty = bar_tfull + kMaxAccStages;
  uint64_t* bar_scfull = bar_tempty + kMaxAccStages;
  uint64_t* bar_scempty = bar_scfull + 2;
  uint64_t* bar_qfull = bar_scempty + 2;
  uint64_t* bar_qempty = bar_qfull + kQueue;
  int4* s_queue = reinterpret_cast<int4*>(bar_qempty + kQueue);     // 16-byte aligned: all parts above are
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_queue + kQueue);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile uint32_t* s_issued = reinterpret_cast<volatile uint32_t*>(s_tmem + 2);    // K blocks whose TMA was issued
  volatile uint32_t* s_consumed = reinterpret_cast<volatile uint32_t*>(s_tmem + 3);  // K blocks whose data arrived
  volatile uint32_t* s_committed = reinterpret_cast<volatile uint32_t*>(s_tmem + 4); // accumulators committed
  volatile uint32_t* s_drained = reinterpret_cast<volatile uint32_t*>(s_tmem + 5);   // accumulators read
  volatile int* s_last_part = reinterpret_cast<volatile int*>(s_tmem + 6);           // split contraction: this CTA closes the tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(bar_full + s, 1); mbar_init(bar_empty + s, 1); }
    for (int s = 0; s < C::kAcc; ++s) { mbar_init(bar_tfull + s, 1); mbar_init(bar_tempty + s, C::kEpiThreads); }
    for (int s = 0; s < 2; ++s) { mbar_init(bar_scfull + s, 32); mbar_init(bar_scempty + s, C::kEpiThreads); }
    for (int s = 0; s < kQueue; ++s) { mbar_init(bar_qfull + s, 1); mbar_init(bar_qempty + s, 64 + C::kEpiThreads); }
    *s_abort = 0; *s_issued = 0; *s_consumed = 0; *s_committed = 0; *s_drained = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tm_a); prefetch_tmap(&tm_x);
    if (DUAL) prefetch_tmap(&tm_b);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  // Everything above touched only shared memory, TMEM and kernel parameters: under a dependent
  // launch it overlaps the tail of the previous kernel. From here on its results are needed.
  // The down GEMM in hand-over mode is the exception: what it reads was written either before the
  // gate/up kernel started (complete by the time this kernel can be scheduled) or by gate/up tiles
  // it waits for one by one.
  const bool handover = !DUAL && p.progress != nullptr;
  if (!handover) dependent_wait();
  dependents_may_launch();
#if !defined(MOE_TIMELINE) || MOE_TIMELINE == 1
  if (DUAL && threadIdx.x == 0) MOE_STAMP_FIRST(p.status, 5);
#endif
  PROBE_START(t_cta);
  const int n_chunks = *p.n_chunks;
  // A long contraction of the down GEMM is summed in `ksplit` parts, each from zero, added in part
  // order: that is the arithmetic whatever the batch. When the tiles are too few to occupy the
  // SMs, the parts become work items of their own (neighbours in the walk, so they run at the same
  // time) and the last one to finish adds them up; otherwise one CTA runs all parts of a tile.
  const int ksplit = DUAL ? 1 : p.ksplit;
  const bool spread = ksplit > 1 && n_chunks * p.tiles_m < 2 * static_cast<int>(gridDim.x);
  const int n_units = n_chunks * p.tiles_m * (spread ? ksplit : 1);
  // K blocks of a work item: one part when spread, else the whole contraction
  auto item_range = [&](int part, int& lo, int& hi) {
    if (spread) k_range(KB, ksplit, part, lo, hi);
    else { lo = 0; hi = KB; }
  };
  const int part_len = (KB + ksplit - 1) / ksplit;     // K blocks per part (the whole contraction when it is not split)

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    {   // warp-uniform loop, one elected lane issues the copies (see the MMA role below)
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      uint32_t it = 0, s = 0, ph = 0, item = 0;
      int ready_chunk = -1;
      bool ok = true;
      PROBE_DECL(probe_stage);
      // The CTA's next item: a fixed stride over the list, or the next free ones of the dispenser.
      // Short items are taken a few at a time (about 16 K blocks' worth), and the claim for the
      // batch after the current one is already in flight: the atomic's round trip (about a
      // microsecond, half the life of a 6-K-block item) is never waited for.
      const int grab = max(1, min(8, 16 / (spread ? (KB + ksplit - 1) / ksplit : KB)));
      int batch_next = 0, batch_end = 0, pending = 0;
      auto claim = [&]() -> int { return lane == 0 ? atomicAdd(p.progress + p.max_chunks, grab) : 0; };
      if (handover) pending = claim();
      auto next_unit = [&](uint32_t ordinal) -> int {
        int u;
        if (handover) {
          if (batch_next == batch_end) {
            batch_next = __shfl_sync(0xffffffffu, pending, 0);
            batch_end = batch_next + grab;
            pending = claim();
          }
          u = batch_next++;
        } else {
          u = blockIdx.x + ordinal * gridDim.x;
        }
        return u < n_units ? u : -1;
      };
      // position of the walk -> (tile position, part), then tile position -> work item
      auto resolve = [&](int& u, int& part) -> Chunk {
        part = 0;
        if (u >= 0 && spread) { part = u % ksplit; u /= ksplit; }
        return load_chunk(p.chunks, u, p.tiles_m);
      };
      int u_next = next_unit(0), part_next = 0;
      Chunk next = resolve(u_next, part_next);
      for (; ok; ++item) {
        const int u = u_next, part = part_next;
        const Chunk ch = next;
        {   // publish the item (or the end mark) to the other roles
          const uint32_t q = item % kQueue;
          if (!__all_sync(0xffffffffu, mbar_wait(bar_qempty + q, ((item / kQueue) & 1u) ^ 1u, s_abort))) {
            if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 6); *s_abort = 1; }
            break;
          }
          if (lane == 0) {
            s_queue[q] = make_int4(u, ch.expert, ch.row0, ch.rows | (part << 8));
            mbar_arrive(bar_qfull + q);
          }
          __syncwarp();
        }
        if (u < 0) {
          if (lane == 0) { PROBE_FLUSH_ROLE(p.status, 2, probe_stage); }
          break;
        }
        u_next = next_unit(item + 1);                          // both in flight during this item
        next = resolve(u_next, part_next);
        if (handover && u / p.tiles_m != ready_chunk) {
          // the chunk's rows of the intermediate activation must be complete before TMA reads them
          if (!__all_sync(0xffffffffu, wait_counter(p.progress + u / p.tiles_m, p.tiles_before, s_abort))) {
            if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 7); *s_abort = 1; }
            break;
          }
          fence_async_global();
          ready_chunk = u / p.tiles_m;
        }
        const int mt = u % p.tiles_m;
        const bool shared_e = ch.expert >= p.n_local;
        const CUtensorMap* ma = shared_e ? &tm_sa : &tm_a;
        const CUtensorMap* mb = shared_e ? &tm_sb : &tm_b;
        const int wrow = (shared_e ? 0 : ch.expert * p.m) + mt * 128;
        const int n16 = (ch.rows + 15) >> 4;
        int kb_lo, kb_hi;
        item_range(part, kb_lo, kb_hi);
        for (int kb = kb_lo; kb < kb_hi; ++it) {
          const int len = step_blocks<DUAL>(kb, kb_hi, part_len);
          const uint32_t bytes = (DUAL ? 2 : len) * C::kABytes + (DUAL ? 1 : len) * n16 * 2048;
          PROBE_START(t_stage);
          if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + s, ph ^ 1u, s_abort))) {
            if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 1); *s_abort = 1; }
            ok = false;
            break;
          }
          PROBE_ADD(probe_stage, t_stage);
          uint8_t* st = stages + s * C::kStageBytes;
          if (elect_one()) {
            mbar_expect_tx(bar_full + s, bytes);
            uint8_t* sb = st + 2 * C::kABytes;
            tma_load_2d(st, ma, kb * 128, wrow, bar_full + s, pol_w);
            if constexpr (DUAL) {
              tma_load_2d(st + C::kABytes, mb, kb * 128, wrow, bar_full + s, pol_w);
            } else if (len == 2) {
              tma_load_2d(st + C::kABytes, ma, (kb + 1) * 128, wrow, bar_full + s, pol_w);
              for (int j = 0; j < n16; ++j)
                tma_load_2d(sb + C::kBBytes + j * 2048, &tm_x, (kb + 1) * 128, ch.row0 + j * 16, bar_full + s, pol_x);
            }
            for (int j = 0; j < n16; ++j) tma_load_2d(sb + j * 2048, &tm_x, kb * 128, ch.row0 + j * 16, bar_full + s, pol_x);
            *s_issued = it + 1;
          }
          __syncwarp();
          if (++s == static_cast<uint32_t>(S)) { s = 0; ph ^= 1u; }
          kb += len;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    // The whole warp runs the loop with warp-uniform values (work item, stage, descriptors) and
    // one elected lane issues: operands of tcgen05.mma live in uniform registers, and a loop run
    // by a single diverged lane had to move every descriptor there per instruction, which made
    // the issue path, not HBM, set the pace of the down GEMM.
    {
      uint32_t it = 0, s = 0, ph = 0;
      bool ok = true;
      PROBE_DECL(probe_acc);
      PROBE_DECL(probe_data);
      for (uint32_t item = 0; ok; ++item) {
        int u = -1;
        Chunk ch;
        if (!__all_sync(0xffffffffu, take_item(s_queue, bar_qfull, bar_qempty, item, s_abort, u, ch))) {
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 8); *s_abort = 1; }
          break;
        }
        if (u < 0) {
          if (lane == 0) { PROBE_FLUSH_ROLE(p.status, 3, probe_acc); PROBE_FLUSH_ROLE(p.status, 4, probe_data); }
          break;
        }
        const uint32_t idesc = idesc_e4m3(128, ((ch.rows + 15) >> 4) * 16);
        int kb_lo, kb_hi;
        item_range(ch.pad, kb_lo, kb_hi);
        for (int kb = kb_lo; kb < kb_hi; ++it) {
          const int len = step_blocks<DUAL>(kb, kb_hi, part_len);
          const uint32_t as = it % C::kAcc, aph = (it / C::kAcc) & 1u;
          PROBE_START(t_acc);
          bool got = mbar_wait(bar_tempty + as, aph ^ 1u, s_abort);
          PROBE_ADD(probe_acc, t_acc);
          PROBE_START(t_data);
          got = got && mbar_wait(bar_full + s, ph, s_abort);
          PROBE_ADD(probe_data, t_data);
          if (!__all_sync(0xffffffffu, got)) {      // one decision for the warp
            if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 2); *s_abort = 1; }
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(stages + s * C::kStageBytes);
          const uint32_t d0 = tmem + as * C::kAccCols;
          if (elect_one()) {
            *s_consumed = it + 1;
            // every operand descriptor of the stage is the first one plus a constant (the start
            // address field counts 16-byte units and no sum leaves it): fewer instructions for
            // the one lane whose instruction stream feeds the tensor pipe
            const uint64_t desc0 = smem_desc_sw128(sa);
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              const uint64_t ad = desc0 + ((k4 * 32) >> 4);
              const uint64_t bd = ad + ((2 * C::kABytes) >> 4);
              mma_f8(d0, ad, bd, idesc, k4 > 0 ? 1u : 0u);
              if constexpr (DUAL) {
                mma_f8(d0 + NT, ad + (C::kABytes >> 4), bd, idesc, k4 > 0 ? 1u : 0u);
              } else if (len == 2) {     // the next K block: its own weight tile, token tile and accumulator
                mma_f8(d0 + NT, ad + (C::kABytes >> 4), bd + (C::kBBytes >> 4), idesc, k4 > 0 ? 1u : 0u);
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
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------ scale loader ------------------------------
    // Each lane waits, loads its share and arrives on its own: no warp-level sync, so a lane that
    // gives up cannot strand the others.
    int ready_chunk = -1;      // the chunk this lane has already seen complete
    for (uint32_t un = 0;; ++un) {
      const uint32_t b = un & 1u, ph = (un >> 1) & 1u;
      int u = -1;
      Chunk ch;
      if (!take_item(s_queue, bar_qfull, bar_qempty, un, s_abort, u, ch) ||
          (u >= 0 && !mbar_wait(bar_scempty + b, ph ^ 1u, s_abort)) ||
          // the previous GEMM's scales of this chunk must be complete (this lane's own acquire)
          (u >= 0 && handover && u / p.tiles_m != ready_chunk &&
           !wait_counter(p.progress + u / p.tiles_m, p.tiles_before, s_abort))) {
        if (!*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 4); *s_abort = 1; }
        break;
      }
      if (u < 0) break;
      ready_chunk = u / p.tiles_m;
      const int mt = u % p.tiles_m;
      const bool shared_e = ch.expert >= p.n_local;
      // The table [kb][NT]: the token's scale (gate/up), or its product with the weight block's scale (down)
      float* ta = s_scales + b * sf;
      float* ws = ta + KB * NT;                                      // gate/up: weight scales [2][kb]
      int* sd = reinterpret_cast<int*>(ws + C::weight_scale_floats(KB));   // [NT] destination row of every token column
      const int cols = ((ch.rows + 15) >> 4) * 16;
      if constexpr (!DUAL) {
        for (int n = lane; n < NT; n += 32)
          sd[n] = n < ch.rows ? (p.row_dest ? p.row_dest[ch.row0 + n] : ch.row0 + n) : 0;
        if (p.ret.base[0]) {
          // expert-parallel return: where every row of the chunk goes home to (its source's slot buffer)
          unsigned long long* sp = reinterpret_cast<unsigned long long*>(sd + NT);
          const int kept = p.ret.offsets[p.ret.n_local];
          for (int n = lane; n < NT; n += 32) {
            unsigned long long at = 0;
            if (n < ch.rows) {
              const int pos = ch.row0 + n;
              const int src = p.ret.row_source[pos];
              const bool routed = pos < kept;
              const int owner = routed ? src / p.ret.cap : p.ret.rank;
              const size_t slot = routed ? static_cast<size_t>(p.ret.recv_slot[src])
                                         : static_cast<size_t>(p.ret.home_tokens) * p.ret.topk + src;
              uint8_t* peer = p.ret.base[0];
#pragma unroll
              for (int r = 1; r < 8; ++r) peer = owner == r ? p.ret.base[r] : peer;
              at = reinterpret_cast<unsigned long long>(peer + p.ret.off_slots + slot * p.m * 2);
            }
            sp[n] = at;
          }
        }
      }
      int kb_lo, kb_hi;
      item_range(ch.pad, kb_lo, kb_hi);
      const int nk = kb_hi - kb_lo;
      const float* wa = (shared_e ? p.s_a_scale : p.w_a_scale + static_cast<size_t>(ch.expert) * p.tiles_m * KB) +
                        static_cast<size_t>(mt) * KB;
      const float* wb = wa;
      if constexpr (DUAL)
        wb = (shared_e ? p.s_b_scale : p.w_b_scale + static_cast<size_t>(ch.expert) * p.tiles_m * KB) +
             static_cast<size_t>(mt) * KB;
      // Token scales are read at L2: a line shared with a neighbouring chunk may have been fetched
      // before that chunk's scales were written.
      if (((KB | kb_lo | nk) & 3) == 0) {
        // a lane takes a row (the transposed stores then fall in different banks), four K blocks
        // per load, eight loads in flight
        const int quads = nk >> 2;
        const float4* wa4 = reinterpret_cast<const float4*>(wa + kb_lo);
        for (int n = lane; n < cols; n += 32) {
          const bool live = n < ch.rows;
          const float4* src =
              reinterpret_cast<const float4*>(p.act_scale + static_cast<size_t>(ch.row0 + (live ? n : 0)) * KB + kb_lo);
          for (int q0 = 0; q0 < quads; q0 += 8) {
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              v[j] = __ldcg(src + min(q0 + j, quads - 1));
              if (!live) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (q0 + j < quads) {
                float* dst = ta + (kb_lo + 4 * (q0 + j)) * NT + n;
                const float4 a4 = DUAL ? make_float4(1.f, 1.f, 1.f, 1.f) : __ldg(wa4 + q0 + j);
                dst[0] = __fmul_rn(a4.x, v[j].x);
                dst[NT] = __fmul_rn(a4.y, v[j].y);
                dst[2 * NT] = __fmul_rn(a4.z, v[j].z);
                dst[3 * NT] = __fmul_rn(a4.w, v[j].w);
              }
            }
          }
        }
      } else {
        for (int i = lane; i < cols * nk; i += 32) {
          const int n = i / nk, kb = kb_lo + i - n * nk;
          const float x = n < ch.rows ? __ldcg(p.act_scale + static_cast<size_t>(ch.row0 + n) * KB + kb) : 0.f;
          ta[kb * NT + n] = DUAL ? x : __fmul_rn(__ldg(wa + kb), x);
        }
      }
      if constexpr (DUAL) {
        for (int kb = kb_lo + lane; kb < kb_hi; kb += 32) {
          ws[kb] = wa[kb];
          ws[KB + kb] = wb[kb];
        }
      }
      mbar_arrive(bar_scfull + b);
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int epi = warp - 3;
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
    const int m = quarter * 32 + lane;            // output channel inside the tile
    const int group = epi >> 2;                   // with 8 epilogue warps: which share of the token columns
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    uint32_t it = 0;
    bool failed = false;
    PROBE_DECL(probe_tfull);
    PROBE_DECL(probe_scales);
    PROBE_DECL(probe_read);
    PROBE_DECL(probe_release);
    PROBE_DECL(probe_fold);
    PROBE_DECL(probe_close);
    for (uint32_t un = 0;; ++un) {
      int u = -1;
      Chunk ch;
      if (!take_item(s_queue, bar_qfull, bar_qempty, un, s_abort, u, ch)) {
        if (!*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 9); *s_abort = 1; }
        failed = true;
      }
      // one decision for all epilogue threads (the item is the same for all of them unless one failed)
      if (epilogue_any<C::kEpiThreads>(failed) || u < 0) {
        if (threadIdx.x == 96) {
          PROBE_FLUSH(p.status, 5, probe_tfull);
          PROBE_FLUSH_ROLE(p.status, 6, probe_scales);
          PROBE_FLUSH_EPI(p.status, 2, probe_read);
          PROBE_FLUSH_EPI(p.status, 3, probe_release);
          PROBE_FLUSH_EPI(p.status, 4, probe_fold);
          PROBE_FLUSH_EPI(p.status, 6, probe_close);
        }
        break;
      }
      const int mt = u % p.tiles_m;
      const int cols = ((ch.rows + 15) >> 4) * 16;            // token columns that were multiplied
      // This thread's columns [col0, cend): two warp groups share the columns the item really has
      // (16/16 of 32, 32/16 of 48, 32/32 of 64), one group takes them all with 4 epilogue warps.
      const int split = cols <= 32 ? 16 : 32;
      const int col0 = group ? split : 0;
      const int cend = (C::kEpiWarps == 8 && group == 0) ? min(split, cols) : cols;
      const int rend = min(ch.rows, cend);                     // ... and the rows among them that exist
      const uint32_t b = un & 1u, sph = (un >> 1) & 1u;
      const float* tab = s_scales + b * sf;         // [kb][NT]: token scales (gate/up) or scale products (down)
      const float* ws = tab + KB * NT;              // gate/up: weight scales [2][kb]
      const int* sd = reinterpret_cast<const int*>(ws + C::weight_scale_floats(KB));
      // down GEMM of an expert-parallel call: the rows' addresses in their sources' slot buffers
      const unsigned long long* sp = (!DUAL && p.ret.base[0]) ? reinterpret_cast<const unsigned long long*>(sd + NT) : nullptr;
      PROBE_START(t_scales);
      if (!failed && !mbar_wait(bar_scfull + b, sph, s_abort)) {
        if (!*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 5); *s_abort = 1; }
        failed = true;
      }
      PROBE_ADD(probe_scales, t_scales);
      float acc_a[C::kCpt];
      float acc_b[C::kCpt];
#pragma unroll
      for (int n = 0; n < C::kCpt; ++n) { acc_a[n] = 0.f; acc_b[n] = 0.f; }
      int kb_lo, kb_hi;
      item_range(ch.pad, kb_lo, kb_hi);
      // one CTA runs every part of a split contraction: acc_a restarts at each part's first K
      // block and acc_b (unused by the down GEMM otherwise) keeps the sum of the finished parts
      const bool parts_here = !DUAL && ksplit > 1 && !spread;
      for (int kb = kb_lo; kb < kb_hi; ++it) {
        const int len = step_blocks<DUAL>(kb, kb_hi, part_len);
        const bool second = DUAL || len == 2;          // the step's second accumulator holds something
        const uint32_t as = it % C::kAcc, aph = (it / C::kAcc) & 1u;
        PROBE_START(t_tfull);
        if (!failed && !mbar_wait(bar_tfull + as, aph, s_abort)) {
          if (!*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 3); *s_abort = 1; }
          failed = true;
        }
        PROBE_ADD(probe_tfull, t_tfull);
        if (failed) { kb += len; continue; }   // keep in step with the other epilogue threads up to the item's end
        tc_fence_after();
        PROBE_START(t_read);
        const bool active = col0 < cend;      // uniform per warp
        uint32_t ra[C::kCpt], rb[C::kCpt];
        if (active) {
          const uint32_t t0 = lane_base + as * C::kAccCols + col0;
#pragma unroll
          for (int g = 0; g < C::kCpt; g += 16) {
            if (col0 + g < cend) {
              tmem_ld16(t0 + g, ra + g);
              if (second) tmem_ld16(t0 + NT + g, rb + g);
            }
          }
          tmem_wait_ld();
        }
        // The values are in registers: hand the accumulators back before folding them, which
        // shortens the round trip that bounds the K blocks per microsecond.
        PROBE_ADD(probe_read, t_read);
        PROBE_START(t_release);
        tc_fence_before();
        mbar_arrive(bar_tempty + as);
        if (m == 0 && epi < 4) *s_drained = it + 1;
        PROBE_ADD(probe_release, t_release);
        PROBE_START(t_fold);
        if (active) {
          // acc += D * (w_scale * x_scale), the product rounded once. Gate/up: gate and up of K block
          // kb share the token scales, the two products are formed here. Down: K blocks kb and kb + 1,
          // folded one after the other into the same sums, their products read from the table.
          const float* sa = tab + kb * NT + col0;
#pragma unroll
          for (int g = 0; g < C::kCpt; g += 16) {
            if (col0 + g < cend) {
              // 16 table entries as four 16-byte loads (col0 and NT are multiples of 16), two columns per instruction
              float s16[16];
#pragma unroll
              for (int j = 0; j < 16; j += 4)
                *reinterpret_cast<float4*>(s16 + j) = *reinterpret_cast<const float4*>(sa + g + j);
              if constexpr (DUAL) {
                const float wa = ws[kb], wb = ws[KB + kb];
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                  float s0, s1;
                  mul2(wa, wa, s16[j], s16[j + 1], s0, s1);
                  fma2(__uint_as_float(ra[g + j]), __uint_as_float(ra[g + j + 1]), s0, s1, acc_a[g + j], acc_a[g + j + 1]);
                }
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                  float s0, s1;
                  mul2(wb, wb, s16[j], s16[j + 1], s0, s1);
                  fma2(__uint_as_float(rb[g + j]), __uint_as_float(rb[g + j + 1]), s0, s1, acc_b[g + j], acc_b[g + j + 1]);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; j += 2)
                  fma2(__uint_as_float(ra[g + j]), __uint_as_float(ra[g + j + 1]), s16[j], s16[j + 1], acc_a[g + j], acc_a[g + j + 1]);
                if (second) {
#pragma unroll
                  for (int j = 0; j < 16; j += 4)
                    *reinterpret_cast<float4*>(s16 + j) = *reinterpret_cast<const float4*>(sa + NT + g + j);
#pragma unroll
                  for (int j = 0; j < 16; j += 2)
                    fma2(__uint_as_float(rb[g + j]), __uint_as_float(rb[g + j + 1]), s16[j], s16[j + 1], acc_a[g + j], acc_a[g + j + 1]);
                }
              }
            }
          }
          if constexpr (!DUAL) {
            const int last = kb + len;          // K blocks folded so far
            if (parts_here && (last % part_len == 0 || last == KB)) {   // a part ends here
#pragma unroll
              for (int n = 0; n < C::kCpt; ++n) {
                acc_b[n] = __fadd_rn(acc_b[n], acc_a[n]);
                acc_a[n] = 0.f;
              }
            }
          }
        }
        PROBE_ADD(probe_fold, t_fold);
        kb += len;
      }
      PROBE_START(t_close);
      // One decision for all epilogue threads: nobody may be left alone at a later barrier.
      if (epilogue_any<C::kEpiThreads>(failed || *s_abort)) break;
      if constexpr (DUAL) {
        epilogue_swiglu_requant_tile<C::kCpt, C::kEpiThreads>(acc_a, acc_b, static_cast<int>(threadIdx.x) - 96, m, col0, NT,
                                                              rend, ch.rows, ch.row0, mt, p.m, s_amax, s_amax + 4 * NT,
                                                              s_tile, p.aq, p.as, p.swiglu);
        // Every epilogue thread's stores precede the closing barrier of the call above, so one
        // thread's fence and release cover them all (the readers are plain loads and TMA).
        if (p.progress && epi == 0 && lane == 0) {
          __threadfence();
          fence_async_global();
          atomicAdd(p.progress + u / p.tiles_m, 1);
        }
      } else {
        if (spread) {
          // This part's fp32 sums go to global memory; the CTA that finishes a tile's last part adds
          // all parts in part order (so the result does not depend on which one that is) and rounds.
          // (destination rows were staged by the scale loader together with the scales)
          const size_t tile_floats = static_cast<size_t>(NT) * 128;
          float* parts = p.partial + static_cast<size_t>(u) * ksplit * tile_floats;
#pragma unroll
          for (int n = 0; n < C::kCpt; ++n)
            if (col0 + n < rend) __stcg(parts + ch.pad * tile_floats + (col0 + n) * 128 + m, acc_a[n]);
          epilogue_sync<C::kEpiThreads>();
          if (epi == 0 && lane == 0) {
            __threadfence();      // after the barrier: this one fence and release cover every thread's stores
            const int before = atomicAdd(p.parts_done + u, 1);
            __threadfence();
            *s_last_part = before == ksplit - 1 ? 1 : 0;
          }
          epilogue_sync<C::kEpiThreads>();
          if (*s_last_part) {
            // eight columns at a time: the loads of all their parts are issued before the first sum (one
            // dependent load per addition made this a chain of columns x parts L2 latencies, 45 us for a
            // 16-row chunk of the Mixtral shape)
            float sums[C::kCpt];
            constexpr int kBatch = 8, kBatchParts = 4;
#pragma unroll
            for (int n0 = 0; n0 < C::kCpt; n0 += kBatch) {
              float v[kBatch][kBatchParts];
#pragma unroll
              for (int c = 0; c < kBatch; ++c)
#pragma unroll
                for (int q = 0; q < kBatchParts; ++q) {
                  const bool live = col0 + n0 + c < rend && q < ksplit;
                  v[c][q] = __ldcg(parts + (live ? q : 0) * tile_floats + (live ? col0 + n0 + c : 0) * 128 + m);
                }
#pragma unroll
              for (int c = 0; c < kBatch; ++c) {
                float sum = 0.f;
                if (col0 + n0 + c < rend) {
#pragma unroll
                  for (int q = 0; q < kBatchParts; ++q)
                    if (q < ksplit) sum = __fadd_rn(sum, v[c][q]);
                  for (int part = kBatchParts; part < ksplit; ++part)
                    sum = __fadd_rn(sum, __ldcg(parts + part * tile_floats + (col0 + n0 + c) * 128 + m));
                }
                sums[n0 + c] = sum;
              }
            }
            epilogue_store_tile<C::kCpt, C::kEpiThreads>(sums, static_cast<int>(threadIdx.x) - 96, m, col0, rend, ch.rows, mt,
                                                         p.m, sd, reinterpret_cast<__nv_bfloat16*>(s_tile), p.out, sp);
          }
        } else {
          // one bf16 rounding of the fp32 sum (megabench/tasks/megamoe.py:149)
          if (parts_here)
            epilogue_store_tile<C::kCpt, C::kEpiThreads>(acc_b, static_cast<int>(threadIdx.x) - 96, m, col0, rend, ch.rows, mt,
                                                         p.m, sd, reinterpret_cast<__nv_bfloat16*>(s_tile), p.out, sp);
          else
            epilogue_store_tile<C::kCpt, C::kEpiThreads>(acc_a, static_cast<int>(threadIdx.x) - 96, m, col0, rend, ch.rows, mt,
                                                         p.m, sd, reinterpret_cast<__nv_bfloat16*>(s_tile), p.out, sp);
        }
      }
      PROBE_ADD(probe_close, t_close);
      mbar_arrive(bar_scempty + b);   // this item's scales are no longer needed
    }
  }

  // ------------------------------ common exit ---------------------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
#if !defined(MOE_TIMELINE) || MOE_TIMELINE == 1
  if (threadIdx.x == 0) MOE_STAMP_LAST(p.status, DUAL ? 6 : 7);
#endif
  if (threadIdx.x == 0) {
    PROBE_DECL(probe_cta);
    PROBE_ADD(probe_cta, t_cta);
    PROBE_FLUSH(p.status, 7, probe_cta);
  }
  if (*s_abort && threadIdx.x == 0) {
    // Give copies and MMAs that were issued but never consumed a bounded chance to land.
    for (uint32_t it = *s_consumed; it < *s_issued; ++it) mbar_wait(bar_full + it % S, (it / S) & 1u);
    for (uint32_t it = *s_drained; it < *s_committed; ++it) mbar_wait(bar_tfull + it % C::kAcc, (it / C::kAcc) & 1u);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
  }
  if constexpr (!DUAL) {
    if (p.fold.y) {
      // Small batches: the combine without a launch of its own. Every CTA of this grid is resident
      // (at most one per SM, and nothing it waits for depends on a CTA that is not), so the grid can
      // meet here: each CTA announces that its slot rows are stored, waits (bounded) for all the
      // others, and then adds up its share of the output in slot order, the combine kernel's
      // arithmetic on the same stored rows.
      if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(p.fold.count, 1);
        if (!wait_counter(p.fold.count, static_cast<int>(gridDim.x))) report(p.status, MOE_ERR_DEVICE_TIMEOUT, 10);
        __threadfence();
      }
      __syncthreads();
      const int vectors = p.m / 8;                      // 8 channels per thread
      const int routed = p.fold.tokens * p.fold.topk;
      for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < p.fold.tokens * vectors; v += gridDim.x * blockDim.x) {
        const int t = v / vectors, c = (v - t * vectors) * 8;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        // eight slots' loads are issued before the first addition; the additions keep the slot order
        for (int s0 = 0; s0 < p.fold.topk; s0 += 8) {
          uint4 raw[8];
          float w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const size_t row = static_cast<size_t>(t) * p.fold.topk + min(s0 + j, p.fold.topk - 1);
            w[j] = p.fold.weights ? p.fold.weights[row] : 1.f;
            raw[j] = __ldcg(reinterpret_cast<const uint4*>(p.out + row * p.m + c));
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (s0 + j < p.fold.topk) {
              const __nv_bfloat16* x8 = reinterpret_cast<const __nv_bfloat16*>(&raw[j]);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(__bfloat162float(x8[i]), w[j]));
            }
          }
        }
        if (p.fold.shared) {
          const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p.out + (static_cast<size_t>(routed) + t) * p.m + c));
          const __nv_bfloat16* x8 = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __bfloat162float(x8[i]));
        }
        uint4 packed;
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(acc[i]);
        if (p.fold.residual) {
          const uint4 raw = *reinterpret_cast<const uint4*>(p.fold.residual + static_cast<size_t>(t) * p.m + c);
          const __nv_bfloat16* x8 = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(__fadd_rn(__bfloat162float(x8[i]), __bfloat162float(o[i])));
        }
        *reinterpret_cast<uint4*>(p.fold.y + static_cast<size_t>(t) * p.m + c) = packed;
      }
    }
  }
  if constexpr (!DUAL) {
    if (p.ret.base[0] && threadIdx.x == 0) {
      // Expert-parallel return: every row this CTA stored into a peer's slot buffer precedes the
      // barrier above; one system-wide fence covers them, and the CTA that is through last tells every
      // source that this owner's rows are home.
      __threadfence_system();
      if (atomicAdd(p.ret.done, 1) == static_cast<int>(gridDim.x) - 1) {
        __threadfence_system();
        for (int r = 0; r < p.ret.world; ++r) {
          uint8_t* peer = p.ret.base[0];
#pragma unroll
          for (int q = 1; q < 8; ++q) peer = r == q ? p.ret.base[q] : peer;
          store_release_sys(reinterpret_cast<uint64_t*>(peer + p.ret.off_flags) + p.ret.rank, p.ret.epoch);
        }
        *p.ret.done = 0;
      }
    }
  }
  // Keep the stream's ordering for whatever follows: this grid does not complete before the
  // gate/up grid has (a CTA that found the dispenser empty idles here until that grid's last
  // tiles are done; one that did work finds it finished).
  if (handover && threadIdx.x == 0) dependent_wait();
}

// ---------------------------------------------------------------------------------------
// Host side: tensor maps and launch.
// ---------------------------------------------------------------------------------------
template <int NT, bool DUAL>
static cudaError_t launch_typed(GemmDev dev, const CUtensorMap* maps, int grid, cudaStream_t stream) {
  using C = GemmCfg<NT, DUAL>;
  static bool configured[64] = {};      // the attribute belongs to the device the call runs on
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<NT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kMaxSmem);
    if (e != cudaSuccess) return e;
    if (device >= 0 && device < 64) configured[device] = true;
  }
  const int cap = dev.stages;           // the caller's cap, 0 = none
  dev.stages = C::stages_for(dev.kblocks);
  if (cap > 0 && cap < dev.stages) dev.stages = cap;
  if (dev.stages < 2) return cudaErrorInvalidValue;
  const int smem = 1024 + dev.stages * C::kStageBytes + C::tail_bytes(dev.kblocks);
  return launch_dependent(grouped_gemm_kernel<NT, DUAL>, dim3(grid), dim3(C::kThreads), smem, stream, maps[0], maps[1],
                          maps[2], maps[3], maps[4], dev);
}

cudaError_t launch_gemm_tc(const GemmArgs& a, cudaStream_t stream, int* launches, int* driver_error) {
  if (a.k % 128 || a.m % 128 || a.k / 128 > kMaxKBlocks) return cudaErrorInvalidValue;
  CUtensorMap maps[5];
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
  rc |= make_map(&maps[4], a.act, a.total_rows, a.k, 16);      // token rows move in boxes of 16
  if (rc) {
    if (driver_error) *driver_error = rc;
    return cudaErrorUnknown;
  }
  GemmDev dev{a.chunks, a.n_chunks, a.m / 128, a.k / 128, a.m, a.n_local, a.max_stages, a.act_scale, a.w_a_scale, a.w_b_scale,
              a.s_a_scale, a.s_b_scale, a.aq, a.as, a.out, a.row_dest, a.status, a.progress, a.max_chunks,
              a.tiles_before, 1, nullptr, nullptr, a.swiglu, a.dual ? FoldCombine{} : a.fold, a.dual ? PeerReturn{} : a.ret};
  if (!a.dual && a.ksplit > 1) {
    const int per = (a.k / 128 + a.ksplit - 1) / a.ksplit;
    if (!a.partial || !a.parts_done || (a.ksplit - 1) * per >= a.k / 128 || a.ksplit > 255) return cudaErrorInvalidValue;
    dev.ksplit = a.ksplit;
    dev.partial = a.partial;
    dev.parts_done = a.parts_done;
  }
  const long long units = static_cast<long long>(a.max_units) * dev.ksplit;
  const int grid = static_cast<int>(max(1ll, min(static_cast<long long>(gemm_sm_count()), units)));
  cudaError_t e;
  if (a.dual) {
    e = a.tile == 16 ? launch_typed<16, true>(dev, maps, grid, stream)
      : a.tile == 32 ? launch_typed<32, true>(dev, maps, grid, stream)
                     : launch_typed<64, true>(dev, maps, grid, stream);
  } else {
    e = a.tile == 16 ? launch_typed<16, false>(dev, maps, grid, stream)
      : a.tile == 32 ? launch_typed<32, false>(dev, maps, grid, stream)
                     : launch_typed<64, false>(dev, maps, grid, stream);
  }
  if (launches) *launches += 1;
  return e;
}

}  // namespace moe
