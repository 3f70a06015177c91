// Persistent grouped GEMM for the MegaMoE-native formats on tcgen05 block-scaled tensor cores.
//
//   D[m, n] = sum over 32-wide K blocks b of  2^(sw[m,b]-127) * 2^(sx[n,b]-127) * sum_k W[m,k] * X[n,k]
//
// W: MXFP4 weights (E2M1 codes, two per byte, one E8M0 scale per 32 input channels,
// megabench/tasks/quantization.py:13-51); X: E4M3 token rows with one E8M0 scale per 32 channels
// (megabench/tasks/megamoe.py:37,125-128). `tcgen05.mma.kind::mxf8f6f4.block_scale` applies both
// scales inside the MMA (K = 32 per instruction = one scale block) and accumulates the whole
// contraction in one fp32 TMEM accumulator, so the epilogue reads each tile once.
//
// Orientation as in the FP8 kernel: weights are the M side (128 output channels per tile), the
// tokens of one expert the N side (16..NT columns). Weight tiles arrive by TMA with the
// 16U4_ALIGN16B element type, which expands the packed 4-bit codes to the one-byte-per-value
// layout the MMA reads from shared memory (HBM traffic stays 4 bits per weight).
//
// Scale factors live in TMEM next to the accumulators: per 128-wide K block 4 columns for the
// gate (or down) rows, 4 for the up rows, up to 2 for the tokens; row r of a tile sits in lane
// r % 32 (replicated in all four lane quarters), column r / 32, byte = 32-wide K block inside the
// 128-wide one. Four warps, one per lane quarter, bring them from global memory through a ring in
// shared memory (cp.async, several groups of four K blocks ahead) and store them with tcgen05.st,
// a group at a time.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 = scale writers,
// warps 6-9 = epilogue (a thread owns one output channel). Every wait is bounded: on expiry the
// role records MOE_ERR_DEVICE_TIMEOUT, raises the CTA's abort flag and all roles fall through to
// the common exit, which waits (bounded) for copies in flight and frees TMEM.
//
// Reference arithmetic: megabench/tasks/megamoe.py:131-150 (operands dequantised exactly to bf16,
// fp32 accumulation, bf16 results), :116-128 (clamped SwiGLU with the routing weight, E4M3
// requantisation with E8M0 scales per 32 channels).
#include "common.cuh"
#include "gemm_mx_common.cuh"
#include "kernels.h"
#include "split_e4m3.cuh"

namespace moe {

constexpr int kMxMaxStages = 12;
constexpr int kMxKPerStage = 2;       // K blocks per pipeline stage: one wait, one release per pair (divides kMxSfGroup)
constexpr int kMxThreads = 320;

template <int NT, bool DUAL>
struct MxCfg {
  static constexpr int kABytes = 128 * 128;     // one byte per value in shared memory
  static constexpr int kATxBytes = 128 * 64;    // what a weight tile counts on the mbarrier: the packed bytes it read
  static constexpr int kXBytes = NT * 128;
  static constexpr int kSubBytes = (DUAL ? 2 : 1) * kABytes + kXBytes;   // one K block of a stage
  static constexpr int kStageBytes = kMxKPerStage * kSubBytes;
  static constexpr int kAccCols = (DUAL ? 2 : 1) * NT;
  static constexpr int kBufCols = kAccCols;
  static constexpr int kSfBase = 2 * kBufCols;  // two accumulator buffers, then the scale factors
  static constexpr int kTailBytes = (2 * kMxMaxStages + 4 + 2 * kMxSfSlots) * 8 + 64;
  // a group's scale bytes in shared memory: 16 per tile row (gate/down, up), then 16 per token row
  static constexpr int kSfXOffset = (DUAL ? 2 : 1) * 2048;
  static constexpr int kSfSlotBytes = kSfXOffset + 1024;
  static constexpr int kFit = (kMxSmem - 1024 - kTailBytes - kMxSfRing * kSfSlotBytes) / kStageBytes;
  static constexpr int kStages = kFit < kMxMaxStages ? kFit : kMxMaxStages;
  static_assert(kSfBase + kMxSfSlots * kMxSfGroup * kMxSfCols <= 512, "TMEM columns");
};

struct MxDev {
  const Chunk* chunks;
  const int32_t* n_chunks;
  int tiles_m, kblocks, m;
  int rows_per_expert;        // rows of the weight matrix one expert owns (2I for linear1, H for linear2)
  int up_offset;              // DUAL: rows between a gate row and its up row (I)
  const uint8_t* w_scales;    // [experts * rows_per_expert, K/32]
  const uint8_t* x_scales;    // [rows, K/32]
  uint8_t* aq;                // DUAL: e4m3 [rows, m]
  uint8_t* as;                // DUAL: E8M0 [rows, m/32]
  __nv_bfloat16* out;         // single: bf16 rows [*, m] at row_dest
  const int32_t* row_dest;
  const float* slot_weight;   // DUAL: routing weight of slot row_dest[row] (NULL = 1)
  float limit;                // DUAL: clamp, 0 = none
  int32_t* status;
  const uint8_t* w_scales_b;  // DUAL: scales of the up rows when they are a tensor of their own (then tm_w2 maps it), else NULL
  int activation;             // DUAL: 0 = clamped SwiGLU, 1 = situ
  int pairs;                  // token columns 2j, 2j+1 are the two E4M3 pieces of one bf16 row
};

template <int NT, bool DUAL>
__global__ void __launch_bounds__(kMxThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_w2,
               const __grid_constant__ CUtensorMap tm_x, const MxDev p) {
  using C = MxCfg<NT, DUAL>;
  constexpr int S = C::kStages;
  constexpr int XC = NT > 32 ? NT / 32 : 1;       // scale columns of the token side
  extern __shared__ uint8_t smem_raw[];
  const int KB = p.kblocks;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stages = base;
  uint8_t* sf_ring = base + S * C::kStageBytes;                       // [kMxSfRing][kSfSlotBytes]
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(sf_ring + kMxSfRing * C::kSfSlotBytes);
  uint64_t* bar_empty = bar_full + kMxMaxStages;
  uint64_t* bar_tfull = bar_empty + kMxMaxStages;
  uint64_t* bar_tempty = bar_tfull + 2;
  uint64_t* bar_sffull = bar_tempty + 2;           // a group's scale factors are in TMEM
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
    for (int s = 0; s < 2; ++s) { mbar_init(bar_tfull + s, 1); mbar_init(bar_tempty + s, 128); }
    for (int s = 0; s < kMxSfSlots; ++s) { mbar_init(bar_sffull + s, 4); mbar_init(bar_sfempty + s, 1); }   // four scale warps
    *s_abort = 0; *s_issued = 0; *s_consumed = 0; *s_committed = 0; *s_drained = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tm_w); prefetch_tmap(&tm_x);
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
  const int n_units = *p.n_chunks * p.tiles_m;
  const int first = blockIdx.x, stride = gridDim.x;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    const uint64_t pol_w = policy_evict_first();
    const uint64_t pol_x = policy_evict_last();
    uint32_t it = 0, s = 0, ph = 0;
    bool ok = true;
    Chunk ahead = chunk_at(p.chunks, first, p.tiles_m, n_units);
    for (int u = first; ok && u < n_units; u += stride) {
      const Chunk ch = ahead;
      ahead = chunk_at(p.chunks, u + stride, p.tiles_m, n_units);
      const int mt = u % p.tiles_m;
      const int wrow = ch.expert * p.rows_per_expert + mt * 128;
      const int n16 = (ch.rows + 15) >> 4;
      const uint32_t bytes = (DUAL ? 2 : 1) * C::kATxBytes + n16 * 2048;      // per K block
      for (int kb0 = 0; kb0 < KB; kb0 += kMxKPerStage, ++it) {
        if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + s, ph ^ 1u, s_abort))) {
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 21); *s_abort = 1; }
          ok = false;
          break;
        }
        const int nk = min(kMxKPerStage, KB - kb0);
        if (elect_one()) {
          mbar_expect_tx(bar_full + s, bytes * nk);
          for (int kk = 0; kk < nk; ++kk) {
            uint8_t* st = stages + s * C::kStageBytes + kk * C::kSubBytes;
            const int kx = (kb0 + kk) * 128;
            if constexpr (DUAL) {
              if (p.w_scales_b) {     // gate and up rows in tensors of their own: two requests
                tma_load_2d(st, &tm_w, kx, wrow, bar_full + s, pol_w);
                tma_load_2d(st + C::kABytes, &tm_w2, kx, wrow, bar_full + s, pol_w);
              } else {
                tma_load_3d(st, &tm_w, kx, mt * 128, 2 * ch.expert, bar_full + s, pol_w);   // gate tile, then up tile
              }
            } else {
              tma_load_2d(st, &tm_w, kx, wrow, bar_full + s, pol_w);                        // x in 4-bit elements
            }
            uint8_t* sx = st + (DUAL ? 2 : 1) * C::kABytes;
            for (int j = 0; j < n16; ++j) tma_load_2d(sx + j * 2048, &tm_x, kx, ch.row0 + j * 16, bar_full + s, pol_x);
          }
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
    Chunk ahead = chunk_at(p.chunks, first, p.tiles_m, n_units);
    for (int u = first; ok && u < n_units; u += stride, ++item) {
      const Chunk ch = ahead;
      ahead = chunk_at(p.chunks, u + stride, p.tiles_m, n_units);
      const int n = ((ch.rows + 15) >> 4) * 16;
      const uint32_t idesc4[4] = {idesc_mx(n, 0), idesc_mx(n, 1), idesc_mx(n, 2), idesc_mx(n, 3)};
      const uint32_t ab = item & 1u, aph = (item >> 1) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty + ab, aph ^ 1u, s_abort))) {
        if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 22); *s_abort = 1; }
        break;
      }
      for (int kb0 = 0; kb0 < KB; kb0 += kMxKPerStage, ++it) {
        // a stage's K blocks lie inside one scale-factor group (kMxKPerStage divides kMxSfGroup)
        const uint32_t slot = gi % kMxSfSlots, in_group0 = kb0 % kMxSfGroup;
        const int nk = min(kMxKPerStage, KB - kb0);
        bool got = mbar_wait(bar_full + s, ph, s_abort);
        if (in_group0 == 0) got = got && mbar_wait(bar_sffull + slot, (gi / kMxSfSlots) & 1u, s_abort);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 23); *s_abort = 1; }
          ok = false;
          break;
        }
        tc_fence_after();
        const bool last = kb0 + nk == KB;
        const bool group_done = in_group0 + nk == kMxSfGroup || last;
        if (elect_one()) {
          *s_consumed = it + 1;
          // every operand descriptor of the stage is the first one plus a constant (the start
          // address field counts 16-byte units and no sum leaves it)
          const uint64_t desc0 = smem_desc_sw128(smem_u32(stages + s * C::kStageBytes));
          const uint32_t d0 = tmem + ab * C::kBufCols;
          const uint32_t sf0 = tmem + C::kSfBase + (slot * kMxSfGroup + in_group0) * kMxSfCols;
#pragma unroll
          for (int kk = 0; kk < kMxKPerStage; ++kk) {
            if (kk < nk) {
              const uint32_t sf = sf0 + kk * kMxSfCols;
#pragma unroll
              for (uint32_t k4 = 0; k4 < 4; ++k4) {
                const uint32_t acc = (kb0 + kk > 0 || k4 > 0) ? 1u : 0u;   // the item's first MMA overwrites
                const uint64_t ad = desc0 + ((kk * C::kSubBytes + k4 * 32) >> 4);
                const uint64_t xd = ad + (((DUAL ? 2 : 1) * C::kABytes) >> 4);
                mma_mx(d0, ad, xd, idesc4[k4], sf, sf + 8, acc);
                if constexpr (DUAL) mma_mx(d0 + NT, ad + (C::kABytes >> 4), xd, idesc4[k4], sf + 4, sf + 8, acc);
              }
            }
          }
          mma_commit(bar_empty + s);                 // the stage may be refilled once these MMAs are done
          if (group_done) mma_commit(bar_sfempty + slot);   // and the group's scale columns rewritten
          if (last) { mma_commit(bar_tfull + ab); *s_committed = item + 1; }
        }
        __syncwarp();
        if (group_done) ++gi;
        if (++s == S) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------ scale writers ------------------------------
    // A group = four K blocks = 16 scale bytes per row. The 128 threads copy the groups to come
    // into a ring in shared memory (cp.async, kMxSfAhead groups ahead across work items: thread t
    // takes tile row t of the weights, of the up rows, and token row t), so that the latency of
    // these small strided reads never meets the MMA. Then warp w fills lane quarter w % 4 of the
    // group's TMEM columns; the four warps store the same values (the MMA wants the scale of tile
    // row r in lane r % 32 of every quarter).
    const int t = static_cast<int>(threadIdx.x) - 64;      // 0..127
    const uint32_t quarter = warp & 3u;
    const int KS = KB * 4;                         // scale bytes per row
    const bool vec = (KS % 16) == 0;
    const int groups = (KB + 3) / 4;
    // the copies' own walk over (work item, group), kMxSfAhead groups ahead of the stores
    int iu = first, ig = 0;
    uint32_t issued = 0;
    Chunk ich = iu < n_units ? p.chunks[iu / p.tiles_m] : Chunk{0, 0, 0, 0};
    auto issue = [&]() {
      if (iu < n_units) {
        uint8_t* slot = sf_ring + (issued % kMxSfRing) * C::kSfSlotBytes;
        const size_t wrow = static_cast<size_t>(ich.expert) * p.rows_per_expert + (iu % p.tiles_m) * 128 + t;
        copy_scale_group(slot + t * 16, p.w_scales + wrow * KS, ig, KB, vec);
        if constexpr (DUAL)
          copy_scale_group(slot + 2048 + t * 16, p.w_scales_b ? p.w_scales_b + wrow * KS : p.w_scales + (wrow + p.up_offset) * KS,
                           ig, KB, vec);
        if (t < NT) {
          uint8_t* dst = slot + C::kSfXOffset + t * 16;
          if (t < ich.rows) copy_scale_group(dst, p.x_scales + static_cast<size_t>(ich.row0 + t) * KS, ig, KB, vec);
          else *reinterpret_cast<uint4*>(dst) = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);   // past the chunk: scale 1, results unused
        }
        if (++ig == groups) {
          ig = 0;
          iu += stride;
          if (iu < n_units) ich = p.chunks[iu / p.tiles_m];
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
          if (t == 0 && !*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 24); *s_abort = 1; }
          ok = false;
          break;
        }
        tc_fence_after();
        const uint8_t* src = sf_ring + (gi % kMxSfRing) * C::kSfSlotBytes;
        uint4 a[4], b[4], x[XC];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          a[c] = *reinterpret_cast<const uint4*>(src + (32 * c + lane) * 16);
          if constexpr (DUAL) b[c] = *reinterpret_cast<const uint4*>(src + 2048 + (32 * c + lane) * 16);
        }
#pragma unroll
        for (int c = 0; c < XC; ++c) x[c] = *reinterpret_cast<const uint4*>(src + C::kSfXOffset + (32 * c + lane) * 16);
        const uint32_t t0 = tmem + ((quarter * 32u) << 16) + C::kSfBase + slot * kMxSfGroup * kMxSfCols;
#define MX_WORD(v, j) ((j) == 0 ? (v).x : (j) == 1 ? (v).y : (j) == 2 ? (v).z : (v).w)
#pragma unroll
        for (int j = 0; j < 4; ++j) {              // a ragged last group stores spare columns nobody reads
          const uint32_t tj = t0 + j * kMxSfCols;
          tmem_st4(tj, MX_WORD(a[0], j), MX_WORD(a[1], j), MX_WORD(a[2], j), MX_WORD(a[3], j));
          if constexpr (DUAL) tmem_st4(tj + 4, MX_WORD(b[0], j), MX_WORD(b[1], j), MX_WORD(b[2], j), MX_WORD(b[3], j));
          tmem_st2(tj + 8, MX_WORD(x[0], j), MX_WORD(x[XC - 1], j));
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
    const int m = quarter * 32 + lane;             // channel inside the tile
    uint32_t item = 0;
    Chunk ahead = chunk_at(p.chunks, first, p.tiles_m, n_units);
    for (int u = first; u < n_units; u += stride, ++item) {
      const Chunk ch = ahead;
      ahead = chunk_at(p.chunks, u + stride, p.tiles_m, n_units);
      const int mt = u % p.tiles_m;
      const int n16 = (ch.rows + 15) >> 4;
      const uint32_t ab = item & 1u, aph = (item >> 1) & 1u;
      // Destination slot and routing weight of the chunk's rows, one row per lane (two rounds for
      // 64 columns), fetched while the MMAs still run; the column loop reads them by shuffle.
      int dest_of[XC];
      float weight_of[XC];
#pragma unroll
      for (int c = 0; c < XC; ++c) {
        const int col = 32 * c + lane;
        const int row = ch.row0 + col;
        dest_of[c] = col < ch.rows ? (p.row_dest ? p.row_dest[row] : row) : 0;
        weight_of[c] = (DUAL && p.slot_weight && col < ch.rows) ? p.slot_weight[dest_of[c]] : 1.f;
      }
      if (!mbar_wait(bar_tfull + ab, aph, s_abort)) {
        if (!*s_abort) { report(p.status, MOE_ERR_DEVICE_TIMEOUT, 25); *s_abort = 1; }
        break;
      }
      tc_fence_after();
      const uint32_t t = tmem + ((quarter * 32u) << 16) + ab * C::kBufCols;
      for (int j = 0; j < n16; ++j) {
        uint32_t g[16], v[16];
        tmem_ld16(t + j * 16, g);
        if constexpr (DUAL) tmem_ld16(t + NT + j * 16, v);
        tmem_wait_ld();
        if (j == n16 - 1) {                        // every column of this accumulator is in registers
          tc_fence_before();
          mbar_arrive(bar_tempty + ab);
          if (threadIdx.x == 6 * 32) *s_drained = item + 1;
        }
        if (p.pairs) {
          // columns 2q, 2q+1 are the two E4M3 pieces of one bf16 row: their results add up to that
          // row's (exact products either way, fp32 sums)
#pragma unroll
          for (int c = 0; c < 16; c += 2) {
            const int col = j * 16 + c;
            if (col >= ch.rows) break;             // uniform across the CTA
            const size_t row = static_cast<size_t>(ch.row0 + col);      // the hi piece's row; the lo piece follows
            const bool upper = XC > 1 && col >= 32;
            const int dest_here = __shfl_sync(0xffffffffu, upper ? dest_of[XC - 1] : dest_of[0], col & 31);
            if constexpr (DUAL) {
              const float gate = bf16_round(__fadd_rn(__uint_as_float(g[c]), __uint_as_float(g[c + 1])));
              const float up = bf16_round(__fadd_rn(__uint_as_float(v[c]), __uint_as_float(v[c + 1])));
              // megabench/tasks/kimi.py:134-135 (situ) or megabench/tasks/megamoe.py:116-122; one bf16 rounding
              float act;
              if (p.activation == 1) {
                act = situ_f32(gate, up);
              } else {
                float gc = gate, uc = up;
                if (p.limit > 0.f) { gc = fminf(gc, p.limit); uc = fminf(fmaxf(uc, -p.limit), p.limit); }
                act = __fmul_rn(__fdiv_rn(gc, __fadd_rn(1.f, expf(-gc))), uc);
              }
              const float one[1] = {bf16_round(act)};
              uint8_t hi[1], lo[1];
              int e_hi, e_lo;
              split_e4m3(one, 32, hi, lo, e_hi, e_lo);       // the warp's 32 channels are one scale block
              p.aq[row * p.m + mt * 128 + m] = hi[0];
              p.aq[(row + 1) * p.m + mt * 128 + m] = lo[0];
              if (lane == 0) {
                p.as[row * (p.m / 32) + mt * 4 + quarter] = static_cast<uint8_t>(e_hi);
                p.as[(row + 1) * (p.m / 32) + mt * 4 + quarter] = static_cast<uint8_t>(e_lo);
              }
            } else {
              p.out[static_cast<size_t>(dest_here >> 1) * p.m + mt * 128 + m] =
                  __float2bfloat16_rn(__fadd_rn(__uint_as_float(g[c]), __uint_as_float(g[c + 1])));
            }
          }
          continue;
        }
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const int col = j * 16 + c;
          if (col >= ch.rows) break;               // uniform across the CTA
          const size_t row = static_cast<size_t>(ch.row0 + col);
          const bool upper = XC > 1 && col >= 32;
          const int dest_here = __shfl_sync(0xffffffffu, upper ? dest_of[XC - 1] : dest_of[0], col & 31);
          const float weight_here = __shfl_sync(0xffffffffu, upper ? weight_of[XC - 1] : weight_of[0], col & 31);
          if constexpr (DUAL) {
            // megabench/tasks/megamoe.py:116-122: bf16 GEMM outputs, clamp, fp32 SwiGLU, routing weight
            float gate = bf16_round(__uint_as_float(g[c]));
            float up = bf16_round(__uint_as_float(v[c]));
            if (p.limit > 0.f) {
              gate = fminf(gate, p.limit);
              up = fminf(fmaxf(up, -p.limit), p.limit);
            }
            float act = __fmul_rn(__fdiv_rn(gate, __fadd_rn(1.f, expf(-gate))), up);
            if (p.slot_weight) act = __fmul_rn(act, weight_here);
            // megabench/tasks/quantization.py:62-84: the warp's 32 channels are one scale block
            const unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(act)));
            const int exponent = max((static_cast<int>(bits) + (0x7FFFFF - 0x600000)) >> 23, 105 + 8) - 8;
            const float inverse = __int_as_float((254 - exponent) << 23);
            p.aq[row * p.m + mt * 128 + m] =
                static_cast<uint8_t>(__nv_cvt_float_to_fp8(__fmul_rn(act, inverse), __NV_SATFINITE, __NV_E4M3));
            if (lane == 0) p.as[row * (p.m / 32) + mt * 4 + quarter] = static_cast<uint8_t>(exponent);
          } else {
            // one bf16 rounding of the fp32 sum (megabench/tasks/megamoe.py:149)
            p.out[static_cast<size_t>(dest_here) * p.m + mt * 128 + m] = __float2bfloat16_rn(__uint_as_float(g[c]));
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
    for (uint32_t it = *s_drained; it < *s_committed; ++it) mbar_wait(bar_tfull + (it & 1u), (it >> 1) & 1u);
    // how far the roles of the first CTA that gave up had come (spare status words)
    if (atomicCAS(p.status + 2, 0, 1 + static_cast<int>(blockIdx.x)) == 0) {
      p.status[3] = *s_issued; p.status[4] = *s_consumed; p.status[5] = *s_committed; p.status[6] = *s_drained;
      p.status[7] = DUAL ? 1 : 2;
    }
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
template <int NT, bool DUAL>
static cudaError_t mx_launch_typed(const MxDev& dev, const CUtensorMap* maps, int grid, cudaStream_t stream) {
  using C = MxCfg<NT, DUAL>;
  static bool configured[64] = {};      // the attribute belongs to the device the call runs on
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    cudaError_t e = cudaFuncSetAttribute(mx_gemm_kernel<NT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMxSmem);
    if (e != cudaSuccess) return e;
    if (device >= 0 && device < 64) configured[device] = true;
  }
  constexpr int smem = 1024 + C::kStages * C::kStageBytes + kMxSfRing * C::kSfSlotBytes + C::kTailBytes;
  static_assert(smem <= kMxSmem, "shared memory of one CTA");
  return launch_dependent(mx_gemm_kernel<NT, DUAL>, dim3(grid), dim3(kMxThreads), smem, stream, maps[0], maps[2], maps[1], dev);
}

cudaError_t launch_gemm_mx(const MxGemmArgs& a, cudaStream_t stream, int* launches, int* driver_error) {
  if (a.tile == 128) return launch_gemm_mx_wide(a, stream, launches, driver_error);
  if (a.k % 128 || a.m % 128 || a.n_experts < 1 || (a.tile != 16 && a.tile != 32 && a.tile != 64)) return cudaErrorInvalidValue;
  const bool apart = a.dual && a.w_blocks_b != nullptr;      // gate and up rows in tensors of their own
  if (apart != (a.dual && a.w_scales_b != nullptr) || (a.pairs && a.tile % 2)) return cudaErrorInvalidValue;
  const int rows_per_expert = (a.dual && !apart) ? 2 * a.m : a.m;
  CUtensorMap maps[3];
  int rc = (a.dual && !apart) ? mx_make_pair_map(&maps[0], a.w_blocks, a.n_experts, a.m, a.k)
                              : mx_make_map(&maps[0], a.w_blocks, static_cast<uint64_t>(a.n_experts) * rows_per_expert, a.k, true, 128);
  rc = rc ? rc : mx_make_map(&maps[1], a.act, a.total_rows, a.k, false, 16);      // token rows move in boxes of 16
  if (apart) rc = rc ? rc : mx_make_map(&maps[2], a.w_blocks_b, static_cast<uint64_t>(a.n_experts) * a.m, a.k, true, 128);
  else maps[2] = maps[0];
  if (rc) {
    if (driver_error) *driver_error = rc;
    return cudaErrorUnknown;
  }
  MxDev dev{a.chunks, a.n_chunks, a.m / 128, a.k / 128, a.m, rows_per_expert, a.dual ? a.m : 0, a.w_scales, a.act_scales,
            a.aq, a.as, a.out, a.row_dest, a.slot_weight, a.limit, a.status, apart ? a.w_scales_b : nullptr, a.activation,
            a.pairs ? 1 : 0};
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int grid = max(1, min(sms, a.max_units));
  cudaError_t e;
  if (a.dual) {
    e = a.tile == 16 ? mx_launch_typed<16, true>(dev, maps, grid, stream)
      : a.tile == 32 ? mx_launch_typed<32, true>(dev, maps, grid, stream)
                     : mx_launch_typed<64, true>(dev, maps, grid, stream);
  } else {
    e = a.tile == 16 ? mx_launch_typed<16, false>(dev, maps, grid, stream)
      : a.tile == 32 ? mx_launch_typed<32, false>(dev, maps, grid, stream)
                     : mx_launch_typed<64, false>(dev, maps, grid, stream);
  }
  if (launches) *launches += 1;
  return e;
}

}  // namespace moe
