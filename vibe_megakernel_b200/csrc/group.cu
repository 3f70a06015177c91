// Token -> expert permutation: a stable counting sort of the routed rows by expert id.
//
// Reference: `torch.sort(ids, stable=True)` + `bincount` (megabench/tasks/megamoe.py:137-138) and
// the owner-order gather of megabench/tasks/megamoe.py:161-168. The result does not depend on
// thread timing: a row's position is offset[expert] + (number of earlier rows with the same
// expert), computed with ballots over the rows in order, never with order-dependent atomics.
#include "common.cuh"
#include "group_tables.cuh"
#include "kernels.h"

namespace moe {

constexpr int kGroupWarps = 8;
constexpr int kMaxGroupRows = 32768;   // ids are staged in shared memory as int16
constexpr int kMaxSegments = 8;        // segments of a segmented input (one per source rank)

// SEG: the input comes in segments (expert-parallel arrivals). The loops are rolled on purpose (one copy
// of the placing code, the segment arithmetic only where SEG asks for it): a version with the counting
// and placing loops unrolled, three times the code, took 20 us longer on 8,192 rows.
template <bool SEG>
__global__ void __launch_bounds__(kGroupWarps * 32) group_rows_kernel(GroupArgs a) {
  extern __shared__ __align__(16) int16_t s_ids[];         // [n rounded up to 256]
  __shared__ int s_count[MOE_MAX_EXPERTS + 1];
  __shared__ int s_offset[MOE_MAX_EXPERTS + 2];
  __shared__ int s_chunk0[MOE_MAX_EXPERTS + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int groups = a.n_local + 1;                        // last one is the shared expert
  dependent_wait();
  dependents_may_launch();
  if (a.zero_status && a.status && blockIdx.x == 0 && tid < 8) a.status[tid] = 0;   // only block 0 reports, later
  wait_for_peers(a.wait);

  // Segmented input (segment s holds seg_counts[s] rows at s * seg_cap): only the rows that exist are
  // walked, in row order, through a compact index c -> row.
  int first_c[kMaxSegments + 1];      // (every index below is a compile-time constant: registers)
  int n_rows = a.n, segments = 0;
  if constexpr (SEG) {
    segments = min(a.n / a.seg_cap, kMaxSegments);
    first_c[0] = 0;
#pragma unroll
    for (int sgm = 0; sgm < kMaxSegments; ++sgm)
      first_c[sgm + 1] = first_c[sgm] + (sgm < segments ? min(max(a.seg_counts[sgm], 0), a.seg_cap) : 0);
    n_rows = first_c[kMaxSegments];
  }
  auto row_of = [&](int c) {
    int r = c;
    if constexpr (SEG) {
#pragma unroll
      for (int sgm = 1; sgm < kMaxSegments; ++sgm)
        if (sgm < segments && c >= first_c[sgm]) r = sgm * a.seg_cap + (c - first_c[sgm]);
    }
    return r;
  };

  // Keys (local expert of a kept row, else -1) into shared memory as int16, padded with -1 to a multiple
  // of 256 rows. The loads of kLoadBatch trips are issued before the first is used (one row per thread
  // and trip, each waited for, cost a block a round trip to the L2 per 256 rows); a plain int32 array
  // is read 16 bytes per thread.
  const int padded = (n_rows + 255) & ~255;
  const long long none = static_cast<long long>(a.id_base) - 1;
  auto key_of = [&](long long id) {
    const long long local = id - a.id_base;
    return local >= 0 && local < a.n_local ? static_cast<int>(local) : -1;
  };
  for (int i = tid; i < groups; i += blockDim.x) s_count[i] = 0;
  constexpr int kLoadBatch = 4;
  if (!SEG && a.ids32 && (n_rows & 3) == 0 && (reinterpret_cast<uintptr_t>(a.ids32) & 15) == 0) {
    const int none32 = a.id_base - 1;
    for (int q0 = tid; q0 < padded / 4; q0 += blockDim.x * kLoadBatch) {
      int4 v[kLoadBatch];
#pragma unroll
      for (int u = 0; u < kLoadBatch; ++u) {
        const int c = 4 * (q0 + u * static_cast<int>(blockDim.x));
        v[u] = c < n_rows ? __ldg(reinterpret_cast<const int4*>(a.ids32 + c)) : make_int4(none32, none32, none32, none32);
      }
#pragma unroll
      for (int u = 0; u < kLoadBatch; ++u) {
        const int c = 4 * (q0 + u * static_cast<int>(blockDim.x));
        if (c < padded)
          *reinterpret_cast<uint2*>(s_ids + c) =
              make_uint2((key_of(v[u].x) & 0xffff) | (static_cast<uint32_t>(key_of(v[u].y)) << 16),
                         (key_of(v[u].z) & 0xffff) | (static_cast<uint32_t>(key_of(v[u].w)) << 16));
      }
    }
  } else {
    for (int c0 = tid; c0 < padded; c0 += blockDim.x * kLoadBatch) {
      long long id[kLoadBatch];
#pragma unroll
      for (int u = 0; u < kLoadBatch; ++u) {
        const int c = c0 + u * static_cast<int>(blockDim.x);
        id[u] = none;
        if (c < n_rows) {
          const int r = row_of(c);
          id[u] = a.ids32 ? static_cast<long long>(a.ids32[r]) : a.ids64[r];
        }
      }
#pragma unroll
      for (int u = 0; u < kLoadBatch; ++u) {
        const int c = c0 + u * static_cast<int>(blockDim.x);
        if (c < padded) s_ids[c] = static_cast<int16_t>(key_of(id[u]));
      }
    }
  }
  __syncthreads();

  // Counts: one shared-memory atomic per distinct expert of a warp's 32 rows (a hot expert, skewed
  // routing, would otherwise serialise hundreds of them on one address, in every block). The lanes
  // with the same key are found by one vote per key bit (match.any took 300 ns per trip with 32
  // distinct keys in a warp, a third of the kernel at 384 experts).
  constexpr int kKeyBits = 10;
  static_assert(MOE_MAX_EXPERTS <= (1 << kKeyBits), "a key fits the votes below");
  const int key_bits = 32 - __clz(max(a.n_local - 1, 1));
#pragma unroll 1
  for (int c0 = warp * 32; c0 < padded; c0 += blockDim.x) {     // whole warps, so that the lanes can vote
    const int key = s_ids[c0 + lane];
    unsigned same = __ballot_sync(0xffffffffu, key >= 0);
#pragma unroll
    for (int bit = 0; bit < kKeyBits; ++bit) {
      if (bit < key_bits) {
        const unsigned set = __ballot_sync(0xffffffffu, (key >> bit) & 1);
        same &= ((key >> bit) & 1) ? set : ~set;
      }
    }
    if (key >= 0 && lane == __ffs(same) - 1) atomicAdd(&s_count[key], __popc(same));
  }
  if (tid == 0) s_count[a.n_local] = a.shared_rows;
  __syncthreads();

  if (warp == 0) group_prefix(s_count, s_offset, s_chunk0, groups, a.tile, lane);
  __syncthreads();

  // Stable rank: warp w walks the keys in order, 256 rows a trip (eight consecutive rows per lane, compared
  // two at a time), and places those of its expert: a row's position is the expert's offset plus the
  // hits in earlier trips, in lower lanes and in the lane's own earlier rows. Trips without a hit, the
  // common case with hundreds of experts, cost one load and a vote.
  const int e = blockIdx.x * kGroupWarps + warp;
  if (e < a.n_local && s_count[e] > 0) {
    int placed = 0;
    const int base = s_offset[e];
    const uint32_t e2 = static_cast<uint32_t>(e) | (static_cast<uint32_t>(e) << 16);
    const unsigned lower = (1u << lane) - 1u;
#pragma unroll 1
    for (int c0 = 0; c0 < padded; c0 += 256) {
      const uint4 v = *reinterpret_cast<const uint4*>(s_ids + c0 + 8 * lane);
      const uint32_t m0 = __vcmpeq2(v.x, e2), m1 = __vcmpeq2(v.y, e2), m2 = __vcmpeq2(v.z, e2), m3 = __vcmpeq2(v.w, e2);
      if (__ballot_sync(0xffffffffu, (m0 | m1 | m2 | m3) != 0) == 0) continue;
      uint32_t hits = (m0 & 1u) | ((m0 >> 15) & 2u) | ((m1 & 1u) << 2) | ((m1 >> 13) & 8u) | ((m2 & 1u) << 4) |
                      ((m2 >> 11) & 32u) | ((m3 & 1u) << 6) | ((m3 >> 9) & 128u);      // bit j: row c0 + 8 lane + j
      const int mine = __popc(hits);                 // 0..8: four votes give the hits in lower lanes and in all
      int before = 0, total = 0;
#pragma unroll
      for (int bit = 0; bit < 4; ++bit) {
        const unsigned m = __ballot_sync(0xffffffffu, (mine >> bit) & 1);
        before += __popc(m & lower) << bit;
        total += __popc(m) << bit;
      }
      int pos = base + placed + before;
#pragma unroll 1
      while (hits) {
        const int r = row_of(c0 + 8 * lane + __ffs(hits) - 1);
        hits &= hits - 1;
        if (a.order) a.order[pos] = r;
        if (a.row_token) a.row_token[pos] = r / a.topk;
        if (a.row_dest) a.row_dest[pos] = r;
        if (a.slot_pos) a.slot_pos[r] = pos;
        ++pos;
      }
      placed += total;
    }
  }

  if (blockIdx.x == 0) group_publish(a, s_count, s_offset, s_chunk0, tid, blockDim.x);
}

cudaError_t launch_group_rows(const GroupArgs& a, cudaStream_t stream, int* launches) {
  if (a.n > kMaxGroupRows || a.n_local > MOE_MAX_EXPERTS) return cudaErrorInvalidValue;
  const int blocks = max(1, (a.n_local + kGroupWarps - 1) / kGroupWarps);
  const size_t smem = static_cast<size_t>(((a.n > 0 ? a.n : 1) + 255) & ~255) * sizeof(int16_t);
  if (smem > 32 * 1024) {      // with the kernel's static tables the default 48 KB would be exceeded
    cudaError_t e = cudaFuncSetAttribute(a.seg_counts ? group_rows_kernel<true> : group_rows_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return e;
  }
  if (a.seg_counts) {
    if (a.seg_cap < 1) return cudaErrorInvalidValue;
    launch_dependent(group_rows_kernel<true>, dim3(blocks), dim3(kGroupWarps * 32), smem, stream, a);
  } else {
    launch_dependent(group_rows_kernel<false>, dim3(blocks), dim3(kGroupWarps * 32), smem, stream, a);
  }
  if (launches) *launches += 1;
  return cudaGetLastError();
}

}  // namespace moe
