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

__global__ void __launch_bounds__(kGroupWarps * 32) group_rows_kernel(GroupArgs a) {
  extern __shared__ int16_t s_ids[];                       // [n]
  __shared__ int s_count[MOE_MAX_EXPERTS + 1];
  __shared__ int s_offset[MOE_MAX_EXPERTS + 2];
  __shared__ int s_chunk0[MOE_MAX_EXPERTS + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int groups = a.n_local + 1;                        // last one is the shared expert
  dependent_wait();
  dependents_may_launch();
  if (a.zero_status && a.status && blockIdx.x == 0 && tid < 8) a.status[tid] = 0;   // only block 0 reports, later
  wait_for_peers(a.wait);

  // Segmented input (expert-parallel arrivals: segment s holds seg_counts[s] rows at s * seg_cap): only
  // the rows that exist are walked, in row order, through a compact index c -> row.
  int first_c[kMaxSegments + 1];      // (every index below is a compile-time constant: registers)
  int n_rows = a.n;
  const int segments = a.seg_counts ? min(a.n / a.seg_cap, kMaxSegments) : 0;
  first_c[0] = 0;
#pragma unroll
  for (int sgm = 0; sgm < kMaxSegments; ++sgm)
    first_c[sgm + 1] = first_c[sgm] + (sgm < segments ? min(max(a.seg_counts[sgm], 0), a.seg_cap) : 0);
  if (a.seg_counts) n_rows = first_c[kMaxSegments];
  auto row_of = [&](int c) {
    int r = c;
    if (segments == 0) return r;      // uniform: plain input
#pragma unroll
    for (int sgm = 1; sgm < kMaxSegments; ++sgm)
      if (sgm < segments && c >= first_c[sgm]) r = sgm * a.seg_cap + (c - first_c[sgm]);
    return r;
  };

  for (int i = tid; i < groups; i += blockDim.x) s_count[i] = 0;
  __syncthreads();
  for (int c0 = warp * 32; c0 < n_rows; c0 += blockDim.x) {     // whole warps, so that the lanes can vote
    const int c = c0 + lane;
    int key = -1;                                             // local expert of a kept row
    if (c < n_rows) {
      const int r = row_of(c);
      const long long id = a.ids32 ? static_cast<long long>(a.ids32[r]) : a.ids64[r];
      const long long local = id - a.id_base;
      if (local >= 0 && local < a.n_local) key = static_cast<int>(local);
      s_ids[c] = static_cast<int16_t>(key);
    }
    // one shared-memory atomic per distinct expert of the warp: a hot expert (skewed routing) would
    // otherwise serialise hundreds of them on one address, in every block
    const unsigned same = __match_any_sync(0xffffffffu, key);
    if (key >= 0 && lane == __ffs(same) - 1) atomicAdd(&s_count[key], __popc(same));
  }
  if (tid == 0) s_count[a.n_local] = a.shared_rows;
  __syncthreads();

  if (warp == 0) group_prefix(s_count, s_offset, s_chunk0, groups, a.tile, lane);
  __syncthreads();

  // Stable rank: warp w walks the rows in order and places those of its expert.
  const int e = blockIdx.x * kGroupWarps + warp;
  if (e < a.n_local && s_count[e] > 0) {
    int placed = 0;
    const int base = s_offset[e];
    for (int c0 = 0; c0 < n_rows; c0 += 32) {
      const int c = c0 + lane;
      const bool hit = c < n_rows && s_ids[c] == e;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int r = row_of(c);
        const int pos = base + placed + __popc(m & ((1u << lane) - 1u));
        if (a.order) a.order[pos] = r;
        if (a.row_token) a.row_token[pos] = r / a.topk;
        if (a.row_dest) a.row_dest[pos] = r;
        if (a.slot_pos) a.slot_pos[r] = pos;
      }
      placed += __popc(m);
    }
  }

  if (blockIdx.x == 0) group_publish(a, s_count, s_offset, s_chunk0, tid, blockDim.x);
}

cudaError_t launch_group_rows(const GroupArgs& a, cudaStream_t stream, int* launches) {
  if (a.n > kMaxGroupRows || a.n_local > MOE_MAX_EXPERTS) return cudaErrorInvalidValue;
  const int blocks = max(1, (a.n_local + kGroupWarps - 1) / kGroupWarps);
  const size_t smem = static_cast<size_t>(a.n > 0 ? a.n : 1) * sizeof(int16_t);
  if (smem > 32 * 1024) {      // with the kernel's static tables the default 48 KB would be exceeded
    cudaError_t e = cudaFuncSetAttribute(group_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return e;
  }
  launch_dependent(group_rows_kernel, dim3(blocks), dim3(kGroupWarps * 32), smem, stream, a);
  if (launches) *launches += 1;
  return cudaGetLastError();
}

}  // namespace moe
