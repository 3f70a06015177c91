// Tables that follow from the per-expert row counts of a grouping: row offsets, the list of work
// items (chunks of at most `tile` rows of one expert) and the rows of the shared expert. Used by
// the permutation kernel and by the fused small-batch routing kernel, so both publish the same
// bytes. Reference for the grouping itself: megabench/tasks/megamoe.py:137-145.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace moe {

// Exclusive prefix of rows and of chunks per expert, by one warp: each lane owns a run of experts.
// s_count[groups] in, s_offset[groups + 1] and s_chunk0[groups + 1] out (the caller synchronises).
// `tile` is a power of two (1, 16, 32 or 64): the chunk counts are shifts, not divisions (a serial
// run of divisions per lane was a microsecond of the small-batch routing kernel's critical path).
__device__ __forceinline__ void group_prefix(const int* s_count, int* s_offset, int* s_chunk0, int groups, int tile,
                                             int lane) {
  const int per = (groups + 31) / 32;
  const int first = lane * per, last = min(first + per, groups);
  const int shift = __ffs(tile) - 1;
  int rows = 0, chunks = 0;
  for (int e = first; e < last; ++e) {
    rows += s_count[e];
    chunks += (s_count[e] + tile - 1) >> shift;
  }
  int rows_before = rows, chunks_before = chunks;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int r = __shfl_up_sync(0xffffffffu, rows_before, off);
    const int c = __shfl_up_sync(0xffffffffu, chunks_before, off);
    if (lane >= off) { rows_before += r; chunks_before += c; }
  }
  rows_before -= rows;
  chunks_before -= chunks;
  for (int e = first; e < last; ++e) {
    s_offset[e] = rows_before;
    s_chunk0[e] = chunks_before;
    rows_before += s_count[e];
    chunks_before += (s_count[e] + tile - 1) >> shift;
  }
  if (last == groups && first < groups) {   // the lane holding the final expert closes the prefix
    s_offset[groups] = rows_before;
    s_chunk0[groups] = chunks_before;
  }
}

// Written once per call (by one block): counters of the GEMMs zeroed, counts, offsets, work items,
// their number, the shared expert's rows, and -1 for positions of `order` no kept row fills.
__device__ __forceinline__ void group_publish(const GroupArgs& a, const int* s_count, const int* s_offset,
                                              const int* s_chunk0, int tid, int nthreads) {
  const int groups = a.n_local + 1;
  if (a.progress)
    for (int i = tid; i < a.progress_len; i += nthreads) a.progress[i] = 0;
  const int kept = s_offset[a.n_local];
  // The shared expert's work items open the list (its rows stay behind the routed rows): its
  // weights may have been requested from HBM ahead of time and should be used while they are
  // still in the L2.
  const int shared_chunks = s_chunk0[groups] - s_chunk0[a.n_local];
  for (int i = tid; i < groups; i += nthreads) {
    a.counts[i] = s_count[i];
    const int c = s_count[i];
    const int nch = (c + a.tile - 1) >> (__ffs(a.tile) - 1);      // the tile is a power of two
    for (int j = 0; a.chunks && j < nch; ++j) {
      const int slot = i == a.n_local ? j : shared_chunks + s_chunk0[i] + j;
      if (slot < a.max_chunks) {
        Chunk ch;
        ch.expert = i;
        ch.row0 = s_offset[i] + j * a.tile;
        ch.rows = min(a.tile, c - j * a.tile);
        ch.pad = j | (nch << 16);      // position among the expert's chunks, and their number
        a.chunks[slot] = ch;
      }
    }
  }
  if (a.offsets)
    for (int i = tid; i <= groups; i += nthreads) a.offsets[i] = s_offset[i];
  if (tid == 0 && a.n_chunks) {
    const int total = s_chunk0[groups];
    // a list that does not fit is not walked at all (the status word says why)
    *a.n_chunks = total > a.max_chunks ? 0 : total;
    if (total > a.max_chunks && a.status) report(a.status, MOE_ERR_DEVICE_BOUNDS, 100);
  }
  // rows of the shared expert follow the routed rows; their output row follows all slot rows
  for (int t = tid; t < a.shared_rows; t += nthreads) {
    if (a.row_token) a.row_token[kept + t] = t;
    if (a.row_dest) a.row_dest[kept + t] = a.n + t;
  }
  if (a.order)
    for (int r = kept + tid; r < a.n; r += nthreads) a.order[r] = -1;
}

}  // namespace moe
