// Host-callable launchers of the layer's kernels (internal to the library).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moe_b200.h"

#include <utility>

namespace moe {

struct Chunk;

// Launch with programmatic stream serialization: the kernel may start while the previous kernel of
// the stream drains; it must call dependent_wait() before reading what that kernel wrote.
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

cudaError_t launch_router(const moe_config_t& cfg, const __nv_bfloat16* x, const float* router, const float* bias,
                          int tokens, float* logits, int32_t* ids32, float* weights, int64_t* ids64,
                          float* weights_out, cudaStream_t stream, int* launches);

cudaError_t launch_router_logits(const __nv_bfloat16* x, const float* router, int tokens, int experts, int hidden,
                                 float* logits, cudaStream_t stream);

struct GroupArgs {
  const int32_t* ids32;   // one of ids32 / ids64 is set
  const int64_t* ids64;
  int n;                  // routed rows
  int id_base, n_local;   // ids in [id_base, id_base + n_local) are kept
  int topk;               // row r belongs to token r / topk
  int shared_rows;        // rows of the shared expert appended as expert n_local (0 = none)
  int tile;               // rows per chunk
  int max_chunks;
  int32_t* counts;        // [n_local + 1]
  int32_t* offsets;       // [n_local + 2]
  int32_t* n_chunks;
  Chunk* chunks;
  int32_t* row_token;     // optional
  int32_t* row_dest;      // optional
  int64_t* order;         // optional, [n]
  int32_t* status;        // optional
  const int32_t* seg_counts;  // optional: rows come in segments of seg_cap, segment s holds seg_counts[s] rows
  int seg_cap;
  int32_t* progress;          // optional: [max_chunks + 4] counters of the GEMMs, zeroed here (see GemmArgs)
};
cudaError_t launch_group_rows(const GroupArgs& a, cudaStream_t stream, int* launches);

cudaError_t launch_quantize(const void* x, int dtype, int rows, int width, const int32_t* gather, uint8_t* q,
                            float* scales, cudaStream_t stream, int* launches);

cudaError_t launch_combine(const __nv_bfloat16* slots, const float* weights, int tokens, int topk, int hidden,
                           int shared, __nv_bfloat16* y, cudaStream_t stream, int* launches);

// Copy rows that arrived in any order (and the home rows of the shared expert) into expert order.
struct GatherArgs {
  const int32_t* row_source;   // grouped position -> arrival index (routed) or home token (shared)
  const int32_t* offsets;      // offsets[n_local] = routed rows kept; shared rows follow
  int n_local, shared_rows, hidden;
  const uint8_t* recv_q;       // arrivals: e4m3 [*, H] and fp32 scales [*, H/128]
  const float* recv_s;
  const uint8_t* xq_home;      // rows of the shared expert
  const float* xs_home;
  uint8_t* xq;                 // grouped output
  float* xs;
};
cudaError_t launch_gather_rows(const GatherArgs& a, int row_blocks, cudaStream_t stream, int* launches);

struct GemmArgs {
  bool dual;                 // true: gate+up with SwiGLU + requantisation; false: down projection
  int tile;                  // tokens per MMA tile: 16, 32 or 64
  int k;                     // contraction length (H for gate/up, I for down)
  int m;                     // output channels per expert (I for gate/up, H for down)
  int n_local;               // routed experts held here; chunk.expert == n_local is the shared expert
  int total_rows;            // rows of the activation buffer
  int max_units;             // upper bound of chunks * (m / 128)
  const Chunk* chunks;
  const int32_t* n_chunks;
  const uint8_t* act;        // e4m3 [total_rows, k]
  const float* act_scale;    // [total_rows, k/128]
  const uint8_t* w_a;        // gate or down, [n_local, m, k]
  const float* w_a_scale;
  const uint8_t* w_b;        // up (dual only)
  const float* w_b_scale;
  const uint8_t* s_a;        // shared expert counterparts (may be NULL when there is none)
  const float* s_a_scale;
  const uint8_t* s_b;
  const float* s_b_scale;
  uint8_t* aq;               // dual: e4m3 [total_rows, m]
  float* as;                 // dual: [total_rows, m/128]
  __nv_bfloat16* out;        // single: bf16 rows [*, m] addressed through row_dest
  const int32_t* row_dest;
  int32_t* status;
  // Hand-over between the two GEMMs of a layer call without a kernel boundary: progress[c] counts
  // the gate/up tiles of work item c that are finished and visible; progress[max_chunks] is the
  // down GEMM's work-item dispenser. The gate/up GEMM increments, the down GEMM (which may be
  // scheduled on SMs the gate/up GEMM has already left) waits per work item and takes items
  // dynamically. NULL = plain kernel-boundary ordering and a static walk.
  int32_t* progress;
  int max_chunks;
  int tiles_before;          // down GEMM: gate/up tiles per work item that must be finished
};
cudaError_t launch_gemm_tc(const GemmArgs& a, cudaStream_t stream, int* launches, int* driver_error);
cudaError_t launch_gemm_simt(const GemmArgs& a, cudaStream_t stream, int* launches);

}  // namespace moe
