/*
 * C ABI of the B200 FP8 mixture-of-experts decode layer.
 *
 * Every entry point takes plain device pointers and sizes. Except moe_ep_buffer_alloc, none
 * allocates device memory: the caller owns inputs, outputs and the scratch workspace. All work is enqueued on `stream`
 * (a cudaStream_t passed as void*). Return value: 0 = ok, > 0 = a cudaError_t, < 0 = one of
 * the MOE_ERR_* codes below. Kernels never trap: a bounded on-device wait that runs out is
 * reported through moe_device_status().
 *
 * The reference these replace is megabench's PyTorch MoE layer (kamahori/vibe-megakernel);
 * each declaration cites the reference lines whose arithmetic it reproduces. Paths are
 * relative to the reference project root.
 */
#ifndef MOE_B200_H_
#define MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_OK 0
#define MOE_ERR_BAD_ARG (-1)
#define MOE_ERR_UNSUPPORTED (-2)
#define MOE_ERR_WORKSPACE (-3)
#define MOE_ERR_DEVICE_TIMEOUT (-4)
#define MOE_ERR_DRIVER (-5)
#define MOE_ERR_DEVICE_BOUNDS (-6)

#define MOE_SCORING_SOFTMAX 0 /* stable top-k of the logits, softmax over the selection */
#define MOE_SCORING_SIGMOID 1 /* sigmoid + selection bias, group-limited, normalised, scaled */
/* p = sqrt(softplus(logit)); selection on p + bias (the same group limit applies when n_group > 1);
 * weights p[ids] / (sum + 1e-20) * routed_scaling: megabench/tasks/dsv41.py:622-626. */
#define MOE_SCORING_SQRT_SOFTPLUS 2
/* The bias is the router's linear-layer bias: scores = logit + bias decide the stable top-k AND
 * enter the softmax over the selection: megabench/tasks/gptoss.py:106-109. */
#define MOE_SCORING_SOFTMAX_BIASED 3

#define MOE_GEMM_TCGEN05 0 /* tcgen05 FP8 MMA, TMEM accumulators, TMA-fed (the product path) */
#define MOE_GEMM_SIMT 1    /* plain CUDA-core check arm used by the tests to localise faults */
/* CUDA-core check arm with the rounding schedule of megabench/tasks/megamoe.py:146-149: both operands
 * dequantised and rounded to bf16, fp32 accumulation over the whole contraction, one bf16 rounding.
 * It shows how much of the tensor-core path's distance to that reference is operand rounding. */
#define MOE_GEMM_SIMT_BF16 2

#define MOE_MAX_EXPERTS 1024
#define MOE_MAX_TOPK 16

typedef struct moe_config {
  int32_t hidden;         /* H, multiple of 128 */
  int32_t inter;          /* I, multiple of 128 */
  int32_t n_experts;      /* routed experts in the whole layer */
  int32_t topk;
  int32_t n_shared;       /* 0 or 1 shared expert of width I */
  int32_t scoring;        /* MOE_SCORING_* */
  int32_t n_group;        /* router groups (1 = no group limit) */
  int32_t topk_group;     /* groups kept */
  float routed_scaling;   /* multiplies the normalised sigmoid weights */
  int32_t ep_world;       /* expert-parallel ranks; rank r owns experts [r*E/world, (r+1)*E/world) */
  int32_t ep_rank;
  int32_t gemm_impl;      /* MOE_GEMM_* */
  /* The MegaMoE form of the expert MLP (megabench/tasks/megamoe.py:116-122,176-182); both 0 = the
   * DeepSeek/GLM form of megabench/tasks/frontier.py:337,352. */
  float swiglu_limit;             /* > 0: gate clamped to at most this, up to +- this, before SwiGLU */
  int32_t weight_before_requant;  /* 1: the routing weight multiplies the SwiGLU output before it is
                                   * requantised and the combine is a plain slot-order sum (one-GPU
                                   * layer and block entry points only) */
} moe_config_t;

/* Device pointers. Layouts are the MoE-block tensors of megabench/tasks/frontier.py:157-176:
 * gate/up e4m3 [E_local, I, H] with fp32 scales [E_local, I/128, H/128]; down e4m3
 * [E_local, H, I] with scales [E_local, H/128, I/128]; shared_* the same without the expert
 * axis; router fp32 [E, H]; router_bias fp32 [E] (may be NULL: treated as zeros). */
typedef struct moe_weights {
  const float* router;
  const float* router_bias;
  const uint8_t* gate;
  const float* gate_scale;
  const uint8_t* up;
  const float* up_scale;
  const uint8_t* down;
  const float* down_scale;
  const uint8_t* shared_gate;
  const float* shared_gate_scale;
  const uint8_t* shared_up;
  const float* shared_up_scale;
  const uint8_t* shared_down;
  const float* shared_down_scale;
} moe_weights_t;

/* Byte offsets of the scratch arrays inside the workspace (tests read intermediates here). */
typedef struct moe_workspace_layout {
  uint64_t total_bytes;
  uint64_t status;        /* int32[8]: [0] device status, [1] detail */
  uint64_t logits;        /* fp32 [T, E] */
  uint64_t topk_ids;      /* int32 [T, topk] */
  uint64_t topk_weights;  /* fp32 [T, topk] */
  uint64_t counts;        /* int32 [E_local + 1] rows per local expert (+ shared) */
  uint64_t offsets;       /* int32 [E_local + 2] exclusive prefix of counts */
  uint64_t n_chunks;      /* int32: number of (expert, row chunk) work items */
  uint64_t chunks;        /* int32 [max_chunks][4]: expert, first row, rows, reserved */
  uint64_t row_token;     /* int32 [rows]: source token of every grouped row */
  uint64_t row_dest;      /* int32 [rows]: output slot row (token*topk+slot; shared: T*topk+token) */
  uint64_t xq;            /* e4m3 [rows, H] grouped activation rows */
  uint64_t xs;            /* fp32 [rows, H/128] */
  uint64_t aq;            /* e4m3 [rows, I] requantised SwiGLU output */
  uint64_t as;            /* fp32 [rows, I/128] */
  uint64_t slots;         /* bf16 [T*topk + T, H] down-projection rows in slot order */
  int32_t rows;           /* T*topk + T*n_shared */
  int32_t max_chunks;
  int32_t token_tile;     /* token rows per MMA tile (16, 32, 64 or 128) chosen for this T */
  int32_t reserved;
} moe_workspace_layout_t;

/* Scratch a call with `tokens` rows needs; fills *layout when it is not NULL. */
int moe_workspace_layout(const moe_config_t* cfg, int32_t tokens, moe_workspace_layout_t* layout);

/* Router: fp32 logits and top-k selection for `tokens` bf16 rows. A logit is summed with fp32 FMAs
 * in 32 per-lane chains that are merged with error-free two-float additions and rounded once
 * (absolute error about 1e-7 at the magnitudes of this layer); the result of a token does not
 * depend on the batch it arrives in. The weight tensors (router, bias, expert matrices) must be
 * complete before the stream operation that precedes a call: kernels fetch them before they
 * wait for that predecessor.
 * Replaces `router.float() @ x.float()` + frontier.route (megabench/tasks/frontier.py:229-242,343)
 * and the stable softmax top-k of megabench/tasks/distributed.py:174-176.
 * expert_ids int64 [T, topk] in choice order; weights fp32 [T, topk]; either may be NULL.
 * Uses the logits / topk_ids / topk_weights arrays of `workspace`. */
int moe_route(const moe_config_t* cfg, const void* x_bf16, const float* router, const float* router_bias,
              int32_t tokens, int64_t* expert_ids, float* weights, void* workspace, size_t workspace_bytes,
              void* stream);

/* The router again, for callers that cannot hand over a workspace because they may not allocate
 * device memory (a plugin given only input and output buffers by a host that forbids cudaMalloc
 * while serving; an FFI wrapper without an allocator). It has no counterpart in the reference.
 * Same arguments and results as moe_route without the workspace: the scratch lives in a static
 * device array inside the library (about 544 KiB held by every GPU that loads the library).
 * Limits: tokens <= MOE_STATIC_ROUTE_MAX_TOKENS and n_experts <= MOE_STATIC_ROUTE_MAX_EXPERTS, else
 * MOE_ERR_TOO_LARGE and nothing is launched.
 * The first call on a device looks up the array's address: make it outside any stream capture.
 * All calls on a GPU share the array, so calls that can overlap on the GPU race; keep them on
 * one stream. Calls no cudaMalloc/cudaFree and no allocating library routine. */
#define MOE_STATIC_ROUTE_MAX_TOKENS 256
#define MOE_STATIC_ROUTE_MAX_EXPERTS 512
#define MOE_ERR_TOO_LARGE (-7)
int moe_route_static(const moe_config_t* cfg, const void* x_bf16, const float* router, const float* router_bias,
                     int32_t tokens, int64_t* expert_ids, float* weights, void* stream);

/* Per-row, per-128-channel e4m3 quantiser: scale = max(amax, 1e-4)/448, q = RNE(x/scale).
 * Replaces pack_fp8_activation(..., scale_format="float") (megabench/tasks/quantization.py:87-109).
 * dtype: 0 = bf16 input, 1 = fp32 input. `width` need not be a multiple of 128 (zero padding).
 * gather (int32[rows], may be NULL) selects the input row of every output row. */
int moe_quantize_rows(const void* x, int32_t dtype, int32_t rows, int32_t width, const int32_t* gather,
                      uint8_t* q, float* scales, void* stream);

/* The same quantiser with power-of-two scales stored as biased exponents (UE8M0), one per `block` =
 * 32 or 128 channels: the activation format of the MXFP4 MegaMoE layer. The exponent comes from the
 * fp32 bits of the block maximum by integer arithmetic, the payload is RNE_e4m3(x * 2^-(e-127)).
 * Replaces pack_fp8_activation(..., block=32, scale_format="e8m0")
 * (megabench/tasks/quantization.py:62-84,87-109). scales uint8 [rows, ceil(width/block)]. */
int moe_quantize_rows_ue8m0(const void* x, int32_t dtype, int32_t rows, int32_t width, int32_t block, uint8_t* q,
                            uint8_t* scales, void* stream);

/* The routed experts in the MegaMoE-native formats: MXFP4 weights and E4M3 token rows, both with one
 * E8M0 scale per 32 input channels; routing is an input. Replaces `megamoe.reference(case, values,
 * serial=True)` (megabench/tasks/megamoe.py:131-182): rows grouped per expert in (token, slot) order,
 * linear1 -> clamped SwiGLU times the routing weight -> E4M3/E8M0 requantisation -> linear2, then the
 * fp32 slot-order sum rounded once to bf16. Device pointers, layouts as megamoe.make_inputs
 * (megabench/tasks/megamoe.py:86-113). */
typedef struct moe_mx_weights {
  const uint8_t* l1_blocks;   /* [E, 2I, H/32, 16] E2M1 codes, low nibble = even channel; gate rows, then up rows */
  const uint8_t* l1_scales;   /* [E, 2I, H/32] E8M0 */
  const uint8_t* l2_blocks;   /* [E, H, I/32, 16] */
  const uint8_t* l2_scales;   /* [E, H, I/32] */
} moe_mx_weights_t;

/* Uses cfg->hidden, inter (multiples of 128), n_experts, topk and swiglu_limit; n_shared must be 0 and
 * ep_world 1. tokens * topk <= 32768. */
int moe_mx_workspace(const moe_config_t* cfg, int32_t tokens, uint64_t* bytes);

/* x_q e4m3 [tokens, H]; x_scales uint8 [tokens, H/32]; topk_idx int64 [tokens, topk] (distinct per
 * token); topk_weights fp32 [tokens, topk]; y bf16 [tokens, H]; order (optional) int64 [tokens*topk].
 * workspace: 256-byte aligned, moe_mx_workspace() bytes. Block pointers 32-byte, scale pointers
 * 16-byte aligned (MOE_ERR_BAD_ARG otherwise). Expert ids are taken as given: a row whose id is
 * outside [0, E) is skipped and leaves its slot of the sum undefined. */
int moe_mx_forward(const moe_config_t* cfg, const moe_mx_weights_t* w, const uint8_t* x_q, const uint8_t* x_scales,
                   const int64_t* topk_idx, const float* topk_weights, int32_t tokens, void* y_bf16, int64_t* order,
                   void* workspace, size_t workspace_bytes, void* stream);

/* The MoE block of the Kimi-K3 decoder layer, all experts on one GPU. Replaces `moe(case, values,
 * normalized, serial=True, group=None)` of megabench/tasks/kimi_layer.py:189-230: sigmoid top-k routing
 * with a selection bias (scaling 1, no groups), a bf16 down-projection of every token into the latent
 * width, routed experts with MXFP4 weights over the bf16 latent rows and the situ activation
 * (megabench/tasks/kimi_layer.py:175-186, megabench/tasks/kimi.py:134-135), the fp32 slot-order weighted
 * sum rounded to bf16, RMSNorm and up-projection of the latent sum, and the shared experts on the
 * full-width token; the two results are added. Device pointers; layouts as
 * megabench/tasks/kimi_layer.py:107-125 makes them. */
typedef struct moe_latent_config {
  int32_t hidden;      /* H, multiple of 128 */
  int32_t latent;      /* latent width L, multiple of 128 */
  int32_t inter;       /* expert intermediate width I, multiple of 128 */
  int32_t n_experts;   /* routed experts, at most MOE_MAX_EXPERTS */
  int32_t topk;
  int32_t n_shared;    /* shared experts: their matrices are n_shared * I wide */
  float latent_eps;    /* epsilon of the latent RMSNorm (1e-5 in the reference) */
} moe_latent_config_t;

typedef struct moe_latent_weights {
  const float* router;          /* fp32 [E, H] (the reference's bf16 router widened: router.float()) */
  const float* router_bias;     /* fp32 [E], may be NULL */
  const void* latent_down;      /* bf16 [L, H] */
  const void* latent_up;        /* bf16 [H, L] */
  const void* latent_norm;      /* bf16 [L] */
  const uint8_t* gate_blocks;   /* [E, I, L/32, 16] E2M1 codes, low nibble = even channel */
  const uint8_t* gate_scales;   /* [E, I, L/32] E8M0 */
  const uint8_t* up_blocks;
  const uint8_t* up_scales;
  const uint8_t* down_blocks;   /* [E, L, I/32, 16] */
  const uint8_t* down_scales;   /* [E, L, I/32] */
  const void* shared_gate;      /* bf16 [n_shared * I, H] */
  const void* shared_up;
  const void* shared_down;      /* bf16 [H, n_shared * I] */
} moe_latent_weights_t;

/* tokens * topk <= 16384 (every routed row travels as two E4M3 rows). */
int moe_latent_workspace(const moe_latent_config_t* cfg, int32_t tokens, uint64_t* bytes);

/* x bf16 [tokens, H] (the layer's normalised tokens) -> y bf16 [tokens, H]; expert_ids int64 [tokens, topk]
 * in choice order and topk_weights fp32 [tokens, topk] are optional outputs (the reference returns the
 * ids sorted per token, megabench/tasks/kimi_layer.py:230). workspace: 256-byte aligned,
 * moe_latent_workspace() bytes. Block pointers 32-byte, scale pointers 16-byte aligned. */
int moe_latent_forward(const moe_latent_config_t* cfg, const moe_latent_weights_t* w, const void* x_bf16, int32_t tokens,
                       void* y_bf16, int64_t* expert_ids, float* topk_weights, void* workspace, size_t workspace_bytes,
                       void* stream);

/* Stable grouping of `n` routed rows by expert id (the token->expert permutation).
 * Replaces `torch.sort(ids, stable=True)` + `bincount` (megabench/tasks/megamoe.py:137-138,161-165).
 * ids int64 [n]; rows whose id is outside [id_base, id_base + n_local) are dropped.
 * order int64 [n] (grouped position -> input row; unused tail = -1), counts int32 [n_local + 1]
 * (rows per expert; the last entry is reserved and written as 0). */
int moe_group_rows(const int64_t* ids, int32_t n, int32_t id_base, int32_t n_local, int64_t* order,
                   int32_t* counts, void* stream);

/* Weighted combine / un-permute of down-projection rows stored in slot order:
 * y[t] = bf16( sum over slot = 0..topk-1, in that order, of fp32(rows[t*topk + slot]) * weights[t*topk + slot],
 * then + fp32(rows[tokens*topk + t]) when `shared` is non-zero ), every product and sum rounded to fp32.
 * Replaces the fp32 slot-order sum with one bf16 rounding of megabench/tasks/megamoe.py:176-182 in
 * its weighted form, megabench/tasks/frontier.py:349-354. rows bf16 [tokens*topk (+ tokens), hidden],
 * weights fp32 [tokens*topk], y bf16 [tokens, hidden]; hidden a multiple of 8, pointers 16-byte aligned. */
int moe_combine(const void* rows_bf16, const float* weights, int32_t tokens, int32_t topk, int32_t hidden,
                int32_t shared, void* y_bf16, void* stream);

/* The experts held by this rank applied to rows that are already quantised: gate/up GEMM, SwiGLU,
 * requantisation, down GEMM; result rows bf16 [n_rows, H] in the order of the input rows.
 * Replaces `experts(...)` of megabench/tasks/megamoe.py:131-150 for the FP8 block-scaled format
 * (rows e4m3 [n_rows, H] + fp32 scales [n_rows, H/128]; local_ids int32 [n_rows] in
 * [0, n_experts/ep_world), or NULL to send every row through the shared expert).
 * moe_experts_workspace gives the scratch size for n_rows. */
int moe_experts_workspace(const moe_config_t* cfg, int32_t n_rows, uint64_t* bytes);
int moe_experts_forward(const moe_config_t* cfg, const moe_weights_t* weights, const uint8_t* rows_q,
                        const float* rows_scale, const int32_t* local_ids, int32_t n_rows, void* out_bf16,
                        void* workspace, size_t workspace_bytes, void* stream);

/* Whole layer on one GPU (ep_world == 1): router, permutation, activation quantiser, grouped
 * gate/up GEMM with SwiGLU + requantisation, grouped down GEMM, shared expert, weighted combine.
 * Replaces the MoE block of megabench/tasks/frontier.py:343-353 batched over tokens with the
 * permutation/combine order of megabench/tasks/megamoe.py:153-182.
 * x bf16 [T, H] -> y bf16 [T, H]; expert_ids int64 [T, topk], topk_weights fp32 [T, topk],
 * order int64 [T*topk] are optional outputs (NULL to skip). Inputs are not modified. */
int moe_layer_forward(const moe_config_t* cfg, const moe_weights_t* weights, const void* x_bf16, int32_t tokens,
                      void* y_bf16, int64_t* expert_ids, float* topk_weights, int64_t* order, void* workspace,
                      size_t workspace_bytes, void* stream);

/* The layer with the step either side of it: RMSNorm of the residual stream in front, residual add
 * behind. Replaces megabench/tasks/frontier.py:335 (`normalized = norm(x, ln2)`, `rms` of
 * megabench/tasks/common.py:13-21) ... :354 (`x = x + output.to(x.dtype)`):
 *   n = bf16 RMSNorm(x) with weight norm_weight_bf16 [H] and eps; weight_in_fp32 != 0 rounds once,
 *   after the fp32 product with the weight (DeepSeek family), 0 rounds the normalised value to bf16
 *   first and multiplies in bf16 (Llama/Qwen/GLM);
 *   x_out = bf16(x + bf16(layer(n))).
 * x_out may be x itself (the stream is then updated in place); the other arguments are those of
 * moe_layer_forward and the same workspace serves both. */
int moe_block_forward(const moe_config_t* cfg, const moe_weights_t* weights, const void* x_bf16,
                      const void* norm_weight_bf16, float eps, int32_t weight_in_fp32, int32_t tokens,
                      void* x_out_bf16, int64_t* expert_ids, float* topk_weights, int64_t* order, void* workspace,
                      size_t workspace_bytes, void* stream);

/* ---- expert parallelism over the GPUs of one node ------------------------------------------
 * Rank r owns experts [r*E/world, (r+1)*E/world) and `tokens` rows of the batch; router, bias and
 * shared expert are replicated (megabench/tasks/megamoe.py:100-105, megabench/tasks/kimi_layer.py:4-6).
 * Replaces exchange_counts/exchange (megabench/tasks/parallel.py:52-68) and the dispatch/combine
 * skeleton of megabench/tasks/megamoe.py:153-182: routed rows are quantised and stored straight
 * into the owning rank's receive buffer by the dispatching kernel (peer stores over NVLink), counts
 * travel with the data, arrival is signalled by per-source flags that the consumer polls with a
 * bounded wait; results come back the same way into the source's slot rows. No host
 * synchronisation and no NCCL call inside a layer call.
 *
 * Every rank allocates one exchange buffer of moe_ep_layout().exchange_bytes (zero-filled once)
 * that its peers can address (moe_ep_buffer_* below, or any other peer-mapped allocation), and
 * passes the array of all ranks' buffer addresses as seen from this process. */
typedef struct moe_ep_layout {
  uint64_t exchange_bytes;   /* peer-visible buffer of every rank */
  uint64_t local_bytes;      /* private scratch of every rank (256-byte aligned) */
  uint64_t flags_dispatch;   /* offsets inside the exchange buffer: uint64[world], one per source */
  uint64_t flags_return;     /* uint64[world], one per owner */
  uint64_t recv_count;       /* int32[world] rows received from each source */
  uint64_t recv_expert;      /* int32[world*cap] local expert id of every received row */
  uint64_t recv_slot;        /* int32[world*cap] slot row (token*topk+slot) at the source */
  uint64_t recv_weight;      /* fp32 [world*cap] routing weight of every received row (MegaMoE form only) */
  uint64_t recv_q;           /* e4m3 [world*cap, H] */
  uint64_t recv_s;           /* fp32 [world*cap, H/128]; MegaMoE form: E8M0 bytes [world*cap, H/32] */
  uint64_t slots;            /* bf16 [cap + max_tokens, H] down-projection rows coming home */
  int32_t cap;               /* rows one source can send to one owner: max_tokens*topk */
  int32_t rows;              /* world*cap + max_tokens: rows this rank may have to multiply */
  int32_t max_chunks;
  int32_t token_tile;
} moe_ep_layout_t;

int moe_ep_layout(const moe_config_t* cfg, int32_t max_tokens, moe_ep_layout_t* layout);

/* One layer call of this rank. `exchange` is void*[world]: every rank's exchange buffer (own one at
 * index ep_rank). `epoch` is 1 on the first call that uses a given `local` buffer (that call clears the
 * buffer's block counters; a first call with another epoch leaves them undefined and every peer then
 * runs into its 2 s wait), grows by one with every call and is the same on all ranks.
 * x bf16 [tokens, H] -> y bf16 [tokens, H]; expert_ids / topk_weights optional as in moe_layer_forward;
 * order (optional) int64 [tokens*topk]: this rank's routed rows in the stable order of their owning
 * rank, the dispatch permutation of megabench/tasks/megamoe.py:161-164.
 * On a bounded wait running out the call still returns; moe_device_status(local, ...) reports it. */
int moe_ep_forward(const moe_config_t* cfg, const moe_weights_t* weights, const void* x_bf16, int32_t tokens,
                   int32_t max_tokens, void* y_bf16, int64_t* expert_ids, float* topk_weights, int64_t* order,
                   void* const* exchange, void* local, size_t local_bytes, uint64_t epoch, void* stream);

/* The routed experts in the MegaMoE-native formats, expert-parallel: the form the reference grades
 * (megabench/cases.py:380-388, `reference(case, values)` of megabench/tasks/megamoe.py:153-182 without
 * `serial`). Every rank passes its own token rows with their routing and the MXFP4 matrices of its
 * experts [rank*E/world, (rank+1)*E/world); the dispatching kernel stores payload, scale bytes, local
 * expert id and routing weight of every routed row into the owner's receive buffer (the four
 * dispatched tensors of megabench/tasks/megamoe.py:167-173), the owner runs linear1 -> clamped SwiGLU
 * times the weight -> requantisation -> linear2 and stores the bf16 rows back into the source's slot
 * rows, the source adds them in slot order. Results equal moe_mx_forward on the whole problem bit
 * for bit (megabench/verify_megamoe.py:44-56,104-105). cfg as for moe_mx_forward with ep_world / ep_rank
 * set and n_experts the experts of the whole layer; tokens and max_tokens count this rank's rows;
 * exchange, local, epoch as for moe_ep_forward, sized by moe_mx_ep_layout. order (optional) int64
 * [tokens*topk]: the stable order of this rank's routed rows by owning rank (rows whose expert id is out
 * of range have no owner, are not sent, and come last). */
int moe_mx_ep_layout(const moe_config_t* cfg, int32_t max_tokens, moe_ep_layout_t* layout);
int moe_mx_ep_forward(const moe_config_t* cfg, const moe_mx_weights_t* w, const uint8_t* x_q, const uint8_t* x_scales,
                      const int64_t* topk_idx, const float* topk_weights, int32_t tokens, int32_t max_tokens,
                      void* y_bf16, int64_t* order, void* const* exchange, void* local, size_t local_bytes,
                      uint64_t epoch, void* stream);

/* The bounded wait the expert-parallel layer uses for its arrival and return flags, on its own:
 * waits until flags[0..world) >= epoch or `timeout_ns` (at most 2 s) has passed; on expiry it writes
 * MOE_ERR_DEVICE_TIMEOUT and 200 + the index of a late flag into status_words (int32[2], as read by
 * moe_device_status) and returns normally. It is how failure detection is exercised without
 * faulting a GPU: a flag that nothing raises makes the wait run out. The reference's counterpart
 * is the process-group timeout of its host-driven collectives (megabench/verify_megamoe.py:149). */
int moe_ep_wait_flags(const uint64_t* flags, int32_t world, uint64_t epoch, uint64_t timeout_ns, void* status_words,
                      void* stream);

/* Peer-visible device memory for the exchange buffer (cudaMalloc + CUDA IPC): allocate and export
 * a 64-byte handle, open a peer's handle (enables peer access), close, free. */
int moe_ep_buffer_alloc(size_t bytes, void** ptr, void* handle64);
int moe_ep_buffer_open(const void* handle64, void** ptr);
int moe_ep_buffer_close(void* ptr);
int moe_ep_buffer_free(void* ptr);

/* Synchronises `stream` and returns the device status word of the workspace: MOE_OK, or
 * MOE_ERR_DEVICE_TIMEOUT / MOE_ERR_DEVICE_BOUNDS when a kernel gave up on a bounded wait or
 * refused an out-of-range index. *detail (may be NULL) receives a code naming the place. */
int moe_device_status(const void* workspace, void* stream, int32_t* detail);

/* Self-check of the epilogue arithmetic (no counterpart in the reference; test infrastructure). The
 * tensor-core epilogues divide without the math library's range check and slow path (a reciprocal
 * and fused residual corrections); this runs n (even) gate/up value pairs and n/2 group scales (device
 * pointers, fp32) through both forms of SwiGLU and of the e4m3 quantisation and writes to counts
 * (device int32[3]): SwiGLU values whose bits differ, e4m3 code pairs that differ, pairs checked. */
int moe_selfcheck_divisions(const float* gate, const float* up, const float* scales, int32_t n, int32_t* counts,
                            void* stream);

/* Number of kernels the last layer call of this thread launched (moe_layer_forward, moe_block_forward,
 * moe_ep_forward, moe_experts_forward, moe_mx_forward, moe_mx_ep_forward, moe_latent_forward). */
int moe_last_launch_count(void);

/* Stage timing for measurements (no counterpart in the reference, whose harness times whole calls
 * with torch.cuda.Event, megabench/harness/benchmark.py:27-38). While enabled, moe_layer_forward
 * records CUDA events on its stream between stages; moe_profile_read waits for the last call and
 * returns the six stage durations in milliseconds: router, permutation, quantiser, gate/up GEMM,
 * down GEMM, combine. Per calling thread. */
int moe_profile_enable(int32_t on);
int moe_profile_read(float* stage_ms, int32_t n);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H_ */
