/*
 * C ABI of libcomfy_b200_moe.so: the HiDream mixture-of-experts feed-forward on B200 (sm_100a).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name starts with `h_`;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - functions return 0 on success or one of the COMFY_MOE_E* codes; they never throw, never
 *     allocate device memory and never synchronise unless the comment says so;
 *   - activations are bf16, row-major, contiguous in the last dimension;
 *   - expert weights use torch.nn.Linear's layout [out_features, in_features] row-major with a
 *     leading dimension `ld` in elements (so a row- or column-slice of a weight can be passed
 *     without copying), dtype bf16 or fp8 e4m3fn with a per-tensor fp32 scale on the device.
 *
 * Reference interface replaced (paths inside the ComfyUI tree):
 *   comfy/ldm/hidream/model.py:242-283   MoEGate
 *   comfy/ldm/hidream/model.py:215-238   FeedForwardSwiGLU
 *   comfy/ldm/hidream/model.py:287-346   MOEFeedForwardSwiGLU.forward / moe_infer
 *   comfy/ops.py:314-358, 379-410        fp8_linear / scaled_fp8_ops.Linear
 */
#ifndef COMFY_B200_MOE_H_
#define COMFY_B200_MOE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COMFY_MOE_ABI_VERSION 9

/* Return codes. */
#define COMFY_MOE_OK 0
#define COMFY_MOE_EINVAL 1        /* null pointer, negative size, misaligned pointer            */
#define COMFY_MOE_EUNSUPPORTED 2  /* shape / dtype / expert count outside what the kernels cover */
#define COMFY_MOE_ECUDA 3         /* a CUDA runtime or driver call failed (launch, encode)       */
#define COMFY_MOE_ETIMEOUT 4      /* a bounded device-side wait ran out (see comfy_moe_read_status) */
#define COMFY_MOE_EDEVICE 5       /* not an sm_100 device, or the driver lacks tensor-map support */
#define COMFY_MOE_ETOOLARGE 6     /* more tokens than the library's built-in scratch array can serve */

/* Element types for weights and for the activations fed to the expert GEMMs. */
#define COMFY_MOE_BF16 0
#define COMFY_MOE_FP32 1
#define COMFY_MOE_FP8_E4M3 2
#define COMFY_MOE_FP16 3

/* Rows of every routed expert's block start on a multiple of this in the permuted layout. */
#define COMFY_MOE_ROW_ALIGN 128
/* Tokens handled by one thread block of the gate / permute kernels (fixes the block-count scratch size). */
#define COMFY_MOE_TOKENS_PER_BLOCK 32
#define COMFY_MOE_MAX_EXPERTS 8
/* A status block is this many int32 words: [0] the sticky device status word (see comfy_moe_read_status), [1] tokens
 * the last gate call flagged as near-ties, [2] elements that the activation quantiser turned into NaN because the
 * reference casts them to e4m3 without a clamp (accumulates; see comfy_moe_permute), [3] reserved. */
#define COMFY_MOE_STATUS_WORDS 4
/* Largest token count comfy_moe_route_static accepts (its scratch is a fixed array inside the library). */
#define COMFY_MOE_STATIC_MAX_TOKENS 131072

int comfy_moe_abi_version(void);
const char* comfy_moe_error_string(int code);

/* Sizes (in elements / rows) of the buffers a caller must provide for `n_tokens` tokens. Pure host arithmetic.
 *   rows_cap      rows of x_perm / h / y_perm: top_k*n_tokens + n_experts*COMFY_MOE_ROW_ALIGN
 *   n_blocks      ceil(n_tokens / COMFY_MOE_TOKENS_PER_BLOCK); block_counts and block_offsets hold n_blocks*n_experts int32
 */
int comfy_moe_plan_sizes(int n_tokens, int n_experts, int top_k, int64_t* rows_cap, int* n_blocks);

/* ---- MoEGate.forward (comfy/ldm/hidream/model.py:263-283) --------------------------------------
 * logits = x . w_gate^T in fp32, softmax over experts, top-2 (largest first, lowest index on exact ties),
 * no renormalisation.  Also writes, per block of COMFY_MOE_TOKENS_PER_BLOCK tokens, how many routed slots
 * went to each expert (input of comfy_moe_route_plan).
 *   x             bf16 [n_tokens, dim]
 *   w_gate        [n_experts, dim], dtype w_dtype (COMFY_MOE_BF16 or COMFY_MOE_FP32)
 *   topk_idx      int32 [n_tokens, 2]          topk_weight  fp32 [n_tokens, 2]
 *   block_counts  int32 [n_blocks, n_experts]  (fully overwritten)
 *   neartie_count int32 [1], may be NULL: incremented for every token whose 2nd and 3rd scores differ by
 *                 less than neartie_eps (caller zeroes it);  neartie_flags uint8 [n_tokens], may be NULL.
 */
int comfy_moe_gate_topk(const void* x, const void* w_gate, int w_dtype, int n_tokens, int dim, int n_experts,
                        int top_k, int32_t* topk_idx, float* topk_weight, int32_t* block_counts,
                        int32_t* neartie_count, uint8_t* neartie_flags, float neartie_eps, void* stream);

/* ---- per-block expert counts for caller-supplied routing (moe_infer takes the indices as an argument,
 * model.py:328): same output as the gate's block_counts.  Ids outside [0, n_experts) are counted nowhere; the
 * permutation maps such slots to row -1 and the combine treats them as zero.
 */
int comfy_moe_route_count(const int32_t* topk_idx, int n_tokens, int n_experts, int32_t* block_counts, void* stream);

/* ---- routing plan: replaces argsort + bincount().cpu().cumsum (model.py:330-332) without a host sync ----
 *   block_counts   int32 [n_blocks, n_experts]  from the gate
 *   block_offsets  int32 [n_blocks, n_experts]  out: rows of expert e that precede block b, within e's block
 *   expert_counts  int32 [n_experts]            out: routed slots per expert (= bincount of topk_idx)
 *   expert_offsets int32 [n_experts + 1]        out: first row of each expert in the permuted layout, each a
 *                                               multiple of COMFY_MOE_ROW_ALIGN; [n_experts] = rows in use
 */
int comfy_moe_route_plan(const int32_t* block_counts, int n_tokens, int n_experts, int32_t* block_offsets,
                         int32_t* expert_counts, int32_t* expert_offsets, void* stream);

/* ---- permutation: replaces x[exp_token_idx] gathers (model.py:338-339) ------------------------------
 * Copies row t of x to row row_map[t*2+k] of x_perm for k = 0,1; order inside an expert block is by slot index
 * (stable), so the layout is reproducible run to run.
 *   x_perm      [rows_cap, dim] in act_dtype: COMFY_MOE_BF16 copies; COMFY_MOE_FP8_E4M3 quantises exactly as
 *               comfy/ops.py:338-343 does.  act_scale NULL (the Linear has no scale_input): clamp to +-448, then
 *               round to nearest even (:339-340).  act_scale given: multiply by bf16(1 / *act_scale) in bf16 and cast
 *               WITHOUT a clamp (:342-343); torch's cast does not saturate, so |v| > 464 and NaN become NaN (byte
 *               0x7f | sign), here as there.
 *   x_q         only for fp8: [n_tokens, dim] e4m3, the un-permuted quantised copy the shared expert reads
 *               (x_q_scale: its own optional scale); may be NULL
 *   row_map     int32 [n_tokens, 2] out
 *   overflow_count  int32 [1], may be NULL: incremented by the number of elements the unclamped cast turned into NaN
 *               (never touched when both scales are NULL), so that such inputs are flagged, not only reproduced
 */
int comfy_moe_permute(const void* x, const int32_t* topk_idx, const int32_t* block_offsets,
                      const int32_t* expert_offsets, int n_tokens, int dim, int n_experts, int act_dtype,
                      const float* act_scale, void* x_perm, void* x_q, const float* x_q_scale,
                      int32_t* row_map, int32_t* overflow_count, void* stream);

/* ---- routing plan and permutation in one launch: comfy_moe_route_plan + comfy_moe_permute -------------------
 * Same outputs (expert_counts, expert_offsets, x_perm, x_q, row_map).  Every block re-sums the per-block counts it
 * needs instead of waiting for a separate single-block scan; beyond 2048 blocks of tokens (65 536 tokens) the call
 * falls back to the two launches and then uses block_offsets_scratch [n_blocks, n_experts].
 */
int comfy_moe_plan_permute(const void* x, const int32_t* topk_idx, const int32_t* block_counts, int n_tokens, int dim,
                           int n_experts, int act_dtype, const float* act_scale, int32_t* block_offsets_scratch,
                           int32_t* expert_counts, int32_t* expert_offsets, void* x_perm, void* x_q,
                           const float* x_q_scale, int32_t* row_map, int32_t* overflow_count, void* stream);

/* ---- debug aid: consistency check of the routing a layer call produced ------------------------------------------
 * (No counterpart in the reference.)  Verifies on the device that every expert id lies inside the layer or its slot is
 * unmapped (row -1), every mapped row lies inside its expert's block and below rows_cap, the offsets are aligned,
 * monotone and leave room for every expert's rows, and the counts add up to the number of mapped slots.  A violation
 * sets the sticky status word to 9 (comfy_moe_read_status then returns COMFY_MOE_ETIMEOUT's sibling COMFY_MOE_EINVAL).
 * status: a status block (word 3 is used as scratch).  Two small kernels and a memset node; meant for debug runs. */
int comfy_moe_validate_routing(const int32_t* topk_idx, const int32_t* row_map, const int32_t* expert_counts,
                               const int32_t* expert_offsets, int n_tokens, int n_experts, int64_t rows_cap,
                               int32_t* status, void* stream);

/* ---- gate + routing plan + permutation for callers that cannot allocate device memory -----------------
 * (No counterpart in the reference: it has no allocation-free mode.)
 * Some hosts of this library may not call cudaMalloc or any allocator between set-up and tear-down: real-time
 * loops that reserve all their device memory at start-up, plugins that are handed a fixed device arena by their
 * host application, processes whose whole device-memory budget is committed before the first frame.  The three
 * routing entry points above need two scratch arrays (block_counts,
 * block_offsets) from the caller; this one does the same three steps with that scratch in a fixed 256 KB device
 * array that is part of the library, so only inputs and outputs are passed.  It calls no allocator of any kind.
 *   inputs    x, w_gate, w_dtype, act_dtype, act_scale, x_q_scale          as comfy_moe_gate_topk / comfy_moe_permute
 *   outputs   topk_idx, topk_weight, expert_counts, expert_offsets, x_perm, x_q (may be NULL), row_map,
 *             neartie_count (may be NULL; caller zeroes)                    exactly what the three calls produce
 * Limits and rules:
 *   - n_tokens <= COMFY_MOE_STATIC_MAX_TOKENS, else COMFY_MOE_ETOOLARGE (nothing is launched);
 *   - the first call on each device looks up the array's device address (one cudaGetSymbolAddress) and keeps it for
 *     the life of the process; make that first call outside any stream capture, and from one thread (the table of
 *     addresses is filled without a lock; later calls only read it).  The address is not looked up again: after a
 *     cudaDeviceReset in the same process it would be stale, so do not use this entry point across a device reset;
 *   - all calls on a device share the one array, so two calls that can overlap on the GPU (different streams
 *     without an ordering between them) race; keep them on one stream or order them with events.  Nothing in the
 *     array has to be cleared between calls: every word a call reads it has written itself.
 */
int comfy_moe_route_static(const void* x, const void* w_gate, int w_dtype, int n_tokens, int dim, int n_experts,
                           int top_k, int act_dtype, const float* act_scale, int32_t* topk_idx, float* topk_weight,
                           int32_t* expert_counts, int32_t* expert_offsets, void* x_perm, void* x_q,
                           const float* x_q_scale, int32_t* row_map, int32_t* neartie_count, void* stream);

/* One SwiGLU feed-forward's weights (FeedForwardSwiGLU, model.py:233-238). */
typedef struct ComfyMoeFfnWeights {
  const void* w1;         /* [hidden, dim], leading dimension ld13 */
  const void* w3;         /* [hidden, dim], leading dimension ld13 */
  const void* w2;         /* [dim, hidden], leading dimension ld2  */
  int64_t ld13;
  int64_t ld2;
  int32_t hidden;         /* multiple of 128 */
  int32_t max_sms;        /* 0 = all SMs.  Read from the shared-expert struct (else from the first group) of a grouped
                             call: its launches then occupy at most this many SMs, the rest stay free for kernels
                             that run beside them on other streams */
  /* fp8 only (NULL = 1.0): per-tensor scales as comfy/ops.py:379-410 stores them */
  const float* scale_w1;
  const float* scale_w3;
  const float* scale_w2;
  const float* scale_in13; /* scale_input shared by w1 and w3 (they see the same activation) */
  const float* scale_in2;  /* scale_input of w2 */
} ComfyMoeFfnWeights;

/* ---- grouped SwiGLU expert GEMM (model.py:238 for every expert, and the shared expert) -------------------
 * Two launches of one persistent tcgen05/TMEM kernel:
 *   h      = silu(a . w1^T) * (a . w3^T)    (bf16 roundings after each of the reference's four steps)
 *   y      = h . w2^T
 * over n_groups row ranges of x_perm, group g = rows [row_start[g], row_start[g] + row_count[g]) with weights
 * h_groups[g] (start and count are DEVICE arrays: no host sync; several groups may name the same expert), and,
 * when `h_shared` is not NULL, one more group over the un-permuted rows.  Group starts need no alignment.
 *   w_dtype        COMFY_MOE_BF16 or COMFY_MOE_FP8_E4M3 (activations x_perm / x_shared / h_* use the same)
 *   x_perm         [rows_cap, dim]        h_perm [rows_cap, hidden] workspace   y_perm bf16 [rows_cap, dim]
 *   x_shared       [n_tokens, dim]        h_shared [n_tokens, hidden_s]         y_shared bf16 [n_tokens, dim]
 *   status         int32 [COMFY_MOE_STATUS_WORDS]: the kernels write a non-zero code to word 0 if a bounded wait ran out (sticky: zeroed by the
 *                  caller once, then only by comfy_moe_read_status after it reported a code)
 * Requires dim % 256 == 0 and hidden % 128 == 0 (COMFY_MOE_EUNSUPPORTED otherwise).
 */
int comfy_moe_grouped_swiglu(int w_dtype, int n_groups, const ComfyMoeFfnWeights* h_groups,
                             const ComfyMoeFfnWeights* h_shared, const int32_t* row_start,
                             const int32_t* row_count, int64_t rows_cap, int n_tokens, int dim, const void* x_perm,
                             void* h_perm, void* y_perm, const void* x_shared, void* h_shared_ws, void* y_shared,
                             int32_t* status, void* stream);

/* ---- grouped GELU-MLP expert GEMM: the experts of the Hunyuan3D-2.1 MoE block ----------------------------------
 * Replaces FeedForward.forward = Linear(dim, hidden, bias) -> exact GELU -> Linear(hidden, dim, bias)
 * (comfy/ldm/hunyuan3dv2_1/hunyuandit.py:8-50) for every routed expert and the shared expert:
 *   h = bf16( gelu( bf16(a . w1^T + b1) ) )        y = bf16( h . w2^T + b2 )
 * bf16 only.  Arguments as comfy_moe_grouped_swiglu.  Requires dim % 256 == 0 and hidden % 256 == 0.
 */
typedef struct ComfyMoeMlpWeights {
  const void* w1;         /* net.0.proj.weight [hidden, dim], leading dimension ld1 */
  const void* b1;         /* net.0.proj.bias [hidden] or NULL */
  const void* w2;         /* net.2.weight [dim, hidden], leading dimension ld2 */
  const void* b2;         /* net.2.bias [dim] or NULL */
  int64_t ld1;
  int64_t ld2;
  int32_t hidden;
  int32_t reserved;
} ComfyMoeMlpWeights;

int comfy_moe_grouped_gelu_mlp(int n_groups, const ComfyMoeMlpWeights* h_groups, const ComfyMoeMlpWeights* h_shared,
                               const int32_t* row_start, const int32_t* row_count, int64_t rows_cap, int n_tokens,
                               int dim, const void* x_perm, void* h_perm, void* y_perm, const void* x_shared,
                               void* h_shared_ws, void* y_shared, int32_t* status, void* stream);

/* comfy_moe_grouped_swiglu for routed groups only, with the second pass writing group i's results to
 * y_out[i] + (row + y_row_shift[i]) * dim instead of one y_perm (y_out: HOST array of n_groups device pointers to
 * bf16 [y_rows_cap, dim] buffers, which may be another GPU's memory mapped here; y_row_shift: DEVICE array).
 * No counterpart in the reference; used by the expert-parallel path to return results while the GEMM runs. */
int comfy_moe_grouped_swiglu_scatter(int w_dtype, int n_groups, const ComfyMoeFfnWeights* h_groups,
                                     const int32_t* row_start, const int32_t* row_count, int64_t rows_cap, int dim,
                                     const void* x_perm, void* h_perm, void* const* h_y_out,
                                     const int32_t* y_row_shift, int64_t y_rows_cap, int32_t* status, void* stream);

/* comfy_moe_grouped_swiglu with options (HOST struct; no counterpart in the reference; what the expert-parallel path
 * is built from):
 *   passes        1 = first pass only (h_perm / h_shared are written), 2 = second pass only (they are read), 0 or 3 =
 *                 both.  Lets a caller run the shared expert's first pass beside other kernels and then fold its second
 *                 pass into the routed groups' launch.
 *   y_out, y_row_shift, y_rows_cap   as comfy_moe_grouped_swiglu_scatter (NULL: results go to y_perm)
 *   arrive_flags  DEVICE array of 32-bit epoch flags, one per source rank (NULL: no waiting).  With it, group i is not
 *                 loaded by the first pass before arrive_flags[group_source[i]] has reached arrive_epoch (acquire at
 *                 system scope, bounded by arrive_budget_cycles, 0 = COMFY_MOE_EP_WAIT_CYCLES; a wait that runs out
 *                 leaves code 7 in the status word).  group_source: HOST array [n_groups], -1 = rows already there.
 *                 So the launch need not be preceded by a wait for every rank: tiles over rows that are there keep
 *                 the tensor pipe busy while other ranks' rows land. */
typedef struct ComfyMoeGroupedOptions {
  int32_t passes;
  int32_t reserved;
  void* const* y_out;
  const int32_t* y_row_shift;
  int64_t y_rows_cap;
  const uint32_t* arrive_flags;
  const int32_t* group_source;
  uint32_t arrive_epoch;
  uint32_t reserved2;
  int64_t arrive_budget_cycles;
} ComfyMoeGroupedOptions;

int comfy_moe_grouped_swiglu_ex(int w_dtype, int n_groups, const ComfyMoeFfnWeights* h_groups,
                                const ComfyMoeFfnWeights* h_shared, const int32_t* row_start, const int32_t* row_count,
                                int64_t rows_cap, int n_tokens, int dim, const void* x_perm, void* h_perm, void* y_perm,
                                const void* x_shared, void* h_shared_ws, void* y_shared,
                                const ComfyMoeGroupedOptions* h_options, int32_t* status, void* stream);

/* ---- weighted combine: replaces mul_ + scatter_reduce_ + shared add (model.py:341-345, 324) ---------------
 * out[t] = bf16( bf16( bf16(w0*y[r0]) + bf16(w1*y[r1]) ) + y_shared[t] ), weights rounded to bf16 first.
 * y_shared may be NULL (routed part only, what moe_infer returns).
 */
int comfy_moe_combine(const void* y_perm, const int32_t* row_map, const float* topk_weight, const void* y_shared,
                      int n_tokens, int dim, void* out, void* stream);

/* Same, for experts whose hidden dimension is split over two GPUs (no counterpart in the reference, which is
 * single-GPU): every row has two partial results, y = bf16(y_a + y_b) replaces the expert output the reference
 * rounds once, then the combine proceeds as above.  Both buffers use the layout row_map refers to.
 */
int comfy_moe_combine_partials(const void* y_perm_a, const void* y_perm_b, const int32_t* row_map,
                               const float* topk_weight, const void* y_shared, int n_tokens, int dim, void* out,
                               void* stream);

/* Everything one layer call needs, for the fused entry point. */
typedef struct ComfyMoeLayer {
  int32_t dim;
  int32_t n_experts;
  int32_t top_k;
  int32_t w_dtype;            /* expert weight dtype */
  int32_t gate_dtype;         /* COMFY_MOE_BF16 or COMFY_MOE_FP32 */
  int32_t reserved;
  const void* w_gate;         /* [n_experts, dim] */
  ComfyMoeFfnWeights experts[COMFY_MOE_MAX_EXPERTS];
  ComfyMoeFfnWeights shared;
} ComfyMoeLayer;

typedef struct ComfyMoeWorkspace {
  int32_t* topk_idx;       /* [n_tokens, 2] */
  float* topk_weight;      /* [n_tokens, 2] */
  int32_t* block_counts;   /* [n_blocks, n_experts] */
  int32_t* block_offsets;  /* [n_blocks, n_experts] */
  int32_t* expert_counts;  /* [n_experts] */
  int32_t* expert_offsets; /* [n_experts + 1] */
  int32_t* row_map;        /* [n_tokens, 2] */
  int32_t* status;         /* [COMFY_MOE_STATUS_WORDS]: [0] device status word (sticky, see comfy_moe_read_status),
                              [1] near-tie count of the last call, [2] e4m3 overflow count (accumulates) */
  void* x_perm;            /* [rows_cap, dim] act dtype */
  void* x_q;               /* fp8 only: [n_tokens, dim] */
  void* h_perm;            /* [rows_cap, hidden] act dtype */
  void* y_perm;            /* bf16 [rows_cap, dim] */
  void* h_shared;          /* [n_tokens, hidden_s] act dtype */
  void* y_shared;          /* bf16 [n_tokens, dim] */
  int64_t rows_cap;
  void* x_mod;             /* bf16 [n_tokens, dim]: normalised + modulated input; only comfy_moe_ffn_block needs it */
} ComfyMoeWorkspace;

/* ---- MOEFeedForwardSwiGLU.forward (model.py:307-325): gate -> plan+permute -> experts -> combine ----
 * x, out: bf16 [n_tokens, dim].  The layer struct and the workspace struct live in HOST memory.
 */
int comfy_moe_forward(const ComfyMoeLayer* h_layer, const ComfyMoeWorkspace* h_ws, const void* x, int n_tokens,
                      void* out, void* stream);

/* ---- MoEBlock.forward in eval mode (comfy/ldm/hunyuan3dv2_1/hunyuandit.py:130-185): gate -> plan+permute ->
 * GELU-MLP experts -> combine (index_add_ of the weighted expert outputs, then + shared_experts(x)).
 * Same workspace struct as comfy_moe_forward (x_q unused); up to COMFY_MOE_MAX_EXPERTS experts, top-2.
 */
typedef struct ComfyMoeMlpLayer {
  int32_t dim;
  int32_t n_experts;
  int32_t top_k;
  int32_t gate_dtype;         /* COMFY_MOE_BF16 or COMFY_MOE_FP32 */
  const void* w_gate;         /* [n_experts, dim] */
  ComfyMoeMlpWeights experts[COMFY_MOE_MAX_EXPERTS];
  ComfyMoeMlpWeights shared;
} ComfyMoeMlpLayer;

int comfy_moe_forward_gelu_mlp(const ComfyMoeMlpLayer* h_layer, const ComfyMoeWorkspace* h_ws, const void* x,
                               int n_tokens, void* out, void* stream);

/* ---- several bias Linears in one launch (operations.Linear, comfy/ops.py:103-115) ----------------------------------
 * out_g = bf16(x_g . w_g^T + bias_g) (fp32 accumulation, one rounding) for up to COMFY_MOE_MAX_EXPERTS + 1 independent
 * groups: one launch of the persistent tcgen05 kernel with the bias epilogue.  Serves the q / k / v projections of
 * HiDreamAttention for image and text tokens (comfy/ldm/hidream/model.py:97-119) as six groups, and its two output
 * projections (:139-144) as two.  bf16; out_features % 256 == 0, in_features % 64 == 0, leading dimensions in elements
 * and multiples of 8; rows may be 0 (group skipped).  status: a status block, see comfy_moe_read_status.
 * At most COMFY_MOE_MAX_EXPERTS + 1 groups, and at most COMFY_MOE_LINEAR_MAX_MAPS DISTINCT operands among them (an x,
 * w or out that several groups name with the same rows, columns and leading dimension counts once); more is
 * COMFY_MOE_EUNSUPPORTED. */
#define COMFY_MOE_LINEAR_MAX_MAPS 22
typedef struct ComfyMoeLinearGroup {
  const void* x;      /* [rows, in_features], leading dimension ld_x */
  const void* w;      /* [out_features, in_features], leading dimension ld_w */
  const void* bias;   /* [out_features] or NULL */
  void* out;          /* [rows, out_features], leading dimension ld_out */
  int64_t ld_x;
  int64_t ld_w;
  int64_t ld_out;
  int32_t rows;
  int32_t in_features;
  int32_t out_features;
  int32_t reserved;
} ComfyMoeLinearGroup;

int comfy_moe_grouped_linear(int n_groups, const ComfyMoeLinearGroup* h_groups, int32_t* status, void* stream);

/* ---- q / k / v glue of the HiDream attention processor (model.py:97-137) ------------------------------------------
 * One pass per projected tensor x [n_tokens, heads * head_dim] (bf16, row stride ld_x):
 *   n   = rms_norm(x, weight, eps) over the whole row as torch.nn.functional.rms_norm computes it for bf16 (fp32
 *         statistics, x * rstd * weight rounded once); weight NULL = no normalisation (the value projection);
 *   out = apply_rope(n, rope) of comfy/ldm/flux/math.py:38-47 on the first rope_pairs pairs of every head (fp32
 *         rotation f[i][0] * n[2p] + f[i][1] * n[2p+1], rounded to bf16); rope NULL = no rotation.
 * Token t = (b, s) with s < tokens_per_batch is written to out + b * out_batch_stride + (out_row_offset + s) * inner
 * and rotated with rope + b * rope_batch_stride + (rope_row_offset + s) * rope_pairs * 4 (fp32 [.., pairs, 2, 2]), so
 * the image part and the text part of a joint sequence land in one [B, S_img + S_txt, heads, head_dim] buffer without
 * the reference's torch.cat.  inner <= 4096, head_dim % 8 == 0.
 */
int comfy_attn_rmsnorm_rope(const void* x, int64_t ld_x, const void* weight, float eps, const float* rope,
                            int64_t rope_batch_stride, int rope_row_offset, int rope_pairs, int n_tokens,
                            int tokens_per_batch, int heads, int head_dim, void* out, int64_t out_batch_stride,
                            int out_row_offset, void* stream);

/* ---- attention forward of the HiDream blocks (model.py:75-76 over attention_pytorch, attention.py:475-516) ---------
 * out[b, s, h, :] = softmax(q[b, s, h, :] . k[b, :, h, :]^T * scale) . v[b, :, h, :]   (no mask, not causal)
 * q [batch, seq_q, heads, 128], k / v [batch, seq_kv, heads, 128], out [batch, seq_q, heads * 128]; bf16, contiguous
 * (the layout comfy_attn_rmsnorm_rope writes and the output projection reads, so nothing is transposed).  Both
 * contractions run on tcgen05 tensor cores with S and O in tensor memory; scores and probabilities never touch HBM.
 * head_dim must be 128 (COMFY_MOE_EUNSUPPORTED otherwise).  status: a status block (code 5: a bounded wait ran out). */
int comfy_attn_forward(const void* q, const void* k, const void* v, int batch, int seq_q, int seq_kv, int heads,
                       int head_dim, float scale, void* out, int32_t* status, void* stream);

/* ---- activation quantiser on its own (comfy/ops.py:338-343) --------------------------------------------------
 * scale NULL:  out = e4m3(clamp(x, +-448))                 (:339-340; round to nearest even)
 * scale given: out = e4m3(bf16(x * bf16(1 / scale)))       (:342-343; NO clamp: beyond the e4m3 range the result is
 *              NaN, as in the reference, and *overflow_count (may be NULL) grows by the number of such elements)
 * x bf16, n_elements a multiple of 16.  What comfy_moe_permute does on the way, for callers that need the quantised
 * copy before the permutation runs (the expert-parallel path quantises the shared expert's input beside the routing
 * kernels).
 */
int comfy_moe_quantize_e4m3(const void* x, const float* scale, int64_t n_elements, void* out, int32_t* overflow_count,
                            void* stream);

/* ---- weight ingest: stochastic rounding to e4m3 (comfy/float.py:3-46) ------------------------------------------
 * What scaled_fp8_ops.Linear.set_weight (comfy/ops.py:418-426) applies to a LoRA-patched weight after dividing it by
 * scale_weight: manual_stochastic_round_to_float8 on one slice.  x: fp32, bf16 or fp16 (x_dtype), rand_fp16: the
 * uniform [0, 1) numbers the reference draws with torch.rand(..., dtype=float16, generator=...) for the slice, out:
 * e4m3 bytes.  Every fp16 rounding of the reference's tensor operations is reproduced, so the same random numbers give
 * the same bytes.
 */
int comfy_moe_stochastic_round_e4m3(const void* x, int x_dtype, const void* rand_fp16, int64_t n_elements, void* out,
                                    void* stream);

/* ---- weight ingest: per-tensor scaled e4m3 -------------------------------------------------------------------------
 * The convention of the scaled-fp8 checkpoints that scaled_fp8_ops.Linear loads (comfy/ops.py:379-410: `weight` in
 * e4m3, `scale_weight` an fp32 scalar):  *scale_out = max|w| / 448 (fp32),  out = e4m3(w / *scale_out), division in fp32,
 * round to nearest even.  Byte-identical to `s = w.float().abs().max() / 448; (w.float() / s).to(float8_e4m3fn)`.
 * w: fp32, bf16 or fp16 (w_dtype), contiguous; scale_out: DEVICE fp32 [1]; out: e4m3 bytes.  Four nodes on `stream`
 * (a 4-byte memset and three kernels), no host synchronisation. */
int comfy_moe_quantize_weight_e4m3(const void* w, int w_dtype, int64_t n_elements, float* scale_out, void* out,
                                   void* stream);

/* ---- expert parallelism over peer memory (one process per GPU, NVLink peer access) ---------------------------
 * No counterpart in the reference (it runs on one GPU).  Tokens stay with their rank; expert e is computed by rank
 * owner0[e] (and, with hidden_splits == 2, by owner1[e], each holding half of the hidden dimension).  Every rank owns
 * a receive buffer [cap_rows, dim] (activation dtype), a result buffer [cap_rows, dim] (bf16) and a flag block
 * (2 * COMFY_MOE_MAX_RANKS zero-initialised uint32), all mapped into every peer; peer_*[r] are rank r's buffers as
 * mapped in the calling process.  One step on each rank, all on one stream:
 *   gate, route_plan -> all-gather of expert_counts into counts_all [world, n_experts] (any collective) ->
 *   comfy_moe_ep_dispatch -> comfy_moe_ep_signal(ARRIVED) -> (shared expert) -> comfy_moe_ep_wait(ARRIVED) ->
 *   comfy_moe_grouped_swiglu over (group_start, group_count) on the receive buffer, results into the result buffer ->
 *   comfy_moe_ep_signal(DONE) -> comfy_moe_ep_wait(DONE) -> comfy_moe_ep_combine.
 * `epoch` must grow by one per step, equally on all ranks.  A wait that runs out of its clock budget (about two
 * seconds) writes a code to `status`; so does a dispatch whose rows do not fit cap_rows (comfy_moe_read_status
 * returns COMFY_MOE_ETIMEOUT / COMFY_MOE_ETOOLARGE).
 *   comfy_moe_ep_dispatch  permutation into the owners' receive buffers (quantising to e4m3 on the way for
 *                          act_dtype FP8, which also fills x_q for the shared expert); row_map[t, k] = row at the
 *                          owner; group_start / group_count [local experts] = this rank's own work list.
 *   comfy_moe_ep_combine   comfy_moe_combine with every routed row read from its owner's result buffer (two
 *                          partial rows summed, rounded to bf16, with a hidden split).
 * Push variant of the return path (y_row_shift not NULL): the work list has one row range per (local expert, source
 * rank), [local experts * world] entries, entry j * world + p being local expert j's rows from source rank
 * (rank + p) % world (own rows first), and y_row_shift[i] = (first row of that range in the source's own
 * expert-major order) - (first row of the range here); comfy_moe_grouped_swiglu_scatter then writes the results of
 * range i into the source rank's return buffer (y_out[i], that rank's memory) while it computes, row_map holds rows
 * of the local return buffer, and the plain comfy_moe_combine / comfy_moe_combine_partials finish the step.
 */
#define COMFY_MOE_MAX_RANKS 8
#define COMFY_MOE_EP_ARRIVED 0
#define COMFY_MOE_EP_DONE 1

typedef struct ComfyMoePeerPlan {
  int32_t world;
  int32_t rank;
  int32_t n_experts;
  int32_t hidden_splits;                      /* 1 or 2 */
  int32_t owner0[COMFY_MOE_MAX_EXPERTS];
  int32_t owner1[COMFY_MOE_MAX_EXPERTS];      /* used when hidden_splits == 2 */
  int64_t cap_rows;
  void* peer_recv[COMFY_MOE_MAX_RANKS];
  void* peer_y[COMFY_MOE_MAX_RANKS];
  uint32_t* peer_flags[COMFY_MOE_MAX_RANKS];
} ComfyMoePeerPlan;

int comfy_moe_ep_dispatch(const ComfyMoePeerPlan* h_plan, const void* x, const int32_t* topk_idx,
                          const int32_t* block_offsets, const int32_t* counts_all, int n_tokens, int dim,
                          int act_dtype, const float* act_scale, void* x_q, const float* x_q_scale, int32_t* row_map,
                          int32_t* group_start, int32_t* group_count, int32_t* y_row_shift, int32_t* status,
                          void* stream);
int comfy_moe_ep_signal(const ComfyMoePeerPlan* h_plan, int kind, uint32_t epoch, void* stream);
int comfy_moe_ep_wait(const ComfyMoePeerPlan* h_plan, int kind, uint32_t epoch, int32_t* status, void* stream);
/* The same wait with the clock budget as an argument (SM cycles; comfy_moe_ep_wait uses COMFY_MOE_EP_WAIT_CYCLES).
 * When the budget runs out before every flag has reached `epoch`, the kernel writes code 7 to *status and returns;
 * the context stays usable and comfy_moe_read_status reports COMFY_MOE_ETIMEOUT. */
#define COMFY_MOE_EP_WAIT_CYCLES 4000000000LL   /* about two seconds of SM clocks */
int comfy_moe_ep_wait_budget(const ComfyMoePeerPlan* h_plan, int kind, uint32_t epoch, int64_t budget_cycles,
                             int32_t* status, void* stream);
int comfy_moe_ep_combine(const ComfyMoePeerPlan* h_plan, const int32_t* topk_idx, const int32_t* row_map,
                         const float* topk_weight, const void* y_shared, int n_tokens, int dim, void* out,
                         void* stream);

/* ---- the element-wise passes a HiDream block runs around its feed-forward (model.py:429-433, 515-523) --------
 * Modulation vectors (shift, scale, gate) are bf16 [batch, dim] views with `*_batch_stride` elements between batch
 * elements (they are chunks of one adaLN output in the reference, so the stride is a multiple of dim); token t
 * belongs to batch element t / tokens_per_batch.
 *
 * comfy_moe_ln_modulate:   out = LayerNorm(x) * (1 + scale) + shift      LayerNorm: eps, no affine, fp32 statistics,
 *                          bf16 output; (1 + scale), the product and the sum each rounded to bf16 as PyTorch does.
 * comfy_moe_gate_residual: out = gate * y + residual                      for a dense feed-forward (text tokens).
 * comfy_moe_combine_block: comfy_moe_combine followed by "gate * (.) + residual" in the same pass.
 */
int comfy_moe_ln_modulate(const void* x, const void* shift, const void* scale, int64_t mod_batch_stride, int n_tokens,
                          int tokens_per_batch, int dim, float eps, void* out, void* stream);
int comfy_moe_gate_residual(const void* y, const void* gate, int64_t gate_batch_stride, const void* residual,
                            int n_tokens, int tokens_per_batch, int dim, void* out, void* stream);
/* comfy_moe_ln_modulate and, on the row each warp has just produced, comfy_moe_gate_topk (model.py:429-431 followed by
 * :263-283), in one pass: same `out`, topk_idx, topk_weight, block_counts, neartie outputs, bit for bit, without the
 * gate's re-read of the modulated tokens and without its launch.  block_counts is zeroed by the call (a memset node on
 * `stream`) and filled with integer atomics.  w_gate: [n_experts, dim], bf16 or fp32; n_experts 2, 4 or 8; top_k 2.
 * One launch and one read of the tokens fewer than the two calls, but not faster at 8192 x 2560 (the gate arithmetic,
 * not memory, bounds both, and here every weight value feeds one token instead of four): comfy_moe_ffn_block makes
 * the two calls. */
int comfy_moe_ln_modulate_gate(const void* x, const void* shift, const void* scale, int64_t mod_batch_stride,
                               int n_tokens, int tokens_per_batch, int dim, float eps, void* out, const void* w_gate,
                               int w_dtype, int n_experts, int top_k, int32_t* topk_idx, float* topk_weight,
                               int32_t* block_counts, int32_t* neartie_count, uint8_t* neartie_flags, float neartie_eps,
                               void* stream);
int comfy_moe_combine_block(const void* y_perm, const int32_t* row_map, const float* topk_weight, const void* y_shared,
                            const void* gate, int64_t gate_batch_stride, const void* residual, int n_tokens,
                            int tokens_per_batch, int dim, void* out, void* stream);

/* ---- feed-forward half of a HiDream block with a MoE (model.py:429-433 / 515-523), six launches ----------
 * (LayerNorm + modulation, gate, plan + permutation, two GEMM passes, combine with gate * (.) + residual)
 *   out = gate * MOEFeedForwardSwiGLU(LayerNorm(x) * (1 + scale) + shift) + x
 * x, out: bf16 [n_tokens, dim] (out may alias nothing else); h_ws->x_mod must be set.
 */
int comfy_moe_ffn_block(const ComfyMoeLayer* h_layer, const ComfyMoeWorkspace* h_ws, const void* x, const void* shift,
                        const void* scale, const void* gate, int64_t mod_batch_stride, int n_tokens,
                        int tokens_per_batch, float eps, void* out, void* stream);

/* The device status word.  Kernels move it from 0 to a code when something went wrong on the device (1-3: a bounded
 * wait of the grouped GEMM's producer / MMA / epilogue role ran out; 5: one of the attention kernel's; 7: a peer's flag did not arrive in time; 8: routed
 * rows did not fit a peer receive buffer and were dropped; 9: the routing check found an inconsistency) and never overwrite a code that is already there; no entry
 * point clears it on the way in.  A caller may therefore share one word among all layers of a model and look at it at
 * a natural synchronisation point (end of a model forward).
 * comfy_moe_read_status synchronises `stream`, copies status[0] to *h_status and returns COMFY_MOE_OK for 0,
 * COMFY_MOE_ETOOLARGE for code 8, COMFY_MOE_EINVAL for code 9 (comfy_moe_validate_routing found an inconsistency) and
 * COMFY_MOE_ETIMEOUT for any other code; a non-zero word is cleared once it has
 * been reported. */
int comfy_moe_read_status(int32_t* status, void* stream, int32_t* h_status);

#ifdef __cplusplus
}
#endif
#endif /* COMFY_B200_MOE_H_ */
