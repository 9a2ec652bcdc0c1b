// Fused entry point and small utilities of the C ABI.
#include "moe_common.cuh"

extern "C" int comfy_moe_abi_version(void) { return COMFY_MOE_ABI_VERSION; }

extern "C" const char* comfy_moe_error_string(int code) {
  switch (code) {
    case COMFY_MOE_OK: return "ok";
    case COMFY_MOE_EINVAL: return "invalid argument (null pointer, negative size or misaligned pointer)";
    case COMFY_MOE_EUNSUPPORTED: return "shape, dtype or expert count not covered by the sm_100a kernels";
    case COMFY_MOE_ECUDA: return "a CUDA runtime or driver call failed";
    case COMFY_MOE_ETIMEOUT: return "a bounded device-side wait ran out";
    case COMFY_MOE_EDEVICE: return "device is not sm_100 or the driver lacks tensor-map support";
    case COMFY_MOE_ETOOLARGE:
      return "token count exceeds COMFY_MOE_STATIC_MAX_TOKENS, the capacity of the library's built-in scratch array";
    default: return "unknown error code";
  }
}

// The status word is sticky: kernels only ever move it from 0 to a code (atomicCAS), no entry point clears it on
// the way in, and this function clears it once it has handed a code to the host.  So a code left by any layer of a
// model is still there when the host looks, however many layers ran after it.
extern "C" int comfy_moe_read_status(int32_t* status, void* stream, int32_t* h_status) {
  if (!status || !h_status) return COMFY_MOE_EINVAL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(h_status, status, sizeof(int32_t), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return COMFY_MOE_ECUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return COMFY_MOE_ECUDA;
  if (*h_status == 0) return COMFY_MOE_OK;
  if (cudaMemsetAsync(status, 0, sizeof(int32_t), s) != cudaSuccess) return COMFY_MOE_ECUDA;
  if (*h_status == 8) return COMFY_MOE_ETOOLARGE;    // routed rows exceed a peer receive buffer
  if (*h_status == 9) return COMFY_MOE_EINVAL;       // the routing check found an inconsistency
  return COMFY_MOE_ETIMEOUT;
}

// Block epilogue requested by comfy_moe_ffn_block: gate * (.) + residual folded into the combine.
struct BlockEpilogue {
  const void* gate;
  int64_t gate_batch_stride;
  const void* residual;
  int tokens_per_batch;
};

// MOEFeedForwardSwiGLU.forward (comfy/ldm/hidream/model.py:307-325) as five launches on one stream:
// gate, routing plan + permutation, two passes of the grouped GEMM, combine.
static int forward_impl(const ComfyMoeLayer* L, const ComfyMoeWorkspace* ws, const void* x, int n_tokens, void* out,
                        void* stream, const BlockEpilogue* epi, bool gate_done = false) {
  if (!L || !ws || n_tokens < 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!x || !out) return COMFY_MOE_EINVAL;
  if (L->top_k != 2 || L->n_experts < 2 || L->n_experts > COMFY_MOE_MAX_EXPERTS) return COMFY_MOE_EUNSUPPORTED;
  if (!ws->topk_idx || !ws->topk_weight || !ws->block_counts || !ws->block_offsets || !ws->expert_counts ||
      !ws->expert_offsets || !ws->row_map || !ws->status || !ws->x_perm || !ws->h_perm || !ws->y_perm ||
      !ws->h_shared || !ws->y_shared)
    return COMFY_MOE_EINVAL;
  int64_t rows_need = 0;
  int rc = comfy_moe_plan_sizes(n_tokens, L->n_experts, L->top_k, &rows_need, nullptr);
  if (rc != COMFY_MOE_OK) return rc;
  if (ws->rows_cap < rows_need) return COMFY_MOE_EINVAL;
  const bool fp8 = L->w_dtype == COMFY_MOE_FP8_E4M3;
  if (fp8 && !ws->x_q) return COMFY_MOE_EINVAL;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!gate_done) {
    // only the near-tie counter starts from zero; the status word keeps whatever an earlier call left in it
    if (cudaMemsetAsync(ws->status + 1, 0, sizeof(int32_t), s) != cudaSuccess) return COMFY_MOE_ECUDA;
    rc = comfy_moe_gate_topk(x, L->w_gate, L->gate_dtype, n_tokens, L->dim, L->n_experts, L->top_k, ws->topk_idx,
                             ws->topk_weight, ws->block_counts, ws->status + 1, nullptr, 1e-6f, stream);
    if (rc != COMFY_MOE_OK) return rc;
  }
  rc = comfy_moe_plan_permute(x, ws->topk_idx, ws->block_counts, n_tokens, L->dim, L->n_experts,
                              fp8 ? COMFY_MOE_FP8_E4M3 : COMFY_MOE_BF16, fp8 ? L->experts[0].scale_in13 : nullptr,
                              ws->block_offsets, ws->expert_counts, ws->expert_offsets, ws->x_perm,
                              fp8 ? ws->x_q : nullptr, fp8 ? L->shared.scale_in13 : nullptr, ws->row_map,
                              ws->status + 2, stream);
  if (rc != COMFY_MOE_OK) return rc;
  rc = comfy_moe_grouped_swiglu(L->w_dtype, L->n_experts, L->experts, &L->shared, ws->expert_offsets,
                                ws->expert_counts, ws->rows_cap, n_tokens, L->dim, ws->x_perm, ws->h_perm, ws->y_perm,
                                fp8 ? ws->x_q : x, ws->h_shared, ws->y_shared, ws->status, stream);
  if (rc != COMFY_MOE_OK) return rc;
  if (epi)
    return comfy_moe_combine_block(ws->y_perm, ws->row_map, ws->topk_weight, ws->y_shared, epi->gate,
                                   epi->gate_batch_stride, epi->residual, n_tokens, epi->tokens_per_batch, L->dim, out,
                                   stream);
  return comfy_moe_combine(ws->y_perm, ws->row_map, ws->topk_weight, ws->y_shared, n_tokens, L->dim, out, stream);
}

extern "C" int comfy_moe_forward(const ComfyMoeLayer* L, const ComfyMoeWorkspace* ws, const void* x, int n_tokens,
                                 void* out, void* stream) {
  return forward_impl(L, ws, x, n_tokens, out, stream, nullptr);
}

// MoEBlock.forward in eval mode (comfy/ldm/hunyuan3dv2_1/hunyuandit.py:130-185): the same five launches with the
// GELU-MLP expert passes in the middle.
extern "C" int comfy_moe_forward_gelu_mlp(const ComfyMoeMlpLayer* L, const ComfyMoeWorkspace* ws, const void* x,
                                          int n_tokens, void* out, void* stream) {
  if (!L || !ws || n_tokens < 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!x || !out) return COMFY_MOE_EINVAL;
  if (L->top_k != 2 || L->n_experts < 2 || L->n_experts > COMFY_MOE_MAX_EXPERTS) return COMFY_MOE_EUNSUPPORTED;
  if (!ws->topk_idx || !ws->topk_weight || !ws->block_counts || !ws->block_offsets || !ws->expert_counts ||
      !ws->expert_offsets || !ws->row_map || !ws->status || !ws->x_perm || !ws->h_perm || !ws->y_perm ||
      !ws->h_shared || !ws->y_shared)
    return COMFY_MOE_EINVAL;
  int64_t rows_need = 0;
  int rc = comfy_moe_plan_sizes(n_tokens, L->n_experts, L->top_k, &rows_need, nullptr);
  if (rc != COMFY_MOE_OK) return rc;
  if (ws->rows_cap < rows_need) return COMFY_MOE_EINVAL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(ws->status + 1, 0, sizeof(int32_t), s) != cudaSuccess) return COMFY_MOE_ECUDA;
  rc = comfy_moe_gate_topk(x, L->w_gate, L->gate_dtype, n_tokens, L->dim, L->n_experts, L->top_k, ws->topk_idx,
                           ws->topk_weight, ws->block_counts, ws->status + 1, nullptr, 1e-6f, stream);
  if (rc != COMFY_MOE_OK) return rc;
  rc = comfy_moe_plan_permute(x, ws->topk_idx, ws->block_counts, n_tokens, L->dim, L->n_experts, COMFY_MOE_BF16,
                              nullptr, ws->block_offsets, ws->expert_counts, ws->expert_offsets, ws->x_perm, nullptr,
                              nullptr, ws->row_map, nullptr, stream);
  if (rc != COMFY_MOE_OK) return rc;
  rc = comfy_moe_grouped_gelu_mlp(L->n_experts, L->experts, &L->shared, ws->expert_offsets, ws->expert_counts,
                                  ws->rows_cap, n_tokens, L->dim, ws->x_perm, ws->h_perm, ws->y_perm, x, ws->h_shared,
                                  ws->y_shared, ws->status, stream);
  if (rc != COMFY_MOE_OK) return rc;
  return comfy_moe_combine(ws->y_perm, ws->row_map, ws->topk_weight, ws->y_shared, n_tokens, L->dim, out, stream);
}

// Feed-forward half of a HiDream block (comfy/ldm/hidream/model.py:429-433): LayerNorm + modulation, the MoE,
// gate * (.) + residual.
extern "C" int comfy_moe_ffn_block(const ComfyMoeLayer* L, const ComfyMoeWorkspace* ws, const void* x,
                                   const void* shift, const void* scale, const void* gate, int64_t mod_batch_stride,
                                   int n_tokens, int tokens_per_batch, float eps, void* out, void* stream) {
  if (!L || !ws || !ws->x_mod) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!ws->topk_idx || !ws->topk_weight || !ws->block_counts || !ws->status) return COMFY_MOE_EINVAL;
  // LayerNorm + modulation, then the gate kernel on its output (which is still in L2).  comfy_moe_ln_modulate_gate does
  // both in one kernel with identical results, but a warp there owns one row, so every gate weight it reads feeds a
  // single FMA; the gate kernel reuses each weight for four tokens, and both kernels are bound by instruction issue:
  // at 8192 x 2560 the two launches take 34 us (46 us from a cold L2), the fused kernel 43 us (59 us).
  int rc = comfy_moe_ln_modulate(x, shift, scale, mod_batch_stride, n_tokens, tokens_per_batch, L->dim, eps, ws->x_mod,
                                 stream);
  if (rc != COMFY_MOE_OK) return rc;
  const BlockEpilogue epi = {gate, mod_batch_stride, x, tokens_per_batch};
  return forward_impl(L, ws, ws->x_mod, n_tokens, out, stream, &epi);
}
