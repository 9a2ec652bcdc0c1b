// Weighted combine of the routed expert outputs plus the shared expert, one pass over HBM.
// Replaces expert_out.mul_(w), scatter_reduce_('sum') into a zeroed cache and "+ shared"
// (comfy/ldm/hidream/model.py:341-345, 324) and reproduces their bf16 rounding points:
//   p_k = bf16(bf16(w_k) * y_k);  r = bf16(p_0 + p_1);  out = bf16(r + shared).
// Thread c owns the 16-byte chunk c of every row; a block handles kTokensPerCombineBlock tokens
// (three row reads and one row write each).
#include "moe_common.cuh"

namespace comfy_b200 {

constexpr int kCombineMaxThreads = 512;          // dim / 8 threads per block: dim <= 4096
// One token per block: three row loads in flight per thread and few registers, so six blocks fit an SM and the
// 8192-token case runs as many short blocks instead of 1.15 waves of long ones (measured 31 us against 42 us with
// eight tokens per block).
constexpr int kTokensPerCombineBlock = 1;

// kTwo: every row has two partial results (an expert whose hidden dimension is split over two GPUs); their sum,
// rounded to bf16, stands in for the expert output the reference rounds once.
template <bool kTwo>
__global__ void __launch_bounds__(kCombineMaxThreads)
combine_kernel(const __nv_bfloat16* __restrict__ y_perm, const __nv_bfloat16* __restrict__ y_perm_b,
               const int32_t* __restrict__ row_map,
               const float* __restrict__ topk_weight, const __nv_bfloat16* __restrict__ y_shared, int n_tokens,
               int dim, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate,
               long long gate_batch_stride, const __nv_bfloat16* __restrict__ residual, int tokens_per_batch) {
  constexpr int kTok = kTokensPerCombineBlock < 4 ? kTokensPerCombineBlock : 4;
  const int tid = threadIdx.x;
  if (tid >= (dim >> 3)) return;
  const int block_tok0 = blockIdx.x * kTokensPerCombineBlock;
  for (int base = 0; base < kTokensPerCombineBlock; base += kTok) {
    const int t0 = block_tok0 + base;
    if (t0 >= n_tokens) break;
    uint4 va[kTok], vb[kTok], vs[kTok];
    uint4 va2[kTwo ? kTok : 1], vb2[kTwo ? kTok : 1];
    float w0[kTok], w1[kTok];
#pragma unroll
    for (int i = 0; i < kTok; ++i) {
      const int t = t0 + i;
      va[i] = vb[i] = vs[i] = make_uint4(0, 0, 0, 0);
      if constexpr (kTwo) va2[i] = vb2[i] = make_uint4(0, 0, 0, 0);
      w0[i] = w1[i] = 0.f;
      if (t < n_tokens) {
        // a negative row means "this slot was routed nowhere": it contributes zero
        const int r0 = __ldg(row_map + 2 * t), r1 = __ldg(row_map + 2 * t + 1);
        w0[i] = round_bf16(__ldg(topk_weight + 2 * t));
        w1[i] = round_bf16(__ldg(topk_weight + 2 * t + 1));
        if (r0 >= 0) va[i] = ld_nc_u4(reinterpret_cast<const uint4*>(y_perm + static_cast<size_t>(r0) * dim) + tid);
        if (r1 >= 0) vb[i] = ld_nc_u4(reinterpret_cast<const uint4*>(y_perm + static_cast<size_t>(r1) * dim) + tid);
        if constexpr (kTwo) {
          if (r0 >= 0) va2[i] = ld_nc_u4(reinterpret_cast<const uint4*>(y_perm_b + static_cast<size_t>(r0) * dim) + tid);
          if (r1 >= 0) vb2[i] = ld_nc_u4(reinterpret_cast<const uint4*>(y_perm_b + static_cast<size_t>(r1) * dim) + tid);
        }
        if (y_shared) vs[i] = ld_nc_u4(reinterpret_cast<const uint4*>(y_shared + static_cast<size_t>(t) * dim) + tid);
      }
    }
#pragma unroll
    for (int i = 0; i < kTok; ++i) {
      const int t = t0 + i;
      if (t >= n_tokens) continue;
      float fa[8], fb[8], fs[8], r[8];
      unpack_bf16x8(va[i], fa);
      unpack_bf16x8(vb[i], fb);
      unpack_bf16x8(vs[i], fs);
      if constexpr (kTwo) {
        float ga[8], gb[8];
        unpack_bf16x8(va2[i], ga);
        unpack_bf16x8(vb2[i], gb);
#pragma unroll
        for (int k = 0; k < 8; ++k) { fa[k] = round_bf16(fa[k] + ga[k]); fb[k] = round_bf16(fb[k] + gb[k]); }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float p0 = round_bf16(w0[i] * fa[k]);
        const float p1 = round_bf16(w1[i] * fb[k]);
        const float routed = round_bf16(p0 + p1);
        r[k] = y_shared ? routed + fs[k] : routed;
      }
      if (gate) {
        // block epilogue (comfy/ldm/hidream/model.py:432-433): gate_mlp * ff(x) + x, each step rounded to bf16
        float fg[8], fr[8];
        unpack_bf16x8(*(reinterpret_cast<const uint4*>(gate + (t / tokens_per_batch) * gate_batch_stride) + tid), fg);
        unpack_bf16x8(ld_nc_u4(reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * dim) + tid), fr);
#pragma unroll
        for (int k = 0; k < 8; ++k) r[k] = round_bf16(fg[k] * round_bf16(r[k])) + fr[k];
      }
      reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * dim)[tid] =
          make_uint4(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]), pack_bf16x2(r[4], r[5]), pack_bf16x2(r[6], r[7]));
    }
  }
}

}  // namespace comfy_b200

using namespace comfy_b200;

static int launch_combine(const void* y_perm, const void* y_perm_b, const int32_t* row_map, const float* topk_weight,
                          const void* y_shared, int n_tokens, int dim, void* out, void* stream,
                          const void* gate = nullptr, long long gate_batch_stride = 0, const void* residual = nullptr,
                          int tokens_per_batch = 1) {
  if (n_tokens < 0 || dim <= 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!y_perm || !row_map || !topk_weight || !out) return COMFY_MOE_EINVAL;
  if (!aligned16(y_perm) || !aligned16(out) || (y_shared && !aligned16(y_shared)) || (y_perm_b && !aligned16(y_perm_b)))
    return COMFY_MOE_EINVAL;
  if ((dim & 7) != 0 || (dim >> 3) > kCombineMaxThreads) return COMFY_MOE_EUNSUPPORTED;
  const int threads = ((dim >> 3) + 31) & ~31;
  const int blocks = (n_tokens + kTokensPerCombineBlock - 1) / kTokensPerCombineBlock;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* ya = static_cast<const __nv_bfloat16*>(y_perm);
  const __nv_bfloat16* yb = static_cast<const __nv_bfloat16*>(y_perm_b);
  const __nv_bfloat16* ys = static_cast<const __nv_bfloat16*>(y_shared);
  const __nv_bfloat16* g = static_cast<const __nv_bfloat16*>(gate);
  const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(residual);
  if (g && (!res || !aligned16(g) || !aligned16(res) || (gate_batch_stride % 8) != 0 || tokens_per_batch <= 0))
    return COMFY_MOE_EINVAL;
  if (yb)
    combine_kernel<true><<<blocks, threads, 0, s>>>(ya, yb, row_map, topk_weight, ys, n_tokens, dim,
                                                    static_cast<__nv_bfloat16*>(out), g, gate_batch_stride, res,
                                                    tokens_per_batch);
  else
    combine_kernel<false><<<blocks, threads, 0, s>>>(ya, nullptr, row_map, topk_weight, ys, n_tokens, dim,
                                                     static_cast<__nv_bfloat16*>(out), g, gate_batch_stride, res,
                                                     tokens_per_batch);
  return check_launch();
}

extern "C" int comfy_moe_combine(const void* y_perm, const int32_t* row_map, const float* topk_weight,
                                 const void* y_shared, int n_tokens, int dim, void* out, void* stream) {
  return launch_combine(y_perm, nullptr, row_map, topk_weight, y_shared, n_tokens, dim, out, stream);
}

extern "C" int comfy_moe_combine_partials(const void* y_perm_a, const void* y_perm_b, const int32_t* row_map,
                                          const float* topk_weight, const void* y_shared, int n_tokens, int dim,
                                          void* out, void* stream) {
  if (!y_perm_b) return COMFY_MOE_EINVAL;
  return launch_combine(y_perm_a, y_perm_b, row_map, topk_weight, y_shared, n_tokens, dim, out, stream);
}

extern "C" int comfy_moe_combine_block(const void* y_perm, const int32_t* row_map, const float* topk_weight,
                                       const void* y_shared, const void* gate, int64_t gate_batch_stride,
                                       const void* residual, int n_tokens, int tokens_per_batch, int dim, void* out,
                                       void* stream) {
  if (!gate || !residual) return COMFY_MOE_EINVAL;
  return launch_combine(y_perm, nullptr, row_map, topk_weight, y_shared, n_tokens, dim, out, stream, gate,
                        gate_batch_stride, residual, tokens_per_batch);
}
