// Weighted combine of the routed expert outputs plus the shared expert, one pass over HBM.
// Replaces expert_out.mul_(w), scatter_reduce_('sum') into a zeroed cache and "+ shared"
// (comfy/ldm/hidream/model.py:341-345, 324) and reproduces their bf16 rounding points:
//   p_k = bf16(bf16(w_k) * y_k);  r = bf16(p_0 + p_1);  out = bf16(r + shared).
#include "moe_common.cuh"

namespace comfy_b200 {

constexpr int kCombineThreads = 256;

__global__ void __launch_bounds__(kCombineThreads)
combine_kernel(const __nv_bfloat16* __restrict__ y_perm, const int32_t* __restrict__ row_map,
               const float* __restrict__ topk_weight, const __nv_bfloat16* __restrict__ y_shared, int n_tokens,
               int dim, __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = kCombineThreads / 32;
  const int chunks = dim >> 3;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < n_tokens; t += gridDim.x * warps_per_block) {
    const int r0 = __ldg(row_map + 2 * t), r1 = __ldg(row_map + 2 * t + 1);
    const float w0 = round_bf16(__ldg(topk_weight + 2 * t));
    const float w1 = round_bf16(__ldg(topk_weight + 2 * t + 1));
    // a negative row means "this slot was routed nowhere": it contributes zero
    const uint4* a = r0 >= 0 ? reinterpret_cast<const uint4*>(y_perm + static_cast<size_t>(r0) * dim) : nullptr;
    const uint4* b = r1 >= 0 ? reinterpret_cast<const uint4*>(y_perm + static_cast<size_t>(r1) * dim) : nullptr;
    const uint4* s = y_shared ? reinterpret_cast<const uint4*>(y_shared + static_cast<size_t>(t) * dim) : nullptr;
    uint4* o = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * dim);
    constexpr int kBatch = 5;
    for (int c0 = lane; c0 < chunks; c0 += 32 * kBatch) {
      uint4 va[kBatch], vb[kBatch], vs[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int c = c0 + 32 * j;
        if (c < chunks) {
          va[j] = a ? ld_nc_u4(a + c) : make_uint4(0, 0, 0, 0);
          vb[j] = b ? ld_nc_u4(b + c) : make_uint4(0, 0, 0, 0);
          vs[j] = s ? ld_nc_u4(s + c) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int c = c0 + 32 * j;
        if (c < chunks) {
          float fa[8], fb[8], fs[8], r[8];
          unpack_bf16x8(va[j], fa);
          unpack_bf16x8(vb[j], fb);
          unpack_bf16x8(vs[j], fs);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float p0 = round_bf16(w0 * fa[i]);
            const float p1 = round_bf16(w1 * fb[i]);
            const float routed = round_bf16(p0 + p1);
            r[i] = s ? routed + fs[i] : routed;
          }
          o[c] = make_uint4(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]), pack_bf16x2(r[4], r[5]),
                            pack_bf16x2(r[6], r[7]));
        }
      }
    }
  }
}

}  // namespace comfy_b200

using namespace comfy_b200;

extern "C" int comfy_moe_combine(const void* y_perm, const int32_t* row_map, const float* topk_weight,
                                 const void* y_shared, int n_tokens, int dim, void* out, void* stream) {
  if (n_tokens < 0 || dim <= 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!y_perm || !row_map || !topk_weight || !out) return COMFY_MOE_EINVAL;
  if (!aligned16(y_perm) || !aligned16(out) || (y_shared && !aligned16(y_shared))) return COMFY_MOE_EINVAL;
  if ((dim & 7) != 0) return COMFY_MOE_EUNSUPPORTED;
  const int warps_per_block = kCombineThreads / 32;
  int blocks = (n_tokens + warps_per_block - 1) / warps_per_block;
  if (blocks > 148 * 8) blocks = 148 * 8;
  combine_kernel<<<blocks, kCombineThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y_perm), row_map, topk_weight, static_cast<const __nv_bfloat16*>(y_shared),
      n_tokens, dim, static_cast<__nv_bfloat16*>(out));
  return check_launch();
}
