// Element-wise passes between the q / k / v projections and the attention call of a HiDream block
// (comfy/ldm/hidream/model.py:97-137): RMSNorm over the whole projected row (torch.nn.functional.rms_norm through
// comfy/rmsnorm.py:14-20: fp32 statistics, one rounding to the activation dtype), the concatenation of image and text
// tokens along the sequence (:120-122), and the rotary embedding (comfy/ldm/flux/math.py:38-47: fp32 2x2 rotation of
// neighbouring pairs, rounded back).  One pass over HBM per projected tensor instead of about ten.
#include "moe_common.cuh"

namespace comfy_b200 {

constexpr int kNormWarps = 8;              // rows per block, one warp each
constexpr int kNormMaxChunks = 16;         // 16-byte chunks per lane: inner dim <= 4096

// One warp per row; the row sits in registers (lane l owns chunks l, l + 32, ...).
//   n   = bf16( x * rsqrt(mean(x^2) + eps) * w )          (weight == nullptr: n = x, no normalisation)
//   out = bf16( f[i][0] * n[2p] + f[i][1] * n[2p+1] )     for the pairs p < rope_pairs of every head, copied otherwise
// The output row of token (b, s) is out + b * out_batch_stride + (out_row_offset + s) * inner, so the image and the
// text part of a joint sequence are written into one buffer by two calls.
template <int kChunksPerLane>
__global__ void __launch_bounds__(kNormWarps * 32, 3)      // three blocks per SM: measured best (27 us against 29 / 31)
rmsnorm_rope_kernel(const __nv_bfloat16* __restrict__ x, long long ld_x, const __nv_bfloat16* __restrict__ weight,
                    float eps, const float* __restrict__ rope, long long rope_batch_stride, int rope_row_offset,
                    int rope_pairs, int n_tokens, int tokens_per_batch, int inner, int head_dim,
                    __nv_bfloat16* __restrict__ out, long long out_batch_stride, int out_row_offset) {
  const int lane = threadIdx.x & 31;
  const int chunks = inner >> 3;
  const float inv_dim = 1.0f / static_cast<float>(inner);
  for (int t = blockIdx.x * kNormWarps + (threadIdx.x >> 5); t < n_tokens; t += gridDim.x * kNormWarps) {
    const uint4* row = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * ld_x);
    uint4 v[kChunksPerLane];
#pragma unroll
    for (int j = 0; j < kChunksPerLane; ++j) {
      const int c = lane + 32 * j;
      v[j] = c < chunks ? ld_nc_u4(row + c) : make_uint4(0, 0, 0, 0);
    }
    float rstd = 1.0f;
    if (weight != nullptr) {
      float sq = 0.f;
#pragma unroll
      for (int j = 0; j < kChunksPerLane; ++j) {
        float f[8];
        unpack_bf16x8(v[j], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) sq = fmaf(f[k], f[k], sq);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
      rstd = rsqrtf(sq * inv_dim + eps);
    }
    const int b = t / tokens_per_batch, s = t - b * tokens_per_batch;
    const float4* rope_row = rope ? reinterpret_cast<const float4*>(rope + b * rope_batch_stride) +
                                        static_cast<size_t>(rope_row_offset + s) * rope_pairs
                                  : nullptr;
    uint4* o_row = reinterpret_cast<uint4*>(out + b * out_batch_stride + static_cast<size_t>(out_row_offset + s) * inner);
    // A lane's chunks are 32 chunks (256 elements) apart: when head_dim divides 256 they all sit at the same place
    // inside their heads and share four rotation matrices, loaded once per row instead of once per chunk.
    const bool same_pairs = (256 % head_dim) == 0;
    const int lane_pair0 = ((lane << 3) % head_dim) >> 1;
    float4 rot[4];
    if (rope_row != nullptr && same_pairs) {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        rot[q] = lane_pair0 + q < rope_pairs ? __ldg(rope_row + lane_pair0 + q) : make_float4(1.f, 0.f, 0.f, 1.f);
    }
#pragma unroll
    for (int j = 0; j < kChunksPerLane; ++j) {
      const int c = lane + 32 * j;
      if (c < chunks) {
        float f[8], n[8], o[8];
        unpack_bf16x8(v[j], f);
        if (weight != nullptr) {
          float w[8];
          unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(weight) + c), w);
#pragma unroll
          for (int k = 0; k < 8; ++k) n[k] = round_bf16(f[k] * rstd * w[k]);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) n[k] = f[k];
        }
        const int pair0 = ((c << 3) % head_dim) >> 1;      // first of this chunk's four pairs inside its head
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (rope_row != nullptr && pair0 + q < rope_pairs) {
            const float4 r = same_pairs ? rot[q] : __ldg(rope_row + pair0 + q);    // f[0][0], f[0][1], f[1][0], f[1][1]
            o[2 * q] = fmaf(r.y, n[2 * q + 1], r.x * n[2 * q]);
            o[2 * q + 1] = fmaf(r.w, n[2 * q + 1], r.z * n[2 * q]);
          } else {
            o[2 * q] = n[2 * q];
            o[2 * q + 1] = n[2 * q + 1];
          }
        }
        o_row[c] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]),
                              pack_bf16x2(o[6], o[7]));
      }
    }
  }
}

}  // namespace comfy_b200

using namespace comfy_b200;

extern "C" int comfy_attn_rmsnorm_rope(const void* x, int64_t ld_x, const void* weight, float eps, const float* rope,
                                       int64_t rope_batch_stride, int rope_row_offset, int rope_pairs, int n_tokens,
                                       int tokens_per_batch, int heads, int head_dim, void* out,
                                       int64_t out_batch_stride, int out_row_offset, void* stream) {
  if (n_tokens < 0 || tokens_per_batch <= 0 || heads <= 0 || head_dim <= 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  const int inner = heads * head_dim;
  if (!x || !out || !aligned16(x) || !aligned16(out) || (weight && !aligned16(weight))) return COMFY_MOE_EINVAL;
  if ((head_dim & 7) != 0 || (inner >> 3) > kNormMaxChunks * 32) return COMFY_MOE_EUNSUPPORTED;
  if (ld_x < inner || (ld_x & 7) != 0 || (out_batch_stride & 7) != 0 || out_row_offset < 0) return COMFY_MOE_EINVAL;
  if (rope) {
    if (rope_pairs <= 0 || rope_pairs * 2 > head_dim || rope_row_offset < 0) return COMFY_MOE_EINVAL;
    if ((reinterpret_cast<uintptr_t>(rope) & 15u) != 0 || (rope_batch_stride & 3) != 0) return COMFY_MOE_EINVAL;
  }
  int blocks = (n_tokens + kNormWarps - 1) / kNormWarps;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const int per_lane = ((inner >> 3) + 31) / 32;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(weight);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
#define COMFY_NORM_LAUNCH(K)                                                                                        \
  rmsnorm_rope_kernel<K><<<blocks, kNormWarps * 32, 0, s>>>(xp, ld_x, wp, eps, rope, rope_batch_stride,             \
                                                            rope_row_offset, rope_pairs, n_tokens, tokens_per_batch, \
                                                            inner, head_dim, op, out_batch_stride, out_row_offset)
  if (per_lane <= 2) COMFY_NORM_LAUNCH(2);
  else if (per_lane <= 4) COMFY_NORM_LAUNCH(4);
  else if (per_lane <= 8) COMFY_NORM_LAUNCH(8);
  else if (per_lane <= 10) COMFY_NORM_LAUNCH(10);
  else if (per_lane <= 12) COMFY_NORM_LAUNCH(12);
  else COMFY_NORM_LAUNCH(16);
#undef COMFY_NORM_LAUNCH
  return check_launch();
}
