// The element-wise passes a HiDream transformer block runs around its feed-forward
// (comfy/ldm/hidream/model.py:429-433 and :515-523):
//     n   = LayerNorm(x)            (eps 1e-6, no affine, fp32 statistics, output in the activation dtype)
//     in  = n * (1 + scale) + shift (per batch element modulation vectors)
//     out = gate * ff(in) + x
// `ln_modulate_kernel` does the first two lines in one pass over HBM; `gate_residual_kernel` does the
// last line for a dense feed-forward (for the MoE it is folded into the combine kernel instead).
// Every bf16 rounding point of the PyTorch composition is kept.
#include "moe_common.cuh"

namespace comfy_b200 {

constexpr int kLnWarps = 8;              // rows per block in flight, one warp each
constexpr int kLnMaxChunks = 16;         // 16-byte chunks per lane: dim <= 16 * 32 * 8 = 4096

// One warp per row: the whole row sits in the warp's registers (lane l owns chunks l, l + 32, ...), the mean and
// the centred second moment are two shuffle reductions, no shared memory and no block barrier.
template <int kChunksPerLane>
__global__ void __launch_bounds__(kLnWarps * 32)
ln_modulate_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ shift,
                   const __nv_bfloat16* __restrict__ scale, long long mod_batch_stride, int n_tokens,
                   int tokens_per_batch, int dim, float eps, __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int chunks = dim >> 3;
  const float inv_dim = 1.0f / static_cast<float>(dim);
  for (int t = blockIdx.x * kLnWarps + (threadIdx.x >> 5); t < n_tokens; t += gridDim.x * kLnWarps) {
    const uint4* row = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * dim);
    uint4 v[kChunksPerLane];
#pragma unroll
    for (int j = 0; j < kChunksPerLane; ++j) {
      const int c = lane + 32 * j;
      v[j] = c < chunks ? ld_nc_u4(row + c) : make_uint4(0, 0, 0, 0);
    }
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kChunksPerLane; ++j) {
      float f[8];
      unpack_bf16x8(v[j], f);
#pragma unroll
      for (int k = 0; k < 8; ++k) sum += f[k];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float mean = sum * inv_dim;
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < kChunksPerLane; ++j) {
      if (lane + 32 * j < chunks) {
        float f[8];
        unpack_bf16x8(v[j], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float d = f[k] - mean;
          sq = fmaf(d, d, sq);
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
    const float rstd = rsqrtf(sq * inv_dim + eps);
    const int b = t / tokens_per_batch;
    const uint4* sc_row = reinterpret_cast<const uint4*>(scale + b * mod_batch_stride);
    const uint4* sh_row = reinterpret_cast<const uint4*>(shift + b * mod_batch_stride);
    uint4* o_row = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * dim);
#pragma unroll
    for (int j = 0; j < kChunksPerLane; ++j) {
      const int c = lane + 32 * j;
      if (c < chunks) {
        float f[8], sc[8], sh[8], o[8];
        unpack_bf16x8(v[j], f);
        unpack_bf16x8(sc_row[c], sc);
        unpack_bf16x8(sh_row[c], sh);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float n = round_bf16((f[k] - mean) * rstd);        // LayerNorm output, activation dtype
          const float one_plus = round_bf16(1.0f + sc[k]);         // (1 + scale) is a bf16 tensor in the reference
          o[k] = round_bf16(n * one_plus) + sh[k];                 // product rounded, sum rounded by the pack
        }
        o_row[c] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]),
                              pack_bf16x2(o[6], o[7]));
      }
    }
  }
}

// out = bf16(bf16(gate[b] * y) + residual), 16 bytes per thread, grid-stride.
__global__ void __launch_bounds__(256)
gate_residual_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ gate,
                     long long gate_batch_stride, const __nv_bfloat16* __restrict__ residual, int n_tokens,
                     int tokens_per_batch, int dim, __nv_bfloat16* __restrict__ out) {
  const int chunks = dim >> 3;
  const long long total = static_cast<long long>(n_tokens) * chunks;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / chunks), c = static_cast<int>(i - static_cast<long long>(t) * chunks);
    const int b = t / tokens_per_batch;
    float fy[8], fg[8], fr[8], o[8];
    unpack_bf16x8(ld_nc_u4(reinterpret_cast<const uint4*>(y) + i), fy);
    unpack_bf16x8(*(reinterpret_cast<const uint4*>(gate + b * gate_batch_stride) + c), fg);
    unpack_bf16x8(ld_nc_u4(reinterpret_cast<const uint4*>(residual) + i), fr);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = round_bf16(fg[k] * fy[k]) + fr[k];
    reinterpret_cast<uint4*>(out)[i] =
        make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
  }
}

// bf16 -> e4m3 with the activation quantiser of comfy/ops.py:338-343.  Without a scale: clamp to +-448, round to
// nearest even.  With one: multiply by bf16(1 / scale), rounded to bf16, and cast WITHOUT a clamp, as the reference does;
// what overflows becomes NaN and is counted.  32 bytes read and 16 written per thread and step.
__global__ void __launch_bounds__(256)
quantize_e4m3_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale, long long n_chunks,
                     uint8_t* __restrict__ out, int32_t* __restrict__ overflow_count) {
  float inv = 1.f;
  bool scaled = false;
  int ovf = 0;
  if (scale) { inv = round_bf16(1.0f / __ldg(scale)); scaled = true; }
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_chunks;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x) + 2 * i;
    float f[16];
    {
      float fa[8], fb[8];
      unpack_bf16x8(ld_nc_u4(src), fa);
      unpack_bf16x8(ld_nc_u4(src + 1), fb);
#pragma unroll
      for (int k = 0; k < 8; ++k) { f[k] = fa[k]; f[8 + k] = fb[k]; }
    }
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float g[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) g[m] = scaled ? round_bf16(f[4 * k + m] * inv) : f[4 * k + m];
      w[k] = scaled ? (static_cast<uint32_t>(f2_to_e4m3x2_nosat(g[0], g[1], ovf)) |
                       (static_cast<uint32_t>(f2_to_e4m3x2_nosat(g[2], g[3], ovf)) << 16))
                    : (static_cast<uint32_t>(f2_to_e4m3x2(g[0], g[1])) |
                       (static_cast<uint32_t>(f2_to_e4m3x2(g[2], g[3])) << 16));
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  if (ovf && overflow_count) atomicAdd(overflow_count, ovf);
}

}  // namespace comfy_b200

using namespace comfy_b200;

static bool modulation_ok(const void* p, long long batch_stride) {
  return p && aligned16(p) && (batch_stride % 8) == 0;
}

extern "C" int comfy_moe_ln_modulate(const void* x, const void* shift, const void* scale, int64_t mod_batch_stride,
                                     int n_tokens, int tokens_per_batch, int dim, float eps, void* out, void* stream) {
  if (n_tokens < 0 || dim <= 0 || tokens_per_batch <= 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!x || !out || !aligned16(x) || !aligned16(out)) return COMFY_MOE_EINVAL;
  if (!modulation_ok(shift, mod_batch_stride) || !modulation_ok(scale, mod_batch_stride)) return COMFY_MOE_EINVAL;
  if ((dim & 7) != 0 || (dim >> 3) > kLnMaxChunks * 32) return COMFY_MOE_EUNSUPPORTED;
  int blocks = (n_tokens + kLnWarps - 1) / kLnWarps;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const int per_lane = ((dim >> 3) + 31) / 32;     // registers hold the row: pick the smallest instantiation that fits
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* shp = static_cast<const __nv_bfloat16*>(shift);
  const __nv_bfloat16* scp = static_cast<const __nv_bfloat16*>(scale);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
#define COMFY_LN_LAUNCH(K) \
  ln_modulate_kernel<K><<<blocks, kLnWarps * 32, 0, s>>>(xp, shp, scp, mod_batch_stride, n_tokens, tokens_per_batch, \
                                                          dim, eps, op)
  if (per_lane <= 2) COMFY_LN_LAUNCH(2);
  else if (per_lane <= 4) COMFY_LN_LAUNCH(4);
  else if (per_lane <= 8) COMFY_LN_LAUNCH(8);
  else if (per_lane <= 10) COMFY_LN_LAUNCH(10);
  else if (per_lane <= 12) COMFY_LN_LAUNCH(12);
  else COMFY_LN_LAUNCH(16);
#undef COMFY_LN_LAUNCH
  return check_launch();
}

extern "C" int comfy_moe_gate_residual(const void* y, const void* gate, int64_t gate_batch_stride,
                                       const void* residual, int n_tokens, int tokens_per_batch, int dim, void* out,
                                       void* stream) {
  if (n_tokens < 0 || dim <= 0 || tokens_per_batch <= 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!y || !residual || !out || !aligned16(y) || !aligned16(residual) || !aligned16(out)) return COMFY_MOE_EINVAL;
  if (!modulation_ok(gate, gate_batch_stride)) return COMFY_MOE_EINVAL;
  if ((dim & 7) != 0) return COMFY_MOE_EUNSUPPORTED;
  const long long total = static_cast<long long>(n_tokens) * (dim >> 3);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  gate_residual_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(gate), gate_batch_stride,
      static_cast<const __nv_bfloat16*>(residual), n_tokens, tokens_per_batch, dim, static_cast<__nv_bfloat16*>(out));
  return check_launch();
}

extern "C" int comfy_moe_quantize_e4m3(const void* x, const float* scale, int64_t n_elements, void* out,
                                       int32_t* overflow_count, void* stream) {
  if (n_elements < 0) return COMFY_MOE_EINVAL;
  if (n_elements == 0) return COMFY_MOE_OK;
  if (!x || !out || !aligned16(x) || !aligned16(out)) return COMFY_MOE_EINVAL;
  if ((n_elements & 15) != 0) return COMFY_MOE_EUNSUPPORTED;
  const long long chunks = n_elements >> 4;
  long long blocks = (chunks + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  quantize_e4m3_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), scale, chunks, static_cast<uint8_t*>(out), overflow_count);
  return check_launch();
}
