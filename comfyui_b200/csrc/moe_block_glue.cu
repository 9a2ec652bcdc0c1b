// The element-wise passes a HiDream transformer block runs around its feed-forward
// (comfy/ldm/hidream/model.py:429-433 and :515-523):
//     n   = LayerNorm(x)            (eps 1e-6, no affine, fp32 statistics, output in the activation dtype)
//     in  = n * (1 + scale) + shift (per batch element modulation vectors)
//     out = gate * ff(in) + x
// `ln_modulate_kernel` does the first two lines in one pass over HBM; `gate_residual_kernel` does the
// last line for a dense feed-forward (for the MoE it is folded into the combine kernel instead).
// Every bf16 rounding point of the PyTorch composition is kept.
#include "moe_common.cuh"
#include "moe_gate.cuh"

namespace comfy_b200 {

__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t w) { return *reinterpret_cast<const __nv_bfloat162*>(&w); }
__device__ __forceinline__ __nv_bfloat162 kOneBf162() { return as_bf162(0x3f803f80u); }      // (1.0, 1.0)

constexpr int kLnWarps = 8;              // rows per block in flight, one warp each
constexpr int kLnMaxChunks = 16;         // 16-byte chunks per lane: dim <= 16 * 32 * 8 = 4096

// One warp per row: the whole row sits in the warp's registers (lane l owns chunks l, l + 32, ...), the mean and
// the centred second moment are two shuffle reductions, no shared memory and no block barrier.
// Arguments of the optional gate that rides on the LayerNorm pass (kGateE > 0): MoEGate.forward on the row the warp has
// just produced.  The warp holds the bf16-rounded output row in registers, lane l owning the same chunks l, l + 32, ...
// the stand-alone gate kernel gives it, so the logits are accumulated in the same order and come out bit for bit
// the same; what the fusion saves is the gate's re-read of the row from memory and its launch.
struct LnGateArgs {
  const void* w_gate;          // [E, dim] as stored (bf16 or fp32), read through L1 (20 KB at dim 2560)
  int32_t* topk_idx;           // [n_tokens, 2]
  float* topk_weight;          // [n_tokens, 2]
  int32_t* block_counts;       // [ceil(n_tokens / kTokensPerBlock), E], zeroed by the caller; filled with atomics
  int32_t* neartie_count;      // may be NULL
  uint8_t* neartie_flags;      // may be NULL
  float neartie_eps;
};

template <int kChunksPerLane, int kGateE = 0, bool kGateW32 = false>
__global__ void __launch_bounds__(kLnWarps * 32)
ln_modulate_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ shift,
                   const __nv_bfloat16* __restrict__ scale, long long mod_batch_stride, int n_tokens,
                   int tokens_per_batch, int dim, float eps, __nv_bfloat16* __restrict__ out, const LnGateArgs gate) {
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
    constexpr int kAcc = kGateE > 0 ? kGateE : 1;
    float acc[kAcc];
#pragma unroll
    for (int e = 0; e < kAcc; ++e) acc[e] = 0.f;
#pragma unroll
    for (int j = 0; j < kChunksPerLane; ++j) {
      const int c = lane + 32 * j;
      if (c < chunks) {
        // n = bf16((x - mean) * rstd) in fp32, two values per conversion; the rest of the line is bf16 arithmetic in the
        // reference (each operation exact in fp32, rounded once to bf16), which is what the packed bf16x2 instructions
        // compute: bf16(1 + scale), bf16(n * .), bf16(. + shift); the _rn forms, which may not be contracted into one fma
        float f[8];
        unpack_bf16x8(v[j], f);
        const uint4 scv = sc_row[c], shv = sh_row[c];
        const uint32_t scw[4] = {scv.x, scv.y, scv.z, scv.w}, shw[4] = {shv.x, shv.y, shv.z, shv.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const __nv_bfloat162 n = __floats2bfloat162_rn((f[2 * k] - mean) * rstd, (f[2 * k + 1] - mean) * rstd);
          const __nv_bfloat162 one_plus = __hadd2_rn(kOneBf162(), as_bf162(scw[k]));
          const __nv_bfloat162 o = __hadd2_rn(__hmul2_rn(n, one_plus), as_bf162(shw[k]));
          ow[k] = *reinterpret_cast<const uint32_t*>(&o);
        }
        const uint4 packed = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        o_row[c] = packed;
        if constexpr (kGateE > 0) {
          float g[8];
          unpack_bf16x8(packed, g);                                // the bf16 values the gate would read back
          gate_accumulate<kGateE, kGateW32>(static_cast<const uint4*>(gate.w_gate), kGateW32 ? chunks * 2 : chunks, c,
                                            g, acc);
        }
      }
    }
    if constexpr (kGateE > 0) {
#pragma unroll
      for (int e = 0; e < kGateE; ++e) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
      }
      int i0, i1;
      float w0, w1;
      bool tie;
      gate_select<kGateE>(acc, gate.neartie_eps, i0, i1, w0, w1, tie);
      if (lane == 0) {
        gate.topk_idx[2 * t] = i0;
        gate.topk_idx[2 * t + 1] = i1;
        gate.topk_weight[2 * t] = w0;
        gate.topk_weight[2 * t + 1] = w1;
        int32_t* counts = gate.block_counts + (t / kTokensPerBlock) * kGateE;
        atomicAdd(counts + i0, 1);                                 // integer atomics: the sums do not depend on order
        atomicAdd(counts + i1, 1);
        if (gate.neartie_flags) gate.neartie_flags[t] = tie ? 1 : 0;
        if (tie && gate.neartie_count) atomicAdd(gate.neartie_count, 1);
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

template <int E, bool W32>
static void launch_ln(int per_lane, int blocks, cudaStream_t s, const __nv_bfloat16* xp, const __nv_bfloat16* shp,
                      const __nv_bfloat16* scp, int64_t mod_batch_stride, int n_tokens, int tokens_per_batch, int dim,
                      float eps, __nv_bfloat16* op, const LnGateArgs& gate) {
#define COMFY_LN_LAUNCH(K) \
  ln_modulate_kernel<K, E, W32><<<blocks, kLnWarps * 32, 0, s>>>(xp, shp, scp, mod_batch_stride, n_tokens, \
                                                                  tokens_per_batch, dim, eps, op, gate)
  // registers hold the row: pick the smallest instantiation that fits
  if (per_lane <= 2) COMFY_LN_LAUNCH(2);
  else if (per_lane <= 4) COMFY_LN_LAUNCH(4);
  else if (per_lane <= 8) COMFY_LN_LAUNCH(8);
  else if (per_lane <= 10) COMFY_LN_LAUNCH(10);
  else if (per_lane <= 12) COMFY_LN_LAUNCH(12);
  else COMFY_LN_LAUNCH(16);
#undef COMFY_LN_LAUNCH
}

static int ln_modulate_impl(const void* x, const void* shift, const void* scale, int64_t mod_batch_stride, int n_tokens,
                            int tokens_per_batch, int dim, float eps, void* out, const LnGateArgs* gate, int gate_dtype,
                            int n_experts, void* stream) {
  if (n_tokens < 0 || dim <= 0 || tokens_per_batch <= 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!x || !out || !aligned16(x) || !aligned16(out)) return COMFY_MOE_EINVAL;
  if (!modulation_ok(shift, mod_batch_stride) || !modulation_ok(scale, mod_batch_stride)) return COMFY_MOE_EINVAL;
  if ((dim & 7) != 0 || (dim >> 3) > kLnMaxChunks * 32) return COMFY_MOE_EUNSUPPORTED;
  int blocks = (n_tokens + kLnWarps - 1) / kLnWarps;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const int per_lane = ((dim >> 3) + 31) / 32;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* shp = static_cast<const __nv_bfloat16*>(shift);
  const __nv_bfloat16* scp = static_cast<const __nv_bfloat16*>(scale);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
  if (!gate) {
    launch_ln<0, false>(per_lane, blocks, s, xp, shp, scp, mod_batch_stride, n_tokens, tokens_per_batch, dim, eps, op,
                        LnGateArgs{});
    return check_launch();
  }
  if (!gate->w_gate || !aligned16(gate->w_gate) || !gate->topk_idx || !gate->topk_weight || !gate->block_counts)
    return COMFY_MOE_EINVAL;
  if (gate_dtype != COMFY_MOE_BF16 && gate_dtype != COMFY_MOE_FP32) return COMFY_MOE_EUNSUPPORTED;
  const int n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  if (cudaMemsetAsync(gate->block_counts, 0, sizeof(int32_t) * n_blocks * n_experts, s) != cudaSuccess)
    return COMFY_MOE_ECUDA;
  const bool w32 = gate_dtype == COMFY_MOE_FP32;
#define COMFY_LN_GATE(E) \
  do { \
    if (w32) launch_ln<E, true>(per_lane, blocks, s, xp, shp, scp, mod_batch_stride, n_tokens, tokens_per_batch, dim, \
                                eps, op, *gate); \
    else launch_ln<E, false>(per_lane, blocks, s, xp, shp, scp, mod_batch_stride, n_tokens, tokens_per_batch, dim, \
                             eps, op, *gate); \
  } while (0)
  switch (n_experts) {
    case 2: COMFY_LN_GATE(2); break;
    case 4: COMFY_LN_GATE(4); break;
    case 8: COMFY_LN_GATE(8); break;
    default: return COMFY_MOE_EUNSUPPORTED;
  }
#undef COMFY_LN_GATE
  return check_launch();
}

extern "C" int comfy_moe_ln_modulate(const void* x, const void* shift, const void* scale, int64_t mod_batch_stride,
                                     int n_tokens, int tokens_per_batch, int dim, float eps, void* out, void* stream) {
  return ln_modulate_impl(x, shift, scale, mod_batch_stride, n_tokens, tokens_per_batch, dim, eps, out, nullptr, 0, 0,
                          stream);
}

// LayerNorm + modulation and, on the row just produced, MoEGate.forward (comfy/ldm/hidream/model.py:429-431 followed
// by :263-283): what comfy_moe_ln_modulate and comfy_moe_gate_topk compute, bit for bit, in one pass over the tokens.
extern "C" int comfy_moe_ln_modulate_gate(const void* x, const void* shift, const void* scale, int64_t mod_batch_stride,
                                          int n_tokens, int tokens_per_batch, int dim, float eps, void* out,
                                          const void* w_gate, int w_dtype, int n_experts, int top_k, int32_t* topk_idx,
                                          float* topk_weight, int32_t* block_counts, int32_t* neartie_count,
                                          uint8_t* neartie_flags, float neartie_eps, void* stream) {
  if (top_k != 2) return COMFY_MOE_EUNSUPPORTED;
  const LnGateArgs gate = {w_gate, topk_idx, topk_weight, block_counts, neartie_count, neartie_flags, neartie_eps};
  return ln_modulate_impl(x, shift, scale, mod_batch_stride, n_tokens, tokens_per_batch, dim, eps, out, &gate, w_dtype,
                          n_experts, stream);
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
