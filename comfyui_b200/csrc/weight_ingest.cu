// Stochastic rounding of a weight tensor to e4m3 as ComfyUI does it when it bakes a LoRA into scaled fp8 weights
// (comfy/float.py:3-46, reached from scaled_fp8_ops.Linear.set_weight, comfy/ops.py:418-426).  The reference is a chain
// of about fifteen fp16 tensor operations; every one of them rounds its result to fp16, and one of them
// (floor(log2 |x|) on an fp16-rounded logarithm) occasionally picks the exponent one too high just below a power of
// two.  The kernel performs the same steps with the same roundings, element by element, so that fed the same uniform
// random numbers it returns the same bytes.
#include <cuda_fp16.h>

#include "moe_common.cuh"

namespace comfy_b200 {

__device__ __forceinline__ float h16(float v) { return __half2float(__float2half_rn(v)); }   // one fp16 rounding

// x: the value already rounded to fp16 (x.half() of the reference); u: uniform [0, 1) as fp16.  Returns the e4m3 byte.
__device__ __forceinline__ uint8_t stochastic_e4m3(float x, float u) {
  constexpr float kBias = 7.0f, kMant = 8.0f;
  if (isnan(x)) return 0x7f;
  const float sign = x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f);
  const float mag = fabsf(x);
  const float lg = h16(log2f(mag));                                   // log2(0) = -inf, handled by the clamp below
  const float exponent = fminf(fmaxf(h16(floorf(lg) + kBias), 0.f), 15.f);
  const bool normal = exponent != 0.f;
  const float p = ldexpf(1.0f, static_cast<int>(exponent - kBias));   // 2 ** (exponent - bias), exact
  float scaled;
  if (normal) scaled = h16(h16(h16(mag / p) - 1.0f) * kMant);
  else scaled = h16(mag * 512.0f);                                    // mag / 2^(-bias + 1 - mantissa bits)
  scaled = h16(scaled + u);
  const float frac = h16(floorf(scaled) / kMant);
  float val;
  if (normal) val = h16(p * h16(1.0f + frac));
  else val = h16(0.015625f * frac);                                   // 2^(-bias + 1) * frac
  float r = h16(sign * val);
  r = fminf(fmaxf(r, -448.f), 448.f);
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(r, __NV_NOSAT, __NV_E4M3));
}

template <typename T>
__device__ __forceinline__ float to_half_value(T v);
template <>
__device__ __forceinline__ float to_half_value<float>(float v) { return h16(v); }
template <>
__device__ __forceinline__ float to_half_value<__nv_bfloat16>(__nv_bfloat16 v) { return h16(__bfloat162float(v)); }
template <>
__device__ __forceinline__ float to_half_value<__half>(__half v) { return __half2float(v); }

template <typename T>
__global__ void __launch_bounds__(256)
stochastic_round_e4m3_kernel(const T* __restrict__ x, const __half* __restrict__ rand, long long n,
                             uint8_t* __restrict__ out) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride)
    out[i] = stochastic_e4m3(to_half_value<T>(x[i]), __half2float(rand[i]));
}

// ------------------------------------------------------------------------------------------------
// Per-tensor scaled e4m3: s = max|w| / 448, wq = (w / s).to(e4m3), the convention of scaled-fp8 checkpoints that
// scaled_fp8_ops.Linear consumes (comfy/ops.py:379-410: weight e4m3, scale_weight fp32 scalar).  Two passes over the
// tensor: the maximum (order-independent, so reproducible), then the division in fp32 and the round-to-nearest-even
// cast; byte-identical to the three torch operations.
// ------------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

// amax_bits: the running maximum of |w| as the bit pattern of a non-negative float (integer order = float order);
// a NaN anywhere makes the result NaN, as torch's max does (its pattern is above +inf's, so it wins the integer max).
template <typename T>
__global__ void __launch_bounds__(256)
absmax_kernel(const T* __restrict__ w, long long n, unsigned int* __restrict__ amax_bits) {
  unsigned int m = 0;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride) {
    const unsigned int b = __float_as_uint(to_f32<T>(w[i])) & 0x7fffffffu;
    m = b > m ? b : m;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const unsigned int o = __shfl_xor_sync(0xffffffffu, m, off);
    m = o > m ? o : m;
  }
  if ((threadIdx.x & 31) == 0 && m) atomicMax(amax_bits, m);
}

template <typename T>
__global__ void __launch_bounds__(256)
scaled_e4m3_kernel(const T* __restrict__ w, long long n, const unsigned int* __restrict__ amax_bits,
                   uint8_t* __restrict__ out) {
  const float s = __fdiv_rn(__uint_as_float(*amax_bits), 448.0f);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride) {
    // |w / s| <= 448 up to one rounding of the division, far from 464 where the cast would leave the format's range
    out[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(__fdiv_rn(to_f32<T>(w[i]), s), __NV_SATFINITE, __NV_E4M3));
  }
}

// The word that held the maximum between the passes becomes the scale, once every block of the cast has read it
// (stream order).
__global__ void amax_to_scale_kernel(float* __restrict__ scale) { *scale = __fdiv_rn(*scale, 448.0f); }

}  // namespace comfy_b200

using namespace comfy_b200;

extern "C" int comfy_moe_quantize_weight_e4m3(const void* w, int w_dtype, int64_t n_elements, float* scale_out,
                                              void* out, void* stream) {
  if (n_elements < 0) return COMFY_MOE_EINVAL;
  if (!scale_out) return COMFY_MOE_EINVAL;
  if (n_elements > 0 && (!w || !out)) return COMFY_MOE_EINVAL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // scale_out doubles as the accumulator of the maximum (the bit pattern of a non-negative float) between the passes
  unsigned int* amax = reinterpret_cast<unsigned int*>(scale_out);
  if (cudaMemsetAsync(amax, 0, sizeof(unsigned int), s) != cudaSuccess) return COMFY_MOE_ECUDA;
  long long blocks = (n_elements + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  const int g = static_cast<int>(blocks);
  uint8_t* o = static_cast<uint8_t*>(out);
#define COMFY_Q(T) \
  do { \
    absmax_kernel<T><<<g, 256, 0, s>>>(static_cast<const T*>(w), n_elements, amax); \
    scaled_e4m3_kernel<T><<<g, 256, 0, s>>>(static_cast<const T*>(w), n_elements, amax, o); \
  } while (0)
  if (w_dtype == COMFY_MOE_FP32) COMFY_Q(float);
  else if (w_dtype == COMFY_MOE_BF16) COMFY_Q(__nv_bfloat16);
  else if (w_dtype == COMFY_MOE_FP16) COMFY_Q(__half);
  else return COMFY_MOE_EUNSUPPORTED;
#undef COMFY_Q
  amax_to_scale_kernel<<<1, 1, 0, s>>>(scale_out);
  return check_launch();
}

extern "C" int comfy_moe_stochastic_round_e4m3(const void* x, int x_dtype, const void* rand_fp16, int64_t n_elements,
                                           void* out, void* stream) {
  if (n_elements < 0) return COMFY_MOE_EINVAL;
  if (n_elements == 0) return COMFY_MOE_OK;
  if (!x || !rand_fp16 || !out) return COMFY_MOE_EINVAL;
  long long blocks = (n_elements + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __half* r = static_cast<const __half*>(rand_fp16);
  uint8_t* o = static_cast<uint8_t*>(out);
  const int g = static_cast<int>(blocks);
  if (x_dtype == COMFY_MOE_FP32)
    stochastic_round_e4m3_kernel<float><<<g, 256, 0, s>>>(static_cast<const float*>(x), r, n_elements, o);
  else if (x_dtype == COMFY_MOE_BF16)
    stochastic_round_e4m3_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), r, n_elements, o);
  else if (x_dtype == COMFY_MOE_FP16)
    stochastic_round_e4m3_kernel<__half><<<g, 256, 0, s>>>(static_cast<const __half*>(x), r, n_elements, o);
  else
    return COMFY_MOE_EUNSUPPORTED;
  return check_launch();
}
