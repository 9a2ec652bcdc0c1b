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

}  // namespace comfy_b200

using namespace comfy_b200;

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
