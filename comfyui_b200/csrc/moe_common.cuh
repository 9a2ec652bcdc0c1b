// Shared helpers for the HiDream MoE kernels: status codes, bf16 rounding, vector loads.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../../include/comfy_b200_moe.h"

namespace comfy_b200 {

constexpr int kTokensPerBlock = COMFY_MOE_TOKENS_PER_BLOCK;
constexpr int kRowAlign = COMFY_MOE_ROW_ALIGN;
constexpr int kMaxExperts = COMFY_MOE_MAX_EXPERTS;

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? COMFY_MOE_OK : COMFY_MOE_ECUDA;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// fp32 -> bf16 -> fp32: one round-to-nearest-even step, used to reproduce the reference's
// per-operation bf16 roundings inside fused fp32 code.
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint4 ld_nc_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Two floats -> two e4m3 bytes, round-to-nearest-even, saturating at +-448 (the clamp of
// comfy/ops.py:339 followed by the cast of :340).
__device__ __forceinline__ uint16_t f2_to_e4m3x2(float lo, float hi) {
  return static_cast<uint16_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

// The same conversion for a value the reference casts WITHOUT clamping first (comfy/ops.py:342-343, the branch taken
// when the Linear has a scale_input): torch's cast to float8_e4m3fn does not saturate.  Everything that rounds past
// 448, i.e. |v| > 464 (464 itself is the tie that still rounds to 448), and NaN become NaN, byte 0x7f with the sign
// of the input.  `overflow` counts the elements this happened to.
__device__ __forceinline__ uint16_t f2_to_e4m3x2_nosat(float lo, float hi, int& overflow) {
  uint16_t r = f2_to_e4m3x2(lo, hi);
  if (!(fabsf(lo) <= 464.f)) { r = (r & 0xff00u) | 0x7fu | ((__float_as_uint(lo) >> 24) & 0x80u); ++overflow; }
  if (!(fabsf(hi) <= 464.f)) { r = (r & 0x00ffu) | 0x7f00u | ((__float_as_uint(hi) >> 16) & 0x8000u); ++overflow; }
  return r;
}

// Layout of a status block (int32 [COMFY_MOE_STATUS_WORDS]).
constexpr int kStatusWord = 0;          // sticky device status code
constexpr int kStatusNearTies = 1;      // near-tie tokens of the last gate call
constexpr int kStatusE4m3Overflow = 2;  // elements the no-clamp quantiser turned into NaN (accumulates)

}  // namespace comfy_b200
