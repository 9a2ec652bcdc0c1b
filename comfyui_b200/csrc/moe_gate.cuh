// The part of MoEGate.forward (comfy/ldm/hidream/model.py:270-283) that follows the logits: softmax over the experts,
// top-2 without renormalisation, and the near-tie test.  Shared by the stand-alone gate kernel and by the LayerNorm +
// modulation kernel that computes the gate on the row it has just produced, so that both yield the same bits.
#pragma once
#include "moe_common.cuh"

namespace comfy_b200 {

// logits[E] (fp32, already reduced over the row) -> indices of the two largest scores (largest first, lowest index on
// exact ties), their softmax scores, and whether 2nd and 3rd place are closer than neartie_eps.
template <int E>
__device__ __forceinline__ void gate_select(const float (&logits)[E], float neartie_eps, int& i0, int& i1, float& w0,
                                            float& w1, bool& tie) {
  float sc[E];
  float mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < E; ++e) { sc[e] = logits[e]; mx = fmaxf(mx, sc[e]); }
  float sum = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) { sc[e] = expf(sc[e] - mx); sum += sc[e]; }
#pragma unroll
  for (int e = 0; e < E; ++e) sc[e] = sc[e] / sum;
  i0 = 0;                                            // strict '>' keeps the lowest index on exact ties
#pragma unroll
  for (int e = 1; e < E; ++e) if (sc[e] > sc[i0]) i0 = e;
  i1 = (i0 == 0) ? 1 : 0;
#pragma unroll
  for (int e = 0; e < E; ++e) if (e != i0 && e != i1 && sc[e] > sc[i1]) i1 = e;
  float third = -1.f;
#pragma unroll
  for (int e = 0; e < E; ++e) if (e != i0 && e != i1) third = fmaxf(third, sc[e]);
  w0 = sc[i0];
  w1 = sc[i1];
  tie = (E > 2) && (sc[i1] - third < neartie_eps);
}

// One 16-byte chunk (8 bf16 activations, already unpacked) against the same chunk of every expert's gate row:
// acc[e] += sum_k f[k] * w[e][k], k ascending.  `w_rows` points at the gate weight as stored (bf16 or fp32, kW32),
// `row_vecs` is the number of 16-byte vectors per weight row and c the chunk index.
template <int E, bool kW32>
__device__ __forceinline__ void gate_accumulate(const uint4* __restrict__ w_rows, int row_vecs, int c,
                                                const float (&f)[8], float (&acc)[E]) {
#pragma unroll
  for (int e = 0; e < E; ++e) {
    float wv[8];
    if constexpr (kW32) {
      const float4 a = reinterpret_cast<const float4*>(w_rows)[e * row_vecs + 2 * c];
      const float4 b = reinterpret_cast<const float4*>(w_rows)[e * row_vecs + 2 * c + 1];
      wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
    } else {
      unpack_bf16x8(w_rows[e * row_vecs + c], wv);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[e] = fmaf(f[k], wv[k], acc[e]);
  }
}

}  // namespace comfy_b200
