// Routing kernels of the HiDream MoE feed-forward: fused gate (logits, softmax, top-2),
// routing plan (per-expert scan) and the row permutation.  All three are HBM-bound; they
// replace comfy/ldm/hidream/model.py:263-283 (MoEGate.forward) and :330-339 (argsort,
// bincount, cumsum on the host, row gathers) without any host synchronisation.
#include "moe_common.cuh"

namespace comfy_b200 {

constexpr int kGateThreads = 256;
constexpr int kGateWarps = kGateThreads / 32;
constexpr int kTokensPerWarp = kTokensPerBlock / kGateWarps;  // 4
static_assert(kTokensPerWarp * kGateWarps == kTokensPerBlock, "block must split evenly over warps");
static_assert(kTokensPerWarp % 2 == 0, "the gate handles tokens in pairs");

// ------------------------------------------------------------------------------------------------
// Gate.  One warp computes two tokens at a time: each lane owns 16-byte chunks (8 bf16) of the row,
// the gate weight sits in shared memory as fp32, logits are reduced with shuffles, softmax and
// top-2 are done redundantly in every lane, lane 0 writes.
// ------------------------------------------------------------------------------------------------
template <int E>
__global__ void __launch_bounds__(kGateThreads)
gate_topk_kernel(const __nv_bfloat16* __restrict__ x, const void* __restrict__ w_gate, int w_dtype, int n_tokens,
                 int dim, int32_t* __restrict__ topk_idx, float* __restrict__ topk_weight,
                 int32_t* __restrict__ block_counts, int32_t* __restrict__ neartie_count,
                 uint8_t* __restrict__ neartie_flags, float neartie_eps) {
  extern __shared__ __align__(16) float w_s[];  // [E][dim]
  __shared__ int hist[E];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;

  if (tid < E) hist[tid] = 0;
  if (w_dtype == COMFY_MOE_FP32) {
    const float* w = static_cast<const float*>(w_gate);
    for (int i = tid; i < E * dim; i += kGateThreads) w_s[i] = w[i];
  } else {
    const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(w_gate);
    for (int i = tid; i < E * dim; i += kGateThreads) w_s[i] = __bfloat162float(w[i]);
  }
  __syncthreads();

  const int chunks = dim >> 3;  // 16-byte chunks per row
  const int block_tok0 = blockIdx.x * kTokensPerBlock;

  for (int pair = 0; pair < kTokensPerWarp / 2; ++pair) {
    const int t0 = block_tok0 + warp * kTokensPerWarp + pair * 2;
    const int t1 = t0 + 1;
    if (t0 >= n_tokens) break;
    const bool has1 = t1 < n_tokens;
    const uint4* r0 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t0) * dim);
    const uint4* r1 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(has1 ? t1 : t0) * dim);

    float acc0[E], acc1[E];
#pragma unroll
    for (int e = 0; e < E; ++e) { acc0[e] = 0.f; acc1[e] = 0.f; }

    constexpr int kBatch = 5;  // chunks per lane in flight per token
    for (int c0 = lane; c0 < chunks; c0 += 32 * kBatch) {
      uint4 v0[kBatch], v1[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int c = c0 + 32 * j;
        if (c < chunks) {
          v0[j] = ld_nc_u4(r0 + c);
          v1[j] = ld_nc_u4(r1 + c);
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int c = c0 + 32 * j;
        if (c < chunks) {
          float f0[8], f1[8];
          unpack_bf16x8(v0[j], f0);
          unpack_bf16x8(v1[j], f1);
#pragma unroll
          for (int e = 0; e < E; ++e) {
            const float4 wa = *reinterpret_cast<const float4*>(w_s + e * dim + c * 8);
            const float4 wb = *reinterpret_cast<const float4*>(w_s + e * dim + c * 8 + 4);
            const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              acc0[e] = fmaf(f0[i], wv[i], acc0[e]);
              acc1[e] = fmaf(f1[i], wv[i], acc1[e]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        acc0[e] += __shfl_xor_sync(0xffffffffu, acc0[e], off);
        acc1[e] += __shfl_xor_sync(0xffffffffu, acc1[e], off);
      }
    }

#pragma unroll
    for (int which = 0; which < 2; ++which) {
      if (which == 1 && !has1) break;
      const int t = which == 0 ? t0 : t1;
      float s[E];
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        s[e] = which == 0 ? acc0[e] : acc1[e];
        mx = fmaxf(mx, s[e]);
      }
      float sum = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        s[e] = expf(s[e] - mx);
        sum += s[e];
      }
#pragma unroll
      for (int e = 0; e < E; ++e) s[e] = s[e] / sum;

      // top-2, strict '>' keeps the lowest index on exact ties
      int i0 = 0;
#pragma unroll
      for (int e = 1; e < E; ++e) if (s[e] > s[i0]) i0 = e;
      int i1 = (i0 == 0) ? 1 : 0;
#pragma unroll
      for (int e = 0; e < E; ++e) if (e != i0 && e != i1 && s[e] > s[i1]) i1 = e;
      float third = -1.f;
#pragma unroll
      for (int e = 0; e < E; ++e) if (e != i0 && e != i1) third = fmaxf(third, s[e]);

      if (lane == 0) {
        topk_idx[2 * t] = i0;
        topk_idx[2 * t + 1] = i1;
        topk_weight[2 * t] = s[i0];
        topk_weight[2 * t + 1] = s[i1];
        atomicAdd(&hist[i0], 1);
        atomicAdd(&hist[i1], 1);
        const bool tie = (E > 2) && (s[i1] - third < neartie_eps);
        if (neartie_flags) neartie_flags[t] = tie ? 1 : 0;
        if (tie && neartie_count) atomicAdd(neartie_count, 1);
      }
    }
  }
  __syncthreads();
  if (tid < E) block_counts[blockIdx.x * E + tid] = hist[tid];
}

// ------------------------------------------------------------------------------------------------
// Per-block expert counts for routing that did not come from the gate kernel (moe_infer is public
// and takes the indices as an argument).  Out-of-range expert ids are counted nowhere.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kTokensPerBlock * 2)
route_count_kernel(const int32_t* __restrict__ topk_idx, int n_tokens, int n_experts,
                   int32_t* __restrict__ block_counts) {
  __shared__ int hist[kMaxExperts];
  const int tid = threadIdx.x;
  if (tid < kMaxExperts) hist[tid] = 0;
  __syncthreads();
  const int slot = blockIdx.x * kTokensPerBlock * 2 + tid;
  const int e = slot < n_tokens * 2 ? topk_idx[slot] : -1;
  for (int k = 0; k < n_experts; ++k) {
    const unsigned m = __ballot_sync(0xffffffffu, e == k);
    if ((tid & 31) == 0 && m) atomicAdd(&hist[k], __popc(m));
  }
  __syncthreads();
  if (tid < n_experts) block_counts[blockIdx.x * n_experts + tid] = hist[tid];
}

// ------------------------------------------------------------------------------------------------
// Routing plan: one thread block scans the per-block counts of every expert.
// ------------------------------------------------------------------------------------------------
constexpr int kPlanThreads = 1024;

__global__ void __launch_bounds__(kPlanThreads)
route_plan_kernel(const int32_t* __restrict__ block_counts, int n_blocks, int n_experts,
                  int32_t* __restrict__ block_offsets, int32_t* __restrict__ expert_counts,
                  int32_t* __restrict__ expert_offsets) {
  __shared__ int warp_sums[kPlanThreads / 32];
  __shared__ int carry;
  __shared__ int totals[kMaxExperts];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int e = 0; e < n_experts; ++e) {
    if (tid == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < n_blocks; base += kPlanThreads) {
      const int b = base + tid;
      const int v = b < n_blocks ? block_counts[b * n_experts + e] : 0;
      int incl = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
      }
      if (lane == 31) warp_sums[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        int ws = warp_sums[lane];
        int wi = ws;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int n = __shfl_up_sync(0xffffffffu, wi, off);
          if (lane >= off) wi += n;
        }
        warp_sums[lane] = wi - ws;  // exclusive prefix of the warp totals
      }
      __syncthreads();
      const int excl = carry + warp_sums[warp] + incl - v;
      if (b < n_blocks) block_offsets[b * n_experts + e] = excl;
      __syncthreads();
      if (tid == kPlanThreads - 1) carry = excl + v;
      __syncthreads();
    }
    if (tid == 0) totals[e] = carry;
    __syncthreads();
  }
  if (tid == 0) {
    int row = 0;
    for (int e = 0; e < n_experts; ++e) {
      expert_counts[e] = totals[e];
      expert_offsets[e] = row;
      row += (totals[e] + kRowAlign - 1) / kRowAlign * kRowAlign;
    }
    expert_offsets[n_experts] = row;
  }
}

// ------------------------------------------------------------------------------------------------
// Permutation.  Block b owns the same tokens as gate block b.  Slots (token, k) are ranked inside
// the block with warp ballots, which gives a stable, atomic-free placement; then every warp copies
// its tokens' rows to both destinations with 16-byte accesses.
// ------------------------------------------------------------------------------------------------
template <bool kFp8>
__global__ void __launch_bounds__(kGateThreads)
permute_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ topk_idx,
               const int32_t* __restrict__ block_offsets, const int32_t* __restrict__ expert_offsets,
               int n_tokens, int dim, int n_experts, const float* __restrict__ act_scale,
               void* __restrict__ x_perm, void* __restrict__ x_q, const float* __restrict__ x_q_scale,
               int32_t* __restrict__ row_map) {
  constexpr int kSlots = kTokensPerBlock * 2;  // 64
  __shared__ int dest_s[kSlots];
  __shared__ int warp_cnt[kSlots / 32][kMaxExperts];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int block_tok0 = blockIdx.x * kTokensPerBlock;

  int my_e = -1, my_rank = 0;
  if (tid < kSlots) {
    const int slot = block_tok0 * 2 + tid;
    if (slot < n_tokens * 2) my_e = topk_idx[slot];
    if (my_e >= n_experts) my_e = -1;   // an id outside the layer routes nowhere
    for (int e = 0; e < n_experts; ++e) {
      const unsigned m = __ballot_sync(0xffffffffu, my_e == e);
      if (my_e == e) my_rank = __popc(m & ((1u << lane) - 1u));
      if (lane == 0) warp_cnt[warp][e] = __popc(m);
    }
  }
  __syncthreads();
  if (tid < kSlots) {
    int d = -1;
    if (my_e >= 0) {
      int before = my_rank;
      for (int w = 0; w < warp; ++w) before += warp_cnt[w][my_e];
      d = expert_offsets[my_e] + block_offsets[blockIdx.x * n_experts + my_e] + before;
    }
    if (block_tok0 * 2 + tid < n_tokens * 2) row_map[block_tok0 * 2 + tid] = d;
    dest_s[tid] = d;
  }
  __syncthreads();

  float inv_p = 1.f, inv_q = 1.f;
  bool scaled_p = false, scaled_q = false;
  if constexpr (kFp8) {
    if (act_scale) { inv_p = round_bf16(1.0f / __ldg(act_scale)); scaled_p = true; }
    if (x_q_scale) { inv_q = round_bf16(1.0f / __ldg(x_q_scale)); scaled_q = true; }
  }

  for (int i = 0; i < kTokensPerWarp; ++i) {
    const int lt = warp * kTokensPerWarp + i;
    const int t = block_tok0 + lt;
    if (t >= n_tokens) break;
    const int d0 = dest_s[2 * lt], d1 = dest_s[2 * lt + 1];
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * dim);
    if constexpr (!kFp8) {
      uint4* o0 = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(x_perm) + static_cast<size_t>(d0) * dim);
      uint4* o1 = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(x_perm) + static_cast<size_t>(d1) * dim);
      const int chunks = dim >> 3;
      constexpr int kBatch = 5;
      for (int c0 = lane; c0 < chunks; c0 += 32 * kBatch) {
        uint4 v[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j)
          if (c0 + 32 * j < chunks) v[j] = ld_nc_u4(src + c0 + 32 * j);
#pragma unroll
        for (int j = 0; j < kBatch; ++j)
          if (c0 + 32 * j < chunks) {
            if (d0 >= 0) o0[c0 + 32 * j] = v[j];
            if (d1 >= 0) o1[c0 + 32 * j] = v[j];
          }
      }
    } else {
      // 16 bf16 (two 16-byte loads) -> 16 e4m3 bytes (one 16-byte store)
      uint8_t* p0 = static_cast<uint8_t*>(x_perm) + static_cast<size_t>(d0) * dim;
      uint8_t* p1 = static_cast<uint8_t*>(x_perm) + static_cast<size_t>(d1) * dim;
      uint8_t* q = x_q ? static_cast<uint8_t*>(x_q) + static_cast<size_t>(t) * dim : nullptr;
      const int chunks = dim >> 4;
      for (int c = lane; c < chunks; c += 32) {
        const uint4 a = ld_nc_u4(src + 2 * c), b = ld_nc_u4(src + 2 * c + 1);
        float f[16];
        {
          float fa[8], fb[8];
          unpack_bf16x8(a, fa);
          unpack_bf16x8(b, fb);
#pragma unroll
          for (int k = 0; k < 8; ++k) { f[k] = fa[k]; f[8 + k] = fb[k]; }
        }
        uint32_t wp[4], wq[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float g[4];
#pragma unroll
          for (int m = 0; m < 4; ++m) g[m] = scaled_p ? round_bf16(f[4 * k + m] * inv_p) : f[4 * k + m];
          wp[k] = static_cast<uint32_t>(f2_to_e4m3x2(g[0], g[1])) |
                  (static_cast<uint32_t>(f2_to_e4m3x2(g[2], g[3])) << 16);
          if (scaled_q == scaled_p && inv_q == inv_p) {
            wq[k] = wp[k];
          } else {
#pragma unroll
            for (int m = 0; m < 4; ++m) g[m] = scaled_q ? round_bf16(f[4 * k + m] * inv_q) : f[4 * k + m];
            wq[k] = static_cast<uint32_t>(f2_to_e4m3x2(g[0], g[1])) |
                    (static_cast<uint32_t>(f2_to_e4m3x2(g[2], g[3])) << 16);
          }
        }
        const uint4 vp = make_uint4(wp[0], wp[1], wp[2], wp[3]);
        if (d0 >= 0) reinterpret_cast<uint4*>(p0)[c] = vp;
        if (d1 >= 0) reinterpret_cast<uint4*>(p1)[c] = vp;
        if (q) reinterpret_cast<uint4*>(q)[c] = make_uint4(wq[0], wq[1], wq[2], wq[3]);
      }
    }
  }
}

}  // namespace comfy_b200

using namespace comfy_b200;

extern "C" int comfy_moe_plan_sizes(int n_tokens, int n_experts, int top_k, int64_t* rows_cap, int* n_blocks) {
  if (n_tokens < 0 || n_experts < 1 || n_experts > kMaxExperts || top_k != 2) return COMFY_MOE_EINVAL;
  if (rows_cap) *rows_cap = static_cast<int64_t>(top_k) * n_tokens + static_cast<int64_t>(n_experts) * kRowAlign;
  if (n_blocks) *n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  return COMFY_MOE_OK;
}

template <int E>
static int launch_gate(const void* x, const void* w_gate, int w_dtype, int n_tokens, int dim, int32_t* topk_idx,
                       float* topk_weight, int32_t* block_counts, int32_t* neartie_count, uint8_t* neartie_flags,
                       float neartie_eps, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(E) * dim * sizeof(float);
  if (smem > 200 * 1024) return COMFY_MOE_EUNSUPPORTED;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(gate_topk_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return COMFY_MOE_ECUDA;
  }
  const int n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  gate_topk_kernel<E><<<n_blocks, kGateThreads, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(x), w_gate, w_dtype, n_tokens, dim, topk_idx, topk_weight, block_counts,
      neartie_count, neartie_flags, neartie_eps);
  return check_launch();
}

extern "C" int comfy_moe_gate_topk(const void* x, const void* w_gate, int w_dtype, int n_tokens, int dim,
                                   int n_experts, int top_k, int32_t* topk_idx, float* topk_weight,
                                   int32_t* block_counts, int32_t* neartie_count, uint8_t* neartie_flags,
                                   float neartie_eps, void* stream) {
  if (n_tokens < 0 || dim <= 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!x || !w_gate || !topk_idx || !topk_weight || !block_counts) return COMFY_MOE_EINVAL;
  if (!aligned16(x) || !aligned16(w_gate)) return COMFY_MOE_EINVAL;
  if (top_k != 2 || (dim & 7) != 0) return COMFY_MOE_EUNSUPPORTED;
  if (w_dtype != COMFY_MOE_BF16 && w_dtype != COMFY_MOE_FP32) return COMFY_MOE_EUNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (n_experts) {
    case 2: return launch_gate<2>(x, w_gate, w_dtype, n_tokens, dim, topk_idx, topk_weight, block_counts, neartie_count, neartie_flags, neartie_eps, s);
    case 4: return launch_gate<4>(x, w_gate, w_dtype, n_tokens, dim, topk_idx, topk_weight, block_counts, neartie_count, neartie_flags, neartie_eps, s);
    case 8: return launch_gate<8>(x, w_gate, w_dtype, n_tokens, dim, topk_idx, topk_weight, block_counts, neartie_count, neartie_flags, neartie_eps, s);
    default: return COMFY_MOE_EUNSUPPORTED;
  }
}

extern "C" int comfy_moe_route_count(const int32_t* topk_idx, int n_tokens, int n_experts, int32_t* block_counts,
                                     void* stream) {
  if (n_tokens < 0 || n_experts < 1 || n_experts > kMaxExperts) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!topk_idx || !block_counts) return COMFY_MOE_EINVAL;
  const int n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  route_count_kernel<<<n_blocks, kTokensPerBlock * 2, 0, static_cast<cudaStream_t>(stream)>>>(
      topk_idx, n_tokens, n_experts, block_counts);
  return check_launch();
}

extern "C" int comfy_moe_route_plan(const int32_t* block_counts, int n_tokens, int n_experts,
                                    int32_t* block_offsets, int32_t* expert_counts, int32_t* expert_offsets,
                                    void* stream) {
  if (n_tokens < 0 || n_experts < 1 || n_experts > kMaxExperts) return COMFY_MOE_EINVAL;
  if (!expert_counts || !expert_offsets) return COMFY_MOE_EINVAL;
  const int n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  if (n_blocks > 0 && (!block_counts || !block_offsets)) return COMFY_MOE_EINVAL;
  route_plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      block_counts, n_blocks, n_experts, block_offsets, expert_counts, expert_offsets);
  return check_launch();
}

extern "C" int comfy_moe_permute(const void* x, const int32_t* topk_idx, const int32_t* block_offsets,
                                 const int32_t* expert_offsets, int n_tokens, int dim, int n_experts,
                                 int act_dtype, const float* act_scale, void* x_perm, void* x_q,
                                 const float* x_q_scale, int32_t* row_map, void* stream) {
  if (n_tokens < 0 || dim <= 0 || n_experts < 1 || n_experts > kMaxExperts) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!x || !topk_idx || !block_offsets || !expert_offsets || !x_perm || !row_map) return COMFY_MOE_EINVAL;
  if (!aligned16(x) || !aligned16(x_perm) || (x_q && !aligned16(x_q))) return COMFY_MOE_EINVAL;
  const int n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (act_dtype == COMFY_MOE_BF16) {
    if ((dim & 7) != 0) return COMFY_MOE_EUNSUPPORTED;
    permute_kernel<false><<<n_blocks, kGateThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), topk_idx,
                                                            block_offsets, expert_offsets, n_tokens, dim, n_experts,
                                                            nullptr, x_perm, nullptr, nullptr, row_map);
  } else if (act_dtype == COMFY_MOE_FP8_E4M3) {
    if ((dim & 15) != 0) return COMFY_MOE_EUNSUPPORTED;
    permute_kernel<true><<<n_blocks, kGateThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), topk_idx,
                                                           block_offsets, expert_offsets, n_tokens, dim, n_experts,
                                                           act_scale, x_perm, x_q, x_q_scale, row_map);
  } else {
    return COMFY_MOE_EUNSUPPORTED;
  }
  return check_launch();
}
