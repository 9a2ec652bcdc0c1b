// Routing kernels of the HiDream MoE feed-forward: fused gate (logits, softmax, top-2),
// routing plan (per-expert scan) and the row permutation.  All three are HBM-bound; they
// replace comfy/ldm/hidream/model.py:263-283 (MoEGate.forward) and :330-339 (argsort,
// bincount, cumsum on the host, row gathers) without any host synchronisation.
//
// A block owns kTokensPerBlock consecutive tokens in both the gate and the permutation; every access is a
// 16-byte chunk per lane, 512 contiguous bytes per warp, with several rows in flight per thread.
#include "moe_common.cuh"
#include "moe_gate.cuh"

namespace comfy_b200 {

constexpr int kMaxRowThreads = 512;    // dim / 8 threads per block: dim <= 4096

__host__ __device__ constexpr int round_up32(int v) { return (v + 31) & ~31; }

// ------------------------------------------------------------------------------------------------
// Gate.  The kernel is bound by instruction issue, not by HBM: 4 dot products of 2560 per token are 10 240 fp32 FMAs,
// and unpacking bf16 weights for them costs as much again, while the token itself is only 5 KB.  So the weight is
// converted to fp32 ONCE per block into shared memory (laid out so that a warp's 16-byte reads are conflict-free), and a
// warp takes FOUR tokens at a time: every weight value read from shared memory feeds four FMAs.  Lane l owns the
// 16-byte chunks l, l + 32, ... of each of its rows, three chunk steps (12 loads per lane) in flight ahead of the
// arithmetic.  Per token the order of operations is the one gate_accumulate uses (chunks ascending, elements
// ascending, then a butterfly reduction), so the logits equal those of the fused LayerNorm + gate kernel bit for bit.
// A block of 8 warps owns the 32 consecutive tokens of one counting block, keeps their expert histogram in shared
// memory and writes it out: no atomics on global memory, nothing to zero beforehand.
// ------------------------------------------------------------------------------------------------
constexpr int kGateWarps = 8;
constexpr int kGateTokensPerWarp = kTokensPerBlock / kGateWarps;   // 4
constexpr int kGateDepth = 3;                                       // chunk steps in flight

// float4 index of half h (elements 4h .. 4h + 3) of chunk c of expert e's row in the shared-memory copy
__device__ __forceinline__ int gate_w_slot(int e, int c, int h, int chunks_pad) {
  return (e * chunks_pad + (c & ~31)) * 2 + h * 32 + (c & 31);
}

template <int E, bool kW32, int kChunksPerLane>
__global__ void __launch_bounds__(kGateWarps * 32, E > 4 ? 1 : 2)
gate_topk_kernel(const __nv_bfloat16* __restrict__ x, const void* __restrict__ w_gate, int n_tokens, int dim,
                 int32_t* __restrict__ topk_idx, float* __restrict__ topk_weight, int32_t* __restrict__ block_counts,
                 int32_t* __restrict__ neartie_count, uint8_t* __restrict__ neartie_flags, float neartie_eps) {
  extern __shared__ float4 w_s[];                      // E x chunks_pad x 2 float4
  __shared__ int hist[E];
  constexpr int T = kGateTokensPerWarp;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunks = dim >> 3;
  const int chunks_pad = round_up32(chunks);
  if constexpr (kW32) {
    const float4* src = static_cast<const float4*>(w_gate);
    for (int q = tid; q < E * chunks * 2; q += kGateWarps * 32) {
      const int e = q / (chunks * 2), r = q - e * chunks * 2;
      w_s[gate_w_slot(e, r >> 1, r & 1, chunks_pad)] = src[q];
    }
  } else {
    const uint4* src = static_cast<const uint4*>(w_gate);
    for (int q = tid; q < E * chunks; q += kGateWarps * 32) {
      const int e = q / chunks, c = q - e * chunks;
      float f[8];
      unpack_bf16x8(src[q], f);
      w_s[gate_w_slot(e, c, 0, chunks_pad)] = make_float4(f[0], f[1], f[2], f[3]);
      w_s[gate_w_slot(e, c, 1, chunks_pad)] = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
  const int n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  for (int tb = blockIdx.x; tb < n_blocks; tb += gridDim.x) {
    if (tid < E) hist[tid] = 0;
    __syncthreads();                                   // weights and histogram ready (previous round's counts written)
    const int t0 = tb * kTokensPerBlock + warp * T;
    const uint4* rows[T];
#pragma unroll
    for (int i = 0; i < T; ++i) {
      const int t = t0 + i < n_tokens ? t0 + i : n_tokens - 1;      // rows past the end repeat the last one, unused
      rows[i] = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * dim);
    }
    uint4 v[kGateDepth][T];
#pragma unroll
    for (int j = 0; j < kGateDepth && j < kChunksPerLane; ++j) {
      const int c = lane + 32 * j;
      if (c < chunks) {
#pragma unroll
        for (int i = 0; i < T; ++i) v[j][i] = ld_nc_u4(rows[i] + c);
      }
    }
    float acc[T][E];
#pragma unroll
    for (int i = 0; i < T; ++i) {
#pragma unroll
      for (int e = 0; e < E; ++e) acc[i][e] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < kChunksPerLane; ++j) {
      const int c = lane + 32 * j;
      uint4 cur[T];
#pragma unroll
      for (int i = 0; i < T; ++i) cur[i] = v[j % kGateDepth][i];
      if (j + kGateDepth < kChunksPerLane) {
        const int cn = lane + 32 * (j + kGateDepth);
        if (cn < chunks) {
#pragma unroll
          for (int i = 0; i < T; ++i) v[j % kGateDepth][i] = ld_nc_u4(rows[i] + cn);
        }
      }
      if (c < chunks) {
        float f[T][8];
#pragma unroll
        for (int i = 0; i < T; ++i) unpack_bf16x8(cur[i], f[i]);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float4 a = w_s[gate_w_slot(e, c, 0, chunks_pad)];
          const float4 b = w_s[gate_w_slot(e, c, 1, chunks_pad)];
          const float wv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
          for (int i = 0; i < T; ++i) {
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[i][e] = fmaf(f[i][k], wv[k], acc[i][e]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < T; ++i) {
#pragma unroll
      for (int e = 0; e < E; ++e) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[i][e] += __shfl_xor_sync(0xffffffffu, acc[i][e], off);
      }
    }
#pragma unroll
    for (int i = 0; i < T; ++i) {
      const int t = t0 + i;
      if (t < n_tokens) {                              // warp-uniform
        int i0, i1;
        float w0, w1;
        bool tie;
        gate_select<E>(acc[i], neartie_eps, i0, i1, w0, w1, tie);
        if (lane == 0) {
          topk_idx[2 * t] = i0;
          topk_idx[2 * t + 1] = i1;
          topk_weight[2 * t] = w0;
          topk_weight[2 * t + 1] = w1;
          atomicAdd(&hist[i0], 1);
          atomicAdd(&hist[i1], 1);
          if (neartie_flags) neartie_flags[t] = tie ? 1 : 0;
          if (tie && neartie_count) atomicAdd(neartie_count, 1);
        }
      }
    }
    __syncthreads();
    if (tid < E) block_counts[tb * E + tid] = hist[tid];
  }
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
// the block with warp ballots, which gives a stable, atomic-free placement; then thread c copies
// chunk c of every row to both destinations, kTok rows in flight.
// bf16: chunk = 8 elements (16 B in, 16 B out).  fp8: chunk = 16 elements (32 B in, 16 B out).
// ------------------------------------------------------------------------------------------------
// kPlan: the routing plan is folded in.  Instead of reading block_offsets / expert_offsets (written by
// route_plan_kernel) every block sums the per-block counts of the blocks before it and of all blocks itself
// (n_blocks * E integers, a few KB from L2), which saves a launch and a serial single-block scan; block 0 also
// publishes expert_counts / expert_offsets for the grouped GEMM.  Used for up to kFusedPlanMaxBlocks blocks.
constexpr int kFusedPlanMaxBlocks = 2048;

template <bool kFp8, bool kPlan>
__global__ void __launch_bounds__(kMaxRowThreads)
permute_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ topk_idx,
               const int32_t* __restrict__ block_offsets, const int32_t* __restrict__ expert_offsets,
               int n_tokens, int dim, int n_experts, const float* __restrict__ act_scale,
               void* __restrict__ x_perm, void* __restrict__ x_q, const float* __restrict__ x_q_scale,
               int32_t* __restrict__ row_map, const int32_t* __restrict__ block_counts, int n_blocks,
               int32_t* __restrict__ expert_counts_out, int32_t* __restrict__ expert_offsets_out,
               int32_t* __restrict__ overflow_count) {
  constexpr int kSlots = kTokensPerBlock * 2;  // 64
  constexpr int kTok = 8;
  __shared__ int dest_s[kSlots];
  __shared__ int warp_cnt[kSlots / 32][kMaxExperts];
  __shared__ int s_before[kMaxExperts];      // rows of expert e that belong to earlier blocks
  __shared__ int s_start[kMaxExperts];       // first row of expert e in the permuted layout
  __shared__ int s_part[kMaxRowThreads / 32][2 * kMaxExperts];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int block_tok0 = blockIdx.x * kTokensPerBlock;

  if constexpr (kPlan) {
    int acc[2 * kMaxExperts];               // [e] = counts of earlier blocks, [kMaxExperts + e] = counts of all blocks
#pragma unroll
    for (int k = 0; k < 2 * kMaxExperts; ++k) acc[k] = 0;
    for (int b = tid; b < n_blocks; b += blockDim.x) {
#pragma unroll
      for (int e = 0; e < kMaxExperts; ++e) {
        if (e < n_experts) {
          const int c = __ldg(block_counts + b * n_experts + e);
          acc[kMaxExperts + e] += c;
          if (b < static_cast<int>(blockIdx.x)) acc[e] += c;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 2 * kMaxExperts; ++k) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], off);
      if (lane == 0) s_part[warp][k] = acc[k];
    }
    __syncthreads();
    if (tid == 0) {
      const int n_warps = blockDim.x >> 5;
      int row = 0;
      for (int e = 0; e < n_experts; ++e) {
        int before = 0, total = 0;
        for (int w = 0; w < n_warps; ++w) { before += s_part[w][e]; total += s_part[w][kMaxExperts + e]; }
        s_before[e] = before;
        s_start[e] = row;
        if (blockIdx.x == 0) { expert_counts_out[e] = total; expert_offsets_out[e] = row; }
        row += (total + kRowAlign - 1) / kRowAlign * kRowAlign;
      }
      if (blockIdx.x == 0) expert_offsets_out[n_experts] = row;
    }
  } else {
    if (tid < n_experts) {
      s_before[tid] = block_offsets[blockIdx.x * n_experts + tid];
      s_start[tid] = expert_offsets[tid];
    }
  }

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
      d = s_start[my_e] + s_before[my_e] + before;
    }
    if (block_tok0 * 2 + tid < n_tokens * 2) row_map[block_tok0 * 2 + tid] = d;
    dest_s[tid] = d;
  }
  __syncthreads();

  const int chunks = kFp8 ? (dim >> 4) : (dim >> 3);
  if (tid >= chunks) return;

  if constexpr (!kFp8) {
    __nv_bfloat16* xp = static_cast<__nv_bfloat16*>(x_perm);
    for (int base = 0; base < kTokensPerBlock; base += kTok) {
      const int t0 = block_tok0 + base;
      if (t0 >= n_tokens) break;
      uint4 v[kTok];
#pragma unroll
      for (int i = 0; i < kTok; ++i)
        if (t0 + i < n_tokens) v[i] = ld_nc_u4(reinterpret_cast<const uint4*>(x + static_cast<size_t>(t0 + i) * dim) + tid);
#pragma unroll
      for (int i = 0; i < kTok; ++i) {
        if (t0 + i < n_tokens) {
          const int d0 = dest_s[2 * (base + i)], d1 = dest_s[2 * (base + i) + 1];
          if (d0 >= 0) reinterpret_cast<uint4*>(xp + static_cast<size_t>(d0) * dim)[tid] = v[i];
          if (d1 >= 0) reinterpret_cast<uint4*>(xp + static_cast<size_t>(d1) * dim)[tid] = v[i];
        }
      }
    }
  } else {
    float inv_p = 1.f, inv_q = 1.f;
    bool scaled_p = false, scaled_q = false;
    if (act_scale) { inv_p = round_bf16(1.0f / __ldg(act_scale)); scaled_p = true; }
    if (x_q_scale) { inv_q = round_bf16(1.0f / __ldg(x_q_scale)); scaled_q = true; }
    const bool same_q = (scaled_q == scaled_p) && (inv_q == inv_p);
    uint8_t* xp = static_cast<uint8_t*>(x_perm);
    uint8_t* xq = static_cast<uint8_t*>(x_q);
    int ovf = 0;                 // elements the reference's unclamped cast turns into NaN (scaled variants only)
    constexpr int kTok8 = 4;
    for (int base = 0; base < kTokensPerBlock; base += kTok8) {
      const int t0 = block_tok0 + base;
      if (t0 >= n_tokens) break;
      uint4 va[kTok8], vb[kTok8];
#pragma unroll
      for (int i = 0; i < kTok8; ++i)
        if (t0 + i < n_tokens) {
          const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t0 + i) * dim) + 2 * tid;
          va[i] = ld_nc_u4(src);
          vb[i] = ld_nc_u4(src + 1);
        }
#pragma unroll
      for (int i = 0; i < kTok8; ++i) {
        if (t0 + i >= n_tokens) continue;
        float f[16];
        {
          float fa[8], fb[8];
          unpack_bf16x8(va[i], fa);
          unpack_bf16x8(vb[i], fb);
#pragma unroll
          for (int k = 0; k < 8; ++k) { f[k] = fa[k]; f[8 + k] = fb[k]; }
        }
        uint32_t wp[4], wq[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float g[4];
#pragma unroll
          for (int m = 0; m < 4; ++m) g[m] = scaled_p ? round_bf16(f[4 * k + m] * inv_p) : f[4 * k + m];
          wp[k] = scaled_p ? (static_cast<uint32_t>(f2_to_e4m3x2_nosat(g[0], g[1], ovf)) |
                              (static_cast<uint32_t>(f2_to_e4m3x2_nosat(g[2], g[3], ovf)) << 16))
                           : (static_cast<uint32_t>(f2_to_e4m3x2(g[0], g[1])) |
                              (static_cast<uint32_t>(f2_to_e4m3x2(g[2], g[3])) << 16));
          if (same_q) {
            wq[k] = wp[k];
          } else {
            int ovf_q = 0;       // the shared expert's copy: counted only when no routed copy is made of the same value
#pragma unroll
            for (int m = 0; m < 4; ++m) g[m] = scaled_q ? round_bf16(f[4 * k + m] * inv_q) : f[4 * k + m];
            wq[k] = scaled_q ? (static_cast<uint32_t>(f2_to_e4m3x2_nosat(g[0], g[1], ovf_q)) |
                                (static_cast<uint32_t>(f2_to_e4m3x2_nosat(g[2], g[3], ovf_q)) << 16))
                             : (static_cast<uint32_t>(f2_to_e4m3x2(g[0], g[1])) |
                                (static_cast<uint32_t>(f2_to_e4m3x2(g[2], g[3])) << 16));
            if (xq) ovf += ovf_q;
          }
        }
        const uint4 vp = make_uint4(wp[0], wp[1], wp[2], wp[3]);
        const int d0 = dest_s[2 * (base + i)], d1 = dest_s[2 * (base + i) + 1];
        if (d0 >= 0) reinterpret_cast<uint4*>(xp + static_cast<size_t>(d0) * dim)[tid] = vp;
        if (d1 >= 0) reinterpret_cast<uint4*>(xp + static_cast<size_t>(d1) * dim)[tid] = vp;
        if (xq) reinterpret_cast<uint4*>(xq + static_cast<size_t>(t0 + i) * dim)[tid] = make_uint4(wq[0], wq[1], wq[2], wq[3]);
      }
    }
    if (ovf && overflow_count) atomicAdd(overflow_count, ovf);
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

static int row_threads(int dim) {
  const int t = round_up32(dim >> 3);
  return t < 64 ? 64 : t;     // the permutation ranks 64 slots with the first two warps
}

template <int E, bool kW32, int K>
static int launch_gate_as(const __nv_bfloat16* x, const void* w_gate, int n_tokens, int dim, int32_t* topk_idx,
                          float* topk_weight, int32_t* block_counts, int32_t* neartie_count, uint8_t* neartie_flags,
                          float neartie_eps, cudaStream_t stream) {
  const int n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  const int grid = n_blocks < 148 * 2 ? n_blocks : 148 * 2;          // two blocks per SM, each converts the weight once
  const size_t smem = static_cast<size_t>(E) * round_up32(dim >> 3) * 2 * sizeof(float4);
  auto kernel = gate_topk_kernel<E, kW32, K>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return COMFY_MOE_ECUDA;
  kernel<<<grid, kGateWarps * 32, smem, stream>>>(x, w_gate, n_tokens, dim, topk_idx, topk_weight, block_counts,
                                                  neartie_count, neartie_flags, neartie_eps);
  return check_launch();
}

template <int E>
static int launch_gate(const void* x, const void* w_gate, int w_dtype, int n_tokens, int dim, int32_t* topk_idx,
                       float* topk_weight, int32_t* block_counts, int32_t* neartie_count, uint8_t* neartie_flags,
                       float neartie_eps, cudaStream_t stream) {
  const int per_lane = ((dim >> 3) + 31) / 32;     // chunk steps per lane: the smallest instantiation that covers the row
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
#define COMFY_GATE_LAUNCH(W32, K) \
  return launch_gate_as<E, W32, K>(xp, w_gate, n_tokens, dim, topk_idx, topk_weight, block_counts, neartie_count, \
                                   neartie_flags, neartie_eps, stream)
#define COMFY_GATE_PICK(W32) \
  do { \
    if (per_lane <= 4) COMFY_GATE_LAUNCH(W32, 4); \
    else if (per_lane <= 10) COMFY_GATE_LAUNCH(W32, 10); \
    else COMFY_GATE_LAUNCH(W32, 16); \
  } while (0)
  if (w_dtype == COMFY_MOE_FP32) COMFY_GATE_PICK(true);
  else COMFY_GATE_PICK(false);
#undef COMFY_GATE_PICK
#undef COMFY_GATE_LAUNCH
}

extern "C" int comfy_moe_gate_topk(const void* x, const void* w_gate, int w_dtype, int n_tokens, int dim,
                                   int n_experts, int top_k, int32_t* topk_idx, float* topk_weight,
                                   int32_t* block_counts, int32_t* neartie_count, uint8_t* neartie_flags,
                                   float neartie_eps, void* stream) {
  if (n_tokens < 0 || dim <= 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!x || !w_gate || !topk_idx || !topk_weight || !block_counts) return COMFY_MOE_EINVAL;
  if (!aligned16(x) || !aligned16(w_gate)) return COMFY_MOE_EINVAL;
  if (top_k != 2 || (dim & 7) != 0 || (dim >> 3) > kMaxRowThreads) return COMFY_MOE_EUNSUPPORTED;
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
                                 const float* x_q_scale, int32_t* row_map, int32_t* overflow_count, void* stream) {
  if (n_tokens < 0 || dim <= 0 || n_experts < 1 || n_experts > kMaxExperts) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!x || !topk_idx || !block_offsets || !expert_offsets || !x_perm || !row_map) return COMFY_MOE_EINVAL;
  if (!aligned16(x) || !aligned16(x_perm) || (x_q && !aligned16(x_q))) return COMFY_MOE_EINVAL;
  if ((dim >> 3) > kMaxRowThreads) return COMFY_MOE_EUNSUPPORTED;
  const int n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (act_dtype == COMFY_MOE_BF16) {
    if ((dim & 7) != 0) return COMFY_MOE_EUNSUPPORTED;
    permute_kernel<false, false><<<n_blocks, row_threads(dim), 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), topk_idx, block_offsets, expert_offsets, n_tokens, dim, n_experts, nullptr,
        x_perm, nullptr, nullptr, row_map, nullptr, 0, nullptr, nullptr, nullptr);
  } else if (act_dtype == COMFY_MOE_FP8_E4M3) {
    if ((dim & 15) != 0) return COMFY_MOE_EUNSUPPORTED;
    permute_kernel<true, false><<<n_blocks, row_threads(dim), 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), topk_idx, block_offsets, expert_offsets, n_tokens, dim, n_experts,
        act_scale, x_perm, x_q, x_q_scale, row_map, nullptr, 0, nullptr, nullptr, overflow_count);
  } else {
    return COMFY_MOE_EUNSUPPORTED;
  }
  return check_launch();
}

// Routing plan and permutation in one launch (what comfy_moe_forward uses for up to kFusedPlanMaxBlocks blocks of
// tokens); same outputs as comfy_moe_route_plan followed by comfy_moe_permute, block_offsets excepted.
extern "C" int comfy_moe_plan_permute(const void* x, const int32_t* topk_idx, const int32_t* block_counts,
                                      int n_tokens, int dim, int n_experts, int act_dtype, const float* act_scale,
                                      int32_t* block_offsets_scratch, int32_t* expert_counts, int32_t* expert_offsets,
                                      void* x_perm, void* x_q, const float* x_q_scale, int32_t* row_map,
                                      int32_t* overflow_count, void* stream) {
  if (n_tokens < 0 || dim <= 0 || n_experts < 1 || n_experts > kMaxExperts) return COMFY_MOE_EINVAL;
  if (!expert_counts || !expert_offsets) return COMFY_MOE_EINVAL;
  const int n_blocks = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  if (n_tokens == 0 || n_blocks > kFusedPlanMaxBlocks) {
    // no rows, or too many blocks for every block to re-sum the counts: the two-launch form
    int rc = comfy_moe_route_plan(block_counts, n_tokens, n_experts, block_offsets_scratch, expert_counts,
                                  expert_offsets, stream);
    if (rc != COMFY_MOE_OK) return rc;
    return comfy_moe_permute(x, topk_idx, block_offsets_scratch, expert_offsets, n_tokens, dim, n_experts, act_dtype,
                             act_scale, x_perm, x_q, x_q_scale, row_map, overflow_count, stream);
  }
  if (!x || !topk_idx || !block_counts || !x_perm || !row_map) return COMFY_MOE_EINVAL;
  if (!aligned16(x) || !aligned16(x_perm) || (x_q && !aligned16(x_q))) return COMFY_MOE_EINVAL;
  if ((dim >> 3) > kMaxRowThreads) return COMFY_MOE_EUNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  if (act_dtype == COMFY_MOE_BF16) {
    if ((dim & 7) != 0) return COMFY_MOE_EUNSUPPORTED;
    permute_kernel<false, true><<<n_blocks, row_threads(dim), 0, s>>>(xp, topk_idx, nullptr, nullptr, n_tokens, dim,
                                                                       n_experts, nullptr, x_perm, nullptr, nullptr,
                                                                       row_map, block_counts, n_blocks, expert_counts,
                                                                       expert_offsets, nullptr);
  } else if (act_dtype == COMFY_MOE_FP8_E4M3) {
    if ((dim & 15) != 0) return COMFY_MOE_EUNSUPPORTED;
    permute_kernel<true, true><<<n_blocks, row_threads(dim), 0, s>>>(xp, topk_idx, nullptr, nullptr, n_tokens, dim,
                                                                      n_experts, act_scale, x_perm, x_q, x_q_scale,
                                                                      row_map, block_counts, n_blocks, expert_counts,
                                                                      expert_offsets, overflow_count);
  } else {
    return COMFY_MOE_EUNSUPPORTED;
  }
  return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Debug aid: checks the routing data structures a layer call left behind and reports the first violation
// through the status word (code 9), instead of letting a bad index become a stray memory access further down.
// Checked: every expert id is inside the layer or the slot is unmapped (-1); every mapped row lies inside its
// expert's block [offset[e], offset[e] + count[e]) and below rows_cap; offsets start at 0, are multiples of the row
// alignment and leave room for each expert's rows; the counts add up to the number of mapped slots.
// ------------------------------------------------------------------------------------------------
namespace comfy_b200 {
constexpr int kStatusRoutingInvalid = 9;

__global__ void __launch_bounds__(256)
validate_routing_kernel(const int32_t* __restrict__ topk_idx, const int32_t* __restrict__ row_map,
                        const int32_t* __restrict__ expert_counts, const int32_t* __restrict__ expert_offsets,
                        int n_tokens, int n_experts, long long rows_cap, int32_t* __restrict__ mapped_slots,
                        int32_t* __restrict__ status) {
  bool bad = false;
  int mapped = 0;
  const long long slots = 2LL * n_tokens;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < slots;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int e = topk_idx[i], r = row_map[i];
    if (e < 0 || e >= n_experts) { bad |= (r != -1); continue; }
    ++mapped;
    const int lo = expert_offsets[e], cnt = expert_counts[e];
    bad |= (r < lo) || (r >= lo + cnt) || (r >= rows_cap);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    long long row = 0;
    for (int e = 0; e < n_experts; ++e) {
      bad |= (expert_offsets[e] != row) || (expert_offsets[e] % kRowAlign != 0) || (expert_counts[e] < 0);
      row += (static_cast<long long>(expert_counts[e]) + kRowAlign - 1) / kRowAlign * kRowAlign;
    }
    bad |= (expert_offsets[n_experts] != row) || (row > rows_cap);
  }
  if (mapped) atomicAdd(mapped_slots, mapped);
  if (bad) atomicCAS(status, 0, kStatusRoutingInvalid);
}

__global__ void validate_total_kernel(const int32_t* __restrict__ expert_counts, int n_experts,
                                      const int32_t* __restrict__ mapped_slots, int32_t* __restrict__ status) {
  long long total = 0;
  for (int e = 0; e < n_experts; ++e) total += expert_counts[e];
  if (total != *mapped_slots) atomicCAS(status, 0, kStatusRoutingInvalid);
}
}  // namespace comfy_b200

extern "C" int comfy_moe_validate_routing(const int32_t* topk_idx, const int32_t* row_map, const int32_t* expert_counts,
                                          const int32_t* expert_offsets, int n_tokens, int n_experts, int64_t rows_cap,
                                          int32_t* status, void* stream) {
  if (n_tokens < 0 || n_experts < 1 || n_experts > kMaxExperts || rows_cap < 0 || !status) return COMFY_MOE_EINVAL;
  if (!expert_counts || !expert_offsets || (n_tokens > 0 && (!topk_idx || !row_map))) return COMFY_MOE_EINVAL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t* mapped = status + 3;                      // the reserved word of the status block serves as the counter
  if (cudaMemsetAsync(mapped, 0, sizeof(int32_t), s) != cudaSuccess) return COMFY_MOE_ECUDA;
  long long blocks = (2LL * n_tokens + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  validate_routing_kernel<<<static_cast<int>(blocks), 256, 0, s>>>(topk_idx, row_map, expert_counts, expert_offsets,
                                                                   n_tokens, n_experts, rows_cap, mapped, status);
  validate_total_kernel<<<1, 1, 0, s>>>(expert_counts, n_experts, mapped, status);
  return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Routing without caller-provided scratch.  The per-block counts and offsets that link the gate, the
// plan and the permutation live in a fixed device array that is part of the library image, so a
// caller that cannot allocate device memory passes only inputs and outputs.
// ------------------------------------------------------------------------------------------------
namespace comfy_b200 {
constexpr int kStaticMaxBlocks = COMFY_MOE_STATIC_MAX_TOKENS / kTokensPerBlock;
// [0]: per-block counts, [1]: per-block offsets.  256 KB, held by every GPU that loads the library.
static __device__ __align__(256) int32_t g_route_scratch[2][kStaticMaxBlocks * kMaxExperts];

// Device address of the array on the current device.  In host code the symbol's name is only a
// handle; the address kernels can use has to be asked for, once per device, with that device current.
static int route_scratch_address(int32_t** out) {
  constexpr int kMaxDevices = 64;
  static int32_t* cached[kMaxDevices] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return COMFY_MOE_ECUDA;
  if (dev < 0 || dev >= kMaxDevices) return COMFY_MOE_EUNSUPPORTED;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_route_scratch) != cudaSuccess || p == nullptr) return COMFY_MOE_ECUDA;
    cached[dev] = static_cast<int32_t*>(p);
  }
  *out = cached[dev];
  return COMFY_MOE_OK;
}
}  // namespace comfy_b200

extern "C" int comfy_moe_route_static(const void* x, const void* w_gate, int w_dtype, int n_tokens, int dim,
                                      int n_experts, int top_k, int act_dtype, const float* act_scale,
                                      int32_t* topk_idx, float* topk_weight, int32_t* expert_counts,
                                      int32_t* expert_offsets, void* x_perm, void* x_q, const float* x_q_scale,
                                      int32_t* row_map, int32_t* neartie_count, void* stream) {
  if (n_tokens < 0) return COMFY_MOE_EINVAL;
  if (n_tokens > COMFY_MOE_STATIC_MAX_TOKENS) return COMFY_MOE_ETOOLARGE;   // the fixed scratch is too small
  if (n_experts < 1 || n_experts > kMaxExperts) return COMFY_MOE_EINVAL;
  int32_t* scratch = nullptr;
  int rc = route_scratch_address(&scratch);
  if (rc != COMFY_MOE_OK) return rc;
  int32_t* block_counts = scratch;
  int32_t* block_offsets = scratch + kStaticMaxBlocks * kMaxExperts;
  // Every scratch word read below is written earlier in this same call (the gate overwrites the counts of
  // all blocks in use, the plan all their offsets), so nothing left by a previous call is ever consumed.
  rc = comfy_moe_gate_topk(x, w_gate, w_dtype, n_tokens, dim, n_experts, top_k, topk_idx, topk_weight, block_counts,
                           neartie_count, nullptr, 1e-6f, stream);
  if (rc != COMFY_MOE_OK) return rc;
  rc = comfy_moe_route_plan(block_counts, n_tokens, n_experts, block_offsets, expert_counts, expert_offsets, stream);
  if (rc != COMFY_MOE_OK) return rc;
  return comfy_moe_permute(x, topk_idx, block_offsets, expert_offsets, n_tokens, dim, n_experts, act_dtype, act_scale,
                           x_perm, x_q, x_q_scale, row_map, nullptr, stream);
}
