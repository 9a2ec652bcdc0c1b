// Expert parallelism over peer memory (NVLink): dispatch and combine without a host synchronisation.
//
// The reference runs on one GPU and has nothing like this; the partitioning follows from the layer
// (comfy/ldm/hidream/model.py:287-346): tokens stay with their rank, a routed expert lives on one rank (or on
// two, each with half of its hidden dimension), and the only exchange is "rows to the expert" and "results back".
//
//   dispatch_kernel   the row permutation, writing every routed row straight into the receive buffer of the rank(s)
//                     that compute its expert (16-byte stores into peer memory; the row's place there follows from
//                     the all-gathered per-rank expert histograms, so no rank asks the host anything)
//   signal / wait     one 32-bit epoch flag per (kind, source rank) in every rank's flag block; a rank raises its
//                     flag at all peers after its dispatch ("arrived") and after its expert GEMM ("done"), and waits,
//                     with a clock budget, for all peers' flags before it consumes what they wrote
//   combine_peer      the weighted combine, reading each routed result from the y buffer of the rank that computed
//                     it (plain 16-byte loads from peer memory)
//
// Every rank keeps one receive buffer and one result buffer of fixed capacity, mapped into all peers.  The order of
// the calls of one step makes single buffers safe: a rank writes into a peer's receive buffer only after its own
// previous combine, which waited for that peer's "done"; a rank overwrites its result buffer only after all peers
// raised "arrived" for the new step, which they do after their previous combine.
#include <cstring>

#include "moe_common.cuh"

namespace comfy_b200 {

constexpr int kMaxRanks = COMFY_MOE_MAX_RANKS;
constexpr int kPeerRowThreads = 512;
constexpr int kStatusPeerTimeout = 7;           // device status word: a peer's flag did not arrive in time
constexpr int kStatusPeerCapacity = 8;          // device status word: the routed rows do not fit the receive buffer

struct PeerParams {
  int world, rank, n_experts, splits;
  int owner[kMaxExperts][2];                    // ranks computing expert e ([1] = -1 without a hidden split)
  uint8_t* recv[kMaxRanks];                     // receive buffer of every rank, as mapped here
  const __nv_bfloat16* y[kMaxRanks];            // result buffer of every rank, as mapped here
  uint32_t* flags[kMaxRanks];                   // flag block of every rank: [2 kinds][kMaxRanks sources]
};

// First row, in the receive buffer of rank q, of the rows that `source` sends for expert e: q's experts in
// increasing order, each holding the rows of source 0, 1, ... one after the other.
__device__ __forceinline__ int recv_row_base(const PeerParams& p, const int32_t* __restrict__ counts_all, int q, int e,
                                             int source) {
  int row = 0;
  for (int f = 0; f < e; ++f) {
    if (p.owner[f][0] == q || p.owner[f][1] == q)
      for (int s = 0; s < p.world; ++s) row += counts_all[s * p.n_experts + f];
  }
  for (int s = 0; s < source; ++s) row += counts_all[s * p.n_experts + e];
  return row;
}

template <bool kFp8>
__global__ void __launch_bounds__(kPeerRowThreads)
dispatch_kernel(const __grid_constant__ PeerParams p, const __nv_bfloat16* __restrict__ x,
                const int32_t* __restrict__ topk_idx, const int32_t* __restrict__ block_offsets,
                const int32_t* __restrict__ counts_all, int n_tokens, int dim, long long cap_rows,
                const float* __restrict__ act_scale, void* __restrict__ x_q, const float* __restrict__ x_q_scale,
                int32_t* __restrict__ row_map, int32_t* __restrict__ group_start, int32_t* __restrict__ group_count,
                int32_t* __restrict__ y_row_shift, int32_t* __restrict__ status) {
  constexpr int kSlots = kTokensPerBlock * 2;
  __shared__ int s_base[kMaxExperts];           // row of this rank's first slot of expert e at the expert's owner(s)
  __shared__ int s_local[kMaxExperts];          // the same slot's row in this rank's own (compact, expert-major) order
  __shared__ int warp_cnt[kSlots / 32][kMaxExperts];
  __shared__ uint8_t* s_dst[kSlots][2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int block_tok0 = blockIdx.x * kTokensPerBlock;
  const int row_bytes = kFp8 ? dim : dim * 2;

  if (tid < p.n_experts) {
    const int e = tid;
    const int q = p.owner[e][0];
    // with a hidden split both owners hold only this expert, so the row is the same at either
    int base = recv_row_base(p, counts_all, q, e, p.rank);
    int total = 0;
    for (int s = 0; s < p.world; ++s) total += counts_all[s * p.n_experts + e];
    const int end_of_group = recv_row_base(p, counts_all, q, e, 0) + total;
    if (end_of_group > cap_rows) { base = -1; atomicCAS(status, 0, kStatusPeerCapacity); }
    const int in_block = n_tokens == 0 ? 0 : block_offsets[blockIdx.x * p.n_experts + e];
    s_base[e] = (base < 0 || n_tokens == 0) ? -1 : base + in_block;
    int local = 0;
    for (int f = 0; f < e; ++f) local += counts_all[p.rank * p.n_experts + f];
    s_local[e] = local + in_block;
    if (blockIdx.x == 0) {
      // this rank's own work list
      int j = 0;
      for (int f = 0; f < e; ++f) j += (p.owner[f][0] == p.rank || p.owner[f][1] == p.rank) ? 1 : 0;
      if (p.owner[e][0] == p.rank || p.owner[e][1] == p.rank) {
        const bool fits = end_of_group <= cap_rows;
        if (y_row_shift == nullptr) {
          // one row range per local expert, all sources together; results stay in this rank's result buffer
          group_start[j] = recv_row_base(p, counts_all, p.rank, e, 0);
          group_count[j] = fits ? total : 0;
        } else {
          // one row range per (local expert, source): the results of source s go straight into s's return buffer,
          // at the rows s's own expert-major order gives them.  The ranges are listed starting with this rank's own
          // rows and then rank + 1, rank + 2, ...: the expert GEMM walks them in this order, so it starts on rows
          // that are certainly there while the peers' rows are still landing, and no two ranks expect the same
          // peer's rows first.
          for (int pos = 0; pos < p.world; ++pos) {
            const int src = (p.rank + pos) % p.world;
            const int g = j * p.world + pos;
            const int start = recv_row_base(p, counts_all, p.rank, e, src);
            int src_local = 0;
            for (int f = 0; f < e; ++f) src_local += counts_all[src * p.n_experts + f];
            group_start[g] = start;
            group_count[g] = fits ? counts_all[src * p.n_experts + e] : 0;
            y_row_shift[g] = src_local - start;
          }
        }
      }
    }
  }

  int my_e = -1, my_rank = 0;
  if (tid < kSlots) {
    const int slot = block_tok0 * 2 + tid;
    if (slot < n_tokens * 2) my_e = topk_idx[slot];
    if (my_e >= p.n_experts) my_e = -1;
    for (int e = 0; e < p.n_experts; ++e) {
      const unsigned m = __ballot_sync(0xffffffffu, my_e == e);
      if (my_e == e) my_rank = __popc(m & ((1u << lane) - 1u));
      if (lane == 0) warp_cnt[warp][e] = __popc(m);
    }
  }
  __syncthreads();
  if (tid < kSlots) {
    int d = -1;
    if (my_e >= 0 && s_base[my_e] >= 0) {
      int before = my_rank;
      for (int w = 0; w < warp; ++w) before += warp_cnt[w][my_e];
      d = s_base[my_e] + before;
    }
    if (block_tok0 * 2 + tid < n_tokens * 2) {
      // pull mode: the row at the owner; push mode: the row of this rank's return buffer the owner writes
      int m = d;
      if (y_row_shift != nullptr && d >= 0) m = s_local[my_e] + (d - s_base[my_e]);
      row_map[block_tok0 * 2 + tid] = m;
    }
    for (int o = 0; o < 2; ++o) {
      const int q = (d >= 0) ? p.owner[my_e][o] : -1;
      s_dst[tid][o] = q >= 0 ? p.recv[q] + static_cast<size_t>(d) * row_bytes : nullptr;
    }
  }
  __syncthreads();

  const int chunks = kFp8 ? (dim >> 4) : (dim >> 3);
  if (tid >= chunks) return;

  if constexpr (!kFp8) {
    constexpr int kTok = 8;
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
#pragma unroll
          for (int k = 0; k < 2; ++k)
#pragma unroll
            for (int o = 0; o < 2; ++o) {
              uint8_t* d = s_dst[2 * (base + i) + k][o];
              if (d) reinterpret_cast<uint4*>(d)[tid] = v[i];
            }
        }
      }
    }
  } else {
    // the activation quantiser of comfy/ops.py:338-343, as in the single-GPU permutation
    float inv_p = 1.f, inv_q = 1.f;
    bool scaled_p = false, scaled_q = false;
    if (act_scale) { inv_p = round_bf16(1.0f / __ldg(act_scale)); scaled_p = true; }
    if (x_q_scale) { inv_q = round_bf16(1.0f / __ldg(x_q_scale)); scaled_q = true; }
    const bool same_q = (scaled_q == scaled_p) && (inv_q == inv_p);
    uint8_t* xq = static_cast<uint8_t*>(x_q);
    int ovf = 0;
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
            int ovf_q = 0;
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
#pragma unroll
        for (int k = 0; k < 2; ++k)
#pragma unroll
          for (int o = 0; o < 2; ++o) {
            uint8_t* d = s_dst[2 * (base + i) + k][o];
            if (d) reinterpret_cast<uint4*>(d)[tid] = vp;
          }
        if (xq) reinterpret_cast<uint4*>(xq + static_cast<size_t>(t0 + i) * dim)[tid] = make_uint4(wq[0], wq[1], wq[2], wq[3]);
      }
    }
    if (ovf) atomicAdd(status + kStatusE4m3Overflow, ovf);
  }
}

// Raises this rank's flag of `kind` at every rank.  Runs after the kernel whose writes it announces (stream order);
// the fence and the release store order those writes before the flag for an observer anywhere in the system.
__global__ void peer_signal_kernel(const __grid_constant__ PeerParams p, int kind, uint32_t epoch) {
  const int r = threadIdx.x;
  if (r >= p.world) return;
  __threadfence_system();
  uint32_t* flag = p.flags[r] + kind * kMaxRanks + p.rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
}

// Waits until every rank's flag of `kind` in this rank's flag block has reached `epoch`.  Bounded: after the clock
// budget the kernel records kStatusPeerTimeout and returns, the host turns that into an error.
__global__ void peer_wait_kernel(const __grid_constant__ PeerParams p, int kind, uint32_t epoch, long long budget,
                                 int32_t* __restrict__ status) {
  const int r = threadIdx.x;
  if (r >= p.world) return;
  const uint32_t* flag = p.flags[p.rank] + kind * kMaxRanks + r;
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) break;
    if (clock64() - t0 > budget) { atomicCAS(status, 0, kStatusPeerTimeout); break; }
    __nanosleep(200);
  }
}

// combine_kernel of the single-GPU path with every routed row read from the rank that computed it.  With a hidden
// split two ranks hold partial results of the same row; their sum, rounded to bf16, stands in for the expert output.
template <bool kTwo>
__global__ void __launch_bounds__(kPeerRowThreads)
combine_peer_kernel(const __grid_constant__ PeerParams p, const int32_t* __restrict__ topk_idx,
                    const int32_t* __restrict__ row_map, const float* __restrict__ topk_weight,
                    const __nv_bfloat16* __restrict__ y_shared, int n_tokens, int dim,
                    __nv_bfloat16* __restrict__ out) {
  const int tid = threadIdx.x;
  if (tid >= (dim >> 3)) return;
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  uint4 v[2][2];
  float w[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int r = __ldg(row_map + 2 * t + k);
    int e = __ldg(topk_idx + 2 * t + k);
    w[k] = round_bf16(__ldg(topk_weight + 2 * t + k));
    v[k][0] = v[k][1] = make_uint4(0, 0, 0, 0);
    if (r >= 0 && e >= 0 && e < p.n_experts) {
      v[k][0] = *(reinterpret_cast<const uint4*>(p.y[p.owner[e][0]] + static_cast<size_t>(r) * dim) + tid);
      if constexpr (kTwo) v[k][1] = *(reinterpret_cast<const uint4*>(p.y[p.owner[e][1]] + static_cast<size_t>(r) * dim) + tid);
    }
  }
  uint4 vs = make_uint4(0, 0, 0, 0);
  if (y_shared) vs = ld_nc_u4(reinterpret_cast<const uint4*>(y_shared + static_cast<size_t>(t) * dim) + tid);
  float fa[8], fb[8], fs[8], r[8];
  unpack_bf16x8(v[0][0], fa);
  unpack_bf16x8(v[1][0], fb);
  unpack_bf16x8(vs, fs);
  if constexpr (kTwo) {
    float ga[8], gb[8];
    unpack_bf16x8(v[0][1], ga);
    unpack_bf16x8(v[1][1], gb);
#pragma unroll
    for (int k = 0; k < 8; ++k) { fa[k] = round_bf16(fa[k] + ga[k]); fb[k] = round_bf16(fb[k] + gb[k]); }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float p0 = round_bf16(w[0] * fa[k]);
    const float p1 = round_bf16(w[1] * fb[k]);
    const float routed = round_bf16(p0 + p1);
    r[k] = y_shared ? routed + fs[k] : routed;
  }
  reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * dim)[tid] =
      make_uint4(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]), pack_bf16x2(r[4], r[5]), pack_bf16x2(r[6], r[7]));
}

static int fill_params(const ComfyMoePeerPlan* plan, PeerParams* p) {
  if (!plan) return COMFY_MOE_EINVAL;
  if (plan->world < 1 || plan->world > kMaxRanks || plan->rank < 0 || plan->rank >= plan->world) return COMFY_MOE_EINVAL;
  if (plan->n_experts < 1 || plan->n_experts > kMaxExperts) return COMFY_MOE_EINVAL;
  if (plan->hidden_splits != 1 && plan->hidden_splits != 2) return COMFY_MOE_EUNSUPPORTED;
  memset(p, 0, sizeof(*p));
  p->world = plan->world; p->rank = plan->rank; p->n_experts = plan->n_experts; p->splits = plan->hidden_splits;
  for (int e = 0; e < plan->n_experts; ++e) {
    const int o0 = plan->owner0[e], o1 = plan->hidden_splits == 2 ? plan->owner1[e] : -1;
    if (o0 < 0 || o0 >= plan->world || o1 >= plan->world || (plan->hidden_splits == 2 && o1 < 0)) return COMFY_MOE_EINVAL;
    p->owner[e][0] = o0; p->owner[e][1] = o1;
  }
  for (int r = 0; r < plan->world; ++r) {
    if (!plan->peer_recv[r] || !plan->peer_y[r] || !plan->peer_flags[r]) return COMFY_MOE_EINVAL;
    if (!aligned16(plan->peer_recv[r]) || !aligned16(plan->peer_y[r])) return COMFY_MOE_EINVAL;
    p->recv[r] = static_cast<uint8_t*>(plan->peer_recv[r]);
    p->y[r] = static_cast<const __nv_bfloat16*>(plan->peer_y[r]);
    p->flags[r] = plan->peer_flags[r];
  }
  return COMFY_MOE_OK;
}

}  // namespace comfy_b200

using namespace comfy_b200;

extern "C" int comfy_moe_ep_dispatch(const ComfyMoePeerPlan* plan, const void* x, const int32_t* topk_idx,
                                     const int32_t* block_offsets, const int32_t* counts_all, int n_tokens, int dim,
                                     int act_dtype, const float* act_scale, void* x_q, const float* x_q_scale,
                                     int32_t* row_map, int32_t* group_start, int32_t* group_count,
                                     int32_t* y_row_shift, int32_t* status, void* stream) {
  PeerParams p;
  int rc = fill_params(plan, &p);
  if (rc != COMFY_MOE_OK) return rc;
  if (n_tokens < 0 || dim <= 0 || plan->cap_rows <= 0) return COMFY_MOE_EINVAL;
  if (!counts_all || !group_start || !group_count || !status) return COMFY_MOE_EINVAL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool fp8 = act_dtype == COMFY_MOE_FP8_E4M3;
  if (!fp8 && act_dtype != COMFY_MOE_BF16) return COMFY_MOE_EUNSUPPORTED;
  if ((dim & (fp8 ? 15 : 7)) != 0 || (dim >> 3) > kPeerRowThreads) return COMFY_MOE_EUNSUPPORTED;
  if (n_tokens > 0 && (!x || !topk_idx || !block_offsets || !row_map || !aligned16(x) || (x_q && !aligned16(x_q))))
    return COMFY_MOE_EINVAL;
  // a rank without tokens still publishes its work list (one block, no rows)
  const int n_blocks = n_tokens > 0 ? (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock : 1;
  const int threads = (((fp8 ? dim >> 4 : dim >> 3) + 31) & ~31) < 64 ? 64 : (((fp8 ? dim >> 4 : dim >> 3) + 31) & ~31);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  if (fp8)
    dispatch_kernel<true><<<n_blocks, threads, 0, s>>>(p, xp, topk_idx, block_offsets, counts_all, n_tokens, dim,
                                                       plan->cap_rows, act_scale, x_q, x_q_scale, row_map, group_start,
                                                       group_count, y_row_shift, status);
  else
    dispatch_kernel<false><<<n_blocks, threads, 0, s>>>(p, xp, topk_idx, block_offsets, counts_all, n_tokens, dim,
                                                        plan->cap_rows, nullptr, nullptr, nullptr, row_map, group_start,
                                                        group_count, y_row_shift, status);
  return check_launch();
}

extern "C" int comfy_moe_ep_signal(const ComfyMoePeerPlan* plan, int kind, uint32_t epoch, void* stream) {
  PeerParams p;
  int rc = fill_params(plan, &p);
  if (rc != COMFY_MOE_OK) return rc;
  if (kind < 0 || kind > 1) return COMFY_MOE_EINVAL;
  peer_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p, kind, epoch);
  return check_launch();
}

extern "C" int comfy_moe_ep_wait_budget(const ComfyMoePeerPlan* plan, int kind, uint32_t epoch, int64_t budget_cycles,
                                        int32_t* status, void* stream) {
  PeerParams p;
  int rc = fill_params(plan, &p);
  if (rc != COMFY_MOE_OK) return rc;
  if (kind < 0 || kind > 1 || !status || budget_cycles <= 0) return COMFY_MOE_EINVAL;
  peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p, kind, epoch, budget_cycles, status);
  return check_launch();
}

extern "C" int comfy_moe_ep_wait(const ComfyMoePeerPlan* plan, int kind, uint32_t epoch, int32_t* status,
                                 void* stream) {
  return comfy_moe_ep_wait_budget(plan, kind, epoch, COMFY_MOE_EP_WAIT_CYCLES, status, stream);
}

extern "C" int comfy_moe_ep_combine(const ComfyMoePeerPlan* plan, const int32_t* topk_idx, const int32_t* row_map,
                                    const float* topk_weight, const void* y_shared, int n_tokens, int dim, void* out,
                                    void* stream) {
  PeerParams p;
  int rc = fill_params(plan, &p);
  if (rc != COMFY_MOE_OK) return rc;
  if (n_tokens < 0 || dim <= 0) return COMFY_MOE_EINVAL;
  if (n_tokens == 0) return COMFY_MOE_OK;
  if (!topk_idx || !row_map || !topk_weight || !out || !aligned16(out) || (y_shared && !aligned16(y_shared)))
    return COMFY_MOE_EINVAL;
  if ((dim & 7) != 0 || (dim >> 3) > kPeerRowThreads) return COMFY_MOE_EUNSUPPORTED;
  const int threads = ((dim >> 3) + 31) & ~31;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* ys = static_cast<const __nv_bfloat16*>(y_shared);
  if (plan->hidden_splits == 2)
    combine_peer_kernel<true><<<n_tokens, threads, 0, s>>>(p, topk_idx, row_map, topk_weight, ys, n_tokens, dim,
                                                           static_cast<__nv_bfloat16*>(out));
  else
    combine_peer_kernel<false><<<n_tokens, threads, 0, s>>>(p, topk_idx, row_map, topk_weight, ys, n_tokens, dim,
                                                            static_cast<__nv_bfloat16*>(out));
  return check_launch();
}
