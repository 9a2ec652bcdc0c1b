// Attention forward for the HiDream blocks on sm_100a: softmax(Q K^T / sqrt(d)) V with the two contractions on
// tcgen05 tensor cores, S and O accumulators in TMEM, K / V tiles fed by TMA.  Replaces the
// scaled_dot_product_attention call behind comfy/ldm/hidream/model.py:75-76 (attention_pytorch,
// comfy/ldm/modules/attention.py:475-516) for the block's shape: bf16, head_dim 128, no mask, not causal.
//
// One CTA computes 256 query rows of one (batch, head), as two tiles a and b of 128 rows, against all keys, 128 keys at
// a time:
//   S_t = Q_t K_j^T          tcgen05.mma, A = Q_t (shared memory), B = K_j (shared memory), D = S_t in TMEM
//   P_t = exp2(c S_t - m)    128 softmax threads per tile, one query row each: the row's scores come out of TMEM into
//                            the thread's registers, so maximum and sum need no shuffles; P goes back to TMEM as bf16,
//                            over the scores it was made from
//   O_t += P_t V_j           tcgen05.mma, A = P_t (TMEM), B = V_j (shared memory, keys along K), D = O_t in TMEM
// The two tiles share every K / V tile in shared memory and alternate on the tensor pipe: while the softmax threads of
// tile a work on S_a, the pipe runs O_b += P_b V and the next S_b, and the other way round, so that exponentials (the
// scarce resource: 16 per clock and SM) and MMAs overlap.  TMEM holds S_a, S_b, O_a, O_b: all 512 columns.  (Steps of
// 64 keys with two S buffers per tile were tried: MMAs with N = 64 ran at half the rate, 0.58 ms against 0.40 ms.)
// The reference maximum m of a row is only raised when a step's maximum exceeds it by more than 8 (in log2 units): P
// then stays below 2^8, which bf16 and the fp32 accumulators hold without loss, and O (which lives in TMEM and would
// have to be read, scaled and written back) is rescaled only on those rare steps; the final division by the row sum
// makes the result independent of the reference point.  So the common case is ONE pass over a step's scores:
// exponentials against the current m and the step's maximum side by side; only when the maximum turns out too large
// (always on the first step) is the step redone after raising m.
// What bounds it (measured at 2 x 20 heads x 4480 x 128, SM-clock stamps of one CTA): a step of 128 keys for both tiles
// needs about 2300 cycles of the tensor pipe (the Q K^T MMAs, both operands from shared memory, run at 80 cycles instead
// of 64: 8 KB of operands per MMA is more than shared memory delivers in 64) and 2048 cycles of the special-function
// unit (4 exponentials per clock and sub-partition; the softmax warps alone, tensor pipe idle, take 0.28 ms for the
// whole problem, the MMA stream alone 0.28 ms too).  The kernel takes about 3700 per step, 0.39 ms: S_t(j+1) cannot be issued
// before P_t(j) has been consumed (they share columns; TMEM has no room for a second S per tile), so each tile's chain is
// softmax (1700 + 230 to store P) -> O_t += P V, S_t = Q K^T (1150) -> barrier latencies (500), and two tiles fill the
// pipe to 60 %.  Two threads per row (16 softmax warps) lengthened the chain by the exchange between them (0.43 ms);
// handing P to the MMA warp in four pieces, so that O += P V follows the softmax piece by piece, cost more in waits
// of the MMA warp (about 150 cycles each even when the barrier is already complete, plus MMA issue that blocks at
// the pipe's rate) than it saved (0.54 ms), and one MMA warp per tile lost the alternation of the two tiles: both
// softmax phases then run at the same time and both MMA phases after them (0.54 ms); polling with test_wait instead
// of try_wait, 16-column loads, and one arrival per thread changed nothing or lost.
// Warps: 0-3 softmax and epilogue of tile a, 4-7 of tile b (TMEM lane quarter = warp index & 3), 8 = MMA issuer and
// TMEM owner, 9 = TMA producer.  Every wait is bounded and reports through the status word like the waits of the
// grouped GEMM.
//
// The COMFY_ATTN_EXPERIMENT_* switches are for timing only (each removes one cost: exponentials, the softmax, the K / V
// loads, the wait for P) and produce wrong results; the library is never built with them.
#include <cuda.h>

#include "moe_common.cuh"
#include "ptx_sm100.cuh"

namespace comfy_b200 {

#ifdef COMFY_ATTN_TRACE
// Development aid, never built into the library: SM-clock stamps of CTA (0, 0, 0), [role][step][event], read back
// with comfy_attn_trace_read.  Roles: 0 / 1 = first softmax warp of tile a / b, 2 = MMA warp.
__device__ long long attn_trace[3][64][12];
#define ATTN_STAMP(role, step, ev) \
  do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (step) >= 0 && (step) < 64) \
         attn_trace[role][step][ev] = clock64(); } while (0)
#else
#define ATTN_STAMP(role, step, ev) do { } while (0)
#endif

constexpr int kAttnD = 128;                    // head dimension
constexpr int kAttnM = 128;                    // query rows per tile
constexpr int kAttnQTiles = 2;                 // query tiles per CTA
constexpr int kAttnN = 128;                    // keys per step
constexpr int kAttnStages = 2;                 // K / V stages in flight
constexpr int kAttnQBoxBytes = 128 * 128;      // one TMA box of Q: 128 rows x 64 bf16 (128 bytes, 128-byte swizzle)
constexpr int kAttnQTileBytes = 2 * kAttnQBoxBytes;
constexpr int kAttnKvBoxBytes = kAttnN * 128;  // one TMA box of K or V: 128 rows x 64 bf16
constexpr int kAttnKvTileBytes = 2 * kAttnKvBoxBytes;   // 128 keys x 128 head-dimension elements
constexpr int kAttnSoftmaxWarps = 4 * kAttnQTiles;
constexpr int kAttnThreads = (kAttnSoftmaxWarps + 2) * 32;
constexpr int kAttnTmemCols = 512;
constexpr size_t kAttnSmem = kAttnQTiles * kAttnQTileBytes + 2 * kAttnStages * kAttnKvTileBytes + 1024;
constexpr int kStatusAttnTimeout = 5;
constexpr float kAttnRescaleThreshold = 8.0f;  // log2 units

__host__ __device__ constexpr uint32_t attn_s_col(int tile) { return tile * 128; }
__host__ __device__ constexpr uint32_t attn_o_col(int tile) { return 256 + tile * 128; }

struct AttnParams {
  CUtensorMap map_q, map_k, map_v;             // [B][S][H * D] bf16; boxes of 128 rows x 64 elements
  __nv_bfloat16* out;                          // [B, S_q, H * D]
  int32_t* status;
  int seq_q, seq_kv, heads;
  float scale_log2;                            // softmax scale * log2(e)
};

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Shared-memory descriptor of a B operand whose N dimension is the contiguous one (V: rows = keys = K of the MMA,
// 64 head-dimension elements per 128-byte row, the other 64 in a second box `box_stride` bytes further), 128-byte
// swizzle: leading byte offset = distance between the two 64-element column blocks, stride byte offset = distance
// between groups of eight keys.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t box_stride) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((box_stride >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (P) is read from tensor memory.
__device__ __forceinline__ void umma_ts_bf16(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
#ifdef COMFY_ATTN_EXPERIMENT_NO_MUFU
  return x * 0.001f + 1.0f;          // timing experiment only: wrong numbers, no special-function unit
#else
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
#endif
}

// One softmax step of one query row (this thread's TMEM lane): the 128 scores of the step against the reference
// maximum.  p = exp2(s * scale - m): one FFMA and one MUFU per element.  The probabilities come back as 64 bf16 pairs,
// their unrounded sum in `sum`, the largest raw score in `raw_max` (four independent chains each).  kMasked: only the
// first `valid` keys of the step exist.
template <bool kMasked>
__device__ __forceinline__ void attn_softmax_step(uint32_t s_tmem, float scale_log2, float neg_m, int valid,
                                                  uint32_t (&pr)[64], float& sum, float& raw_max) {
  float part[4] = {0.f, 0.f, 0.f, 0.f};
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  // All 128 scores are requested at once and waited for once: a TMEM load takes several hundred cycles while the tensor
  // pipe works on the other tile, and tcgen05.wait::ld waits for every load in flight.
  uint32_t sr[4][32];
#pragma unroll
  for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(s_tmem + c * 32, sr[c]);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float s0 = __uint_as_float(sr[c][i]), s1 = __uint_as_float(sr[c][i + 1]);
      if constexpr (kMasked) {
        if (c * 32 + i >= valid) s0 = -INFINITY;
        if (c * 32 + i + 1 >= valid) s1 = -INFINITY;
      }
      mx[(i >> 1) & 3] = fmaxf(mx[(i >> 1) & 3], fmaxf(s0, s1));
      const float e0 = fast_exp2(fmaf(s0, scale_log2, neg_m));
      const float e1 = fast_exp2(fmaf(s1, scale_log2, neg_m));
      part[(i >> 1) & 3] += e0 + e1;
      pr[c * 16 + (i >> 1)] = pack_bf16x2(e0, e1);
    }
  }
  sum = (part[0] + part[1]) + (part[2] + part[3]);
  raw_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

// (10 warps put three on one SM sub-partition, whose 16384 registers then allow 168 per thread)
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full;
  __shared__ __align__(8) uint64_t k_full[kAttnStages], k_empty[kAttnStages];
  __shared__ __align__(8) uint64_t v_full[kAttnStages], v_empty[kAttnStages];
  __shared__ __align__(8) uint64_t s_full[kAttnQTiles];
  __shared__ __align__(8) uint64_t p_ready[kAttnQTiles];
  __shared__ __align__(8) uint64_t o_done[kAttnQTiles][2];     // by step parity, like the S buffers
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* k_smem = smem + kAttnQTiles * kAttnQTileBytes;
  uint8_t* v_smem = k_smem + kAttnStages * kAttnKvTileBytes;

  const int head = blockIdx.y, batch = blockIdx.z;
  const int q_row0 = blockIdx.x * (kAttnQTiles * kAttnM);
  const int n_kv = (p.seq_kv + kAttnN - 1) / kAttnN;
  const int col0 = head * kAttnD;              // first element of this head inside a token's H * D row

  if (tid == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < kAttnStages; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < kAttnQTiles; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_ready[t], 4);            // one arrival per softmax warp
      for (int b = 0; b < 2; ++b) mbar_init(&o_done[t][b], 1);
    }
    fence_mbar_init();
    abort_flag = 0;
  }
  if (warp == kAttnSoftmaxWarps) { tmem_alloc(&tmem_slot, kAttnTmemCols); tmem_relinquish(); }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_ptr = &abort_flag;
  auto give_up = [&]() {
    if (lane == 0) { atomicCAS(p.status, 0, kStatusAttnTimeout); abort_flag = 1; }
  };

  if (warp == kAttnSoftmaxWarps + 1) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_arrive_expect_tx(&q_full, kAttnQTiles * kAttnQTileBytes);
#pragma unroll
      for (int t = 0; t < kAttnQTiles; ++t) {
        tma_load_3d(q_smem + t * kAttnQTileBytes, &p.map_q, &q_full, col0, q_row0 + t * kAttnM, batch);
        tma_load_3d(q_smem + t * kAttnQTileBytes + kAttnQBoxBytes, &p.map_q, &q_full, col0 + 64, q_row0 + t * kAttnM, batch);
      }
    }
    __syncwarp();
    bool ok = true;
#ifdef COMFY_ATTN_EXPERIMENT_NO_LOADS
    const int n_loads = n_kv < kAttnStages ? n_kv : kAttnStages;     // timing experiment only: K / V loaded once
#else
    const int n_loads = n_kv;
#endif
    for (int j = 0; j < n_loads && ok; ++j) {
      const int s = j % kAttnStages;
      const uint32_t ph = (j / kAttnStages) & 1u;
      ok = mbar_wait_warp(&k_empty[s], ph ^ 1u, abort_ptr);
      if (!ok) { give_up(); break; }
      if (elect_one()) {
        mbar_arrive_expect_tx(&k_full[s], kAttnKvTileBytes);
        tma_load_3d(k_smem + s * kAttnKvTileBytes, &p.map_k, &k_full[s], col0, j * kAttnN, batch);
        tma_load_3d(k_smem + s * kAttnKvTileBytes + kAttnKvBoxBytes, &p.map_k, &k_full[s], col0 + 64, j * kAttnN, batch);
      }
      __syncwarp();
      ok = mbar_wait_warp(&v_empty[s], ph ^ 1u, abort_ptr);
      if (!ok) { give_up(); break; }
      if (elect_one()) {
        mbar_arrive_expect_tx(&v_full[s], kAttnKvTileBytes);
        tma_load_3d(v_smem + s * kAttnKvTileBytes, &p.map_v, &v_full[s], col0, j * kAttnN, batch);
        tma_load_3d(v_smem + s * kAttnKvTileBytes + kAttnKvBoxBytes, &p.map_v, &v_full[s], col0 + 64, j * kAttnN, batch);
      }
      __syncwarp();
    }
  } else if (warp == kAttnSoftmaxWarps) {
    // ------------------------------------------------------------------ MMA issuer
    // Order on the tensor pipe: S_a(0) S_b(0) | O_a(0) S_a(1) | O_b(0) S_b(1) | O_a(1) S_a(2) | ...
    // S_t(j+1) overwrites the columns whose first half holds P_t(j); it is issued after O_t(j), and the pipe executes
    // MMAs of one shape from one thread in order (all MMAs here are 128 x 128 x 16).
    constexpr uint32_t idesc_qk = umma_idesc<false>(kAttnM, kAttnN);
    constexpr uint32_t idesc_pv = umma_idesc<false>(kAttnM, kAttnD) | (1u << 16);     // B with N contiguous
    bool ok = mbar_wait_warp(&q_full, 0, abort_ptr);
    const uint32_t q_addr = smem_u32(q_smem);

    // The eight MMAs of one product differ only in the start addresses inside their descriptors (16-byte units in the low
    // bits): one 64-bit add with a constant each, so that issuing an MMA costs a handful of instructions (the MMAs here
    // last 64 to 80 cycles; an issue loop that rebuilds descriptors takes about 100 per MMA).
    auto mma_qk = [&](int t, int j) {                // S_t(j) = Q_t K_j^T; the last tile to use K_j frees its stage
      const int s = j % kAttnStages;
      const uint64_t q_desc = umma_desc_k_sw128(q_addr + t * kAttnQTileBytes);
      const uint64_t k_desc = umma_desc_k_sw128(smem_u32(k_smem + s * kAttnKvTileBytes));
      const uint32_t d_tmem = tmem_base + attn_s_col(t);
#pragma unroll
      for (int kk = 0; kk < kAttnD / 16; ++kk) {
        // 16 elements of the head dimension = 32 bytes inside a box; the second 64 elements live in the second box
        umma_ss<false>(d_tmem, q_desc + (((kk >> 2) * kAttnQBoxBytes + (kk & 3) * 32) >> 4),
                       k_desc + (((kk >> 2) * kAttnKvBoxBytes + (kk & 3) * 32) >> 4), idesc_qk, kk != 0 ? 1u : 0u);
      }
      umma_commit(&s_full[t]);
      if (t == kAttnQTiles - 1) umma_commit(&k_empty[s]);
    };
    auto mma_pv = [&](int t, int j) {                // O_t += P_t(j) V_j; the last tile to use V_j frees its stage
      const int s = j % kAttnStages;
      const uint64_t v_desc = umma_desc_mn_sw128(smem_u32(v_smem + s * kAttnKvTileBytes), kAttnKvBoxBytes);
      const uint32_t p_tmem = tmem_base + attn_s_col(t);
      const uint32_t o_tmem = tmem_base + attn_o_col(t);
      const uint32_t acc0 = j != 0 ? 1u : 0u;
#pragma unroll
      for (int kk = 0; kk < kAttnN / 16; ++kk) {
        // 16 keys = two groups of eight rows (2048 bytes); 16 bf16 of P = 8 columns of TMEM
        umma_ts_bf16(o_tmem, p_tmem + kk * 8, v_desc + ((kk * 2048) >> 4), idesc_pv, kk != 0 ? 1u : acc0);
      }
      umma_commit(&o_done[t][j & 1]);
      if (t == kAttnQTiles - 1) umma_commit(&v_empty[s]);
    };
    // K_j / V_j are in shared memory.  Asked ahead of time (the tiles arrive a whole step before they are needed), so that
    // these waits, which cost about 150 cycles even on a completed barrier, stay off the chain P ready -> MMAs issued.
    auto wait_k = [&](int j) -> bool {
#ifdef COMFY_ATTN_EXPERIMENT_NO_LOADS
      if (j >= kAttnStages) return true;
#endif
      return mbar_wait_warp(&k_full[j % kAttnStages], (j / kAttnStages) & 1u, abort_ptr);
    };
    auto wait_v = [&](int j) -> bool {
#ifdef COMFY_ATTN_EXPERIMENT_NO_LOADS
      if (j >= kAttnStages) return true;
#endif
      return mbar_wait_warp(&v_full[j % kAttnStages], (j / kAttnStages) & 1u, abort_ptr);
    };

#ifdef COMFY_ATTN_EXPERIMENT_SOFTMAX_ONLY
    ok = false;                                      // timing experiment only: the tensor pipe stays idle
#endif
    if (ok) ok = wait_k(0);
    if (ok) {
      tc_fence_after_sync();
      if (elect_one()) {
        for (int t = 0; t < kAttnQTiles; ++t) mma_qk(t, 0);
      }
      __syncwarp();
    }
    for (int j = 0; j < n_kv && ok; ++j) {
      ok = wait_v(j) && (j + 1 >= n_kv || wait_k(j + 1));
      for (int t = 0; t < kAttnQTiles && ok; ++t) {
        ATTN_STAMP(2, j, 6 * t);
#ifndef COMFY_ATTN_EXPERIMENT_NO_PWAIT
        ok = mbar_wait_warp(&p_ready[t], j & 1u, abort_ptr);
        if (!ok) break;
#endif
        tc_fence_after_sync();
        ATTN_STAMP(2, j, 6 * t + 1);
        if (elect_one()) {
          mma_pv(t, j);
          if (j + 1 < n_kv) mma_qk(t, j + 1);
        }
        __syncwarp();
        ATTN_STAMP(2, j, 6 * t + 5);
      }
    }
#ifndef COMFY_ATTN_EXPERIMENT_SOFTMAX_ONLY
    if (!ok) give_up();
#endif
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: one query row per thread
    const int t = warp >> 2;                                   // query tile of this warp
    const int row = (warp & 3) * 32 + lane;                    // row inside the tile = TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t o_tmem = lane_base + attn_o_col(t);
    float m_ref = -INFINITY, l_sum = 0.f;                      // m_ref in units of score times scale_log2
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const uint32_t s_tmem = lane_base + attn_s_col(t);
      if ((warp & 3) == 0) ATTN_STAMP(t, j, 0);
#ifndef COMFY_ATTN_EXPERIMENT_SOFTMAX_ONLY
      ok = mbar_wait_warp(&s_full[t], j & 1u, abort_ptr);
      if (!ok) { give_up(); break; }
#endif
      tc_fence_after_sync();
      if ((warp & 3) == 0) ATTN_STAMP(t, j, 1);
      const int valid = p.seq_kv - j * kAttnN;                 // only the last step can hold fewer than 128 keys
      const bool partial = valid < kAttnN;
#ifdef COMFY_ATTN_EXPERIMENT_NO_SOFTMAX
      if (j >= 0) {                                            // timing experiment only: no softmax work at all
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[t]);
        continue;
      }
#endif
      uint32_t pr[64];
      float sum, raw_max;
      if (partial) attn_softmax_step<true>(s_tmem, p.scale_log2, -m_ref, valid, pr, sum, raw_max);
      else attn_softmax_step<false>(s_tmem, p.scale_log2, -m_ref, valid, pr, sum, raw_max);
      // the probabilities above are good unless some row's maximum lies more than the threshold above its reference
      // (always so on the first step); tcgen05.ld / st are warp-wide, so the warp decides together
      const float mx = raw_max * p.scale_log2;
#ifdef COMFY_ATTN_EXPERIMENT_SOFTMAX_ONLY
      const bool raise = mx > 1e30f;                           // timing experiment only: the scores are whatever TMEM held
#else
      const bool raise = mx > m_ref + kAttnRescaleThreshold;
#endif
      if (__any_sync(0xffffffffu, raise)) {
        const float m_new = raise ? mx : m_ref;
        const float factor = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
        if (j > 0) {
          // O holds the sum over steps 0 .. j-1 once the MMAs of step j-1 have finished.  (One barrier per step parity:
          // a parity wait is only sound while the waiter is less than two phases behind.)
          ok = mbar_wait_warp(&o_done[t][(j - 1) & 1], ((j - 1) >> 1) & 1u, abort_ptr);
          if (!ok) { give_up(); break; }
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(o_tmem + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st_32x32b_x32(o_tmem + c * 32, o);
          }
          tmem_st_wait();
        }
        l_sum *= factor;
        m_ref = m_new;
        // the scores are still in TMEM: redo the step against the new reference
        if (partial) attn_softmax_step<true>(s_tmem, p.scale_log2, -m_ref, valid, pr, sum, raw_max);
        else attn_softmax_step<false>(s_tmem, p.scale_log2, -m_ref, valid, pr, sum, raw_max);
      }
      l_sum += sum;
      if ((warp & 3) == 0) ATTN_STAMP(t, j, 2);
      {                                                        // P over the first 64 columns of the scores it came from
        uint32_t half[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < 32; ++i) half[i] = pr[h * 32 + i];
          tmem_st_32x32b_x32(s_tmem + h * 32, half);
        }
      }
      if ((warp & 3) == 0) ATTN_STAMP(t, j, 4);
      tmem_st_wait();                                          // warp-wide: every lane's probabilities are in TMEM
      if ((warp & 3) == 0) ATTN_STAMP(t, j, 5);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
      if ((warp & 3) == 0) ATTN_STAMP(t, j, 3);
    }
#ifndef COMFY_ATTN_EXPERIMENT_SOFTMAX_ONLY
    if (ok) {
      ok = mbar_wait_warp(&o_done[t][(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1u, abort_ptr);
      if (!ok) give_up();
    }
#endif
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.0f / l_sum;
      const int q_row = q_row0 + t * kAttnM + row;
      __nv_bfloat16* o_row = p.out + (static_cast<size_t>(batch) * p.seq_q + q_row) * (static_cast<size_t>(p.heads) * kAttnD) + col0;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(o_tmem + c * 32, o);
        tmem_ld_wait();
        if (q_row < p.seq_q) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
            q.y = pack_bf16x2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
            q.z = pack_bf16x2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
            q.w = pack_bf16x2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
            reinterpret_cast<uint4*>(o_row + c * 32)[i] = q;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_ptr) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);     // copies in flight may still land in shared memory
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kAttnSoftmaxWarps) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kAttnTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn3)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [B][S][H * D] bf16, contiguous; boxes of box_rows rows x 64 elements, 128-byte swizzle, rows past S read as zero.
static int make_attn_map(CUtensorMap* map, const void* base, int64_t batch, int64_t seq, int64_t row_elems, int box_rows) {
  static EncodeTiledFn3 encode = nullptr;
  if (!encode) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return COMFY_MOE_EDEVICE;
    encode = reinterpret_cast<EncodeTiledFn3>(ptr);
  }
  if (!base || !aligned16(base)) return COMFY_MOE_EINVAL;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(row_elems), static_cast<cuuint64_t>(seq), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_elems) * 2, static_cast<cuuint64_t>(row_elems) * seq * 2};
  cuuint32_t box[3] = {64u, static_cast<cuuint32_t>(box_rows), 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? COMFY_MOE_OK : COMFY_MOE_ECUDA;
}

}  // namespace comfy_b200

using namespace comfy_b200;

#ifdef COMFY_ATTN_TRACE
extern "C" int comfy_attn_trace_read(long long* host) {
  return cudaMemcpyFromSymbol(host, attn_trace, sizeof(attn_trace)) == cudaSuccess ? COMFY_MOE_OK : COMFY_MOE_ECUDA;
}
#endif

extern "C" int comfy_attn_forward(const void* q, const void* k, const void* v, int batch, int seq_q, int seq_kv,
                                  int heads, int head_dim, float scale, void* out, int32_t* status, void* stream) {
  if (batch < 0 || seq_q < 0 || seq_kv < 0 || heads <= 0 || !status) return COMFY_MOE_EINVAL;
  if (head_dim != kAttnD) return COMFY_MOE_EUNSUPPORTED;
  if (batch == 0 || seq_q == 0) return COMFY_MOE_OK;
  if (seq_kv == 0 || !q || !k || !v || !out || !aligned16(out)) return COMFY_MOE_EINVAL;
  if (batch > 65535 || heads > 65535) return COMFY_MOE_EUNSUPPORTED;
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return COMFY_MOE_ECUDA;
  if (major != 10) return COMFY_MOE_EDEVICE;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  const int64_t row = static_cast<int64_t>(heads) * kAttnD;
  int rc;
  if ((rc = make_attn_map(&p.map_q, q, batch, seq_q, row, kAttnM)) != COMFY_MOE_OK) return rc;
  if ((rc = make_attn_map(&p.map_k, k, batch, seq_kv, row, kAttnN)) != COMFY_MOE_OK) return rc;
  if ((rc = make_attn_map(&p.map_v, v, batch, seq_kv, row, kAttnN)) != COMFY_MOE_OK) return rc;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = status;
  p.seq_q = seq_q; p.seq_kv = seq_kv; p.heads = heads;
  p.scale_log2 = scale * 1.4426950408889634f;
  constexpr int kMaxDevices = 64;
  static bool configured[kMaxDevices] = {false};
  if (dev < 0 || dev >= kMaxDevices || !configured[dev]) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kAttnSmem)) != cudaSuccess)
      return COMFY_MOE_ECUDA;
    if (dev >= 0 && dev < kMaxDevices) configured[dev] = true;
  }
  dim3 grid((seq_q + kAttnQTiles * kAttnM - 1) / (kAttnQTiles * kAttnM), heads, batch);
  attn_fwd_kernel<<<grid, kAttnThreads, kAttnSmem, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch();
}
