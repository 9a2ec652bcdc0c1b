// Grouped SwiGLU expert GEMM for sm_100a: TMA-fed tcgen05.mma with fp32 accumulators in TMEM.
//
// One persistent kernel, launched twice per layer call:
//   pass 1 (kSwiglu):  h[m, j]  = silu(a[m,:] . w1[j,:]) * (a[m,:] . w3[j,:])
//   pass 2 (plain):    y[m, n]  = h[m,:] . w2[n,:]
// over "groups" = row ranges [row_start[g], row_start[g] + row_count[g]) of the permuted activations,
// each with its own expert's weights (start and count live on the device, so no host sync is needed),
// plus, optionally, the shared expert over the un-permuted rows.  Rows are independent, so a tile may
// hang over the end of its group: the loads read whatever follows, the stores are predicated.
// It replaces the three F.linear calls, F.silu and the product of
// FeedForwardSwiGLU.forward (comfy/ldm/hidream/model.py:238) for all experts at once, and in the
// fp8 variant the clamp / cast / torch._scaled_mm sequence of comfy/ops.py:338-348.
//
// CTA layout (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2-9 = epilogue (TMEM -> registers -> global): two warps per TMEM lane quarter, half of the columns each.
//
// kCtas = 2 (the default): two CTAs on an SM pair form a cluster and share one
// tcgen05.mma.cta_group::2 stream.  A cluster tile is 256 rows x 256 accumulator columns; each CTA
// loads its own 128 rows of A and HALF of the B tile (128 rows), so shared-memory fill traffic and
// L2->SM traffic per flop drop by a third against a single-CTA 128 x 256 tile.  In pass 1 the 256
// accumulator columns are 128 of w1 (loaded by CTA 0) next to the matching 128 of w3 (CTA 1), so one
// MMA stream yields both halves of the SwiGLU and the epilogue emits 128 columns of h.  All loads are
// plain (single-destination) TMA loads; the pair is coordinated with mbarriers only:
//   full[s]        lives in CTA 0; CTA 0's producer arms it with the bytes of both CTAs' loads, both
//                  CTAs' loads complete on it;
//   empty[s]       one per CTA; CTA 0's MMA thread commits to both once a stage has been consumed;
//   tmem_full[a]   one per CTA, committed to by CTA 0's MMA thread when a tile's accumulator is done;
//   tmem_empty[a]  lives in CTA 0; the epilogue warps of both CTAs arrive on it.
// kCtas = 1 is the same code with every pair degenerate (one CTA, 128-row tiles, the CTA loads both B
// boxes itself).
// Shared memory: kStages x (A 16 KB + B 32/kCtas KB), 128-byte swizzle.  TMEM: 2 x 256 columns, so the
// epilogue of tile i overlaps the MMAs of tile i+1.
#include <cuda.h>
#include <memory>

#include "moe_common.cuh"
#include "ptx_sm100.cuh"

namespace comfy_b200 {

constexpr int kBlockM = 128;                      // rows per CTA per tile
constexpr int kBlockN = 256;                      // accumulator columns per tile
constexpr int kRowBytes = 128;                    // bytes of K per operand row per stage
constexpr int kAccStages = 2;
constexpr int kABytes = kBlockM * kRowBytes;      // 16 KB
constexpr int kBBoxBytes = 128 * kRowBytes;       // 16 KB: one 128-row B box
constexpr int kOutStageBytes = 2 * kABytes;      // epilogue staging tile: 128 rows x 256 bytes
constexpr int kEpilogueWarps = 8;                 // two per TMEM lane quarter, each taking half of the columns
constexpr int kGemmThreads = 64 + 32 * kEpilogueWarps;
constexpr int kTmemCols = kAccStages * kBlockN;   // 512
constexpr int kBandTiles = 32;                    // row tiles per band of a row-fastest pass (8192 rows on SM pairs)
constexpr int kMaxGroups = kMaxExperts + 1;
constexpr int kMaxMaps = COMFY_MOE_LINEAR_MAX_MAPS;
static_assert(kMaxMaps >= 4 + 2 * kMaxGroups, "the SwiGLU passes use four activation maps and two weight maps per group");

template <int kCtas> struct GemmShape {
  static constexpr int kTileM = kBlockM * kCtas;
  static constexpr int kBBoxes = 2 / kCtas;                                  // B boxes each CTA loads
  static constexpr int kStageBytes = kABytes + kBBoxes * kBBoxBytes;          // 48 KB or 32 KB
  static constexpr int kStages = kCtas == 1 ? 4 : 6;
  static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + kOutStageBytes + 1024;  // + alignment slack
};

// Device-side status codes written to *status when a bounded wait gives up.
constexpr int kStatusProducerTimeout = 1;
constexpr int kStatusMmaTimeout = 2;
constexpr int kStatusEpilogueTimeout = 3;
constexpr int kStatusArrivalTimeout = 7;          // a source rank's "rows arrived" flag did not come in time

struct GemmGroup {
  int a_map;          // index of the A tensor map
  int b0_map;         // first 128-row B box
  int b1_map;         // second 128-row B box
  int b1_row_off;     // its row offset relative to the first box (0 in pass 1, 128 in pass 2)
  int k_blocks;       // K / (kRowBytes / element size)
  int n_tiles;        // tiles along the output columns
  int routed_index;   // >= 0: rows [row_start[i], row_start[i] + row_count[i]);  < 0: rows [0, static_rows)
  int static_rows;
  int out_map;        // tensor map of the output (TMA stores)
  int reserved;
  void* out;          // output base
  long long ld_out;   // output leading dimension in elements
  const float* scale_a;        // fp8: activation scale (NULL = 1)
  const float* scale_b0;       // fp8: weight scale of the first box
  const float* scale_b1;       // fp8: weight scale of the second box
  const float* out_scale;      // fp8 pass 1: scale_input of w2 (h is multiplied by bf16(1/s) before the cast)
  const __nv_bfloat16* bias;   // kBiasAct instantiations: bias over the output columns (NULL = none)
  int gelu;                    // kBiasAct instantiations: 1 = exact (erf) GELU on the bf16-rounded sum
  int wait_source;             // >= 0: the group's rows come from this rank; its "arrived" flag gates the first load
};

struct alignas(64) GemmParams {
  CUtensorMap maps[kMaxMaps];
  GemmGroup groups[kMaxGroups];
  const int32_t* row_start;
  const int32_t* row_count;
  int32_t* status;
  int num_groups;
  int m_fastest;      // plain passes: 1 = row tiles fastest (short K, wide N), 0 = column tiles fastest
  const int32_t* out_shift;   // optional, device, per routed group: output row = input row + out_shift[i] (results that
                              // are written straight into another buffer's layout, e.g. a peer's return buffer)
  // optional (expert parallelism): arrive_flags[r] reaches arrive_epoch once rank r's rows are in the A operand; a
  // group with wait_source = r is not loaded before that.  Replaces a wait for ALL ranks in front of the launch: the
  // rows this GPU routed to itself are there already, and the tiles over them keep the tensor pipe busy while the
  // other ranks' rows land.
  const uint32_t* arrive_flags;
  uint32_t arrive_epoch;
  int reserved3;
  long long arrive_budget;    // clock budget of one such wait
};

// The SwiGLU epilogue works on pairs of neighbouring columns held as bf16x2, so that every rounding the reference
// performs on its bf16 tensors (after w1 x, after w3 x, after silu, after the product) is one packed conversion or one
// packed multiply for two elements.  silu itself is fp32 math on the rounded value, as PyTorch computes it.
__device__ __forceinline__ float silu_f32(float a) { return __fdividef(a, 1.0f + __expf(-a)); }
__device__ __forceinline__ float bf16x2_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16x2_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  // the fp32 product of two bf16 values is exact, so one rounding here equals "multiply in fp32, round to bf16"
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <bool kFp8, bool kSwiglu, int kCtas, bool kBiasAct = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
  using Shape = GemmShape<kCtas>;
  constexpr int kStages = Shape::kStages;
  constexpr int kStageBytes = Shape::kStageBytes;
  constexpr int kTileM = Shape::kTileM;
  constexpr bool kPair = kCtas == 2;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t tmem_full_bar[kAccStages];
  __shared__ __align__(8) uint64_t tmem_empty_bar[kAccStages];
  __shared__ __align__(8) uint64_t drain_bar;
  __shared__ __align__(8) uint64_t epi_bar;        // the epilogue warps meet here (bounded, unlike bar.sync)
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int s_tile_start[kMaxGroups + 1];
  __shared__ int s_m_tiles[kMaxGroups];
  __shared__ int s_row_base[kMaxGroups];
  __shared__ int s_row_limit[kMaxGroups];
  __shared__ int s_out_shift[kMaxGroups];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;   // 0 = leader of the pair
  const int unit = blockIdx.x / kCtas;                         // index of this CTA (pair) among the workers
  const int n_units = gridDim.x / kCtas;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < kAccStages; ++s) { mbar_init(&tmem_full_bar[s], 1); mbar_init(&tmem_empty_bar[s], kEpilogueWarps * kCtas); }
    mbar_init(&drain_bar, 1);
    mbar_init(&epi_bar, 32 * kEpilogueWarps);
    fence_mbar_init();
    abort_flag = 0;
    int start = 0;
    for (int g = 0; g < p.num_groups; ++g) {
      const GemmGroup& grp = p.groups[g];
      int base, rows, limit;
      if (grp.routed_index >= 0) {
        base = p.row_start[grp.routed_index];
        rows = p.row_count[grp.routed_index];
        if (rows < 0) rows = 0;
        limit = base + rows;
      } else {
        base = 0;
        rows = grp.static_rows;
        limit = rows;
      }
      const int m_tiles = (rows + kTileM - 1) / kTileM;
      s_tile_start[g] = start;
      s_m_tiles[g] = m_tiles;
      s_row_base[g] = base;
      s_row_limit[g] = limit;
      s_out_shift[g] = (p.out_shift && grp.routed_index >= 0) ? p.out_shift[grp.routed_index] : 0;
      start += m_tiles * grp.n_tiles;
    }
    s_tile_start[p.num_groups] = start;
  }
  if (warp == 1) {
    if constexpr (kPair) { tmem_alloc_pair(&tmem_slot, kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(&tmem_slot, kTmemCols); tmem_relinquish(); }
  }
  __syncwarp();
  tc_fence_before_sync();
  if constexpr (kPair) cluster_sync_all();     // the peer's barriers must exist before anything signals them
  else __syncthreads();
  tc_fence_after_sync();

  const uint32_t tmem_base = tmem_slot;
  const int total_tiles = s_tile_start[p.num_groups];
  volatile int* abort_ptr = &abort_flag;

  // Which tiles this CTA (pair) computes, in order.  Tiles are dealt round-robin.  In pass 2 the trailing
  // un-permuted group (the shared expert) has a shorter K than the routed groups, so its tiles cost about half:
  // they are dealt in a second round-robin that first serves the workers that got one routed tile fewer, which
  // evens out the load (12.1 -> 11.6 routed-tile units on the busiest worker for the HiDream shapes).
  int main_tiles = total_tiles;
  if (!kSwiglu && p.num_groups > 1 && p.groups[p.num_groups - 1].routed_index < 0)
    main_tiles = s_tile_start[p.num_groups - 1];
  const int my_main = unit < main_tiles ? (main_tiles - unit + n_units - 1) / n_units : 0;
  const int rr = main_tiles % n_units;                        // workers [0, rr) hold one main tile more
  const int light = n_units - rr;                             // number of workers served by the first partial round
  const int pos = (unit - rr + n_units) % n_units;            // my place in the order rr, rr+1, ..., rr-1
  auto tile_at = [&](int i) -> int {
    if (i < my_main) return unit + i * n_units;
    const int q = i - my_main;
    int j;
    if (pos < light) j = q == 0 ? pos : light + pos + (q - 1) * n_units;
    else j = light + pos + q * n_units;
    const int t = main_tiles + j;
    return t < total_tiles ? t : -1;
  };
  constexpr int kElemsPerRow = kFp8 ? kRowBytes : kRowBytes / 2;   // K elements per stage

  auto decode = [&](int t, int& g, int& m_tile, int& n_tile) {
    g = 0;
    while (t >= s_tile_start[g + 1]) ++g;
    const int local = t - s_tile_start[g];
    if (kSwiglu || p.m_fastest) {
      // pass 1: row tiles fastest inside a band of kBandTiles row tiles.  The CTAs running together share a few
      // weight panels and sweep the band's rows, which stay in L2 (K = dim is short: a band is at most 42 MB)
      // while every weight panel passes once per band.  A group with fewer row tiles than a band (the HiDream
      // shapes at 8192 tokens) is one band: weights read from HBM once.  Without the bands a group of 100 000
      // rows would re-read all of its activations from HBM for every weight panel.
      const int mt = s_m_tiles[g];
      const int per_band = kBandTiles * p.groups[g].n_tiles;
      const int band = local / per_band;
      const int rem = local - band * per_band;
      const int m0 = band * kBandTiles;
      const int in_band = (mt - m0) < kBandTiles ? (mt - m0) : kBandTiles;
      n_tile = rem / in_band;
      m_tile = m0 + (rem - n_tile * in_band);
    } else {
      // pass 2: column tiles fastest.  K = hidden is long, so a row tile of h is 1.7 MB; running all
      // column tiles of a few row tiles together reads every row of h from HBM once while w2 stays in L2.
      const int nt = p.groups[g].n_tiles;
      m_tile = local / nt;
      n_tile = local - m_tile * nt;
    }
  };

  // The producer and MMA warps stay converged: every lane runs the loops and the waits, and the instructions
  // that must come from a single thread are issued under elect.sync.  (Running these loops in one divergent
  // lane costs about 40 extra cycles per MMA and caps the tensor pipe near 78 %; measured.)
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs of a pair)
    uint32_t it = 0;
    bool ok = true;
    uint32_t arrived = 0;           // sources whose flag this warp has already seen at the current epoch
    for (int i = 0, t; (t = tile_at(i)) >= 0 && ok; ++i) {
      int g, m_tile, n_tile;
      decode(t, g, m_tile, n_tile);
      const GemmGroup& grp = p.groups[g];
      if (p.arrive_flags != nullptr && grp.wait_source >= 0 && !((arrived >> grp.wait_source) & 1u)) {
        ok = flag_wait_warp(p.arrive_flags + grp.wait_source, p.arrive_epoch, p.arrive_budget, abort_ptr);
        if (!ok) {
          if (lane == 0) { atomicCAS(p.status, 0, kStatusArrivalTimeout); abort_flag = 1; }
          break;
        }
        arrived |= 1u << grp.wait_source;
        fence_proxy_async_all();    // the rows were written with ordinary stores; the loads below are tensor-map loads
      }
      const CUtensorMap* map_a = &p.maps[grp.a_map];
      const int a_row = s_row_base[g] + m_tile * kTileM + static_cast<int>(cta_rank) * kBlockM;
      const int b_row = n_tile * (kSwiglu ? 128 : kBlockN);
      const int kb_count = grp.k_blocks;
      for (int kb = 0; kb < kb_count; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        ok = mbar_wait_warp(&empty_bar[s], ph ^ 1u, abort_ptr);
        if (!ok) {
          if (lane == 0) { atomicCAS(p.status, 0, kStatusProducerTimeout); abort_flag = 1; }
          break;
        }
        uint8_t* stage = smem + static_cast<size_t>(s) * kStageBytes;
        if (elect_one()) {
          if constexpr (kPair) {
            const uint32_t full_leader = mapa_shared(smem_u32(&full_bar[s]), 0);
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * kStageBytes);
            tma_load_2d_pair(stage, map_a, full_leader, kb * kElemsPerRow, a_row);
            const CUtensorMap* map_b = &p.maps[cta_rank == 0 ? grp.b0_map : grp.b1_map];
            tma_load_2d_pair(stage + kABytes, map_b, full_leader, kb * kElemsPerRow,
                             b_row + (cta_rank == 0 ? 0 : grp.b1_row_off));
          } else {
            mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
            tma_load_2d(stage, map_a, &full_bar[s], kb * kElemsPerRow, a_row);
            tma_load_2d(stage + kABytes, &p.maps[grp.b0_map], &full_bar[s], kb * kElemsPerRow, b_row);
            tma_load_2d(stage + kABytes + kBBoxBytes, &p.maps[grp.b1_map], &full_bar[s], kb * kElemsPerRow,
                        b_row + grp.b1_row_off);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (cta_rank == 0) {
      constexpr uint32_t idesc = umma_idesc<kFp8>(kTileM, kBlockN);
      uint32_t it = 0, tile_count = 0;
      bool ok = true;
      for (int i = 0, t; (t = tile_at(i)) >= 0 && ok; ++i, ++tile_count) {
        int g, m_tile, n_tile;
        decode(t, g, m_tile, n_tile);
        const int kb_count = p.groups[g].k_blocks;
        const uint32_t as = tile_count & 1u;
        const uint32_t aph = (tile_count >> 1) & 1u;
        ok = mbar_wait_warp(&tmem_empty_bar[as], aph ^ 1u, abort_ptr);
        if (!ok) {
          if (lane == 0) { atomicCAS(p.status, 0, kStatusMmaTimeout); abort_flag = 1; }
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * kBlockN;
        for (int kb = 0; kb < kb_count; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          ok = mbar_wait_warp(&full_bar[s], ph, abort_ptr);
          if (!ok) {
            if (lane == 0) { atomicCAS(p.status, 0, kStatusMmaTimeout); abort_flag = 1; }
            break;
          }
          tc_fence_after_sync();
          if (elect_one()) {
            {
              const uint32_t a_addr = smem_u32(smem + static_cast<size_t>(s) * kStageBytes);
              const uint64_t a_desc = umma_desc_k_sw128(a_addr);
              const uint64_t b_desc = umma_desc_k_sw128(a_addr + kABytes);
#pragma unroll
              for (int k = 0; k < kRowBytes / 32; ++k) {
                // every MMA consumes 32 bytes of K per row: advance the start address by 32 B (2 units of 16 B)
                if constexpr (kPair) umma_ss_pair<kFp8>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                else umma_ss<kFp8>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
              }
              // free the stage, in both CTAs, once these MMAs have read it
              if constexpr (kPair) {
                const uint32_t e_local = smem_u32(&empty_bar[s]);
                umma_commit_pair(mapa_shared(e_local, 0));
                umma_commit_pair(mapa_shared(e_local, 1));
              } else {
                umma_commit(&empty_bar[s]);
              }
            }
          }
          __syncwarp();
        }
        if (ok && elect_one()) {
          if constexpr (kPair) {
            const uint32_t f_local = smem_u32(&tmem_full_bar[as]);
            umma_commit_pair(mapa_shared(f_local, 0));
            umma_commit_pair(mapa_shared(f_local, 1));
          } else {
            umma_commit(&tmem_full_bar[as]);
          }
        }
        __syncwarp();
      }
      // make sure nothing issued by this warp is still running before TMEM is released
      if (elect_one()) {
        if constexpr (kPair) umma_commit_pair(mapa_shared(smem_u32(&drain_bar), 0));
        else umma_commit(&drain_bar);
      }
      __syncwarp();
      mbar_wait(&drain_bar, 0, abort_ptr);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps per CTA)
    // TMEM -> registers -> (math) -> swizzled staging tile in shared memory -> TMA store.  Full 128-byte lines
    // leave the SM instead of 16-byte pieces of 32 different rows.  A tile that hangs over the end of its group
    // (its last rows belong to the next group) is written with predicated stores from registers instead.
    const int quarter = warp & 3;   // TMEM lanes this warp may read: [32*quarter, 32*quarter + 32)
    const int col_half = (warp - 2) >> 2;   // which half of the tile's columns this warp converts
    const bool issuer = warp == 2 && lane == 0;
    uint8_t* stage_out = smem + static_cast<size_t>(kStages) * kStageBytes;    // kOutStageBytes, 1024-aligned
    const int r_in_tile = quarter * 32 + lane;
    uint8_t* stage_row = stage_out + r_in_tile * 128;
    const int sw = r_in_tile & 7;
    uint32_t epi_phase = 0;
    bool epi_ok = true;
    // All epilogue threads arrive and wait with the usual clock budget; a warp that gave up elsewhere can
    // therefore never leave the others parked at a hardware barrier.
    auto epi_sync = [&]() {
      mbar_arrive(&epi_bar);
      if (!mbar_wait_warp(&epi_bar, epi_phase, abort_ptr)) epi_ok = false;
      epi_phase ^= 1u;
    };
    uint32_t tile_count = 0;
    for (int i = 0, t; epi_ok && (t = tile_at(i)) >= 0; ++i, ++tile_count) {
      int g, m_tile, n_tile;
      decode(t, g, m_tile, n_tile);
      const GemmGroup& grp = p.groups[g];
      const uint32_t as = tile_count & 1u;
      const uint32_t aph = (tile_count >> 1) & 1u;
      const bool ok = mbar_wait_warp(&tmem_full_bar[as], aph, abort_ptr);
      if (!ok) {
        if (lane == 0) { atomicCAS(p.status, 0, kStatusEpilogueTimeout); abort_flag = 1; }
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * kBlockN;
      const int row_in0 = s_row_base[g] + m_tile * kTileM + static_cast<int>(cta_rank) * kBlockM;
      const bool valid = (row_in0 + r_in_tile < s_row_limit[g]);
      const int row0 = row_in0 + s_out_shift[g];     // where the tile's first row goes in the output
      const int row = row0 + r_in_tile;
      // whole tile inside the group (or clipped by the tensor's own bounds, for the un-permuted group)
      const bool tile_tma = (grp.routed_index < 0 || row_in0 + kBlockM <= s_row_limit[g]);
      const CUtensorMap* map_out = &p.maps[grp.out_map];

      float alpha0 = 1.f, alpha1 = 1.f, out_inv = 1.f;
      uint32_t out_inv2 = 0;
      bool out_scaled = false;
      if constexpr (kFp8) {
        const float sa = grp.scale_a ? __ldg(grp.scale_a) : 1.f;
        alpha0 = sa * (grp.scale_b0 ? __ldg(grp.scale_b0) : 1.f);
        alpha1 = sa * (grp.scale_b1 ? __ldg(grp.scale_b1) : 1.f);
        if (kSwiglu && grp.out_scale) { out_inv = round_bf16(1.0f / __ldg(grp.out_scale)); out_scaled = true; }
        out_inv2 = pack_bf16x2(out_inv, out_inv);
      }

      // hand the accumulator stage back to the MMA warp: called once every TMEM read of the tile has landed in
      // registers, i.e. before the math and the stores, so the next tile's MMAs never wait for them
      auto release_tmem = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kPair) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty_bar[as]), 0));
          else mbar_arrive(&tmem_empty_bar[as]);
        }
      };

      if constexpr (kSwiglu) {
        const int col0 = n_tile * 128;
        const int c_first = 2 * col_half;           // this warp's two chunks of 32 output columns
        uint32_t ra[2][32], rb[2][32];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          tmem_ld_32x32b_x32(taddr + (c_first + i) * 32, ra[i]);
          tmem_ld_32x32b_x32(taddr + 128 + (c_first + i) * 32, rb[i]);
        }
        tmem_ld_wait();
        release_tmem();
        if (tile_tma) {
          if (issuer) bulk_wait_read_all();         // the previous tile's store has finished reading the staging tile
          epi_sync();
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int c = c_first + i;
          uint32_t hp[16];                        // h for columns 2j, 2j+1 of this chunk, bf16x2
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float a0 = __uint_as_float(ra[i][2 * j]), a1 = __uint_as_float(ra[i][2 * j + 1]);
            float b0 = __uint_as_float(rb[i][2 * j]), b1 = __uint_as_float(rb[i][2 * j + 1]);
            if constexpr (kFp8) { a0 *= alpha0; a1 *= alpha0; b0 *= alpha1; b1 *= alpha1; }
            const uint32_t a2 = pack_bf16x2(a0, a1);
            const uint32_t b2 = pack_bf16x2(b0, b1);
            const uint32_t s2 = pack_bf16x2(silu_f32(bf16x2_lo(a2)), silu_f32(bf16x2_hi(a2)));
            hp[j] = mul_bf16x2(s2, b2);
            if constexpr (kFp8) { if (out_scaled) hp[j] = mul_bf16x2(hp[j], out_inv2); }
          }
          if constexpr (kFp8) {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              w[j] = static_cast<uint32_t>(f2_to_e4m3x2(bf16x2_lo(hp[2 * j]), bf16x2_hi(hp[2 * j]))) |
                     (static_cast<uint32_t>(f2_to_e4m3x2(bf16x2_lo(hp[2 * j + 1]), bf16x2_hi(hp[2 * j + 1]))) << 16);
            if (out_scaled) {
              // w2 has a scale_input: the reference casts h * (1 / scale) without a clamp, so what lies beyond the e4m3
              // range is NaN there.  Rare by construction; the saturated bytes are patched only when a value qualifies.
              int ovf = 0;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float lo = bf16x2_lo(hp[j]), hi = bf16x2_hi(hp[j]);
                if (!(fabsf(lo) <= 464.f) || !(fabsf(hi) <= 464.f)) {
                  const uint32_t pair = f2_to_e4m3x2_nosat(lo, hi, ovf);
                  w[j >> 1] = (j & 1) ? ((w[j >> 1] & 0x0000ffffu) | (pair << 16)) : ((w[j >> 1] & 0xffff0000u) | pair);
                }
              }
              if (ovf && valid) atomicAdd(p.status + kStatusE4m3Overflow, ovf);
            }
            if (tile_tma) {
              // one 128-byte row per tile row: this chunk is pieces 2c and 2c+1
              *reinterpret_cast<uint4*>(stage_row + (((2 * c) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
              *reinterpret_cast<uint4*>(stage_row + (((2 * c + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
            } else if (valid) {
              uint8_t* o = static_cast<uint8_t*>(grp.out) + static_cast<long long>(row) * grp.ld_out + col0 + c * 32;
              reinterpret_cast<uint4*>(o)[0] = make_uint4(w[0], w[1], w[2], w[3]);
              reinterpret_cast<uint4*>(o)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          } else {
            uint4 q[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) q[j] = make_uint4(hp[4 * j], hp[4 * j + 1], hp[4 * j + 2], hp[4 * j + 3]);
            if (tile_tma) {
              // two boxes of 64 columns (128 bytes per row each): chunk c is pieces 4(c&1) .. +3 of box c>>1
              uint8_t* box_row = stage_row + (c >> 1) * kABytes;
#pragma unroll
              for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(box_row + ((((c & 1) * 4 + j) ^ sw) << 4)) = q[j];
            } else if (valid) {
              __nv_bfloat16* o = static_cast<__nv_bfloat16*>(grp.out) + static_cast<long long>(row) * grp.ld_out + col0 + c * 32;
#pragma unroll
              for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(o)[j] = q[j];
            }
          }
        }
        if (tile_tma) {
          fence_proxy_async_smem();
          epi_sync();
          if (issuer) {
            tma_store_2d(map_out, stage_out, col0, row0);
            if constexpr (!kFp8) tma_store_2d(map_out, stage_out + kABytes, col0 + 64, row0);
            bulk_commit_group();
          }
        }
      } else {
        const int col0 = n_tile * kBlockN;
        __nv_bfloat16* o_row = static_cast<__nv_bfloat16*>(grp.out) + static_cast<long long>(row) * grp.ld_out + col0;
        // this warp's four chunks of 32 columns: two in each 128-column half of the tile, all read up front
        uint32_t r[4][32];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          tmem_ld_32x32b_x32(taddr + ((i >> 1) * 4 + 2 * col_half + (i & 1)) * 32, r[i]);
        tmem_ld_wait();
        release_tmem();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (tile_tma) {
            if (issuer) bulk_wait_read_all();
            epi_sync();
          }
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const int cc = 2 * col_half + k;      // chunk inside the half
            const int c = half * 4 + cc;          // chunk inside the tile
            const uint32_t* rv = r[half * 2 + k];
            uint4 q[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float v[8];
#pragma unroll
              for (int m = 0; m < 8; ++m) {
                v[m] = __uint_as_float(rv[8 * j + m]);
                if constexpr (kFp8) v[m] *= (half == 0 ? alpha0 : alpha1);
              }
              if constexpr (kBiasAct) {
                // nn.Linear with a bias: the sum is formed in fp32 and rounded once; GELU (exact, erf) is then
                // fp32 math on that bf16 value, rounded once more by the pack below
                if (grp.bias) {
                  float bv[8];
                  unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(grp.bias + col0 + c * 32) + j), bv);
#pragma unroll
                  for (int m = 0; m < 8; ++m) v[m] += bv[m];
                }
                if (grp.gelu) {
#pragma unroll
                  for (int m = 0; m < 8; ++m) {
                    const float t = round_bf16(v[m]);
                    v[m] = 0.5f * t * (1.0f + erff(t * 0.70710678118654752440f));
                  }
                }
              }
              q[j] = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                pack_bf16x2(v[6], v[7]));
            }
            if (tile_tma) {
              uint8_t* box_row = stage_row + (cc >> 1) * kABytes;
#pragma unroll
              for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(box_row + ((((cc & 1) * 4 + j) ^ sw) << 4)) = q[j];
            } else if (valid) {
              __nv_bfloat16* o = o_row + c * 32;
#pragma unroll
              for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(o)[j] = q[j];
            }
          }
          if (tile_tma) {
            fence_proxy_async_smem();
            epi_sync();
            if (issuer) {
              tma_store_2d(map_out, stage_out, col0 + half * 128, row0);
              tma_store_2d(map_out, stage_out + kABytes, col0 + half * 128 + 64, row0);
              bulk_commit_group();
            }
          }
        }
      }
    }
    if (!epi_ok && lane == 0) { atomicCAS(p.status, 0, kStatusEpilogueTimeout); abort_flag = 1; }
    if (issuer) bulk_wait_all();     // stores must have left shared memory (and landed) before the CTA exits
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_ptr) {
    // a wait gave up: give copies still in flight time to land before shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  tc_fence_before_sync();
  if constexpr (kPair) cluster_sync_all();    // neither CTA may leave while its peer can still touch it
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (kPair) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ==================================================================================== host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// [rows, cols] row-major with leading dimension ld (elements); boxes of 128 rows x 128 bytes.
// An encoded map is a pure function of these arguments (it holds the address and the layout, not the data), so the
// maps are remembered per calling thread in a small direct-mapped table: the 48 layers of a model with their ~20 maps
// each are encoded once, not once per call.
struct MapMemo {
  const void* base;
  int64_t rows, cols, ld;
  int fp8;      // -1 = empty
  CUtensorMap map;
};
constexpr int kMapMemoSlots = 2048;

static int make_map(CUtensorMap* map, const void* base, bool fp8, int64_t rows, int64_t cols, int64_t ld) {
  static thread_local std::unique_ptr<MapMemo[]> memo;
  if (!memo) {
    memo.reset(new MapMemo[kMapMemoSlots]);
    for (int i = 0; i < kMapMemoSlots; ++i) memo[i].fp8 = -1;
  }
  uint64_t hsh = reinterpret_cast<uintptr_t>(base) >> 4;
  hsh = (hsh ^ static_cast<uint64_t>(rows) * 0x9e3779b97f4a7c15ull ^ static_cast<uint64_t>(cols) * 0xc2b2ae3d27d4eb4full ^
         static_cast<uint64_t>(ld) * 0x165667b19e3779f9ull ^ (fp8 ? 0x27d4eb2full : 0ull));
  hsh ^= hsh >> 29;
  MapMemo& slot = memo[(hsh * 0x9e3779b97f4a7c15ull) >> 53];   // top 11 bits
  static_assert(kMapMemoSlots == 1 << 11, "slot index takes the top 11 bits of the hash");
  if (slot.fp8 == static_cast<int>(fp8) && slot.base == base && slot.rows == rows && slot.cols == cols && slot.ld == ld) {
    *map = slot.map;
    return COMFY_MOE_OK;
  }
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return COMFY_MOE_EDEVICE;
  const int es = fp8 ? 1 : 2;
  if (!base || !aligned16(base) || rows <= 0 || cols <= 0 || (ld * es) % 16 != 0) return COMFY_MOE_EINVAL;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * es};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kRowBytes / es), 128u};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = encode(map, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                      const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return COMFY_MOE_ECUDA;
  slot.base = base; slot.rows = rows; slot.cols = cols; slot.ld = ld; slot.fp8 = static_cast<int>(fp8);
  slot.map = *map;
  return COMFY_MOE_OK;
}

static int device_sm_count(int* sms) {
  static int cached_dev = -1, cached_sms = 0, cached_major = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return COMFY_MOE_ECUDA;
  if (dev != cached_dev) {
    int n = 0, major = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return COMFY_MOE_ECUDA;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return COMFY_MOE_ECUDA;
    cached_dev = dev; cached_sms = n; cached_major = major;
  }
  if (cached_major != 10) return COMFY_MOE_EDEVICE;
  *sms = cached_sms;
  return COMFY_MOE_OK;
}

// CTAs per tile: SM pairs (cta_group::2) by default; they move a third less data from L2 per flop, which
// under the B200's power cap shows up as higher clocks.  COMFY_B200_GEMM_CTAS=1 selects the single-CTA
// variant of the same kernel (same results) for comparison runs.
static int gemm_ctas() {
  static int ctas = 0;
  if (ctas == 0) {
    const char* env = getenv("COMFY_B200_GEMM_CTAS");
    ctas = (env && env[0] == '1') ? 1 : 2;
  }
  return ctas;
}

template <bool kFp8, bool kSwiglu, int kCtas, bool kBiasAct = false>
static int launch_gemm_impl(const GemmParams& params, int64_t max_tiles, int sms, cudaStream_t stream) {
  auto kernel = grouped_gemm_kernel<kFp8, kSwiglu, kCtas, kBiasAct>;
  constexpr size_t smem = GemmShape<kCtas>::kSmemBytes;
  // the shared-memory opt-in is a per-device property of the kernel
  constexpr int kMaxDevices = 64;
  static bool configured[kMaxDevices] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return COMFY_MOE_ECUDA;
  if (dev < 0 || dev >= kMaxDevices || !configured[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return COMFY_MOE_ECUDA;
    if (dev >= 0 && dev < kMaxDevices) configured[dev] = true;
  }
  int64_t units = sms / kCtas;
  if (max_tiles < units) units = max_tiles;
  if (units <= 0) return COMFY_MOE_OK;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(units * kCtas), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, params) != cudaSuccess) return COMFY_MOE_ECUDA;
  return check_launch();
}

template <bool kFp8, bool kSwiglu, bool kBiasAct = false>
static int launch_gemm(const GemmParams& params, int64_t tiles_single, int64_t tiles_pair, int sms, cudaStream_t stream) {
  if (gemm_ctas() == 1) return launch_gemm_impl<kFp8, kSwiglu, 1, kBiasAct>(params, tiles_single, sms, stream);
  return launch_gemm_impl<kFp8, kSwiglu, 2, kBiasAct>(params, tiles_pair, sms, stream);
}

}  // namespace comfy_b200

using namespace comfy_b200;

// Both passes for n_experts routed groups and the optional un-permuted group.  With `y_out` (one base pointer per
// routed group, any of them possibly another GPU's memory) the second pass writes group i's rows to
// y_out[i] at row (input row + y_row_shift[i]) instead of into y_perm.
static int grouped_swiglu_impl(int w_dtype, int n_experts, const ComfyMoeFfnWeights* h_experts,
                               const ComfyMoeFfnWeights* h_shared, const int32_t* row_start,
                               const int32_t* row_count, int64_t rows_cap, int n_tokens, int dim, const void* x_perm,
                               void* h_perm, void* y_perm, const void* x_shared, void* h_shared_ws, void* y_shared,
                               int32_t* status, void* stream, const ComfyMoeGroupedOptions* opt) {
  void* const* y_out = opt ? opt->y_out : nullptr;
  const int32_t* y_row_shift = opt ? opt->y_row_shift : nullptr;
  const int64_t y_rows_cap = opt ? opt->y_rows_cap : 0;
  const int passes = (opt && opt->passes) ? opt->passes : 3;
  if (passes < 1 || passes > 3) return COMFY_MOE_EINVAL;
  if (opt && opt->arrive_flags && !opt->group_source) return COMFY_MOE_EINVAL;
  if (n_experts < 0 || n_experts > kMaxExperts || dim <= 0 || n_tokens < 0 || rows_cap < 0) return COMFY_MOE_EINVAL;
  if (y_out && (!y_row_shift || y_rows_cap <= 0)) return COMFY_MOE_EINVAL;
  if (y_out && !y_perm) y_perm = y_out[0];     // only its non-nullness is checked below
  if (w_dtype != COMFY_MOE_BF16 && w_dtype != COMFY_MOE_FP8_E4M3) return COMFY_MOE_EUNSUPPORTED;
  if (!status) return COMFY_MOE_EINVAL;
  if (n_experts > 0 && (!h_experts || !row_start || !row_count || !x_perm || !h_perm || !y_perm || rows_cap <= 0))
    return COMFY_MOE_EINVAL;
  const bool has_shared = h_shared != nullptr && n_tokens > 0;
  if (has_shared && (!x_shared || !h_shared_ws || !y_shared)) return COMFY_MOE_EINVAL;
  if (n_experts == 0 && !has_shared) return COMFY_MOE_OK;
  if (dim % kBlockN != 0) return COMFY_MOE_EUNSUPPORTED;
  const bool fp8 = w_dtype == COMFY_MOE_FP8_E4M3;
  const int k_elems = fp8 ? kRowBytes : kRowBytes / 2;
  if (dim % k_elems != 0) return COMFY_MOE_EUNSUPPORTED;

  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != COMFY_MOE_OK) return rc;
  {
    const int limit = h_shared ? h_shared->max_sms : (n_experts > 0 && h_experts ? h_experts[0].max_sms : 0);
    if (limit >= 2 && limit < sms) sms = limit & ~1;
  }

  GemmParams p1, p2;
  memset(&p1, 0, sizeof(p1));
  memset(&p2, 0, sizeof(p2));
  p1.row_start = p2.row_start = row_start;
  p1.row_count = p2.row_count = row_count;
  p1.status = p2.status = status;
  int64_t tiles1[2] = {0, 0}, tiles2[2] = {0, 0};   // upper bounds on tiles, [0] 128-row tiles, [1] 256-row tiles
  int n_maps1 = 0, n_maps2 = 0, g = 0;

  int hidden_routed = 0;
  if (n_experts > 0) {
    hidden_routed = h_experts[0].hidden;
    for (int e = 0; e < n_experts; ++e)
      if (h_experts[e].hidden != hidden_routed) return COMFY_MOE_EUNSUPPORTED;
    if (hidden_routed <= 0 || hidden_routed % 128 != 0 || hidden_routed % k_elems != 0) return COMFY_MOE_EUNSUPPORTED;
    // A operands of the routed groups: the permuted activations and the permuted hidden activations
    if ((rc = make_map(&p1.maps[n_maps1], x_perm, fp8, rows_cap, dim, dim)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[n_maps2], h_perm, fp8, rows_cap, hidden_routed, hidden_routed)) != COMFY_MOE_OK) return rc;
    const int a1 = n_maps1++, a2 = n_maps2++;
    // outputs: pass 1 stores h through the same map pass 2 reads it with; pass 2 stores y_perm
    if ((rc = make_map(&p1.maps[n_maps1], h_perm, fp8, rows_cap, hidden_routed, hidden_routed)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[n_maps2], y_perm, false, y_out ? y_rows_cap : rows_cap, dim, dim)) != COMFY_MOE_OK)
      return rc;
    const int o1 = n_maps1++, o2 = n_maps2++;
    if (y_out) p2.out_shift = y_row_shift;
    // every group may end in a partial tile
    const int64_t m_tiles_cap[2] = {(rows_cap + kBlockM - 1) / kBlockM + n_experts,
                                    (rows_cap + 2 * kBlockM - 1) / (2 * kBlockM) + n_experts};
    for (int e = 0; e < n_experts; ++e, ++g) {
      const ComfyMoeFfnWeights& w = h_experts[e];
      if (!w.w1 || !w.w2 || !w.w3) return COMFY_MOE_EINVAL;
      if ((rc = make_map(&p1.maps[n_maps1], w.w1, fp8, w.hidden, dim, w.ld13)) != COMFY_MOE_OK) return rc;
      if ((rc = make_map(&p1.maps[n_maps1 + 1], w.w3, fp8, w.hidden, dim, w.ld13)) != COMFY_MOE_OK) return rc;
      if ((rc = make_map(&p2.maps[n_maps2], w.w2, fp8, dim, w.hidden, w.ld2)) != COMFY_MOE_OK) return rc;
      GemmGroup& g1 = p1.groups[g];
      g1.a_map = a1; g1.b0_map = n_maps1; g1.b1_map = n_maps1 + 1; g1.b1_row_off = 0;
      g1.k_blocks = dim / k_elems; g1.n_tiles = w.hidden / 128; g1.routed_index = e; g1.static_rows = 0;
      g1.out = h_perm; g1.ld_out = w.hidden; g1.out_map = o1;
      g1.scale_a = w.scale_in13; g1.scale_b0 = w.scale_w1; g1.scale_b1 = w.scale_w3; g1.out_scale = w.scale_in2;
      g1.wait_source = -1;
      if (opt && opt->arrive_flags) {
        const int src = opt->group_source[e];
        if (src >= 32) return COMFY_MOE_EINVAL;
        g1.wait_source = src;
      }
      GemmGroup& g2 = p2.groups[g];
      g2.a_map = a2; g2.b0_map = n_maps2; g2.b1_map = n_maps2; g2.b1_row_off = 128; g2.out_map = o2;
      g2.k_blocks = w.hidden / k_elems; g2.n_tiles = dim / kBlockN; g2.routed_index = e; g2.static_rows = 0;
      g2.out = y_perm; g2.ld_out = dim;
      g2.scale_a = w.scale_in2; g2.scale_b0 = w.scale_w2; g2.scale_b1 = w.scale_w2; g2.out_scale = nullptr;
      n_maps1 += 2; n_maps2 += 1;
      if (y_out) {
        if (!y_out[e]) return COMFY_MOE_EINVAL;
        if ((rc = make_map(&p2.maps[n_maps2], y_out[e], false, y_rows_cap, dim, dim)) != COMFY_MOE_OK) return rc;
        g2.out = y_out[e];
        g2.out_map = n_maps2++;
      }
    }
    for (int v = 0; v < 2; ++v) {
      tiles1[v] += m_tiles_cap[v] * (hidden_routed / 128);
      tiles2[v] += m_tiles_cap[v] * (dim / kBlockN);
    }
  }
  if (has_shared) {
    const ComfyMoeFfnWeights& w = *h_shared;
    if (!w.w1 || !w.w2 || !w.w3) return COMFY_MOE_EINVAL;
    if (w.hidden <= 0 || w.hidden % 128 != 0 || w.hidden % k_elems != 0) return COMFY_MOE_EUNSUPPORTED;
    if ((rc = make_map(&p1.maps[n_maps1], x_shared, fp8, n_tokens, dim, dim)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p1.maps[n_maps1 + 1], w.w1, fp8, w.hidden, dim, w.ld13)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p1.maps[n_maps1 + 2], w.w3, fp8, w.hidden, dim, w.ld13)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[n_maps2], h_shared_ws, fp8, n_tokens, w.hidden, w.hidden)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[n_maps2 + 1], w.w2, fp8, dim, w.hidden, w.ld2)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p1.maps[n_maps1 + 3], h_shared_ws, fp8, n_tokens, w.hidden, w.hidden)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[n_maps2 + 2], y_shared, false, n_tokens, dim, dim)) != COMFY_MOE_OK) return rc;
    GemmGroup& g1 = p1.groups[g];
    g1.a_map = n_maps1; g1.b0_map = n_maps1 + 1; g1.b1_map = n_maps1 + 2; g1.b1_row_off = 0;
    g1.k_blocks = dim / k_elems; g1.n_tiles = w.hidden / 128; g1.routed_index = -1; g1.static_rows = n_tokens;
    g1.out = h_shared_ws; g1.ld_out = w.hidden; g1.out_map = n_maps1 + 3;
    g1.scale_a = w.scale_in13; g1.scale_b0 = w.scale_w1; g1.scale_b1 = w.scale_w3; g1.out_scale = w.scale_in2;
    g1.wait_source = -1;
    GemmGroup& g2 = p2.groups[g];
    g2.a_map = n_maps2; g2.b0_map = n_maps2 + 1; g2.b1_map = n_maps2 + 1; g2.b1_row_off = 128;
    g2.k_blocks = w.hidden / k_elems; g2.n_tiles = dim / kBlockN; g2.routed_index = -1; g2.static_rows = n_tokens;
    g2.out = y_shared; g2.ld_out = dim; g2.out_map = n_maps2 + 2;
    g2.scale_a = w.scale_in2; g2.scale_b0 = w.scale_w2; g2.scale_b1 = w.scale_w2; g2.out_scale = nullptr;
    for (int v = 0; v < 2; ++v) {
      const int64_t tile_m = kBlockM * (v + 1);
      const int64_t m_tiles = (n_tokens + tile_m - 1) / tile_m;
      tiles1[v] += m_tiles * (w.hidden / 128);
      tiles2[v] += m_tiles * (dim / kBlockN);
    }
    ++g;
  }
  p1.num_groups = p2.num_groups = g;
  if (opt && opt->arrive_flags) {
    p1.arrive_flags = opt->arrive_flags;
    p1.arrive_epoch = opt->arrive_epoch;
    p1.arrive_budget = opt->arrive_budget_cycles > 0 ? opt->arrive_budget_cycles : COMFY_MOE_EP_WAIT_CYCLES;
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (passes & 1) {
    rc = fp8 ? launch_gemm<true, true>(p1, tiles1[0], tiles1[1], sms, s)
             : launch_gemm<false, true>(p1, tiles1[0], tiles1[1], sms, s);
    if (rc != COMFY_MOE_OK) return rc;
  }
  if (passes & 2) {
    rc = fp8 ? launch_gemm<true, false>(p2, tiles2[0], tiles2[1], sms, s)
             : launch_gemm<false, false>(p2, tiles2[0], tiles2[1], sms, s);
  }
  return rc;
}

extern "C" int comfy_moe_grouped_swiglu(int w_dtype, int n_experts, const ComfyMoeFfnWeights* h_experts,
                                        const ComfyMoeFfnWeights* h_shared, const int32_t* row_start,
                                        const int32_t* row_count, int64_t rows_cap, int n_tokens, int dim,
                                        const void* x_perm, void* h_perm, void* y_perm, const void* x_shared,
                                        void* h_shared_ws, void* y_shared, int32_t* status, void* stream) {
  return grouped_swiglu_impl(w_dtype, n_experts, h_experts, h_shared, row_start, row_count, rows_cap, n_tokens, dim,
                             x_perm, h_perm, y_perm, x_shared, h_shared_ws, y_shared, status, stream, nullptr);
}

extern "C" int comfy_moe_grouped_swiglu_ex(int w_dtype, int n_groups, const ComfyMoeFfnWeights* h_groups,
                                           const ComfyMoeFfnWeights* h_shared, const int32_t* row_start,
                                           const int32_t* row_count, int64_t rows_cap, int n_tokens, int dim,
                                           const void* x_perm, void* h_perm, void* y_perm, const void* x_shared,
                                           void* h_shared_ws, void* y_shared, const ComfyMoeGroupedOptions* h_options,
                                           int32_t* status, void* stream) {
  return grouped_swiglu_impl(w_dtype, n_groups, h_groups, h_shared, row_start, row_count, rows_cap, n_tokens, dim,
                             x_perm, h_perm, y_perm, x_shared, h_shared_ws, y_shared, status, stream, h_options);
}

extern "C" int comfy_moe_grouped_swiglu_scatter(int w_dtype, int n_groups, const ComfyMoeFfnWeights* h_groups,
                                                const int32_t* row_start, const int32_t* row_count, int64_t rows_cap,
                                                int dim, const void* x_perm, void* h_perm, void* const* h_y_out,
                                                const int32_t* y_row_shift, int64_t y_rows_cap, int32_t* status,
                                                void* stream) {
  if (!h_y_out || n_groups <= 0) return COMFY_MOE_EINVAL;
  ComfyMoeGroupedOptions opt;
  memset(&opt, 0, sizeof(opt));
  opt.y_out = h_y_out;
  opt.y_row_shift = y_row_shift;
  opt.y_rows_cap = y_rows_cap;
  return grouped_swiglu_impl(w_dtype, n_groups, h_groups, nullptr, row_start, row_count, rows_cap, 0, dim, x_perm,
                             h_perm, nullptr, nullptr, nullptr, nullptr, status, stream, &opt);
}

// GELU-MLP experts (Linear + bias, exact GELU, Linear + bias): the feed-forward of the Hunyuan3D-2.1 MoE block
// (comfy/ldm/hunyuan3dv2_1/hunyuandit.py:8-50).  Both launches are plain passes of the same kernel with the
// bias / activation epilogue; the first one walks row tiles fastest because its K (= dim) is short and its N wide.
extern "C" int comfy_moe_grouped_gelu_mlp(int n_experts, const ComfyMoeMlpWeights* h_experts,
                                          const ComfyMoeMlpWeights* h_shared, const int32_t* row_start,
                                          const int32_t* row_count, int64_t rows_cap, int n_tokens, int dim,
                                          const void* x_perm, void* h_perm, void* y_perm, const void* x_shared,
                                          void* h_shared_ws, void* y_shared, int32_t* status, void* stream) {
  if (n_experts < 0 || n_experts > kMaxExperts || dim <= 0 || n_tokens < 0 || rows_cap < 0) return COMFY_MOE_EINVAL;
  if (!status) return COMFY_MOE_EINVAL;
  if (n_experts > 0 && (!h_experts || !row_start || !row_count || !x_perm || !h_perm || !y_perm || rows_cap <= 0))
    return COMFY_MOE_EINVAL;
  const bool has_shared = h_shared != nullptr && n_tokens > 0;
  if (has_shared && (!x_shared || !h_shared_ws || !y_shared)) return COMFY_MOE_EINVAL;
  if (n_experts == 0 && !has_shared) return COMFY_MOE_OK;
  constexpr int k_elems = kRowBytes / 2;
  if (dim % kBlockN != 0) return COMFY_MOE_EUNSUPPORTED;

  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != COMFY_MOE_OK) return rc;

  GemmParams p1, p2;
  memset(&p1, 0, sizeof(p1));
  memset(&p2, 0, sizeof(p2));
  p1.row_start = p2.row_start = row_start;
  p1.row_count = p2.row_count = row_count;
  p1.status = p2.status = status;
  p1.m_fastest = 1;
  int64_t tiles1[2] = {0, 0}, tiles2[2] = {0, 0};
  int n_maps1 = 0, n_maps2 = 0, g = 0;

  auto weights_ok = [&](const ComfyMoeMlpWeights& w) -> int {
    if (!w.w1 || !w.w2) return COMFY_MOE_EINVAL;
    if ((w.b1 && !aligned16(w.b1)) || (w.b2 && !aligned16(w.b2))) return COMFY_MOE_EINVAL;
    if (w.hidden <= 0 || w.hidden % kBlockN != 0) return COMFY_MOE_EUNSUPPORTED;
    return COMFY_MOE_OK;
  };
  auto fill = [&](GemmGroup& g1, GemmGroup& g2, const ComfyMoeMlpWeights& w, int a1, int b1, int o1, int a2, int b2,
                  int o2, int routed_index, int static_rows, void* h_out, void* y_out) {
    g1.a_map = a1; g1.b0_map = b1; g1.b1_map = b1; g1.b1_row_off = 128; g1.out_map = o1;
    g1.k_blocks = dim / k_elems; g1.n_tiles = w.hidden / kBlockN; g1.routed_index = routed_index;
    g1.static_rows = static_rows; g1.out = h_out; g1.ld_out = w.hidden;
    g1.bias = static_cast<const __nv_bfloat16*>(w.b1); g1.gelu = 1;
    g2.a_map = a2; g2.b0_map = b2; g2.b1_map = b2; g2.b1_row_off = 128; g2.out_map = o2;
    g2.k_blocks = w.hidden / k_elems; g2.n_tiles = dim / kBlockN; g2.routed_index = routed_index;
    g2.static_rows = static_rows; g2.out = y_out; g2.ld_out = dim;
    g2.bias = static_cast<const __nv_bfloat16*>(w.b2); g2.gelu = 0;
  };

  if (n_experts > 0) {
    const int hidden = h_experts[0].hidden;
    for (int e = 0; e < n_experts; ++e) {
      if ((rc = weights_ok(h_experts[e])) != COMFY_MOE_OK) return rc;
      if (h_experts[e].hidden != hidden) return COMFY_MOE_EUNSUPPORTED;
    }
    if ((rc = make_map(&p1.maps[0], x_perm, false, rows_cap, dim, dim)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p1.maps[1], h_perm, false, rows_cap, hidden, hidden)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[0], h_perm, false, rows_cap, hidden, hidden)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[1], y_perm, false, rows_cap, dim, dim)) != COMFY_MOE_OK) return rc;
    n_maps1 = n_maps2 = 2;
    const int64_t m_tiles_cap[2] = {(rows_cap + kBlockM - 1) / kBlockM + n_experts,
                                    (rows_cap + 2 * kBlockM - 1) / (2 * kBlockM) + n_experts};
    for (int e = 0; e < n_experts; ++e, ++g) {
      const ComfyMoeMlpWeights& w = h_experts[e];
      if ((rc = make_map(&p1.maps[n_maps1], w.w1, false, w.hidden, dim, w.ld1)) != COMFY_MOE_OK) return rc;
      if ((rc = make_map(&p2.maps[n_maps2], w.w2, false, dim, w.hidden, w.ld2)) != COMFY_MOE_OK) return rc;
      fill(p1.groups[g], p2.groups[g], w, 0, n_maps1, 1, 0, n_maps2, 1, e, 0, h_perm, y_perm);
      ++n_maps1; ++n_maps2;
    }
    for (int v = 0; v < 2; ++v) {
      tiles1[v] += m_tiles_cap[v] * (hidden / kBlockN);
      tiles2[v] += m_tiles_cap[v] * (dim / kBlockN);
    }
  }
  if (has_shared) {
    const ComfyMoeMlpWeights& w = *h_shared;
    if ((rc = weights_ok(w)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p1.maps[n_maps1], x_shared, false, n_tokens, dim, dim)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p1.maps[n_maps1 + 1], w.w1, false, w.hidden, dim, w.ld1)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p1.maps[n_maps1 + 2], h_shared_ws, false, n_tokens, w.hidden, w.hidden)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[n_maps2], h_shared_ws, false, n_tokens, w.hidden, w.hidden)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[n_maps2 + 1], w.w2, false, dim, w.hidden, w.ld2)) != COMFY_MOE_OK) return rc;
    if ((rc = make_map(&p2.maps[n_maps2 + 2], y_shared, false, n_tokens, dim, dim)) != COMFY_MOE_OK) return rc;
    fill(p1.groups[g], p2.groups[g], w, n_maps1, n_maps1 + 1, n_maps1 + 2, n_maps2, n_maps2 + 1, n_maps2 + 2, -1,
         n_tokens, h_shared_ws, y_shared);
    for (int v = 0; v < 2; ++v) {
      const int64_t tile_m = kBlockM * (v + 1);
      const int64_t m_tiles = (n_tokens + tile_m - 1) / tile_m;
      tiles1[v] += m_tiles * (w.hidden / kBlockN);
      tiles2[v] += m_tiles * (dim / kBlockN);
    }
    ++g;
  }
  p1.num_groups = p2.num_groups = g;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if ((rc = launch_gemm<false, false, true>(p1, tiles1[0], tiles1[1], sms, s)) != COMFY_MOE_OK) return rc;
  return launch_gemm<false, false, true>(p2, tiles2[0], tiles2[1], sms, s);
}

// Several bias Linears in one launch: out_g = x_g . w_g^T + b_g for up to kMaxGroups independent (x, w, b, out) sets,
// each a plain pass of the kernel above with the bias epilogue.  Replaces the torch.nn.functional.linear calls behind
// operations.Linear (comfy/ops.py:103-115) where a block runs several of them on the same tokens: the q / k / v
// projections of HiDreamAttention for image and text tokens (comfy/ldm/hidream/model.py:97-119) are six groups of one
// launch, the two output projections (:139-144) two groups of another.
extern "C" int comfy_moe_grouped_linear(int n_groups, const ComfyMoeLinearGroup* h_groups, int32_t* status, void* stream) {
  if (n_groups < 0 || n_groups > kMaxGroups || !status) return COMFY_MOE_EINVAL;
  if (n_groups == 0) return COMFY_MOE_OK;
  if (!h_groups) return COMFY_MOE_EINVAL;
  constexpr int k_elems = kRowBytes / 2;
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != COMFY_MOE_OK) return rc;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.status = status;
  p.m_fastest = 1;            // K is short: sweep the rows under each weight panel
  int64_t tiles[2] = {0, 0};
  int n_maps = 0, g = 0;
  // Operands that several groups share (the tokens under the q, k and v projections, a weight under the per-batch
  // groups of a strided output) get ONE tensor map; GemmParams holds COMFY_MOE_LINEAR_MAX_MAPS of them.
  struct MapKey { const void* base; int64_t rows, cols, ld; };
  MapKey keys[kMaxMaps];
  auto map_for = [&](const void* base, int64_t rows, int64_t cols, int64_t ld, int* index) -> int {
    for (int m = 0; m < n_maps; ++m) {
      if (keys[m].base == base && keys[m].rows == rows && keys[m].cols == cols && keys[m].ld == ld) {
        *index = m;
        return COMFY_MOE_OK;
      }
    }
    if (n_maps >= kMaxMaps) return COMFY_MOE_EUNSUPPORTED;
    const int made = make_map(&p.maps[n_maps], base, false, rows, cols, ld);
    if (made != COMFY_MOE_OK) return made;
    keys[n_maps] = MapKey{base, rows, cols, ld};
    *index = n_maps++;
    return COMFY_MOE_OK;
  };
  for (int i = 0; i < n_groups; ++i) {
    const ComfyMoeLinearGroup& L = h_groups[i];
    if (L.rows < 0 || L.in_features <= 0 || L.out_features <= 0) return COMFY_MOE_EINVAL;
    if (L.rows == 0) continue;
    if (!L.x || !L.w || !L.out) return COMFY_MOE_EINVAL;
    if (L.bias && !aligned16(L.bias)) return COMFY_MOE_EINVAL;
    if (L.out_features % kBlockN != 0 || L.in_features % k_elems != 0) return COMFY_MOE_EUNSUPPORTED;
    int a_map = 0, b_map = 0, o_map = 0;
    if ((rc = map_for(L.x, L.rows, L.in_features, L.ld_x, &a_map)) != COMFY_MOE_OK) return rc;
    if ((rc = map_for(L.w, L.out_features, L.in_features, L.ld_w, &b_map)) != COMFY_MOE_OK) return rc;
    if ((rc = map_for(L.out, L.rows, L.out_features, L.ld_out, &o_map)) != COMFY_MOE_OK) return rc;
    GemmGroup& grp = p.groups[g];
    grp.a_map = a_map; grp.b0_map = b_map; grp.b1_map = b_map; grp.b1_row_off = 128; grp.out_map = o_map;
    grp.k_blocks = L.in_features / k_elems; grp.n_tiles = L.out_features / kBlockN;
    grp.routed_index = -1; grp.static_rows = L.rows;
    grp.out = L.out; grp.ld_out = L.ld_out;
    grp.bias = static_cast<const __nv_bfloat16*>(L.bias); grp.gelu = 0;
    for (int v = 0; v < 2; ++v) {
      const int64_t tile_m = kBlockM * (v + 1);
      tiles[v] += (L.rows + tile_m - 1) / tile_m * grp.n_tiles;
    }
    ++g;
  }
  if (g == 0) return COMFY_MOE_OK;
  p.num_groups = g;
  return launch_gemm<false, false, true>(p, tiles[0], tiles[1], sms, static_cast<cudaStream_t>(stream));
}
