// Quantised / bf16 Linear as a persistent, warp-specialised tcgen05 GEMM.
//
//   out[m,n] = epilogue( sum_k A[m,k] * W[n,k] )      A: [M,K], W: [N,K], K contiguous in both
//
// One CTA per SM walks output tiles of 128 x BLOCK_N - or one CTA pair per two SMs tiles of 256 x 256 with one
// cta_group::2 MMA, each CTA staging 128 rows of A and half of the W rows (no multicast).  Up to two problems
// share a launch (their tile lists are concatenated).  Warp 0 feeds a ring of shared-memory stages with plain TMA
// loads (128-byte swizzle, one 128-byte K-slab per stage), warp 1 issues tcgen05.mma (32 bytes of K per
// instruction) into one of two TMEM accumulators, and eight epilogue warps (two per TMEM lane quadrant, half of the
// tile's columns each) drain the other accumulator with tcgen05.ld and apply the fused epilogue: dequantisation
// scales, bias, per-head RMSNorm + RoPE on q/k columns, GELU / SiLU, gate-residual, routing of column ranges to two
// outputs.  Tiles of 32 rows x 128 bytes (64 bf16 columns, or 128 e4m3 columns for an 8-bit output range) go to TMA
// stores through a swizzled staging slot per warp; per-row epilogue inputs - the residual block, the RoPE factors -
// come into the same slot by TMA loads, so every global access of the epilogue moves whole 128-byte lines.
//
// HBM layout: A and W are row-major with K contiguous, so both operands are
// "K-major" for the tensor core and no transpose or repack is ever needed; the
// FP8/INT8 payload is the plain [N,K] byte matrix produced by the prepack.
#include <mutex>

#include "common.cuh"
#include "dsb.h"

namespace dsb {

constexpr int kBlockM = 128;
constexpr int kSlabBytes = 128;  // bytes of K per stage row (one swizzle row)
constexpr int kGemmThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps

__device__ __forceinline__ uint32_t pack_e4m3x4_sat(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

struct GemmEpilogue {
  const float* row_scale;
  const float* col_scale;
  int col_scale_stride;
  const float* bias;
  int act;
  int act_col0;
  const float* gate;
  int has_resid;
  int split_col;
  int* status;
  // fused per-head QK-RMSNorm + RoPE on the projection's q and k column ranges (nq_w == nullptr: off)
  const float* nq_w;   // [128] weights of the q heads (columns [0, d_model))
  const float* nk_w;   // [128] weights of the k heads (columns [d_model, 2 d_model))
  int has_rope;  // RoPE table (fp16 [rows][64] (cos, sin)) is reached through the problem's staging-load tensor map
  int rope_row0;
  int d_model;
  float norm_eps;
  // e4m3 output (unit scale, saturating) instead of bf16 for the first / second output range: the consumer GEMM then
  // needs no row quantiser.  Only with 256-wide tiles: a warp's two 64-column blocks share one 128-byte staging row.
  int out0_e4m3, out1_e4m3;
};

struct alignas(64) GemmProblem {
  CUtensorMap a, b, o0, o1, r;  // operands, the two output ranges, the residual
  GemmEpilogue ep;
  int M, N, K;
  int tiles_m, num_tiles, num_kb;  // for the tile shape the launch uses
  int tiles_n, panel;              // tiles are walked in panels of `panel` row tiles, see tile_coords
};
// Order in which the persistent CTAs walk a problem's tiles.  Walking all row tiles of one column tile before the next
// column tile re-reads the whole activation matrix once per column tile; when it does not fit the L2 (32760 x 5120 in
// 8 bits = 168 MB) that is tiles_n passes over it from HBM - 9 GB for a 32760 x 5120 -> 13824 projection, which made
// those launches HBM-bound at about 4.4 TB/s.  So the rows are cut into panels of `panel` row tiles whose activations
// (at most ~32 MB) stay in the L2 together with the weight while every column tile of the panel is computed:
// inside a panel the row tile runs fastest.  tl -> (row tile, column tile).
__device__ __forceinline__ void tile_coords(const GemmProblem& P, int tl, int* mt, int* nt) {
  const int per_panel = P.panel * P.tiles_n;
  const int pn = tl / per_panel;
  const int within = tl - pn * per_panel;
  const int rows = min(P.panel, P.tiles_m - pn * P.panel);  // the last panel may be lower
  const int n = within / rows;
  *nt = n;
  *mt = pn * P.panel + (within - n * rows);
}

// Up to two independent problems (same format and tile shape) share one persistent launch: the tile list of the
// second follows the first, so a small problem (the 512-row text stream) fills the SMs its big sibling leaves idle.
struct alignas(64) GemmGroup {
  GemmProblem p[2];
  int count;
};

constexpr int kEpiWarps = 8;               // two per TMEM lane quadrant, each draining half of the tile's columns
constexpr int kStageSlotBytes = 32 * 128;  // 32 rows x 64 bf16
constexpr int kStageBytes = kEpiWarps * kStageSlotBytes;

// CTAS = 1: one CTA computes 128 x BLOCK_N.  CTAS = 2: a CTA pair computes 256 x BLOCK_N with one tcgen05.mma
// (cta_group::2); each CTA stages 128 rows of A and BLOCK_N/2 rows of W, which halves the shared-memory bytes
// per flop (the single-CTA kernel is bound by that traffic) and the L2 reads of W.
template <int BLOCK_N, int CTAS, bool TABLE>
struct GemmSmem {
  static constexpr int kStageA = kBlockM * kSlabBytes;
  static constexpr int kStageB = (BLOCK_N / CTAS) * kSlabBytes;
  static constexpr int kStage = kStageA + kStageB;
  // per epilogue warp: four per-column parameter vectors (scale, bias, gate, head-norm weight) of its BLOCK_N/2 columns
  static constexpr int kParamFloats = 4 * (BLOCK_N / 2);
  static constexpr int kParamBytes = TABLE ? kEpiWarps * kParamFloats * 4 : 0;
  static constexpr int kBarBytes = 256;
  static constexpr int kFixed = kStageBytes + kParamBytes + kBarBytes + 1024;  // + alignment slack
  static constexpr int kStages = (227 * 1024 - kFixed) / kStage;   // 32-KiB stages: 6 (5 with the table); 48-KiB: 4 (3)
  static constexpr int kTotal = kStages * kStage + kFixed;
};

// EPI: which epilogue the launch needs, decided on the host from the problem description.  The generic epilogue tests
// its options at run time inside the per-group code (residual? activation from which column? e4m3 output? a
// normalised head?); those warp-uniform branches and the code they guard cost the drain of a tile about 15 % at
// K = 3072 (4096 x 3072 -> 12288 with GELU and e4m3 output: 134 -> 114 us with the options fixed at compile time),
// so the common cases are instantiated with their options as constants.
enum : int {
  EPI_GENERIC = 0,  // everything decided at run time (split outputs, activation on a column range, other activations)
  EPI_PLAIN = 1,    // scales + bias, bf16 out
  EPI_RESID = 2,    // ... + gate * (.) + residual, bf16 out
  EPI_GELU = 3,     // ... + GELU-tanh on every column, bf16 out
  EPI_GELU8 = 4,    // ... + GELU-tanh on every column, e4m3 out (unit scale)
  EPI_NORM = 5,     // per-head RMSNorm (+ RoPE) on the q and k columns, bf16 out, nothing else
  EPI_NORM_GELU8 = 6,  // ... and GELU-tanh from act_col0 on, those columns (second output) as e4m3: q|k|v|mlp projection
};

template <int KIND, int BLOCK_N, int CTAS, bool TABLE, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_kernel(const __grid_constant__ GemmGroup g) {
  using SM = GemmSmem<BLOCK_N, CTAS, TABLE>;
  constexpr int kStages = SM::kStages;
  constexpr int kElemBytes = (KIND == KIND_F16) ? 2 : 1;
  constexpr int kSlabElems = kSlabBytes / kElemBytes;
  constexpr uint32_t kTmemCols = 2 * BLOCK_N;
  constexpr int kTileM = kBlockM * CTAS;  // rows of one scheduled tile (both CTAs of a pair)
  constexpr uint32_t kIdesc =
      (KIND == KIND_F16)  ? make_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 0, 0, kTileM, BLOCK_N)
      : (KIND == KIND_F8) ? make_idesc(DFMT_F32, FMT_E4M3, FMT_E4M3, 0, 0, kTileM, BLOCK_N)
                          : make_idesc(DFMT_S32, FMT_S8, FMT_S8, 0, 0, kTileM, BLOCK_N);
  const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int unit = blockIdx.x / CTAS;        // which CTA (pair) of the persistent grid
  const int num_units = gridDim.x / CTAS;

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows = 1024 bytes.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem + kStages * SM::kStage;  // 1024-aligned: stages are multiples of 16 KiB
  float* param_base = reinterpret_cast<float*>(stage_base + kStageBytes);
  uint8_t* bar_base = stage_base + kStageBytes + SM::kParamBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* resid_bar = tmem_empty + 2;  // kEpiWarps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(resid_bar + kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], CTAS * kEpiWarps * 32);
    }
    for (int i = 0; i < kEpiWarps; ++i) mbar_init(&resid_bar[i], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&g.p[0].a);
    tma_prefetch_desc(&g.p[0].b);
    tma_prefetch_desc(&g.p[0].o0);
  }
  if (warp == 1) {
    if constexpr (CTAS == 2) {
      tmem_alloc_cg2(tmem_slot, kTmemCols);
      tmem_relinquish_cg2();
    } else {
      tmem_alloc(tmem_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // the peer's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_first = g.p[0].num_tiles;
  const int num_tiles = tiles_first + (g.count > 1 ? g.p[1].num_tiles : 0);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = unit; t < num_tiles; t += num_units) {
        const GemmProblem& P = g.p[t >= tiles_first ? 1 : 0];
        const int tl = t >= tiles_first ? t - tiles_first : t;
        int mt, nt;
        tile_coords(P, tl, &mt, &nt);
        const int m0 = mt * kTileM + static_cast<int>(cta_rank) * kBlockM;
        const int n0 = nt * BLOCK_N + static_cast<int>(cta_rank) * (BLOCK_N / CTAS);
        const int num_kb = P.num_kb;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) goto producer_done;
          uint8_t* sa = smem + stage * SM::kStage;
          uint8_t* sb = sa + SM::kStageA;
          if constexpr (CTAS == 2) {
            // both CTAs' bytes are counted on the leader's barrier, which the leader arms for the pair
            if (leader) mbar_expect_tx(&full_bar[stage], 2 * SM::kStage);
            const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);
            tma_load_2d_cg2(sa, &P.a, bar, kb * kSlabElems, m0);
            tma_load_2d_cg2(sb, &P.b, bar, kb * kSlabElems, n0);
          } else {
            mbar_expect_tx(&full_bar[stage], SM::kStage);
            tma_load_2d(sa, &P.a, &full_bar[stage], kb * kSlabElems, m0);
            tma_load_2d(sb, &P.b, &full_bar[stage], kb * kSlabElems, n0);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  producer_done:;
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (leader) {
      // the whole warp runs the loop (descriptors stay warp-uniform); one elected lane issues
      const uint32_t el = elect_one();
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = unit; t < num_tiles; t += num_units, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag)) goto mma_done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        const int num_kb = g.p[t >= tiles_first ? 1 : 0].num_kb;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_spin(&full_bar[stage], phase, abort_flag)) goto mma_done;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * SM::kStage);
          const uint64_t adesc = make_desc_k_sw128(sa);
          const uint64_t bdesc = make_desc_k_sw128(sa + SM::kStageA);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // advancing 32 bytes along K inside the swizzle row = +2 in the (addr >> 4) field
            mma_ss_elect<KIND, CTAS>(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc, (kb | k) != 0 ? 1u : 0u, el);
          }
          if constexpr (CTAS == 2) {  // the stage is free in both CTAs once these MMAs have read it
            tc_commit_cg2_elect(smem_u32(&empty_bar[stage]), el);
            tc_commit_cg2_elect(mapa_u32(smem_u32(&empty_bar[stage]), 1), el);
          } else {
            tc_commit_elect(&empty_bar[stage], el);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if constexpr (CTAS == 2) {
          tc_commit_cg2_elect(smem_u32(&tmem_full[acc]), el);
          tc_commit_cg2_elect(mapa_u32(smem_u32(&tmem_full[acc]), 1), el);
        } else {
          tc_commit_elect(&tmem_full[acc], el);
        }
      }
    }
  mma_done:;
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int ew = warp - 2;
    const int half = ew >> 2;  // which half of the tile's 64-column blocks this warp drains
    uint8_t* sbuf = stage_base + ew * kStageSlotBytes;
    float* ptab = param_base + ew * SM::kParamFloats;
    uint64_t* rbar = resid_bar + ew;
    uint32_t rphase = 0;
    constexpr int kBlocksPerWarp = BLOCK_N / 64 / 2;
    const uint32_t row_off = static_cast<uint32_t>(lane) * 128u;
    const uint32_t sw = static_cast<uint32_t>(lane & 7);
    int it = 0;
    for (int t = unit; t < num_tiles; t += num_units, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const GemmProblem& P = g.p[t >= tiles_first ? 1 : 0];
      const GemmEpilogue& ep = P.ep;
      const int M = P.M, N = P.N;
      const int tl = t >= tiles_first ? t - tiles_first : t;
      int mt, nt;
      tile_coords(P, tl, &mt, &nt);
      const int m0 = mt * kTileM + static_cast<int>(cta_rank) * kBlockM;
      const int n0 = nt * BLOCK_N;
      const int r0 = m0 + quad * 32;
      const int m = r0 + lane;
      // Fused QK-RMSNorm (+RoPE): with 256-wide tiles this warp's 128 columns are exactly one head, one row per
      // thread, so the row's sum of squares needs no cross-thread traffic - just a first pass over TMEM.
      const int head_col0 = n0 + half * 128;
      constexpr bool kAnyNorm = (EPI == EPI_GENERIC || EPI == EPI_NORM || EPI == EPI_NORM_GELU8) && BLOCK_N == 256;
      const bool fuse_norm = kAnyNorm && ep.nq_w != nullptr && head_col0 < 2 * ep.d_model && head_col0 < N;
      const bool rope_tile = fuse_norm && ep.has_rope;
      const bool has_resid = (EPI == EPI_GENERIC) ? (ep.has_resid != 0) : (EPI == EPI_RESID);
      // The tile-shaped epilogue input of this warp's FIRST 64-column block (residual rows, or RoPE factors) does not
      // depend on the accumulator: request it before waiting for the MMAs, so its L2 round trip runs under them.
      // The staging slot must first have been read out by the previous tile's store.
      const int pre_nb = n0 + half * kBlocksPerWarp * 64;
      const bool pre_issued = (has_resid || rope_tile) && pre_nb < N;
      if (pre_issued) {
        if (lane == 0) {
          bulk_wait_read<0>();
          mbar_expect_tx(rbar, kStageSlotBytes);
          if (rope_tile)
            tma_load_2d(sbuf, &P.r, rbar, pre_nb - head_col0, ep.rope_row0 + r0);
          else
            tma_load_2d(sbuf, &P.r, rbar, pre_nb, r0);
        }
        __syncwarp();
      }
      // Per-column epilogue parameters (per-channel scale, bias, gate, head-norm weight) of this warp's column range:
      // lane l fetches kPer consecutive columns' values once per tile, before the accumulator is ready.  (Loading
      // them group by group from global memory, right where they are used, cost a serial L2 round trip per group.)
      // TABLE: they go into the warp's own table in shared memory and the 8-column groups below read theirs back as
      // two 16-byte broadcasts per vector.  Otherwise they stay in registers and are handed round by warp shuffles:
      // 8 shuffles per vector and group, and the shuffle unit issues one per cycle for the whole SM - measured 5-8 %
      // of the whole GEMM at K = 3072, where the epilogue is the longer half of the pipeline; at K >= 5120 the mainloop
      // is, and the sixth operand stage the table's 16 KiB would displace is worth more (1-7 %).
      constexpr int kWarpCols = BLOCK_N / 2, kPer = kWarpCols / 32;
      constexpr bool kNeedGate = EPI == EPI_GENERIC || EPI == EPI_RESID;
      const int wcol0 = n0 + half * kWarpCols;
      float p_cs[kPer], p_bias[kPer], p_gate[kPer], p_hw[kPer];
      {
        const int c = wcol0 + lane * kPer;
        const bool in = c < N;
        const bool chan = ep.col_scale && ep.col_scale_stride;
        const float* hw = (wcol0 < ep.d_model) ? ep.nq_w : ep.nk_w;
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          p_cs[j] = (in && chan) ? __ldg(ep.col_scale + c + j) : 1.f;
          p_bias[j] = (in && ep.bias) ? __ldg(ep.bias + c + j) : 0.f;
          p_gate[j] = (kNeedGate && in && ep.gate) ? __ldg(ep.gate + c + j) : 1.f;
          p_hw[j] = (fuse_norm && hw) ? __ldg(hw + ((lane * kPer + j) & 127)) : 1.f;
        }
        if constexpr (TABLE) {
          __syncwarp();  // every lane has read the previous tile's values
#pragma unroll
          for (int j = 0; j < kPer; ++j) {
            ptab[0 * kWarpCols + lane * kPer + j] = p_cs[j];
            ptab[1 * kWarpCols + lane * kPer + j] = p_bias[j];
            if constexpr (kNeedGate) ptab[2 * kWarpCols + lane * kPer + j] = p_gate[j];
            if constexpr (kAnyNorm) ptab[3 * kWarpCols + lane * kPer + j] = p_hw[j];
          }
          __syncwarp();
        }
      }
      // the 8 values of vector `which` (0 scale, 1 bias, 2 gate, 3 norm weight) for the column group that starts at
      // column c8 (a multiple of 8) of the warp's range
      auto pick8 = [&](int which, int c8, float (&out)[8]) {
        if constexpr (TABLE) {
          const float4 lo = *reinterpret_cast<const float4*>(ptab + which * kWarpCols + c8);
          const float4 hi = *reinterpret_cast<const float4*>(ptab + which * kWarpCols + c8 + 4);
          out[0] = lo.x, out[1] = lo.y, out[2] = lo.z, out[3] = lo.w;
          out[4] = hi.x, out[5] = hi.y, out[6] = hi.z, out[7] = hi.w;
        } else {
          const float(&mine)[kPer] = which == 0 ? p_cs : which == 1 ? p_bias : which == 2 ? p_gate : p_hw;
#pragma unroll
          for (int j = 0; j < 8; ++j) out[j] = __shfl_sync(0xffffffffu, mine[j % kPer], c8 / kPer + j / kPer);
        }
      };
      // the row's activation scale is fetched before the wait as well
      const float rs = (ep.row_scale && m < M) ? __ldg(ep.row_scale + m) : 1.0f;
      const float rs_t = (ep.col_scale && !ep.col_scale_stride) ? rs * __ldg(ep.col_scale) : rs;  // per-tensor scale folded in
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      const bool second = n0 >= ep.split_col;
      const CUtensorMap* tmap_out = second ? &P.o1 : &P.o0;
      const bool out8 = (BLOCK_N == 256) && (EPI == EPI_GENERIC      ? ((second ? ep.out1_e4m3 : ep.out0_e4m3) != 0)
                                             : EPI == EPI_NORM_GELU8 ? second
                                                                     : (EPI == EPI_GELU8));
      const int col_shift = second ? ep.split_col : 0;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BLOCK_N;
      float rnorm = 1.0f;
      if (fuse_norm) {
        float ss = 0.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + half * 128 + c * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float cs8[8], b8[8];
            pick8(0, c * 32 + g * 8, cs8);
            pick8(1, c * 32 + g * 8, b8);
#pragma unroll
            for (int j = 0; j < 8; ++j) cs8[j] *= rs_t;   // rs_t = row scale x per-tensor scale (1 if per-channel)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float a;
              if constexpr (KIND == KIND_I8)
                a = static_cast<float>(static_cast<int>(r[g * 8 + j]));
              else
                a = __uint_as_float(r[g * 8 + j]);
              const float v = fmaf(a, cs8[j], b8[j]);
              ss = fmaf(v, v, ss);
            }
          }
        }
        rnorm = rsqrtf(ss * (1.0f / 128.0f) + ep.norm_eps);
      }
      bool alive = true;
#pragma unroll 1
      for (int cb = half * kBlocksPerWarp; cb < (half + 1) * kBlocksPerWarp && alive; ++cb) {
        const int nb = n0 + cb * 64;
        if (nb >= N) break;  // uniform across the warp
        // this warp's previous store must have read the staging slot out (an e4m3 tile fills the slot with both of
        // the warp's blocks, 64 bytes per row each, before it is stored)
        const int cb_local = cb - half * kBlocksPerWarp;
        if (!(out8 && cb_local > 0)) {
          if (lane == 0) bulk_wait_read<0>();
          __syncwarp();
        }
        // Tile-shaped epilogue input, fetched by TMA into this warp's staging slot (32 rows x 128 bytes, the slot the
        // output block is then written over cell by cell): the residual block, or for a normalised head the RoPE
        // factors of these rows - 32 pairs of fp16 (cos, sin) are the same 128 bytes per row as 64 bf16 outputs.
        const bool do_rope = rope_tile;
        if (has_resid || do_rope) {
          if (lane == 0 && !(pre_issued && nb == pre_nb)) {  // the first block's input is already on its way
            mbar_expect_tx(rbar, kStageSlotBytes);
            if (do_rope)
              tma_load_2d(sbuf, &P.r, rbar, nb - head_col0, ep.rope_row0 + r0);
            else
              tma_load_2d(sbuf, &P.r, rbar, nb, r0);
          }
          if (!mbar_wait(rbar, rphase, abort_flag)) {
            alive = false;
            break;
          }
          rphase ^= 1u;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int nc = nb + h * 32;
          uint32_t r[32];
          tmem_ld32(t_row + cb * 64 + h * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int n = nc + g * 8;
            uint8_t* cell = sbuf + row_off + (((static_cast<uint32_t>(h * 4 + g)) ^ sw) << 4);
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if constexpr (KIND == KIND_I8)
                v[j] = static_cast<float>(static_cast<int>(r[g * 8 + j]));
              else
                v[j] = __uint_as_float(r[g * 8 + j]);
            }
            if (n < N) {
              const int c8 = cb_local * 64 + h * 32 + g * 8;   // first column of the group inside the warp's range
              {
                float cs8[8], b8[8];
                pick8(0, c8, cs8);
                pick8(1, c8, b8);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = fmaf(v[j], cs8[j] * rs_t, b8[j]);
              }
              if (fuse_norm) {
                float w8[8];
                pick8(3, c8, w8);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= rnorm * w8[j];
                if (do_rope) {
                  const uint4 cs4 = *reinterpret_cast<const uint4*>(cell);  // (cos, sin) of the four pairs, fp16
                  const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&cs4.x));
                  const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&cs4.y));
                  const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&cs4.z));
                  const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&cs4.w));
                  float t0 = f0.x * v[0] - f0.y * v[1], t1 = f0.y * v[0] + f0.x * v[1];
                  v[0] = t0, v[1] = t1;
                  t0 = f1.x * v[2] - f1.y * v[3], t1 = f1.y * v[2] + f1.x * v[3];
                  v[2] = t0, v[3] = t1;
                  t0 = f2.x * v[4] - f2.y * v[5], t1 = f2.y * v[4] + f2.x * v[5];
                  v[4] = t0, v[5] = t1;
                  t0 = f3.x * v[6] - f3.y * v[7], t1 = f3.y * v[6] + f3.x * v[7];
                  v[6] = t0, v[7] = t1;
                }
              }
              if constexpr (EPI == EPI_GELU || EPI == EPI_GELU8) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
              } else if constexpr (EPI == EPI_NORM_GELU8) {
                if (n >= ep.act_col0) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
                }
              } else if constexpr (EPI == EPI_GENERIC) {
                if (ep.act != DSB_ACT_NONE && n >= ep.act_col0) {
                  if (ep.act == DSB_ACT_GELU_TANH) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
                  } else if (ep.act == DSB_ACT_SILU) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = silu(v[j]);
                  } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = gelu_erf(v[j]);
                  }
                }
              }
              if (has_resid) {
                const uint4 rr = *reinterpret_cast<const uint4*>(cell);
                const uint32_t ru[4] = {rr.x, rr.y, rr.z, rr.w};
                float gte[8];
                pick8(2, c8, gte);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = unpack_bf16x2(ru[j]);
                  v[2 * j] = f.x + gte[2 * j] * v[2 * j];
                  v[2 * j + 1] = f.y + gte[2 * j + 1] * v[2 * j + 1];
                }
              }
            }
            if (out8) {
              // eight e4m3 values = half a 16-byte chunk of the 128-byte row that holds the warp's 128 columns
              uint8_t* cell8 = sbuf + row_off + (((static_cast<uint32_t>(cb_local * 4 + h * 2 + (g >> 1))) ^ sw) << 4) +
                               (g & 1) * 8;
              uint2 o8;
              o8.x = pack_e4m3x4_sat(v[0], v[1], v[2], v[3]);
              o8.y = pack_e4m3x4_sat(v[4], v[5], v[6], v[7]);
              *reinterpret_cast<uint2*>(cell8) = o8;
            } else {
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]);
              o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]);
              o.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(cell) = o;
            }
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          if (!out8) {
            tma_store_2d(tmap_out, sbuf, nb - col_shift, r0);
            bulk_commit();
          } else if (cb_local + 1 == kBlocksPerWarp || nb + 64 >= N) {
            tma_store_2d(tmap_out, sbuf, n0 + half * 128 - col_shift, r0);
            bulk_commit();
          }
        }
      }
      tc_fence_before();
      if constexpr (CTAS == 2) {  // the leader's MMA thread waits for the epilogues of both CTAs
        if (leader) mbar_arrive(&tmem_empty[acc]);
        else mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
      } else {
        mbar_arrive(&tmem_empty[acc]);
      }
      if (!alive) break;
    }
    if (lane == 0) bulk_wait<0>();  // every store of this warp has left shared memory and been written
  }

  // Common exit: on the abort path give copies still in flight time to land
  // before shared memory and TMEM go back to the SM.
  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // neither CTA leaves (or frees TMEM) while its peer may still use it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (CTAS == 2) tmem_dealloc_cg2(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && g.p[0].ep.status) atomicCAS(g.p[0].ep.status, 0, DSB_ERR_TIMEOUT);
}

template <int KIND, int BLOCK_N, int CTAS, bool TABLE, int EPI>
static int launch_group(GemmGroup& grp, cudaStream_t st) {
  using SM = GemmSmem<BLOCK_N, CTAS, TABLE>;
  auto kern = gemm_kernel<KIND, BLOCK_N, CTAS, TABLE, EPI>;
  DSB_ENSURE_SMEM(kern, SM::kTotal);
  int tiles = 0;
  for (int i = 0; i < grp.count; ++i) tiles += grp.p[i].num_tiles;
  if constexpr (CTAS == 1) {
    const int grid = tiles < sm_count() ? tiles : sm_count();
    kern<<<grid, kGemmThreads, SM::kTotal, st>>>(grp);
  } else {
    // persistent grid = the CTA pairs the device can hold at once (GPCs with an odd SM count leave one SM out)
    static int resident_pairs[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DSB_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = SM::kTotal;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (resident_pairs[dev] == 0) {
      cfg.gridDim = dim3(sm_count() & ~1, 1, 1);
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = sm_count() / 2;
      resident_pairs[dev] = n;
    }
    const int units = resident_pairs[dev];
    cfg.gridDim = dim3((tiles < units ? tiles : units) * CTAS, 1, 1);
    cfg.stream = st;
    if (cudaLaunchKernelEx(&cfg, kern, grp) != cudaSuccess) return DSB_ERR_CUDA;
  }
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

// Tile width: 256 columns unless that leaves SMs idle that 128-wide tiles would fill.
static int pick_block_n(int M, int N) {
  const int tm = (M + kBlockM - 1) / kBlockM;
  const int t256 = tm * ((N + 255) / 256);
  const int t128 = tm * ((N + 127) / 128);
  const int sms = sm_count();
  if (N <= 128) return 128;
  if (t256 >= sms) {
    // compare the waves each choice needs, counting a 128-wide tile as half the work
    const double w256 = static_cast<double>((t256 + sms - 1) / sms);
    const double w128 = 0.5 * static_cast<double>((t128 + sms - 1) / sms);
    return (w128 < w256 * 0.92) ? 128 : 256;
  }
  return 128;
}

}  // namespace dsb

using namespace dsb;

// Validates one problem and fills everything of it that does not depend on the tile shape.
static int check_problem(const dsb_gemm_args& a, int fmt, int* status, GemmProblem* P) {
  if (a.M < 0 || a.N < 0 || a.K <= 0 || (a.N & 7)) return DSB_ERR_ARG;
  if (a.M == 0 || a.N == 0) return DSB_OK;
  if (!a.A || !a.W || !a.out0) return DSB_ERR_ARG;
  const int esz = (fmt == DSB_FMT_BF16) ? 2 : 1;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al16(a.A) || !al16(a.W) || !al16(a.out0) || (a.out1 && !al16(a.out1)) || (a.resid && !al16(a.resid)) ||
      (a.bias && !al16(a.bias)) || (a.gate && !al16(a.gate)) ||
      (a.col_scale && a.col_scale_stride && !al16(a.col_scale)))
    return DSB_ERR_ARG;
  if (((a.lda * esz) & 15) || ((a.ldw * esz) & 15) || (a.ld_out0 & 7) || (a.ld_resid & 7) || (a.ld_out1 & 7))
    return DSB_ERR_ARG;
  if (a.col_scale_stride != 0 && a.col_scale_stride != 1) return DSB_ERR_ARG;
  if (a.act < DSB_ACT_NONE || a.act > DSB_ACT_GELU) return DSB_ERR_ARG;
  int split_col = a.split_col;
  if (!a.out1) split_col = INT32_MAX;
  else if (split_col < 0 || (split_col % 256) != 0) return DSB_ERR_ARG;
  if (a.gate && !a.resid) return DSB_ERR_ARG;
  const bool o0_8 = a.out0_fmt == DSB_FMT_E4M3, o1_8 = a.out1 && a.out1_fmt == DSB_FMT_E4M3;
  if ((a.out0_fmt != DSB_FMT_BF16 && !o0_8) || (a.out1 && a.out1_fmt != DSB_FMT_BF16 && !o1_8)) return DSB_ERR_ARG;
  if ((o0_8 || o1_8) && a.resid) return DSB_ERR_ARG;                      // the residual form writes bf16
  if (o0_8 && (a.nq_w || (a.ld_out0 & 15))) return DSB_ERR_ARG;           // normalised heads stay bf16
  if (o1_8 && (a.ld_out1 & 15)) return DSB_ERR_ARG;
  if (a.resid && a.out1) return DSB_ERR_ARG;  // the residual form writes one output
  if (a.nq_w) {
    if (!a.nk_w || a.d_model <= 0 || (a.d_model % 128) || 2 * a.d_model > a.N || a.resid || !al16(a.nq_w) ||
        !al16(a.nk_w) || (a.rope && !al16(a.rope)))
      return DSB_ERR_ARG;
  }
  GemmEpilogue& ep = P->ep;
  ep.row_scale = a.row_scale;
  ep.col_scale = a.col_scale;
  ep.col_scale_stride = a.col_scale_stride;
  ep.bias = a.bias;
  ep.act = a.act;
  ep.act_col0 = a.act_col0;
  ep.gate = a.gate;
  ep.has_resid = a.resid ? 1 : 0;
  ep.split_col = split_col;
  ep.status = status;
  ep.nq_w = a.nq_w;
  ep.nk_w = a.nk_w;
  ep.has_rope = (a.nq_w && a.rope) ? 1 : 0;
  ep.rope_row0 = a.rope_row0;
  ep.d_model = a.d_model;
  ep.norm_eps = a.norm_eps;
  ep.out0_e4m3 = o0_8 ? 1 : 0;
  ep.out1_e4m3 = o1_8 ? 1 : 0;
  P->M = a.M, P->N = a.N, P->K = a.K;
  // bf16 output / residual tiles of 32 rows x 64 columns (128 bytes per row, 128-byte swizzle)
  const int n0cols = a.out1 ? (split_col < a.N ? split_col : a.N) : a.N;
  // bf16 ranges: blocks of 32 rows x 64 columns; e4m3 ranges: 32 rows x 128 columns (128 bytes per row either way)
  if ((o0_8 ? make_tmap_2d(&P->o0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.out0, a.M, n0cols, a.ld_out0, 32, 128)
            : make_tmap_2d(&P->o0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.out0, a.M, n0cols, a.ld_out0 * 2, 32, 64)) !=
      DSB_OK)
    return DSB_ERR_CUDA;
  P->o1 = P->o0;
  if (a.out1 && split_col < a.N &&
      (o1_8 ? make_tmap_2d(&P->o1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.out1, a.M, a.N - split_col, a.ld_out1, 32, 128)
            : make_tmap_2d(&P->o1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.out1, a.M, a.N - split_col, a.ld_out1 * 2, 32,
                           64)) != DSB_OK)
    return DSB_ERR_CUDA;
  P->r = P->o0;
  if (a.resid &&
      make_tmap_2d(&P->r, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.resid, a.M, a.N, a.ld_resid * 2, 32, 64) != DSB_OK)
    return DSB_ERR_CUDA;
  // RoPE table rows [0, rope_row0 + M) of 64 (cos, sin) fp16 pairs = 128 halves = 256 bytes per row
  if (ep.has_rope && make_tmap_2d(&P->r, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.rope,
                                  static_cast<int64_t>(a.rope_row0) + a.M, 128, 256, 32, 64) != DSB_OK)
    return DSB_ERR_CUDA;
  return DSB_OK;
}

// Operand maps and tile counts for the chosen tile shape.
static int shape_problem(const dsb_gemm_args& a, int fmt, int bn, int ctas, GemmProblem* P) {
  const int esz = (fmt == DSB_FMT_BF16) ? 2 : 1;
  const int slab_elems = kSlabBytes / esz;
  const CUtensorMapDataType dt =
      (fmt == DSB_FMT_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  if (make_tmap_2d(&P->a, dt, esz, a.A, a.M, a.K, a.lda * esz, kBlockM, slab_elems) != DSB_OK) return DSB_ERR_CUDA;
  if (make_tmap_2d(&P->b, dt, esz, a.W, a.N, a.K, a.ldw * esz, bn / ctas, slab_elems) != DSB_OK) return DSB_ERR_CUDA;
  P->tiles_m = (a.M + kBlockM * ctas - 1) / (kBlockM * ctas);
  P->tiles_n = (a.N + bn - 1) / bn;
  P->num_tiles = P->tiles_m * P->tiles_n;
  // panel height: activations of a panel <= ~32 MB, at least 4 row tiles, and a panel at least two waves of tiles
  {
    const int64_t tile_bytes = static_cast<int64_t>(kBlockM) * ctas * a.K * esz;
    int64_t g = (32ll << 20) / (tile_bytes > 0 ? tile_bytes : 1);
    if (g < 4) g = 4;
    const int64_t min_g = (2ll * sm_count() / ctas + P->tiles_n - 1) / P->tiles_n;
    if (g < min_g) g = min_g;
    if (g > P->tiles_m) g = P->tiles_m;
    P->panel = static_cast<int>(g);
  }
  P->num_kb = (a.K + slab_elems - 1) / slab_elems;
  return DSB_OK;
}

extern "C" int dsb_gemm_group(const dsb_gemm_args* args, int count, int fmt, int* status, void* stream) {
  if (!args || count < 1 || count > 2) return DSB_ERR_ARG;
  if (fmt != DSB_FMT_BF16 && fmt != DSB_FMT_E4M3 && fmt != DSB_FMT_INT8) return DSB_ERR_ARG;
  GemmGroup grp;
  const dsb_gemm_args* live[2];
  grp.count = 0;
  for (int i = 0; i < count; ++i) {
    const int rc = check_problem(args[i], fmt, status, &grp.p[grp.count]);
    if (rc != DSB_OK) return rc;
    if (args[i].M == 0 || args[i].N == 0) continue;  // an empty product: nothing to read or write
    live[grp.count++] = &args[i];
  }
  if (grp.count == 0) return DSB_OK;
  // one tile shape for the launch, chosen for the first (larger) problem; the fused norm needs a whole head per
  // epilogue warp, i.e. 256-wide tiles
  bool any_norm = false;
  for (int i = 0; i < grp.count; ++i)
    any_norm = any_norm || live[i]->nq_w != nullptr || live[i]->out0_fmt == DSB_FMT_E4M3 ||
               (live[i]->out1 && live[i]->out1_fmt == DSB_FMT_E4M3);  // both need a warp's full 128 columns
  const int bn = any_norm ? 256 : pick_block_n(live[0]->M, live[0]->N);
  // CTA pairs (256 x 256 tiles) when the first problem has enough rows to fill them
  const bool pair = bn == 256 && live[0]->M > 256 && live[0]->N >= 256;
  for (int i = 0; i < grp.count; ++i) {
    const int rc = shape_problem(*live[i], fmt, bn, pair ? 2 : 1, &grp.p[i]);
    if (rc != DSB_OK) return rc;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // Short reductions (at most 32 K slabs: K <= 4096 in 8 bits, 2048 in bf16) leave the epilogue as the longer half of
  // the pipeline: those launches take the kernel with the parameter table, the others the one with the deeper ring.
  const bool table = grp.p[0].num_kb <= 32;
  // the epilogue instantiation every problem of the launch fits (see the EPI enum); 128-wide tiles keep the generic one
  auto classify = [](const dsb_gemm_args& a) {
    const bool o8 = a.out0_fmt == DSB_FMT_E4M3;
    const bool split = a.out1 != nullptr;
    if (a.nq_w) {
      if (!split && !o8 && a.act == DSB_ACT_NONE && !a.resid) return int(EPI_NORM);
      if (split && !o8 && a.out1_fmt == DSB_FMT_E4M3 && a.act == DSB_ACT_GELU_TANH && a.act_col0 == a.split_col && !a.resid)
        return int(EPI_NORM_GELU8);
      return int(EPI_GENERIC);
    }
    if (split) return int(EPI_GENERIC);
    if (a.resid) return (a.act == DSB_ACT_NONE && !o8) ? int(EPI_RESID) : int(EPI_GENERIC);
    if (a.act == DSB_ACT_GELU_TANH && a.act_col0 <= 0) return o8 ? int(EPI_GELU8) : int(EPI_GELU);
    if (a.act == DSB_ACT_NONE && !o8) return int(EPI_PLAIN);
    return int(EPI_GENERIC);
  };
  int epi = bn == 256 ? classify(*live[0]) : int(EPI_GENERIC);
  for (int i = 1; i < grp.count; ++i)
    if (classify(*live[i]) != epi) epi = EPI_GENERIC;
#define DSB_GEMM_EPI(KIND, TABLE, EPI)                                          \
  (pair ? launch_group<KIND, 256, 2, TABLE, EPI>(grp, st) : launch_group<KIND, 256, 1, TABLE, EPI>(grp, st))
#define DSB_GEMM_SHAPE(KIND, TABLE)                                             \
  (bn != 256             ? launch_group<KIND, 128, 1, TABLE, EPI_GENERIC>(grp, st) \
   : epi == EPI_PLAIN    ? DSB_GEMM_EPI(KIND, TABLE, EPI_PLAIN)                 \
   : epi == EPI_RESID    ? DSB_GEMM_EPI(KIND, TABLE, EPI_RESID)                 \
   : epi == EPI_GELU     ? DSB_GEMM_EPI(KIND, TABLE, EPI_GELU)                  \
   : epi == EPI_GELU8    ? DSB_GEMM_EPI(KIND, TABLE, EPI_GELU8)                 \
   : epi == EPI_NORM     ? DSB_GEMM_EPI(KIND, TABLE, EPI_NORM)                  \
   : epi == EPI_NORM_GELU8 ? DSB_GEMM_EPI(KIND, TABLE, EPI_NORM_GELU8)          \
                         : DSB_GEMM_EPI(KIND, TABLE, EPI_GENERIC))
#define DSB_GEMM_DISPATCH(KIND) (table ? DSB_GEMM_SHAPE(KIND, true) : DSB_GEMM_SHAPE(KIND, false))
  if (fmt == DSB_FMT_BF16) return DSB_GEMM_DISPATCH(KIND_F16);
  if (fmt == DSB_FMT_E4M3) return DSB_GEMM_DISPATCH(KIND_F8);
  return DSB_GEMM_DISPATCH(KIND_I8);
#undef DSB_GEMM_DISPATCH
#undef DSB_GEMM_SHAPE
#undef DSB_GEMM_EPI
}

extern "C" int dsb_gemm(const void* A, int64_t lda, const void* W, int64_t ldw, int fmt, int M, int N, int K,
                        const float* row_scale, const float* col_scale, int col_scale_stride, const float* bias,
                        int act, int act_col0, const float* gate, const void* resid, int64_t ld_resid, void* out0,
                        int64_t ld_out0, void* out1, int64_t ld_out1, int split_col, int* status, void* stream) {
  dsb_gemm_args a = {};
  a.A = A, a.lda = lda, a.W = W, a.ldw = ldw, a.M = M, a.N = N, a.K = K;
  a.row_scale = row_scale, a.col_scale = col_scale, a.col_scale_stride = col_scale_stride, a.bias = bias;
  a.act = act, a.act_col0 = act_col0, a.gate = gate, a.resid = resid, a.ld_resid = ld_resid;
  a.out0 = out0, a.ld_out0 = ld_out0, a.out1 = out1, a.ld_out1 = ld_out1, a.split_col = split_col;
  return dsb_gemm_group(&a, 1, fmt, status, stream);
}

extern "C" int dsb_gemm_qkv(const void* A, int64_t lda, const void* W, int64_t ldw, int fmt, int M, int N, int K,
                            const float* row_scale, const float* col_scale, int col_scale_stride, const float* bias,
                            int act, int act_col0, void* out0, int64_t ld_out0, void* out1, int64_t ld_out1,
                            int split_col, const float* nq_w, const float* nk_w, int d_model, const void* rope,
                            int rope_row0, float norm_eps, int* status, void* stream) {
  if (!nq_w || !nk_w) return DSB_ERR_ARG;
  dsb_gemm_args a = {};
  a.A = A, a.lda = lda, a.W = W, a.ldw = ldw, a.M = M, a.N = N, a.K = K;
  a.row_scale = row_scale, a.col_scale = col_scale, a.col_scale_stride = col_scale_stride, a.bias = bias;
  a.act = act, a.act_col0 = act_col0;
  a.out0 = out0, a.ld_out0 = ld_out0, a.out1 = out1, a.ld_out1 = ld_out1, a.split_col = split_col;
  a.nq_w = nq_w, a.nk_w = nk_w, a.d_model = d_model, a.rope = rope, a.rope_row0 = rope_row0, a.norm_eps = norm_eps;
  return dsb_gemm_group(&a, 1, fmt, status, stream);
}
