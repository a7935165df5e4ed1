// Mask-free attention (joint text+image self-attention, Wan self- and
// cross-attention) as a tcgen05 flash-attention kernel, head_dim 128, bf16.
//
// One CTA owns two 128-row query tiles of one (batch, head) and streams the
// keys/values in tiles of 128.  Roles:
//   warp 0      TMA producer: Q once, then a 2-stage ring of K and of V tiles
//               (plain tiled loads, 128-byte swizzle, two 64-column halves)
//   warp 1      MMA issuer:   S_q = Q_q K_j^T  (SS, both operands K-major)
//                             O_q += P_q V_j   (TS: P read from TMEM, V MN-major)
//               The whole warp runs the issue loop, so descriptors stay warp-uniform, and one elected lane issues;
//               it polls the P barriers without suspending (a hand-over then costs a few cycles, not a wake-up).
//   warps 4-11  softmax of query tile 0, two threads per query row: warps 4-7 own key columns [0,64) of the
//               score tile, warps 8-11 own [64,128)
//   warps 12-19 softmax of query tile 1, same split
// TMEM (512 columns): S_0 | S_1 | O_0 | O_1, 128 fp32 columns each.  Each softmax thread turns its 64 scores into
// 32 columns of packed bf16 probabilities written over the FIRST half of its own 64 score columns, so P_q sits in
// columns [0,32) and [64,96) of S_q and no thread ever writes where another thread still has scores to read.
// S_q(j+1) is issued only after O_q += P_q(j) V_j, and the two query tiles ping-pong on the tensor core.
// P is handed over in two parts: the first 32 keys of each 64-key half as soon as their store has landed (a quarter
// of the way into the second chunk's exponentials), the rest at the end, so half of P.V runs under the softmax.
//
// The exponentials use a REFERENCE maximum that is one tile stale: p = exp2(s*c - m_ref) with m_ref = the row's
// maximum over all earlier key tiles.  Row sums and O carry the same reference, so the result is exact; entries of
// the current tile that exceed m_ref simply give p > 1 (fp32/bf16 have the range).  That takes the row-maximum
// reduction - and the exchange of it between the two threads of a row - off the S -> P -> MMA critical path: the
// threads publish their running maxima after they hand P over, and pick the partner's value up one tile later.
// Only the first tile computes its maximum before exponentiating.  m_ref is refreshed (O and the sums rescaled)
// when the running maximum has grown by more than 2^8.
//
// m_ref is always an INTEGER (in log2 units): rescaling by 2^(integer) is exact in floating point, so the bf16
// rounding of a probability does not depend on which reference it was computed against.  The result therefore equals
// "P = bf16(exp2(s*c - M)), O = P V / sum(exp2(s*c - M))" for ANY integer M, whatever the tile schedule - which is
// what the CPU restatement used by the parity tests evaluates (with M = ceil of the row maximum).
#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "dsb.h"

namespace dsb {

constexpr int kAttnThreads = 640;  // 4 control warps + 16 softmax warps
constexpr int kTileQ = 128;
constexpr int kTileKV = 128;
constexpr int kNQ = 2;
constexpr int kKVStages = 2;
constexpr int kRefresh = 1;  // the reference maximum is re-examined every kRefresh key tiles (power of two)
constexpr int kTileBytes = 128 * 128 * 2;  // 32 KiB: one 128 x 128 bf16 tile as two 64-column halves
constexpr int kHalfBytes = kTileBytes / 2;
constexpr int kXchgSlots = 2 * 2 * 128 * 3;  // [q][half][row] x {running maximum (even tile, odd tile), row sum}
constexpr int kAttnSmem = (kNQ + 2 * kKVStages) * kTileBytes + 256 + kXchgSlots * 8 + 1024;

constexpr int kMaxParts = 8;
constexpr int kWsRow = 132;  // floats per row of a partial result (528 bytes: rows stay 16-byte aligned)
// The query rows (and, independently, the output rows) may be cut into up to kMaxParts equal row ranges that live in
// different buffers - e.g. in the memory of different GPUs of a sequence-parallel group, where rank r holds the
// queries of its own tokens and receives the output rows of its own tokens from every rank.
struct AttnQMaps {
  CUtensorMap m[kMaxParts];
};
struct AttnParams {
  __nv_bfloat16* o;
  __nv_bfloat16* o_part[kMaxParts];
  int out_e4m3;         // 1: the output is written as e4m3 (1 byte per element; strides count elements = bytes)
  // Work items (query-tile pair, head) are numbered head-major along grid.x.  Items from n_full on - the ones that
  // would form a partly filled last wave - are each cut into `split` CTAs over contiguous key ranges; those CTAs
  // leave unnormalised partial results in `ws` and attn_combine_kernel finishes the rows.
  int n_pairs, n_full, split;
  float* ws;            // [tail item][part][256 rows][kWsRow floats]: 128 output columns, reference exponent, row sum
  int q_rows_per_part;  // 0: one query buffer (map 0); else a multiple of kTileQ
  int o_rows_per_part;  // 0: one output buffer (o); else row s goes to o_part[s / o_rows_per_part]
  int64_t o_stride_b, o_stride_s, o_stride_h;
  int Sq, Sk;
  float scale_log2;  // sm_scale * log2(e)
  // position of the (s, h, b) coordinates inside the tensor-map coordinate list (after d)
  int q_pos[3], k_pos[3], v_pos[3];
  int* status;
};

// Hand-over of one float between the two threads of a query row: a 64-bit slot {sequence number, value} written with
// one store; the reader spins (bounded) until the sequence number it expects is there.
__device__ __forceinline__ void xchg_publish(unsigned long long* slot, uint32_t seq, float v) {
  *reinterpret_cast<volatile unsigned long long*>(slot) =
      (static_cast<unsigned long long>(seq) << 32) | static_cast<unsigned long long>(__float_as_uint(v));
}
__device__ __forceinline__ bool xchg_read(const unsigned long long* slot, uint32_t seq, float* v,
                                          volatile int* abort_flag) {
  {
    const unsigned long long w = *reinterpret_cast<const volatile unsigned long long*>(slot);
    if (static_cast<uint32_t>(w >> 32) == seq) {  // the usual case: published long ago
      *v = __uint_as_float(static_cast<uint32_t>(w));
      return true;
    }
  }
  const long long t0 = clock64();
  uint32_t spins = 0;
  for (;;) {
    const unsigned long long w = *reinterpret_cast<const volatile unsigned long long*>(slot);
    if (static_cast<uint32_t>(w >> 32) == seq) {
      *v = __uint_as_float(static_cast<uint32_t>(w));
      return true;
    }
    if (((++spins) & 0xffu) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, const int (&pos)[3], int s0,
                                          int h, int b) {
  int c[3];
  c[pos[0]] = s0;
  c[pos[1]] = h;
  c[pos[2]] = b;
  tma_load_4d(dst, m, bar, 0, c[0], c[1], c[2]);
  tma_load_4d(dst + kHalfBytes, m, bar, 64, c[0], c[1], c[2]);
}

#define mbar_arrive(bar) mbar_arrive(bar)

// SPLIT: the launch has items cut along the keys (see AttnParams); the plain instantiation carries none of that code.
template <bool SPLIT>
__global__ void __launch_bounds__(kAttnThreads, 1)
    flash_attn_kernel(const __grid_constant__ AttnQMaps qmaps, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kNQ * kTileBytes;
  uint8_t* sV = sK + kKVStages * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kKVStages * kTileBytes);
  uint64_t* q_full = bars;                  // 1
  uint64_t* k_full = bars + 1;              // kKVStages
  uint64_t* k_empty = k_full + kKVStages;   // kKVStages
  uint64_t* v_full = k_empty + kKVStages;   // kKVStages
  uint64_t* v_empty = v_full + kKVStages;   // kKVStages
  uint64_t* s_full = v_empty + kKVStages;   // kNQ
  uint64_t* p_full = s_full + kNQ;          // kNQ: P of the first 32 keys of both key halves is in TMEM
  uint64_t* p_rest = p_full + kNQ;          // kNQ: ... and of the other 32
  uint64_t* o_full = p_rest + kNQ;          // kNQ
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + kNQ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned long long* xchg = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int item = blockIdx.x, part = 0, nparts = 1;
  if constexpr (SPLIT) {
    if (item >= p.n_full) {
      const int t = item - p.n_full;
      part = t % p.split;
      item = p.n_full + t / p.split;
      nparts = p.split;
    }
  }
  const int q0 = (item % p.n_pairs) * (kNQ * kTileQ);
  const int h = item / p.n_pairs;
  const int b = blockIdx.z;
  const int nkv_all = (p.Sk + kTileKV - 1) / kTileKV;
  const int jb = SPLIT ? static_cast<int>(static_cast<int64_t>(part) * nkv_all / nparts) : 0;  // first key tile of this CTA
  const int nkv = SPLIT ? static_cast<int>(static_cast<int64_t>(part + 1) * nkv_all / nparts) - jb : nkv_all;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kKVStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int q = 0; q < kNQ; ++q) {
      mbar_init(&s_full[q], 1);
      mbar_init(&p_full[q], 256);
      mbar_init(&p_rest[q], 256);
      mbar_init(&o_full[q], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  for (int i = threadIdx.x; i < kXchgSlots; i += blockDim.x) xchg[i] = 0ull;  // sequence 0 = nothing published
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&qmaps.m[0]);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, kNQ * kTileBytes);
      for (int q = 0; q < kNQ; ++q) {
        int s0 = q0 + q * kTileQ, part = 0;
        if (p.q_rows_per_part > 0) {  // a 128-row tile never straddles two parts
          part = min(s0 / p.q_rows_per_part, kMaxParts - 1);
          s0 -= part * p.q_rows_per_part;
        }
        load_tile(sQ + q * kTileBytes, &qmaps.m[part], q_full, p.q_pos, s0, h, b);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < nkv; ++j) {
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&k_full[st], kTileBytes);
        load_tile(sK + st * kTileBytes, &tmap_k, &k_full[st], p.k_pos, (jb + j) * kTileKV, h, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&v_full[st], kTileBytes);
        load_tile(sV + st * kTileBytes, &tmap_v, &v_full[st], p.v_pos, (jb + j) * kTileKV, h, b);
        if (++st == kKVStages) {
          st = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    {
      // the whole warp runs this loop so that descriptors and addresses stay warp-uniform; one elected lane issues
      const uint32_t leader = elect_one();
      constexpr uint32_t idesc_qk = make_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 0, 0, 128, 128);
      constexpr uint32_t idesc_pv = make_idesc(DFMT_F32, FMT_BF16, FMT_BF16, 0, 1, 128, 128);
      // One tcgen05.mma here is only 64 tensor-core cycles of work, so the issuing thread must not spend more than
      // a few instructions per MMA: every descriptor is a base computed once plus a compile-time offset in the
      // low word (the address field, in 16-byte units, never carries into the upper word).
      const uint64_t q_desc0 = make_desc_k_sw128(smem_u32(sQ));
      const uint64_t k_desc0 = make_desc_k_sw128(smem_u32(sK));
      const uint64_t v_desc0 = make_desc_mn_sw128(smem_u32(sV), kHalfBytes, 1024);
      constexpr uint32_t kTile16 = kTileBytes >> 4, kHalf16 = kHalfBytes >> 4;
      auto issue_qk = [&](int q, int st) {
        const uint64_t ad0 = q_desc0 + static_cast<uint32_t>(q) * kTile16;
        const uint64_t bd0 = k_desc0 + static_cast<uint32_t>(st) * kTile16;
        const uint32_t d = tmem_base + q * 128;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * kHalf16 + 2 * (kk & 3);
          mma_ss_f16_elect(d, ad0 + off, bd0 + off, idesc_qk, kk > 0 ? 1u : 0u, leader);
        }
      };
      // O_q += P_q V for the 16-key groups kk in {g, g+1, g+4, g+5}: g = 0 are the keys whose probabilities every
      // softmax thread writes first (its first 32 of 64 columns), g = 2 the rest
      auto issue_pv = [&](int q, int st, int g, bool accumulate) {
        const uint64_t bd0 = v_desc0 + static_cast<uint32_t>(st) * kTile16;
        const uint32_t d = tmem_base + 256 + q * 128;
        const uint32_t a = tmem_base + q * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int kk = g + (i & 1) + (i >> 1) * 4;
          // 16 keys per instruction = 16 rows of 128 bytes (2048 bytes = 128 units) further into the V tile
          // P of keys [0,64) lives in columns [0,32) of S_q, P of keys [64,128) in columns [64,96)
          mma_ts_f16_elect(d, a + (kk >> 2) * 64 + (kk & 3) * 8, bd0 + kk * 128u, idesc_pv, (accumulate || i > 0) ? 1u : 0u,
                           leader);
        }
      };
      int kst = 0, vst = 0;
      uint32_t kph = 0, vph = 0;
      if (!mbar_wait(q_full, 0, abort_flag)) goto mma_done;
      if (!mbar_wait(&k_full[kst], kph, abort_flag)) goto mma_done;
      tc_fence_after();
      for (int q = 0; q < kNQ; ++q) {
        issue_qk(q, kst);
        tc_commit_elect(&s_full[q], leader);
      }
      tc_commit_elect(&k_empty[kst], leader);
      if (++kst == kKVStages) kst = 0, kph ^= 1;
      for (int j = 0; j < nkv; ++j) {
        const bool has_next = (j + 1) < nkv;
        if (!mbar_wait(&v_full[vst], vph, abort_flag)) goto mma_done;
        if (has_next && !mbar_wait(&k_full[kst], kph, abort_flag)) goto mma_done;
        for (int q = 0; q < kNQ; ++q) {
          if (!mbar_wait_spin(&p_full[q], j & 1, abort_flag)) goto mma_done;
          tc_fence_after();
          issue_pv(q, vst, 0, j > 0);
          if (!mbar_wait_spin(&p_rest[q], j & 1, abort_flag)) goto mma_done;
          tc_fence_after();
          issue_pv(q, vst, 2, true);
          if (has_next) {
            issue_qk(q, kst);
            tc_commit_elect(&s_full[q], leader);
          } else {
            tc_commit_elect(&o_full[q], leader);
          }
        }
        tc_commit_elect(&v_empty[vst], leader);
        if (++vst == kKVStages) vst = 0, vph ^= 1;
        if (has_next) {
          tc_commit_elect(&k_empty[kst], leader);
          if (++kst == kKVStages) kst = 0, kph ^= 1;
        }
      }
    }
  mma_done:;
  } else if (warp >= 4) {
    // ----------------------------------------------------------------- softmax
    const int ws = warp - 4;
    const int q = ws >> 3;
    const int half = (ws >> 2) & 1;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_off + q * 128 + half * 64;        // my 64 score columns; P goes to the first 32
    const uint32_t t_o = tmem_base + lane_off + 256 + q * 128 + half * 64;  // my half of the output columns
    unsigned long long* slot_mine = xchg + ((q * 2 + half) * 128 + row) * 3;  // {max even tile, max odd tile, sum}
    const unsigned long long* slot_other = xchg + ((q * 2 + (half ^ 1)) * 128 + row) * 3;
    const float cs = p.scale_log2;
    const float inv_cs = 1.0f / cs;
    float m_ref = 0.f;       // reference maximum (log2 units) the exponentials, the row sum and O currently use
    float run_max = -INFINITY;  // this thread's running maximum of raw scores over its columns, all tiles so far
    // four running maxima and four partial row sums live across the key tiles (folded only when published / at the
    // end), so no per-tile reduction chain sits between the last exponential and the hand-over of P
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    float2 ls2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      if (!mbar_wait(&s_full[q], j & 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int valid = min(kTileKV, p.Sk - (jb + j) * kTileKV) - half * 64;  // valid columns among my 64 (may be <= 0)
      bool handed = false;  // p_full already signalled for this tile
      if (j == 0) {
        // first tile: the row maximum must be known before anything is exponentiated
        uint32_t s0[32], s1[32];
        tmem_ld32(t_s, s0);
        tmem_ld32(t_s + 32, s1);
        tc_wait_ld();
        float m0 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i < valid) m0 = fmaxf(m0, __uint_as_float(s0[i]));
          if (32 + i < valid) m0 = fmaxf(m0, __uint_as_float(s1[i]));
        }
        run_max = m0;
        xchg_publish(&slot_mine[0], 1u, m0);
        float mo;
        if (!xchg_read(&slot_other[0], 1u, &mo, abort_flag)) {
          ok = false;
          break;
        }
        m_ref = ceilf(fmaxf(m0, mo) * cs);  // at least one key of the tile is valid, so this is finite
        float ls = 0.f;
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = (2 * i < valid) ? fast_exp2(fmaf(__uint_as_float(s0[2 * i]), cs, -m_ref)) : 0.f;
          const float p1 = (2 * i + 1 < valid) ? fast_exp2(fmaf(__uint_as_float(s0[2 * i + 1]), cs, -m_ref)) : 0.f;
          ls += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st16(t_s, pk);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = (32 + 2 * i < valid) ? fast_exp2(fmaf(__uint_as_float(s1[2 * i]), cs, -m_ref)) : 0.f;
          const float p1 = (33 + 2 * i < valid) ? fast_exp2(fmaf(__uint_as_float(s1[2 * i + 1]), cs, -m_ref)) : 0.f;
          ls += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st16(t_s + 16, pk);
        ls2[0].x = ls;
        mx[0] = m0;
      } else {
        // first score chunk on its way from TMEM while the (already published) partner maximum is read
        uint32_t sc[32];
        tmem_ld32(t_s, sc);
        if (kRefresh == 1 || (j & (kRefresh - 1)) == 1) {
          // every kRefresh-th tile: is the reference maximum still close enough to the running maximum of the row?
          // (the partner published its running maximum after tile j-1)
          float mo;
          if (!xchg_read(&slot_other[((j - 1) / kRefresh) & 1], static_cast<uint32_t>(j), &mo, abort_flag)) {
            ok = false;
            break;
          }
          const float m_run = fmaxf(run_max, mo) * cs;
          if (__any_sync(0xffffffffu, m_run > m_ref + 8.0f)) {
            // both warps of these rows see the same values, so both take this branch.  O is idle: S_q(j) is only
            // signalled after O_q += P_q(j-1) V has completed.
            const float m_upd = fmaxf(m_ref, ceilf(m_run));
            const float alpha = __int_as_float(max(0, 127 + static_cast<int>(m_ref - m_upd)) << 23);
            m_ref = m_upd;
            ls2[0].x *= alpha, ls2[0].y *= alpha, ls2[1].x *= alpha, ls2[1].y *= alpha;
            tc_wait_ld();
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
              uint32_t r[32];
              tmem_ld32(t_o + c * 32, r);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st32(t_o + c * 32, r);
            }
          }
        }
        const float2 cs2 = make_float2(cs, cs), nm2 = make_float2(-m_ref, -m_ref);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (c == 1) tmem_ld32(t_s + 32, sc);
          tc_wait_ld();
          uint32_t pk[16];
          if (valid >= 64) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              if (c == 1 && i == 8) {
                // the first chunk's P store has had half a chunk of arithmetic to land: hand the first 32 keys over
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(&p_full[q]);
                handed = true;
              }
              const float2 a = make_float2(__uint_as_float(sc[2 * i]), __uint_as_float(sc[2 * i + 1]));
              const float2 x = __ffma2_rn(a, cs2, nm2);
              // the clamp only matters for rows whose scores jump by more than 2^100 from one key tile to the next
              const float2 pp = make_float2(fast_exp2(fminf(x.x, 100.f)), fast_exp2(fminf(x.y, 100.f)));
              mx[i & 3] = max3f(mx[i & 3], a.x, a.y);
              ls2[i & 1] = __fadd2_rn(ls2[i & 1], pp);
              pk[i] = pack_bf16x2(pp.x, pp.y);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int c0 = c * 32 + 2 * i;
              const float a0 = __uint_as_float(sc[2 * i]), a1 = __uint_as_float(sc[2 * i + 1]);
              const float p0 = (c0 < valid) ? fast_exp2(fminf(fmaf(a0, cs, -m_ref), 100.f)) : 0.f;
              const float p1 = (c0 + 1 < valid) ? fast_exp2(fminf(fmaf(a1, cs, -m_ref), 100.f)) : 0.f;
              if (c0 < valid) mx[i & 3] = fmaxf(mx[i & 3], a0);
              if (c0 + 1 < valid) mx[i & 3] = fmaxf(mx[i & 3], a1);
              ls2[i & 1].x += p0;
              ls2[i & 1].y += p1;
              pk[i] = pack_bf16x2(p0, p1);
            }
          }
          tmem_st16(t_s + c * 16, pk);
        }
      }
      tc_wait_st();
      tc_fence_before();
      if (!handed) mbar_arrive(&p_full[q]);
      mbar_arrive(&p_rest[q]);
      // off the critical path: publish my running maximum for the partner to use at the next tile (slot by tile
      // parity: the partner cannot be two tiles ahead, S_q(j+2) needs this thread's P_q(j+1))
      if (j > 0 && (j & (kRefresh - 1)) == 0) {
        // A score more than 2^100 above the reference was exponentiated as 2^100 (the clamp), so the running maximum
        // - and with it the next reference - may only follow it that far: the row then stays finite and is
        // dominated by that key, as it should be.
        const float lim = (m_ref + 100.f) * inv_cs;
#pragma unroll
        for (int i = 0; i < 4; ++i) mx[i] = fminf(mx[i], lim);
        run_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        xchg_publish(&slot_mine[(j / kRefresh) & 1], static_cast<uint32_t>(j + 1), run_max);
      }
    }
    if (ok && mbar_wait(&o_full[q], 0, abort_flag)) {
      tc_fence_after();
      const float l = (ls2[0].x + ls2[0].y) + (ls2[1].x + ls2[1].y);
      xchg_publish(&slot_mine[2], 0x7fffffffu, l);
      float lo = 0.f;
      ok = xchg_read(&slot_other[2], 0x7fffffffu, &lo, abort_flag);
      const int sq = q0 + q * kTileQ + row;
      if (SPLIT && nparts > 1) {
        // one key range of a split item: O (relative to 2^m_ref), m_ref and the row sum go to the workspace
        float* wrow = p.ws + ((static_cast<int64_t>(item - p.n_full) * nparts + part) * (kNQ * kTileQ) + q * kTileQ + row) * kWsRow;
        if (half == 0) {
          wrow[128] = m_ref;
          wrow[129] = l + lo;
        }
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(t_o + c * 32, r);
          tc_wait_ld();
          if (ok) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
              *reinterpret_cast<uint4*>(wrow + half * 64 + c * 32 + g * 4) =
                  make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
          }
        }
      } else {
      const float inv = 1.0f / (l + lo);
      __nv_bfloat16* obase = p.o + static_cast<int64_t>(b) * p.o_stride_b;
      int so = sq;
      if (p.o_rows_per_part > 0) {
        const int part = min(sq / p.o_rows_per_part, kMaxParts - 1);
        obase = p.o_part[part];
        so = sq - part * p.o_rows_per_part;
      }
      const int64_t ooff = static_cast<int64_t>(so) * p.o_stride_s + static_cast<int64_t>(h) * p.o_stride_h + half * 64;
      __nv_bfloat16* orow = obase + ooff;
      // e4m3 output (the operand of a following FP8 Linear with unit activation scale): the value is rounded to bf16
      // first and then cast with saturation, i.e. exactly what a bf16 output followed by dsb_cast_quant gives
      uint8_t* orow8 = reinterpret_cast<uint8_t*>(p.o) + static_cast<int64_t>(b) * p.o_stride_b + ooff;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(t_o + c * 32, r);
        tc_wait_ld();
        if (ok && sq < p.Sq) {
          if (p.out_e4m3) {
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 lo = unpack_bf16x2(pack_bf16x2(__uint_as_float(r[g * 16 + j * 4 + 0]) * inv,
                                                            __uint_as_float(r[g * 16 + j * 4 + 1]) * inv));
                const float2 hi = unpack_bf16x2(pack_bf16x2(__uint_as_float(r[g * 16 + j * 4 + 2]) * inv,
                                                            __uint_as_float(r[g * 16 + j * 4 + 3]) * inv));
                const __nv_fp8x2_storage_t a8 = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3);
                const __nv_fp8x2_storage_t b8 = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3);
                w[j] = static_cast<uint32_t>(a8) | (static_cast<uint32_t>(b8) << 16);
              }
              *reinterpret_cast<uint4*>(orow8 + c * 32 + g * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]) * inv, __uint_as_float(r[g * 8 + 1]) * inv);
              o.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]) * inv, __uint_as_float(r[g * 8 + 3]) * inv);
              o.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]) * inv, __uint_as_float(r[g * 8 + 5]) * inv);
              o.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]) * inv, __uint_as_float(r[g * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
            }
          }
        }
      }
      }  // whole-row result
    }
  }

  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, 0, DSB_ERR_TIMEOUT);
}

// Finishes the rows of the split items: with M = max over parts of m_p, O = sum_p 2^(m_p - M) O_p and
// l = sum_p 2^(m_p - M) l_p (the m_p are integers, so the factors are exact), out = O / l.  One warp per row,
// four columns per lane.
__global__ void __launch_bounds__(256) attn_combine_kernel(AttnParams p, int tail_items) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int rows = kNQ * kTileQ;
  if (gw >= tail_items * rows) return;
  const int ti = gw / rows, r = gw % rows;
  const int item = p.n_full + ti;
  const int sq = (item % p.n_pairs) * rows + r;
  const int h = item / p.n_pairs;
  if (sq >= p.Sq) return;
  const float* base = p.ws + (static_cast<int64_t>(ti) * p.split * rows + r) * kWsRow;
  float M = -INFINITY;
  for (int s = 0; s < p.split; ++s) M = fmaxf(M, base[static_cast<int64_t>(s) * rows * kWsRow + 128]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l = 0.f;
  for (int s = 0; s < p.split; ++s) {
    const float* pr = base + static_cast<int64_t>(s) * rows * kWsRow;
    const float w = exp2f(pr[128] - M);
    const float4 o = *reinterpret_cast<const float4*>(pr + lane * 4);
    acc.x = fmaf(w, o.x, acc.x), acc.y = fmaf(w, o.y, acc.y), acc.z = fmaf(w, o.z, acc.z), acc.w = fmaf(w, o.w, acc.w);
    l = fmaf(w, pr[129], l);
  }
  const float inv = 1.0f / l;
  __nv_bfloat16* obase = p.o;
  int so = sq;
  if (p.o_rows_per_part > 0) {
    const int part = min(sq / p.o_rows_per_part, kMaxParts - 1);
    obase = p.o_part[part];
    so = sq - part * p.o_rows_per_part;
  }
  __nv_bfloat16* orow = obase + static_cast<int64_t>(so) * p.o_stride_s + static_cast<int64_t>(h) * p.o_stride_h + lane * 4;
  uint2 o2;
  o2.x = pack_bf16x2(acc.x * inv, acc.y * inv);
  o2.y = pack_bf16x2(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(orow) = o2;
}

// Rank-4 tensor map over (d, then s/h/b ordered by ascending stride); box = 64 x 128 rows of s.
static int make_tmap_attn(CUtensorMap* out, int (&pos)[3], const void* base, int S, int H, int B, int64_t ss,
                          int64_t sh, int64_t sb) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return DSB_ERR_CUDA;
  struct Dim {
    uint64_t size, stride;
    uint32_t box;
    int id;
  } d[3] = {{static_cast<uint64_t>(S), static_cast<uint64_t>(ss) * 2, 128u, 0},
            {static_cast<uint64_t>(H), static_cast<uint64_t>(sh) * 2, 1u, 1},
            {static_cast<uint64_t>(B), static_cast<uint64_t>(sb) * 2, 1u, 2}};
  // a dimension of extent 1 never moves: give it a stride that keeps the list ascending
  std::stable_sort(d, d + 3, [](const Dim& a, const Dim& b2) {
    if ((a.size == 1) != (b2.size == 1)) return b2.size == 1;
    return a.stride < b2.stride;
  });
  uint64_t prev = 256;  // bytes of one row of d
  for (int i = 0; i < 3; ++i) {
    if (d[i].size == 1) d[i].stride = prev * (i == 0 ? 1 : d[i - 1].size);
    if (d[i].stride == 0 || (d[i].stride & 15)) return DSB_ERR_ARG;
    prev = d[i].stride;
  }
  for (int i = 0; i < 3; ++i) pos[d[i].id] = i;
  const cuuint64_t dims[4] = {128, d[0].size, d[1].size, d[2].size};
  const cuuint64_t strides[3] = {d[0].stride, d[1].stride, d[2].stride};
  const cuuint32_t box[4] = {64, d[0].box, d[1].box, d[2].box};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DSB_OK : DSB_ERR_CUDA;
}

}  // namespace dsb

using namespace dsb;

// q_parts / o_parts: nullptr for one buffer (q / o), else n equal row ranges in separate buffers
static int launch_attn(const void* q, const void* const* q_parts, int n_q_parts, int q_rows_per_part, const void* k,
                       const void* v, void* o, void* const* o_parts, int n_o_parts, int o_rows_per_part, int B, int H,
                       int Sq, int Sk, int head_dim, int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                       int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_b,
                       int64_t v_stride_s, int64_t v_stride_h, int64_t o_stride_b, int64_t o_stride_s,
                       int64_t o_stride_h, float sm_scale, int out_e4m3, void* ws, int64_t ws_bytes, int* status,
                       void* stream) {
  if (!k || !v || B <= 0 || H <= 0 || Sq < 0 || Sk <= 0) return DSB_ERR_ARG;
  if (ws && ((reinterpret_cast<uintptr_t>(ws) & 15u) || ws_bytes < 0)) return DSB_ERR_ARG;
  if (out_e4m3 && (o_parts || ((o_stride_s | o_stride_h | o_stride_b) & 15))) return DSB_ERR_ARG;
  if (head_dim != 128) return DSB_ERR_UNSUPPORTED;
  if (B > 65535) return DSB_ERR_UNSUPPORTED;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al16(k) || !al16(v)) return DSB_ERR_ARG;
  if (q_parts) {
    if (B != 1 || n_q_parts < 1 || n_q_parts > kMaxParts || q_rows_per_part <= 0 || (q_rows_per_part % kTileQ) ||
        static_cast<int64_t>(n_q_parts) * q_rows_per_part < Sq)
      return DSB_ERR_ARG;
    for (int i = 0; i < n_q_parts; ++i)
      if (!q_parts[i] || !al16(q_parts[i])) return DSB_ERR_ARG;
  } else if (!q || !al16(q)) {
    return DSB_ERR_ARG;
  }
  if (o_parts) {
    if (B != 1 || n_o_parts < 1 || n_o_parts > kMaxParts || o_rows_per_part <= 0 ||
        static_cast<int64_t>(n_o_parts) * o_rows_per_part < Sq)
      return DSB_ERR_ARG;
    for (int i = 0; i < n_o_parts; ++i)
      if (!o_parts[i] || !al16(o_parts[i])) return DSB_ERR_ARG;
  } else if (!o || !al16(o)) {
    return DSB_ERR_ARG;
  }
  const int64_t strides[] = {q_stride_s, q_stride_h, k_stride_s, k_stride_h, v_stride_s, v_stride_h,
                             o_stride_s, o_stride_h, q_stride_b, k_stride_b, v_stride_b, o_stride_b};
  for (int64_t s : strides)
    if (s < 0 || (s & 7)) return DSB_ERR_ARG;
  if (Sq == 0) return DSB_OK;
  AttnParams p = {};
  AttnQMaps qm;
  CUtensorMap tk, tv;
  int rc;
  if (q_parts) {
    // every part is a buffer of q_rows_per_part rows (rows past Sq are read but never used), so all maps share one
    // coordinate order; unused slots repeat the last part
    for (int i = 0; i < kMaxParts; ++i) {
      const void* base = q_parts[i < n_q_parts ? i : n_q_parts - 1];
      if ((rc = make_tmap_attn(&qm.m[i], p.q_pos, base, q_rows_per_part, H, 1, q_stride_s, q_stride_h, q_stride_b)) !=
          DSB_OK)
        return rc;
    }
    p.q_rows_per_part = q_rows_per_part;
  } else {
    if ((rc = make_tmap_attn(&qm.m[0], p.q_pos, q, Sq, H, B, q_stride_s, q_stride_h, q_stride_b)) != DSB_OK) return rc;
    for (int i = 1; i < kMaxParts; ++i) qm.m[i] = qm.m[0];
  }
  if ((rc = make_tmap_attn(&tk, p.k_pos, k, Sk, H, B, k_stride_s, k_stride_h, k_stride_b)) != DSB_OK) return rc;
  if ((rc = make_tmap_attn(&tv, p.v_pos, v, Sk, H, B, v_stride_s, v_stride_h, v_stride_b)) != DSB_OK) return rc;
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  if (o_parts) {
    for (int i = 0; i < kMaxParts; ++i)
      p.o_part[i] = reinterpret_cast<__nv_bfloat16*>(o_parts[i < n_o_parts ? i : n_o_parts - 1]);
    p.o_rows_per_part = o_rows_per_part;
  }
  p.out_e4m3 = out_e4m3 ? 1 : 0;
  p.o_stride_b = o_stride_b;
  p.o_stride_s = o_stride_s;
  p.o_stride_h = o_stride_h;
  p.Sq = Sq;
  p.Sk = Sk;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.status = status;
  DSB_ENSURE_SMEM(flash_attn_kernel<false>, kAttnSmem);
  DSB_ENSURE_SMEM(flash_attn_kernel<true>, kAttnSmem);
  const int n_pairs = (Sq + kNQ * kTileQ - 1) / (kNQ * kTileQ);
  const int64_t items = static_cast<int64_t>(n_pairs) * H;
  if (items > 0x3fffffff) return DSB_ERR_UNSUPPORTED;
  p.n_pairs = n_pairs;
  p.n_full = static_cast<int>(items);
  p.split = 1;
  p.ws = nullptr;
  // One CTA per SM: the items run in waves of sm_count().  A partly filled last wave costs a whole item's duration
  // (measured: 590 items on 148 SMs 1.94 ms, 595 items 2.34 ms at 32760 keys), so when the caller provides a
  // workspace its items are cut along the keys into as many CTAs as fill that wave, plus a combine pass.
  int tail = 0;
  if (ws && B == 1 && !out_e4m3) {
    const int sms = sm_count();
    const int nkv = (Sk + kTileKV - 1) / kTileKV;
    tail = static_cast<int>(items % sms);
    // cut in `split`: the last wave's items take ceil(tail * split / sms) rounds of 1/split of an item's duration
    // (plus a few per cent per CTA for prologue, partial-result stores and the combine pass)
    int split = 1;
    if (tail > 0 && items > sms) {
      double best = 1.0;
      for (int sp = 2; sp <= 4; ++sp) {
        if (nkv / sp < 8) break;  // every key range keeps at least 8 tiles
        const double cost = static_cast<double>((static_cast<int64_t>(tail) * sp + sms - 1) / sms) / sp + 0.05;
        if (cost < best - 1e-9) best = cost, split = sp;
      }
    }
    const int64_t need = static_cast<int64_t>(tail) * split * (kNQ * kTileQ) * kWsRow * 4;
    if (split >= 2 && need <= ws_bytes) {
      p.split = split;
      p.n_full = static_cast<int>(items) - tail;
      p.ws = reinterpret_cast<float*>(ws);
    }
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int ctas = p.n_full + (p.split > 1 ? tail * p.split : 0);
  dim3 grid(ctas, 1, B);
  if (p.split > 1)
    flash_attn_kernel<true><<<grid, kAttnThreads, kAttnSmem, st>>>(qm, tk, tv, p);
  else
    flash_attn_kernel<false><<<grid, kAttnThreads, kAttnSmem, st>>>(qm, tk, tv, p);
  if (cudaGetLastError() != cudaSuccess) return DSB_ERR_CUDA;
  if (p.split > 1) {
    const int warps = tail * kNQ * kTileQ;
    attn_combine_kernel<<<(warps + 7) / 8, 256, 0, st>>>(p, tail);
  }
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

extern "C" int dsb_flash_attn(const void* q, const void* k, const void* v, void* o, int B, int H, int Sq, int Sk,
                              int head_dim, int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                              int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_b,
                              int64_t v_stride_s, int64_t v_stride_h, int64_t o_stride_b, int64_t o_stride_s,
                              int64_t o_stride_h, float sm_scale, int* status, void* stream) {
  return launch_attn(q, nullptr, 0, 0, k, v, o, nullptr, 0, 0, B, H, Sq, Sk, head_dim, q_stride_b, q_stride_s, q_stride_h,
                     k_stride_b, k_stride_s, k_stride_h, v_stride_b, v_stride_s, v_stride_h, o_stride_b, o_stride_s,
                     o_stride_h, sm_scale, 0, nullptr, 0, status, stream);
}

extern "C" int dsb_flash_attn_out8(const void* q, const void* k, const void* v, void* o, int B, int H, int Sq, int Sk,
                                   int head_dim, int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                                   int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_b,
                                   int64_t v_stride_s, int64_t v_stride_h, int64_t o_stride_b, int64_t o_stride_s,
                                   int64_t o_stride_h, float sm_scale, int* status, void* stream) {
  return launch_attn(q, nullptr, 0, 0, k, v, o, nullptr, 0, 0, B, H, Sq, Sk, head_dim, q_stride_b, q_stride_s, q_stride_h,
                     k_stride_b, k_stride_s, k_stride_h, v_stride_b, v_stride_s, v_stride_h, o_stride_b, o_stride_s,
                     o_stride_h, sm_scale, 1, nullptr, 0, status, stream);
}

extern "C" int dsb_flash_attn_parts(const void* const* q_parts, int n_q_parts, int q_rows_per_part, const void* k,
                                    const void* v, void* const* o_parts, int n_o_parts, int o_rows_per_part, int H,
                                    int Sq, int Sk, int head_dim, int64_t q_stride_s, int64_t q_stride_h,
                                    int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_s, int64_t v_stride_h,
                                    int64_t o_stride_s, int64_t o_stride_h, float sm_scale, void* workspace,
                                    int64_t workspace_bytes, int* status, void* stream) {
  if (!q_parts || !o_parts) return DSB_ERR_ARG;
  return launch_attn(nullptr, q_parts, n_q_parts, q_rows_per_part, k, v, nullptr, o_parts, n_o_parts, o_rows_per_part, 1,
                     H, Sq, Sk, head_dim, 0, q_stride_s, q_stride_h, 0, k_stride_s, k_stride_h, 0, v_stride_s,
                     v_stride_h, 0, o_stride_s, o_stride_h, sm_scale, 0, workspace, workspace_bytes, status, stream);
}

extern "C" int64_t dsb_flash_attn_workspace_bytes(void) {
  // a last wave of at most sm_count() - 1 items, cut in at most four
  return static_cast<int64_t>(sm_count()) * 4 * (kNQ * kTileQ) * kWsRow * 4;
}
