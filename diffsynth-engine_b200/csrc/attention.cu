// Mask-free attention (joint text+image self-attention, Wan self- and
// cross-attention) as a tcgen05 flash-attention kernel, head_dim 128, bf16.
//
// One CTA owns two 128-row query tiles of one (batch, head) and streams the
// keys/values in tiles of 128.  Roles:
//   warp 0      TMA producer: Q once, then a 2-stage ring of K and of V tiles
//               (plain tiled loads, 128-byte swizzle, two 64-column halves)
//   warp 1      MMA issuer:   S_q = Q_q K_j^T  (SS, both operands K-major)
//                             O_q += P_q V_j   (TS: P read from TMEM, V MN-major)
//   warps 4-7   softmax of query tile 0 (one thread per query row)
//   warps 8-11  softmax of query tile 1
// TMEM (512 columns): S_0 | S_1 | O_0 | O_1, 128 fp32 columns each; the bf16
// probabilities P_q overwrite the first 64 columns of S_q, so S_q(j+1) is issued
// only after O_q += P_q(j) V_j, and the two query tiles ping-pong on the tensor
// core while the other one is in its softmax.
// The running maximum is refreshed lazily (only when it grows by more than 2^8),
// which keeps O's rescale out of the common path; it is exact because O and the
// row sum carry the same reference maximum.
#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "dsb.h"

namespace dsb {

constexpr int kAttnThreads = 384;
constexpr int kTileQ = 128;
constexpr int kTileKV = 128;
constexpr int kNQ = 2;
constexpr int kKVStages = 2;
constexpr int kTileBytes = 128 * 128 * 2;  // 32 KiB: one 128 x 128 bf16 tile as two 64-column halves
constexpr int kHalfBytes = kTileBytes / 2;
constexpr int kCtrlRegs = 72;      // registers per thread kept by the control warps
constexpr int kSoftmaxRegs = 208;  // registers per thread of the softmax warps
constexpr int kAttnSmem = (kNQ + 2 * kKVStages) * kTileBytes + 256 + 1024;

struct AttnParams {
  __nv_bfloat16* o;
  int64_t o_stride_b, o_stride_s, o_stride_h;
  int Sq, Sk;
  float scale_log2;  // sm_scale * log2(e)
  // position of the (s, h, b) coordinates inside the tensor-map coordinate list (after d)
  int q_pos[3], k_pos[3], v_pos[3];
  int* status;
};

template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
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

__global__ void __launch_bounds__(kAttnThreads, 1)
    flash_attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
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
  uint64_t* p_full = s_full + kNQ;          // kNQ
  uint64_t* o_full = p_full + kNQ;          // kNQ
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + kNQ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * (kNQ * kTileQ);
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int nkv = (p.Sk + kTileKV - 1) / kTileKV;

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
      mbar_init(&p_full[q], 128);
      mbar_init(&o_full[q], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
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

  // Registers move from the four control warps (TMA, MMA, two idle) to the softmax warps, which hold a whole
  // 128-wide score row per thread.  The kernel launches with 168 registers per thread (384 threads); the 128
  // control threads give back 168-72 = 96 each (12288), the 256 softmax threads take 208-168 = 40 each (10240).
  // The increase must never ask for more than was released: setmaxnreg.inc blocks until it is satisfied.
  static_assert((168 - kCtrlRegs) * 128 >= (kSoftmaxRegs - 168) * 256, "setmaxnreg.inc could never be satisfied");
  if (warp < 4) reg_dealloc<kCtrlRegs>();
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, kNQ * kTileBytes);
      for (int q = 0; q < kNQ; ++q) load_tile(sQ + q * kTileBytes, &tmap_q, q_full, p.q_pos, q0 + q * kTileQ, h, b);
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < nkv; ++j) {
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&k_full[st], kTileBytes);
        load_tile(sK + st * kTileBytes, &tmap_k, &k_full[st], p.k_pos, j * kTileKV, h, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&v_full[st], kTileBytes);
        load_tile(sV + st * kTileBytes, &tmap_v, &v_full[st], p.v_pos, j * kTileKV, h, b);
        if (++st == kKVStages) {
          st = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
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
          constexpr uint32_t dummy = 0;
          (void)dummy;
          const uint32_t off = (kk >> 2) * kHalf16 + 2 * (kk & 3);
          mma_ss<KIND_F16>(d, ad0 + off, bd0 + off, idesc_qk, kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int q, int st, bool accumulate) {
        const uint64_t bd0 = v_desc0 + static_cast<uint32_t>(st) * kTile16;
        const uint32_t d = tmem_base + 256 + q * 128;
        const uint32_t a = tmem_base + q * 128;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 keys per instruction = 16 rows of 128 bytes (2048 bytes = 128 units) further into the V tile
          mma_ts_f16(d, a + kk * 8, bd0 + kk * 128u, idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
        }
      };
      int kst = 0, vst = 0;
      uint32_t kph = 0, vph = 0;
      if (!mbar_wait(q_full, 0, abort_flag)) goto mma_done;
      if (!mbar_wait(&k_full[kst], kph, abort_flag)) goto mma_done;
      tc_fence_after();
      for (int q = 0; q < kNQ; ++q) {
        issue_qk(q, kst);
        tc_commit(&s_full[q]);
      }
      tc_commit(&k_empty[kst]);
      if (++kst == kKVStages) kst = 0, kph ^= 1;
      for (int j = 0; j < nkv; ++j) {
        const bool has_next = (j + 1) < nkv;
        if (!mbar_wait(&v_full[vst], vph, abort_flag)) goto mma_done;
        if (has_next && !mbar_wait(&k_full[kst], kph, abort_flag)) goto mma_done;
        for (int q = 0; q < kNQ; ++q) {
          if (!mbar_wait(&p_full[q], j & 1, abort_flag)) goto mma_done;
          tc_fence_after();
          issue_pv(q, vst, j > 0);
          if (has_next) {
            issue_qk(q, kst);
            tc_commit(&s_full[q]);
          } else {
            tc_commit(&o_full[q]);
          }
        }
        tc_commit(&v_empty[vst]);
        if (++vst == kKVStages) vst = 0, vph ^= 1;
        if (has_next) {
          tc_commit(&k_empty[kst]);
          if (++kst == kKVStages) kst = 0, kph ^= 1;
        }
      }
    }
  mma_done:;
  } else if (warp >= 4) {
    // ----------------------------------------------------------------- softmax
    reg_alloc<kSoftmaxRegs>();
    const int q = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_off + q * 128;
    const uint32_t t_o = tmem_base + lane_off + 256 + q * 128;
    const float cs = p.scale_log2;
    float m = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      if (!mbar_wait(&s_full[q], j & 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int valid = min(kTileKV, p.Sk - j * kTileKV);
      // the whole score row (128 fp32) in registers: four loads in flight, one wait
      uint32_t s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, reinterpret_cast<uint32_t(&)[32]>(s[c * 32]));
      tc_wait_ld();
      if (valid != kTileKV) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i >= valid) s[i] = 0xff800000u;  // -inf: masked keys of the last tile
      }
      float mx[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) mx[a] = __uint_as_float(s[a]);
#pragma unroll
      for (int i = 8; i < 128; ++i) mx[i & 7] = fmaxf(mx[i & 7], __uint_as_float(s[i]));
      const float mrow = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                               fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
      const float m_new = mrow * cs;
      if (j == 0) {
        m = m_new;
      } else if (__any_sync(0xffffffffu, m_new > m + 8.0f)) {
        const float m_upd = fmaxf(m, m_new);
        const float alpha = fast_exp2(m - m_upd);
        m = m_upd;
        l *= alpha;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(t_o + c * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(t_o + c * 32, r);
        }
      }
      // probabilities, written over S as packed bf16 (64 columns)
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(s[c * 32 + 2 * i]), cs, -m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(s[c * 32 + 2 * i + 1]), cs, -m));
          ls[i & 3] += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st16(t_s + c * 16, pk);
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[q]);
    }
    if (ok && mbar_wait(&o_full[q], 0, abort_flag)) {
      tc_fence_after();
      const int sq = q0 + q * kTileQ + row;
      const float inv = 1.0f / l;
      __nv_bfloat16* orow = p.o + static_cast<int64_t>(b) * p.o_stride_b + static_cast<int64_t>(sq) * p.o_stride_s +
                            static_cast<int64_t>(h) * p.o_stride_h;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(t_o + c * 32, r);
        tc_wait_ld();
        if (sq < p.Sq) {
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

extern "C" int dsb_flash_attn(const void* q, const void* k, const void* v, void* o, int B, int H, int Sq, int Sk,
                              int head_dim, int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                              int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_b,
                              int64_t v_stride_s, int64_t v_stride_h, int64_t o_stride_b, int64_t o_stride_s,
                              int64_t o_stride_h, float sm_scale, int* status, void* stream) {
  if (!q || !k || !v || !o || B <= 0 || H <= 0 || Sq < 0 || Sk <= 0) return DSB_ERR_ARG;
  if (head_dim != 128) return DSB_ERR_UNSUPPORTED;
  if (H > 65535 || B > 65535) return DSB_ERR_UNSUPPORTED;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al16(q) || !al16(k) || !al16(v) || !al16(o)) return DSB_ERR_ARG;
  const int64_t strides[] = {q_stride_s, q_stride_h, k_stride_s, k_stride_h, v_stride_s, v_stride_h,
                             o_stride_s, o_stride_h, q_stride_b, k_stride_b, v_stride_b, o_stride_b};
  for (int64_t s : strides)
    if (s < 0 || (s & 7)) return DSB_ERR_ARG;
  if (Sq == 0) return DSB_OK;
  AttnParams p;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_attn(&tq, p.q_pos, q, Sq, H, B, q_stride_s, q_stride_h, q_stride_b)) != DSB_OK) return rc;
  if ((rc = make_tmap_attn(&tk, p.k_pos, k, Sk, H, B, k_stride_s, k_stride_h, k_stride_b)) != DSB_OK) return rc;
  if ((rc = make_tmap_attn(&tv, p.v_pos, v, Sk, H, B, v_stride_s, v_stride_h, v_stride_b)) != DSB_OK) return rc;
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.o_stride_b = o_stride_b;
  p.o_stride_s = o_stride_s;
  p.o_stride_h = o_stride_h;
  p.Sq = Sq;
  p.Sk = Sk;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.status = status;
  DSB_ENSURE_SMEM(flash_attn_kernel, kAttnSmem);
  dim3 grid((Sq + kNQ * kTileQ - 1) / (kNQ * kTileQ), H, B);
  flash_attn_kernel<<<grid, kAttnThreads, kAttnSmem, reinterpret_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}
