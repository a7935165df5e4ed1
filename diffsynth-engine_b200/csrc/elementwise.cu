// Bandwidth-bound kernels of the DiT step: AdaLN (LayerNorm + shift/scale,
// optionally emitting the FP8/INT8 operand of the next GEMM with its per-row
// scale), gate-residual, per-head and full-width QK-RMSNorm with RoPE, row
// quantisation, the M=1 modulation/embedding GEMV, and the flow-match Euler
// update.  All global accesses are 128-bit; one CTA (or one warp) owns a row
// so every reduction stays on chip.
#include "common.cuh"
#include "dsb.h"

namespace dsb {

constexpr int kRowThreads = 128;

struct alignas(16) bf16x8 {
  uint32_t u[4];
};

__device__ __forceinline__ float block_sum_128(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}
__device__ __forceinline__ float block_max_128(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  return fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  // satfinite conversion; inputs are already scaled into [-448, 448].
  __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}
__device__ __forceinline__ uint32_t pack_s8x4(float a, float b, float c, float d) {
  // round-half-even, clamp to [-127, 127]
  int ia = max(-127, min(127, __float2int_rn(a)));
  int ib = max(-127, min(127, __float2int_rn(b)));
  int ic = max(-127, min(127, __float2int_rn(c)));
  int id = max(-127, min(127, __float2int_rn(d)));
  return (ia & 0xff) | ((ib & 0xff) << 8) | ((ic & 0xff) << 16) | ((id & 0xff) << 24);
}

// Per-row scale shared by the quantising kernels: amax / qmax, with a floor so
// an all-zero row gives scale 1 (and a zero payload) instead of a division by 0.
__device__ __forceinline__ float row_scale_from_amax(float amax, float qmax) {
  return amax > 0.f ? amax / qmax : 1.0f;
}

// ------------------------------------------------------------ row prefetch ring
// The row quantiser walks rows with persistent CTAs and keeps the next kRing-1 rows of each CTA in flight while one
// is processed: thread t copies its own 16-byte vectors (t, t+T, t+2T, ...) of a row into a slot of a shared-memory
// ring with cp.async and later reads exactly those vectors back itself, so the ring needs no barrier - only
// cp.async.wait_group.  Measured at 32760 x 5120: 146 -> 107 us (3.4 -> 4.7 TB/s).  The LayerNorm and RMSNorm kernels
// keep one row per CTA: they are bound by instruction issue (fp32 math on bf16 data plus per-column parameters), not
// by bytes in flight - with the ring they were no faster (RMSNorm) or slower (LayerNorm: fewer resident warps).
constexpr int kRing = 4;
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// SRC(vi) -> global address of 16-byte vector vi of the row; THREADS = blockDim.x
template <int NV, int THREADS, typename SRC>
__device__ __forceinline__ void ring_issue(uint4* ring, int slot, int nvec, bool row_exists, SRC src) {
  if (row_exists) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * THREADS;
      if (vi < nvec) cp_async16(ring + (slot * NV + i) * THREADS + threadIdx.x, src(vi));
    }
  }
  cp_async_commit();  // an empty group keeps the group count in step with the iteration count
}
template <int NV, int THREADS>
__device__ __forceinline__ uint4 ring_read(const uint4* ring, int slot, int i) {
  return ring[(slot * NV + i) * THREADS + threadIdx.x];
}
// grid of a persistent row kernel: the CTAs the device holds at once, at most one per row
template <auto KERNEL>
static int persistent_grid(int threads, size_t smem, int rows) {
  static int per_sm[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (per_sm[dev] == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, KERNEL, threads, smem) != cudaSuccess || n <= 0) n = 1;
    per_sm[dev] = n;
  }
  const int64_t cap = static_cast<int64_t>(per_sm[dev]) * sm_count();
  return static_cast<int>(rows < cap ? rows : cap);
}

// ------------------------------------------------------------ ln_modulate
// y = LayerNorm(x; eps, no affine) * (1 + scale[d]) + shift[d]
// NV = 128-bit vectors per thread (row width D <= 128 * 8 * NV).
// OUT: 0 bf16, 1 e4m3 + row scale, 2 int8 + row scale.
template <int NV, int OUT>
__global__ void __launch_bounds__(kRowThreads, (NV <= 6 ? 7 : 4)) ln_modulate_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x,
                                                                  const float* __restrict__ shift_a,
                                                                  const float* __restrict__ scale_a, int split_row,
                                                                  const float* __restrict__ shift_b,
                                                                  const float* __restrict__ scale_b, void* __restrict__ y,
                                                                  int64_t ld_y, float* __restrict__ row_scale, int M,
                                                                  int D, float eps) {
  __shared__ float red[4];
  const int row = blockIdx.x;
  if (row >= M) return;
  // rows below split_row take the first modulation vectors, the rest the second (text rows precede image rows
  // in the joint hidden-state buffer, each stream with its own AdaLN output)
  const float* shift = row < split_row ? shift_a : shift_b;
  const float* scale = row < split_row ? scale_a : scale_b;
  const int nvec = D >> 3;
  const __nv_bfloat16* xr = x + static_cast<int64_t>(row) * ld_x;
  // The row stays in registers as 4 x float2 per 128-bit vector and every pass uses the packed fp32 instructions
  // (two lanes per issue slot): the kernel is bound by instruction issue, not by bytes in flight - at 5120-wide rows
  // the scalar form spent ~600 issue slots per thread and row.  Same operations in the same order as the scalar form:
  // ((x - mean) * rstd) * (1 + scale) + shift with the last two fused.
  float2 v[NV][4];
  float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * kRowThreads;
    if (vi < nvec) {
      bf16x8 p = *reinterpret_cast<const bf16x8*>(xr + vi * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i][j] = unpack_bf16x2(p.u[j]);
        s2 = __fadd2_rn(s2, v[i][j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[i][j] = make_float2(0.f, 0.f);
    }
  }
  const float mean = block_sum_128(s2.x + s2.y, red) / static_cast<float>(D);
  const float2 nmean = make_float2(-mean, -mean);
  float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * kRowThreads;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i][j] = __fadd2_rn(v[i][j], nmean);   // the centred value is kept for the last pass
        q2 = __ffma2_rn(v[i][j], v[i][j], q2);
      }
    }
  }
  const float var = block_sum_128(q2.x + q2.y, red) / static_cast<float>(D);
  const float rstd = rsqrtf(var + eps);
  const float2 rstd2 = make_float2(rstd, rstd), one2 = make_float2(1.f, 1.f);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * kRowThreads;
    if (vi < nvec) {
      const float4 sc0 = *reinterpret_cast<const float4*>(scale + vi * 8);
      const float4 sc1 = *reinterpret_cast<const float4*>(scale + vi * 8 + 4);
      const float4 sh0 = *reinterpret_cast<const float4*>(shift + vi * 8);
      const float4 sh1 = *reinterpret_cast<const float4*>(shift + vi * 8 + 4);
      const float2 sc[4] = {make_float2(sc0.x, sc0.y), make_float2(sc0.z, sc0.w), make_float2(sc1.x, sc1.y),
                            make_float2(sc1.z, sc1.w)};
      const float2 sh[4] = {make_float2(sh0.x, sh0.y), make_float2(sh0.z, sh0.w), make_float2(sh1.x, sh1.y),
                            make_float2(sh1.z, sh1.w)};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 o = __ffma2_rn(__fmul2_rn(v[i][j], rstd2), __fadd2_rn(one2, sc[j]), sh[j]);
        v[i][j] = o;
        amax = fmaxf(amax, fmaxf(fabsf(o.x), fabsf(o.y)));
      }
    }
  }
  if constexpr (OUT == 0) {
    __nv_bfloat16* yr = reinterpret_cast<__nv_bfloat16*>(y) + static_cast<int64_t>(row) * ld_y;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * kRowThreads;
      if (vi < nvec) {
        bf16x8 p;
#pragma unroll
        for (int j = 0; j < 4; ++j) p.u[j] = pack_bf16x2(v[i][j].x, v[i][j].y);
        *reinterpret_cast<bf16x8*>(yr + vi * 8) = p;
      }
    }
  } else {
    amax = block_max_128(amax, red);
    const float qmax = (OUT == 1) ? 448.0f : 127.0f;
    const float sc = row_scale_from_amax(amax, qmax);
    const float inv = 1.0f / sc;
    const float2 inv2 = make_float2(inv, inv);
    if (threadIdx.x == 0) row_scale[row] = sc;
    uint8_t* yr = reinterpret_cast<uint8_t*>(y) + static_cast<int64_t>(row) * ld_y;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * kRowThreads;
      if (vi < nvec) {
        float2 t[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = __fmul2_rn(v[i][j], inv2);
        uint2 p;
        if constexpr (OUT == 1) {
          p.x = pack_e4m3x4(t[0].x, t[0].y, t[1].x, t[1].y);
          p.y = pack_e4m3x4(t[2].x, t[2].y, t[3].x, t[3].y);
        } else {
          p.x = pack_s8x4(t[0].x, t[0].y, t[1].x, t[1].y);
          p.y = pack_s8x4(t[2].x, t[2].y, t[3].x, t[3].y);
        }
        *reinterpret_cast<uint2*>(yr + vi * 8) = p;
      }
    }
  }
}

template <int OUT>
static int launch_ln_modulate(const void* x, int64_t ld_x, const float* shift, const float* scale, int split_row,
                              const float* shift_b, const float* scale_b, void* y, int64_t ld_y, float* row_scale,
                              int M, int D, float eps, cudaStream_t st) {
  const int nv = (D / 8 + kRowThreads - 1) / kRowThreads;
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
#define DSB_LN_CASE(NV)                                                                                         \
  case NV:                                                                                                      \
    ln_modulate_kernel<NV, OUT><<<M, kRowThreads, 0, st>>>(xp, ld_x, shift, scale, split_row, shift_b, scale_b, y, ld_y, \
                                                           row_scale, M, D, eps);                                  \
    break;
  switch (nv) {
    DSB_LN_CASE(1) DSB_LN_CASE(2) DSB_LN_CASE(3) DSB_LN_CASE(4) DSB_LN_CASE(5) DSB_LN_CASE(6) DSB_LN_CASE(7)
    DSB_LN_CASE(8)
    default:
      return DSB_ERR_UNSUPPORTED;
  }
#undef DSB_LN_CASE
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

// ---------------------------------------------------------- gate_residual
// out = x + gate[d] * y   (gate == nullptr: out = x + y)
__global__ void __launch_bounds__(256) gate_residual_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x,
                                                            const __nv_bfloat16* __restrict__ y, int64_t ld_y,
                                                            const float* __restrict__ gate,
                                                            __nv_bfloat16* __restrict__ out, int64_t ld_o, int M,
                                                            int D) {
  const int nvec = D >> 3;
  const int64_t total = static_cast<int64_t>(M) * nvec;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / nvec;
    const int c = static_cast<int>(i - r * nvec) * 8;
    bf16x8 a = *reinterpret_cast<const bf16x8*>(x + r * ld_x + c);
    bf16x8 b = *reinterpret_cast<const bf16x8*>(y + r * ld_y + c);
    float g[8];
    if (gate) {
      const float4 g0 = *reinterpret_cast<const float4*>(gate + c);
      const float4 g1 = *reinterpret_cast<const float4*>(gate + c + 4);
      g[0] = g0.x, g[1] = g0.y, g[2] = g0.z, g[3] = g0.w, g[4] = g1.x, g[5] = g1.y, g[6] = g1.z, g[7] = g1.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = 1.f;
    }
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fa = unpack_bf16x2(a.u[j]), fb = unpack_bf16x2(b.u[j]);
      o.u[j] = pack_bf16x2(fa.x + g[2 * j] * fb.x, fa.y + g[2 * j + 1] * fb.y);
    }
    *reinterpret_cast<bf16x8*>(out + r * ld_o + c) = o;
  }
}

// ---------------------------------------------------- rmsnorm_rope_heads
// Per-head RMSNorm (head_dim 128, weight[128]) followed by RoPE on adjacent
// pairs, in place, for `nsel` head groups (q and k) of a [S, ld] buffer.
// One warp per (token, head).  rope == nullptr skips the rotation.
// rope row for token s is rope[(rope_row0 + s) * 64 + j] = (cos, sin).
__global__ void __launch_bounds__(256) rmsnorm_rope_heads_kernel(__nv_bfloat16* __restrict__ buf, int64_t ld, int S,
                                                                 int H, int nsel, const float* __restrict__ w_q,
                                                                 const float* __restrict__ w_k,
                                                                 const float2* __restrict__ rope, int rope_row0,
                                                                 float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int64_t wid = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int64_t total = static_cast<int64_t>(S) * nsel * H;
  if (wid >= total) return;
  const int s = static_cast<int>(wid / (nsel * H));
  const int hh = static_cast<int>(wid - static_cast<int64_t>(s) * (nsel * H));  // [0, nsel*H): q heads then k heads
  const float* w = (hh < H) ? w_q : w_k;
  __nv_bfloat16* p = buf + static_cast<int64_t>(s) * ld + hh * 128 + lane * 4;
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
  float ss = a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
  ss = warp_sum(ss);
  const float r = rsqrtf(ss * (1.0f / 128.0f) + eps);
  const float4 wv = *reinterpret_cast<const float4*>(w + lane * 4);
  float x0 = a.x * r * wv.x, x1 = a.y * r * wv.y, x2 = b.x * r * wv.z, x3 = b.y * r * wv.w;
  if (rope) {
    const float2* rr = rope + (static_cast<int64_t>(rope_row0) + s) * 64 + lane * 2;
    const float2 c0 = rr[0], c1 = rr[1];
    const float y0 = c0.x * x0 - c0.y * x1, y1 = c0.y * x0 + c0.x * x1;
    const float y2 = c1.x * x2 - c1.y * x3, y3 = c1.y * x2 + c1.x * x3;
    x0 = y0, x1 = y1, x2 = y2, x3 = y3;
  }
  uint2 o;
  o.x = pack_bf16x2(x0, x1);
  o.y = pack_bf16x2(x2, x3);
  *reinterpret_cast<uint2*>(p) = o;
}

// ------------------------------------------------------ rmsnorm_full_rope
// RMSNorm over the whole row (all heads, width D = H*128) with weight[D],
// then per-head RoPE (same 64 (cos,sin) pairs for every head of a token).
// One CTA per row; in place.  rope == nullptr skips the rotation.
// The output may be "chunked": column c of row m goes to out[(c / chunk_cols) * chunk_stride + m * ld_out +
// c % chunk_cols] - the per-peer-contiguous send layout of a head/sequence all-to-all ([P][rows][D/P]).
template <int NV>
__global__ void __launch_bounds__(kRowThreads) rmsnorm_full_rope_kernel(const __nv_bfloat16* buf, int64_t ld,
                                                                        __nv_bfloat16* out, int64_t ld_out,
                                                                        int chunk_cols, int64_t chunk_stride, int M,
                                                                        int D, const float* __restrict__ w,
                                                                        const float2* __restrict__ rope,
                                                                        int rope_row0, float eps) {
  __shared__ float red[4];
  const int row = blockIdx.x;
  if (row >= M) return;
  const int nvec = D >> 3;
  const __nv_bfloat16* xr = buf + static_cast<int64_t>(row) * ld;
  // this row's RoPE factors (512 bytes, used only after the reduction) start their trip from L2 now
  if (rope && threadIdx.x < 4)
    asm volatile("prefetch.global.L1 [%0];" ::"l"(rope + (static_cast<int64_t>(rope_row0) + row) * 64 + threadIdx.x * 16));
  // packed fp32 arithmetic (two lanes per issue slot), operations in the order of the scalar form: (x * r) * w
  float2 v[NV][4];
  float2 ss2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * kRowThreads;
    if (vi < nvec) {
      bf16x8 p = *reinterpret_cast<const bf16x8*>(xr + vi * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i][j] = unpack_bf16x2(p.u[j]);
        ss2 = __ffma2_rn(v[i][j], v[i][j], ss2);
      }
    }
  }
  const float r = rsqrtf(block_sum_128(ss2.x + ss2.y, red) / static_cast<float>(D) + eps);
  const float2 r2 = make_float2(r, r);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * kRowThreads;
    if (vi < nvec) {
      const float4 w0 = *reinterpret_cast<const float4*>(w + vi * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(w + vi * 8 + 4);
      const float2 ww[4] = {make_float2(w0.x, w0.y), make_float2(w0.z, w0.w), make_float2(w1.x, w1.y),
                            make_float2(w1.z, w1.w)};
      float2 o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = __fmul2_rn(__fmul2_rn(v[i][j], r2), ww[j]);
      if (rope) {
        const int pair0 = ((vi * 8) & 127) >> 1;  // pair index inside the head
        const float2* rr = rope + (static_cast<int64_t>(rope_row0) + row) * 64 + pair0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 c = rr[j];
          const float a = o[j].x, b = o[j].y;
          o[j].x = c.x * a - c.y * b;
          o[j].y = c.y * a + c.x * b;
        }
      }
      bf16x8 p;
#pragma unroll
      for (int j = 0; j < 4; ++j) p.u[j] = pack_bf16x2(o[j].x, o[j].y);
      const int col = vi * 8;
      const int ck = col / chunk_cols;
      *reinterpret_cast<bf16x8*>(out + ck * chunk_stride + static_cast<int64_t>(row) * ld_out + (col - ck * chunk_cols)) =
          p;
    }
  }
}

// ------------------------------------------------------------- quant_rows
// bf16 [M, K] -> e4m3 or int8 [M, K] plus row_scale[M] (dynamic, amax based).
// Rows of up to 256 * NV 16-byte vectors (K <= 8192 with NV = 4): persistent CTAs with the prefetch ring, the row is
// read once and held in registers between the amax pass and the quantising pass.
template <int OUT, int NV>
__global__ void __launch_bounds__(256) quant_rows_ring_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x,
                                                              int chunk_cols, int64_t chunk_stride,
                                                              uint8_t* __restrict__ y, int64_t ld_y,
                                                              float* __restrict__ row_scale, int M, int K) {
  __shared__ float red[8];
  extern __shared__ uint4 ring[];
  const int nvec = K >> 3;
  const int stride = gridDim.x;
  // chunked input: column c of row m lives at x[(c / chunk_cols) * chunk_stride + m * ld_x + c % chunk_cols]
  // (what a sequence/head all-to-all delivers: [P][rows][K/P]); chunk_cols == K is the plain row-major case
  auto issue = [&](int slot, int r) {
    const __nv_bfloat16* xrow = x + static_cast<int64_t>(r) * ld_x;
    ring_issue<NV, 256>(ring, slot, nvec, r < M, [&](int vi) {
      const int col = vi * 8;
      const int ck = col / chunk_cols;
      return xrow + ck * chunk_stride + (col - ck * chunk_cols);
    });
  };
#pragma unroll
  for (int k = 0; k < kRing - 1; ++k) issue(k, blockIdx.x + k * stride);
  int it = 0;
  for (int row = blockIdx.x; row < M; row += stride, ++it) {
    issue((it + kRing - 1) % kRing, row + (kRing - 1) * stride);
    cp_async_wait<kRing - 1>();
    const int slot = it % kRing;
    float f[NV][8];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (threadIdx.x + i * 256 < nvec) {
        const uint4 pu = ring_read<NV, 256>(ring, slot, i);
        const uint32_t u[4] = {pu.x, pu.y, pu.z, pu.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = unpack_bf16x2(u[j]);
          f[i][2 * j] = t.x, f[i][2 * j + 1] = t.y;
          amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
        }
      }
    }
    amax = warp_max(amax);
    __syncthreads();  // the previous row's readers of red[] are done
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
    const float qmax = (OUT == 1) ? 448.0f : 127.0f;
    const float sc = row_scale_from_amax(amax, qmax);
    const float inv = 1.0f / sc;
    if (threadIdx.x == 0) row_scale[row] = sc;
    uint8_t* yr = y + static_cast<int64_t>(row) * ld_y;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * 256;
      if (vi < nvec) {
        uint2 o;
        if constexpr (OUT == 1) {
          o.x = pack_e4m3x4(f[i][0] * inv, f[i][1] * inv, f[i][2] * inv, f[i][3] * inv);
          o.y = pack_e4m3x4(f[i][4] * inv, f[i][5] * inv, f[i][6] * inv, f[i][7] * inv);
        } else {
          o.x = pack_s8x4(f[i][0] * inv, f[i][1] * inv, f[i][2] * inv, f[i][3] * inv);
          o.y = pack_s8x4(f[i][4] * inv, f[i][5] * inv, f[i][6] * inv, f[i][7] * inv);
        }
        *reinterpret_cast<uint2*>(yr + vi * 8) = o;
      }
    }
  }
}

// Wider rows: one CTA per row, the row is read twice (the second read is served by L1/L2).
template <int OUT>
__global__ void __launch_bounds__(256) quant_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x,
                                                         int chunk_cols, int64_t chunk_stride,
                                                         uint8_t* __restrict__ y, int64_t ld_y,
                                                         float* __restrict__ row_scale, int M, int K) {
  __shared__ float red[8];
  const int row = blockIdx.x;
  if (row >= M) return;
  const int nvec = K >> 3;
  // chunked input: column c of row m lives at x[(c / chunk_cols) * chunk_stride + m * ld_x + c % chunk_cols]
  // (what a sequence/head all-to-all delivers: [P][rows][K/P]); chunk_cols == K is the plain row-major case
  const __nv_bfloat16* xrow = x + static_cast<int64_t>(row) * ld_x;
  auto src = [&](int vi) {
    const int col = vi * 8;
    const int ck = col / chunk_cols;
    return xrow + ck * chunk_stride + (col - ck * chunk_cols);
  };
  float amax = 0.f;
  for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
    bf16x8 p = *reinterpret_cast<const bf16x8*>(src(vi));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(p.u[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float qmax = (OUT == 1) ? 448.0f : 127.0f;
  const float sc = row_scale_from_amax(amax, qmax);
  const float inv = 1.0f / sc;
  if (threadIdx.x == 0) row_scale[row] = sc;
  uint8_t* yr = y + static_cast<int64_t>(row) * ld_y;
  for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
    bf16x8 p = *reinterpret_cast<const bf16x8*>(src(vi));
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = unpack_bf16x2(p.u[j]);
      f[2 * j] = t.x * inv;
      f[2 * j + 1] = t.y * inv;
    }
    uint2 o;
    if constexpr (OUT == 1) {
      o.x = pack_e4m3x4(f[0], f[1], f[2], f[3]);
      o.y = pack_e4m3x4(f[4], f[5], f[6], f[7]);
    } else {
      o.x = pack_s8x4(f[0], f[1], f[2], f[3]);
      o.y = pack_s8x4(f[4], f[5], f[6], f[7]);
    }
    *reinterpret_cast<uint2*>(yr + vi * 8) = o;
  }
}

// ------------------------------------------------------------- patchify / unpatchify
// Latents [C, F, 2*gh, 2*gw] (bf16, contiguous) <-> token rows: token t = (f*gh + y)*gw + z holds the 2 x 2 patch
// (rows 2y, 2y+1; columns 2z, 2z+1) of every channel of frame f.
// patchify: feature c*4 + py*2 + pz (what a Conv3d / Conv2d with kernel = stride = (1,2,2) sees as one Linear input
// row); rows [row0, row0 + n_rows) are written, rows past the last token as zeros; OUT 0 writes bf16, 1 / 2 write the
// row quantised to e4m3 / int8 with its dynamic scale (the rule of quant_rows_kernel).  One warp per token, a lane
// per (channel, patch row) pair = two adjacent latents = one 4-byte load.
template <int OUT>
__global__ void __launch_bounds__(256) patchify_kernel(const __nv_bfloat16* __restrict__ lat, int C, int F, int gh, int gw,
                                                       int row0, int n_rows, void* __restrict__ out, int64_t ld_out,
                                                       float* __restrict__ row_scale) {
  constexpr int kMaxPairs = 8;  // pairs per lane: C*2 <= 256
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= n_rows) return;
  const int64_t t = static_cast<int64_t>(row0) + warp;
  const int64_t tokens = static_cast<int64_t>(F) * gh * gw;
  const int npairs = C * 2;
  float2 v[kMaxPairs];
  float amax = 0.f;
  const int z = static_cast<int>(t % gw), y = static_cast<int>((t / gw) % gh), f = static_cast<int>(t / (static_cast<int64_t>(gw) * gh));
#pragma unroll
  for (int i = 0; i < kMaxPairs; ++i) {
    const int pr = lane + i * 32;  // pair index = c*2 + py
    v[i] = make_float2(0.f, 0.f);
    if (pr < npairs && t < tokens) {
      const int c = pr >> 1, py = pr & 1;
      const int64_t src = ((static_cast<int64_t>(c) * F + f) * (2 * gh) + 2 * y + py) * (2 * gw) + 2 * z;
      v[i] = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(lat + src));
      amax = fmaxf(amax, fmaxf(fabsf(v[i].x), fabsf(v[i].y)));
    }
  }
  if constexpr (OUT == 0) {
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(out) + static_cast<int64_t>(warp) * ld_out;
#pragma unroll
    for (int i = 0; i < kMaxPairs; ++i) {
      const int pr = lane + i * 32;
      if (pr < npairs) *reinterpret_cast<uint32_t*>(orow + pr * 2) = pack_bf16x2(v[i].x, v[i].y);
    }
  } else {
    amax = warp_max(amax);
    const float sc = row_scale_from_amax(amax, OUT == 1 ? 448.0f : 127.0f);
    const float inv = 1.0f / sc;
    if (lane == 0) row_scale[warp] = sc;
    uint8_t* orow = reinterpret_cast<uint8_t*>(out) + static_cast<int64_t>(warp) * ld_out;
#pragma unroll
    for (int i = 0; i < kMaxPairs; ++i) {
      const int pr = lane + i * 32;
      if (pr < npairs) {
        const uint32_t q = (OUT == 1) ? pack_e4m3x4(v[i].x * inv, v[i].y * inv, 0.f, 0.f)
                                      : pack_s8x4(v[i].x * inv, v[i].y * inv, 0.f, 0.f);
        *reinterpret_cast<uint16_t*>(orow + pr * 2) = static_cast<uint16_t>(q & 0xffffu);
      }
    }
  }
}

// unpatchify: token rows [tokens, >= C*4] -> latents [C, F, 2*gh, 2*gw].  c_fastest = 1: feature (py*2 + pz)*C + c
// (Wan head, "(x y z c)", models/wan/wan_dit.py:307-317); 0: feature c*4 + py*2 + pz (Flux, flux_dit.py:369-374).
// One thread per horizontally adjacent output pair.
__global__ void __launch_bounds__(256) unpatchify_kernel(const __nv_bfloat16* __restrict__ tok, int64_t ld_tok, int C, int F,
                                                         int gh, int gw, int c_fastest, __nv_bfloat16* __restrict__ out) {
  const int64_t total = static_cast<int64_t>(C) * F * (2 * gh) * gw;  // pairs
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int z = static_cast<int>(i % gw);
    int64_t r = i / gw;
    const int yy = static_cast<int>(r % (2 * gh));
    r /= 2 * gh;
    const int f = static_cast<int>(r % F);
    const int c = static_cast<int>(r / F);
    const int y = yy >> 1, py = yy & 1;
    const __nv_bfloat16* row = tok + ((static_cast<int64_t>(f) * gh + y) * gw + z) * ld_tok;
    const int f0 = c_fastest ? (py * 2) * C + c : c * 4 + py * 2;
    const int f1 = c_fastest ? (py * 2 + 1) * C + c : c * 4 + py * 2 + 1;
    __nv_bfloat162 o;
    o.x = row[f0];
    o.y = row[f1];
    *reinterpret_cast<__nv_bfloat162*>(out + i * 2) = o;
  }
}

// ------------------------------------------------------------- cast_quant
// bf16 [M, D] -> e4m3 (saturating, round-to-nearest-even) or int8 (round-half-even, clamp +-127) with no scale:
// the values are already in the operand's units.  Fills the K-extension columns of a quantised activation
// buffer with the LoRA down-projection.  SPLIT (e4m3 only): writes [head | remainder | head] at column offsets
// 0, D, 2D, where head = e4m3(x) and remainder = e4m3(x - head), so that the pair carries about 7 mantissa bits.
__device__ __forceinline__ float e4m3_value(float v) {
  const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  const __half_raw h = __nv_cvt_fp8_to_halfraw(q, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

template <int OUT, bool SPLIT>
__global__ void __launch_bounds__(256) cast_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x,
                                                         uint8_t* __restrict__ y, int64_t ld_y, int M, int D) {
  const int nvec = D >> 3;
  const int64_t total = static_cast<int64_t>(M) * nvec;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / nvec;
    const int c = static_cast<int>(i - r * nvec) * 8;
    bf16x8 p = *reinterpret_cast<const bf16x8*>(x + r * ld_x + c);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = unpack_bf16x2(p.u[j]);
      f[2 * j] = t.x, f[2 * j + 1] = t.y;
    }
    uint2 o;
    if constexpr (OUT == 1) {
      o.x = pack_e4m3x4(f[0], f[1], f[2], f[3]);
      o.y = pack_e4m3x4(f[4], f[5], f[6], f[7]);
    } else {
      o.x = pack_s8x4(f[0], f[1], f[2], f[3]);
      o.y = pack_s8x4(f[4], f[5], f[6], f[7]);
    }
    uint8_t* dst = y + r * ld_y + c;
    *reinterpret_cast<uint2*>(dst) = o;
    if constexpr (SPLIT) {
      *reinterpret_cast<uint2*>(dst + 2 * D) = o;
      float g[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = f[j] - e4m3_value(f[j]);
      uint2 lo;
      lo.x = pack_e4m3x4(g[0], g[1], g[2], g[3]);
      lo.y = pack_e4m3x4(g[4], g[5], g[6], g[7]);
      *reinterpret_cast<uint2*>(dst + D) = lo;
    }
  }
}

// ---------------------------------------------------------- dequant_q8_0
// GGUF Q8_0 -> bf16: one thread per block of 32 weights (34 bytes: fp16 d, 32 x int8).  A block is only 2-byte
// aligned, so it is read as 17 halfwords; the thread writes 64 contiguous bytes.  out = bf16(bf16(d) * q), the
// product the reference forms when its compute dtype is bf16.
__global__ void __launch_bounds__(256) dequant_q8_0_kernel(const uint16_t* __restrict__ raw, int64_t row_halfwords,
                                                           __nv_bfloat16* __restrict__ out, int64_t ld_out, int N,
                                                           int blocks_per_row) {
  const int64_t total = static_cast<int64_t>(N) * blocks_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = i / blocks_per_row;
    const int kb = static_cast<int>(i - n * blocks_per_row);
    const uint16_t* src = raw + n * row_halfwords + static_cast<int64_t>(kb) * 17;
    const __half_raw hr = {__ldg(src)};
    const float d = __bfloat162float(__float2bfloat16_rn(__half2float(*reinterpret_cast<const __half*>(&hr))));
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint16_t w = __ldg(src + 1 + j);
      const float q0 = static_cast<float>(static_cast<int8_t>(w & 0xffu));
      const float q1 = static_cast<float>(static_cast<int8_t>(w >> 8));
      o[j] = pack_bf16x2(d * q0, d * q1);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + n * ld_out + static_cast<int64_t>(kb) * 32);
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
  }
}

// ---------------------------------------------------------- dequant_q4_k
// GGUF Q4_K -> bf16: super-blocks of 256 weights in 144 bytes (fp16 d, fp16 dmin, 12 bytes of eight 6-bit scales and
// eight 6-bit mins, 128 bytes of 4-bit quants).  One thread per sub-block of 32 weights.  The arithmetic repeats the
// reference's bf16 evaluation order: (bf16(d) * sc) rounded, (bf16(dmin) * m) rounded, (that * q) rounded, minus.
__device__ __forceinline__ float rbf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__global__ void __launch_bounds__(256) dequant_q4_k_kernel(const uint8_t* __restrict__ raw, int64_t row_bytes,
                                                           __nv_bfloat16* __restrict__ out, int64_t ld_out, int N,
                                                           int subs_per_row) {
  const int64_t total = static_cast<int64_t>(N) * subs_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = i / subs_per_row;
    const int sb = static_cast<int>(i - n * subs_per_row);  // sub-block inside the row
    const int j = sb & 7;
    const uint8_t* blk = raw + n * row_bytes + static_cast<int64_t>(sb >> 3) * 144;
    const uint4 head = __ldg(reinterpret_cast<const uint4*>(blk));  // d, dmin, 12 scale bytes
    const __half_raw hd = {static_cast<unsigned short>(head.x & 0xffffu)};
    const __half_raw hm = {static_cast<unsigned short>(head.x >> 16)};
    const float d = rbf(__half2float(*reinterpret_cast<const __half*>(&hd)));
    const float dmin = rbf(__half2float(*reinterpret_cast<const __half*>(&hm)));
    const uint32_t w[3] = {head.y, head.z, head.w};
    auto sbyte = [&](int k) { return (w[k >> 2] >> ((k & 3) * 8)) & 0xffu; };
    uint32_t sc, mn;
    if (j < 4) {
      sc = sbyte(j) & 63u;
      mn = sbyte(j + 4) & 63u;
    } else {
      sc = (sbyte(j + 4) & 15u) | ((sbyte(j - 4) >> 6) << 4);
      mn = (sbyte(j + 4) >> 4) | ((sbyte(j) >> 6) << 4);
    }
    const float dsc = rbf(d * static_cast<float>(sc));
    const float dm = rbf(dmin * static_cast<float>(mn));
    const uint4* qp = reinterpret_cast<const uint4*>(blk + 16 + (j >> 1) * 32);
    const int shift = (j & 1) * 4;
    uint4* dst = reinterpret_cast<uint4*>(out + n * ld_out + static_cast<int64_t>(sb) * 32);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint4 qv = __ldg(qp + h);
      const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
      uint32_t o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t b0 = (qw[k >> 1] >> ((k & 1) * 16)) & 0xffu, b1 = (qw[k >> 1] >> ((k & 1) * 16 + 8)) & 0xffu;
        const float q0 = static_cast<float>((b0 >> shift) & 15u), q1 = static_cast<float>((b1 >> shift) & 15u);
        o[k] = pack_bf16x2(rbf(dsc * q0) - dm, rbf(dsc * q1) - dm);
      }
      dst[2 * h] = make_uint4(o[0], o[1], o[2], o[3]);
      dst[2 * h + 1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
  }
}

// ------------------------------------------------------ GGUF block formats (generic path)
// One thread turns 16 consecutive weights of a row into bf16, for every block format the reference dequantises
// (utils/gguf.py:171-368).  Arithmetic and rounding follow the reference with a bf16 compute dtype: the fp16 block
// scales are rounded to bf16, and every product and every sum is rounded to bf16 again, in the reference's order.
// Block sizes such as 18, 22, 110 or 210 bytes leave nothing aligned, so the bytes are fetched one by one (this
// runs once per weight, when a checkpoint is attached).
enum : int { GG_Q4_0 = 2, GG_Q4_1 = 3, GG_Q5_0 = 6, GG_Q5_1 = 7, GG_Q8_0 = 8, GG_Q2_K = 10, GG_Q3_K = 11, GG_Q4_K = 12,
             GG_Q5_K = 13, GG_Q6_K = 14 };

__device__ __forceinline__ float gg_f16(const uint8_t* p) {   // fp16 field -> bf16-rounded float
  const __half_raw h = {static_cast<unsigned short>(__ldg(p) | (static_cast<unsigned>(__ldg(p + 1)) << 8))};
  return rbf(__half2float(*reinterpret_cast<const __half*>(&h)));
}
__device__ __forceinline__ uint32_t gg_u32(const uint8_t* p) {
  return __ldg(p) | (static_cast<uint32_t>(__ldg(p + 1)) << 8) | (static_cast<uint32_t>(__ldg(p + 2)) << 16) |
         (static_cast<uint32_t>(__ldg(p + 3)) << 24);
}
// the eight 6-bit (scale, min) pairs of a K-quant super-block (get_scale_min, gguf.py:158-168)
__device__ __forceinline__ void gg_k_scale(const uint8_t* s, int j, uint32_t* sc, uint32_t* mn) {
  if (j < 4) {
    *sc = __ldg(s + j) & 63u;
    *mn = __ldg(s + j + 4) & 63u;
  } else {
    *sc = (__ldg(s + j + 4) & 15u) | ((__ldg(s + j - 4) >> 6) << 4);
    *mn = (__ldg(s + j + 4) >> 4) | ((__ldg(s + j) >> 6) << 4);
  }
}

template <int T>
__device__ __forceinline__ void gg_deq16(const uint8_t* blk, int v0, float (&o)[16]) {
  if constexpr (T == GG_Q4_0 || T == GG_Q4_1 || T == GG_Q5_0 || T == GG_Q5_1) {
    constexpr bool kHasMin = (T == GG_Q4_1 || T == GG_Q5_1), kFive = (T == GG_Q5_0 || T == GG_Q5_1);
    const float d = gg_f16(blk), m = kHasMin ? gg_f16(blk + 2) : 0.f;
    const uint8_t* hp = blk + (kHasMin ? 4 : 2);
    const uint8_t* qs = hp + (kFive ? 4 : 0);
    const uint32_t qh = kFive ? gg_u32(hp) : 0u;
    const int shift = v0 >= 16 ? 4 : 0;   // values 0..15 are the low nibbles of the 16 bytes, 16..31 the high ones
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      int q = (__ldg(qs + i) >> shift) & 15;
      if (kFive) q |= static_cast<int>((qh >> (v0 + i)) & 1u) << 4;
      if (T == GG_Q4_0) q -= 8;
      if (T == GG_Q5_0) q -= 16;
      const float dq = rbf(d * static_cast<float>(q));
      o[i] = kHasMin ? rbf(dq + m) : dq;
    }
  } else if constexpr (T == GG_Q8_0) {
    const float d = gg_f16(blk);
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = rbf(d * static_cast<float>(static_cast<int8_t>(__ldg(blk + 2 + v0 + i))));
  } else if constexpr (T == GG_Q2_K) {
    const uint32_t s = __ldg(blk + (v0 >> 4));
    const float dl = rbf(gg_f16(blk + 80) * static_cast<float>(s & 15u));
    const float ml = rbf(gg_f16(blk + 82) * static_cast<float>(s >> 4));
    const uint8_t* qs = blk + 16 + (v0 >> 7) * 32 + (v0 & 31);
    const int sh = ((v0 & 127) >> 5) * 2;
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = rbf(rbf(dl * static_cast<float>((__ldg(qs + i) >> sh) & 3)) - ml);
  } else if constexpr (T == GG_Q3_K) {
    const int k = v0 >> 4;
    const uint8_t* s = blk + 96;
    const int low = k < 8 ? (__ldg(s + k) & 15) : (__ldg(s + k - 8) >> 4);
    const int high = (__ldg(s + 8 + (k & 3)) >> (2 * (k >> 2))) & 3;
    const float dl = rbf(gg_f16(blk + 108) * static_cast<float>((low | (high << 4)) - 32));
    const uint8_t* qs = blk + 32 + (v0 >> 7) * 32 + (v0 & 31);
    const uint8_t* hm = blk + (v0 & 31);
    const int sh = ((v0 & 127) >> 5) * 2, hb = v0 >> 5;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int q = ((__ldg(qs + i) >> sh) & 3) - ((((__ldg(hm + i) >> hb) & 1) ^ 1) << 2);
      o[i] = rbf(dl * static_cast<float>(q));
    }
  } else if constexpr (T == GG_Q4_K || T == GG_Q5_K) {
    const int j = v0 >> 5;
    uint32_t sc, mn;
    gg_k_scale(blk + 4, j, &sc, &mn);
    const float dsc = rbf(gg_f16(blk) * static_cast<float>(sc)), dm = rbf(gg_f16(blk + 2) * static_cast<float>(mn));
    const uint8_t* qs = blk + (T == GG_Q5_K ? 48 : 16) + (j >> 1) * 32 + (v0 & 31);
    const uint8_t* qh = blk + 16 + (v0 & 31);
    const int sh = (j & 1) * 4;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      int q = (__ldg(qs + i) >> sh) & 15;
      if (T == GG_Q5_K) q |= ((__ldg(qh + i) >> j) & 1) << 4;
      o[i] = rbf(rbf(dsc * static_cast<float>(q)) - dm);
    }
  } else {  // GG_Q6_K
    const int h = v0 >> 7, r = v0 & 127;
    const float dl = rbf(gg_f16(blk + 208) * static_cast<float>(static_cast<int8_t>(__ldg(blk + 192 + (v0 >> 4)))));
    const uint8_t* ql = blk + h * 64 + (r & 63);
    const uint8_t* qh = blk + 128 + h * 32 + (r & 31);
    const int sl = (r >> 6) * 4, shh = (r >> 5) * 2;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int q = (((__ldg(ql + i) >> sl) & 15) | (((__ldg(qh + i) >> shh) & 3) << 4)) - 32;
      o[i] = rbf(dl * static_cast<float>(q));
    }
  }
}

template <int T>
__global__ void __launch_bounds__(256) dequant_gguf_kernel(const uint8_t* __restrict__ raw, int64_t row_bytes,
                                                           __nv_bfloat16* __restrict__ out, int64_t ld_out, int N, int K,
                                                           int type_size, int block_size) {
  const int groups = K >> 4;
  const int64_t total = static_cast<int64_t>(N) * groups;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = i / groups;
    const int col = static_cast<int>(i - n * groups) << 4;
    const uint8_t* blk = raw + n * row_bytes + static_cast<int64_t>(col / block_size) * type_size;
    float o[16];
    gg_deq16<T>(blk, col % block_size, o);
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) w[k] = pack_bf16x2(o[2 * k], o[2 * k + 1]);
    uint4* dst = reinterpret_cast<uint4*>(out + n * ld_out + col);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// ------------------------------------------------------------------- gemv
// y[n] = (sum_k W[n,k] * f(x[k])) * w_scale[n or 0] + bias[n].  The activation vector is staged once per CTA
// in shared memory; each warp walks groups of four consecutive rows so that every 64-byte read of the
// activations serves four weight rows and four 16-byte weight loads per lane are in flight.
// WFMT: 0 bf16, 1 e4m3, 2 int8.  act_in: DSB_ACT_NONE or DSB_ACT_SILU on x; act_out: any DSB_ACT_* on y.
template <int WFMT>
__device__ __forceinline__ void dequant16(const uint4& p, float (&w)[16]) {
  const uint32_t u[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if constexpr (WFMT == 1) {
      const __half2_raw h0 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(u[j] & 0xffffu), __NV_E4M3);
      const __half2_raw h1 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(u[j] >> 16), __NV_E4M3);
      const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&h0));
      const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&h1));
      w[4 * j] = f0.x, w[4 * j + 1] = f0.y, w[4 * j + 2] = f1.x, w[4 * j + 3] = f1.y;
    } else {
      const int v = static_cast<int>(u[j]);
      w[4 * j] = static_cast<float>(static_cast<int8_t>(v & 0xff));
      w[4 * j + 1] = static_cast<float>(static_cast<int8_t>((v >> 8) & 0xff));
      w[4 * j + 2] = static_cast<float>(static_cast<int8_t>((v >> 16) & 0xff));
      w[4 * j + 3] = static_cast<float>(static_cast<int8_t>((v >> 24) & 0xff));
    }
  }
}

template <int WFMT>
__global__ void __launch_bounds__(256) gemv_kernel(const void* __restrict__ W, int64_t ld_w_bytes,
                                                   const float* __restrict__ x, const float* __restrict__ w_scale,
                                                   int w_scale_stride, const float* __restrict__ bias,
                                                   float* __restrict__ y, int N, int K, int act_in, int act_out,
                                                   int accumulate) {
  extern __shared__ float xs[];
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    float t = x[k];
    xs[k] = act_in == DSB_ACT_SILU ? silu(t) : t;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  constexpr int R = 4;
  constexpr int EPL = (WFMT == 0) ? 8 : 16;  // elements per 16-byte load
  const int groups = (N + R - 1) / R;
  for (int g = blockIdx.x * warps + (threadIdx.x >> 5); g < groups; g += gridDim.x * warps) {
    const int n0 = g * R;
    const uint8_t* wr[R];
#pragma unroll
    for (int r = 0; r < R; ++r)
      wr[r] = reinterpret_cast<const uint8_t*>(W) + static_cast<int64_t>(min(n0 + r, N - 1)) * ld_w_bytes;
    float acc[R] = {0.f, 0.f, 0.f, 0.f};
    for (int k = lane * EPL; k < K; k += 32 * EPL) {
      uint4 p[R];
#pragma unroll
      for (int r = 0; r < R; ++r) p[r] = *reinterpret_cast<const uint4*>(wr[r] + k * (WFMT == 0 ? 2 : 1));
      float xv[EPL];
#pragma unroll
      for (int e = 0; e < EPL; e += 4) {
        const float4 t = *reinterpret_cast<const float4*>(xs + k + e);
        xv[e] = t.x, xv[e + 1] = t.y, xv[e + 2] = t.z, xv[e + 3] = t.w;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if constexpr (WFMT == 0) {
          const uint32_t u[4] = {p[r].x, p[r].y, p[r].z, p[r].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16x2(u[j]);
            acc[r] += f.x * xv[2 * j] + f.y * xv[2 * j + 1];
          }
        } else {
          float w[16];
          dequant16<WFMT>(p[r], w);
#pragma unroll
          for (int e = 0; e < 16; ++e) acc[r] += w[e] * xv[e];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
    if (lane < R && n0 + lane < N) {
      const int n = n0 + lane;
      float a = acc[0];
      if (lane == 1) a = acc[1];
      if (lane == 2) a = acc[2];
      if (lane == 3) a = acc[3];
      const float sc = w_scale ? w_scale[static_cast<int64_t>(n) * w_scale_stride] : 1.0f;
      float o = a * sc + (bias ? bias[n] : 0.f);
      if (act_out == DSB_ACT_SILU) o = silu(o);
      if (act_out == DSB_ACT_GELU_TANH) o = gelu_tanh(o);
      if (act_out == DSB_ACT_GELU) o = gelu_erf(o);
      y[n] = accumulate ? y[n] + o : o;
    }
  }
}

// ------------------------------------------------------------ euler step
// out = cast(latents_fp32 + model_out * dt); optional inpaint blend
// model_out' = model_out * mask + init * (1 - mask) applied first.
__global__ void __launch_bounds__(256) euler_step_kernel(const __nv_bfloat16* __restrict__ latents,
                                                         const __nv_bfloat16* __restrict__ model_out,
                                                         const __nv_bfloat16* __restrict__ init,
                                                         const __nv_bfloat16* __restrict__ mask, float dt,
                                                         __nv_bfloat16* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float m = __bfloat162float(model_out[i]);
    if (mask) {
      // the reference evaluates the blend in the model-output dtype
      const float k = __bfloat162float(mask[i]);
      const float a = __bfloat162float(__float2bfloat16(m * k));
      const float om = __bfloat162float(__float2bfloat16(1.0f - k));
      const float b = __bfloat162float(__float2bfloat16(__bfloat162float(init[i]) * om));
      m = __bfloat162float(__float2bfloat16(a + b));
    }
    // bf16 tensor times a 0-dim fp32 sigma difference stays bf16 in the reference
    const float step = __bfloat162float(__float2bfloat16(m * dt));
    out[i] = __float2bfloat16(__bfloat162float(latents[i]) + step);
  }
}
__global__ void __launch_bounds__(256) euler_step_f32_kernel(const float* __restrict__ latents,
                                                             const float* __restrict__ model_out,
                                                             const float* __restrict__ init,
                                                             const float* __restrict__ mask, float dt,
                                                             float* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float m = model_out[i];
    if (mask) m = m * mask[i] + init[i] * (1.0f - mask[i]);
    out[i] = latents[i] + m * dt;
  }
}

// ------------------------------------------------------- timestep embedding
// mode 0: fp32 sinusoid [cos | sin], freq_i = exp(-ln(10000) * i / half)      (Flux)
// mode 1: fp64 sinusoid [cos | sin], freq_i = 10000^(-i / half)               (Wan)
__global__ void timestep_embedding_kernel(const float* __restrict__ t, int n, int dim, float t_scale, int mode,
                                          int round_bf16, float* __restrict__ out) {
  const int half = dim / 2;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * half) return;
  const int r = idx / half, i = idx - r * half;
  float c, s;
  if (mode == 0) {
    const float exponent = -9.210340371976184f * static_cast<float>(i) / static_cast<float>(half);
    const float ang = (t[r] * t_scale) * expf(exponent);
    c = cosf(ang), s = sinf(ang);
  } else {
    const double ang = static_cast<double>(t[r] * t_scale) * pow(10000.0, -static_cast<double>(i) / half);
    c = static_cast<float>(cos(ang)), s = static_cast<float>(sin(ang));
  }
  if (round_bf16) {
    c = __bfloat162float(__float2bfloat16(c));
    s = __bfloat162float(__float2bfloat16(s));
  }
  out[r * dim + i] = c;
  out[r * dim + half + i] = s;
}

// ------------------------------------------------- CFG combine + euler step
// model_out = neg + cfg * (pos - neg), then the flow-match Euler update, in one pass.  The bf16 form rounds where
// the reference's tensor expression rounds (each elementwise op yields a bf16 tensor).
__global__ void __launch_bounds__(256) cfg_euler_step_kernel(const __nv_bfloat16* __restrict__ latents,
                                                             const __nv_bfloat16* __restrict__ pos,
                                                             const __nv_bfloat16* __restrict__ neg, float cfg, float dt,
                                                             __nv_bfloat16* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float p = __bfloat162float(pos[i]), q = __bfloat162float(neg[i]);
    const float m = rbf(q + rbf(cfg * rbf(p - q)));
    out[i] = __float2bfloat16(__bfloat162float(latents[i]) + rbf(m * dt));
  }
}
__global__ void __launch_bounds__(256) cfg_euler_step_f32_kernel(const float* __restrict__ latents,
                                                                 const float* __restrict__ pos,
                                                                 const float* __restrict__ neg, float cfg, float dt,
                                                                 float* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float m = neg[i] + cfg * (pos[i] - neg[i]);
    out[i] = latents[i] + m * dt;
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace dsb

using namespace dsb;

extern "C" {

int dsb_ln_modulate(const void* x, int64_t ld_x, const float* shift, const float* scale, void* y, int64_t ld_y,
                    float* row_scale, int M, int D, float eps, int out_fmt, void* stream) {
  return dsb_ln_modulate2(x, ld_x, shift, scale, M, shift, scale, y, ld_y, row_scale, M, D, eps, out_fmt, stream);
}

int dsb_ln_modulate2(const void* x, int64_t ld_x, const float* shift, const float* scale, int split_row,
                     const float* shift_b, const float* scale_b, void* y, int64_t ld_y, float* row_scale, int M, int D,
                     float eps, int out_fmt, void* stream) {
  if (M == 0 && D > 0 && !(D & 7)) return DSB_OK;
  if (!shift_b || !scale_b || !aligned16(shift_b) || !aligned16(scale_b)) return DSB_ERR_ARG;
  if (!x || !shift || !scale || !y || M < 0 || D <= 0 || (D & 7) || (ld_x & 7) || !aligned16(x) || !aligned16(y) ||
      !aligned16(shift) || !aligned16(scale))
    return DSB_ERR_ARG;
  if (out_fmt != DSB_FMT_BF16 && !row_scale) return DSB_ERR_ARG;
  if ((out_fmt == DSB_FMT_BF16 && (ld_y & 7)) || (out_fmt != DSB_FMT_BF16 && (ld_y & 15))) return DSB_ERR_ARG;
  if (M == 0) return DSB_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (out_fmt) {
    case DSB_FMT_BF16:
      return launch_ln_modulate<0>(x, ld_x, shift, scale, split_row, shift_b, scale_b, y, ld_y, row_scale, M, D, eps, st);
    case DSB_FMT_E4M3:
      return launch_ln_modulate<1>(x, ld_x, shift, scale, split_row, shift_b, scale_b, y, ld_y, row_scale, M, D, eps, st);
    case DSB_FMT_INT8:
      return launch_ln_modulate<2>(x, ld_x, shift, scale, split_row, shift_b, scale_b, y, ld_y, row_scale, M, D, eps, st);
    default:
      return DSB_ERR_ARG;
  }
}

int dsb_gate_residual(const void* x, int64_t ld_x, const void* y, int64_t ld_y, const float* gate, void* out,
                      int64_t ld_o, int M, int D, void* stream) {
  if (M == 0 && D > 0 && !(D & 7)) return DSB_OK;
  if (!x || !y || !out || M < 0 || D <= 0 || (D & 7) || (ld_x & 7) || (ld_y & 7) || (ld_o & 7) || !aligned16(x) ||
      !aligned16(y) || !aligned16(out) || (gate && !aligned16(gate)))
    return DSB_ERR_ARG;
  if (M == 0) return DSB_OK;
  const int64_t total = static_cast<int64_t>(M) * (D / 8);
  int blocks = static_cast<int>((total + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  gate_residual_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ld_x, reinterpret_cast<const __nv_bfloat16*>(y), ld_y, gate,
      reinterpret_cast<__nv_bfloat16*>(out), ld_o, M, D);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_rmsnorm_rope_heads(void* buf, int64_t ld, int S, int H, int head_dim, int nsel, const float* w_q,
                           const float* w_k, const float* rope, int rope_row0, float eps, void* stream) {
  if (!buf || !w_q || S < 0 || H <= 0 || head_dim != 128 || (nsel != 1 && nsel != 2) || (nsel == 2 && !w_k) ||
      (ld & 7) || !aligned16(buf) || !aligned16(w_q) || (w_k && !aligned16(w_k)) || (rope && !aligned16(rope)))
    return DSB_ERR_ARG;
  if (S == 0) return DSB_OK;
  const int64_t total = static_cast<int64_t>(S) * nsel * H;
  const int blocks = static_cast<int>((total + 7) / 8);
  rmsnorm_rope_heads_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(buf), ld, S, H, nsel, w_q, w_k ? w_k : w_q,
      reinterpret_cast<const float2*>(rope), rope_row0, eps);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_rmsnorm_full(const void* x, int64_t ld_x, void* out, int64_t ld_out, int out_chunk_cols,
                     int64_t out_chunk_stride, int M, int D, const float* w, const float* rope, int rope_row0,
                     float eps, void* stream) {
  if (M == 0 && D > 0 && !(D & 127)) return DSB_OK;
  if (!x || !out || !w || M < 0 || D <= 0 || (D & 127) || (ld_x & 7) || (ld_out & 7) || !aligned16(x) ||
      !aligned16(out) || !aligned16(w) || (rope && !aligned16(rope)))
    return DSB_ERR_ARG;
  if (out_chunk_cols == 0) out_chunk_cols = D, out_chunk_stride = 0;
  if (out_chunk_cols < 0 || (out_chunk_cols & 7) || (D % out_chunk_cols) || (out_chunk_stride & 7)) return DSB_ERR_ARG;
  const int nv = (D / 8 + kRowThreads - 1) / kRowThreads;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
  const float2* rp = reinterpret_cast<const float2*>(rope);
#define DSB_RMS_CASE(NV)                                                                                          \
  case NV:                                                                                                        \
    rmsnorm_full_rope_kernel<NV><<<M, kRowThreads, 0, st>>>(b, ld_x, o, ld_out, out_chunk_cols, out_chunk_stride, \
                                                           M, D, w, rp, rope_row0, eps);                        \
    break;
  switch (nv) {
    DSB_RMS_CASE(1) DSB_RMS_CASE(2) DSB_RMS_CASE(3) DSB_RMS_CASE(4) DSB_RMS_CASE(5) DSB_RMS_CASE(6) DSB_RMS_CASE(7)
    DSB_RMS_CASE(8)
    default:
      return DSB_ERR_UNSUPPORTED;
  }
#undef DSB_RMS_CASE
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

static int quant_rows_impl(const void* x, int64_t ld_x, int chunk_cols, int64_t chunk_stride, void* y, int64_t ld_y,
                           float* row_scale, int M, int K, int out_fmt, void* stream);

int dsb_quant_rows(const void* x, int64_t ld_x, void* y, int64_t ld_y, float* row_scale, int M, int K, int out_fmt,
                   void* stream) {
  return quant_rows_impl(x, ld_x, K, 0, y, ld_y, row_scale, M, K, out_fmt, stream);
}

int dsb_quant_rows_chunked(const void* x, int64_t ld_x, int chunk_cols, int64_t chunk_stride, void* y, int64_t ld_y,
                           float* row_scale, int M, int K, int out_fmt, void* stream) {
  if (chunk_cols <= 0 || (chunk_cols & 7) || K <= 0 || (K % chunk_cols) || (chunk_stride & 7)) return DSB_ERR_ARG;
  return quant_rows_impl(x, ld_x, chunk_cols, chunk_stride, y, ld_y, row_scale, M, K, out_fmt, stream);
}

}  // extern "C"

static int quant_rows_impl(const void* x, int64_t ld_x, int chunk_cols, int64_t chunk_stride, void* y, int64_t ld_y,
                           float* row_scale, int M, int K, int out_fmt, void* stream) {
  if (M == 0 && K > 0 && !(K & 7)) return DSB_OK;
  if (!x || !y || !row_scale || M < 0 || K <= 0 || (K & 7) || (ld_x & 7) || (ld_y & 15) || !aligned16(x) ||
      !aligned16(y))
    return DSB_ERR_ARG;
  if (M == 0) return DSB_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  uint8_t* yp = reinterpret_cast<uint8_t*>(y);
  if (out_fmt != DSB_FMT_E4M3 && out_fmt != DSB_FMT_INT8) return DSB_ERR_ARG;
  const int nv = (K / 8 + 255) / 256;
#define DSB_QR_RING(OUT, NV)                                                                                  \
  {                                                                                                           \
    constexpr size_t smem = static_cast<size_t>(kRing) * NV * 256 * 16;                                       \
    DSB_ENSURE_SMEM((quant_rows_ring_kernel<OUT, NV>), static_cast<int>(smem));                               \
    const int grid = persistent_grid<quant_rows_ring_kernel<OUT, NV>>(256, smem, M);                          \
    if (grid <= 0) return DSB_ERR_CUDA;                                                                       \
    quant_rows_ring_kernel<OUT, NV><<<grid, 256, smem, st>>>(xp, ld_x, chunk_cols, chunk_stride, yp, ld_y,    \
                                                             row_scale, M, K);                                \
  }
#define DSB_QR_FMT(OUT)                                                                                       \
  switch (nv) {                                                                                               \
    case 1: DSB_QR_RING(OUT, 1) break;                                                                        \
    case 2: DSB_QR_RING(OUT, 2) break;                                                                        \
    case 3: DSB_QR_RING(OUT, 3) break;                                                                        \
    case 4: DSB_QR_RING(OUT, 4) break;                                                                        \
    default:                                                                                                  \
      quant_rows_kernel<OUT><<<M, 256, 0, st>>>(xp, ld_x, chunk_cols, chunk_stride, yp, ld_y, row_scale, M, K); \
  }
  if (out_fmt == DSB_FMT_E4M3) {
    DSB_QR_FMT(1)
  } else {
    DSB_QR_FMT(2)
  }
#undef DSB_QR_FMT
#undef DSB_QR_RING
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

extern "C" {

int dsb_dequant_q8_0(const void* blocks, int64_t row_bytes, int N, int K, void* out, int64_t ld_out, void* stream) {
  if (N < 0 || K <= 0 || (K & 31) || (row_bytes & 1) || row_bytes < static_cast<int64_t>(K / 32) * 34 || (ld_out & 7))
    return DSB_ERR_ARG;
  if (N == 0) return DSB_OK;
  if (!blocks || !out || (reinterpret_cast<uintptr_t>(blocks) & 1u) || !aligned16(out)) return DSB_ERR_ARG;
  const int bpr = K / 32;
  const int64_t total = static_cast<int64_t>(N) * bpr;
  int nblk = static_cast<int>((total + 255) / 256);
  const int cap = sm_count() * 16;
  if (nblk > cap) nblk = cap;
  dequant_q8_0_kernel<<<nblk, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint16_t*>(blocks), row_bytes / 2, reinterpret_cast<__nv_bfloat16*>(out), ld_out, N, bpr);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_dequant_q4_k(const void* blocks, int64_t row_bytes, int N, int K, void* out, int64_t ld_out, void* stream) {
  if (N < 0 || K <= 0 || (K & 255) || (row_bytes & 15) || row_bytes < static_cast<int64_t>(K / 256) * 144 || (ld_out & 7))
    return DSB_ERR_ARG;
  if (N == 0) return DSB_OK;
  if (!blocks || !out || !aligned16(blocks) || !aligned16(out)) return DSB_ERR_ARG;
  const int spr = K / 32;
  const int64_t total = static_cast<int64_t>(N) * spr;
  int nblk = static_cast<int>((total + 255) / 256);
  const int cap = sm_count() * 16;
  if (nblk > cap) nblk = cap;
  dequant_q4_k_kernel<<<nblk, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(blocks), row_bytes, reinterpret_cast<__nv_bfloat16*>(out), ld_out, N, spr);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_dequant_gguf(int ggml_type, const void* blocks, int64_t row_bytes, int N, int K, void* out, int64_t ld_out,
                     void* stream) {
  int tsz, bsz;
  switch (ggml_type) {
    case GG_Q4_0: tsz = 18, bsz = 32; break;
    case GG_Q4_1: tsz = 20, bsz = 32; break;
    case GG_Q5_0: tsz = 22, bsz = 32; break;
    case GG_Q5_1: tsz = 24, bsz = 32; break;
    case GG_Q8_0: tsz = 34, bsz = 32; break;
    case GG_Q2_K: tsz = 84, bsz = 256; break;
    case GG_Q3_K: tsz = 110, bsz = 256; break;
    case GG_Q4_K: tsz = 144, bsz = 256; break;
    case GG_Q5_K: tsz = 176, bsz = 256; break;
    case GG_Q6_K: tsz = 210, bsz = 256; break;
    default: return DSB_ERR_UNSUPPORTED;
  }
  if (N < 0 || K <= 0 || (K % bsz) || (ld_out & 7) || row_bytes < static_cast<int64_t>(K / bsz) * tsz) return DSB_ERR_ARG;
  if (N == 0) return DSB_OK;
  if (!blocks || !out || !aligned16(out)) return DSB_ERR_ARG;
  const int64_t total = static_cast<int64_t>(N) * (K >> 4);
  int nblk = static_cast<int>((total + 255) / 256);
  const int cap = sm_count() * 16;
  if (nblk > cap) nblk = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const uint8_t* rp = reinterpret_cast<const uint8_t*>(blocks);
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(out);
#define DSB_GG(T) case T: dequant_gguf_kernel<T><<<nblk, 256, 0, st>>>(rp, row_bytes, op, ld_out, N, K, tsz, bsz); break;
  switch (ggml_type) {
    DSB_GG(GG_Q4_0) DSB_GG(GG_Q4_1) DSB_GG(GG_Q5_0) DSB_GG(GG_Q5_1) DSB_GG(GG_Q8_0) DSB_GG(GG_Q2_K) DSB_GG(GG_Q3_K)
    DSB_GG(GG_Q4_K) DSB_GG(GG_Q5_K) DSB_GG(GG_Q6_K)
  }
#undef DSB_GG
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_cast_quant(const void* x, int64_t ld_x, void* y, int64_t ld_y, int M, int D, int out_fmt, int split,
                   void* stream) {
  if (M < 0 || D <= 0 || (D & 7) || (ld_x & 7) || (ld_y & 7)) return DSB_ERR_ARG;
  if (split && out_fmt != DSB_FMT_E4M3) return DSB_ERR_ARG;
  if (M == 0) return DSB_OK;
  if (!x || !y || !aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 7u)) return DSB_ERR_ARG;
  const int64_t total = static_cast<int64_t>(M) * (D >> 3);
  int blocks = static_cast<int>((total + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  uint8_t* yp = reinterpret_cast<uint8_t*>(y);
  if (out_fmt == DSB_FMT_E4M3 && split)
    cast_quant_kernel<1, true><<<blocks, 256, 0, st>>>(xp, ld_x, yp, ld_y, M, D);
  else if (out_fmt == DSB_FMT_E4M3)
    cast_quant_kernel<1, false><<<blocks, 256, 0, st>>>(xp, ld_x, yp, ld_y, M, D);
  else if (out_fmt == DSB_FMT_INT8)
    cast_quant_kernel<2, false><<<blocks, 256, 0, st>>>(xp, ld_x, yp, ld_y, M, D);
  else
    return DSB_ERR_ARG;
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_gemv(const void* W, int64_t ld_w, int w_fmt, const float* x, const float* w_scale, int w_scale_stride,
             const float* bias, float* y, int N, int K, int act_in, int act_out, int accumulate, void* stream) {
  if (!W || !x || !y || N < 0 || K <= 0 || !aligned16(W)) return DSB_ERR_ARG;
  const int esz = (w_fmt == DSB_FMT_BF16) ? 2 : 1;
  const int kq = (w_fmt == DSB_FMT_BF16) ? 8 : 16;
  if ((K % kq) || ((ld_w * esz) & 15)) return DSB_ERR_ARG;
  if (static_cast<size_t>(K) * 4 > 96 * 1024) return DSB_ERR_UNSUPPORTED;
  if (N == 0) return DSB_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t smem = static_cast<size_t>(K) * 4;
  const int64_t ldb = ld_w * esz;
  int blocks = (N + 31) / 32;  // one warp per group of four rows
#define DSB_GEMV(F)                                                                                             \
  {                                                                                                             \
    auto kern = gemv_kernel<F>;                                                                                 \
    DSB_ENSURE_SMEM(kern, 96 * 1024);                                                                           \
    int occ = 1;                                                                                                \
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, 256, smem) != cudaSuccess || occ < 1) occ = 1; \
    if (blocks > occ * sm_count()) blocks = occ * sm_count(); /* exactly the resident set: no second wave */     \
    gemv_kernel<F><<<blocks, 256, smem, st>>>(W, ldb, x, w_scale, w_scale_stride, bias, y, N, K, act_in, act_out, \
                                               accumulate);                                                       \
  }
  if (w_fmt == DSB_FMT_BF16) DSB_GEMV(0)
  else if (w_fmt == DSB_FMT_E4M3) DSB_GEMV(1)
  else if (w_fmt == DSB_FMT_INT8) DSB_GEMV(2)
  else return DSB_ERR_ARG;
#undef DSB_GEMV
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_timestep_embedding(const float* t, int n, int dim, float t_scale, int mode, int round_bf16, float* out,
                           void* stream) {
  if (!t || !out || n <= 0 || dim <= 0 || (dim & 1) || (mode != 0 && mode != 1)) return DSB_ERR_ARG;
  const int total = n * (dim / 2);
  timestep_embedding_kernel<<<(total + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      t, n, dim, t_scale, mode, round_bf16, out);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_cfg_euler_step(const void* latents, const void* pos, const void* neg, float cfg_scale, float dt, void* out,
                       int64_t n, int is_f32, void* stream) {
  if (!latents || !pos || !neg || !out || n < 0) return DSB_ERR_ARG;
  if (n == 0) return DSB_OK;
  int blocks = static_cast<int>((n + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (is_f32)
    cfg_euler_step_f32_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(latents),
                                                      reinterpret_cast<const float*>(pos),
                                                      reinterpret_cast<const float*>(neg), cfg_scale, dt,
                                                      reinterpret_cast<float*>(out), n);
  else
    cfg_euler_step_kernel<<<blocks, 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(latents), reinterpret_cast<const __nv_bfloat16*>(pos),
        reinterpret_cast<const __nv_bfloat16*>(neg), cfg_scale, dt, reinterpret_cast<__nv_bfloat16*>(out), n);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_patchify(const void* latents, int C, int F, int gh, int gw, int row0, int n_rows, int out_fmt, void* out,
                 int64_t ld_out, float* row_scale, void* stream) {
  if (C <= 0 || C > 128 || F <= 0 || gh <= 0 || gw <= 0 || row0 < 0 || n_rows < 0) return DSB_ERR_ARG;
  if (n_rows == 0) return DSB_OK;
  if (!latents || !out || (reinterpret_cast<uintptr_t>(latents) & 3u) || ld_out < C * 4) return DSB_ERR_ARG;
  const int blocks = (n_rows + 7) / 8;  // 8 warps = 8 tokens per CTA
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16* lat = reinterpret_cast<const __nv_bfloat16*>(latents);
  if (out_fmt == DSB_FMT_BF16) {
    if ((reinterpret_cast<uintptr_t>(out) & 3u) || (ld_out & 1)) return DSB_ERR_ARG;
    patchify_kernel<0><<<blocks, 256, 0, st>>>(lat, C, F, gh, gw, row0, n_rows, out, ld_out, nullptr);
  } else if (out_fmt == DSB_FMT_E4M3 || out_fmt == DSB_FMT_INT8) {
    if (!row_scale || (reinterpret_cast<uintptr_t>(out) & 1u) || (ld_out & 1)) return DSB_ERR_ARG;
    if (out_fmt == DSB_FMT_E4M3)
      patchify_kernel<1><<<blocks, 256, 0, st>>>(lat, C, F, gh, gw, row0, n_rows, out, ld_out, row_scale);
    else
      patchify_kernel<2><<<blocks, 256, 0, st>>>(lat, C, F, gh, gw, row0, n_rows, out, ld_out, row_scale);
  } else {
    return DSB_ERR_ARG;
  }
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_unpatchify(const void* tokens, int64_t ld_tok, int C, int F, int gh, int gw, int c_fastest, void* out,
                   void* stream) {
  if (C <= 0 || F <= 0 || gh <= 0 || gw <= 0 || ld_tok < C * 4) return DSB_ERR_ARG;
  if (!tokens || !out || (reinterpret_cast<uintptr_t>(out) & 3u) || (reinterpret_cast<uintptr_t>(tokens) & 1u))
    return DSB_ERR_ARG;
  const int64_t total = static_cast<int64_t>(C) * F * (2 * gh) * gw;
  int blocks = static_cast<int>((total + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  unpatchify_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(tokens), ld_tok, C, F, gh, gw, c_fastest ? 1 : 0,
      reinterpret_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

int dsb_euler_step(const void* latents, const void* model_out, const void* init, const void* mask, float dt, void* out,
                   int64_t n, int is_f32, void* stream) {
  if (!latents || !model_out || !out || n < 0 || (mask && !init)) return DSB_ERR_ARG;
  if (n == 0) return DSB_OK;
  int blocks = static_cast<int>((n + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (is_f32)
    euler_step_f32_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(latents),
                                                  reinterpret_cast<const float*>(model_out),
                                                  reinterpret_cast<const float*>(init),
                                                  reinterpret_cast<const float*>(mask), dt,
                                                  reinterpret_cast<float*>(out), n);
  else
    euler_step_kernel<<<blocks, 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(latents), reinterpret_cast<const __nv_bfloat16*>(model_out),
        reinterpret_cast<const __nv_bfloat16*>(init), reinterpret_cast<const __nv_bfloat16*>(mask), dt,
        reinterpret_cast<__nv_bfloat16*>(out), n);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

}  // extern "C"
