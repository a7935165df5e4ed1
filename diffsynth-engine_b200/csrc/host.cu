// Host-side helpers shared by the kernels (tensor-map encoding through the
// runtime's driver entry point, SM count cache) and the weight prepack.
#include <mutex>

#include "common.cuh"
#include "dsb.h"

namespace dsb {

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  });
  return fn;
}

int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows,
                 uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return DSB_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || (pitch_bytes & 15u) || box_cols * elem_bytes != 128u ||
      box_rows > 256u || rows == 0 || cols == 0)
    return DSB_ERR_ARG;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DSB_OK : DSB_ERR_CUDA;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ------------------------------------------------------------ weight prepack
template <bool SRC_BF16>
__device__ __forceinline__ float load_w(const void* W, int64_t idx) {
  if constexpr (SRC_BF16)
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(W)[idx]);
  else
    return reinterpret_cast<const float*>(W)[idx];
}

// amax over the whole matrix (atomicMax on the bit pattern of a non-negative float)
template <bool SRC_BF16>
__global__ void __launch_bounds__(256) amax_all_kernel(const void* __restrict__ W, int64_t ld, int N, int K,
                                                       float* __restrict__ work) {
  float a = 0.f;
  const int64_t total = static_cast<int64_t>(N) * K;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / K;
    a = fmaxf(a, fabsf(load_w<SRC_BF16>(W, r * ld + (i - r * K))));
  }
  a = warp_max(a);
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(work), __float_as_int(a));
}

// One CTA per output row: per-channel amax (or the global one from `work`), then quantise.
template <bool SRC_BF16, int FMT>
__global__ void __launch_bounds__(256) pack_rows_kernel(const void* __restrict__ W, int64_t ld, uint8_t* __restrict__ Wq,
                                                        int64_t ld_q, float* __restrict__ scales, int N, int K,
                                                        int per_channel, const float* __restrict__ work) {
  __shared__ float red[8];
  const int n = blockIdx.x;
  const float qmax = (FMT == DSB_FMT_E4M3) ? 448.0f : 127.0f;
  float amax;
  if (per_channel) {
    float a = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) a = fmaxf(a, fabsf(load_w<SRC_BF16>(W, n * ld + k)));
    a = warp_max(a);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  } else {
    amax = *work;
  }
  const float s = amax > 0.f ? amax / qmax : 1.0f;
  if (threadIdx.x == 0) {
    if (per_channel) scales[n] = s;
    else if (n == 0) scales[0] = s;
  }
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    // true division, as the oracle does; then clamp, then convert
    float q = load_w<SRC_BF16>(W, n * ld + k) / s;
    q = fminf(fmaxf(q, -qmax), qmax);
    uint8_t o;
    if constexpr (FMT == DSB_FMT_E4M3)
      o = static_cast<uint8_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3));
    else
      o = static_cast<uint8_t>(static_cast<int8_t>(__float2int_rn(q)));
    Wq[n * ld_q + k] = o;
  }
}

// The give-up path of the bounded waits, exercised on purpose: one warp waits on a barrier that nothing ever
// arrives at, with a short cycle budget; a second warp stands for the other roles of a real kernel, polls the abort
// flag and leaves when it is raised.  Both meet at the common exit, where the status word is written - the same
// sequence the GEMM and attention kernels run when a wait of theirs runs out.
__global__ void __launch_bounds__(64) wait_timeout_selftest_kernel(long long limit_cycles, int* status, int* left) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    if (threadIdx.x == 0) mbar_wait_limit(&bar, 0, abort_flag, limit_cycles);   // nobody arrives: must give up
  } else if (threadIdx.x == 32) {
    // a neighbour role: its own (long) wait on the same barrier ends as soon as the first role has given up
    const bool done = mbar_wait(&bar, 0, abort_flag);
    if (left) *left = done ? 0 : 1;
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && status) atomicCAS(status, 0, DSB_ERR_TIMEOUT);
}

// A barrier among the ranks of a sequence-parallel group (one process and one GPU per rank).  flags.f[r] is rank r's
// flag array (one int per rank) in memory that every rank has mapped.  Thread t tells rank t "rank `rank` has
// reached `epoch`" (slot [rank] of rank t's array) and then waits until rank t has told this rank the same.  The
// system-scope fence before the signal orders everything earlier launches of this stream wrote - to any rank's
// memory - before it; the acquire on the waiting side makes those writes visible to later launches of the waiter.
// Epochs only grow, so a rank that is already one barrier ahead never blocks a slower one.  The wait is bounded.
struct RankFlags {
  int* f[8];
};
__global__ void __launch_bounds__(32) rank_barrier_kernel(RankFlags flags, int n, int rank, int epoch,
                                                          long long limit_cycles, int* status) {
  const int t = threadIdx.x;
  if (t >= n) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags.f[t] + rank), "r"(epoch) : "memory");
  const int* mine = flags.f[rank] + t;
  // after one barrier of this process has timed out the run is lost anyway: later barriers do not wait again
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
  const long long t0 = clock64();
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v - epoch >= 0) return;
    if (clock64() - t0 > limit_cycles) break;
    __nanosleep(100);
  }
  if (status) atomicCAS(status, 0, DSB_ERR_TIMEOUT);
}

}  // namespace dsb

using namespace dsb;

extern "C" int dsb_version(void) { return 100; }

extern "C" int dsb_rank_barrier(int* const* flags, int n_ranks, int rank, int epoch, long long limit_cycles,
                                int* status, void* stream) {
  if (!flags || n_ranks < 1 || n_ranks > 8 || rank < 0 || rank >= n_ranks || limit_cycles <= 0) return DSB_ERR_ARG;
  RankFlags f = {};
  for (int i = 0; i < n_ranks; ++i) {
    if (!flags[i] || (reinterpret_cast<uintptr_t>(flags[i]) & 3u)) return DSB_ERR_ARG;
    f.f[i] = flags[i];
  }
  rank_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(f, n_ranks, rank, epoch, limit_cycles, status);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

extern "C" int dsb_selftest_wait_timeout(long long limit_cycles, int* status, int* neighbour_left, void* stream) {
  if (!status || limit_cycles <= 0 || limit_cycles > kWaitLimitCycles) return DSB_ERR_ARG;
  wait_timeout_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(limit_cycles, status,
                                                                                      neighbour_left);
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}

extern "C" int dsb_pack_quant_weight(const void* W, int64_t ld_w, int src_is_bf16, void* Wq, int64_t ld_q,
                                     float* scales, int N, int K, int fmt, int per_channel, float* work,
                                     void* stream) {
  if (!W || !Wq || !scales || N <= 0 || K <= 0) return DSB_ERR_ARG;
  if (fmt != DSB_FMT_E4M3 && fmt != DSB_FMT_INT8) return DSB_ERR_ARG;
  if (fmt == DSB_FMT_INT8 && !per_channel) return DSB_ERR_ARG;
  if (!per_channel && !work) return DSB_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* q = reinterpret_cast<uint8_t*>(Wq);
  if (!per_channel) {
    if (cudaMemsetAsync(work, 0, sizeof(float), st) != cudaSuccess) return DSB_ERR_CUDA;
    const int blocks = sm_count() * 4;
    if (src_is_bf16)
      amax_all_kernel<true><<<blocks, 256, 0, st>>>(W, ld_w, N, K, work);
    else
      amax_all_kernel<false><<<blocks, 256, 0, st>>>(W, ld_w, N, K, work);
  }
#define DSB_PACK(SRC, F) pack_rows_kernel<SRC, F><<<N, 256, 0, st>>>(W, ld_w, q, ld_q, scales, N, K, per_channel, work)
  if (fmt == DSB_FMT_E4M3) {
    if (src_is_bf16) DSB_PACK(true, DSB_FMT_E4M3);
    else DSB_PACK(false, DSB_FMT_E4M3);
  } else {
    if (src_is_bf16) DSB_PACK(true, DSB_FMT_INT8);
    else DSB_PACK(false, DSB_FMT_INT8);
  }
#undef DSB_PACK
  return cudaGetLastError() == cudaSuccess ? DSB_OK : DSB_ERR_CUDA;
}
