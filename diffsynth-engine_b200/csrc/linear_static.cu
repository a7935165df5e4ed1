// dsb_linear_static: the quantised Linear for callers that may not allocate device memory.
//
// The ordinary path (dsb_quant_rows followed by dsb_gemm) needs two intermediates that are neither input
// nor output: the 8-bit copy of the activation and one scale per row.  Normally the caller allocates them.
// Some callers cannot: a plugin that runs inside another runtime's fixed memory plan, a host binding (cgo, JNI,
// a C plugin ABI) that only ever hands over the tensors it was given, or code that runs at a point where
// cudaMalloc is not permitted.  For them this file keeps the two intermediates in a file-scope __device__
// array, so the entry point takes inputs and outputs only and calls no allocator of any kind.
//
// Cost and limits: every GPU that loads libdsb.so holds the array (kMaxActBytes + 256 KiB) until the process
// exits.  A problem with more than kMaxActBytes activation elements (M*K) or more than kMaxRows rows is rejected
// with DSB_ERR_TOO_LARGE.  All calls share the one array and it keeps the last call's contents: nothing in it
// has to start at zero (each call overwrites exactly the M*K bytes and M scales it later reads), but two calls
// that overlap on the GPU - different streams, or different host threads - race on it.  Callers serialise.
//
// In host code the array's NAME is a host-side stand-in, not a device address, so the device address is looked
// up once per device with cudaGetSymbolAddress (with that device current) and cached.  That lookup happens in
// the first call on each device; make that first call outside any stream capture.
#include <mutex>

#include "common.cuh"
#include "dsb.h"

namespace {

constexpr size_t kMaxActBytes = size_t(64) << 20;  // 64 Mi elements of quantised activation (1 byte each)
constexpr int kMaxRows = 65536;                    // one fp32 scale per activation row

static __device__ __align__(256) unsigned char g_linear_scratch[kMaxActBytes + size_t(kMaxRows) * sizeof(float)];

std::mutex g_mu;
unsigned char* g_scratch_addr[64] = {nullptr};  // device address of g_linear_scratch, per device ordinal

int scratch_of_current_device(unsigned char** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DSB_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_linear_scratch);
    if (e != cudaSuccess || p == nullptr) return DSB_ERR_CUDA;
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[dev];
  return DSB_OK;
}

}  // namespace

extern "C" int dsb_linear_static(const void* x, int64_t ld_x, const void* Wq, int64_t ld_w, int w_fmt, int M, int N,
                                 int K, const float* w_scale, int w_scale_stride, const float* bias, int act,
                                 void* out, int64_t ld_out, int* status, void* stream) {
  if (w_fmt != DSB_FMT_E4M3 && w_fmt != DSB_FMT_INT8) return DSB_ERR_ARG;
  if (M < 0 || N < 0 || K <= 0 || (K & 15) || !w_scale) return DSB_ERR_ARG;
  if (static_cast<size_t>(M) * static_cast<size_t>(K) > kMaxActBytes || M > kMaxRows) return DSB_ERR_TOO_LARGE;
  if (M == 0 || N == 0) return DSB_OK;
  unsigned char* scratch = nullptr;
  int rc = scratch_of_current_device(&scratch);
  if (rc != DSB_OK) return rc;
  float* row_scale = reinterpret_cast<float*>(scratch + kMaxActBytes);
  rc = dsb_quant_rows(x, ld_x, scratch, K, row_scale, M, K, w_fmt, stream);
  if (rc != DSB_OK) return rc;
  return dsb_gemm(scratch, K, Wq, ld_w, w_fmt, M, N, K, row_scale, w_scale, w_scale_stride, bias, act, 0, nullptr,
                  nullptr, 0, out, ld_out, nullptr, 0, N, status, stream);
}
