// Host plumbing of the C ABI: feature query, status word, tensor-map encoding.
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "host_common.h"

namespace wk {

namespace {
constexpr int kMaxDevices = 64;
int* g_status[kMaxDevices] = {};
int g_sms[kMaxDevices] = {};
std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn encode_fn() {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) !=
          cudaSuccess ||
      qres != cudaDriverEntryPointSuccess) {
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

int encode_tmap(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return WK_E_CUDA;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (uint32_t i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult r = fn(map, dtype, rank, const_cast<void*>(base), gdim, gstr, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : WK_E_ARG;
}

int* status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 64) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, 64) != cudaSuccess) return nullptr;
    g_status[dev] = p;
  }
  return g_status[dev];
}

int device_arch_of(int dev) {
  // compute capability 10.x -> 100; remembered per device (0 = not asked yet)
  static int known[kMaxDevices] = {};
  if (dev < 0 || dev >= kMaxDevices) return WK_E_ARG;
  if (known[dev]) return known[dev];
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    cudaGetLastError();  // leave no sticky error behind for the caller's next launch check
    return WK_E_CUDA;
  }
  known[dev] = major == 10 ? 100 : WK_E_UNSUPPORTED;
  return known[dev];
}

int require_sm100() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return WK_E_CUDA;
  const int arch = device_arch_of(dev);
  return arch == 100 ? 0 : arch;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  if (!g_sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

int allow_smem(const void* func, int bytes) {
  // remembered per (kernel, device): the attribute belongs to the device's context
  constexpr int kMaxFuncs = 32;
  static const void* funcs[kMaxFuncs] = {};
  static bool done[kMaxFuncs][kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return WK_E_CUDA;
  std::lock_guard<std::mutex> lock(g_mu);
  int slot = -1;
  for (int i = 0; i < kMaxFuncs; ++i) {
    if (funcs[i] == func || funcs[i] == nullptr) {
      slot = i;
      break;
    }
  }
  if (slot >= 0 && funcs[slot] == func && done[slot][dev]) return 0;
  if (cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
    return WK_E_CUDA;
  if (slot >= 0) {
    funcs[slot] = func;
    done[slot][dev] = true;
  }
  return 0;
}

}  // namespace wk

extern "C" {

int wk_query(const char* feature) {
  if (!feature) return WK_E_ARG;
  static const char* const kYes[] = {"gemm",       "gemm_fp8",   "gemm_mx",      "gemm_mx_out", "gemm_gelu",
                                     "gemm_dgelu", "gemm_accum", "attn_fwd_fp8", "attn_bwd_fp8", "attn_fwd", "attn_bwd"};
  for (const char* f : kYes)
    if (!strcmp(f, feature)) return 1;
  return WK_E_ARG;  // every feature name of the reference is built; anything else is not a feature
}

int wk_device_arch(int device) {
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    return WK_E_CUDA;
  }
  return wk::device_arch_of(device);
}

int wk_status(void) {
  int* p = wk::status_word();
  if (!p) return WK_E_CUDA;
  if (cudaDeviceSynchronize() != cudaSuccess) return WK_E_CUDA;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return WK_E_CUDA;
  if (v != 0 && cudaMemset(p, 0, sizeof(int)) != cudaSuccess) return WK_E_CUDA;
  return v;
}

const char* wk_error_string(int code) {
  switch (code) {
    case 0: return "ok";
    case WK_E_ARG: return "argument rejected (size, stride, alignment or null pointer)";
    case WK_E_CUDA: return "CUDA runtime or driver error";
    case WK_E_UNSUPPORTED: return "device is not compute capability 10.x";
    case WK_E_TOO_LARGE: return "problem too large for the library's fixed scratch array";
    case wk::WK_ERR_TIMEOUT_LOAD: return "kernel gave up waiting for a TMA load";
    case wk::WK_ERR_TIMEOUT_EMPTY: return "kernel gave up waiting for a free pipeline stage";
    case wk::WK_ERR_TIMEOUT_MMA: return "kernel gave up waiting for the tensor core";
    case wk::WK_ERR_TIMEOUT_TMEM: return "kernel gave up waiting for a drained accumulator";
    case wk::WK_ERR_TIMEOUT_P: return "kernel gave up waiting for softmax output";
    case wk::WK_ERR_RANGE: return "attention scores span more than 2^100 within a row";
    default: return "unknown code";
  }
}

}  // extern "C"
