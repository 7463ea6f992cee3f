// Host-side helpers shared by the C-ABI entry points: tensor-map encoding through
// the driver entry point (no link-time dependency on libcuda), the per-device
// status word the kernels report bounded-wait failures to, and argument checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/warpy_b200.h"

namespace wk {

// Returns 0 and fills *map, or a negative WK_E_* code.
int encode_tmap(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes /* rank-1 entries */,
                const uint32_t* box, CUtensorMapSwizzle swizzle);

// Device pointer of the int status word of the current device (allocated on first use).
int* status_word();

// 100 for a device of compute capability 10.x, WK_E_UNSUPPORTED for any other, WK_E_CUDA if it cannot be asked.
int device_arch_of(int dev);

// 0 if the current device can run this library's kernels, else the negative code an entry point returns
// (WK_E_UNSUPPORTED for a device that is not compute capability 10.x).  Allocates nothing.
int require_sm100();

// Number of SMs of the current device (cached).
int sm_count();

// Raises the dynamic shared memory limit of `func` once per process.
int allow_smem(const void* func, int bytes);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace wk

#define WK_CUDA_OK(expr)                    \
  do {                                      \
    cudaError_t e__ = (expr);               \
    if (e__ != cudaSuccess) return WK_E_CUDA; \
  } while (0)
