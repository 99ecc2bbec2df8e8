// Shared host/device helpers of the C-ABI library: error reporting, element
// type conversion and small warp utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/matterformer_b200.h"

namespace mf {

// ---- host: per-thread error text ------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_error(cudaError_t err, const char* what);

#define MF_CHECK_ARG(cond, ...)                 \
  do {                                          \
    if (!(cond)) {                              \
      ::mf::set_error(__VA_ARGS__);             \
      return MF_ERR_INVALID_ARGUMENT;           \
    }                                           \
  } while (0)

#define MF_CHECK_LAUNCH(what)                                   \
  do {                                                          \
    cudaError_t e__ = cudaGetLastError();                       \
    if (e__ != cudaSuccess) return ::mf::cuda_error(e__, what); \
  } while (0)

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
// Kernels read and write tensors through 16-byte vector accesses: every tensor base must sit on a 16-byte boundary
// (a view that starts inside another tensor may not).  NULL counts as aligned (optional tensors).
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
#define MF_CHECK_ALIGNED(name, ...)                                                                          \
  do {                                                                                                       \
    const void* ptrs__[] = {__VA_ARGS__};                                                                    \
    for (const void* q__ : ptrs__)                                                                           \
      if (!::mf::aligned16(q__)) {                                                                           \
        ::mf::set_error("%s: tensor at %p is not 16-byte aligned (pass tensors that start on a 16-byte boundary)", \
                        name, q__);                                                                          \
        return MF_ERR_INVALID_ARGUMENT;                                                                      \
      }                                                                                                      \
  } while (0)

// ---- device: index checks of debug builds ----------------------------------------
// Built with -DMF_DEBUG_BOUNDS (MF_DEBUG_BOUNDS=1 python -m matterformer_b200.build), the table and bitmap lookups
// of the tensor-core kernels check their index first: one outside [0, limit) is recorded in the kernel's status word
// (MF_ERR_BOUNDS) and replaced by 0, so that the access itself stays in range and nothing faults.  The memory checker
// of the toolkit is not available on every machine this library is developed on; this is the stand-in.  Release
// builds use the index as it is.
#ifdef MF_DEBUG_BOUNDS
__device__ __forceinline__ long long checked_index(long long i, long long n, int32_t* status) {
  if (i >= 0 && i < n) return i;
  if (status) atomicExch(status, MF_ERR_BOUNDS);
  return 0;
}
#define MF_IDX(idx, limit, status) (::mf::checked_index((long long)(idx), (long long)(limit), (status)))
#else
#define MF_IDX(idx, limit, status) (idx)
#endif

// ---- device: element conversion ------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Dispatch a generic lambda on the element type named by an MF_DTYPE_* code.
#define MF_DISPATCH_DTYPE(dtype, T, ...)                         \
  switch (dtype) {                                               \
    case MF_DTYPE_F32: {                                         \
      using T = float;                                           \
      __VA_ARGS__;                                               \
    } break;                                                     \
    case MF_DTYPE_BF16: {                                        \
      using T = __nv_bfloat16;                                   \
      __VA_ARGS__;                                               \
    } break;                                                     \
    case MF_DTYPE_F16: {                                         \
      using T = __half;                                          \
      __VA_ARGS__;                                               \
    } break;                                                     \
    default:                                                     \
      ::mf::set_error("unsupported dtype code %d", (int)(dtype)); \
      return MF_ERR_INVALID_ARGUMENT;                            \
  }

}  // namespace mf

namespace mf {
// Kernel timing aid (see mf_profile_enable): record an event on `stream` before/after a main kernel.
void profile_mark(int which, bool begin, cudaStream_t stream);
}  // namespace mf
