// Column sums of a row-major matrix: out[c] = sum_r x[r, c], fp32 accumulation, fp32 result.
//
// The bias gradient of every Linear layer of the trunk (AdaLNBlock.forward, models/transformer.py:228-316: the input
// and output projections of the attention, the two layers of the MLP, the AdaLN modulation) is such a sum over all
// tokens of the batch: 30 k rows of 512 to 2560 bf16 values at the benchmark batch.  Two kernels, both with a fixed
// order of additions (no atomics): a block sums a band of rows for 256 columns, every lane holding eight neighbouring
// columns (one 16-byte load per row for bf16), the eight warps of the block are added in warp order, and a second
// kernel adds the bands in band order.  HBM-bound: the matrix is read once.
//
// The MLP of the block has a GELU (tanh form, models/transformer.py:137-152) between its two layers; its backward pass,
// dpre = dact * gelu'(pre), produces exactly the matrix whose column sums are the first layer's bias gradient, so the
// band kernel also exists in a form that computes dpre from (pre, dact), stores it and sums it in the same sweep.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/matterformer_b200.h"
#include "common.cuh"

namespace mf {
namespace {

constexpr int kWarps = 8;
constexpr int kColsPerBlock = 256;  // 32 lanes x 8 columns
constexpr int kMaxBands = 256;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) v[2 * e] = __uint_as_float(w[e] << 16), v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
    w[e] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// GELU, tanh form: 0.5 x (1 + tanh(beta (x + kappa x^3))), and its derivative
constexpr float kGeluBeta = 0.7978845608028654f;  // sqrt(2 / pi)
constexpr float kGeluKappa = 0.044715f;
// kFast (bf16 tensors): the hardware tanh (relative error about 2^-11, below the 2^-9 of the bf16 result); fp32
// tensors take tanhf
template <bool kFast>
__device__ __forceinline__ float tanh_of(float v) {
  if constexpr (kFast) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(v));
    return t;
  } else {
    return tanhf(v);
  }
}
template <bool kFast>
__device__ __forceinline__ float gelu_tanh(float x) {
  const float t = tanh_of<kFast>(kGeluBeta * (x + kGeluKappa * x * x * x));
  return 0.5f * x * (1.f + t);
}
template <bool kFast>
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float t = tanh_of<kFast>(kGeluBeta * (x + kGeluKappa * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * kGeluBeta * (1.f + 3.f * kGeluKappa * x * x);
}

template <typename T>
__global__ void gelu_tanh_fwd_kernel(const T* __restrict__ x, long long n, T* __restrict__ y) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  float v[8];
  load8<T>(x + i, v);
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = gelu_tanh<sizeof(T) == 2>(v[e]);
  store8<T>(y + i, v);
}

// grid (column groups, bands); part[band][C].  kGelu: x is the pre-activation, dy the gradient of the activation;
// dx = dy * gelu'(x) is stored and summed.
template <typename T, bool kGelu>
__global__ void __launch_bounds__(kWarps * 32) column_sums_band_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                                      T* __restrict__ dx, long long rows, int C,
                                                                      long long rows_per_band, float* __restrict__ part) {
  __shared__ float red[kWarps][kColsPerBlock];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * kColsPerBlock + 8 * lane;
  const long long r0 = (long long)blockIdx.y * rows_per_band;
  const long long r1 = r0 + rows_per_band < rows ? r0 + rows_per_band : rows;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < C) {
    long long r = r0 + warp;
    for (; r + 3 * kWarps < r1; r += 4 * kWarps) {  // four rows in flight per lane
      float v[4][8], g[kGelu ? 4 : 1][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        load8<T>(x + (r + u * kWarps) * C + col, v[u]);
        if constexpr (kGelu) load8<T>(dy + (r + u * kWarps) * C + col, g[u]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if constexpr (kGelu) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[u][e] = g[u][e] * gelu_tanh_grad<sizeof(T) == 2>(v[u][e]);
          store8<T>(dx + (r + u * kWarps) * C + col, v[u]);
          if constexpr (sizeof(T) == 2) {  // what the next consumer reads is the rounded value: sum that
#pragma unroll
            for (int e = 0; e < 8; ++e) v[u][e] = __bfloat162float(__float2bfloat16_rn(v[u][e]));
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += v[u][e];
      }
    }
    for (; r < r1; r += kWarps) {
      float v[8];
      load8<T>(x + r * C + col, v);
      if constexpr (kGelu) {
        float g[8];
        load8<T>(dy + r * C + col, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = g[e] * gelu_tanh_grad<sizeof(T) == 2>(v[e]);
        store8<T>(dx + r * C + col, v);
        if constexpr (sizeof(T) == 2) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __bfloat162float(__float2bfloat16_rn(v[e]));
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[warp][8 * lane + e] = acc[e];
  __syncthreads();
  const int c = blockIdx.x * kColsPerBlock + threadIdx.x;
  if (c < C) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) tot += red[w][threadIdx.x];
    part[(size_t)blockIdx.y * C + c] = tot;
  }
}

// Adds the bands: a block of 32 x 8 threads owns 32 columns; thread (x, y) adds the bands y, y + 8, ... (four loads in
// flight), then the eight slices are added in slice order.
__global__ void __launch_bounds__(256) column_sums_final_kernel(const float* __restrict__ part, int bands, int C,
                                                                float* __restrict__ out) {
  __shared__ float red[8][32];
  const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + x;
  float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
  if (c < C) {
    int b = y;
    for (; b + 24 < bands; b += 32) {
      const float v0 = part[(size_t)b * C + c], v1 = part[(size_t)(b + 8) * C + c];
      const float v2 = part[(size_t)(b + 16) * C + c], v3 = part[(size_t)(b + 24) * C + c];
      t0 += v0, t1 += v1, t2 += v2, t3 += v3;
    }
    for (; b < bands; b += 8) t0 += part[(size_t)b * C + c];
  }
  red[y][x] = (t0 + t1) + (t2 + t3);
  __syncthreads();
  if (y == 0 && c < C) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w][x];
    out[c] = tot;
  }
}

// bands: enough blocks to fill the GPU a few times over, at least 32 rows per band
int bands_for(long long rows, int cols) {
  const int groups = (cols + kColsPerBlock - 1) / kColsPerBlock;
  long long bands = (4 * 148 + groups - 1) / groups;
  const long long by_rows = (rows + 31) / 32;
  if (bands > by_rows) bands = by_rows;
  if (bands > kMaxBands) bands = kMaxBands;
  if (bands < 1) bands = 1;
  return (int)bands;
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" size_t mf_column_sums_workspace_bytes(int64_t rows, int32_t cols) {
  if (rows < 0 || cols < 1) return 0;
  return (size_t)bands_for(rows, cols) * (size_t)cols * sizeof(float);
}

extern "C" int mf_column_sums(const void* x, int32_t dtype, int64_t rows, int32_t cols, float* out, void* workspace,
                              size_t workspace_bytes, void* stream) {
  MF_CHECK_ARG(rows >= 0 && cols >= 1 && cols % 8 == 0, "mf_column_sums: cols must be a positive multiple of 8, rows >= 0");
  MF_CHECK_ARG(dtype == MF_DTYPE_F32 || dtype == MF_DTYPE_BF16, "mf_column_sums: tensor type must be float32 or bfloat16");
  MF_CHECK_ARG(out != nullptr && (rows == 0 || x != nullptr), "mf_column_sums: null tensor");
  MF_CHECK_ARG(reinterpret_cast<uintptr_t>(x) % 16 == 0, "mf_column_sums: x must start on a 16-byte boundary");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    cudaError_t e = cudaMemsetAsync(out, 0, (size_t)cols * sizeof(float), s);
    return e == cudaSuccess ? MF_OK : cuda_error(e, "cudaMemsetAsync(mf_column_sums)");
  }
  const int bands = bands_for(rows, cols);
  if (workspace == nullptr || workspace_bytes < (size_t)bands * cols * sizeof(float)) {
    set_error("mf_column_sums: workspace too small (%zu bytes needed)", (size_t)bands * cols * sizeof(float));
    return MF_ERR_WORKSPACE_TOO_SMALL;
  }
  float* part = static_cast<float*>(workspace);
  const long long rows_per_band = (rows + bands - 1) / bands;
  const dim3 grid((cols + kColsPerBlock - 1) / kColsPerBlock, bands);
  if (dtype == MF_DTYPE_BF16)
    column_sums_band_kernel<__nv_bfloat16, false><<<grid, kWarps * 32, 0, s>>>(static_cast<const __nv_bfloat16*>(x), nullptr,
                                                                               nullptr, rows, cols, rows_per_band, part);
  else
    column_sums_band_kernel<float, false><<<grid, kWarps * 32, 0, s>>>(static_cast<const float*>(x), nullptr, nullptr, rows,
                                                                       cols, rows_per_band, part);
  MF_CHECK_LAUNCH("column_sums_band_kernel");
  column_sums_final_kernel<<<(cols + 31) / 32, 256, 0, s>>>(part, bands, cols, out);
  MF_CHECK_LAUNCH("column_sums_final_kernel");
  return MF_OK;
}

extern "C" int mf_gelu_tanh_fwd(const void* x, int32_t dtype, int64_t n, void* y, void* stream) {
  MF_CHECK_ARG(n >= 0 && n % 8 == 0, "mf_gelu_tanh_fwd: the element count must be a multiple of 8");
  MF_CHECK_ARG(dtype == MF_DTYPE_F32 || dtype == MF_DTYPE_BF16, "mf_gelu_tanh_fwd: tensor type must be float32 or bfloat16");
  if (n == 0) return MF_OK;
  MF_CHECK_ARG(x && y, "mf_gelu_tanh_fwd: null tensor");
  MF_CHECK_ARG(reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0,
               "mf_gelu_tanh_fwd: tensors must start on 16-byte boundaries");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((n / 8 + 255) / 256);
  if (dtype == MF_DTYPE_BF16)
    gelu_tanh_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n,
                                                                static_cast<__nv_bfloat16*>(y));
  else
    gelu_tanh_fwd_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), n, static_cast<float*>(y));
  MF_CHECK_LAUNCH("gelu_tanh_fwd_kernel");
  return MF_OK;
}

extern "C" int mf_gelu_tanh_bwd(const void* x, const void* dy, int32_t dtype, int64_t rows, int32_t cols, void* dx,
                                float* column_sums, void* workspace, size_t workspace_bytes, void* stream) {
  MF_CHECK_ARG(rows >= 0 && cols >= 1 && cols % 8 == 0, "mf_gelu_tanh_bwd: cols must be a positive multiple of 8, rows >= 0");
  MF_CHECK_ARG(dtype == MF_DTYPE_F32 || dtype == MF_DTYPE_BF16, "mf_gelu_tanh_bwd: tensor type must be float32 or bfloat16");
  MF_CHECK_ARG(column_sums != nullptr, "mf_gelu_tanh_bwd: null tensor");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    cudaError_t e = cudaMemsetAsync(column_sums, 0, (size_t)cols * sizeof(float), s);
    return e == cudaSuccess ? MF_OK : cuda_error(e, "cudaMemsetAsync(mf_gelu_tanh_bwd)");
  }
  MF_CHECK_ARG(x && dy && dx, "mf_gelu_tanh_bwd: null tensor");
  MF_CHECK_ARG(reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(dy) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(dx) % 16 == 0,
               "mf_gelu_tanh_bwd: tensors must start on 16-byte boundaries");
  const int bands = bands_for(rows, cols);
  if (workspace == nullptr || workspace_bytes < (size_t)bands * cols * sizeof(float)) {
    set_error("mf_gelu_tanh_bwd: workspace too small (%zu bytes needed)", (size_t)bands * cols * sizeof(float));
    return MF_ERR_WORKSPACE_TOO_SMALL;
  }
  float* part = static_cast<float*>(workspace);
  const long long rows_per_band = (rows + bands - 1) / bands;
  const dim3 grid((cols + kColsPerBlock - 1) / kColsPerBlock, bands);
  if (dtype == MF_DTYPE_BF16)
    column_sums_band_kernel<__nv_bfloat16, true><<<grid, kWarps * 32, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), rows,
        cols, rows_per_band, part);
  else
    column_sums_band_kernel<float, true><<<grid, kWarps * 32, 0, s>>>(static_cast<const float*>(x), static_cast<const float*>(dy),
                                                                      static_cast<float*>(dx), rows, cols, rows_per_band, part);
  MF_CHECK_LAUNCH("column_sums_band_kernel");
  column_sums_final_kernel<<<(cols + 31) / 32, 256, 0, s>>>(part, bands, cols, column_sums);
  MF_CHECK_LAUNCH("column_sums_final_kernel");
  return MF_OK;
}
