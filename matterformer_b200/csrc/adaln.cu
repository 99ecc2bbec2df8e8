// Fused element-wise passes of the trunk's adaptive-LayerNorm block
// (src/matterformer/models/transformer.py:242-253, 308-316):
//   h = LayerNorm(x) * (1 + scale_b) + shift_b        (no affine parameters; statistics over the channels)
//   y = x + gate_b * a
// with x the residual stream (B, N, C) in fp32 or bf16, shift / scale / gate per molecule (B, C) in fp32, h and a in
// fp32 or bf16; arithmetic in fp32.
// The reference runs each as a chain of separate element-wise kernels over the (B, N, C) tensor; these kernels
// read and write it once.  One CTA per molecule: a warp per token row, per-column sums over the molecule's
// tokens (the gradients of shift, scale and gate) in registers, combined across warps in a fixed order.
#include <cuda_bf16.h>

#include "common.cuh"

namespace mf {
namespace {

constexpr int kAdaWarps = 8;
constexpr int kAdaMaxPerLane = 32;  // channels per lane: C <= 1024

template <typename T>
__device__ __forceinline__ float ld_f32(const T* p);
template <>
__device__ __forceinline__ float ld_f32<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void st_f32(T* p, float v);
template <>
__device__ __forceinline__ void st_f32<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st_f32<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename TX, typename TH>
__global__ void __launch_bounds__(kAdaWarps * 32) ln_modulate_fwd_kernel(const TX* __restrict__ x,
                                                                         const float* __restrict__ shift,
                                                                         const float* __restrict__ scale, int N, int C,
                                                                         float eps, TH* __restrict__ h,
                                                                         float* __restrict__ mean_out,
                                                                         float* __restrict__ rstd_out) {
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* sh = shift + (size_t)b * C;
  const float* sc = scale + (size_t)b * C;
  for (int n = warp; n < N; n += kAdaWarps) {
    const size_t row = (size_t)b * N + n;
    const TX* xr = x + row * C;
    float s = 0.f;
    for (int c = lane; c < C; c += 32) s += ld_f32<TX>(xr + c);
    const float mean = warp_sum(s) / (float)C;
    float v = 0.f;
    for (int c = lane; c < C; c += 32) {
      const float d = ld_f32<TX>(xr + c) - mean;
      v = fmaf(d, d, v);
    }
    const float rstd = rsqrtf(warp_sum(v) / (float)C + eps);
    for (int c = lane; c < C; c += 32)
      st_f32<TH>(h + row * C + c, fmaf((ld_f32<TX>(xr + c) - mean) * rstd, 1.f + sc[c], sh[c]));
    if (lane == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
  }
}

// dx, and per molecule dshift[c] = sum_n dh, dscale[c] = sum_n dh * xhat
template <typename TX, typename TH>
__global__ void __launch_bounds__(kAdaWarps * 32) ln_modulate_bwd_kernel(const TH* __restrict__ dh,
                                                                         const TX* __restrict__ x,
                                                                         const float* __restrict__ scale,
                                                                         const float* __restrict__ mean_in,
                                                                         const float* __restrict__ rstd_in, int N, int C,
                                                                         TX* __restrict__ dx,
                                                                         float* __restrict__ dshift,
                                                                         float* __restrict__ dscale) {
  extern __shared__ float part[];  // [kAdaWarps][C]
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* sc = scale + (size_t)b * C;
  float a_shift[kAdaMaxPerLane], a_scale[kAdaMaxPerLane];
#pragma unroll
  for (int t = 0; t < kAdaMaxPerLane; ++t) a_shift[t] = 0.f, a_scale[t] = 0.f;
  for (int n = warp; n < N; n += kAdaWarps) {
    const size_t row = (size_t)b * N + n;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int t = 0; t < kAdaMaxPerLane; ++t) {
      const int c = lane + 32 * t;
      if (c < C) {
        const float g0 = ld_f32<TH>(dh + row * C + c);
        const float xh = (ld_f32<TX>(x + row * C + c) - mean) * rstd;
        const float g = g0 * (1.f + sc[c]);
        s1 += g;
        s2 = fmaf(g, xh, s2);
        a_shift[t] += g0;
        a_scale[t] = fmaf(g0, xh, a_scale[t]);
      }
    }
    s1 = warp_sum(s1) / (float)C;
    s2 = warp_sum(s2) / (float)C;
#pragma unroll
    for (int t = 0; t < kAdaMaxPerLane; ++t) {
      const int c = lane + 32 * t;
      if (c < C) {
        const float g = ld_f32<TH>(dh + row * C + c) * (1.f + sc[c]);
        const float xh = (ld_f32<TX>(x + row * C + c) - mean) * rstd;
        st_f32<TX>(dx + row * C + c, rstd * (g - s1 - xh * s2));
      }
    }
  }
  // column sums over the molecule's tokens: the warps' partial sums, added in warp order
  for (int pass = 0; pass < 2; ++pass) {
    __syncthreads();
#pragma unroll
    for (int t = 0; t < kAdaMaxPerLane; ++t) {
      const int c = lane + 32 * t;
      if (c < C) part[warp * C + c] = pass == 0 ? a_shift[t] : a_scale[t];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += kAdaWarps * 32) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kAdaWarps; ++w) tot += part[w * C + c];
      (pass == 0 ? dshift : dscale)[(size_t)b * C + c] = tot;
    }
  }
}

template <typename TX, typename TA>
__global__ void gated_residual_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ gate,
                                          const TA* __restrict__ a, int N, int C, long long total,
                                          TX* __restrict__ y) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (int)(i % C);
  const long long bq = i / ((long long)N * C);
  st_f32<TX>(y + i, fmaf(gate[bq * C + c], ld_f32<TA>(a + i), ld_f32<TX>(x + i)));
}

// da = dy * gate_b (in a's type), dgate[b,c] = sum_n dy * a
template <typename TX, typename TA>
__global__ void __launch_bounds__(kAdaWarps * 32) gated_residual_bwd_kernel(const TX* __restrict__ dy,
                                                                            const float* __restrict__ gate,
                                                                            const TA* __restrict__ a, int N, int C,
                                                                            TA* __restrict__ da,
                                                                            float* __restrict__ dgate) {
  extern __shared__ float part[];  // [kAdaWarps][C]
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* gt = gate + (size_t)b * C;
  float acc[kAdaMaxPerLane];
#pragma unroll
  for (int t = 0; t < kAdaMaxPerLane; ++t) acc[t] = 0.f;
  for (int n = warp; n < N; n += kAdaWarps) {
    const size_t row = (size_t)b * N + n;
#pragma unroll
    for (int t = 0; t < kAdaMaxPerLane; ++t) {
      const int c = lane + 32 * t;
      if (c < C) {
        const float g = ld_f32<TX>(dy + row * C + c);
        acc[t] = fmaf(g, ld_f32<TA>(a + row * C + c), acc[t]);
        st_f32<TA>(da + row * C + c, g * gt[c]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kAdaMaxPerLane; ++t) {
    const int c = lane + 32 * t;
    if (c < C) part[warp * C + c] = acc[t];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += kAdaWarps * 32) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kAdaWarps; ++w) tot += part[w * C + c];
    dgate[(size_t)b * C + c] = tot;
  }
}

int check_sizes(const char* name, int batch, int tokens, int channels, int half_dtype) {
  MF_CHECK_ARG(batch >= 0 && tokens >= 0 && channels >= 1, "%s: bad size", name);
  MF_CHECK_ARG(channels <= 32 * kAdaMaxPerLane, "%s: at most %d channels, got %d", name, 32 * kAdaMaxPerLane, channels);
  MF_CHECK_ARG(half_dtype == MF_DTYPE_F32 || half_dtype == MF_DTYPE_BF16, "%s: tensor type must be float32 or bfloat16",
               name);
  return MF_OK;
}

}  // namespace
}  // namespace mf

using namespace mf;

// dispatch on the two tensor types (fp32 / bf16 each)
#define MF_ADA_DISPATCH(xcode, hcode, TX, TH, ...)                          \
  do {                                                                      \
    if ((xcode) == MF_DTYPE_BF16 && (hcode) == MF_DTYPE_BF16) {             \
      using TX = __nv_bfloat16;                                             \
      using TH = __nv_bfloat16;                                             \
      __VA_ARGS__;                                                          \
    } else if ((xcode) == MF_DTYPE_BF16) {                                  \
      using TX = __nv_bfloat16;                                             \
      using TH = float;                                                     \
      __VA_ARGS__;                                                          \
    } else if ((hcode) == MF_DTYPE_BF16) {                                  \
      using TX = float;                                                     \
      using TH = __nv_bfloat16;                                             \
      __VA_ARGS__;                                                          \
    } else {                                                                \
      using TX = float;                                                     \
      using TH = float;                                                     \
      __VA_ARGS__;                                                          \
    }                                                                       \
  } while (0)

extern "C" int mf_ln_modulate_fwd(const void* x, int32_t x_dtype, const float* shift, const float* scale, int32_t batch,
                                  int32_t tokens, int32_t channels, float eps, int32_t h_dtype, void* h, float* mean,
                                  float* rstd, void* stream) {
  int rc = check_sizes("mf_ln_modulate_fwd", batch, tokens, channels, h_dtype);
  if (rc == MF_OK) rc = check_sizes("mf_ln_modulate_fwd", batch, tokens, channels, x_dtype);
  if (rc != MF_OK) return rc;
  if (batch == 0 || tokens == 0) return MF_OK;
  MF_CHECK_ARG(x && shift && scale && h && mean && rstd, "mf_ln_modulate_fwd: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MF_ADA_DISPATCH(x_dtype, h_dtype, TX, TH,
                  (ln_modulate_fwd_kernel<TX, TH><<<batch, kAdaWarps * 32, 0, s>>>(
                      static_cast<const TX*>(x), shift, scale, tokens, channels, eps, static_cast<TH*>(h), mean, rstd)));
  MF_CHECK_LAUNCH("ln_modulate_fwd_kernel");
  return MF_OK;
}

extern "C" int mf_ln_modulate_bwd(const void* dh, int32_t dh_dtype, const void* x, int32_t x_dtype, const float* scale,
                                  const float* mean, const float* rstd, int32_t batch, int32_t tokens, int32_t channels,
                                  void* dx, float* dshift, float* dscale, void* stream) {
  int rc = check_sizes("mf_ln_modulate_bwd", batch, tokens, channels, dh_dtype);
  if (rc == MF_OK) rc = check_sizes("mf_ln_modulate_bwd", batch, tokens, channels, x_dtype);
  if (rc != MF_OK) return rc;
  if (batch == 0) return MF_OK;
  MF_CHECK_ARG(dh && x && scale && mean && rstd && dx && dshift && dscale, "mf_ln_modulate_bwd: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)kAdaWarps * channels * sizeof(float);
  MF_ADA_DISPATCH(x_dtype, dh_dtype, TX, TH,
                  (ln_modulate_bwd_kernel<TX, TH><<<batch, kAdaWarps * 32, smem, s>>>(
                      static_cast<const TH*>(dh), static_cast<const TX*>(x), scale, mean, rstd, tokens, channels,
                      static_cast<TX*>(dx), dshift, dscale)));
  MF_CHECK_LAUNCH("ln_modulate_bwd_kernel");
  return MF_OK;
}

extern "C" int mf_gated_residual_fwd(const void* x, int32_t x_dtype, const float* gate, const void* a, int32_t a_dtype,
                                     int32_t batch, int32_t tokens, int32_t channels, void* y, void* stream) {
  int rc = check_sizes("mf_gated_residual_fwd", batch, tokens, channels, a_dtype);
  if (rc == MF_OK) rc = check_sizes("mf_gated_residual_fwd", batch, tokens, channels, x_dtype);
  if (rc != MF_OK) return rc;
  const long long total = (long long)batch * tokens * channels;
  if (total == 0) return MF_OK;
  MF_CHECK_ARG(x && gate && a && y, "mf_gated_residual_fwd: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((total + 255) / 256);
  MF_ADA_DISPATCH(x_dtype, a_dtype, TX, TA,
                  (gated_residual_fwd_kernel<TX, TA><<<blocks, 256, 0, s>>>(
                      static_cast<const TX*>(x), gate, static_cast<const TA*>(a), tokens, channels, total,
                      static_cast<TX*>(y))));
  MF_CHECK_LAUNCH("gated_residual_fwd_kernel");
  return MF_OK;
}

extern "C" int mf_gated_residual_bwd(const void* dy, int32_t dy_dtype, const float* gate, const void* a, int32_t a_dtype,
                                     int32_t batch, int32_t tokens, int32_t channels, void* da, float* dgate,
                                     void* stream) {
  int rc = check_sizes("mf_gated_residual_bwd", batch, tokens, channels, a_dtype);
  if (rc == MF_OK) rc = check_sizes("mf_gated_residual_bwd", batch, tokens, channels, dy_dtype);
  if (rc != MF_OK) return rc;
  if (batch == 0) return MF_OK;
  MF_CHECK_ARG(dy && gate && a && da && dgate, "mf_gated_residual_bwd: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)kAdaWarps * channels * sizeof(float);
  MF_ADA_DISPATCH(dy_dtype, a_dtype, TX, TA,
                  (gated_residual_bwd_kernel<TX, TA><<<batch, kAdaWarps * 32, smem, s>>>(
                      static_cast<const TX*>(dy), gate, static_cast<const TA*>(a), tokens, channels,
                      static_cast<TA*>(da), dgate)));
  MF_CHECK_LAUNCH("gated_residual_bwd_kernel");
  return MF_OK;
}
