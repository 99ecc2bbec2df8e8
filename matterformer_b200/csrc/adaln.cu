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

// two neighbouring channels at a time: 4-byte (bf16) or 8-byte (fp32) accesses, fully used 128-byte lines per warp
template <typename T>
__device__ __forceinline__ float2 ld2(const T* p);
template <>
__device__ __forceinline__ float2 ld2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <>
__device__ __forceinline__ float2 ld2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T>
__device__ __forceinline__ void st2(T* p, float a, float b);
template <>
__device__ __forceinline__ void st2<float>(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
template <>
__device__ __forceinline__ void st2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// Channels come in pairs (C even): lane l owns channels 2l + 64t, 2l + 64t + 1.
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
    float xv[kAdaMaxPerLane];
    float s = 0.f;
#pragma unroll
    for (int t = 0; t < kAdaMaxPerLane / 2; ++t) {
      const int c = 2 * lane + 64 * t;
      float2 v = make_float2(0.f, 0.f);
      if (c < C) v = ld2<TX>(xr + c);
      xv[2 * t] = v.x, xv[2 * t + 1] = v.y;
      s += v.x + v.y;
    }
    const float mean = warp_sum(s) / (float)C;
    float v2 = 0.f;
#pragma unroll
    for (int t = 0; t < kAdaMaxPerLane / 2; ++t) {
      const int c = 2 * lane + 64 * t;
      if (c < C) {
        const float d0 = xv[2 * t] - mean, d1 = xv[2 * t + 1] - mean;
        v2 = fmaf(d0, d0, fmaf(d1, d1, v2));
      }
    }
    const float rstd = rsqrtf(warp_sum(v2) / (float)C + eps);
#pragma unroll
    for (int t = 0; t < kAdaMaxPerLane / 2; ++t) {
      const int c = 2 * lane + 64 * t;
      if (c < C) {
        const float2 sc2 = *reinterpret_cast<const float2*>(sc + c), sh2 = *reinterpret_cast<const float2*>(sh + c);
        st2<TH>(h + row * C + c, fmaf((xv[2 * t] - mean) * rstd, 1.f + sc2.x, sh2.x),
                fmaf((xv[2 * t + 1] - mean) * rstd, 1.f + sc2.y, sh2.y));
      }
    }
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
    for (int t = 0; t < kAdaMaxPerLane / 2; ++t) {
      const int c = 2 * lane + 64 * t;
      if (c < C) {
        const float2 g0 = ld2<TH>(dh + row * C + c), xx = ld2<TX>(x + row * C + c);
        const float2 sc2 = *reinterpret_cast<const float2*>(sc + c);
        const float xh0 = (xx.x - mean) * rstd, xh1 = (xx.y - mean) * rstd;
        const float g_0 = g0.x * (1.f + sc2.x), g_1 = g0.y * (1.f + sc2.y);
        s1 += g_0 + g_1;
        s2 = fmaf(g_0, xh0, fmaf(g_1, xh1, s2));
        a_shift[2 * t] += g0.x, a_shift[2 * t + 1] += g0.y;
        a_scale[2 * t] = fmaf(g0.x, xh0, a_scale[2 * t]);
        a_scale[2 * t + 1] = fmaf(g0.y, xh1, a_scale[2 * t + 1]);
      }
    }
    s1 = warp_sum(s1) / (float)C;
    s2 = warp_sum(s2) / (float)C;
    // second sweep over the row (it is in L1 now) rather than 64 more registers per thread
#pragma unroll
    for (int t = 0; t < kAdaMaxPerLane / 2; ++t) {
      const int c = 2 * lane + 64 * t;
      if (c < C) {
        const float2 g0 = ld2<TH>(dh + row * C + c), xx = ld2<TX>(x + row * C + c);
        const float2 sc2 = *reinterpret_cast<const float2*>(sc + c);
        const float xh0 = (xx.x - mean) * rstd, xh1 = (xx.y - mean) * rstd;
        st2<TX>(dx + row * C + c, rstd * (g0.x * (1.f + sc2.x) - s1 - xh0 * s2),
                rstd * (g0.y * (1.f + sc2.y) - s1 - xh1 * s2));
      }
    }
  }
  // column sums over the molecule's tokens: the warps' partial sums, added in warp order
  for (int pass = 0; pass < 2; ++pass) {
    __syncthreads();
#pragma unroll
    for (int t = 0; t < kAdaMaxPerLane / 2; ++t) {
      const int c = 2 * lane + 64 * t;
      if (c < C) {
        part[warp * C + c] = pass == 0 ? a_shift[2 * t] : a_scale[2 * t];
        part[warp * C + c + 1] = pass == 0 ? a_shift[2 * t + 1] : a_scale[2 * t + 1];
      }
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

// eight neighbouring channels per thread (C a multiple of 8)
template <typename TX, typename TA>
__global__ void gated_residual_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ gate,
                                          const TA* __restrict__ a, int N, int C, long long total,
                                          TX* __restrict__ y) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= total) return;
  const int c = (int)(i % C);
  const long long bq = i / ((long long)N * C);
  const float* g = gate + bq * C + c;
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    const float2 xx = ld2<TX>(x + i + e), aa = ld2<TA>(a + i + e);
    st2<TX>(y + i + e, fmaf(g[e], aa.x, xx.x), fmaf(g[e + 1], aa.y, xx.y));
  }
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
    for (int t = 0; t < kAdaMaxPerLane / 2; ++t) {
      const int c = 2 * lane + 64 * t;
      if (c < C) {
        const float2 g = ld2<TX>(dy + row * C + c), aa = ld2<TA>(a + row * C + c);
        const float2 gg = *reinterpret_cast<const float2*>(gt + c);
        acc[2 * t] = fmaf(g.x, aa.x, acc[2 * t]);
        acc[2 * t + 1] = fmaf(g.y, aa.y, acc[2 * t + 1]);
        st2<TA>(da + row * C + c, g.x * gg.x, g.y * gg.y);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kAdaMaxPerLane / 2; ++t) {
    const int c = 2 * lane + 64 * t;
    if (c < C) part[warp * C + c] = acc[2 * t], part[warp * C + c + 1] = acc[2 * t + 1];
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
  MF_CHECK_ARG(channels <= 32 * kAdaMaxPerLane && channels % 8 == 0, "%s: channels must be a multiple of 8, at most %d, got %d",
               name, 32 * kAdaMaxPerLane, channels);
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
  MF_CHECK_ALIGNED("mf_ln_modulate_fwd", x, shift, scale, h);
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
  MF_CHECK_ALIGNED("mf_ln_modulate_bwd", dh, x, scale, dx, dshift, dscale);
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
  MF_CHECK_ALIGNED("mf_gated_residual_fwd", x, gate, a, y);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((total / 8 + 255) / 256);
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
  MF_CHECK_ALIGNED("mf_gated_residual_bwd", dy, gate, a, da, dgate);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)kAdaWarps * channels * sizeof(float);
  MF_ADA_DISPATCH(dy_dtype, a_dtype, TX, TA,
                  (gated_residual_bwd_kernel<TX, TA><<<batch, kAdaWarps * 32, smem, s>>>(
                      static_cast<const TX*>(dy), gate, static_cast<const TA*>(a), tokens, channels,
                      static_cast<TA*>(da), dgate)));
  MF_CHECK_LAUNCH("gated_residual_bwd_kernel");
  return MF_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Head split / merge: the projections of an attention layer come out of one GEMM as (B, N, G, H, D) (G = 5 for the
// 2-simplicial layer: q, k1, v1, k2, v2; 3 for q, k, v) and the attention kernels want G tensors (B, H, N, D).
// One pass with 16-byte accesses on both sides instead of G strided copies; group g can be scaled on the way (the
// 1/sqrt(D) of the queries).  The merge is the inverse (and the backward pass of the split).
// ---------------------------------------------------------------------------------------------------------------
namespace mf {
namespace {

constexpr int kMaxGroups = 8;
struct HeadGroups {
  void* ptr[kMaxGroups];
  float scale[kMaxGroups];
};

template <typename T>
__device__ __forceinline__ uint4 scale16(uint4 v, float s);
template <>
__device__ __forceinline__ uint4 scale16<float>(uint4 v, float s) {
  float4 f = *reinterpret_cast<float4*>(&v);
  f.x *= s, f.y *= s, f.z *= s, f.w *= s;
  return *reinterpret_cast<uint4*>(&f);
}
template <>
__device__ __forceinline__ uint4 scale16<__nv_bfloat16>(uint4 v, float s) {
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    h[e] = __floats2bfloat162_rn(f.x * s, f.y * s);
  }
  return v;
}

// kSplit: packed -> groups, else groups -> packed (a null group reads as zeros).  One 16-byte chunk per thread.
template <typename T, bool kSplit>
__global__ void head_layout_kernel(T* __restrict__ packed, HeadGroups g, int G, int N, int H, int chunks_per_row,
                                   long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // chunk index on the packed side
  if (i >= total) return;
  const int c = (int)(i % chunks_per_row);
  long long r = i / chunks_per_row;
  const int h = (int)(r % H);
  r /= H;
  const int gi = (int)(r % G);
  r /= G;
  const int n = (int)(r % N);
  const long long b = r / N;
  uint4* pk = reinterpret_cast<uint4*>(packed) + i;
  uint4* gp = reinterpret_cast<uint4*>(g.ptr[gi]);
  const long long off = ((b * H + h) * N + n) * chunks_per_row + c;
  const float s = g.scale[gi];
  if (kSplit) {
    uint4 v = *pk;
    if (s != 1.f) v = scale16<T>(v, s);
    gp[off] = v;
  } else {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (gp) {
      v = gp[off];
      if (s != 1.f) v = scale16<T>(v, s);
    }
    *pk = v;
  }
}

int head_layout(bool split, void* packed, void* const* groups, const float* scales, int G, int B, int N, int H, int D,
                int dtype, cudaStream_t s, const char* name) {
  MF_CHECK_ARG(G >= 1 && G <= kMaxGroups && B >= 0 && N >= 0 && H >= 1 && D >= 1, "%s: bad size", name);
  MF_CHECK_ARG(dtype == MF_DTYPE_F32 || dtype == MF_DTYPE_BF16, "%s: tensor type must be float32 or bfloat16", name);
  const int es = dtype == MF_DTYPE_F32 ? 4 : 2;
  MF_CHECK_ARG((D * es) % 16 == 0, "%s: a head row must be a multiple of 16 bytes, got %d", name, D * es);
  if (B == 0 || N == 0) return MF_OK;
  MF_CHECK_ARG(packed && groups, "%s: null pointer argument", name);
  HeadGroups g{};
  for (int i = 0; i < G; ++i) {
    g.ptr[i] = groups[i];
    g.scale[i] = scales ? scales[i] : 1.f;
    MF_CHECK_ARG(!split || g.ptr[i], "%s: null output tensor %d", name, i);
    MF_CHECK_ARG((reinterpret_cast<uintptr_t>(g.ptr[i]) & 15u) == 0, "%s: tensor %d is not 16-byte aligned", name, i);
  }
  MF_CHECK_ARG((reinterpret_cast<uintptr_t>(packed) & 15u) == 0, "%s: packed tensor is not 16-byte aligned", name);
  const int cpr = D * es / 16;
  const long long total = (long long)B * N * G * H * cpr;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MF_DTYPE_F32) {
    if (split) head_layout_kernel<float, true><<<blocks, 256, 0, s>>>(static_cast<float*>(packed), g, G, N, H, cpr, total);
    else head_layout_kernel<float, false><<<blocks, 256, 0, s>>>(static_cast<float*>(packed), g, G, N, H, cpr, total);
  } else {
    if (split)
      head_layout_kernel<__nv_bfloat16, true><<<blocks, 256, 0, s>>>(static_cast<__nv_bfloat16*>(packed), g, G, N, H, cpr,
                                                                     total);
    else
      head_layout_kernel<__nv_bfloat16, false><<<blocks, 256, 0, s>>>(static_cast<__nv_bfloat16*>(packed), g, G, N, H, cpr,
                                                                      total);
  }
  MF_CHECK_LAUNCH("head_layout_kernel");
  return MF_OK;
}

}  // namespace
}  // namespace mf

extern "C" int mf_split_heads(const void* packed, void* const* outs, const float* scales, int32_t groups, int32_t batch,
                              int32_t tokens, int32_t heads, int32_t head_dim, int32_t dtype, void* stream) {
  return mf::head_layout(true, const_cast<void*>(packed), outs, scales, groups, batch, tokens, heads, head_dim, dtype,
                         static_cast<cudaStream_t>(stream), "mf_split_heads");
}

extern "C" int mf_merge_heads(void* const* ins, const float* scales, void* packed, int32_t groups, int32_t batch,
                              int32_t tokens, int32_t heads, int32_t head_dim, int32_t dtype, void* stream) {
  return mf::head_layout(false, packed, ins, scales, groups, batch, tokens, heads, head_dim, dtype,
                         static_cast<cudaStream_t>(stream), "mf_merge_heads");
}
