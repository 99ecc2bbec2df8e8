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
constexpr int kAdaVec = 4;  // at most four 8-channel vectors per lane: C <= 8 * 32 * 4 = 1024 (kernels are built for 1, 2 and 4)

// Eight neighbouring channels at a time: 16-byte (bf16) or 2 x 16-byte (fp32) accesses.  Lane l owns the vectors
// l, l + 32, l + 64, l + 96 of a row (vector v = channels 8v .. 8v + 7).
template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void ld8<float>(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
template <>
__device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) v[2 * e] = __uint_as_float(w[e] << 16), v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void st8<float>(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
    w[e] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename TX, typename TH, int VEC>
__global__ void __launch_bounds__(kAdaWarps * 32) ln_modulate_fwd_kernel(const TX* __restrict__ x,
                                                                         const float* __restrict__ shift,
                                                                         const float* __restrict__ scale, int N, int C,
                                                                         float eps, TH* __restrict__ h,
                                                                         float* __restrict__ mean_out,
                                                                         float* __restrict__ rstd_out) {
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* sh = shift + (size_t)b * C;
  const float* sc = scale + (size_t)b * C;
  const int nvec = C >> 3;
  const float inv_c = 1.f / (float)C;
  for (int n = warp; n < N; n += kAdaWarps) {
    const size_t row = (size_t)b * N + n;
    const TX* xr = x + row * C;
    float xv[VEC][8];
    float s = 0.f;
#pragma unroll
    for (int t = 0; t < VEC; ++t) {
      const int v = lane + 32 * t;
      if (v < nvec) {
        ld8<TX>(xr + 8 * v, xv[t]);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += xv[t][e];
      }
    }
    const float mean = warp_sum(s) * inv_c;
    float v2 = 0.f;
#pragma unroll
    for (int t = 0; t < VEC; ++t) {
      if (lane + 32 * t < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float d = xv[t][e] - mean;
          v2 = fmaf(d, d, v2);
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(v2) * inv_c + eps);
#pragma unroll
    for (int t = 0; t < VEC; ++t) {
      const int v = lane + 32 * t;
      if (v < nvec) {
        float scv[8], shv[8], out[8];
        ld8<float>(sc + 8 * v, scv);
        ld8<float>(sh + 8 * v, shv);
#pragma unroll
        for (int e = 0; e < 8; ++e) out[e] = fmaf((xv[t][e] - mean) * rstd, 1.f + scv[e], shv[e]);
        st8<TH>(h + row * C + 8 * v, out);
      }
    }
    if (lane == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
  }
}

// Column sums over a molecule's tokens: every warp's partial sums, added in warp order.  acc[t][e] belongs to channel
// 8 (lane + 32 t) + e.
template <int VEC>
__device__ __forceinline__ void molecule_column_sums(float* part, const float (&acc)[VEC][8], int C, float* dst) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nvec = C >> 3;
  __syncthreads();
#pragma unroll
  for (int t = 0; t < VEC; ++t) {
    const int v = lane + 32 * t;
    if (v < nvec) st8<float>(part + warp * C + 8 * v, acc[t]);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += kAdaWarps * 32) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kAdaWarps; ++w) tot += part[w * C + c];
    dst[c] = tot;
  }
}

// dx, and per molecule dshift[c] = sum_n dh, dscale[c] = sum_n dh * xhat.  One sweep: the row's dh and xhat stay in
// registers between the two row sums and the store.
template <typename TX, typename TH, int VEC>
__global__ void __launch_bounds__(kAdaWarps * 32) ln_modulate_bwd_kernel(const TH* __restrict__ dh,
                                                                         const TX* __restrict__ x,
                                                                         const float* __restrict__ scale,
                                                                         const float* __restrict__ mean_in,
                                                                         const float* __restrict__ rstd_in, int N, int C,
                                                                         TX* __restrict__ dx,
                                                                         float* __restrict__ dshift,
                                                                         float* __restrict__ dscale) {
  extern __shared__ __align__(16) float part[];  // [kAdaWarps][C]
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* sc = scale + (size_t)b * C;
  const int nvec = C >> 3;
  const float inv_c = 1.f / (float)C;
  float a_shift[VEC][8], a_scale[VEC][8], one_plus[VEC][8];
#pragma unroll
  for (int t = 0; t < VEC; ++t) {
    const int v = lane + 32 * t;
#pragma unroll
    for (int e = 0; e < 8; ++e) a_shift[t][e] = 0.f, a_scale[t][e] = 0.f, one_plus[t][e] = 1.f;
    if (v < nvec) {
      ld8<float>(sc + 8 * v, one_plus[t]);
#pragma unroll
      for (int e = 0; e < 8; ++e) one_plus[t][e] += 1.f;
    }
  }
  for (int n = warp; n < N; n += kAdaWarps) {
    const size_t row = (size_t)b * N + n;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float g[VEC][8], xh[VEC][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int t = 0; t < VEC; ++t) {
      const int v = lane + 32 * t;
      if (v < nvec) {
        ld8<TH>(dh + row * C + 8 * v, g[t]);
        ld8<TX>(x + row * C + 8 * v, xh[t]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[t][e] = (xh[t][e] - mean) * rstd;
          a_shift[t][e] += g[t][e];
          a_scale[t][e] = fmaf(g[t][e], xh[t][e], a_scale[t][e]);
          g[t][e] *= one_plus[t][e];  // gradient of the normalised row
          s1 += g[t][e];
          s2 = fmaf(g[t][e], xh[t][e], s2);
        }
      }
    }
    s1 = warp_sum(s1) * inv_c;
    s2 = warp_sum(s2) * inv_c;
#pragma unroll
    for (int t = 0; t < VEC; ++t) {
      const int v = lane + 32 * t;
      if (v < nvec) {
        float out[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) out[e] = rstd * (g[t][e] - s1 - xh[t][e] * s2);
        st8<TX>(dx + row * C + 8 * v, out);
      }
    }
  }
  molecule_column_sums(part, a_shift, C, dshift + (size_t)b * C);
  molecule_column_sums(part, a_scale, C, dscale + (size_t)b * C);
}

// y = x + gate_b * a; rows flagged in `pad` (nullable, (B, N) bytes) become zeros.  One vector of eight channels per thread.
template <typename TX, typename TA>
__global__ void gated_residual_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ gate,
                                          const TA* __restrict__ a, const uint8_t* __restrict__ pad, int N, int C,
                                          long long total, TX* __restrict__ y) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= total) return;
  const int c = (int)(i % C);
  const long long row = i / C;
  float out[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (!(pad && pad[row])) {
    float xv[8], av[8], gv[8];
    ld8<TX>(x + i, xv);
    ld8<TA>(a + i, av);
    ld8<float>(gate + (row / N) * C + c, gv);
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = fmaf(gv[e], av[e], xv[e]);
  }
  st8<TX>(y + i, out);
}

// da = dy * gate_b (in a's type), dgate[b,c] = sum_n dy * a; with `pad`, flagged rows count as dy = 0 and
// dx = dy with those rows cleared is written as well (without it the gradient of x is dy itself).
template <typename TX, typename TA, int VEC>
__global__ void __launch_bounds__(kAdaWarps * 32) gated_residual_bwd_kernel(const TX* __restrict__ dy,
                                                                            const float* __restrict__ gate,
                                                                            const TA* __restrict__ a,
                                                                            const uint8_t* __restrict__ pad, int N, int C,
                                                                            TA* __restrict__ da, TX* __restrict__ dx,
                                                                            float* __restrict__ dgate) {
  extern __shared__ __align__(16) float part[];  // [kAdaWarps][C]
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* gt = gate + (size_t)b * C;
  const int nvec = C >> 3;
  float acc[VEC][8], gv[VEC][8];
#pragma unroll
  for (int t = 0; t < VEC; ++t) {
    const int v = lane + 32 * t;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[t][e] = 0.f, gv[t][e] = 0.f;
    if (v < nvec) ld8<float>(gt + 8 * v, gv[t]);
  }
  for (int n = warp; n < N; n += kAdaWarps) {
    const size_t row = (size_t)b * N + n;
    const bool hidden = pad && pad[row];
#pragma unroll
    for (int t = 0; t < VEC; ++t) {
      const int v = lane + 32 * t;
      if (v < nvec) {
        float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, av[8], out[8];
        if (!hidden) {
          ld8<TX>(dy + row * C + 8 * v, g);
          ld8<TA>(a + row * C + 8 * v, av);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[t][e] = fmaf(g[e], av[e], acc[t][e]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) out[e] = g[e] * gv[t][e];
        st8<TA>(da + row * C + 8 * v, out);
        if (dx) st8<TX>(dx + row * C + 8 * v, g);
      }
    }
  }
  molecule_column_sums(part, acc, C, dgate + (size_t)b * C);
}

int check_sizes(const char* name, int batch, int tokens, int channels, int half_dtype) {
  MF_CHECK_ARG(batch >= 0 && tokens >= 0 && channels >= 1, "%s: bad size", name);
  MF_CHECK_ARG(channels <= 256 * kAdaVec && channels % 8 == 0, "%s: channels must be a multiple of 8, at most %d, got %d",
               name, 256 * kAdaVec, channels);
  MF_CHECK_ARG(half_dtype == MF_DTYPE_F32 || half_dtype == MF_DTYPE_BF16, "%s: tensor type must be float32 or bfloat16",
               name);
  return MF_OK;
}

}  // namespace
}  // namespace mf

using namespace mf;

// dispatch on the 8-channel vectors a lane holds per row: 1 (C <= 256), 2 (C <= 512) or 4 (C <= 1024)
#define MF_ADA_VEC(channels, VEC, ...)   \
  do {                                   \
    if ((channels) <= 256) {             \
      constexpr int VEC = 1;             \
      __VA_ARGS__;                       \
    } else if ((channels) <= 512) {      \
      constexpr int VEC = 2;             \
      __VA_ARGS__;                       \
    } else {                             \
      constexpr int VEC = 4;             \
      __VA_ARGS__;                       \
    }                                    \
  } while (0)

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
                  MF_ADA_VEC(channels, VEC,
                             (ln_modulate_fwd_kernel<TX, TH, VEC><<<batch, kAdaWarps * 32, 0, s>>>(
                                 static_cast<const TX*>(x), shift, scale, tokens, channels, eps, static_cast<TH*>(h), mean,
                                 rstd))));
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
                  MF_ADA_VEC(channels, VEC,
                             (ln_modulate_bwd_kernel<TX, TH, VEC><<<batch, kAdaWarps * 32, smem, s>>>(
                                 static_cast<const TH*>(dh), static_cast<const TX*>(x), scale, mean, rstd, tokens, channels,
                                 static_cast<TX*>(dx), dshift, dscale))));
  MF_CHECK_LAUNCH("ln_modulate_bwd_kernel");
  return MF_OK;
}

extern "C" int mf_gated_residual_fwd(const void* x, int32_t x_dtype, const float* gate, const void* a, int32_t a_dtype,
                                     const uint8_t* pad, int32_t batch, int32_t tokens, int32_t channels, void* y,
                                     void* stream) {
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
                      static_cast<const TX*>(x), gate, static_cast<const TA*>(a), pad, tokens, channels, total,
                      static_cast<TX*>(y))));
  MF_CHECK_LAUNCH("gated_residual_fwd_kernel");
  return MF_OK;
}

extern "C" int mf_gated_residual_bwd(const void* dy, int32_t dy_dtype, const float* gate, const void* a, int32_t a_dtype,
                                     const uint8_t* pad, int32_t batch, int32_t tokens, int32_t channels, void* da,
                                     void* dx, float* dgate, void* stream) {
  int rc = check_sizes("mf_gated_residual_bwd", batch, tokens, channels, a_dtype);
  if (rc == MF_OK) rc = check_sizes("mf_gated_residual_bwd", batch, tokens, channels, dy_dtype);
  if (rc != MF_OK) return rc;
  if (batch == 0) return MF_OK;
  MF_CHECK_ARG(dy && gate && a && da && dgate, "mf_gated_residual_bwd: null pointer argument");
  MF_CHECK_ALIGNED("mf_gated_residual_bwd", dy, gate, a, da, dx, dgate);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)kAdaWarps * channels * sizeof(float);
  MF_ADA_DISPATCH(dy_dtype, a_dtype, TX, TA,
                  MF_ADA_VEC(channels, VEC,
                             (gated_residual_bwd_kernel<TX, TA, VEC><<<batch, kAdaWarps * 32, smem, s>>>(
                                 static_cast<const TX*>(dy), gate, static_cast<const TA*>(a), pad, tokens, channels,
                                 static_cast<TA*>(da), static_cast<TX*>(dx), dgate))));
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
