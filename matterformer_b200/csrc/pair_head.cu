// Equivariant coordinate head of the denoiser (models/qm9.py:478-501 of the reference, on the pair geometry of
// geometry/adapters.py:83-125): for every ordered pair of real atoms (i, j), i != j,
//
//   w_ij     = w_out . silu(a_i + b_j + W_rbf rbf(|x_i - x_j| / rms)) + b_out
//   raw_i    = sum_j w_ij (x_i - x_j) / n                     n = real atoms of the molecule
//   out_i    = raw_i - mean over real atoms of raw            (0 on padding)
//
// where a = h W_i^T and b = h W_j^T + b_0 are the two halves of the pair MLP's first Linear applied to the trunk output
// (two small GEMMs done by the caller), rbf_r(d) = exp(-gamma (d - c_r)^2) and rms is the root-mean-square radius of the
// molecule.  The reference materialises cat[h_i, h_j, rbf_ij] as a (B, N, N, 2d+16) tensor and runs the MLP on it;
// here nothing of size N^2 x channels ever reaches memory.
//
// Mapping: a warp owns one atom ("owner") and walks its partners; lane l holds channels l, l+32, l+64, l+96 of the
// 128-wide hidden layer, with its 4 x 16 slice of W_rbf in registers.  The real partners of a chunk of 64 atoms are
// compacted into shared memory (positions, index, fp32 vectors), so the walk has no branches: the diagonal pair gets a
// zero factor.  The 16 radial basis values of 32 partners are computed one partner per lane and handed round through
// shared memory.  In the forward pass every lane keeps its own share of sum_j w_ij (x_i - x_j); the lanes are summed
// once per owner.  CTAs of four warps, several per SM, so that one CTA's staging overlaps another's arithmetic.
//
// The backward pass runs the same walk twice so that every sum has one owner and a fixed order (no atomics, results
// are reproducible): once with the owner as i (gives grad a_i and the parameter gradients, accumulated in registers
// over all work of a CTA and reduced over CTAs by a second kernel) and once with the owner as j (gives grad b_j).
// Coordinates are inputs of the denoiser, not parameters: no gradient with respect to them is produced.
#include <cstddef>

#include "common.cuh"

namespace mf {
namespace {

constexpr int kHid = 128;                   // hidden width of the pair MLP
constexpr int kRbf = 16;                    // radial basis functions
constexpr int kWarps = 4;                   // owners worked on at a time
constexpr int kPer = kHid / 32;             // channels per lane
constexpr int kChunk = 64;                  // atoms whose real members are staged at a time
constexpr int kRbfStride = 20;              // floats per partner in the hand-over buffer (16 + 4: conflict-free 16-byte stores)
constexpr int kParamFloats = kHid * kRbf + kHid + 1;  // grad W_rbf, grad w_out, grad b_out

enum PairMode { kForward = 0, kBackwardRows = 1, kBackwardCols = 2 };

struct PairHeadParams {
  const void* a;
  const void* b;
  const float* coords;
  const uint8_t* valid;
  const float* w_rbf;
  const float* w_out;
  const float* b_out;
  const float* centers;
  float gamma;
  int batch, tokens;
  int rows_per_item;      // owners per work item, a multiple of kWarps; kWarps when the molecule needs several chunks
  float* out;             // forward: raw_i (before the mean is removed)
  const float* grad_out;  // backward
  void* grad_vec;         // backward: grad a (rows) or grad b (cols)
  float* partials;        // backward rows: (gridDim.x, kParamFloats)
};

struct __align__(16) PairShared {
  float part[kChunk][kHid];   // vectors of the real partners, compacted
  float4 pxyz[kChunk];        // their positions; w holds the atom index as an integer (-1: filler)
  float4 pg[kChunk];          // their share of the output gradient (backward, owner = j)
  float rbf[kWarps][32 * kRbfStride];  // radial basis values of 32 partners per warp (read and written 16 bytes at a time)
  int src[kChunk];            // their atom indices
  int count;                  // how many there are
};
static_assert(offsetof(PairShared, pxyz) % 16 == 0 && offsetof(PairShared, pg) % 16 == 0 &&
                  offsetof(PairShared, rbf) % 16 == 0 && (32 * kRbfStride * sizeof(float)) % 16 == 0 &&
                  (kRbfStride * sizeof(float)) % 16 == 0,
              "16-byte accesses into PairShared");

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x, v[1] = x.y, v[2] = x.z, v[3] = x.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 x = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(x.x << 16), v[1] = __uint_as_float(x.x & 0xffff0000u);
  v[2] = __uint_as_float(x.y << 16), v[3] = __uint_as_float(x.y & 0xffff0000u);
}

template <typename T, int MODE>
__global__ void __launch_bounds__(kWarps * 32) pair_head_kernel(const PairHeadParams p) {
  constexpr int U = MODE == kBackwardRows ? 1 : 2;  // partners per step of the walk
  extern __shared__ __align__(16) unsigned char smem_raw[];
  PairShared& sm = *reinterpret_cast<PairShared*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.tokens;
  const int row_blocks = (N + p.rows_per_item - 1) / p.rows_per_item;
  const long long items = (long long)p.batch * row_blocks;
  const bool one_chunk = N <= kChunk;  // then the partners are staged once per work item

  // the lane's slice of the parameters
  float wr[kPer][kRbf], wo[kPer];
#pragma unroll
  for (int m = 0; m < kPer; ++m) {
    wo[m] = p.w_out[lane + 32 * m];
#pragma unroll
    for (int r = 0; r < kRbf; ++r) wr[m][r] = p.w_rbf[(lane + 32 * m) * kRbf + r];
  }
  const float b_out = p.b_out[0];
  const T* own_src = static_cast<const T*>(MODE == kBackwardCols ? p.b : p.a);
  const T* partner_src = static_cast<const T*>(MODE == kBackwardCols ? p.a : p.b);

  // parameter gradients of everything this CTA works on (owner = i pass only)
  float g_wr[MODE == kBackwardRows ? kPer : 1][MODE == kBackwardRows ? kRbf : 1] = {};
  float g_wo[kPer] = {};
  float g_bo = 0.f;

  for (long long item = blockIdx.x; item < items; item += gridDim.x) {
    const int b = (int)(item / row_blocks);
    const int r0 = (int)(item % row_blocks) * p.rows_per_item;
    const float* xyz = p.coords + (size_t)b * N * 3;
    const uint8_t* val = p.valid + (size_t)b * N;

    // molecule statistics, every warp for itself in one fixed order
    float cnt = 0.f, sq = 0.f, gs[3] = {0.f, 0.f, 0.f};
    for (int t = lane; t < N; t += 32) {
      if (val[t]) {
        const float x = xyz[t * 3], y = xyz[t * 3 + 1], z = xyz[t * 3 + 2];
        cnt += 1.f;
        sq += x * x + y * y + z * z;
        if (MODE != kForward) {
          const float* g = p.grad_out + ((size_t)b * N + t) * 3;
          gs[0] += g[0], gs[1] += g[1], gs[2] += g[2];
        }
      }
    }
    cnt = warp_sum(cnt), sq = warp_sum(sq);
    const float rms = fmaxf(sqrtf(fmaxf(sq / fmaxf(cnt, 1.f), 1e-8f)), 1e-8f);
    const float inv_n = 1.f / fmaxf(cnt, 1.f);
    float gmean[3] = {0.f, 0.f, 0.f};
    if (MODE != kForward) {
#pragma unroll
      for (int c = 0; c < 3; ++c) gmean[c] = warp_sum(gs[c]) * inv_n;
    }

    for (int o = r0 + warp; o - warp < min(r0 + p.rows_per_item, N); o += kWarps) {  // same trip count in every warp
      const bool own_valid = o < N && val[o] != 0;
      float ox = 0.f, oy = 0.f, oz = 0.f, own[kPer] = {};
      float og[3] = {0.f, 0.f, 0.f};  // owner's share of the output gradient (owner = i)
      if (own_valid) {
        ox = xyz[o * 3], oy = xyz[o * 3 + 1], oz = xyz[o * 3 + 2];
#pragma unroll
        for (int m = 0; m < kPer; ++m) own[m] = to_f32(own_src[((size_t)b * N + o) * kHid + lane + 32 * m]);
        if (MODE == kBackwardRows) {
          const float* g = p.grad_out + ((size_t)b * N + o) * 3;
#pragma unroll
          for (int c = 0; c < 3; ++c) og[c] = (g[c] - gmean[c]) * inv_n;
        }
      }
      float acc[3] = {0.f, 0.f, 0.f};   // forward: this lane's share of sum_j w_ij (x_i - x_j)
      float dsum[3] = {0.f, 0.f, 0.f};  // forward: sum_j (x_i - x_j), for the bias of the second Linear
      float g_vec[kPer] = {};           // backward: grad a_i or grad b_j

      for (int t0 = 0; t0 < N; t0 += kChunk) {
        if (!one_chunk || o - warp == r0) {
          __syncthreads();  // nobody reads the previous chunk any more
          if (warp == 0) {  // compact the chunk's real atoms
            int base = 0;
#pragma unroll
            for (int half = 0; half < kChunk / 32; ++half) {
              const int t = t0 + half * 32 + lane;
              const bool v = t < N && val[t] != 0;
              const unsigned mask = __ballot_sync(0xffffffffu, v);
              if (v) {
                const int pos = base + __popc(mask & ((1u << lane) - 1u));
                sm.pxyz[pos] = make_float4(xyz[t * 3], xyz[t * 3 + 1], xyz[t * 3 + 2], __int_as_float(t));
                sm.src[pos] = t;
                if (MODE == kBackwardCols) {
                  const float* g = p.grad_out + ((size_t)b * N + t) * 3;
                  sm.pg[pos] = make_float4((g[0] - gmean[0]) * inv_n, (g[1] - gmean[1]) * inv_n, (g[2] - gmean[2]) * inv_n, 0.f);
                }
              }
              base += __popc(mask);
            }
            if (lane == 0) {
              sm.count = base;
              if (base < kChunk) {  // filler that completes the last step of the walk
                sm.pxyz[base] = make_float4(0.f, 0.f, 0.f, __int_as_float(-1));
                sm.pg[base] = make_float4(0.f, 0.f, 0.f, 0.f);
              }
            }
          }
          __syncthreads();
          const int rows = min(kChunk, (sm.count + U - 1) / U * U);
          for (int e = tid; e < rows * (kHid / 4); e += kWarps * 32) {
            const int k = e / (kHid / 4), c4 = (e % (kHid / 4)) * 4;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (k < sm.count) load4<T>(partner_src + ((size_t)b * N + sm.src[k]) * kHid + c4, v);
            *reinterpret_cast<float4*>(&sm.part[k][c4]) = make_float4(v[0], v[1], v[2], v[3]);
          }
          __syncthreads();
        }
        if (!own_valid) continue;  // whole warp: a padded owner has no pairs
        const int steps_end = min(kChunk, (sm.count + U - 1) / U * U);

        for (int s0 = 0; s0 < steps_end; s0 += 32) {
          {  // radial basis of partner s0 + lane, for the other lanes to read
            float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s0 + lane < steps_end) q = sm.pxyz[s0 + lane];
            const float dx = ox - q.x, dy = oy - q.y, dz = oz - q.z;
            const float dn = sqrtf(fmaxf(dx * dx + dy * dy + dz * dz, 0.f)) / rms;
            float* dst = &sm.rbf[warp][lane * kRbfStride];
            __syncwarp();  // the previous block's readers are done
#pragma unroll
            for (int r = 0; r < kRbf; r += 4) {
              float e[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float u = dn - p.centers[r + k];
                e[k] = __expf(-p.gamma * u * u);
              }
              *reinterpret_cast<float4*>(dst + r) = make_float4(e[0], e[1], e[2], e[3]);
            }
            __syncwarp();
          }
          const int t_end = min(32, steps_end - s0);
          for (int tt = 0; tt < t_end; tt += U) {
            float rb[U][kRbf], d[U][3], dw[U], keep[U], wsum[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const float4 q = sm.pxyz[s0 + tt + u];
              const int j = __float_as_int(q.w);
              keep[u] = (j != o && j >= 0) ? 1.f : 0.f;  // the diagonal and the filler carry no weight
#pragma unroll
              for (int r = 0; r < kRbf; r += 4) {
                const float4 e = *reinterpret_cast<const float4*>(&sm.rbf[warp][(tt + u) * kRbfStride + r]);
                rb[u][r] = e.x, rb[u][r + 1] = e.y, rb[u][r + 2] = e.z, rb[u][r + 3] = e.w;
              }
              // x_i - x_j with i the first index of the pair
              const float sgn = MODE == kBackwardCols ? -1.f : 1.f;
              d[u][0] = sgn * (ox - q.x), d[u][1] = sgn * (oy - q.y), d[u][2] = sgn * (oz - q.z);
              dw[u] = 0.f, wsum[u] = 0.f;
              if (MODE == kBackwardRows) dw[u] = keep[u] * (og[0] * d[u][0] + og[1] * d[u][1] + og[2] * d[u][2]);
              if (MODE == kBackwardCols) {
                const float4 g4 = sm.pg[s0 + tt + u];
                dw[u] = keep[u] * (g4.x * d[u][0] + g4.y * d[u][1] + g4.z * d[u][2]);
              }
            }
#pragma unroll
            for (int m = 0; m < kPer; ++m) {
#pragma unroll
              for (int u = 0; u < U; ++u) {
                float pre = own[m] + sm.part[s0 + tt + u][lane + 32 * m];
#pragma unroll
                for (int r = 0; r < kRbf; ++r) pre = fmaf(wr[m][r], rb[u][r], pre);
                const float sig = __fdividef(1.f, 1.f + __expf(-pre));
                if (MODE == kForward) {
                  wsum[u] = fmaf(wo[m], pre * sig, wsum[u]);
                } else {
                  const float dh = dw[u] * wo[m] * sig * fmaf(pre, 1.f - sig, 1.f);
                  g_vec[m] += dh;
                  if constexpr (MODE == kBackwardRows) {
                    g_wo[m] = fmaf(dw[u], pre * sig, g_wo[m]);
#pragma unroll
                    for (int r = 0; r < kRbf; ++r) g_wr[m][r] = fmaf(dh, rb[u][r], g_wr[m][r]);
                  }
                }
              }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              if (MODE == kForward) {
                const float w = wsum[u] * keep[u];
#pragma unroll
                for (int c = 0; c < 3; ++c) acc[c] = fmaf(w, d[u][c], acc[c]), dsum[c] = fmaf(keep[u], d[u][c], dsum[c]);
              }
              if (MODE == kBackwardRows) g_bo += dw[u];
            }
          }
        }
      }

      if (o < N) {
        if (MODE == kForward) {
#pragma unroll
          for (int c = 0; c < 3; ++c) acc[c] = (warp_sum(acc[c]) + b_out * dsum[c]) * inv_n;
          if (lane < 3) p.out[((size_t)b * N + o) * 3 + lane] = lane == 0 ? acc[0] : lane == 1 ? acc[1] : acc[2];
        } else {
          T* dst = static_cast<T*>(p.grad_vec) + ((size_t)b * N + o) * kHid;
#pragma unroll
          for (int m = 0; m < kPer; ++m) dst[lane + 32 * m] = from_f32<T>(g_vec[m]);
        }
      }
    }
  }

  if constexpr (MODE == kBackwardRows) {
    // warps add their sums into one shared copy in warp order, then the CTA writes its line of partial sums
    __syncthreads();
    float* red = &sm.part[0][0];
    for (int w = 0; w < kWarps; ++w) {
      if (warp == w) {
#pragma unroll
        for (int m = 0; m < kPer; ++m) {
          const int c = lane + 32 * m;
#pragma unroll
          for (int r = 0; r < kRbf; ++r) red[c * kRbf + r] = (w ? red[c * kRbf + r] : 0.f) + g_wr[m][r];
          red[kHid * kRbf + c] = (w ? red[kHid * kRbf + c] : 0.f) + g_wo[m];
        }
        if (lane == 0) red[kHid * kRbf + kHid] = (w ? red[kHid * kRbf + kHid] : 0.f) + g_bo;
      }
      __syncthreads();
    }
    float* dst = p.partials + (size_t)blockIdx.x * kParamFloats;
    for (int e = tid; e < kParamFloats; e += kWarps * 32) dst[e] = red[e];
  }
}

// out_i = raw_i - mean over the molecule's real atoms; zero on padding.  One warp per molecule.
__global__ void pair_head_center_kernel(float* out, const uint8_t* valid, int batch, int tokens) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (b >= batch) return;
  float* o = out + (size_t)b * tokens * 3;
  const uint8_t* v = valid + (size_t)b * tokens;
  float cnt = 0.f, s[3] = {0.f, 0.f, 0.f};
  for (int t = lane; t < tokens; t += 32)
    if (v[t]) cnt += 1.f, s[0] += o[t * 3], s[1] += o[t * 3 + 1], s[2] += o[t * 3 + 2];
  cnt = fmaxf(warp_sum(cnt), 1.f);
#pragma unroll
  for (int c = 0; c < 3; ++c) s[c] = warp_sum(s[c]) / cnt;
  for (int t = lane; t < tokens; t += 32)
#pragma unroll
    for (int c = 0; c < 3; ++c) o[t * 3 + c] = v[t] ? o[t * 3 + c] - s[c] : 0.f;
}

// Sums the CTAs' lines of partial parameter gradients in CTA order.
__global__ void pair_head_param_sum_kernel(const float* partials, int lines, float* g_w_rbf, float* g_w_out,
                                           float* g_b_out) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= kParamFloats) return;
  float s = 0.f;
  for (int l = 0; l < lines; ++l) s += partials[(size_t)l * kParamFloats + e];
  if (e < kHid * kRbf) g_w_rbf[e] = s;
  else if (e < kHid * kRbf + kHid) g_w_out[e - kHid * kRbf] = s;
  else g_b_out[0] = s;
}

int check_args(const char* name, const MfPairHeadArgs* a, bool backward) {
  MF_CHECK_ARG(a != nullptr, "%s: null argument block", name);
  MF_CHECK_ARG(a->batch >= 0 && a->tokens >= 0, "%s: negative size", name);
  MF_CHECK_ARG(a->dtype == MF_DTYPE_F32 || a->dtype == MF_DTYPE_BF16, "%s: a / b must be float32 or bfloat16", name);
  MF_CHECK_ARG(a->hidden == kHid && a->n_rbf == kRbf, "%s: built for a hidden width of %d and %d radial basis functions, got %d and %d",
               name, kHid, kRbf, a->hidden, a->n_rbf);
  MF_CHECK_ARG((long long)a->batch * a->tokens < (1LL << 31) / kHid, "%s: batch * tokens too large", name);
  if (a->batch == 0 || a->tokens == 0) return MF_OK;
  MF_CHECK_ARG(a->a && a->b && a->coords && a->valid && a->w_rbf && a->w_out && a->b_out && a->centers,
               "%s: null input pointer", name);
  MF_CHECK_ALIGNED(name, a->a, a->b, a->w_rbf, a->w_out);
  if (!backward) {
    MF_CHECK_ARG(a->out != nullptr, "%s: null output pointer", name);
  } else {
    MF_CHECK_ARG(a->grad_out && a->grad_a && a->grad_b && a->grad_w_rbf && a->grad_w_out && a->grad_b_out,
                 "%s: null gradient pointer", name);
    MF_CHECK_ALIGNED(name, a->grad_a, a->grad_b);
  }
  return MF_OK;
}

PairHeadParams params_of(const MfPairHeadArgs* a) {
  PairHeadParams p{};
  p.a = a->a, p.b = a->b, p.coords = a->coords, p.valid = a->valid;
  p.w_rbf = a->w_rbf, p.w_out = a->w_out, p.b_out = a->b_out, p.centers = a->centers;
  p.gamma = a->gamma, p.batch = a->batch, p.tokens = a->tokens;
  p.out = a->out, p.grad_out = a->grad_out;
  return p;
}

// Persistent grid: as many CTAs as fit on the device at once (two or three per SM, by registers), never more than
// there are work items.
template <typename T, int MODE>
int grid_size(long long items, int* blocks) {
  int dev = 0, sms = 0, per_sm = 0;
  cudaError_t e = cudaFuncSetAttribute(pair_head_kernel<T, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)sizeof(PairShared));
  if (e == cudaSuccess) e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess)
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pair_head_kernel<T, MODE>, kWarps * 32, sizeof(PairShared));
  if (e != cudaSuccess) return cuda_error(e, "pair_head_kernel: launch configuration");
  const long long cap = (long long)sms * (per_sm > 0 ? per_sm : 1);
  *blocks = (int)(items < cap ? items : cap);
  return MF_OK;
}

template <int MODE>
int grid_size_dtype(int dtype, long long items, int* blocks) {
  return dtype == MF_DTYPE_F32 ? grid_size<float, MODE>(items, blocks) : grid_size<__nv_bfloat16, MODE>(items, blocks);
}

template <typename T, int MODE>
int launch(const PairHeadParams& p, int blocks, cudaStream_t s) {
  pair_head_kernel<T, MODE><<<blocks, kWarps * 32, sizeof(PairShared), s>>>(p);
  MF_CHECK_LAUNCH("pair_head_kernel");
  return MF_OK;
}

template <int MODE>
int launch_dtype(int dtype, const PairHeadParams& p, int blocks, cudaStream_t s) {
  return dtype == MF_DTYPE_F32 ? launch<float, MODE>(p, blocks, s) : launch<__nv_bfloat16, MODE>(p, blocks, s);
}

// Owners per work item.  A molecule that fits one chunk is staged once per item, so items should be as large as the
// balance of a persistent grid allows (about eight items per SM); larger molecules take one round of owners per item.
int plan_items(const MfPairHeadArgs* a, int* rows_per_item, long long* items) {
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_error(e, "mf_pair_head: device query");
  int rows = kWarps;
  if (a->tokens <= kChunk) {
    const long long split = (8LL * sms + a->batch - 1) / a->batch;  // row blocks wanted per molecule
    rows = (int)((a->tokens + split - 1) / split);
    rows = (rows + kWarps - 1) / kWarps * kWarps;
  }
  *rows_per_item = rows;
  *items = (long long)a->batch * ((a->tokens + rows - 1) / rows);
  return MF_OK;
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" size_t mf_pair_head_bwd_workspace_bytes(const MfPairHeadArgs* a) {
  if (!a || a->batch <= 0 || a->tokens <= 0) return 0;
  int blocks = 0, rows = 0;
  long long items = 0;
  if (plan_items(a, &rows, &items) != MF_OK || grid_size_dtype<kBackwardRows>(a->dtype, items, &blocks) != MF_OK) return 0;
  return (size_t)blocks * kParamFloats * sizeof(float);
}

extern "C" int mf_pair_head_fwd(const MfPairHeadArgs* a, void* stream) {
  int rc = check_args("mf_pair_head_fwd", a, false);
  if (rc != MF_OK || a->batch == 0 || a->tokens == 0) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int blocks = 0, rows = 0;
  long long items = 0;
  rc = plan_items(a, &rows, &items);
  if (rc == MF_OK) rc = grid_size_dtype<kForward>(a->dtype, items, &blocks);
  if (rc != MF_OK) return rc;
  PairHeadParams p = params_of(a);
  p.rows_per_item = rows;
  rc = launch_dtype<kForward>(a->dtype, p, blocks, s);
  if (rc != MF_OK) return rc;
  pair_head_center_kernel<<<(a->batch + 7) / 8, 256, 0, s>>>(a->out, a->valid, a->batch, a->tokens);
  MF_CHECK_LAUNCH("pair_head_center_kernel");
  return MF_OK;
}

extern "C" int mf_pair_head_bwd(const MfPairHeadArgs* a, void* stream) {
  int rc = check_args("mf_pair_head_bwd", a, true);
  if (rc != MF_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a->batch == 0 || a->tokens == 0) {  // no pairs: the parameter gradients are zero
    if (a->grad_w_rbf && a->grad_w_out && a->grad_b_out) {
      cudaError_t e = cudaMemsetAsync(a->grad_w_rbf, 0, sizeof(float) * kHid * kRbf, s);
      if (e == cudaSuccess) e = cudaMemsetAsync(a->grad_w_out, 0, sizeof(float) * kHid, s);
      if (e == cudaSuccess) e = cudaMemsetAsync(a->grad_b_out, 0, sizeof(float), s);
      if (e != cudaSuccess) return cuda_error(e, "mf_pair_head_bwd: memset");
    }
    return MF_OK;
  }
  int blocks = 0, col_blocks = 0, rows = 0;
  long long items = 0;
  rc = plan_items(a, &rows, &items);
  if (rc == MF_OK) rc = grid_size_dtype<kBackwardRows>(a->dtype, items, &blocks);
  if (rc == MF_OK) rc = grid_size_dtype<kBackwardCols>(a->dtype, items, &col_blocks);
  if (rc != MF_OK) return rc;
  const size_t need = (size_t)blocks * kParamFloats * sizeof(float);
  MF_CHECK_ARG(a->workspace && a->workspace_bytes >= need, "mf_pair_head_bwd: workspace of %zu bytes needed, %zu given", need,
               a->workspace_bytes);
  PairHeadParams p = params_of(a);
  p.rows_per_item = rows;
  p.partials = static_cast<float*>(a->workspace);
  p.grad_vec = a->grad_a;
  rc = launch_dtype<kBackwardRows>(a->dtype, p, blocks, s);
  if (rc != MF_OK) return rc;
  p.grad_vec = a->grad_b;
  rc = launch_dtype<kBackwardCols>(a->dtype, p, col_blocks, s);
  if (rc != MF_OK) return rc;
  pair_head_param_sum_kernel<<<(kParamFloats + 255) / 256, 256, 0, s>>>(p.partials, blocks, a->grad_w_rbf, a->grad_w_out,
                                                                        a->grad_b_out);
  MF_CHECK_LAUNCH("pair_head_param_sum_kernel");
  return MF_OK;
}
