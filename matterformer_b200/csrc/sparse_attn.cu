// Radius block-sparse attention and local-window attention over cell-sorted
// tokens, forward and backward.
//
// Both operators are softmax attention with a per-pair visibility mask, the
// computation F.scaled_dot_product_attention performs for the reference's
// RotaryMultiheadAttention (src/matterformer/models/regular_attention.py:251-268)
// when it is handed an additive 0/-inf mask; here the mask is never
// materialised:
//   radius : pairs come from the block list; inside an active 32x32 block the
//            visible pairs are the set bits of the block's bitmap
//   local  : key j is visible to query i iff i-w/2 <= j <= i+w/2-1
//
// One warp owns one row (a query in the forward and dq kernels, a key in the
// dk/dv kernel); its partner rows come in groups of 32, one per lane, for the
// dot products, and are then revisited one by one with the lanes spread over
// the head dimension for the weighted sums.  No atomics: every output row has
// exactly one owner, so results are bit-identical from run to run.
#include "common.cuh"
#include "simplicial_sm100.cuh"
#include "sparse_attn_mma.cuh"
#include "sparse_attn_sm100.cuh"

namespace mf {
namespace {

enum { SP_FWD = 0, SP_DQ = 1, SP_DKV = 2 };

struct SparseParams {
  const void* q;
  const void* k;
  const void* v;
  const void* grad_out;
  const float* lse;
  const float* delta;
  const int32_t* num_atoms;
  const int32_t* block_count;
  const int32_t* block_cols;
  const uint32_t* block_mask;
  void* out;
  float* lse_out;
  void* dq;
  void* dk;
  void* dv;
  int H, N, window, tiles;
  float scale;
};

// 8 consecutive elements -> fp32
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&o)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
  o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    o[2 * t] = __uint_as_float(w[t] << 16);
    o[2 * t + 1] = __uint_as_float(w[t] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&o)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 f = __half22float2(h[t]);
    o[2 * t] = f.x;
    o[2 * t + 1] = f.y;
  }
}

// dot product of a partner row in global memory with an owner row in shared memory
template <typename T, int D>
__device__ __forceinline__ float row_dot(const T* row, const float* own) {
  float s = 0.f;
#pragma unroll
  for (int d0 = 0; d0 < D; d0 += 8) {
    float x[8];
    load8<T>(row + d0, x);
    const float4 a = *reinterpret_cast<const float4*>(own + d0);
    const float4 b = *reinterpret_cast<const float4*>(own + d0 + 4);
    s = fmaf(x[0], a.x, s); s = fmaf(x[1], a.y, s); s = fmaf(x[2], a.z, s); s = fmaf(x[3], a.w, s);
    s = fmaf(x[4], b.x, s); s = fmaf(x[5], b.y, s); s = fmaf(x[6], b.z, s); s = fmaf(x[7], b.w, s);
  }
  return s;
}

// Partner groups of an owner row.  group(t) yields the first partner row of group t and the
// bitmap of visible lanes.
template <bool kRadius, int MODE>
struct Partners {
  int count;
  // radius
  const int32_t* cols;
  const uint32_t* masks;  // base of mask[b][tile(o)][*][*]
  int lane_row;           // o % 32
  // local
  int first, lo, hi;

  __device__ __forceinline__ Partners(const SparseParams& p, int b, int o, int n) {
    if (kRadius) {
      const int tile = o >> 5;
      count = p.block_count[(size_t)b * p.tiles + tile];
      cols = p.block_cols + ((size_t)b * p.tiles + tile) * p.tiles;
      masks = p.block_mask + ((size_t)b * p.tiles + tile) * p.tiles * 32;
      lane_row = o & 31;
      first = lo = hi = 0;
    } else {
      const int half = p.window / 2;
      // query i sees keys [i-half, i+half-1]; key j is seen by queries [j-half+1, j+half]
      lo = (MODE == SP_DKV) ? o - half + 1 : o - half;
      hi = (MODE == SP_DKV) ? o + half : o + half - 1;
      lo = max(lo, 0);
      hi = min(hi, n - 1);
      first = lo;
      count = (hi >= lo) ? (hi - lo + 32) / 32 : 0;
      cols = nullptr;
      masks = nullptr;
      lane_row = 0;
    }
  }
  __device__ __forceinline__ void group(int t, int& row0, uint32_t& word) const {
    if (kRadius) {
      const int J = cols[t];
      row0 = 32 * J;
      // The bitmap is symmetric (distances are), so the same word serves queries looking at
      // keys and keys looking at queries.
      word = masks[(size_t)J * 32 + lane_row];
    } else {
      row0 = first + 32 * t;
      const int rem = hi - row0 + 1;
      word = rem >= 32 ? 0xffffffffu : ((1u << rem) - 1u);
    }
  }
};

template <typename T, int D, bool kRadius, int MODE>
__global__ void __launch_bounds__(128) sparse_attn_kernel(SparseParams p) {
  constexpr int DPL = D / 32;  // head-dim elements per lane in the weighted sums
  __shared__ __align__(16) float own_s[4][2][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, b = bh / p.H;
  const int N = p.N;
  const int n = min(p.num_atoms[b], N);
  const int o = blockIdx.x * 4 + warp;
  if (o >= N) return;
  const size_t base = (size_t)bh * N * D;
  const T* Q = static_cast<const T*>(p.q) + base;
  const T* K = static_cast<const T*>(p.k) + base;
  const T* V = static_cast<const T*>(p.v) + base;
  const T* dO = (MODE == SP_FWD) ? nullptr : static_cast<const T*>(p.grad_out) + base;
  const bool owner_ok = o < n;

  // partner matrices: A is dotted with own_a to give the logit, B with own_b to give dP
  //   FWD/DQ : owner = query -> own_a = q_o, partners A = K, own_b = dO_o, partners B = V
  //   DKV    : owner = key   -> own_a = k_o, partners A = Q, own_b = v_o,  partners B = dO
  const T* PA = (MODE == SP_DKV) ? Q : K;
  const T* PB = (MODE == SP_DKV) ? dO : V;
  float* own_a = own_s[warp][0];
  float* own_b = own_s[warp][1];
  if (owner_ok) {
    const T* ra = ((MODE == SP_DKV) ? K : Q) + (size_t)o * D;
    const T* rb = (MODE == SP_FWD) ? nullptr : ((MODE == SP_DKV) ? V : dO) + (size_t)o * D;
#pragma unroll
    for (int r = 0; r < DPL; ++r) {
      own_a[lane + 32 * r] = to_f32<T>(ra[lane + 32 * r]);
      if (MODE != SP_FWD) own_b[lane + 32 * r] = to_f32<T>(rb[lane + 32 * r]);
    }
  }
  __syncwarp();

  float acc0[DPL], acc1[DPL];
#pragma unroll
  for (int r = 0; r < DPL; ++r) acc0[r] = acc1[r] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  float own_lse = 0.f, own_delta = 0.f;
  if (MODE == SP_DQ && owner_ok) {
    own_lse = p.lse[(size_t)bh * N + o];
    own_delta = p.delta[(size_t)bh * N + o];
  }

  if (owner_ok) {
    const Partners<kRadius, MODE> parts(p, b, o, n);
    for (int t = 0; t < parts.count; ++t) {
      int row0;
      uint32_t word;
      parts.group(t, row0, word);
      if (word == 0u) continue;
      const int row = row0 + lane;
      const bool vis = (word >> lane) & 1u;
      float s = 0.f, c0 = 0.f, c1 = 0.f;
      if (vis) {
        s = row_dot<T, D>(PA + (size_t)row * D, own_a) * p.scale;
        if (MODE == SP_FWD) {
          // c0 is filled after the running maximum is known
        } else {
          const float l = (MODE == SP_DQ) ? own_lse : p.lse[(size_t)bh * N + row];
          const float dl = (MODE == SP_DQ) ? own_delta : p.delta[(size_t)bh * N + row];
          const float pr = expf(s - l);
          const float dp = row_dot<T, D>(PB + (size_t)row * D, own_b);
          c0 = pr * (dp - dl) * p.scale;  // dS
          c1 = pr;                        // P
        }
      }
      if (MODE == SP_FWD) {
        const float gmax = warp_max(vis ? s : -INFINITY);
        const float m_new = fmaxf(m_run, gmax);
        const float alpha = expf(m_run - m_new);  // 0 on the first visible group
        c0 = vis ? expf(s - m_new) : 0.f;
        l_run = l_run * alpha + warp_sum(c0);
#pragma unroll
        for (int r = 0; r < DPL; ++r) acc0[r] *= alpha;
        m_run = m_new;
      }
      // weighted sums over the visible partners, lanes spread over the head dimension
      uint32_t rest = word;
      while (rest) {
        const int c = __ffs(rest) - 1;
        rest &= rest - 1;
        const float w0 = __shfl_sync(0xffffffffu, c0, c);
        const size_t roff = (size_t)(row0 + c) * D;
        if (MODE == SP_FWD) {
#pragma unroll
          for (int r = 0; r < DPL; ++r) acc0[r] = fmaf(w0, to_f32<T>(V[roff + lane + 32 * r]), acc0[r]);
        } else if (MODE == SP_DQ) {
#pragma unroll
          for (int r = 0; r < DPL; ++r) acc0[r] = fmaf(w0, to_f32<T>(K[roff + lane + 32 * r]), acc0[r]);
        } else {
          const float w1 = __shfl_sync(0xffffffffu, c1, c);
#pragma unroll
          for (int r = 0; r < DPL; ++r) {
            acc0[r] = fmaf(w0, to_f32<T>(Q[roff + lane + 32 * r]), acc0[r]);   // dK += dS * q
            acc1[r] = fmaf(w1, to_f32<T>(dO[roff + lane + 32 * r]), acc1[r]);  // dV += P * dO
          }
        }
      }
    }
  }

  const size_t ooff = base + (size_t)o * D;
  if (MODE == SP_FWD) {
    const bool have = owner_ok && l_run > 0.f;
    const float inv = have ? 1.f / l_run : 0.f;
#pragma unroll
    for (int r = 0; r < DPL; ++r) static_cast<T*>(p.out)[ooff + lane + 32 * r] = from_f32<T>(acc0[r] * inv);
    if (lane == 0) p.lse_out[(size_t)bh * N + o] = have ? m_run + logf(l_run) : 0.f;
  } else if (MODE == SP_DQ) {
#pragma unroll
    for (int r = 0; r < DPL; ++r) static_cast<T*>(p.dq)[ooff + lane + 32 * r] = from_f32<T>(acc0[r]);
  } else {
#pragma unroll
    for (int r = 0; r < DPL; ++r) {
      static_cast<T*>(p.dk)[ooff + lane + 32 * r] = from_f32<T>(acc0[r]);
      static_cast<T*>(p.dv)[ooff + lane + 32 * r] = from_f32<T>(acc1[r]);
    }
  }
}

template <typename T>
__global__ void sparse_delta_kernel(const T* __restrict__ grad_out, const T* __restrict__ out,
                                    float* __restrict__ delta, int rows, int D) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float s = 0.f;
  for (int d = lane; d < D; d += 32)
    s = fmaf(to_f32<T>(grad_out[(size_t)row * D + d]), to_f32<T>(out[(size_t)row * D + d]), s);
  s = warp_sum(s);
  if (lane == 0) delta[row] = s;
}

template <typename T, int D, bool kRadius>
int launch_sparse(const MfSparseAttnArgs& a, bool backward, cudaStream_t s) {
  SparseParams p{};
  p.q = a.q;
  p.k = a.k;
  p.v = a.v;
  p.grad_out = a.grad_out;
  p.lse = a.lse;
  p.num_atoms = a.num_atoms;
  p.block_count = a.block_count;
  p.block_cols = a.block_cols;
  p.block_mask = a.block_mask;
  p.out = a.out;
  p.lse_out = a.lse;
  p.dq = a.dq;
  p.dk = a.dk;
  p.dv = a.dv;
  p.H = a.heads;
  p.N = a.tokens;
  p.window = a.window;
  p.tiles = (a.tokens + 31) / 32;
  p.scale = a.scale;
  const int BH = a.batch * a.heads;
  dim3 grid((a.tokens + 3) / 4, BH);
  if (!backward) {
    sparse_attn_kernel<T, D, kRadius, SP_FWD><<<grid, 128, 0, s>>>(p);
    MF_CHECK_LAUNCH("sparse_attn_kernel<fwd>");
    return MF_OK;
  }
  float* delta = static_cast<float*>(a.workspace);
  p.delta = delta;
  const int rows = BH * a.tokens;
  sparse_delta_kernel<T><<<(rows + 3) / 4, 128, 0, s>>>(static_cast<const T*>(a.grad_out),
                                                          static_cast<const T*>(a.out), delta, rows, D);
  MF_CHECK_LAUNCH("sparse_delta_kernel");
  sparse_attn_kernel<T, D, kRadius, SP_DQ><<<grid, 128, 0, s>>>(p);
  MF_CHECK_LAUNCH("sparse_attn_kernel<dq>");
  sparse_attn_kernel<T, D, kRadius, SP_DKV><<<grid, 128, 0, s>>>(p);
  MF_CHECK_LAUNCH("sparse_attn_kernel<dkv>");
  return MF_OK;
}

template <bool kRadius>
int run_sparse(const MfSparseAttnArgs* a, bool backward, void* stream, const char* name) {
  MF_CHECK_ARG(a != nullptr, "%s: null argument struct", name);
  MF_CHECK_ARG(a->batch >= 0 && a->heads >= 0 && a->tokens >= 0, "%s: negative size", name);
  MF_CHECK_ARG(a->head_dim == 32 || a->head_dim == 64 || a->head_dim == 128,
               "%s: head_dim must be 32, 64 or 128, got %d", name, (int)a->head_dim);
  if (a->batch == 0 || a->heads == 0 || a->tokens == 0) return MF_OK;
  MF_CHECK_ARG(a->q && a->k && a->v && a->num_atoms && a->out && a->lse, "%s: null tensor pointer", name);
  MF_CHECK_ALIGNED(name, a->q, a->k, a->v, a->out, a->grad_out, a->dq, a->dk, a->dv);
  if (kRadius) {
    MF_CHECK_ARG(a->block_count && a->block_cols && a->block_mask, "%s: block list pointers are required", name);
  } else {
    MF_CHECK_ARG(a->window >= 2 && a->window % 2 == 0, "%s: window must be a positive even number, got %d", name,
                 (int)a->window);
  }
  if (backward) {
    MF_CHECK_ARG(a->grad_out && a->dq && a->dk && a->dv, "%s: null gradient pointer", name);
    const size_t need = mf_sparse_attn_bwd_workspace_bytes(a);
    if (!a->workspace || a->workspace_bytes < need) {
      set_error("%s: workspace of %zu bytes needed, %zu given", name, need, a->workspace_bytes);
      return MF_ERR_WORKSPACE_TOO_SMALL;
    }
  }
  if (a->batch == 0 || a->heads == 0 || a->tokens == 0) return MF_OK;
  MF_CHECK_ARG((long long)a->batch * a->heads <= 65535, "%s: batch*heads above 65535", name);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // bf16 runs on the tensor cores; fp32 (1e-4 parity needs fp32 products) and fp16 use the CUDA-core kernels
  if (a->dtype == MF_DTYPE_BF16) {
    // 128-row tcgen05 tiles where the operator is close to dense attention with a bit mask (radius lists at a few
    // hundred atoms and more); the 32-row warp-level tiles for short structures and for the narrow band
    const bool fits = sparse_attn_sm100_applies(*a, backward);
    MF_CHECK_ARG(a->backend != MF_SPARSE_BACKEND_TCGEN05 || fits,
                 "%s: the tcgen05 kernels need bf16, head_dim 64, a multiple of four and at most 8192 tokens, 16-byte "
                 "aligned tensors and the driver's tensor-map encoder", name);
    const bool tc = a->backend == MF_SPARSE_BACKEND_TCGEN05 ||
                    (a->backend == MF_SPARSE_BACKEND_AUTO && fits && kRadius && a->tokens >= 256);
    if (tc) return backward ? sparse_attn_sm100_bwd(*a, kRadius, s) : sparse_attn_sm100_fwd(*a, kRadius, s);
    return backward ? sparse_attn_mma_bwd(*a, kRadius, s) : sparse_attn_mma_fwd(*a, kRadius, s);
  }
  MF_DISPATCH_DTYPE(a->dtype, T, {
    switch (a->head_dim) {
      case 32: return launch_sparse<T, 32, kRadius>(*a, backward, s);
      case 64: return launch_sparse<T, 64, kRadius>(*a, backward, s);
      default: return launch_sparse<T, 128, kRadius>(*a, backward, s);
    }
  });
  return MF_OK;
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" size_t mf_sparse_attn_bwd_workspace_bytes(const MfSparseAttnArgs* a) {
  if (!a) return 0;
  // per query dO . out and (tcgen05 kernels) the log-sum-exp in the log2 domain
  return 2 * align_up((size_t)a->batch * a->heads * a->tokens * sizeof(float), 256);
}
extern "C" int mf_radius_attn_fwd(const MfSparseAttnArgs* a, void* stream) {
  return run_sparse<true>(a, false, stream, "mf_radius_attn_fwd");
}
extern "C" int mf_radius_attn_bwd(const MfSparseAttnArgs* a, void* stream) {
  return run_sparse<true>(a, true, stream, "mf_radius_attn_bwd");
}
extern "C" int mf_local_attn_fwd(const MfSparseAttnArgs* a, void* stream) {
  return run_sparse<false>(a, false, stream, "mf_local_attn_fwd");
}
extern "C" int mf_local_attn_bwd(const MfSparseAttnArgs* a, void* stream) {
  return run_sparse<false>(a, true, stream, "mf_local_attn_bwd");
}
extern "C" int mf_sparse_attn_status(int32_t* host_status, void* stream) {
  MF_CHECK_ARG(host_status != nullptr, "mf_sparse_attn_status: null pointer");
  return sparse_attn_sm100_status(host_status, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------------------------
// Band attention on the packed projection of an attention layer: q, k, v are read inside the (B,N,3,H,D) output of
// the layer's input GEMM and out is written as (B,N,H*D), so the head split before and the merge after the core
// (and their counterparts in the backward pass) do not exist.  bf16, the warp-level tile kernels.
// ---------------------------------------------------------------------------------------------------------------
namespace mf {
namespace {
int run_local_packed(const MfLocalAttnPackedArgs* a, bool backward, void* stream, const char* name) {
  MF_CHECK_ARG(a != nullptr, "%s: null argument struct", name);
  MF_CHECK_ARG(a->batch >= 0 && a->heads >= 0 && a->tokens >= 0, "%s: negative size", name);
  MF_CHECK_ARG(a->head_dim == 32 || a->head_dim == 64 || a->head_dim == 128, "%s: head_dim must be 32, 64 or 128, got %d",
               name, (int)a->head_dim);
  MF_CHECK_ARG(a->window >= 2 && a->window % 2 == 0, "%s: window must be a positive even number, got %d", name,
               (int)a->window);
  if (a->batch == 0 || a->heads == 0 || a->tokens == 0) return MF_OK;
  MF_CHECK_ARG((long long)a->batch * a->heads <= 65535, "%s: batch*heads above 65535", name);
  MF_CHECK_ARG(a->qkv && a->num_atoms && a->out && a->lse, "%s: null tensor pointer", name);
  MF_CHECK_ALIGNED(name, a->qkv, a->out, a->grad_out, a->grad_qkv);
  const long long hd = (long long)a->heads * a->head_dim;
  MfSparseAttnArgs s{};
  s.batch = a->batch, s.heads = a->heads, s.tokens = a->tokens, s.head_dim = a->head_dim;
  s.dtype = MF_DTYPE_BF16, s.window = a->window, s.scale = a->scale, s.backend = MF_SPARSE_BACKEND_MMA;
  const __nv_bfloat16* qkv = static_cast<const __nv_bfloat16*>(a->qkv);
  s.q = qkv, s.k = qkv + hd, s.v = qkv + 2 * hd;
  s.num_atoms = a->num_atoms, s.out = a->out, s.lse = a->lse;
  if (backward) {
    MF_CHECK_ARG(a->grad_out && a->grad_qkv, "%s: null gradient pointer", name);
    __nv_bfloat16* g = static_cast<__nv_bfloat16*>(a->grad_qkv);
    s.grad_out = a->grad_out, s.dq = g, s.dk = g + hd, s.dv = g + 2 * hd;
    const size_t need = mf_sparse_attn_bwd_workspace_bytes(&s);
    if (!a->workspace || a->workspace_bytes < need) {
      set_error("%s: workspace of %zu bytes needed, %zu given", name, need, a->workspace_bytes);
      return MF_ERR_WORKSPACE_TOO_SMALL;
    }
    s.workspace = a->workspace, s.workspace_bytes = a->workspace_bytes;
  }
  const RowLayout in{(long long)a->tokens * 3 * hd, (long long)a->head_dim, 3 * hd};  // a group's rows in (B,N,3,H,D)
  const RowLayout act{(long long)a->tokens * hd, (long long)a->head_dim, hd};          // (B,N,H,D)
  return local_attn_mma_layouts(s, in, act, backward, static_cast<cudaStream_t>(stream));
}
}  // namespace
}  // namespace mf

extern "C" size_t mf_local_attn_packed_bwd_workspace_bytes(const MfLocalAttnPackedArgs* a) {
  if (!a) return 0;
  MfSparseAttnArgs s{};
  s.batch = a->batch, s.heads = a->heads, s.tokens = a->tokens;
  return mf_sparse_attn_bwd_workspace_bytes(&s);
}
extern "C" int mf_local_attn_packed_fwd(const MfLocalAttnPackedArgs* a, void* stream) {
  return run_local_packed(a, false, stream, "mf_local_attn_packed_fwd");
}
extern "C" int mf_local_attn_packed_bwd(const MfLocalAttnPackedArgs* a, void* stream) {
  return run_local_packed(a, true, stream, "mf_local_attn_packed_bwd");
}
