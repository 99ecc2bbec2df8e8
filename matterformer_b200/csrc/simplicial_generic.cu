// 2-simplicial attention on CUDA cores in fp32: the path for fp32 inputs
// (1e-4 parity needs fp32 products), for head sizes and token counts the
// tensor-core kernel does not take, and the cross-check for that kernel.
//
// One kernel template covers the forward pass and the three kinds of gradient.
// Every warp owns one row ("owner"), the 32 lanes own 32 consecutive keys of
// the second key set ("inner") and the block walks over the remaining index
// ("middle") in tiles of 32 rows staged in shared memory:
//
//   mode FWD : owner = query i, middle = j, inner = k   -> out[i,:], lse[i]
//   mode DQ  : owner = query i, middle = j, inner = k   -> dq[i,:]
//   mode DK  : owner = key   j, middle = i, inner = k   -> dk1[j,:]
//   mode DV  : owner = key   j, middle = i, inner = k   -> dv1[j,:]
//
// dk2/dv2 come from the DK/DV modes with the two key/value sets exchanged
// (the operator is symmetric under (k1,v1,j) <-> (k2,v2,k)).  All reductions
// run in a fixed order, so results are bit-identical from run to run.
//
// Semantics follow simplicial_attention_torch_from_projected
// (src/matterformer/models/simplicial_attention.py:206-344 of the reference).
#include "common.cuh"
#include "simplicial.cuh"

namespace mf {

namespace {

enum { MODE_FWD = 0, MODE_DQ = 1, MODE_DK = 2, MODE_DV = 3 };

struct GenericParams {
  const void* own_a;
  const void* own_b;
  const void* mid_a;
  const void* mid_b;
  const void* inn_a;
  const void* inn_b;
  const float* lse;    // (BH,N) per query
  const float* delta;  // (BH,N) per query
  const uint8_t* query_valid;
  const uint8_t* key_valid;
  const uint8_t* pair_valid;
  int pv_transposed;  // 1 when the two key sets are exchanged (owner/inner come from sets 2/1)
  // factorized logit bias gate_i * (u_ij + v_ik + w_jk), fp32, (BH,N,N) / (BH,N); null when absent
  const float* bu;
  const float* bv;
  const float* bw;
  const float* bgate;
  float* du;     // DQ mode: (BH,N,N), written for visible (i,j)
  float* dvb;    // DQ mode: (BH,N,N)
  float* dw;     // DK mode, sets not exchanged: (BH,N,N)
  float* dgate;  // DQ mode: (BH,N)
  int H, N, D;
  float* out_f32;
  float* lse_out;
  void* out_t;
};

template <typename T, int DMAX>
__device__ __forceinline__ void load_tile(float* dst, const T* src, int row0, int N, int D) {
  constexpr int DS = DMAX + 4;
  for (int idx = threadIdx.x; idx < 32 * DMAX; idx += blockDim.x) {
    const int r = idx / DMAX, c = idx % DMAX;
    const int row = row0 + r;
    float v = 0.f;
    if (row < N && c < D) v = to_f32<T>(src[(size_t)row * D + c]);
    dst[r * DS + c] = v;
  }
}

template <typename T, int DMAX, int MODE>
__global__ void __launch_bounds__(128) simplicial_generic_kernel(GenericParams p) {
  constexpr int DS = DMAX + 4;
  constexpr int R = DMAX / 32;
  extern __shared__ __align__(16) float smem_f[];
  float* mid_a = smem_f;
  float* mid_b = mid_a + 32 * DS;
  float* inn_a = mid_b + 32 * DS;
  float* inn_b = inn_a + 32 * DS;
  float* tbuf = inn_b + 32 * DS;  // [4][2][DMAX]
  __shared__ float mid_lse[32], mid_delta[32], mid_gate[32];
  __shared__ int mid_ok[32];
  __shared__ int any_flag;

  const int N = p.N, D = p.D;
  const int bh = blockIdx.y;
  const int b = bh / p.H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int o = blockIdx.x * 4 + warp;
  const size_t base = (size_t)bh * N * D;

  const uint8_t* qv = p.query_valid + (size_t)b * N;
  const uint8_t* kv = p.key_valid + (size_t)b * N;
  const uint8_t* pv = p.pair_valid ? p.pair_valid + (size_t)b * N * N : nullptr;
  constexpr bool kOwnerIsQuery = (MODE == MODE_FWD || MODE == MODE_DQ);
  constexpr bool kNeedDp = (MODE == MODE_DQ || MODE == MODE_DK);
  constexpr bool kUseB = (MODE == MODE_FWD || MODE == MODE_DV);  // accumulate with the value tiles

  const bool owner_ok = (o < N) && (kOwnerIsQuery ? qv[o] > 0 : kv[o] > 0);

  // owner rows in registers: lane holds d = lane + 32 r
  float own_a[R], own_b[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = lane + 32 * r;
    own_a[r] = 0.f;
    own_b[r] = 0.f;
    if (owner_ok && d < D) {
      own_a[r] = to_f32<T>(static_cast<const T*>(p.own_a)[base + (size_t)o * D + d]);
      if (kNeedDp) own_b[r] = to_f32<T>(static_cast<const T*>(p.own_b)[base + (size_t)o * D + d]);
    }
  }
  float own_lse = 0.f, own_delta = 0.f;
  if (MODE == MODE_DQ && owner_ok) {
    own_lse = p.lse[(size_t)bh * N + o];
    own_delta = p.delta[(size_t)bh * N + o];
  }

  float acc[DMAX];
#pragma unroll
  for (int d = 0; d < DMAX; ++d) acc[d] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  float* tw = tbuf + warp * 2 * DMAX;
  float* t2w = tw + DMAX;
  // factorized bias: which tensor supplies the per-middle scalar, the per-(middle, lane) term and the
  // per-lane term depends on the roles (see the table at bias_terms below)
  const bool has_bias = p.bu != nullptr;
  const size_t bhNN = (size_t)bh * N * N;
  float* du_acc = tbuf + 4 * 2 * DMAX + warp * N;  // DQ mode: sum over k of dS for every j of this warp's query
  const bool want_du = MODE == MODE_DQ && has_bias && p.du != nullptr;
  if (want_du)
    for (int t = lane; t < N; t += 32) du_acc[t] = 0.f;
  float own_gate = 0.f, dgate_acc = 0.f;
  if (has_bias && kOwnerIsQuery && owner_ok) own_gate = p.bgate[(size_t)bh * N + o];

  // does this block have anything to do?
  if (threadIdx.x == 0) any_flag = 0;
  __syncthreads();
  if (owner_ok && lane == 0) any_flag = 1;
  __syncthreads();
  const bool block_active = any_flag != 0;

  if (block_active) {
    for (int kc = 0; kc < N; kc += 32) {
      const int k = kc + lane;
      const bool inner_ok = (k < N) && kv[k] > 0;
      if (__syncthreads_or(inner_ok) == 0) continue;
      load_tile<T, DMAX>(inn_a, static_cast<const T*>(p.inn_a) + base, kc, N, D);
      load_tile<T, DMAX>(inn_b, static_cast<const T*>(p.inn_b) + base, kc, N, D);
      // bias_terms: logits get gate_i * (t_m + t_ml + t_l) with
      //   owner = query i           : t_m = u[i,j]  t_ml = w[j,k]  t_l = v[i,k]
      //   owner = key j (set 1)     : t_m = u[i,j]  t_ml = v[i,k]  t_l = w[j,k]
      //   owner = key k (exchanged) : t_m = v[i,k]  t_ml = u[i,j]  t_l = w[j,k]   (inner lane = j)
      float t_l = 0.f, lane_acc = 0.f;  // lane_acc: sum over the middle index of (gate *) dS for this lane's key
      if (has_bias && owner_ok && inner_ok) {
        if (kOwnerIsQuery) t_l = p.bv[bhNN + (size_t)o * N + k];
        else t_l = p.pv_transposed ? p.bw[bhNN + (size_t)k * N + o] : p.bw[bhNN + (size_t)o * N + k];
      }
      for (int mc = 0; mc < N; mc += 32) {
        __syncthreads();  // previous middle tile fully consumed
        if (threadIdx.x < 32) {
          const int m = mc + threadIdx.x;
          int ok = 0;
          float l = 0.f, dl = 0.f;
          if (m < N) {
            ok = kOwnerIsQuery ? (kv[m] > 0) : (qv[m] > 0);
            if (!kOwnerIsQuery && ok) {
              l = p.lse[(size_t)bh * N + m];
              if (MODE == MODE_DK) dl = p.delta[(size_t)bh * N + m];
              if (has_bias) mid_gate[threadIdx.x] = p.bgate[(size_t)bh * N + m];
            }
          }
          mid_ok[threadIdx.x] = ok;
          mid_lse[threadIdx.x] = l;
          mid_delta[threadIdx.x] = dl;
        }
        const bool chunk_any = __syncthreads_or(threadIdx.x < 32 ? mid_ok[threadIdx.x] : 0) != 0;
        if (!chunk_any) continue;
        load_tile<T, DMAX>(mid_a, static_cast<const T*>(p.mid_a) + base, mc, N, D);
        load_tile<T, DMAX>(mid_b, static_cast<const T*>(p.mid_b) + base, mc, N, D);
        __syncthreads();
        if (!owner_ok) continue;

        for (int mm = 0; mm < 32; ++mm) {
          if (!mid_ok[mm]) continue;
          const int m = mc + mm;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const int d = lane + 32 * r;
            tw[d] = own_a[r] * mid_a[mm * DS + d];
            if (kNeedDp) t2w[d] = own_b[r] * mid_b[mm * DS + d];
          }
          __syncwarp();
          // visibility of the key pair (j,k)
          bool visible = inner_ok;
          if (visible && pv) {
            const int j = kOwnerIsQuery ? m : o;
            visible = p.pv_transposed ? (pv[(size_t)k * N + j] > 0) : (pv[(size_t)j * N + k] > 0);
          }
          float s = 0.f, dp = 0.f;
          {
            const float4* t4 = reinterpret_cast<const float4*>(tw);
            const float4* a4 = reinterpret_cast<const float4*>(inn_a + lane * DS);
#pragma unroll
            for (int d4 = 0; d4 < DMAX / 4; ++d4) {
              const float4 x = t4[d4], y = a4[d4];
              s = fmaf(x.x, y.x, s);
              s = fmaf(x.y, y.y, s);
              s = fmaf(x.z, y.z, s);
              s = fmaf(x.w, y.w, s);
            }
            if (kNeedDp) {
              const float4* u4 = reinterpret_cast<const float4*>(t2w);
              const float4* b4 = reinterpret_cast<const float4*>(inn_b + lane * DS);
#pragma unroll
              for (int d4 = 0; d4 < DMAX / 4; ++d4) {
                const float4 x = u4[d4], y = b4[d4];
                dp = fmaf(x.x, y.x, dp);
                dp = fmaf(x.y, y.y, dp);
                dp = fmaf(x.z, y.z, dp);
                dp = fmaf(x.w, y.w, dp);
              }
            }
          }
          float bias_sum = 0.f;
          if (has_bias && visible) {
            float t_m, t_ml;
            if (kOwnerIsQuery) {
              t_m = p.bu[bhNN + (size_t)o * N + m];
              t_ml = p.bw[bhNN + (size_t)m * N + k];
            } else if (!p.pv_transposed) {
              t_m = p.bu[bhNN + (size_t)m * N + o];
              t_ml = p.bv[bhNN + (size_t)m * N + k];
            } else {
              t_m = p.bv[bhNN + (size_t)m * N + o];
              t_ml = p.bu[bhNN + (size_t)m * N + k];
            }
            bias_sum = (t_m + t_ml) + t_l;
            s = fmaf(kOwnerIsQuery ? own_gate : mid_gate[mm], bias_sum, s);
          }
          float coef = 0.f;
          if (visible) {
            if (MODE == MODE_FWD) {
              if (s > m_run) {
                const float sc = expf(m_run - s);  // 0 when m_run = -inf
                l_run *= sc;
#pragma unroll
                for (int d = 0; d < DMAX; ++d) acc[d] *= sc;
                m_run = s;
              }
              coef = expf(s - m_run);
              l_run += coef;
            } else {
              const float l = kOwnerIsQuery ? own_lse : mid_lse[mm];
              const float pr = expf(s - l);
              if (MODE == MODE_DV) {
                coef = pr;
              } else {
                const float dl = kOwnerIsQuery ? own_delta : mid_delta[mm];
                coef = pr * (dp - dl);
              }
            }
          }
          if (has_bias && MODE == MODE_DQ) {  // coef = dS of (i, j = m, k = lane's key)
            lane_acc += coef;
            dgate_acc = fmaf(coef, bias_sum, dgate_acc);
            if (want_du) {
              const float row_sum = warp_sum(coef);
              if (lane == 0) du_acc[m] += row_sum;
            }
          }
          if (has_bias && MODE == MODE_DK && !p.pv_transposed) lane_acc = fmaf(mid_gate[mm], coef, lane_acc);
          if (coef != 0.f) {
            const float4* m4 = reinterpret_cast<const float4*>((kUseB ? mid_b : mid_a) + mm * DS);
            const float4* i4 = reinterpret_cast<const float4*>((kUseB ? inn_b : inn_a) + lane * DS);
#pragma unroll
            for (int d4 = 0; d4 < DMAX / 4; ++d4) {
              const float4 x = m4[d4], y = i4[d4];
              acc[4 * d4 + 0] = fmaf(coef * x.x, y.x, acc[4 * d4 + 0]);
              acc[4 * d4 + 1] = fmaf(coef * x.y, y.y, acc[4 * d4 + 1]);
              acc[4 * d4 + 2] = fmaf(coef * x.z, y.z, acc[4 * d4 + 2]);
              acc[4 * d4 + 3] = fmaf(coef * x.w, y.w, acc[4 * d4 + 3]);
            }
          }
          __syncwarp();
        }
      }
      if (has_bias && owner_ok && inner_ok) {
        if (MODE == MODE_DQ && p.dvb) p.dvb[bhNN + (size_t)o * N + k] = own_gate * lane_acc;       // dv[i,k]
        if (MODE == MODE_DK && !p.pv_transposed && p.dw) p.dw[bhNN + (size_t)o * N + k] = lane_acc;  // dw[j,k]
      }
      __syncthreads();  // inner tiles are reloaded next
    }
  }

  if (MODE == MODE_DQ && has_bias && owner_ok) {
    __syncwarp();
    if (want_du)
      for (int t = lane; t < N; t += 32) p.du[bhNN + (size_t)o * N + t] = own_gate * du_acc[t];
    const float tot = warp_sum(dgate_acc);
    if (lane == 0 && p.dgate) p.dgate[(size_t)bh * N + o] = tot;
  }
  if (o >= N) return;
  // ---- combine the 32 lanes (fixed butterfly order) and write the owner's row
  float sc = 1.f, l_tot = 1.f, m_tot = 0.f;
  if (MODE == MODE_FWD) {
    m_tot = warp_max(m_run);
    sc = (m_run == -INFINITY) ? 0.f : expf(m_run - m_tot);
    l_tot = warp_sum(l_run * sc);
  }
  float res[R];
#pragma unroll
  for (int r = 0; r < R; ++r) res[r] = 0.f;
#pragma unroll
  for (int d = 0; d < DMAX; ++d) {
    const float v = warp_sum(acc[d] * sc);
    if ((d & 31) == lane) res[d >> 5] = v;
  }
  const bool have = owner_ok && (MODE != MODE_FWD || l_tot > 0.f);
  const float inv = (MODE == MODE_FWD && have) ? 1.f / l_tot : 1.f;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = lane + 32 * r;
    if (d < D) {
      const float v = have ? res[r] * inv : 0.f;
      const size_t off = base + (size_t)o * D + d;
      if (MODE == MODE_FWD) {
        p.out_f32[off] = v;
        if (p.out_t) static_cast<T*>(p.out_t)[off] = from_f32<T>(v);
      } else {
        static_cast<T*>(p.out_t)[off] = from_f32<T>(v);
      }
    }
  }
  if (MODE == MODE_FWD && lane == 0) p.lse_out[(size_t)bh * N + o] = have ? m_tot + logf(l_tot) : 0.f;
}

template <typename T>
__global__ void delta_kernel(const T* __restrict__ grad_out, const float* __restrict__ out, float* __restrict__ delta,
                             int rows, int D) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float s = 0.f;
  for (int d = lane; d < D; d += 32) s = fmaf(to_f32<T>(grad_out[(size_t)row * D + d]), out[(size_t)row * D + d], s);
  s = warp_sum(s);
  if (lane == 0) delta[row] = s;
}

template <typename T, int DMAX, int MODE>
int launch_mode(const GenericParams& p, int BH, cudaStream_t stream) {
  constexpr int DS = DMAX + 4;
  const size_t smem = (size_t)(4 * 32 * DS + 4 * 2 * DMAX + 4 * p.N) * sizeof(float);
  auto kern = simplicial_generic_kernel<T, DMAX, MODE>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_error(e, "cudaFuncSetAttribute(simplicial_generic)");
  }
  dim3 grid((p.N + 3) / 4, BH);
  kern<<<grid, 128, smem, stream>>>(p);
  MF_CHECK_LAUNCH("simplicial_generic_kernel");
  return MF_OK;
}

template <typename T, int MODE>
int launch_mode_d(const GenericParams& p, int BH, cudaStream_t stream) {
  if (p.D <= 32) return launch_mode<T, 32, MODE>(p, BH, stream);
  if (p.D <= 64) return launch_mode<T, 64, MODE>(p, BH, stream);
  return launch_mode<T, 128, MODE>(p, BH, stream);
}

}  // namespace

size_t simplicial_generic_bwd_workspace_bytes(const MfSimplicialBwdArgs& a) {
  return align_up((size_t)a.batch * a.heads * a.tokens * sizeof(float), 256);
}

int simplicial_generic_fwd(const MfSimplicialFwdArgs& a, cudaStream_t stream) {
  GenericParams p{};
  p.own_a = a.q;
  p.mid_a = a.k1;
  p.mid_b = a.v1;
  p.inn_a = a.k2;
  p.inn_b = a.v2;
  p.query_valid = a.query_valid;
  p.key_valid = a.pair_key_valid;
  p.pair_valid = a.pair_valid;
  p.pv_transposed = 0;
  p.bu = a.u;
  p.bv = a.v_bias;
  p.bw = a.w;
  p.bgate = a.gate;
  p.H = a.heads;
  p.N = a.tokens;
  p.D = a.head_dim;
  p.out_f32 = a.out;
  p.lse_out = a.lse;
  p.out_t = a.out_cast;
  const int BH = a.batch * a.heads;
  MF_DISPATCH_DTYPE(a.dtype, T, return (launch_mode_d<T, MODE_FWD>(p, BH, stream)));
  return MF_OK;
}

int simplicial_generic_bwd(const MfSimplicialBwdArgs& a, cudaStream_t stream) {
  const int BH = a.batch * a.heads;
  const int rows = BH * a.tokens;
  float* delta = static_cast<float*>(a.workspace);
  MF_DISPATCH_DTYPE(a.dtype, T, {
    delta_kernel<T><<<(rows + 3) / 4, 128, 0, stream>>>(static_cast<const T*>(a.grad_out), a.out, delta, rows,
                                                          a.head_dim);
    MF_CHECK_LAUNCH("delta_kernel");
    GenericParams p{};
    p.lse = a.lse;
    p.delta = delta;
    p.query_valid = a.query_valid;
    p.key_valid = a.pair_key_valid;
    p.pair_valid = a.pair_valid;
    p.H = a.heads;
    p.N = a.tokens;
    p.D = a.head_dim;
    p.bu = a.u;
    p.bv = a.v_bias;
    p.bw = a.w;
    p.bgate = a.gate;
    p.du = a.du;
    p.dvb = a.dv_bias;
    p.dw = a.dw;
    p.dgate = a.dgate;
    int rc;
    // dq: owner = query (also du, dv_bias, dgate); dk1: owner = first key set (also dw)
    p.own_a = a.q;
    p.own_b = a.grad_out;
    p.mid_a = a.k1;
    p.mid_b = a.v1;
    p.inn_a = a.k2;
    p.inn_b = a.v2;
    p.pv_transposed = 0;
    p.out_t = a.dq;
    if ((rc = launch_mode_d<T, MODE_DQ>(p, BH, stream)) != MF_OK) return rc;
    // dk1 / dv1: owner = first key set
    p.own_a = a.k1;
    p.own_b = a.v1;
    p.mid_a = a.q;
    p.mid_b = a.grad_out;
    p.out_t = a.dk1;
    if ((rc = launch_mode_d<T, MODE_DK>(p, BH, stream)) != MF_OK) return rc;
    p.out_t = a.dv1;
    if ((rc = launch_mode_d<T, MODE_DV>(p, BH, stream)) != MF_OK) return rc;
    // dk2 / dv2: the two key sets exchanged
    p.own_a = a.k2;
    p.own_b = a.v2;
    p.inn_a = a.k1;
    p.inn_b = a.v1;
    p.pv_transposed = 1;
    p.out_t = a.dk2;
    if ((rc = launch_mode_d<T, MODE_DK>(p, BH, stream)) != MF_OK) return rc;
    p.out_t = a.dv2;
    if ((rc = launch_mode_d<T, MODE_DV>(p, BH, stream)) != MF_OK) return rc;
  });
  return MF_OK;
}

}  // namespace mf
