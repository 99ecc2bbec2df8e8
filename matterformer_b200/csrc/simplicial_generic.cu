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
constexpr int kResMax = 32;  // largest rank of the low-rank residuals the kernels take

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
  // low-rank residuals (kRes kernels), fp32.  Angle: logits += agate_i * ra^-1/2 * sum_r al[i,j,r] ar[i,k,r];
  // message: out_i += rm^-1/2 * sum_r (sum_jk attn_ijk ml[i,j,r] mr[i,k,r]) basis[h,r,:].  Ranks at most kResMax.
  const float* al;      // (BH,N,N,ra)
  const float* ar;      // (BH,N,N,ra)
  const float* agate;   // (BH,N)
  const float* ml;      // (BH,N,N,rm)
  const float* mr;      // (BH,N,N,rm)
  const float* basis;   // (H,rm,D)
  int ra, rm;
  float a_scale, m_scale;  // ra^-1/2, rm^-1/2
  float* gb;       // (BH,N,rm) scratch: dO_i . basis_r, written by the DQ pass and read by the DK passes
  float* dal;      // DQ mode outputs, zero-filled by the caller: (BH,N,N,ra)
  float* dar;      // (BH,N,N,ra)
  float* dagate;   // (BH,N)
  float* dml;      // (BH,N,N,rm)
  float* dmr;      // (BH,N,N,rm)
  float* mcoef;    // (BH,N,rm): rm^-1/2 sum_jk attn ml mr, from which the caller forms the gradient of basis
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

template <typename T, int DMAX, int MODE, bool kRes>
__global__ void __launch_bounds__(128) simplicial_generic_kernel(GenericParams p) {
  constexpr int DS = DMAX + 4;
  constexpr int R = DMAX / 32;
  extern __shared__ __align__(16) float smem_f[];
  float* mid_a = smem_f;
  float* mid_b = mid_a + 32 * DS;
  float* inn_a = mid_b + 32 * DS;
  float* inn_b = inn_a + 32 * DS;
  float* tbuf = inn_b + 32 * DS;  // [4][2][DMAX]
  __shared__ float mid_lse[32], mid_delta[32], mid_gate[32], mid_agate[32];
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
  // low-rank residuals
  const bool has_angle = kRes && p.al != nullptr, has_msg = kRes && p.ml != nullptr;
  const int ra = p.ra, rm = p.rm;
  float own_agate = 0.f, dagate_acc = 0.f;
  float c_acc[kRes && MODE == MODE_FWD ? kResMax : 1];   // FWD: un-normalised message coefficients of this lane
  float my_gb = 0.f, my_coef = 0.f;                       // DQ: lane r holds dO_i . basis_r and the coefficient c_ir
  float* gbw = du_acc + 4 * N - warp * N + warp * kResMax;  // per-warp [kResMax] behind the du accumulators
  if constexpr (kRes) {
    if (has_angle && kOwnerIsQuery && owner_ok) own_agate = p.agate[(size_t)bh * N + o];
    if constexpr (MODE == MODE_FWD) {
#pragma unroll
      for (int r = 0; r < kResMax; ++r) c_acc[r] = 0.f;
    }
    if (MODE == MODE_DQ && has_msg) {
      // gb_r = dO_i . basis[h,r,:]; the row of dO sits in own_b (lane holds d = lane + 32 t)
      const int hh = bh % p.H;
      for (int r = 0; r < rm; ++r) {
        float part = 0.f;
#pragma unroll
        for (int t = 0; t < R; ++t) {
          const int d = lane + 32 * t;
          if (d < D) part = fmaf(own_b[t], p.basis[((size_t)hh * rm + r) * D + d], part);
        }
        const float tot = warp_sum(part);
        if (lane == r) my_gb = tot;
      }
      if (lane < rm) {
        gbw[lane] = my_gb;
        if (o < N) p.gb[((size_t)bh * N + o) * rm + lane] = owner_ok ? my_gb : 0.f;
      }
      __syncwarp();
    }
  }

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
      // DQ with residuals: sums over the middle index j of dS al[i,j,r] and P ml[i,j,r] for this lane's key k
      float dar_acc[kRes && MODE == MODE_DQ ? kResMax : 1], dmr_acc[kRes && MODE == MODE_DQ ? kResMax : 1];
      if constexpr (kRes && MODE == MODE_DQ) {
#pragma unroll
        for (int r = 0; r < kResMax; ++r) dar_acc[r] = 0.f, dmr_acc[r] = 0.f;
      }
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
              if (has_angle) mid_agate[threadIdx.x] = p.agate[(size_t)bh * N + m];
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
          // low-rank residuals of element (i, j, k): rows (i,j) of the left factors, (i,k) of the right factors
          float angle_dot = 0.f;
          size_t ij = 0, ik = 0;
          if constexpr (kRes) {
            if (visible) {
              const int qi = kOwnerIsQuery ? o : m;
              const int kj = kOwnerIsQuery ? m : (p.pv_transposed ? k : o);
              const int kk = kOwnerIsQuery ? k : (p.pv_transposed ? o : k);
              ij = ((size_t)bh * N + qi) * N + kj;
              ik = ((size_t)bh * N + qi) * N + kk;
              if (has_angle) {
                const float* a = p.al + ij * ra;
                const float* b2 = p.ar + ik * ra;
                float t = 0.f;
                for (int r = 0; r < ra; ++r) t = fmaf(__ldg(a + r), __ldg(b2 + r), t);
                angle_dot = t * p.a_scale;
                s = fmaf(kOwnerIsQuery ? own_agate : mid_agate[mm], angle_dot, s);
              }
              if (has_msg && kNeedDp) {  // d out / d attn gets the message term: rm^-1/2 sum_r ml mr (dO_i . basis_r)
                const float* a = p.ml + ij * rm;
                const float* b2 = p.mr + ik * rm;
                const float* g = kOwnerIsQuery ? gbw : p.gb + ((size_t)bh * N + qi) * rm;
                float t = 0.f;
                for (int r = 0; r < rm; ++r) t = fmaf(__ldg(a + r) * __ldg(b2 + r), g[r], t);
                dp = fmaf(t, p.m_scale, dp);
              }
            }
          }
          float coef = 0.f, pr = 0.f;
          if (visible) {
            if (MODE == MODE_FWD) {
              if (s > m_run) {
                const float sc = expf(m_run - s);  // 0 when m_run = -inf
                l_run *= sc;
#pragma unroll
                for (int d = 0; d < DMAX; ++d) acc[d] *= sc;
                if constexpr (kRes && MODE == MODE_FWD) {
#pragma unroll
                  for (int r = 0; r < kResMax; ++r) c_acc[r] *= sc;
                }
                m_run = s;
              }
              coef = expf(s - m_run);
              l_run += coef;
            } else {
              const float l = kOwnerIsQuery ? own_lse : mid_lse[mm];
              pr = expf(s - l);
              if (MODE == MODE_DV) {
                coef = pr;
              } else {
                const float dl = kOwnerIsQuery ? own_delta : mid_delta[mm];
                coef = pr * (dp - dl);
              }
            }
          }
          if constexpr (kRes && MODE == MODE_FWD) {
            if (has_msg && coef != 0.f) {
              const float* a = p.ml + ij * rm;
              const float* b2 = p.mr + ik * rm;
#pragma unroll
              for (int r = 0; r < kResMax; ++r)
                if (r < rm) c_acc[r] = fmaf(coef * __ldg(a + r), __ldg(b2 + r), c_acc[r]);
            }
          }
          if constexpr (kRes && MODE == MODE_DQ) {  // coef = dS, pr = P of (i, j = m, k = lane's key)
            if (has_angle) {
              dagate_acc = fmaf(coef, angle_dot, dagate_acc);
              const float* a = p.al + ij * ra;   // ij, ik are 0 for invisible elements, where coef = 0
              const float* b2 = p.ar + ik * ra;
              float mine = 0.f;
#pragma unroll
              for (int r = 0; r < kResMax; ++r) {
                if (r < ra) {  // uniform
                  if (visible) dar_acc[r] = fmaf(coef, __ldg(a + r), dar_acc[r]);
                  const float tot = warp_sum(visible ? coef * __ldg(b2 + r) : 0.f);  // sum over k of dS ar[i,k,r]
                  if (lane == r) mine = tot;
                }
              }
              if (owner_ok && lane < ra && p.dal)
                p.dal[(((size_t)bh * N + o) * N + m) * ra + lane] += own_agate * p.a_scale * mine;
            }
            if (has_msg) {
              const float* a = p.ml + ij * rm;
              const float* b2 = p.mr + ik * rm;
              float mine = 0.f;
#pragma unroll
              for (int r = 0; r < kResMax; ++r) {
                if (r < rm) {
                  if (visible) dmr_acc[r] = fmaf(pr, __ldg(a + r), dmr_acc[r]);
                  const float tot = warp_sum(visible ? pr * __ldg(b2 + r) : 0.f);  // sum over k of P mr[i,k,r]
                  if (lane == r) mine = tot;
                }
              }
              if (owner_ok && lane < rm) {
                const size_t row = (((size_t)bh * N + o) * N + m) * rm + lane;
                if (p.dml) p.dml[row] += p.m_scale * my_gb * mine;
                my_coef = fmaf(p.m_scale * __ldg(p.ml + row), mine, my_coef);
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
      if constexpr (kRes && MODE == MODE_DQ) {
        if (owner_ok && inner_ok) {
          const size_t row = ((size_t)bh * N + o) * N + k;
          if (has_angle && p.dar)
            for (int r = 0; r < ra; ++r) p.dar[row * ra + r] = own_agate * p.a_scale * dar_acc[r];
          if (has_msg && p.dmr)
            for (int r = 0; r < rm; ++r) p.dmr[row * rm + r] = p.m_scale * gbw[r] * dmr_acc[r];
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
  if constexpr (kRes && MODE == MODE_DQ) {
    if (owner_ok) {
      if (has_angle) {
        const float tot = warp_sum(dagate_acc);
        if (lane == 0 && p.dagate) p.dagate[(size_t)bh * N + o] = tot;
      }
      if (has_msg && lane < rm && p.mcoef) p.mcoef[((size_t)bh * N + o) * rm + lane] = my_coef;
    }
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
  if constexpr (kRes && MODE == MODE_FWD) {
    if (has_msg) {  // out_i += rm^-1/2 sum_r c_ir basis[h,r,:], with c_ir normalised like the rest of the row below
      const int hh = bh % p.H;
#pragma unroll
      for (int r = 0; r < kResMax; ++r) {
        if (r < rm) {
          const float cr = warp_sum(c_acc[r] * sc) * p.m_scale;
#pragma unroll
          for (int t = 0; t < R; ++t) {
            const int d = lane + 32 * t;
            if (d < D) res[t] = fmaf(cr, p.basis[((size_t)hh * rm + r) * D + d], res[t]);
          }
        }
      }
    }
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

template <typename T, int DMAX, int MODE, bool kRes>
int launch_mode_r(const GenericParams& p, int BH, cudaStream_t stream) {
  constexpr int DS = DMAX + 4;
  const size_t smem = (size_t)(4 * 32 * DS + 4 * 2 * DMAX + 4 * p.N + 4 * kResMax) * sizeof(float);
  auto kern = simplicial_generic_kernel<T, DMAX, MODE, kRes>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_error(e, "cudaFuncSetAttribute(simplicial_generic)");
  }
  dim3 grid((p.N + 3) / 4, BH);
  kern<<<grid, 128, smem, stream>>>(p);
  MF_CHECK_LAUNCH("simplicial_generic_kernel");
  return MF_OK;
}

template <typename T, int DMAX, int MODE>
int launch_mode(const GenericParams& p, int BH, cudaStream_t stream) {
  if (p.al != nullptr || p.ml != nullptr) return launch_mode_r<T, DMAX, MODE, true>(p, BH, stream);
  return launch_mode_r<T, DMAX, MODE, false>(p, BH, stream);
}

template <typename T, int MODE>
int launch_mode_d(const GenericParams& p, int BH, cudaStream_t stream) {
  if (p.D <= 32) return launch_mode<T, 32, MODE>(p, BH, stream);
  if (p.D <= 64) return launch_mode<T, 64, MODE>(p, BH, stream);
  return launch_mode<T, 128, MODE>(p, BH, stream);
}

}  // namespace

size_t simplicial_generic_bwd_workspace_bytes(const MfSimplicialBwdArgs& a) {
  // delta (BH,N), then dO_i . basis_r (BH,N,message_rank) when the message residual is present
  const size_t rows = (size_t)a.batch * a.heads * a.tokens;
  return align_up(rows * sizeof(float), 256) + align_up(rows * (size_t)(a.message_left ? a.message_rank : 0) * sizeof(float), 256);
}

namespace {
template <typename Args>
void set_residuals(GenericParams& p, const Args& a) {
  p.al = a.angle_left;
  p.ar = a.angle_right;
  p.agate = a.angle_gate;
  p.ml = a.message_left;
  p.mr = a.message_right;
  p.basis = a.message_basis;
  p.ra = a.angle_left ? a.angle_rank : 0;
  p.rm = a.message_left ? a.message_rank : 0;
  p.a_scale = p.ra > 0 ? 1.f / sqrtf((float)p.ra) : 0.f;
  p.m_scale = p.rm > 0 ? 1.f / sqrtf((float)p.rm) : 0.f;
}
}  // namespace

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
  set_residuals(p, a);
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
    set_residuals(p, a);
    p.gb = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + align_up((size_t)rows * sizeof(float), 256));
    p.dal = a.dangle_left;
    p.dar = a.dangle_right;
    p.dagate = a.dangle_gate;
    p.dml = a.dmessage_left;
    p.dmr = a.dmessage_right;
    p.mcoef = a.message_coeff;
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
