// Radius block-sparse and local-window attention on the warp-level tensor cores (mma.sync m16n8k16, bf16).
//
// Same operators and semantics as sparse_attn.cu (masked softmax attention as computed by
// F.scaled_dot_product_attention for the reference's RotaryMultiheadAttention,
// src/matterformer/models/regular_attention.py:251-268); this file is the bf16 path.  These operators move
// little data per FLOP only on paper: with 32-row tiles the work per byte is small enough that the legacy
// warp-level MMA is the right tool, the tile operands come through shared memory with cp.async double
// buffering, and nothing is reshaped into large GEMMs.
//
// One CTA of two warps owns a tile of 32 "owner" rows of one (batch, head) and walks over its partner blocks
// of 32 rows; each warp handles 16 owner rows.
//   FWD : owners = queries, partners = key blocks   -> out, lse           (online softmax)
//   DQ  : owners = queries, partners = key blocks   -> dq
//   DKV : owners = keys,    partners = query blocks -> dk, dv             (scores computed transposed)
// Partner blocks and the per-row visibility words come from the radius block list / bitmaps, or from the
// band i - w/2 <= j <= i + w/2 - 1.  Every output row has one owner: no atomics, bit-identical reruns.
#include "common.cuh"
#include "simplicial_sm100.cuh"
#include "sparse_attn_mma.cuh"

namespace mf {
namespace {

enum { M_FWD = 0, M_DQ = 1, M_DKV = 2 };
// partner blocks in the shared-memory ring: the band walk is short (three blocks at window 64), so it keeps two
// blocks in flight; the radius walk is long and gains more from the occupancy of a two-stage ring
template <bool kRadius>
constexpr int kSparseStages = kRadius ? 2 : 3;
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLn2F = 0.6931471805599453f;

struct MmaParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* grad_out;
  const float* lse;
  float* delta;  // written by the DQ pass, read by the DKV pass
  const int32_t* num_atoms;
  const int32_t* block_count;
  const int32_t* block_cols;
  const uint32_t* block_mask;
  __nv_bfloat16* out;
  float* lse_out;
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int H, N, window, tiles;
  float scale;
  RowLayout in;   // rows of q, k, v and of dq, dk, dv: (B,H,N,D) contiguous, or slices of a packed (B,N,3,H,D) projection
  RowLayout act;  // rows of out and grad_out: (B,H,N,D) contiguous, or (B,N,H*D)
};

__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// bits c of a 32-row block starting at row kb with lo <= kb + c <= hi
__device__ __forceinline__ uint32_t range_word(int kb, int lo, int hi) {
  const int a = max(lo - kb, 0), b = min(hi - kb, 31);
  if (a > b) return 0u;
  const int len = b - a + 1;
  return (len >= 32 ? 0xffffffffu : ((1u << len) - 1u)) << a;
}

// 32 x D tile, row-major bf16 in global -> padded rows in shared memory; rows >= row_limit become zeros
template <int D>
__device__ __forceinline__ void load_tile_async(uint32_t smem_tile, const __nv_bfloat16* src, long long row_stride,
                                                int row0, int row_limit) {
  constexpr int LD = D + 8;
  constexpr int CHUNKS = 32 * (D / 8);
  for (int idx = threadIdx.x; idx < CHUNKS; idx += 64) {
    const int r = idx / (D / 8), c = idx % (D / 8);
    const int row = row0 + r;
    const bool ok = row >= 0 && row < row_limit;
    cp_async16(smem_tile + (r * LD + c * 8) * 2, src + (ok ? row : 0) * row_stride + c * 8, ok);
  }
}

// A fragments (16 rows x D) of a tile for all k-steps: frag[ks][4]
template <int D>
__device__ __forceinline__ void load_a_frags(uint32_t (&frag)[D / 16][4], uint32_t smem_tile, int row0, int lane) {
  constexpr int LD = D + 8;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
    ldmatrix_x4(frag[ks], smem_tile + ((row0 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8) * 2);
}

// c[nt] (16 x 8 each, nt = 0..3: 32 partner rows) = A (16 x D) . B^T where B is a 32 x D tile (rows = partners)
template <int D>
__device__ __forceinline__ void gemm_rows(float (&c)[4][4], const uint32_t (&a)[D / 16][4], uint32_t smem_b, int lane) {
  constexpr int LD = D + 8;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) c[nt][e] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int np = 0; np < 2; ++np) {  // two n-tiles (16 partner rows) per ldmatrix.x4
      uint32_t b[4];
      ldmatrix_x4(b, smem_b + ((np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8) * 2);
      mma_bf16(c[2 * np], a[ks], b[0], b[1]);
      mma_bf16(c[2 * np + 1], a[ks], b[2], b[3]);
    }
  }
}

// acc (16 x D) += P (16 x 32, given as C fragments p[nt]) . B where B is a 32 x D tile (rows = the 32 partners)
template <int D>
__device__ __forceinline__ void gemm_acc(float (&acc)[D / 8][4], const float (&p)[4][4], uint32_t smem_b, int lane) {
  constexpr int LD = D + 8;
#pragma unroll
  for (int kk = 0; kk < 2; ++kk) {  // 16 partner rows per k-step
    uint32_t a[4];
    a[0] = pack2_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack2_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack2_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack2_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {  // two n-tiles (16 columns of D) per ldmatrix.x4.trans
      uint32_t b[4];
      ldmatrix_x4_trans(b, smem_b + ((kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + np * 16 + (lane >> 4) * 8) * 2);
      mma_bf16(acc[2 * np], a, b[0], b[1]);
      mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// 16 x D accumulator -> bf16 rows in global memory (rows >= row_limit are skipped)
template <int D>
__device__ __forceinline__ void store_acc(__nv_bfloat16* dst, long long row_stride, const float (&acc)[D / 8][4],
                                          int row_g, int row_limit, int lane, float mul_lo, float mul_hi) {
  const int t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const int col = nt * 8 + 2 * t;
    if (row_g < row_limit)
      *reinterpret_cast<uint32_t*>(dst + row_g * row_stride + col) = pack2_bf16(acc[nt][0] * mul_lo, acc[nt][1] * mul_lo);
    if (row_g + 8 < row_limit)
      *reinterpret_cast<uint32_t*>(dst + (row_g + 8) * row_stride + col) =
          pack2_bf16(acc[nt][2] * mul_hi, acc[nt][3] * mul_hi);
  }
}

// Partner blocks of an owner tile and the visibility word of an owner row against a partner block.
template <bool kRadius, int MODE>
struct BlockWalk {
  int count, first_block, n, half;
  const int32_t* cols;
  const uint32_t* masks;

  __device__ __forceinline__ BlockWalk(const MmaParams& p, int b, int tile, int n_) : n(n_) {
    half = p.window / 2;
    if (kRadius) {
      count = (tile * 32 < n) ? p.block_count[(size_t)b * p.tiles + tile] : 0;
      cols = p.block_cols + ((size_t)b * p.tiles + tile) * p.tiles;
      masks = p.block_mask + ((size_t)b * p.tiles + tile) * p.tiles * 32;
      first_block = 0;
    } else {
      // query i sees keys [i-half, i+half-1]; key j is seen by queries [j-half+1, j+half]
      const int lo = max(0, tile * 32 - half + (MODE == M_DKV ? 1 : 0));
      const int hi = min(n - 1, tile * 32 + 31 + half - (MODE == M_DKV ? 0 : 1));
      first_block = lo >> 5;
      count = (tile * 32 < n && hi >= lo) ? (hi >> 5) - first_block + 1 : 0;
      cols = nullptr;
      masks = nullptr;
    }
  }
  __device__ __forceinline__ int block_row0(int t) const { return 32 * (kRadius ? cols[t] : first_block + t); }
  // owner row `orow` (index inside the structure) against the partner block starting at row kb
  __device__ __forceinline__ uint32_t word(int t, int kb, int orow) const {
    if (orow >= n) return 0u;
    if (kRadius) return masks[(size_t)cols[t] * 32 + (orow & 31)];  // symmetric bitmap: serves both directions
    const int lo = orow - half + (MODE == M_DKV ? 1 : 0), hi = orow + half - (MODE == M_DKV ? 0 : 1);
    return range_word(kb, max(lo, 0), min(hi, n - 1));
  }
};

template <int D, bool kRadius, int MODE>
__global__ void __launch_bounds__(64) sparse_attn_mma_kernel(MmaParams p) {
  constexpr int LD = D + 8;
  constexpr int TILE_BYTES = 32 * LD * 2;
  constexpr int S = kSparseStages<kRadius>;  // partner blocks in the ring: S - 1 of them are in flight while one is used
  extern __shared__ __align__(16) uint8_t smem_dyn[];
  // own_a | own_b | part_a[S] | part_b[S] | part_lse[S][32] | part_delta[S][32]
  const uint32_t s_own_a = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dyn));
  const uint32_t s_own_b = s_own_a + TILE_BYTES;
  const uint32_t s_part_a = s_own_b + TILE_BYTES;
  const uint32_t s_part_b = s_part_a + S * TILE_BYTES;
  float* part_lse = reinterpret_cast<float*>(smem_dyn + (2 + 2 * S) * TILE_BYTES);
  float* part_delta = part_lse + S * 32;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int tile = blockIdx.x, bh = blockIdx.y, b = bh / p.H;
  const int N = p.N;
  const int n = min(p.num_atoms[b], N);
  const long long in_base = p.in.at(b, bh - b * p.H, 0), act_base = p.act.at(b, bh - b * p.H, 0);
  const long long rs_in = p.in.token, rs_act = p.act.token;  // elements between neighbouring tokens of a head
  const __nv_bfloat16* Q = p.q + in_base;
  const __nv_bfloat16* K = p.k + in_base;
  const __nv_bfloat16* V = p.v + in_base;
  const __nv_bfloat16* dO = (MODE == M_FWD) ? nullptr : p.grad_out + act_base;
  // owners: queries (FWD, DQ) or keys (DKV); "a" tiles feed the logits, "b" tiles feed dP
  const __nv_bfloat16* OWN_A = (MODE == M_DKV) ? K : Q;
  const __nv_bfloat16* OWN_B = (MODE == M_DKV) ? V : dO;
  const __nv_bfloat16* PART_A = (MODE == M_DKV) ? Q : K;
  const __nv_bfloat16* PART_B = (MODE == M_DKV) ? dO : V;
  const long long own_b_rs = (MODE == M_DKV) ? rs_in : rs_act, part_b_rs = (MODE == M_DKV) ? rs_act : rs_in;

  const BlockWalk<kRadius, MODE> walk(p, b, tile, n);
  const int row0 = tile * 32;
  const int my_row = row0 + warp * 16 + g;  // this thread's rows: my_row and my_row + 8

  // ---- owner tiles and the first partner block
  load_tile_async<D>(s_own_a, OWN_A, rs_in, row0, n);
  if (MODE != M_FWD) load_tile_async<D>(s_own_b, OWN_B, own_b_rs, row0, n);
  auto load_partner = [&](int t, int stage) {
    const int kb = walk.block_row0(t);
    load_tile_async<D>(s_part_a + stage * TILE_BYTES, PART_A, rs_in, kb, n);
    load_tile_async<D>(s_part_b + stage * TILE_BYTES, PART_B, part_b_rs, kb, n);
    if (MODE == M_DKV && threadIdx.x < 32) {
      const int row = kb + threadIdx.x;
      part_lse[stage * 32 + threadIdx.x] = row < n ? p.lse[(size_t)bh * N + row] * kLog2eF : INFINITY;
      part_delta[stage * 32 + threadIdx.x] = row < n ? p.delta[(size_t)bh * N + row] : 0.f;
    }
  };
  // one commit group per partner block (the owner tiles ride in the first); groups are committed even when
  // empty so that "all but the newest S - 2 groups" always means "everything up to the block used next"
  if (walk.count > 0) load_partner(0, 0);
  cp_async_commit();
#pragma unroll
  for (int t = 1; t < S - 1; ++t) {
    if (t < walk.count) load_partner(t, t);
    cp_async_commit();
  }
  cp_async_wait<S - 2>();
  __syncthreads();

  uint32_t a_frag[D / 16][4], b_frag[D / 16][4];
  load_a_frags<D>(a_frag, s_own_a, warp * 16, lane);
  if (MODE != M_FWD) load_a_frags<D>(b_frag, s_own_b, warp * 16, lane);

  float acc0[D / 8][4], acc1[(MODE == M_DKV) ? D / 8 : 1][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc0[i][e] = 0.f;
  if constexpr (MODE == M_DKV) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc1[i][e] = 0.f;
  }
  const float sc2 = p.scale * kLog2eF;  // logits in the log2 domain
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float lse_lo = INFINITY, lse_hi = INFINITY, dl_lo = 0.f, dl_hi = 0.f;
  if (MODE == M_DQ) {
    // delta = dO . out per row, formed here by the four lanes that share a row (each D/4 columns) and left in
    // global memory for the key-centric pass that follows on the same stream
    auto row_delta = [&](int row) {
      float d = 0.f;
      if (row < n) {
        const uint4* go = reinterpret_cast<const uint4*>(dO + row * rs_act + t4 * (D / 4));
        const uint4* oo = reinterpret_cast<const uint4*>(p.out + act_base + row * rs_act + t4 * (D / 4));
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          const uint4 a = __ldg(go + c), o = __ldg(oo + c);
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            d = fmaf(__uint_as_float(aw[e] << 16), __uint_as_float(ow[e] << 16), d);
            d = fmaf(__uint_as_float(aw[e] & 0xffff0000u), __uint_as_float(ow[e] & 0xffff0000u), d);
          }
        }
      }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      if (t4 == 0 && row < N) p.delta[(size_t)bh * N + row] = d;
      return d;
    };
    dl_lo = row_delta(my_row);
    dl_hi = row_delta(my_row + 8);
    if (my_row < n) lse_lo = p.lse[(size_t)bh * N + my_row] * kLog2eF;
    if (my_row + 8 < n) lse_hi = p.lse[(size_t)bh * N + my_row + 8] * kLog2eF;
  }

  for (int t = 0; t < walk.count; ++t) {
    const int stage = t % S;
    if (t + S - 1 < walk.count) load_partner(t + S - 1, (t + S - 1) % S);  // refills the block used last iteration
    cp_async_commit();
    const int kb = walk.block_row0(t);
    const uint32_t w_lo = walk.word(t, kb, my_row), w_hi = walk.word(t, kb, my_row + 8);
    const uint32_t any = __ballot_sync(0xffffffffu, (w_lo | w_hi) != 0u);
    if (any != 0u) {  // warp-uniform: some row of this warp sees some partner of the block
      float s[4][4];
      gemm_rows<D>(s, a_frag, s_part_a + stage * TILE_BYTES, lane);
      if (MODE == M_FWD) {
        // ---- online softmax over the visible partners
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = nt * 8 + 2 * t4 + (e & 1);
            const bool vis = ((e < 2 ? w_lo : w_hi) >> col) & 1u;
            s[nt][e] = vis ? s[nt][e] * sc2 : -INFINITY;
            if (e < 2) mx_lo = fmaxf(mx_lo, s[nt][e]); else mx_hi = fmaxf(mx_hi, s[nt][e]);
          }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float mu_lo = mn_lo == -INFINITY ? 0.f : mn_lo, mu_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float al_lo = m_lo == -INFINITY ? 0.f : exp2_fast(m_lo - mu_lo);
        const float al_hi = m_hi == -INFINITY ? 0.f : exp2_fast(m_hi - mu_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float pr = exp2_fast(s[nt][e] - (e < 2 ? mu_lo : mu_hi));  // exp2(-inf) = 0 for masked pairs
            s[nt][e] = pr;
            if (e < 2) sum_lo += pr; else sum_hi += pr;
          }
        l_lo = l_lo * al_lo + sum_lo;  // per-thread partial sums; the quad is combined at the end
        l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          acc0[i][0] *= al_lo;
          acc0[i][1] *= al_lo;
          acc0[i][2] *= al_hi;
          acc0[i][3] *= al_hi;
        }
        gemm_acc<D>(acc0, s, s_part_b + stage * TILE_BYTES, lane);
      } else {
        float dp[4][4];
        gemm_rows<D>(dp, b_frag, s_part_b + stage * TILE_BYTES, lane);
        float ds[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = nt * 8 + 2 * t4 + (e & 1);
            const bool vis = ((e < 2 ? w_lo : w_hi) >> col) & 1u;
            float l, dl;
            if (MODE == M_DQ) {
              l = e < 2 ? lse_lo : lse_hi;
              dl = e < 2 ? dl_lo : dl_hi;
            } else {  // per partner column (a query)
              l = part_lse[stage * 32 + col];
              dl = part_delta[stage * 32 + col];
            }
            const float pr = vis ? exp2_fast(fmaf(s[nt][e], sc2, -l)) : 0.f;
            s[nt][e] = pr;
            ds[nt][e] = pr * (dp[nt][e] - dl) * p.scale;
          }
        gemm_acc<D>(acc0, ds, s_part_a + stage * TILE_BYTES, lane);                       // dq += dS.K | dk += dS^T.Q
        if constexpr (MODE == M_DKV) gemm_acc<D>(acc1, s, s_part_b + stage * TILE_BYTES, lane);  // dv += P^T.dO
      }
    }
    cp_async_wait<S - 2>();
    __syncthreads();  // next block landed; this block's buffers may be refilled by the next iteration's loads
  }

  // ---- write the owner rows
  if (MODE == M_FWD) {
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
    store_acc<D>(p.out + act_base, rs_act, acc0, my_row, N, lane, inv_lo, inv_hi);
    if (t4 == 0) {
      if (my_row < N) p.lse_out[(size_t)bh * N + my_row] = l_lo > 0.f ? (m_lo + log2f(l_lo)) * kLn2F : 0.f;
      if (my_row + 8 < N) p.lse_out[(size_t)bh * N + my_row + 8] = l_hi > 0.f ? (m_hi + log2f(l_hi)) * kLn2F : 0.f;
    }
  } else if (MODE == M_DQ) {
    store_acc<D>(p.dq + in_base, rs_in, acc0, my_row, N, lane, 1.f, 1.f);
  } else if constexpr (MODE == M_DKV) {
    store_acc<D>(p.dk + in_base, rs_in, acc0, my_row, N, lane, 1.f, 1.f);
    store_acc<D>(p.dv + in_base, rs_in, acc1, my_row, N, lane, 1.f, 1.f);
  }
}

template <int D, bool kRadius, int MODE>
int launch_one(const MmaParams& p, int BH, cudaStream_t s) {
  constexpr int smem = (2 + 2 * kSparseStages<kRadius>) * 32 * (D + 8) * 2 + kSparseStages<kRadius> * 256;
  auto kern = sparse_attn_mma_kernel<D, kRadius, MODE>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_error(e, "cudaFuncSetAttribute(sparse_attn_mma_kernel)");
  }
  kern<<<dim3(p.tiles, BH), 64, smem, s>>>(p);
  MF_CHECK_LAUNCH("sparse_attn_mma_kernel");
  return MF_OK;
}

template <int D, bool kRadius>
int launch_all(const MfSparseAttnArgs& a, const RowLayout* layouts, bool backward, cudaStream_t s) {
  MmaParams p{};
  p.in = p.act = RowLayout{(long long)a.heads * a.tokens * D, (long long)a.tokens * D, (long long)D};
  if (layouts) p.in = layouts[0], p.act = layouts[1];
  p.q = static_cast<const __nv_bfloat16*>(a.q);
  p.k = static_cast<const __nv_bfloat16*>(a.k);
  p.v = static_cast<const __nv_bfloat16*>(a.v);
  p.grad_out = static_cast<const __nv_bfloat16*>(a.grad_out);
  p.lse = a.lse;
  p.num_atoms = a.num_atoms;
  p.block_count = a.block_count;
  p.block_cols = a.block_cols;
  p.block_mask = a.block_mask;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.lse_out = a.lse;
  p.dq = static_cast<__nv_bfloat16*>(a.dq);
  p.dk = static_cast<__nv_bfloat16*>(a.dk);
  p.dv = static_cast<__nv_bfloat16*>(a.dv);
  p.H = a.heads;
  p.N = a.tokens;
  p.window = a.window;
  p.tiles = (a.tokens + 31) / 32;
  p.scale = a.scale;
  const int BH = a.batch * a.heads;
  if (!backward) return launch_one<D, kRadius, M_FWD>(p, BH, s);
  float* delta = static_cast<float*>(a.workspace);
  p.delta = delta;
  int rc = launch_one<D, kRadius, M_DQ>(p, BH, s);  // also writes delta
  if (rc != MF_OK) return rc;
  return launch_one<D, kRadius, M_DKV>(p, BH, s);
}

template <bool kRadius>
int dispatch_d(const MfSparseAttnArgs& a, const RowLayout* layouts, bool backward, cudaStream_t s) {
  switch (a.head_dim) {
    case 32: return launch_all<32, kRadius>(a, layouts, backward, s);
    case 64: return launch_all<64, kRadius>(a, layouts, backward, s);
    default: return launch_all<128, kRadius>(a, layouts, backward, s);
  }
}

}  // namespace

int sparse_attn_mma_fwd(const MfSparseAttnArgs& a, bool radius, cudaStream_t stream) {
  return radius ? dispatch_d<true>(a, nullptr, false, stream) : dispatch_d<false>(a, nullptr, false, stream);
}
int sparse_attn_mma_bwd(const MfSparseAttnArgs& a, bool radius, cudaStream_t stream) {
  return radius ? dispatch_d<true>(a, nullptr, true, stream) : dispatch_d<false>(a, nullptr, true, stream);
}
int local_attn_mma_layouts(const MfSparseAttnArgs& a, const RowLayout& in, const RowLayout& act, bool backward,
                           cudaStream_t stream) {
  const RowLayout l[2] = {in, act};
  return dispatch_d<false>(a, l, backward, stream);
}

}  // namespace mf
