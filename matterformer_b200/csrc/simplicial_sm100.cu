// 2-simplicial attention on the Blackwell tensor cores (tcgen05 + tensor memory).
//
// Formulation.  For a tile of 128 queries (one per TMEM lane / thread) the kernel
// walks over the first key index j.  With A_j = Q_tile o k1_j (each query row
// scaled column-wise by k1_j, rewritten into shared memory every step) the
// trilinear logits of step j are one GEMM
//     S_j[i,k] = sum_d q[i,d] k1[j,d] k2[k,d] = (A_j . K2^T)[i,k]          (tcgen05.mma, fp32 in TMEM)
// with a constant K2 tile.  The softmax runs over the whole (j,k) plane with a
// running maximum and sum per query row, exactly like flash attention's, and
//     out[i,:] = sum_j v1_j o (P_j . V2)[i,:]                                (tcgen05.mma, A = P_j from TMEM)
// where the per-column scaling by v1_j is applied while the 128x64 product is
// drained from tensor memory into the fp32 register accumulator.
//
// Semantics follow simplicial_attention_torch_from_projected of the reference
// (src/matterformer/models/simplicial_attention.py:206-344); the interface is the one of
// triton_simplicial_attention_forward/backward (triton_simplicial_attention.py:790-926, 929-1204).
//
// Every wait on an mbarrier is bounded; when one expires the CTA records an error
// code in the status word at the start of the workspace, frees its tensor memory
// and returns.
#include "common.cuh"
#include "simplicial.cuh"
#include "sm100_primitives.cuh"
#include "tensor_map.cuh"
#include "simplicial_sm100.cuh"
#include "simplicial_rows.cuh"

#include <mutex>

namespace mf {
namespace {

constexpr int kTmemCols = 256;  // S/P in columns [0,192), P.V2 product in [192,256)
constexpr int kColW = 192;

// ---------------------------------------------------------------------------
// Per-batch extents and a heaviest-first launch order.
// ---------------------------------------------------------------------------
// one warp per batch element: the last valid key / query index + 1
__global__ void extent_kernel(const uint8_t* __restrict__ query_valid, const uint8_t* __restrict__ key_valid, int B,
                              int N, BatchInfo* __restrict__ info, int32_t* __restrict__ status) {
  if (blockIdx.x == 0 && threadIdx.x < 64) status[threadIdx.x] = 0;  // the 256-byte status block
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  int nk = 0, nq = 0, cnt = 0;
  for (int t = lane; t < N; t += 32) {
    if (key_valid[(size_t)b * N + t]) {
      nk = t + 1;
      ++cnt;
    }
    if (query_valid[(size_t)b * N + t]) nq = t + 1;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    nk = max(nk, __shfl_xor_sync(0xffffffffu, nk, o));
    nq = max(nq, __shfl_xor_sync(0xffffffffu, nq, o));
    cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  }
  if (lane == 0) {
    info[b].n_keys = nk;
    info[b].n_queries = nq;
    info[b].reserved0 = cnt;  // number of valid keys
    info[b].reserved1 = 0;
  }
}

// rank by cost (descending), ties by index: a stable, deterministic order; one warp per batch element, its lanes
// striding over the elements it is compared with
__global__ void order_kernel(const BatchInfo* __restrict__ info, int B, int32_t* __restrict__ order) {
  const int b = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (b >= B) return;  // uniform per warp
  auto cost = [&](int i) {
    return (long long)info[i].n_keys * info[i].n_keys * ((info[i].n_queries + kTileM - 1) / kTileM);
  };
  const long long cb = cost(b);
  int rank = 0;
  for (int o = lane; o < B; o += 32) {
    const long long co = cost(o);
    rank += (co > cb) || (co == cb && o < b);
  }
  rank = __reduce_add_sync(0xffffffffu, rank);
  if (lane == 0) order[rank] = b;
}

struct FwdParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k1;
  const __nv_bfloat16* v1;
  const __nv_bfloat16* k2;
  const __nv_bfloat16* v2;
  const uint8_t* query_valid;
  const uint8_t* key_valid;
  const uint8_t* pair_valid;
  float* out;
  float* lse;
  __nv_bfloat16* out_cast;
  const BatchInfo* info;
  const int32_t* order;
  int32_t* status;
  // factorized logit bias gate_i * ((u_ij + v_ik) + w_jk), fp32, (B,H,N,N) x 3 and (B,H,N); packed-heads kernel only
  const float* u;
  const float* v_bias;
  const float* w;
  const float* gate;
  int bias_vec4;       // rows of v_bias and w start on 16-byte boundaries
  int H, N, q_tiles;
  RowLayout in;        // rows of q, k1, v1, k2, v2
  RowLayout act;       // rows of out_cast
  float q_scale;       // applied to q on load; 1 or another power of two (exact in bf16)
  int use_tma;         // K2 / V2 tiles arrive through the tensor maps below (else plain loads)
  CUtensorMap tm_k2;   // (B*H, N, 64) bf16, boxes of 32 rows, 128-byte swizzle
  CUtensorMap tm_v2;
};

// shared memory map (dynamic, 1024-byte aligned)
constexpr int kSmemK2 = 0;                                // [192][64] bf16, 128B-swizzled, K-major B operand
constexpr int kSmemV2 = kSmemK2 + kMaxKeys * 128;         // [192][64] bf16, 128B-swizzled, MN-major B operand
constexpr int kSmemA = kSmemV2 + kMaxKeys * 128;          // [128][64] bf16, 128B-swizzled, K-major A operand
constexpr int kSmemPv = kSmemA + kTileM * 128;            // [192][6] pair_valid bit rows
constexpr int kSmemFwdBytes = kSmemPv + kMaxKeys * 6 * 4;
constexpr int kSmemFwdAlloc = kSmemFwdBytes + 1024;       // slack for the manual 1024-byte alignment

// kPacked: molecules of at most 32 tokens.  One CTA then serves four heads of a molecule: warp w holds the 32
// query rows of head 4g+w, the K2 / V2 tiles stack the four heads' keys (row 32w'+k = key k of head 4g+w'), the
// logit GEMM computes all 128 x 128 head combinations and only the diagonal 32 x 32 blocks are used: each row
// reads the 32 columns of its own head and writes zeros as the probabilities of the other heads' keys.
// kBias: the factorized geometry bias of the reference kernel (triton_simplicial_attention.py:244-262) is added to the
// logits in fp32 before the softmax: gate_i * ((u_ij + v_ik) + w_jk), the three terms summed first, as the reference sums
// them.  u_ij is one value per row and step, the rows v_i. and w_j. are read through the caches.  One head per tile: the
// biased logits of the maximum pass are written back over the logits in tensor memory, so that the exponential pass reads
// them instead of forming the bias again.
template <bool kPacked, bool kBias = false>
__global__ void __launch_bounds__(128, 2) simplicial_fwd_sm100_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar_s, bar_w, bar_kv;
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t kmask[6];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // heaviest molecules first
  const int per_b = kPacked ? p.H / 4 : p.H * p.q_tiles;
  const int b = p.order[blockIdx.x / per_b];
  const int bh0 = kPacked ? b * p.H + 4 * (int)(blockIdx.x % per_b) : 0;  // packed: first of the CTA's four heads
  const int h = kPacked ? 4 * (int)(blockIdx.x % per_b) + warp : (int)(blockIdx.x % per_b) / p.q_tiles;
  const int qt = kPacked ? 0 : blockIdx.x % p.q_tiles;
  const int N = p.N;
  const int bh = b * p.H + h;
  const size_t base = (size_t)bh * N * kD;           // fp32 out and lse: always (B,H,N,D)
  const long long in_base = p.in.at(b, h, 0);         // this head's rows of q, k1, v1, k2, v2
  const long long act_base = p.act.at(b, h, 0);       // ... of out_cast
  const int n_keys = p.info[b].n_keys;
  const int n_queries = p.info[b].n_queries;
  const int row = kPacked ? lane : qt * kTileM + tid;  // this thread's query
  const bool row_in = row < N;
  const bool row_ok = row_in && p.query_valid[(size_t)b * N + row] > 0;

  // ---- nothing to attend to: write zeros and leave (uniform per CTA)
  if (qt * kTileM >= n_queries || n_keys == 0) {
    if (row_in) {
      float4* o = reinterpret_cast<float4*>(p.out + base + (size_t)row * kD);
#pragma unroll
      for (int c = 0; c < kD / 4; ++c) o[c] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p.out_cast) {
        uint4* oc = reinterpret_cast<uint4*>(p.out_cast + act_base + row * p.act.token);
#pragma unroll
        for (int c = 0; c < kD / 8; ++c) oc[c] = make_uint4(0, 0, 0, 0);
      }
      p.lse[(size_t)bh * N + row] = 0.f;
    }
    return;
  }
  const int nk_pad = kPacked ? 128 : (n_keys + 15) & ~15;  // MMA N (multiple of 16)
  const int n_chunks = (nk_pad + 31) >> 5;
  const bool warp_live = kPacked || qt * kTileM + warp * 32 < n_queries;

  // ---- set-up: barriers, tensor memory, key masks, operand tiles
  if (tid == 0) {
    mbar_init(&bar_s, 1);
    mbar_init(&bar_w, 1);
    mbar_init(&bar_kv, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, kTmemCols);
    tmem_relinquish();
  }
  if (tid < 6) {
    uint32_t w = 0;
    for (int e = 0; e < 32; ++e) {
      const int k = tid * 32 + e;
      if (k < n_keys && p.key_valid[(size_t)b * N + k] > 0) w |= 1u << e;
    }
    kmask[tid] = w;
  }
  __syncthreads();
  {
    uint32_t* pvbits = reinterpret_cast<uint32_t*>(smem + kSmemPv);
    const uint8_t* pv = p.pair_valid ? p.pair_valid + (size_t)b * N * N : nullptr;
    for (int idx = tid; idx < n_keys * 6; idx += 128) {
      const int j = idx / 6, c = idx % 6;
      uint32_t w = 0xffffffffu;
      if (pv) {
        w = 0;
        for (int e = 0; e < 32; ++e) {
          const int k = c * 32 + e;
          if (k < n_keys && pv[(size_t)j * N + k] > 0) w |= 1u << e;
        }
      }
      pvbits[idx] = w;
    }
    // K2 / V2 tiles.  Through the copy engine: one bulk tensor load per 32 rows and tile, all signalling one
    // mbarrier; rows of invalid keys are cleared once the data has landed (below).  Otherwise by plain loads,
    // with rows of invalid keys and padding rows zero-filled.
    if (p.use_tma) {
      if (tid == 0) {
        mbar_arrive_expect_tx(&bar_kv, (uint32_t)n_chunks * 2u * kTmaBoxRows * 128u);
        for (int c = 0; c < n_chunks; ++c) {  // packed: box c = the (at most 32) keys of head c of the CTA
          const int row0 = kPacked ? 0 : c * kTmaBoxRows, mat = kPacked ? bh0 + c : bh;
          tma_load_rows(smem + kSmemK2 + c * kTmaBoxRows * 128, &p.tm_k2, row0, mat, &bar_kv);
          tma_load_rows(smem + kSmemV2 + c * kTmaBoxRows * 128, &p.tm_v2, row0, mat, &bar_kv);
        }
      }
    } else {
      for (int idx = tid; idx < nk_pad * 8; idx += 128) {
        const int r = idx >> 3, c = idx & 7;
        const int key = kPacked ? (r & 31) : r;  // packed: tile row 32w'+k holds key k of head w'
        // packed: row r of the tile belongs to head 4g + (r >> 5), the CTA's heads being bh0 % H .. bh0 % H + 3
        const long long src = kPacked ? p.in.at(b, (bh0 - b * p.H) + (r >> 5), key) : in_base + r * p.in.token;
        uint4 vk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
        if ((kmask[key >> 5] >> (key & 31)) & 1u) {
          vk = __ldg(reinterpret_cast<const uint4*>(p.k2 + src) + c);
          vv = __ldg(reinterpret_cast<const uint4*>(p.v2 + src) + c);
        }
        const uint32_t off = r * 128 + ((c ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(smem + kSmemK2 + off) = vk;
        *reinterpret_cast<uint4*>(smem + kSmemV2 + off) = vv;
      }
    }
  }
  // this thread's query row as 32 bf16x2 words
  uint32_t qreg[32];
  {
    const uint4* qp = reinterpret_cast<const uint4*>(p.q + in_base + row * p.in.token);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row_ok) v = __ldg(qp + c);
      qreg[4 * c + 0] = v.x;
      qreg[4 * c + 1] = v.y;
      qreg[4 * c + 2] = v.z;
      qreg[4 * c + 3] = v.w;
    }
    if (p.q_scale != 1.f) {
      const __nv_bfloat162 sc = __float2bfloat162_rn(p.q_scale);
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const __nv_bfloat162 t = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&qreg[c]), sc);
        qreg[c] = *reinterpret_cast<const uint32_t*>(&t);
      }
    }
  }
  bool bad = false;
  if (p.use_tma) {
    bad |= !mbar_wait(&bar_kv, 0);
    if (!bad)  // rows of invalid keys must be zero whatever the padded tokens hold
      for (int idx = tid; idx < nk_pad * 8; idx += 128) {
        const int r = idx >> 3, c = idx & 7;
        const int key = kPacked ? (r & 31) : r;
        if (!((kmask[key >> 5] >> (key & 31)) & 1u)) {
          const uint32_t off = r * 128 + ((c ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(smem + kSmemK2 + off) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(smem + kSmemV2 + off) = make_uint4(0, 0, 0, 0);
        }
      }
  }
  fence_smem_to_async_proxy();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tmem_row = tmem + ((uint32_t)(warp * 32) << 16);
  const uint32_t sA = smem_u32(smem + kSmemA);
  const uint32_t sK2 = smem_u32(smem + kSmemK2);
  const uint32_t sV2 = smem_u32(smem + kSmemV2);
  const uint32_t* pvbits = reinterpret_cast<const uint32_t*>(smem + kSmemPv);
  const uint32_t idesc_s = make_idesc_bf16(kTileM, nk_pad, false, false);
  const uint32_t idesc_w = make_idesc_bf16(kTileM, kD, false, true);
  // descriptors are built once; the issue loops only step them (see desc_advance)
  const uint64_t dA_k = make_smem_desc_sw128(sA, 0, 1024), dK2_k = make_smem_desc_sw128(sK2, 0, 1024);
  const uint64_t dV2_mn = make_smem_desc_sw128(sV2, kMaxKeys * 128, 1024);

  float o_acc[kD];
#pragma unroll
  for (int d = 0; d < kD; ++d) o_acc[d] = 0.f;
  float m_run = -INFINITY;  // running maximum in the log2 domain
  float l_run = 0.f;
  uint32_t phase = 0;

  // bias operands of this thread's row (kBias): the gate, and the rows of u and v_bias
  const size_t nn = (size_t)N * N;
  const float gate_i = (kBias && row_ok) ? p.gate[(size_t)bh * N + row] : 0.f;
  const float* u_row = kBias ? p.u + (size_t)bh * nn + (size_t)(row_ok ? row : 0) * N : nullptr;
  const float* v_row = kBias ? p.v_bias + (size_t)bh * nn + (size_t)(row_ok ? row : 0) * N : nullptr;

  for (int j = 0; j < n_keys; ++j) {
    if (!((kmask[j >> 5] >> (j & 31)) & 1u)) continue;  // uniform
    const float u_ij = kBias ? __ldg(u_row + j) : 0.f;
    // ---- A_j = Q o k1_j  (one row per thread)
    {
      const uint4* kp = reinterpret_cast<const uint4*>(p.k1 + in_base + j * p.in.token);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 kk = __ldg(kp + c);
        uint4 a;
        __nv_bfloat162 t;
        t = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&qreg[4 * c + 0]), *reinterpret_cast<const __nv_bfloat162*>(&kk.x));
        a.x = *reinterpret_cast<uint32_t*>(&t);
        t = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&qreg[4 * c + 1]), *reinterpret_cast<const __nv_bfloat162*>(&kk.y));
        a.y = *reinterpret_cast<uint32_t*>(&t);
        t = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&qreg[4 * c + 2]), *reinterpret_cast<const __nv_bfloat162*>(&kk.z));
        a.z = *reinterpret_cast<uint32_t*>(&t);
        t = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&qreg[4 * c + 3]), *reinterpret_cast<const __nv_bfloat162*>(&kk.w));
        a.w = *reinterpret_cast<uint32_t*>(&t);
        *reinterpret_cast<uint4*>(smem + kSmemA + tid * 128 + ((c ^ (tid & 7)) << 4)) = a;
      }
    }
    {  // the k1 / v1 rows of the next step: one 128-byte line each, on their way to L1 while this step runs
      int jn = j + 1;
      while (jn < n_keys && !((kmask[jn >> 5] >> (jn & 31)) & 1u)) ++jn;
      if (lane == 0 && jn < n_keys) {
        asm volatile("prefetch.global.L1 [%0];" ::"l"(p.k1 + in_base + jn * p.in.token));
        asm volatile("prefetch.global.L1 [%0];" ::"l"(p.v1 + in_base + jn * p.in.token));
      }
    }
    fence_smem_to_async_proxy();
    tc_fence_before_sync();
    __syncthreads();
    // ---- S_j = A_j . K2^T
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks)
        umma_ss(tmem, desc_advance(dA_k, 32 * ks), desc_advance(dK2_k, 32 * ks), idesc_s, ks > 0);
      umma_commit(&bar_s);
    }
    bad |= !mbar_wait(&bar_s, phase);
    tc_fence_after_sync();

    float alpha = 1.f;
    if (warp_live) {  // warps whose 32 rows all lie beyond the last valid query skip the row work
    // Both passes keep two 32-column chunks in flight: the tensor-memory load of chunk c+1 is issued
    // before chunk c is processed, and independent partial maxima / sums keep the dependency chains short.
    // ---- pass 1: row maximum over the visible columns
    const uint32_t* pvrow = pvbits + j * 6;
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    auto max_chunk = [&](const uint32_t (&s)[32], int c) {
      const uint32_t word = kmask[c] & pvrow[c];
      if (word == 0xffffffffu) {
#pragma unroll
        for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(s[e]));
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          mx4[e & 3] = fmaxf(mx4[e & 3], ((word >> e) & 1u) ? __uint_as_float(s[e]) : -INFINITY);
      }
    };
    // packed heads: the row has one chunk, the 32 columns of its own head; it stays in registers for pass 2
    const uint32_t tmem_srow = tmem_row + (kPacked ? 32 * warp : 0);
    const int row_chunks = kPacked ? 1 : n_chunks;
    uint32_t sa[32], sb[32];
    tmem_ld32(tmem_srow, sa);
    if constexpr (kBias && kPacked) {  // the row's one chunk: logits += gate_i * ((u_ij + v_ik) + w_jk) for its head's keys
      const float* w_row = p.w + (size_t)bh * nn + (size_t)j * N;
      float bsum[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) bsum[e] = e < N ? (u_ij + __ldg(v_row + e)) + __ldg(w_row + e) : 0.f;
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) sa[e] = __float_as_uint(fmaf(gate_i, bsum[e], __uint_as_float(sa[e])));
    }
    // one head per tile with the bias: add it to chunk c and put the chunk back for pass 2
    auto bias_chunk = [&](uint32_t (&s)[32], int c) {
      if constexpr (kBias && !kPacked) {
        const float* w_row = p.w + (size_t)bh * nn + (size_t)j * N;
        if (p.bias_vec4) {  // rows of v_bias and w start on 16-byte boundaries: four keys per load
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const int k = 32 * c + e;
            if (k < N) {
              const float4 vv = __ldg(reinterpret_cast<const float4*>(v_row + k));
              const float4 ww = __ldg(reinterpret_cast<const float4*>(w_row + k));
              s[e] = __float_as_uint(fmaf(gate_i, (u_ij + vv.x) + ww.x, __uint_as_float(s[e])));
              s[e + 1] = __float_as_uint(fmaf(gate_i, (u_ij + vv.y) + ww.y, __uint_as_float(s[e + 1])));
              s[e + 2] = __float_as_uint(fmaf(gate_i, (u_ij + vv.z) + ww.z, __uint_as_float(s[e + 2])));
              s[e + 3] = __float_as_uint(fmaf(gate_i, (u_ij + vv.w) + ww.w, __uint_as_float(s[e + 3])));
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int k = 32 * c + e;
            if (k < N) {
              const float bsum = (u_ij + __ldg(v_row + k)) + __ldg(w_row + k);
              s[e] = __float_as_uint(fmaf(gate_i, bsum, __uint_as_float(s[e])));
            }
          }
        }
        tmem_st16(tmem_srow + 32 * c, reinterpret_cast<const uint32_t(&)[16]>(s[0]));
        tmem_st16(tmem_srow + 32 * c + 16, reinterpret_cast<const uint32_t(&)[16]>(s[16]));
      }
    };
    for (int c = 0; c < row_chunks; c += 2) {
      tmem_ld_wait();
      if (c + 1 < row_chunks) tmem_ld32(tmem_srow + 32 * (c + 1), sb);
      bias_chunk(sa, c);
      max_chunk(sa, c);
      if (c + 1 < row_chunks) {
        tmem_ld_wait();
        if (c + 2 < row_chunks) tmem_ld32(tmem_srow + 32 * (c + 2), sa);
        bias_chunk(sb, c + 1);
        max_chunk(sb, c + 1);
      }
    }
    if constexpr (kBias && !kPacked) tmem_st_wait();  // the biased logits are in tensor memory before they are read again
    if (!kPacked) tmem_ld32(tmem_srow, sa);  // first chunk of pass 2
    const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
    const float m_new = fmaxf(m_run, mx * kLog2e);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_use);
    m_run = m_new;

    // ---- pass 2: P = exp2(S log2e - m), packed to bf16 into the columns S occupied.  P chunk c lands on
    // columns [16c, 16c+16), which lie below every S chunk still to be read.
    float ps4[4] = {0.f, 0.f, 0.f, 0.f};
    auto exp_chunk = [&](const uint32_t (&s)[32], int c) {
      const uint32_t word = kmask[c] & pvrow[c];
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float p0 = fast_exp2(fmaf(__uint_as_float(s[e]), kLog2e, -m_use));
        float p1 = fast_exp2(fmaf(__uint_as_float(s[e + 1]), kLog2e, -m_use));
        if (word != 0xffffffffu) {
          p0 = ((word >> e) & 1u) ? p0 : 0.f;
          p1 = ((word >> (e + 1)) & 1u) ? p1 : 0.f;
        }
        ps4[(e >> 1) & 3] += p0 + p1;
        pk[e >> 1] = pack_bf16x2(p0, p1);
      }
      tmem_st16(tmem_row + 16 * (kPacked ? warp : c), pk);
    };
    for (int c = 0; c < row_chunks; c += 2) {
      tmem_ld_wait();
      if (c + 1 < row_chunks) tmem_ld32(tmem_srow + 32 * (c + 1), sb);
      exp_chunk(sa, c);
      if (c + 1 < row_chunks) {
        tmem_ld_wait();
        if (c + 2 < row_chunks) tmem_ld32(tmem_srow + 32 * (c + 2), sa);
        exp_chunk(sb, c + 1);
      }
    }
    if (kPacked) {  // probabilities of the other heads' keys: zeros over the cross-head logits
      uint32_t zero16[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) zero16[e] = 0u;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c != warp) tmem_st16(tmem_row + 16 * c, zero16);
    }
    const float psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
    l_run = l_run * alpha + psum;
    }
    tmem_st_wait();
    tc_fence_before_sync();
    if (__syncthreads_or(bad)) {
      bad = true;
      break;
    }
    // ---- W_j = P_j . V2
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < kMaxKeys / 16; ++ks)
        if (ks < nk_pad / 16) umma_ts(tmem + kColW, tmem + 8 * ks, desc_advance(dV2_mn, 2048 * ks), idesc_w, ks > 0);
      umma_commit(&bar_w);
    }
    // v1_j while the MMA runs
    uint4 v1w[8];
    {
      const uint4* vp = reinterpret_cast<const uint4*>(p.v1 + in_base + j * p.in.token);
#pragma unroll
      for (int c = 0; c < 8; ++c) v1w[c] = __ldg(vp + c);
    }
    bad |= !mbar_wait(&bar_w, phase);
    tc_fence_after_sync();
    phase ^= 1u;
    // ---- out += v1_j o W_j
#pragma unroll
    for (int half = 0; half < 2 && warp_live; ++half) {
      uint32_t w[32];
      tmem_ld32(tmem_row + kColW + 32 * half, w);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 vv = v1w[4 * half + c];
        const uint32_t vw[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int d = 32 * half + 8 * c + 2 * t;
          const float v_lo = __uint_as_float(vw[t] << 16);
          const float v_hi = __uint_as_float(vw[t] & 0xffff0000u);
          o_acc[d] = fmaf(o_acc[d], alpha, __uint_as_float(w[8 * c + 2 * t]) * v_lo);
          o_acc[d + 1] = fmaf(o_acc[d + 1], alpha, __uint_as_float(w[8 * c + 2 * t + 1]) * v_hi);
        }
      }
    }
    tc_fence_before_sync();  // the next step's MMAs overwrite what was just read
  }

  // ---- epilogue
  bad = __syncthreads_or(bad) != 0;
  if (bad && tid == 0) atomicExch(p.status, MF_ERR_DEVICE_TIMEOUT);
  if (row_in) {
    const bool have = row_ok && l_run > 0.f && !bad;
    const float inv = have ? 1.f / l_run : 0.f;
    float4* o = reinterpret_cast<float4*>(p.out + base + (size_t)row * kD);
#pragma unroll
    for (int c = 0; c < kD / 4; ++c)
      o[c] = make_float4(o_acc[4 * c] * inv, o_acc[4 * c + 1] * inv, o_acc[4 * c + 2] * inv, o_acc[4 * c + 3] * inv);
    if (p.out_cast) {
      uint4* oc = reinterpret_cast<uint4*>(p.out_cast + act_base + row * p.act.token);
#pragma unroll
      for (int c = 0; c < kD / 8; ++c) {
        uint4 v;
        v.x = pack_bf16x2(o_acc[8 * c + 0] * inv, o_acc[8 * c + 1] * inv);
        v.y = pack_bf16x2(o_acc[8 * c + 2] * inv, o_acc[8 * c + 3] * inv);
        v.z = pack_bf16x2(o_acc[8 * c + 4] * inv, o_acc[8 * c + 5] * inv);
        v.w = pack_bf16x2(o_acc[8 * c + 6] * inv, o_acc[8 * c + 7] * inv);
        oc[c] = v;
      }
    }
    p.lse[(size_t)bh * N + row] = have ? (m_run + log2f(l_run)) * kLn2 : 0.f;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

size_t simplicial_schedule_layout(int B, size_t* info_off, size_t* order_off) {
  size_t off = kStatusBytes;
  *info_off = off;
  off += align_up((size_t)B * sizeof(BatchInfo), 256);
  *order_off = off;
  off += align_up((size_t)B * sizeof(int32_t), 256);
  return off;
}

int cached_max_row_tiles(int tokens) {
  static std::mutex mu;
  static int table[kMaxKeys + 1] = {};
  if (tokens < 1) return 1;
  if (tokens > kMaxKeys) tokens = kMaxKeys;
  std::lock_guard<std::mutex> lock(mu);
  if (table[tokens] == 0) table[tokens] = max_row_tiles(tokens);
  return table[tokens];
}

int launch_schedule(const uint8_t* query_valid, const uint8_t* key_valid, int B, int N, BatchInfo* info,
                    int32_t* order, int32_t* status, cudaStream_t stream) {
  extent_kernel<<<(B + 7) / 8, 256, 0, stream>>>(query_valid, key_valid, B, N, info, status);
  MF_CHECK_LAUNCH("extent_kernel");
  order_kernel<<<(B + 7) / 8, 256, 0, stream>>>(info, B, order);
  MF_CHECK_LAUNCH("order_kernel");
  return MF_OK;
}

bool simplicial_sm100_supports(int dtype, int precision, int tokens, int head_dim) {
  return dtype == MF_DTYPE_BF16 && precision == MF_PRECISION_BF16_TC && head_dim == kD && tokens <= kMaxKeys &&
         tokens >= 1;
}

size_t simplicial_sm100_fwd_workspace_bytes(const MfSimplicialFwdArgs& a) {
  size_t i, o;
  return simplicial_schedule_layout(a.batch, &i, &o);
}

int simplicial_sm100_fwd(const MfSimplicialFwdArgs& a, cudaStream_t stream) {
  return simplicial_sm100_fwd_layouts(a, nullptr, stream);
}

int simplicial_sm100_fwd_layouts(const MfSimplicialFwdArgs& a, const TileLayouts* layouts, cudaStream_t stream) {
  size_t info_off, order_off;
  simplicial_schedule_layout(a.batch, &info_off, &order_off);
  char* ws = static_cast<char*>(a.workspace);
  FwdParams p{};
  p.q = static_cast<const __nv_bfloat16*>(a.q);
  p.k1 = static_cast<const __nv_bfloat16*>(a.k1);
  p.v1 = static_cast<const __nv_bfloat16*>(a.v1);
  p.k2 = static_cast<const __nv_bfloat16*>(a.k2);
  p.v2 = static_cast<const __nv_bfloat16*>(a.v2);
  p.query_valid = a.query_valid;
  p.key_valid = a.pair_key_valid;
  p.pair_valid = a.pair_valid;
  p.out = a.out;
  p.lse = a.lse;
  p.out_cast = static_cast<__nv_bfloat16*>(a.out_cast);
  p.status = reinterpret_cast<int32_t*>(ws);
  BatchInfo* info = reinterpret_cast<BatchInfo*>(ws + info_off);
  int32_t* order = reinterpret_cast<int32_t*>(ws + order_off);
  p.info = info;
  p.order = order;
  p.H = a.heads;
  p.N = a.tokens;
  p.q_tiles = (a.tokens + kTileM - 1) / kTileM;
  p.u = a.u, p.v_bias = a.v_bias, p.w = a.w, p.gate = a.gate;
  p.bias_vec4 = a.tokens % 4 == 0 && reinterpret_cast<uintptr_t>(a.v_bias) % 16 == 0 && reinterpret_cast<uintptr_t>(a.w) % 16 == 0;
  p.in = p.act = contiguous_rows(a.heads, a.tokens);
  p.q_scale = 1.f;
  if (layouts) {  // rows that are not (B,H,N,D) contiguous come by plain loads: the tensor maps describe that form only
    p.in = layouts->in, p.act = layouts->act, p.q_scale = layouts->q_scale;
    p.use_tma = 0;
  } else {
    p.use_tma = make_rows_tensor_map(&p.tm_k2, a.k2, a.tokens, a.batch * a.heads) &&
                make_rows_tensor_map(&p.tm_v2, a.v2, a.tokens, a.batch * a.heads);
  }
  int rc = launch_schedule(a.query_valid, a.pair_key_valid, a.batch, a.tokens, info, order, p.status, stream);
  if (rc != MF_OK) return rc;
  const bool packed = simplicial_sm100_packs_heads(a.tokens, a.heads);
  const bool bias = a.u != nullptr;
  auto kern = bias ? (packed ? simplicial_fwd_sm100_kernel<true, true> : simplicial_fwd_sm100_kernel<false, true>)
                   : (packed ? simplicial_fwd_sm100_kernel<true, false> : simplicial_fwd_sm100_kernel<false, false>);
  {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFwdAlloc);
    if (e != cudaSuccess) return cuda_error(e, "cudaFuncSetAttribute(simplicial_fwd_sm100_kernel)");
  }
  const long long blocks = packed ? (long long)a.batch * (a.heads / 4) : (long long)a.batch * a.heads * p.q_tiles;
  profile_mark(MF_PROFILE_SIMPLICIAL_FWD, true, stream);
  kern<<<(unsigned)blocks, 128, kSmemFwdAlloc, stream>>>(p);
  profile_mark(MF_PROFILE_SIMPLICIAL_FWD, false, stream);
  MF_CHECK_LAUNCH("simplicial_fwd_sm100_kernel");
  return MF_OK;
}

}  // namespace mf

// ---------------------------------------------------------------------------
// Forward pass for callers that cannot allocate device memory
// ---------------------------------------------------------------------------
// The tensor-core forward kernel needs a little scratch (status word, per-molecule extents, launch
// order).  mf_simplicial_fwd takes it from the caller; this variant keeps it in the library image
// instead, so a caller that only holds its input and output buffers -- a plugin running inside someone
// else's memory pool, a real-time loop that may not touch the allocator, code that runs after the
// framework's allocator has been frozen -- can still launch the kernel.  Every GPU that loads the
// library carries the array (about 80 KB) until the process exits.
#include <mutex>

#define MF_NOALLOC_MAX_BATCH 4096
namespace {
constexpr size_t kNoAllocScratchBytes =
    mf::kStatusBytes + MF_NOALLOC_MAX_BATCH * sizeof(mf::BatchInfo) + MF_NOALLOC_MAX_BATCH * sizeof(int32_t) + 512;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address: the address each
// device gave the array is looked up once per device (with that device current) and cached here.
constexpr int kMaxDevices = 64;
void* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;
}  // namespace

extern "C" int mf_simplicial_fwd_noalloc(const MfSimplicialFwdArgs* args, void* stream) {
  using namespace mf;
  MF_CHECK_ARG(args != nullptr, "mf_simplicial_fwd_noalloc: null argument struct");
  MF_CHECK_ARG(args->batch >= 0 && args->heads >= 0 && args->tokens >= 0, "mf_simplicial_fwd_noalloc: negative size");
  if (args->batch > MF_NOALLOC_MAX_BATCH) {
    set_error("mf_simplicial_fwd_noalloc: batch %d exceeds the built-in scratch (at most %d molecules per call); "
              "split the batch or use mf_simplicial_fwd with a caller-provided workspace",
              (int)args->batch, MF_NOALLOC_MAX_BATCH);
    return MF_ERR_INVALID_ARGUMENT;
  }
  if (args->batch == 0 || args->heads == 0 || args->tokens == 0) return MF_OK;
  if (!simplicial_sm100_supports(args->dtype, args->precision, args->tokens, args->head_dim) ||
      args->backend == MF_BACKEND_GENERIC || args->u || args->v_bias || args->w || args->gate || args->angle_left ||
      args->message_left) {
    set_error("mf_simplicial_fwd_noalloc: only the tensor-core forward kernel has this variant (bf16 inputs, "
              "precision bf16_tc, head_dim 64, tokens <= %d); other problems need no scratch in mf_simplicial_fwd",
              kMaxKeys);
    return MF_ERR_UNSUPPORTED;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_error(e, "mf_simplicial_fwd_noalloc: cudaGetDevice");
  MF_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "mf_simplicial_fwd_noalloc: device index %d out of range", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {  // first call on this device: resolve the symbol's device address
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (e != cudaSuccess) return cuda_error(e, "mf_simplicial_fwd_noalloc: cudaGetSymbolAddress");
      g_noalloc_ptr[dev] = ptr;
    }
    scratch = g_noalloc_ptr[dev];
  }
  MfSimplicialFwdArgs a = *args;
  a.workspace = scratch;
  a.workspace_bytes = kNoAllocScratchBytes;
  if (simplicial_sm100_fwd_workspace_bytes(a) > kNoAllocScratchBytes) {
    set_error("mf_simplicial_fwd_noalloc: internal scratch too small for batch %d", (int)a.batch);
    return MF_ERR_WORKSPACE_TOO_SMALL;
  }
  // Same validation and launch as the allocating entry point; the status word at the start of the scratch is
  // cleared by the first kernel of every call, nothing else has to start at zero.
  return mf_simplicial_fwd(&a, stream);
}

// The status word of the last mf_simplicial_fwd_noalloc call on the current device, copied to a caller-provided host
// integer by one asynchronous copy on `stream` (no allocation); the caller synchronises the stream before reading it.
extern "C" int mf_simplicial_noalloc_status(int32_t* host_status, void* stream) {
  using namespace mf;
  MF_CHECK_ARG(host_status != nullptr, "mf_simplicial_noalloc_status: null output pointer");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_error(e, "mf_simplicial_noalloc_status: cudaGetDevice");
  MF_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "mf_simplicial_noalloc_status: device index %d out of range", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    scratch = g_noalloc_ptr[dev];
  }
  if (!scratch) {  // nothing has run on this device yet: there is no status to report
    *host_status = MF_OK;
    return MF_OK;
  }
  e = cudaMemcpyAsync(host_status, scratch, sizeof(int32_t), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_error(e, "mf_simplicial_noalloc_status: cudaMemcpyAsync");
  return MF_OK;
}

// ---------------------------------------------------------------------------
// Self-test of the bounded waits
// ---------------------------------------------------------------------------
namespace mf {
namespace {
// One warp waits on a barrier that nobody ever arrives on, with the given limit instead of the production one; when
// the wait gives up the kernel reports the way every tensor-core kernel does and returns.
__global__ void wait_timeout_selftest_kernel(int32_t* status, long long limit_cycles) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  const long long t0 = clock64();
  const bool ok = mbar_wait_for(&bar, 0, limit_cycles);
  if (threadIdx.x == 0) {
    status[0] = ok ? MF_OK : MF_ERR_DEVICE_TIMEOUT;
    const long long dt = clock64() - t0;
    status[1] = dt > 0x7fffffffll ? 0x7fffffff : (int32_t)dt;
  }
}
}  // namespace
}  // namespace mf

extern "C" int mf_selftest_wait_timeout(int32_t* status, int64_t limit_cycles, void* stream) {
  using namespace mf;
  MF_CHECK_ARG(status != nullptr, "mf_selftest_wait_timeout: null status pointer");
  MF_CHECK_ARG(limit_cycles >= 1 && limit_cycles <= (1ll << 31), "mf_selftest_wait_timeout: limit must be in [1, 2^31] clocks");
  wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, (long long)limit_cycles);
  MF_CHECK_LAUNCH("wait_timeout_selftest_kernel");
  return MF_OK;
}
