// Backward pass of 2-simplicial attention on the Blackwell tensor cores.
//
// One CTA owns a 128-query tile x a 128-key slab of the second key set (index k)
// of one (batch, head) and walks over the first key index j.  Per step, with
//   A1_j = Q o k1_j   and   A2_j = dO o v1_j      (rewritten into shared memory every step)
// six GEMMs run on tcgen05 with fp32 accumulators in tensor memory:
//   S_j   = A1_j . K2^T          logits (recomputed)              M=128 N<=128 K=64
//   dP_j  = A2_j . V2^T          d(out)/d(prob)                   M=128 N<=128 K=64
//   U_j   = dS_j . K2            -> dq += U_j o k1_j,  dk1_j = colsum_i(Q o U_j)
//   W_j   = P_j  . V2            -> dv1_j = colsum_i(dO o W_j)
//   dK2  += dS_j^T . A1_j        accumulated in TMEM over every j
//   dV2  += P_j^T  . A2_j        accumulated in TMEM over every j
// with P_j = exp(S_j - lse_i) and dS_j = P_j o (dP_j - delta_i), delta_i = dO_i . out_i,
// formed by the worker threads (one query row each), written as bf16 to shared memory, where
// the bytes serve as MN-major A operand of dK2 and dV2, and packed in place into tensor memory,
// from where they are the A operand of U and W.  These are the six products of the reference's
// backward kernel (src/matterformer/models/triton_simplicial_attention.py:553,611,626,627,644,645).
//
// Partial results of the (query tile, key slab) CTAs of one (batch, head) go to
// fp32 scratch and are summed in a fixed order by a finalize kernel: there are no
// floating-point atomics, so gradients are bit-identical from run to run.
//
// Threads: 384 = three warp groups.
//   group 0 (warps 0-3) holds the q rows : builds A1, drains U
//   group 1 (warps 4-7) holds the dO rows: builds A2, drains W
//   both form P and dS of their rows, one 64-column half of the slab (X, then Y) at a time
//   group 2: one thread issues every tcgen05.mma from descriptors built once; the group hands
//            its registers to the workers (setmaxnreg), which only works when the CTA has
//            three full warp groups for the register pool to come from.
// The MMAs of one half run while the workers process the other half; issuer -> workers
// hand-offs are tcgen05.commit on mbarriers, workers -> issuer hand-offs are mbarriers with
// 256 arrivals.
// Every mbarrier wait is bounded; on expiry the CTA reports through the status word and
// leaves after freeing its tensor memory.
#include "common.cuh"
#include "simplicial.cuh"
#include "simplicial_sm100.cuh"
#include "sm100_primitives.cuh"
#include "tensor_map.cuh"

namespace mf {
namespace {

constexpr int kSlab = 128;          // keys of the second set per CTA
constexpr int kBwdTmemCols = 512;
constexpr int kColS = 0;            // S    [0,128)
constexpr int kColDP = 128;         // dP   [128,256)
constexpr int kColU = 256;          // U    [256,320)
constexpr int kColWb = 320;         // W    [320,384)
constexpr int kColDK2 = 384;        // dK2  [384,448)
constexpr int kColDV2 = 448;        // dV2  [448,512)
constexpr int kMaskWords = kMaxKeys / 32;

// shared memory map (dynamic, 1024-byte aligned)
constexpr int kOffK2 = 0;                       // [128][64] bf16 swizzled: slab of K2
constexpr int kOffV2 = kOffK2 + kSlab * 128;    // [128][64]            : slab of V2
constexpr int kOffA1 = kOffV2 + kSlab * 128;    // 2 stages x [128][64] : Q o k1_j
constexpr int kOffA2 = kOffA1 + 2 * kTileM * 128;  // 2 stages x [128][64]: dO o v1_j
constexpr int kOffP = kOffA2 + 2 * kTileM * 128;   // 2 chunks x [128][64]: P_j   (chunk = 64 logit columns)
constexpr int kOffDS = kOffP + 2 * kTileM * 128;   // 2 chunks x [128][64]: dS_j
constexpr int kOffPv = kOffDS + 2 * kTileM * 128;  // [192][6] pair_valid bit rows
constexpr int kOffRed = kOffPv + kMaxKeys * kMaskWords * 4;  // 2 x [8 warps][64] column-sum partials
constexpr int kSmemBwdBytes = kOffRed + 2 * 8 * 64 * 4;
constexpr int kSmemBwdAlloc = kSmemBwdBytes + 1024;
// with the factorized bias, four heads per tile: per row the running sum over the steps of dS (the gradient of v_bias),
// [128][33] fp32
constexpr int kOffDvb = kSmemBwdBytes;
constexpr int kDvbStride = 33;  // odd: the rows of a warp fall into different banks
// with the factorized bias, one head per tile: the four row groups' column sums of gate_i dS of a step (the gradient of
// w), 2 steps x [4][128] fp32, and the column halves' row sums of dS (the gradient of u) and of dS x bias (the
// gradient of the gate), 2 steps x [128] fp32
constexpr int kOffDwRed = kSmemBwdBytes;
constexpr int kOffDuRed = kOffDwRed + 2 * 4 * kSlab * 4;
static_assert(kOffDuRed + 2 * kTileM * 4 <= kOffDvb + kTileM * kDvbStride * 4, "the bias scratch of both variants fits one size");
constexpr int kSmemBwdBiasAlloc = kOffDvb + kTileM * kDvbStride * 4 + 1024;

struct BwdParams {
  const __nv_bfloat16* grad_out;
  const __nv_bfloat16* q;
  const __nv_bfloat16* k1;
  const __nv_bfloat16* v1;
  const __nv_bfloat16* k2;
  const __nv_bfloat16* v2;
  const float* lse;
  const float* delta;
  const uint8_t* query_valid;
  const uint8_t* key_valid;
  const uint8_t* pair_valid;
  // fp32 partials, each (BH, N, 64)
  float* dq_part;   // [slab]
  float* dk2_part;  // [q_tile]
  float* dv2_part;  // [q_tile]
  float* dk1_part;  // [q_tile][slab]
  float* dv1_part;  // [q_tile][slab]
  const BatchInfo* info;
  const int32_t* order;
  int32_t* status;
  int H, N, q_tiles, slabs;
  size_t part_stride;  // BH * N * 64
  // factorized logit bias gate_i * ((u_ij + v_ik) + w_jk) and its gradients, fp32, (B,H,N,N) x 3 and (B,H,N);
  // packed-heads kernel only
  const float* u;
  const float* v_bias;
  const float* w;
  const float* gate;
  float* du;
  float* dv_bias;
  float* dw;
  float* dgate;
  int dv_vec4;         // rows of dv_bias start on 16-byte boundaries: four keys per reduction
  int bias_vec4;       // likewise the rows of v_bias and w: four keys per load
  // four heads per tile: one CTA holds every contribution to its heads' gradients and writes them itself, in bf16
  __nv_bfloat16* gq;
  __nv_bfloat16* gk1;
  __nv_bfloat16* gv1;
  __nv_bfloat16* gk2;
  __nv_bfloat16* gv2;
  RowLayout in;        // rows of q, k1, v1, k2, v2 and of the five gradients
  RowLayout act;       // rows of grad_out
  float q_scale;       // applied to q on load and to dq on store; 1 or another power of two
  int use_tma;         // K2 / V2 slabs arrive through the tensor maps below (else plain loads)
  CUtensorMap tm_k2;   // (B*H, N, 64) bf16, boxes of 32 rows, 128-byte swizzle
  CUtensorMap tm_v2;
};

template <typename T>
__global__ void delta_bf16_kernel(const __nv_bfloat16* __restrict__ grad_out, RowLayout go, int H, int N,
                                  const float* __restrict__ out, float* __restrict__ delta, int rows) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (b, h, n) in the order of out and delta
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int n = row % N, bh = row / N;
  const __nv_bfloat162 g = reinterpret_cast<const __nv_bfloat162*>(grad_out + go.at(bh / H, bh % H, n))[lane];
  const float2 o = reinterpret_cast<const float2*>(out + (size_t)row * kD)[lane];
  float s = fmaf(__bfloat162float(g.x), o.x, __bfloat162float(g.y) * o.y);
  s = warp_sum(s);
  if (lane == 0) delta[row] = s;
}

// Additions to global memory that return nothing (the thread does not wait for them).  Additions of one thread to one
// address take effect in program order, so a location with a single writer accumulates in a fixed order.
__device__ __forceinline__ void red_add(float* addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add4(float* addr, float a, float b, float c, float d) {  // 16-byte aligned
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Sum over the 32 lanes of a warp of a 32-vector held by every lane: lane l returns the total of column l.
// Fixed exchange pattern -> deterministic.
__device__ __forceinline__ float warp_column_sums32(float (&v)[32], int lane) {
#pragma unroll
  for (int off = 16, n = 16; off >= 1; off >>= 1, n >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int t = 0; t < n; ++t) {
      const float send = upper ? v[t] : v[t + n];
      const float keep = upper ? v[t + n] : v[t];
      v[t] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return v[0];
}

// Sum over the 32 lanes of a warp of a 64-vector held by every lane.  Returns in (r0, r1) the
// totals of columns 2*lane and 2*lane+1.  Fixed exchange pattern -> deterministic.
__device__ __forceinline__ void warp_column_sums(float (&v)[64], int lane, float& r0, float& r1) {
#pragma unroll
  for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int t = 0; t < n; ++t) {
      const float send = upper ? v[t] : v[t + n];
      const float keep = upper ? v[t + n] : v[t];
      v[t] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  r0 = v[0];
  r1 = v[1];
}

constexpr int kBwdThreads = 384;   // 8 worker warps + one warp group that holds the issuing warp
constexpr int kIssuerThread = 256;

// kPacked: molecules of at most 32 tokens.  One CTA serves four heads of a molecule: tile row 32w+i is query i
// of head 4g+w, slab row 32w+k is key k of the same head.  The logit GEMMs compute all 128 x 128 combinations;
// a row uses the 32 columns of its own head and its probabilities for the other heads' keys are written as
// zeros, which keeps the four products that follow block-diagonal.
// kBias: the factorized geometry bias of the reference kernel enters the recomputed logits, and its four gradients leave
// the same element-wise pass (triton_simplicial_attention.py:660-682): du_ij = gate_i sum_k dS, dv_ik = gate_i sum_j dS,
// dw_jk = sum_i gate_i dS, dgate_i = sum_jk dS ((u_ij + v_ik) + w_jk).
// Four heads per tile: a row's 32 live logits of a step are all in one thread and the 32 rows of a head are the lanes of
// one warp, so every sum is local or one shuffle tree; dv accumulates over the steps in a shared-memory row private to
// the thread, and every gradient element has one writer.
// One head per tile: a (row, key) pair belongs to one thread of one CTA, which adds gate_i dS to dv_bias in global
// memory step by step (one writer per address: fixed order).  The sums over a row's keys are combined between the two
// column halves of the CTA through shared memory and between the (at most two) key slabs by an atomic addition; the
// sums over the rows go warp -> four row groups (shared memory) -> the (at most two) query tiles (atomic addition).
// Two addends commute, so the results do not depend on the order in which the CTAs run.
template <bool kPacked, bool kBias = false>
__global__ void __maxnreg__(168) simplicial_bwd_sm100_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar_sx, bar_sy, bar_uw, bar_fin;  // signalled by tcgen05.commit
  __shared__ uint64_t bar_px, bar_py, bar_a, bar_a0;     // 256 worker arrivals each
  __shared__ uint64_t bar_kv;                             // bulk tensor copies of the K2 / V2 slab
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t kmask[kMaskWords];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_worker = tid < 256;
  const int grp = (tid >> 7) & 1;  // 0: q side, 1: dO side
  const int r = tid & 127;         // row of the tile
  const int per_b = kPacked ? p.H / 4 : p.H * p.q_tiles * p.slabs;
  const int b = p.order[blockIdx.x / per_b];
  int rem = blockIdx.x % per_b;
  const int hh = r >> 5;                                       // packed: which of the CTA's four heads this row is
  const int bh0 = kPacked ? b * p.H + 4 * rem : 0;             // packed: first of the CTA's four heads
  const int h = kPacked ? 4 * rem + hh : rem / (p.q_tiles * p.slabs);
  rem %= p.q_tiles * p.slabs;
  const int qt = kPacked ? 0 : rem / p.slabs;
  const int slab = kPacked ? 0 : rem % p.slabs;
  const int N = p.N;
  const int bh = b * p.H + h;
  const size_t base = (size_t)bh * N * kD;      // partial planes, lse, delta: always (B,H,N,D)
  const long long in_base = p.in.at(b, h, 0);    // this head's rows of q, k1, v1, k2, v2
  const int n_keys = p.info[b].n_keys;
  const int n_queries = p.info[b].n_queries;
  if (qt * kTileM >= n_queries || slab * kSlab >= n_keys) {  // nothing to attend to (uniform per CTA)
    if constexpr (kPacked) {  // the gradients of the CTA's four heads are zeros
      for (int idx = tid; idx < 4 * N * 8; idx += kBwdThreads) {
        const long long off = p.in.at(b, bh0 - b * p.H + idx / (N * 8), (idx >> 3) % N) + 8 * (idx & 7);
        const uint4 z = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(p.gq + off) = z;
        *reinterpret_cast<uint4*>(p.gk1 + off) = z;
        *reinterpret_cast<uint4*>(p.gv1 + off) = z;
        *reinterpret_cast<uint4*>(p.gk2 + off) = z;
        *reinterpret_cast<uint4*>(p.gv2 + off) = z;
      }
    }
    return;  // one head per tile: the finalize kernel never reads this CTA's partials
  }

  const int k0 = slab * kSlab;                                  // first key of the slab
  const int nk_slab = min(kSlab, n_keys - k0);                  // keys in the slab
  const int nk_pad = kPacked ? kSlab : (nk_slab + 15) & ~15;    // MMA N of the logit GEMMs
  const int row = kPacked ? (r & 31) : qt * kTileM + r;
  const bool row_ok = is_worker && row < N && p.query_valid[(size_t)b * N + row] > 0;

  if (tid == 0) {
    mbar_init(&bar_sx, 1);
    mbar_init(&bar_sy, 1);
    mbar_init(&bar_uw, 1);
    mbar_init(&bar_fin, 1);
    mbar_init(&bar_px, 256);
    mbar_init(&bar_py, 256);
    mbar_init(&bar_a, 256);
    mbar_init(&bar_a0, 256);
    mbar_init(&bar_kv, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, kBwdTmemCols);
    tmem_relinquish();
  }
  if (tid < kMaskWords) {
    uint32_t w = 0;
    for (int e = 0; e < 32; ++e) {
      const int k = tid * 32 + e;
      if (k < n_keys && p.key_valid[(size_t)b * N + k] > 0) w |= 1u << e;
    }
    kmask[tid] = w;
  }
  __syncthreads();
  uint32_t* pvbits_w = reinterpret_cast<uint32_t*>(smem + kOffPv);
  {
    const uint8_t* pv = p.pair_valid ? p.pair_valid + (size_t)b * N * N : nullptr;
    for (int idx = tid; idx < n_keys * kMaskWords; idx += kBwdThreads) {
      const int j = idx / kMaskWords, c = idx % kMaskWords;
      uint32_t w = 0xffffffffu;
      if (pv) {
        w = 0;
        for (int e = 0; e < 32; ++e) {
          const int k = c * 32 + e;
          if (k < n_keys && pv[(size_t)j * N + k] > 0) w |= 1u << e;
        }
      }
      pvbits_w[idx] = w;
    }
    // slab of K2 / V2: all 128 rows are written (zeros beyond the slab and for invalid keys).  Through the
    // copy engine: four boxes of 32 rows per tile on one mbarrier, rows of invalid keys cleared after the
    // data has landed (below); rows past the end of the matrix are zero-filled by the copy itself.
    if (p.use_tma) {
      if (tid == 0) {
        mbar_arrive_expect_tx(&bar_kv, (uint32_t)(kSlab / kTmaBoxRows) * 2u * kTmaBoxRows * 128u);
        for (int c = 0; c < kSlab / kTmaBoxRows; ++c) {  // packed: box c = the keys of head c of the CTA
          const int row0 = kPacked ? 0 : k0 + c * kTmaBoxRows, mat = kPacked ? bh0 + c : bh;
          tma_load_rows(smem + kOffK2 + c * kTmaBoxRows * 128, &p.tm_k2, row0, mat, &bar_kv);
          tma_load_rows(smem + kOffV2 + c * kTmaBoxRows * 128, &p.tm_v2, row0, mat, &bar_kv);
        }
      }
    } else {
      for (int idx = tid; idx < kSlab * 8; idx += kBwdThreads) {
        const int rr = idx >> 3, c = idx & 7;
        const int k = kPacked ? (rr & 31) : k0 + rr;  // packed: slab row 32w'+k holds key k of head w'
        const long long src = kPacked ? p.in.at(b, (bh0 - b * p.H) + (rr >> 5), k) : in_base + k * p.in.token;
        uint4 vk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
        if (k < n_keys && ((kmask[k >> 5] >> (k & 31)) & 1u)) {
          vk = __ldg(reinterpret_cast<const uint4*>(p.k2 + src) + c);
          vv = __ldg(reinterpret_cast<const uint4*>(p.v2 + src) + c);
        }
        const uint32_t off = rr * 128 + ((c ^ (rr & 7)) << 4);
        *reinterpret_cast<uint4*>(smem + kOffK2 + off) = vk;
        *reinterpret_cast<uint4*>(smem + kOffV2 + off) = vv;
      }
    }
    // P / dS tiles start as zeros: columns the element-wise pass never writes must not hold junk,
    // because the transposed products read all 128 key rows of the slab
    for (int idx = tid; idx < 4 * kTileM * 8; idx += kBwdThreads)
      *reinterpret_cast<uint4*>(smem + kOffP + idx * 16) = make_uint4(0, 0, 0, 0);
    if constexpr (kBias && !kPacked) {  // column-sum slots of warps and column halves without work stay zero
      for (int idx = tid; idx < 2 * 4 * kSlab + 2 * kTileM; idx += kBwdThreads)
        reinterpret_cast<float*>(smem + kOffDwRed)[idx] = 0.f;
    }
  }
  // Row data of the workers; loaded inside the worker branch so that it is not live where the roles split.
  uint32_t xreg[32];
  float lse2 = INFINITY, delta = 0.f;
  bool kv_ok = true;
  if (p.use_tma) {
    kv_ok = mbar_wait(&bar_kv, 0);
    if (kv_ok)
      for (int idx = tid; idx < kSlab * 8; idx += kBwdThreads) {
        const int rr = idx >> 3, c = idx & 7;
        const int k = kPacked ? (rr & 31) : k0 + rr;
        if (!(k < n_keys && ((kmask[k >> 5] >> (k & 31)) & 1u))) {
          const uint32_t off = rr * 128 + ((c ^ (rr & 7)) << 4);
          *reinterpret_cast<uint4*>(smem + kOffK2 + off) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(smem + kOffV2 + off) = make_uint4(0, 0, 0, 0);
        }
      }
  }
  fence_smem_to_async_proxy();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tmem_row = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  const uint32_t sK2 = smem_u32(smem + kOffK2), sV2 = smem_u32(smem + kOffV2);
  const uint32_t sA1 = smem_u32(smem + kOffA1), sA2 = smem_u32(smem + kOffA2);
  const uint32_t sP = smem_u32(smem + kOffP), sDS = smem_u32(smem + kOffDS);
  const uint32_t* pvbits = reinterpret_cast<const uint32_t*>(smem + kOffPv);
  float* red = reinterpret_cast<float*>(smem + kOffRed);
    const uint32_t idesc_uw = make_idesc_bf16(kTileM, kD, false, true);     // A K-major, B MN-major
  const uint32_t idesc_acc = make_idesc_bf16(kTileM, kD, true, true);     // A MN-major (transposed), B MN-major
  // 32-column chunks this thread handles; warps whose 32 rows all lie beyond the last valid query have no
  // row work at all (their rows of P and dS stay at the zeros written during set-up)
  const bool warp_live = kPacked || qt * kTileM + (warp & 3) * 32 < n_queries;
  const int nk_x = min(64, nk_pad), nk_y = nk_pad - nk_x;  // logit columns of the two halves of the slab
  const int ks_x = nk_x / 16, ks_y = nk_y / 16;
  // packed: the row's own head occupies column block hh = 2*half + group of exactly one (half, group) pair
  const bool live_x = kPacked ? (hh == grp) : (warp_live && 32 * grp < nk_x);
  const bool live_y = kPacked ? (hh == 2 + grp) : (warp_live && 32 * grp < nk_y);
  const uint32_t idesc_x = make_idesc_bf16(kTileM, nk_x, false, false);
  const uint32_t idesc_y = make_idesc_bf16(kTileM, nk_y > 0 ? nk_y : 16, false, false);

  float dq_acc[kD];

  // builds this group's scaled operand for step j into stage `st`
  auto build_operand = [&](int j, int st) {
    const __nv_bfloat16* src = (grp == 0 ? p.k1 : p.v1) + in_base + j * p.in.token;
    const uint4* kp = reinterpret_cast<const uint4*>(src);
    uint8_t* dst = smem + (grp == 0 ? kOffA1 : kOffA2) + st * (kTileM * 128) + r * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 kk = __ldg(kp + c);
      const uint32_t kw[4] = {kk.x, kk.y, kk.z, kk.w};
      uint32_t aw[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        __nv_bfloat162 m = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&xreg[4 * c + t]),
                                   *reinterpret_cast<const __nv_bfloat162*>(&kw[t]));
        aw[t] = *reinterpret_cast<uint32_t*>(&m);
      }
      *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = make_uint4(aw[0], aw[1], aw[2], aw[3]);
    }
  };
  // Low words of the operand descriptors (see make_desc_lo): built once, stepped by (bytes >> 4) per MMA.
  const uint32_t lA1_k = make_desc_lo(sA1, 0), lA2_k = make_desc_lo(sA2, 0);
  const uint32_t lK2_k = make_desc_lo(sK2, 0), lV2_k = make_desc_lo(sV2, 0);
  const uint32_t lK2_mn = make_desc_lo(sK2, kSlab * 128), lV2_mn = make_desc_lo(sV2, kSlab * 128);
  const uint32_t lDS_t = make_desc_lo(sDS, kTileM * 128), lP_t = make_desc_lo(sP, kTileM * 128);
  const uint32_t lA1_mn = make_desc_lo(sA1, kTileM * 128), lA2_mn = make_desc_lo(sA2, kTileM * 128);
  constexpr uint32_t kStage16 = (kTileM * 128) >> 4;  // one operand stage, in descriptor units
  auto issue_logits = [&](int st) {  // S and dP of the operands in stage st, one pair of tiles per half
    const uint32_t a1 = lA1_k + st * kStage16, a2 = lA2_k + st * kStage16;
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) umma_ss_lo(tmem + kColS, a1 + 2 * ks, lK2_k + 2 * ks, idesc_x, ks > 0);
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) umma_ss_lo(tmem + kColDP, a2 + 2 * ks, lV2_k + 2 * ks, idesc_x, ks > 0);
    umma_commit(&bar_sx);
    if (nk_y > 0) {  // keys 64.. of the slab: rows 64.. of the K2 / V2 tiles, columns 64.. of S / dP
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks)
        umma_ss_lo(tmem + kColS + 64, a1 + 2 * ks, lK2_k + 512 + 2 * ks, idesc_y, ks > 0);
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks)
        umma_ss_lo(tmem + kColDP + 64, a2 + 2 * ks, lV2_k + 512 + 2 * ks, idesc_y, ks > 0);
      umma_commit(&bar_sy);
    }
  };

  // ---- the step loop
  // Warps 0-7 (256 "workers", two per query row) do the row work; lane 0 of warp 8 only issues MMAs.  Issuing
  // blocks while the tensor pipe is busy, so it must not sit in a thread the others wait for.  The slab's logit
  // columns are handled as two halves, X = columns [0,64) and Y = [64,128), each with its own S / dP tiles:
  //   workers: pass over X | pass over Y | build next operands | wait U,W | drain U, W
  //   issuer :      wait X | U_X, W_X | wait Y | U_Y, W_Y, commit | dK2+=, dV2+= | wait operands | next S, dP
  // Hand-offs are mbarriers (workers arrive 256 times; the issuer signals with tcgen05.commit); after the first
  // expired wait every later wait is skipped so that all parties still leave the loop together.
  // Group g of the workers handles columns [32g, 32g+32) of each half.
  int j = 0;
  while (j < n_keys && !((kmask[j >> 5] >> (j & 31)) & 1u)) ++j;
  int st = 0;
  uint32_t phase = 0;
  bool bad = !kv_ok;
  bool first = true;
  int j_prev = -1;  // step whose column sums wait in `red` to be stored
  int step = 0;     // parity selects the `red` buffer
  // one half of the element-wise pass: P and dS of 32 columns as bf16 into shared memory (operands of the
  // transposed products) and, packed, over the S / dP columns just read (A operands of U and W)
  // bias operands and gradient sums of this thread's row (kBias)
  const size_t nn = (size_t)p.N * p.N;
  const float gate_i = (kBias && row_ok) ? p.gate[(size_t)bh * N + row] : 0.f;
  const float* u_row = kBias ? p.u + (size_t)bh * nn + (size_t)(row_ok ? row : 0) * N : nullptr;
  const float* v_row = kBias ? p.v_bias + (size_t)bh * nn + (size_t)(row_ok ? row : 0) * N : nullptr;
  float* dvb_row = reinterpret_cast<float*>(smem + kOffDvb) + r * kDvbStride;  // sum over the steps of dS of this row
  float* dwred = reinterpret_cast<float*>(smem + kOffDwRed);                   // [2][4][128], zeroed during set-up
  float* dured = reinterpret_cast<float*>(smem + kOffDuRed);                   // [2][128]
  float dgate_acc = 0.f;
  float du_step = 0.f;  // one head per tile: this thread's part of sum_k dS of the current step
  if constexpr (kBias && kPacked) {
    if (is_worker && (live_x || live_y)) {  // the thread that will form this row's dS
#pragma unroll
      for (int e = 0; e < 32; ++e) dvb_row[e] = 0.f;
    }
  }
  // the bias of this thread's 32 columns of one half of step jj: (u_ij + v_ik) + w_jk.  It does not depend on the
  // products, so it is fetched before the wait for the logits and is in registers when they arrive.
  float bsum[kBias ? 32 : 1];
  auto load_bias = [&](int half, int jj) {
    if constexpr (kBias) {
      const int col = 64 * half + 32 * grp;
      const float* w_row = p.w + (size_t)bh * nn + (size_t)jj * N;
      const float u_ij = __ldg(u_row + jj);
      const int kb = kPacked ? 0 : k0 + col;  // first key of this thread's 32 columns
      if (!kPacked && p.bias_vec4) {  // rows of v_bias and w start on 16-byte boundaries: four keys per load
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float4 vv = make_float4(0.f, 0.f, 0.f, 0.f), ww = vv;
          const bool in = kb + e < N;
          if (in) {
            vv = __ldg(reinterpret_cast<const float4*>(v_row + kb + e));
            ww = __ldg(reinterpret_cast<const float4*>(w_row + kb + e));
          }
          bsum[e] = in ? (u_ij + vv.x) + ww.x : 0.f;
          bsum[e + 1] = in ? (u_ij + vv.y) + ww.y : 0.f;
          bsum[e + 2] = in ? (u_ij + vv.z) + ww.z : 0.f;
          bsum[e + 3] = in ? (u_ij + vv.w) + ww.w : 0.f;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) bsum[e] = kb + e < N ? (u_ij + __ldg(v_row + kb + e)) + __ldg(w_row + kb + e) : 0.f;
      }
    }
  };
  auto half_pass = [&](int half, int jj) {
    const int col = 64 * half + 32 * grp;  // column inside the slab
    uint32_t s[32], dp[32];
    tmem_ld32(tmem_row + kColS + col, s);
    tmem_ld32(tmem_row + kColDP + col, dp);
    tmem_ld_wait();
    if constexpr (kBias) {
#pragma unroll
      for (int e = 0; e < 32; ++e) s[e] = __float_as_uint(fmaf(gate_i, bsum[e], __uint_as_float(s[e])));
    }
    const int wi = kPacked ? 0 : (k0 + col) >> 5;  // packed: the block's 32 columns are keys 0..31 of the row's head
    const uint32_t word = kmask[MF_IDX(wi, kMaskWords, p.status)] & pvbits[MF_IDX(jj * kMaskWords + wi, kMaxKeys * kMaskWords, p.status)];
    uint8_t* prow = smem + kOffP + half * (kTileM * 128) + r * 128;
    uint8_t* dsrow = smem + kOffDS + half * (kTileM * 128) + r * 128;
    uint32_t pk[16], dk[16];
    float dsum = 0.f;                  // kBias: sum_k dS of the row (du_ij)
    float gds[kBias ? 32 : 1];         // kBias: gate_i dS per key, for the column sums over the head's rows (dw_jk)
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {  // 8 columns = one 16-byte chunk at a time
      uint32_t* pw = pk + 4 * q4;
      uint32_t* dw = dk + 4 * q4;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int e = 8 * q4 + 2 * t;
        float p0 = fast_exp2(fmaf(__uint_as_float(s[e]), kLog2e, -lse2));
        float p1 = fast_exp2(fmaf(__uint_as_float(s[e + 1]), kLog2e, -lse2));
        if (word != 0xffffffffu) {
          p0 = ((word >> e) & 1u) ? p0 : 0.f;
          p1 = ((word >> (e + 1)) & 1u) ? p1 : 0.f;
        }
        const float d0 = p0 * (__uint_as_float(dp[e]) - delta);
        const float d1 = p1 * (__uint_as_float(dp[e + 1]) - delta);
        if constexpr (kBias) {
          dsum += d0 + d1;
          dgate_acc = fmaf(d0, bsum[e], fmaf(d1, bsum[e + 1], dgate_acc));
          if constexpr (kPacked) {
            dvb_row[e] += d0;
            dvb_row[e + 1] += d1;
          }
          gds[e] = gate_i * d0;
          gds[e + 1] = gate_i * d1;
        }
        pw[t] = pack_bf16x2(p0, p1);
        dw[t] = pack_bf16x2(d0, d1);
      }
      const int cc = 4 * grp + q4;  // 16-byte chunk index inside the 128-byte row
      const uint32_t off = (cc ^ (r & 7)) << 4;
      *reinterpret_cast<uint4*>(prow + off) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
      *reinterpret_cast<uint4*>(dsrow + off) = make_uint4(dw[0], dw[1], dw[2], dw[3]);
    }
    tmem_st16(tmem_row + kColS + col, pk);
    tmem_st16(tmem_row + kColDP + col, dk);
    if constexpr (kBias && kPacked) {
      if (row_ok && p.du) p.du[(size_t)bh * nn + (size_t)row * N + jj] = gate_i * dsum;
      const float tot = warp_column_sums32(gds, lane);  // the warp's lanes are the 32 queries of this head
      if (lane < N && p.dw) p.dw[(size_t)bh * nn + (size_t)jj * N + lane] = tot;
    }
    if constexpr (kBias && !kPacked) {
      du_step += dsum;
      const int kb = k0 + col;
      if (row_ok && p.dv_bias) {  // dv_bias[i, k] += gate_i dS: this thread is the only writer of its 32 addresses
        float* dst = p.dv_bias + (size_t)bh * nn + (size_t)row * N + kb;
        if (p.dv_vec4) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            if (kb + e < N) red_add4(dst + e, gds[e], gds[e + 1], gds[e + 2], gds[e + 3]);
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (kb + e < N) red_add(dst + e, gds[e]);
        }
      }
      const float tot = warp_column_sums32(gds, lane);  // over the warp's 32 rows; lane = column
      dwred[(step & 1) * 512 + (warp & 3) * kSlab + col + lane] = tot;
    }
  };
  // packed: the 32 columns of another head in this row: zero probabilities over the cross-head logits (the
  // shared-memory copies of P and dS keep the zeros written during set-up)
  auto zero_pass = [&](int half) {
    const int col = 64 * half + 32 * grp;
    uint32_t zero16[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) zero16[e] = 0u;
    tmem_st16(tmem_row + kColS + col, zero16);
    tmem_st16(tmem_row + kColDP + col, zero16);
  };
  // U += dS.K2 and W += P.V2 over the keys of one half; A operands from tensor memory
  auto issue_uw = [&](int half, int ks_count) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)  // 16 keys = 8 packed columns; keys 32.. of a half sit 32 columns further
      if (ks < ks_count)
        umma_ts_lo(tmem + kColU, tmem + kColDP + 64 * half + 32 * (ks >> 1) + 8 * (ks & 1),
                   lK2_mn + 128 * (4 * half + ks), idesc_uw, half > 0 || ks > 0);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      if (ks < ks_count)
        umma_ts_lo(tmem + kColWb, tmem + kColS + 64 * half + 32 * (ks >> 1) + 8 * (ks & 1),
                   lV2_mn + 128 * (4 * half + ks), idesc_uw, half > 0 || ks > 0);
  };
  // the column sums of step jj wait in red[buf]; 64 threads of each group add the four warp partials
  auto store_column_sums = [&](int jj, int buf) {
    if (kPacked) {  // one head per warp: nothing to add, two of the 4 x 64 sums per thread
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int w = (r >> 6) + 2 * t, d = r & 63;
        const float tot = red[MF_IDX((buf & 1) * 512 + (grp * 4 + w) * 64 + d, 1024, p.status)];
        (grp == 0 ? p.gk1 : p.gv1)[p.in.at(b, bh0 - b * p.H + w, jj) + d] = __float2bfloat16_rn(tot);
      }
    } else if (r < 64) {
      const float* rp = red + (buf & 1) * 512 + (grp * 4) * 64 + r;
      const float tot = (rp[0] + rp[64]) + (rp[128] + rp[192]);
      float* dst = (grp == 0 ? p.dk1_part : p.dv1_part) + (size_t)(qt * p.slabs + slab) * p.part_stride + base +
                   (size_t)jj * kD + r;
      *dst = tot;
    }
  };

  auto wait_on = [&](uint64_t* bar, uint32_t ph) {
    if (!bad) bad = !mbar_wait(bar, ph);
  };
  // Registers: 384 threads start with 168 each (three warps per scheduler).  The third warp group (the issuing
  // warp and three idle ones) drops to 56 and the eight worker warps take the 4 x 112 registers it frees:
  // 8 x 224 + 4 x 56 = 12 x 168.  Register hand-over works per warp group, hence the idle warps.  Everything
  // the workers do from here on, including the epilogue, stays inside their branch so that it may use the
  // larger budget.
  if (warp >= 8) {
    // ------------------------------------------------------------------ issuer
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (tid == kIssuerThread) {
      if (j < n_keys) {  // first step's operands
        wait_on(&bar_a0, 0);
        tc_fence_after_sync();
        issue_logits(0);
      }
      while (j < n_keys) {
        int jn = j + 1;
        while (jn < n_keys && !((kmask[jn >> 5] >> (jn & 31)) & 1u)) ++jn;
        wait_on(&bar_px, phase);
        tc_fence_after_sync();
        issue_uw(0, ks_x);
        if (nk_y > 0) {
          wait_on(&bar_py, phase);
          tc_fence_after_sync();
          issue_uw(1, ks_y);
        }
        umma_commit(&bar_uw);  // the drain only needs U and W; the accumulated transposed products run behind it
        {
          const uint32_t b1 = lA1_mn + st * kStage16, b2 = lA2_mn + st * kStage16;
#pragma unroll
          for (int ks = 0; ks < kTileM / 16; ++ks)  // K runs over the 128 query rows
            umma_ss_lo(tmem + kColDK2, lDS_t + 128 * ks, b1 + 128 * ks, idesc_acc, !(first && ks == 0));
#pragma unroll
          for (int ks = 0; ks < kTileM / 16; ++ks)
            umma_ss_lo(tmem + kColDV2, lP_t + 128 * ks, b2 + 128 * ks, idesc_acc, !(first && ks == 0));
        }
        first = false;
        if (jn < n_keys) {
          wait_on(&bar_a, phase);  // next operands built, and every worker is done reading S / dP
          tc_fence_after_sync();
          issue_logits(st ^ 1);
        }
        phase ^= 1u;
        j = jn;
        st ^= 1;
      }
      umma_commit(&bar_fin);
    }
  } else {
    // ------------------------------------------------------------------ workers
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // this thread's row of q (group 0) or dO (group 1) as 32 bf16x2 words
    {
      const __nv_bfloat16* src = grp == 0 ? p.q + in_base + row * p.in.token : p.grad_out + p.act.at(b, h, row);
      const uint4* xp = reinterpret_cast<const uint4*>(src);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row_ok) v = __ldg(xp + c);
        xreg[4 * c + 0] = v.x;
        xreg[4 * c + 1] = v.y;
        xreg[4 * c + 2] = v.z;
        xreg[4 * c + 3] = v.w;
      }
      if (grp == 0 && p.q_scale != 1.f) {
        const __nv_bfloat162 sc = __float2bfloat162_rn(p.q_scale);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const __nv_bfloat162 t = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&xreg[c]), sc);
          xreg[c] = *reinterpret_cast<const uint32_t*>(&t);
        }
      }
    }
    // exp2(S log2e - lse log2e); an invalid row keeps +inf so that every probability is 0
    if (row_ok) {
      lse2 = p.lse[(size_t)bh * N + row] * kLog2e;
      delta = p.delta[(size_t)bh * N + row];
    }
#pragma unroll
    for (int d = 0; d < kD; ++d) dq_acc[d] = 0.f;
    if (j < n_keys) {  // first step's operands
      build_operand(j, 0);
      fence_smem_to_async_proxy();
      tc_fence_before_sync();
      mbar_arrive(&bar_a0);
    }
    while (j < n_keys) {
      int jn = j + 1;
      while (jn < n_keys && !((kmask[jn >> 5] >> (jn & 31)) & 1u)) ++jn;
      if (lane == 0 && jn < n_keys) {  // the rows scaled into the next operands: one 128-byte line each
        const __nv_bfloat16* nxt = (grp == 0 ? p.k1 : p.v1) + in_base + jn * p.in.token;
        asm volatile("prefetch.global.L1 [%0];" ::"l"(nxt));
      }
      if (live_x) load_bias(0, j);
      wait_on(&bar_sx, phase);
      tc_fence_after_sync();
      du_step = 0.f;
      if (live_x) half_pass(0, j);
      else if (kPacked) zero_pass(0);
      if constexpr (kBias && !kPacked) {  // the other column half's part of du_ij, read after this step's arrivals
        if (grp == 1) dured[(step & 1) * kTileM + r] = du_step;
      }
      tmem_st_wait();
      fence_smem_to_async_proxy();
      tc_fence_before_sync();  // also orders the previous drain's reads of U, W before the products issued next
      mbar_arrive(&bar_px);
      if (nk_y > 0) {
        if (live_y) load_bias(1, j);
        wait_on(&bar_sy, phase);
        tc_fence_after_sync();
        if (live_y) half_pass(1, j);
        else if (kPacked) zero_pass(1);
        if constexpr (kBias && !kPacked) {
          if (grp == 1) dured[(step & 1) * kTileM + r] = du_step;
        }
        tmem_st_wait();
        fence_smem_to_async_proxy();
        tc_fence_before_sync();
        mbar_arrive(&bar_py);
      }
      if (jn < n_keys) {
        build_operand(jn, st ^ 1);
        fence_smem_to_async_proxy();
        tc_fence_before_sync();
        mbar_arrive(&bar_a);
      }
      const uint4* k1p = reinterpret_cast<const uint4*>(p.k1 + in_base + j * p.in.token);
      wait_on(&bar_uw, phase);
      tc_fence_after_sync();
      phase ^= 1u;
      // U, W of this step exist, so every worker has passed its arrivals of this step and thereby finished the
      // previous drain: the previous step's column sums are complete in `red` (other buffer than this step's)
      if (j_prev >= 0) store_column_sums(j_prev, step ^ 1);
      if constexpr (kBias && !kPacked) {
        // likewise this step's sums of dS: every worker wrote its parts before the arrivals that U and W waited for
        if (grp == 0) {
          const float* dr = dwred + (step & 1) * 512 + r;
          const float tot = (dr[0] + dr[kSlab]) + (dr[2 * kSlab] + dr[3 * kSlab]);
          if (k0 + r < N && p.dw) atomicAdd(p.dw + (size_t)bh * nn + (size_t)j * N + k0 + r, tot);  // <= 2 query tiles
          const float du_ij = du_step + dured[(step & 1) * kTileM + r];
          if (row_ok && p.du) atomicAdd(p.du + (size_t)bh * nn + (size_t)row * N + j, gate_i * du_ij);  // <= 2 key slabs
        }
      }
      // ---- drain: group 0 reads U (dq, dk1_j), group 1 reads W (dv1_j)
      float* red_j = red + (step & 1) * 512;
      if (!warp_live) {
        *reinterpret_cast<float2*>(red_j + warp * 64 + 2 * lane) = make_float2(0.f, 0.f);
      } else {
        float cvec[64];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t w[32];
          tmem_ld32(tmem_row + (grp == 0 ? kColU : kColWb) + 32 * half, w);
          uint4 k1w[4];  // k1_j, the 32 columns of this half (group 0 only)
          if (grp == 0) {
#pragma unroll
            for (int c = 0; c < 4; ++c) k1w[c] = __ldg(k1p + 4 * half + c);
          }
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const int d = 32 * half + 2 * t;
            const uint32_t xw = xreg[d >> 1];
            const float x_lo = __uint_as_float(xw << 16), x_hi = __uint_as_float(xw & 0xffff0000u);
            const float u0 = __uint_as_float(w[2 * t]), u1 = __uint_as_float(w[2 * t + 1]);
            cvec[d] = x_lo * u0;
            cvec[d + 1] = x_hi * u1;
            if (grp == 0) {
              const uint4 kq = k1w[(d >> 3) & 3];
              const uint32_t kwv[4] = {kq.x, kq.y, kq.z, kq.w};
              const uint32_t kw = kwv[(d >> 1) & 3];
              dq_acc[d] = fmaf(u0, __uint_as_float(kw << 16), dq_acc[d]);
              dq_acc[d + 1] = fmaf(u1, __uint_as_float(kw & 0xffff0000u), dq_acc[d + 1]);
            }
          }
        }
        float c0, c1;
        warp_column_sums(cvec, lane, c0, c1);
        *reinterpret_cast<float2*>(red_j + warp * 64 + 2 * lane) = make_float2(c0, c1);
      }
      first = false;
      j_prev = j;
      step ^= 1;
      j = jn;
      st ^= 1;
    }
    if (j_prev >= 0) {
      asm volatile("bar.sync 1, 256;" ::: "memory");  // every worker's last column sums are in `red`
      store_column_sums(j_prev, step ^ 1);
    }
    // ---- epilogue: the last step's accumulated products are still in flight (the issuer committed bar_fin)
    wait_on(&bar_fin, 0);
    tc_fence_after_sync();
    if constexpr (kBias && !kPacked) {  // the two column halves' parts of dgate_i meet in shared memory
      if (grp == 1) dured[r] = dgate_acc;
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    if (bad) {
      atomicExch(p.status, MF_ERR_DEVICE_TIMEOUT);
    } else {
      if constexpr (kBias && !kPacked) {
        if (grp == 0 && row_ok && p.dgate) atomicAdd(p.dgate + (size_t)bh * N + row, dgate_acc + dured[r]);  // <= 2 key slabs
      }
      if constexpr (kBias && kPacked) {
        if ((live_x || live_y) && row_ok) {  // the thread that formed this row's dS
          if (p.dv_bias)
            for (int e = 0; e < N && e < 32; ++e) p.dv_bias[(size_t)bh * nn + (size_t)row * N + e] = gate_i * dvb_row[e];
          if (p.dgate) p.dgate[(size_t)bh * N + row] = dgate_acc;
        }
      }
      if constexpr (kPacked) {
        // rows of first keys that no step visited: zeros (same thread-to-element mapping as store_column_sums)
        for (int jj = 0; jj < N; ++jj) {
          if ((kmask[jj >> 5] >> (jj & 31)) & 1u) continue;  // uniform
#pragma unroll
          for (int t = 0; t < 2; ++t)
            (grp == 0 ? p.gk1 : p.gv1)[p.in.at(b, bh0 - b * p.H + (r >> 6) + 2 * t, jj) + (r & 63)] = __float2bfloat16_rn(0.f);
        }
        if (grp == 0 && row < N) {
          const float sc = row_ok ? p.q_scale : 0.f;
          uint4* dst = reinterpret_cast<uint4*>(p.gq + p.in.at(b, h, row));
#pragma unroll
          for (int c = 0; c < kD / 8; ++c)
            dst[c] = make_uint4(pack_bf16x2(dq_acc[8 * c] * sc, dq_acc[8 * c + 1] * sc),
                                pack_bf16x2(dq_acc[8 * c + 2] * sc, dq_acc[8 * c + 3] * sc),
                                pack_bf16x2(dq_acc[8 * c + 4] * sc, dq_acc[8 * c + 5] * sc),
                                pack_bf16x2(dq_acc[8 * c + 6] * sc, dq_acc[8 * c + 7] * sc));
        }
      } else if (grp == 0 && row < N) {
        float4* dst = reinterpret_cast<float4*>(p.dq_part + (size_t)slab * p.part_stride + base + (size_t)row * kD);
#pragma unroll
        for (int c = 0; c < kD / 4; ++c)
          dst[c] = make_float4(dq_acc[4 * c], dq_acc[4 * c + 1], dq_acc[4 * c + 2], dq_acc[4 * c + 3]);
      }
      // accumulators: lane r of tensor memory = key k0 + r; group 0 stores dK2, group 1 dV2
      const int k = kPacked ? (r & 31) : k0 + r;  // packed: lane 32w+k = key k of head w, this thread's own head
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t w[32];
        tmem_ld32(tmem_row + (grp == 0 ? kColDK2 : kColDV2) + 32 * half, w);
        tmem_ld_wait();
        if constexpr (kPacked) {
          if (k < N) {
            const bool live = !first && k < n_keys && ((kmask[k >> 5] >> (k & 31)) & 1u);
            uint4* dst = reinterpret_cast<uint4*>((grp == 0 ? p.gk2 : p.gv2) + p.in.at(b, h, k) + 32 * half);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 o = make_uint4(0, 0, 0, 0);
              if (live)
                o = make_uint4(pack_bf16x2(__uint_as_float(w[8 * c]), __uint_as_float(w[8 * c + 1])),
                               pack_bf16x2(__uint_as_float(w[8 * c + 2]), __uint_as_float(w[8 * c + 3])),
                               pack_bf16x2(__uint_as_float(w[8 * c + 4]), __uint_as_float(w[8 * c + 5])),
                               pack_bf16x2(__uint_as_float(w[8 * c + 6]), __uint_as_float(w[8 * c + 7])));
              dst[c] = o;
            }
          }
        } else if (k < n_keys && !first) {
          float4* dst = reinterpret_cast<float4*>((grp == 0 ? p.dk2_part : p.dv2_part) + (size_t)qt * p.part_stride +
                                                  base + (size_t)k * kD + 32 * half);
#pragma unroll
          for (int c = 0; c < 8; ++c)
            dst[c] = make_float4(__uint_as_float(w[4 * c]), __uint_as_float(w[4 * c + 1]),
                                 __uint_as_float(w[4 * c + 2]), __uint_as_float(w[4 * c + 3]));
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kBwdTmemCols);
}

// Four heads per tile: the gradients are final when the main kernel ends; only after an expired device-side wait
// (status word set) are they all overwritten with zeros, as the finalize kernel does for the other shapes.
__global__ void simplicial_bwd_zero_on_error_kernel(BwdParams p, int BH) {
  if (p.status[0] == 0) return;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 8 elements
  if (idx >= (long long)BH * p.N * (kD / 8)) return;
  const int row = (int)((idx / (kD / 8)) % p.N), bh = (int)(idx / ((long long)(kD / 8) * p.N));
  const long long off = p.in.at(bh / p.H, bh % p.H, row) + 8 * (idx % (kD / 8));
  const uint4 z = make_uint4(0, 0, 0, 0);
  *reinterpret_cast<uint4*>(p.gq + off) = z;
  *reinterpret_cast<uint4*>(p.gk1 + off) = z;
  *reinterpret_cast<uint4*>(p.gv1 + off) = z;
  *reinterpret_cast<uint4*>(p.gk2 + off) = z;
  *reinterpret_cast<uint4*>(p.gv2 + off) = z;
}

// Sums the partials in a fixed order and writes the five gradients in bf16; rows of padded
// tokens (and of keys that take part in no pair) get exact zeros.
__global__ void simplicial_bwd_finalize_kernel(BwdParams p, __nv_bfloat16* __restrict__ dq,
                                               __nv_bfloat16* __restrict__ dk1, __nv_bfloat16* __restrict__ dv1,
                                               __nv_bfloat16* __restrict__ dk2, __nv_bfloat16* __restrict__ dv2,
                                               int BH) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 4 elements
  const long long total = (long long)BH * p.N * (kD / 4);
  if (idx >= total) return;
  const int d4 = (int)(idx % (kD / 4));
  const int row = (int)((idx / (kD / 4)) % p.N);
  const int bh = (int)(idx / ((long long)(kD / 4) * p.N));
  const int b = bh / p.H;
  const int n_keys = p.info[b].n_keys, n_queries = p.info[b].n_queries;
  const int nqt = (n_queries + kTileM - 1) / kTileM, nsl = (n_keys + kSlab - 1) / kSlab;
  const size_t off = ((size_t)bh * p.N + row) * kD + 4 * d4;             // in the partial planes
  const long long dst = p.in.at(b, bh - b * p.H, row) + 4 * d4;          // in the gradient tensors
  const bool sane = p.status[0] == 0;  // after an expired device-side wait every gradient is written as zeros
  const bool q_ok = sane && row < n_queries && p.query_valid[(size_t)b * p.N + row] > 0 && n_keys > 0;
  const bool k_ok = sane && row < n_keys && p.key_valid[(size_t)b * p.N + row] > 0 && n_queries > 0;
  auto add4 = [](float4& a, const float4 v) {
    a.x += v.x;
    a.y += v.y;
    a.z += v.z;
    a.w += v.w;
  };
  auto store4 = [](__nv_bfloat16* dst, const float4 v) {
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dst) = o;
  };
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  if (q_ok)
    for (int s = 0; s < nsl; ++s) add4(a, *reinterpret_cast<const float4*>(p.dq_part + (size_t)s * p.part_stride + off));
  a.x *= p.q_scale, a.y *= p.q_scale, a.z *= p.q_scale, a.w *= p.q_scale;
  store4(dq + dst, a);
  float4 k2v = make_float4(0.f, 0.f, 0.f, 0.f), v2v = k2v, k1v = k2v, v1v = k2v;
  if (k_ok) {
    for (int t = 0; t < nqt; ++t) {
      add4(k2v, *reinterpret_cast<const float4*>(p.dk2_part + (size_t)t * p.part_stride + off));
      add4(v2v, *reinterpret_cast<const float4*>(p.dv2_part + (size_t)t * p.part_stride + off));
      for (int s = 0; s < nsl; ++s) {
        add4(k1v, *reinterpret_cast<const float4*>(p.dk1_part + (size_t)(t * p.slabs + s) * p.part_stride + off));
        add4(v1v, *reinterpret_cast<const float4*>(p.dv1_part + (size_t)(t * p.slabs + s) * p.part_stride + off));
      }
    }
  }
  store4(dk2 + dst, k2v);
  store4(dv2 + dst, v2v);
  store4(dk1 + dst, k1v);
  store4(dv1 + dst, v1v);
}

struct BwdLayout {
  size_t info, order, delta, dq, dk2, dv2, dk1, dv1, total;
};

BwdLayout bwd_layout(int B, int H, int N) {
  BwdLayout l{};
  const int q_tiles = (N + kTileM - 1) / kTileM, slabs = (N + kSlab - 1) / kSlab;
  const size_t part = align_up((size_t)B * H * N * kD * sizeof(float), 256);
  size_t off = kStatusBytes;
  l.info = off;
  off += align_up((size_t)B * sizeof(BatchInfo), 256);
  l.order = off;
  off += align_up((size_t)B * sizeof(int32_t), 256);
  l.delta = off;
  off += align_up((size_t)B * H * N * sizeof(float), 256);
  l.dq = off;
  off += part * slabs;
  l.dk2 = off;
  off += part * q_tiles;
  l.dv2 = off;
  off += part * q_tiles;
  l.dk1 = off;
  off += part * q_tiles * slabs;
  l.dv1 = off;
  off += part * q_tiles * slabs;
  l.total = off;
  return l;
}

}  // namespace

size_t simplicial_sm100_bwd_workspace_bytes(const MfSimplicialBwdArgs& a) {
  return bwd_layout(a.batch, a.heads, a.tokens).total;
}

int simplicial_sm100_bwd(const MfSimplicialBwdArgs& a, cudaStream_t stream) {
  return simplicial_sm100_bwd_layouts(a, nullptr, stream);
}

int simplicial_sm100_bwd_layouts(const MfSimplicialBwdArgs& a, const TileLayouts* layouts, cudaStream_t stream) {
  const BwdLayout l = bwd_layout(a.batch, a.heads, a.tokens);
  char* ws = static_cast<char*>(a.workspace);
  const int BH = a.batch * a.heads;
  BwdParams p{};
  p.grad_out = static_cast<const __nv_bfloat16*>(a.grad_out);
  p.q = static_cast<const __nv_bfloat16*>(a.q);
  p.k1 = static_cast<const __nv_bfloat16*>(a.k1);
  p.v1 = static_cast<const __nv_bfloat16*>(a.v1);
  p.k2 = static_cast<const __nv_bfloat16*>(a.k2);
  p.v2 = static_cast<const __nv_bfloat16*>(a.v2);
  p.lse = a.lse;
  p.query_valid = a.query_valid;
  p.key_valid = a.pair_key_valid;
  p.pair_valid = a.pair_valid;
  p.status = reinterpret_cast<int32_t*>(ws);
  p.in = p.act = contiguous_rows(a.heads, a.tokens);
  p.q_scale = 1.f;
  p.u = a.u, p.v_bias = a.v_bias, p.w = a.w, p.gate = a.gate;
  p.du = a.du, p.dv_bias = a.dv_bias, p.dw = a.dw, p.dgate = a.dgate;
  p.gq = static_cast<__nv_bfloat16*>(a.dq), p.gk1 = static_cast<__nv_bfloat16*>(a.dk1);
  p.gv1 = static_cast<__nv_bfloat16*>(a.dv1), p.gk2 = static_cast<__nv_bfloat16*>(a.dk2);
  p.gv2 = static_cast<__nv_bfloat16*>(a.dv2);
  if (layouts) {  // rows that are not (B,H,N,D) contiguous come by plain loads: the tensor maps describe that form only
    p.in = layouts->in, p.act = layouts->act, p.q_scale = layouts->q_scale;
    p.use_tma = 0;
  } else {
    p.use_tma = make_rows_tensor_map(&p.tm_k2, a.k2, a.tokens, BH) && make_rows_tensor_map(&p.tm_v2, a.v2, a.tokens, BH);
  }
  BatchInfo* info = reinterpret_cast<BatchInfo*>(ws + l.info);
  int32_t* order = reinterpret_cast<int32_t*>(ws + l.order);
  float* delta = reinterpret_cast<float*>(ws + l.delta);
  p.info = info;
  p.order = order;
  p.delta = delta;
  p.dq_part = reinterpret_cast<float*>(ws + l.dq);
  p.dk2_part = reinterpret_cast<float*>(ws + l.dk2);
  p.dv2_part = reinterpret_cast<float*>(ws + l.dv2);
  p.dk1_part = reinterpret_cast<float*>(ws + l.dk1);
  p.dv1_part = reinterpret_cast<float*>(ws + l.dv1);
  p.H = a.heads;
  p.N = a.tokens;
  p.q_tiles = (a.tokens + kTileM - 1) / kTileM;
  p.slabs = (a.tokens + kSlab - 1) / kSlab;
  p.part_stride = align_up((size_t)BH * a.tokens * kD * sizeof(float), 256) / sizeof(float);

  int rc = launch_schedule(a.query_valid, a.pair_key_valid, a.batch, a.tokens, info, order, p.status, stream);
  if (rc != MF_OK) return rc;
  const int rows = BH * a.tokens;
  delta_bf16_kernel<float><<<(rows + 7) / 8, 256, 0, stream>>>(p.grad_out, p.act, a.heads, a.tokens, a.out, delta, rows);
  MF_CHECK_LAUNCH("delta_bf16_kernel");
  const bool packed = simplicial_sm100_packs_heads(a.tokens, a.heads);
  const bool bias = a.u != nullptr;
  p.dv_vec4 = bias && a.dv_bias && a.tokens % 4 == 0 && reinterpret_cast<uintptr_t>(a.dv_bias) % 16 == 0;
  p.bias_vec4 = bias && a.tokens % 4 == 0 && reinterpret_cast<uintptr_t>(a.v_bias) % 16 == 0 &&
                reinterpret_cast<uintptr_t>(a.w) % 16 == 0;
  auto kern = bias ? (packed ? simplicial_bwd_sm100_kernel<true, true> : simplicial_bwd_sm100_kernel<false, true>)
                   : (packed ? simplicial_bwd_sm100_kernel<true, false> : simplicial_bwd_sm100_kernel<false, false>);
  const int smem_alloc = bias ? kSmemBwdBiasAlloc : kSmemBwdAlloc;
  {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_alloc);
    if (e != cudaSuccess) return cuda_error(e, "cudaFuncSetAttribute(simplicial_bwd_sm100_kernel)");
  }
  const long long blocks = packed ? (long long)a.batch * (a.heads / 4) : (long long)BH * p.q_tiles * p.slabs;
  profile_mark(MF_PROFILE_SIMPLICIAL_BWD, true, stream);
  kern<<<(unsigned)blocks, kBwdThreads, smem_alloc, stream>>>(p);
  profile_mark(MF_PROFILE_SIMPLICIAL_BWD, false, stream);
  MF_CHECK_LAUNCH("simplicial_bwd_sm100_kernel");
  if (packed) {
    const long long total8 = (long long)rows * (kD / 8);
    simplicial_bwd_zero_on_error_kernel<<<(unsigned)((total8 + 255) / 256), 256, 0, stream>>>(p, BH);
    MF_CHECK_LAUNCH("simplicial_bwd_zero_on_error_kernel");
    return MF_OK;
  }
  const long long total4 = (long long)rows * (kD / 4);
  simplicial_bwd_finalize_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, stream>>>(
      p, static_cast<__nv_bfloat16*>(a.dq), static_cast<__nv_bfloat16*>(a.dk1), static_cast<__nv_bfloat16*>(a.dv1),
      static_cast<__nv_bfloat16*>(a.dk2), static_cast<__nv_bfloat16*>(a.dv2), BH);
  MF_CHECK_LAUNCH("simplicial_bwd_finalize_kernel");
  return MF_OK;
}

}  // namespace mf
