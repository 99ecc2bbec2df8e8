// Backward pass of 2-simplicial attention on the Blackwell tensor cores, row-packed.
//
// One CTA owns one (batch, head) and one slab of at most 128 keys of the second key set (index k).  Every row
// of its 128-row tile carries its own (query i, first key j) pair (see simplicial_rows.cuh); the CTA walks over
// all query ranges of the molecule and, inside a range, over groups of first keys.  Per step, with
//   A1[r,:] = q[i_r,:] o k1[j_r,:]   and   A2[r,:] = dO[i_r,:] o v1[j_r,:]     (rewritten into shared memory)
// seven GEMMs run on tcgen05 with fp32 accumulators in tensor memory:
//   S   = A1 . K2^T            logits (recomputed)
//   dP  = A2 . V2^T            d(out)/d(prob)
//   U   = dS . K2              -> dq[i_r] += U[r] o k1[j_r]        (registers of both groups; rows of one query merged per range)
//   W   = P  . V2
//   dK2 += dS^T . A1           accumulated in tensor memory over every step and every query range
//   dV2 += P^T  . A2           likewise
//   D   = [q o U | dO o W]^T . Sel^T   column sums per group of rows: dk1[j_g] and dv1[j_g]
// with P = exp(S - lse_i), dS = P o (dP - delta_i), delta_i = dO_i . out_i.  The first six are the products of
// the reference's backward kernel (src/matterformer/models/triton_simplicial_attention.py:553,611,626,627,644,
// 645); the seventh replaces a cross-lane reduction: the element-wise products q o U and dO o W go to shared
// memory as bf16 and a GEMM against a 0/1 selector sums the rows of each group (M = 128 output columns,
// N = 16 groups, K = 128 rows), so the column sums of a step cost one narrow MMA instead of a shuffle tree.
//
// dK2 / dV2 leave the CTA as final bf16 rows (no other CTA contributes to them).  dq and dk1 / dv1 are written
// as fp32 partials per key slab and summed in a fixed order by the finalize kernel; within a CTA dk1 / dv1
// partials are accumulated over the query ranges by plain read-modify-write of addresses only this CTA
// touches.  There are no floating-point atomics: gradients are bit-identical from run to run.
//
// Threads: 384.  Warps 0-3 hold the q rows (build A1, drain U), warps 4-7 the dO rows (build A2, drain W); both
// form P and dS, each on every other 32-column chunk; one thread of warp 8 issues every tcgen05.mma; warp 9
// runs ahead and stages the k1 / v1 rows of the coming steps in shared memory, so that no worker waits on a
// global load.  The element-wise pass handles the slab as two halves of 64 logit columns so that U and W of the
// first half are issued while the second is still being processed.  Hand-offs are mbarriers (one elected lane
// per warp arrives); every wait is bounded and an expired wait is reported through the status word.
#include "common.cuh"
#include "simplicial.cuh"
#include "simplicial_rows.cuh"
#include "simplicial_sm100.cuh"
#include "sm100_primitives.cuh"
#include "tensor_map.cuh"

namespace mf {
namespace {

constexpr int kSlab = 128;          // keys of the second set per CTA (at most)
constexpr int kBwdThreads = 384;  // 8 worker warps + one warp group that holds the issuing warp
constexpr int kBwdIssuer = 256;
constexpr int kBwdTmemCols = 512;
constexpr int kColS = 0;            // S    [0,128): half X = [0,64), half Y = [64,128)
constexpr int kColDP = 128;         // dP   [128,256)
constexpr int kColU = 256;          // U    [256,320)
constexpr int kColWb = 320;         // W    [320,384)
constexpr int kColDK2 = 384;        // dK2  [384,448)
constexpr int kColDV2 = 448;        // dV2  [448,512)
constexpr int kColD = kColS + 16;   // column sums: 16 columns left free by the packed probabilities of chunk 0
constexpr int kMaskWords = kMaxKeys / 32;

// shared memory map (dynamic, 1024-byte aligned)
constexpr int kOffK2 = 0;                          // [128][64] bf16 swizzled: slab of K2
constexpr int kOffV2 = kOffK2 + kSlab * 128;       // [128][64]            : slab of V2
constexpr int kOffA1 = kOffV2 + kSlab * 128;       // 2 stages x [128][64] : q_i o k1_j per row
constexpr int kOffA2 = kOffA1 + 2 * kTileM * 128;  // 2 stages x [128][64] : dO_i o v1_j per row
constexpr int kOffP = kOffA2 + 2 * kTileM * 128;   // 2 halves x [128][64] : P
constexpr int kOffDS = kOffP + 2 * kTileM * 128;   // 2 halves x [128][64] : dS
constexpr int kOffX = kOffDS + 2 * kTileM * 128;   // [128][64] q o U, then [128][64] dO o W
constexpr int kOffSel = kOffX + 2 * kTileM * 128;  // [16][128] bf16 swizzled: Sel[g][r] = 1 iff row r belongs to group g
constexpr int kRowStages = 4;                      // steps the loader warp may run ahead
constexpr int kOffRows = kOffSel + 16 * 256;       // 4 stages x {k1, v1} x [8][64] bf16: rows of a step's first keys
constexpr int kOffK1f = kOffRows + kRowStages * 2 * kMaxGroups * kD * 2;  // 4 stages x [8][64] fp32: the k1 rows again
constexpr int kOffPv = kOffK1f + kRowStages * kMaxGroups * kD * 4;        // [192][6] pair_valid bit rows
constexpr int kSmemBytes = kOffPv + kMaxKeys * kMaskWords * 4;
constexpr int kSmemAlloc = kSmemBytes + 1024;

struct RowsBwdParams {
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
  __nv_bfloat16* dk2;  // final
  __nv_bfloat16* dv2;  // final
  float* dq_part;      // [slab] x (BH, N, 64) fp32
  float* dk1_part;     // [slab]
  float* dv1_part;     // [slab]
  const BatchInfo* info;
  const int32_t* order;
  int32_t* status;
  int H, N, slabs_max;
  size_t part_stride;  // elements per partial plane
  int use_tma;
  CUtensorMap tm_k2;   // (B*H, N, 64) bf16, boxes of 32 rows, 128-byte swizzle
  CUtensorMap tm_v2;
};

// Key slabs of a molecule: equal widths, multiples of 32 so that mask words line up with 32-column chunks.
__host__ __device__ inline int slab_count(int n_keys) { return (n_keys + kSlab - 1) / kSlab; }
__host__ __device__ inline int slab_width(int n_keys) {
  const int s = slab_count(n_keys);
  return s > 0 ? (((n_keys + s - 1) / s + 31) & ~31) : 0;
}

__global__ void delta_rows_kernel(const __nv_bfloat16* __restrict__ grad_out, const float* __restrict__ out,
                                  float* __restrict__ delta, int rows) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat162 g = reinterpret_cast<const __nv_bfloat162*>(grad_out + (size_t)row * kD)[lane];
  const float2 o = reinterpret_cast<const float2*>(out + (size_t)row * kD)[lane];
  float s = fmaf(__bfloat162float(g.x), o.x, __bfloat162float(g.y) * o.y);
  s = warp_sum(s);
  if (lane == 0) delta[row] = s;
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__global__ void __maxnreg__(168) simplicial_rows_bwd_kernel(const __grid_constant__ RowsBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar_sx, bar_uw, bar_d, bar_fin;          // signalled by tcgen05.commit
  __shared__ uint64_t bar_px, bar_py, bar_a, bar_x;            // one arrival per worker warp
  __shared__ uint64_t bar_full[kRowStages], bar_empty[kRowStages];  // loader warp <-> workers
  __shared__ uint64_t bar_kv;                                   // bulk tensor copies of the K2 / V2 slab
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t kmask[kMaskWords];
  __shared__ uint8_t jlist[kMaxKeys];

  const int tid = threadIdx.x, warp = tid >> 5;
  const bool is_worker = tid < 256;
  const int grp = (tid >> 7) & 1;  // 0: q side, 1: dO side
  const int r = tid & 127;         // row of the tile
  const int per_b = p.H * p.slabs_max;
  const int b = p.order[blockIdx.x / per_b];
  const int rem = blockIdx.x % per_b;
  const int h = rem / p.slabs_max, slab = rem % p.slabs_max;
  const int N = p.N;
  const int bh = b * p.H + h;
  const size_t base = (size_t)bh * N * kD;
  const int n_keys = p.info[b].n_keys;
  const int n_queries = p.info[b].n_queries;
  const int nj = p.info[b].reserved0;  // valid first keys
  const RowPlan plan = plan_rows(n_queries, nj);
  if (plan.tiles == 0 || slab >= slab_count(n_keys)) return;  // the finalize kernel writes the zeros
  const int slab_w = slab_width(n_keys);
  const int k0 = slab * slab_w;                     // first key of the slab (multiple of 32)
  const int nk_slab = min(slab_w, n_keys - k0);     // keys in the slab
  if (nk_slab <= 0) return;
  // MMA N of the logit GEMMs: whole 32-column chunks, so that every column a worker reads has been written (keys
  // beyond the slab's last have zero K2 / V2 rows)
  const int nk_pad = (nk_slab + 31) & ~31;
  const int rt = plan.rows_per_tile, G = plan.groups, steps = plan.steps;

  if (tid == 0) {
    mbar_init(&bar_sx, 1);
    mbar_init(&bar_uw, 1);
    mbar_init(&bar_d, 1);
    mbar_init(&bar_fin, 1);
    mbar_init(&bar_px, 8);
    mbar_init(&bar_py, 8);
    mbar_init(&bar_a, 8);
    mbar_init(&bar_x, 8);
    for (int i = 0; i < kRowStages; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_empty[i], 8);
    }
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
  if (tid < kMaxKeys && ((kmask[tid >> 5] >> (tid & 31)) & 1u)) {  // compacted list of the valid first keys
    int pos = __popc(kmask[tid >> 5] & ((1u << (tid & 31)) - 1u));
    for (int c = 0; c < (tid >> 5); ++c) pos += __popc(kmask[c]);
    jlist[pos] = (uint8_t)tid;
  }
  auto key_live = [&](int rr) {  // slab row rr holds a key that takes part
    const int k = k0 + rr;
    return rr < nk_slab && ((kmask[k >> 5] >> (k & 31)) & 1u);
  };
  {
    uint32_t* pvbits_w = reinterpret_cast<uint32_t*>(smem + kOffPv);
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
    // slab of K2 / V2: all 128 rows are written (zeros beyond the slab and for invalid keys).  Through the copy
    // engine: four boxes of 32 rows per tile on one mbarrier, rows that must be zero cleared afterwards.
    if (p.use_tma) {
      if (tid == 0) {
        mbar_arrive_expect_tx(&bar_kv, (uint32_t)(kSlab / kTmaBoxRows) * 2u * kTmaBoxRows * 128u);
        for (int c = 0; c < kSlab / kTmaBoxRows; ++c) {
          tma_load_rows(smem + kOffK2 + c * kTmaBoxRows * 128, &p.tm_k2, k0 + c * kTmaBoxRows, bh, &bar_kv);
          tma_load_rows(smem + kOffV2 + c * kTmaBoxRows * 128, &p.tm_v2, k0 + c * kTmaBoxRows, bh, &bar_kv);
        }
      }
    } else {
      for (int idx = tid; idx < kSlab * 8; idx += kBwdThreads) {
        const int rr = idx >> 3, c = idx & 7;
        uint4 vk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
        if (key_live(rr)) {
          vk = __ldg(reinterpret_cast<const uint4*>(p.k2 + base + (size_t)(k0 + rr) * kD) + c);
          vv = __ldg(reinterpret_cast<const uint4*>(p.v2 + base + (size_t)(k0 + rr) * kD) + c);
        }
        const uint32_t off = rr * 128 + ((c ^ (rr & 7)) << 4);
        *reinterpret_cast<uint4*>(smem + kOffK2 + off) = vk;
        *reinterpret_cast<uint4*>(smem + kOffV2 + off) = vv;
      }
    }
    // P / dS / q o U / dO o W tiles start as zeros: rows and columns the element-wise passes never write must
    // not hold junk, because the transposed products and the column-sum product read every row
    for (int idx = tid; idx < 6 * kTileM * 8; idx += kBwdThreads)
      *reinterpret_cast<uint4*>(smem + kOffP + idx * 16) = make_uint4(0, 0, 0, 0);
    // selector: Sel[g][r] = 1 iff r / rows_per_tile == g (g < groups); 16 rows x 128 columns, two 64-column blocks
    if (tid < 256) {
      const int m = tid >> 4, cc = tid & 15;
      uint32_t wv[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int r0 = cc * 8 + 2 * t;
        const uint32_t lo = (m < G && r0 / rt == m) ? 0x3F80u : 0u;
        const uint32_t hi = (m < G && (r0 + 1) / rt == m) ? 0x3F80u : 0u;
        wv[t] = lo | (hi << 16);
      }
      uint8_t* dst = smem + kOffSel + (cc >> 3) * 2048 + m * 128 + (((cc & 7) ^ (m & 7)) << 4);
      *reinterpret_cast<uint4*>(dst) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
    }
  }
  bool bad = false;
  if (p.use_tma) {
    bad = !mbar_wait(&bar_kv, 0);
    if (!bad)
      for (int idx = tid; idx < kSlab * 8; idx += kBwdThreads) {
        const int rr = idx >> 3, c = idx & 7;
        if (!key_live(rr)) {
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
  const int nk_x = min(64, nk_pad), nk_y = nk_pad - nk_x;  // logit columns of the two halves of the slab
  const int ks_x = nk_x / 16, ks_y = nk_y / 16;

  auto wait_on = [&](uint64_t* bar, uint32_t ph) {
    if (!bad) bad = !mbar_wait(bar, ph);
  };

  // Registers: 384 threads start with 168 each (three warps per scheduler).  The third warp group (the issuing
  // warp and three idle ones) drops to 88 and the eight worker warps take what it frees: 8 x 208 + 4 x 88
  // = 12 x 168.  The hand-over works per warp group, hence the idle warps; the raise blocks until the registers
  // exist in the CTA's own pool, so the two figures must never add up to more than the launch allocation.
  static_assert(8 * 208 + 4 * 88 <= 12 * 168, "register hand-over exceeds the CTA's pool");
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
  if (tid == kBwdIssuer) {
    // ------------------------------------------------------------------ issuer
    const uint32_t sK2 = smem_u32(smem + kOffK2), sV2 = smem_u32(smem + kOffV2);
    const uint32_t lA1_k = make_desc_lo(smem_u32(smem + kOffA1), 0), lA2_k = make_desc_lo(smem_u32(smem + kOffA2), 0);
    const uint32_t lK2_k = make_desc_lo(sK2, 0), lV2_k = make_desc_lo(sV2, 0);
    const uint32_t lK2_mn = make_desc_lo(sK2, kSlab * 128), lV2_mn = make_desc_lo(sV2, kSlab * 128);
    const uint32_t lDS_t = make_desc_lo(smem_u32(smem + kOffDS), kTileM * 128);
    const uint32_t lP_t = make_desc_lo(smem_u32(smem + kOffP), kTileM * 128);
    const uint32_t lA1_mn = make_desc_lo(smem_u32(smem + kOffA1), kTileM * 128);
    const uint32_t lA2_mn = make_desc_lo(smem_u32(smem + kOffA2), kTileM * 128);
    const uint32_t lX_t = make_desc_lo(smem_u32(smem + kOffX), kTileM * 128);
    const uint32_t lSel = make_desc_lo(smem_u32(smem + kOffSel), 0);
    constexpr uint32_t kStage16 = (kTileM * 128) >> 4;  // one operand stage, in descriptor units
    const uint32_t idesc_s = make_idesc_bf16(kTileM, nk_pad, false, false);
    const uint32_t idesc_uw = make_idesc_bf16(kTileM, kD, false, true);    // A from tensor memory, B MN-major
    const uint32_t idesc_acc = make_idesc_bf16(kTileM, kD, true, true);    // A MN-major (transposed), B MN-major
    const uint32_t idesc_sum = make_idesc_bf16(kTileM, 16, true, false);   // A MN-major (transposed), B K-major
    auto issue_logits = [&](int st) {  // S and dP of the operands in stage st, the whole slab width at once
      const uint32_t a1 = lA1_k + st * kStage16, a2 = lA2_k + st * kStage16;
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) umma_ss_lo(tmem + kColS, a1 + 2 * ks, lK2_k + 2 * ks, idesc_s, ks > 0);
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) umma_ss_lo(tmem + kColDP, a2 + 2 * ks, lV2_k + 2 * ks, idesc_s, ks > 0);
      umma_commit(&bar_sx);
    };
    // U += dS.K2 and W += P.V2 over the keys of one half; A operands from tensor memory, where the packed
    // values sit over the first 16 columns of the 32-column chunk they came from
    auto issue_uw = [&](int half, int ks_count) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        if (ks < ks_count)
          umma_ts_lo(tmem + kColU, tmem + kColDP + 64 * half + 32 * (ks >> 1) + 8 * (ks & 1),
                     lK2_mn + 128 * (4 * half + ks), idesc_uw, half > 0 || ks > 0);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        if (ks < ks_count)
          umma_ts_lo(tmem + kColWb, tmem + kColS + 64 * half + 32 * (ks >> 1) + 8 * (ks & 1),
                     lV2_mn + 128 * (4 * half + ks), idesc_uw, half > 0 || ks > 0);
    };
    auto issue_sums = [&]() {  // D[c, g] = sum_r [q o U | dO o W][r, c] Sel[g, r]
#pragma unroll
      for (int ks = 0; ks < kTileM / 16; ++ks)
        umma_ss_lo(tmem + kColD, lX_t + 128 * ks, lSel + (ks < 4 ? 2 * ks : 128 + 2 * (ks - 4)), idesc_sum, ks > 0);
      umma_commit(&bar_d);
    };
    uint32_t it = 0;  // steps issued so far: every barrier completes once per step, so its parity is it & 1
    for (int t = 0; t < plan.tiles; ++t) {
      wait_on(&bar_a, it & 1);
      tc_fence_after_sync();
      issue_logits(it & 1);
      for (int s = 0; s < steps; ++s, ++it) {
        const int st = it & 1;
        wait_on(&bar_px, it & 1);
        tc_fence_after_sync();
        if (s >= 1) {  // the previous step's q o U / dO o W rows are complete (their owners passed the drain)
          wait_on(&bar_x, (it - 1) & 1);
          tc_fence_after_sync();
          issue_sums();
        }
        issue_uw(0, ks_x);
        if (nk_y > 0) {
          wait_on(&bar_py, it & 1);
          tc_fence_after_sync();
          issue_uw(1, ks_y);
        }
        umma_commit(&bar_uw);  // the drain only needs U and W; the accumulated transposed products run behind it
        {
          const uint32_t b1 = lA1_mn + st * kStage16, b2 = lA2_mn + st * kStage16;
#pragma unroll
          for (int ks = 0; ks < kTileM / 16; ++ks)  // K runs over the 128 rows of the tile
            umma_ss_lo(tmem + kColDK2, lDS_t + 128 * ks, b1 + 128 * ks, idesc_acc, !(it == 0 && ks == 0));
#pragma unroll
          for (int ks = 0; ks < kTileM / 16; ++ks)
            umma_ss_lo(tmem + kColDV2, lP_t + 128 * ks, b2 + 128 * ks, idesc_acc, !(it == 0 && ks == 0));
        }
        if (s + 1 < steps) {
          wait_on(&bar_a, (it + 1) & 1);  // next operands built, and every worker is done reading S / dP and D
          tc_fence_after_sync();
          issue_logits((it + 1) & 1);
        }
      }
      wait_on(&bar_x, (it - 1) & 1);  // last step of the range
      tc_fence_after_sync();
      issue_sums();
    }
    umma_commit(&bar_fin);
  } else if (warp == 9) {
    // ------------------------------------------------------------------ loader
    // Stages, up to kRowStages steps ahead of the workers, the k1 and v1 rows of each step's first keys (bf16, for
    // the operand builds) and the k1 rows once more as fp32 (for dq += U o k1_j).  Lane l handles the 16-byte
    // pieces l, l + 32, l + 64, l + 96 of the 2 x 8 rows.
    const int lane = tid & 31;
    float* k1f_w = reinterpret_cast<float*>(smem + kOffK1f);
    uint32_t gi = 0;
    for (int t = 0; t < plan.tiles; ++t)
      for (int s = 0; s < steps; ++s, ++gi) {
        const int stg = gi & (kRowStages - 1);
        if (gi >= kRowStages) wait_on(&bar_empty[stg], ((gi / kRowStages) - 1) & 1);
        uint4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c = lane + 32 * q, which = c >> 6, gg = (c >> 3) & 7, part = c & 7;
          const int jj = s * G + gg;
          v[q] = make_uint4(0, 0, 0, 0);
          if (gg < G && jj < nj)
            v[q] = __ldg(reinterpret_cast<const uint4*>((which == 0 ? p.k1 : p.v1) + base + (size_t)jlist[jj] * kD) + part);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c = lane + 32 * q, which = c >> 6, gg = (c >> 3) & 7, part = c & 7;
          *reinterpret_cast<uint4*>(smem + kOffRows + ((stg * 2 + which) * kMaxGroups + gg) * (kD * 2) + part * 16) = v[q];
          if (which == 0) {
            const uint32_t w4[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
            float f[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              f[2 * e] = __uint_as_float(w4[e] << 16);
              f[2 * e + 1] = __uint_as_float(w4[e] & 0xffff0000u);
            }
            float4* dst = reinterpret_cast<float4*>(k1f_w + (stg * kMaxGroups + gg) * kD + part * 8);
            dst[0] = make_float4(f[0], f[1], f[2], f[3]);
            dst[1] = make_float4(f[4], f[5], f[6], f[7]);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_full[stg]);
      }
  }
  } else {
    // ------------------------------------------------------------------ workers
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const uint32_t tmem_row = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t* pvbits = reinterpret_cast<const uint32_t*>(smem + kOffPv);
    const int lane = tid & 31;
    const float* k1f = reinterpret_cast<const float*>(smem + kOffK1f);
    // one arrival per warp: every lane orders its own writes, the warp converges, one lane arrives
    auto warp_arrive = [&](uint64_t* bar) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };
    const int g = r / rt, ii = r - g * rt;
    const bool slot_ok = g < G;
    // rows [G * rt, 128) never carry a pair: warps made of such rows only take part in the hand-offs; their
    // rows of P, dS, q o U and dO o W keep the zeros written during set-up
    const bool warp_live = (warp & 3) * 32 < G * rt;
    const bool live_x = warp_live && 32 * grp < nk_x;
    const bool live_y = warp_live && 32 * grp < nk_y;
    // partial column sums of this thread's output column (readers: the 128 threads of the q side)
    float* part_col = (r < 64 ? p.dk1_part : p.dv1_part) + (size_t)slab * p.part_stride + base + (r & 63);

    uint32_t xreg[32];
    float dq_acc[32];  // dq columns [32 grp, 32 grp + 32) of this thread's row: the two groups share the accumulation
    float lse2 = INFINITY, delta = 0.f;
    bool row_ok = false;
    int i = 0;
    uint32_t it = 0;

    // operand rows of tile step s (global step index gi): the k1 / v1 rows come from the loader warp's stage
    auto build_operand = [&](int s, uint32_t gi) {
      const int stg = gi & (kRowStages - 1), st = gi & 1;
      wait_on(&bar_full[stg], (gi / kRowStages) & 1);
      const int jj = s * G + g;
      const bool ok = row_ok && jj < nj;
      const uint4* kp = reinterpret_cast<const uint4*>(smem + kOffRows + ((stg * 2 + grp) * kMaxGroups + (slot_ok ? g : 0)) * (kD * 2));
      uint8_t* dst = smem + (grp == 0 ? kOffA1 : kOffA2) + st * (kTileM * 128) + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 a = make_uint4(0, 0, 0, 0);
        if (ok) {
          const uint4 kk = kp[c];
          const uint32_t kw[4] = {kk.x, kk.y, kk.z, kk.w};
          uint32_t aw[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            __nv_bfloat162 m = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&xreg[4 * c + t]),
                                       *reinterpret_cast<const __nv_bfloat162*>(&kw[t]));
            aw[t] = *reinterpret_cast<uint32_t*>(&m);
          }
          a = make_uint4(aw[0], aw[1], aw[2], aw[3]);
        }
        *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = a;
      }
      fence_smem_to_async_proxy();
      tc_fence_before_sync();
      warp_arrive(&bar_a);
    };
    // one half of the element-wise pass: P and dS of 32 columns as bf16 into shared memory (operands of the
    // transposed products) and, packed, over the S / dP columns just read (A operands of U and W)
    auto half_pass = [&](int half, int s) {
      const int col = 64 * half + 32 * grp;  // column inside the slab
      const int jj = s * G + g;
      const bool ok = row_ok && jj < nj;
      const int wi = (k0 + col) >> 5;
      const uint32_t word = ok ? (kmask[MF_IDX(wi, kMaskWords, p.status)] &
                                  pvbits[MF_IDX(jlist[MF_IDX(jj, kMaxKeys, p.status)] * kMaskWords + wi, kMaxKeys * kMaskWords, p.status)])
                               : 0u;
      // When only invalid keys are hidden, no per-column select is needed: their K2 / V2 rows are zero, so whatever
      // P and dS hold in their columns reaches neither U, W nor dq, and their own dK2 / dV2 rows are written as zeros.
      const bool selects = word != kmask[wi] || lse2 < -64.f;  // (the bound keeps exp2(-lse) and its products finite)
      uint8_t* prow = smem + kOffP + half * (kTileM * 128) + r * 128;
      uint8_t* dsrow = smem + kOffDS + half * (kTileM * 128) + r * 128;
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {  // 16 columns at a time keeps the live registers low
        uint32_t sv[16], dp[16];
        tmem_ld16(tmem_row + kColS + col + 16 * sub, sv);
        tmem_ld16(tmem_row + kColDP + col + 16 * sub, dp);
        tmem_ld_wait();
        uint32_t pk[8], dk[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const int e = 2 * t;
          float p0 = fast_exp2(fmaf(__uint_as_float(sv[e]), kLog2e, -lse2));
          float p1 = fast_exp2(fmaf(__uint_as_float(sv[e + 1]), kLog2e, -lse2));
          if (selects) {
            p0 = ((word >> (16 * sub + e)) & 1u) ? p0 : 0.f;
            p1 = ((word >> (16 * sub + e + 1)) & 1u) ? p1 : 0.f;
          }
          const float d0 = p0 * (__uint_as_float(dp[e]) - delta);
          const float d1 = p1 * (__uint_as_float(dp[e + 1]) - delta);
          pk[t] = pack_bf16x2(p0, p1);
          dk[t] = pack_bf16x2(d0, d1);
        }
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {  // 8 columns = one 16-byte chunk of the 128-byte row
          const int cc = 4 * grp + 2 * sub + q2;
          const uint32_t off = (cc ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(prow + off) = make_uint4(pk[4 * q2], pk[4 * q2 + 1], pk[4 * q2 + 2], pk[4 * q2 + 3]);
          *reinterpret_cast<uint4*>(dsrow + off) = make_uint4(dk[4 * q2], dk[4 * q2 + 1], dk[4 * q2 + 2], dk[4 * q2 + 3]);
        }
        // packed values over the first 16 columns of the 32-column chunk: sub-chunk 0 -> [0,8), 1 -> [8,16); both lie
        // below the columns of sub-chunk 1 still to be read only for sub 0 ([0,8) < 16), and sub 1 has been read
        tmem_st8(tmem_row + kColS + col + 8 * sub, pk);
        tmem_st8(tmem_row + kColDP + col + 8 * sub, dk);
      }
    };
    // column sums of step sp: values already in the partial plane (later query ranges add to them) ...
    float oldv[kMaxGroups];
    auto prefetch_sums = [&](int t, int sp) {
#pragma unroll
      for (int m = 0; m < kMaxGroups; ++m) {
        oldv[m] = 0.f;
        if (grp == 0 && t > 0 && m < G && sp * G + m < nj) oldv[m] = part_col[(size_t)jlist[sp * G + m] * kD];
      }
    };
    // ... and the store of old + new once the column-sum product has completed
    auto commit_sums = [&](int sp) {
      wait_on(&bar_d, (it - 1) & 1);
      tc_fence_after_sync();
      if (grp == 0) {
        uint32_t dv[16];
        tmem_ld16(tmem_row + kColD, dv);
        tmem_ld_wait();
#pragma unroll
        for (int m = 0; m < kMaxGroups; ++m)
          if (m < G && sp * G + m < nj) part_col[(size_t)jlist[sp * G + m] * kD] = oldv[m] + __uint_as_float(dv[m]);
      }
      tc_fence_before_sync();
    };

    for (int t = 0; t < plan.tiles; ++t) {
      // ---- this range's row: q (group 0) or dO (group 1) as 32 bf16x2 words, lse and delta of the query
      i = t * rt + ii;
      row_ok = slot_ok && i < n_queries && p.query_valid[(size_t)b * N + i] > 0;
      {
        const uint4* xp = reinterpret_cast<const uint4*>((grp == 0 ? p.q : p.grad_out) + base + (size_t)(row_ok ? i : 0) * kD);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 v = make_uint4(0, 0, 0, 0);
          if (row_ok) v = __ldg(xp + c);
          xreg[4 * c + 0] = v.x;
          xreg[4 * c + 1] = v.y;
          xreg[4 * c + 2] = v.z;
          xreg[4 * c + 3] = v.w;
        }
      }
      // exp2(S log2e - lse log2e); a row without a query keeps +inf so that every probability is 0
      lse2 = INFINITY;
      delta = 0.f;
      if (row_ok) {
        lse2 = p.lse[(size_t)bh * N + i] * kLog2e;
        delta = p.delta[(size_t)bh * N + i];
      }
#pragma unroll
      for (int d = 0; d < 32; ++d) dq_acc[d] = 0.f;
      build_operand(0, it);

      for (int s = 0; s < steps; ++s, ++it) {
        const int st = it & 1;
        if (s >= 1) prefetch_sums(t, s - 1);
        wait_on(&bar_sx, it & 1);
        tc_fence_after_sync();
        if (live_x) half_pass(0, s);
        tmem_st_wait();
        fence_smem_to_async_proxy();
        tc_fence_before_sync();  // also orders the previous drain's reads of U, W before the products issued next
        warp_arrive(&bar_px);
        if (nk_y > 0) {
          if (live_y) half_pass(1, s);
          tmem_st_wait();
          fence_smem_to_async_proxy();
          tc_fence_before_sync();
          warp_arrive(&bar_py);
        }
        if (s >= 1) commit_sums(s - 1);
        if (s + 1 < steps) build_operand(s + 1, it + 1);
        wait_on(&bar_uw, it & 1);
        tc_fence_after_sync();
        // ---- drain: group 0 reads U (q o U), group 1 reads W (dO o W); dq += U o k1_j is shared: group 0 takes
        // columns [0,32) from the half of U it holds anyway, group 1 loads columns [32,64) of U once more
        if (warp_live) {
          uint8_t* xrow = smem + kOffX + grp * (kTileM * 128) + r * 128;
          const float4* kf = reinterpret_cast<const float4*>(k1f + ((it & (kRowStages - 1)) * kMaxGroups + (slot_ok ? g : 0)) * kD + 32 * grp);
          auto add_dq = [&](const uint32_t (&w)[32]) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const float4 ka = kf[c];
              dq_acc[4 * c + 0] = fmaf(__uint_as_float(w[4 * c + 0]), ka.x, dq_acc[4 * c + 0]);
              dq_acc[4 * c + 1] = fmaf(__uint_as_float(w[4 * c + 1]), ka.y, dq_acc[4 * c + 1]);
              dq_acc[4 * c + 2] = fmaf(__uint_as_float(w[4 * c + 2]), ka.z, dq_acc[4 * c + 2]);
              dq_acc[4 * c + 3] = fmaf(__uint_as_float(w[4 * c + 3]), ka.w, dq_acc[4 * c + 3]);
            }
          };
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t w[32];
            tmem_ld32(tmem_row + (grp == 0 ? kColU : kColWb) + 32 * half, w);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t xw[4];
#pragma unroll
              for (int t2 = 0; t2 < 4; ++t2) {
                const int e = 8 * c + 2 * t2;
                const uint32_t ub = pack_bf16x2(__uint_as_float(w[e]), __uint_as_float(w[e + 1]));
                __nv_bfloat162 m = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&ub),
                                           *reinterpret_cast<const __nv_bfloat162*>(&xreg[16 * half + 4 * c + t2]));
                xw[t2] = *reinterpret_cast<uint32_t*>(&m);
              }
              *reinterpret_cast<uint4*>(xrow + (((4 * half + c) ^ (r & 7)) << 4)) = make_uint4(xw[0], xw[1], xw[2], xw[3]);
            }
            if (grp == 0 && half == 0) add_dq(w);
          }
          if (grp == 1) {
            uint32_t w[32];
            tmem_ld32(tmem_row + kColU + 32, w);
            tmem_ld_wait();
            add_dq(w);
          }
        }
        fence_smem_to_async_proxy();
        tc_fence_before_sync();
        warp_arrive(&bar_x);
        if (lane == 0) mbar_arrive(&bar_empty[it & (kRowStages - 1)]);  // the step's staged rows are free (after the warp converged)
      }
      // ---- end of the range: last column sums, then dq of the range (rows of one query summed over the groups)
      prefetch_sums(t, steps - 1);
      commit_sums(steps - 1);  // also: every product issued so far has completed
      float* dq_dst = p.dq_part + (size_t)slab * p.part_stride + base;
      if (G == 1) {
        if (slot_ok && i < n_queries) {
          float4* dst = reinterpret_cast<float4*>(dq_dst + (size_t)i * kD + 32 * grp);
#pragma unroll
          for (int c = 0; c < 8; ++c)
            dst[c] = make_float4(dq_acc[4 * c], dq_acc[4 * c + 1], dq_acc[4 * c + 2], dq_acc[4 * c + 3]);
        }
      } else {
        float* stage = reinterpret_cast<float*>(smem + kOffA1);  // [128][64] fp32 over the two idle A1 stages
        named_barrier(1, 256);
#pragma unroll
        for (int c = 0; c < 8; ++c)  // float4 index rotated by the row to spread the banks
          reinterpret_cast<float4*>(stage + r * kD)[(8 * grp + c) ^ (r & 15)] =
              make_float4(dq_acc[4 * c], dq_acc[4 * c + 1], dq_acc[4 * c + 2], dq_acc[4 * c + 3]);
        named_barrier(1, 256);
        if (g == 0 && i < n_queries) {  // thread (r, grp) sums columns [32 grp, 32 grp + 32) in a fixed order
          float4 acc[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int gg = 0; gg < G; ++gg) {
            const int r2 = gg * rt + r;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const float4 v = reinterpret_cast<const float4*>(stage + r2 * kD)[(8 * grp + c) ^ (r2 & 15)];
              acc[c].x += v.x;
              acc[c].y += v.y;
              acc[c].z += v.z;
              acc[c].w += v.w;
            }
          }
          float4* dst = reinterpret_cast<float4*>(dq_dst + (size_t)i * kD + 32 * grp);
#pragma unroll
          for (int c = 0; c < 8; ++c) dst[c] = acc[c];
        }
        named_barrier(1, 256);  // the next range's operands overwrite the staging area
      }
    }
    // ---- epilogue: accumulators: lane r of tensor memory = key k0 + r; group 0 stores dK2, group 1 dV2
    wait_on(&bar_fin, 0);
    tc_fence_after_sync();
    {
      __nv_bfloat16* dst = (grp == 0 ? p.dk2 : p.dv2) + base + (size_t)(k0 + r) * kD;
      const bool store = !bad && r < nk_slab;
      const bool live = key_live(r);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t w[32];
        tmem_ld32(tmem_row + (grp == 0 ? kColDK2 : kColDV2) + 32 * half, w);  // whole warps: the load is warp-wide
        tmem_ld_wait();
        if (store) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 v = make_uint4(0, 0, 0, 0);  // an invalid key's row is exactly zero
            if (live) {
              v.x = pack_bf16x2(__uint_as_float(w[8 * c + 0]), __uint_as_float(w[8 * c + 1]));
              v.y = pack_bf16x2(__uint_as_float(w[8 * c + 2]), __uint_as_float(w[8 * c + 3]));
              v.z = pack_bf16x2(__uint_as_float(w[8 * c + 4]), __uint_as_float(w[8 * c + 5]));
              v.w = pack_bf16x2(__uint_as_float(w[8 * c + 6]), __uint_as_float(w[8 * c + 7]));
            }
            reinterpret_cast<uint4*>(dst + 32 * half)[c] = v;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  bad = __syncthreads_or(bad) != 0;
  if (bad && tid == 0) atomicExch(p.status, MF_ERR_DEVICE_TIMEOUT);
  if (warp == 0) tmem_dealloc(tmem, kBwdTmemCols);
}

// Sums the partial planes in a fixed order and writes dq, dk1, dv1 in bf16; rows of padded tokens get exact
// zeros, and so do the rows of dk2 / dv2 that no CTA of the main kernel owns.  When a bounded wait expired
// anywhere (status word set) every gradient is written as zeros.
__global__ void simplicial_rows_bwd_finalize_kernel(RowsBwdParams p, __nv_bfloat16* __restrict__ dq,
                                                    __nv_bfloat16* __restrict__ dk1, __nv_bfloat16* __restrict__ dv1,
                                                    int BH) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 4 elements
  const long long total = (long long)BH * p.N * (kD / 4);
  if (idx >= total) return;
  const int d4 = (int)(idx % (kD / 4));
  const int row = (int)((idx / (kD / 4)) % p.N);
  const int bh = (int)(idx / ((long long)(kD / 4) * p.N));
  const int b = bh / p.H;
  const int n_keys = p.info[b].n_keys, n_queries = p.info[b].n_queries, nj = p.info[b].reserved0;
  const bool failed = p.status[0] != 0;
  const bool active = n_queries > 0 && nj > 0 && !failed;
  const int nsl = slab_count(n_keys);
  const size_t off = ((size_t)bh * p.N + row) * kD + 4 * d4;
  const bool q_ok = active && row < n_queries && p.query_valid[(size_t)b * p.N + row] > 0;
  const bool k_ok = active && row < n_keys && p.key_valid[(size_t)b * p.N + row] > 0;
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
  store4(dq + off, a);
  float4 k1v = make_float4(0.f, 0.f, 0.f, 0.f), v1v = k1v;
  if (k_ok)
    for (int s = 0; s < nsl; ++s) {
      add4(k1v, *reinterpret_cast<const float4*>(p.dk1_part + (size_t)s * p.part_stride + off));
      add4(v1v, *reinterpret_cast<const float4*>(p.dv1_part + (size_t)s * p.part_stride + off));
    }
  store4(dk1 + off, k1v);
  store4(dv1 + off, v1v);
  if (!(active && row < n_keys)) {
    store4(p.dk2 + off, make_float4(0.f, 0.f, 0.f, 0.f));
    store4(p.dv2 + off, make_float4(0.f, 0.f, 0.f, 0.f));
  }
}

struct RowsBwdLayout {
  size_t info, order, delta, dq, dk1, dv1, total;
  int slabs_max;
  size_t part;  // bytes per partial plane
};

RowsBwdLayout rows_bwd_layout(int B, int H, int N) {
  RowsBwdLayout l{};
  l.slabs_max = (N + kSlab - 1) / kSlab;
  l.part = align_up((size_t)B * H * N * kD * sizeof(float), 256);
  size_t off = simplicial_schedule_layout(B, &l.info, &l.order);
  l.delta = off;
  off += align_up((size_t)B * H * N * sizeof(float), 256);
  l.dq = off;
  off += l.part * l.slabs_max;
  l.dk1 = off;
  off += l.part * l.slabs_max;
  l.dv1 = off;
  off += l.part * l.slabs_max;
  l.total = off;
  return l;
}

}  // namespace

size_t simplicial_rows_bwd_workspace_bytes(const MfSimplicialBwdArgs& a) {
  return rows_bwd_layout(a.batch, a.heads, a.tokens).total;
}

int simplicial_rows_bwd(const MfSimplicialBwdArgs& a, cudaStream_t stream) {
  const RowsBwdLayout l = rows_bwd_layout(a.batch, a.heads, a.tokens);
  char* ws = static_cast<char*>(a.workspace);
  const int BH = a.batch * a.heads;
  RowsBwdParams p{};
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
  p.dk2 = static_cast<__nv_bfloat16*>(a.dk2);
  p.dv2 = static_cast<__nv_bfloat16*>(a.dv2);
  p.status = reinterpret_cast<int32_t*>(ws);
  p.use_tma = make_rows_tensor_map(&p.tm_k2, a.k2, a.tokens, BH) && make_rows_tensor_map(&p.tm_v2, a.v2, a.tokens, BH);
  BatchInfo* info = reinterpret_cast<BatchInfo*>(ws + l.info);
  int32_t* order = reinterpret_cast<int32_t*>(ws + l.order);
  float* delta = reinterpret_cast<float*>(ws + l.delta);
  p.info = info;
  p.order = order;
  p.delta = delta;
  p.dq_part = reinterpret_cast<float*>(ws + l.dq);
  p.dk1_part = reinterpret_cast<float*>(ws + l.dk1);
  p.dv1_part = reinterpret_cast<float*>(ws + l.dv1);
  p.H = a.heads;
  p.N = a.tokens;
  p.slabs_max = l.slabs_max;
  p.part_stride = l.part / sizeof(float);

  int rc = launch_schedule(a.query_valid, a.pair_key_valid, a.batch, a.tokens, info, order, p.status, stream);
  if (rc != MF_OK) return rc;
  const int rows = BH * a.tokens;
  delta_rows_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(p.grad_out, a.out, delta, rows);
  MF_CHECK_LAUNCH("delta_rows_kernel");
  {
    cudaError_t e = cudaFuncSetAttribute(simplicial_rows_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
    if (e != cudaSuccess) return cuda_error(e, "cudaFuncSetAttribute(simplicial_rows_bwd_kernel)");
  }
  const long long blocks = (long long)BH * p.slabs_max;
  profile_mark(MF_PROFILE_SIMPLICIAL_BWD, true, stream);
  simplicial_rows_bwd_kernel<<<(unsigned)blocks, kBwdThreads, kSmemAlloc, stream>>>(p);
  profile_mark(MF_PROFILE_SIMPLICIAL_BWD, false, stream);
  MF_CHECK_LAUNCH("simplicial_rows_bwd_kernel");
  const long long total4 = (long long)rows * (kD / 4);
  simplicial_rows_bwd_finalize_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, stream>>>(
      p, static_cast<__nv_bfloat16*>(a.dq), static_cast<__nv_bfloat16*>(a.dk1), static_cast<__nv_bfloat16*>(a.dv1), BH);
  MF_CHECK_LAUNCH("simplicial_rows_bwd_finalize_kernel");
  return MF_OK;
}

}  // namespace mf
