// Radius block-sparse and local-window attention on the Blackwell tensor cores (tcgen05.mma, accumulators in tensor
// memory, operand tiles by bulk tensor copies), bf16, head_dim 64.
//
// Same operators and semantics as sparse_attn.cu / sparse_attn_mma.cu (masked softmax attention as computed by
// F.scaled_dot_product_attention for the reference's RotaryMultiheadAttention,
// src/matterformer/models/regular_attention.py:251-268).  At the sizes where the radius block list is nearly full
// (a 6 A cutoff in a 15-30 A cell leaves few 32 x 32 blocks empty) the operator is dense attention with a bit mask,
// and 128-row tcgen05 tiles beat the 32-row warp-level tiles by a wide margin.
//
// One CTA owns a tile of 128 "owner" rows of one (batch, head) and walks over the partner tiles of 64 rows that hold
// at least one visible pair.  Three passes share one skeleton:
//   FWD : owners = queries, partners = keys    S = Q.K^T              -> P -> W = P.V, out = out*alpha + W   (registers)
//   DQ  : owners = queries, partners = keys    S = Q.K^T, dP = dO.V^T -> dS -> dQ += dS.K                   (tensor memory)
//   DKV : owners = keys,    partners = queries S^T = K.Q^T, dP^T = V.dO^T -> P^T, dS^T -> dV += P^T.dO, dK += dS^T.Q
// P and dS never touch shared memory: the row owners pack them to bf16 over the fp32 columns they came from and the
// second product of a step takes its A operand from tensor memory.  Every output row has one owner: no atomics,
// bit-identical reruns.
//
// Roles: 8 (forward) or 16 (backward) warps own the rows, two or four threads per row, each taking a share of the 64
// partner columns of a step and of the head dimension; one thread of the next warp issues every tcgen05.mma, one
// thread of the last warp every bulk tensor copy (ring of partner stages).  S and dP are double-buffered in tensor memory: the first products of step t+2 are issued right behind
// the second products of step t (the tensor pipe runs them in order), so the row owners find step t+1 ready when
// they are done with step t; in the forward pass P.V of a step is drained one step late for the same reason.
// Hand-offs are mbarriers; every wait is bounded and an expired wait is reported through a status word.
#include "common.cuh"
#include "sm100_primitives.cuh"
#include "sparse_attn_sm100.cuh"
#include "tensor_map.cuh"

namespace mf {

__device__ int32_t g_sparse_tc_status = 0;  // last device-side error of the kernels in this file (0 = none)

namespace {

enum { T_FWD = 0, T_DQ = 1, T_DKV = 2 };
constexpr int kHd = 64;            // head dimension
constexpr int kOwn = 128;          // owner rows per CTA
constexpr int kPart = 64;          // partner rows per step
constexpr int kMaxPartTiles = 128; // tokens <= 8192
constexpr int kBoxRows = 64;       // rows per bulk tensor copy
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLn2F = 0.6931471805599453f;

// Per pass: row-owner warps, partner stages in flight, CTAs per SM, tensor-memory columns.  The first products of two
// steps are in flight at a time (two buffers each for S and dP), so a stage is busy for three steps.
//   FWD     : S[2] 64 columns each, W[2] 64 each      = 256 columns, two CTAs per SM of 8 row-owner warps, 5 stages
//   DQ, DKV : {S, dP}[2] 128 each, dQ | dK 64, dV 64  = 384 -> 512 columns, one CTA per SM of 16 row-owner warps, 8 stages
// A row is shared by kSplit threads (one per warp of the same lane quarter), each taking kCols of the 64 partner
// columns of a step and kCols of the 64 output columns.
template <int MODE>
struct TcShape {
  static constexpr bool kFwd = MODE == T_FWD;
  static constexpr int kWorkerWarps = kFwd ? 8 : 16;
  static constexpr int kWorkers = kWorkerWarps * 32;
  static constexpr int kThreads = kWorkers + 96;  // + two issuing warps and the copy warp (one thread of each works)
  static constexpr int kSplit = kWorkerWarps / 4;
  static constexpr int kCols = kPart / kSplit;
  // first packed column of the 16 partners of MMA k-group kg: every thread packs over its own columns
  __host__ __device__ static constexpr int kPackedCol(int kg) { return kCols * (kg / (kCols / 16)) + 8 * (kg % (kCols / 16)); }
  static constexpr int kStages = kFwd ? 5 : 8;
  static constexpr int kCtasPerSm = kFwd ? 2 : 1;
  static constexpr int kTmemCols = kFwd ? 256 : 512;
  __host__ __device__ static constexpr int kColS(int buf) { return kFwd ? 64 * buf : 128 * buf; }
  __host__ __device__ static constexpr int kColDP(int buf) { return 128 * buf + 64; }
  __host__ __device__ static constexpr int kColW(int buf) { return 128 + 64 * buf; }  // FWD
  static constexpr int kColAcc0 = 256, kColAcc1 = 320;             // DQ: dQ; DKV: dK, dV
  // shared memory map (dynamic, 1024-byte aligned); every tile is [rows][64] bf16 in 128-byte swizzled lines
  static constexpr int kOffOwnA = 0;                                        // 128 rows: Q | Q | K
  static constexpr int kOffOwnB = kOffOwnA + kOwn * 128;                    // 128 rows: - | dO | V
  static constexpr int kOffPartA = kFwd ? kOffOwnB : kOffOwnB + kOwn * 128;  // stages x 64 rows: K | K | Q
  static constexpr int kOffPartB = kOffPartA + kStages * kPart * 128;       // stages x 64 rows: V | V | dO
  static constexpr int kSmemBytes = kOffPartB + kStages * kPart * 128;
  static constexpr int kSmemAlloc = kSmemBytes + 1024;
};

struct TcParams {
  const __nv_bfloat16* grad_out;
  const __nv_bfloat16* out_in;
  const float* lse_in;
  float* delta;  // scale * dO . out per query: written by the DQ pass, read by the DKV pass
  float* lse2;   // log-sum-exp per query in the log2 domain: likewise
  const int32_t* num_atoms;
  const int32_t* block_count;
  const int32_t* block_cols;
  const uint32_t* block_mask;
  __nv_bfloat16* out;
  float* lse_out;
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int H, N, window, T32;
  float scale;
  CUtensorMap tm_own_a, tm_own_b, tm_part_a, tm_part_b;  // (B*H, N, 64) bf16, boxes of 64 rows, 128-byte swizzle
};

__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// A read-only load that stays where it is written: the compiler may not sink it towards its first use, which is a
// whole step later.
__device__ __forceinline__ uint32_t ld_pinned(const uint32_t* ptr) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(ptr));
  return v;
}
// tensor memory <-> registers for 16 or 32 fp32 columns, 8 or 16 packed words
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st16(taddr, r); }
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t (&r)[8]) { tmem_st8(taddr, r); }
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// bits c of a 32-row block starting at row kb with lo <= kb + c <= hi
__device__ __forceinline__ uint32_t range_word(int kb, int lo, int hi) {
  const int a = max(lo - kb, 0), b = min(hi - kb, 31);
  if (a > b) return 0u;
  const int len = b - a + 1;
  return (len >= 32 ? 0xffffffffu : ((1u << len) - 1u)) << a;
}

template <int MODE, bool kRadius>
__global__ void __launch_bounds__(TcShape<MODE>::kThreads, TcShape<MODE>::kCtasPerSm) sparse_tc_kernel(const __grid_constant__ TcParams p) {
  using Sh = TcShape<MODE>;
  constexpr int kStages = Sh::kStages, kTcThreads = Sh::kThreads, kC = Sh::kCols;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar_own, bar_s[2], bar_p[2], bar_w[2];
  __shared__ uint64_t bar_full[kStages], bar_free[kStages];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t present[kMaxPartTiles];  // per partner tile: bit (owner 32-row block * 2 + partner 32-row block)
  __shared__ uint16_t steplist[kMaxPartTiles];
  __shared__ int nsteps_s;
  __shared__ float xch[2][Sh::kSplit][kOwn];   // [step parity][column part][row]: values the threads of a row swap

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = tid & 127, part = (tid >> 7) & (Sh::kSplit - 1);  // row, and which kC columns of it
  const int col0 = part * kC;
  const int ot = blockIdx.x, bh = blockIdx.y, b = bh / p.H;
  const int N = p.N;
  const int n = min(p.num_atoms[b], N);
  const int row0 = ot * kOwn;
  const size_t base = (size_t)bh * N * kHd;
  const int half = p.window >> 1;

  // ---- which partner tiles hold a visible pair
  const int part_tiles = (n + kPart - 1) / kPart;
  for (int i = tid; i < kMaxPartTiles; i += kTcThreads) present[i] = 0u;
  __syncthreads();
  if (row0 < n) {
    if (kRadius) {
      for (int rb = 0; rb < 4; ++rb) {
        const int rt = ot * 4 + rb;
        if (rt * 32 >= n) break;
        const int cnt = p.block_count[(size_t)b * p.T32 + rt];
        const int32_t* cols = p.block_cols + ((size_t)b * p.T32 + rt) * p.T32;
        for (int i = tid; i < cnt; i += kTcThreads) {
          const int ct = cols[i];
          if (ct >= 0 && (ct >> 1) < part_tiles) atomicOr(&present[ct >> 1], 1u << (rb * 2 + (ct & 1)));
        }
      }
    } else {
      // band: owner row i sees partners i - half .. i + half - 1 (the transposed band when the owners are keys)
      const int lo = max(0, row0 - half + (MODE == T_DKV ? 1 : 0));
      const int hi = min(n - 1, min(row0 + kOwn - 1, n - 1) + half - (MODE == T_DKV ? 0 : 1));
      for (int pt = tid; pt < part_tiles; pt += kTcThreads)
        if (pt * kPart <= hi && pt * kPart + kPart - 1 >= lo) present[pt] = 0xffu;
    }
  }
  __syncthreads();
  if (tid == 0) {
    int c = 0;
    for (int pt = 0; pt < part_tiles; ++pt)
      if (present[pt]) steplist[c++] = (uint16_t)pt;
    nsteps_s = c;
  }
  __syncthreads();
  const int nsteps = nsteps_s;

  if (nsteps == 0) {  // uniform per CTA: padding only, or nothing visible.  The rows get zeros.
    const int rows = min(kOwn, N - row0);
    if (MODE == T_FWD) {
      for (int i = tid; i < rows * 8; i += kTcThreads) reinterpret_cast<uint4*>(p.out + base + (size_t)row0 * kHd)[i] = make_uint4(0, 0, 0, 0);
      for (int i = tid; i < rows; i += kTcThreads) p.lse_out[(size_t)bh * N + row0 + i] = 0.f;
    } else if (MODE == T_DQ) {
      for (int i = tid; i < rows * 8; i += kTcThreads) reinterpret_cast<uint4*>(p.dq + base + (size_t)row0 * kHd)[i] = make_uint4(0, 0, 0, 0);
      for (int i = tid; i < rows; i += kTcThreads) p.delta[(size_t)bh * N + row0 + i] = 0.f, p.lse2[(size_t)bh * N + row0 + i] = 0.f;
    } else {
      for (int i = tid; i < rows * 8; i += kTcThreads) {
        reinterpret_cast<uint4*>(p.dk + base + (size_t)row0 * kHd)[i] = make_uint4(0, 0, 0, 0);
        reinterpret_cast<uint4*>(p.dv + base + (size_t)row0 * kHd)[i] = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }

  // ---- set-up: barriers, tensor memory
  if (tid == 0) {
    mbar_init(&bar_own, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_p[i], Sh::kWorkerWarps);  // one arrival per row-owner warp
      mbar_init(&bar_w[i], 1);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_free[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, Sh::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;

  bool bad = false;
  auto wait_on = [&](uint64_t* bar, uint32_t ph) {
    if (!bad) bad = !mbar_wait(bar, ph);
  };

  if (tid == Sh::kWorkers + 64) {
    // ------------------------------------------------------------------ bulk tensor copies
    constexpr uint32_t kStageBytes = 2u * kPart * 128u;
    auto load_stage = [&](int t) {
      const int stg = t % kStages, row = steplist[MF_IDX(t, kMaxPartTiles, &g_sparse_tc_status)] * kPart;
      mbar_arrive_expect_tx(&bar_full[stg], kStageBytes);
      tma_load_rows(smem + Sh::kOffPartA + stg * kPart * 128, &p.tm_part_a, row, bh, &bar_full[stg]);
      tma_load_rows(smem + Sh::kOffPartB + stg * kPart * 128, &p.tm_part_b, row, bh, &bar_full[stg]);
    };
    tma_prefetch_map(&p.tm_own_a);
    if (MODE != T_FWD) tma_prefetch_map(&p.tm_own_b);
    tma_prefetch_map(&p.tm_part_a);
    tma_prefetch_map(&p.tm_part_b);
    mbar_arrive_expect_tx(&bar_own, (MODE == T_FWD ? 1u : 2u) * kOwn * 128u);
#pragma unroll
    for (int c = 0; c < kOwn / kBoxRows; ++c) {
      tma_load_rows(smem + Sh::kOffOwnA + c * kBoxRows * 128, &p.tm_own_a, row0 + c * kBoxRows, bh, &bar_own);
      if (MODE != T_FWD) tma_load_rows(smem + Sh::kOffOwnB + c * kBoxRows * 128, &p.tm_own_b, row0 + c * kBoxRows, bh, &bar_own);
    }
    for (int t = 0; t < kStages && t < nsteps; ++t) load_stage(t);
    for (int t = kStages; t < nsteps; ++t) {  // a stage is free once the products of its previous step have completed
      wait_on(&bar_free[t % kStages], ((t / kStages) - 1) & 1);
      if (bad) break;
      load_stage(t);
    }
  } else if (tid == Sh::kWorkers || tid == Sh::kWorkers + 32) {
    // ------------------------------------------------------------------ MMAs
    // Two issuing threads in warps of different schedulers, so that neither the issue slots of one scheduler nor the
    // instruction stream of one thread limits the MMA rate: the first issues the products of P / dS, the second the
    // logit products.  The tensor pipe orders the MMAs of one thread only, so the second thread waits for the
    // completion of the products that read the buffer it is about to overwrite.
    const uint32_t l_own_a = make_desc_lo(smem_u32(smem + Sh::kOffOwnA), 0), l_own_b = make_desc_lo(smem_u32(smem + Sh::kOffOwnB), 0);
    const uint32_t l_part_a = make_desc_lo(smem_u32(smem + Sh::kOffPartA), 0), l_part_b = make_desc_lo(smem_u32(smem + Sh::kOffPartB), 0);
    constexpr uint32_t kStageStep = (kPart * 128) >> 4;  // descriptor units between partner stages
    const uint32_t idesc_kk = make_idesc_bf16(kOwn, kPart, false, false);  // both operands K-major: rows . rows^T
    const uint32_t idesc_mn = make_idesc_bf16(kOwn, kHd, false, true);     // A from tensor memory, B MN-major: P . rows
    if (tid == Sh::kWorkers) {
      for (int t = 0; t < nsteps; ++t) {  // products whose A operand is the packed P / dS of step t
        const int buf = t & 1;
        const uint32_t pa = l_part_a + (t % kStages) * kStageStep, pb = l_part_b + (t % kStages) * kStageStep;
        wait_on(&bar_p[buf], (t >> 1) & 1);
        tc_fence_after_sync();
#pragma unroll
        for (int kg = 0; kg < kPart / 16; ++kg) {  // 16 partners per MMA: 8 packed columns, 16 shared-memory lines
          const uint32_t acol = Sh::kPackedCol(kg);
          if (MODE == T_FWD) umma_ts_lo(tmem + Sh::kColW(buf), tmem + Sh::kColS(buf) + acol, pb + 128 * kg, idesc_mn, kg > 0);
          if (MODE == T_DQ) umma_ts_lo(tmem + Sh::kColAcc0, tmem + Sh::kColDP(buf) + acol, pa + 128 * kg, idesc_mn, t > 0 || kg > 0);
          if (MODE == T_DKV) {
            umma_ts_lo(tmem + Sh::kColAcc1, tmem + Sh::kColS(buf) + acol, pb + 128 * kg, idesc_mn, t > 0 || kg > 0);
            umma_ts_lo(tmem + Sh::kColAcc0, tmem + Sh::kColDP(buf) + acol, pa + 128 * kg, idesc_mn, t > 0 || kg > 0);
          }
        }
        umma_commit(&bar_free[t % kStages]);  // the stage and the S / dP buffer of step t are free
        if (MODE == T_FWD) umma_commit(&bar_w[buf]);
        else if (t == nsteps - 1) umma_commit(&bar_w[0]);
      }
    } else {
      wait_on(&bar_own, 0);
      for (int t = 0; t < nsteps; ++t) {  // S (and dP) of step t into buffer t & 1
        const int buf = t & 1;
        const uint32_t pa = l_part_a + (t % kStages) * kStageStep, pb = l_part_b + (t % kStages) * kStageStep;
        wait_on(&bar_full[t % kStages], (t / kStages) & 1);
        if (t >= 2) wait_on(&bar_free[(t - 2) % kStages], ((t - 2) / kStages) & 1);  // the buffer's previous user is done
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < kHd / 16; ++ks) umma_ss_lo(tmem + Sh::kColS(buf), l_own_a + 2 * ks, pa + 2 * ks, idesc_kk, ks > 0);
        if (MODE != T_FWD) {
#pragma unroll
          for (int ks = 0; ks < kHd / 16; ++ks) umma_ss_lo(tmem + Sh::kColDP(buf), l_own_b + 2 * ks, pb + 2 * ks, idesc_kk, ks > 0);
        }
        umma_commit(&bar_s[buf]);
      }
    }
  } else if (tid < Sh::kWorkers) {
    // ------------------------------------------------------------------ row owners
    const uint32_t tmem_row = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int orow = row0 + r;
    const bool row_ok = orow < n;
    const float sc2 = p.scale * kLog2eF;  // logits in the log2 domain
    auto warp_arrive = [&](uint64_t* bar) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };
    // Visibility of the 32 partners around this thread's kC columns of step t for its owner row.  The word is fetched
    // a step ahead and not touched until it is needed, so the load never stalls the row owner.
    constexpr uint32_t kAllBits = kC == 32 ? 0xffffffffu : ((1u << (kC & 31)) - 1u);
    auto word_of = [&](int t) -> uint32_t {
      const int pt = steplist[t];
      const int ct = 2 * pt + (col0 >> 5), kb = ct * 32;
      if (!row_ok) return 0u;
      if (kRadius) {
        if (!((present[pt] >> ((r >> 5) * 2 + (col0 >> 5))) & 1u)) return 0u;
        return ld_pinned(p.block_mask + (((size_t)b * p.T32 + MF_IDX(orow >> 5, p.T32, &g_sparse_tc_status)) * p.T32 +
                                         MF_IDX(ct, p.T32, &g_sparse_tc_status)) * 32 + (orow & 31));  // symmetric bitmap
      }
      const int lo = orow - half + (MODE == T_DKV ? 1 : 0), hi = orow + half - (MODE == T_DKV ? 0 : 1);
      return range_word(kb, max(lo, 0), min(hi, n - 1));
    };
    // partner rows beyond the structure's last atom hold whatever the padded tokens hold: clear them before they
    // become the B operand of a product (zero probabilities times a non-finite value would not be zero)
    auto clear_padding = [&](int t) {
      const int pt = steplist[t], stg = t % kStages;
      const int first = n - pt * kPart;  // first padded row of the tile
      if (first >= kPart) return;
      wait_on(&bar_full[stg], (t / kStages) & 1);
      for (int i = tid; i < (kPart - first) * 8; i += Sh::kWorkers) {
        const int row = first + (i >> 3), c = i & 7;
        *reinterpret_cast<uint4*>(smem + Sh::kOffPartA + stg * kPart * 128 + row * 128 + c * 16) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(smem + Sh::kOffPartB + stg * kPart * 128 + row * 128 + c * 16) = make_uint4(0, 0, 0, 0);
      }
      fence_smem_to_async_proxy();
    };

    float o_acc[kC];     // FWD: this thread's part of the output row
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    float lse2 = INFINITY, dlt = 0.f;  // DQ: the owner row's log-sum-exp (log2 domain) and scale * dO . out
    if (MODE == T_FWD) {
#pragma unroll
      for (int d = 0; d < kC; ++d) o_acc[d] = 0.f;
    }
    // FWD: out = out * alpha + P.V of step t, taken from tensor memory one step late (its product runs meanwhile)
    auto drain = [&](int t) {
      wait_on(&bar_w[t & 1], (t >> 1) & 1);
      tc_fence_after_sync();
      uint32_t w[kC];
      tmem_ld_cols(tmem_row + Sh::kColW(t & 1) + col0, w);
      tmem_ld_wait();
#pragma unroll
      for (int d = 0; d < kC; ++d) o_acc[d] = fmaf(o_acc[d], alpha_prev, __uint_as_float(w[d]));
      tc_fence_before_sync();
    };
    if (MODE == T_DQ) {
      float d = 0.f;
      if (row_ok) {
        const uint4* go = reinterpret_cast<const uint4*>(p.grad_out + base + (size_t)orow * kHd + col0);
        const uint4* oo = reinterpret_cast<const uint4*>(p.out_in + base + (size_t)orow * kHd + col0);
#pragma unroll
        for (int c = 0; c < kC / 8; ++c) {
          const uint4 a = __ldg(go + c), o = __ldg(oo + c);
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            d = fmaf(__uint_as_float(aw[e] << 16), __uint_as_float(ow[e] << 16), d);
            d = fmaf(__uint_as_float(aw[e] & 0xffff0000u), __uint_as_float(ow[e] & 0xffff0000u), d);
          }
        }
        lse2 = p.lse_in[(size_t)bh * N + orow] * kLog2eF;
      }
      xch[0][part][r] = d;
      named_barrier(1 + (warp & 3), 32 * Sh::kSplit);  // the warps that share these 32 rows
      dlt = 0.f;
#pragma unroll
      for (int q = 0; q < Sh::kSplit; ++q) dlt += xch[0][q][r];
      dlt *= p.scale;  // dS = P (dP - delta) scale = P (dP scale - delta scale)
      if (part == 0 && orow < N) {
        p.delta[(size_t)bh * N + orow] = row_ok ? dlt : 0.f;
        p.lse2[(size_t)bh * N + orow] = row_ok ? lse2 : 0.f;
      }
      named_barrier(1 + (warp & 3), 32 * Sh::kSplit);  // xch[0] is reused by the first steps
    }

    uint32_t word_next = word_of(0);
    for (int t = 0; t < nsteps; ++t) {
      const int buf = t & 1;
      const uint32_t word = (word_next >> (col0 & 31)) & kAllBits;  // this thread's kC partners in the low bits
      if (t + 1 < nsteps) word_next = word_of(t + 1);
      const int kb = steplist[t] * kPart + col0;  // first partner row of this thread's columns
      clear_padding(t);
      wait_on(&bar_s[buf], (t >> 1) & 1);
      tc_fence_after_sync();
      uint32_t sv[kC];
      tmem_ld_cols(tmem_row + Sh::kColS(buf) + col0, sv);
      tmem_ld_wait();
      // hidden pairs become -inf once; every later use (maximum, exp2) then needs no further test
      if (word != kAllBits) {
#pragma unroll
        for (int e = 0; e < kC; ++e) sv[e] = ((word >> e) & 1u) ? sv[e] : 0xff800000u;
      }
      if (MODE == T_FWD) {
        // ---- online softmax over the visible partners (the scale is positive: it commutes with the maximum)
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < kC; e += 2) mx4[(e >> 1) & 3] = max3(mx4[(e >> 1) & 3], __uint_as_float(sv[e]), __uint_as_float(sv[e + 1]));
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc2;
        xch[buf][part][r] = mx;
        named_barrier(1 + (warp & 3), 32 * Sh::kSplit);
#pragma unroll
        for (int q = 0; q < Sh::kSplit; ++q) mx = fmaxf(mx, xch[buf][q][r]);
        const float m_new = fmaxf(m_run, mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = (m_run == -INFINITY) ? 0.f : exp2_fast(m_run - m_use);
        m_run = m_new;
        uint32_t pk[kC / 2];
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int e = 0; e < kC; e += 2) {
          const float p0 = exp2_fast(fmaf(__uint_as_float(sv[e]), sc2, -m_use));  // exp2(-inf) = 0 for hidden pairs
          const float p1 = exp2_fast(fmaf(__uint_as_float(sv[e + 1]), sc2, -m_use));
          ps0 += p0;
          ps1 += p1;
          pk[e >> 1] = pack_bf16x2(p0, p1);
        }
        l_run = l_run * alpha + (ps0 + ps1);
        tmem_st_cols(tmem_row + Sh::kColS(buf) + col0, pk);
        tmem_st_wait();
        tc_fence_before_sync();
        warp_arrive(&bar_p[buf]);
        if (t >= 1) drain(t - 1);
        alpha_prev = alpha;
      } else {
        uint32_t dp[kC];
        tmem_ld_cols(tmem_row + Sh::kColDP(buf) + col0, dp);
        tmem_ld_wait();
        // dP of a hidden pair is multiplied by a zero probability, which is only safe when it is finite: in the one
        // tile that reaches past the last atom the padded partners' rows may hold anything
        if (n - steplist[t] * kPart < kPart) {
#pragma unroll
          for (int e = 0; e < kC; ++e) dp[e] = ((word >> e) & 1u) ? dp[e] : 0u;
        }
        uint32_t pk_p[kC / 2], pk_ds[kC / 2];
#pragma unroll
        for (int e4 = 0; e4 < kC; e4 += 4) {
          float l4[4], d4[4];
          if (MODE == T_DQ) {
#pragma unroll
            for (int k = 0; k < 4; ++k) l4[k] = lse2, d4[k] = dlt;
          } else {  // per partner column (a query); all lanes of a warp read the same addresses
            float4 lv = make_float4(0.f, 0.f, 0.f, 0.f), dv = lv;  // (the token count is a multiple of four)
            if (kb + e4 < N) {
              lv = __ldg(reinterpret_cast<const float4*>(p.lse2 + (size_t)bh * N + kb + e4));
              dv = __ldg(reinterpret_cast<const float4*>(p.delta + (size_t)bh * N + kb + e4));
            }
            l4[0] = lv.x, l4[1] = lv.y, l4[2] = lv.z, l4[3] = lv.w;
            d4[0] = dv.x, d4[1] = dv.y, d4[2] = dv.z, d4[3] = dv.w;
          }
          float pr[4], ds[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int e = e4 + k;
            pr[k] = exp2_fast(fmaf(__uint_as_float(sv[e]), sc2, -l4[k]));  // 0 for hidden pairs
            ds[k] = pr[k] * fmaf(__uint_as_float(dp[e]), p.scale, -d4[k]);
          }
          pk_ds[e4 >> 1] = pack_bf16x2(ds[0], ds[1]);
          pk_ds[(e4 >> 1) + 1] = pack_bf16x2(ds[2], ds[3]);
          if (MODE == T_DKV) {
            pk_p[e4 >> 1] = pack_bf16x2(pr[0], pr[1]);
            pk_p[(e4 >> 1) + 1] = pack_bf16x2(pr[2], pr[3]);
          }
        }
        if (MODE == T_DKV) tmem_st_cols(tmem_row + Sh::kColS(buf) + col0, pk_p);
        tmem_st_cols(tmem_row + Sh::kColDP(buf) + col0, pk_ds);
        tmem_st_wait();
        tc_fence_before_sync();
        warp_arrive(&bar_p[buf]);
      }
    }

    // ---- write the owner rows
    if (MODE == T_FWD) {
      drain(nsteps - 1);
      xch[nsteps & 1][part][r] = l_run;
      named_barrier(1 + (warp & 3), 32 * Sh::kSplit);
      float l_row = 0.f;
#pragma unroll
      for (int q = 0; q < Sh::kSplit; ++q) l_row += xch[nsteps & 1][q][r];
      const bool have = row_ok && l_row > 0.f && !bad;
      const float inv = have ? 1.f / l_row : 0.f;
      if (orow < N) {
        uint4* o = reinterpret_cast<uint4*>(p.out + base + (size_t)orow * kHd + col0);
#pragma unroll
        for (int c = 0; c < kC / 8; ++c) {
          uint4 v;
          v.x = pack_bf16x2(o_acc[8 * c + 0] * inv, o_acc[8 * c + 1] * inv);
          v.y = pack_bf16x2(o_acc[8 * c + 2] * inv, o_acc[8 * c + 3] * inv);
          v.z = pack_bf16x2(o_acc[8 * c + 4] * inv, o_acc[8 * c + 5] * inv);
          v.w = pack_bf16x2(o_acc[8 * c + 6] * inv, o_acc[8 * c + 7] * inv);
          o[c] = have ? v : make_uint4(0, 0, 0, 0);
        }
        if (part == 0) p.lse_out[(size_t)bh * N + orow] = have ? (m_run + log2f(l_row)) * kLn2F : 0.f;
      }
    } else {
      wait_on(&bar_w[0], 0);
      tc_fence_after_sync();
      const bool have = row_ok && !bad;
#pragma unroll
      for (int which = 0; which < (MODE == T_DKV ? 2 : 1); ++which) {
        uint32_t w[kC];
        tmem_ld_cols(tmem_row + (which ? Sh::kColAcc1 : Sh::kColAcc0) + col0, w);
        tmem_ld_wait();
        __nv_bfloat16* dst = MODE == T_DQ ? p.dq : (which ? p.dv : p.dk);
        if (orow < N) {
          uint4* o = reinterpret_cast<uint4*>(dst + base + (size_t)orow * kHd + col0);
#pragma unroll
          for (int c = 0; c < kC / 8; ++c) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(w[8 * c + 0]), __uint_as_float(w[8 * c + 1]));
            v.y = pack_bf16x2(__uint_as_float(w[8 * c + 2]), __uint_as_float(w[8 * c + 3]));
            v.z = pack_bf16x2(__uint_as_float(w[8 * c + 4]), __uint_as_float(w[8 * c + 5]));
            v.w = pack_bf16x2(__uint_as_float(w[8 * c + 6]), __uint_as_float(w[8 * c + 7]));
            o[c] = have ? v : make_uint4(0, 0, 0, 0);
          }
        }
      }
      tc_fence_before_sync();
    }
  }

  tc_fence_before_sync();
  bad = __syncthreads_or(bad) != 0;
  if (bad && tid == 0) atomicExch(&g_sparse_tc_status, MF_ERR_DEVICE_TIMEOUT);
  if (warp == 0) tmem_dealloc(tmem, Sh::kTmemCols);
}

template <int MODE, bool kRadius>
int launch_one(const TcParams& p, int tiles, int BH, cudaStream_t s) {
  auto kern = sparse_tc_kernel<MODE, kRadius>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcShape<MODE>::kSmemAlloc);
  if (e != cudaSuccess) return cuda_error(e, "cudaFuncSetAttribute(sparse_tc_kernel)");
  kern<<<dim3(tiles, BH), TcShape<MODE>::kThreads, TcShape<MODE>::kSmemAlloc, s>>>(p);
  MF_CHECK_LAUNCH("sparse_tc_kernel");
  return MF_OK;
}

template <bool kRadius>
int run_tc(const MfSparseAttnArgs& a, bool backward, cudaStream_t s) {
  TcParams p{};
  p.grad_out = static_cast<const __nv_bfloat16*>(a.grad_out);
  p.out_in = static_cast<const __nv_bfloat16*>(a.out);
  p.lse_in = a.lse;
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
  p.T32 = (a.tokens + 31) / 32;
  p.scale = a.scale;
  p.delta = static_cast<float*>(a.workspace);
  p.lse2 = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + align_up((size_t)a.batch * a.heads * a.tokens * sizeof(float), 256));
  const int BH = a.batch * a.heads, tiles = (a.tokens + kOwn - 1) / kOwn;
  CUtensorMap tq, tk, tv, tdo;
  bool ok = make_rows_tensor_map(&tq, a.q, a.tokens, BH, kBoxRows) && make_rows_tensor_map(&tk, a.k, a.tokens, BH, kBoxRows) &&
            make_rows_tensor_map(&tv, a.v, a.tokens, BH, kBoxRows);
  if (backward) ok = ok && make_rows_tensor_map(&tdo, a.grad_out, a.tokens, BH, kBoxRows);
  if (!ok) {
    set_error("sparse attention (tcgen05): a tensor map could not be encoded (driver result %d; q %p k %p v %p dO %p, %d tokens, "
              "%d matrices)", last_tensor_map_result(), a.q, a.k, a.v, a.grad_out, a.tokens, BH);
    return MF_ERR_UNSUPPORTED;
  }
  if (!backward) {
    p.tm_own_a = tq, p.tm_own_b = tq, p.tm_part_a = tk, p.tm_part_b = tv;
    return launch_one<T_FWD, kRadius>(p, tiles, BH, s);
  }
  p.tm_own_a = tq, p.tm_own_b = tdo, p.tm_part_a = tk, p.tm_part_b = tv;
  int rc = launch_one<T_DQ, kRadius>(p, tiles, BH, s);  // also writes delta
  if (rc != MF_OK) return rc;
  p.tm_own_a = tk, p.tm_own_b = tv, p.tm_part_a = tq, p.tm_part_b = tdo;
  return launch_one<T_DKV, kRadius>(p, tiles, BH, s);
}

}  // namespace

bool sparse_attn_sm100_applies(const MfSparseAttnArgs& a, bool backward) {
  if (a.dtype != MF_DTYPE_BF16 || a.head_dim != kHd || a.tokens > kMaxPartTiles * kPart || !tensor_maps_available()) return false;
  if (a.tokens % 4) return false;  // the per-query statistics are read four at a time
  if (!(a.scale > 0.f)) return false;  // the row maximum is taken before the logits are scaled
  if ((long long)a.batch * a.heads > 65535) return false;
  const void* ptrs[] = {a.q, a.k, a.v, a.out, a.lse, backward ? a.grad_out : a.q, backward ? a.dq : a.q,
                        backward ? a.dk : a.q, backward ? a.dv : a.q, backward ? a.workspace : a.q};
  for (const void* q : ptrs)
    if (!aligned16(q)) return false;
  return true;
}
int sparse_attn_sm100_fwd(const MfSparseAttnArgs& a, bool radius, cudaStream_t stream) {
  return radius ? run_tc<true>(a, false, stream) : run_tc<false>(a, false, stream);
}
int sparse_attn_sm100_bwd(const MfSparseAttnArgs& a, bool radius, cudaStream_t stream) {
  return radius ? run_tc<true>(a, true, stream) : run_tc<false>(a, true, stream);
}
int sparse_attn_sm100_status(int32_t* host_status, cudaStream_t stream) {
  cudaError_t e = cudaMemcpyFromSymbolAsync(host_status, g_sparse_tc_status, sizeof(int32_t), 0, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_error(e, "sparse attention status read-back");
  return MF_OK;
}

}  // namespace mf
