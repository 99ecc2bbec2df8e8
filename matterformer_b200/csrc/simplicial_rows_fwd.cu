// 2-simplicial attention forward on the Blackwell tensor cores, row-packed and warp-specialised.
//
// Every row of the 128-row tcgen05 tile carries its own (query i, first key j) pair (see simplicial_rows.cuh):
// with A[r,:] = q[i_r,:] o k1[j_r,:] the trilinear logits of a step are one GEMM
//     S[r,k] = sum_d q[i_r,d] k1[j_r,d] k2[k,d] = (A . K2^T)[r,k]               (tcgen05.mma, fp32 in tensor memory)
// against the constant K2 tile, the softmax over the whole (j,k) plane runs online per row (running maximum and
// sum, as in flash attention) and
//     out[i,:] = sum_j v1[j,:] o (P_j . V2)[i,:]                                 (tcgen05.mma, A = P from tensor memory)
// is accumulated in registers while the 128x64 product is drained from tensor memory.  Rows that share a query
// (one per group of first keys) are merged at the end like the splits of a split-k softmax.
//
// Roles (640 threads): warps 0-15 own the rows, four threads per row, each taking every fourth 32-column chunk of
// the logits and a quarter of the output columns; one thread of warp 16 issues every tcgen05.mma; warp 17 runs ahead
// and stages the k1 / v1 rows of the coming steps in shared memory, so that no row owner waits on a global load
// (warps 18-19 only lend their registers).  The logits are
// double-buffered in tensor memory, so the GEMM of step s+1 runs under the softmax of step s and the P.V2
// product of step s under the softmax of step s+1.  Hand-offs are mbarriers; every wait is bounded and an
// expired wait is reported through the status word.
//
// Semantics follow simplicial_attention_torch_from_projected of the reference
// (src/matterformer/models/simplicial_attention.py:206-344); the interface is the one of
// triton_simplicial_attention_forward (src/matterformer/models/triton_simplicial_attention.py:790-926).
#include "common.cuh"
#include "simplicial.cuh"
#include "simplicial_rows.cuh"
#include "simplicial_sm100.cuh"
#include "sm100_primitives.cuh"
#include "tensor_map.cuh"

namespace mf {
namespace {

// A row is shared by kSplit threads, one in each of kSplit warps with the same lane quarter: every thread takes
// every kSplit-th 32-column chunk of the logits and 64 / kSplit of the output columns.  With four threads per row
// the CTA runs sixteen row-owner warps, four per scheduler: the kernel is bound by dependency stalls of the
// row owners' instruction streams (a warp issues once every six to seven clocks), not by any pipe, so the number of
// warps a scheduler can choose from is what sets its rate.
constexpr int kSplit = 4;
constexpr int kWorkerWarps = 4 * kSplit;
constexpr int kWorkers = 32 * kWorkerWarps;
constexpr int kFwdThreads = kWorkers + 128;  // + one warp group that holds the issuing warp and the loader warp
constexpr int kFwdIssuer = kWorkers;
constexpr int kLoaderWarp = kWorkerWarps + 1;
constexpr int kDc = kD / kSplit;                      // output columns per thread
constexpr int kCpt = (kMaxKeys / 32 + kSplit - 1) / kSplit;  // logit chunks per thread, at most
// registers: the launch gives every thread kRegLaunch; the aux warp group drops to kRegAux and the row owners
// take what that frees (setmaxnreg works per warp group, and a raise blocks until the registers exist in the CTA's pool)
constexpr int kRegLaunch = kSplit == 2 ? 168 : 96;
constexpr int kRegAux = 56;
constexpr int kRegWorker = kSplit == 2 ? 224 : 104;
static_assert(kWorkerWarps * kRegWorker + 4 * kRegAux <= (kWorkerWarps + 4) * kRegLaunch, "register hand-over exceeds the CTA's pool");
static_assert(kFwdThreads * kRegLaunch <= 65536, "launch registers exceed the register file");
constexpr int kFwdTmemCols = 512;
constexpr int kColS = 0;      // two logit buffers of 192 columns
constexpr int kColW = 384;    // two P.V2 buffers of 64 columns
constexpr int kMaskWords = kMaxKeys / 32;

// shared memory map (dynamic, 1024-byte aligned)
constexpr int kOffK2 = 0;                                   // [192][64] bf16 swizzled, K-major B operand
constexpr int kOffV2 = kOffK2 + kMaxKeys * 128;             // [192][64] bf16 swizzled, MN-major B operand
constexpr int kOffA = kOffV2 + kMaxKeys * 128;              // 2 stages x [128][64] bf16 swizzled: q_i o k1_j per row
constexpr int kRowStages = 8;  // steps the loader warp may run ahead; a step's rows stay live for four steps
constexpr int kOffK1 = kOffA + 2 * kTileM * 128;            // 8 stages x [8][64] bf16: k1 rows of a step's first keys
constexpr int kOffV1f = kOffK1 + kRowStages * kMaxGroups * kD * 2;  // 8 stages x [8][64] fp32: the v1 rows
constexpr int kOffPv = kOffV1f + kRowStages * kMaxGroups * kD * 4;  // [192][6] pair_valid bit rows
constexpr int kOffXch = kOffPv + kMaxKeys * kMaskWords * 4; // [2 steps][kSplit][128] row maxima, [kSplit][128] row sums
constexpr int kOffMl = kOffXch + 3 * kSplit * kTileM * 4;   // [128][2] running maximum / sum of every row (merge)
constexpr int kSmemBytes = kOffMl + 2 * kTileM * 4;
constexpr int kSmemAlloc = kSmemBytes + 1024;

struct RowsFwdParams {
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
  int H, N, tiles_max;
  int use_tma;
  CUtensorMap tm_k2;  // (B*H, N, 64) bf16, boxes of 32 rows, 128-byte swizzle
  CUtensorMap tm_v2;
};

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__global__ void __maxnreg__(kRegLaunch) simplicial_rows_fwd_kernel(const __grid_constant__ RowsFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar_a[2], bar_s[2], bar_p[2], bar_w[2], bar_kv;
  __shared__ uint64_t bar_full[kRowStages], bar_empty[kRowStages];  // loader warp <-> row owners
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t kmask[kMaskWords];
  __shared__ uint8_t jlist[kMaxKeys];

  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & 127, part = (tid >> 7) & (kSplit - 1);  // tile row, and which share of it this thread takes
  const int per_b = p.H * p.tiles_max;
  const int b = p.order[blockIdx.x / per_b];
  const int rem = blockIdx.x % per_b;
  const int h = rem / p.tiles_max, qt = rem % p.tiles_max;
  const int N = p.N;
  const int bh = b * p.H + h;
  const size_t base = (size_t)bh * N * kD;
  const int n_keys = p.info[b].n_keys;
  const int n_queries = p.info[b].n_queries;
  const int nj = p.info[b].reserved0;  // valid first keys
  const RowPlan plan = plan_rows(n_queries, nj);

  // ---- rows no tile covers (beyond the last valid query, or everything when nothing can be attended to)
  if (qt == 0) {
    const int z0 = plan.tiles > 0 ? n_queries : 0;
    for (int idx = tid; idx < (N - z0) * (kD / 4); idx += kFwdThreads)
      reinterpret_cast<float4*>(p.out + base + (size_t)z0 * kD)[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p.out_cast)
      for (int idx = tid; idx < (N - z0) * (kD / 8); idx += kFwdThreads)
        reinterpret_cast<uint4*>(p.out_cast + base + (size_t)z0 * kD)[idx] = make_uint4(0, 0, 0, 0);
    for (int idx = z0 + tid; idx < N; idx += kFwdThreads) p.lse[(size_t)bh * N + idx] = 0.f;
  }
  if (plan.tiles == 0 || qt >= plan.tiles) return;  // uniform per CTA

  const int rt = plan.rows_per_tile, G = plan.groups, steps = plan.steps;
  // MMA N of the logit GEMM: whole 32-column chunks, so that every column a row owner reads has been written
  // (keys beyond the last valid one have zero K2 / V2 rows: their logits are exactly 0, their products vanish)
  const int nk_pad = (n_keys + 31) & ~31;
  const int n_chunks = (nk_pad + 31) >> 5;

  // ---- set-up: barriers, tensor memory, key masks, first-key list, operand tiles
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_a[i], kWorkerWarps);  // one arrival per row-owner warp
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_p[i], kWorkerWarps);
      mbar_init(&bar_w[i], 1);
    }
    for (int i = 0; i < kRowStages; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_empty[i], kWorkerWarps);
    }
    mbar_init(&bar_kv, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, kFwdTmemCols);
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
  {
    uint32_t* pvbits_w = reinterpret_cast<uint32_t*>(smem + kOffPv);
    const uint8_t* pv = p.pair_valid ? p.pair_valid + (size_t)b * N * N : nullptr;
    for (int idx = tid; idx < n_keys * kMaskWords; idx += kFwdThreads) {
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
    // K2 / V2 tiles: bulk tensor copies of 32 rows each on one mbarrier (rows past the end of the matrix are
    // zero-filled by the copy engine, rows of invalid keys are cleared below), or plain loads.
    if (p.use_tma) {
      if (tid == 0) {
        mbar_arrive_expect_tx(&bar_kv, (uint32_t)n_chunks * 2u * kTmaBoxRows * 128u);
        for (int c = 0; c < n_chunks; ++c) {
          tma_load_rows(smem + kOffK2 + c * kTmaBoxRows * 128, &p.tm_k2, c * kTmaBoxRows, bh, &bar_kv);
          tma_load_rows(smem + kOffV2 + c * kTmaBoxRows * 128, &p.tm_v2, c * kTmaBoxRows, bh, &bar_kv);
        }
      }
    } else {
      for (int idx = tid; idx < n_chunks * 32 * 8; idx += kFwdThreads) {
        const int rr = idx >> 3, c = idx & 7;
        uint4 vk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
        if (rr < n_keys && ((kmask[rr >> 5] >> (rr & 31)) & 1u)) {
          vk = __ldg(reinterpret_cast<const uint4*>(p.k2 + base + (size_t)rr * kD) + c);
          vv = __ldg(reinterpret_cast<const uint4*>(p.v2 + base + (size_t)rr * kD) + c);
        }
        const uint32_t off = rr * 128 + ((c ^ (rr & 7)) << 4);
        *reinterpret_cast<uint4*>(smem + kOffK2 + off) = vk;
        *reinterpret_cast<uint4*>(smem + kOffV2 + off) = vv;
      }
    }
  }
  bool bad = false;
  if (p.use_tma) {
    bad |= !mbar_wait(&bar_kv, 0);
    if (!bad)  // rows of invalid keys must be zero whatever the padded tokens hold
      for (int idx = tid; idx < n_chunks * 32 * 8; idx += kFwdThreads) {
        const int rr = idx >> 3, c = idx & 7;
        if (!(rr < n_keys && ((kmask[rr >> 5] >> (rr & 31)) & 1u))) {
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

  auto wait_on = [&](uint64_t* bar, uint32_t ph) {
    if (!bad) bad = !mbar_wait(bar, ph);
  };

  if (warp >= kWorkerWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegAux));
  if (tid == kFwdIssuer) {
    // ------------------------------------------------------------------ issuer
    const uint32_t lA = make_desc_lo(smem_u32(smem + kOffA), 0), lK2 = make_desc_lo(smem_u32(smem + kOffK2), 0);
    const uint32_t lV2 = make_desc_lo(smem_u32(smem + kOffV2), kMaxKeys * 128);
    const uint32_t idesc_s = make_idesc_bf16(kTileM, nk_pad, false, false);
    const uint32_t idesc_w = make_idesc_bf16(kTileM, kD, false, true);
    auto issue_logits = [&](int s) {  // S(s) = A(s) . K2^T into logit buffer s & 1
      const int buf = s & 1;
      const uint32_t a = lA + buf * ((kTileM * 128) >> 4);
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) umma_ss_lo(tmem + kColS + buf * kMaxKeys, a + 2 * ks, lK2 + 2 * ks, idesc_s, ks > 0);
      umma_commit(&bar_s[buf]);
    };
    auto issue_pv = [&](int s) {  // W(s) = P(s) . V2; P sits packed over the first 16 columns of every 32-column chunk
      const int buf = s & 1;
      for (int kg = 0; kg < nk_pad / 16; ++kg)
        umma_ts_lo(tmem + kColW + buf * kD, tmem + kColS + buf * kMaxKeys + 32 * (kg >> 1) + 8 * (kg & 1), lV2 + 128 * kg,
                   idesc_w, kg > 0);
      umma_commit(&bar_w[buf]);
    };
    wait_on(&bar_a[0], 0);
    tc_fence_after_sync();
    issue_logits(0);
    for (int s = 0; s < steps; ++s) {
      if (s + 1 < steps) {
        wait_on(&bar_a[(s + 1) & 1], ((s + 1) >> 1) & 1);
        tc_fence_after_sync();
        issue_logits(s + 1);
      }
      wait_on(&bar_p[s & 1], (s >> 1) & 1);
      tc_fence_after_sync();
      issue_pv(s);
    }
  } else if (warp == kLoaderWarp) {
    // ------------------------------------------------------------------ loader
    // Stages, up to kRowStages steps ahead, the k1 rows of each step's first keys (bf16, for the operand build) and
    // the v1 rows as fp32 (for out += v1_j o W).  Lane l handles the 16-byte pieces l, l + 32, l + 64, l + 96.
    const int lane = tid & 31;
    float* v1f_w = reinterpret_cast<float*>(smem + kOffV1f);
    for (int s = 0; s < steps; ++s) {
      const int stg = s & (kRowStages - 1);
      if (s >= kRowStages) wait_on(&bar_empty[stg], ((s / kRowStages) - 1) & 1);
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
        if (which == 0) {
          *reinterpret_cast<uint4*>(smem + kOffK1 + (stg * kMaxGroups + gg) * (kD * 2) + part * 16) = v[q];
        } else {
          const uint32_t w4[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
          float f[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            f[2 * e] = __uint_as_float(w4[e] << 16);
            f[2 * e + 1] = __uint_as_float(w4[e] & 0xffff0000u);
          }
          float4* dst = reinterpret_cast<float4*>(v1f_w + (stg * kMaxGroups + gg) * kD + part * 8);
          dst[0] = make_float4(f[0], f[1], f[2], f[3]);
          dst[1] = make_float4(f[4], f[5], f[6], f[7]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_full[stg]);
    }
  }
  } else {
    // ------------------------------------------------------------------ row owners
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegWorker));
    const uint32_t tmem_row = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t* pvbits = reinterpret_cast<const uint32_t*>(smem + kOffPv);
    const int lane = tid & 31;
    const float* v1f = reinterpret_cast<const float*>(smem + kOffV1f);
    // one arrival per warp: every lane orders its own writes, the warp converges, one lane arrives
    auto warp_arrive = [&](uint64_t* bar) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };
    // the kSplit warps that share 32 rows meet at named barrier 1 + (lane quarter)
    auto row_barrier = [&]() { named_barrier(1 + (warp & 3), 32 * kSplit); };
    float* xmax = reinterpret_cast<float*>(smem + kOffXch);          // [2][kSplit][128]
    float* xsum = xmax + 2 * kSplit * kTileM;                         // [kSplit][128]
    float* ml = reinterpret_cast<float*>(smem + kOffMl);             // [128][2]
    const int g = r / rt, ii = r - g * rt;
    const bool slot_ok = g < G;
    const int i = qt * rt + ii;
    const bool row_ok = slot_ok && i < n_queries && p.query_valid[(size_t)b * N + i] > 0;
    // rows [G * rt, 128) never carry a pair: warps made of such rows only take part in the hand-offs
    const bool warp_live = (warp & 3) * 32 < G * rt;
    const int nc = (n_chunks - part + kSplit - 1) / kSplit;  // this thread's chunks: part, part + kSplit, ...

    // this thread's share of the query row as bf16x2 words
    uint32_t qreg[kDc / 2];
    {
      const uint4* qp = reinterpret_cast<const uint4*>(p.q + base + (size_t)(row_ok ? i : 0) * kD + kDc * part);
#pragma unroll
      for (int c = 0; c < kDc / 8; ++c) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row_ok) v = __ldg(qp + c);
        qreg[4 * c + 0] = v.x;
        qreg[4 * c + 1] = v.y;
        qreg[4 * c + 2] = v.z;
        qreg[4 * c + 3] = v.w;
      }
    }
    // operand rows of step s: A[r,:] = q_i o k1_j (zeros when the row has no pair in this step), this thread's columns
    auto build = [&](int s) {
      const int stg = s & (kRowStages - 1);
      wait_on(&bar_full[stg], (s / kRowStages) & 1);
      const int jj = s * G + g;
      const bool ok = row_ok && jj < nj;
      const uint4* kp = reinterpret_cast<const uint4*>(smem + kOffK1 + (stg * kMaxGroups + (slot_ok ? g : 0)) * (kD * 2) + 2 * kDc * part);
      uint8_t* dst = smem + kOffA + (s & 1) * (kTileM * 128) + r * 128;
#pragma unroll
      for (int c = 0; c < kDc / 8; ++c) {
        uint4 a = make_uint4(0, 0, 0, 0);
        if (ok) {
          const uint4 kk = kp[c];
          const uint32_t kw[4] = {kk.x, kk.y, kk.z, kk.w};
          uint32_t aw[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            __nv_bfloat162 m = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&qreg[4 * c + t]),
                                       *reinterpret_cast<const __nv_bfloat162*>(&kw[t]));
            aw[t] = *reinterpret_cast<uint32_t*>(&m);
          }
          a = make_uint4(aw[0], aw[1], aw[2], aw[3]);
        }
        *reinterpret_cast<uint4*>(dst + ((((kDc / 8) * part + c) ^ (r & 7)) << 4)) = a;
      }
      fence_smem_to_async_proxy();
      tc_fence_before_sync();
      warp_arrive(&bar_a[s & 1]);
    };
    // out = out * alpha + v1_j o W of step sp, this thread's kDc columns
    float o_acc[kDc];
#pragma unroll
    for (int d = 0; d < kDc; ++d) o_acc[d] = 0.f;
    float alpha_prev = 1.f;   // rescale factor of the step whose product is drained next
    auto drain = [&](int sp) {
      wait_on(&bar_w[sp & 1], (sp >> 1) & 1);
      tc_fence_after_sync();
      if (warp_live) {
        uint32_t w[kDc];
        if constexpr (kDc == 32) tmem_ld32(tmem_row + kColW + (sp & 1) * kD + kDc * part, reinterpret_cast<uint32_t(&)[32]>(w));
        else tmem_ld16(tmem_row + kColW + (sp & 1) * kD + kDc * part, reinterpret_cast<uint32_t(&)[16]>(w));
        const float4* vf = reinterpret_cast<const float4*>(v1f + ((sp & (kRowStages - 1)) * kMaxGroups + (slot_ok ? g : 0)) * kD + kDc * part);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < kDc / 4; ++c) {
          const float4 v = vf[c];
          o_acc[4 * c + 0] = fmaf(o_acc[4 * c + 0], alpha_prev, __uint_as_float(w[4 * c + 0]) * v.x);
          o_acc[4 * c + 1] = fmaf(o_acc[4 * c + 1], alpha_prev, __uint_as_float(w[4 * c + 1]) * v.y);
          o_acc[4 * c + 2] = fmaf(o_acc[4 * c + 2], alpha_prev, __uint_as_float(w[4 * c + 2]) * v.z);
          o_acc[4 * c + 3] = fmaf(o_acc[4 * c + 3], alpha_prev, __uint_as_float(w[4 * c + 3]) * v.w);
        }
        tc_fence_before_sync();
      }
    };

    float m_run = -INFINITY;  // running maximum in the log2 domain (shared by the threads of a row)
    float l_run = 0.f;        // this thread's part of the running sum

    build(0);
    if (steps > 1) build(1);
    for (int s = 0; s < steps; ++s) {
      const int buf = s & 1;
      const uint32_t srow = tmem_row + kColS + buf * kMaxKeys;
      wait_on(&bar_s[buf], (s >> 1) & 1);
      tc_fence_after_sync();
      const int jj = s * G + g;
      const bool ok = row_ok && jj < nj;
      const uint32_t* pvrow = pvbits + MF_IDX((ok ? jlist[MF_IDX(jj, kMaxKeys, p.status)] : 0) * kMaskWords, kMaxKeys * kMaskWords, p.status);
      float alpha = 1.f;
      // ---- first pass over this thread's chunks: the row maximum (the logits are read again for the exponentials,
      // which costs a tensor-memory load and saves 32 registers per chunk)
      uint32_t word[kCpt];
      float mx = -INFINITY;
      if (warp_live) {
#pragma unroll
        for (int t = 0; t < kCpt; ++t) {
          word[t] = 0;
          if (t < nc) {
            const int c = part + kSplit * t;
            uint32_t sv[32];
            tmem_ld32(srow + 32 * c, sv);
            word[t] = ok ? (kmask[c] & pvrow[c]) : 0u;
            tmem_ld_wait();
            // Only invalid keys are hidden (the pair mask removes nothing here): their K2 rows are zero, so their
            // logits are exact zeros and the plain maximum is right whenever it is positive.
            bool plain = word[t] == kmask[c] && word[t] != 0u;
            float c4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // independent chains keep the dependency depth low
            if (plain) {
#pragma unroll
              for (int e = 0; e < 32; e += 2)
                c4[(e >> 1) & 3] = max3(c4[(e >> 1) & 3], __uint_as_float(sv[e]), __uint_as_float(sv[e + 1]));
              const float cm = fmaxf(fmaxf(c4[0], c4[1]), fmaxf(c4[2], c4[3]));
              if (word[t] == 0xffffffffu || cm > 0.f) mx = fmaxf(mx, cm);
              else plain = false;  // the maximum may come from a padded column: take the exact path
            }
            if (!plain && word[t] != 0u) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) c4[q4] = -INFINITY;
#pragma unroll
              for (int e = 0; e < 32; e += 2)
                c4[(e >> 1) & 3] = max3(c4[(e >> 1) & 3], ((word[t] >> e) & 1u) ? __uint_as_float(sv[e]) : -INFINITY,
                                        ((word[t] >> (e + 1)) & 1u) ? __uint_as_float(sv[e + 1]) : -INFINITY);
              mx = fmaxf(mx, fmaxf(fmaxf(c4[0], c4[1]), fmaxf(c4[2], c4[3])));
            }
          }
        }
      }
      xmax[(buf * kSplit + part) * kTileM + r] = mx;
      row_barrier();
      if (warp_live) {
#pragma unroll
        for (int q4 = 0; q4 < kSplit; ++q4) mx = fmaxf(mx, xmax[(buf * kSplit + q4) * kTileM + r]);
        const float m_new = fmaxf(m_run, mx * kLog2e);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_use);
        m_run = m_new;
        // ---- second pass: P = exp2(S log2e - m), packed to bf16 over the first 16 columns of the chunk it came from
        float psum = 0.f;
#pragma unroll
        for (int t = 0; t < kCpt; ++t) {
          if (t < nc) {
            const int c = part + kSplit * t;
            uint32_t pk[16];
            uint32_t sv[32];
            tmem_ld32(srow + 32 * c, sv);  // (by whole warps: a tensor-memory load must not sit under a per-lane condition)
            tmem_ld_wait();
            if (word[t] == 0u) {
#pragma unroll
              for (int e = 0; e < 16; ++e) pk[e] = 0u;
            } else {
              float ps0 = 0.f, ps1 = 0.f;
              if (word[t] == kmask[c] && m_use > -64.f) {  // (the bound keeps exp2(-m) finite)
                // only invalid keys are hidden: no per-column selects.  Their logits are exact zeros, so each adds
                // exp2(-m) to the plain sum (taken off again below) and nothing to P.V2 (their V2 rows are zero).
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                  const float p0 = fast_exp2(fmaf(__uint_as_float(sv[e]), kLog2e, -m_use));
                  const float p1 = fast_exp2(fmaf(__uint_as_float(sv[e + 1]), kLog2e, -m_use));
                  ps0 += p0;
                  ps1 += p1;
                  pk[e >> 1] = pack_bf16x2(p0, p1);
                }
                psum += ps0 + ps1;
                if (word[t] != 0xffffffffu) psum = fmaf(-(float)(32 - __popc(word[t])), fast_exp2(-m_use), psum);
              } else {
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                  float p0 = fast_exp2(fmaf(__uint_as_float(sv[e]), kLog2e, -m_use));
                  float p1 = fast_exp2(fmaf(__uint_as_float(sv[e + 1]), kLog2e, -m_use));
                  p0 = ((word[t] >> e) & 1u) ? p0 : 0.f;
                  p1 = ((word[t] >> (e + 1)) & 1u) ? p1 : 0.f;
                  ps0 += p0;
                  ps1 += p1;
                  pk[e >> 1] = pack_bf16x2(p0, p1);
                }
                psum += ps0 + ps1;
              }
            }
            tmem_st16(srow + 32 * c, pk);
          }
        }
        l_run = l_run * alpha + psum;
        tmem_st_wait();
      }
      tc_fence_before_sync();
      warp_arrive(&bar_p[buf]);

      // ---- out = out * alpha + v1_j o W of the previous step, whose product has long finished
      if (s >= 1) {
        drain(s - 1);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_empty[(s - 1) & (kRowStages - 1)]);  // the step's staged rows are free
      }
      alpha_prev = alpha;
      if (s + 2 < steps) build(s + 2);
    }
    drain(steps - 1);  // the last step's product

    // ---- epilogue: the row's sum from its threads, then the rows of one query merged over the groups
    xsum[part * kTileM + r] = l_run;
    row_barrier();
    float l_row = 0.f;
#pragma unroll
    for (int q4 = 0; q4 < kSplit; ++q4) l_row += xsum[q4 * kTileM + r];
    float m_row = m_run;
    if (G > 1) {
      float* ostage = reinterpret_cast<float*>(smem + kOffA);  // [128][64] fp32; every product has completed
      named_barrier(5, kWorkers);
      if (part == 0) {
        ml[2 * r] = m_row;
        ml[2 * r + 1] = l_row;
      }
#pragma unroll
      for (int c = 0; c < kDc / 4; ++c)  // float4 index rotated by the row to spread the banks
        reinterpret_cast<float4*>(ostage + r * kD)[((kDc / 4) * part + c) ^ (r & 15)] =
            make_float4(o_acc[4 * c], o_acc[4 * c + 1], o_acc[4 * c + 2], o_acc[4 * c + 3]);
      named_barrier(5, kWorkers);
      if (g == 0) {
        float m_all = -INFINITY;
        for (int gg = 0; gg < G; ++gg) m_all = fmaxf(m_all, ml[2 * (gg * rt + r)]);
        float l_all = 0.f;
#pragma unroll
        for (int d = 0; d < kDc; ++d) o_acc[d] = 0.f;
        for (int gg = 0; gg < G; ++gg) {  // fixed order
          const int r2 = gg * rt + r;
          const float mg = ml[2 * r2];
          const float sc = (mg == -INFINITY) ? 0.f : fast_exp2(mg - m_all);
          l_all = fmaf(ml[2 * r2 + 1], sc, l_all);
#pragma unroll
          for (int c = 0; c < kDc / 4; ++c) {
            const float4 v = reinterpret_cast<const float4*>(ostage + r2 * kD)[((kDc / 4) * part + c) ^ (r2 & 15)];
            o_acc[4 * c + 0] = fmaf(v.x, sc, o_acc[4 * c + 0]);
            o_acc[4 * c + 1] = fmaf(v.y, sc, o_acc[4 * c + 1]);
            o_acc[4 * c + 2] = fmaf(v.z, sc, o_acc[4 * c + 2]);
            o_acc[4 * c + 3] = fmaf(v.w, sc, o_acc[4 * c + 3]);
          }
        }
        m_row = m_all;
        l_row = l_all;
      }
    }
    if (g == 0 && i < n_queries) {
      const bool have = row_ok && l_row > 0.f && !bad;
      const float inv = have ? 1.f / l_row : 0.f;
      float4* o = reinterpret_cast<float4*>(p.out + base + (size_t)i * kD + kDc * part);
#pragma unroll
      for (int c = 0; c < kDc / 4; ++c)
        o[c] = make_float4(have ? o_acc[4 * c] * inv : 0.f, have ? o_acc[4 * c + 1] * inv : 0.f,
                           have ? o_acc[4 * c + 2] * inv : 0.f, have ? o_acc[4 * c + 3] * inv : 0.f);
      if (p.out_cast) {
        uint4* oc = reinterpret_cast<uint4*>(p.out_cast + base + (size_t)i * kD + kDc * part);
#pragma unroll
        for (int c = 0; c < kDc / 8; ++c) {
          uint4 v;
          v.x = have ? pack_bf16x2(o_acc[8 * c + 0] * inv, o_acc[8 * c + 1] * inv) : 0u;
          v.y = have ? pack_bf16x2(o_acc[8 * c + 2] * inv, o_acc[8 * c + 3] * inv) : 0u;
          v.z = have ? pack_bf16x2(o_acc[8 * c + 4] * inv, o_acc[8 * c + 5] * inv) : 0u;
          v.w = have ? pack_bf16x2(o_acc[8 * c + 6] * inv, o_acc[8 * c + 7] * inv) : 0u;
          oc[c] = v;
        }
      }
      if (part == 0) p.lse[(size_t)bh * N + i] = have ? (m_row + log2f(l_row)) * kLn2 : 0.f;
    }
  }

  tc_fence_before_sync();
  bad = __syncthreads_or(bad) != 0;
  if (bad && tid == 0) atomicExch(p.status, MF_ERR_DEVICE_TIMEOUT);
  if (warp == 0) tmem_dealloc(tmem, kFwdTmemCols);
}

}  // namespace

int simplicial_rows_fwd(const MfSimplicialFwdArgs& a, cudaStream_t stream) {
  size_t info_off, order_off;
  simplicial_schedule_layout(a.batch, &info_off, &order_off);
  char* ws = static_cast<char*>(a.workspace);
  RowsFwdParams p{};
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
  p.tiles_max = cached_max_row_tiles(a.tokens);
  p.use_tma = make_rows_tensor_map(&p.tm_k2, a.k2, a.tokens, a.batch * a.heads) &&
              make_rows_tensor_map(&p.tm_v2, a.v2, a.tokens, a.batch * a.heads);
  int rc = launch_schedule(a.query_valid, a.pair_key_valid, a.batch, a.tokens, info, order, p.status, stream);
  if (rc != MF_OK) return rc;
  {
    cudaError_t e = cudaFuncSetAttribute(simplicial_rows_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
    if (e != cudaSuccess) return cuda_error(e, "cudaFuncSetAttribute(simplicial_rows_fwd_kernel)");
  }
  const long long blocks = (long long)a.batch * a.heads * p.tiles_max;
  profile_mark(MF_PROFILE_SIMPLICIAL_FWD, true, stream);
  simplicial_rows_fwd_kernel<<<(unsigned)blocks, kFwdThreads, kSmemAlloc, stream>>>(p);
  profile_mark(MF_PROFILE_SIMPLICIAL_FWD, false, stream);
  MF_CHECK_LAUNCH("simplicial_rows_fwd_kernel");
  return MF_OK;
}

}  // namespace mf
