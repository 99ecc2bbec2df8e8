// Interface between the C-ABI layer of the sparse attention operators and their tensor-core (mma.sync, bf16)
// kernels, plus the warp-level MMA helpers those kernels use.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/matterformer_b200.h"

namespace mf {

// bf16 inputs, head_dim 32 / 64 / 128.  `radius` selects the block-list variant, otherwise the band variant.
int sparse_attn_mma_fwd(const MfSparseAttnArgs& a, bool radius, cudaStream_t stream);
int sparse_attn_mma_bwd(const MfSparseAttnArgs& a, bool radius, cudaStream_t stream);
// The band variant with rows that are not (B,H,N,D) contiguous: `in` for q, k, v, dq, dk, dv; `act` for out, grad_out.
struct RowLayout;
int local_attn_mma_layouts(const MfSparseAttnArgs& a, const RowLayout& in, const RowLayout& act, bool backward,
                           cudaStream_t stream);

// ---- warp-level tensor-core helpers (m16n8k16, bf16 operands, fp32 accumulate) ---------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
// d (16x8, fp32) += a (16x16, row) * b (16x8, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr, bool valid) {
  const int bytes = valid ? 16 : 0;  // zero-fill when the source row does not exist
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace mf
