/*
 * matterformer_b200 -- C ABI of the B200 (sm_100a) attention kernels.
 *
 * Conventions shared by every entry point
 *  - All tensor pointers are DEVICE pointers to contiguous row-major arrays
 *    whose shapes are given in the comments; sizes are plain integers.
 *  - The caller owns every buffer (inputs, outputs and workspaces) and keeps it
 *    alive until the work enqueued on `stream` has completed.  Unless an entry
 *    point says otherwise the library allocates nothing, frees nothing and
 *    keeps no pointer after it returns.
 *  - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the
 *    call returns without synchronising.
 *  - Return value: 0 on success, a negative MF_ERR_* code otherwise; the text
 *    of the last error on the calling thread is returned by mf_last_error().
 *  - Entry points are re-entrant.  Global state: a per-device cache of driver attributes and of the address of the
 *    built-in scratch of mf_simplicial_fwd_noalloc (written once per device, under a lock), a lazily filled table of
 *    grid bounds, and the kernel-timing aid of mf_profile_enable / mf_profile_read (event lists under a lock; off by
 *    default).
 *  - Tensors are read and written with 16-byte vector accesses: every tensor pointer must be 16-byte aligned.  The
 *    simplicial entry points send problems with unaligned tensors to the element-wise CUDA-core kernel; every other
 *    entry point returns MF_ERR_INVALID_ARGUMENT.
 *  - "ref:" comments name the interface of the reference implementation
 *    (stases/Matterformer, paths relative to that project) that the entry point
 *    replaces or, where the reference has no such operator, the reference
 *    primitives whose composition defines its semantics.
 */
#ifndef MATTERFORMER_B200_H_
#define MATTERFORMER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MF_OK 0
#define MF_ERR_INVALID_ARGUMENT (-1)
#define MF_ERR_UNSUPPORTED (-2)
#define MF_ERR_WORKSPACE_TOO_SMALL (-3)
#define MF_ERR_CUDA (-4)
#define MF_ERR_DEVICE_TIMEOUT (-5)
#define MF_ERR_BOUNDS (-6) /* status-word value only: a debug build (-DMF_DEBUG_BOUNDS) saw an index out of range */

/* element types of q/k/v style tensors */
#define MF_DTYPE_F32 0
#define MF_DTYPE_BF16 1
#define MF_DTYPE_F16 2

/* ref: SUPPORTED_SIMPLICIAL_PRECISIONS, src/matterformer/models/triton_simplicial_attention.py:13 */
#define MF_PRECISION_BF16_TC 0
#define MF_PRECISION_TF32 1
#define MF_PRECISION_IEEE_FP32 2

/* Which implementation a simplicial call is allowed to use. */
#define MF_BACKEND_AUTO 0    /* tensor-core (tcgen05) kernel when the problem qualifies, else the fp32 CUDA-core kernel */
#define MF_BACKEND_GENERIC 1 /* always the fp32 CUDA-core kernel */
#define MF_BACKEND_TCGEN05 2 /* tensor-core kernel (row-packed) or MF_ERR_UNSUPPORTED */
#define MF_BACKEND_TCGEN05_TILES 3 /* tensor-core kernels with one query per tile row, or MF_ERR_UNSUPPORTED */

/* ------------------------------------------------------------------------- */
/* 2-simplicial attention                                                     */
/* ------------------------------------------------------------------------- */

/*
 * Arguments of the forward pass.
 * ref: triton_simplicial_attention_forward(q,k1,v1,k2,v2,*,query_valid,pair_key_valid,pair_valid,u,v_bias,w,gate,
 *      angle_*,message_*,precision) -> (out, lse, out_fp32),
 *      src/matterformer/models/triton_simplicial_attention.py:790-926.
 *
 * logits[b,h,i,j,k] = sum_d q[b,h,i,d] k1[b,h,j,d] k2[b,h,k,d]   (q arrives pre-scaled)
 * pair (j,k) visible iff pair_key_valid[b,j] && pair_key_valid[b,k] && (pair_valid == NULL || pair_valid[b,j,k])
 * attn = softmax over visible (j,k); out[b,h,i,:] = sum_jk attn v1[b,h,j,:] * v2[b,h,k,:]
 * A query that is invalid or sees no pair gets out = 0 and lse = 0.
 */
typedef struct MfSimplicialFwdArgs {
  int32_t batch, heads, tokens, head_dim;
  int32_t dtype;     /* MF_DTYPE_* of q,k1,v1,k2,v2 and out_cast */
  int32_t precision; /* MF_PRECISION_* */
  int32_t backend;   /* MF_BACKEND_* */
  int32_t reserved0;
  const void* q;  /* (B,H,N,D) */
  const void* k1; /* (B,H,N,D) */
  const void* v1; /* (B,H,N,D) */
  const void* k2; /* (B,H,N,D) */
  const void* v2; /* (B,H,N,D) */
  const uint8_t* query_valid;    /* (B,N) bytes, >0 = valid */
  const uint8_t* pair_key_valid; /* (B,N) */
  const uint8_t* pair_valid;     /* (B,N,N) or NULL */
  /* Geometry-bias operands of the reference interface (u, v_bias, w, gate, angle_*, message_*).
   * Factorized bias: logits += gate[b,h,i] * (u[b,h,i,j] + v_bias[b,h,i,k] + w[b,h,j,k]); the four
   * tensors are fp32, contiguous, u / v_bias / w of shape (B,H,N,N) and gate of shape (B,H,N), and are
   * given all together or not at all.  A bf16 call with them (head_dim 64, at most 192 tokens, no residual
   * operands) runs on the tcgen05 tile kernels, which sum the three terms in fp32 before adding them to the logit;
   * any other call with them runs on the CUDA-core kernel.
   * Low-rank angle residual: logits += angle_gate[b,h,i] * R^-1/2 * sum_r angle_left[b,h,i,j,r] *
   * angle_right[b,h,i,k,r]; low-rank message residual: out[b,h,i,:] += R^-1/2 * sum_r (sum_jk attn *
   * message_left[b,h,i,j,r] * message_right[b,h,i,k,r]) * message_basis[h,r,:]  (simplicial_attention.py:50-104,
   * 330-337).  fp32, contiguous, (B,H,N,N,R) / (B,H,N) / (H,R,D), ranks at most 32; each group is given
   * complete or not at all.  Calls with a residual operand run on the CUDA-core kernel. */
  const float* u;
  const float* v_bias;
  const float* w;
  const float* gate;
  const float* angle_left;
  const float* angle_right;
  const float* angle_gate;
  const float* message_left;
  const float* message_right;
  const float* message_basis;
  int32_t angle_rank, message_rank;
  float* out;     /* (B,H,N,D) fp32, written for every row (zeros where invalid) */
  float* lse;     /* (B,H,N)   fp32 natural-log sum of exp over visible pairs */
  void* out_cast; /* optional (B,H,N,D) copy of out in `dtype`; may be NULL */
  void* workspace; /* mf_simplicial_fwd_workspace_bytes() bytes, 256-byte aligned; may be NULL when that is 0 */
  size_t workspace_bytes;
} MfSimplicialFwdArgs;

/*
 * Arguments of the backward pass.
 * ref: triton_simplicial_attention_backward(grad_out,q,k1,v1,k2,v2,out,lse,*,masks,...,need_*) -> 15-tuple,
 *      src/matterformer/models/triton_simplicial_attention.py:929-1204.
 * Gradients are written for every row: rows of padded tokens receive exact zeros.
 * The reduction order is fixed, so results are bit-identical from run to run.
 */
typedef struct MfSimplicialBwdArgs {
  int32_t batch, heads, tokens, head_dim;
  int32_t dtype;
  int32_t precision;
  int32_t backend;
  int32_t reserved0;
  const void* grad_out; /* (B,H,N,D) in `dtype` */
  const void* q;
  const void* k1;
  const void* v1;
  const void* k2;
  const void* v2;
  const float* out; /* (B,H,N,D) fp32 saved by the forward pass */
  const float* lse; /* (B,H,N) fp32 saved by the forward pass */
  const uint8_t* query_valid;
  const uint8_t* pair_key_valid;
  const uint8_t* pair_valid; /* or NULL */
  void* dq; /* (B,H,N,D) in `dtype` */
  void* dk1;
  void* dv1;
  void* dk2;
  void* dv2;
  void* workspace; /* mf_simplicial_bwd_workspace_bytes() bytes, 256-byte aligned */
  size_t workspace_bytes;
  /* Factorized bias of the forward call (all four or none, fp32, same shapes) and the gradients
   * the reference returns for it (triton_simplicial_attention.py:929-1204, outputs du, dv, dw, dgate).
   * du, dv_bias, dw are (B,H,N,N) fp32, dgate is (B,H,N) fp32; the caller zero-fills them, the call
   * writes the entries of visible (query, key) combinations.  Each may be NULL when not needed. */
  const float* u;
  const float* v_bias;
  const float* w;
  const float* gate;
  float* du;
  float* dv_bias;
  float* dw;
  float* dgate;
  /* Low-rank residuals of the forward call and their gradients, same shapes, fp32, zero-filled by the caller;
   * each output may be NULL.  message_coeff (B,H,N,message_rank) receives R^-1/2 sum_jk attn * message_left *
   * message_right, from which the caller forms d message_basis[h,r,:] = sum_{b,i} message_coeff[b,h,i,r] *
   * grad_out[b,h,i,:].  With the message residual the workspace grows (mf_simplicial_bwd_workspace_bytes). */
  const float* angle_left;
  const float* angle_right;
  const float* angle_gate;
  const float* message_left;
  const float* message_right;
  const float* message_basis;
  int32_t angle_rank, message_rank;
  float* dangle_left;
  float* dangle_right;
  float* dangle_gate;
  float* dmessage_left;
  float* dmessage_right;
  float* message_coeff;
} MfSimplicialBwdArgs;

/* Bytes of scratch the calls below need for these sizes (0 is possible). */
size_t mf_simplicial_fwd_workspace_bytes(const MfSimplicialFwdArgs* args);
size_t mf_simplicial_bwd_workspace_bytes(const MfSimplicialBwdArgs* args);

/* Which kernel family a call with these arguments runs on: MF_BACKEND_TCGEN05 or MF_BACKEND_GENERIC.  (No counterpart
 * in the reference.)  Only the tensor-core kernels leave a status word at the start of the workspace. */
int mf_simplicial_fwd_backend(const MfSimplicialFwdArgs* args);
int mf_simplicial_bwd_backend(const MfSimplicialBwdArgs* args);

/* How the row-packed tensor-core kernels lay a molecule with `n_queries` queries (1 + index of the last valid
 * one) and `valid_keys` valid keys onto 128-row tiles: plan[0] = query ranges, plan[1] = queries per range,
 * plan[2] = first keys handled per step, plan[3] = steps per range (all 0 when either count is 0).  Host-only
 * arithmetic, the same function the kernels evaluate; exported so that callers can size and balance batches by
 * attention cost (ranges * steps tile-steps per molecule and head).  (No counterpart in the reference.) */
int mf_simplicial_row_plan(int32_t n_queries, int32_t valid_keys, int32_t plan[4]);

/* ref: triton_simplicial_attention_forward, triton_simplicial_attention.py:790-926 */
int mf_simplicial_fwd(const MfSimplicialFwdArgs* args, void* stream);
/* ref: triton_simplicial_attention_backward, triton_simplicial_attention.py:929-1204 */
int mf_simplicial_bwd(const MfSimplicialBwdArgs* args, void* stream);

/*
 * Forward pass that allocates nothing and needs no caller workspace.  (No counterpart in the reference.)
 *
 * For callers that cannot hand the library scratch memory because they cannot allocate any: code embedded in
 * another runtime's memory pool, loops that must stay off the allocator once they are running, or hosts whose
 * allocator has been shut down or frozen.  They pass inputs and outputs only; `workspace` / `workspace_bytes`
 * of the struct are ignored.  The scratch the tensor-core kernel needs (status word, per-molecule extents, launch
 * order) lives in an array that is part of the library image on every GPU that loads it, sized for at most 4096
 * molecules per call; a larger `batch` is rejected with MF_ERR_INVALID_ARGUMENT.  Only problems the tensor-core
 * forward kernel takes are accepted (bf16, precision bf16_tc, head_dim 64, tokens <= 192; otherwise
 * MF_ERR_UNSUPPORTED -- such problems need no scratch in mf_simplicial_fwd anyway).
 *
 * The first call on each device looks up the array's device address, so make that first call outside any stream
 * capture.  All calls on a device share the one array: calls whose kernels may overlap on the GPU (different
 * streams, different host threads) race on it and must be serialised by the caller.  The array keeps the previous
 * call's contents; the only part that must start at zero, the status word, is cleared by the call itself.
 * Results are identical to mf_simplicial_fwd.
 */
int mf_simplicial_fwd_noalloc(const MfSimplicialFwdArgs* args, void* stream);

/* The status word that the last mf_simplicial_fwd_noalloc call on the current device left in the built-in scratch
 * (MF_OK, or MF_ERR_DEVICE_TIMEOUT when a bounded device-side wait gave up), copied into *host_status by one
 * asynchronous copy on `stream`; synchronise the stream before reading it.  Allocates nothing.  (No counterpart in
 * the reference.) */
int mf_simplicial_noalloc_status(int32_t* host_status, void* stream);

/* Self-test of the bounded device-side waits (no counterpart in the reference).  Launches one warp that waits, with
 * `limit_cycles` SM clocks as its limit instead of the production limit of about a second, on a barrier that is
 * never signalled.  The wait gives up, the kernel writes MF_ERR_DEVICE_TIMEOUT to status[0] and the clocks it
 * waited to status[1] (two device int32) and returns: the path every tensor-core kernel takes when a hand-off never
 * arrives, exercised without hanging or faulting anything. */
int mf_selftest_wait_timeout(int32_t* status, int64_t limit_cycles, void* stream);

/* ------------------------------------------------------------------------- */
/* Periodic geometry: kNN, cell sort, radius block list                       */
/* ------------------------------------------------------------------------- */

/*
 * Minimum-image squared distance used by every geometry entry point (and by the
 * CPU oracle, operation for operation, so integer results are bit-exact):
 *   delta = (x_i - x_j) + offset            fractional, offset in {-1,0,1}^3
 *   r_x = fma(delta_2, L20, fma(delta_1, L10, delta_0 * L00))
 *   r_y = fma(delta_2, L21, delta_1 * L11)
 *   r_z = delta_2 * L22
 *   d2  = fma(r_z, r_z, fma(r_y, r_y, r_x * r_x))
 * minimised over the 27 offsets visited in the order (-1,-1,-1), (-1,-1,0), ... (1,1,1)
 * with the first minimum winning, where L is the lower-triangular cell whose rows are
 * the lattice vectors.
 * ref: PeriodicGeometryAdapter.forward, src/matterformer/geometry/adapters.py:176-190
 *      (offset order :141-149, first-minimum argmin :185); cell from
 *      lattice_latent_to_lower_triangular, src/matterformer/geometry/lattice.py:12-62.
 */

/*
 * Periodic k nearest neighbours of every atom.
 * ref: the reference's active package has no kNN operator; semantics = ascending stable sort of the
 *      minimum-image distances above (adapters.py:176-190) with self excluded, first k kept; the only
 *      kNN statement in the project is the non-periodic legacy/rapidash_v5/models/rapidash_utils.py:139-193.
 * frac (B,N,3) fp32 fractional coordinates; cell (B,3,3) fp32 lower-triangular; num_atoms (B) int32
 * (atoms [0,num_atoms[b]) are real).  Outputs idx (B,N,k) int32 and dist2 (B,N,k) fp32 (may be NULL),
 * sorted by (d2, index); missing neighbours and rows of padded atoms hold -1 / +inf.  1 <= k <= 32.
 */
int mf_knn_topk(const float* frac, const float* cell, const int32_t* num_atoms, int32_t batch, int32_t n_max,
                int32_t k, int32_t include_self, int32_t* idx, float* dist2, void* stream);

/*
 * The same k nearest neighbours, bit for bit, found with a cell list instead of all pairs.
 * ref: as mf_knn_topk.
 * grid_dims (B,3) int32: bins per axis, each in [1,16]; bounds (B,2) fp32: [min over axes of (perpendicular cell
 * width / bins on that axis), half the smallest perpendicular width], both rounded DOWN (they are used as lower
 * bounds on distances to atoms that were not visited).  workspace: mf_knn_cells_workspace_bytes().
 * Structures with a coordinate outside [0,1) are searched exhaustively.
 * mf_knn_search_grid fills grid_dims and bounds from the cell and the atom count (bin edge about 1.25x the radius
 * of a sphere that holds k atoms at the mean density).
 */
int mf_knn_search_grid(const float* cell, const int32_t* num_atoms, int32_t batch, int32_t n_max, int32_t k,
                       int32_t* grid_dims, float* bounds, void* stream);
size_t mf_knn_cells_workspace_bytes(int32_t batch, int32_t n_max);
int mf_knn_topk_cells(const float* frac, const float* cell, const int32_t* num_atoms, const int32_t* grid_dims,
                      const float* bounds, int32_t batch, int32_t n_max, int32_t k, int32_t include_self,
                      int32_t* idx, float* dist2, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Cell sort + radius block list.
 * ref: no counterpart in the reference; the per-pair criterion is sqrt(min-image d2) <= cutoff with the
 *      distances of adapters.py:176-190, self pair included (d = 0).
 * Atoms are binned on a grid of grid_dims[b] = (gx,gy,gz) cells over the wrapped fractional coordinates,
 * sorted by (linear cell index, original index) and cut into tiles of 32 consecutive sorted atoms.
 * Outputs (T = ceil(n_max/32)):
 *   perm        (B,N)      int32  original index of the s-th sorted atom (padding: identity tail)
 *   block_count (B,T)      int32  number of active column tiles of each row tile
 *   block_cols  (B,T,T)    int32  ascending active column tiles, -1 padded
 *   block_mask  (B,T,T,32) uint32 for column tile J (dense index, not list position): bit c of word r is set
 *                                 iff sorted atoms 32*I+r and 32*J+c are both real and within the cutoff
 * A block is active iff its mask has a set bit.  workspace: mf_radius_blocks_workspace_bytes().
 */
size_t mf_radius_blocks_workspace_bytes(int32_t batch, int32_t n_max);
int mf_cell_sort_blocklist(const float* frac, const float* cell, const int32_t* num_atoms, const int32_t* grid_dims,
                           int32_t batch, int32_t n_max, float cutoff, int32_t* perm, int32_t* block_count,
                           int32_t* block_cols, uint32_t* block_mask, void* workspace, size_t workspace_bytes,
                           void* stream);

/* ------------------------------------------------------------------------- */
/* Radius block-sparse attention and local-window attention                   */
/* ------------------------------------------------------------------------- */

/*
 * Softmax attention restricted to the pairs of a radius block list, tokens in cell-sorted order.
 * ref: composition of reference primitives -- additive 0/finfo.min mask from the min-image distances fed to
 *      F.scaled_dot_product_attention as RotaryMultiheadAttention.forward does,
 *      src/matterformer/models/regular_attention.py:251-268, scale head_dim^-1/2.
 * q,k,v,out (B,H,N,D) in `dtype` (bf16/f16/f32), D in {32,64,128}; lse (B,H,N) fp32; rows without any
 * visible key give out = 0, lse = 0.
 */
#define MF_SPARSE_BACKEND_AUTO 0    /* tcgen05 tiles for radius lists over >= 256 tokens, else warp-level tiles */
#define MF_SPARSE_BACKEND_MMA 1     /* 32-row tiles on mma.sync */
#define MF_SPARSE_BACKEND_TCGEN05 2 /* 128-row tiles on tcgen05 + bulk tensor copies: bf16, head_dim 64, tokens a
                                       multiple of four and <= 8192, 16-byte aligned tensors */
typedef struct MfSparseAttnArgs {
  int32_t batch, heads, tokens, head_dim;
  int32_t dtype;
  int32_t window; /* local-window attention only: keys i-window/2 .. i+window/2-1 */
  float scale;    /* logits = scale * q.k */
  int32_t backend; /* MF_SPARSE_BACKEND_*: bf16 calls only; other types always use the CUDA-core kernels */
  const void* q;
  const void* k;
  const void* v;
  const int32_t* num_atoms;   /* (B) */
  const int32_t* block_count; /* radius only */
  const int32_t* block_cols;  /* radius only */
  const uint32_t* block_mask; /* radius only */
  void* out;                  /* fwd: written; bwd: read */
  float* lse;                 /* fwd: written; bwd: read */
  const void* grad_out;       /* bwd only */
  void* dq;                   /* bwd only */
  void* dk;
  void* dv;
  void* workspace; /* bwd: mf_sparse_attn_bwd_workspace_bytes() bytes */
  size_t workspace_bytes;
} MfSparseAttnArgs;

size_t mf_sparse_attn_bwd_workspace_bytes(const MfSparseAttnArgs* args);
int mf_radius_attn_fwd(const MfSparseAttnArgs* args, void* stream);
int mf_radius_attn_bwd(const MfSparseAttnArgs* args, void* stream);

/*
 * Band attention over the (cell-sorted) token order: key j is visible to query i iff
 * i - window/2 <= j <= i + window/2 - 1 and both are real atoms.
 * ref: same masked-SDPA composition as above (regular_attention.py:251-268) with a band mask.
 */
int mf_local_attn_fwd(const MfSparseAttnArgs* args, void* stream);
int mf_local_attn_bwd(const MfSparseAttnArgs* args, void* stream);

/*
 * Band attention on the packed projection of an attention layer.  `nn.MultiheadAttention` (the MHA layers of the
 * reference trunk, transformer.py:228-316) projects to (B,N,3*H*D), splits that into three head-major tensors and
 * permutes the core's output back; here q, k, v are read inside qkv (B,N,3,H,D) bf16 and out is written as (B,N,H*D)
 * bf16.  The backward call reads out and lse of the forward call, takes grad_out (B,N,H*D) and writes grad_qkv
 * (B,N,3,H,D).  Semantics of mf_local_attn_fwd / mf_local_attn_bwd; bf16; head_dim 32, 64 or 128.
 */
typedef struct MfLocalAttnPackedArgs {
  int32_t batch, heads, tokens, head_dim;
  int32_t window;
  float scale;
  const void* qkv;
  const int32_t* num_atoms; /* (B) */
  void* out;
  float* lse;               /* (B,H,N) */
  const void* grad_out;     /* backward only from here on */
  void* grad_qkv;
  void* workspace;          /* mf_local_attn_packed_bwd_workspace_bytes() bytes */
  size_t workspace_bytes;
} MfLocalAttnPackedArgs;

size_t mf_local_attn_packed_bwd_workspace_bytes(const MfLocalAttnPackedArgs* args);
int mf_local_attn_packed_fwd(const MfLocalAttnPackedArgs* args, void* stream);
int mf_local_attn_packed_bwd(const MfLocalAttnPackedArgs* args, void* stream);

/*
 * Status word of the tcgen05 sparse-attention kernels (no counterpart in the reference): 0, or
 * MF_ERR_DEVICE_TIMEOUT once a bounded device-side wait has expired (the outputs of that call are then
 * undefined).  Waits for `stream`, copies four bytes, allocates nothing.
 */
int mf_sparse_attn_status(int32_t* host_status, void* stream);

/* ------------------------------------------------------------------------- */
/* Errors                                                                     */
/* ------------------------------------------------------------------------- */

/* Copies the calling thread's last error text (NUL terminated) into buf; returns its length. */
size_t mf_last_error(char* buf, size_t buf_len);

/* Library version, e.g. 100 = 0.1.0 */
int mf_version(void);

/* Capabilities found on this machine, as a bit set.  (No counterpart in the reference.)
 * bit 0 (MF_FEATURE_TENSOR_MAPS): the driver's tensor-map encoder is available, so the tensor-core
 * simplicial kernels receive their K2 / V2 tiles through bulk tensor copies; otherwise they use plain loads. */
#define MF_FEATURE_TENSOR_MAPS 1
int mf_feature_flags(void);

/* ------------------------------------------------------------------------- */
/* Fused element-wise passes of the adaptive-LayerNorm block                  */
/* ------------------------------------------------------------------------- */

/*
 * h[b,n,:] = LayerNorm(x[b,n,:]) * (1 + scale[b,:]) + shift[b,:]   (statistics over the channels, no affine
 * parameters), the `modulate(norm(x), shift, scale)` of AdaLNBlock.forward, transformer.py:242-253, which the
 * reference evaluates as separate element-wise kernels.  x (B,N,C) contiguous, fp32 or bf16 (x_dtype), shift / scale
 * fp32 (B,C), h fp32 or bf16 (h_dtype); arithmetic in fp32.  mean and rstd (B,N) are saved for the backward call,
 * which returns dx (in x's type) and dshift, dscale (B,C) fp32 = sums over the tokens of a molecule.  C is a multiple
 * of 8, at most 1024.
 */
int mf_ln_modulate_fwd(const void* x, int32_t x_dtype, const float* shift, const float* scale, int32_t batch,
                       int32_t tokens, int32_t channels, float eps, int32_t h_dtype, void* h, float* mean, float* rstd,
                       void* stream);
int mf_ln_modulate_bwd(const void* dh, int32_t dh_dtype, const void* x, int32_t x_dtype, const float* scale,
                       const float* mean, const float* rstd, int32_t batch, int32_t tokens, int32_t channels, void* dx,
                       float* dshift, float* dscale, void* stream);

/*
 * y = x + gate[b,:] * a, the gated residual of AdaLNBlock.forward, transformer.py:308-316.  x, y (B,N,C) fp32 or bf16
 * (x_dtype), gate fp32 (B,C), a fp32 or bf16 (a_dtype).  `pad` (NULL or (B,N) bytes, non-zero = padded token) folds in
 * the `x.masked_fill(pad_mask[..., None], 0)` that the trunk applies before the next block (transformer.py, the loop
 * of TransformerTrunk.forward): flagged rows of y are zeros.  The backward call takes dy in x's type and returns
 * da = dy * gate (in a's type) and dgate (B,C) fp32; the gradient of x is dy itself, or, with `pad`, dy with the
 * flagged rows cleared, written to `dx` (flagged rows then contribute nothing to da and dgate either).
 */
int mf_gated_residual_fwd(const void* x, int32_t x_dtype, const float* gate, const void* a, int32_t a_dtype,
                          const uint8_t* pad, int32_t batch, int32_t tokens, int32_t channels, void* y, void* stream);
int mf_gated_residual_bwd(const void* dy, int32_t dy_dtype, const float* gate, const void* a, int32_t a_dtype,
                          const uint8_t* pad, int32_t batch, int32_t tokens, int32_t channels, void* da, void* dx,
                          float* dgate, void* stream);

/*
 * out[c] = sum_r x[r, c]: the bias gradient of a Linear layer (the sum of its output gradient over all tokens), which
 * autograd forms for every Linear of AdaLNBlock.forward, transformer.py:228-316.  x (rows, cols) row-major fp32 or
 * bf16, starting on a 16-byte boundary, cols a multiple of 8; out (cols) fp32; fp32 accumulation in a fixed order
 * (bit-identical from run to run).  `workspace`: mf_column_sums_workspace_bytes(rows, cols) bytes.
 */
size_t mf_column_sums_workspace_bytes(int64_t rows, int32_t cols);
int mf_column_sums(const void* x, int32_t dtype, int64_t rows, int32_t cols, float* out, void* workspace,
                   size_t workspace_bytes, void* stream);

/*
 * GELU in its tanh form, the activation of the block's MLP (`Mlp`, transformer.py:137-152: nn.GELU(approximate="tanh")):
 * y = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), evaluated in fp32.  Forward: n elements (a multiple of 8) of
 * fp32 or bf16.  Backward: x = the pre-activation (rows, cols), dy = the gradient of the activation; writes
 * dx = dy * gelu'(x) and column_sums[c] = sum_r dx[r, c] (fp32; of the values as stored), which is the bias gradient
 * of the Linear layer that produced x.  Workspace as for mf_column_sums.  Tensors start on 16-byte boundaries.
 */
int mf_gelu_tanh_fwd(const void* x, int32_t dtype, int64_t n, void* y, void* stream);
int mf_gelu_tanh_bwd(const void* x, const void* dy, int32_t dtype, int64_t rows, int32_t cols, void* dx,
                     float* column_sums, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Head split / merge around the attention cores.  The projection GEMM of a layer writes (B,N,G,H,D) (G = 5: q, k1,
 * v1, k2, v2 of `_project_inputs`, simplicial_attention.py:718-725; G = 3: q, k, v) and the kernels take G tensors
 * (B,H,N,D); the reference gets there by G transposing copies.  mf_split_heads does it in one pass and multiplies
 * group g by scales[g] (host array of G floats or NULL; the D^-1/2 of the queries); mf_merge_heads is the inverse
 * and the split's backward pass (a NULL entry of `ins` is read as zeros).  fp32 or bf16, head rows of a multiple
 * of 16 bytes, 16-byte aligned tensors, G <= 8.  `outs` / `ins` are host arrays of G device pointers.
 */
int mf_split_heads(const void* packed, void* const* outs, const float* scales, int32_t groups, int32_t batch,
                   int32_t tokens, int32_t heads, int32_t head_dim, int32_t dtype, void* stream);
int mf_merge_heads(void* const* ins, const float* scales, void* packed, int32_t groups, int32_t batch, int32_t tokens,
                   int32_t heads, int32_t head_dim, int32_t dtype, void* stream);

/* ------------------------------------------------------------------------- */
/* 2-simplicial attention on the packed projection                           */
/* ------------------------------------------------------------------------- */

/*
 * `SimplicialAttention._project_inputs` (simplicial_attention.py:718-725) turns the (B,N,5*H*D) output of the layer's
 * input GEMM into five contiguous (B,H,N,D) tensors by five transposing copies and a multiply of the queries, and
 * `SimplicialAttention.forward` (:965) permutes the attention output back to (B,N,H*D) for `out_proj`.  These entry
 * points read the projection where the GEMM left it (proj (B,N,5,H,D) bf16; group 0 = q, then k1, v1, k2, v2), scale
 * the queries by q_scale on load (a power of two, D^-1/2 at D = 64), write `out` as (B,N,H*D) bf16 and, in the backward
 * call, all five gradients into grad_proj (B,N,5,H,D) bf16, the gradient of the unscaled projection.  out32 (B,H,N,D)
 * fp32 and lse (B,H,N) fp32 are written by the forward call and read by the backward call, as in mf_simplicial_fwd /
 * mf_simplicial_bwd, whose semantics (masks, zero rows, reproducibility) apply.  Served shapes: head_dim 64, at most 32
 * tokens, heads a multiple of four (the kernels that pack four heads into one 128-row tile); MF_ERR_UNSUPPORTED
 * otherwise.  16-byte aligned tensors; workspaces from the two *_workspace_bytes functions.
 */
typedef struct MfSimplicialPackedArgs {
  int32_t batch, heads, tokens, head_dim;
  float q_scale;
  int32_t reserved0;
  const void* proj;
  const uint8_t* query_valid;    /* (B,N) bytes, >0 = valid */
  const uint8_t* pair_key_valid; /* (B,N) */
  const uint8_t* pair_valid;     /* (B,N,N) or NULL */
  float* out32;
  float* lse;
  void* out;            /* forward */
  const void* grad_out; /* backward: (B,N,H*D) bf16 */
  void* grad_proj;      /* backward */
  void* workspace;
  size_t workspace_bytes;
} MfSimplicialPackedArgs;

size_t mf_simplicial_packed_fwd_workspace_bytes(const MfSimplicialPackedArgs* args);
size_t mf_simplicial_packed_bwd_workspace_bytes(const MfSimplicialPackedArgs* args);
int mf_simplicial_packed_fwd(const MfSimplicialPackedArgs* args, void* stream);
int mf_simplicial_packed_bwd(const MfSimplicialPackedArgs* args, void* stream);

/* ------------------------------------------------------------------------- */
/* Equivariant coordinate head                                               */
/* ------------------------------------------------------------------------- */

/*
 * `QM9EDMModel._equivariant_coord_delta`, models/qm9.py:478-501, on the pair geometry of
 * `NonPeriodicGeometryAdapter.forward`, geometry/adapters.py:83-125, and the radial basis of `_distance_rbf`,
 * models/qm9.py:460-469.  The reference builds cat[h_i, h_j, rbf_ij] as a (B,N,N,2d+16) tensor and applies
 * pair_head = Linear(2d+16, 128) -> SiLU -> Linear(128, 1) to it.  Here the caller applies the first Linear's two
 * d-wide column blocks to the trunk output once per atom (a = h W[:, :d]^T, b = h W[:, d:2d]^T + bias, (B,N,128) fp32
 * or bf16) and the kernel does the rest per pair without storing anything of size N^2 x channels:
 *   w_ij = w_out . silu(a_i + b_j + w_rbf exp(-gamma (|x_i - x_j| / rms - centers)^2)) + b_out   (0 on padding, i = j)
 *   out_i = (1/n) sum_j w_ij (x_i - x_j), minus its mean over the molecule's real atoms; 0 on padding.
 * coords (B,N,3) fp32, valid (B,N) bytes (non-zero = real atom), w_rbf (128,16) = W[:, 2d:], w_out (128), b_out (1),
 * centers (16), all fp32 on the device.  The backward call takes grad_out (B,N,3) fp32 and returns grad_a, grad_b (in
 * dtype), grad_w_rbf, grad_w_out, grad_b_out (fp32); it needs mf_pair_head_bwd_workspace_bytes of workspace.  No
 * gradient with respect to the coordinates is produced (they are inputs of the denoiser).  Sums run in a fixed order:
 * results are reproducible from call to call.
 */
typedef struct MfPairHeadArgs {
  int32_t batch, tokens;
  int32_t hidden; /* 128 */
  int32_t n_rbf;  /* 16 */
  int32_t dtype;  /* of a, b, grad_a, grad_b: MF_DTYPE_F32 or MF_DTYPE_BF16 */
  float gamma;
  const void* a;
  const void* b;
  const float* coords;
  const uint8_t* valid;
  const float* w_rbf;
  const float* w_out;
  const float* b_out;
  const float* centers;
  float* out;            /* forward */
  const float* grad_out; /* backward from here on */
  void* grad_a;
  void* grad_b;
  float* grad_w_rbf;
  float* grad_w_out;
  float* grad_b_out;
  void* workspace;
  size_t workspace_bytes;
} MfPairHeadArgs;

size_t mf_pair_head_bwd_workspace_bytes(const MfPairHeadArgs* args);
int mf_pair_head_fwd(const MfPairHeadArgs* args, void* stream);
int mf_pair_head_bwd(const MfPairHeadArgs* args, void* stream);

/* ------------------------------------------------------------------------- */
/* Kernel timing (measurement aid; no counterpart in the reference)           */
/* ------------------------------------------------------------------------- */

#define MF_PROFILE_SIMPLICIAL_FWD 0 /* the tensor-core forward kernel */
#define MF_PROFILE_SIMPLICIAL_BWD 1 /* the tensor-core backward kernel */

/*
 * While enabled, each listed kernel is bracketed by a pair of CUDA events on the stream it is launched
 * on.  mf_profile_read waits for the recorded events of `which`, returns the summed device time in
 * milliseconds and the number of launches, and forgets them.  Off by default; not thread safe.
 */
int mf_profile_enable(int32_t on);
int mf_profile_read(int32_t which, double* total_ms, int32_t* launches);

#ifdef __cplusplus
}
#endif
#endif /* MATTERFORMER_B200_H_ */
