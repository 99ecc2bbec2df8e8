// 2-simplicial attention on the projection as the layer's GEMM leaves it.
//
// `SimplicialAttention._project_inputs` (src/matterformer/models/simplicial_attention.py:718-725) computes one GEMM
// (B,N,C) -> (B,N,5*H*D), then reshapes, permutes and scales it into five contiguous (B,H,N,D) tensors (five
// transposing copies and a multiply), and the layer undoes the permutation before `out_proj` (:965).  These entry
// points take the GEMM's output as it is -- rows of q, k1, v1, k2, v2 are slices of the packed tensor, addressed
// with strides -- apply the query scale on load, write the attention output as (B,N,H*D) and the five gradients
// straight into one (B,N,5,H,D) tensor, so neither pass over the activations exists any more.  They run the
// packed-heads tile kernels (simplicial_sm100.cu, simplicial_sm100_bwd.cu) and therefore serve molecules of at most
// 32 tokens with a multiple of four heads of 64 channels in bf16: the trunk's shape.
#include "common.cuh"
#include "simplicial.cuh"
#include "simplicial_sm100.cuh"

namespace mf {
namespace {

int check_packed(const MfSimplicialPackedArgs* a, const char* name, bool backward) {
  MF_CHECK_ARG(a != nullptr, "%s: null argument struct", name);
  MF_CHECK_ARG(a->batch >= 0 && a->heads >= 0 && a->tokens >= 0, "%s: negative size", name);
  if (a->head_dim != kD || a->tokens > 32 || a->heads % 4 != 0) {
    set_error("%s: serves head_dim 64, at most 32 tokens and a multiple of four heads (got head_dim %d, %d tokens, %d heads); "
              "split the heads and call mf_simplicial_fwd / mf_simplicial_bwd otherwise", name, (int)a->head_dim,
              (int)a->tokens, (int)a->heads);
    return MF_ERR_UNSUPPORTED;
  }
  if (a->batch == 0 || a->heads == 0 || a->tokens == 0) return MF_OK;
  MF_CHECK_ARG((long long)a->batch * a->heads <= 65535, "%s: batch*heads above 65535", name);
  MF_CHECK_ARG(a->proj && a->query_valid && a->pair_key_valid && a->out32 && a->lse, "%s: null pointer argument", name);
  {  // the scale goes onto q in bf16: it has to be a power of two to be exact there
    int e = 0;
    MF_CHECK_ARG(a->q_scale > 0.f && frexpf(a->q_scale, &e) == 0.5f, "%s: q_scale must be a power of two, got %g", name,
                 (double)a->q_scale);
  }
  MF_CHECK_ALIGNED(name, a->proj, a->out32, a->out, a->grad_out, a->grad_proj);
  if (!backward) {
    MF_CHECK_ARG(a->out != nullptr, "%s: null output pointer", name);
  } else {
    MF_CHECK_ARG(a->grad_out && a->grad_proj, "%s: null gradient pointer", name);
  }
  return MF_OK;
}

TileLayouts packed_layouts(const MfSimplicialPackedArgs* a) {
  const long long hd = (long long)a->heads * kD;
  TileLayouts l;
  l.in = RowLayout{(long long)a->tokens * 5 * hd, (long long)kD, 5 * hd};  // (B,N,5,H,D): a group's rows
  l.act = RowLayout{(long long)a->tokens * hd, (long long)kD, hd};         // (B,N,H,D)
  l.q_scale = a->q_scale;
  return l;
}

MfSimplicialFwdArgs as_fwd(const MfSimplicialPackedArgs* a) {
  const __nv_bfloat16* proj = static_cast<const __nv_bfloat16*>(a->proj);
  const long long hd = (long long)a->heads * kD;
  MfSimplicialFwdArgs f{};
  f.batch = a->batch, f.heads = a->heads, f.tokens = a->tokens, f.head_dim = a->head_dim;
  f.dtype = MF_DTYPE_BF16, f.precision = MF_PRECISION_BF16_TC, f.backend = MF_BACKEND_TCGEN05_TILES;
  f.q = proj, f.k1 = proj + hd, f.v1 = proj + 2 * hd, f.k2 = proj + 3 * hd, f.v2 = proj + 4 * hd;
  f.query_valid = a->query_valid, f.pair_key_valid = a->pair_key_valid, f.pair_valid = a->pair_valid;
  f.out = a->out32, f.lse = a->lse, f.out_cast = a->out;
  f.workspace = a->workspace, f.workspace_bytes = a->workspace_bytes;
  return f;
}

MfSimplicialBwdArgs as_bwd(const MfSimplicialPackedArgs* a) {
  const __nv_bfloat16* proj = static_cast<const __nv_bfloat16*>(a->proj);
  __nv_bfloat16* g = static_cast<__nv_bfloat16*>(a->grad_proj);
  const long long hd = (long long)a->heads * kD;
  MfSimplicialBwdArgs r{};
  r.batch = a->batch, r.heads = a->heads, r.tokens = a->tokens, r.head_dim = a->head_dim;
  r.dtype = MF_DTYPE_BF16, r.precision = MF_PRECISION_BF16_TC, r.backend = MF_BACKEND_TCGEN05_TILES;
  r.grad_out = a->grad_out;
  r.q = proj, r.k1 = proj + hd, r.v1 = proj + 2 * hd, r.k2 = proj + 3 * hd, r.v2 = proj + 4 * hd;
  r.out = a->out32, r.lse = a->lse;
  r.query_valid = a->query_valid, r.pair_key_valid = a->pair_key_valid, r.pair_valid = a->pair_valid;
  r.dq = g, r.dk1 = g + hd, r.dv1 = g + 2 * hd, r.dk2 = g + 3 * hd, r.dv2 = g + 4 * hd;
  r.workspace = a->workspace, r.workspace_bytes = a->workspace_bytes;
  return r;
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" size_t mf_simplicial_packed_fwd_workspace_bytes(const MfSimplicialPackedArgs* a) {
  if (!a || a->batch <= 0) return 0;
  const MfSimplicialFwdArgs f = as_fwd(a);
  return simplicial_sm100_fwd_workspace_bytes(f);
}

extern "C" size_t mf_simplicial_packed_bwd_workspace_bytes(const MfSimplicialPackedArgs* a) {
  if (!a || a->batch <= 0) return 0;
  const MfSimplicialBwdArgs r = as_bwd(a);
  return simplicial_sm100_bwd_workspace_bytes(r);
}

extern "C" int mf_simplicial_packed_fwd(const MfSimplicialPackedArgs* a, void* stream) {
  int rc = check_packed(a, "mf_simplicial_packed_fwd", false);
  if (rc != MF_OK || a->batch == 0 || a->heads == 0 || a->tokens == 0) return rc;
  const MfSimplicialFwdArgs f = as_fwd(a);
  const size_t need = simplicial_sm100_fwd_workspace_bytes(f);
  if (!a->workspace || a->workspace_bytes < need) {
    set_error("mf_simplicial_packed_fwd: workspace of %zu bytes needed, %zu given", need, a->workspace_bytes);
    return MF_ERR_WORKSPACE_TOO_SMALL;
  }
  const TileLayouts l = packed_layouts(a);
  return simplicial_sm100_fwd_layouts(f, &l, static_cast<cudaStream_t>(stream));
}

extern "C" int mf_simplicial_packed_bwd(const MfSimplicialPackedArgs* a, void* stream) {
  int rc = check_packed(a, "mf_simplicial_packed_bwd", true);
  if (rc != MF_OK || a->batch == 0 || a->heads == 0 || a->tokens == 0) return rc;
  const MfSimplicialBwdArgs r = as_bwd(a);
  const size_t need = simplicial_sm100_bwd_workspace_bytes(r);
  if (!a->workspace || a->workspace_bytes < need) {
    set_error("mf_simplicial_packed_bwd: workspace of %zu bytes needed, %zu given", need, a->workspace_bytes);
    return MF_ERR_WORKSPACE_TOO_SMALL;
  }
  const TileLayouts l = packed_layouts(a);
  return simplicial_sm100_bwd_layouts(r, &l, static_cast<cudaStream_t>(stream));
}
