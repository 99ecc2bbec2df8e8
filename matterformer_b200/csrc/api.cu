// C-ABI entry points for 2-simplicial attention plus the error plumbing shared
// by every entry point of the library.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"
#include "tensor_map.cuh"
#include "simplicial.cuh"
#include "simplicial_rows.cuh"

namespace mf {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_error(cudaError_t err, const char* what) {
  set_error("%s: CUDA error %d (%s)", what, (int)err, cudaGetErrorString(err));
  return MF_ERR_CUDA;
}

namespace {

template <typename Args>
int check_common(const Args* a, const char* name) {
  MF_CHECK_ARG(a != nullptr, "%s: null argument struct", name);
  MF_CHECK_ARG(a->batch >= 0 && a->heads >= 0 && a->tokens >= 0 && a->head_dim > 0, "%s: negative size", name);
  MF_CHECK_ARG(a->head_dim <= 128, "%s: only supports head_dim <= 128, got %d", name, (int)a->head_dim);
  MF_CHECK_ARG(a->dtype == MF_DTYPE_F32 || a->dtype == MF_DTYPE_BF16 || a->dtype == MF_DTYPE_F16,
               "%s: only supports float16/bfloat16/float32 inputs, got dtype code %d", name, (int)a->dtype);
  MF_CHECK_ARG(a->precision >= MF_PRECISION_BF16_TC && a->precision <= MF_PRECISION_IEEE_FP32,
               "%s: unknown precision code %d", name, (int)a->precision);
  MF_CHECK_ARG(a->backend >= MF_BACKEND_AUTO && a->backend <= MF_BACKEND_TCGEN05_TILES, "%s: unknown backend code %d",
               name, (int)a->backend);
  if (a->batch == 0 || a->heads == 0 || a->tokens == 0) return MF_OK;  // nothing to read or write
  MF_CHECK_ARG(a->q && a->k1 && a->v1 && a->k2 && a->v2, "%s: null q/k/v pointer", name);
  MF_CHECK_ARG(a->query_valid && a->pair_key_valid, "%s: null mask pointer", name);
  MF_CHECK_ARG((long long)a->batch * a->heads <= 65535, "%s: batch*heads above 65535", name);
  return MF_OK;
}

// The factorized bias comes as four tensors or not at all.
template <typename Args>
int check_bias(const Args* a, const char* name) {
  const int n = (a->u != nullptr) + (a->v_bias != nullptr) + (a->w != nullptr) + (a->gate != nullptr);
  MF_CHECK_ARG(n == 0 || n == 4, "%s: u, v_bias, w and gate must be given together (got %d of 4)", name, n);
  const int na = (a->angle_left != nullptr) + (a->angle_right != nullptr) + (a->angle_gate != nullptr);
  MF_CHECK_ARG(na == 0 || na == 3, "%s: angle_left, angle_right and angle_gate must be given together", name);
  const int nm = (a->message_left != nullptr) + (a->message_right != nullptr) + (a->message_basis != nullptr);
  MF_CHECK_ARG(nm == 0 || nm == 3, "%s: message_left, message_right and message_basis must be given together", name);
  if ((na && (a->angle_rank < 1 || a->angle_rank > 32)) || (nm && (a->message_rank < 1 || a->message_rank > 32))) {
    set_error("%s: residual ranks must be in [1, 32] (angle %d, message %d)", name, (int)a->angle_rank,
              (int)a->message_rank);
    return MF_ERR_UNSUPPORTED;
  }
  return MF_OK;
}

inline bool vectors_aligned(const MfSimplicialFwdArgs* a) {
  return aligned16(a->q) && aligned16(a->k1) && aligned16(a->v1) && aligned16(a->k2) && aligned16(a->v2) &&
         aligned16(a->out) && aligned16(a->out_cast);
}
inline bool vectors_aligned(const MfSimplicialBwdArgs* a) {
  return aligned16(a->q) && aligned16(a->k1) && aligned16(a->v1) && aligned16(a->k2) && aligned16(a->v2) &&
         aligned16(a->grad_out) && aligned16(a->out) && aligned16(a->dq) && aligned16(a->dk1) && aligned16(a->dv1) &&
         aligned16(a->dk2) && aligned16(a->dv2);
}

template <typename Args>
bool has_factorized_bias(const Args* a) {
  return a->u || a->v_bias || a->w || a->gate;
}

template <typename Args>
bool wants_tcgen05(const Args* a, int* rc, const char* name) {
  *rc = MF_OK;
  // The factorized bias is built into the tile kernels, not into the row-packed ones; the low-rank residuals run on the
  // CUDA-core kernel.
  const bool has_residual = a->angle_left || a->message_left;
  const bool bias_ok = !has_residual && (!has_factorized_bias(a) || a->backend != MF_BACKEND_TCGEN05);
  // the tensor-core kernels move rows with 16-byte vector accesses; tensors that do not start on a 16-byte boundary
  // (a view into the middle of another tensor) go to the CUDA-core kernel, which loads element by element
  const bool ok = bias_ok && simplicial_sm100_supports(a->dtype, a->precision, a->tokens, a->head_dim) &&
                  vectors_aligned(a);
  if (a->backend == MF_BACKEND_GENERIC) return false;
  if ((a->backend == MF_BACKEND_TCGEN05 || a->backend == MF_BACKEND_TCGEN05_TILES) && !ok) {
    set_error("%s: the tcgen05 kernels need bf16 inputs with precision bf16_tc, head_dim 64, tokens <= 192, tensors "
              "that start on 16-byte boundaries and no residual operands; the factorized bias is built into the tile "
              "kernels only", name);
    *rc = MF_ERR_UNSUPPORTED;
    return false;
  }
  return ok;
}

// Which of the two tensor-core kernel families serves a qualifying call.  Molecules of at most 32 tokens with a
// multiple of four heads run fastest with four heads sharing one tile (measured on B200 at 1024 molecules of up to 29
// atoms: 0.39 / 0.94 ms forward / backward against 0.93 / 1.25 ms row-packed); everything else is row-packed.
template <typename Args>
bool uses_tile_kernels(const Args* a) {
  if (a->backend == MF_BACKEND_TCGEN05_TILES || has_factorized_bias(a)) return true;
  return a->backend == MF_BACKEND_AUTO && simplicial_sm100_packs_heads(a->tokens, a->heads);
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" size_t mf_last_error(char* buf, size_t buf_len) {
  const size_t n = strlen(g_error);
  if (buf && buf_len > 0) {
    const size_t c = n < buf_len - 1 ? n : buf_len - 1;
    memcpy(buf, g_error, c);
    buf[c] = '\0';
  }
  return n;
}

extern "C" int mf_version(void) { return 100; }

extern "C" int mf_feature_flags(void) { return tensor_maps_available() ? MF_FEATURE_TENSOR_MAPS : 0; }

extern "C" size_t mf_simplicial_fwd_workspace_bytes(const MfSimplicialFwdArgs* a) {
  if (!a) return 0;
  int rc;
  if (wants_tcgen05(a, &rc, "mf_simplicial_fwd")) return simplicial_sm100_fwd_workspace_bytes(*a);
  return 0;
}

extern "C" size_t mf_simplicial_bwd_workspace_bytes(const MfSimplicialBwdArgs* a) {
  if (!a) return 0;
  int rc;
  if (wants_tcgen05(a, &rc, "mf_simplicial_bwd"))
    return uses_tile_kernels(a) ? simplicial_sm100_bwd_workspace_bytes(*a) : simplicial_rows_bwd_workspace_bytes(*a);
  return simplicial_generic_bwd_workspace_bytes(*a);
}

extern "C" int mf_simplicial_fwd_backend(const MfSimplicialFwdArgs* a) {
  if (!a) return MF_BACKEND_GENERIC;
  int rc;
  return wants_tcgen05(a, &rc, "mf_simplicial_fwd_backend") ? MF_BACKEND_TCGEN05 : MF_BACKEND_GENERIC;
}

extern "C" int mf_simplicial_bwd_backend(const MfSimplicialBwdArgs* a) {
  if (!a) return MF_BACKEND_GENERIC;
  int rc;
  return wants_tcgen05(a, &rc, "mf_simplicial_bwd_backend") ? MF_BACKEND_TCGEN05 : MF_BACKEND_GENERIC;
}

extern "C" int mf_simplicial_row_plan(int32_t n_queries, int32_t valid_keys, int32_t plan[4]) {
  MF_CHECK_ARG(plan != nullptr, "mf_simplicial_row_plan: null output pointer");
  MF_CHECK_ARG(n_queries >= 0 && valid_keys >= 0, "mf_simplicial_row_plan: negative count");
  const RowPlan rp = plan_rows(n_queries, valid_keys);
  plan[0] = rp.tiles;
  plan[1] = rp.rows_per_tile;
  plan[2] = rp.groups;
  plan[3] = rp.steps;
  return MF_OK;
}

extern "C" int mf_simplicial_fwd(const MfSimplicialFwdArgs* a, void* stream) {
  int rc = check_common(a, "mf_simplicial_fwd");
  if (rc != MF_OK) return rc;
  if (a->batch == 0 || a->heads == 0 || a->tokens == 0) return MF_OK;
  MF_CHECK_ARG(a->out && a->lse, "mf_simplicial_fwd: null output pointer");
  if ((rc = check_bias(a, "mf_simplicial_fwd")) != MF_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tc = wants_tcgen05(a, &rc, "mf_simplicial_fwd");
  if (rc != MF_OK) return rc;
  const size_t need = mf_simplicial_fwd_workspace_bytes(a);
  if (need > 0 && (!a->workspace || a->workspace_bytes < need)) {
    set_error("mf_simplicial_fwd: workspace of %zu bytes needed, %zu given", need, a->workspace_bytes);
    return MF_ERR_WORKSPACE_TOO_SMALL;
  }
  if (!tc) return simplicial_generic_fwd(*a, s);
  return uses_tile_kernels(a) ? simplicial_sm100_fwd(*a, s) : simplicial_rows_fwd(*a, s);
}

extern "C" int mf_simplicial_bwd(const MfSimplicialBwdArgs* a, void* stream) {
  int rc = check_common(a, "mf_simplicial_bwd");
  if (rc != MF_OK) return rc;
  if (a->batch == 0 || a->heads == 0 || a->tokens == 0) return MF_OK;
  MF_CHECK_ARG(a->grad_out && a->out && a->lse, "mf_simplicial_bwd: null saved-tensor pointer");
  MF_CHECK_ARG(a->dq && a->dk1 && a->dv1 && a->dk2 && a->dv2, "mf_simplicial_bwd: null gradient pointer");
  if ((rc = check_bias(a, "mf_simplicial_bwd")) != MF_OK) return rc;
  MF_CHECK_ARG(a->u || !(a->du || a->dv_bias || a->dw || a->dgate),
               "mf_simplicial_bwd: bias gradients requested without the bias operands");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tc = wants_tcgen05(a, &rc, "mf_simplicial_bwd");
  if (rc != MF_OK) return rc;
  const size_t need = mf_simplicial_bwd_workspace_bytes(a);
  if (need > 0 && (!a->workspace || a->workspace_bytes < need)) {
    set_error("mf_simplicial_bwd: workspace of %zu bytes needed, %zu given", need, a->workspace_bytes);
    return MF_ERR_WORKSPACE_TOO_SMALL;
  }
  if (!tc) return simplicial_generic_bwd(*a, s);
  return uses_tile_kernels(a) ? simplicial_sm100_bwd(*a, s) : simplicial_rows_bwd(*a, s);
}

// ---------------------------------------------------------------------------
// kernel timing aid
// ---------------------------------------------------------------------------
#include <vector>

#include <atomic>
#include <mutex>

namespace mf {
namespace {
std::atomic<bool> g_profile_on{false};
std::mutex g_profile_mutex;                    // guards the event lists
std::vector<cudaEvent_t> g_profile_events[2];  // begin, end, begin, end, ...
}  // namespace

void profile_mark(int which, bool begin, cudaStream_t stream) {
  if (!g_profile_on.load(std::memory_order_relaxed) || which < 0 || which > 1) return;
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  std::vector<cudaEvent_t>& ev = g_profile_events[which];
  if (begin != (ev.size() % 2 == 0)) return;  // unpaired call: ignore
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, stream);
  ev.push_back(e);
}
}  // namespace mf

extern "C" int mf_profile_enable(int32_t on) {
  g_profile_on.store(on != 0);
  return MF_OK;
}

extern "C" int mf_profile_read(int32_t which, double* total_ms, int32_t* launches) {
  MF_CHECK_ARG(which == MF_PROFILE_SIMPLICIAL_FWD || which == MF_PROFILE_SIMPLICIAL_BWD,
               "mf_profile_read: unknown kernel id %d", (int)which);
  MF_CHECK_ARG(total_ms && launches, "mf_profile_read: null output pointer");
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  std::vector<cudaEvent_t>& ev = g_profile_events[which];
  double total = 0.0;
  int n = 0;
  for (size_t i = 0; i + 1 < ev.size(); i += 2) {
    cudaError_t e = cudaEventSynchronize(ev[i + 1]);
    if (e != cudaSuccess) return cuda_error(e, "mf_profile_read");
    float ms = 0.f;
    e = cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
    if (e != cudaSuccess) return cuda_error(e, "mf_profile_read");
    total += ms;
    ++n;
  }
  for (cudaEvent_t e : ev) cudaEventDestroy(e);
  ev.clear();
  *total_ms = total;
  *launches = n;
  return MF_OK;
}
