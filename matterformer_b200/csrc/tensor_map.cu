// Host-side encoding of the tensor maps declared in tensor_map.cuh.  The driver's encoder is looked up through
// the runtime (cudaGetDriverEntryPoint), so the library does not link against libcuda.
#include "tensor_map.cuh"

#include <mutex>

namespace mf {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

}  // namespace

bool tensor_maps_available() { return encoder() != nullptr; }

static thread_local int g_last_encode_result = 0;
int last_tensor_map_result() { return g_last_encode_result; }

bool make_rows_tensor_map(CUtensorMap* map, const void* base, int rows_per_matrix, int matrices, int box_rows) {
  EncodeTiledFn fn = encoder();
  g_last_encode_result = -1;  // refused before the driver was asked
  if (!fn || !base || rows_per_matrix <= 0 || matrices <= 0 || box_rows <= 0 || box_rows > 256 || box_rows % 8) return false;
  if (reinterpret_cast<uintptr_t>(base) & 15u) return false;  // the copy engine needs a 16-byte aligned base
  const cuuint64_t dims[3] = {64, (cuuint64_t)rows_per_matrix, (cuuint64_t)matrices};
  const cuuint64_t strides[2] = {128, (cuuint64_t)rows_per_matrix * 128};  // bytes, dimensions 1 and 2
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  CUtensorMap tmp;
  auto encode = [&]() {
    return fn(&tmp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem_strides,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // The encoder wants a context bound to the calling thread.  A host thread that has only been handed cached
    // device memory so far (the backward thread of an autograd engine, say) has none yet: a no-op runtime call
    // binds the device's primary context, then the encoding goes through.
    (void)cudaFree(nullptr);
    r = encode();
  }
  g_last_encode_result = (int)r;
  if (r != CUDA_SUCCESS) return false;
  *map = tmp;
  return true;
}

}  // namespace mf
