// Tensor maps (TMA descriptors) for the row-major bf16 operand matrices of the attention kernels, and the
// device-side bulk tensor load that uses them.
//
// A (B*H, N, 64) bf16 tensor is described as a 3-D map {64, N, B*H} with 128-byte swizzle, so that a box of
// 32 rows lands in shared memory in exactly the layout the tcgen05 shared-memory descriptors of this library
// expect (128-byte lines, 16-byte chunk index XOR-ed with row % 8, tiles 1024-byte aligned).  Rows beyond N
// are filled with zeros by the copy engine.  Loads always start at column 0, which satisfies the 16-byte
// alignment rule for the innermost coordinate.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mf {

constexpr int kTmaBoxRows = 32;

// Encodes the map on the host.  Allocates nothing.  Returns false (and leaves *map untouched) when the driver
// entry point is missing or the tensor does not meet the alignment rules; callers then use plain loads.
// `box_rows` rows per copy (a multiple of 8, at most 256); the simplicial kernels use kTmaBoxRows.
bool make_rows_tensor_map(CUtensorMap* map, const void* base, int rows_per_matrix, int matrices, int box_rows = 32);
// Result of the calling thread's last make_rows_tensor_map: the driver's code (0 = success), or -1 when the
// arguments were refused before the driver was asked.
int last_tensor_map_result();
// Whether the driver's encoder could be found at all.
bool tensor_maps_available();

#ifdef __CUDACC__
// Brings a tensor map (a kernel parameter) into the descriptor cache ahead of its first copy.
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// One box (the map's box rows) x 64 bf16 columns of matrix `mat`, starting at row `row0`, into `smem_dst`
// (1024-byte aligned); completion is signalled on `bar` with the byte count of the box.
__device__ __forceinline__ void tma_load_rows(void* smem_dst, const CUtensorMap* map, int row0, int mat,
                                              uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
      "l"(map), "r"(0), "r"(row0), "r"(mat), "r"((uint32_t)__cvta_generic_to_shared(bar))
      : "memory");
}
#endif

}  // namespace mf
