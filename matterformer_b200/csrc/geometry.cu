// Periodic geometry kernels: minimum-image distances, k nearest neighbours,
// cell sort and the radius block list with its per-block pair bitmaps.
//
// Every distance is evaluated with one fixed sequence of IEEE fp32 operations
// (see min_image_d2) that the CPU oracle repeats operation for operation, so
// the integer outputs (neighbour indices, permutation, block lists, bitmaps)
// can be compared bit for bit.
//
// Distance semantics follow PeriodicGeometryAdapter.forward of the reference
// (src/matterformer/geometry/adapters.py:176-190): fractional delta plus each of
// the 27 lattice offsets in itertools.product(range(-1,2), repeat=3) order,
// squared length under the cell metric, first minimum wins.
#include "common.cuh"
#include "geometry.cuh"

namespace mf {

namespace {

// ---------------------------------------------------------------------------
// kNN: one thread per query atom, candidates streamed through shared memory,
// the k best kept as a sorted register list.  Candidates arrive in ascending
// index order and only a strictly smaller distance displaces an entry, so ties
// resolve to the lower index.
// ---------------------------------------------------------------------------
template <int KMAX>
__global__ void __launch_bounds__(128) knn_kernel(const float* __restrict__ frac, const float* __restrict__ cell,
                                                  const int32_t* __restrict__ num_atoms, int n_max, int k,
                                                  int include_self, int32_t* __restrict__ idx,
                                                  float* __restrict__ dist2) {
  __shared__ float sx[128], sy[128], sz[128];
  const int b = blockIdx.y;
  const int n = min(num_atoms[b], n_max);
  const int i = blockIdx.x * 128 + threadIdx.x;
  const float* pos = frac + (size_t)b * n_max * 3;
  const Cell c = load_cell(cell + (size_t)b * 9);
  const bool active = i < n;
  float xi = 0.f, yi = 0.f, zi = 0.f;
  if (active) {
    xi = pos[3 * i + 0];
    yi = pos[3 * i + 1];
    zi = pos[3 * i + 2];
  }
  float bd[KMAX];
  int bi[KMAX];
#pragma unroll
  for (int t = 0; t < KMAX; ++t) {
    bd[t] = INFINITY;
    bi[t] = -1;
  }
  for (int j0 = 0; j0 < n; j0 += 128) {
    __syncthreads();
    const int jl = j0 + threadIdx.x;
    if (jl < n) {
      sx[threadIdx.x] = pos[3 * jl + 0];
      sy[threadIdx.x] = pos[3 * jl + 1];
      sz[threadIdx.x] = pos[3 * jl + 2];
    }
    __syncthreads();
    if (!active) continue;
    const int cnt = min(128, n - j0);
    for (int t = 0; t < cnt; ++t) {
      const int j = j0 + t;
      if (j == i && !include_self) continue;
      const float d2 = min_image_d2(xi, yi, zi, sx[t], sy[t], sz[t], c);
      if (d2 < bd[KMAX - 1]) {
        float cd = d2;
        int ci = j;
        bool shifting = false;
#pragma unroll
        for (int s = 0; s < KMAX; ++s) {
          const bool sw = shifting || (cd < bd[s]);
          const float td = bd[s];
          const int ti = bi[s];
          bd[s] = sw ? cd : td;
          bi[s] = sw ? ci : ti;
          cd = sw ? td : cd;
          ci = sw ? ti : ci;
          shifting = sw;
        }
      }
    }
  }
  if (i < n_max) {
    int32_t* oi = idx + ((size_t)b * n_max + i) * k;
    float* od = dist2 ? dist2 + ((size_t)b * n_max + i) * k : nullptr;
#pragma unroll
    for (int t = 0; t < KMAX; ++t) {
      if (t < k) {
        oi[t] = active ? bi[t] : -1;
        if (od) od[t] = active ? bd[t] : INFINITY;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// cell sort
// ---------------------------------------------------------------------------
__global__ void cell_key_kernel(const float* __restrict__ frac, const int32_t* __restrict__ num_atoms,
                                const int32_t* __restrict__ grid_dims, int n_max, int32_t* __restrict__ keys) {
  const int b = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_max) return;
  const int n = min(num_atoms[b], n_max);
  int key = INT32_MAX;
  if (i < n) {
    const float* p = frac + ((size_t)b * n_max + i) * 3;
    const int gx = grid_dims[3 * b + 0], gy = grid_dims[3 * b + 1], gz = grid_dims[3 * b + 2];
    key = (cell_coord(p[0], gx) * gy + cell_coord(p[1], gy)) * gz + cell_coord(p[2], gz);
  }
  keys[(size_t)b * n_max + i] = key;
}

// rank of atom i = number of atoms with a smaller (key, index); padded atoms keep their place.
__global__ void __launch_bounds__(256) cell_rank_kernel(const int32_t* __restrict__ keys,
                                                        const int32_t* __restrict__ num_atoms, int n_max,
                                                        int32_t* __restrict__ perm) {
  __shared__ int32_t sk[256];
  const int b = blockIdx.y;
  const int n = min(num_atoms[b], n_max);
  const int i = blockIdx.x * 256 + threadIdx.x;
  const int32_t* kb = keys + (size_t)b * n_max;
  const int32_t ki = (i < n) ? kb[i] : INT32_MAX;
  int rank = 0;
  for (int j0 = 0; j0 < n; j0 += 256) {
    __syncthreads();
    if (j0 + threadIdx.x < n) sk[threadIdx.x] = kb[j0 + threadIdx.x];
    __syncthreads();
    const int cnt = min(256, n - j0);
    if (i < n) {
      for (int t = 0; t < cnt; ++t) {
        const int32_t kj = sk[t];
        rank += (kj < ki) || (kj == ki && (j0 + t) < i);
      }
    }
  }
  if (i < n)
    perm[(size_t)b * n_max + rank] = i;
  else if (i < n_max)
    perm[(size_t)b * n_max + i] = i;
}

// one block per (column tile J, row tile I, batch); warp r = row of the tile, lane c = column
__global__ void __launch_bounds__(1024) block_mask_kernel(const float* __restrict__ frac,
                                                          const float* __restrict__ cell,
                                                          const int32_t* __restrict__ num_atoms,
                                                          const int32_t* __restrict__ perm, int n_max, int tiles,
                                                          float cutoff, uint32_t* __restrict__ block_mask,
                                                          int32_t* __restrict__ active) {
  const int J = blockIdx.x, I = blockIdx.y, b = blockIdx.z;
  const int r = threadIdx.x >> 5, cidx = threadIdx.x & 31;
  const int n = min(num_atoms[b], n_max);
  const int si = 32 * I + r, sj = 32 * J + cidx;
  const float* pos = frac + (size_t)b * n_max * 3;
  const int32_t* pb = perm + (size_t)b * n_max;
  bool hit = false;
  if (si < n && sj < n) {
    const Cell c = load_cell(cell + (size_t)b * 9);
    const int ai = pb[si], aj = pb[sj];
    const float d2 = min_image_d2(pos[3 * ai], pos[3 * ai + 1], pos[3 * ai + 2], pos[3 * aj], pos[3 * aj + 1],
                                  pos[3 * aj + 2], c);
    hit = __fsqrt_rn(d2) <= cutoff;
  }
  const uint32_t word = __ballot_sync(0xffffffffu, hit);
  if (cidx == 0) block_mask[(((size_t)b * tiles + I) * tiles + J) * 32 + r] = word;
  const int any = __syncthreads_or(hit);
  if (threadIdx.x == 0) active[((size_t)b * tiles + I) * tiles + J] = any;
}

__global__ void block_compact_kernel(const int32_t* __restrict__ active, int tiles, int total_rows,
                                     int32_t* __restrict__ block_count, int32_t* __restrict__ block_cols) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;  // flattened (b, I)
  if (row >= total_rows) return;
  const int32_t* a = active + (size_t)row * tiles;
  int32_t* cols = block_cols + (size_t)row * tiles;
  int cnt = 0;
  for (int J = 0; J < tiles; ++J)
    if (a[J]) cols[cnt++] = J;
  block_count[row] = cnt;
  for (int t = cnt; t < tiles; ++t) cols[t] = -1;
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" int mf_knn_topk(const float* frac, const float* cell, const int32_t* num_atoms, int32_t batch,
                           int32_t n_max, int32_t k, int32_t include_self, int32_t* idx, float* dist2,
                           void* stream) {
  MF_CHECK_ARG(batch >= 0 && n_max >= 0, "mf_knn_topk: negative size");
  MF_CHECK_ARG(k >= 1 && k <= 32, "mf_knn_topk: k must be in [1, 32], got %d", (int)k);
  if (batch == 0 || n_max == 0) return MF_OK;
  MF_CHECK_ARG(frac && cell && num_atoms && idx, "mf_knn_topk: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((n_max + 127) / 128, batch);
  if (k <= 16)
    knn_kernel<16><<<grid, 128, 0, s>>>(frac, cell, num_atoms, n_max, k, include_self, idx, dist2);
  else
    knn_kernel<32><<<grid, 128, 0, s>>>(frac, cell, num_atoms, n_max, k, include_self, idx, dist2);
  MF_CHECK_LAUNCH("knn_kernel");
  return MF_OK;
}

extern "C" size_t mf_radius_blocks_workspace_bytes(int32_t batch, int32_t n_max) {
  const size_t tiles = (size_t)(n_max + 31) / 32;
  return align_up((size_t)batch * n_max * sizeof(int32_t), 256) + align_up((size_t)batch * tiles * tiles * 4, 256);
}

extern "C" int mf_cell_sort_blocklist(const float* frac, const float* cell, const int32_t* num_atoms,
                                      const int32_t* grid_dims, int32_t batch, int32_t n_max, float cutoff,
                                      int32_t* perm, int32_t* block_count, int32_t* block_cols,
                                      uint32_t* block_mask, void* workspace, size_t workspace_bytes, void* stream) {
  MF_CHECK_ARG(batch >= 0 && n_max >= 0, "mf_cell_sort_blocklist: negative size");
  MF_CHECK_ARG(cutoff >= 0.f, "mf_cell_sort_blocklist: cutoff must be non-negative");
  if (batch == 0 || n_max == 0) return MF_OK;
  MF_CHECK_ARG(frac && cell && num_atoms && grid_dims && perm && block_count && block_cols && block_mask,
               "mf_cell_sort_blocklist: null pointer argument");
  const size_t need = mf_radius_blocks_workspace_bytes(batch, n_max);
  if (!workspace || workspace_bytes < need) {
    set_error("mf_cell_sort_blocklist: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    return MF_ERR_WORKSPACE_TOO_SMALL;
  }
  MF_CHECK_ARG(batch <= 65535, "mf_cell_sort_blocklist: batch above 65535");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tiles = (n_max + 31) / 32;
  int32_t* keys = static_cast<int32_t*>(workspace);
  int32_t* active = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) +
                                               align_up((size_t)batch * n_max * sizeof(int32_t), 256));
  cell_key_kernel<<<dim3((n_max + 255) / 256, batch), 256, 0, s>>>(frac, num_atoms, grid_dims, n_max, keys);
  MF_CHECK_LAUNCH("cell_key_kernel");
  cell_rank_kernel<<<dim3((n_max + 255) / 256, batch), 256, 0, s>>>(keys, num_atoms, n_max, perm);
  MF_CHECK_LAUNCH("cell_rank_kernel");
  block_mask_kernel<<<dim3(tiles, tiles, batch), 1024, 0, s>>>(frac, cell, num_atoms, perm, n_max, tiles, cutoff,
                                                               block_mask, active);
  MF_CHECK_LAUNCH("block_mask_kernel");
  const int rows = batch * tiles;
  block_compact_kernel<<<(rows + 127) / 128, 128, 0, s>>>(active, tiles, rows, block_count, block_cols);
  MF_CHECK_LAUNCH("block_compact_kernel");
  return MF_OK;
}
