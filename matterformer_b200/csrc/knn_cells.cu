// Periodic k nearest neighbours with a cell list.
//
// Same result, bit for bit, as the all-pairs kernel (and the CPU oracle): the k smallest
// (minimum-image d2, index) pairs per atom.  Atoms are binned on a per-structure grid over their
// fractional coordinates and every query visits the bins within s cells of its own, s = 1, 2, ...
// A search of half-width s is complete as soon as k neighbours are known and the k-th distance is
// below s*h, where h = min over the axes of (perpendicular cell width / bins on that axis): any atom
// in an unvisited bin lies at least s bins away along some axis, so each of its 27 images is
// farther than s*h.  Candidates are inserted under the lexicographic order (d2, index), so the
// result does not depend on the order in which bins or atoms inside a bin are visited.
//
// A candidate normally costs one distance evaluation instead of 27: the image chosen by rounding the
// fractional delta is the minimum image whenever it is closer than half the smallest cell width, and
// its d2 is evaluated with the same operation sequence the 27-image search uses for that image; a
// candidate whose rounded image is farther than that needs the full search only while the list of
// the k best still holds an entry that far away.
//
// Structures with a coordinate outside [0,1) (where the reference's 27 offsets of the unwrapped
// coordinates are not the nearest images) are searched exhaustively.
#include "common.cuh"
#include "geometry.cuh"

namespace mf {
namespace {

constexpr int kMaxBinsPerAxis = 16;
constexpr int kMaxBins = kMaxBinsPerAxis * kMaxBinsPerAxis * kMaxBinsPerAxis;

struct KnnWorkspace {
  int32_t* counts;   // (B, kMaxBins + 1) bin sizes, then exclusive starts
  int32_t* cursor;   // (B, kMaxBins) fill cursors
  int32_t* keys;     // (B, N) bin of every atom
  int32_t* flags;    // (B) 1 when a coordinate lies outside [0,1)
  float4* sorted;    // (B, N) x, y, z, original index (as int bits), grouped by bin
};

__global__ void knn_zero_kernel(int32_t* counts, int32_t* flags, int B) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < B * (kMaxBins + 1)) counts[i] = 0;
  if (i < B) flags[i] = 0;
}

__global__ void knn_count_kernel(const float* __restrict__ frac, const int32_t* __restrict__ num_atoms,
                                 const int32_t* __restrict__ grid_dims, int n_max, KnnWorkspace w) {
  const int b = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = min(num_atoms[b], n_max);
  if (i >= n) return;
  const float* p = frac + ((size_t)b * n_max + i) * 3;
  const int gx = grid_dims[3 * b], gy = grid_dims[3 * b + 1], gz = grid_dims[3 * b + 2];
  const float x = p[0], y = p[1], z = p[2];
  if (!(x >= 0.f && x < 1.f && y >= 0.f && y < 1.f && z >= 0.f && z < 1.f)) w.flags[b] = 1;
  const int key = (cell_coord(x, gx) * gy + cell_coord(y, gy)) * gz + cell_coord(z, gz);
  w.keys[(size_t)b * n_max + i] = key;
  atomicAdd(&w.counts[(size_t)b * (kMaxBins + 1) + key], 1);
}

// exclusive scan of the bin sizes of one structure (one block per structure, bins <= 4096)
__global__ void __launch_bounds__(1024) knn_scan_kernel(const int32_t* __restrict__ grid_dims, KnnWorkspace w) {
  __shared__ int32_t part[1024];
  const int b = blockIdx.x;
  const int bins = grid_dims[3 * b] * grid_dims[3 * b + 1] * grid_dims[3 * b + 2];
  int32_t* c = w.counts + (size_t)b * (kMaxBins + 1);
  const int per = (bins + 1023) / 1024;  // consecutive bins per thread
  const int lo = threadIdx.x * per;
  int sum = 0;
  for (int t = 0; t < per; ++t)
    if (lo + t < bins) sum += c[lo + t];
  part[threadIdx.x] = sum;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int v = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
    __syncthreads();
    part[threadIdx.x] += v;
    __syncthreads();
  }
  int run = part[threadIdx.x] - sum;  // exclusive prefix of this thread's first bin
  for (int t = 0; t < per; ++t) {
    if (lo + t < bins) {
      const int v = c[lo + t];
      c[lo + t] = run;
      w.cursor[(size_t)b * kMaxBins + lo + t] = run;
      run += v;
    }
  }
  if (threadIdx.x == 1023) c[bins] = part[1023];
}

__global__ void knn_fill_kernel(const float* __restrict__ frac, const int32_t* __restrict__ num_atoms, int n_max,
                                KnnWorkspace w) {
  const int b = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = min(num_atoms[b], n_max);
  if (i >= n) return;
  const float* p = frac + ((size_t)b * n_max + i) * 3;
  const int key = w.keys[(size_t)b * n_max + i];
  const int slot = atomicAdd(&w.cursor[(size_t)b * kMaxBins + key], 1);
  w.sorted[(size_t)b * n_max + slot] = make_float4(p[0], p[1], p[2], __int_as_float(i));
}

// Bins per axis and the two distance bounds of the search, one thread per structure (double precision; the
// bounds are rounded down because they serve as lower bounds on distances to atoms that were not visited).
__global__ void knn_grid_kernel(const float* __restrict__ cell, const int32_t* __restrict__ num_atoms, int B, int n_max,
                                int k, int32_t* __restrict__ grid_dims, float* __restrict__ bounds) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const float* c = cell + (size_t)b * 9;
  const double a0 = c[0], a1 = c[1], a2 = c[2], b0 = c[3], b1 = c[4], b2 = c[5], c0 = c[6], c1 = c[7], c2 = c[8];
  // cross products b x c, c x a, a x b
  const double bc0 = b1 * c2 - b2 * c1, bc1 = b2 * c0 - b0 * c2, bc2 = b0 * c1 - b1 * c0;
  const double ca0 = c1 * a2 - c2 * a1, ca1 = c2 * a0 - c0 * a2, ca2 = c0 * a1 - c1 * a0;
  const double ab0 = a1 * b2 - a2 * b1, ab1 = a2 * b0 - a0 * b2, ab2 = a0 * b1 - a1 * b0;
  const double vol = fmax(fabs(a0 * bc0 + a1 * bc1 + a2 * bc2), 1e-12);
  const double w[3] = {vol / fmax(sqrt(bc0 * bc0 + bc1 * bc1 + bc2 * bc2), 1e-12),
                       vol / fmax(sqrt(ca0 * ca0 + ca1 * ca1 + ca2 * ca2), 1e-12),
                       vol / fmax(sqrt(ab0 * ab0 + ab1 * ab1 + ab2 * ab2), 1e-12)};
  const double n = fmax((double)min(num_atoms[b], n_max), 1.0);
  // bin edge ~ 1.25 x the radius of a sphere holding k atoms at the mean density
  const double r_est = 1.25 * cbrt(3.0 * k * vol / (4.0 * 3.14159265358979323846 * n));
  double h = 1e300, wmin = 1e300;
  for (int a = 0; a < 3; ++a) {
    const int g = (int)fmin(fmax(floor(w[a] / r_est), 1.0), (double)kMaxBinsPerAxis);
    grid_dims[3 * b + a] = g;
    h = fmin(h, w[a] / g);
    wmin = fmin(wmin, w[a]);
  }
  bounds[2 * b] = __double2float_rd(h * (1.0 - 1e-6));
  bounds[2 * b + 1] = __double2float_rd(0.5 * wmin * (1.0 - 1e-6));
}

// ---------------------------------------------------------------------------------------------------------------
// Warp-cooperative search.  One warp serves one bin of the grid: the atoms of the 3 x 3 x 3 bins around it are the
// candidates of every query atom in the bin, so they are gathered once into shared memory (own bin first, then the
// face, edge and corner neighbours, so that the list of the k best tightens early).  For one query at a time the 32
// lanes evaluate 32 candidates, and the k best live in a list spread over the lanes (lane t holds entry t, sorted by
// (d2, index)): a candidate that beats the last entry is broadcast and every lane either keeps its entry, takes the
// candidate, or takes its left neighbour's entry.  Queries whose k-th distance does not prove the first shell
// complete, structures searched exhaustively and neighbourhoods larger than the shared-memory list fall back to
// scanning bins straight from global memory with the same list logic.  The result does not depend on the order of
// candidates, so it is the same, bit for bit, as the one-thread-per-query search.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kWarpCand = 384;  // candidates per warp in shared memory (a 27-bin neighbourhood holds about 216)

__constant__ int8_t kShellOrder[27][3] = {
    {0, 0, 0},
    {-1, 0, 0}, {1, 0, 0}, {0, -1, 0}, {0, 1, 0}, {0, 0, -1}, {0, 0, 1},
    {-1, -1, 0}, {-1, 1, 0}, {1, -1, 0}, {1, 1, 0}, {-1, 0, -1}, {-1, 0, 1}, {1, 0, -1}, {1, 0, 1},
    {0, -1, -1}, {0, -1, 1}, {0, 1, -1}, {0, 1, 1},
    {-1, -1, -1}, {-1, -1, 1}, {-1, 1, -1}, {-1, 1, 1}, {1, -1, -1}, {1, -1, 1}, {1, 1, -1}, {1, 1, 1}};

template <int KMAX>
__global__ void __launch_bounds__(128) knn_warp_kernel(const float* __restrict__ cell,
                                                       const int32_t* __restrict__ num_atoms,
                                                       const int32_t* __restrict__ grid_dims,
                                                       const float* __restrict__ bounds, int n_max, int k,
                                                       int include_self, KnnWorkspace w, int32_t* __restrict__ idx,
                                                       float* __restrict__ dist2) {
  __shared__ float4 cand_s[4][kWarpCand];
  __shared__ float2 surv_s[4][kWarpCand];  // (d2, index bits) of the candidates within the first shell's reach
  const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gx = grid_dims[3 * b], gy = grid_dims[3 * b + 1], gz = grid_dims[3 * b + 2];
  const int n = min(num_atoms[b], n_max);
  const float4* sorted = w.sorted + (size_t)b * n_max;
  const int32_t* start = w.counts + (size_t)b * (kMaxBins + 1);
  const Cell c = load_cell(cell + (size_t)b * 9);
  // the grid has a fixed number of warps per structure; each takes every (warps per structure)-th bin
  for (int bin = blockIdx.x * 4 + warp; bin < gx * gy * gz; bin += gridDim.x * 4) {
  const int q0 = start[bin], q1 = start[bin + 1];
  if (q0 == q1) continue;
  const float h = bounds[2 * b];           // min over axes of width / bins, rounded down
  const float half_w = bounds[2 * b + 1];  // half the smallest perpendicular width, rounded down
  const float fast_limit2 = half_w * half_w * (1.f - 1e-4f);
  const bool exhaustive = w.flags[b] != 0;
  const int cz = bin % gz, cy = (bin / gz) % gy, cx = bin / (gy * gz);
  const int need = min(k, include_self ? n : n - 1);  // neighbours that exist
  float4* cand = cand_s[warp];
  float2* surv = surv_s[warp];

  // ---- the first shell's candidates, gathered once for all queries of the bin
  const bool ordered = !exhaustive && gx >= 3 && gy >= 3 && gz >= 3;
  const bool covers_all = exhaustive || (gx <= 3 && gy <= 3 && gz <= 3);
  int n_cand = 0;
  bool in_smem = ordered;
  if (ordered) {
    // lane t < 27 looks up the extent of neighbour bin t; one prefix sum places every bin's atoms in the list, and the
    // copies of the 27 bins are independent loads (two round trips to memory instead of one per bin)
    int e0 = 0, cnt = 0;
    if (lane < 27) {
      const int bx = (cx + kShellOrder[lane][0] + gx) % gx, by = (cy + kShellOrder[lane][1] + gy) % gy,
                bz = (cz + kShellOrder[lane][2] + gz) % gz;
      const int ob = (bx * gy + by) * gz + bz;
      e0 = start[ob];
      cnt = start[ob + 1] - e0;
    }
    int off = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, off, o);
      if (lane >= o) off += v;
    }
    n_cand = __shfl_sync(0xffffffffu, off, 31);
    off -= cnt;
    if (n_cand > kWarpCand) {
      in_smem = false;
    } else {
      for (int t = 0; t < 27; ++t) {
        const int e0_t = __shfl_sync(0xffffffffu, e0, t), c_t = __shfl_sync(0xffffffffu, cnt, t),
                  o_t = __shfl_sync(0xffffffffu, off, t);
        for (int e = lane; e < c_t; e += 32) cand[o_t + e] = __ldg(sorted + e0_t + e);
      }
    }
    __syncwarp();
  }

  // the list of the k best, entry t on lane t
  float d = INFINITY;
  int id = 0x7fffffff;
  int my_id = -1;
  float4 me = make_float4(0.f, 0.f, 0.f, 0.f);
  auto before = [](float cd, int ci, float ed, int ei) { return cd < ed || (cd == ed && ci < ei); };
  // A shell that does not cover every bin only counts if the k-th distance ends up below its reach (else the
  // search is repeated with a wider shell), so candidates at or beyond the reach can be dropped unseen.
  float keep_below = INFINITY;
  // d2 of one candidate per lane (INF where it does not count).  The image chosen by rounding the fractional delta is
  // the minimum image whenever it is closer than half the smallest cell width; a candidate whose rounded image is
  // farther needs the 27-image search only if something that far away could still be kept.
  auto distance = [&](float4 o, bool ok, float far_kept) {
    float d2 = INFINITY;
    if (ok && (include_self || __float_as_int(o.w) != my_id)) {
      if (!exhaustive) {
        const float dx = __fsub_rn(me.x, o.x), dy = __fsub_rn(me.y, o.y), dz = __fsub_rn(me.z, o.z);
        // -rint(delta) for |delta| < 1 (ties at +-0.5 go to 0), by comparison: cheaper than three conversions
        const float ox = dx > 0.5f ? -1.f : (dx < -0.5f ? 1.f : 0.f), oy = dy > 0.5f ? -1.f : (dy < -0.5f ? 1.f : 0.f),
                    oz = dz > 0.5f ? -1.f : (dz < -0.5f ? 1.f : 0.f);
        d2 = image_d2(dx, dy, dz, ox, oy, oz, c);
        if (d2 >= fast_limit2 && far_kept >= fast_limit2) d2 = min_image_d2(me.x, me.y, me.z, o.x, o.y, o.z, c);
      } else {
        d2 = min_image_d2(me.x, me.y, me.z, o.x, o.y, o.z, c);
      }
    }
    return d2;
  };
  // the lanes' candidates (d2, oid) that beat the current last entry, inserted one at a time
  auto insert_batch = [&](float d2, int oid, float worst_d, int worst_i) {
    uint32_t pass = __ballot_sync(0xffffffffu, d2 < keep_below && before(d2, oid, worst_d, worst_i));
    while (pass) {
      const int src = __ffs(pass) - 1;
      pass &= pass - 1;
      const float cd = __shfl_sync(0xffffffffu, d2, src);
      const int ci = __shfl_sync(0xffffffffu, oid, src);
      const uint32_t bal = __ballot_sync(0xffffffffu, lane < KMAX && before(cd, ci, d, id));
      const float pd = __shfl_up_sync(0xffffffffu, d, 1);
      const int pi = __shfl_up_sync(0xffffffffu, id, 1);
      if (bal == 0u) continue;  // earlier insertions of this batch pushed it out
      const int pos = __ffs(bal) - 1;
      if (lane == pos) {
        d = cd;
        id = ci;
      } else if (lane > pos && lane < KMAX) {
        d = pd;
        id = pi;
      }
    }
  };
  // 32 candidates, one per lane (valid where `ok`)
  auto consider = [&](float4 o, bool ok) {
    const float worst_d = __shfl_sync(0xffffffffu, d, KMAX - 1);
    const int worst_i = __shfl_sync(0xffffffffu, id, KMAX - 1);
    insert_batch(distance(o, ok, fminf(worst_d, keep_below)), __float_as_int(o.w), worst_d, worst_i);
  };
  // the lanes' 32 entries sorted ascending by (d2, index) across the warp (bitonic network, 15 exchanges)
  auto sort_lanes = [&]() {
#pragma unroll
    for (int k2 = 2; k2 <= 32; k2 <<= 1) {
#pragma unroll
      for (int j = k2 >> 1; j > 0; j >>= 1) {
        const float pd = __shfl_xor_sync(0xffffffffu, d, j);
        const int pi = __shfl_xor_sync(0xffffffffu, id, j);
        const bool keep_min = ((lane & j) == 0) == ((lane & k2) == 0);
        const bool take = keep_min ? before(pd, pi, d, id) : before(d, id, pd, pi);
        if (take) {
          d = pd;
          id = pi;
        }
      }
    }
  };
  // all atoms of the bins within s of the query's bin, straight from global memory
  auto scan_shell = [&](int s) {
    const int nx = exhaustive ? gx : min(2 * s + 1, gx);
    const int ny = exhaustive ? gy : min(2 * s + 1, gy);
    const int nz = exhaustive ? gz : min(2 * s + 1, gz);
    for (int ix = 0; ix < nx; ++ix) {
      const int bx = ((cx - s + ix) % gx + gx) % gx;
      for (int iy = 0; iy < ny; ++iy) {
        const int by = ((cy - s + iy) % gy + gy) % gy;
        for (int iz = 0; iz < nz; ++iz) {
          const int bz = ((cz - s + iz) % gz + gz) % gz;
          const int ob = (bx * gy + by) * gz + bz;
          const int e0 = start[ob], e1 = start[ob + 1];
          for (int e = e0; e < e1; e += 32) {
            const bool ok = e + lane < e1;
            consider(ok ? __ldg(sorted + e + lane) : make_float4(0.f, 0.f, 0.f, 0.f), ok);
          }
        }
      }
    }
    return nx == gx && ny == gy && nz == gz;  // every bin was visited
  };

  const int s_max = max(max(gx, gy), gz);
  for (int q = q0; q < q1; ++q) {
    me = __ldg(sorted + q);
    my_id = __float_as_int(me.w);
    d = INFINITY;
    id = 0x7fffffff;
    int s = 1;
    bool all_bins;
    keep_below = (covers_all || exhaustive || s_max <= 1) ? INFINITY : h * h * (1.f - 2e-5f);
    if (in_smem) {
      // first every candidate's distance, keeping those within the shell's reach; then the first 32 survivors are
      // sorted across the lanes in one go and become the list, the rest (few) are inserted one at a time
      int m = 0;
      for (int c0 = 0; c0 < n_cand; c0 += 32) {
        const bool ok = c0 + lane < n_cand;
        const float4 o = ok ? cand[c0 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float d2 = distance(o, ok, keep_below);
        const bool keep = d2 < keep_below;  // also drops the INF of lanes without a candidate
        const uint32_t bal = __ballot_sync(0xffffffffu, keep);
        if (keep) surv[m + __popc(bal & ((1u << lane) - 1u))] = make_float2(d2, o.w);
        m += __popc(bal);
      }
      __syncwarp();
      if (lane < m) {
        const float2 sv = surv[lane];
        d = sv.x;
        id = __float_as_int(sv.y);
      }
      sort_lanes();
      if (lane >= KMAX) {
        d = INFINITY;
        id = 0x7fffffff;
      }
      for (int c0 = 32; c0 < m; c0 += 32) {
        const bool ok = c0 + lane < m;
        const float2 sv = ok ? surv[c0 + lane] : make_float2(INFINITY, __int_as_float(0x7fffffff));
        const float worst_d = __shfl_sync(0xffffffffu, d, KMAX - 1);
        const int worst_i = __shfl_sync(0xffffffffu, id, KMAX - 1);
        insert_batch(sv.x, __float_as_int(sv.y), worst_d, worst_i);
      }
      __syncwarp();  // the survivor buffer is rewritten for the next query
      all_bins = covers_all;
    } else {
      all_bins = scan_shell(1);
    }
    // complete when the needed neighbours are known and the farthest of them is inside the searched shell
    while (!all_bins && !exhaustive) {
      const float reach = (float)s * h;
      const float kth = need >= 1 ? __shfl_sync(0xffffffffu, d, need - 1) : 0.f;
      if (kth < reach * reach * (1.f - 2e-5f) || s >= s_max) break;
      ++s;
      d = INFINITY;
      id = 0x7fffffff;
      {  // the reach of the new shell, unless it is the last one (every bin, or the largest half-width)
        const bool last = (2 * s + 1 >= gx && 2 * s + 1 >= gy && 2 * s + 1 >= gz) || s >= s_max;
        const float reach_s = (float)s * h;
        keep_below = last ? INFINITY : reach_s * reach_s * (1.f - 2e-5f);
      }
      all_bins = scan_shell(s);
    }
    if (lane < k) {
      const bool have = d < INFINITY;
      idx[((size_t)b * n_max + my_id) * k + lane] = have ? id : -1;
      if (dist2) dist2[((size_t)b * n_max + my_id) * k + lane] = have ? d : INFINITY;
    }
  }
  __syncwarp();  // the shared-memory list is refilled for the next bin
  }
}

// rows of padded atoms: no neighbours
__global__ void knn_pad_rows_kernel(const int32_t* __restrict__ num_atoms, int n_max, int k, int32_t* __restrict__ idx,
                                    float* __restrict__ dist2) {
  const int b = blockIdx.y;
  const int n = min(num_atoms[b], n_max);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // (row - n) * k + t
  const long long total = (long long)(n_max - n) * k;
  if (i >= total) return;
  const size_t off = ((size_t)b * n_max + n) * k + i;
  idx[off] = -1;
  if (dist2) dist2[off] = INFINITY;
}

KnnWorkspace carve(void* ws, int B, int N) {
  char* p = static_cast<char*>(ws);
  KnnWorkspace w;
  w.counts = reinterpret_cast<int32_t*>(p);
  p += align_up((size_t)B * (kMaxBins + 1) * 4, 256);
  w.cursor = reinterpret_cast<int32_t*>(p);
  p += align_up((size_t)B * kMaxBins * 4, 256);
  w.keys = reinterpret_cast<int32_t*>(p);
  p += align_up((size_t)B * N * 4, 256);
  w.flags = reinterpret_cast<int32_t*>(p);
  p += align_up((size_t)B * 4, 256);
  w.sorted = reinterpret_cast<float4*>(p);
  return w;
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" size_t mf_knn_cells_workspace_bytes(int32_t batch, int32_t n_max) {
  const size_t B = batch, N = n_max;
  return align_up(B * (kMaxBins + 1) * 4, 256) + align_up(B * kMaxBins * 4, 256) + align_up(B * N * 4, 256) +
         align_up(B * 4, 256) + align_up(B * N * sizeof(float4), 256);
}

extern "C" int mf_knn_search_grid(const float* cell, const int32_t* num_atoms, int32_t batch, int32_t n_max, int32_t k,
                                  int32_t* grid_dims, float* bounds, void* stream) {
  MF_CHECK_ARG(batch >= 0 && n_max >= 0 && k >= 1, "mf_knn_search_grid: bad size");
  if (batch == 0) return MF_OK;
  MF_CHECK_ARG(cell && num_atoms && grid_dims && bounds, "mf_knn_search_grid: null pointer argument");
  knn_grid_kernel<<<(batch + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(cell, num_atoms, batch, n_max, k,
                                                                                      grid_dims, bounds);
  MF_CHECK_LAUNCH("knn_grid_kernel");
  return MF_OK;
}

extern "C" int mf_knn_topk_cells(const float* frac, const float* cell, const int32_t* num_atoms,
                                 const int32_t* grid_dims, const float* bounds, int32_t batch, int32_t n_max,
                                 int32_t k, int32_t include_self, int32_t* idx, float* dist2, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  MF_CHECK_ARG(batch >= 0 && n_max >= 0, "mf_knn_topk_cells: negative size");
  MF_CHECK_ARG(k >= 1 && k <= 32, "mf_knn_topk_cells: k must be in [1, 32], got %d", (int)k);
  if (batch == 0 || n_max == 0) return MF_OK;
  MF_CHECK_ARG(frac && cell && num_atoms && grid_dims && bounds && idx, "mf_knn_topk_cells: null pointer argument");
  MF_CHECK_ARG(batch <= 65535, "mf_knn_topk_cells: batch above 65535");
  const size_t need = mf_knn_cells_workspace_bytes(batch, n_max);
  if (!workspace || workspace_bytes < need) {
    set_error("mf_knn_topk_cells: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    return MF_ERR_WORKSPACE_TOO_SMALL;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KnnWorkspace w = carve(workspace, batch, n_max);
  const int zero_n = batch * (kMaxBins + 1);
  knn_zero_kernel<<<(zero_n + 255) / 256, 256, 0, s>>>(w.counts, w.flags, batch);
  MF_CHECK_LAUNCH("knn_zero_kernel");
  dim3 per_atom((n_max + 255) / 256, batch);
  knn_count_kernel<<<per_atom, 256, 0, s>>>(frac, num_atoms, grid_dims, n_max, w);
  MF_CHECK_LAUNCH("knn_count_kernel");
  knn_scan_kernel<<<batch, 1024, 0, s>>>(grid_dims, w);
  MF_CHECK_LAUNCH("knn_scan_kernel");
  knn_fill_kernel<<<per_atom, 256, 0, s>>>(frac, num_atoms, n_max, w);
  MF_CHECK_LAUNCH("knn_fill_kernel");
  dim3 grid(64, batch);  // 256 warps per structure, each taking every 256th bin
  if (k <= 16)
    knn_warp_kernel<16><<<grid, 128, 0, s>>>(cell, num_atoms, grid_dims, bounds, n_max, k, include_self, w, idx, dist2);
  else
    knn_warp_kernel<32><<<grid, 128, 0, s>>>(cell, num_atoms, grid_dims, bounds, n_max, k, include_self, w, idx, dist2);
  MF_CHECK_LAUNCH("knn_warp_kernel");
  const long long pad = (long long)n_max * k;
  knn_pad_rows_kernel<<<dim3((unsigned)((pad + 255) / 256), batch), 256, 0, s>>>(num_atoms, n_max, k, idx, dist2);
  MF_CHECK_LAUNCH("knn_pad_rows_kernel");
  return MF_OK;
}
