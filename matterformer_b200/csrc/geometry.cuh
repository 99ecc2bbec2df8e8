// Device functions shared by the periodic-geometry kernels: the fixed-order minimum-image distance and
// the grid cell of a fractional coordinate.  One definition, so every kernel (and the CPU oracle that
// repeats it operation for operation) produces the same bits.
#pragma once

#include <cuda_runtime.h>
#include <math.h>

namespace mf {

struct Cell {
  float l00, l10, l11, l20, l21, l22;
};

__device__ __forceinline__ Cell load_cell(const float* cell) {
  Cell c;
  c.l00 = cell[0];
  c.l10 = cell[3];
  c.l11 = cell[4];
  c.l20 = cell[6];
  c.l21 = cell[7];
  c.l22 = cell[8];
  return c;
}

// Squared minimum-image distance; see the formula in include/matterformer_b200.h.
// Explicit round-to-nearest intrinsics: the compiler may neither fuse nor reorder them.
__device__ __forceinline__ float min_image_d2(float xi, float yi, float zi, float xj, float yj, float zj,
                                              const Cell& c) {
  const float dx = __fsub_rn(xi, xj), dy = __fsub_rn(yi, yj), dz = __fsub_rn(zi, zj);
  float best = INFINITY;
#pragma unroll
  for (int ox = -1; ox <= 1; ++ox) {
    const float ax = __fadd_rn(dx, (float)ox);
    const float rx0 = __fmul_rn(ax, c.l00);
#pragma unroll
    for (int oy = -1; oy <= 1; ++oy) {
      const float ay = __fadd_rn(dy, (float)oy);
      const float rx1 = __fmaf_rn(ay, c.l10, rx0);
      const float ry0 = __fmul_rn(ay, c.l11);
#pragma unroll
      for (int oz = -1; oz <= 1; ++oz) {
        const float az = __fadd_rn(dz, (float)oz);
        const float rx = __fmaf_rn(az, c.l20, rx1);
        const float ry = __fmaf_rn(az, c.l21, ry0);
        const float rz = __fmul_rn(az, c.l22);
        const float d2 = __fmaf_rn(rz, rz, __fmaf_rn(ry, ry, __fmul_rn(rx, rx)));
        if (d2 < best) best = d2;  // strict: the first minimum wins
      }
    }
  }
  return best;
}

// squared length of one image: delta + (ox, oy, oz), same operation sequence as inside min_image_d2
__device__ __forceinline__ float image_d2(float dx, float dy, float dz, float ox, float oy, float oz, const Cell& c) {
  const float ax = __fadd_rn(dx, ox), ay = __fadd_rn(dy, oy), az = __fadd_rn(dz, oz);
  const float rx = __fmaf_rn(az, c.l20, __fmaf_rn(ay, c.l10, __fmul_rn(ax, c.l00)));
  const float ry = __fmaf_rn(az, c.l21, __fmul_rn(ay, c.l11));
  const float rz = __fmul_rn(az, c.l22);
  return __fmaf_rn(rz, rz, __fmaf_rn(ry, ry, __fmul_rn(rx, rx)));
}

__device__ __forceinline__ int cell_coord(float f, int g) {
  const float w = __fsub_rn(f, floorf(f));  // wrapped to [0,1]
  int c = (int)__fmul_rn(w, (float)g);
  return min(max(c, 0), g - 1);
}

}  // namespace mf
