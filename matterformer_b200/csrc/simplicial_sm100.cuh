// Definitions shared by the forward and backward tensor-core simplicial kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mf {

constexpr int kD = 64;          // head dimension handled by the tensor-core kernels
constexpr int kTileM = 128;     // queries per CTA = TMEM lanes
constexpr int kMaxKeys = 192;   // upper bound on the key count
constexpr int kStatusBytes = 256;

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct BatchInfo {
  int32_t n_keys;     // 1 + index of the last valid key (0 when none)
  int32_t n_queries;  // 1 + index of the last valid query
  int32_t reserved0;  // number of valid keys
  int32_t reserved1;
};

// Where row `token` of head `head` of batch element `batch` starts, in elements: (B,H,N,64) contiguous by default;
// the token-major form addresses slices of a packed projection (B,N,G,H,64) or a (B,N,H*64) activation directly.
struct RowLayout {
  long long batch, head, token;
  __host__ __device__ long long at(int b, int h, int n) const { return b * batch + h * head + n * token; }
};
inline RowLayout contiguous_rows(int heads, int tokens) {
  return RowLayout{(long long)heads * tokens * kD, (long long)tokens * kD, (long long)kD};
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Fills info[b] and a heaviest-first order of the batch; zeroes the status word.
int launch_schedule(const uint8_t* query_valid, const uint8_t* key_valid, int B, int N, BatchInfo* info,
                    int32_t* order, int32_t* status, cudaStream_t stream);

struct TileLayouts {   // non-default row layouts of a tile-kernel call (see RowLayout)
  RowLayout in;        // q, k1, v1, k2, v2 and their gradients
  RowLayout act;       // out_cast (forward), grad_out (backward)
  float q_scale;       // q is multiplied by this on load (a power of two), dq on store
};

// Offsets of the per-molecule extents and of the launch order behind the status block; returns the bytes used.
size_t simplicial_schedule_layout(int B, size_t* info_off, size_t* order_off);
// max_row_tiles(tokens) of simplicial_rows.cuh, computed once per token count.
int cached_max_row_tiles(int tokens);

}  // namespace mf
