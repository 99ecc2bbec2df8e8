/*
 * CPU restatement of the periodic geometry used by the kernels (TEST INFRASTRUCTURE).
 *
 * Only tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py load this file's
 * shared object; the product never does.
 *
 * The distance follows PeriodicGeometryAdapter.forward of the reference
 * (src/matterformer/geometry/adapters.py:176-190): fractional delta plus each of the 27 lattice
 * offsets in itertools.product(range(-1,2), repeat=3) order (:141-149), squared length under the
 * cell metric, first minimum wins (argmin, :185).  The reference evaluates delta^T G delta with an
 * einsum whose summation order is unspecified; this restatement (and the CUDA kernels, operation
 * for operation) evaluates |delta L|^2 with one fixed sequence of fp32 operations instead, so
 * integer results can be compared bit for bit:
 *     r_x = fma(d2, L20, fma(d1, L10, d0*L00)); r_y = fma(d2, L21, d1*L11); r_z = d2*L22
 *     dist2 = fma(r_z, r_z, fma(r_y, r_y, r_x*r_x))
 * Parity with the reference's own arithmetic is checked in tests against golden vectors the
 * reference produced (tests/golden/), up to pairs whose distances differ by a few ulp.
 *
 * kNN semantics: ascending (dist2, index) order, self excluded unless asked, first k; the only kNN
 * statement in the reference project is the non-periodic legacy/rapidash_v5/models/rapidash_utils.py:139-193.
 *
 * Compile with -ffp-contract=off so the compiler neither fuses nor splits the operations above.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- a minimal parallel-for over pthreads (no OpenMP runtime on the build image) ---- */
static int g_threads = 1;
void mfo_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
int mfo_get_threads(void) { return g_threads; }

typedef void (*task_fn)(int index, void* ctx);
typedef struct { task_fn fn; void* ctx; int count; int next; pthread_mutex_t mu; } pool_t;

static void* pool_worker(void* arg) {
  pool_t* p = (pool_t*)arg;
  for (;;) {
    pthread_mutex_lock(&p->mu);
    const int i = p->next++;
    pthread_mutex_unlock(&p->mu);
    if (i >= p->count) break;
    p->fn(i, p->ctx);
  }
  return NULL;
}

static void parallel_for(int count, task_fn fn, void* ctx) {
  pool_t p;
  p.fn = fn; p.ctx = ctx; p.count = count; p.next = 0;
  pthread_mutex_init(&p.mu, NULL);
  int nt = g_threads < count ? g_threads : count;
  if (nt <= 1) {
    for (int i = 0; i < count; ++i) fn(i, ctx);
  } else {
    pthread_t th[256];
    for (int t = 0; t < nt; ++t) pthread_create(&th[t], NULL, pool_worker, &p);
    for (int t = 0; t < nt; ++t) pthread_join(th[t], NULL);
  }
  pthread_mutex_destroy(&p.mu);
}

static inline float min_image_d2(const float* pi, const float* pj, const float* cell) {
  const float l00 = cell[0], l10 = cell[3], l11 = cell[4], l20 = cell[6], l21 = cell[7], l22 = cell[8];
  const float dx = pi[0] - pj[0], dy = pi[1] - pj[1], dz = pi[2] - pj[2];
  float best = INFINITY;
  for (int ox = -1; ox <= 1; ++ox) {
    const float ax = dx + (float)ox;
    const float rx0 = ax * l00;
    for (int oy = -1; oy <= 1; ++oy) {
      const float ay = dy + (float)oy;
      const float rx1 = fmaf(ay, l10, rx0);
      const float ry0 = ay * l11;
      for (int oz = -1; oz <= 1; ++oz) {
        const float az = dz + (float)oz;
        const float rx = fmaf(az, l20, rx1);
        const float ry = fmaf(az, l21, ry0);
        const float rz = az * l22;
        const float d2 = fmaf(rz, rz, fmaf(ry, ry, rx * rx));
        if (d2 < best) best = d2;
      }
    }
  }
  return best;
}

/* all-pairs minimum-image squared distances of one structure: out (n,n) */
void mfo_pair_dist2(const float* frac, const float* cell, int n, float* out) {
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) out[(size_t)i * n + j] = min_image_d2(frac + 3 * i, frac + 3 * j, cell);
}

typedef struct {
  const float* frac; const float* cell; const int32_t* num_atoms; int batch, n_max, k, include_self, chunks;
  int32_t* idx; float* dist2;
} knn_ctx;

#define KNN_ROWS_PER_TASK 256

static void knn_task(int task, void* vctx) {
  const knn_ctx* a = (const knn_ctx*)vctx;
  const int b = task / a->chunks, chunk = task % a->chunks;
  const int n_max = a->n_max, k = a->k, include_self = a->include_self;
  int32_t* idx = a->idx; float* dist2 = a->dist2;
  {
    const int n = a->num_atoms[b] < n_max ? a->num_atoms[b] : n_max;
    const float* pos = a->frac + (size_t)b * n_max * 3;
    const float* c = a->cell + (size_t)b * 9;
    float* bd = (float*)malloc(sizeof(float) * (size_t)k);
    int32_t* bi = (int32_t*)malloc(sizeof(int32_t) * (size_t)k);
    const int i_end = (chunk + 1) * KNN_ROWS_PER_TASK < n_max ? (chunk + 1) * KNN_ROWS_PER_TASK : n_max;
    for (int i = chunk * KNN_ROWS_PER_TASK; i < i_end; ++i) {
      for (int t = 0; t < k; ++t) { bd[t] = INFINITY; bi[t] = -1; }
      if (i < n) {
        for (int j = 0; j < n; ++j) {
          if (j == i && !include_self) continue;
          const float d2 = min_image_d2(pos + 3 * i, pos + 3 * j, c);
          if (!(d2 < bd[k - 1])) continue;
          int t = k - 1; /* insert after every entry with distance <= d2 */
          while (t > 0 && bd[t - 1] > d2) { bd[t] = bd[t - 1]; bi[t] = bi[t - 1]; --t; }
          bd[t] = d2; bi[t] = j;
        }
      }
      memcpy(idx + ((size_t)b * n_max + i) * k, bi, sizeof(int32_t) * (size_t)k);
      if (dist2) memcpy(dist2 + ((size_t)b * n_max + i) * k, bd, sizeof(float) * (size_t)k);
    }
    free(bd); free(bi);
  }
}

/* kNN over a batch; same output convention as mf_knn_topk */
void mfo_knn_topk(const float* frac, const float* cell, const int32_t* num_atoms, int batch, int n_max, int k,
                  int include_self, int32_t* idx, float* dist2) {
  knn_ctx a = {frac, cell, num_atoms, batch, n_max, k, include_self, (n_max + KNN_ROWS_PER_TASK - 1) / KNN_ROWS_PER_TASK,
               idx, dist2};
  parallel_for(batch * a.chunks, knn_task, &a);
}

static inline int cell_coord(float f, int g) {
  const float w = f - floorf(f);
  int c = (int)(w * (float)g);
  if (c < 0) c = 0;
  if (c > g - 1) c = g - 1;
  return c;
}

typedef struct {
  const float* frac; const float* cell; const int32_t* num_atoms; const int32_t* grid_dims; int batch, n_max;
  float cutoff; int32_t* perm; int32_t* block_count; int32_t* block_cols; uint32_t* block_mask;
} blk_ctx;

static void blocklist_task(int b, void* vctx) {
  const blk_ctx* a = (const blk_ctx*)vctx;
  const int n_max = a->n_max;
  const float cutoff = a->cutoff;
  const int32_t* grid_dims = a->grid_dims;
  int32_t* perm = a->perm; int32_t* block_count = a->block_count; int32_t* block_cols = a->block_cols;
  uint32_t* block_mask = a->block_mask;
  const int tiles = (n_max + 31) / 32;
  {
    const int n = a->num_atoms[b] < n_max ? a->num_atoms[b] : n_max;
    const float* pos = a->frac + (size_t)b * n_max * 3;
    const float* c = a->cell + (size_t)b * 9;
    const int gx = grid_dims[3 * b], gy = grid_dims[3 * b + 1], gz = grid_dims[3 * b + 2];
    int32_t* keys = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n_max > 0 ? n_max : 1));
    int32_t* pb = perm + (size_t)b * n_max;
    for (int i = 0; i < n; ++i)
      keys[i] = (cell_coord(pos[3 * i], gx) * gy + cell_coord(pos[3 * i + 1], gy)) * gz + cell_coord(pos[3 * i + 2], gz);
    for (int i = 0; i < n; ++i) {
      int rank = 0;
      for (int j = 0; j < n; ++j) rank += (keys[j] < keys[i]) || (keys[j] == keys[i] && j < i);
      pb[rank] = i;
    }
    for (int i = n; i < n_max; ++i) pb[i] = i;
    for (int I = 0; I < tiles; ++I) {
      int cnt = 0;
      int32_t* cols = block_cols + ((size_t)b * tiles + I) * tiles;
      for (int J = 0; J < tiles; ++J) {
        uint32_t* words = block_mask + (((size_t)b * tiles + I) * tiles + J) * 32;
        int any = 0;
        for (int r = 0; r < 32; ++r) {
          uint32_t w = 0;
          const int si = 32 * I + r;
          for (int cc = 0; cc < 32; ++cc) {
            const int sj = 32 * J + cc;
            if (si < n && sj < n) {
              const float d2 = min_image_d2(pos + 3 * pb[si], pos + 3 * pb[sj], c);
              if (sqrtf(d2) <= cutoff) w |= (1u << cc);
            }
          }
          words[r] = w;
          any |= (w != 0);
        }
        if (any) cols[cnt++] = J;
      }
      block_count[(size_t)b * tiles + I] = cnt;
      for (int t = cnt; t < tiles; ++t) cols[t] = -1;
    }
    free(keys);
  }
}

/* cell sort + block list + pair bitmaps; same output convention as mf_cell_sort_blocklist */
void mfo_cell_sort_blocklist(const float* frac, const float* cell, const int32_t* num_atoms, const int32_t* grid_dims,
                             int batch, int n_max, float cutoff, int32_t* perm, int32_t* block_count,
                             int32_t* block_cols, uint32_t* block_mask) {
  blk_ctx a = {frac, cell, num_atoms, grid_dims, batch, n_max, cutoff, perm, block_count, block_cols, block_mask};
  parallel_for(batch, blocklist_task, &a);
}
