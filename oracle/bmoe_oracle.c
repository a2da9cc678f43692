/*
 * bmoe_oracle.c - CPU restatement of the reference algorithms on the MoE
 * grouped-GEMM hot path. TEST INFRASTRUCTURE ONLY: tests, the smoke check and
 * the CPU-baseline leg of the benchmark may load this; the engine never does.
 *
 * Each function names the reference code it restates (paths relative to the
 * reference project root):
 *   orc_generate_counts      src/workload/workload.cpp:13-49,100-113
 *                            (+ GNU libstdc++ 13 std::mt19937_64,
 *                            std::generate_canonical<double,53> and
 *                            std::discrete_distribution, bits/random.tcc)
 *   orc_workload_metrics     src/workload/workload.cpp:127-172
 *   orc_build_tiles          src/scheduler/scheduler.cpp:37-60, 80-103
 *   orc_simulate             src/scheduler/scheduler.cpp:62-70, 105-145
 *   orc_schedule_metrics     src/scheduler/scheduler.cpp:147-211
 *   orc_routing_features     python/blackwell_moe_tirx/dispatch.py:42-83
 *   orc_select_variant       python/blackwell_moe_tirx/dispatch.py:86-114
 *   orc_probe_checksum       src/kernels/scheduler_probe.cu:18-47
 *   orc_grouped_gemm_*       FP32 sequential-k loop of
 *                            baselines/cutlass/test_correctness.cu:139-157 and
 *                            tests/test_sm100_dense_correctness.cu:113-129
 *
 * Pinning: the integer functions are checked against the reference's own
 * compiled sources (oracle/_ref, see build_oracle.py) and against fixtures in
 * tests/golden/ generated from the reference; the GEMM loop is checked against
 * the reference's known-answer inputs, whose FP32 sums are exact.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_EXPORT __attribute__((visibility("default")))

typedef struct orc_tile {
  uint32_t expert_id, tile_m, tile_n, valid_m, valid_n;
} orc_tile;

/* ------------------------------------------------------------------------ */
/* mt19937_64 (Matsumoto & Nishimura), as std::mt19937_64                    */
/* ------------------------------------------------------------------------ */
typedef struct {
  uint64_t mt[312];
  int index;
} orc_mt64;

static void mt64_seed(orc_mt64* g, uint64_t seed) {
  g->mt[0] = seed;
  for (int i = 1; i < 312; ++i) {
    g->mt[i] = 6364136223846793005ULL * (g->mt[i - 1] ^ (g->mt[i - 1] >> 62)) + (uint64_t)i;
  }
  g->index = 312;
}

static uint64_t mt64_next(orc_mt64* g) {
  if (g->index >= 312) {
    const uint64_t upper = 0xFFFFFFFF80000000ULL, lower = 0x7FFFFFFFULL;
    for (int i = 0; i < 312; ++i) {
      const uint64_t x = (g->mt[i] & upper) | (g->mt[(i + 1) % 312] & lower);
      uint64_t xa = x >> 1;
      if (x & 1ULL) xa ^= 0xB5026F5AA96619E9ULL;
      g->mt[i] = g->mt[(i + 156) % 312] ^ xa;
    }
    g->index = 0;
  }
  uint64_t y = g->mt[g->index++];
  y ^= (y >> 29) & 0x5555555555555555ULL;
  y ^= (y << 17) & 0x71D67FFFEDA60000ULL;
  y ^= (y << 37) & 0xFFF7EEE000000000ULL;
  y ^= y >> 43;
  return y;
}

/* std::generate_canonical<double, 53> over a 64-bit engine: one draw, divided
 * by 2^64, clamped below 1. */
static double canonical53(orc_mt64* g) {
  const double r = (double)mt64_next(g) / 18446744073709551616.0;
  return r >= 1.0 ? nextafter(1.0, 0.0) : r;
}

/* ------------------------------------------------------------------------ */
/* Workload generator                                                        */
/* ------------------------------------------------------------------------ */
static int fraction_ok(double x) { return x >= 0.0 && x <= 1.0; }

/* distribution: 0 uniform, 1 heavy_hitter, 2 sparse, 3 zipf (the reference's
 * four), 4 heavy_sparse (engine-side family without a reference counterpart:
 * the heavy-hitter rule for the leading experts, the sparse rule's count of idle
 * experts at the BACK, the rest shared evenly; same draw machinery).
 * Returns 0, or -1 for a configuration the reference rejects. */
ORC_EXPORT int orc_generate_counts(uint32_t experts, uint64_t total_tokens,
                                   uint32_t distribution, uint64_t seed,
                                   double zipf_alpha, double heavy_fraction,
                                   double heavy_share, double inactive_fraction,
                                   uint32_t* counts_out) {
  if (experts == 0 || distribution > 4 || !(zipf_alpha > 0.0)) return -1;
  if (!fraction_ok(heavy_fraction) || heavy_fraction == 0.0 ||
      !fraction_ok(heavy_share) || !fraction_ok(inactive_fraction)) {
    return -1;
  }
  double* w = (double*)malloc(sizeof(double) * experts);
  double* cp = (double*)malloc(sizeof(double) * experts);
  if (!w || !cp) { free(w); free(cp); return -1; }
  for (uint32_t i = 0; i < experts; ++i) w[i] = 1.0;
  if (distribution == 3) {
    for (uint32_t i = 0; i < experts; ++i) w[i] = 1.0 / pow((double)(i + 1), zipf_alpha);
  } else if (distribution == 1) {
    uint32_t heavy = (uint32_t)ceil(experts * heavy_fraction);
    if (heavy < 1) heavy = 1;
    const uint32_t light = experts - heavy;
    const double hw = heavy_share / heavy;
    const double lw = light == 0 ? 0.0 : (1.0 - heavy_share) / light;
    for (uint32_t i = 0; i < experts; ++i) w[i] = i < heavy ? hw : lw;
  } else if (distribution == 2) {
    uint32_t silent = (uint32_t)floor(experts * inactive_fraction);
    if (silent > experts - 1) silent = experts - 1;
    for (uint32_t i = 0; i < silent; ++i) w[i] = 0.0;
  } else if (distribution == 4) {
    uint32_t silent = (uint32_t)floor(experts * inactive_fraction);
    if (silent > experts - 1) silent = experts - 1;
    uint32_t heavy = (uint32_t)ceil(experts * heavy_fraction);
    if (heavy < 1) heavy = 1;
    if (heavy > experts - silent) heavy = experts - silent;
    const uint32_t light = experts - silent - heavy;
    const double hw = (light == 0 ? 1.0 : heavy_share) / heavy;
    const double lw = light == 0 ? 0.0 : (1.0 - heavy_share) / light;
    for (uint32_t i = 0; i < experts; ++i) {
      w[i] = i < heavy ? hw : (i < heavy + light ? lw : 0.0);
    }
  }
  memset(counts_out, 0, sizeof(uint32_t) * experts);

  orc_mt64 gen;
  mt64_seed(&gen, seed);
  if (experts < 2) {
    /* A distribution over fewer than two weights always returns 0 and does
     * not touch the engine. */
    counts_out[0] = (uint32_t)total_tokens;
  } else {
    double sum = 0.0;
    for (uint32_t i = 0; i < experts; ++i) sum += w[i];
    double run = 0.0;
    for (uint32_t i = 0; i < experts; ++i) {
      run += w[i] / sum; /* normalise, then partial sums, left to right */
      cp[i] = run;
    }
    cp[experts - 1] = 1.0;
    for (uint64_t t = 0; t < total_tokens; ++t) {
      const double p = canonical53(&gen);
      /* lower_bound: first index with cp[index] >= p */
      uint32_t lo = 0, hi = experts;
      while (lo < hi) {
        const uint32_t mid = lo + (hi - lo) / 2;
        if (cp[mid] < p) lo = mid + 1; else hi = mid;
      }
      counts_out[lo] += 1;
    }
  }
  free(w);
  free(cp);
  return 0;
}

static double population_cv(const double* v, size_t n) {
  if (n == 0) return 0.0;
  double s = 0.0;
  for (size_t i = 0; i < n; ++i) s += v[i];
  const double mean = s / (double)n;
  if (mean == 0.0) return 0.0;
  double ss = 0.0;
  for (size_t i = 0; i < n; ++i) {
    const double d = v[i] - mean;
    ss += d * d;
  }
  return sqrt(ss / (double)n) / mean;
}

/* out[0..5] = mean, cv, max/mean, inactive ratio, small-M ratio, tile cv;
 * out_int[0] = active experts, out_int[1] = total tiles. */
ORC_EXPORT int orc_workload_metrics(const uint32_t* counts, uint32_t experts,
                                    uint32_t n, uint32_t tile_m, uint32_t tile_n,
                                    double* out, uint64_t* out_int) {
  memset(out, 0, sizeof(double) * 6);
  out_int[0] = out_int[1] = 0;
  if (experts == 0) return 0;
  if (tile_m == 0 || tile_n == 0) return -1;
  double* tok = (double*)malloc(sizeof(double) * experts);
  double* til = (double*)malloc(sizeof(double) * experts);
  const uint32_t n_tiles = (n + tile_n - 1) / tile_n;
  uint64_t sum = 0;
  uint32_t largest = 0, silent = 0, small = 0;
  for (uint32_t e = 0; e < experts; ++e) {
    const uint32_t c = counts[e];
    sum += c;
    if (c > largest) largest = c;
    if (c == 0) ++silent;
    if (c > 0 && c < tile_m) ++small;
    if (c > 0) out_int[0] += 1;
    const uint64_t m_tiles = c == 0 ? 0 : (c + tile_m - 1) / tile_m;
    const uint64_t tiles = m_tiles * n_tiles;
    out_int[1] += tiles;
    tok[e] = (double)c;
    til[e] = (double)tiles;
  }
  out[0] = (double)sum / experts;
  out[1] = population_cv(tok, experts);
  out[5] = population_cv(til, experts);
  out[2] = out[0] == 0.0 ? 0.0 : largest / out[0];
  out[3] = (double)silent / experts;
  out[4] = (double)small / experts;
  free(tok);
  free(til);
  return 0;
}

/* ------------------------------------------------------------------------ */
/* Worklist                                                                  */
/* ------------------------------------------------------------------------ */
static uint64_t emit_expert(orc_tile* out, uint64_t cap, uint64_t at, uint32_t e,
                            uint32_t rows, uint32_t n, uint32_t tile_m,
                            uint32_t tile_n, uint32_t raster) {
  const uint32_t m_tiles = rows == 0 ? 0 : (rows + tile_m - 1) / tile_m;
  const uint32_t n_tiles = (n + tile_n - 1) / tile_n;
  const uint32_t outer = raster ? n_tiles : m_tiles;
  const uint32_t inner = raster ? m_tiles : n_tiles;
  for (uint32_t o = 0; o < outer; ++o) {
    for (uint32_t i = 0; i < inner; ++i) {
      const uint32_t tm = raster ? i : o;
      const uint32_t tn = raster ? o : i;
      if (at < cap) {
        orc_tile t;
        t.expert_id = e;
        t.tile_m = tm;
        t.tile_n = tn;
        t.valid_m = rows - tm * tile_m < tile_m ? rows - tm * tile_m : tile_m;
        t.valid_n = n - tn * tile_n < tile_n ? n - tn * tile_n : tile_n;
        out[at] = t;
      }
      ++at;
    }
  }
  return at;
}

/* order: 0 expert-major, 1 experts by descending tile count (stable).
 * raster: 0 tile_n fastest (reference), 1 tile_m fastest.
 * Returns the number of tiles (records beyond `cap` are not written), or
 * UINT64_MAX for zero tile dimensions. */
ORC_EXPORT uint64_t orc_build_tiles(const uint32_t* counts, uint32_t experts,
                                    uint32_t n, uint32_t tile_m, uint32_t tile_n,
                                    uint32_t order, uint32_t raster, orc_tile* out,
                                    uint64_t cap) {
  if (tile_m == 0 || tile_n == 0) return UINT64_MAX;
  uint32_t* visit = (uint32_t*)malloc(sizeof(uint32_t) * (experts ? experts : 1));
  for (uint32_t e = 0; e < experts; ++e) visit[e] = e;
  if (order == 1) {
    /* Stable insertion sort by descending tile count. The column-tile factor
     * is common to all experts, so the row-tile count is the key. */
    for (uint32_t i = 1; i < experts; ++i) {
      const uint32_t v = visit[i];
      const uint32_t kv = (counts[v] + tile_m - 1) / tile_m;
      uint32_t j = i;
      while (j > 0 && (counts[visit[j - 1]] + tile_m - 1) / tile_m < kv) {
        visit[j] = visit[j - 1];
        --j;
      }
      visit[j] = v;
    }
  }
  uint64_t at = 0;
  for (uint32_t p = 0; p < experts; ++p) {
    const uint32_t e = visit[p];
    at = emit_expert(out, cap, at, e, counts[e], n, tile_m, tile_n, raster);
  }
  free(visit);
  return at;
}

/* scheduler: SchedulerKind ordinal (0 expert order, 1 static persistent,
 * 2 dynamic queue, 3 compacted, 4 auto). tiles_out gets the per-CTA lists back
 * to back, cta_offsets[cta_count + 1] the boundaries. Returns the tile count
 * or UINT64_MAX on invalid input. */
ORC_EXPORT uint64_t orc_simulate(uint32_t scheduler, const uint32_t* counts,
                                 uint32_t experts, uint32_t n, uint32_t tile_m,
                                 uint32_t tile_n, uint32_t cta_count,
                                 orc_tile* tiles_out, uint64_t* cta_offsets) {
  if (cta_count == 0 || tile_m == 0 || tile_n == 0 || scheduler > 4) return UINT64_MAX;
  const uint64_t total =
      orc_build_tiles(counts, experts, n, tile_m, tile_n, 0, 0, NULL, 0);
  orc_tile* flat = (orc_tile*)malloc(sizeof(orc_tile) * (total ? total : 1));
  orc_build_tiles(counts, experts, n, tile_m, tile_n, scheduler == 1 ? 1 : 0, 0, flat, total);
  uint32_t* owner = (uint32_t*)malloc(sizeof(uint32_t) * (total ? total : 1));
  uint64_t* load = (uint64_t*)calloc(cta_count, sizeof(uint64_t));
  if (scheduler == 2) {
    for (uint64_t i = 0; i < total; ++i) {
      uint32_t best = 0;
      for (uint32_t c = 1; c < cta_count; ++c) {
        if (load[c] < load[best]) best = c;
      }
      owner[i] = best;
      uint64_t cost = (uint64_t)flat[i].valid_m * flat[i].valid_n;
      load[best] += cost ? cost : 1;
    }
  } else {
    for (uint64_t i = 0; i < total; ++i) owner[i] = (uint32_t)(i % cta_count);
  }
  uint64_t* fill = (uint64_t*)calloc(cta_count + 1, sizeof(uint64_t));
  for (uint64_t i = 0; i < total; ++i) fill[owner[i] + 1] += 1;
  for (uint32_t c = 0; c < cta_count; ++c) fill[c + 1] += fill[c];
  memcpy(cta_offsets, fill, sizeof(uint64_t) * (cta_count + 1));
  for (uint64_t i = 0; i < total; ++i) tiles_out[fill[owner[i]]++] = flat[i];
  free(fill);
  free(load);
  free(owner);
  free(flat);
  return total;
}

/* ints[0..5] = total tiles, valid, padded, expert switches, min, max tiles per
 * CTA; reals[0..5] = mean work, max work, cv, tail ratio, est. utilisation,
 * useful-work ratio. */
ORC_EXPORT int orc_schedule_metrics(const orc_tile* tiles, const uint64_t* cta_offsets,
                                    uint32_t cta_count, uint32_t tile_m,
                                    uint32_t tile_n, uint64_t* ints, double* reals) {
  memset(ints, 0, sizeof(uint64_t) * 6);
  memset(reals, 0, sizeof(double) * 6);
  if (tile_m == 0 || tile_n == 0) return -1;
  if (cta_count == 0) return 0;
  double* work = (double*)malloc(sizeof(double) * cta_count);
  ints[4] = UINT64_MAX;
  for (uint32_t c = 0; c < cta_count; ++c) {
    const uint64_t b = cta_offsets[c], e = cta_offsets[c + 1];
    const uint64_t cnt = e - b;
    ints[0] += cnt;
    if (cnt < ints[4]) ints[4] = cnt;
    if (cnt > ints[5]) ints[5] = cnt;
    uint64_t valid = 0;
    for (uint64_t i = b; i < e; ++i) {
      valid += (uint64_t)tiles[i].valid_m * tiles[i].valid_n;
      if (i > b && tiles[i].expert_id != tiles[i - 1].expert_id) ints[3] += 1;
    }
    ints[1] += valid;
    work[c] = (double)valid;
  }
  ints[2] = ints[0] * ((uint64_t)tile_m * tile_n);
  double sum = 0.0, peak = work[0];
  for (uint32_t c = 0; c < cta_count; ++c) {
    sum += work[c];
    if (work[c] > peak) peak = work[c];
  }
  reals[0] = sum / (double)cta_count;
  reals[1] = peak;
  if (reals[0] > 0.0) {
    double ss = 0.0;
    for (uint32_t c = 0; c < cta_count; ++c) {
      const double d = work[c] - reals[0];
      ss += d * d;
    }
    reals[2] = sqrt(ss / (double)cta_count) / reals[0];
    reals[3] = reals[1] / reals[0];
  }
  if (reals[1] > 0.0) reals[4] = (double)ints[1] / ((double)cta_count * reals[1]);
  if (ints[2] > 0) reals[5] = (double)ints[1] / (double)ints[2];
  free(work);
  return 0;
}

/* ------------------------------------------------------------------------ */
/* Dispatch                                                                  */
/* ------------------------------------------------------------------------ */
/* CPython >= 3.12 sums floats with Neumaier's compensated algorithm
 * (Python/bltinmodule.c, builtin_sum); the reference's variance sums go
 * through it, so the restatement does too. */
typedef struct { double sum, comp; } orc_pysum;

static void pysum_add(orc_pysum* s, double x) {
  const double t = s->sum + x;
  if (fabs(s->sum) >= fabs(x)) s->comp += (s->sum - t) + x;
  else s->comp += (x - t) + s->sum;
  s->sum = t;
}

static double pysum_result(const orc_pysum* s) {
  return (s->comp != 0.0 && isfinite(s->comp)) ? s->sum + s->comp : s->sum;
}

/* out[0..8] = mean_m, cv_m, max/mean, inactive ratio, small-M ratio (over
 * active experts, count <= tile_m), expert tile cv, max tiles/mean,
 * tiles per CTA, useful-work ratio; *active_tiles = tile total. */
ORC_EXPORT int orc_routing_features(const uint32_t* counts, uint32_t experts,
                                    uint32_t n, uint32_t tile_m, uint32_t tile_n,
                                    uint32_t cta_count, double* out,
                                    uint64_t* active_tiles) {
  memset(out, 0, sizeof(double) * 9);
  out[8] = 1.0;
  *active_tiles = 0;
  if (tile_m == 0 || tile_n == 0 || cta_count == 0) return -1;
  uint64_t sum = 0, largest = 0, active = 0, small = 0;
  for (uint32_t e = 0; e < experts; ++e) {
    sum += counts[e];
    if (counts[e] > largest) largest = counts[e];
    if (counts[e] > 0) {
      ++active;
      if (counts[e] <= tile_m) ++small;
    }
  }
  if (experts) {
    const double mean = (double)sum / (double)experts;
    out[0] = mean;
    if (mean != 0.0) {
      orc_pysum ss = {0.0, 0.0};
      for (uint32_t e = 0; e < experts; ++e) pysum_add(&ss, pow((double)counts[e] - mean, 2.0));
      out[1] = sqrt(pysum_result(&ss) / (double)experts) / mean;
      out[2] = (double)largest / mean;
    }
    out[3] = 1.0 - (double)active / (double)experts;
  }
  if (active) out[4] = (double)small / (double)active;

  const uint64_t whole_n = n / tile_n;
  const uint64_t all_n = ((uint64_t)n + tile_n - 1) / tile_n;
  uint64_t tile_sum = 0, tile_max = 0, m_tile_sum = 0;
  for (uint32_t e = 0; e < experts; ++e) {
    const uint64_t mt = ((uint64_t)counts[e] + tile_m - 1) / tile_m;
    const uint64_t t = mt * whole_n;
    tile_sum += t;
    m_tile_sum += mt;
    if (t > tile_max) tile_max = t;
  }
  if (experts) {
    const double mean_t = (double)tile_sum / (double)experts;
    if (mean_t != 0.0) {
      orc_pysum ss = {0.0, 0.0};
      for (uint32_t e = 0; e < experts; ++e) {
        const uint64_t t = (((uint64_t)counts[e] + tile_m - 1) / tile_m) * whole_n;
        pysum_add(&ss, pow((double)t - mean_t, 2.0));
      }
      out[5] = sqrt(pysum_result(&ss) / (double)experts) / mean_t;
      out[6] = (double)tile_max / mean_t;
    }
  }
  *active_tiles = m_tile_sum * all_n;
  out[7] = (double)*active_tiles / (double)cta_count;
  const uint64_t padded = *active_tiles * (uint64_t)tile_m * tile_n;
  if (padded) out[8] = (double)(sum * n) / (double)padded;
  return 0;
}

/* Returns 0 v0_nonpersistent, 1 v1_static_ws, 2 v2_dynamic, 3 v3_chunked,
 * 4 v4_hybrid with the bootstrap thresholds 1.0 / 0.25 / 2.0 / 4.0 / 1.0 / 0.5. */
ORC_EXPORT uint32_t orc_select_variant(double tiles_per_cta, double cv_m,
                                       double inactive_ratio) {
  if (tiles_per_cta <= 1.0) return 0;
  if (cv_m <= 0.25) return 1;
  if (tiles_per_cta < 2.0) return 1;
  if (tiles_per_cta >= 4.0 && (cv_m >= 1.0 || inactive_ratio >= 0.5)) return 4;
  if (tiles_per_cta >= 4.0) return 3;
  return 2;
}

/* ------------------------------------------------------------------------ */
/* Scheduler probe checksum                                                  */
/* ------------------------------------------------------------------------ */
static uint64_t mix64(uint64_t v) {
  v ^= v >> 30;
  v *= 0xbf58476d1ce4e5b9ULL;
  v ^= v >> 27;
  v *= 0x94d049bb133111ebULL;
  return v ^ (v >> 31);
}

ORC_EXPORT uint64_t orc_probe_checksum(const orc_tile* tile, uint32_t work_scale) {
  const uint64_t valid = (uint64_t)tile->valid_m * tile->valid_n;
  uint32_t rounds = work_scale * (uint32_t)((valid + 4095) / 4096);
  if (rounds < 1) rounds = 1;
  uint64_t all = 0;
  for (uint32_t thread = 0; thread < 256; ++thread) {
    uint64_t v = ((uint64_t)tile->expert_id << 48) ^ ((uint64_t)tile->tile_m << 32) ^
                 ((uint64_t)tile->tile_n << 16) ^ thread;
    for (uint32_t r = 0; r < rounds; ++r) v = mix64(v + r + 0x9e3779b97f4a7c15ULL);
    all ^= v;
  }
  return all;
}

/* ------------------------------------------------------------------------ */
/* Grouped GEMM                                                              */
/* ------------------------------------------------------------------------ */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Round to nearest, ties to even (NaN stays NaN). */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

#define ORC_COLS 128

/* acc[c] += a * bt[c] for a block of columns, exactly as the scalar loop does
 * per output element (FP32 multiply, FP32 add, ascending k). */
__attribute__((target_clones("avx512f", "avx2", "default")))
static void row_block_f32(const uint16_t* a_row, const float* bt, uint32_t k,
                          uint32_t cols, float* acc) {
  for (uint32_t c = 0; c < ORC_COLS; ++c) acc[c] = 0.0f;
  for (uint32_t kk = 0; kk < k; ++kk) {
    const float a = bf16_to_f32(a_row[kk]);
    const float* b = bt + (size_t)kk * ORC_COLS;
    for (uint32_t c = 0; c < ORC_COLS; ++c) acc[c] += a * b[c];
  }
  (void)cols;
}

__attribute__((target_clones("avx512f", "avx2", "default")))
static void row_block_f64(const uint16_t* a_row, const float* bt, uint32_t k,
                          double* acc) {
  for (uint32_t c = 0; c < ORC_COLS; ++c) acc[c] = 0.0;
  for (uint32_t kk = 0; kk < k; ++kk) {
    const double a = (double)bf16_to_f32(a_row[kk]);
    const float* b = bt + (size_t)kk * ORC_COLS;
    for (uint32_t c = 0; c < ORC_COLS; ++c) acc[c] += a * (double)b[c];
  }
}

/* Packed grouped GEMM on BF16 bit patterns.
 *   a      [sum(counts), k]  rows of expert 0, then expert 1, ...
 *   b      [experts, n, k]   (weights stored row-major [n, k] per expert)
 *   d_bf16 [sum(counts), n]  FP32 sequential-k result rounded to BF16 (may be NULL)
 *   d_f32  [sum(counts), n]  the unrounded FP32 sum (may be NULL)
 *   d_f64  [sum(counts), n]  FP64-accumulated value (may be NULL)
 * Only rows r (index inside the expert) with r % row_stride == row_phase are
 * computed; others are left untouched. threads <= 0 uses all cores. Returns
 * the number of rows computed. */
static uint64_t grouped_gemm_impl(const uint16_t* a, const uint16_t* b,
                                  const uint32_t* counts, uint32_t experts,
                                  uint32_t n, uint32_t k, uint16_t* d_bf16,
                                  float* d_f32, double* d_f64,
                                  uint32_t row_stride, uint32_t row_phase,
                                  uint32_t col_block_stride, uint32_t col_block_phase,
                                  int threads, uint64_t* elements_out) {
  if (row_stride == 0) row_stride = 1;
  if (col_block_stride == 0) col_block_stride = 1;
  uint64_t elements = 0;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  uint64_t rows_done = 0;
  uint64_t row_base = 0;
  float* bt = (float*)malloc(sizeof(float) * (size_t)k * ORC_COLS);
  for (uint32_t e = 0; e < experts; ++e) {
    const uint32_t rows = counts[e];
    if (rows == 0) continue;
    const uint16_t* be = b + (size_t)e * n * k;
    for (uint32_t c0 = 0; c0 < n; c0 += ORC_COLS) {
      const uint32_t cols = n - c0 < ORC_COLS ? n - c0 : ORC_COLS;
      if ((c0 / ORC_COLS) % col_block_stride != col_block_phase) continue;
      for (uint32_t r = row_phase; r < rows; r += row_stride) elements += cols;
      /* Transposed FP32 copy of the weight block: bt[kk][c]. */
#pragma omp parallel for schedule(static)
      for (uint32_t kk = 0; kk < k; ++kk) {
        float* dst = bt + (size_t)kk * ORC_COLS;
        for (uint32_t c = 0; c < cols; ++c) dst[c] = bf16_to_f32(be[(size_t)(c0 + c) * k + kk]);
        for (uint32_t c = cols; c < ORC_COLS; ++c) dst[c] = 0.0f;
      }
#pragma omp parallel for schedule(dynamic, 4)
      for (uint32_t r = row_phase; r < rows; r += row_stride) {
        const uint16_t* a_row = a + (size_t)(row_base + r) * k;
        const size_t out = (size_t)(row_base + r) * n + c0;
        if (d_bf16 != NULL || d_f32 != NULL) {
          float acc[ORC_COLS];
          row_block_f32(a_row, bt, k, cols, acc);
          for (uint32_t c = 0; c < cols; ++c) {
            if (d_f32) d_f32[out + c] = acc[c];
            if (d_bf16) d_bf16[out + c] = f32_to_bf16(acc[c]);
          }
        }
        if (d_f64 != NULL) {
          double acc64[ORC_COLS];
          row_block_f64(a_row, bt, k, acc64);
          for (uint32_t c = 0; c < cols; ++c) d_f64[out + c] = acc64[c];
        }
      }
    }
    for (uint32_t r = row_phase; r < rows; r += row_stride) ++rows_done;
    row_base += rows;
  }
  free(bt);
  if (elements_out != NULL) *elements_out = elements;
  return rows_done;
}

ORC_EXPORT uint64_t orc_grouped_gemm(const uint16_t* a, const uint16_t* b,
                                     const uint32_t* counts, uint32_t experts,
                                     uint32_t n, uint32_t k, uint16_t* d_bf16,
                                     float* d_f32, double* d_f64,
                                     uint32_t row_stride, uint32_t row_phase,
                                     int threads) {
  return grouped_gemm_impl(a, b, counts, experts, n, k, d_bf16, d_f32, d_f64, row_stride,
                           row_phase, 1, 0, threads, NULL);
}

/* The same loop over a SAMPLE OF COLUMN BLOCKS: all rows of every expert, but only the
 * 128-column blocks whose index % col_block_stride == col_block_phase. Every sampled
 * block does what the full problem does for it (weight block made ready once, then all
 * rows), so the time per output element is that of the full problem; a row sample is
 * not (the per-expert weight preparation is then shared by fewer rows). Used to time a
 * bounded part of a large configuration. Returns the number of output elements
 * computed (FLOPs = 2 * k * elements). */
ORC_EXPORT uint64_t orc_grouped_gemm_column_sample(const uint16_t* a, const uint16_t* b,
                                                   const uint32_t* counts, uint32_t experts,
                                                   uint32_t n, uint32_t k, uint16_t* d_bf16,
                                                   uint32_t col_block_stride,
                                                   uint32_t col_block_phase, int threads) {
  uint64_t elements = 0;
  grouped_gemm_impl(a, b, counts, experts, n, k, d_bf16, NULL, NULL, 1, 0, col_block_stride,
                    col_block_phase, threads, &elements);
  return elements;
}

/* Weighted top-k combine: out[t,:] = bf16(sum_j w[t,j] * float(src[row[t,j],:])),
 * FP32, one fmaf per term, j ascending, one rounding to BF16. The reference has
 * no such function (its callers own the un-permute, agent/search_space.yaml:13);
 * this states the engine's definition of the step on the CPU. Rows < 0 or
 * >= src_rows are dropped assignments. weights may be NULL (all 1.0f). */
ORC_EXPORT int orc_combine_topk(const uint16_t* src, uint64_t src_rows, const int64_t* row,
                                const float* weights, uint64_t tokens, uint32_t top_k,
                                uint32_t n, uint16_t* out) {
  if (src == NULL || row == NULL || out == NULL || top_k == 0) return -1;
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < (int64_t)tokens; ++t) {
    for (uint32_t c = 0; c < n; ++c) {
      float acc = 0.0f;
      for (uint32_t j = 0; j < top_k; ++j) {
        const int64_t r = row[(uint64_t)t * top_k + j];
        if (r < 0 || (uint64_t)r >= src_rows) continue;
        const float w = weights != NULL ? weights[(uint64_t)t * top_k + j] : 1.0f;
        acc = fmaf(w, bf16_to_f32(src[(uint64_t)r * n + c]), acc);
      }
      out[(uint64_t)t * n + c] = f32_to_bf16(acc);
    }
  }
  return 0;
}

ORC_EXPORT int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* FP8 E4M3 operands                                                         */
/* ------------------------------------------------------------------------ */
/* The reference declares DataType::kFp8E4M3 (include/blackwell_moe/kernels/
 * grouped_gemm.cuh:10) and implements nothing for it, so there is nothing of the
 * reference's to follow here: these state the OCP 8-bit floating point format E4M3
 * (1 sign, 4 exponent bits with bias 7, 3 mantissa bits; no infinities, S.1111.111 is
 * NaN, largest finite value 448) and the engine's definition of the FP8 grouped GEMM:
 * every operand byte decoded exactly, then the BF16 contract's loop. Every E4M3 value is
 * exactly representable in BF16, so decoding to BF16 bit patterns and calling
 * orc_grouped_gemm IS the FP8 oracle. */
static inline float e4m3_to_f32(uint8_t v) {
  const uint32_t sign = v >> 7, exponent = (v >> 3) & 15u, mantissa = v & 7u;
  float magnitude;
  if (exponent == 15u && mantissa == 7u) {
    magnitude = NAN;
  } else if (exponent == 0u) {
    magnitude = ldexpf((float)mantissa, -9);             /* subnormal: m/8 * 2^-6 */
  } else {
    magnitude = ldexpf((float)(8u + mantissa), (int)exponent - 10);   /* (1 + m/8) * 2^(e-7) */
  }
  return sign ? -magnitude : magnitude;
}

ORC_EXPORT void orc_e4m3_to_bf16(const uint8_t* src, uint64_t count, uint16_t* dst) {
  for (uint64_t i = 0; i < count; ++i) dst[i] = f32_to_bf16(e4m3_to_f32(src[i]));
}

ORC_EXPORT float orc_e4m3_to_f32(uint8_t v) { return e4m3_to_f32(v); }

/* Round to nearest, ties to even, saturating to +-448 (NaN stays NaN). */
ORC_EXPORT uint8_t orc_f32_to_e4m3(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
  const float a = fabsf(f);
  if (a != a) return (uint8_t)(sign | 0x7fu);
  if (a >= 448.0f) return (uint8_t)(sign | 0x7eu);
  if (a < ldexpf(1.0f, -6)) {
    /* subnormal range: multiples of 2^-9 */
    const float q = nearbyintf(ldexpf(a, 9));            /* 0 .. 8, ties to even */
    return (uint8_t)(sign | (uint8_t)q);                 /* 8 = smallest normal, 0x08 */
  }
  int e;
  const float frac = frexpf(a, &e);                      /* a = frac * 2^e, frac in [0.5, 1) */
  float q = nearbyintf(ldexpf(frac, 4));                 /* 8 .. 16 */
  if (q == 16.0f) { q = 8.0f; ++e; }
  const uint32_t exponent = (uint32_t)(e - 1 + 7);
  const uint32_t code = (exponent << 3) | ((uint32_t)q - 8u);
  return (uint8_t)(sign | (code > 0x7eu ? 0x7eu : code));
}

ORC_EXPORT uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
ORC_EXPORT float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
