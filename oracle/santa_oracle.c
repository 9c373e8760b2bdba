/*
 * santa_oracle.c -- CPU restatement of the S2ANTA decode-attention sampler and
 * estimators (fixed "Flash" tile budgets and proportional "Prop" tile budgets).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the parity tests,
 * the smoke test and the benchmark's CPU-baseline leg compare the CUDA path
 * against.  Nothing in the shipped product path links, imports or calls it.
 *
 * Every function cites the reference file:line it restates (paths relative to
 * the OPUSLab/SANTA tree):
 *   F.cpp = flash_style_fused_santa_fixed_tile_budgets/santa_cuda.cpp
 *   F.cu  = flash_style_fused_santa_fixed_tile_budgets/santa_cuda_kernel.cu
 *   P.cpp = santa_fused_proportional_tile_budgets/santa_cuda.cpp
 *   P.cu  = santa_fused_proportional_tile_budgets/santa_cuda_kernel.cu
 *
 * Parity pinning.  The reference ships no golden vectors or known-answer tests
 * for this path.  The integer and IEEE-exact parts below (tile rule, budget
 * rule, splitmix64 offsets, score order, systematic counts, compaction,
 * largest-remainder apportionment) are pinned against fixtures under
 * tests/golden/ that were produced by running the reference's own kernels on a
 * B200 (see tests/golden/README.md).  Two hardware-approximate primitives the
 * reference uses on the GPU -- ex2.approx behind __expf and div.approx under
 * --use_fast_math -- cannot be reproduced bit-for-bit on a CPU; they are
 * modelled with exp2f()/IEEE division here and every entry point that depends
 * on them also accepts the GPU's values as an injected input so that the
 * downstream integer results can still be compared bit-exactly.
 *
 * Build:  make -C oracle   (gcc -O2 -ffp-contract=off -mfma -mf16c)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__GNUC__)
#define SANTA_API __attribute__((visibility("default")))
#else
#define SANTA_API
#endif

/* ------------------------------------------------------------------ */
/* 16-bit storage types                                                */
/* ------------------------------------------------------------------ */

static inline float bf16_to_f32(uint16_t v) {
  uint32_t w = (uint32_t)v << 16;
  float f;
  memcpy(&f, &w, 4);
  return f;
}

/* round-to-nearest-even, NaN -> quiet NaN (what __float2bfloat16 does) */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t w;
  memcpy(&w, &f, 4);
  if ((w & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
  uint32_t lsb = (w >> 16) & 1u;
  w += 0x7fffu + lsb;
  return (uint16_t)(w >> 16);
}

static inline float f16_to_f32(uint16_t v) {
  _Float16 h;
  memcpy(&h, &v, 2);
  return (float)h;
}

static inline uint16_t f32_to_f16(float f) {
  _Float16 h = (_Float16)f; /* RN-even, like __float2half_rn */
  uint16_t v;
  memcpy(&v, &h, 2);
  return v;
}

static inline float load16(const uint16_t *p, int is_bf16) {
  return is_bf16 ? bf16_to_f32(*p) : f16_to_f32(*p);
}
static inline uint16_t store16(float f, int is_bf16) {
  return is_bf16 ? f32_to_bf16(f) : f32_to_f16(f);
}

SANTA_API void santa_or_f32_to_16(const float *src, uint16_t *dst, long n, int is_bf16) {
  for (long i = 0; i < n; ++i) dst[i] = store16(src[i], is_bf16);
}
SANTA_API void santa_or_16_to_f32(const uint16_t *src, float *dst, long n, int is_bf16) {
  for (long i = 0; i < n; ++i) dst[i] = load16(src + i, is_bf16);
}

/* model of __expf(x): fp32 multiply by log2(e), then 2^y (the GPU uses the
 * ex2.approx unit for the second step; exp2f is the CPU stand-in). */
static inline float expf_model(float x) { return exp2f(x * 1.4426950408889634f); }

/* ------------------------------------------------------------------ */
/* Host rules                                                          */
/* ------------------------------------------------------------------ */

/* F.cpp:36-44, P.cpp:61-77 -- tile size from the valid length */
SANTA_API int santa_or_block_n(int L, int block_n) {
  if (block_n > 0) return block_n;
  if (L <= 1536) return 32;
  if (L <= 3072) return 64;
  return 256;
}

/* F.cpp:202-208 -- number of tiles and the fixed per-tile sample budget */
SANTA_API void santa_or_flash_budget(int L, int block_n, long S, int *T_c, int *S_per_tile) {
  int tc = (L + block_n - 1) / block_n;
  int spt = 0;
  if (S > 0) {
    spt = (int)(S / tc);
    if (spt < 1) spt = 1;
  }
  *T_c = tc;
  *S_per_tile = spt;
}

/* F.cu:74-87 == P.cu:557-570 -- per-(head, tile) stratification offset */
static inline uint64_t mix64(uint64_t x) {
  uint64_t z = x + 0x9e3779b97f4a7c15ULL;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
  return z ^ (z >> 31);
}
SANTA_API float santa_or_u01(uint64_t seed, int h, int t) {
  /* int -> uint64 conversion sign-extends, exactly as uint64_t(h) does */
  uint64_t key = seed ^ (((uint64_t)(int64_t)h << 32) ^ (uint64_t)(int64_t)t);
  uint64_t r = mix64(key);
  double u = (double)(r >> 11) * (1.0 / 9007199254740992.0);
  return (float)u;
}

/* ------------------------------------------------------------------ */
/* Scores                                                              */
/* ------------------------------------------------------------------ */

/* F.cu:161-221 / P.cu:317-379 -- "vec" score order.
 * 32 lane partials, each a 4-term fma chain over dims 4i..4i+3 of
 * (fp32(q)*q_scale) x fp32(k), then the shfl_down tree 16,8,4,2,1 read at
 * lane 0.  q16:[H,128]  K16:[L_storage,KVH,128]  scores:[H,L] (head-major). */
SANTA_API void santa_or_scores_vec(const uint16_t *q16, const uint16_t *K16, int is_bf16,
                                   int H, int KVH, int L, float q_scale, float *scores) {
  const int D = 128;
  const int GH = H / KVH;
  float *qs = (float *)malloc(sizeof(float) * (size_t)H * D);
  for (int i = 0; i < H * D; ++i) qs[i] = load16(q16 + i, is_bf16) * q_scale;
  for (int n = 0; n < L; ++n) {
    for (int kv = 0; kv < KVH; ++kv) {
      float kf[128];
      const uint16_t *kp = K16 + ((size_t)n * KVH + kv) * D;
      for (int d = 0; d < D; ++d) kf[d] = load16(kp + d, is_bf16);
      for (int g = 0; g < GH; ++g) {
        const float *qh = qs + (size_t)(kv * GH + g) * D;
        float p[32];
        for (int i = 0; i < 32; ++i) {
          float s = 0.f;
          s = fmaf(qh[4 * i + 0], kf[4 * i + 0], s);
          s = fmaf(qh[4 * i + 1], kf[4 * i + 1], s);
          s = fmaf(qh[4 * i + 2], kf[4 * i + 2], s);
          s = fmaf(qh[4 * i + 3], kf[4 * i + 3], s);
          p[i] = s;
        }
        for (int off = 16; off > 0; off >>= 1)
          for (int i = 0; i < off; ++i) p[i] = p[i] + p[i + off];
        scores[(size_t)(kv * GH + g) * L + n] = p[0];
      }
    }
  }
  free(qs);
}

/* P.cu:126-187 -- tensor-core ("WMMA") score path used by Prop when the vec
 * path does not apply: q*scale is ROUNDED to the storage type, products are
 * accumulated in fp32 in 16-wide k-steps.  The accumulation order inside one
 * tensor-core step is hardware-defined; this model sums the 16 products of a
 * k-step in double and rounds once per step, which agrees with the GPU to a
 * few ulps (callers inject the GPU's scores when exact downstream results are
 * needed). */
SANTA_API void santa_or_scores_mma(const uint16_t *q16, const uint16_t *K16, int is_bf16,
                                   int H, int KVH, int L, int D, float q_scale, float *scores) {
  const int GH = H / KVH;
  float *qs = (float *)malloc(sizeof(float) * (size_t)H * D);
  for (int i = 0; i < H * D; ++i)
    qs[i] = load16(&(uint16_t){store16(load16(q16 + i, is_bf16) * q_scale, is_bf16)}, is_bf16);
  for (int n = 0; n < L; ++n)
    for (int kv = 0; kv < KVH; ++kv) {
      const uint16_t *kp = K16 + ((size_t)n * KVH + kv) * D;
      for (int g = 0; g < GH; ++g) {
        const float *qh = qs + (size_t)(kv * GH + g) * D;
        float acc = 0.f;
        for (int k0 = 0; k0 < D; k0 += 16) {
          double part = 0.0;
          for (int k = k0; k < k0 + 16; ++k) part += (double)qh[k] * (double)load16(kp + k, is_bf16);
          acc = (float)((double)acc + part);
        }
        scores[(size_t)(kv * GH + g) * L + n] = acc;
      }
    }
  free(qs);
}

/* ------------------------------------------------------------------ */
/* Tile statistics                                                     */
/* ------------------------------------------------------------------ */

/* F.cu:223-273 / P.cu:381-440 -- per (head, tile): m_t = max score,
 * u = __expf(s - m_t) (kept in fp32 for the sum, rounded to the storage type
 * for sampling) and ell_t = sum of the unrounded u in the reference's order:
 *   thread `tid` of a block of NW warps owns head g = tid%4 and rows
 *   tid/4 + (8*NW)*j, j ascending; a 32-lane shfl_down tree per warp (the
 *   lanes of the other heads add exact zeros); warps summed w = 0..NW-1.
 * NW = 8 for block_n == 256, else 4 (F.cu:520-521,558-560).
 * scores:[H,L]; m_tiles, ell_tiles:[H,T_c]; u16:[H,L] storage-type bits.
 * If u16_inject != NULL its values replace the modelled exp (ell is then
 * summed from fp32 u recomputed by the model -- pass ell_inject too when the
 * GPU's ell is wanted downstream). */
static float ell_reference_order(const float *u, int tile_len, int NW) {
  const int RPP = 8 * NW; /* rows covered by one pass of the block */
  float W[8];
  for (int w = 0; w < NW; ++w) {
    float V[8];
    for (int k = 0; k < 8; ++k) {
      float acc = 0.f;
      for (int r = 8 * w + k; r < tile_len; r += RPP) acc += u[r];
      V[k] = acc;
    }
    W[w] = ((V[0] + V[4]) + (V[2] + V[6])) + ((V[1] + V[5]) + (V[3] + V[7]));
  }
  float ell = 0.f;
  for (int w = 0; w < NW; ++w) ell += W[w];
  return ell;
}

SANTA_API void santa_or_tile_stats_vec(const float *scores, int H, int L, int block_n, int is_bf16,
                                       float *m_tiles, float *ell_tiles, uint16_t *u16) {
  const int T_c = (L + block_n - 1) / block_n;
  const int NW = (block_n == 256) ? 8 : 4;
  float *u = (float *)malloc(sizeof(float) * (size_t)block_n);
  for (int h = 0; h < H; ++h)
    for (int t = 0; t < T_c; ++t) {
      const int n0 = t * block_n;
      const int tile_len = (n0 + block_n <= L) ? block_n : (L - n0);
      const float *s = scores + (size_t)h * L + n0;
      float m = -INFINITY;
      for (int r = 0; r < tile_len; ++r) m = fmaxf(m, s[r]);
      for (int r = 0; r < tile_len; ++r) {
        u[r] = expf_model(s[r] - m);
        u16[(size_t)h * L + n0 + r] = store16(u[r], is_bf16);
      }
      m_tiles[(size_t)h * T_c + t] = m;
      ell_tiles[(size_t)h * T_c + t] = ell_reference_order(u, tile_len, NW);
    }
  free(u);
}

/* P.cu:190-265 -- tile statistics of the tensor-core path: each warp owns 16
 * consecutive rows; lane r sums its 16 u values in order; warps are summed
 * w = 0..block_n/16-1. */
SANTA_API void santa_or_tile_stats_mma(const float *scores, int H, int L, int block_n, int is_bf16,
                                       float *m_tiles, float *ell_tiles, uint16_t *u16) {
  const int T_c = (L + block_n - 1) / block_n;
  for (int h = 0; h < H; ++h)
    for (int t = 0; t < T_c; ++t) {
      const int n0 = t * block_n;
      const int tile_len = (n0 + block_n <= L) ? block_n : (L - n0);
      const float *s = scores + (size_t)h * L + n0;
      float m = -INFINITY;
      for (int r = 0; r < tile_len; ++r) m = fmaxf(m, s[r]);
      float ell = 0.f;
      for (int w0 = 0; w0 < block_n; w0 += 16) {
        float part = 0.f;
        for (int r = w0; r < w0 + 16 && r < tile_len; ++r) {
          float u = expf_model(s[r] - m);
          part += u;
          u16[(size_t)h * L + n0 + r] = store16(u, is_bf16);
        }
        ell += part;
      }
      m_tiles[(size_t)h * T_c + t] = m;
      ell_tiles[(size_t)h * T_c + t] = ell;
    }
}

/* ------------------------------------------------------------------ */
/* Systematic counts                                                   */
/* ------------------------------------------------------------------ */

/* F.cu:275-311 == P.cu:777-807 -- one warp walks the tile in 32-row chunks.
 * x = u16*invdel; inclusive Hillis-Steele scan (offsets 1,2,4,8,16), exclusive
 * prefix pre = scan - x, carried chunk total, and
 *   c = clamp(int(floorf(a0 + carry + pre + x) - floorf(a0 + carry + pre)), 0, 32767). */
static void systematic_counts_tile(const uint16_t *u16, int is_bf16, int tile_len, float invdel,
                                   float a0, int16_t *c_out) {
  float carry = 0.f;
  for (int base = 0; base < tile_len; base += 32) {
    float x[32], res[32], nxt[32];
    for (int lane = 0; lane < 32; ++lane) {
      const int r = base + lane;
      x[lane] = (r < tile_len && invdel > 0.f) ? load16(u16 + r, is_bf16) * invdel : 0.f;
      res[lane] = x[lane];
    }
    for (int off = 1; off < 32; off <<= 1) {
      for (int lane = 0; lane < 32; ++lane)
        nxt[lane] = (lane >= off) ? (res[lane] + res[lane - off]) : res[lane];
      memcpy(res, nxt, sizeof(res));
    }
    const int remain = tile_len - base;
    const int last_lane = remain > 32 ? 31 : remain - 1;
    for (int lane = 0; lane < 32; ++lane) {
      const int r = base + lane;
      if (r >= tile_len) break;
      const float pre = res[lane] - x[lane];
      const float pre_g = carry + pre;
      const float cum_g = pre_g + x[lane];
      const float f_prev = floorf(a0 + pre_g);
      const float f_curr = floorf(a0 + cum_g);
      int c = (int)(f_curr - f_prev);
      if (c < 0) c = 0;
      if (c > 32767) c = 32767;
      c_out[r] = (int16_t)c;
    }
    /* chunk_total = (pre + x) at the last valid lane */
    const float chunk_total = (res[last_lane] - x[last_lane]) + x[last_lane];
    carry += chunk_total;
  }
}

/* Flash counts for one sequence.  F.cu:275-311 with
 *   invdel = (S_per_tile > 0 && ell > 1e-20) ? S_per_tile / ell : 0   (F.cu:279-280)
 *   a0     = u01(seed, b*H + h, t)                                   (F.cu:281)
 * u16:[H,L]; ell_tiles:[H,T_c]; counts:[H,L].
 * `rng_head0` is b*H (the head index of head 0 in the RNG key) and
 * `tile0` the global index of tile 0 (0 for an unsharded call).
 * invdel_inject:[H,T_c] replaces the division when not NULL (the GPU divides
 * with div.approx under --use_fast_math). */
SANTA_API void santa_or_flash_counts(const uint16_t *u16, const float *ell_tiles, int is_bf16,
                                     int H, int L, int block_n, int S_per_tile, uint64_t seed,
                                     int rng_head0, int tile0, const float *invdel_inject,
                                     int16_t *counts, float *a0_out, float *invdel_out) {
  const int T_c = (L + block_n - 1) / block_n;
  for (int h = 0; h < H; ++h)
    for (int t = 0; t < T_c; ++t) {
      const int n0 = t * block_n;
      const int tile_len = (n0 + block_n <= L) ? block_n : (L - n0);
      const float ell = ell_tiles[(size_t)h * T_c + t];
      float invdel = (S_per_tile > 0 && ell > 1e-20f) ? ((float)S_per_tile / ell) : 0.f;
      if (invdel_inject) invdel = invdel_inject[(size_t)h * T_c + t];
      const float a0 = santa_or_u01(seed, rng_head0 + h, tile0 + t);
      if (a0_out) a0_out[(size_t)h * T_c + t] = a0;
      if (invdel_out) invdel_out[(size_t)h * T_c + t] = invdel;
      systematic_counts_tile(u16 + (size_t)h * L + n0, is_bf16, tile_len, invdel, a0,
                             counts + (size_t)h * L + n0);
    }
}

/* Prop counts for one sequence: same walk with per-tile invdelta/a0 tables
 * from the budget step (P.cu:771-808).  Tables are [H,T_c]. */
SANTA_API void santa_or_prop_counts(const uint16_t *u16, int is_bf16, int H, int L, int block_n,
                                    const float *invdelta, const float *a0, int16_t *counts) {
  const int T_c = (L + block_n - 1) / block_n;
  for (int h = 0; h < H; ++h)
    for (int t = 0; t < T_c; ++t) {
      const int n0 = t * block_n;
      const int tile_len = (n0 + block_n <= L) ? block_n : (L - n0);
      systematic_counts_tile(u16 + (size_t)h * L + n0, is_bf16, tile_len,
                             invdelta[(size_t)h * T_c + t], a0[(size_t)h * T_c + t],
                             counts + (size_t)h * L + n0);
    }
}

/* F.cu:314-345 / P.cu:810-838 -- a row is gathered when any head of its
 * kv-group drew it; rows are emitted in ascending order.  rowflag:[KVH,L]
 * (0/1), vrows:[KVH] = number of flagged rows (F.cu:475-508, P.cu:869-899). */
SANTA_API void santa_or_rowflags(const int16_t *counts, int H, int KVH, int L, uint8_t *rowflag,
                                 int *vrows) {
  const int GH = H / KVH;
  for (int kv = 0; kv < KVH; ++kv) {
    int cnt = 0;
    for (int n = 0; n < L; ++n) {
      int sum = 0;
      for (int g = 0; g < GH; ++g) sum += counts[(size_t)(kv * GH + g) * L + n];
      const uint8_t f = sum > 0;
      if (rowflag) rowflag[(size_t)kv * L + n] = f;
      cnt += f;
    }
    vrows[kv] = cnt;
  }
}

/* ------------------------------------------------------------------ */
/* Estimators                                                          */
/* ------------------------------------------------------------------ */

/* Flash: F.cu:347-379 (per-tile sum of c*V, ascending rows, fp32 fma) then
 * F.cu:386-470 (m* = max_t m_t, w_t = __expf(m_t - m*) * ell_t, Z by the
 * 256-thread strided partials + binary tree, out = sum_t w_t*o_t / (Z*S_per_tile)).
 * V16:[L_storage,KVH,128]; counts:[H,L]; out_f32:[H,128]; out16 may be NULL. */
SANTA_API void santa_or_flash_estimate(const int16_t *counts, const uint16_t *V16, int is_bf16,
                                       int H, int KVH, int L, int block_n, int S_per_tile,
                                       const float *m_tiles, const float *ell_tiles,
                                       float *out_f32, uint16_t *out16, float *m_star) {
  const int D = 128;
  const int GH = H / KVH;
  const int T_c = (L + block_n - 1) / block_n;
  float *w = (float *)malloc(sizeof(float) * (size_t)T_c);
  float *ot = (float *)malloc(sizeof(float) * (size_t)T_c * D);
  for (int h = 0; h < H; ++h) {
    const int kv = h / GH;
    for (int t = 0; t < T_c; ++t) {
      float *o = ot + (size_t)t * D;
      for (int d = 0; d < D; ++d) o[d] = 0.f;
      const int n0 = t * block_n;
      const int n1 = (n0 + block_n <= L) ? n0 + block_n : L;
      for (int n = n0; n < n1; ++n) {
        const int c = counts[(size_t)h * L + n];
        if (c == 0) continue;
        const float cf = (float)c;
        const uint16_t *vp = V16 + ((size_t)n * KVH + kv) * D;
        for (int d = 0; d < D; ++d) o[d] = fmaf(cf, load16(vp + d, is_bf16), o[d]);
      }
    }
    float ms = -INFINITY;
    for (int t = 0; t < T_c; ++t) ms = fmaxf(ms, m_tiles[(size_t)h * T_c + t]);
    float red[256];
    for (int i = 0; i < 256; ++i) red[i] = 0.f;
    for (int t = 0; t < T_c; ++t) {
      w[t] = expf_model(m_tiles[(size_t)h * T_c + t] - ms) * ell_tiles[(size_t)h * T_c + t];
      red[t & 255] += w[t];
    }
    for (int s = 128; s > 0; s >>= 1)
      for (int i = 0; i < s; ++i) red[i] += red[i + s];
    const float Z = red[0];
    const float inv_norm = (S_per_tile > 0 && Z > 0.f) ? (1.0f / (Z * (float)S_per_tile)) : 0.f;
    for (int d = 0; d < D; ++d) {
      float num = 0.f;
      for (int t = 0; t < T_c; ++t) num = fmaf(w[t], ot[(size_t)t * D + d], num);
      const float y = num * inv_norm;
      out_f32[(size_t)h * D + d] = y;
      if (out16) out16[(size_t)h * D + d] = store16(y, is_bf16);
    }
    if (m_star) m_star[h] = ms;
  }
  free(w);
  free(ot);
}

/* Prop: P.cu:843-863 (sum of c*V over all tiles; the reference adds tiles in
 * a nondeterministic atomic order -- ascending tile order is used here) and
 * P.cpp:333 / P.cu:976-985 (scale by 1/S, cast). */
SANTA_API void santa_or_prop_estimate(const int16_t *counts, const uint16_t *V16, int is_bf16,
                                      int H, int KVH, int L, int D, int block_n, long S,
                                      float *out_f32, uint16_t *out16) {
  const int GH = H / KVH;
  const int T_c = (L + block_n - 1) / block_n;
  const float scale = (S > 0) ? (1.0f / (float)S) : 0.f;
  float *o = (float *)malloc(sizeof(float) * (size_t)D);
  float *acc = (float *)malloc(sizeof(float) * (size_t)D);
  for (int h = 0; h < H; ++h) {
    const int kv = h / GH;
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    for (int t = 0; t < T_c; ++t) {
      const int n0 = t * block_n;
      const int n1 = (n0 + block_n <= L) ? n0 + block_n : L;
      int any = 0;
      for (int d = 0; d < D; ++d) o[d] = 0.f;
      for (int n = n0; n < n1; ++n) {
        const int c = counts[(size_t)h * L + n];
        if (c == 0) continue;
        any = 1;
        const float cf = (float)c;
        const uint16_t *vp = V16 + ((size_t)n * KVH + kv) * D;
        /* P.cu:854: acc += cf * v (contracted to one fma by the compiler) */
        for (int d = 0; d < D; ++d) o[d] = fmaf(cf, load16(vp + d, is_bf16), o[d]);
      }
      if (any)
        for (int d = 0; d < D; ++d) acc[d] += o[d];
    }
    for (int d = 0; d < D; ++d) {
      const float y = acc[d] * scale;
      out_f32[(size_t)h * D + d] = y;
      if (out16) out16[(size_t)h * D + d] = store16(y, is_bf16);
    }
  }
  free(o);
  free(acc);
}

/* ------------------------------------------------------------------ */
/* Prop tile budgets                                                   */
/* ------------------------------------------------------------------ */

/* P.cu:577-726 -- per head: m* = max_t m_t; W_t = __expf(m_t - m*) * ell_t;
 * Z = sum W_t; q_t = S * (W_t / Z); base = floor(q_t); the S - sum(base)
 * leftover samples go to the tiles with the largest frac_t = q_t - base +
 * 1e-7*u01(seed,h,t), ranked by the same bitonic network (descending, padded
 * to a power of two with -inf/-1); invdelta_t = S_t/ell_t; a0_t = u01(seed,h,t).
 *
 * Z order.  The reference adds 128 per-thread partial sums (thread i owns
 * tiles t = i, i+128, ...) into shared memory with atomicAdd, whose order is
 * not defined.  The canonical order used here -- and by the CUDA path -- is
 * thread 0, 1, ..., 127.
 * flags bit0: frac = fma(1e-7, u01, q - base) instead of mul-then-add.
 * flags bit1: per-thread partial z += fma(e, ell, z) instead of mul-then-add.
 * (whether the reference binary contracts these is a compiler decision; the
 * tests pin the choice that matches the reference build.)
 * W_inject:[H,T_c] replaces the modelled W_t when not NULL. */
SANTA_API void santa_or_prop_budgets(const float *m_tiles, const float *ell_tiles, int H, int T_c,
                                     long S_in, uint64_t seed, int flags, const float *W_inject,
                                     float *m_star, int *S_tiles, float *invdelta, float *a0,
                                     float *W_out) {
  const int S = (int)S_in;
  int N = 1;
  while (N < T_c) N <<= 1;
  float *frac = (float *)malloc(sizeof(float) * (size_t)N);
  int *idx = (int *)malloc(sizeof(int) * (size_t)N);
  float *W = (float *)malloc(sizeof(float) * (size_t)T_c);
  for (int h = 0; h < H; ++h) {
    const float *mt = m_tiles + (size_t)h * T_c;
    const float *el = ell_tiles + (size_t)h * T_c;
    float ms = -3.402823466e+38f; /* -FLT_MAX, P.cu:600 */
    for (int t = 0; t < T_c; ++t) ms = fmaxf(ms, mt[t]);
    if (m_star) m_star[h] = ms;

    float zl[128];
    for (int i = 0; i < 128; ++i) zl[i] = 0.f;
    for (int t = 0; t < T_c; ++t) {
      float e = expf_model(mt[t] - ms);
      W[t] = W_inject ? W_inject[(size_t)h * T_c + t] : e * el[t];
      if ((flags & 2) && !W_inject)
        zl[t & 127] = fmaf(e, el[t], zl[t & 127]);
      else
        zl[t & 127] += W[t];
      if (W_out) W_out[(size_t)h * T_c + t] = W[t];
    }
    float Z = 0.f;
    for (int i = 0; i < 128; ++i) Z += zl[i];

    if (S <= 0 || !(Z > 0.f)) {
      for (int t = 0; t < T_c; ++t) {
        S_tiles[(size_t)h * T_c + t] = 0;
        invdelta[(size_t)h * T_c + t] = 0.f;
        a0[(size_t)h * T_c + t] = santa_or_u01(seed, h, t);
      }
      continue;
    }

    int sum_base = 0;
    for (int t = 0; t < T_c; ++t) {
      const float q = (float)S * (W[t] / Z);
      const int b = (int)floorf(q);
      S_tiles[(size_t)h * T_c + t] = b;
      sum_base += b;
      const float ft = q - (float)b;
      const float u = santa_or_u01(seed, h, t);
      frac[t] = (flags & 1) ? fmaf(1.0e-7f, u, ft) : (ft + 1.0e-7f * u);
      idx[t] = t;
    }
    for (int t = T_c; t < N; ++t) {
      frac[t] = -INFINITY;
      idx[t] = -1;
    }
    int rem = S - sum_base;
    if (rem < 0) rem = 0;
    if (rem > T_c) rem = T_c;

    /* bitonic network, final order descending (P.cu:686-707).  Positions
     * >= T_c are virtual: they read as (-inf, -1) and are never stored.  When
     * T_c is not a power of two an ascending sub-block can push a real entry
     * into a virtual slot, where it is dropped and a (-inf, -1) takes its
     * place; such a tile can then never receive a leftover sample and the
     * budgets may sum to less than S.  That is the reference's behaviour and
     * is reproduced on purpose (same loads, same stores, same comparison). */
    for (int k = 2; k <= N; k <<= 1)
      for (int j = k >> 1; j > 0; j >>= 1)
        for (int i = 0; i < N; ++i) {
          const int ixj = i ^ j;
          if (ixj <= i) continue;
          const int up = (i & k) != 0;
          float ai = (i < T_c) ? frac[i] : -INFINITY;
          float aj = (ixj < T_c) ? frac[ixj] : -INFINITY;
          int ii = (i < T_c) ? idx[i] : -1;
          int ij = (ixj < T_c) ? idx[ixj] : -1;
          if ((ai > aj) == up) {
            float tf = ai; ai = aj; aj = tf;
            int ti = ii; ii = ij; ij = ti;
          }
          if (i < T_c) { frac[i] = ai; idx[i] = ii; }
          if (ixj < T_c) { frac[ixj] = aj; idx[ixj] = ij; }
        }
    for (int r = 0; r < rem; ++r)
      if (idx[r] >= 0) S_tiles[(size_t)h * T_c + idx[r]] += 1;

    for (int t = 0; t < T_c; ++t) {
      const int St = S_tiles[(size_t)h * T_c + t];
      invdelta[(size_t)h * T_c + t] = (St > 0 && el[t] > 1e-20f) ? ((float)St / el[t]) : 0.f;
      a0[(size_t)h * T_c + t] = santa_or_u01(seed, h, t);
    }
  }
  free(frac);
  free(idx);
  free(W);
}

/* ------------------------------------------------------------------ */
/* Split-KV merge (used for the sequence-sharded decode)               */
/* ------------------------------------------------------------------ */

/* Merge G partial results of the Flash estimator.  Partial r carries, per
 * head, m_r (max score of its tiles), Z_r = sum_t exp(m_t - m_r)*ell_t and
 * A_r[d] = sum_t exp(m_t - m_r)*ell_t*o_t[d].  The merged estimator is
 * algebraically F.cu:386-470 over the union of the tiles:
 *   m* = max_r m_r;  out = sum_r e^{m_r-m*} A_r / (S_per_tile * sum_r e^{m_r-m*} Z_r).
 * part layout: [G][H][D+2] with A at [0,D), m at D, Z at D+1. */
SANTA_API void santa_or_merge_partials(const float *part, int G, int H, int D, int S_per_tile,
                                       float *out_f32, float *m_star) {
  const int W = D + 2;
  for (int h = 0; h < H; ++h) {
    float ms = -INFINITY;
    for (int r = 0; r < G; ++r) ms = fmaxf(ms, part[((size_t)r * H + h) * W + D]);
    double Z = 0.0;
    for (int r = 0; r < G; ++r) {
      const float *p = part + ((size_t)r * H + h) * W;
      Z += (double)p[D + 1] * exp((double)p[D] - (double)ms);
    }
    for (int d = 0; d < D; ++d) {
      double num = 0.0;
      for (int r = 0; r < G; ++r) {
        const float *p = part + ((size_t)r * H + h) * W;
        num += (double)p[d] * exp((double)p[D] - (double)ms);
      }
      out_f32[(size_t)h * D + d] =
          (S_per_tile > 0 && Z > 0.0) ? (float)(num / (Z * (double)S_per_tile)) : 0.f;
    }
    if (m_star) m_star[h] = ms;
  }
}
