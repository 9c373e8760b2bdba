// common.cuh -- device helpers shared by the Flash and Prop translation units.
//
// Everything here is header-only so that each translation unit compiles it
// under its own floating-point flags: the Flash unit is built with
// --use_fast_math (approximate division, flush-to-zero) and the Prop unit
// without, exactly as the reference builds its two extensions
// (flash_style_fused_santa_fixed_tile_budgets/setup.py:15-20,
//  santa_fused_proportional_tile_budgets/setup.py:39-42).  Sampled row counts
// are only reproducible bit-for-bit when those flags agree.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstdint>

namespace santa {

constexpr int kD = 128;             // head_dim of the vectorised kernels
constexpr int kGH = 4;              // query heads per kv-head of the vectorised kernels
constexpr int kRowBytes = kD * 2;   // one K/V row of one kv-head
constexpr int kChunkRows = 32;      // rows per sampler chunk (one row per lane, as in the reference scan)
constexpr int kStageRows = 32;      // rows staged per pipeline slot
constexpr int kStageBytes = kStageRows * kRowBytes;
constexpr int kGroupWarps = 8;      // one warp per kv-head column of a column group
constexpr int kMaxCtas = 256;       // upper bound on persistent CTAs (>= SM count)
constexpr int kPartialStride = 132; // floats per (slot, warp, head): A[128], m, Z, pad
constexpr uint32_t kSpinLimit = 1u << 22;  // polls; with the sleep between polls this is seconds

// status word values (0 = ok)
enum : int {
  kStatusOk = 0,
  kStatusStageTimeout = 1,    // a staged K piece never arrived
  kStatusHandoffTimeout = 2,  // a score buffer was never handed over between the warps of a column
  kStatusBadPosition = 3,     // an append position outside the cache was skipped
  kStatusPeerTimeout = 4,     // a rank's partial never arrived in the exchange buffer
  kStatusBadIndex = 5,        // checked build only: an index left its array; the access was skipped
};

// Checked build (-DSANTA_B200_CHECKS, `python -m santa_b200._build --checks`): every index that
// depends on data or on the work split is compared with the extent of its array before the access.
// A failed check writes kStatusBadIndex to the status word and the access is skipped -- nothing
// traps, the context stays usable, and the host reads the word as after any call.  In the normal
// build the macro is the constant `true` and the checks cost nothing.  (Stands in for a memory
// checker where none can be run; same idea as the reference's SANTA_DEBUG asserts,
// santa_fused_proportional_tile_budgets/santa_cuda_kernel.cu:24-38, without the trap.)
#ifdef SANTA_B200_CHECKS
#define SANTA_IN_RANGE(idx, extent, status_ptr)                                         \
  (((unsigned long long)(idx) < (unsigned long long)(extent))                           \
       ? true                                                                           \
       : (((status_ptr) != nullptr ? (void)atomicExch((status_ptr), kStatusBadIndex) : (void)0), false))
#else
#define SANTA_IN_RANGE(idx, extent, status_ptr) (true)
#endif

// ---------------------------------------------------------------- RNG
// splitmix64 finaliser over seed ^ (h << 32 ^ t); top 53 bits -> [0,1] double
// -> float.  Restates flash_style_fused_santa_fixed_tile_budgets/
// santa_cuda_kernel.cu:74-87 (same function at
// santa_fused_proportional_tile_budgets/santa_cuda_kernel.cu:557-570).
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t x) {
  uint64_t z = x + 0x9e3779b97f4a7c15ULL;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
  return z ^ (z >> 31);
}
__host__ __device__ __forceinline__ float u01_from_seed(uint64_t seed, int h, int t) {
  const uint64_t key = seed ^ ((uint64_t(int64_t(h)) << 32) ^ uint64_t(int64_t(t)));
  const uint64_t r = mix64(key);
  const double u = double(r >> 11) * (1.0 / 9007199254740992.0);
  return float(u);
}

// ---------------------------------------------------------------- 16-bit storage
template <typename TK>
struct Store16;

template <>
struct Store16<__nv_bfloat16> {
  // two packed values -> two floats (element 0 in the low half)
  static __device__ __forceinline__ float2 unpack(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
  // round to storage precision, return as float
  static __device__ __forceinline__ float round(float x) {
    return __bfloat162float(__float2bfloat16(x));
  }
  static __device__ __forceinline__ uint16_t bits(float x) {
    return __bfloat16_as_ushort(__float2bfloat16(x));
  }
};

template <>
struct Store16<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ uint16_t bits(float x) {
    return __half_as_ushort(__float2half_rn(x));
  }
};

// ---------------------------------------------------------------- tensor-core step
// One m16n8k16 step, fp32 accumulate, 16-bit operands of the storage type.
template <typename TK>
struct MmaOp;
template <>
struct MmaOp<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};
template <>
struct MmaOp<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};

// ---------------------------------------------------------------- async staging
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the phase did not complete within the limit.
// Between polls the warp sleeps `backoff_ns`, so that a waiting warp does not
// take issue slots from the warps it is waiting for.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t backoff_ns = 32) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(backoff_ns);
  }
  return false;
}
// One bulk asynchronous copy global -> shared, completion counted on `bar`.
// Source, destination and size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// One tiled TMA load of a 4-D box (coordinates innermost first) global -> shared.
// `tmap` must live in kernel-parameter, constant or global memory.  The
// innermost coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], "
      "[%6];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// ---------------------------------------------------------------- cross-device combine
// int32 control words at the start of a rank's exchange buffer (after the arrival counters)
constexpr int kPeerDoneIndex = 32;    // rows finished by the receiving side in this step
constexpr int kPeerStepIndex = 33;    // steps completed so far (device-counted epochs)
constexpr int kPeerStatusIndex = 34;  // 4 once a wait on this buffer ran out

// Folds n raw Flash partials of one (sequence, head) row -- A[128], m, Z each, `stride` floats apart,
// produced for disjoint tile sets -- in index order and writes the normalised row: the reference's
// finalize (flash_style_fused_santa_fixed_tile_budgets/santa_cuda_kernel.cu:386-470) over the union
// of the tiles,
//   m* = max_r m_r,  out = sum_r e^{m_r-m*} A_r / (S_per_tile * sum_r e^{m_r-m*} Z_r).
// One warp per row, lane l owns dims 4l..4l+3.  Every operation is spelled out, so that all
// translation units (whatever their floating-point flags) produce the same bits.
template <typename TK>
__device__ __forceinline__ void combine_rows(const float* rows, size_t stride, int n, int S_per_tile, int lane,
                                             TK* out_row, float* m_star_row) {
  constexpr int W = kD + 2;
  (void)W;
  float ms = -CUDART_INF_F;
  for (int r = 0; r < n; ++r) ms = fmaxf(ms, __ldcg(rows + size_t(r) * stride + kD));
  float zs = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = 0; r < n; ++r) {
    const float* p = rows + size_t(r) * stride;
    const float e = __expf(__fsub_rn(__ldcg(p + kD), ms));
    zs = __fmaf_rn(e, __ldcg(p + kD + 1), zs);
    const float2 a01 = __ldcg(reinterpret_cast<const float2*>(p) + 2 * lane);
    const float2 a23 = __ldcg(reinterpret_cast<const float2*>(p) + 2 * lane + 1);
    acc.x = __fmaf_rn(e, a01.x, acc.x);
    acc.y = __fmaf_rn(e, a01.y, acc.y);
    acc.z = __fmaf_rn(e, a23.x, acc.z);
    acc.w = __fmaf_rn(e, a23.y, acc.w);
  }
  const float inv = (S_per_tile > 0 && zs > 0.f) ? __frcp_rn(__fmul_rn(zs, (float)S_per_tile)) : 0.f;
  uint2 wv;
  wv.x = uint32_t(Store16<TK>::bits(__fmul_rn(acc.x, inv))) | (uint32_t(Store16<TK>::bits(__fmul_rn(acc.y, inv))) << 16);
  wv.y = uint32_t(Store16<TK>::bits(__fmul_rn(acc.z, inv))) | (uint32_t(Store16<TK>::bits(__fmul_rn(acc.w, inv))) << 16);
  *reinterpret_cast<uint2*>(out_row + 4 * lane) = wv;
  if (lane == 0 && m_star_row != nullptr) *m_star_row = ms;
}

// Bounded wait of lanes 0..world-1 on one int32 word each (lane r: `word_of_lane`) until it holds
// `want` or -- counters -- has passed it; system-scope acquire loads, sleeping between polls.
// The bound is one second of the GPU's nanosecond timer (and a poll count, should the timer stand
// still).  Returns true on every lane when all arrived within the bound.
constexpr unsigned long long kPeerWaitNs = 1000000000ull;
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool peer_wait(const int* word_of_lane, bool polls, unsigned want, bool counter) {
  bool ok = true;
  if (polls) {
    ok = false;
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(word_of_lane) : "memory");
      if (counter ? (int(unsigned(v) - want) >= 0) : (unsigned(v) == want)) {
        ok = true;
        break;
      }
      if ((spin & 63u) == 63u && global_timer_ns() - t0 > kPeerWaitNs) break;
      __nanosleep(200);
    }
  }
  return __all_sync(0xffffffffu, ok);
}

// The last row of a step to finish on the receiving side puts the row counter back to zero and
// advances the buffer's step counter; rows whose wait ran out count too, so that the counters never
// stay half-way and this rank stays in step with the others.
__device__ __forceinline__ void peer_step_done(int* ctl, int rows_per_step) {
  __threadfence();
  if (atomicAdd(ctl + kPeerDoneIndex, 1) == rows_per_step - 1) {
    ctl[kPeerDoneIndex] = 0;
    __threadfence();
    atomicAdd(ctl + kPeerStepIndex, 1);
  }
}

// ---------------------------------------------------------------- work split
// `items` work items are dealt to `ctas` CTAs in contiguous, balanced ranges:
// CTA i owns [lo(i), lo(i+1)) with lo(i) = floor(i*items/ctas).
__host__ __device__ __forceinline__ long long range_lo(long long i, long long items, long long ctas) {
  return (i * items) / ctas;
}
// the CTA whose range contains item x: the largest i with lo(i) <= x
__host__ __device__ __forceinline__ int cta_of_item(long long x, long long items, long long ctas) {
  return int(((x + 1) * ctas - 1) / items);
}

// ---------------------------------------------------------------- ragged batches
// A ragged batch gives every sequence its own length through a device array.  Work items are
// ordered (sequence, column group, tile); `start[b]` is the first item of sequence b and
// start[nseq] the item total.  Lengths are clamped to [0, max_len], so that a bad entry can
// neither index outside the cache nor change the item arithmetic between kernels.
constexpr int kMaxRaggedSeqs = 1024;

__device__ __forceinline__ int ragged_len(const int* __restrict__ seq_lens, int b, int max_len) {
  const int n = __ldg(seq_lens + b);
  return n < 0 ? 0 : (n > max_len ? max_len : n);
}

// Built by one full warp; `start` has nseq + 1 entries in shared memory.
__device__ __forceinline__ void build_item_starts(const int* __restrict__ seq_lens, int nseq, int max_len, int bn,
                                                  int groups_per_seq, int* start, int lane) {
  int carry = 0;
  for (int base = 0; base < nseq; base += 32) {
    const int b = base + lane;
    int n = 0;
    if (b < nseq) n = ((ragged_len(seq_lens, b, max_len) + bn - 1) / bn) * groups_per_seq;
    int incl = n;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (b < nseq) start[b] = carry + incl - n;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) start[nseq] = carry;
}

// ---------------------------------------------------------------- weighted split (Prop, second pass)
// A (kv-head, tile) unit of Prop's second pass costs more in a short sequence than in a long one: the
// budget S is spread over fewer tiles, so every tile holds more samples (more rows to gather, no head
// without a budget).  Measured on uniform batches at S = 256, per unit and warp with all warps busy:
// 11.4 / 8.0 / 6.3 / 5.5 us at 32 / 64 / 128 / 256 tiles, i.e. about 4.9 + 0.8 * S / T.  A ragged
// batch is therefore cut into ranges of equal WEIGHT, not of equal item count: every item of a
// sequence of T tiles weighs prop_unit_weight(T, S), item k of sequence b starts at weight
// wstart[b] + k * w_b, and range i owns the items whose start lies in [lo(i), lo(i + 1)) with
// lo(i) = floor(i * W / ranges) -- range_lo / cta_of_item in weight space.  With no more than
// W / max_b(w_b) ranges every range holds at least one item.
__host__ __device__ __forceinline__ int prop_unit_weight(int T, long long S) {
  if (T <= 0) return 49;
  long long r = S > 0 ? (8 * S + T / 2) / T : 0;
  if (r > 512) r = 512;
  return int(49 + r);
}

// Built by one full warp: wstart[b] = weight before sequence b (nseq + 1 entries); returns the largest
// weight of a sequence that has items (0 if none has).
__device__ __forceinline__ int build_weight_starts(const int* __restrict__ seq_lens, int nseq, int max_len, int bn,
                                                   int groups_per_seq, long long S, long long* wstart, int lane) {
  long long carry = 0;
  int wmax = 0;
  for (int base = 0; base < nseq; base += 32) {
    const int b = base + lane;
    long long n = 0;
    if (b < nseq) {
      const int T = (ragged_len(seq_lens, b, max_len) + bn - 1) / bn;
      const int w = prop_unit_weight(T, S);
      n = (long long)T * groups_per_seq * w;
      if (T > 0) wmax = wmax > w ? wmax : w;
    }
    long long incl = n;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const long long t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (b < nseq) wstart[b] = carry + incl - n;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) wstart[nseq] = carry;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const int o = __shfl_xor_sync(0xffffffffu, wmax, off);
    wmax = wmax > o ? wmax : o;
  }
  return wmax;
}

// The first item whose weight start is >= wpos (0 <= wpos <= wstart[nseq]); `start` / `wstart` are the
// item and weight prefixes over the sequences, each of which has groups_per_seq items per tile.
__host__ __device__ __forceinline__ long long item_at_weight(const int* start, const long long* wstart, int nseq,
                                                             long long wpos, int groups_per_seq, long long S) {
  int lo = 0, hi = nseq;  // the largest b < nseq with wstart[b] <= wpos
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (wstart[mid] <= wpos)
      lo = mid;
    else
      hi = mid;
  }
  const int n_b = start[lo + 1] - start[lo];
  const int w = prop_unit_weight(n_b / groups_per_seq, S);
  long long k = (wpos - wstart[lo] + w - 1) / w;
  if (k > n_b) k = n_b;
  return (long long)start[lo] + k;
}

// The sequence owning item `it` (0 <= it < start[nseq]): the largest b with start[b] <= it.
__device__ __forceinline__ int seq_of_item(const int* start, int nseq, int it) {
  int lo = 0, hi = nseq;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (start[mid] <= it)
      lo = mid;
    else
      hi = mid;
  }
  return lo;
}
}  // namespace santa
