// sampler.cuh -- per-tile sampling steps executed by one warp on a tile whose
// four heads' scores (or tile-local weights) sit in shared memory as one float4
// per row: tile statistics, systematic counts with row compaction, and the
// sparse sum of V rows.  Shared by the Flash kernel, Prop's first pass (tile
// statistics) and Prop's second pass (counts and V).  Every step follows the
// reference's floating-point order so that the sampled counts are identical.
#pragma once

#include "common.cuh"
#include "santa_abi_internal.h"

namespace santa {

// Tile statistics, flash_style_fused_santa_fixed_tile_budgets/santa_cuda_kernel.cu:223-273
// (== santa_fused_proportional_tile_budgets/santa_cuda_kernel.cu:381-440).
// In: sb[r] = scores of row r (4 heads).  Out: sb[r] = u = __expf(s - m) in fp32
// (0 on rows >= tile_len of a started 32-row chunk), m[g] = max score,
// ell[g] = sum of u in the reference's order: thread-strided partials (chunk
// parity selects the 32-row half when the reference block has 8 warps), an
// 8-row tree per reference warp, reference warps added in order.
template <int NW>
__device__ __forceinline__ void tile_stats(float4* sb, int tile_len, int lane, float (&m)[kGH], float (&ell)[kGH]) {
  constexpr int NH = NW / 4;
  const int nch = (tile_len + kChunkRows - 1) / kChunkRows;
#pragma unroll
  for (int g = 0; g < kGH; ++g) m[g] = -CUDART_INF_F;
#pragma unroll 4
  for (int ch = 0; ch < nch; ++ch) {
    if (ch * kChunkRows + lane < tile_len) {
      const float4 s = sb[ch * kChunkRows + lane];
      m[0] = fmaxf(m[0], s.x);
      m[1] = fmaxf(m[1], s.y);
      m[2] = fmaxf(m[2], s.z);
      m[3] = fmaxf(m[3], s.w);
    }
  }
  // shuffles of the four heads are issued back to back so that their latencies overlap
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    float o[kGH];
#pragma unroll
    for (int g = 0; g < kGH; ++g) o[g] = __shfl_xor_sync(0xffffffffu, m[g], off);
#pragma unroll
    for (int g = 0; g < kGH; ++g) m[g] = fmaxf(m[g], o[g]);
  }

  float V0[kGH], V1[kGH];
#pragma unroll
  for (int g = 0; g < kGH; ++g) V0[g] = V1[g] = 0.f;
#pragma unroll 2
  for (int ch = 0; ch < nch; ++ch) {
    const bool valid = ch * kChunkRows + lane < tile_len;
    float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid) {
      const float4 s = sb[ch * kChunkRows + lane];
      u.x = __expf(s.x - m[0]);
      u.y = __expf(s.y - m[1]);
      u.z = __expf(s.z - m[2]);
      u.w = __expf(s.w - m[3]);
    }
    sb[ch * kChunkRows + lane] = u;
    if (NH == 2 && (ch & 1)) {
      V1[0] = __fadd_rn(V1[0], u.x);
      V1[1] = __fadd_rn(V1[1], u.y);
      V1[2] = __fadd_rn(V1[2], u.z);
      V1[3] = __fadd_rn(V1[3], u.w);
    } else {
      V0[0] = __fadd_rn(V0[0], u.x);
      V0[1] = __fadd_rn(V0[1], u.y);
      V0[2] = __fadd_rn(V0[2], u.z);
      V0[3] = __fadd_rn(V0[3], u.w);
    }
  }
  // per-head value order (reference): 8-row tree (xor 4,2,1), then the reference warps in order
  // (lane groups 0,8,16,24 of the even half, then of the odd half when the block has 8 warps).
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) {
    float o0[kGH], o1[kGH];
#pragma unroll
    for (int g = 0; g < kGH; ++g) {
      o0[g] = __shfl_xor_sync(0xffffffffu, V0[g], off);
      if (NH == 2) o1[g] = __shfl_xor_sync(0xffffffffu, V1[g], off);
    }
#pragma unroll
    for (int g = 0; g < kGH; ++g) {
      V0[g] = __fadd_rn(V0[g], o0[g]);
      if (NH == 2) V1[g] = __fadd_rn(V1[g], o1[g]);
    }
  }
  float w[2 * 4][kGH];
#pragma unroll
  for (int k = 0; k < 4; ++k)
#pragma unroll
    for (int g = 0; g < kGH; ++g) {
      w[k][g] = __shfl_sync(0xffffffffu, V0[g], 8 * k);
      if (NH == 2) w[4 + k][g] = __shfl_sync(0xffffffffu, V1[g], 8 * k);
    }
#pragma unroll
  for (int g = 0; g < kGH; ++g) {
    float e = w[0][g];
#pragma unroll
    for (int k = 1; k < 4 * NH; ++k) e = __fadd_rn(e, w[k][g]);
    ell[g] = e;
  }
}

// Optional per-row trace targets of tile_counts (all may be null).
struct RowTrace {
  uint16_t* u16;    // storage bits of u for head g at u16[g * head_stride + row]; needs counts too
  int16_t* counts;  // same indexing
  int* rowmask;     // + row index
  size_t head_stride;
  int* status;      // the call's status word (checked build)
  int rows_left;    // rows of the V tensor from the tile's first row to the end of its sequence's storage
  // V row of the tile's first row for this kv-head and the bytes between rows (or null): a row is
  // prefetched into L2 the moment the counts show it is sampled, so that the gather after the last
  // chunk finds it there instead of waiting a DRAM round trip
  const unsigned char* vrow0;
  size_t row_stride;
};

__device__ __forceinline__ void prefetch_row_l2(const unsigned char* row) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(row));
  asm volatile("prefetch.global.L2 [%0];" ::"l"(row + 128));
}

// Systematic counts and row compaction of one tile,
// flash_style_fused_santa_fixed_tile_budgets/santa_cuda_kernel.cu:275-345
// (== santa_fused_proportional_tile_budgets/santa_cuda_kernel.cu:771-838).
// In: sb[r] = u (fp32, or already rounded to the storage type), invdel[g], a0[g].
// Out: the emit list overwrites sb in place -- entry i (16 bytes: four 16-bit
// counts, row index within the tile) describes the i-th gathered row in
// ascending row order and lands on row i, which has been consumed by then.
// Returns the number of gathered rows.
// ROUNDED: sb already holds values of the storage type (Prop's second pass reads them from the
// stash), so the rounding step is skipped.
// TWO: two chunks per iteration (more instruction-level parallelism, more registers) or one.
template <typename TK, bool ROUNDED = false, bool TWO = true>
__device__ __forceinline__ int tile_counts(float4* sb, int tile_len, int lane, const float (&invdel)[kGH],
                                           const float (&a0)[kGH], const RowTrace& tr) {
  const int nch = (tile_len + kChunkRows - 1) / kChunkRows;
  float carry[kGH];
#pragma unroll
  for (int g = 0; g < kGH; ++g) carry[g] = 0.f;
  int n_emit = 0;
  uint4* emit = reinterpret_cast<uint4*>(sb);
  // Two chunks (A = ch, B = ch+1) per iteration: their scans are independent, so the shuffles of
  // the eight (chunk, head) chains are issued back to back and their latencies overlap.  Only the
  // final additions of B need A's chunk total (the carried prefix).
#pragma unroll 1
  for (int ch = 0; ch < nch; ch += (TWO ? 2 : 1)) {
    const int remainA = tile_len - ch * kChunkRows;
    const int remainB = remainA - kChunkRows;  // <= 0 when chunk B does not exist
    const bool hasB = TWO && remainB > 0;
    const int lastA = remainA > 32 ? 31 : remainA - 1;
    const int lastB = remainB > 32 ? 31 : (hasB ? remainB - 1 : 0);
    const bool validA = lane < remainA;
    const bool validB = TWO && lane < remainB;
    const float4 uA4 = sb[ch * kChunkRows + lane];
    const float4 uB4 = hasB ? sb[(ch + 1) * kChunkRows + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float uA[kGH] = {uA4.x, uA4.y, uA4.z, uA4.w};
    const float uB[kGH] = {uB4.x, uB4.y, uB4.z, uB4.w};
    float xA[kGH], xB[kGH], rA[kGH], rB[kGH];
#pragma unroll
    for (int g = 0; g < kGH; ++g) {
      const float ruA = ROUNDED ? uA[g] : Store16<TK>::round(uA[g]);
      const float ruB = ROUNDED ? uB[g] : Store16<TK>::round(uB[g]);
      xA[g] = (validA && invdel[g] > 0.f) ? __fmul_rn(ruA, invdel[g]) : 0.f;
      xB[g] = (validB && invdel[g] > 0.f) ? __fmul_rn(ruB, invdel[g]) : 0.f;
      rA[g] = xA[g];
      rB[g] = xB[g];
    }
    // inclusive Hillis-Steele scans (offsets 1,2,4,8,16)
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      float nA[kGH], nB[kGH];
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        nA[g] = __shfl_up_sync(0xffffffffu, rA[g], off);
        nB[g] = __shfl_up_sync(0xffffffffu, rB[g], off);
      }
      if (lane >= off) {
#pragma unroll
        for (int g = 0; g < kGH; ++g) {
          rA[g] = __fadd_rn(rA[g], nA[g]);
          rB[g] = __fadd_rn(rB[g], nB[g]);
        }
      }
    }
    float preA[kGH], preB[kGH], totA[kGH], totB[kGH];
#pragma unroll
    for (int g = 0; g < kGH; ++g) {
      preA[g] = __fsub_rn(rA[g], xA[g]);
      preB[g] = __fsub_rn(rB[g], xB[g]);
      totA[g] = __shfl_sync(0xffffffffu, __fadd_rn(preA[g], xA[g]), lastA);
      totB[g] = __shfl_sync(0xffffffffu, __fadd_rn(preB[g], xB[g]), lastB);
    }
    int cA[kGH], cB[kGH];
#pragma unroll
    for (int g = 0; g < kGH; ++g) {
      // int(floorf(b) - floorf(a)) == floor-to-int(b) - floor-to-int(a): both floors are exact
      // integers far below 2^24 (they are bounded by the tile budget plus one)
      const float carryB = __fadd_rn(carry[g], totA[g]);
      const float pgA = __fadd_rn(carry[g], preA[g]);
      const float cgA = __fadd_rn(pgA, xA[g]);
      const float pgB = __fadd_rn(carryB, preB[g]);
      const float cgB = __fadd_rn(pgB, xB[g]);
      int a = __float2int_rd(__fadd_rn(a0[g], cgA)) - __float2int_rd(__fadd_rn(a0[g], pgA));
      int b = __float2int_rd(__fadd_rn(a0[g], cgB)) - __float2int_rd(__fadd_rn(a0[g], pgB));
      a = a < 0 ? 0 : (a > 32767 ? 32767 : a);
      b = b < 0 ? 0 : (b > 32767 ? 32767 : b);
      cA[g] = validA ? a : 0;
      cB[g] = validB ? b : 0;
      carry[g] = hasB ? __fadd_rn(carryB, totB[g]) : carryB;
    }
    if (tr.counts != nullptr) {
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        const size_t o = size_t(g) * tr.head_stride + ch * kChunkRows + lane;
        if (validA) {
          if (tr.u16 != nullptr) tr.u16[o] = Store16<TK>::bits(uA[g]);
          tr.counts[o] = (int16_t)cA[g];
        }
        if (validB) {
          if (tr.u16 != nullptr) tr.u16[o + kChunkRows] = Store16<TK>::bits(uB[g]);
          tr.counts[o + kChunkRows] = (int16_t)cB[g];
        }
      }
    }
    // compaction in ascending row order: A's rows, then B's
    const bool flagA = (cA[0] + cA[1] + cA[2] + cA[3]) > 0;
    const bool flagB = (cB[0] + cB[1] + cB[2] + cB[3]) > 0;
    const uint32_t maskA = __ballot_sync(0xffffffffu, flagA);
    const uint32_t maskB = __ballot_sync(0xffffffffu, flagB);
    __syncwarp();
    const uint32_t lt = (1u << lane) - 1u;
    if (flagA && SANTA_IN_RANGE(n_emit + __popc(maskA & lt), kChunkRows * ((tile_len + kChunkRows - 1) / kChunkRows), tr.status)) {
      emit[n_emit + __popc(maskA & lt)] =
          make_uint4((uint32_t)cA[0] | ((uint32_t)cA[1] << 16), (uint32_t)cA[2] | ((uint32_t)cA[3] << 16),
                     (uint32_t)(ch * kChunkRows + lane), 0u);
      if (tr.rowmask != nullptr) tr.rowmask[ch * kChunkRows + lane] = 1;
      if (tr.vrow0 != nullptr) prefetch_row_l2(tr.vrow0 + size_t(ch * kChunkRows + lane) * tr.row_stride);
    }
    if (flagB && SANTA_IN_RANGE(n_emit + __popc(maskA) + __popc(maskB & lt), kChunkRows * ((tile_len + kChunkRows - 1) / kChunkRows), tr.status)) {
      emit[n_emit + __popc(maskA) + __popc(maskB & lt)] =
          make_uint4((uint32_t)cB[0] | ((uint32_t)cB[1] << 16), (uint32_t)cB[2] | ((uint32_t)cB[3] << 16),
                     (uint32_t)((ch + 1) * kChunkRows + lane), 0u);
      if (tr.rowmask != nullptr) tr.rowmask[(ch + 1) * kChunkRows + lane] = 1;
      if (tr.vrow0 != nullptr) prefetch_row_l2(tr.vrow0 + size_t((ch + 1) * kChunkRows + lane) * tr.row_stride);
    }
    n_emit += __popc(maskA) + __popc(maskB);
  }
  __syncwarp();
  return n_emit;
}

// The same for a tile in which only NA < 4 of the heads have a budget (Prop, long contexts: most
// (head, tile) pairs get none).  A head without budget has step 0, so all its counts are zero and its
// scans can be left out entirely: the NA active heads (bits of `active`, ascending) are gathered into
// dense arrays, run through the same arithmetic, and their counts scattered back.  Bit-identical to
// tile_counts on the same input.
__device__ __forceinline__ float pick4(const float4& v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}
template <typename TK, bool ROUNDED, bool TWO, int NA>
__device__ __forceinline__ int tile_counts_some(float4* sb, int tile_len, int lane, const float (&invdel)[kGH],
                                                const float (&a0)[kGH], const RowTrace& tr, uint32_t active) {
  int hs[NA];
  float inv[NA], off0[NA], carry[NA];
  {
    uint32_t m = active;
#pragma unroll
    for (int k = 0; k < NA; ++k) {
      hs[k] = __ffs(m) - 1;
      m &= m - 1u;
      inv[k] = hs[k] == 0 ? invdel[0] : (hs[k] == 1 ? invdel[1] : (hs[k] == 2 ? invdel[2] : invdel[3]));
      off0[k] = hs[k] == 0 ? a0[0] : (hs[k] == 1 ? a0[1] : (hs[k] == 2 ? a0[2] : a0[3]));
      carry[k] = 0.f;
    }
  }
  const int nch = (tile_len + kChunkRows - 1) / kChunkRows;
  int n_emit = 0;
  uint4* emit = reinterpret_cast<uint4*>(sb);
#pragma unroll 1
  for (int ch = 0; ch < nch; ch += (TWO ? 2 : 1)) {
    const int remainA = tile_len - ch * kChunkRows;
    const int remainB = remainA - kChunkRows;
    const bool hasB = TWO && remainB > 0;
    const int lastA = remainA > 32 ? 31 : remainA - 1;
    const int lastB = remainB > 32 ? 31 : (hasB ? remainB - 1 : 0);
    const bool validA = lane < remainA;
    const bool validB = TWO && lane < remainB;
    const float4 uA4 = sb[ch * kChunkRows + lane];
    const float4 uB4 = hasB ? sb[(ch + 1) * kChunkRows + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
    float xA[NA], xB[NA], rA[NA], rB[NA];
#pragma unroll
    for (int k = 0; k < NA; ++k) {
      const float uA = pick4(uA4, hs[k]), uB = pick4(uB4, hs[k]);
      const float ruA = ROUNDED ? uA : Store16<TK>::round(uA);
      const float ruB = ROUNDED ? uB : Store16<TK>::round(uB);
      xA[k] = validA ? __fmul_rn(ruA, inv[k]) : 0.f;
      xB[k] = validB ? __fmul_rn(ruB, inv[k]) : 0.f;
      rA[k] = xA[k];
      rB[k] = xB[k];
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float nA[NA], nB[NA];
#pragma unroll
      for (int k = 0; k < NA; ++k) {
        nA[k] = __shfl_up_sync(0xffffffffu, rA[k], o);
        nB[k] = __shfl_up_sync(0xffffffffu, rB[k], o);
      }
      if (lane >= o) {
#pragma unroll
        for (int k = 0; k < NA; ++k) {
          rA[k] = __fadd_rn(rA[k], nA[k]);
          rB[k] = __fadd_rn(rB[k], nB[k]);
        }
      }
    }
    int c4A[kGH] = {0, 0, 0, 0}, c4B[kGH] = {0, 0, 0, 0};
#pragma unroll
    for (int k = 0; k < NA; ++k) {
      const float preA = __fsub_rn(rA[k], xA[k]);
      const float preB = __fsub_rn(rB[k], xB[k]);
      const float totA = __shfl_sync(0xffffffffu, __fadd_rn(preA, xA[k]), lastA);
      const float totB = __shfl_sync(0xffffffffu, __fadd_rn(preB, xB[k]), lastB);
      const float carryB = __fadd_rn(carry[k], totA);
      const float pgA = __fadd_rn(carry[k], preA);
      const float cgA = __fadd_rn(pgA, xA[k]);
      const float pgB = __fadd_rn(carryB, preB);
      const float cgB = __fadd_rn(pgB, xB[k]);
      int a = __float2int_rd(__fadd_rn(off0[k], cgA)) - __float2int_rd(__fadd_rn(off0[k], pgA));
      int b = __float2int_rd(__fadd_rn(off0[k], cgB)) - __float2int_rd(__fadd_rn(off0[k], pgB));
      a = a < 0 ? 0 : (a > 32767 ? 32767 : a);
      b = b < 0 ? 0 : (b > 32767 ? 32767 : b);
      a = validA ? a : 0;
      b = validB ? b : 0;
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        c4A[g] = (hs[k] == g) ? a : c4A[g];
        c4B[g] = (hs[k] == g) ? b : c4B[g];
      }
      carry[k] = hasB ? __fadd_rn(carryB, totB) : carryB;
    }
    if (tr.counts != nullptr) {
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        const size_t o = size_t(g) * tr.head_stride + ch * kChunkRows + lane;
        if (validA) tr.counts[o] = (int16_t)c4A[g];
        if (validB) tr.counts[o + kChunkRows] = (int16_t)c4B[g];
      }
    }
    const bool flagA = (c4A[0] + c4A[1] + c4A[2] + c4A[3]) > 0;
    const bool flagB = (c4B[0] + c4B[1] + c4B[2] + c4B[3]) > 0;
    const uint32_t maskA = __ballot_sync(0xffffffffu, flagA);
    const uint32_t maskB = __ballot_sync(0xffffffffu, flagB);
    __syncwarp();
    const uint32_t lt = (1u << lane) - 1u;
    const int room = kChunkRows * nch;
    (void)room;  // only the checked build reads it
    if (flagA && SANTA_IN_RANGE(n_emit + __popc(maskA & lt), room, tr.status)) {
      emit[n_emit + __popc(maskA & lt)] =
          make_uint4((uint32_t)c4A[0] | ((uint32_t)c4A[1] << 16), (uint32_t)c4A[2] | ((uint32_t)c4A[3] << 16),
                     (uint32_t)(ch * kChunkRows + lane), 0u);
      if (tr.rowmask != nullptr) tr.rowmask[ch * kChunkRows + lane] = 1;
      if (tr.vrow0 != nullptr) prefetch_row_l2(tr.vrow0 + size_t(ch * kChunkRows + lane) * tr.row_stride);
    }
    if (flagB && SANTA_IN_RANGE(n_emit + __popc(maskA) + __popc(maskB & lt), room, tr.status)) {
      emit[n_emit + __popc(maskA) + __popc(maskB & lt)] =
          make_uint4((uint32_t)c4B[0] | ((uint32_t)c4B[1] << 16), (uint32_t)c4B[2] | ((uint32_t)c4B[3] << 16),
                     (uint32_t)((ch + 1) * kChunkRows + lane), 0u);
      if (tr.rowmask != nullptr) tr.rowmask[(ch + 1) * kChunkRows + lane] = 1;
      if (tr.vrow0 != nullptr) prefetch_row_l2(tr.vrow0 + size_t((ch + 1) * kChunkRows + lane) * tr.row_stride);
    }
    n_emit += __popc(maskA) + __popc(maskB);
  }
  __syncwarp();
  return n_emit;
}

// Sparse sum of c*V over the emit list, ascending rows, fp32 fma per head
// (flash_style_fused_santa_fixed_tile_budgets/santa_cuda_kernel.cu:347-379,
// santa_fused_proportional_tile_budgets/santa_cuda_kernel.cu:843-857).
// Lane l accumulates dims 4l..4l+3 of each head; eight rows are in flight.
// `vrow0` points at the V row of the tile's first row for this kv-head.
template <typename TK>
__device__ __forceinline__ void gather_rows(const float4* sb, int n_emit, const unsigned char* __restrict__ vrow0,
                                            size_t row_stride, int lane, float (&o)[kGH][4], int* status = nullptr,
                                            int rows_left = 0) {
  (void)status;
  (void)rows_left;
  constexpr int kInFlight = 8;
  const uint4* emit = reinterpret_cast<const uint4*>(sb);
#pragma unroll 1
  for (int i0 = 0; i0 < n_emit; i0 += kInFlight) {
    uint2 vv[kInFlight];
#pragma unroll
    for (int k = 0; k < kInFlight; ++k) {
#ifdef SANTA_B200_CHECKS
      vv[k] = make_uint2(0u, 0u);  // a skipped row contributes nothing
#endif
      if (i0 + k < n_emit && SANTA_IN_RANGE(emit[i0 + k].z, rows_left, status))
        vv[k] = __ldg(reinterpret_cast<const uint2*>(vrow0 + size_t(emit[i0 + k].z) * row_stride) + lane);
    }
#pragma unroll
    for (int k = 0; k < kInFlight; ++k) {
      if (i0 + k < n_emit) {
        const uint4 en = emit[i0 + k];
        const float2 va = Store16<TK>::unpack(vv[k].x), vb = Store16<TK>::unpack(vv[k].y);
        const int cg4[kGH] = {int(en.x & 0xffffu), int(en.x >> 16), int(en.y & 0xffffu), int(en.y >> 16)};
#pragma unroll
        for (int g = 0; g < kGH; ++g) {
          if (cg4[g] != 0) {
            const float cf = (float)cg4[g];
            o[g][0] = fmaf(cf, va.x, o[g][0]);
            o[g][1] = fmaf(cf, va.y, o[g][1]);
            o[g][2] = fmaf(cf, vb.x, o[g][2]);
            o[g][3] = fmaf(cf, vb.y, o[g][3]);
          }
        }
      }
    }
  }
  __syncwarp();
}

// ---------------------------------------------------------------- work split over column slots
// A CTA has kGroupWarps column slots.  With group width gw (a power of two
// <= 8) the slots form 8/gw slot groups of gw columns.  The (column group,
// tile) items -- column groups being gw consecutive columns -- are cut into nvg
// contiguous, balanced ranges, one per virtual group, and the virtual groups
// are dealt to the CTAs in contiguous, balanced runs: CTA c runs the virtual
// groups [lo(c), lo(c+1)) with lo(c) = floor(c * nvg / ctas), one per slot
// group.  A CTA's slot groups therefore hold neighbouring item ranges and the
// CTAs' item totals differ by at most one item, also when the virtual groups'
// own sizes differ (a problem of few tiles per slot).
struct WarpWork {
  int vg, col_in_group;
  long long lo, hi;
};

__device__ __forceinline__ WarpWork warp_work(const WorkSplit& w, int cta, int ctas, int slot) {
  WarpWork r;
  const int first = int(range_lo(cta, w.nvg, ctas));
  const int count = int(range_lo(cta + 1, w.nvg, ctas)) - first;  // <= 8 / gw by construction of nvg
  const int sg = slot / w.gw;
  r.vg = (sg < count) ? first + sg : w.nvg;
  r.col_in_group = slot % w.gw;
  if (r.vg < w.nvg) {
    r.lo = range_lo(r.vg, w.items, w.nvg);
    r.hi = range_lo(r.vg + 1, w.items, w.nvg);
  } else {
    r.lo = r.hi = 0;
  }
  return r;
}

}  // namespace santa
