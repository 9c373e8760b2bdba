// stream_scores.cuh -- the K-streaming front end shared by the Flash kernel and
// Prop's first pass: a warp stages 32-row pieces of one kv-head's K rows in
// shared memory with tiled TMA loads (cp.async.bulk.tensor) and forms the four query heads'
// scores for every row in the reference's exact floating-point order.
//
// Score order being reproduced (flash_style_fused_santa_fixed_tile_budgets/
// santa_cuda_kernel.cu:161-221, santa_fused_proportional_tile_budgets/
// santa_cuda_kernel.cu:317-379): reference lane i in [0,32) owns dims 4i..4i+3
// and forms p_i = fma(q3,k3,fma(q2,k2,fma(q1,k1,fma(q0,k0,0)))) with
// q = fp32(q16)*q_scale; the row's score is the shfl_down tree
//   a_i=p_i+p_{i+16}, b_i=a_i+a_{i+8}, c_i=b_i+b_{i+4}, d_i=c_i+c_{i+2}, s=d_0+d_1.
//
// Mapping used here: 8 threads per row.  Thread j of a row group owns the
// reference lanes j, j+8, j+16, j+24, so the first two tree levels are register
// adds; the eight b_j of a row then go through a small shared-memory exchange
// and one thread per (row, head) finishes the tree (7 adds) -- cheaper than
// three shuffle levels per head.  The two partials of a register pair are
// computed by one packed fma.rn.f32x2, which is IEEE-identical to two scalar
// fmas; addition commutes, so operand order never changes a bit.
//
// Shared-memory banks: rows are 256 B apart, so the two row groups of a
// half-warp would hit the same banks.  Odd row groups therefore visit the
// four 64-byte segments of their row in the order 1,0,3,2 instead of 0,1,2,3
// and keep their query registers permuted the same way; the per-thread code is
// uniform and conflict-free.
#pragma once

#include "common.cuh"

namespace santa {

constexpr int kRedStride = 36;                  // floats per row in the exchange buffer (bank-conflict free)
constexpr int kRedFloats = 16 * kRedStride;         // one exchange per 16 rows

// Query registers of one thread: qp[g][h][i] = (q[g][slot 2h][i], q[g][slot 2h+1][i])
// where slot s of this thread covers reference lane j + 8*(s ^ odd).
struct QRegs {
  float2 qp[kGH][2][4];
};

template <typename TK>
__device__ __forceinline__ void load_q(const TK* __restrict__ q_head0, float q_scale, int lane, QRegs& Q) {
  const int j = lane & 7;
  const int odd = (lane >> 3) & 1;
#pragma unroll
  for (int g = 0; g < kGH; ++g) {
    const uint2* qrow = reinterpret_cast<const uint2*>(q_head0 + g * kD);
    float qs[4][4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const uint2 w = qrow[j + 8 * (s ^ odd)];
      const float2 lo = Store16<TK>::unpack(w.x), hi = Store16<TK>::unpack(w.y);
      qs[s][0] = lo.x * q_scale;
      qs[s][1] = lo.y * q_scale;
      qs[s][2] = hi.x * q_scale;
      qs[s][3] = hi.y * q_scale;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) Q.qp[g][h][i] = make_float2(qs[2 * h][i], qs[2 * h + 1][i]);
  }
}

// Raw K words of one thread for one step of four rows (its four 8-byte slots).
struct KRaw {
  uint2 w[4];
};

__device__ __forceinline__ void load_k4(const unsigned char* __restrict__ rows, int step, int lane, KRaw& k) {
  const int j = lane & 7;
  const int rr = lane >> 3;
  const int odd = rr & 1;
  const unsigned char* rp = rows + (4 * step + rr) * kRowBytes + j * 8;
  k.w[0] = *reinterpret_cast<const uint2*>(rp + odd * 64);
  k.w[1] = *reinterpret_cast<const uint2*>(rp + (odd ^ 1) * 64);
  k.w[2] = *reinterpret_cast<const uint2*>(rp + odd * 64 + 128);
  k.w[3] = *reinterpret_cast<const uint2*>(rp + (odd ^ 1) * 64 + 128);
}

// b_j of the thread's row for the four heads, written to the exchange buffer.
template <typename TK>
__device__ __forceinline__ void partial_rows4(const KRaw& k, const QRegs& Q, float* __restrict__ red, int step,
                                              int lane) {
  const int j = lane & 7;
  const int rr = lane >> 3;
  const float2 k0a = Store16<TK>::unpack(k.w[0].x), k0b = Store16<TK>::unpack(k.w[0].y);
  const float2 k1a = Store16<TK>::unpack(k.w[1].x), k1b = Store16<TK>::unpack(k.w[1].y);
  const float2 k2a = Store16<TK>::unpack(k.w[2].x), k2b = Store16<TK>::unpack(k.w[2].y);
  const float2 k3a = Store16<TK>::unpack(k.w[3].x), k3b = Store16<TK>::unpack(k.w[3].y);
  float2 kp[2][4];
  kp[0][0] = make_float2(k0a.x, k1a.x);
  kp[0][1] = make_float2(k0a.y, k1a.y);
  kp[0][2] = make_float2(k0b.x, k1b.x);
  kp[0][3] = make_float2(k0b.y, k1b.y);
  kp[1][0] = make_float2(k2a.x, k3a.x);
  kp[1][1] = make_float2(k2a.y, k3a.y);
  kp[1][2] = make_float2(k2b.x, k3b.x);
  kp[1][3] = make_float2(k2b.y, k3b.y);
  float b[kGH];
#pragma unroll
  for (int g = 0; g < kGH; ++g) {
    float2 a01 = make_float2(0.f, 0.f), a23 = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a01 = __ffma2_rn(Q.qp[g][0][i], kp[0][i], a01);
      a23 = __ffma2_rn(Q.qp[g][1][i], kp[1][i], a23);
    }
    const float2 t = __fadd2_rn(a01, a23);  // (a_j, a_{j+8}) in either order
    b[g] = __fadd_rn(t.x, t.y);             // b_j
  }
  *reinterpret_cast<float4*>(red + (4 * step + rr) * kRedStride + 4 * j) = make_float4(b[0], b[1], b[2], b[3]);
}

// Scores of 16 consecutive rows (half of a staged 32-row piece).  `rows` points at the first
// of them in the staging buffer, `red` at this slot's exchange buffer (kRedFloats floats) and
// `score_out` at 64 floats laid out [row][head].  The K words of the next
// four-row step are fetched while the current step is multiplied, and a single
// exchange finishes all 16 rows.  Rows that were not staged produce garbage
// the caller masks.
template <typename TK>
__device__ __forceinline__ void score_rows16(const unsigned char* __restrict__ rows, const QRegs& Q,
                                             float* __restrict__ red, float* __restrict__ score_out, int lane) {
  KRaw k0, k1;
  load_k4(rows, 0, lane, k0);
  load_k4(rows, 1, lane, k1);
  partial_rows4<TK>(k0, Q, red, 0, lane);
  load_k4(rows, 2, lane, k0);
  partial_rows4<TK>(k1, Q, red, 1, lane);
  load_k4(rows, 3, lane, k1);
  partial_rows4<TK>(k0, Q, red, 2, lane);
  partial_rows4<TK>(k1, Q, red, 3, lane);
  __syncwarp();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float* rd = red + (8 * h + (lane >> 2)) * kRedStride + (lane & 3);
    const float c0 = __fadd_rn(rd[0], rd[16]);
    const float c1 = __fadd_rn(rd[4], rd[20]);
    const float c2 = __fadd_rn(rd[8], rd[24]);
    const float c3 = __fadd_rn(rd[12], rd[28]);
    const float d0 = __fadd_rn(c0, c2);
    const float d1 = __fadd_rn(c1, c3);
    score_out[32 * h + lane] = __fadd_rn(d0, d1);
  }
  __syncwarp();
}

// ---------------------------------------------------------------- tensor-core scores (opt-in)
// The same scores from the tensor cores: NOT the reference's floating-point order, hence an opt-in
// mode whose sampled counts can differ from the reference's on rare rows.  The four query heads of
// the group, scaled in fp32 like the exact path, are split into a high and a low 16-bit part
// (q = hi + lo up to 2^-17 relative); the eight columns of an m16n8k16 step hold hi of heads 0..3
// and lo of heads 0..3, the 16 rows are 16 K rows, and the score of (row, head) is the sum of the
// two columns.  Products of two 16-bit values are exact in fp32, so the result differs from the
// exact path only by the order and rounding of the fp32 accumulation inside the tensor core.
//
// Staging for this path: a 32-row piece arrives as two TMA boxes of 64 elements x 32 rows with the
// 128-byte swizzle (16-byte chunk index XOR row mod 8), so that ldmatrix reads eight rows of one
// k-chunk without bank conflicts.  Stage buffers are 1024-byte aligned.
struct QFrag {
  uint32_t b[kD / 16][2];  // B fragments of the eight k-steps
};

template <typename TK>
__device__ __forceinline__ void load_q_frag(const TK* __restrict__ q_head0, float q_scale, int lane, QFrag& Q) {
  const int n = lane >> 2;       // column of the fragment: heads 0..3 high parts, then their low parts
  const int kk = 2 * (lane & 3);
  const TK* qrow = q_head0 + (n & 3) * kD;
#pragma unroll
  for (int ks = 0; ks < kD / 16; ++ks)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const float2 f = Store16<TK>::unpack(*reinterpret_cast<const uint32_t*>(qrow + ks * 16 + half * 8 + kk));
      const float x0 = f.x * q_scale, x1 = f.y * q_scale;
      const float h0 = Store16<TK>::round(x0), h1 = Store16<TK>::round(x1);
      const float v0 = (n < kGH) ? h0 : __fsub_rn(x0, h0);
      const float v1 = (n < kGH) ? h1 : __fsub_rn(x1, h1);
      Q.b[ks][half] = uint32_t(Store16<TK>::bits(v0)) | (uint32_t(Store16<TK>::bits(v1)) << 16);
    }
}

// Scores of 16 consecutive rows of a swizzled piece.  `piece` is the shared-memory address of the
// piece (1024-byte aligned: rows 0..31 x elements 0..63, then the same rows x elements 64..127),
// `rb` selects its first or second 16 rows, `score_out` points at 64 floats laid out [row][head].
template <typename TK>
__device__ __forceinline__ void score_rows16_mma(uint32_t piece, int rb, const QFrag& Q,
                                                 float* __restrict__ score_out, int lane) {
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  const int row = rb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;  // the row whose address this lane supplies
#pragma unroll
  for (int ks = 0; ks < kD / 16; ++ks) {
    const int chunk = 2 * (ks & 3) + (lane >> 4);
    const uint32_t addr = piece + (ks >> 2) * (kStageBytes / 2) + row * 128 + ((chunk ^ (row & 7)) << 4);
    uint32_t a[4];
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                 : "r"(addr));
    MmaOp<TK>::mma(c, a, Q.b[ks]);
  }
  // c0,c1: row lane/4, columns 2*(lane%4), +1;  c2,c3: row lane/4 + 8.  high + low part of a head
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] = __fadd_rn(c[i], __shfl_xor_sync(0xffffffffu, c[i], 2));
  if ((lane & 3) < 2) {
    float2* so = reinterpret_cast<float2*>(score_out);
    so[(lane >> 2) * 2 + (lane & 3)] = make_float2(c[0], c[1]);
    so[((lane >> 2) + 8) * 2 + (lane & 3)] = make_float2(c[2], c[3]);
  }
  __syncwarp();
}

// Per-warp staging ring: kStages pieces of kStageRows rows x 256 B, one mbarrier each.
template <int kStages>
struct WarpRing {
  unsigned char* data;  // kStages * kStageBytes, 128-byte aligned
  uint32_t bar0;        // shared address of the first of kStages barriers
  uint32_t count;       // stages consumed so far by this warp (selects slot and parity)

  __device__ __forceinline__ void init(unsigned char* d, uint64_t* bars, int lane) {
    data = d;
    bar0 = smem_u32(bars);
    count = 0;
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8 * s, 1);
      mbar_fence_init();
    }
  }
  // Stage rows [row0, row0+kStageRows) of K column (b, kv) into the slot that
  // global stage number `g` maps to: one tiled TMA load of a {128, 1, 16, 1}
  // box from the [B][L_storage][KVH][128] tensor `tmap` describes.  Rows past
  // the end of the storage read as zeros; the caller masks rows past the valid
  // length.
  // SWZ: the map describes {64, 1, 32, 1} boxes with the 128-byte swizzle (tensor-core score path):
  // two loads fill the slot, elements 0..63 of the rows first, elements 64..127 behind them.
  template <bool SWZ = false>
  __device__ __forceinline__ void issue(uint32_t g, const void* tmap, int b, int kv, int row0, int lane) {
    if (lane == 0) {
      const uint32_t st = g % kStages;
      const uint32_t bar = bar0 + 8 * st;
      mbar_arrive_expect_tx(bar, kStageBytes);
      const uint32_t dst = smem_u32(data + st * kStageBytes);
      if (SWZ) {
        tma_load_4d(dst, tmap, 0, kv, row0, b, bar);
        tma_load_4d(dst + kStageBytes / 2, tmap, kD / 2, kv, row0, b, bar);
      } else {
        tma_load_4d(dst, tmap, 0, kv, row0, b, bar);
      }
    }
  }
  __device__ __forceinline__ const unsigned char* stage_ptr(uint32_t g) const {
    return data + (g % kStages) * kStageBytes;
  }
  __device__ __forceinline__ bool wait(uint32_t g) const {
    return mbar_wait_bounded(bar0 + 8 * (g % kStages), (g / kStages) & 1u);
  }
};

}  // namespace santa
