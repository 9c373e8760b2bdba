// stream_scores.cuh -- the K-streaming front end shared by the Flash kernel and
// Prop's first pass: a warp stages 32-row chunks of one kv-head's K rows in
// shared memory with bulk asynchronous copies and forms the four query heads'
// scores for every row in the reference's exact floating-point order.
//
// Score order being reproduced (flash_style_fused_santa_fixed_tile_budgets/
// santa_cuda_kernel.cu:161-221, santa_fused_proportional_tile_budgets/
// santa_cuda_kernel.cu:317-379): reference lane i in [0,32) owns dims 4i..4i+3
// and forms p_i = fma(q3,k3,fma(q2,k2,fma(q1,k1,fma(q0,k0,0)))) with
// q = fp32(q16)*q_scale; the row's score is the shfl_down tree
//   a_i=p_i+p_{i+16}, b_i=a_i+a_{i+8}, c_i=b_i+b_{i+4}, d_i=c_i+c_{i+2}, s=d_0+d_1.
//
// Mapping used here: 8 threads per row (4 rows per warp step).  Thread j of a
// row group owns the reference lanes j, j+8, j+16, j+24, so the first two tree
// levels are register adds and the last three are xor-shuffles inside the
// 8-thread group (addition commutes, so the butterfly yields the same bits as
// the one-sided tree).  The two partials of a register pair are computed by
// one packed fma.rn.f32x2, which is IEEE-identical to two scalar fmas.
//
// Shared-memory banks: rows are 256 B apart, so the two row groups of a
// half-warp would hit the same banks.  Odd row groups therefore visit the
// four 64-byte segments of their row in the order 1,0,3,2 instead of 0,1,2,3
// and keep their query registers permuted the same way; the per-thread code is
// uniform and conflict-free.
#pragma once

#include "common.cuh"

namespace santa {

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

// Scores of the 32 rows of one staged chunk: on return lane l holds the four
// heads' scores of row l in s_out.  Rows that were not staged produce garbage
// the caller masks.
template <typename TK>
__device__ __forceinline__ void score_chunk(const unsigned char* __restrict__ stage, const QRegs& Q,
                                            int lane, float (&s_out)[kGH]) {
  const int j = lane & 7;
  const int rr = lane >> 3;
  const int odd = rr & 1;
  const unsigned char* pA = stage + (8 * rr) * kRowBytes + j * 8 + odd * 64;
  const unsigned char* pB = stage + (8 * rr) * kRowBytes + j * 8 + (odd ^ 1) * 64;
#pragma unroll
  for (int ii = 0; ii < 8; ++ii) {
    const uint2 w0 = *reinterpret_cast<const uint2*>(pA + ii * kRowBytes);
    const uint2 w1 = *reinterpret_cast<const uint2*>(pB + ii * kRowBytes);
    const uint2 w2 = *reinterpret_cast<const uint2*>(pA + ii * kRowBytes + 128);
    const uint2 w3 = *reinterpret_cast<const uint2*>(pB + ii * kRowBytes + 128);
    const float2 k0a = Store16<TK>::unpack(w0.x), k0b = Store16<TK>::unpack(w0.y);
    const float2 k1a = Store16<TK>::unpack(w1.x), k1b = Store16<TK>::unpack(w1.y);
    const float2 k2a = Store16<TK>::unpack(w2.x), k2b = Store16<TK>::unpack(w2.y);
    const float2 k3a = Store16<TK>::unpack(w3.x), k3b = Store16<TK>::unpack(w3.y);
    float2 kp[2][4];
    kp[0][0] = make_float2(k0a.x, k1a.x);
    kp[0][1] = make_float2(k0a.y, k1a.y);
    kp[0][2] = make_float2(k0b.x, k1b.x);
    kp[0][3] = make_float2(k0b.y, k1b.y);
    kp[1][0] = make_float2(k2a.x, k3a.x);
    kp[1][1] = make_float2(k2a.y, k3a.y);
    kp[1][2] = make_float2(k2b.x, k3b.x);
    kp[1][3] = make_float2(k2b.y, k3b.y);
#pragma unroll
    for (int g = 0; g < kGH; ++g) {
      float2 a01 = make_float2(0.f, 0.f), a23 = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a01 = __ffma2_rn(Q.qp[g][0][i], kp[0][i], a01);
        a23 = __ffma2_rn(Q.qp[g][1][i], kp[1][i], a23);
      }
      const float2 t = __fadd2_rn(a01, a23);  // (a_j, a_{j+8}) in either order
      float b = __fadd_rn(t.x, t.y);
      b = __fadd_rn(b, __shfl_xor_sync(0xffffffffu, b, 4));
      b = __fadd_rn(b, __shfl_xor_sync(0xffffffffu, b, 2));
      b = __fadd_rn(b, __shfl_xor_sync(0xffffffffu, b, 1));
      if (ii == j) s_out[g] = b;
    }
  }
}

// Per-warp staging ring: kStages chunks of 32 rows x 256 B, one mbarrier each.
template <int kStages>
struct WarpRing {
  unsigned char* data;  // kStages * kStageBytes, 128-byte aligned
  uint32_t bar0;        // shared address of the first of kStages barriers
  uint32_t count;       // chunks consumed so far by this warp (selects stage and parity)

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
  // Stage rows [row0, row0+32) of a K column whose rows lie `row_stride` bytes
  // apart into the stage that global chunk number `g` maps to.  Rows at or
  // beyond `row_end` are not copied.
  __device__ __forceinline__ void issue(uint32_t g, const unsigned char* col_base, size_t row_stride,
                                        int row0, int row_end, int lane) {
    const uint32_t st = g % kStages;
    const int row = row0 + lane;
    const bool v = row < row_end;
    const uint32_t nvalid = __popc(__ballot_sync(0xffffffffu, v));
    const uint32_t bar = bar0 + 8 * st;
    if (lane == 0) mbar_arrive_expect_tx(bar, nvalid * kRowBytes);
    __syncwarp();
    if (v)
      bulk_g2s(smem_u32(data + st * kStageBytes + lane * kRowBytes), col_base + size_t(row) * row_stride,
               kRowBytes, bar);
  }
  __device__ __forceinline__ const unsigned char* stage_ptr(uint32_t g) const {
    return data + (g % kStages) * kStageBytes;
  }
  __device__ __forceinline__ bool wait(uint32_t g) const {
    return mbar_wait_bounded(bar0 + 8 * (g % kStages), (g / kStages) & 1u);
  }
};

}  // namespace santa
