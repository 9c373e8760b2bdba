// flash_kernels.cu -- S2ANTA-Flash decode attention (fixed per-tile sample
// budget) for sm_100a.  Two launches on one stream, chained with programmatic
// dependent launch:
//   flash_decode_kernel  persistent, one CTA per SM; streams K once through TMA,
//                        samples rows by systematic resampling inside every
//                        tile, gathers the sampled V rows and folds tiles into
//                        a running log-sum-exp state; every CTA writes one
//                        partial (A[128], m, Z per head) per column group it
//                        touched;
//   flash_merge_kernel   one small CTA per (batch, head) folds the partials into
//                        out / m_star / vrows (or an unnormalised partial for a
//                        cross-device combine).
//
// Replaces, with identical sampled row counts, the reference's
//   fused_tiles_vec_gqa_gh4_d128_bn   (flash_style_fused_santa_fixed_tile_budgets/santa_cuda_kernel.cu:96-380)
//   finalize_weighted_out_kernel      (same file :386-470)
//   reduce_vrows_kernel               (same file :475-508)
//
// This translation unit must be compiled with --use_fast_math, like the
// reference's Flash extension (its setup.py:15-20): the per-tile step
// S_per_tile/ell is then the same approximate division and exp the same
// flush-to-zero ex2, which the sampled counts depend on.
//
// Work layout.  A "column" is one (batch, kv-head) pair; eight consecutive
// columns form a column group, so that the eight 256-byte K rows of a token are
// fetched together.  Work items are (column group, tile) pairs; CTA i owns a
// contiguous balanced range of them.  A CTA has sixteen warps, two per column:
//   * the SCORE warp of a column owns a TMA staging ring, streams the column's
//     K rows and writes the four heads' scores of a tile into one of two score
//     buffers;
//   * the SAMPLER warp of the column turns a finished score buffer into tile
//     statistics, sampled counts, the sparse sum of V rows and the running
//     log-sum-exp state.
// The two warps hand buffers over through a full/empty pair of mbarriers per
// buffer, so K keeps streaming while the previous tile is being sampled.  No
// warp ever synchronises with another column.  All hot loops are rolled so that
// the instruction footprint stays small; every wait is bounded.

#include <cooperative_groups.h>

#include "santa_abi_internal.h"
#include "stream_scores.cuh"

namespace santa {

constexpr int kFlashStages = 4;
constexpr int kMaxTileRows = 256;
constexpr int kScoreBytes = kMaxTileRows * kGH * 4;  // one score buffer: scores, then u, then the emit list
constexpr int kColSmem = kFlashStages * kStageBytes + 2 * kScoreBytes + kRedFloats * 4;
constexpr int kColBars = kFlashStages + 4;           // ring + full[2] + empty[2]
constexpr int kCtaWarps = 2 * kGroupWarps;
constexpr size_t kFlashSmemBytes = size_t(kGroupWarps) * kColSmem + size_t(kGroupWarps) * kColBars * 8;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <typename TK, int BN>
__global__ void __launch_bounds__(kCtaWarps * 32, 1) flash_decode_kernel(const __grid_constant__ FlashParams p) {
  constexpr int NW = (BN == 256) ? 8 : 4;    // warps of the reference block (fixes the ell order)
  constexpr int NH = NW / 4;                 // 32-row halves per reference pass

  extern __shared__ __align__(128) unsigned char smem[];
  const int cta_warp = threadIdx.x >> 5;
  const int warp = cta_warp & (kGroupWarps - 1);  // column within the column group
  const bool is_sampler = cta_warp >= kGroupWarps;
  const int lane = threadIdx.x & 31;

  unsigned char* cbase = smem + size_t(warp) * kColSmem;
  float* scorebufs = reinterpret_cast<float*>(cbase + kFlashStages * kStageBytes);
  float* red = reinterpret_cast<float*>(cbase + kFlashStages * kStageBytes + 2 * kScoreBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + size_t(kGroupWarps) * kColSmem) + warp * kColBars;
  const uint32_t bar_full = smem_u32(bars + kFlashStages);       // [2]
  const uint32_t bar_empty = smem_u32(bars + kFlashStages + 2);  // [2]

  WarpRing<kFlashStages> ring;
  if (!is_sampler) {
    ring.init(cbase, bars, lane);
    if (lane == 0) {
      mbar_init(bar_full, 1);
      mbar_init(bar_full + 8, 1);
      mbar_init(bar_empty, 1);
      mbar_init(bar_empty + 8, 1);
      mbar_fence_init();
    }
  }
  __syncthreads();

  const TK* __restrict__ Qg = static_cast<const TK*>(p.q);
  const unsigned char* __restrict__ Vg = static_cast<const unsigned char*>(p.V);
  const size_t row_stride = size_t(p.KVH) * kRowBytes;

  const long long lo = range_lo(blockIdx.x, p.items, gridDim.x);
  const long long hi = range_lo(blockIdx.x + 1, p.items, gridDim.x);
  bool dead = false;     // set when a wait ran out; the status word then says why
  uint32_t handoff = 0;  // tiles handed over so far on this column (selects buffer and parity)

  long long it = lo;
  while (it < hi) {
    const int cg = int(it / p.T_c);
    const int t_lo = int(it - (long long)cg * p.T_c);
    const int t_hi = (hi - it < (long long)(p.T_c - t_lo)) ? t_lo + int(hi - it) : p.T_c;
    const int col = cg * kGroupWarps + warp;
    const bool active = col < p.ncol;
    const int slot = blockIdx.x + cg;  // distinct for every (CTA, column group) pair that occurs
    const int b = active ? col / p.KVH : 0;
    const int kv = col - b * p.KVH;
    const int h0 = kv * kGH;

    if (active && !is_sampler) {
      // =========================== SCORE warp ===============================
      QRegs Q;
      load_q<TK>(Qg + (size_t(b) * p.H + h0) * kD, p.q_scale, lane, Q);
      const int row_base = t_lo * BN;
      const int row_end = (t_hi * BN < p.L_valid) ? t_hi * BN : p.L_valid;
      const int npieces = (row_end - row_base + kStageRows - 1) / kStageRows;
      int issued = 0;
      for (; issued < kFlashStages && issued < npieces; ++issued)
        ring.issue(ring.count + issued, &p.tmK, b, kv, row_base + issued * kStageRows, lane);

#pragma unroll 1
      for (int t = t_lo; t < t_hi; ++t, ++handoff) {
        const int n0 = t * BN;
        const int tile_len = (p.L_valid - n0 < BN) ? (p.L_valid - n0) : BN;
        const uint32_t buf = handoff & 1u;
        float* scorebuf = scorebufs + buf * (kScoreBytes / 4);
        // wait until the sampler has released this buffer (passes at once the first two times)
        if (!dead && !mbar_wait_bounded(bar_empty + 8 * buf, ((handoff >> 1) & 1u) ^ 1u)) {
          dead = true;
          if (lane == 0) atomicExch(p.status, kStatusHandoffTimeout);
        }
        const int npc = (tile_len + kStageRows - 1) / kStageRows;
#pragma unroll 1
        for (int pc = 0; pc < npc; ++pc) {
          if (!dead && !ring.wait(ring.count)) {
            dead = true;
            if (lane == 0) atomicExch(p.status, kStatusStageTimeout);
          }
          const unsigned char* st = ring.stage_ptr(ring.count);
          score_rows8<TK>(st, Q, red, scorebuf + (pc * kStageRows) * kGH, lane);
          score_rows8<TK>(st + 8 * kRowBytes, Q, red, scorebuf + (pc * kStageRows + 8) * kGH, lane);
          if (issued < npieces && !dead) {
            ring.issue(ring.count + kFlashStages, &p.tmK, b, kv, row_base + issued * kStageRows, lane);
            ++issued;
          }
          ++ring.count;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full + 8 * buf);
      }
    } else if (active) {
      // ========================== SAMPLER warp ==============================
      const unsigned char* vcol = Vg + (size_t(b) * p.L_storage * p.KVH + kv) * kRowBytes;
      float M[kGH], Z[kGH], A[kGH][4];
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        M[g] = -CUDART_INF_F;
        Z[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) A[g][i] = 0.f;
      }
      int vrow_count = 0;

#pragma unroll 1
      for (int t = t_lo; t < t_hi; ++t, ++handoff) {
        const int n0 = t * BN;
        const int tile_len = (p.L_valid - n0 < BN) ? (p.L_valid - n0) : BN;
        const int nch = (tile_len + kChunkRows - 1) / kChunkRows;
        const uint32_t buf = handoff & 1u;
        float* scorebuf = scorebufs + buf * (kScoreBytes / 4);
        if (!dead && !mbar_wait_bounded(bar_full + 8 * buf, (handoff >> 1) & 1u)) {
          dead = true;
          if (lane == 0) atomicExch(p.status, kStatusHandoffTimeout);
        }
        const float4* sb4 = reinterpret_cast<const float4*>(scorebuf);
        float4* sb4w = reinterpret_cast<float4*>(scorebuf);

        // ---- tile statistics (reference :223-273) -------------------------
        float m[kGH], ell[kGH];
#pragma unroll
        for (int g = 0; g < kGH; ++g) m[g] = -CUDART_INF_F;
#pragma unroll 1
        for (int ch = 0; ch < nch; ++ch) {
          if (ch * kChunkRows + lane < tile_len) {
            const float4 s = sb4[ch * kChunkRows + lane];
            m[0] = fmaxf(m[0], s.x);
            m[1] = fmaxf(m[1], s.y);
            m[2] = fmaxf(m[2], s.z);
            m[3] = fmaxf(m[3], s.w);
          }
        }
#pragma unroll
        for (int g = 0; g < kGH; ++g)
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) m[g] = fmaxf(m[g], __shfl_xor_sync(0xffffffffu, m[g], off));

        // u = exp(s - m) replaces the scores in place; ell is summed in the
        // reference's order: per-thread strided partials (chunk parity picks
        // the half for block_n 256), an 8-row tree per reference warp, then
        // the reference warps in order.
        float V0[kGH], V1[kGH];
#pragma unroll
        for (int g = 0; g < kGH; ++g) V0[g] = V1[g] = 0.f;
#pragma unroll 1
        for (int ch = 0; ch < nch; ++ch) {
          const bool valid = ch * kChunkRows + lane < tile_len;
          float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
          if (valid) {
            const float4 s = sb4[ch * kChunkRows + lane];
            u.x = __expf(s.x - m[0]);
            u.y = __expf(s.y - m[1]);
            u.z = __expf(s.z - m[2]);
            u.w = __expf(s.w - m[3]);
          }
          sb4w[ch * kChunkRows + lane] = u;
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
#pragma unroll
        for (int g = 0; g < kGH; ++g) {
          float x0 = V0[g], x1 = V1[g];
          x0 = __fadd_rn(x0, __shfl_xor_sync(0xffffffffu, x0, 4));
          x0 = __fadd_rn(x0, __shfl_xor_sync(0xffffffffu, x0, 2));
          x0 = __fadd_rn(x0, __shfl_xor_sync(0xffffffffu, x0, 1));
          float e = __shfl_sync(0xffffffffu, x0, 0);
          e = __fadd_rn(e, __shfl_sync(0xffffffffu, x0, 8));
          e = __fadd_rn(e, __shfl_sync(0xffffffffu, x0, 16));
          e = __fadd_rn(e, __shfl_sync(0xffffffffu, x0, 24));
          if (NH == 2) {
            x1 = __fadd_rn(x1, __shfl_xor_sync(0xffffffffu, x1, 4));
            x1 = __fadd_rn(x1, __shfl_xor_sync(0xffffffffu, x1, 2));
            x1 = __fadd_rn(x1, __shfl_xor_sync(0xffffffffu, x1, 1));
            e = __fadd_rn(e, __shfl_sync(0xffffffffu, x1, 0));
            e = __fadd_rn(e, __shfl_sync(0xffffffffu, x1, 8));
            e = __fadd_rn(e, __shfl_sync(0xffffffffu, x1, 16));
            e = __fadd_rn(e, __shfl_sync(0xffffffffu, x1, 24));
          }
          ell[g] = e;
        }

        // ---- systematic counts (reference :275-311) -----------------------
        float invdel[kGH], a0[kGH], carry[kGH];
#pragma unroll
        for (int g = 0; g < kGH; ++g) {
          invdel[g] = (p.S_per_tile > 0 && ell[g] > 1e-20f) ? ((float)p.S_per_tile / ell[g]) : 0.0f;
          a0[g] = u01_from_seed(p.seed, (p.batch_offset + b) * p.H + h0 + g, p.tile_offset + t);
          carry[g] = 0.f;
        }
        int n_emit = 0;
        uint4* emit = reinterpret_cast<uint4*>(scorebuf);  // entry i overwrites row i, which is already consumed
#pragma unroll 1
        for (int ch = 0; ch < nch; ++ch) {
          const int remain = tile_len - ch * kChunkRows;
          const int last_lane = remain > 32 ? 31 : remain - 1;
          const bool valid = lane < remain;
          const float4 u4 = sb4[ch * kChunkRows + lane];
          const float uu[kGH] = {u4.x, u4.y, u4.z, u4.w};
          int c[kGH];
#pragma unroll
          for (int g = 0; g < kGH; ++g) {
            const float u16v = Store16<TK>::round(uu[g]);
            const float xv = (valid && invdel[g] > 0.f) ? __fmul_rn(u16v, invdel[g]) : 0.f;
            float res = xv;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
              const float nb = __shfl_up_sync(0xffffffffu, res, off);
              if (lane >= off) res = __fadd_rn(res, nb);
            }
            const float pre = __fsub_rn(res, xv);
            const float pre_g = __fadd_rn(carry[g], pre);
            const float cum_g = __fadd_rn(pre_g, xv);
            const float f_prev = floorf(__fadd_rn(a0[g], pre_g));
            const float f_curr = floorf(__fadd_rn(a0[g], cum_g));
            int cc = (int)__fsub_rn(f_curr, f_prev);
            cc = cc < 0 ? 0 : cc;
            cc = cc > 32767 ? 32767 : cc;
            c[g] = valid ? cc : 0;
            const float chunk_total = __shfl_sync(0xffffffffu, __fadd_rn(pre, xv), last_lane);
            carry[g] = __fadd_rn(carry[g], chunk_total);
          }
          if (p.dbg_u != nullptr && valid) {
#pragma unroll
            for (int g = 0; g < kGH; ++g) {
              const size_t o = (size_t(b) * p.H + h0 + g) * p.L_valid + n0 + ch * kChunkRows + lane;
              p.dbg_u[o] = Store16<TK>::bits(uu[g]);
              p.dbg_c[o] = (int16_t)c[g];
            }
          }
          // ---- compaction (reference :314-345): ascending row order -------
          const bool flag = (c[0] + c[1] + c[2] + c[3]) > 0;
          const uint32_t mask = __ballot_sync(0xffffffffu, flag);
          __syncwarp();
          if (flag) {
            const int pos = n_emit + __popc(mask & ((1u << lane) - 1u));
            emit[pos] = make_uint4((uint32_t)c[0] | ((uint32_t)c[1] << 16), (uint32_t)c[2] | ((uint32_t)c[3] << 16),
                                   (uint32_t)(ch * kChunkRows + lane), 0u);
            if (p.rowmask != nullptr)
              p.rowmask[(size_t(b) * p.KVH + kv) * p.L_valid + n0 + ch * kChunkRows + lane] = 1;
          }
          n_emit += __popc(mask);
        }
        vrow_count += n_emit;
        if (p.dbg_m != nullptr && lane < kGH) {
          float mv = m[0], ev = ell[0];
#pragma unroll
          for (int g = 1; g < kGH; ++g) {
            mv = (lane == g) ? m[g] : mv;
            ev = (lane == g) ? ell[g] : ev;
          }
          const size_t o = (size_t(b) * p.H + h0 + lane) * p.T_c + t;
          p.dbg_m[o] = mv;
          p.dbg_ell[o] = ev;
        }
        __syncwarp();

        // ---- sparse sum of c*V (reference :347-379), 4 rows in flight ----
        float o[kGH][4];
#pragma unroll
        for (int g = 0; g < kGH; ++g)
#pragma unroll
          for (int i = 0; i < 4; ++i) o[g][i] = 0.f;
#pragma unroll 1
        for (int i0 = 0; i0 < n_emit; i0 += 4) {
          uint4 en[4];
          uint2 vv[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (i0 + k < n_emit) {
              en[k] = emit[i0 + k];
              vv[k] = __ldg(reinterpret_cast<const uint2*>(vcol + size_t(n0 + (int)en[k].z) * row_stride) + lane);
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (i0 + k < n_emit) {
              const float2 va = Store16<TK>::unpack(vv[k].x), vb = Store16<TK>::unpack(vv[k].y);
              const int cg4[kGH] = {int(en[k].x & 0xffffu), int(en[k].x >> 16), int(en[k].y & 0xffffu),
                                    int(en[k].y >> 16)};
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

        // ---- fold the tile into the running (m, Z, A) state ---------------
#pragma unroll
        for (int g = 0; g < kGH; ++g) {
          const float m_new = fmaxf(M[g], m[g]);
          const float so = __expf(M[g] - m_new);
          const float st = __expf(m[g] - m_new) * ell[g];
          Z[g] = Z[g] * so + st;
#pragma unroll
          for (int i = 0; i < 4; ++i) A[g][i] = A[g][i] * so + st * o[g][i];
          M[g] = m_new;
        }
        if (lane == 0) mbar_arrive(bar_empty + 8 * buf);  // the __syncwarp above ordered every lane's reads
      }  // tiles

      // ---- publish this column's partial ---------------------------------
      float* ps = p.partials + (size_t(slot) * kGroupWarps + warp) * (kGH * kPartialStride);
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        reinterpret_cast<float4*>(ps + g * kPartialStride)[lane] = make_float4(A[g][0], A[g][1], A[g][2], A[g][3]);
        if (lane == 0) {
          ps[g * kPartialStride + kD] = M[g];
          ps[g * kPartialStride + kD + 1] = Z[g];
        }
      }
      if (lane == 0) p.partial_vrows[slot * kGroupWarps + warp] = vrow_count;
    } else {
      handoff += uint32_t(t_hi - t_lo);
    }
    it += (t_hi - t_lo);
  }
}

// Folds the partials of one (column, head) pair.  Launched as a programmatic
// dependent of flash_decode_kernel: it may become resident early and waits for
// the producer grid before touching its results.
//   m* = max_v m_v;  w_v = exp(m_v - m*);  Z = sum_v w_v Z_v;  A = sum_v w_v A_v;
//   out = A / (Z * S_per_tile)            (reference :436-468 over all tiles)
template <typename TK>
__global__ void __launch_bounds__(128) flash_merge_kernel(const FlashMergeParams p) {
  cudaGridDependencySynchronize();
  __shared__ float s_w[kMaxCtas];
  __shared__ float s_red[4];
  __shared__ int s_redi[4];
  __shared__ float4 s_acc[4][32];

  const int col = blockIdx.x >> 2;
  const int g = blockIdx.x & 3;
  const int cg = col / kGroupWarps;
  const int w = col - cg * kGroupWarps;
  const int b = col / p.KVH;
  const int kv = col - b * p.KVH;
  const int tid = threadIdx.x, lane = tid & 31, wq = tid >> 5;

  const int v_first = cta_of_item((long long)cg * p.T_c, p.items, p.ctas);
  const int v_last = cta_of_item((long long)(cg + 1) * p.T_c - 1, p.items, p.ctas);
  const int nv = v_last - v_first + 1;
  auto partial = [&](int v) {
    return p.partials + ((size_t(v + cg) * kGroupWarps + w) * kGH + g) * kPartialStride;
  };

  // phase 1: m*
  float mloc = -CUDART_INF_F;
  for (int i = tid; i < nv; i += 128) {
    const float mv = __ldcg(partial(v_first + i) + kD);
    s_w[i] = mv;
    mloc = fmaxf(mloc, mv);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, off));
  if (lane == 0) s_red[wq] = mloc;
  __syncthreads();
  const float ms = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
  __syncthreads();

  // phase 2: weights, Z, gathered-row count
  float zloc = 0.f;
  int vloc = 0;
  for (int i = tid; i < nv; i += 128) {
    const float e = __expf(s_w[i] - ms);
    zloc += e * __ldcg(partial(v_first + i) + kD + 1);
    if (g == 0 && p.vrows != nullptr) vloc += __ldcg(p.partial_vrows + (v_first + i + cg) * kGroupWarps + w);
    s_w[i] = e;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    zloc += __shfl_xor_sync(0xffffffffu, zloc, off);
    vloc += __shfl_xor_sync(0xffffffffu, vloc, off);
  }
  if (lane == 0) {
    s_red[wq] = zloc;
    s_redi[wq] = vloc;
  }
  __syncthreads();
  const float zs = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);

  // phase 3: A, four partials in flight per warp
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i0 = wq; i0 < nv; i0 += 16) {
    float e[4];
    float4 a[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = i0 + 4 * k;
      e[k] = (i < nv) ? s_w[i] : 0.f;
      a[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < nv) a[k] = __ldcg(reinterpret_cast<const float4*>(partial(v_first + i)) + lane);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      acc.x += e[k] * a[k].x;
      acc.y += e[k] * a[k].y;
      acc.z += e[k] * a[k].z;
      acc.w += e[k] * a[k].w;
    }
  }
  s_acc[wq][lane] = acc;
  __syncthreads();
  if (wq == 0) {
    const float4 a1 = s_acc[1][lane], a2 = s_acc[2][lane], a3 = s_acc[3][lane];
    acc.x = (acc.x + a1.x) + (a2.x + a3.x);
    acc.y = (acc.y + a1.y) + (a2.y + a3.y);
    acc.z = (acc.z + a1.z) + (a2.z + a3.z);
    acc.w = (acc.w + a1.w) + (a2.w + a3.w);
    const size_t bh = size_t(b) * p.H + kv * kGH + g;
    if (p.partial_out != nullptr) {
      // raw merged partial for a cross-device combine: A[128], m, Z
      float* po = p.partial_out + bh * (kD + 2);
      po[4 * lane + 0] = acc.x;
      po[4 * lane + 1] = acc.y;
      po[4 * lane + 2] = acc.z;
      po[4 * lane + 3] = acc.w;
      if (lane == 0) {
        po[kD] = ms;
        po[kD + 1] = zs;
      }
    }
    if (p.out != nullptr) {
      const float inv = (p.S_per_tile > 0 && zs > 0.f) ? 1.0f / (zs * (float)p.S_per_tile) : 0.f;
      TK* op = static_cast<TK*>(p.out) + bh * kD + 4 * lane;
      uint2 wv;
      wv.x = uint32_t(Store16<TK>::bits(acc.x * inv)) | (uint32_t(Store16<TK>::bits(acc.y * inv)) << 16);
      wv.y = uint32_t(Store16<TK>::bits(acc.z * inv)) | (uint32_t(Store16<TK>::bits(acc.w * inv)) << 16);
      *reinterpret_cast<uint2*>(op) = wv;
    }
    if (lane == 0) {
      if (p.m_star != nullptr) p.m_star[bh] = ms;
      if (g == 0 && p.vrows != nullptr) p.vrows[b * p.KVH + kv] = (s_redi[0] + s_redi[1]) + (s_redi[2] + s_redi[3]);
    }
  }
}

template <typename TK, int BN>
static cudaError_t launch_one(const FlashParams& p, const FlashMergeParams& mp, int grid, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(flash_decode_kernel<TK, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kFlashSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  flash_decode_kernel<TK, BN><<<grid, kCtaWarps * 32, kFlashSmemBytes, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(p.ncol) * kGH);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, flash_merge_kernel<TK>, mp);
}

cudaError_t launch_flash(const FlashParams& p, const FlashMergeParams& mp, int dtype, int block_n, int grid,
                         cudaStream_t stream) {
  if (dtype == 0) {
    if (block_n == 32) return launch_one<__nv_bfloat16, 32>(p, mp, grid, stream);
    if (block_n == 64) return launch_one<__nv_bfloat16, 64>(p, mp, grid, stream);
    return launch_one<__nv_bfloat16, 256>(p, mp, grid, stream);
  }
  if (block_n == 32) return launch_one<__half, 32>(p, mp, grid, stream);
  if (block_n == 64) return launch_one<__half, 64>(p, mp, grid, stream);
  return launch_one<__half, 256>(p, mp, grid, stream);
}

}  // namespace santa
