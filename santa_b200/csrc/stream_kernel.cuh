// stream_kernel.cuh -- the persistent K-streaming kernel behind Flash decode and
// Prop's first pass (vec path).  One CTA per SM, sixteen warps, two per column
// slot:
//   * the SCORE warp of a slot owns a TMA staging ring, streams its column's K
//     rows and writes the four heads' scores of a tile into one of two score
//     buffers (stream_scores.cuh);
//   * the SAMPLER warp of the slot turns a finished score buffer into tile
//     statistics and -- Flash -- sampled counts, the sparse sum of V rows and a
//     running log-sum-exp state, or -- Prop pass 1 -- the stashed tile-local
//     weights (sampler.cuh).
// The two warps hand buffers over through a full/empty pair of mbarriers per
// buffer, so K keeps streaming while the previous tile is being sampled.  No
// warp ever synchronises with another slot.  All hot loops are rolled so that
// the instruction footprint stays small; every wait is bounded and reports
// through the status word instead of hanging.
//
// Included by flash_kernels.cu (compiled with --use_fast_math) and
// prop_kernels.cu (compiled without); each instantiates only its own mode.
#pragma once

#include <type_traits>

#include "sampler.cuh"
#include "stream_scores.cuh"

namespace santa {

constexpr int kModeFlash = 0;
constexpr int kModePropPass1 = 1;

constexpr int kStreamStages = 2;
constexpr int kMaxTileRows = 256;
constexpr int kScoreBytes = kMaxTileRows * kGH * 4;  // one score buffer: scores, then u, then the emit list
// Dynamic shared memory, from a 1024-byte aligned base (the swizzled staging of the tensor-core score
// path needs it): the staging rings of the eight slots, then per slot two score buffers and the
// exchange buffer of the exact score path, then the mbarriers.
constexpr int kSlotRing = kStreamStages * kStageBytes;
constexpr int kSlotRest = 2 * kScoreBytes + kRedFloats * 4;
constexpr int kSlotBars = kStreamStages + 4;  // ring + full[2] + empty[2]
constexpr int kCtaWarps = 2 * kGroupWarps;
constexpr size_t kStreamSmemBytes =
    1024 + size_t(kGroupWarps) * (kSlotRing + kSlotRest) + size_t(kGroupWarps) * kSlotBars * 8;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// RAGGED: per-sequence lengths from p.seq_lens (a compile-time switch, so that the uniform kernel
// carries none of the look-up state).
// MMA: scores from the tensor cores (stream_scores.cuh, opt-in): p.tmK then describes swizzled
// half-row boxes.  Everything after the scores is the same code.
template <typename TK, int BN, int MODE, bool RAGGED = false, bool MMA = false>
__global__ void __launch_bounds__(kCtaWarps * 32, 1) stream_kernel(const __grid_constant__ StreamParams p) {
  constexpr int NW = (BN == 256) ? 8 : 4;  // warps of the reference block (fixes the ell order)

  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int cta_warp = threadIdx.x >> 5;
  const int slot = cta_warp & (kGroupWarps - 1);
  const bool is_sampler = cta_warp >= kGroupWarps;
  const int lane = threadIdx.x & 31;

  unsigned char* sbase = smem + size_t(slot) * kSlotRing;
  unsigned char* srest = smem + size_t(kGroupWarps) * kSlotRing + size_t(slot) * kSlotRest;
  float* scorebufs = reinterpret_cast<float*>(srest);
  float* red = reinterpret_cast<float*>(srest + 2 * kScoreBytes);
  uint64_t* bars =
      reinterpret_cast<uint64_t*>(smem + size_t(kGroupWarps) * (kSlotRing + kSlotRest)) + slot * kSlotBars;
  const uint32_t bar_full = smem_u32(bars + kStreamStages);       // [2]
  const uint32_t bar_empty = smem_u32(bars + kStreamStages + 2);  // [2]

  if (threadIdx.x == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tmK) : "memory");
  __shared__ int s_start[kMaxRaggedSeqs + 1];
  constexpr bool ragged = RAGGED;
  WarpRing<kStreamStages> ring;
  if (!is_sampler) {
    ring.init(sbase, bars, lane);
    if (lane == 0) {
      mbar_init(bar_full, 1);
      mbar_init(bar_full + 8, 1);
      mbar_init(bar_empty, 1);
      mbar_init(bar_empty + 8, 1);
      mbar_fence_init();
    }
  }
  // The kernel is launched as a programmatic dependent of whatever precedes it on the stream (the
  // previous decode call's merge, the RoPE/append launch): the set-up above overlaps that kernel's
  // tail; nothing below may run before it has completed -- it produced q, the new K/V rows and the
  // lengths, and it still reads the workspace this kernel is about to overwrite.
  cudaGridDependencySynchronize();
  if (ragged && cta_warp == kCtaWarps - 1)
    build_item_starts(p.seq_lens, p.nseq, p.L_valid, BN, p.KVH / p.ws.gw, s_start, lane);
  __syncthreads();

  const TK* __restrict__ Qg = static_cast<const TK*>(p.q);
  const unsigned char* __restrict__ Vg = static_cast<const unsigned char*>(p.V);
  const size_t row_stride = size_t(p.KVH) * kRowBytes;
  WorkSplit split = p.ws;
  if (ragged) {  // the item total is only known here; never more groups than items
    split.items = s_start[p.nseq];
    split.nvg = (split.items < (long long)split.nvg) ? int(split.items) : split.nvg;
  }
  const WarpWork ww = warp_work(split, blockIdx.x, gridDim.x, slot);

  bool dead = false;     // set when a wait ran out; the status word then says why
  uint32_t handoff = 0;  // tiles handed over so far on this slot (selects buffer and parity)

  long long it = ww.lo;
  while (it < ww.hi) {
    // item -> (column group, first tile); L_b / T_b are the column's length and tile count
    int cg, t_lo, b, kv, L_b, T_b;
    bool active;
    if (!ragged) {
      L_b = p.L_valid;
      T_b = p.ws.T_c;
      cg = int(it / T_b);
      t_lo = int(it - (long long)cg * T_b);
      const int col = cg * p.ws.gw + ww.col_in_group;
      active = col < p.ws.ncol;
      b = active ? col / p.KVH : 0;
      kv = col - b * p.KVH;
    } else {
      b = seq_of_item(s_start, p.nseq, int(it));
      L_b = ragged_len(p.seq_lens, b, p.L_valid);
      T_b = (L_b + BN - 1) / BN;
      const int rel = int(it) - s_start[b];
      const int cgs = rel / T_b;
      t_lo = rel - cgs * T_b;
      cg = b * (p.KVH / p.ws.gw) + cgs;
      kv = cgs * p.ws.gw + ww.col_in_group;
      active = true;
    }
    const int t_hi = (ww.hi - it < (long long)(T_b - t_lo)) ? t_lo + int(ww.hi - it) : T_b;
    const int h0 = kv * kGH;

    if (active && !is_sampler) {
      // =========================== SCORE warp ===============================
      const int row_base = t_lo * BN;
      const int row_end = (t_hi * BN < L_b) ? t_hi * BN : L_b;
      const int npieces = (row_end - row_base + kStageRows - 1) / kStageRows;
      int issued = 0;  // the K pieces do not depend on q: start them before fetching q
      for (; issued < kStreamStages && issued < npieces; ++issued)
        ring.template issue<MMA>(ring.count + issued, &p.tmK, b, kv, row_base + issued * kStageRows, lane);
      typename std::conditional<MMA, QFrag, QRegs>::type Q;
      if constexpr (MMA)
        load_q_frag<TK>(Qg + (size_t(b) * p.H + h0) * kD, p.q_scale, lane, Q);
      else
        load_q<TK>(Qg + (size_t(b) * p.H + h0) * kD, p.q_scale, lane, Q);

#pragma unroll 1
      for (int t = t_lo; t < t_hi; ++t, ++handoff) {
        const int n0 = t * BN;
        const int tile_len = (L_b - n0 < BN) ? (L_b - n0) : BN;
        const uint32_t buf = handoff & 1u;
        float* scorebuf = scorebufs + buf * (kScoreBytes / 4);
        // wait until the sampler has released this buffer (passes at once the first two times)
        if (!dead && !mbar_wait_bounded(bar_empty + 8 * buf, ((handoff >> 1) & 1u) ^ 1u, 128)) {
          dead = true;
          if (lane == 0) atomicExch(p.status, kStatusHandoffTimeout);
        }
        int npc = (tile_len + kStageRows - 1) / kStageRows;
        if (!SANTA_IN_RANGE(npc * kStageRows - 1, kMaxTileRows, p.status)) npc = 0;  // a piece past the score buffer
#pragma unroll 1
        for (int pc = 0; pc < npc; ++pc) {
          if (!dead && !ring.wait(ring.count)) {
            dead = true;
            if (lane == 0) atomicExch(p.status, kStatusStageTimeout);
          }
          const unsigned char* st = ring.stage_ptr(ring.count);
          if constexpr (MMA) {
            score_rows16_mma<TK>(smem_u32(st), 0, Q, scorebuf + (pc * kStageRows) * kGH, lane);
            score_rows16_mma<TK>(smem_u32(st), 1, Q, scorebuf + (pc * kStageRows + 16) * kGH, lane);
          } else {
            score_rows16<TK>(st, Q, red, scorebuf + (pc * kStageRows) * kGH, lane);
            score_rows16<TK>(st + 16 * kRowBytes, Q, red, scorebuf + (pc * kStageRows + 16) * kGH, lane);
          }
          if (issued < npieces && !dead) {
            ring.template issue<MMA>(ring.count + kStreamStages, &p.tmK, b, kv, row_base + issued * kStageRows, lane);
            ++issued;
          }
          ++ring.count;
        }
        __syncwarp();
        if constexpr (MMA) {
          // With the scores coming from the tensor cores this warp has time to spare and the sampler
          // warp is the one that bounds a slot: the tile statistics (max, exp, ell) move over here.
          // m and ell travel in the exchange buffer, which the tensor-core path does not use otherwise.
          float ms[kGH], es[kGH];
          tile_stats<NW>(reinterpret_cast<float4*>(scorebuf), tile_len, lane, ms, es);
          if (lane < kGH) {
            float mv = ms[0], ev = es[0];
#pragma unroll
            for (int g = 1; g < kGH; ++g) {
              mv = (lane == g) ? ms[g] : mv;
              ev = (lane == g) ? es[g] : ev;
            }
            red[buf * 2 * kGH + lane] = mv;
            red[buf * 2 * kGH + kGH + lane] = ev;
          }
          __syncwarp();
        }
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
        const int tile_len = (L_b - n0 < BN) ? (L_b - n0) : BN;
        const uint32_t buf = handoff & 1u;
        float4* sb = reinterpret_cast<float4*>(scorebufs + buf * (kScoreBytes / 4));
        if (!dead && !mbar_wait_bounded(bar_full + 8 * buf, (handoff >> 1) & 1u, 256)) {
          dead = true;
          if (lane == 0) atomicExch(p.status, kStatusHandoffTimeout);
        }

        float m[kGH], ell[kGH];
        if constexpr (MMA) {  // computed by the score warp (see there)
#pragma unroll
          for (int g = 0; g < kGH; ++g) {
            m[g] = red[buf * 2 * kGH + g];
            ell[g] = red[buf * 2 * kGH + kGH + g];
          }
        } else {
          tile_stats<NW>(sb, tile_len, lane, m, ell);
        }
        const size_t bh0 = size_t(b) * p.H + h0;

        if (MODE == kModePropPass1) {
          // tile statistics and the stash of rounded weights for the second pass
          // (santa_fused_proportional_tile_budgets/santa_cuda_kernel.cu:404-440)
          const int nch = (tile_len + kChunkRows - 1) / kChunkRows;
#pragma unroll 1
          for (int ch = 0; ch < nch; ++ch) {
            const int r = ch * kChunkRows + lane;
            if (r < tile_len && SANTA_IN_RANGE(n0 + r, p.len_stride, p.status)) {
              const float4 u = sb[r];
              const uint32_t w01 = uint32_t(Store16<TK>::bits(u.x)) | (uint32_t(Store16<TK>::bits(u.y)) << 16);
              const uint32_t w23 = uint32_t(Store16<TK>::bits(u.z)) | (uint32_t(Store16<TK>::bits(u.w)) << 16);
              // one 8-byte word per row: the four heads of the group side by side
              reinterpret_cast<uint2*>(p.stash)[(size_t(b) * p.KVH + kv) * p.len_stride + n0 + r] =
                  make_uint2(w01, w23);
              if (p.dbg_u != nullptr) {
                uint16_t* sp = p.dbg_u + bh0 * p.len_stride + n0 + r;
                sp[0] = uint16_t(w01 & 0xffffu);
                sp[size_t(p.len_stride)] = uint16_t(w01 >> 16);
                sp[2 * size_t(p.len_stride)] = uint16_t(w23 & 0xffffu);
                sp[3 * size_t(p.len_stride)] = uint16_t(w23 >> 16);
              }
            }
          }
          __syncwarp();
        }
        // Flash budget rule (santa_cuda.cpp:202-208); a ragged batch applies it to each length
        const int spt = (RAGGED && MODE == kModeFlash) ? (p.S_total > 0 ? (p.S_total / T_b > 1 ? p.S_total / T_b : 1) : 0)
                                                       : p.S_per_tile;
        float invdel[kGH];
#pragma unroll
        for (int g = 0; g < kGH; ++g)
          invdel[g] = (spt > 0 && ell[g] > 1e-20f) ? ((float)spt / ell[g]) : 0.0f;
        if (p.m_tiles != nullptr && lane < kGH) {
          float mv = m[0], ev = ell[0], iv = invdel[0];
#pragma unroll
          for (int g = 1; g < kGH; ++g) {
            mv = (lane == g) ? m[g] : mv;
            ev = (lane == g) ? ell[g] : ev;
            iv = (lane == g) ? invdel[g] : iv;
          }
          const size_t o = (bh0 + lane) * p.tile_stride + t;
          if (SANTA_IN_RANGE(t, p.tile_stride, p.status) && SANTA_IN_RANGE(bh0 + lane, size_t(p.nseq) * p.H, p.status)) {
            p.m_tiles[o] = mv;
            p.ell_tiles[o] = ev;
            if (p.dbg_invdel != nullptr) p.dbg_invdel[o] = iv;
          }
        }

        if (MODE == kModeFlash) {
          // systematic counts, compaction, sparse V sum, running merge
          // the four heads' offsets are computed on lanes 0..3 in parallel and broadcast
          const float a0_lane = u01_from_seed(p.seed, (p.batch_offset + b) * p.H + h0 + (lane & 3), p.tile_offset + t);
          float a0[kGH];
#pragma unroll
          for (int g = 0; g < kGH; ++g) a0[g] = __shfl_sync(0xffffffffu, a0_lane, g);
          RowTrace tr;
          tr.status = p.status;
          tr.rows_left = p.L_storage - n0;
          tr.vrow0 = vcol + size_t(n0) * row_stride;
          tr.row_stride = row_stride;
          tr.head_stride = size_t(p.len_stride);
          tr.u16 = p.dbg_u ? p.dbg_u + bh0 * p.len_stride + n0 : nullptr;
          tr.counts = p.dbg_c ? p.dbg_c + bh0 * p.len_stride + n0 : nullptr;
          tr.rowmask = p.rowmask ? p.rowmask + (size_t(b) * p.KVH + kv) * p.len_stride + n0 : nullptr;
          const int n_emit = tile_counts<TK>(sb, tile_len, lane, invdel, a0, tr);
          vrow_count += n_emit;

          float o[kGH][4];
#pragma unroll
          for (int g = 0; g < kGH; ++g)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[g][i] = 0.f;
          gather_rows<TK>(sb, n_emit, vcol + size_t(n0) * row_stride, row_stride, lane, o, p.status, tr.rows_left);

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
        }
        if (lane == 0) mbar_arrive(bar_empty + 8 * buf);  // every lane's reads were ordered by a __syncwarp
      }  // tiles

      if (MODE == kModeFlash) {
        // ---- publish this column's partial -------------------------------
        const size_t pslot = size_t(ww.vg + cg) * p.ws.gw + ww.col_in_group;
        float* ps = p.partials + pslot * (kGH * kPartialStride);
        if (SANTA_IN_RANGE(pslot, p.partial_slots, p.status)) {
#pragma unroll
        for (int g = 0; g < kGH; ++g) {
          reinterpret_cast<float4*>(ps + g * kPartialStride)[lane] = make_float4(A[g][0], A[g][1], A[g][2], A[g][3]);
          if (lane == 0) {
            ps[g * kPartialStride + kD] = M[g];
            ps[g * kPartialStride + kD + 1] = Z[g];
          }
        }
        if (lane == 0) p.partial_vrows[pslot] = vrow_count;
        }
      }
    } else {
      handoff += uint32_t(t_hi - t_lo);
    }
    it += (t_hi - t_lo);
  }
}

}  // namespace santa
