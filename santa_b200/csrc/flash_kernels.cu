// flash_kernels.cu -- S2ANTA-Flash decode attention (fixed per-tile sample
// budget) for sm_100a: one persistent launch that streams K once, samples rows
// by systematic resampling inside every tile, gathers the sampled V rows and
// merges tiles with a running log-sum-exp; the last CTA to finish a column
// group folds the per-CTA partials into the output, so there is no second
// launch and no device-side wait.
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
// columns form a column group handled by the eight warps of a CTA, so that the
// eight 256-byte K rows of a token are fetched together.  Work items are
// (column group, tile) pairs; CTA i owns a contiguous balanced range of them.
// Each warp is autonomous: it owns a staging ring fed by its own bulk copies
// and never synchronises with the other warps while streaming.

#include "santa_abi_internal.h"
#include "stream_scores.cuh"

namespace santa {

constexpr int kFlashStages = 3;
constexpr int kEmitCap = 256;  // at most one entry per row of a tile
constexpr size_t kFlashSmemBytes = size_t(kWarpsPerCta) * (kFlashStages * kStageBytes + kEmitCap * 8 + kEmitCap) +
                                   size_t(kWarpsPerCta) * kFlashStages * 8;

template <typename TK, int BN>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 1) flash_decode_kernel(const FlashParams p) {
  constexpr int CPT = BN / kChunkRows;       // chunks per tile
  constexpr int NW = (BN == 256) ? 8 : 4;    // warps of the reference block (fixes the ell order)
  constexpr int NH = NW / 4;                 // 32-row halves per reference pass
  constexpr int NJ = CPT / NH;               // reference passes over the tile

  extern __shared__ __align__(128) unsigned char smem[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  unsigned char* ring_mem = smem + size_t(warp) * (kFlashStages * kStageBytes);
  unsigned char* aux = smem + size_t(kWarpsPerCta) * (kFlashStages * kStageBytes);
  uint2* em_cnt = reinterpret_cast<uint2*>(aux + size_t(warp) * kEmitCap * 8);
  uint8_t* em_row = aux + size_t(kWarpsPerCta) * kEmitCap * 8 + size_t(warp) * kEmitCap;
  uint64_t* bars =
      reinterpret_cast<uint64_t*>(aux + size_t(kWarpsPerCta) * (kEmitCap * 8 + kEmitCap)) + warp * kFlashStages;
  __shared__ int s_last;

  WarpRing<kFlashStages> ring;
  ring.init(ring_mem, bars, lane);
  __syncthreads();

  const TK* __restrict__ Qg = static_cast<const TK*>(p.q);
  const unsigned char* __restrict__ Kg = static_cast<const unsigned char*>(p.K);
  const unsigned char* __restrict__ Vg = static_cast<const unsigned char*>(p.V);
  const size_t row_stride = size_t(p.KVH) * kRowBytes;

  const long long lo = range_lo(blockIdx.x, p.items, gridDim.x);
  const long long hi = range_lo(blockIdx.x + 1, p.items, gridDim.x);
  bool dead = false;  // set when a staged chunk never arrived

  long long it = lo;
  while (it < hi) {
    const int cg = int(it / p.T_c);
    const int t_lo = int(it - (long long)cg * p.T_c);
    const int t_hi = (hi - it < (long long)(p.T_c - t_lo)) ? t_lo + int(hi - it) : p.T_c;
    const int col = cg * kWarpsPerCta + warp;
    const bool active = col < p.ncol;
    const int slot = blockIdx.x + cg;

    if (active) {
      const int b = col / p.KVH;
      const int kv = col - b * p.KVH;
      const int h0 = kv * kGH;
      QRegs Q;
      load_q<TK>(Qg + (size_t(b) * p.H + h0) * kD, p.q_scale, lane, Q);
      const unsigned char* kcol = Kg + (size_t(b) * p.L_storage * p.KVH + kv) * kRowBytes;
      const unsigned char* vcol = Vg + (size_t(b) * p.L_storage * p.KVH + kv) * kRowBytes;

      const int nchunks = (t_hi - t_lo) * CPT;
      const int row_base = t_lo * BN;
      int issued = 0;
      for (; issued < kFlashStages && issued < nchunks; ++issued)
        ring.issue(ring.count + issued, kcol, row_stride, row_base + issued * kChunkRows, p.L_valid, lane);

      float M[kGH], Z[kGH], A[kGH][4];
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        M[g] = -CUDART_INF_F;
        Z[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) A[g][i] = 0.f;
      }
      int vrow_count = 0;

      for (int t = t_lo; t < t_hi; ++t) {
        const int n0 = t * BN;
        const int tile_len = (p.L_valid - n0 < BN) ? (p.L_valid - n0) : BN;

        // ---- stream the tile's chunks, scores stay in registers ----------
        float sc[CPT][kGH];
#pragma unroll
        for (int ch = 0; ch < CPT; ++ch) {
          if (!dead && !ring.wait(ring.count)) {
            dead = true;
            if (lane == 0) atomicExch(p.status, kStatusStageTimeout);
          }
          score_chunk<TK>(ring.stage_ptr(ring.count), Q, lane, sc[ch]);
          __syncwarp();
          if (issued < nchunks && !dead) {
            ring.issue(ring.count + kFlashStages, kcol, row_stride, row_base + issued * kChunkRows, p.L_valid,
                       lane);
            ++issued;
          }
          ++ring.count;
        }

        // ---- tile statistics (reference :223-273) -------------------------
        float m[kGH], ell[kGH];
#pragma unroll
        for (int g = 0; g < kGH; ++g) {
          float v = -CUDART_INF_F;
#pragma unroll
          for (int ch = 0; ch < CPT; ++ch) {
            const bool valid = ch * kChunkRows + lane < tile_len;
            sc[ch][g] = valid ? sc[ch][g] : -CUDART_INF_F;
            v = fmaxf(v, sc[ch][g]);
          }
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
          m[g] = v;
        }
#pragma unroll
        for (int g = 0; g < kGH; ++g) {
#pragma unroll
          for (int ch = 0; ch < CPT; ++ch) sc[ch][g] = __expf(sc[ch][g] - m[g]);  // u, fp32; 0 on masked rows
          // ell in the reference's order: per-thread strided partials, an
          // 8-row tree per reference warp, reference warps summed in order.
          float x[NH];
#pragma unroll
          for (int hf = 0; hf < NH; ++hf) {
            float v = sc[hf][g];
#pragma unroll
            for (int jj = 1; jj < NJ; ++jj) v = __fadd_rn(v, sc[jj * NH + hf][g]);
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
            x[hf] = v;
          }
          float e = __shfl_sync(0xffffffffu, x[0], 0);
#pragma unroll
          for (int w = 1; w < NW; ++w) e = __fadd_rn(e, __shfl_sync(0xffffffffu, x[w / 4], 8 * (w & 3)));
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
#pragma unroll
        for (int ch = 0; ch < CPT; ++ch) {
          const int remain = tile_len - ch * kChunkRows;
          if (remain > 0) {  // warp-uniform
            const int last_lane = remain > 32 ? 31 : remain - 1;
            const bool valid = lane < remain;
            int c[kGH];
#pragma unroll
            for (int g = 0; g < kGH; ++g) {
              const float u16v = Store16<TK>::round(sc[ch][g]);
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
              if (p.dbg_u != nullptr && valid) {
                const size_t o = (size_t(b) * p.H + h0 + g) * p.L_valid + n0 + ch * kChunkRows + lane;
                p.dbg_u[o] = Store16<TK>::bits(sc[ch][g]);
                p.dbg_c[o] = (int16_t)c[g];
              }
            }
            // ---- compaction (reference :314-345): ascending row order -----
            const bool flag = (c[0] + c[1] + c[2] + c[3]) > 0;
            const uint32_t mask = __ballot_sync(0xffffffffu, flag);
            if (flag) {
              const int pos = n_emit + __popc(mask & ((1u << lane) - 1u));
              em_row[pos] = (uint8_t)(ch * kChunkRows + lane);
              em_cnt[pos] = make_uint2((uint32_t)c[0] | ((uint32_t)c[1] << 16), (uint32_t)c[2] | ((uint32_t)c[3] << 16));
              if (p.rowmask != nullptr)
                p.rowmask[(size_t(b) * p.KVH + kv) * p.L_valid + n0 + ch * kChunkRows + lane] = 1;
            }
            n_emit += __popc(mask);
          }
        }
        vrow_count += n_emit;
        if (p.dbg_m != nullptr && lane < kGH) {
          // select without dynamic register indexing
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

        // ---- sparse sum of c*V (reference :347-379), 8 rows in flight ----
        float o[kGH][4];
#pragma unroll
        for (int g = 0; g < kGH; ++g)
#pragma unroll
          for (int i = 0; i < 4; ++i) o[g][i] = 0.f;
        for (int i0 = 0; i0 < n_emit; i0 += 8) {
          uint2 vv[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (i0 + k < n_emit) {
              const int n = n0 + em_row[i0 + k];
              vv[k] = __ldg(reinterpret_cast<const uint2*>(vcol + size_t(n) * row_stride) + lane);
            }
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (i0 + k < n_emit) {
              const uint2 cw = em_cnt[i0 + k];
              const float2 va = Store16<TK>::unpack(vv[k].x), vb = Store16<TK>::unpack(vv[k].y);
              const int cg4[kGH] = {int(cw.x & 0xffffu), int(cw.x >> 16), int(cw.y & 0xffffu), int(cw.y >> 16)};
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
      }  // tiles

      // ---- publish this warp's partial -----------------------------------
      float* ps = p.partials + (size_t(slot) * kWarpsPerCta + warp) * (kGH * kPartialStride);
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        reinterpret_cast<float4*>(ps + g * kPartialStride)[lane] = make_float4(A[g][0], A[g][1], A[g][2], A[g][3]);
        if (lane == 0) {
          ps[g * kPartialStride + kD] = M[g];
          ps[g * kPartialStride + kD + 1] = Z[g];
        }
      }
      if (lane == 0) p.partial_vrows[slot * kWarpsPerCta + warp] = vrow_count;
    }  // active

    // ---- last CTA of the column group merges -------------------------------
    __threadfence();
    __syncthreads();
    const int cta_first = cta_of_item((long long)cg * p.T_c, p.items, gridDim.x);
    const int cta_last = cta_of_item((long long)(cg + 1) * p.T_c - 1, p.items, gridDim.x);
    if (threadIdx.x == 0) {
      const unsigned expected = unsigned(cta_last - cta_first + 1);
      const unsigned old = atomicAdd(&p.tickets[cg], 1u);
      s_last = (old == expected - 1u);
      if (s_last) p.tickets[cg] = 0u;  // leave the workspace ready for the next call
    }
    __syncthreads();
    if (s_last && active) {
      __threadfence();
      const int b = col / p.KVH;
      const int kv = col - b * p.KVH;
      int vr = 0;
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        const int h = kv * kGH + g;
        float ms = -CUDART_INF_F;
        for (int c = cta_first; c <= cta_last; ++c) {
          const float* ps = p.partials + ((size_t(c + cg) * kWarpsPerCta + warp) * kGH + g) * kPartialStride;
          ms = fmaxf(ms, __ldcg(ps + kD));
        }
        float zs = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = cta_first; c <= cta_last; ++c) {
          const float* ps = p.partials + ((size_t(c + cg) * kWarpsPerCta + warp) * kGH + g) * kPartialStride;
          const float e = __expf(__ldcg(ps + kD) - ms);
          const float4 a = __ldcg(reinterpret_cast<const float4*>(ps) + lane);
          zs += e * __ldcg(ps + kD + 1);
          acc.x += e * a.x;
          acc.y += e * a.y;
          acc.z += e * a.z;
          acc.w += e * a.w;
        }
        const size_t bh = size_t(b) * p.H + h;
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
          uint2 w;
          w.x = uint32_t(Store16<TK>::bits(acc.x * inv)) | (uint32_t(Store16<TK>::bits(acc.y * inv)) << 16);
          w.y = uint32_t(Store16<TK>::bits(acc.z * inv)) | (uint32_t(Store16<TK>::bits(acc.w * inv)) << 16);
          *reinterpret_cast<uint2*>(op) = w;
        }
        if (lane == 0 && p.m_star != nullptr) p.m_star[bh] = ms;
      }
      if (p.vrows != nullptr) {
        for (int c = cta_first + lane; c <= cta_last; c += 32) vr += __ldcg(p.partial_vrows + (c + cg) * kWarpsPerCta + warp);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) vr += __shfl_xor_sync(0xffffffffu, vr, off);
        if (lane == 0) p.vrows[b * p.KVH + kv] = vr;
      }
    }
    __syncthreads();  // s_last is reused by the next segment
    it += (t_hi - t_lo);
  }
}

template <typename TK, int BN>
static cudaError_t launch_one(const FlashParams& p, int grid, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(flash_decode_kernel<TK, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kFlashSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  flash_decode_kernel<TK, BN><<<grid, kWarpsPerCta * 32, kFlashSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_flash(const FlashParams& p, int dtype, int block_n, int grid, cudaStream_t stream) {
  if (dtype == 0) {
    if (block_n == 32) return launch_one<__nv_bfloat16, 32>(p, grid, stream);
    if (block_n == 64) return launch_one<__nv_bfloat16, 64>(p, grid, stream);
    return launch_one<__nv_bfloat16, 256>(p, grid, stream);
  }
  if (block_n == 32) return launch_one<__half, 32>(p, grid, stream);
  if (block_n == 64) return launch_one<__half, 64>(p, grid, stream);
  return launch_one<__half, 256>(p, grid, stream);
}

}  // namespace santa
