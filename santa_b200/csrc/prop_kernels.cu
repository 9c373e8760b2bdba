// prop_kernels.cu -- S2ANTA-Prop decode attention (per-head sample budget split
// over tiles in proportion to their softmax mass) for sm_100a.  Four launches on
// one stream, each a programmatic dependent of the one before:
//   pass 1   tile statistics m_t, ell_t and the stash of rounded tile-local
//            weights u = exp(s - m_t): the persistent TMA-streaming kernel of
//            stream_kernel.cuh when block_n == 256, else a tensor-core kernel;
//   budgets  one CTA per head: m*, Z, largest-remainder apportionment of S over
//            the tiles, per-tile step S_t/ell_t and offset;
//   pass 2   systematic counts from the stash, row compaction, sparse V sum, one
//            partial per warp;
//   merge    sums the partials in a fixed order, scales by 1/S, casts.
//
// Replaces the reference's santa_fused_proportional_tile_budgets/
// santa_cuda_kernel.cu kernels: pass1_tiles_kernel_vec_gqa_gh4_d128_bn256
// (:278-441), pass1_tiles_kernel_wmma_gqa_x (:87-267), tile_budgets_kernel
// (:577-726), pass2_grouped_tile_fused_atomic_kernel_x (:734-864),
// cast_scale_out_kernel (:976-985) and reduce_vrows_kernel (:869-899).
//
// Compiled WITHOUT --use_fast_math, like the reference's Prop extension (its
// setup.py:39-42): divisions here are IEEE.
//
// Determinism.  The reference sums Z with shared-memory atomics and the output
// with global atomics, so it is not run-to-run reproducible.  This file fixes
// one order for each (per-thread partials added thread 0..127 for Z; tiles in
// ascending order per warp and warps in ascending order for the output).

#include <cooperative_groups.h>

#include "stream_kernel.cuh"

namespace santa {

// ------------------------------------------------------------------ pass 1, tensor-core path
// One CTA per (tile, kv-head), one warp per 16 K rows; GH <= 8 query heads per kv-head, any head
// dimension D that is a multiple of 16.  The scores are formed exactly like the reference's
// 16x16x16 WMMA steps (santa_cuda_kernel.cu:126-188: q*scale rounded to the storage type, fp32
// accumulation over 16-wide k steps in ascending order); a 16x16x16 WMMA step is two m16n8k16 MMAs
// on the two 8-column halves, with the heads in the first GH of the 16 rows.  Tile statistics
// follow santa_cuda_kernel.cu:190-265: per warp and head a sequential 16-term sum of u, warps
// added in ascending order.  The stash is [kv-head][row][GH] 16-bit.
template <typename TK>
__global__ void prop_pass1_mma_kernel(const TK* __restrict__ Q, const TK* __restrict__ K, int H, int KVH, int GH,
                                      int D, int L, int bn, int T_c, float q_scale, float* __restrict__ m_tiles,
                                      float* __restrict__ ell_tiles, uint16_t* __restrict__ stash,
                                      uint16_t* __restrict__ dbg_u) {
  extern __shared__ float smf[];
  const int t = blockIdx.x, kv = blockIdx.y;
  const int NWARP = blockDim.x >> 5;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = t * bn;
  float* Ct = smf + w * 256;                 // [16 heads][16 rows of K]
  float* rowMax = smf + NWARP * 256;         // [16][NWARP]
  float* rowEll = rowMax + 16 * NWARP;       // [16][NWARP]
  float* mRow = rowEll + 16 * NWARP;         // [16]

  const int r0 = lane >> 2, c0 = 2 * (lane & 3);
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  for (int k0 = 0; k0 < D; k0 += 16) {
    uint32_t a[4] = {0u, 0u, 0u, 0u};
    if (r0 < GH) {  // rows GH..15 are padding (GH <= 8: the rows r0+8 are never used)
      const TK* qp = Q + (size_t(kv) * GH + r0) * D + k0 + c0;
      const float2 lo = Store16<TK>::unpack(*reinterpret_cast<const uint32_t*>(qp));
      const float2 hi = Store16<TK>::unpack(*reinterpret_cast<const uint32_t*>(qp + 8));
      a[0] = uint32_t(Store16<TK>::bits(lo.x * q_scale)) | (uint32_t(Store16<TK>::bits(lo.y * q_scale)) << 16);
      a[2] = uint32_t(Store16<TK>::bits(hi.x * q_scale)) | (uint32_t(Store16<TK>::bits(hi.y * q_scale)) << 16);
    }
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const int n = n0 + 16 * w + 8 * nb + r0;
      uint32_t b[2] = {0u, 0u};
      if (n < L) {
        const TK* kp = K + (size_t(n) * KVH + kv) * D + k0 + c0;
        b[0] = *reinterpret_cast<const uint32_t*>(kp);
        b[1] = *reinterpret_cast<const uint32_t*>(kp + 8);
      }
      MmaOp<TK>::mma(acc[nb], a, b);
    }
  }
#pragma unroll
  for (int nb = 0; nb < 2; ++nb) {
    Ct[r0 * 16 + 8 * nb + c0] = acc[nb][0];
    Ct[r0 * 16 + 8 * nb + c0 + 1] = acc[nb][1];
    Ct[(r0 + 8) * 16 + 8 * nb + c0] = acc[nb][2];
    Ct[(r0 + 8) * 16 + 8 * nb + c0 + 1] = acc[nb][3];
  }
  __syncthreads();
  if (lane < 16) {
    float mp = -CUDART_INF_F;
    if (lane < GH)
      for (int j = 0; j < 16; ++j)
        if (n0 + 16 * w + j < L) mp = fmaxf(mp, Ct[lane * 16 + j]);
    rowMax[lane * NWARP + w] = mp;
  }
  __syncthreads();
  if (w == 0 && lane < 16) {
    float mv = -CUDART_INF_F;
    for (int ww = 0; ww < NWARP; ++ww) mv = fmaxf(mv, rowMax[lane * NWARP + ww]);
    mRow[lane] = (lane < GH) ? mv : -CUDART_INF_F;
  }
  __syncthreads();
  if (lane < 16) {
    float ep = 0.f;
    if (lane < GH) {
      const float mr = mRow[lane];
      const int h = kv * GH + lane;
      for (int j = 0; j < 16; ++j) {
        const int n = n0 + 16 * w + j;
        if (n < L) {
          const float u = __expf(Ct[lane * 16 + j] - mr);
          ep = __fadd_rn(ep, u);
          const uint16_t ub = Store16<TK>::bits(u);
          stash[(size_t(kv) * L + n) * GH + lane] = ub;  // [kv][row][head of the group]
          if (dbg_u != nullptr) dbg_u[size_t(h) * L + n] = ub;
        }
      }
    }
    rowEll[lane * NWARP + w] = ep;
  }
  __syncthreads();
  if (w == 0 && lane < GH) {
    float e = 0.f;
    for (int ww = 0; ww < NWARP; ++ww) e = __fadd_rn(e, rowEll[lane * NWARP + ww]);
    const int h = kv * GH + lane;
    m_tiles[size_t(h) * T_c + t] = mRow[lane];
    ell_tiles[size_t(h) * T_c + t] = e;
  }
}

// ------------------------------------------------------------------ budgets
// The bitonic network of the budgets kernel on up to 256 keys, run by ONE warp in registers instead of
// by the CTA in shared memory with a barrier per stage (36 stages for 256 keys).  Lane l holds the
// elements l*R .. l*R+R-1 of the N = 32*R positions (R = 1 also serves N < 32).  Same comparators in
// the same order as the shared-memory form below: pair (i, i^j) with i < i^j, direction from bit k of
// i, swap iff (a_i > a_j) == up; positions >= T_c are virtual -- they read as (-inf, -1) and whatever
// a comparator would have put there is dropped -- so they are reset after every stage.
template <int R>
__device__ __forceinline__ void warp_bitonic(float (&f)[R], int (&ix)[R], int N, int T_c, int lane) {
#pragma unroll 1
  for (int k = 2; k <= N; k <<= 1) {
    // stages whose partner sits in another lane (lane ^ (j / R), same register): rolled
#pragma unroll 1
    for (int j = k >> 1; j >= R; j >>= 1) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = lane * R + r;
        const float of = __shfl_xor_sync(0xffffffffu, f[r], j / R);
        const int oi = __shfl_xor_sync(0xffffffffu, ix[r], j / R);
        const bool lower = (i & j) == 0;
        const bool up = ((lower ? i : (i ^ j)) & k) != 0;
        const float a_low = lower ? f[r] : of, a_high = lower ? of : f[r];
        if ((a_low > a_high) == up) {
          f[r] = of;
          ix[r] = oi;
        }
        if (i >= T_c) {
          f[r] = -CUDART_INF_F;
          ix[r] = -1;
        }
      }
    }
    // stages whose partner is register r ^ j of this lane: j is a compile-time constant
#pragma unroll
    for (int j = R / 2; j > 0; j >>= 1) {
      if (j < k) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if ((r & j) == 0) {
            const int i = lane * R + r;
            const bool up = (i & k) != 0;
            if ((f[r] > f[r | j]) == up) {
              const float tf = f[r];
              f[r] = f[r | j];
              f[r | j] = tf;
              const int ti = ix[r];
              ix[r] = ix[r | j];
              ix[r | j] = ti;
            }
            if (i >= T_c) {
              f[r] = -CUDART_INF_F;
              ix[r] = -1;
            }
            if ((i | j) >= T_c) {
              f[r | j] = -CUDART_INF_F;
              ix[r | j] = -1;
            }
          }
        }
      }
    }
  }
}

// Sort the keys in `frac` (shared memory, T_c of them) with the network above and give the first `rem`
// positions' tiles one more sample each.
template <int R>
__device__ __forceinline__ void warp_sort_and_top_up(const float* frac, int* bud, int N, int T_c, int rem, int lane) {
  float f[R];
  int ix[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane * R + r;
    f[r] = (i < T_c) ? frac[i] : -CUDART_INF_F;
    ix[r] = (i < T_c) ? i : -1;
  }
  warp_bitonic<R>(f, ix, N, T_c, lane);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane * R + r;
    if (i < rem && ix[r] >= 0) bud[ix[r]] += 1;  // the entries are distinct tiles
  }
}

// One CTA of 128 threads per head; restates tile_budgets_kernel
// (santa_cuda_kernel.cu:577-726) step by step: m* = max_t m_t,
// W_t = __expf(m_t - m*) * ell_t, Z, q_t = S * (W_t / Z), floor, fractional part
// plus 1e-7*u01 jitter, the bitonic network (descending, virtual -inf padding
// that is never stored), +1 for the first S - sum(floor) entries,
// invdelta_t = S_t / ell_t, a0_t = u01(seed, h, t).
// flags bit0: jitter added with one fma; bit1: thread partials of Z with fma.
// Ragged batches: blockIdx.y is the sequence, its tile count comes from seq_lens and its rows of
// the tables are tile_stride apart; every sequence uses the head index h in the random stream,
// exactly like one call per sequence.
__global__ void __launch_bounds__(128) prop_budgets_kernel(const float* __restrict__ m_tiles_all,
                                                           const float* __restrict__ ell_tiles_all, int T_uniform,
                                                           const int* __restrict__ seq_lens, int max_len, int bn,
                                                           int tile_stride, int S, uint64_t seed, int flags,
                                                           float* __restrict__ m_star_all,
                                                           int* __restrict__ S_tiles_all,
                                                           float* __restrict__ invdelta_all,
                                                           float* __restrict__ a0_tile_all) {
  cudaGridDependencySynchronize();
  extern __shared__ unsigned char smraw[];
  const int T_c = seq_lens ? (ragged_len(seq_lens, blockIdx.y, max_len) + bn - 1) / bn : T_uniform;
  // per-tile tables of this head, all in shared memory: sort keys, sort payload, ell, budgets, offsets
  float* frac = reinterpret_cast<float*>(smraw);
  int* idx = reinterpret_cast<int*>(frac + tile_stride);
  float* ells = reinterpret_cast<float*>(idx + tile_stride);
  int* bud = reinterpret_cast<int*>(ells + tile_stride);
  float* offs = reinterpret_cast<float*>(bud + tile_stride);
  __shared__ float s_part[128];
  __shared__ float s_bcast;
  __shared__ float s_wmax[4];
  __shared__ int s_wsum[4];
  const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wq = tid >> 5;
  const size_t row = (size_t(blockIdx.y) * gridDim.x + h) * tile_stride;
  const float* mt = m_tiles_all + row;
  const float* el = ell_tiles_all + row;
  int* S_tiles = S_tiles_all + row;
  float* invdelta = invdelta_all + row;
  float* a0_tile = a0_tile_all + row;
  float* m_star = m_star_all ? m_star_all + size_t(blockIdx.y) * gridDim.x : nullptr;

  // m* (a maximum is the same in any order); ell and the random offsets ride along
  float lm = -3.402823466e+38f;
  for (int t = tid; t < T_c; t += 128) {
    const float v = __ldcg(mt + t);
    ells[t] = __ldcg(el + t);
    frac[t] = v;
    lm = fmaxf(lm, v);
    offs[t] = u01_from_seed(seed, h, t);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) lm = fmaxf(lm, __shfl_xor_sync(0xffffffffu, lm, off));
  if (lane == 0) s_wmax[wq] = lm;
  __syncthreads();
  const float mstar = fmaxf(fmaxf(s_wmax[0], s_wmax[1]), fmaxf(s_wmax[2], s_wmax[3]));
  if (tid == 0 && m_star != nullptr) m_star[h] = mstar;

  // W_t and Z: per-thread partials in tile order, then thread 0 adds the 128 partials in order
  float zl = 0.f;
  for (int t = tid; t < T_c; t += 128) {
    const float e = __expf(frac[t] - mstar);
    const float W = __fmul_rn(e, ells[t]);
    frac[t] = W;
    zl = (flags & 2) ? __fmaf_rn(e, ells[t], zl) : __fadd_rn(zl, W);
  }
  s_part[tid] = zl;
  __syncthreads();
  if (tid == 0) {
    float z = 0.f;
    for (int i = 0; i < 128; ++i) z = __fadd_rn(z, s_part[i]);
    s_bcast = z;
  }
  __syncthreads();
  const float Z = s_bcast;

  if (S <= 0 || !(Z > 0.0f)) {
    for (int t = tid; t < T_c; t += 128) {
      S_tiles[t] = 0;
      invdelta[t] = 0.0f;
      a0_tile[t] = offs[t];
    }
    return;
  }

  int bl = 0;
  for (int t = tid; t < T_c; t += 128) {
    const float q = __fmul_rn((float)S, __fdiv_rn(frac[t], Z));
    const int b = (int)floorf(q);
    bud[t] = b;
    bl += b;
    const float ft = __fsub_rn(q, (float)b);
    const float u = offs[t];
    frac[t] = (flags & 1) ? __fmaf_rn(1.0e-7f, u, ft) : __fadd_rn(ft, __fmul_rn(1.0e-7f, u));
    idx[t] = t;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) bl += __shfl_xor_sync(0xffffffffu, bl, off);
  if (lane == 0) s_wsum[wq] = bl;
  __syncthreads();
  int rem = S - ((s_wsum[0] + s_wsum[1]) + (s_wsum[2] + s_wsum[3]));
  rem = rem < 0 ? 0 : rem;
  rem = rem > T_c ? T_c : rem;

  int N = 1;
  while (N < T_c) N <<= 1;
  if (N <= 256) {  // one warp sorts in registers: no barrier per stage
    if (wq == 0) {
      if (N <= 32)
        warp_sort_and_top_up<1>(frac, bud, N, T_c, rem, lane);
      else if (N == 64)
        warp_sort_and_top_up<2>(frac, bud, N, T_c, rem, lane);
      else if (N == 128)
        warp_sort_and_top_up<4>(frac, bud, N, T_c, rem, lane);
      else
        warp_sort_and_top_up<8>(frac, bud, N, T_c, rem, lane);
    }
    N = 0;  // skips the shared-memory network and its top-up below
    rem = 0;
  }
  for (int k = 2; k <= N; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < N; i += 128) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const bool up = (i & k) != 0;
          float ai = (i < T_c) ? frac[i] : -CUDART_INF_F;
          float aj = (ixj < T_c) ? frac[ixj] : -CUDART_INF_F;
          int ii = (i < T_c) ? idx[i] : -1;
          int ij = (ixj < T_c) ? idx[ixj] : -1;
          if ((ai > aj) == up) {
            const float tf = ai; ai = aj; aj = tf;
            const int ti = ii; ii = ij; ij = ti;
          }
          if (i < T_c) { frac[i] = ai; idx[i] = ii; }
          if (ixj < T_c) { frac[ixj] = aj; idx[ixj] = ij; }
        }
      }
      __syncthreads();
    }
  }
  for (int r = tid; r < rem; r += 128) {
    const int best = idx[r];
    if (best >= 0) bud[best] += 1;  // the entries of idx are distinct tiles
  }
  __syncthreads();
  for (int t = tid; t < T_c; t += 128) {
    const float ell = ells[t];
    const int St = bud[t];
    S_tiles[t] = St;
    invdelta[t] = (St > 0 && ell > 1e-20f) ? __fdiv_rn((float)St, ell) : 0.0f;
    a0_tile[t] = offs[t];
  }
}

// ------------------------------------------------------------------ pass 2
struct Pass2Params {
  const void* V;            // [nseq,L_storage,KVH,128]
  const uint16_t* stash;    // [nseq,H,len_stride]
  const float* invdelta;    // [nseq,H,tile_stride]
  const float* a0;          // [nseq,H,tile_stride]
  int H, KVH, L, bn, T_c;   // L, T_c: the uniform length / tile count, or the length bound when ragged
  int L_storage, len_stride, tile_stride;
  const int* seq_lens;      // [nseq] device lengths, or null
  int nseq;
  WorkSplit ws;             // gw == 1: one column (sequence, kv-head) per warp
  float* partials;          // [nvg + columns][4][128]
  int* partial_vrows;       // [nvg + columns]
  long long partial_slots;  // nvg + columns (the checked build compares slots with it)
  int* status;              // the call's status word
  long long S;              // the per-head budget: enters the weights of a ragged batch's split
  int16_t* dbg_c;           // [nseq,H,len_stride] or null
  int* rowmask;             // [nseq,KVH,len_stride] or null
};

constexpr int kPass2Warps = 8;
constexpr int kPass2CtasPerSm = 2;  // resident CTAs per SM (register-limited)
// Two chunks per scan iteration; one chunk with three resident CTAs was measured 7 % slower (spills).
constexpr bool kPass2TwoChunks = true;

// One warp per (kv-head, tile range): counts from the stash, compaction,
// sparse V sum (santa_cuda_kernel.cu:771-863), tiles in ascending order.
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// dynamic shared memory of one pass-2 CTA: per warp a tile of unpacked weights (later the emit
// list), the raw stash rows of the tile being fetched, and that tile's four steps and offsets
constexpr int kPass2RawBytes = kMaxTileRows * 8;
constexpr int kPass2WarpSmem = kMaxTileRows * 16 + kPass2RawBytes + 32;
constexpr int kPass2Smem = kPass2Warps * kPass2WarpSmem;

template <typename TK>
__global__ void __launch_bounds__(kPass2Warps * 32, kPass2CtasPerSm) prop_pass2_kernel(const Pass2Params p) {
  extern __shared__ __align__(16) unsigned char s_dyn[];
  __shared__ int s_start[kMaxRaggedSeqs + 1];
  __shared__ long long s_wstart[kMaxRaggedSeqs + 1];
  __shared__ int s_wmax;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool ragged = p.seq_lens != nullptr;
  if (ragged) {  // lengths are inputs of the call, not results of the preceding kernels
    if (warp == 0) build_item_starts(p.seq_lens, p.nseq, p.L, p.bn, p.KVH, s_start, lane);
    if (warp == 1) {
      const int wmax = build_weight_starts(p.seq_lens, p.nseq, p.L, p.bn, p.KVH, p.S, s_wstart, lane);
      if (lane == 0) s_wmax = wmax;
    }
    __syncthreads();
  }
  cudaGridDependencySynchronize();
  long long items = p.ws.items;
  int nvg = p.ws.nvg;
  if (ragged) {  // ranges of equal weight, never more than hold an item each
    items = s_start[p.nseq];
    const long long fit = s_wmax > 0 ? s_wstart[p.nseq] / s_wmax : 0;
    nvg = (fit < (long long)nvg) ? int(fit) : nvg;
  }
  // The item ranges are dealt to the warps with a stride of the grid: the eight warps of a CTA (and
  // the CTAs that share an SM) work on ranges spread over the whole batch.  Ranges differ in cost --
  // a short sequence puts several samples into every tile, a long one leaves tiles empty -- and with
  // neighbouring ranges in one CTA the SMs that drew the expensive sequences ran half as long again
  // as the average.  Which warp runs a range does not change any result.
  const int vg = warp * int(gridDim.x) + int(blockIdx.x);
  if (vg >= nvg) return;
  long long lo, hi;
  if (ragged) {
    const long long W = s_wstart[p.nseq];
    lo = item_at_weight(s_start, s_wstart, p.nseq, range_lo(vg, W, nvg), p.KVH, p.S);
    hi = item_at_weight(s_start, s_wstart, p.nseq, range_lo(vg + 1, W, nvg), p.KVH, p.S);
  } else {
    lo = range_lo(vg, items, nvg);
    hi = range_lo(vg + 1, items, nvg);
  }
  float4* sb = reinterpret_cast<float4*>(s_dyn + size_t(warp) * kPass2WarpSmem);
  uint2* raw = reinterpret_cast<uint2*>(s_dyn + size_t(warp) * kPass2WarpSmem + kMaxTileRows * 16);
  float* par = reinterpret_cast<float*>(s_dyn + size_t(warp) * kPass2WarpSmem + kMaxTileRows * 16 + kPass2RawBytes);
  const size_t row_stride = size_t(p.KVH) * kRowBytes;
  const size_t ls = size_t(p.len_stride);

  long long it = lo;
  while (it < hi) {
    int b = 0, kv, t_lo, L_b = p.L, T_b = p.T_c;
    if (!ragged) {
      kv = int(it / T_b);
      t_lo = int(it - (long long)kv * T_b);
    } else {
      b = seq_of_item(s_start, p.nseq, int(it));
      L_b = ragged_len(p.seq_lens, b, p.L);
      T_b = (L_b + p.bn - 1) / p.bn;
      const int rel = int(it) - s_start[b];
      kv = rel / T_b;
      t_lo = rel - kv * T_b;
    }
    const int t_hi = (hi - it < (long long)(T_b - t_lo)) ? t_lo + int(hi - it) : T_b;
    const int h0 = kv * kGH;
    const size_t bh0 = size_t(b) * p.H + h0;
    const unsigned char* vcol =
        static_cast<const unsigned char*>(p.V) + (size_t(b) * p.L_storage * p.KVH + kv) * kRowBytes;
    const uint2* stash_col = reinterpret_cast<const uint2*>(p.stash) + (size_t(b) * p.KVH + kv) * ls;
    float acc[kGH][4];
#pragma unroll
    for (int g = 0; g < kGH; ++g)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[g][i] = 0.f;
    int vrow_count = 0;

    // Asynchronous fetch of a tile's stash rows (one 8-byte word per row) and of its four steps and
    // offsets into this warp's shared memory: issued one tile ahead, so that the latency of the
    // second pass's only streamed input hides behind the previous tile's counting and gathering.
    auto fetch = [&](int t) {
      const int n0 = t * p.bn;
      const int tile_len = (L_b - n0 < p.bn) ? (L_b - n0) : p.bn;
#pragma unroll
      for (int ch = 0; ch < kMaxTileRows / kChunkRows; ++ch) {
        const int r = ch * kChunkRows + lane;
        if (r < tile_len && SANTA_IN_RANGE(n0 + r, p.len_stride, p.status)) cp_async8(raw + r, stash_col + n0 + r);
      }
      if (lane < 2 * kGH) {
        const float* src = (lane < kGH ? p.invdelta : p.a0) + (bh0 + (lane & (kGH - 1))) * p.tile_stride + t;
        cp_async4(par + lane, src);
      }
    };
    fetch(t_lo);

#pragma unroll 1
    for (int t = t_lo; t < t_hi; ++t) {
      cp_async_wait_all();
      __syncwarp();
      float invdel[kGH], a0[kGH];
#pragma unroll
      for (int g = 0; g < kGH; ++g) {
        invdel[g] = par[g];
        a0[g] = par[kGH + g];
      }
      const int n0 = t * p.bn;
      const int tile_len = (L_b - n0 < p.bn) ? (L_b - n0) : p.bn;
      // a tile without budget on any of its four heads samples nothing: every count is zero
      const bool empty = !(invdel[0] > 0.f || invdel[1] > 0.f || invdel[2] > 0.f || invdel[3] > 0.f);
      if (!empty) {
#pragma unroll
        for (int ch = 0; ch < kMaxTileRows / kChunkRows; ++ch) {
          const int r = ch * kChunkRows + lane;
          const uint2 w = (r < tile_len) ? raw[r] : make_uint2(0u, 0u);
          const float2 f01 = Store16<TK>::unpack(w.x), f23 = Store16<TK>::unpack(w.y);
          sb[r] = make_float4(f01.x, f01.y, f23.x, f23.y);
        }
      }
      __syncwarp();                      // raw and par are consumed: the next tile may land
      if (t + 1 < t_hi) fetch(t + 1);
      if (empty) continue;
      RowTrace tr;
      tr.status = p.status;
      tr.rows_left = p.L_storage - n0;
      tr.vrow0 = vcol + size_t(n0) * row_stride;
      tr.row_stride = row_stride;
      tr.head_stride = ls;
      tr.u16 = nullptr;
      tr.counts = p.dbg_c ? p.dbg_c + bh0 * ls + n0 : nullptr;
      tr.rowmask = p.rowmask ? p.rowmask + (size_t(b) * p.KVH + kv) * ls + n0 : nullptr;
      // heads of this tile without a budget sample nothing: only the others are scanned
      const uint32_t active = (invdel[0] > 0.f ? 1u : 0u) | (invdel[1] > 0.f ? 2u : 0u) | (invdel[2] > 0.f ? 4u : 0u) |
                              (invdel[3] > 0.f ? 8u : 0u);
      int n_emit;
      switch (__popc(active)) {
        case 1: n_emit = tile_counts_some<TK, true, kPass2TwoChunks, 1>(sb, tile_len, lane, invdel, a0, tr, active); break;
        case 2: n_emit = tile_counts_some<TK, true, kPass2TwoChunks, 2>(sb, tile_len, lane, invdel, a0, tr, active); break;
        case 3: n_emit = tile_counts_some<TK, true, kPass2TwoChunks, 3>(sb, tile_len, lane, invdel, a0, tr, active); break;
        default: n_emit = tile_counts<TK, true, kPass2TwoChunks>(sb, tile_len, lane, invdel, a0, tr); break;
      }
      vrow_count += n_emit;
      float o[kGH][4];
#pragma unroll
      for (int g = 0; g < kGH; ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[g][i] = 0.f;
      gather_rows<TK>(sb, n_emit, vcol + size_t(n0) * row_stride, row_stride, lane, o, p.status, tr.rows_left);
      if (n_emit > 0) {
#pragma unroll
        for (int g = 0; g < kGH; ++g)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[g][i] = __fadd_rn(acc[g][i], o[g][i]);
      }
    }
    const size_t pslot = size_t(vg) + size_t(b) * p.KVH + kv;
    float* ps = p.partials + pslot * (kGH * kD);
    if (SANTA_IN_RANGE(pslot, p.partial_slots, p.status)) {
#pragma unroll
      for (int g = 0; g < kGH; ++g)
        reinterpret_cast<float4*>(ps + g * kD)[lane] = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
      if (lane == 0) p.partial_vrows[pslot] = vrow_count;
    }
    it += (t_hi - t_lo);
  }
}

// ------------------------------------------------------------------ merge
struct PropMergeParams {
  const float* partials;
  const int* partial_vrows;
  int KVH, T_c;
  const int* seq_lens;  // ragged: [nseq] device lengths, else null
  int nseq, max_len, bn;
  WorkSplit ws;
  float scale;   // 1/S, or 0 when S <= 0 (santa_cuda.cpp:333)
  long long S;   // the per-head budget (weights of a ragged batch's split)
  void* out;     // [nseq,H,128]
  int* vrows;    // [nseq,KVH] or null
};

// One CTA of 8 warps per (kv-head, head): warp w adds the partials v = first+w, first+w+8, ... in
// ascending order, then the eight sums are added in warp order -- a fixed order, so repeated calls
// give identical bits.
constexpr int kMergeWarps = 8;
template <typename TK>
__global__ void __launch_bounds__(kMergeWarps * 32) prop_merge_kernel(const PropMergeParams p) {
  __shared__ float4 s_acc[kMergeWarps][32];
  __shared__ int s_vr[kMergeWarps];
  __shared__ int s_wmx[kMergeWarps];
  __shared__ long long s_wbefore[kMergeWarps], s_wtotal[kMergeWarps];
  const int col = blockIdx.x >> 2;  // (sequence, kv-head)
  const int kv = col, g = blockIdx.x & 3, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  long long items = p.ws.items, item0 = (long long)col * p.T_c;
  int nvg = p.ws.nvg, T_b = p.T_c;
  long long item_last = item0 + T_b - 1;
  if (p.seq_lens != nullptr) {
    // The second pass cut its ranges in weight space (prop_unit_weight): this column's place there is
    // the weight of the sequences before it, times KVH, plus its own offset.
    const int b = col / p.KVH, kvb = col - b * p.KVH;
    int wmx = 0;
    long long wbefore = 0, wtotal = 0;
    for (int i = threadIdx.x; i < p.nseq; i += kMergeWarps * 32) {
      const int t = (ragged_len(p.seq_lens, i, p.max_len) + p.bn - 1) / p.bn;
      const int wi = prop_unit_weight(t, p.S);
      wtotal += (long long)t * wi;
      wbefore += (i < b) ? (long long)t * wi : 0;
      if (t > 0) wmx = wmx > wi ? wmx : wi;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      wbefore += __shfl_xor_sync(0xffffffffu, wbefore, off);
      wtotal += __shfl_xor_sync(0xffffffffu, wtotal, off);
      const int o = __shfl_xor_sync(0xffffffffu, wmx, off);
      wmx = wmx > o ? wmx : o;
    }
    if (lane == 0) {
      s_wbefore[w] = wbefore;
      s_wtotal[w] = wtotal;
      s_wmx[w] = wmx;
    }
    __syncthreads();
    wmx = 0;
    wbefore = wtotal = 0;
    for (int k = 0; k < kMergeWarps; ++k) {
      wbefore += s_wbefore[k];
      wtotal += s_wtotal[k];
      wmx = wmx > s_wmx[k] ? wmx : s_wmx[k];
    }
    T_b = (ragged_len(p.seq_lens, b, p.max_len) + p.bn - 1) / p.bn;
    const long long w_b = prop_unit_weight(T_b, p.S);
    // from here on `items`, `item0` and `item_last` are weights: the total and the weight starts of
    // the column's first and last item
    items = wtotal * p.KVH;
    const long long fit = wmx > 0 ? items / wmx : 0;
    nvg = (fit < (long long)nvg) ? int(fit) : nvg;
    item0 = wbefore * p.KVH + (long long)kvb * T_b * w_b;
    item_last = item0 + (long long)(T_b - 1) * w_b;
  }
  cudaGridDependencySynchronize();
  int v_first = 0, v_last = -1;  // an empty sequence contributes nothing
  if (T_b > 0) {
    v_first = cta_of_item(item0, items, nvg);
    v_last = cta_of_item(item_last, items, nvg);
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int v0 = v_first + w; v0 <= v_last; v0 += 4 * kMergeWarps) {
    float4 a[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      a[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      const int v = v0 + k * kMergeWarps;
      if (v <= v_last) a[k] = __ldcg(reinterpret_cast<const float4*>(p.partials + (size_t(v + kv) * kGH + g) * kD) + lane);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      acc.x += a[k].x;
      acc.y += a[k].y;
      acc.z += a[k].z;
      acc.w += a[k].w;
    }
  }
  int vr = 0;
  if (g == 0 && p.vrows != nullptr)
    for (int v = v_first + threadIdx.x; v <= v_last; v += kMergeWarps * 32) vr += __ldcg(p.partial_vrows + v + kv);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) vr += __shfl_xor_sync(0xffffffffu, vr, off);
  s_acc[w][lane] = acc;
  if (lane == 0) s_vr[w] = vr;
  __syncthreads();
  if (w == 0) {
#pragma unroll
    for (int k = 1; k < kMergeWarps; ++k) {
      const float4 b = s_acc[k][lane];
      acc.x += b.x;
      acc.y += b.y;
      acc.z += b.z;
      acc.w += b.w;
    }
    TK* op = static_cast<TK*>(p.out) + (size_t(kv) * kGH + g) * kD + 4 * lane;
    uint2 wv;
    wv.x = uint32_t(Store16<TK>::bits(acc.x * p.scale)) | (uint32_t(Store16<TK>::bits(acc.y * p.scale)) << 16);
    wv.y = uint32_t(Store16<TK>::bits(acc.z * p.scale)) | (uint32_t(Store16<TK>::bits(acc.w * p.scale)) << 16);
    *reinterpret_cast<uint2*>(op) = wv;
    if (g == 0 && p.vrows != nullptr && lane == 0) {
      int t = 0;
      for (int k = 0; k < kMergeWarps; ++k) t += s_vr[k];
      p.vrows[kv] = t;
    }
  }
}

// ------------------------------------------------------------------ pass 2 and merge for any GH <= 8, D % 16 == 0
// The shapes the vectorised kernels above do not cover (they are written for GH == 4, D == 128) go
// through these two: the arithmetic of the reference's pass2_grouped_tile_fused_atomic_kernel_x
// (santa_cuda_kernel.cu:734-864) with one warp per query head of the group, and a merge that adds
// the tiles in ascending order instead of the reference's atomics (deterministic).
struct Pass2GenericParams {
  const void* V;          // [L,KVH,D]
  const uint16_t* stash;  // [KVH][L][GH]
  const float* invdelta;  // [H,T_c]
  const float* a0;        // [H,T_c]
  const int* S_tiles;     // [H,T_c]
  int H, KVH, GH, D, L, bn, T_c;
  float* partials;        // [KVH][T_c][GH][D]
  int* partial_vrows;     // [KVH][T_c]
  int16_t* dbg_c;         // [H,L] or null
  int* rowmask;           // [KVH,L] or null
  int* status;            // the call's status word
};

template <typename TK>
__global__ void prop_pass2_generic_kernel(const Pass2GenericParams p) {
  cudaGridDependencySynchronize();
  extern __shared__ __align__(16) unsigned char s_dyn[];
  int16_t* c_tile = reinterpret_cast<int16_t*>(s_dyn);                       // [GH][bn]
  int* emit = reinterpret_cast<int*>(s_dyn + size_t(p.GH) * p.bn * 2);      // [bn]
  __shared__ int s_emit_len;
  const int kv = blockIdx.x, t = blockIdx.y;
  const int g = threadIdx.x >> 5, lane = threadIdx.x & 31;  // one warp per head of the group
  const int h = kv * p.GH + g;
  const int n0 = t * p.bn;
  const int tile_len = (p.L - n0 < p.bn) ? (p.L - n0) : p.bn;
  const size_t ht = size_t(h) * p.T_c + t;

  // counts of head g (santa_cuda_kernel.cu:771-808), the scan as in tile_counts of sampler.cuh
  {
    const float invdel = p.invdelta[ht], a0 = p.a0[ht];
    float carry = 0.f;
    for (int base = 0; base < tile_len; base += kChunkRows) {
      const int r = base + lane;
      const bool valid = r < tile_len;
      float x = 0.f;
      if (valid && invdel > 0.f) {
        const uint32_t ub = p.stash[(size_t(kv) * p.L + n0 + r) * p.GH + g];
        x = __fmul_rn(Store16<TK>::unpack(ub).x, invdel);
      }
      float res = x;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float nb = __shfl_up_sync(0xffffffffu, res, off);
        if (lane >= off) res = __fadd_rn(res, nb);
      }
      const float pre = __fsub_rn(res, x);
      const int remain = tile_len - base;
      const int last = remain > 32 ? 31 : remain - 1;
      const float tot = __shfl_sync(0xffffffffu, __fadd_rn(pre, x), last);
      const float pg = __fadd_rn(carry, pre);
      const float cg = __fadd_rn(pg, x);
      int c = __float2int_rd(__fadd_rn(a0, cg)) - __float2int_rd(__fadd_rn(a0, pg));
      c = c < 0 ? 0 : (c > 32767 ? 32767 : c);
      if (valid) {
        c_tile[g * p.bn + r] = (int16_t)c;
        if (p.dbg_c != nullptr) p.dbg_c[size_t(h) * p.L + n0 + r] = (int16_t)c;
      }
      carry = __fadd_rn(carry, tot);
    }
  }
  __syncthreads();
  // rows sampled by any head, ascending (:810-838)
  if (g == 0) {
    int n_emit = 0;
    for (int base = 0; base < tile_len; base += kChunkRows) {
      const int r = base + lane;
      int sum = 0;
      if (r < tile_len)
        for (int gg = 0; gg < p.GH; ++gg) sum += c_tile[gg * p.bn + r];
      const bool flag = sum > 0;
      const uint32_t mask = __ballot_sync(0xffffffffu, flag);
      if (flag && SANTA_IN_RANGE(n_emit + __popc(mask & ((1u << lane) - 1u)), p.bn, p.status)) {
        emit[n_emit + __popc(mask & ((1u << lane) - 1u))] = r;
        if (p.rowmask != nullptr) p.rowmask[size_t(kv) * p.L + n0 + r] = 1;
      }
      n_emit += __popc(mask);
    }
    if (lane == 0) {
      s_emit_len = n_emit;
      p.partial_vrows[size_t(kv) * p.T_c + t] = n_emit;
    }
  }
  __syncthreads();
  // sparse sum of c*V for head g (:843-857): lane l owns dims l, l+32, ...
  const int n_emit = s_emit_len;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const TK* Vt = static_cast<const TK*>(p.V);
  for (int i = 0; i < n_emit; ++i) {
    const int r = emit[i];
    if (!SANTA_IN_RANGE(r, tile_len, p.status)) continue;
    const int c = c_tile[g * p.bn + r];
    if (c != 0) {
      const float cf = (float)c;
      const uint16_t* vrow = reinterpret_cast<const uint16_t*>(Vt + (size_t(n0 + r) * p.KVH + kv) * p.D);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int d = lane + 32 * k;
        if (d < p.D) acc[k] = fmaf(cf, Store16<TK>::unpack(uint32_t(vrow[d])).x, acc[k]);
      }
    }
  }
  float* po = p.partials + ((size_t(kv) * p.T_c + t) * p.GH + g) * p.D;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int d = lane + 32 * k;
    if (d < p.D) po[d] = acc[k];
  }
}

// One CTA per head: out[h, :] = (sum over tiles, ascending, of the tile's partial) / S.
template <typename TK>
__global__ void prop_merge_generic_kernel(const float* __restrict__ partials, const int* __restrict__ partial_vrows,
                                          const int* __restrict__ S_tiles, int KVH, int GH, int D, int T_c,
                                          float scale, TK* __restrict__ out, int* __restrict__ vrows) {
  cudaGridDependencySynchronize();
  const int h = blockIdx.x, kv = h / GH, g = h - kv * GH;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int t = 0; t < T_c; ++t)
      if (S_tiles[size_t(h) * T_c + t] > 0) acc = __fadd_rn(acc, __ldcg(partials + ((size_t(kv) * T_c + t) * GH + g) * D + d));
    reinterpret_cast<uint16_t*>(out)[size_t(h) * D + d] = Store16<TK>::bits(acc * scale);
  }
  if (g == 0 && vrows != nullptr && threadIdx.x == 0) {
    int n = 0;
    for (int t = 0; t < T_c; ++t) n += __ldcg(partial_vrows + size_t(kv) * T_c + t);
    vrows[kv] = n;
  }
}

// ------------------------------------------------------------------ launch
template <typename KernelT, typename... Args>
static cudaError_t launch_dependent(KernelT kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <typename TK>
static cudaError_t launch_prop_t(const PropParams& p, int grid, cudaStream_t stream) {
  static bool configured[64] = {};
  static bool configured2[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t e;
  const int H = p.sp.H, KVH = p.sp.KVH, L = p.sp.L_valid;
  if (p.use_vec) {
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      const void* kernels[4] = {(const void*)stream_kernel<TK, 256, kModePropPass1, false, false>,
                                (const void*)stream_kernel<TK, 256, kModePropPass1, true, false>,
                                (const void*)stream_kernel<TK, 256, kModePropPass1, false, true>,
                                (const void*)stream_kernel<TK, 256, kModePropPass1, true, true>};
      for (const void* k : kernels) {
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStreamSmemBytes);
        if (e != cudaSuccess) return e;
      }
      configured[dev] = true;
    }
    const bool ragged = p.sp.seq_lens != nullptr;
    if (p.sp.score_mma)
      e = ragged ? launch_dependent(stream_kernel<TK, 256, kModePropPass1, true, true>, dim3(grid),
                                    dim3(kCtaWarps * 32), kStreamSmemBytes, stream, p.sp)
                 : launch_dependent(stream_kernel<TK, 256, kModePropPass1, false, true>, dim3(grid),
                                    dim3(kCtaWarps * 32), kStreamSmemBytes, stream, p.sp);
    else
      e = ragged ? launch_dependent(stream_kernel<TK, 256, kModePropPass1, true, false>, dim3(grid),
                                    dim3(kCtaWarps * 32), kStreamSmemBytes, stream, p.sp)
                 : launch_dependent(stream_kernel<TK, 256, kModePropPass1, false, false>, dim3(grid),
                                    dim3(kCtaWarps * 32), kStreamSmemBytes, stream, p.sp);
    if (e != cudaSuccess) return e;
  } else {
    const int nwarp = p.block_n / 16;
    const size_t smem = size_t(nwarp * 256 + 2 * 16 * nwarp + 16) * sizeof(float);
    prop_pass1_mma_kernel<TK><<<dim3(p.T_c, KVH), nwarp * 32, smem, stream>>>(
        static_cast<const TK*>(p.sp.q), static_cast<const TK*>(p.K), H, KVH, H / KVH, p.D, L, p.block_n, p.T_c,
        p.sp.q_scale, p.sp.m_tiles, p.sp.ell_tiles, p.sp.stash, p.sp.dbg_u);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  const int nseq = p.sp.seq_lens ? p.sp.nseq : 1;
  const size_t budget_smem = size_t(p.sp.tile_stride) * 20;  // five per-tile tables
  if (budget_smem > 48 * 1024) {
    e = cudaFuncSetAttribute(prop_budgets_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget_smem);
    if (e != cudaSuccess) return e;
  }
  e = launch_dependent(prop_budgets_kernel, dim3(H, nseq), dim3(128), budget_smem, stream,
                       (const float*)p.sp.m_tiles, (const float*)p.sp.ell_tiles, p.T_c, p.sp.seq_lens, L,
                       p.block_n, p.sp.tile_stride, p.S, p.sp.seed, p.flags, p.m_star, p.S_tiles, p.invdelta, p.a0);
  if (e != cudaSuccess) return e;

  const int GH = H / KVH;
  if (GH != kGH || p.D != kD) {
    // shapes outside the vectorised kernels: one CTA per (kv-head, tile), one warp per head of the group
    Pass2GenericParams pg{};
    pg.V = p.sp.V;
    pg.stash = p.sp.stash;
    pg.invdelta = p.invdelta;
    pg.a0 = p.a0;
    pg.S_tiles = p.S_tiles;
    pg.H = H;
    pg.KVH = KVH;
    pg.GH = GH;
    pg.D = p.D;
    pg.L = L;
    pg.bn = p.block_n;
    pg.T_c = p.T_c;
    pg.partials = p.partials;
    pg.partial_vrows = p.partial_vrows;
    pg.dbg_c = p.dbg_c;
    pg.rowmask = p.rowmask;
    pg.status = p.sp.status;
    const size_t smem2 = size_t(GH) * p.block_n * 2 + size_t(p.block_n) * 4;
    e = launch_dependent(prop_pass2_generic_kernel<TK>, dim3(KVH, p.T_c), dim3(GH * 32), smem2, stream, pg);
    if (e != cudaSuccess) return e;
    const float scale = (p.S > 0) ? (1.0f / (float)p.S) : 0.0f;
    return launch_dependent(prop_merge_generic_kernel<TK>, dim3(H), dim3(128), 0, stream,
                            (const float*)p.partials, (const int*)p.partial_vrows, (const int*)p.S_tiles, KVH, GH,
                            p.D, p.T_c, scale, static_cast<TK*>(p.out), p.vrows);
  }

  Pass2Params p2{};
  p2.V = p.sp.V;
  p2.stash = p.sp.stash;
  p2.invdelta = p.invdelta;
  p2.a0 = p.a0;
  p2.H = H;
  p2.KVH = KVH;
  p2.L = L;
  p2.bn = p.block_n;
  p2.T_c = p.T_c;
  p2.L_storage = p.sp.L_storage;
  p2.len_stride = p.sp.len_stride;
  p2.tile_stride = p.sp.tile_stride;
  p2.seq_lens = p.sp.seq_lens;
  p2.nseq = nseq;
  p2.ws.gw = 1;
  p2.ws.T_c = p.T_c;
  p2.ws.ncol = nseq * KVH;
  p2.ws.items = (long long)nseq * KVH * p.T_c;  // ragged: an upper bound, the kernels count the real items
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long max_warps = (long long)prop_pass2_max_groups(sms);
  p2.ws.nvg = int(p2.ws.items < max_warps ? p2.ws.items : max_warps);
  p2.partials = p.partials;
  p2.partial_vrows = p.partial_vrows;
  p2.partial_slots = max_warps + (long long)nseq * KVH;
  p2.status = p.sp.status;
  p2.S = p.S;
  p2.dbg_c = p.dbg_c;
  p2.rowmask = p.rowmask;
  const int grid2 = (p2.ws.nvg + kPass2Warps - 1) / kPass2Warps;
  if (dev >= 0 && dev < 64 && !configured2[dev]) {
    e = cudaFuncSetAttribute(prop_pass2_kernel<TK>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPass2Smem);
    if (e != cudaSuccess) return e;
    configured2[dev] = true;
  }
  e = launch_dependent(prop_pass2_kernel<TK>, dim3(grid2), dim3(kPass2Warps * 32), kPass2Smem, stream, p2);
  if (e != cudaSuccess) return e;

  PropMergeParams pm{};
  pm.partials = p.partials;
  pm.partial_vrows = p.partial_vrows;
  pm.KVH = KVH;
  pm.T_c = p.T_c;
  pm.seq_lens = p.sp.seq_lens;
  pm.nseq = nseq;
  pm.max_len = L;
  pm.bn = p.block_n;
  pm.ws = p2.ws;
  pm.scale = (p.S > 0) ? (1.0f / (float)p.S) : 0.0f;
  pm.S = p.S;
  pm.out = p.out;
  pm.vrows = p.vrows;
  return launch_dependent(prop_merge_kernel<TK>, dim3(nseq * KVH * kGH), dim3(kMergeWarps * 32), 0, stream, pm);
}

cudaError_t launch_prop(const PropParams& p, int dtype, int grid, cudaStream_t stream) {
  return dtype == 0 ? launch_prop_t<__nv_bfloat16>(p, grid, stream) : launch_prop_t<__half>(p, grid, stream);
}

// Upper bound on pass-2 warps for workspace sizing (must match launch_prop_t).
int prop_pass2_max_groups(int sms) { return sms * kPass2CtasPerSm * kPass2Warps; }

}  // namespace santa
