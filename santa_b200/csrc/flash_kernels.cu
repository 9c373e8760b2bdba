// flash_kernels.cu -- S2ANTA-Flash decode attention (fixed per-tile sample
// budget) for sm_100a.  Two launches on one stream, chained with programmatic
// dependent launch:
//   stream_kernel<.., kModeFlash>  persistent, one CTA per SM (stream_kernel.cuh):
//                        streams K once through TMA, samples rows by systematic
//                        resampling inside every tile, gathers the sampled V
//                        rows and folds tiles into a running log-sum-exp state;
//                        every column slot writes one partial (A[128], m, Z per
//                        head) per column group it touched;
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

#include <cooperative_groups.h>

#include "stream_kernel.cuh"

namespace santa {

// Folds the partials of one (column, head) pair.  Launched as a programmatic
// dependent of flash_decode_kernel: it may become resident early and waits for
// the producer grid before touching its results.
//   m* = max_v m_v;  w_v = exp(m_v - m*);  Z = sum_v w_v Z_v;  A = sum_v w_v A_v;
//   out = A / (Z * S_per_tile)            (reference :436-468 over all tiles)
constexpr int kFlashMergeWarps = 8;    // warps of one merge CTA
constexpr int kFlashMergeInFlight = 8; // partial vectors each warp keeps in flight
template <typename TK>
__global__ void __launch_bounds__(kFlashMergeWarps * 32) flash_merge_kernel(const FlashMergeParams p) {
  constexpr int NW = kFlashMergeWarps, NT = kFlashMergeWarps * 32, NF = kFlashMergeInFlight;
  __shared__ float s_w[kMaxCtas * kGroupWarps];
  __shared__ float s_z[kMaxCtas * kGroupWarps];
  __shared__ float s_red[NW];
  __shared__ int s_redi[NW];
  __shared__ int s_before[NW], s_total[NW];
  __shared__ float4 s_acc[NW][32];

  const int col = blockIdx.x >> 2;
  const int g = blockIdx.x & 3;
  const int gw = p.ws.gw;
  const int b = col / p.KVH;
  const int kv = col - b * p.KVH;
  const int tid = threadIdx.x, lane = tid & 31, wq = tid >> 5;
  int cg = col / gw;
  const int w = col - cg * gw;
  int T_c = p.ws.T_c, spt = p.S_per_tile, nvg = p.ws.nvg;
  long long items = p.ws.items, item0 = (long long)cg * T_c;
  if (p.seq_lens != nullptr) {
    // ragged batch: column groups never span sequences; the items of the sequences before this one
    // come first (the lengths are inputs of the call, so they may be read before the producer ends)
    int before = 0, total = 0;
    for (int i = tid; i < p.nseq; i += NT) {
      const int t = (ragged_len(p.seq_lens, i, p.max_len) + p.bn - 1) / p.bn;
      total += t;
      before += (i < b) ? t : 0;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      before += __shfl_xor_sync(0xffffffffu, before, off);
      total += __shfl_xor_sync(0xffffffffu, total, off);
    }
    if (lane == 0) {
      s_before[wq] = before;
      s_total[wq] = total;
    }
    __syncthreads();
    before = total = 0;
#pragma unroll
    for (int k = 0; k < NW; ++k) {
      before += s_before[k];
      total += s_total[k];
    }
    const int gps = p.KVH / gw, cgs = kv / gw;
    T_c = (ragged_len(p.seq_lens, b, p.max_len) + p.bn - 1) / p.bn;
    spt = (p.S_total > 0 && T_c > 0) ? (p.S_total / T_c > 1 ? p.S_total / T_c : 1) : 0;
    cg = b * gps + cgs;
    items = (long long)total * gps;
    nvg = (items < (long long)nvg) ? int(items) : nvg;
    item0 = ((long long)before * gps) + (long long)cgs * T_c;
  }
  cudaGridDependencySynchronize();

  int v_first = 0, v_last = -1;  // an empty sequence has no partials
  if (T_c > 0) {
    v_first = cta_of_item(item0, items, nvg);
    v_last = cta_of_item(item0 + T_c - 1, items, nvg);
  }
  int nv = v_last - v_first + 1;
  if (nv > 0 && !SANTA_IN_RANGE(size_t(v_last + cg) * gw + w, p.partial_slots, p.status)) nv = 0;
  if (!SANTA_IN_RANGE(nv, kMaxCtas * kGroupWarps + 1, p.status)) nv = 0;  // the weights live in shared memory
  auto partial = [&](int v) {
    return p.partials + ((size_t(v + cg) * gw + w) * kGH + g) * kPartialStride;
  };

  // All loads of a merge of up to NW * NF partials are issued before anything depends on them: the
  // first NF partial vectors of every warp (phase 3 below) together with every partial's (m, Z) pair.
  float4 a_pre[NF];
#pragma unroll
  for (int k = 0; k < NF; ++k) {
    const int i = wq + NW * k;
    a_pre[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < nv) a_pre[k] = __ldcg(reinterpret_cast<const float4*>(partial(v_first + i)) + lane);
  }

  // phase 1: m* (Z rides along in the same 8-byte load)
  float mloc = -CUDART_INF_F;
  for (int i = tid; i < nv; i += NT) {
    const float2 mz = __ldcg(reinterpret_cast<const float2*>(partial(v_first + i) + kD));
    s_w[i] = mz.x;
    s_z[i] = mz.y;
    mloc = fmaxf(mloc, mz.x);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, off));
  if (lane == 0) s_red[wq] = mloc;
  __syncthreads();
  float ms = s_red[0];
#pragma unroll
  for (int k = 1; k < NW; ++k) ms = fmaxf(ms, s_red[k]);
  __syncthreads();

  // phase 2: weights, Z, gathered-row count
  float zloc = 0.f;
  int vloc = 0;
  for (int i = tid; i < nv; i += NT) {
    const float e = __expf(s_w[i] - ms);
    zloc += e * s_z[i];
    if (g == 0 && p.vrows != nullptr) vloc += __ldcg(p.partial_vrows + size_t(v_first + i + cg) * gw + w);
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
  float zs = 0.f;
  int vrows_total = 0;
#pragma unroll
  for (int k = 0; k < NW; ++k) {  // a fixed order: repeated calls give identical bits
    zs += s_red[k];
    vrows_total += s_redi[k];
  }

  // phase 3: A, NF partials in flight per warp (the first NF were fetched above)
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i0 = wq; i0 < nv; i0 += NW * NF) {
    float e[NF];
    float4 a[NF];
#pragma unroll
    for (int k = 0; k < NF; ++k) {
      const int i = i0 + NW * k;
      e[k] = (i < nv) ? s_w[i] : 0.f;
      a[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i0 == wq)
        a[k] = a_pre[k];
      else if (i < nv)
        a[k] = __ldcg(reinterpret_cast<const float4*>(partial(v_first + i)) + lane);
    }
#pragma unroll
    for (int k = 0; k < NF; ++k) {
      acc.x += e[k] * a[k].x;
      acc.y += e[k] * a[k].y;
      acc.z += e[k] * a[k].z;
      acc.w += e[k] * a[k].w;
    }
  }
  s_acc[wq][lane] = acc;
  __syncthreads();
  if (wq == 0) {
#pragma unroll
    for (int k = 1; k < NW; ++k) {
      const float4 ak = s_acc[k][lane];
      acc.x += ak.x;
      acc.y += ak.y;
      acc.z += ak.z;
      acc.w += ak.w;
    }
    const size_t bh = size_t(b) * p.H + kv * kGH + g;
    if (p.partial_out != nullptr) {
      // raw merged partial for a cross-device combine: A[128], m, Z
      float* po = p.partial_out + bh * (kD + 2);
      reinterpret_cast<float2*>(po)[2 * lane] = make_float2(acc.x, acc.y);
      reinterpret_cast<float2*>(po)[2 * lane + 1] = make_float2(acc.z, acc.w);
      if (lane == 0) reinterpret_cast<float2*>(po)[kD / 2] = make_float2(ms, zs);
    }
    bool combined = false;
    if (p.px.world > 0) {
      // the same partial into every rank's exchange buffer: plain peer stores; then -- the row's stores
      // having happened before the warp's barrier -- the signalling lanes release them at system scope
      // and mark the row (its epoch) and count it for the receiver
      const int BH = int(gridDim.x);
      int* ctl = reinterpret_cast<int*>(p.px.base[p.px.rank]);
      // device-counted epochs: this step is (steps completed so far) + 1
      const unsigned epoch = p.px.epoch != 0 ? p.px.epoch : unsigned(__ldcg(ctl + kPeerStepIndex)) + 1u;
      const int parity = int(epoch & 1u);
      for (int r = 0; r < p.px.world; ++r) {
        float* po = reinterpret_cast<float*>(p.px.base[r] + peer_data_offset(parity, p.px.world, p.px.rank, BH)) +
                    bh * (kD + 2);
        reinterpret_cast<float2*>(po)[2 * lane] = make_float2(acc.x, acc.y);
        reinterpret_cast<float2*>(po)[2 * lane + 1] = make_float2(acc.z, acc.w);
        if (lane == 0) reinterpret_cast<float2*>(po)[kD / 2] = make_float2(ms, zs);
      }
      __syncwarp();
      if (lane < p.px.world) {
        __threadfence_system();
        volatile int* flag =
            reinterpret_cast<volatile int*>(p.px.base[lane] + peer_row_flag_offset(parity, p.px.world, p.px.rank, BH)) + bh;
        *flag = int(epoch);  // read by the combining form of this call on the receiving rank
        if (!p.px.combine)   // counted by the separate wait-and-combine kernel
          atomicAdd_system(reinterpret_cast<int*>(p.px.base[lane]) + parity * kMaxPeers + p.px.rank, 1);
      }
      if (p.px.combine) {
        // the receiving half for this row, without a second kernel: wait (bounded) until every rank's
        // row of this epoch sits in the local buffer, then fold them in rank order
        const int* my_flag = reinterpret_cast<const int*>(p.px.base[p.px.rank] +
                                                          peer_row_flag_offset(parity, p.px.world, lane, BH)) + bh;
        const bool ok = peer_wait(my_flag, lane < p.px.world, epoch, false);
        TK* op = static_cast<TK*>(p.out) + bh * kD;
        if (!ok) {
          if (lane == 0) {
            atomicExch(p.status, kStatusPeerTimeout);
            atomicExch(ctl + kPeerStatusIndex, kStatusPeerTimeout);
            if (p.m_star != nullptr) p.m_star[bh] = -CUDART_INF_F;
          }
          *reinterpret_cast<uint2*>(op + 4 * lane) = make_uint2(0u, 0u);
        } else {
          const float* rows = reinterpret_cast<const float*>(p.px.base[p.px.rank] +
                                                             peer_data_offset(parity, p.px.world, 0, BH)) + bh * (kD + 2);
          combine_rows<TK>(rows, size_t(BH) * (kD + 2), p.px.world, spt, lane, op, p.m_star ? p.m_star + bh : nullptr);
        }
        if (p.px.epoch == 0 && lane == 0) peer_step_done(ctl, BH);
        combined = true;
      }
    }
    if (p.out != nullptr && !combined) {
      const float inv = (spt > 0 && zs > 0.f) ? 1.0f / (zs * (float)spt) : 0.f;
      TK* op = static_cast<TK*>(p.out) + bh * kD + 4 * lane;
      uint2 wv;
      wv.x = uint32_t(Store16<TK>::bits(acc.x * inv)) | (uint32_t(Store16<TK>::bits(acc.y * inv)) << 16);
      wv.y = uint32_t(Store16<TK>::bits(acc.z * inv)) | (uint32_t(Store16<TK>::bits(acc.w * inv)) << 16);
      *reinterpret_cast<uint2*>(op) = wv;
    }
    if (lane == 0) {
      if (p.m_star != nullptr && !combined) p.m_star[bh] = ms;
      if (g == 0 && p.vrows != nullptr) p.vrows[b * p.KVH + kv] = vrows_total;
    }
  }
}

template <typename TK, int BN, bool MMA>
static cudaError_t launch_one(const StreamParams& p, const FlashMergeParams& mp, int grid, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(stream_kernel<TK, BN, kModeFlash, false, MMA>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStreamSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(stream_kernel<TK, BN, kModeFlash, true, MMA>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStreamSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(grid));
  cfg.blockDim = dim3(kCtaWarps * 32);
  cfg.dynamicSmemBytes = kStreamSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = (p.seq_lens != nullptr)
                      ? cudaLaunchKernelEx(&cfg, stream_kernel<TK, BN, kModeFlash, true, MMA>, p)
                      : cudaLaunchKernelEx(&cfg, stream_kernel<TK, BN, kModeFlash, false, MMA>, p);
  if (e != cudaSuccess) return e;

  cfg.gridDim = dim3(unsigned(p.ws.ncol) * kGH);
  cfg.blockDim = dim3(kFlashMergeWarps * 32);
  cfg.dynamicSmemBytes = 0;
  return cudaLaunchKernelEx(&cfg, flash_merge_kernel<TK>, mp);
}

template <typename TK>
static cudaError_t launch_bn(const StreamParams& p, const FlashMergeParams& mp, int block_n, int grid,
                             cudaStream_t stream) {
  if (p.score_mma) {
    if (block_n == 32) return launch_one<TK, 32, true>(p, mp, grid, stream);
    if (block_n == 64) return launch_one<TK, 64, true>(p, mp, grid, stream);
    return launch_one<TK, 256, true>(p, mp, grid, stream);
  }
  if (block_n == 32) return launch_one<TK, 32, false>(p, mp, grid, stream);
  if (block_n == 64) return launch_one<TK, 64, false>(p, mp, grid, stream);
  return launch_one<TK, 256, false>(p, mp, grid, stream);
}

cudaError_t launch_flash(const StreamParams& p, const FlashMergeParams& mp, int dtype, int block_n, int grid,
                         cudaStream_t stream) {
  return dtype == 0 ? launch_bn<__nv_bfloat16>(p, mp, block_n, grid, stream)
                    : launch_bn<__half>(p, mp, block_n, grid, stream);
}

}  // namespace santa
