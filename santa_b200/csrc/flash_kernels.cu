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
template <typename TK>
__global__ void __launch_bounds__(128) flash_merge_kernel(const FlashMergeParams p) {
  __shared__ float s_w[kMaxCtas * kGroupWarps];
  __shared__ float s_z[kMaxCtas * kGroupWarps];
  __shared__ float s_red[4];
  __shared__ int s_redi[4];
  __shared__ int s_before[4], s_total[4];
  __shared__ float4 s_acc[4][32];

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
    for (int i = tid; i < p.nseq; i += 128) {
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
    before = (s_before[0] + s_before[1]) + (s_before[2] + s_before[3]);
    total = (s_total[0] + s_total[1]) + (s_total[2] + s_total[3]);
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
  const int nv = v_last - v_first + 1;
  auto partial = [&](int v) {
    return p.partials + ((size_t(v + cg) * gw + w) * kGH + g) * kPartialStride;
  };

  // All loads of a small merge are issued before anything depends on them: the first four partial
  // vectors of every warp (phase 3 below) together with every partial's (m, Z) pair.
  float4 a_pre[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = wq + 4 * k;
    a_pre[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < nv) a_pre[k] = __ldcg(reinterpret_cast<const float4*>(partial(v_first + i)) + lane);
  }

  // phase 1: m* (Z rides along in the same 8-byte load)
  float mloc = -CUDART_INF_F;
  for (int i = tid; i < nv; i += 128) {
    const float2 mz = __ldcg(reinterpret_cast<const float2*>(partial(v_first + i) + kD));
    s_w[i] = mz.x;
    s_z[i] = mz.y;
    mloc = fmaxf(mloc, mz.x);
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
  const float zs = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);

  // phase 3: A, four partials in flight per warp (the first four were fetched above)
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i0 = wq; i0 < nv; i0 += 16) {
    float e[4];
    float4 a[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = i0 + 4 * k;
      e[k] = (i < nv) ? s_w[i] : 0.f;
      a[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i0 == wq)
        a[k] = a_pre[k];
      else if (i < nv)
        a[k] = __ldcg(reinterpret_cast<const float4*>(partial(v_first + i)) + lane);
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
    if (p.px.world > 0) {
      // the same partial into every rank's exchange buffer: plain peer stores, made visible system-wide,
      // then one arrival count per receiver (released after the whole row is out)
      const int BH = int(gridDim.x);
      int parity = p.px.parity;
      if (parity < 0)  // device-counted epochs: this step is (steps completed so far) + 1
        parity = (__ldcg(reinterpret_cast<const int*>(p.px.base[p.px.rank]) + kPeerStepIndex) + 1) & 1;
      for (int r = 0; r < p.px.world; ++r) {
        float* po = reinterpret_cast<float*>(p.px.base[r] + peer_data_offset(parity, p.px.world, p.px.rank, BH)) +
                    bh * (kD + 2);
        po[4 * lane + 0] = acc.x;
        po[4 * lane + 1] = acc.y;
        po[4 * lane + 2] = acc.z;
        po[4 * lane + 3] = acc.w;
        if (lane == 0) {
          po[kD] = ms;
          po[kD + 1] = zs;
        }
      }
      __threadfence_system();
      __syncwarp();
      if (lane < p.px.world)
        atomicAdd_system(reinterpret_cast<int*>(p.px.base[lane]) + parity * kMaxPeers + p.px.rank, 1);
    }
    if (p.out != nullptr) {
      const float inv = (spt > 0 && zs > 0.f) ? 1.0f / (zs * (float)spt) : 0.f;
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
static cudaError_t launch_one(const StreamParams& p, const FlashMergeParams& mp, int grid, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(stream_kernel<TK, BN, kModeFlash, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStreamSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(stream_kernel<TK, BN, kModeFlash, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kStreamSmemBytes);
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
  cudaError_t e = (p.seq_lens != nullptr) ? cudaLaunchKernelEx(&cfg, stream_kernel<TK, BN, kModeFlash, true>, p)
                                          : cudaLaunchKernelEx(&cfg, stream_kernel<TK, BN, kModeFlash, false>, p);
  if (e != cudaSuccess) return e;

  cfg.gridDim = dim3(unsigned(p.ws.ncol) * kGH);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = 0;
  return cudaLaunchKernelEx(&cfg, flash_merge_kernel<TK>, mp);
}

cudaError_t launch_flash(const StreamParams& p, const FlashMergeParams& mp, int dtype, int block_n, int grid,
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
