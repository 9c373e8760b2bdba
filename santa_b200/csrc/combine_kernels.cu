// combine_kernels.cu -- log-sum-exp combine of unnormalised Flash partials that
// were produced for disjoint tile sets of the same sequences, e.g. by the ranks
// of a sequence-sharded decode after an all-gather.  Partial r holds, per
// (batch, head): A_r[128], m_r, Z_r with
//   A_r = sum_t exp(m_t - m_r) ell_t o_t,   Z_r = sum_t exp(m_t - m_r) ell_t,
// and the combined result is the reference's finalize over the union of tiles
// (flash_style_fused_santa_fixed_tile_budgets/santa_cuda_kernel.cu:386-470):
//   m* = max_r m_r,  out = sum_r e^{m_r-m*} A_r / (S_per_tile * sum_r e^{m_r-m*} Z_r).
#include "common.cuh"
#include "santa_abi_internal.h"

namespace santa {

template <typename TK>
__global__ void __launch_bounds__(32) lse_combine_kernel(const float* __restrict__ partials, int G, int BH,
                                                         int S_per_tile, TK* __restrict__ out,
                                                         float* __restrict__ m_star) {
  const int bh = blockIdx.x, lane = threadIdx.x;
  constexpr int W = kD + 2;
  float ms = -CUDART_INF_F;
  for (int r = 0; r < G; ++r) ms = fmaxf(ms, partials[(size_t(r) * BH + bh) * W + kD]);
  float zs = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = 0; r < G; ++r) {
    const float* p = partials + (size_t(r) * BH + bh) * W;
    const float e = __expf(p[kD] - ms);
    zs += e * p[kD + 1];
    acc.x += e * p[4 * lane + 0];
    acc.y += e * p[4 * lane + 1];
    acc.z += e * p[4 * lane + 2];
    acc.w += e * p[4 * lane + 3];
  }
  const float inv = (S_per_tile > 0 && zs > 0.f) ? 1.0f / (zs * (float)S_per_tile) : 0.f;
  TK* op = out + size_t(bh) * kD + 4 * lane;
  uint2 wv;
  wv.x = uint32_t(Store16<TK>::bits(acc.x * inv)) | (uint32_t(Store16<TK>::bits(acc.y * inv)) << 16);
  wv.y = uint32_t(Store16<TK>::bits(acc.z * inv)) | (uint32_t(Store16<TK>::bits(acc.w * inv)) << 16);
  *reinterpret_cast<uint2*>(op) = wv;
  if (lane == 0 && m_star != nullptr) m_star[bh] = ms;
}

// The receiving half of the peer exchange.  One warp per (batch, head) row: lane g < world polls sender
// g's arrival counter (every sender adds 1 per row it has delivered, `expected` in total by this epoch)
// with system-scope acquire loads and a bounded, sleeping wait; then the rows are combined as above.
template <typename TK>
__global__ void __launch_bounds__(32) lse_combine_wait_kernel(unsigned char* __restrict__ base, int world,
                                                              unsigned epoch_arg, int BH, int S_per_tile,
                                                              TK* __restrict__ out, float* __restrict__ m_star,
                                                              int* __restrict__ status) {
  const int bh = blockIdx.x, lane = threadIdx.x;
  int* ctl = reinterpret_cast<int*>(base);
  // epoch 0: count the epochs on the device (the same launch, replayed from a graph, serves every step)
  const bool counted = epoch_arg == 0;
  const unsigned epoch = counted ? unsigned(__ldcg(ctl + kPeerStepIndex)) + 1u : epoch_arg;
  const int parity = int(epoch & 1u);
  // every sender has added BH to its counter of this parity once per epoch of that parity so far
  const unsigned expected = ((epoch + unsigned(parity)) >> 1) * unsigned(BH);
  bool ok = true;
  if (lane < world) {
    const int* flag = reinterpret_cast<const int*>(base) + parity * kMaxPeers + lane;
    ok = false;
    for (int spin = 0; spin < kSpinLimit; ++spin) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (int(unsigned(v) - expected) >= 0) {  // wrap-safe: the counters run for the life of the buffer
        ok = true;
        break;
      }
      __nanosleep(200);
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  TK* op = out + size_t(bh) * kD + 4 * lane;
  if (!ok) {  // report and leave a defined result; nothing was consumed, the step counter stays
    if (lane == 0 && status != nullptr) atomicExch(status, kStatusPeerTimeout);
    *reinterpret_cast<uint2*>(op) = make_uint2(0u, 0u);
    if (lane == 0 && m_star != nullptr) m_star[bh] = -CUDART_INF_F;
    return;
  }
  constexpr int W = kD + 2;
  const float* partials = reinterpret_cast<const float*>(base + peer_data_offset(parity, world, 0, BH));
  float ms = -CUDART_INF_F;
  for (int r = 0; r < world; ++r) ms = fmaxf(ms, __ldcg(partials + (size_t(r) * BH + bh) * W + kD));
  float zs = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = 0; r < world; ++r) {
    const float* p = partials + (size_t(r) * BH + bh) * W;
    const float e = __expf(__ldcg(p + kD) - ms);
    zs += e * __ldcg(p + kD + 1);
    acc.x += e * __ldcg(p + 4 * lane + 0);
    acc.y += e * __ldcg(p + 4 * lane + 1);
    acc.z += e * __ldcg(p + 4 * lane + 2);
    acc.w += e * __ldcg(p + 4 * lane + 3);
  }
  const float inv = (S_per_tile > 0 && zs > 0.f) ? 1.0f / (zs * (float)S_per_tile) : 0.f;
  uint2 wv;
  wv.x = uint32_t(Store16<TK>::bits(acc.x * inv)) | (uint32_t(Store16<TK>::bits(acc.y * inv)) << 16);
  wv.y = uint32_t(Store16<TK>::bits(acc.z * inv)) | (uint32_t(Store16<TK>::bits(acc.w * inv)) << 16);
  *reinterpret_cast<uint2*>(op) = wv;
  if (lane == 0 && m_star != nullptr) m_star[bh] = ms;
  if (counted && lane == 0) {
    // the last row to finish advances the step counter: every row has read it by then
    __threadfence();
    if (atomicAdd(ctl + kPeerDoneIndex, 1) == BH - 1) {
      ctl[kPeerDoneIndex] = 0;
      __threadfence();
      atomicAdd(ctl + kPeerStepIndex, 1);
    }
  }
}

cudaError_t launch_lse_combine_wait(unsigned char* local_base, int world, unsigned epoch, int BH,
                                    int S_per_tile, int dtype, void* out, float* m_star, int* status,
                                    cudaStream_t stream) {
  if (dtype == 0)
    lse_combine_wait_kernel<__nv_bfloat16><<<BH, 32, 0, stream>>>(local_base, world, epoch, BH, S_per_tile,
                                                                 static_cast<__nv_bfloat16*>(out), m_star, status);
  else
    lse_combine_wait_kernel<__half><<<BH, 32, 0, stream>>>(local_base, world, epoch, BH, S_per_tile,
                                                          static_cast<__half*>(out), m_star, status);
  return cudaGetLastError();
}

cudaError_t launch_lse_combine(const float* partials, int G, int BH, int S_per_tile, int dtype, void* out,
                               float* m_star, cudaStream_t stream) {
  if (dtype == 0)
    lse_combine_kernel<__nv_bfloat16><<<BH, 32, 0, stream>>>(partials, G, BH, S_per_tile,
                                                            static_cast<__nv_bfloat16*>(out), m_star);
  else
    lse_combine_kernel<__half><<<BH, 32, 0, stream>>>(partials, G, BH, S_per_tile, static_cast<__half*>(out), m_star);
  return cudaGetLastError();
}

}  // namespace santa
