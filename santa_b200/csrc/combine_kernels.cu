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
  combine_rows<TK>(partials + size_t(bh) * W, size_t(BH) * W, G, S_per_tile, lane, out + size_t(bh) * kD,
                   m_star ? m_star + bh : nullptr);
}

// The receiving half of the peer exchange as a kernel of its own.  One warp per (batch, head) row: lane
// r < world polls sender r's arrival counter (every sender adds 1 per row it has delivered, `expected` in
// total by this epoch) with system-scope acquire loads and a bounded, sleeping wait; then the rows are
// combined as above.
template <typename TK>
__global__ void __launch_bounds__(32) lse_combine_wait_kernel(unsigned char* __restrict__ base, int world,
                                                              unsigned epoch_arg, int BH, int S_per_tile,
                                                              TK* __restrict__ out, float* __restrict__ m_star,
                                                              int* __restrict__ status) {
  cudaGridDependencySynchronize();  // a programmatic dependent of the decode call that sends this rank's rows
  const int bh = blockIdx.x, lane = threadIdx.x;
  int* ctl = reinterpret_cast<int*>(base);
  // epoch 0: count the epochs on the device (the same launch, replayed from a graph, serves every step)
  const bool counted = epoch_arg == 0;
  const unsigned epoch = counted ? unsigned(__ldcg(ctl + kPeerStepIndex)) + 1u : epoch_arg;
  const int parity = int(epoch & 1u);
  // every sender has added BH to its counter of this parity once per epoch of that parity so far
  const unsigned expected = ((epoch + unsigned(parity)) >> 1) * unsigned(BH);
  const bool ok = peer_wait(ctl + parity * kMaxPeers + lane, lane < world, expected, true);
  TK* op = out + size_t(bh) * kD;
  if (!ok) {  // report and leave a defined result
    if (lane == 0) {
      if (status != nullptr) atomicExch(status, kStatusPeerTimeout);
      atomicExch(ctl + kPeerStatusIndex, kStatusPeerTimeout);
      if (m_star != nullptr) m_star[bh] = -CUDART_INF_F;
    }
    *reinterpret_cast<uint2*>(op + 4 * lane) = make_uint2(0u, 0u);
  } else {
    constexpr int W = kD + 2;
    const float* rows = reinterpret_cast<const float*>(base + peer_data_offset(parity, world, 0, BH)) + size_t(bh) * W;
    combine_rows<TK>(rows, size_t(BH) * W, world, S_per_tile, lane, op, m_star ? m_star + bh : nullptr);
  }
  if (counted && lane == 0) peer_step_done(ctl, BH);
}

cudaError_t launch_lse_combine_wait(unsigned char* local_base, int world, unsigned epoch, int BH,
                                    int S_per_tile, int dtype, void* out, float* m_star, int* status,
                                    cudaStream_t stream) {
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(BH));
  cfg.blockDim = dim3(32);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (dtype == 0)
    return cudaLaunchKernelEx(&cfg, lse_combine_wait_kernel<__nv_bfloat16>, local_base, world, epoch, BH, S_per_tile,
                              static_cast<__nv_bfloat16*>(out), m_star, status);
  return cudaLaunchKernelEx(&cfg, lse_combine_wait_kernel<__half>, local_base, world, epoch, BH, S_per_tile,
                            static_cast<__half*>(out), m_star, status);
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
