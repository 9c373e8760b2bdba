// rope_kernels.cu -- the step in front of the decode-attention call, fused into one launch:
// rotary position embedding of the new token's q and k, append of the rotated k and of v to the
// NHD cache at the token's position, and the packed q [B,H,D] the attention kernels read.
//
// Replaces, bit for bit, this sequence of the reference runtime
// (tutorial_code/runtime_common.py:540-556):
//     q,k,v = view(B,1,heads,D).transpose(1,2).contiguous()
//     q, k = apply_rotary_pos_emb(q, k, cos, sin)       (runtime_common.py:165-185)
//     kc[:, pos].copy_(k[:, :, 0, :]);  vc[:, pos].copy_(v[:, :, 0, :])
//     q_bhd = q[:, :, 0, :].contiguous()
// which is a dozen small elementwise launches and copies per layer.
//
// Arithmetic of apply_rotary_pos_emb on 16-bit tensors: every elementwise op computes in fp32 and
// rounds its result to the storage type, so
//     x_embed[d] = rn( rn(x[d]*cos[d]) + rn(rot[d]*sin[d]) ),   rot = cat(-x[64:], x[:64]).
// The products of two 16-bit values are exact in fp32; the three roundings are reproduced here.
// Compiled without fast-math; the explicit _rn intrinsics keep the compiler from fusing them.

#include "common.cuh"
#include "santa_abi_internal.h"

namespace santa {

template <typename TK>
__device__ __forceinline__ float rn16(float x) {
  return Store16<TK>::round(x);
}

// One warp per head vector of 128 elements; lane l owns dims 4l..4l+3, its rotation partner is
// lane l^16.  Vectors: B*H of q, then B*KVH of k, then B*KVH of v.
template <typename TK>
__global__ void __launch_bounds__(128) rope_append_kernel(const RopeAppendParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nq = p.B * p.H, nk = p.B * p.KVH;
  if (warp >= nq + 2 * nk) return;
  int b, kind, head;
  if (warp < nq) {
    kind = 0;
    b = warp / p.H;
    head = warp - b * p.H;
  } else {
    const int r = warp - nq;
    kind = (r < nk) ? 1 : 2;
    const int rr = (r < nk) ? r : r - nk;
    b = rr / p.KVH;
    head = rr - b * p.KVH;
  }
  const int pos = p.pos_dev ? __ldg(p.pos_dev + b) : p.pos;
  // the first B warps also publish the new lengths (position + 1) for the attention call
  if (warp < p.B && lane == 0 && p.seq_lens_out != nullptr)
    p.seq_lens_out[warp] = (p.pos_dev ? __ldg(p.pos_dev + warp) : p.pos) + 1;
  const bool pos_ok = pos >= 0 && pos < p.L_storage;
  if (!pos_ok && kind != 0) {
    if (lane == 0 && p.status != nullptr) atomicExch(p.status, kStatusBadPosition);
    return;  // never write outside the cache
  }

  const unsigned char* src;
  // projections may be slices of one fused [B, (H+2*KVH)*D] tensor: per-sequence strides in elements
  if (kind == 0)
    src = static_cast<const unsigned char*>(p.q_proj) + size_t(b) * p.q_stride * 2 + size_t(head) * kRowBytes;
  else if (kind == 1)
    src = static_cast<const unsigned char*>(p.k_proj) + size_t(b) * p.k_stride * 2 + size_t(head) * kRowBytes;
  else
    src = static_cast<const unsigned char*>(p.v_proj) + size_t(b) * p.v_stride * 2 + size_t(head) * kRowBytes;
  uint2 xw = *(reinterpret_cast<const uint2*>(src) + lane);

  if (kind != 2) {
    const uint2 cw = *(reinterpret_cast<const uint2*>(static_cast<const unsigned char*>(p.cos) + size_t(b) * kRowBytes) + lane);
    const uint2 sw = *(reinterpret_cast<const uint2*>(static_cast<const unsigned char*>(p.sin) + size_t(b) * kRowBytes) + lane);
    const float2 x01 = Store16<TK>::unpack(xw.x), x23 = Store16<TK>::unpack(xw.y);
    const float2 c01 = Store16<TK>::unpack(cw.x), c23 = Store16<TK>::unpack(cw.y);
    const float2 s01 = Store16<TK>::unpack(sw.x), s23 = Store16<TK>::unpack(sw.y);
    const float x[4] = {x01.x, x01.y, x23.x, x23.y};
    const float c[4] = {c01.x, c01.y, c23.x, c23.y};
    const float s[4] = {s01.x, s01.y, s23.x, s23.y};
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float partner = __shfl_xor_sync(0xffffffffu, x[i], 16);
      const float rot = (lane < 16) ? -partner : partner;  // cat(-x2, x1)
      const float a = rn16<TK>(__fmul_rn(x[i], c[i]));
      const float r = rn16<TK>(__fmul_rn(rot, s[i]));
      y[i] = __fadd_rn(a, r);
    }
    xw.x = uint32_t(Store16<TK>::bits(y[0])) | (uint32_t(Store16<TK>::bits(y[1])) << 16);
    xw.y = uint32_t(Store16<TK>::bits(y[2])) | (uint32_t(Store16<TK>::bits(y[3])) << 16);
  }

  unsigned char* dst;
  if (kind == 0)
    dst = static_cast<unsigned char*>(p.q_out) + (size_t(b) * p.H + head) * kRowBytes;
  else
    dst = static_cast<unsigned char*>(kind == 1 ? p.k_cache : p.v_cache) +
          ((size_t(b) * p.L_storage + pos) * p.KVH + head) * kRowBytes;
  *(reinterpret_cast<uint2*>(dst) + lane) = xw;
}

cudaError_t launch_rope_append(const RopeAppendParams& p, int dtype, cudaStream_t stream) {
  const int warps = p.B * (p.H + 2 * p.KVH);
  const int grid = (warps + 3) / 4;
  if (dtype == 0)
    rope_append_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(p);
  else
    rope_append_kernel<__half><<<grid, 128, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace santa
