// santa_abi_internal.h -- parameter blocks passed from the C-ABI layer (capi.cu)
// to the kernel launchers of each translation unit.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "common.cuh"

namespace santa {

// how (column group, tile) items are dealt to the column slots of the CTAs
struct WorkSplit {
  int gw;           // columns per column group (1, 2, 4 or 8)
  int nvg;          // virtual groups that own work
  int T_c;          // tiles per column
  int ncol;         // columns = sequences * kv-heads
  long long items;  // column groups * T_c
};

// Streaming kernels: Flash decode and Prop's first pass.
struct StreamParams {
  CUtensorMap tmK;  // K as a [B][L_storage][KVH][128] 16-bit tensor, box {128,1,32,1}; with score_mma
                    // box {64,1,32,1} and the 128-byte swizzle
  int score_mma;    // 1: scores from the tensor cores (opt-in), 0: the reference's fp32 order
  const void* q;    // [B,H,128]
  const void* V;    // [B,L_storage,KVH,128]
  int H, KVH;
  int L_valid, L_storage;
  WorkSplit ws;
  int S_per_tile;  // Flash: fixed per-tile budget (uniform batch)
  int S_total;     // Flash, ragged batch: S; the per-tile budget max(1, S / T_b) follows each length
  float q_scale;
  uint64_t seed;
  int batch_offset, tile_offset;
  int* status;  // one word
  // Ragged batch (Prop pass 1): per-sequence lengths on the device, clamped to [0, L_valid];
  // null for a uniform batch.  Column groups then never span sequences (gw divides KVH) and the
  // item total is computed by the kernel.
  const int* seq_lens;  // [nseq] or null
  int nseq;
  int tile_stride;  // tiles per (sequence, head) row of m_tiles / ell_tiles
  int len_stride;   // rows per (sequence, head) row of stash / trace arrays
  // Flash: per (virtual group, column group) partials, read by the merge kernel
  float* partials;     // [nvg + column groups][gw][4][kPartialStride]
  int* partial_vrows;  // [nvg + column groups][gw]
  long long partial_slots;  // (nvg + column groups) * gw: the extent the checked build compares slots with
  // Prop pass 1 outputs / Flash trace ([B,H,T_c]); Flash: may be null
  float* m_tiles;
  float* ell_tiles;
  // Prop pass 1: rounded tile-local weights, [sequence][kv-head][len_stride][4 heads] 16-bit
  uint16_t* stash;
  // trace (may be null)
  float* dbg_invdel;  // [B,H,T_c]                    (Flash)
  uint16_t* dbg_u;    // [B,H,len_stride]             (Flash; Prop pass 1: the stash per head)
  int16_t* dbg_c;     // [B,H,L_valid]
  int* rowmask;       // [B,KVH,L_valid]
};

// Peer exchange: layout of one rank's buffer and what the kernels need of it.
//   [0, 256)   int32 control words: arrival counters [2 parities][kMaxPeers senders], then the
//              words named below
//   then       int32 row flags [2 parities][world senders][BH rows]: the epoch of the row last stored
//   then       fp32 rows      [2 parities][world senders][BH rows][130]
constexpr int kMaxPeers = 16;
constexpr size_t kPeerFlagBytes = 256;
__host__ __device__ inline size_t peer_row_flags_bytes(int world, int BH) {
  return (size_t(2) * world * BH * sizeof(int) + 255) / 256 * 256;
}
__host__ __device__ inline size_t peer_row_flag_offset(int parity, int world, int sender, int BH) {
  return kPeerFlagBytes + ((size_t(parity) * world + sender) * BH) * sizeof(int);
}
__host__ __device__ inline size_t peer_data_offset(int parity, int world, int sender, int BH) {
  return kPeerFlagBytes + peer_row_flags_bytes(world, BH) + ((size_t(parity) * world + sender) * BH) * 130 * sizeof(float);
}
struct PeerScatter {
  int world, rank;                // world == 0: no exchange
  unsigned epoch;                 // 0: the epoch is the local buffer's step counter + 1
  int combine;                    // 1: the sending kernel also waits for the other ranks' rows and combines
  unsigned char* base[kMaxPeers]; // every rank's buffer as mapped here
};

struct FlashMergeParams {
  int H, KVH, S_per_tile;
  // ragged batch: device lengths (else null), their bound, the tile size and S
  const int* seq_lens;
  int nseq, max_len, bn, S_total;
  WorkSplit ws;
  const float* partials;
  const int* partial_vrows;
  long long partial_slots;
  void* out;           // [B,H,128] storage dtype or nullptr
  float* m_star;       // [B,H] or nullptr
  int* vrows;          // [B,KVH] or nullptr
  float* partial_out;  // [B,H,130] or nullptr
  PeerScatter px;      // also store the partial into every rank's exchange buffer
  int* status;         // the workspace's status word
};

cudaError_t launch_flash(const StreamParams& p, const FlashMergeParams& mp, int dtype, int block_n, int grid,
                         cudaStream_t stream);

// Prop: pass 1 (vec streaming or tensor-core), budgets, pass 2, merge.
struct PropParams {
  StreamParams sp;      // pass 1 (vec path) -- also carries q, V, H, KVH, L, ws, status, stash, m/ell tiles
  const void* K;        // [L,KVH,D]
  int D;                // head dimension; with H / KVH != 4 or D != 128 the generic pass 2 / merge run
  int block_n, T_c;
  int use_vec;          // 1: streaming vec pass 1, 0: tensor-core pass 1
  int S;
  int flags;            // bit0/bit1: fma contraction choices of the budget step
  // workspace tables [H,T_c]
  int* S_tiles;
  float* invdelta;
  float* a0;
  float* m_star;        // [H] output
  // pass 2 partials
  float* partials;      // [nvg + column groups][gw][4][128]; generic shapes: [KVH][T_c][GH][D]
  int* partial_vrows;
  // outputs
  void* out;            // [H,128] storage dtype
  int* vrows;           // [KVH] or nullptr
  // trace (may be null)
  int16_t* dbg_c;       // [H,L]
  int* rowmask;         // [KVH,L]
};

cudaError_t launch_prop(const PropParams& p, int dtype, int grid, cudaStream_t stream);
int prop_pass2_max_groups(int sms);

// RoPE of the new token's q/k + append of k/v to the cache + packed q.
struct RopeAppendParams {
  const void* q_proj;   // [B,H,128], sequences q_stride elements apart
  const void* k_proj;   // [B,KVH,128]
  const void* v_proj;   // [B,KVH,128]
  long long q_stride, k_stride, v_stride;
  const void* cos;      // [B,128]
  const void* sin;      // [B,128]
  int B, H, KVH, L_storage;
  int pos;              // host position, used when pos_dev is null
  const int* pos_dev;   // [B] device positions or null
  void* k_cache;        // [B,L_storage,KVH,128]
  void* v_cache;
  void* q_out;          // [B,H,128]
  int* seq_lens_out;    // [B] or null: position + 1
  int* status;          // one word or null
};
cudaError_t launch_rope_append(const RopeAppendParams& p, int dtype, cudaStream_t stream);

// Cross-device combine of G unnormalised partials [G][BH][130].
// Wait for `world` partials of one parity in the local exchange buffer, then combine them.
// epoch == 0: the epoch is the buffer's own step counter + 1, advanced by the kernel when it is done.
cudaError_t launch_lse_combine_wait(unsigned char* local_base, int world, unsigned epoch, int BH,
                                    int S_per_tile, int dtype, void* out, float* m_star, int* status,
                                    cudaStream_t stream);
cudaError_t launch_lse_combine(const float* partials, int G, int BH, int S_per_tile, int dtype, void* out,
                               float* m_star, cudaStream_t stream);

}  // namespace santa
