// santa_abi_internal.h -- parameter blocks passed from the C-ABI layer (capi.cu)
// to the kernel launchers of each translation unit.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace santa {

struct FlashParams {
  CUtensorMap tmK;  // K as a [B][L_storage][KVH][128] 16-bit tensor, box {128,1,16,1}
  const void* q;  // [B,H,128]
  const void* K;  // [B,L_storage,KVH,128]
  const void* V;
  int B, H, KVH;
  int L_valid, L_storage;
  int T_c;         // tiles per sequence in this call
  int S_per_tile;  // fixed per-tile budget
  float q_scale;
  uint64_t seed;
  int batch_offset, tile_offset;
  int ncol;         // B*KVH columns
  long long items;  // column groups * T_c
  // workspace (written here, read by the merge kernel)
  int* status;         // one word
  float* partials;     // [grid + column groups][8][4][kPartialStride]
  int* partial_vrows;  // [grid + column groups][8]
  // trace
  float* dbg_m;
  float* dbg_ell;
  uint16_t* dbg_u;
  int16_t* dbg_c;
  int* rowmask;
};

struct FlashMergeParams {
  int H, KVH, T_c, S_per_tile;
  long long items;
  int ctas;  // grid of the decode kernel
  const float* partials;
  const int* partial_vrows;
  void* out;           // [B,H,128] storage dtype or nullptr
  float* m_star;       // [B,H] or nullptr
  int* vrows;          // [B,KVH] or nullptr
  float* partial_out;  // [B,H,130] or nullptr
};

cudaError_t launch_flash(const FlashParams& p, const FlashMergeParams& mp, int dtype, int block_n, int grid,
                         cudaStream_t stream);

}  // namespace santa
