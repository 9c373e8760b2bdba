/*
 * santa_b200.h -- C ABI of the B200 (sm_100a) S2ANTA decode-attention library.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless the
 * comment says otherwise; `stream` is a cudaStream_t passed as void*.  All
 * entry points are asynchronous on `stream`, never synchronise the host, and
 * never allocate: scratch memory is a caller-provided workspace.  Return value:
 * 0 on success, a negative SANTA_E_* code otherwise (santa_strerror() gives
 * the text).  There is no CPU fallback anywhere in the library.
 *
 * Each entry point names the reference interface it replaces, by file:line in
 * the OPUSLab/SANTA tree:
 *   F.cpp = flash_style_fused_santa_fixed_tile_budgets/santa_cuda.cpp
 *   F.cu  = flash_style_fused_santa_fixed_tile_budgets/santa_cuda_kernel.cu
 *   P.cpp = santa_fused_proportional_tile_budgets/santa_cuda.cpp
 *   P.cu  = santa_fused_proportional_tile_budgets/santa_cuda_kernel.cu
 */
#ifndef SANTA_B200_H_
#define SANTA_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define SANTA_API __attribute__((visibility("default")))
#else
#define SANTA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define SANTA_DTYPE_BF16 0
#define SANTA_DTYPE_F16 1

#define SANTA_OK 0
#define SANTA_E_DTYPE (-1)      /* dtype is not SANTA_DTYPE_BF16 / SANTA_DTYPE_F16 */
#define SANTA_E_SHAPE (-2)      /* unsupported H/KVH/D combination */
#define SANTA_E_LENGTH (-3)     /* valid length <= 0 or > storage length */
#define SANTA_E_BLOCK_N (-4)    /* block_n not supported by this entry point */
#define SANTA_E_WORKSPACE (-5)  /* workspace NULL, misaligned or too small */
#define SANTA_E_ALIGN (-6)      /* q/K/V/out pointer not 16-byte aligned */
#define SANTA_E_CUDA (-7)       /* a CUDA runtime call failed; see santa_last_cuda_error() */
#define SANTA_E_ARG (-8)        /* NULL required pointer or inconsistent optional arguments */
#define SANTA_E_TOO_LARGE (-9)  /* size beyond what the no-allocation entry point supports */

SANTA_API const char* santa_strerror(int code);
/* cudaError_t value of the most recent failing CUDA call made by the library on this host thread. */
SANTA_API int santa_last_cuda_error(void);
/* Library ABI version (bumped on any signature change). */
SANTA_API int santa_abi_version(void);

/* ---- host-side rules (pure functions, no CUDA) --------------------------- */

/* Tile size from the valid length: explicit block_n > 0 wins, else L<=1536 -> 32,
 * L<=3072 -> 64, else 256.  Replaces _normalize_block_n, F.cpp:36-44 / P.cpp:61-77. */
SANTA_API int santa_block_n_rule(int L_valid, int block_n);

/* Tiles and fixed per-tile budget: T_c = ceil(L/block_n), S_per_tile = S>0 ? max(1, S/T_c) : 0.
 * Replaces F.cpp:202-208. */
SANTA_API void santa_flash_budget(int L_valid, int block_n, int64_t S, int* T_c, int* S_per_tile);

/* Per-(head, tile) stratification offset in [0,1].  Replaces u01_from_seed, F.cu:74-87 == P.cu:557-570. */
SANTA_API float santa_u01(uint64_t seed, int head_index, int tile_index);

/* ---- optional extensions of the Flash decode ------------------------------ */

typedef struct santa_flash_ext {
  /* Added to the batch index in the RNG key (head index b*H+h, F.cu:281) so that a batch-sharded
   * call reproduces the unsharded call's samples.  0 = reference behaviour. */
  int batch_offset;
  /* Global index of this call's tile 0 in the RNG key, for a sequence-sharded call.  0 = reference. */
  int tile_offset;
  /* If >= 0, replaces the S_per_tile computed from S and this call's own tile count (a sequence
   * shard must use the budget of the WHOLE sequence).  -1 = reference rule. */
  int s_per_tile_override;
  int reserved0;
  /* If not NULL: [B,H,130] fp32 unnormalised partial result per head -- A[128], m, Z -- such that
   * out = A / (Z * S_per_tile) and partials of disjoint tile sets combine with santa_lse_combine().
   * `out` may then be NULL. */
  float* partial_out;
  /* Debug/trace outputs, each may be NULL.  m_tiles, ell_tiles: [B,H,T_c] fp32 (the reference's
   * workspace tensors of the same names, F.cpp:219-229).  u16: [B,H,L_valid] storage-type bits of
   * the rounded tile-local weights; counts: [B,H,L_valid] int16 sampled row counts (u16 and counts
   * must be given together).  rowmask: [B,KVH,L_valid] int32, set to 1 for gathered rows (caller
   * zero-fills; F.cpp:223). */
  float* m_tiles;
  float* ell_tiles;
  uint16_t* u16;
  int16_t* counts;
  int32_t* rowmask;
} santa_flash_ext;

/* Bytes of workspace santa_flash_decode needs on the current device for this problem. */
SANTA_API size_t santa_flash_workspace_bytes(int B, int KVH, int L_valid, int block_n);

/*
 * S2ANTA-Flash decode attention for a batch of same-length sequences.
 * Replaces the launch sequence of decode_systematic_scalar/_batched, F.cpp:174-343
 * (launch_fused_tiles_vec_gqa_gh4_d128_bn{32,64,256}_{bf16,f16}, launch_finalize_weighted_{bf16,f16},
 * launch_reduce_vrows; declared F.cpp:56-120).
 *
 *   q      [B,H,D]            storage dtype, contiguous
 *   K, V   [B,L_storage,KVH,D] storage dtype, contiguous; rows [0,L_valid) are used
 *   out    [B,H,D]            storage dtype
 *   m_star [B,H]              fp32, max scaled score per head
 *   vrows  [B,KVH] int32 or NULL: number of distinct V rows gathered
 * Requires D == 128, H == 4*KVH, block_n in {0,32,64,256}, 16-byte aligned q/K/V/out.
 * S <= 0 is legal and yields zeros.
 *
 * workspace: santa_flash_workspace_bytes() bytes, 256-byte aligned.  It must be zero-filled once
 * before its first use; every successful call leaves it ready for the next.  Calls that share a
 * workspace must be ordered on one stream.  The first int32 after the call is a status word
 * (santa_workspace_status()).
 */
SANTA_API int santa_flash_decode(const void* q, const void* K, const void* V, int dtype, int B, int H, int KVH, int D,
                       int L_valid, int L_storage, int64_t S, uint64_t seed, int block_n, void* out,
                       float* m_star, int32_t* vrows, void* workspace, size_t workspace_bytes,
                       const santa_flash_ext* ext, void* stream);

/* Device address of the int32 status word inside a workspace (0 = ok, 1 = a staged K chunk never
 * arrived and the result is invalid).  Read it after synchronising the stream. */
SANTA_API int32_t* santa_workspace_status(void* workspace);

#ifdef __cplusplus
}
#endif
#endif /* SANTA_B200_H_ */
