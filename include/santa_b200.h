/*
 * santa_b200.h -- C ABI of the B200 (sm_100a) S2ANTA decode-attention library.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless the
 * comment says otherwise; `stream` is a cudaStream_t passed as void*.  All
 * entry points are asynchronous on `stream`, never synchronise the host, and
 * never allocate: scratch memory is a caller-provided workspace (one entry
 * point, santa_flash_decode_noalloc, brings its own fixed scratch instead).
 * Return value: 0 on success, a negative SANTA_E_* code otherwise
 * (santa_strerror() gives the text).  There is no CPU fallback anywhere in the
 * library.
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
#define SANTA_E_SHAPE (-2)      /* unsupported H/KVH/D combination (see each entry point) */
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

/* Exchange of Flash partials between the ranks of a sequence-sharded decode through peer-mapped device
 * memory (NVLink), without a collective library.  Every rank owns one exchange buffer of
 * santa_peer_exchange_bytes() bytes, zero-filled once, and maps all of them (CUDA IPC, symmetric memory):
 * peer_buffer[r] is the address of rank r's buffer in THIS process.  A decode call whose ext names a
 * santa_peer_exchange stores its [B,H,130] partial into every rank's buffer (plain peer stores, then a
 * system-scope release of a per-sender arrival counter); santa_lse_combine_wait() on every rank waits,
 * with a bound, until all `world` partials of the same epoch have arrived in its own buffer and folds
 * them.  `epoch` counts the steps (1, 2, 3, ...; the same value on every rank for the same step);
 * buffers alternate with its parity, so the ranks only have to stay within one step of each other --
 * which the wait itself guarantees.  epoch == 0 on every rank selects device-counted epochs: each
 * buffer carries its own step counter, read by the kernels and advanced by santa_lse_combine_wait, so
 * that a decode + wait pair captured once in a CUDA graph can be replayed for every step.
 * With SANTA_PEER_COMBINE in `flags` the decode call does the receiving half itself: the kernel that
 * stored a row waits (bounded) for the same row from every other rank and writes the combined `out` /
 * `m_star` of santa_flash_decode -- one call per step, no santa_lse_combine_wait.  A wait that ran out
 * leaves zeros in its rows and 4 in the workspace's status word and in santa_peer_exchange_status();
 * the step still counts, so that this rank stays in step with the others; after such a failure all
 * ranks re-zero their buffers behind a barrier before the exchange is used again.
 * No counterpart in the reference (single device). */
#define SANTA_PEER_COMBINE 1u
typedef struct santa_peer_exchange {
  int world;             /* ranks taking part, 1..16 */
  int rank;              /* this rank */
  uint32_t epoch;        /* >= 1, or 0 = counted on the device */
  uint32_t flags;        /* 0 or SANTA_PEER_COMBINE */
  void* peer_buffer[16]; /* [world] used */
} santa_peer_exchange;

/* How the scores q.K are formed (santa_flash_ext.score_mode, santa_prop_ext.score_mode).
 *   SANTA_SCORE_EXACT   fp32 multiply-adds in the reference's order (F.cu:161-221, P.cu:317-379): the
 *                       sampled row counts equal the reference's bit for bit.  The default.
 *   SANTA_SCORE_TENSOR  tensor cores (mma.sync m16n8k16, fp32 accumulate); the fp32-scaled query is
 *                       split into two 16-bit parts, so the scores agree with the exact ones to about
 *                       1e-6 relative, but not bit for bit: on rare rows a sampled count moves to a
 *                       neighbouring row.  Takes the score arithmetic off the fp32 pipe, which is
 *                       what bounds the exact mode.  Opt-in; never chosen by the library itself. */
#define SANTA_SCORE_EXACT 0
#define SANTA_SCORE_TENSOR 1

typedef struct santa_flash_ext {
  /* Added to the batch index in the RNG key (head index b*H+h, F.cu:281) so that a batch-sharded
   * call reproduces the unsharded call's samples.  0 = reference behaviour. */
  int batch_offset;
  /* Global index of this call's tile 0 in the RNG key, for a sequence-sharded call.  0 = reference. */
  int tile_offset;
  /* If >= 0, replaces the S_per_tile computed from S and this call's own tile count (a sequence
   * shard must use the budget of the WHOLE sequence).  -1 = reference rule. */
  int s_per_tile_override;
  int score_mode; /* SANTA_SCORE_EXACT (0, the reference's arithmetic) or SANTA_SCORE_TENSOR */
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
  /* [B,H,T_c] fp32 or NULL: the per-tile sampling step S_per_tile/ell_t as the device computed it
   * (an approximate division, F.cu:279-280). */
  float* invdel;
  /* If not NULL: the partial (as partial_out) is also stored into every rank's exchange buffer. */
  const santa_peer_exchange* peer;
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
 *   out    [B,H,D]            storage dtype; device memory, or pinned (device-accessible) host memory --
 *                             the merge kernel then stores the result over the bus, no separate copy
 *   m_star [B,H]              fp32, max scaled score per head
 *   vrows  [B,KVH] int32 or NULL: number of distinct V rows gathered
 * Requires D == 128, H == 4*KVH, block_n in {0,32,64,256}, 16-byte aligned q/K/V/out.
 * S <= 0 is legal and yields zeros.
 *
 * workspace: santa_flash_workspace_bytes() bytes, 256-byte aligned.  Zero-fill it once before its
 * first use (only the status word has to start at 0).  Calls that share a workspace must be
 * ordered on one stream.  The first int32 after the call is a status word
 * (santa_workspace_status()).
 */
SANTA_API int santa_flash_decode(const void* q, const void* K, const void* V, int dtype, int B, int H, int KVH, int D,
                       int L_valid, int L_storage, int64_t S, uint64_t seed, int block_n, void* out,
                       float* m_star, int32_t* vrows, void* workspace, size_t workspace_bytes,
                       const santa_flash_ext* ext, void* stream);

/* Device address of the int32 status word inside a workspace.  0 = ok; 1 = a staged K piece never
 * arrived, 2 = a score buffer was never handed over (the result is invalid); 3 = santa_rope_append
 * skipped a position outside the cache; 4 = a rank's rows never arrived in a peer exchange; 5 = the
 * bounds-checked build of the library (-DSANTA_B200_CHECKS) caught an index outside its array and
 * skipped the access.  The word is sticky.  Read it after synchronising the stream. */
SANTA_API int32_t* santa_workspace_status(void* workspace);

/*
 * The same decode as santa_flash_decode for callers that cannot hand over a workspace: inference
 * servers that give all free device memory to their KV-cache pool at start-up and forbid any
 * allocation on the decode path (cudaMalloc stalls the whole device and may fail once memory is
 * fragmented), and plain C / cgo hosts that have no device allocator of their own.  The scratch
 * lives in a fixed SANTA_NOALLOC_SCRATCH_BYTES array inside the library; the entry point calls no
 * cudaMalloc, cudaFree or any allocating routine.  This entry point has no counterpart in the
 * reference.
 *
 * Arguments, results and error codes are those of santa_flash_decode without the workspace pair.
 * A problem whose scratch need (santa_flash_workspace_bytes) exceeds SANTA_NOALLOC_SCRATCH_BYTES is
 * rejected with SANTA_E_TOO_LARGE before anything is launched; with 8 kv-heads that is roughly
 * more than 100 sequences per call.
 *
 * The first call on a device looks up the device address of the array (with that device current).
 * Under CUDA's lazy module loading that first call is also the moment the device sets the array's
 * 4 MiB aside -- from then on every such GPU holds them until the process exits -- so make it
 * before the device's free memory is given away (a KV-cache pool sized to "all that is left"), and
 * outside any stream capture.  All calls on a device share the one array and nothing in it is
 * cleared between calls: every call overwrites what it reads, except the status word, which starts
 * at zero when the module is loaded and from then on only changes when a bounded wait inside a
 * kernel ran out (1 or 2, see santa_workspace_status; the result of that call is invalid).  Read it
 * through santa_noalloc_status() after synchronising the stream; a caller that has seen a non-zero
 * value puts it back to zero itself (cudaMemsetAsync on that address).  Two calls whose kernels
 * may overlap on the GPU (different streams, no ordering) race on the array -- order them.
 */
#define SANTA_NOALLOC_SCRATCH_BYTES (4u << 20)
SANTA_API int santa_flash_decode_noalloc(const void* q, const void* K, const void* V, int dtype, int B, int H, int KVH,
                               int D, int L_valid, int L_storage, int64_t S, uint64_t seed, int block_n, void* out,
                               float* m_star, int32_t* vrows, const santa_flash_ext* ext, void* stream);

/* Device address of the status word santa_flash_decode_noalloc uses on the CURRENT device, or NULL
 * before that entry point's first call on it.  No counterpart in the reference. */
SANTA_API int32_t* santa_noalloc_status(void);

/* Bytes of workspace santa_flash_decode_ragged needs on the current device (0 on bad arguments). */
SANTA_API size_t santa_flash_ragged_workspace_bytes(int B, int KVH, int max_len, int block_n);

/*
 * S2ANTA-Flash decode attention with PER-SEQUENCE LENGTHS READ FROM DEVICE MEMORY.  No counterpart
 * in the reference, whose entry point takes one host-side valid_len for the whole batch
 * (F.cpp:188-191): this is the variant for a decode step captured once in a CUDA graph and replayed
 * while the cache grows -- the step before it (tutorial_code/runtime_common.py:551-557) bumps the
 * lengths on the device -- and for batches whose sequences differ in length.
 * Sequence b gets exactly the result of santa_flash_decode on that sequence alone with
 * L_valid = seq_lens[b], the same block_n and ext.batch_offset = batch_offset + b (the random stream
 * is keyed by b*H + h, F.cu:281); with all lengths equal to L it therefore equals the uniform call
 * with valid_len = L.  The per-tile budget max(1, S / ceil(len_b / block_n)) follows each length.
 *
 *   seq_lens [B] int32 in DEVICE memory, read when the kernels run; clamped to [0, max_len]
 *   max_len  host-side bound, 0 < max_len <= L_storage; sizes the workspace
 *   block_n  32, 64 or 256; <= 0 applies the reference's rule to max_len.  The host cannot see
 *            the lengths, so a caller that wants the rule's tile size re-plans (and re-captures)
 *            when its lengths cross 1536 / 3072.
 * Other arguments as santa_flash_decode (out is required).  A sequence of length 0 yields a zero
 * output row.  B <= 1024.  Of `ext` only batch_offset and the trace arrays may be set; the trace
 * arrays are laid out [B,H,ceil(max_len/block_n)] and [B,H,max_len] (rowmask [B,KVH,max_len]).
 */
SANTA_API int santa_flash_decode_ragged(const void* q, const void* K, const void* V, int dtype, int B, int H, int KVH,
                                        int D, int L_storage, const int32_t* seq_lens, int max_len, int64_t S,
                                        uint64_t seed, int block_n, void* out, float* m_star, int32_t* vrows,
                                        void* workspace, size_t workspace_bytes, const santa_flash_ext* ext,
                                        void* stream);

/* ---- Prop decode ----------------------------------------------------------- */

typedef struct santa_prop_ext {
  /* First-pass kernel choice, the reference's SANTA_PASS1 switch (P.cpp:39-51): 0 = auto (streaming
   * vec kernel when block_n == 256, tensor-core kernel otherwise), 1 = force the tensor-core kernel,
   * 2 = force the vec kernel (block_n <= 0 then means 256; any other block_n is an error). */
  int pass1_mode;
  /* Rounding choices of the budget step that the reference leaves to its compiler: bit0 = the 1e-7
   * jitter is added with one fused multiply-add, bit1 = the per-thread partial sums of Z use a fused
   * multiply-add.  The default (no ext) is 3. */
  int flags;
  /* Trace outputs, each may be NULL; when given they are used instead of workspace memory.
   * m_tiles, ell_tiles: [H,T_c] fp32; u16: [H,L] storage-type bits of the rounded tile-local weights
   * (the reference's u_stash, transposed); counts: [H,L] int16 sampled row counts; rowmask: [KVH,L]
   * int32 set to 1 on gathered rows (caller zero-fills); S_tiles: [H,T_c] int32 per-tile budgets;
   * invdelta, a0: [H,T_c] fp32 per-tile step and offset. */
  float* m_tiles;
  float* ell_tiles;
  uint16_t* u16;
  int16_t* counts;
  int32_t* rowmask;
  int32_t* S_tiles;
  float* invdelta;
  float* a0;
  /* SANTA_SCORE_EXACT (0) or SANTA_SCORE_TENSOR: applies to the streaming first pass (block_n == 256);
   * the small-tile first pass already is the reference's own tensor-core arithmetic. */
  int score_mode;
  int reserved;
} santa_prop_ext;

/* Bytes of workspace santa_prop_decode needs on the current device for this problem. */
SANTA_API size_t santa_prop_workspace_bytes(int H, int KVH, int D, int L, int block_n);

/*
 * S2ANTA-Prop decode attention for ONE sequence.  Replaces the launch sequence of
 * decode_systematic_scalar, P.cpp:270-352 (launch_pass1_tiles_{vec,wmma}_gqa_{bf16,f16},
 * launch_tile_budgets, launch_pass2_grouped_fused_atomic_{bf16,f16}, launch_cast_scale_out_{bf16,f16},
 * launch_reduce_vrows; declared P.cpp:81-138).
 *
 *   q      [H,D]       storage dtype, contiguous
 *   K, V   [L,KVH,D]   storage dtype, contiguous (every row is used)
 *   out    [H,D]       storage dtype
 *   m_star [H]         fp32
 *   vrows  [KVH] int32 or NULL
 * Shapes: any H % KVH == 0 with up to 8 query heads per kv-head and any D % 16 == 0 up to 256, like
 * the reference (P.cpp:212-247; its second pass launches 128 x GH threads, P.cu:924-927, hence the 8).
 * H == 4*KVH with D == 128 runs the vectorised kernels (streaming first pass when block_n == 256),
 * every other shape the tensor-core first pass and a generic second pass, both with the reference's
 * arithmetic.  block_n <= 0 (auto) or a multiple of 16 up to 256; at most 11 622 tiles per sequence
 * (2.9 M tokens at 256-row tiles; SANTA_E_TOO_LARGE beyond).
 * The output is summed in a fixed order, so repeated calls give identical bits (the reference
 * accumulates with atomics and does not).  Workspace rules as for santa_flash_decode.
 */
SANTA_API int santa_prop_decode(const void* q, const void* K, const void* V, int dtype, int H, int KVH, int D, int L,
                      int64_t S, uint64_t seed, int block_n, void* out, float* m_star, int32_t* vrows,
                      void* workspace, size_t workspace_bytes, const santa_prop_ext* ext, void* stream);

/* Bytes of workspace santa_prop_decode_ragged needs on the current device (0 on bad arguments). */
SANTA_API size_t santa_prop_ragged_workspace_bytes(int B, int H, int KVH, int D, int max_len);

/*
 * S2ANTA-Prop decode attention for a RAGGED BATCH in one launch sequence.  Replaces the per-sequence
 * loop the reference's adapter runs over decode_systematic_scalar
 * (tutorial_code/attention_backends.py:491-500): sequence b gets exactly the result of
 * santa_prop_decode(q[b], K[b,:len_b], V[b,:len_b], ..., block_n = 256) -- the same tile statistics,
 * budgets, random offsets (keyed by the head index h, not b*H+h, as in the loop) and sampled row counts;
 * outputs agree up to the fp32 order in which per-warp partial sums are added.
 *
 *   q        [B,H,D]             storage dtype, contiguous
 *   K, V     [B,L_storage,KVH,D] storage dtype, contiguous; rows [0, len_b) of sequence b are used
 *   seq_lens [B] int32 in DEVICE memory, read by the kernels when they run (so a captured CUDA graph
 *            follows lengths that change between replays); each entry is clamped to [0, max_len]
 *   max_len  host-side bound on the lengths, 0 < max_len <= L_storage; sizes the workspace
 *   out      [B,H,D] storage dtype;  m_star [B,H] fp32;  vrows [B,KVH] int32 or NULL
 * Tiles are 256 rows (what the reference's rule picks for every length above 3072; a shorter sequence
 * gets the result of the per-sequence call with block_n = 256, not of its 32/64-row rule).  A
 * sequence of length 0 yields a zero output row.  B <= 1024.  Trace arrays of `ext` are laid out
 * [B,H,ceil(max_len/256)] and [B,H,max_len] (rowmask [B,KVH,max_len]); pass1_mode must be 0 or 2.
 */
SANTA_API int santa_prop_decode_ragged(const void* q, const void* K, const void* V, int dtype, int B, int H, int KVH,
                                       int D, int L_storage, const int32_t* seq_lens, int max_len, int64_t S,
                                       uint64_t seed, void* out, float* m_star, int32_t* vrows, void* workspace,
                                       size_t workspace_bytes, const santa_prop_ext* ext, void* stream);

/* ---- the step in front of the attention call -------------------------------- */

/*
 * Rotary embedding of the new token's q and k, append of k and v to the cache, packed q -- one
 * launch.  Replaces the tensor code between the projections and the attention call in the
 * reference runtime, tutorial_code/runtime_common.py:540-556 (view/transpose/contiguous,
 * apply_rotary_pos_emb :165-185, kc[:, pos].copy_, vc[:, pos].copy_, q[:, :, 0, :].contiguous()),
 * with the same three roundings per element: rn(rn(x*cos) + rn(rotate_half(x)*sin)).
 *
 *   q_proj [B,H,D], k_proj/v_proj [B,KVH,D]   the projections of ONE new token per sequence
 *   q_stride, k_stride, v_stride              elements between consecutive sequences of each projection
 *                                             (multiples of 4); <= 0 means dense.  Slices of one fused
 *                                             [B,(H+2*KVH)*D] projection are passed without a copy
 *   cos, sin [B,D]                            rotary tables of each sequence's position
 *   k_cache, v_cache [B,L_storage,KVH,D]      row `position` of every sequence is overwritten
 *   pos       host position of all sequences, used when pos_dev is NULL (0 <= pos < L_storage)
 *   pos_dev   [B] int32 positions in DEVICE memory or NULL; read when the kernel runs; a position
 *             outside [0, L_storage) is skipped (nothing is written for that sequence's k/v) and
 *             *status, if given, is set to 3
 *   q_out [B,H,D]                             rotated q, the layout santa_flash_decode reads
 *   seq_lens_out [B] int32 or NULL            position + 1: the lengths for the *_ragged decode calls
 *   status  one int32 in device memory or NULL
 * All tensors in the storage dtype, contiguous, 8-byte aligned; D == 128.  q_proj, k_proj and v_proj may
 * also point into pinned (page-locked, device-mapped) host memory: the kernel reads them over PCIe,
 * which replaces a separate host-to-device copy of a decode step's inputs.
 */
SANTA_API int santa_rope_append(const void* q_proj, const void* k_proj, const void* v_proj, int64_t q_stride,
                                int64_t k_stride, int64_t v_stride, const void* cos, const void* sin, int dtype,
                                int B, int H, int KVH, int D, void* k_cache, void* v_cache, int L_storage, int pos,
                                const int32_t* pos_dev, void* q_out, int32_t* seq_lens_out, int32_t* status,
                                void* stream);

/* ---- split-KV combine ------------------------------------------------------- */

/* Bytes of one rank's exchange buffer for `world` ranks and BH = B*H (batch x heads) partial rows. */
SANTA_API size_t santa_peer_exchange_bytes(int world, int BH);

/* Device address of the int32 inside an exchange buffer (this rank's own) that becomes 4 when a
 * bounded wait on that buffer ran out.  Read it after synchronising the stream. */
SANTA_API int32_t* santa_peer_exchange_status(void* own_buffer);

/*
 * The receiving half of the peer exchange: wait until the partials of px->epoch from all px->world
 * ranks have arrived in this rank's buffer (px->peer_buffer[px->rank]), then combine them exactly as
 * santa_lse_combine does.  The wait is bounded (about a second); when it runs out the kernel writes 4
 * to *status (device int32, may be NULL), stores zeros and returns, so the context stays usable.
 * Asynchronous on `stream`; call it after the decode call of the same epoch.
 */
SANTA_API int santa_lse_combine_wait(const santa_peer_exchange* px, int BH, int D, int S_per_tile, int dtype,
                                     void* out, float* m_star, int32_t* status, void* stream);

/*
 * Combine G unnormalised Flash partials (santa_flash_ext.partial_out of G calls over disjoint tile
 * sets of the same sequences): partials is [G][BH][130] fp32 -- A[128], m, Z.  Writes
 * out [BH,128] (storage dtype) = sum_r e^{m_r-m*} A_r / (S_per_tile * sum_r e^{m_r-m*} Z_r) and
 * m_star [BH] (may be NULL).  This is the reference's finalize (F.cu:386-470) over the union of the
 * tiles; the reference itself has no multi-device path.
 */
SANTA_API int santa_lse_combine(const float* partials, int G, int BH, int D, int S_per_tile, int dtype, void* out,
                      float* m_star, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SANTA_B200_H_ */
