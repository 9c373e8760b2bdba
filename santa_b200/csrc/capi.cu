// capi.cu -- the extern "C" boundary of libsanta_b200.so (declared in
// include/santa_b200.h): argument validation, the reference's host-side rules,
// workspace carving and kernel launches.  No allocation, no host
// synchronisation, no fallback path.

#include "../../include/santa_b200.h"
#include "common.cuh"
#include "santa_abi_internal.h"

#include <cmath>

namespace {

thread_local int g_last_cuda_error = 0;

int cuda_fail(cudaError_t e) {
  g_last_cuda_error = int(e);
  return SANTA_E_CUDA;
}

int sm_count_of_current_device(int* out) {
  static int cached[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev >= 0 && dev < 64 && cached[dev] > 0) {
    *out = cached[dev];
    return SANTA_OK;
  }
  int n = 0;
  e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev >= 0 && dev < 64) cached[dev] = n;
  *out = n;
  return SANTA_OK;
}

// cuTensorMapEncodeTiled, looked up through the runtime so that the library
// does not link against libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Tensor map of a K cache [B][L_storage][KVH][128] of 16-bit elements with a
// {128, 1, kStageRows, 1} box: one kv-head's rows of kStageRows tokens.
// swizzled: {64, 1, kStageRows, 1} boxes with the 128-byte swizzle (two per piece), the staging of
// the tensor-core score path.
int encode_k_map(CUtensorMap* tm, const void* K, int B, int L_storage, int KVH, bool swizzled = false) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return cuda_fail(cudaErrorNotSupported);
  const cuuint64_t dims[4] = {cuuint64_t(santa::kD), cuuint64_t(KVH), cuuint64_t(L_storage), cuuint64_t(B)};
  const cuuint64_t strides[3] = {cuuint64_t(santa::kRowBytes), cuuint64_t(KVH) * santa::kRowBytes,
                                 cuuint64_t(L_storage) * KVH * santa::kRowBytes};
  const cuuint32_t box[4] = {cuuint32_t(swizzled ? santa::kD / 2 : santa::kD), 1u, cuuint32_t(santa::kStageRows), 1u};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(K), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  return SANTA_OK;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Deal (column group, tile) items to the 8 column slots of each persistent CTA (the device side is
// warp_work in sampler.cuh).  For every group width the items are cut into one range per virtual
// group and the virtual groups are dealt to the CTAs in contiguous runs; the cost of a width is the
// column-tiles of its busiest CTA.  Wide groups fetch whole token rows together, so a narrower width
// only replaces a wider one when it takes at least 3 % off that cost -- which it does when the
// problem has only one or two tiles per slot and whole tiles would otherwise be dealt unevenly.
// `within` > 0 restricts the width to divisors of it (ragged batches: a column group must not
// span two sequences, so the width has to divide KVH).
santa::WorkSplit make_split(int ncol, int T_c, int sms, int* grid, int within = 0) {
  santa::WorkSplit best{};
  long long best_load = -1;
  for (int gw = santa::kGroupWarps; gw >= 1; gw >>= 1) {
    if (within > 0 && within % gw != 0) continue;
    const long long ncg = (ncol + gw - 1) / gw;
    const long long items = ncg * T_c;
    const long long slots = (long long)sms * (santa::kGroupWarps / gw);
    const long long nvg = items < slots ? items : slots;
    const long long ctas = nvg < sms ? nvg : sms;
    long long busiest = 0;  // items of the busiest CTA
    for (long long c = 0; c < ctas; ++c) {
      const long long v0 = santa::range_lo(c, nvg, ctas), v1 = santa::range_lo(c + 1, nvg, ctas);
      const long long n = santa::range_lo(v1, items, nvg) - santa::range_lo(v0, items, nvg);
      busiest = n > busiest ? n : busiest;
    }
    const long long load = busiest * gw;
    if (best_load < 0 || load * 100 < best_load * 97) {
      best_load = load;
      best.gw = gw;
      best.nvg = int(nvg);
      best.T_c = T_c;
      best.ncol = ncol;
      best.items = items;
      *grid = int(ctas);
    }
  }
  return best;
}

struct FlashPlan {
  int block_n, T_c, grid;
  santa::WorkSplit ws;
  size_t off_pvrows, off_partials, total, slots;
};

int plan_flash(int B, int KVH, int L_valid, int block_n, FlashPlan* pl) {
  if (B <= 0 || KVH <= 0) return SANTA_E_SHAPE;
  if (L_valid <= 0) return SANTA_E_LENGTH;
  const int bn = santa_block_n_rule(L_valid, block_n);
  if (bn != 32 && bn != 64 && bn != 256) return SANTA_E_BLOCK_N;
  int sms = 0;
  if (int rc = sm_count_of_current_device(&sms)) return rc;
  if (sms > santa::kMaxCtas) sms = santa::kMaxCtas;
  pl->block_n = bn;
  pl->T_c = (L_valid + bn - 1) / bn;
  pl->ws = make_split(B * KVH, pl->T_c, sms, &pl->grid);
  const size_t ncg = (size_t(B) * KVH + pl->ws.gw - 1) / pl->ws.gw;
  const size_t slots = (size_t(pl->ws.nvg) + ncg) * pl->ws.gw;
  pl->slots = slots;
  pl->off_pvrows = 256;
  pl->off_partials = pl->off_pvrows + align_up(slots * 4, 256);
  pl->total = pl->off_partials + slots * santa::kGH * santa::kPartialStride * sizeof(float);
  return SANTA_OK;
}

struct PropPlan {
  int block_n, T_c, grid, use_vec;
  santa::WorkSplit ws;
  size_t off_m, off_ell, off_S, off_inv, off_a0, off_stash, off_pvrows, off_partials, total;
};

int plan_prop(int H, int KVH, int D, int L, int block_n, int pass1_mode, PropPlan* pl) {
  // the reference takes any H % KVH == 0 and D % 16 == 0 (P.cpp:155-166, :212-247); its second pass
  // launches 128 x GH threads per block (P.cu:924-927), which bounds GH by 8
  if (KVH <= 0 || H <= 0 || H % KVH != 0 || H / KVH > 8 || D <= 0 || D % 16 != 0 || D > 256) return SANTA_E_SHAPE;
  if (L <= 0) return SANTA_E_LENGTH;
  const int GH = H / KVH;
  const bool vec_shape = GH == santa::kGH && D == santa::kD;
  int bn = block_n;
  if (bn <= 0) bn = (pass1_mode == 2) ? 256 : santa_block_n_rule(L, 0);  // P.cpp:69-77
  if (bn % 16 != 0 || bn > 256) return SANTA_E_BLOCK_N;
  if (pass1_mode == 2 && (bn != 256 || !vec_shape)) return SANTA_E_BLOCK_N;  // P.cpp:230-234
  int sms = 0;
  if (int rc = sm_count_of_current_device(&sms)) return rc;
  if (sms > santa::kMaxCtas) sms = santa::kMaxCtas;
  pl->block_n = bn;
  pl->T_c = (L + bn - 1) / bn;
  if (size_t(pl->T_c) * 20 > size_t(227) * 1024) return SANTA_E_TOO_LARGE;  // budget tables live in shared memory
  pl->use_vec = (vec_shape && bn == 256 && pass1_mode != 1) ? 1 : 0;  // P.cpp:215-229
  pl->ws = make_split(KVH, pl->T_c, sms, &pl->grid);
  const size_t ht = align_up(size_t(H) * pl->T_c * 4, 256);
  pl->off_m = 256;
  pl->off_ell = pl->off_m + ht;
  pl->off_S = pl->off_ell + ht;
  pl->off_inv = pl->off_S + ht;
  pl->off_a0 = pl->off_inv + ht;
  pl->off_stash = pl->off_a0 + ht;
  pl->off_pvrows = pl->off_stash + align_up(size_t(H) * L * 2, 256);
  if (vec_shape) {
    const size_t slots = size_t(santa::prop_pass2_max_groups(sms)) + KVH;
    pl->off_partials = pl->off_pvrows + align_up(slots * 4, 256);
    pl->total = pl->off_partials + slots * santa::kGH * santa::kD * sizeof(float);
  } else {  // one partial per (kv-head, tile): [KVH][T_c][GH][D]
    const size_t tiles = size_t(KVH) * pl->T_c;
    pl->off_partials = pl->off_pvrows + align_up(tiles * 4, 256);
    pl->total = pl->off_partials + tiles * GH * D * sizeof(float);
  }
  return SANTA_OK;
}

// Ragged Flash batch: planned for the length bound; column groups stay inside a sequence.
int plan_flash_ragged(int B, int KVH, int max_len, int block_n, FlashPlan* pl) {
  if (B <= 0 || KVH <= 0) return SANTA_E_SHAPE;
  if (B > santa::kMaxRaggedSeqs) return SANTA_E_TOO_LARGE;
  if (max_len <= 0) return SANTA_E_LENGTH;
  const int bn = santa_block_n_rule(max_len, block_n);
  if (bn != 32 && bn != 64 && bn != 256) return SANTA_E_BLOCK_N;
  int sms = 0;
  if (int rc = sm_count_of_current_device(&sms)) return rc;
  if (sms > santa::kMaxCtas) sms = santa::kMaxCtas;
  pl->block_n = bn;
  pl->T_c = (max_len + bn - 1) / bn;
  if ((long long)B * KVH * pl->T_c >= (1LL << 31)) return SANTA_E_TOO_LARGE;
  pl->ws = make_split(B * KVH, pl->T_c, sms, &pl->grid, KVH);
  const size_t ncg = size_t(B) * (KVH / pl->ws.gw);
  const size_t slots = (size_t(pl->ws.nvg) + ncg) * pl->ws.gw;
  pl->slots = slots;
  pl->off_pvrows = 256;
  pl->off_partials = pl->off_pvrows + align_up(slots * 4, 256);
  pl->total = pl->off_partials + slots * santa::kGH * santa::kPartialStride * sizeof(float);
  return SANTA_OK;
}

// Ragged Prop batch: tables and the stash are laid out for the length bound, [B,H,T_max] and
// [B,H,max_len]; the work split assumes every sequence as long as the bound (the kernels count
// the real items).
struct PropRaggedPlan {
  int T_max, grid;
  santa::WorkSplit ws;
  size_t off_m, off_ell, off_S, off_inv, off_a0, off_stash, off_pvrows, off_partials, total;
};

int plan_prop_ragged(int B, int H, int KVH, int D, int max_len, PropRaggedPlan* pl) {
  if (KVH <= 0 || D != santa::kD || H != santa::kGH * KVH) return SANTA_E_SHAPE;
  if (B <= 0 || B > santa::kMaxRaggedSeqs) return SANTA_E_TOO_LARGE;
  if (max_len <= 0) return SANTA_E_LENGTH;
  int sms = 0;
  if (int rc = sm_count_of_current_device(&sms)) return rc;
  if (sms > santa::kMaxCtas) sms = santa::kMaxCtas;
  pl->T_max = (max_len + 255) / 256;
  if ((long long)B * KVH * pl->T_max >= (1LL << 31)) return SANTA_E_TOO_LARGE;
  if (size_t(pl->T_max) * 20 > size_t(227) * 1024) return SANTA_E_TOO_LARGE;  // budget tables live in shared memory
  pl->ws = make_split(B * KVH, pl->T_max, sms, &pl->grid, KVH);
  const size_t ht = align_up(size_t(B) * H * pl->T_max * 4, 256);
  pl->off_m = 256;
  pl->off_ell = pl->off_m + ht;
  pl->off_S = pl->off_ell + ht;
  pl->off_inv = pl->off_S + ht;
  pl->off_a0 = pl->off_inv + ht;
  pl->off_stash = pl->off_a0 + ht;
  pl->off_pvrows = pl->off_stash + align_up(size_t(B) * H * max_len * 2, 256);
  const size_t slots = size_t(santa::prop_pass2_max_groups(sms)) + size_t(B) * KVH;
  pl->off_partials = pl->off_pvrows + align_up(slots * 4, 256);
  pl->total = pl->off_partials + slots * santa::kGH * santa::kD * sizeof(float);
  return SANTA_OK;
}

}  // namespace

extern "C" {

const char* santa_strerror(int code) {
  switch (code) {
    case SANTA_OK: return "ok";
    case SANTA_E_DTYPE: return "dtype must be bf16 or f16";
    case SANTA_E_SHAPE:
      return "unsupported shape: Flash and the ragged calls take D=128 and H/KVH=4; santa_prop_decode takes "
             "H%KVH==0 with H/KVH<=8 and D a multiple of 16 up to 256";
    case SANTA_E_LENGTH: return "valid_len must be > 0 and must not exceed the storage length";
    case SANTA_E_BLOCK_N: return "block_n must be 0 (auto) or one of {32,64,256}";
    case SANTA_E_WORKSPACE: return "workspace is NULL, not 256-byte aligned, or too small";
    case SANTA_E_ALIGN: return "q/K/V/out pointers must be 16-byte aligned";
    case SANTA_E_CUDA: return "a CUDA runtime call failed";
    case SANTA_E_ARG: return "missing or inconsistent argument";
    case SANTA_E_TOO_LARGE: return "problem size beyond the limit of this entry point";
    default: return "unknown error";
  }
}

int santa_last_cuda_error(void) { return g_last_cuda_error; }
int santa_abi_version(void) { return 3; }

int santa_block_n_rule(int L_valid, int block_n) {
  if (block_n > 0) return block_n;
  if (L_valid <= 1536) return 32;
  if (L_valid <= 3072) return 64;
  return 256;
}

void santa_flash_budget(int L_valid, int block_n, int64_t S, int* T_c, int* S_per_tile) {
  const int tc = (L_valid + block_n - 1) / block_n;
  int spt = 0;
  if (S > 0) {
    spt = int(S / tc);
    if (spt < 1) spt = 1;
  }
  if (T_c) *T_c = tc;
  if (S_per_tile) *S_per_tile = spt;
}

float santa_u01(uint64_t seed, int head_index, int tile_index) {
  return santa::u01_from_seed(seed, head_index, tile_index);
}

size_t santa_flash_workspace_bytes(int B, int KVH, int L_valid, int block_n) {
  FlashPlan pl;
  if (plan_flash(B, KVH, L_valid, block_n, &pl) != SANTA_OK) return 0;
  return pl.total;
}

size_t santa_prop_workspace_bytes(int H, int KVH, int D, int L, int block_n) {
  PropPlan pl;
  // the vec-forcing mode can only enlarge block_n, never the workspace
  if (plan_prop(H, KVH, D, L, block_n, 0, &pl) != SANTA_OK) return 0;
  return pl.total;
}

int32_t* santa_workspace_status(void* workspace) { return static_cast<int32_t*>(workspace); }

int santa_flash_decode(const void* q, const void* K, const void* V, int dtype, int B, int H, int KVH, int D,
                       int L_valid, int L_storage, int64_t S, uint64_t seed, int block_n, void* out,
                       float* m_star, int32_t* vrows, void* workspace, size_t workspace_bytes,
                       const santa_flash_ext* ext, void* stream) {
  if (dtype != SANTA_DTYPE_BF16 && dtype != SANTA_DTYPE_F16) return SANTA_E_DTYPE;
  if (!q || !K || !V) return SANTA_E_ARG;
  if (D != santa::kD || KVH <= 0 || H != santa::kGH * KVH || B <= 0) return SANTA_E_SHAPE;
  if (L_valid <= 0 || L_valid > L_storage) return SANTA_E_LENGTH;
  const bool want_partial = ext && ext->partial_out;
  const bool want_peer = ext && ext->peer;
  if (!out && !want_partial && !want_peer) return SANTA_E_ARG;
  if (want_peer) {
    const santa_peer_exchange* px = ext->peer;
    if (px->world < 1 || px->world > santa::kMaxPeers || px->rank < 0 || px->rank >= px->world) return SANTA_E_ARG;
    for (int r = 0; r < px->world; ++r)
      if (!px->peer_buffer[r] || (reinterpret_cast<uintptr_t>(px->peer_buffer[r]) & 255u)) return SANTA_E_ARG;
    if ((px->flags & SANTA_PEER_COMBINE) && !out) return SANTA_E_ARG;  // the combined result needs a place
  }
  if (ext && ((ext->u16 == nullptr) != (ext->counts == nullptr))) return SANTA_E_ARG;
  if (ext && ((ext->m_tiles == nullptr) != (ext->ell_tiles == nullptr))) return SANTA_E_ARG;
  if (ext && ext->score_mode != SANTA_SCORE_EXACT && ext->score_mode != SANTA_SCORE_TENSOR) return SANTA_E_ARG;
  if (!aligned16(q) || !aligned16(K) || !aligned16(V) || (out && !aligned16(out))) return SANTA_E_ALIGN;

  FlashPlan pl;
  if (int rc = plan_flash(B, KVH, L_valid, block_n, &pl)) return rc;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < pl.total)
    return SANTA_E_WORKSPACE;

  int T_c = 0, spt = 0;
  santa_flash_budget(L_valid, pl.block_n, S, &T_c, &spt);
  if (ext && ext->s_per_tile_override >= 0) spt = ext->s_per_tile_override;

  unsigned char* ws = static_cast<unsigned char*>(workspace);
  santa::StreamParams p{};
  p.score_mma = (ext && ext->score_mode == SANTA_SCORE_TENSOR) ? 1 : 0;
  if (int rc = encode_k_map(&p.tmK, K, B, L_storage, KVH, p.score_mma != 0)) return rc;
  p.q = q;
  p.V = V;
  p.H = H;
  p.KVH = KVH;
  p.L_valid = L_valid;
  p.L_storage = L_storage;
  p.seq_lens = nullptr;
  p.nseq = B;
  p.tile_stride = pl.T_c;
  p.len_stride = L_valid;
  p.ws = pl.ws;
  p.S_per_tile = spt;
  p.S_total = 0;
  p.q_scale = 1.0f / std::sqrt((float)D);  // F.cpp:210
  p.seed = seed;
  p.batch_offset = ext ? ext->batch_offset : 0;
  p.tile_offset = ext ? ext->tile_offset : 0;
  p.status = reinterpret_cast<int*>(ws);
  p.partial_vrows = reinterpret_cast<int*>(ws + pl.off_pvrows);
  p.partials = reinterpret_cast<float*>(ws + pl.off_partials);
  p.partial_slots = (long long)pl.slots;
  p.m_tiles = ext ? ext->m_tiles : nullptr;
  p.ell_tiles = ext ? ext->ell_tiles : nullptr;
  p.stash = nullptr;
  p.dbg_invdel = (ext && ext->m_tiles) ? ext->invdel : nullptr;
  p.dbg_u = ext ? ext->u16 : nullptr;
  p.dbg_c = ext ? ext->counts : nullptr;
  p.rowmask = ext ? ext->rowmask : nullptr;

  santa::FlashMergeParams mp{};
  mp.H = H;
  mp.KVH = KVH;
  mp.S_per_tile = spt;
  mp.ws = pl.ws;
  mp.partials = p.partials;
  mp.partial_vrows = p.partial_vrows;
  mp.partial_slots = p.partial_slots;
  mp.out = out;
  mp.m_star = m_star;
  mp.vrows = vrows;
  mp.partial_out = want_partial ? ext->partial_out : nullptr;
  mp.status = p.status;
  if (ext && ext->peer) {
    const santa_peer_exchange* px = ext->peer;
    mp.px.world = px->world;
    mp.px.rank = px->rank;
    mp.px.epoch = px->epoch;
    mp.px.combine = (px->flags & SANTA_PEER_COMBINE) ? 1 : 0;
    for (int r = 0; r < px->world; ++r) mp.px.base[r] = static_cast<unsigned char*>(px->peer_buffer[r]);
  }

  cudaError_t e = santa::launch_flash(p, mp, dtype, pl.block_n, pl.grid, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  return SANTA_OK;
}

size_t santa_flash_ragged_workspace_bytes(int B, int KVH, int max_len, int block_n) {
  FlashPlan pl;
  if (plan_flash_ragged(B, KVH, max_len, block_n, &pl) != SANTA_OK) return 0;
  return pl.total;
}

int santa_flash_decode_ragged(const void* q, const void* K, const void* V, int dtype, int B, int H, int KVH, int D,
                              int L_storage, const int32_t* seq_lens, int max_len, int64_t S, uint64_t seed,
                              int block_n, void* out, float* m_star, int32_t* vrows, void* workspace,
                              size_t workspace_bytes, const santa_flash_ext* ext, void* stream) {
  if (dtype != SANTA_DTYPE_BF16 && dtype != SANTA_DTYPE_F16) return SANTA_E_DTYPE;
  if (!q || !K || !V || !out || !seq_lens) return SANTA_E_ARG;
  if (D != santa::kD || KVH <= 0 || H != santa::kGH * KVH || B <= 0) return SANTA_E_SHAPE;
  if (max_len <= 0 || max_len > L_storage) return SANTA_E_LENGTH;
  if (ext && (ext->tile_offset != 0 || ext->s_per_tile_override >= 0 || ext->partial_out != nullptr))
    return SANTA_E_ARG;  // the sequence-sharding extensions belong to the uniform entry point
  if (ext && ((ext->u16 == nullptr) != (ext->counts == nullptr))) return SANTA_E_ARG;
  if (ext && ((ext->m_tiles == nullptr) != (ext->ell_tiles == nullptr))) return SANTA_E_ARG;
  if (ext && ext->score_mode != SANTA_SCORE_EXACT && ext->score_mode != SANTA_SCORE_TENSOR) return SANTA_E_ARG;
  if (!aligned16(q) || !aligned16(K) || !aligned16(V) || !aligned16(out)) return SANTA_E_ALIGN;

  FlashPlan pl;
  if (int rc = plan_flash_ragged(B, KVH, max_len, block_n, &pl)) return rc;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < pl.total)
    return SANTA_E_WORKSPACE;
  const int S32 = S > 2147483647LL ? 2147483647 : (S < 0 ? 0 : int(S));

  unsigned char* ws = static_cast<unsigned char*>(workspace);
  santa::StreamParams p{};
  p.score_mma = (ext && ext->score_mode == SANTA_SCORE_TENSOR) ? 1 : 0;
  if (int rc = encode_k_map(&p.tmK, K, B, L_storage, KVH, p.score_mma != 0)) return rc;
  p.q = q;
  p.V = V;
  p.H = H;
  p.KVH = KVH;
  p.L_valid = max_len;
  p.L_storage = L_storage;
  p.seq_lens = seq_lens;
  p.nseq = B;
  p.tile_stride = pl.T_c;
  p.len_stride = max_len;
  p.ws = pl.ws;
  p.S_per_tile = 0;
  p.S_total = S32;
  p.q_scale = 1.0f / std::sqrt((float)D);  // F.cpp:210
  p.seed = seed;
  p.batch_offset = ext ? ext->batch_offset : 0;
  p.tile_offset = 0;
  p.status = reinterpret_cast<int*>(ws);
  p.partial_vrows = reinterpret_cast<int*>(ws + pl.off_pvrows);
  p.partials = reinterpret_cast<float*>(ws + pl.off_partials);
  p.partial_slots = (long long)pl.slots;
  p.m_tiles = ext ? ext->m_tiles : nullptr;
  p.ell_tiles = ext ? ext->ell_tiles : nullptr;
  p.stash = nullptr;
  p.dbg_invdel = (ext && ext->m_tiles) ? ext->invdel : nullptr;
  p.dbg_u = ext ? ext->u16 : nullptr;
  p.dbg_c = ext ? ext->counts : nullptr;
  p.rowmask = ext ? ext->rowmask : nullptr;

  santa::FlashMergeParams mp{};
  mp.H = H;
  mp.KVH = KVH;
  mp.S_per_tile = 0;
  mp.seq_lens = seq_lens;
  mp.nseq = B;
  mp.max_len = max_len;
  mp.bn = pl.block_n;
  mp.S_total = S32;
  mp.ws = pl.ws;
  mp.partials = p.partials;
  mp.partial_vrows = p.partial_vrows;
  mp.partial_slots = p.partial_slots;
  mp.out = out;
  mp.m_star = m_star;
  mp.vrows = vrows;
  mp.partial_out = nullptr;

  cudaError_t e = santa::launch_flash(p, mp, dtype, pl.block_n, pl.grid, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  return SANTA_OK;
}

int santa_prop_decode(const void* q, const void* K, const void* V, int dtype, int H, int KVH, int D, int L, int64_t S,
                      uint64_t seed, int block_n, void* out, float* m_star, int32_t* vrows, void* workspace,
                      size_t workspace_bytes, const santa_prop_ext* ext, void* stream) {
  if (dtype != SANTA_DTYPE_BF16 && dtype != SANTA_DTYPE_F16) return SANTA_E_DTYPE;
  if (!q || !K || !V || !out || !m_star) return SANTA_E_ARG;
  if (!aligned16(q) || !aligned16(K) || !aligned16(V) || !aligned16(out)) return SANTA_E_ALIGN;
  const int mode = ext ? ext->pass1_mode : 0;
  if (mode < 0 || mode > 2) return SANTA_E_ARG;
  if (ext && ext->score_mode != SANTA_SCORE_EXACT && ext->score_mode != SANTA_SCORE_TENSOR) return SANTA_E_ARG;
  PropPlan pl;
  if (int rc = plan_prop(H, KVH, D, L, block_n, mode, &pl)) return rc;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < pl.total)
    return SANTA_E_WORKSPACE;
  unsigned char* ws = static_cast<unsigned char*>(workspace);

  santa::PropParams p{};
  santa::StreamParams& sp = p.sp;
  sp.score_mma = (pl.use_vec && ext && ext->score_mode == SANTA_SCORE_TENSOR) ? 1 : 0;
  if (pl.use_vec)
    if (int rc = encode_k_map(&sp.tmK, K, 1, L, KVH, sp.score_mma != 0)) return rc;
  sp.q = q;
  sp.V = V;
  sp.H = H;
  sp.KVH = KVH;
  sp.L_valid = L;
  sp.L_storage = L;
  sp.seq_lens = nullptr;
  sp.nseq = 1;
  sp.tile_stride = pl.T_c;
  sp.len_stride = L;
  sp.ws = pl.ws;
  sp.S_per_tile = 0;
  sp.q_scale = 1.0f / std::sqrt((float)D);  // P.cpp:208
  sp.seed = seed;
  sp.status = reinterpret_cast<int*>(ws);
  sp.m_tiles = (ext && ext->m_tiles) ? ext->m_tiles : reinterpret_cast<float*>(ws + pl.off_m);
  sp.ell_tiles = (ext && ext->ell_tiles) ? ext->ell_tiles : reinterpret_cast<float*>(ws + pl.off_ell);
  sp.stash = reinterpret_cast<uint16_t*>(ws + pl.off_stash);
  sp.dbg_u = ext ? ext->u16 : nullptr;
  p.K = K;
  p.D = D;
  p.block_n = pl.block_n;
  p.T_c = pl.T_c;
  p.use_vec = pl.use_vec;
  p.S = S > 2147483647LL ? 2147483647 : (S < -2147483647LL ? -2147483647 : int(S));
  p.flags = ext ? ext->flags : 3;
  p.S_tiles = (ext && ext->S_tiles) ? ext->S_tiles : reinterpret_cast<int*>(ws + pl.off_S);
  p.invdelta = (ext && ext->invdelta) ? ext->invdelta : reinterpret_cast<float*>(ws + pl.off_inv);
  p.a0 = (ext && ext->a0) ? ext->a0 : reinterpret_cast<float*>(ws + pl.off_a0);
  p.m_star = m_star;
  p.partial_vrows = reinterpret_cast<int*>(ws + pl.off_pvrows);
  p.partials = reinterpret_cast<float*>(ws + pl.off_partials);
  p.out = out;
  p.vrows = vrows;
  p.dbg_c = ext ? ext->counts : nullptr;
  p.rowmask = ext ? ext->rowmask : nullptr;
  cudaError_t e = santa::launch_prop(p, dtype, pl.grid, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  return SANTA_OK;
}

size_t santa_prop_ragged_workspace_bytes(int B, int H, int KVH, int D, int max_len) {
  PropRaggedPlan pl;
  if (plan_prop_ragged(B, H, KVH, D, max_len, &pl) != SANTA_OK) return 0;
  return pl.total;
}

int santa_prop_decode_ragged(const void* q, const void* K, const void* V, int dtype, int B, int H, int KVH, int D,
                             int L_storage, const int32_t* seq_lens, int max_len, int64_t S, uint64_t seed,
                             void* out, float* m_star, int32_t* vrows, void* workspace, size_t workspace_bytes,
                             const santa_prop_ext* ext, void* stream) {
  if (dtype != SANTA_DTYPE_BF16 && dtype != SANTA_DTYPE_F16) return SANTA_E_DTYPE;
  if (!q || !K || !V || !out || !m_star || !seq_lens) return SANTA_E_ARG;
  if (!aligned16(q) || !aligned16(K) || !aligned16(V) || !aligned16(out)) return SANTA_E_ALIGN;
  if (max_len <= 0 || max_len > L_storage) return SANTA_E_LENGTH;
  if (ext && ext->pass1_mode != 0 && ext->pass1_mode != 2) return SANTA_E_ARG;
  if (ext && ext->score_mode != SANTA_SCORE_EXACT && ext->score_mode != SANTA_SCORE_TENSOR) return SANTA_E_ARG;
  PropRaggedPlan pl;
  if (int rc = plan_prop_ragged(B, H, KVH, D, max_len, &pl)) return rc;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < pl.total)
    return SANTA_E_WORKSPACE;
  unsigned char* ws = static_cast<unsigned char*>(workspace);

  santa::PropParams p{};
  santa::StreamParams& sp = p.sp;
  sp.score_mma = (ext && ext->score_mode == SANTA_SCORE_TENSOR) ? 1 : 0;
  if (int rc = encode_k_map(&sp.tmK, K, B, L_storage, KVH, sp.score_mma != 0)) return rc;
  sp.q = q;
  sp.V = V;
  sp.H = H;
  sp.KVH = KVH;
  sp.L_valid = max_len;
  sp.L_storage = L_storage;
  sp.seq_lens = seq_lens;
  sp.nseq = B;
  sp.tile_stride = pl.T_max;
  sp.len_stride = max_len;
  sp.ws = pl.ws;
  sp.S_per_tile = 0;
  sp.q_scale = 1.0f / std::sqrt((float)D);  // P.cpp:208
  sp.seed = seed;
  sp.status = reinterpret_cast<int*>(ws);
  sp.m_tiles = (ext && ext->m_tiles) ? ext->m_tiles : reinterpret_cast<float*>(ws + pl.off_m);
  sp.ell_tiles = (ext && ext->ell_tiles) ? ext->ell_tiles : reinterpret_cast<float*>(ws + pl.off_ell);
  sp.stash = reinterpret_cast<uint16_t*>(ws + pl.off_stash);
  sp.dbg_u = ext ? ext->u16 : nullptr;
  p.K = K;
  p.D = D;
  p.block_n = 256;
  p.T_c = pl.T_max;
  p.use_vec = 1;
  p.S = S > 2147483647LL ? 2147483647 : (S < -2147483647LL ? -2147483647 : int(S));
  p.flags = ext ? ext->flags : 3;
  p.S_tiles = (ext && ext->S_tiles) ? ext->S_tiles : reinterpret_cast<int*>(ws + pl.off_S);
  p.invdelta = (ext && ext->invdelta) ? ext->invdelta : reinterpret_cast<float*>(ws + pl.off_inv);
  p.a0 = (ext && ext->a0) ? ext->a0 : reinterpret_cast<float*>(ws + pl.off_a0);
  p.m_star = m_star;
  p.partial_vrows = reinterpret_cast<int*>(ws + pl.off_pvrows);
  p.partials = reinterpret_cast<float*>(ws + pl.off_partials);
  p.out = out;
  p.vrows = vrows;
  p.dbg_c = ext ? ext->counts : nullptr;
  p.rowmask = ext ? ext->rowmask : nullptr;
  cudaError_t e = santa::launch_prop(p, dtype, pl.grid, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  return SANTA_OK;
}

int32_t* santa_peer_exchange_status(void* own_buffer) {
  return own_buffer ? static_cast<int32_t*>(own_buffer) + santa::kPeerStatusIndex : nullptr;
}

size_t santa_peer_exchange_bytes(int world, int BH) {
  if (world < 1 || world > santa::kMaxPeers || BH <= 0) return 0;
  return align_up(santa::peer_data_offset(2, world, 0, BH), 256);
}

int santa_lse_combine_wait(const santa_peer_exchange* px, int BH, int D, int S_per_tile, int dtype, void* out,
                           float* m_star, int32_t* status, void* stream) {
  if (dtype != SANTA_DTYPE_BF16 && dtype != SANTA_DTYPE_F16) return SANTA_E_DTYPE;
  if (!px || !out || BH <= 0) return SANTA_E_ARG;
  if (D != santa::kD) return SANTA_E_SHAPE;
  if (px->world < 1 || px->world > santa::kMaxPeers || px->rank < 0 || px->rank >= px->world) return SANTA_E_ARG;
  if (!px->peer_buffer[px->rank]) return SANTA_E_ARG;
  cudaError_t e = santa::launch_lse_combine_wait(static_cast<unsigned char*>(px->peer_buffer[px->rank]), px->world,
                                                 px->epoch, BH, S_per_tile, dtype, out, m_star, status,
                                                 static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  return SANTA_OK;
}

int santa_lse_combine(const float* partials, int G, int BH, int D, int S_per_tile, int dtype, void* out,
                      float* m_star, void* stream) {
  if (dtype != SANTA_DTYPE_BF16 && dtype != SANTA_DTYPE_F16) return SANTA_E_DTYPE;
  if (!partials || !out || G <= 0 || BH <= 0) return SANTA_E_ARG;
  if (D != santa::kD) return SANTA_E_SHAPE;
  cudaError_t e = santa::launch_lse_combine(partials, G, BH, S_per_tile, dtype, out, m_star,
                                            static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  return SANTA_OK;
}

int santa_rope_append(const void* q_proj, const void* k_proj, const void* v_proj, int64_t q_stride, int64_t k_stride,
                      int64_t v_stride, const void* cos, const void* sin, int dtype, int B, int H, int KVH, int D,
                      void* k_cache, void* v_cache, int L_storage, int pos, const int32_t* pos_dev, void* q_out,
                      int32_t* seq_lens_out, int32_t* status, void* stream) {
  if (dtype != SANTA_DTYPE_BF16 && dtype != SANTA_DTYPE_F16) return SANTA_E_DTYPE;
  if (!q_proj || !k_proj || !v_proj || !cos || !sin || !k_cache || !v_cache || !q_out) return SANTA_E_ARG;
  if (D != santa::kD || B <= 0 || H <= 0 || KVH <= 0 || L_storage <= 0) return SANTA_E_SHAPE;
  if (!pos_dev && (pos < 0 || pos >= L_storage)) return SANTA_E_LENGTH;
  if (q_stride <= 0) q_stride = int64_t(H) * D;
  if (k_stride <= 0) k_stride = int64_t(KVH) * D;
  if (v_stride <= 0) v_stride = int64_t(KVH) * D;
  if ((q_stride | k_stride | v_stride) & 3) return SANTA_E_ALIGN;  // rows stay 8-byte aligned
  const void* ptrs[] = {q_proj, k_proj, v_proj, cos, sin, k_cache, v_cache, q_out};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 7u) return SANTA_E_ALIGN;  // 8-byte vector accesses
  santa::RopeAppendParams p{};
  p.q_proj = q_proj;
  p.k_proj = k_proj;
  p.v_proj = v_proj;
  p.q_stride = q_stride;
  p.k_stride = k_stride;
  p.v_stride = v_stride;
  p.cos = cos;
  p.sin = sin;
  p.B = B;
  p.H = H;
  p.KVH = KVH;
  p.L_storage = L_storage;
  p.pos = pos;
  p.pos_dev = pos_dev;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.q_out = q_out;
  p.seq_lens_out = seq_lens_out;
  p.status = status;
  cudaError_t e = santa::launch_rope_append(p, dtype, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  return SANTA_OK;
}

// ---- no-allocation variant of the Flash decode ---------------------------------------------
// Scratch for callers that cannot provide a workspace.  In host code this name is only a
// stand-in for the device array: its device address comes from cudaGetSymbolAddress, once per
// device, and is what the kernels receive.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SANTA_NOALLOC_SCRATCH_BYTES];

static void* scratch_of_device[64] = {};

int32_t* santa_noalloc_status(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  return static_cast<int32_t*>(scratch_of_device[dev]);  // the status word is the array's first word
}

int santa_flash_decode_noalloc(const void* q, const void* K, const void* V, int dtype, int B, int H, int KVH, int D,
                               int L_valid, int L_storage, int64_t S, uint64_t seed, int block_n, void* out,
                               float* m_star, int32_t* vrows, const santa_flash_ext* ext, void* stream) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= 64) return SANTA_E_ARG;
  if (scratch_of_device[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);  // set-up: first call on this device
    if (e != cudaSuccess) return cuda_fail(e);
    scratch_of_device[dev] = ptr;
  }
  void* scratch = scratch_of_device[dev];
  // sizes beyond the fixed array are refused; argument errors are left to the common path below
  const size_t need = santa_flash_workspace_bytes(B, KVH, L_valid, block_n);
  if (need > size_t(SANTA_NOALLOC_SCRATCH_BYTES)) return SANTA_E_TOO_LARGE;
  // The array keeps the previous call's contents.  Every word a call reads it has written before,
  // except the status word: that one is zero from the module's load image and is left alone here, so
  // that a time-out reported by an earlier call stays readable (santa_noalloc_status).
  return santa_flash_decode(q, K, V, dtype, B, H, KVH, D, L_valid, L_storage, S, seed, block_n, out, m_star, vrows,
                            scratch, size_t(SANTA_NOALLOC_SCRATCH_BYTES), ext, stream);
}

}  // extern "C"
