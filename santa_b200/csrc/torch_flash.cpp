// torch_flash.cpp -- the `santa_flash_batch_cuda` Python module: a thin
// pybind11/ATen shim over the C ABI of libsanta_b200.so.
//
// Same names, argument order, defaults, tensor layouts, return tuple and error
// messages as the reference module of that name
// (flash_style_fused_santa_fixed_tile_budgets/santa_cuda.cpp:123-360), so that
// tutorial_code/attention_backends.py (SantaFlashBackend, :513-515) imports and
// calls it unchanged.  ATen supplies tensors, the current stream and the
// caching allocator; all arithmetic is in the CUDA library.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>
#include <type_traits>

#include "santa_b200.h"

namespace py = pybind11;

namespace {

// Argument errors surface in Python as RuntimeError with the reference's
// message text (the reference raises them through TORCH_CHECK).
inline void cat_into(std::string&) {}
template <typename T, typename... Rest>
inline void cat_into(std::string& s, const T& v, const Rest&... rest) {
  if constexpr (std::is_arithmetic_v<T>)
    s += std::to_string(v);
  else
    s += v;
  cat_into(s, rest...);
}
template <typename... Args>
[[noreturn]] inline void fail(const Args&... args) {
  std::string msg;
  cat_into(msg, args...);
  throw std::runtime_error(msg);
}
#define SANTA_CHECK(cond, ...) \
  do {                         \
    if (!(cond)) fail(__VA_ARGS__); \
  } while (0)

struct ShapeInfo {
  bool batched;
  int B, H, D, L_storage, KVH;
};

ShapeInfo check_inputs(const at::Tensor& q_h, const at::Tensor& K_g, const at::Tensor& V_g) {
  SANTA_CHECK(q_h.is_cuda(), "q_h must be CUDA");
  SANTA_CHECK(K_g.is_cuda() && V_g.is_cuda(), "K_g and V_g must be CUDA");
  SANTA_CHECK(q_h.scalar_type() == at::kBFloat16 || q_h.scalar_type() == at::kHalf, "q_h must be bf16 or f16");
  SANTA_CHECK(K_g.scalar_type() == at::kBFloat16 || K_g.scalar_type() == at::kHalf, "K_g must be bf16 or f16");
  SANTA_CHECK(K_g.scalar_type() == V_g.scalar_type(), "K_g and V_g must have the same dtype");
  SANTA_CHECK(q_h.scalar_type() == K_g.scalar_type(), "q_h dtype must match K_g/V_g dtype");
  SANTA_CHECK(q_h.device() == K_g.device() && q_h.device() == V_g.device(), "device mismatch");
  SANTA_CHECK(K_g.is_contiguous() && V_g.is_contiguous(),
              "K_g/V_g must be contiguous. Expected [L,KVH,D] for single or [B,L,KVH,D] for batch.");
  ShapeInfo s{};
  if (q_h.dim() == 2) {
    SANTA_CHECK(K_g.dim() == 3 && V_g.dim() == 3, "Single-request path expects q_h [H,D], K_g/V_g [L,KVH,D]");
    SANTA_CHECK(K_g.sizes() == V_g.sizes(), "K_g and V_g must have the same shape");
    SANTA_CHECK(q_h.size(1) == K_g.size(2), "D mismatch (q_h.size(1) vs K_g.size(2))");
    s = {false, 1, (int)q_h.size(0), (int)q_h.size(1), (int)K_g.size(0), (int)K_g.size(1)};
    return s;
  }
  SANTA_CHECK(q_h.dim() == 3 && K_g.dim() == 4 && V_g.dim() == 4,
              "Batched path expects q_h [B,H,D], K_g/V_g [B,L,KVH,D]");
  SANTA_CHECK(K_g.sizes() == V_g.sizes(), "K_g and V_g must have the same shape");
  SANTA_CHECK(q_h.size(0) == K_g.size(0), "Batch mismatch between q_h and K_g/V_g");
  SANTA_CHECK(q_h.size(2) == K_g.size(3), "D mismatch (q_h.size(2) vs K_g.size(3))");
  s = {true, (int)q_h.size(0), (int)q_h.size(1), (int)q_h.size(2), (int)K_g.size(1), (int)K_g.size(2)};
  return s;
}

// One scratch tensor per (device, stream): calls on a stream are ordered, so
// they can share it.  Grown on demand; the old tensor goes back to the caching
// allocator, which keeps stream order.
at::Tensor& workspace_for(const at::Tensor& like, cudaStream_t stream, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, at::Tensor> cache;
  std::lock_guard<std::mutex> lock(mu);
  at::Tensor& ws = cache[{(int)like.get_device(), stream}];
  if (!ws.defined() || (size_t)ws.numel() < bytes) {
    const int64_t n = (int64_t)std::max<size_t>(bytes, size_t(4) << 20);
    ws = at::zeros({n}, like.options().dtype(at::kByte));
  }
  return ws;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> decode_systematic(at::Tensor q_h, at::Tensor K_g, at::Tensor V_g,
                                                                 int64_t S, uint64_t seed, int64_t block_n,
                                                                 bool want_vrows, int64_t valid_len,
                                                                 int64_t score_mode) {
  const ShapeInfo info = check_inputs(q_h, K_g, V_g);
  const int B = info.B, H = info.H, D = info.D, KVH = info.KVH, L_storage = info.L_storage;
  const int L = (valid_len > 0) ? (int)valid_len : L_storage;
  SANTA_CHECK(L > 0, "valid_len must be > 0; got ", L);
  SANTA_CHECK(L <= L_storage, "valid_len exceeds storage length: valid_len=", L, " storage=", L_storage);
  SANTA_CHECK(D == 128, "This build supports only D=128. Got D=", D);
  SANTA_CHECK(H % KVH == 0, "H must be divisible by KVH. Got H=", H, " KVH=", KVH);
  SANTA_CHECK(H / KVH == 4, "This build supports only GH=4 (H/KVH). Got GH=", H / KVH, " (H=", H, " KVH=", KVH, ")");
  const int bn = santa_block_n_rule(L, (int)block_n);
  SANTA_CHECK(bn == 32 || bn == 64 || bn == 256, "block_n must be 0 (auto) or one of {32,64,256}. Got block_n=", bn);

  // argument errors are raised above, before any device state is touched
  const c10::cuda::CUDAGuard guard(q_h.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto q = q_h.contiguous();

  auto optsF = q.options().dtype(at::kFloat);
  auto optsI = q.options().dtype(at::kInt);
  at::Tensor out = info.batched ? at::empty({B, H, D}, q.options()) : at::empty({H, D}, q.options());
  at::Tensor m_star = info.batched ? at::empty({B, H}, optsF) : at::empty({H}, optsF);
  at::Tensor vrows = at::empty({0}, optsI);
  if (want_vrows) vrows = info.batched ? at::empty({B, KVH}, optsI) : at::empty({KVH}, optsI);

  const size_t ws_bytes = santa_flash_workspace_bytes(B, KVH, L, bn);
  SANTA_CHECK(ws_bytes > 0, "santa_b200: could not size the workspace");
  at::Tensor& ws = workspace_for(q, stream.stream(), ws_bytes);

  // score_mode: not part of the reference's signature; 0 (the default) is the reference's arithmetic
  SANTA_CHECK(score_mode == SANTA_SCORE_EXACT || score_mode == SANTA_SCORE_TENSOR, "score_mode must be 0 or 1");
  santa_flash_ext ext{};
  ext.s_per_tile_override = -1;
  ext.score_mode = (int)score_mode;
  const int rc = santa_flash_decode(q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(),
                                    q.scalar_type() == at::kBFloat16 ? SANTA_DTYPE_BF16 : SANTA_DTYPE_F16, B, H, KVH,
                                    D, L, L_storage, S, seed, bn, out.data_ptr(), m_star.data_ptr<float>(),
                                    want_vrows ? vrows.data_ptr<int>() : nullptr, ws.data_ptr(), (size_t)ws.numel(),
                                    score_mode ? &ext : nullptr, (void*)stream.stream());
  SANTA_CHECK(rc == SANTA_OK, "santa_b200: ", santa_strerror(rc), " (code ", rc, ", cuda ", santa_last_cuda_error(),
              ")");
  return std::make_tuple(out, m_star, vrows);
}

// Per-sequence lengths from a device tensor; not part of the reference module (its entry point
// takes one host-side valid_len, santa_cuda.cpp:188-191).  Nothing on the host depends on the
// lengths' values, so a captured CUDA graph of this call follows lengths that change between replays.
std::tuple<at::Tensor, at::Tensor, at::Tensor> decode_systematic_ragged(at::Tensor q_h, at::Tensor K_g,
                                                                        at::Tensor V_g, at::Tensor seq_lens,
                                                                        int64_t S, uint64_t seed, int64_t block_n,
                                                                        bool want_vrows, int64_t max_len,
                                                                        int64_t score_mode) {
  const ShapeInfo info = check_inputs(q_h, K_g, V_g);
  SANTA_CHECK(info.batched, "Ragged path expects q_h [B,H,D], K_g/V_g [B,L,KVH,D]");
  const int B = info.B, H = info.H, D = info.D, KVH = info.KVH, L_storage = info.L_storage;
  SANTA_CHECK(D == 128, "This build supports only D=128. Got D=", D);
  SANTA_CHECK(H % KVH == 0 && H / KVH == 4, "This build supports only GH=4 (H/KVH). Got H=", H, " KVH=", KVH);
  SANTA_CHECK(seq_lens.scalar_type() == at::kInt && seq_lens.dim() == 1 && seq_lens.size(0) == B,
              "seq_lens must be an int32 tensor with one length per sequence");
  const int mlen = max_len > 0 ? (int)max_len : L_storage;
  SANTA_CHECK(mlen <= L_storage, "max_len exceeds storage length: max_len=", mlen, " storage=", L_storage);
  SANTA_CHECK(B <= 1024, "The ragged path takes at most 1024 sequences. Got B=", B);
  const int bn = santa_block_n_rule(mlen, (int)block_n);
  SANTA_CHECK(bn == 32 || bn == 64 || bn == 256, "block_n must be 0 (auto) or one of {32,64,256}. Got block_n=", bn);

  const c10::cuda::CUDAGuard guard(q_h.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto q = q_h.contiguous();
  at::Tensor lens = seq_lens.is_cuda() ? seq_lens.contiguous() : seq_lens.to(q.device(), /*non_blocking=*/false);
  SANTA_CHECK(lens.device() == q.device(), "seq_lens must be on q_h's device or on the CPU");

  at::Tensor out = at::empty({B, H, D}, q.options());
  at::Tensor m_star = at::empty({B, H}, q.options().dtype(at::kFloat));
  at::Tensor vrows = want_vrows ? at::empty({B, KVH}, q.options().dtype(at::kInt))
                                : at::empty({0}, q.options().dtype(at::kInt));
  const size_t ws_bytes = santa_flash_ragged_workspace_bytes(B, KVH, mlen, bn);
  SANTA_CHECK(ws_bytes > 0, "santa_b200: could not size the workspace");
  at::Tensor& ws = workspace_for(q, stream.stream(), ws_bytes);
  SANTA_CHECK(score_mode == SANTA_SCORE_EXACT || score_mode == SANTA_SCORE_TENSOR, "score_mode must be 0 or 1");
  santa_flash_ext ext{};
  ext.s_per_tile_override = -1;
  ext.score_mode = (int)score_mode;
  const int rc = santa_flash_decode_ragged(
      q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(), q.scalar_type() == at::kBFloat16 ? SANTA_DTYPE_BF16 : SANTA_DTYPE_F16,
      B, H, KVH, D, L_storage, lens.data_ptr<int>(), mlen, S, seed, bn, out.data_ptr(), m_star.data_ptr<float>(),
      want_vrows ? vrows.data_ptr<int>() : nullptr, ws.data_ptr(), (size_t)ws.numel(), score_mode ? &ext : nullptr,
      (void*)stream.stream());
  SANTA_CHECK(rc == SANTA_OK, "santa_b200: ", santa_strerror(rc), " (code ", rc, ", cuda ", santa_last_cuda_error(),
              ")");
  return std::make_tuple(out, m_star, vrows);
}

// Sequence-sharded decode (no counterpart in the reference, which is single-device): this rank's
// shard of the cache sampled with the GLOBAL tile index and the GLOBAL per-tile budget; returns the
// unnormalised partial [B,H,130] fp32 (A[128], m, Z per head) that `lse_combine` folds across ranks.
at::Tensor decode_systematic_partial(at::Tensor q_h, at::Tensor K_g, at::Tensor V_g, int64_t S, uint64_t seed,
                                     int64_t block_n, int64_t valid_len, int64_t batch_offset, int64_t tile_offset,
                                     int64_t s_per_tile) {
  const ShapeInfo info = check_inputs(q_h, K_g, V_g);
  SANTA_CHECK(info.batched, "Batched path expects q_h [B,H,D], K_g/V_g [B,L,KVH,D]");
  const int B = info.B, H = info.H, D = info.D, KVH = info.KVH, L_storage = info.L_storage;
  const int L = (valid_len > 0) ? (int)valid_len : L_storage;
  SANTA_CHECK(L <= L_storage, "valid_len exceeds storage length: valid_len=", L, " storage=", L_storage);
  SANTA_CHECK(D == 128 && H % KVH == 0 && H / KVH == 4, "This build supports only D=128 and GH=4 (H/KVH)");
  const int bn = santa_block_n_rule(L, (int)block_n);
  SANTA_CHECK(bn == 32 || bn == 64 || bn == 256, "block_n must be 0 (auto) or one of {32,64,256}. Got block_n=", bn);
  const c10::cuda::CUDAGuard guard(q_h.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto q = q_h.contiguous();
  at::Tensor part = at::empty({B, H, D + 2}, q.options().dtype(at::kFloat));
  const size_t ws_bytes = santa_flash_workspace_bytes(B, KVH, L, bn);
  SANTA_CHECK(ws_bytes > 0, "santa_b200: could not size the workspace");
  at::Tensor& ws = workspace_for(q, stream.stream(), ws_bytes);
  santa_flash_ext ext{};
  ext.batch_offset = (int)batch_offset;
  ext.tile_offset = (int)tile_offset;
  ext.s_per_tile_override = (int)s_per_tile;
  ext.partial_out = part.data_ptr<float>();
  const int rc = santa_flash_decode(q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(),
                                    q.scalar_type() == at::kBFloat16 ? SANTA_DTYPE_BF16 : SANTA_DTYPE_F16, B, H, KVH,
                                    D, L, L_storage, S, seed, bn, nullptr, nullptr, nullptr, ws.data_ptr(),
                                    (size_t)ws.numel(), &ext, (void*)stream.stream());
  SANTA_CHECK(rc == SANTA_OK, "santa_b200: ", santa_strerror(rc), " (code ", rc, ", cuda ", santa_last_cuda_error(),
              ")");
  return part;
}

santa_peer_exchange make_peer(const std::vector<int64_t>& peer_ptrs, int64_t rank, int64_t epoch,
                              bool combine = false) {
  SANTA_CHECK(!peer_ptrs.empty() && peer_ptrs.size() <= 16, "peer_ptrs must hold 1..16 buffer addresses");
  SANTA_CHECK(rank >= 0 && rank < (int64_t)peer_ptrs.size() && epoch >= 0, "bad rank / epoch of the peer exchange");
  santa_peer_exchange px{};
  px.world = (int)peer_ptrs.size();
  px.rank = (int)rank;
  px.epoch = (uint32_t)epoch;
  px.flags = combine ? SANTA_PEER_COMBINE : 0u;
  for (size_t r = 0; r < peer_ptrs.size(); ++r) px.peer_buffer[r] = reinterpret_cast<void*>(peer_ptrs[r]);
  return px;
}

// Sequence-sharded decode whose partial goes straight into every rank's exchange buffer (peer-mapped
// device memory) instead of through a collective.  combine = true: the same call also waits for the
// other ranks' rows and returns the combined (out, m_star); combine = false: it returns two empty
// tensors and `lse_combine_wait` is the receiving half.
std::tuple<at::Tensor, at::Tensor> decode_systematic_exchange(at::Tensor q_h, at::Tensor K_g, at::Tensor V_g,
                                                              int64_t S, uint64_t seed, int64_t block_n,
                                                              int64_t valid_len, int64_t batch_offset,
                                                              int64_t tile_offset, int64_t s_per_tile,
                                                              std::vector<int64_t> peer_ptrs, int64_t rank,
                                                              int64_t epoch, bool combine) {
  const ShapeInfo info = check_inputs(q_h, K_g, V_g);
  SANTA_CHECK(info.batched, "Batched path expects q_h [B,H,D], K_g/V_g [B,L,KVH,D]");
  const int B = info.B, H = info.H, D = info.D, KVH = info.KVH, L_storage = info.L_storage;
  const int L = (valid_len > 0) ? (int)valid_len : L_storage;
  SANTA_CHECK(L <= L_storage, "valid_len exceeds storage length: valid_len=", L, " storage=", L_storage);
  SANTA_CHECK(D == 128 && H % KVH == 0 && H / KVH == 4, "This build supports only D=128 and GH=4 (H/KVH)");
  const int bn = santa_block_n_rule(L, (int)block_n);
  SANTA_CHECK(bn == 32 || bn == 64 || bn == 256, "block_n must be 0 (auto) or one of {32,64,256}. Got block_n=", bn);
  const santa_peer_exchange px = make_peer(peer_ptrs, rank, epoch, combine);
  const c10::cuda::CUDAGuard guard(q_h.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto q = q_h.contiguous();
  const size_t ws_bytes = santa_flash_workspace_bytes(B, KVH, L, bn);
  SANTA_CHECK(ws_bytes > 0, "santa_b200: could not size the workspace");
  at::Tensor& ws = workspace_for(q, stream.stream(), ws_bytes);
  at::Tensor out = combine ? at::empty({B, H, D}, q.options()) : at::empty({0}, q.options());
  at::Tensor m_star = combine ? at::empty({B, H}, q.options().dtype(at::kFloat))
                              : at::empty({0}, q.options().dtype(at::kFloat));
  santa_flash_ext ext{};
  ext.batch_offset = (int)batch_offset;
  ext.tile_offset = (int)tile_offset;
  ext.s_per_tile_override = (int)s_per_tile;
  ext.peer = &px;
  const int rc = santa_flash_decode(q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(),
                                    q.scalar_type() == at::kBFloat16 ? SANTA_DTYPE_BF16 : SANTA_DTYPE_F16, B, H, KVH,
                                    D, L, L_storage, S, seed, bn, combine ? out.data_ptr() : nullptr,
                                    combine ? m_star.data_ptr<float>() : nullptr, nullptr, ws.data_ptr(),
                                    (size_t)ws.numel(), &ext, (void*)stream.stream());
  SANTA_CHECK(rc == SANTA_OK, "santa_b200: ", santa_strerror(rc), " (code ", rc, ", cuda ", santa_last_cuda_error(),
              ")");
  return std::make_tuple(out, m_star);
}

std::tuple<at::Tensor, at::Tensor> lse_combine_wait(std::vector<int64_t> peer_ptrs, int64_t rank, int64_t epoch,
                                                    int64_t B, int64_t H, int64_t s_per_tile, bool bf16,
                                                    at::Tensor status) {
  SANTA_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1,
              "status must be a CUDA int32 tensor");
  const santa_peer_exchange px = make_peer(peer_ptrs, rank, epoch);
  const c10::cuda::CUDAGuard guard(status.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  at::Tensor out = at::empty({B, H, 128}, status.options().dtype(bf16 ? at::kBFloat16 : at::kHalf));
  at::Tensor m_star = at::empty({B, H}, status.options().dtype(at::kFloat));
  const int rc = santa_lse_combine_wait(&px, (int)(B * H), 128, (int)s_per_tile,
                                        bf16 ? SANTA_DTYPE_BF16 : SANTA_DTYPE_F16, out.data_ptr(),
                                        m_star.data_ptr<float>(), status.data_ptr<int>(), (void*)stream.stream());
  SANTA_CHECK(rc == SANTA_OK, "santa_b200: ", santa_strerror(rc), " (code ", rc, ")");
  return std::make_tuple(out, m_star);
}

// Fold partials [G,B,H,130] fp32 of G disjoint tile sets into (out [B,H,128], m_star [B,H]).
std::tuple<at::Tensor, at::Tensor> lse_combine(at::Tensor partials, int64_t s_per_tile, bool bf16) {
  SANTA_CHECK(partials.is_cuda() && partials.scalar_type() == at::kFloat && partials.is_contiguous() &&
                  partials.dim() == 4 && partials.size(3) == 130,
              "partials must be a contiguous CUDA fp32 tensor [G,B,H,130]");
  const c10::cuda::CUDAGuard guard(partials.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int G = (int)partials.size(0), B = (int)partials.size(1), H = (int)partials.size(2);
  at::Tensor out = at::empty({B, H, 128}, partials.options().dtype(bf16 ? at::kBFloat16 : at::kHalf));
  at::Tensor m_star = at::empty({B, H}, partials.options());
  const int rc = santa_lse_combine(partials.data_ptr<float>(), G, B * H, 128, (int)s_per_tile,
                                   bf16 ? SANTA_DTYPE_BF16 : SANTA_DTYPE_F16, out.data_ptr(),
                                   m_star.data_ptr<float>(), (void*)stream.stream());
  SANTA_CHECK(rc == SANTA_OK, "santa_b200: ", santa_strerror(rc), " (code ", rc, ")");
  return std::make_tuple(out, m_star);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("decode_systematic_partial", &decode_systematic_partial, py::arg("q_h"), py::arg("K_g"), py::arg("V_g"),
        py::arg("S"), py::arg("seed") = 42ULL, py::arg("block_n") = 0, py::arg("valid_len") = -1,
        py::arg("batch_offset") = 0, py::arg("tile_offset") = 0, py::arg("s_per_tile") = -1);
  m.def("decode_systematic_exchange", &decode_systematic_exchange, py::arg("q_h"), py::arg("K_g"), py::arg("V_g"),
        py::arg("S"), py::arg("seed"), py::arg("block_n"), py::arg("valid_len"), py::arg("batch_offset"),
        py::arg("tile_offset"), py::arg("s_per_tile"), py::arg("peer_ptrs"), py::arg("rank"), py::arg("epoch"),
        py::arg("combine") = false);
  m.def("lse_combine_wait", &lse_combine_wait, py::arg("peer_ptrs"), py::arg("rank"), py::arg("epoch"), py::arg("B"),
        py::arg("H"), py::arg("s_per_tile"), py::arg("bf16"), py::arg("status"));
  m.def("lse_combine", &lse_combine, py::arg("partials"), py::arg("s_per_tile"), py::arg("bf16") = true);
  m.def("decode_systematic_ragged", &decode_systematic_ragged, py::arg("q_h"), py::arg("K_g"), py::arg("V_g"),
        py::arg("seq_lens"), py::arg("S"), py::arg("seed") = 42ULL, py::arg("block_n") = 0,
        py::arg("want_vrows") = false, py::arg("max_len") = -1, py::kw_only(), py::arg("score_mode") = 0);
  // the reference's signature (santa_cuda.cpp:346-359), plus one keyword-only extra that defaults to its behaviour
  m.def("decode_systematic_scalar", &decode_systematic, py::arg("q_h"), py::arg("K_g"), py::arg("V_g"), py::arg("S"),
        py::arg("seed") = 42ULL, py::arg("block_n") = 0, py::arg("want_vrows") = false, py::arg("valid_len") = -1,
        py::kw_only(), py::arg("score_mode") = 0);
  m.def("decode_systematic_batched", &decode_systematic, py::arg("q_h"), py::arg("K_g"), py::arg("V_g"), py::arg("S"),
        py::arg("seed") = 42ULL, py::arg("block_n") = 0, py::arg("want_vrows") = false, py::arg("valid_len") = -1,
        py::kw_only(), py::arg("score_mode") = 0);
}
