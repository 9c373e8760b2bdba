// torch_prop.cpp -- the `santa_prop_batch_cuda` Python module: a thin
// pybind11/ATen shim over the C ABI of libsanta_b200.so.
//
// Same name, argument order, defaults, tensor layouts, return tuple and error
// messages as the reference module of that name
// (santa_fused_proportional_tile_budgets/santa_cuda.cpp:141-359).  Like the
// reference it exposes ONLY decode_systematic_scalar, takes a single sequence
// (q_h [H,D]) and has no valid_len argument: tutorial_code/attention_backends.py
// (:476-500) relies on the batched call failing with a TypeError that names
// valid_len and then loops over the batch.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <stdexcept>
#include <string>
#include <tuple>
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

// SANTA_PASS1 = auto | gqa (perhead) | vec (gqa_vec), santa_cuda.cpp:39-51
int pass1_mode_from_env() {
  const char* env = std::getenv("SANTA_PASS1");
  if (!env) return 0;
  std::string s(env);
  std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return (char)std::tolower(c); });
  if (s == "gqa" || s == "perhead") return 1;
  if (s == "vec" || s == "gqa_vec") return 2;
  return 0;
}

at::Tensor& workspace_for(const at::Tensor& like, cudaStream_t stream, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, at::Tensor> cache;
  std::lock_guard<std::mutex> lock(mu);
  at::Tensor& ws = cache[{(int)like.get_device(), stream}];
  if (!ws.defined() || (size_t)ws.numel() < bytes) {
    const int64_t n = (int64_t)std::max<size_t>(bytes, size_t(8) << 20);
    ws = at::zeros({n}, like.options().dtype(at::kByte));
  }
  return ws;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> decode_systematic_scalar(at::Tensor q_h, at::Tensor K_g,
                                                                        at::Tensor V_g, int64_t S, uint64_t seed,
                                                                        int64_t block_n, bool want_vrows,
                                                                        int64_t score_mode) {
  SANTA_CHECK(q_h.is_cuda(), "q_h must be CUDA");
  SANTA_CHECK(K_g.is_cuda() && V_g.is_cuda(), "K_g and V_g must be CUDA");
  SANTA_CHECK(q_h.scalar_type() == at::kBFloat16 || q_h.scalar_type() == at::kHalf, "q_h must be bf16 or f16");
  SANTA_CHECK((K_g.scalar_type() == at::kBFloat16 || K_g.scalar_type() == at::kHalf) &&
                  K_g.scalar_type() == V_g.scalar_type(),
              "K_g/V_g must be bf16 or f16 and match");
  SANTA_CHECK(q_h.scalar_type() == K_g.scalar_type(), "q_h dtype must match K_g/V_g");
  SANTA_CHECK(q_h.dim() == 2 && K_g.dim() == 3 && V_g.dim() == 3, "bad ranks");
  SANTA_CHECK(q_h.device() == K_g.device() && q_h.device() == V_g.device(), "device mismatch");
  SANTA_CHECK(K_g.sizes() == V_g.sizes(), "K_g and V_g must have the same shape");
  SANTA_CHECK(q_h.size(1) == K_g.size(2), "D mismatch (q_h.size(1) vs K_g.size(2))");
  SANTA_CHECK(q_h.size(0) % K_g.size(1) == 0, "H must be divisible by KVH (expected KVH == K_g.size(1) for NHD)");
  SANTA_CHECK(K_g.is_contiguous() && V_g.is_contiguous(), "K_g/V_g must be contiguous with layout [L, KVH, D] (NHD)");

  const int H = (int)q_h.size(0), D = (int)q_h.size(1), L = (int)K_g.size(0), KVH = (int)K_g.size(1);
  // any GH and D % 16 == 0 like the reference (santa_cuda.cpp:212-247); its second pass launches 128 x GH
  // threads per block (santa_cuda_kernel.cu:924-927), which bounds GH by 8
  SANTA_CHECK(H / KVH <= 8, "This build supports up to 8 query heads per kv-head. Got GH=", H / KVH);
  SANTA_CHECK(D <= 256, "This build supports head dimensions up to 256. Got D=", D);
  const int mode = pass1_mode_from_env();
  int bn = (int)block_n;
  if (bn <= 0) bn = (mode == 2) ? 256 : santa_block_n_rule(L, 0);
  SANTA_CHECK(mode != 2 || (H / KVH == 4 && D == 128 && bn == 256),
              "SANTA_PASS1=vec requires GH=4, D=128, block_n=256. Got GH=", H / KVH, " D=", D, " block_n=", bn);
  SANTA_CHECK(D % 16 == 0 && bn % 16 == 0,
              "Pass-1 WMMA-GQA requires D % 16 == 0 and block_n % 16 == 0. Got D=", D, " block_n=", bn);
  SANTA_CHECK(bn <= 256, "This build supports block_n up to 256. Got block_n=", bn);

  // argument errors are raised above, before any device state is touched
  const c10::cuda::CUDAGuard guard(q_h.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto q = q_h.contiguous();

  at::Tensor out = at::empty({H, D}, q.options());
  at::Tensor m_star = at::empty({H}, q.options().dtype(at::kFloat));
  at::Tensor vrows = at::empty({want_vrows ? (int64_t)KVH : (int64_t)0}, q.options().dtype(at::kInt));

  const size_t ws_bytes = santa_prop_workspace_bytes(H, KVH, D, L, bn);
  SANTA_CHECK(ws_bytes > 0, "santa_b200: could not size the workspace");
  at::Tensor& ws = workspace_for(q, stream.stream(), ws_bytes);
  SANTA_CHECK(score_mode == SANTA_SCORE_EXACT || score_mode == SANTA_SCORE_TENSOR, "score_mode must be 0 or 1");
  santa_prop_ext ext{};
  ext.pass1_mode = mode;
  ext.flags = 3;
  ext.score_mode = (int)score_mode;  // not part of the reference's signature; 0 is its arithmetic
  const int rc = santa_prop_decode(q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(),
                                   q.scalar_type() == at::kBFloat16 ? SANTA_DTYPE_BF16 : SANTA_DTYPE_F16, H, KVH, D,
                                   L, S, seed, bn, out.data_ptr(), m_star.data_ptr<float>(),
                                   want_vrows ? vrows.data_ptr<int>() : nullptr, ws.data_ptr(), (size_t)ws.numel(),
                                   &ext, (void*)stream.stream());
  SANTA_CHECK(rc == SANTA_OK, "santa_b200: ", santa_strerror(rc), " (code ", rc, ", cuda ", santa_last_cuda_error(),
              ")");
  return std::make_tuple(out, m_star, vrows);
}

// Ragged batch in one launch sequence; not part of the reference module.  It is exported under
// its own name: the reference adapter treats a module that has `decode_systematic_batched` as truly
// batched with Flash semantics (tutorial_code/attention_backends.py:447), which this is not --
// every sequence here uses the head index h in the random stream, as the adapter's per-sequence
// loop does (attention_backends.py:491-500).
std::tuple<at::Tensor, at::Tensor, at::Tensor> decode_systematic_ragged(at::Tensor q_bh, at::Tensor K_g,
                                                                        at::Tensor V_g, at::Tensor seq_lens,
                                                                        int64_t S, uint64_t seed, bool want_vrows,
                                                                        int64_t max_len, int64_t score_mode) {
  SANTA_CHECK(q_bh.is_cuda() && K_g.is_cuda() && V_g.is_cuda(), "q_bh, K_g and V_g must be CUDA");
  SANTA_CHECK(q_bh.scalar_type() == at::kBFloat16 || q_bh.scalar_type() == at::kHalf, "q_bh must be bf16 or f16");
  SANTA_CHECK(K_g.scalar_type() == q_bh.scalar_type() && V_g.scalar_type() == q_bh.scalar_type(),
              "q_bh dtype must match K_g/V_g");
  SANTA_CHECK(q_bh.dim() == 3 && K_g.dim() == 4 && V_g.dim() == 4,
              "Ragged path expects q_bh [B,H,D], K_g/V_g [B,L,KVH,D]");
  SANTA_CHECK(q_bh.device() == K_g.device() && q_bh.device() == V_g.device(), "device mismatch");
  SANTA_CHECK(K_g.sizes() == V_g.sizes(), "K_g and V_g must have the same shape");
  SANTA_CHECK(q_bh.size(0) == K_g.size(0), "Batch mismatch between q_bh and K_g/V_g");
  SANTA_CHECK(q_bh.size(2) == K_g.size(3), "D mismatch (q_bh.size(2) vs K_g.size(3))");
  SANTA_CHECK(K_g.is_contiguous() && V_g.is_contiguous(), "K_g/V_g must be contiguous with layout [B, L, KVH, D]");
  const int B = (int)q_bh.size(0), H = (int)q_bh.size(1), D = (int)q_bh.size(2);
  const int L_storage = (int)K_g.size(1), KVH = (int)K_g.size(2);
  SANTA_CHECK(D == 128 && H == 4 * KVH, "This build supports only D=128 and GH=4 (H/KVH). Got D=", D, " H=", H,
              " KVH=", KVH);
  SANTA_CHECK(seq_lens.scalar_type() == at::kInt && seq_lens.dim() == 1 && seq_lens.size(0) == B,
              "seq_lens must be an int32 tensor with one length per sequence");
  const int mlen = max_len > 0 ? (int)max_len : L_storage;
  SANTA_CHECK(mlen <= L_storage, "max_len exceeds storage length: max_len=", mlen, " storage=", L_storage);
  SANTA_CHECK(B <= 1024, "The ragged path takes at most 1024 sequences. Got B=", B);

  const c10::cuda::CUDAGuard guard(q_bh.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto q = q_bh.contiguous();
  // lengths are read on the device when the kernels run; a host tensor is copied over
  at::Tensor lens = seq_lens.is_cuda() ? seq_lens.contiguous() : seq_lens.to(q.device(), /*non_blocking=*/false);
  SANTA_CHECK(lens.device() == q.device(), "seq_lens must be on q_bh's device or on the CPU");

  at::Tensor out = at::empty({B, H, D}, q.options());
  at::Tensor m_star = at::empty({B, H}, q.options().dtype(at::kFloat));
  at::Tensor vrows = want_vrows ? at::empty({B, KVH}, q.options().dtype(at::kInt))
                                : at::empty({0}, q.options().dtype(at::kInt));
  const size_t ws_bytes = santa_prop_ragged_workspace_bytes(B, H, KVH, D, mlen);
  SANTA_CHECK(ws_bytes > 0, "santa_b200: could not size the workspace");
  at::Tensor& ws = workspace_for(q, stream.stream(), ws_bytes);
  SANTA_CHECK(score_mode == SANTA_SCORE_EXACT || score_mode == SANTA_SCORE_TENSOR, "score_mode must be 0 or 1");
  santa_prop_ext ext{};
  ext.flags = 3;
  ext.score_mode = (int)score_mode;
  const int rc = santa_prop_decode_ragged(
      q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(), q.scalar_type() == at::kBFloat16 ? SANTA_DTYPE_BF16 : SANTA_DTYPE_F16,
      B, H, KVH, D, L_storage, lens.data_ptr<int>(), mlen, S, seed, out.data_ptr(), m_star.data_ptr<float>(),
      want_vrows ? vrows.data_ptr<int>() : nullptr, ws.data_ptr(), (size_t)ws.numel(), &ext,
      (void*)stream.stream());
  SANTA_CHECK(rc == SANTA_OK, "santa_b200: ", santa_strerror(rc), " (code ", rc, ", cuda ", santa_last_cuda_error(),
              ")");
  return std::make_tuple(out, m_star, vrows);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("decode_systematic_ragged", &decode_systematic_ragged, py::arg("q_bh"), py::arg("K_g"), py::arg("V_g"),
        py::arg("seq_lens"), py::arg("S"), py::arg("seed") = 42ULL, py::arg("want_vrows") = false,
        py::arg("max_len") = -1, py::kw_only(), py::arg("score_mode") = 0);
  // the reference's signature (santa_cuda.cpp:354-359) plus one keyword-only extra that defaults to its behaviour
  m.def("decode_systematic_scalar", &decode_systematic_scalar, py::arg("q_h"), py::arg("K_g"), py::arg("V_g"),
        py::arg("S"), py::arg("seed") = 42ULL, py::arg("block_n") = 0, py::arg("want_vrows") = false,
        py::kw_only(), py::arg("score_mode") = 0);
}
