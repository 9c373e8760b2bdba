// A plain C++ host of the C ABI: no PyTorch, no Python.  Fills q/K/V with a fixed integer recurrence
// (the GPU test generates the same bits in Python), runs santa_flash_decode and prints the output's
// 16-bit patterns so that the test can compare them with the Python mirror's result.
//   usage: capi_host B L KVH S seed
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../include/santa_b200.h"

static uint16_t bf16_bits(uint32_t& state) {          // small values in (-2, 2), exactly representable
  state = state * 1664525u + 1013904223u;
  const int v = int((state >> 16) & 0xff) - 128;       // -128..127
  const float f = float(v) / 64.0f;
  uint32_t u;
  memcpy(&u, &f, 4);
  return uint16_t(u >> 16);
}

#define CK(x)                                                              \
  do {                                                                     \
    cudaError_t e_ = (x);                                                  \
    if (e_ != cudaSuccess) {                                               \
      fprintf(stderr, "cuda error %s at %s\n", cudaGetErrorString(e_), #x); \
      return 2;                                                            \
    }                                                                      \
  } while (0)

int main(int argc, char** argv) {
  if (argc != 6) return 1;
  const int B = atoi(argv[1]), L = atoi(argv[2]), KVH = atoi(argv[3]), S = atoi(argv[4]);
  const uint64_t seed = strtoull(argv[5], nullptr, 10);
  const int H = 4 * KVH, D = 128;
  std::vector<uint16_t> q(size_t(B) * H * D), K(size_t(B) * L * KVH * D), V(K.size());
  uint32_t st = 12345u;
  for (auto& x : q) x = bf16_bits(st);
  for (auto& x : K) x = bf16_bits(st);
  for (auto& x : V) x = bf16_bits(st);
  void *dq, *dK, *dV, *dout, *dws;
  float* dm;
  int32_t* dvr;
  CK(cudaMalloc(&dq, q.size() * 2));
  CK(cudaMalloc(&dK, K.size() * 2));
  CK(cudaMalloc(&dV, V.size() * 2));
  CK(cudaMalloc(&dout, q.size() * 2));
  CK(cudaMalloc(&dm, size_t(B) * H * 4));
  CK(cudaMalloc(&dvr, size_t(B) * KVH * 4));
  CK(cudaMemcpy(dq, q.data(), q.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dK, K.data(), K.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dV, V.data(), V.size() * 2, cudaMemcpyHostToDevice));
  const size_t wsb = santa_flash_workspace_bytes(B, KVH, L, 0);
  if (wsb == 0) return 3;
  CK(cudaMalloc(&dws, wsb));
  CK(cudaMemset(dws, 0, wsb));
  const int rc = santa_flash_decode(dq, dK, dV, SANTA_DTYPE_BF16, B, H, KVH, D, L, L, S, seed, 0, dout, dm, dvr, dws, wsb,
                                    nullptr, nullptr);
  if (rc != SANTA_OK) {
    fprintf(stderr, "santa_flash_decode: %s\n", santa_strerror(rc));
    return 4;
  }
  CK(cudaDeviceSynchronize());
  int32_t status = 0;
  CK(cudaMemcpy(&status, santa_workspace_status(dws), 4, cudaMemcpyDeviceToHost));
  std::vector<uint16_t> out(q.size());
  std::vector<int32_t> vr(size_t(B) * KVH);
  CK(cudaMemcpy(out.data(), dout, out.size() * 2, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(vr.data(), dvr, vr.size() * 4, cudaMemcpyDeviceToHost));
  printf("status %d\nvrows", status);
  for (int v : vr) printf(" %d", v);
  printf("\nout");
  for (uint16_t x : out) printf(" %u", unsigned(x));
  printf("\n");
  return 0;
}
