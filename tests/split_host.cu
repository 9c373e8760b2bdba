// Host-side check of the work-split arithmetic that the kernels share (santa_b200/csrc/common.cuh):
// the equal-count split (range_lo / cta_of_item) and the weighted split of a ragged Prop batch
// (prop_unit_weight / item_at_weight).  Compiled with nvcc as a plain host program by the CPU suite;
// nothing runs on a GPU.  For random ragged batches it checks that the ranges tile the items exactly
// once, that none is empty, and that the range the merge kernel computes for a column's first and
// last item (cta_of_item in weight space) is the range that owns that item.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../santa_b200/csrc/common.cuh"

using namespace santa;

static unsigned long long rng_state = 88172645463325252ull;
static unsigned rnd() {
  rng_state ^= rng_state << 13;
  rng_state ^= rng_state >> 7;
  rng_state ^= rng_state << 17;
  return unsigned(rng_state >> 11);
}

int main() {
  const int bn = 256;
  const long long budgets[] = {0, 1, 3, 64, 256, 2048};
  const int kvhs[] = {1, 2, 8};
  const int groups[] = {1, 3, 8, 64, 2368};
  long long checked_items = 0;
  for (int trial = 0; trial < 4000; ++trial) {
    const int nseq = 1 + rnd() % 12, KVH = kvhs[rnd() % 3];
    const long long S = budgets[rnd() % 6];
    std::vector<int> T(nseq), start(nseq + 1, 0);
    std::vector<long long> wstart(nseq + 1, 0);
    int wmax = 0;
    for (int b = 0; b < nseq; ++b) {
      const int pick = rnd() % 6;
      const int len = pick == 0 ? 0 : pick == 1 ? 1 : pick == 2 ? 255 : pick == 3 ? 256 : pick == 4 ? 257 : 1 + rnd() % 70000;
      T[b] = (len + bn - 1) / bn;
      const int w = prop_unit_weight(T[b], S);
      start[b + 1] = start[b] + T[b] * KVH;
      wstart[b + 1] = wstart[b] + (long long)T[b] * KVH * w;
      if (T[b] > 0 && w > wmax) wmax = w;
    }
    const long long items = start[nseq], W = wstart[nseq];
    const long long fit = wmax > 0 ? W / wmax : 0;
    const int cap = groups[rnd() % 5];
    const int nvg = int(fit < cap ? fit : cap);
    if (items == 0) {
      if (nvg != 0) { std::printf("FAIL: ranges for an empty batch\n"); return 1; }
      continue;
    }
    if (nvg < 1) { std::printf("FAIL: no range for %lld items\n", items); return 1; }
    std::vector<int> owner(items, -1);
    for (int vg = 0; vg < nvg; ++vg) {
      const long long lo = item_at_weight(start.data(), wstart.data(), nseq, range_lo(vg, W, nvg), KVH, S);
      const long long hi = item_at_weight(start.data(), wstart.data(), nseq, range_lo(vg + 1, W, nvg), KVH, S);
      if (!(lo < hi) || hi > items) { std::printf("FAIL: empty or overlong range %d in trial %d\n", vg, trial); return 1; }
      for (long long x = lo; x < hi; ++x) {
        if (owner[x] != -1) { std::printf("FAIL: item owned twice\n"); return 1; }
        owner[x] = vg;
      }
    }
    for (long long x = 0; x < items; ++x)
      if (owner[x] < 0) { std::printf("FAIL: item %lld of trial %d without a range\n", x, trial); return 1; }
    for (int b = 0; b < nseq; ++b) {
      if (T[b] == 0) continue;
      const long long w = prop_unit_weight(T[b], S);
      for (int kv = 0; kv < KVH; ++kv) {
        const long long w0 = wstart[b] + (long long)kv * T[b] * w, w1 = w0 + (long long)(T[b] - 1) * w;
        const long long x0 = start[b] + (long long)kv * T[b];
        if (cta_of_item(w0, W, nvg) != owner[x0] || cta_of_item(w1, W, nvg) != owner[x0 + T[b] - 1]) {
          std::printf("FAIL: the merge kernel's range of a column differs from the owner (trial %d)\n", trial);
          return 1;
        }
      }
    }
    // the equal-count split of the same items
    for (long long x = 0; x < items; x += 1 + items / 97) {
      const int n2 = int(items < cap ? items : cap);
      const int c = cta_of_item(x, items, n2);
      if (!(range_lo(c, items, n2) <= x && x < range_lo(c + 1, items, n2))) { std::printf("FAIL: cta_of_item\n"); return 1; }
    }
    checked_items += items;
  }
  std::printf("ok %lld\n", checked_items);
  return 0;
}
