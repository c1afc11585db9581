// Driver for the address / undefined-behaviour sanitizer build of the host-side LRU bookkeeping
// (csrc/sparse_kv_offload.cpp): random selections over many sequences with threads, capacity
// overflow, release and re-use.  Exits 0 when every invariant holds and the sanitizers stay silent.
#include <cstdio>
#include <cstdlib>
#include <set>
#include <vector>

extern "C" {
void* b200_sko_create(int slots_per_sequence);
void b200_sko_destroy(void* h);
void b200_sko_release(void* h, long seq_id);
int b200_sko_update(void* h, const long* seq_ids, int B, const int* topk, int k, int* slots, int* miss_tok,
                    int* miss_slot, int* miss_count, int num_threads);
void b200_sko_stats(void* h, long* out);
}

#define CHECK(c)                                                    \
  do {                                                              \
    if (!(c)) { std::printf("FAILED %s line %d\n", #c, __LINE__); return 1; } \
  } while (0)

int main() {
  const int cap = 24, B = 16, k = 8;
  void* h = b200_sko_create(cap);
  CHECK(h != nullptr);
  CHECK(b200_sko_create(0) == nullptr);
  std::vector<long> ids(B);
  for (int b = 0; b < B; b++) ids[b] = 100 + b;
  std::vector<int> topk(B * k), slots(B * k), mt(B * k), ms(B * k), mc(B);
  unsigned seed = 12345;
  auto rnd = [&](int n) { seed = seed * 1103515245u + 12345u; return (int)((seed >> 8) % (unsigned)n); };
  for (int step = 0; step < 400; step++) {
    for (int b = 0; b < B; b++) {
      std::set<int> used;
      for (int i = 0; i < k; i++) {
        int t = rnd(10) == 0 ? -1 : rnd(64);
        topk[b * k + i] = t;
      }
    }
    const int rc = b200_sko_update(h, ids.data(), B, topk.data(), k, slots.data(), mt.data(), ms.data(), mc.data(),
                                   1 + step % 4);
    CHECK(rc == 0);
    for (int b = 0; b < B; b++) {
      CHECK(mc[b] >= 0 && mc[b] <= k);
      for (int i = 0; i < k; i++) {
        const int t = topk[b * k + i], s = slots[b * k + i];
        CHECK((t < 0) == (s < 0));
        CHECK(s < cap);
        for (int j = 0; j < i; j++)            // two different tokens never share a slot within one step
          if (topk[b * k + j] >= 0 && t >= 0 && topk[b * k + j] != t) CHECK(slots[b * k + j] != s);
      }
      for (int i = 0; i < mc[b]; i++) CHECK(ms[b * k + i] >= 0 && ms[b * k + i] < cap && mt[b * k + i] >= 0);
    }
    if (step % 50 == 49) b200_sko_release(h, ids[step % B]);
  }
  // a selection with more distinct tokens than the pool holds is refused, not corrupted
  void* small = b200_sko_create(4);
  long one = 7;
  int sel[8] = {0, 1, 2, 3, 4, 5, 6, 7}, so[8], a[8], c[8], n[1];
  CHECK(b200_sko_update(small, &one, 1, sel, 8, so, a, c, n, 1) == 1);
  int ok_sel[8] = {0, 1, 2, 3, -1, -1, -1, -1};
  CHECK(b200_sko_update(small, &one, 1, ok_sel, 8, so, a, c, n, 1) == 0);
  long st[3];
  b200_sko_stats(h, st);
  CHECK(st[0] > 0 && st[1] > 0 && st[2] > 0);
  b200_sko_destroy(small);
  b200_sko_destroy(h);
  std::printf("OK hits=%ld misses=%ld evictions=%ld\n", st[0], st[1], st[2]);
  return 0;
}
