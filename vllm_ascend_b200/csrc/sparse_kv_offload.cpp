// Host-side resident-set bookkeeping for sparse-attention KV offload.
//
// With sparse attention only the top-k tokens picked by the indexer are read per step, so the
// full KV of a sequence can live in host memory and the GPU keeps a small per-sequence pool of
// token slots.  Every step, for each sequence, this module maps the selected tokens to device
// slots: hits keep their slot, misses take the least recently used slot of the sequence and
// are reported as (host token -> device slot) copies.  The work is independent per sequence
// and runs on a few host threads.  Native counterpart of the reference's sparse_kv_offload.cpp
// (OpenMP LRU / resident-set maintenance, vllm_ascend/distributed/kv_transfer/sparse_kv_offload/).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <list>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#define SKO_API extern "C" __attribute__((visibility("default")))

namespace {

struct SeqState {
  int capacity = 0;
  std::unordered_map<int, int> slot_of;                  // token -> slot
  std::list<int> lru;                                    // tokens, most recent first
  std::unordered_map<int, std::list<int>::iterator> pos; // token -> place in lru
  std::vector<int> free_slots;
};

struct Manager {
  int capacity;
  std::unordered_map<long, SeqState> seqs;
  std::mutex mu;
  long hits = 0, misses = 0, evictions = 0;
};

SeqState& seq_of(Manager* m, long id) {
  std::lock_guard<std::mutex> g(m->mu);
  auto it = m->seqs.find(id);
  if (it == m->seqs.end()) {
    SeqState s;
    s.capacity = m->capacity;
    s.free_slots.resize(m->capacity);
    for (int i = 0; i < m->capacity; i++) s.free_slots[i] = m->capacity - 1 - i;
    it = m->seqs.emplace(id, std::move(s)).first;
  }
  return it->second;
}

// returns number of misses written; -1 when the selection does not fit the pool
int update_one(SeqState& s, const int* topk, int k, int* slots, int* miss_tok, int* miss_slot,
               long* hits, long* evictions) {
  int n_miss = 0;
  // first pass: touch hits so they cannot be evicted by this step's misses
  for (int i = 0; i < k; i++) {
    const int tok = topk[i];
    if (tok < 0) { slots[i] = -1; continue; }
    auto it = s.slot_of.find(tok);
    if (it != s.slot_of.end()) {
      slots[i] = it->second;
      s.lru.erase(s.pos[tok]);
      s.lru.push_front(tok);
      s.pos[tok] = s.lru.begin();
      (*hits)++;
    } else {
      slots[i] = -2;
    }
  }
  int protected_count = 0;
  for (int i = 0; i < k; i++) protected_count += slots[i] >= 0;
  for (int i = 0; i < k; i++) {
    if (slots[i] != -2) continue;
    const int tok = topk[i];
    auto dup = s.slot_of.find(tok);            // the same token twice in one selection
    if (dup != s.slot_of.end()) { slots[i] = dup->second; continue; }
    int slot;
    if (!s.free_slots.empty()) {
      slot = s.free_slots.back();
      s.free_slots.pop_back();
    } else {
      if ((int)s.lru.size() <= protected_count) return -1;   // every resident token is needed now
      const int victim = s.lru.back();
      s.lru.pop_back();
      slot = s.slot_of[victim];
      s.slot_of.erase(victim);
      s.pos.erase(victim);
      (*evictions)++;
    }
    s.slot_of[tok] = slot;
    s.lru.push_front(tok);
    s.pos[tok] = s.lru.begin();
    protected_count++;
    slots[i] = slot;
    miss_tok[n_miss] = tok;
    miss_slot[n_miss] = slot;
    n_miss++;
  }
  return n_miss;
}

}  // namespace

SKO_API void* b200_sko_create(int slots_per_sequence) {
  if (slots_per_sequence <= 0) return nullptr;
  Manager* m = new Manager();
  m->capacity = slots_per_sequence;
  return m;
}

SKO_API void b200_sko_destroy(void* h) { delete (Manager*)h; }

SKO_API void b200_sko_release(void* h, long seq_id) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  m->seqs.erase(seq_id);
}

// seq_ids [B]; topk [B, k] token positions (-1 = unused entry).
// out: slots [B, k] device slot of every selected token (-1 for unused entries);
//      miss_tok / miss_slot [B, k] with miss_count [B] valid entries per row: the copies to issue.
// Returns 0, or 1 + the index of the first sequence whose selection exceeds the pool.
SKO_API int b200_sko_update(void* h, const long* seq_ids, int B, const int* topk, int k, int* slots,
                            int* miss_tok, int* miss_slot, int* miss_count, int num_threads) {
  Manager* m = (Manager*)h;
  std::vector<SeqState*> states(B);
  for (int b = 0; b < B; b++) states[b] = &seq_of(m, seq_ids[b]);
  if (num_threads < 1) num_threads = 1;
  num_threads = std::min(num_threads, std::max(1, B));
  std::vector<long> hits(num_threads, 0), evs(num_threads, 0);
  std::vector<int> bad(num_threads, 0);
  auto work = [&](int tid) {
    for (int b = tid; b < B; b += num_threads) {
      const int n = update_one(*states[b], topk + (long)b * k, k, slots + (long)b * k,
                               miss_tok + (long)b * k, miss_slot + (long)b * k, &hits[tid], &evs[tid]);
      if (n < 0) { miss_count[b] = 0; if (!bad[tid]) bad[tid] = b + 1; }
      else miss_count[b] = n;
    }
  };
  if (num_threads == 1) {
    work(0);
  } else {
    std::vector<std::thread> ts;
    for (int t = 0; t < num_threads; t++) ts.emplace_back(work, t);
    for (auto& t : ts) t.join();
  }
  long h_sum = 0, e_sum = 0, miss_sum = 0;
  for (int t = 0; t < num_threads; t++) { h_sum += hits[t]; e_sum += evs[t]; }
  for (int b = 0; b < B; b++) miss_sum += miss_count[b];
  {
    std::lock_guard<std::mutex> g(m->mu);
    m->hits += h_sum; m->evictions += e_sum; m->misses += miss_sum;
  }
  for (int t = 0; t < num_threads; t++) if (bad[t]) return bad[t];
  return 0;
}

SKO_API void b200_sko_stats(void* h, long* out3) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  out3[0] = m->hits; out3[1] = m->misses; out3[2] = m->evictions;
}
