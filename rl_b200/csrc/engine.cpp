// Host runtime of the generation engine: paged-KV block manager with reference counts (prefix
// sharing between the samples of one prompt, copy-on-write of the partial tail block), and a
// continuous-batching scheduler (admission by free blocks / running limit / prefill token budget,
// preemption by recompute when blocks run out).
//
// The model forward, attention and sampling run as CUDA kernels driven from Python; this file owns
// the bookkeeping that decides, every step, which sequences prefill, which decode, and where each
// new token's K/V goes. It is the in-house counterpart of the scheduler and block manager that the
// reference gets from vLLM (nemo_rl/models/generation/vllm/vllm_worker.py:570-597).
//
// Plain C ABI; all handles are opaque pointers. Not thread-safe: one engine, one driver thread.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <unordered_map>
#include <vector>

#define RLB_API extern "C" __attribute__((visibility("default")))

namespace {

enum SeqState : int { WAITING = 0, RUNNING = 1, FINISHED = 2 };

struct Seq {
  long long id = 0;
  int prompt_len = 0;
  int max_new = 0;
  int num_tokens = 0;      // tokens whose K/V is (or is about to be) in the cache
  int num_generated = 0;
  int state = WAITING;
  long long share_with = -1;  // id of a sequence with an identical prompt whose blocks can be shared
  bool prefilled = false;
  long long arrival = 0;
  std::vector<int> blocks;
  std::vector<unsigned long long> hashes;  // content hash of every full block of the prompt (chained: covers the prefix)
  int cached_prefix = 0;                   // tokens of the current admission whose K/V were found in the prefix cache
};

struct Engine {
  int num_blocks, block_size, max_running, max_prefill_tokens;
  std::vector<int> free_list;
  std::vector<int> refcount;
  std::unordered_map<long long, Seq> seqs;
  std::deque<long long> waiting;
  std::vector<long long> running;
  long long clock = 0;
  long long n_preempt = 0;
  int lookahead = 1;   // decode steps the host wants to run between two visits (multi-step decode)
  int window = 1;      // steps granted by the last schedule() call
  // Prefix cache: full prompt blocks are registered under the hash of the token prefix they end. A registered block whose
  // last user has finished keeps its contents and waits in `cached_free` (oldest first) until a request with the same
  // prefix takes it over again or the allocator runs out of plain free blocks and evicts it.
  std::unordered_map<unsigned long long, int> cache_table;   // prefix hash -> block
  std::vector<unsigned long long> block_hash;                // per block: its hash (valid when block_cached)
  std::vector<char> block_cached;
  std::deque<int> cached_free;
  long long cache_hits = 0, cache_queries = 0, cache_evictions = 0;
  // scratch of the last schedule() call
  std::vector<long long> prefill_ids, decode_ids, shared_ids;
  std::vector<int> copy_src, copy_dst;

  int blocks_for(int tokens) const { return (tokens + block_size - 1) / block_size; }
  int available_blocks() const { return static_cast<int>(free_list.size() + cached_free.size()); }
  void forget_block(int b) {
    if (block_cached[b]) {
      auto it = cache_table.find(block_hash[b]);
      if (it != cache_table.end() && it->second == b) cache_table.erase(it);
      block_cached[b] = 0;
    }
  }
  int alloc_block() {
    int b;
    if (!free_list.empty()) {
      b = free_list.back();
      free_list.pop_back();
    } else if (!cached_free.empty()) {
      b = cached_free.front();   // evict the block that has been unused for the longest time
      cached_free.pop_front();
      forget_block(b);
      ++cache_evictions;
    } else {
      return -1;
    }
    refcount[b] = 1;
    return b;
  }
  void release_block(int b) {
    if (--refcount[b] == 0) {
      if (block_cached[b]) cached_free.push_back(b);
      else free_list.push_back(b);
    }
  }
  // Takes a cached block into use again (it may be waiting in cached_free or be shared with a running sequence).
  void retain_cached(int b) {
    if (refcount[b] == 0) {
      auto it = std::find(cached_free.begin(), cached_free.end(), b);
      if (it != cached_free.end()) cached_free.erase(it);
    }
    ++refcount[b];
  }
  void register_block(int b, unsigned long long h) {
    if (block_cached[b] || cache_table.count(h)) return;
    cache_table[h] = b;
    block_hash[b] = h;
    block_cached[b] = 1;
  }
  void release_seq(Seq& s) {
    for (int b : s.blocks) release_block(b);
    s.blocks.clear();
  }
  // Grows `s` to hold `tokens` tokens. Returns false (and changes nothing) when blocks run out.
  bool ensure_capacity(Seq& s, int tokens) {
    const int need = blocks_for(tokens) - static_cast<int>(s.blocks.size());
    if (need <= 0) return true;
    if (available_blocks() < need) return false;
    for (int i = 0; i < need; ++i) s.blocks.push_back(alloc_block());
    return true;
  }
};

}  // namespace

RLB_API void* rlb_engine_create(int num_blocks, int block_size, int max_running, int max_prefill_tokens) {
  if (num_blocks <= 0 || block_size <= 0 || max_running <= 0) return nullptr;
  Engine* e = new Engine();
  e->num_blocks = num_blocks;
  e->block_size = block_size;
  e->max_running = max_running;
  e->max_prefill_tokens = max_prefill_tokens > 0 ? max_prefill_tokens : (1 << 30);
  e->refcount.assign(num_blocks, 0);
  e->block_hash.assign(num_blocks, 0ull);
  e->block_cached.assign(num_blocks, 0);
  e->free_list.reserve(num_blocks);
  for (int b = num_blocks - 1; b >= 0; --b) e->free_list.push_back(b);
  return e;
}

RLB_API void rlb_engine_destroy(void* h) { delete static_cast<Engine*>(h); }

RLB_API int rlb_engine_num_free_blocks(void* h) { return static_cast<Engine*>(h)->available_blocks(); }
RLB_API int rlb_engine_num_running(void* h) { return static_cast<int>(static_cast<Engine*>(h)->running.size()); }
RLB_API int rlb_engine_num_waiting(void* h) { return static_cast<int>(static_cast<Engine*>(h)->waiting.size()); }
RLB_API long long rlb_engine_num_preemptions(void* h) { return static_cast<Engine*>(h)->n_preempt; }

// Adds a request. share_with: id of an earlier request with the same prompt tokens (or -1). Returns 0,
// or -1 when the id exists / the request can never fit.
RLB_API int rlb_engine_add(void* h, long long id, int prompt_len, int max_new_tokens, long long share_with) {
  Engine* e = static_cast<Engine*>(h);
  if (e->seqs.count(id) || prompt_len <= 0) return -1;
  if (e->blocks_for(prompt_len + max_new_tokens) > e->num_blocks) return -1;
  Seq s;
  s.id = id;
  s.prompt_len = prompt_len;
  s.max_new = max_new_tokens;
  s.share_with = share_with;
  s.arrival = e->clock++;
  e->seqs.emplace(id, std::move(s));
  e->waiting.push_back(id);
  return 0;
}

// Plans one engine step.
//  * running sequences get room for one more token; when blocks run out the most recently arrived
//    running sequence is preempted (blocks freed, back to the head of the waiting queue, recompute);
//  * waiting sequences are admitted in order while blocks, the running limit and the prefill token
//    budget allow. A sequence whose `share_with` partner has been prefilled in an earlier step (or is
//    being prefilled in this one) reuses the partner's full prompt blocks by reference and receives a
//    private copy of the partial tail block, so it needs no prefill compute of its own.
// Counts are returned through n_*; the id lists are read with rlb_engine_get_*.
RLB_API int rlb_engine_schedule(void* h, int* n_prefill, int* n_shared, int* n_decode, int* n_copies) {
  Engine* e = static_cast<Engine*>(h);
  e->prefill_ids.clear();
  e->decode_ids.clear();
  e->shared_ids.clear();
  e->copy_src.clear();
  e->copy_dst.clear();

  // 1. decode slots for the running set (oldest first so that preemption hits the youngest)
  std::sort(e->running.begin(), e->running.end(),
            [&](long long a, long long b) { return e->seqs[a].arrival < e->seqs[b].arrival; });
  // Multi-step decode: every running sequence gets room for `window` more tokens (never beyond its own limit), so that
  // the device can run that many steps from the block table alone. When the free blocks do not cover the full
  // look-ahead for everybody, this call falls back to single steps (and to preemption if even those do not fit).
  int want = e->lookahead;
  if (want > 1) {
    long long need = 0;
    for (long long id : e->running) {
      const Seq& s = e->seqs[id];
      const int rem = std::max(1, s.max_new - s.num_generated);
      need += std::max(0, e->blocks_for(s.num_tokens + std::min(want, rem)) - static_cast<int>(s.blocks.size()));
    }
    if (need > static_cast<long long>(e->available_blocks())) want = 1;
  }
  e->window = want;
  size_t i = 0;
  while (i < e->running.size()) {
    Seq& s = e->seqs[e->running[i]];
    if (e->ensure_capacity(s, s.num_tokens + std::min(want, std::max(1, s.max_new - s.num_generated)))) {
      ++i;
      continue;
    }
    // out of blocks: preempt the youngest running sequence (possibly this one)
    long long victim_id = e->running.back();
    Seq& v = e->seqs[victim_id];
    e->release_seq(v);
    v.state = WAITING;
    v.prefilled = false;
    // recompute from scratch: generated tokens become part of the prompt on re-admission
    v.num_tokens = 0;
    e->running.pop_back();
    e->waiting.push_front(victim_id);
    ++e->n_preempt;
    if (victim_id == s.id) break;  // everything at and after i is gone
  }
  for (long long id : e->running) e->decode_ids.push_back(id);

  // 2. admission
  int prefill_tokens = 0;
  while (!e->waiting.empty() && static_cast<int>(e->running.size()) < e->max_running) {
    const long long id = e->waiting.front();
    Seq& s = e->seqs[id];
    const int context = s.prompt_len + s.num_generated;  // recompute includes what was generated
    Seq* partner = nullptr;
    if (s.share_with >= 0 && s.num_generated == 0) {
      auto it = e->seqs.find(s.share_with);
      if (it != e->seqs.end() && it->second.state == RUNNING && it->second.prefilled &&
          it->second.prompt_len == s.prompt_len &&
          static_cast<int>(it->second.blocks.size()) >= e->blocks_for(s.prompt_len))
        partner = &it->second;
    }
    if (partner) {
      const int full = s.prompt_len / e->block_size;
      const int total = e->blocks_for(s.prompt_len + 1);
      const int fresh = total - full;
      if (e->available_blocks() < fresh) break;
      for (int b = 0; b < full; ++b) {
        s.blocks.push_back(partner->blocks[b]);
        ++e->refcount[partner->blocks[b]];
      }
      for (int b = full; b < total; ++b) s.blocks.push_back(e->alloc_block());
      if (s.prompt_len % e->block_size) {
        e->copy_src.push_back(partner->blocks[full]);
        e->copy_dst.push_back(s.blocks[full]);
      }
      s.num_tokens = s.prompt_len;
      s.prefilled = true;
      s.state = RUNNING;
      e->shared_ids.push_back(id);
    } else {
      // prefix cache: the longest run of leading full prompt blocks whose hashes are registered is taken over by
      // reference; at least one token is always left to compute (its logits start the generation)
      int hit = 0;
      if (s.blocks.empty() && !s.hashes.empty()) {
        const int max_blocks_hit = std::min(static_cast<int>(s.hashes.size()), (context - 1) / e->block_size);
        ++e->cache_queries;
        while (hit < max_blocks_hit) {
          auto it = e->cache_table.find(s.hashes[hit]);
          if (it == e->cache_table.end()) break;
          ++hit;
        }
      }
      const int fresh_tokens = context - hit * e->block_size;
      if (prefill_tokens > 0 && prefill_tokens + fresh_tokens > e->max_prefill_tokens) break;
      for (int b = 0; b < hit; ++b) {
        const int blk = e->cache_table[s.hashes[b]];
        e->retain_cached(blk);
        s.blocks.push_back(blk);
      }
      if (!e->ensure_capacity(s, context + 1)) {
        e->release_seq(s);   // gives the borrowed prefix back (it stays cached)
        break;
      }
      if (hit) ++e->cache_hits;
      s.cached_prefix = hit * e->block_size;
      prefill_tokens += fresh_tokens;
      s.num_tokens = context;
      s.prefilled = true;  // true once this step's prefill kernels have run; partners see it from the next admission on
      s.state = RUNNING;
      e->prefill_ids.push_back(id);
    }
    e->running.push_back(id);
    e->waiting.pop_front();
  }
  *n_prefill = static_cast<int>(e->prefill_ids.size());
  *n_shared = static_cast<int>(e->shared_ids.size());
  *n_decode = static_cast<int>(e->decode_ids.size());
  *n_copies = static_cast<int>(e->copy_src.size());
  return 0;
}

RLB_API void rlb_engine_get_lists(void* h, long long* prefill_ids, long long* shared_ids, long long* decode_ids,
                                  int* copy_src, int* copy_dst) {
  Engine* e = static_cast<Engine*>(h);
  if (prefill_ids) std::copy(e->prefill_ids.begin(), e->prefill_ids.end(), prefill_ids);
  if (shared_ids) std::copy(e->shared_ids.begin(), e->shared_ids.end(), shared_ids);
  if (decode_ids) std::copy(e->decode_ids.begin(), e->decode_ids.end(), decode_ids);
  if (copy_src) std::copy(e->copy_src.begin(), e->copy_src.end(), copy_src);
  if (copy_dst) std::copy(e->copy_dst.begin(), e->copy_dst.end(), copy_dst);
}

// Fills, for `n` sequence ids: the block table rows (padded with 0 to `max_blocks`), the current
// token counts (context lengths before the step's new token), and the cache slot of the next token.
RLB_API int rlb_engine_fill_tables(void* h, const long long* ids, int n, int max_blocks, int* block_table,
                                   int* context_lens, long long* next_slots) {
  Engine* e = static_cast<Engine*>(h);
  for (int i = 0; i < n; ++i) {
    auto it = e->seqs.find(ids[i]);
    if (it == e->seqs.end()) return -1;
    const Seq& s = it->second;
    const int nb = static_cast<int>(s.blocks.size());
    if (nb > max_blocks) return -2;
    int* row = block_table + static_cast<long long>(i) * max_blocks;
    std::memcpy(row, s.blocks.data(), sizeof(int) * nb);
    std::memset(row + nb, 0, sizeof(int) * (max_blocks - nb));
    if (context_lens) context_lens[i] = s.num_tokens;
    if (next_slots) {
      const int blk = s.num_tokens / e->block_size;
      next_slots[i] = blk < nb ? static_cast<long long>(s.blocks[blk]) * e->block_size + s.num_tokens % e->block_size
                               : -1;
    }
  }
  return 0;
}

// Cache slots of tokens [first, first+count) of one sequence (used by prefill to scatter K/V).
RLB_API int rlb_engine_fill_slots(void* h, long long id, int first, int count, long long* slots) {
  Engine* e = static_cast<Engine*>(h);
  auto it = e->seqs.find(id);
  if (it == e->seqs.end()) return -1;
  const Seq& s = it->second;
  for (int t = 0; t < count; ++t) {
    const int pos = first + t;
    const int blk = pos / e->block_size;
    if (blk >= static_cast<int>(s.blocks.size())) return -2;
    slots[t] = static_cast<long long>(s.blocks[blk]) * e->block_size + pos % e->block_size;
  }
  return 0;
}

// Records one generated token for every id; `finished[i]` != 0 retires the sequence (its blocks are
// released). A sequence that reached max_new tokens is retired as well; the return value is the
// number of sequences retired by this call, and finished[i] is set to 2 for length-retired ones.
RLB_API int rlb_engine_commit(void* h, const long long* ids, int n, int* finished) {
  Engine* e = static_cast<Engine*>(h);
  int retired = 0;
  for (int i = 0; i < n; ++i) {
    auto it = e->seqs.find(ids[i]);
    if (it == e->seqs.end()) continue;
    Seq& s = it->second;
    ++s.num_tokens;
    ++s.num_generated;
    bool done = finished[i] != 0;
    if (!done && s.num_generated >= s.max_new) {
      done = true;
      finished[i] = 2;
    }
    if (done) {
      e->release_seq(s);
      s.state = FINISHED;
      e->running.erase(std::remove(e->running.begin(), e->running.end(), s.id), e->running.end());
      e->seqs.erase(it);
      ++retired;
    }
  }
  return retired;
}

// Multi-step decode: sets how many decode steps the next schedule() calls should reserve blocks for (>= 1).
RLB_API void rlb_engine_set_lookahead(void* h, int steps) { static_cast<Engine*>(h)->lookahead = steps < 1 ? 1 : steps; }
// Steps granted by the last schedule() call (the look-ahead, or 1 when blocks were short).
RLB_API int rlb_engine_window(void* h) { return static_cast<Engine*>(h)->window; }

// Records counts[i] generated tokens for every id (the result of a window of decode steps). finished[i] != 0 retires
// the sequence; one that reached its limit is retired too and gets finished[i] = 2. Returns the number retired.
RLB_API int rlb_engine_commit_n(void* h, const long long* ids, int n, const int* counts, int* finished) {
  Engine* e = static_cast<Engine*>(h);
  int retired = 0;
  for (int i = 0; i < n; ++i) {
    auto it = e->seqs.find(ids[i]);
    if (it == e->seqs.end()) continue;
    Seq& s = it->second;
    s.num_tokens += counts[i];
    s.num_generated += counts[i];
    bool done = finished[i] != 0;
    if (!done && s.num_generated >= s.max_new) {
      done = true;
      finished[i] = 2;
    }
    if (done) {
      e->release_seq(s);
      s.state = FINISHED;
      e->running.erase(std::remove(e->running.begin(), e->running.end(), s.id), e->running.end());
      e->seqs.erase(it);
      ++retired;
    }
  }
  return retired;
}

// The first sampled token of a freshly prefilled sequence does not occupy a cache slot yet (its K/V
// is written by the next decode step); this variant counts the token as generated without growing
// the cached length.
RLB_API int rlb_engine_commit_first(void* h, const long long* ids, int n, int* finished) {
  Engine* e = static_cast<Engine*>(h);
  int retired = 0;
  for (int i = 0; i < n; ++i) {
    auto it = e->seqs.find(ids[i]);
    if (it == e->seqs.end()) continue;
    Seq& s = it->second;
    ++s.num_generated;
    bool done = finished[i] != 0;
    if (!done && s.num_generated >= s.max_new) {
      done = true;
      finished[i] = 2;
    }
    if (done) {
      e->release_seq(s);
      s.state = FINISHED;
      e->running.erase(std::remove(e->running.begin(), e->running.end(), s.id), e->running.end());
      e->seqs.erase(it);
      ++retired;
    }
  }
  return retired;
}

RLB_API int rlb_engine_seq_info(void* h, long long id, int* num_tokens, int* num_generated, int* state) {
  Engine* e = static_cast<Engine*>(h);
  auto it = e->seqs.find(id);
  if (it == e->seqs.end()) return -1;
  if (num_tokens) *num_tokens = it->second.num_tokens;
  if (num_generated) *num_generated = it->second.num_generated;
  if (state) *state = it->second.state;
  return 0;
}

// Drops every request and returns all blocks (end of a generation phase / KV cache invalidation).
RLB_API void rlb_engine_reset(void* h) {
  Engine* e = static_cast<Engine*>(h);
  e->seqs.clear();
  e->waiting.clear();
  e->running.clear();
  e->free_list.clear();
  e->cached_free.clear();
  e->cache_table.clear();
  std::fill(e->refcount.begin(), e->refcount.end(), 0);
  std::fill(e->block_cached.begin(), e->block_cached.end(), 0);
  for (int b = e->num_blocks - 1; b >= 0; --b) e->free_list.push_back(b);
}

// Prefix cache. `hashes[i]` identifies the content of the first (i + 1) * block_size prompt tokens of request `id` (the
// caller chains them, so equal hashes mean equal prefixes). Set before the request is scheduled.
RLB_API int rlb_engine_set_hashes(void* h, long long id, const unsigned long long* hashes, int n) {
  Engine* e = static_cast<Engine*>(h);
  auto it = e->seqs.find(id);
  if (it == e->seqs.end() || n < 0) return -1;
  it->second.hashes.assign(hashes, hashes + n);
  return 0;
}
// Tokens of the request's current admission that came out of the prefix cache (a multiple of the block size).
RLB_API int rlb_engine_cached_prefix(void* h, long long id) {
  Engine* e = static_cast<Engine*>(h);
  auto it = e->seqs.find(id);
  return it == e->seqs.end() ? -1 : it->second.cached_prefix;
}
// Registers the full prompt blocks of a request whose prefill has run, so that later requests can take them over.
RLB_API int rlb_engine_register_prefix(void* h, long long id) {
  Engine* e = static_cast<Engine*>(h);
  auto it = e->seqs.find(id);
  if (it == e->seqs.end()) return -1;
  Seq& s = it->second;
  const int n = std::min(static_cast<int>(s.hashes.size()), std::min(static_cast<int>(s.blocks.size()), s.prompt_len / e->block_size));
  for (int b = 0; b < n; ++b) e->register_block(s.blocks[b], s.hashes[b]);
  return n;
}
// hits / queries / evictions of the prefix cache since creation.
RLB_API void rlb_engine_cache_stats(void* h, long long* hits, long long* queries, long long* evictions, long long* cached_blocks) {
  Engine* e = static_cast<Engine*>(h);
  if (hits) *hits = e->cache_hits;
  if (queries) *queries = e->cache_queries;
  if (evictions) *evictions = e->cache_evictions;
  if (cached_blocks) *cached_blocks = static_cast<long long>(e->cache_table.size());
}
