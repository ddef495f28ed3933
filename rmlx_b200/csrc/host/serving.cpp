// Host-side serving core: the KV block manager (free list, per-sequence block tables, reference
// counts with copy-on-write, prefix adoption, speculative rollback), the prefix cache (radix tree
// from whole blocks of token ids to KV block ids with least-recently-used leaf eviction) and the
// continuous-batching scheduler (waiting queue, active set, block-aware admission, one chunk of one
// prompt per step interleaved with everyone else's decode step).
//
// These are the native forms of what the reference implements in Rust:
// BlockManager / PagedKvCache bookkeeping (crates/rmlx-nn/src/paged_kv_cache.rs:36-631),
// PrefixCache (crates/rmlx-nn/src/prefix_cache.rs:27-330) and Scheduler
// (crates/rmlx-nn/src/scheduler.rs:19-352). The Python classes of the same names keep the same
// behaviour and serve as the oracle in the tests; the C ABI below is what they are compared with
// and what the serving engine uses when the host library is present.
//
// None of the three classes locks: a serving engine drives them from one thread (the reference's
// are likewise single-owner `&mut self` types).
//
// Return codes: 0 ok, -1 unknown / already existing sequence, -2 bad argument or state,
// -3 out of blocks. Counts are returned as non-negative ints.
#include <algorithm>
#include <cstdint>
#include <deque>
#include <map>
#include <unordered_map>
#include <vector>

namespace {

constexpr int kOk = 0, kNoSeq = -1, kBad = -2, kOutOfBlocks = -3;

// ------------------------------------------------------------------------------------------------
// Block manager
// ------------------------------------------------------------------------------------------------
class BlockManager {
 public:
  BlockManager(int num_blocks, int block_size, int reserved)
      : block_size_(block_size), reserved_(reserved), ref_(num_blocks, 0) {
    // hand out low block ids first (the free list is a stack with the lowest id on top)
    for (int b = num_blocks - 1; b >= reserved; --b) free_.push_back(b);
  }
  int block_size() const { return block_size_; }
  int num_free() const { return static_cast<int>(free_.size()); }
  bool has(int64_t seq) const { return seqs_.count(seq) != 0; }
  int seq_len(int64_t seq) const {
    auto it = seqs_.find(seq);
    return it == seqs_.end() ? 0 : it->second.len;
  }
  const std::vector<int>* table(int64_t seq) const {
    auto it = seqs_.find(seq);
    return it == seqs_.end() ? nullptr : &it->second.table;
  }
  int blocks_needed(int64_t seq, int new_tokens) const {
    auto it = seqs_.find(seq);
    const int cur = it == seqs_.end() ? 0 : it->second.len;
    const int have = it == seqs_.end() ? 0 : static_cast<int>(it->second.table.size());
    const int need = (cur + new_tokens + block_size_ - 1) / block_size_;
    return std::max(0, need - have);
  }
  int add_sequence(int64_t seq) {
    if (has(seq)) return kNoSeq;
    seqs_[seq] = Seq{};
    return kOk;
  }
  // Makes room for new_tokens more tokens. A shared, partly filled last block is replaced by a
  // fresh one first; the (src, dst) pair is reported so the caller copies the page.
  int reserve(int64_t seq, int new_tokens, int* copy_src, int* copy_dst, int* n_copies) {
    *n_copies = 0;
    if (new_tokens < 0) return kBad;
    if (!has(seq)) seqs_[seq] = Seq{};
    if (blocks_needed(seq, new_tokens) > num_free()) return kOutOfBlocks;
    Seq& s = seqs_[seq];
    if (new_tokens > 0 && !s.table.empty() && s.len % block_size_ != 0) {
      const int last = s.table.back();
      if (ref_[last] > 1) {
        if (blocks_needed(seq, new_tokens) + 1 > num_free()) return kOutOfBlocks;
        const int nb = take();
        *copy_src = last;
        *copy_dst = nb;
        *n_copies = 1;
        drop(last);
        s.table.back() = nb;
      }
    }
    const int need = blocks_needed(seq, new_tokens);
    for (int i = 0; i < need; ++i) s.table.push_back(take());
    return kOk;
  }
  int commit(int64_t seq, int new_tokens) {
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return kNoSeq;
    it->second.len += new_tokens;
    return kOk;
  }
  int fork(int64_t parent, int64_t child) {
    auto it = seqs_.find(parent);
    if (it == seqs_.end() || has(child)) return kNoSeq;
    Seq c = it->second;
    for (int b : c.table) ++ref_[b];
    seqs_[child] = c;
    return kOk;
  }
  int adopt(int64_t seq, const int* blocks, int n, int num_tokens) {
    auto it = seqs_.find(seq);
    if (it != seqs_.end() && (!it->second.table.empty() || it->second.len != 0)) return kBad;
    if (n < 0 || num_tokens < 0 || num_tokens > n * block_size_) return kBad;
    for (int i = 0; i < n; ++i)
      if (blocks[i] < 0 || blocks[i] >= static_cast<int>(ref_.size()) || ref_[blocks[i]] <= 0) return kBad;
    Seq& s = seqs_[seq];
    s.table.assign(blocks, blocks + n);
    s.len = num_tokens;
    for (int i = 0; i < n; ++i) ++ref_[blocks[i]];
    return kOk;
  }
  int retain(int block) {
    if (block < 0 || block >= static_cast<int>(ref_.size()) || ref_[block] <= 0) return kBad;
    ++ref_[block];
    return kOk;
  }
  int release(int block) {
    if (block < 0 || block >= static_cast<int>(ref_.size()) || ref_[block] <= 0) return kBad;
    drop(block);
    return kOk;
  }
  int trim(int64_t seq, int num_tokens) {
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return kNoSeq;
    Seq& s = it->second;
    const int nl = std::max(0, s.len - num_tokens);
    const size_t keep = static_cast<size_t>((nl + block_size_ - 1) / block_size_);
    while (s.table.size() > keep) {
      drop(s.table.back());
      s.table.pop_back();
    }
    s.len = nl;
    return kOk;
  }
  // Sliding-window sequences: release the pages that lie entirely before the last keep_tokens
  // tokens. Their table entries become 0, the reserved page (attention with a window never reads
  // them; positions keep indexing the table by pos / block_size). Returns the number released,
  // or a negative code. Needs a reserved page.
  int drop_front(int64_t seq, int keep_tokens) {
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return kNoSeq;
    if (reserved_ < 1 || keep_tokens < 0) return kBad;
    Seq& s = it->second;
    const int first_needed = std::max(0, s.len - keep_tokens) / block_size_;
    int n = 0;
    for (int i = 0; i < first_needed && i < static_cast<int>(s.table.size()); ++i) {
      if (s.table[i] >= reserved_) { drop(s.table[i]); s.table[i] = 0; ++n; }
    }
    return n;
  }
  int free_sequence(int64_t seq) {
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return kOk;       // freeing an unknown sequence is a no-op
    for (int b : it->second.table) drop(b);
    seqs_.erase(it);
    return kOk;
  }
  int ref_count(int block) const {
    return block < 0 || block >= static_cast<int>(ref_.size()) ? -1 : ref_[block];
  }

 private:
  struct Seq {
    std::vector<int> table;
    int len = 0;
  };
  int take() {
    const int b = free_.back();
    free_.pop_back();
    ref_[b] = 1;
    return b;
  }
  void drop(int b) {
    if (b < reserved_) return;               // a released front page (entry 0) holds no reference
    if (--ref_[b] == 0) free_.push_back(b);
  }
  int block_size_;
  int reserved_;
  std::vector<int> ref_;
  std::vector<int> free_;
  std::unordered_map<int64_t, Seq> seqs_;
};

}  // namespace

namespace {

// ------------------------------------------------------------------------------------------------
// Prefix cache: a radix tree whose edges are whole blocks of token ids
// ------------------------------------------------------------------------------------------------
class PrefixCache {
 public:
  PrefixCache(int block_size, int max_blocks) : bs_(block_size), max_blocks_(max_blocks) {}
  ~PrefixCache() { destroy(&root_); }

  int size() const { return num_blocks_; }
  int64_t hits() const { return hits_; }
  int64_t misses() const { return misses_; }

  // Records blocks[i] as the page of the i-th full block of tokens; appends the block ids that
  // were newly recorded (chunks already present keep the block they had).
  void insert(const int* tokens, int n, const int* blocks, int nb, std::vector<int>* fresh) {
    Node* node = &root_;
    const int64_t now = ++clock_;
    const int chunks = std::min(n / bs_, nb);
    for (int c = 0; c < chunks; ++c) {
      std::vector<int> key(tokens + c * bs_, tokens + (c + 1) * bs_);
      auto it = node->children.find(key);
      Node* nxt;
      if (it == node->children.end()) {
        nxt = new Node();
        nxt->parent = node;
        nxt->block = blocks[c];
        nxt->self = node->children.emplace(key, nxt).first;
        ++num_blocks_;
        fresh->push_back(blocks[c]);
      } else {
        nxt = it->second;
      }
      nxt->last_used = now;
      node = nxt;
    }
    if (max_blocks_ > 0 && num_blocks_ > max_blocks_) evict(num_blocks_ - max_blocks_, &pending_);
  }
  // Longest cached prefix: appends its block ids, returns how many.
  int lookup(const int* tokens, int n, std::vector<int>* blocks) {
    Node* node = &root_;
    const int64_t now = ++clock_;
    int found = 0;
    for (int c = 0; c < n / bs_; ++c) {
      std::vector<int> key(tokens + c * bs_, tokens + (c + 1) * bs_);
      auto it = node->children.find(key);
      if (it == node->children.end()) break;
      node = it->second;
      node->last_used = now;
      blocks->push_back(node->block);
      ++found;
    }
    if (found) ++hits_; else ++misses_;
    return found;
  }
  // Drops up to n least-recently-used leaves; appends their block ids.
  void evict(int n, std::vector<int>* victims) {
    for (int i = 0; i < n; ++i) {
      Node* best = nullptr;
      std::vector<Node*> stack{&root_};
      while (!stack.empty()) {
        Node* nd = stack.back();
        stack.pop_back();
        if (nd != &root_ && nd->children.empty() && (!best || nd->last_used < best->last_used)) best = nd;
        for (auto& kv : nd->children) stack.push_back(kv.second);
      }
      if (!best) return;
      victims->push_back(best->block);
      best->parent->children.erase(best->self);
      delete best;
      --num_blocks_;
    }
  }
  // Hands over up to cap of the blocks that insert() pushed out to stay under max_blocks.
  std::vector<int> take_pending(int cap) {
    const size_t n = std::min(pending_.size(), static_cast<size_t>(std::max(0, cap)));
    std::vector<int> v(pending_.begin(), pending_.begin() + n);
    pending_.erase(pending_.begin(), pending_.begin() + n);
    return v;
  }

 private:
  struct Node {
    std::map<std::vector<int>, Node*> children;
    std::map<std::vector<int>, Node*>::iterator self;
    Node* parent = nullptr;
    int block = -1;
    int64_t last_used = 0;
  };
  static void destroy(Node* nd) {
    for (auto& kv : nd->children) {
      destroy(kv.second);
      delete kv.second;
    }
    nd->children.clear();
  }
  int bs_, max_blocks_;
  Node root_;
  int num_blocks_ = 0;
  int64_t clock_ = 0, hits_ = 0, misses_ = 0;
  std::vector<int> pending_;
};

}  // namespace

namespace {

// ------------------------------------------------------------------------------------------------
// Continuous-batching scheduler
// ------------------------------------------------------------------------------------------------
class Scheduler {
 public:
  Scheduler(int max_batch, int64_t eos, int max_prefill_chunk, bool manage_blocks)
      : max_batch_(max_batch), eos_(eos), chunk_(max_prefill_chunk), manage_(manage_blocks) {}

  int add_request(int64_t seq, const int* prompt, int n, int max_out) {
    if (n <= 0) return kBad;
    waiting_.push_back(Request{seq, std::vector<int>(prompt, prompt + n), max_out});
    return kOk;
  }
  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_active() const { return static_cast<int>(order_.size()); }

  // A token came out for seq in the previous step: 1 if that ends the sequence (it is dropped from
  // the active set; its blocks are the caller's to free), else 0.
  int finish(int64_t seq, int64_t token) {
    auto it = active_.find(seq);
    if (it == active_.end()) return 0;
    if (token != eos_ && it->second.generated < it->second.max_out) return 0;
    active_.erase(it);
    order_.erase(std::find(order_.begin(), order_.end(), seq));
    return 1;
  }
  // Admits the oldest waiting request if a batch slot and the blocks of its first chunk are
  // available. Returns its id (the caller registers it with the KV cache and reports how many
  // prompt tokens it found cached) or -1.
  int64_t admit_next(const BlockManager& bm) {
    if (waiting_.empty() || num_active() >= max_batch_) return -1;
    Request& r = waiting_.front();
    const int first = std::min<int>(static_cast<int>(r.prompt.size()), chunk_);
    if ((first + bm.block_size() - 1) / bm.block_size() > bm.num_free()) return -1;
    const int64_t seq = r.seq;
    Active a;
    a.prompt.swap(r.prompt);
    a.max_out = r.max_out;
    waiting_.pop_front();
    active_.emplace(seq, std::move(a));
    order_.push_back(seq);
    return seq;
  }
  int set_cached(int64_t seq, int cached) {
    auto it = active_.find(seq);
    if (it == active_.end()) return kNoSeq;
    // the last prompt token always runs: its logits give the first generated token
    const int cap = static_cast<int>(it->second.prompt.size()) - 1;
    it->second.progress = std::max(0, std::min(cached, cap));
    return kOk;
  }
  // One chunk of the oldest unfinished prompt; every other fully prefilled sequence decodes.
  // prefill[3] = {seq, lo, hi} (seq -1: none). Returns the number of decode ids written.
  int plan(BlockManager* bm, int64_t* prefill, int64_t* decode, int cap) {
    prefill[0] = -1; prefill[1] = prefill[2] = 0;
    int64_t chosen = -1;
    for (int64_t seq : order_) {
      Active& a = active_[seq];
      if (a.progress >= static_cast<int>(a.prompt.size())) continue;
      const int lo = a.progress;
      const int hi = std::min<int>(static_cast<int>(a.prompt.size()), lo + chunk_);
      bool room = bm->blocks_needed(seq, hi - lo) <= bm->num_free();
      if (room && manage_) {
        int s, d, n;
        room = bm->reserve(seq, hi - lo, &s, &d, &n) == kOk;   // may still fail on a copy-on-write block
        if (room) bm->commit(seq, hi - lo);
      }
      if (room) {
        a.progress = hi;
        prefill[0] = seq; prefill[1] = lo; prefill[2] = hi;
        chosen = seq;
      }
      break;                      // only the oldest unfinished prompt is considered
    }
    int n_dec = 0;
    for (int64_t seq : order_) {
      Active& a = active_[seq];
      if (a.progress < static_cast<int>(a.prompt.size()) || seq == chosen) continue;
      if (bm->blocks_needed(seq, 1) > bm->num_free()) continue;   // stalls until blocks free up
      if (manage_) {
        int s, d, n;
        if (bm->reserve(seq, 1, &s, &d, &n) != kOk) continue;
      }
      if (n_dec < cap) decode[n_dec++] = seq;
    }
    return n_dec;
  }
  int update(BlockManager* bm, int64_t seq) {
    auto it = active_.find(seq);
    if (it == active_.end()) return kNoSeq;
    ++it->second.generated;
    if (manage_) bm->commit(seq, 1);
    return kOk;
  }
  int prompt(int64_t seq, int lo, int hi, int* out) const {
    auto it = active_.find(seq);
    if (it == active_.end()) return kNoSeq;
    const auto& p = it->second.prompt;
    lo = std::max(0, lo);
    hi = std::min<int>(hi, static_cast<int>(p.size()));
    for (int i = lo; i < hi; ++i) out[i - lo] = p[i];
    return std::max(0, hi - lo);
  }
  int info(int64_t seq, int* out) const {
    auto it = active_.find(seq);
    if (it == active_.end()) return kNoSeq;
    out[0] = static_cast<int>(it->second.prompt.size());
    out[1] = it->second.progress;
    out[2] = it->second.generated;
    return kOk;
  }

 private:
  struct Request {
    int64_t seq;
    std::vector<int> prompt;
    int max_out;
  };
  struct Active {
    std::vector<int> prompt;
    int max_out = 0, generated = 0, progress = 0;
  };
  int max_batch_;
  int64_t eos_;
  int chunk_;
  bool manage_;
  std::deque<Request> waiting_;
  std::unordered_map<int64_t, Active> active_;
  std::vector<int64_t> order_;     // admission order (the oldest unfinished prompt goes first)
};

int copy_out(const std::vector<int>& v, int* out, int cap) {
  const int n = std::min<int>(static_cast<int>(v.size()), cap);
  for (int i = 0; i < n; ++i) out[i] = v[i];
  return n;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------
#define BM(h) static_cast<BlockManager*>(h)
#define PC(h) static_cast<PrefixCache*>(h)
#define SC(h) static_cast<Scheduler*>(h)

extern "C" {

void* rmlx_bm_create(int num_blocks, int block_size, int reserved) {
  if (num_blocks < 1 || block_size < 1 || reserved < 0 || reserved > num_blocks) return nullptr;
  return new BlockManager(num_blocks, block_size, reserved);
}
void rmlx_bm_destroy(void* h) { delete BM(h); }
int rmlx_bm_num_free(void* h) { return BM(h)->num_free(); }
int rmlx_bm_has(void* h, int64_t seq) { return BM(h)->has(seq) ? 1 : 0; }
int rmlx_bm_seq_len(void* h, int64_t seq) { return BM(h)->seq_len(seq); }
int rmlx_bm_blocks_needed(void* h, int64_t seq, int n) { return BM(h)->blocks_needed(seq, n); }
int rmlx_bm_add_sequence(void* h, int64_t seq) { return BM(h)->add_sequence(seq); }
int rmlx_bm_reserve(void* h, int64_t seq, int n, int* src, int* dst, int* n_copies) {
  return BM(h)->reserve(seq, n, src, dst, n_copies);
}
int rmlx_bm_commit(void* h, int64_t seq, int n) { return BM(h)->commit(seq, n); }
int rmlx_bm_fork(void* h, int64_t parent, int64_t child) { return BM(h)->fork(parent, child); }
int rmlx_bm_adopt(void* h, int64_t seq, const int* blocks, int n, int tokens) {
  return BM(h)->adopt(seq, blocks, n, tokens);
}
int rmlx_bm_retain(void* h, int block) { return BM(h)->retain(block); }
int rmlx_bm_release(void* h, int block) { return BM(h)->release(block); }
int rmlx_bm_trim(void* h, int64_t seq, int n) { return BM(h)->trim(seq, n); }
int rmlx_bm_drop_front(void* h, int64_t seq, int keep) { return BM(h)->drop_front(seq, keep); }
int rmlx_bm_free_sequence(void* h, int64_t seq) { return BM(h)->free_sequence(seq); }
int rmlx_bm_ref_count(void* h, int block) { return BM(h)->ref_count(block); }
// Block table of seq into out (at most cap entries); returns its full length, -1 if unknown.
int rmlx_bm_table(void* h, int64_t seq, int* out, int cap) {
  const std::vector<int>* t = BM(h)->table(seq);
  if (!t) return -1;
  copy_out(*t, out, cap);
  return static_cast<int>(t->size());
}

void* rmlx_pc_create(int block_size, int max_blocks) {
  return block_size < 1 ? nullptr : new PrefixCache(block_size, max_blocks);
}
void rmlx_pc_destroy(void* h) { delete PC(h); }
int rmlx_pc_len(void* h) { return PC(h)->size(); }
int64_t rmlx_pc_hits(void* h) { return PC(h)->hits(); }
int64_t rmlx_pc_misses(void* h) { return PC(h)->misses(); }
int rmlx_pc_insert(void* h, const int* tokens, int n, const int* blocks, int nb, int* fresh, int cap) {
  std::vector<int> v;
  PC(h)->insert(tokens, n, blocks, nb, &v);
  return copy_out(v, fresh, cap);
}
int rmlx_pc_lookup(void* h, const int* tokens, int n, int* blocks, int cap) {
  std::vector<int> v;
  PC(h)->lookup(tokens, n, &v);
  return copy_out(v, blocks, cap);
}
int rmlx_pc_evict(void* h, int n, int* victims, int cap) {
  std::vector<int> v;
  PC(h)->evict(std::min(n, cap), &v);
  return copy_out(v, victims, cap);
}
int rmlx_pc_take_evicted(void* h, int* victims, int cap) {
  return copy_out(PC(h)->take_pending(cap), victims, cap);
}

void* rmlx_sched_create(int max_batch, int64_t eos, int max_prefill_chunk, int manage_blocks) {
  if (max_batch < 1 || max_prefill_chunk < 1) return nullptr;
  return new Scheduler(max_batch, eos, max_prefill_chunk, manage_blocks != 0);
}
void rmlx_sched_destroy(void* h) { delete SC(h); }
int rmlx_sched_add_request(void* h, int64_t seq, const int* prompt, int n, int max_out) {
  return SC(h)->add_request(seq, prompt, n, max_out);
}
int rmlx_sched_num_waiting(void* h) { return SC(h)->num_waiting(); }
int rmlx_sched_num_active(void* h) { return SC(h)->num_active(); }
int rmlx_sched_finish(void* h, int64_t seq, int64_t token) { return SC(h)->finish(seq, token); }
int64_t rmlx_sched_admit_next(void* h, void* bm) { return SC(h)->admit_next(*BM(bm)); }
int rmlx_sched_set_cached(void* h, int64_t seq, int cached) { return SC(h)->set_cached(seq, cached); }
int rmlx_sched_plan(void* h, void* bm, int64_t* prefill, int64_t* decode, int cap) {
  return SC(h)->plan(BM(bm), prefill, decode, cap);
}
int rmlx_sched_update(void* h, void* bm, int64_t seq) { return SC(h)->update(BM(bm), seq); }
// Bulk forms for the binding: one call per step instead of one per sequence.
// finish_many: tokens of the previous step for n sequences; writes the ids that ended, returns how many.
int rmlx_sched_finish_many(void* h, const int64_t* seqs, const int64_t* tokens, int n, int64_t* ended) {
  int k = 0;
  for (int i = 0; i < n; ++i)
    if (SC(h)->finish(seqs[i], tokens[i])) ended[k++] = seqs[i];
  return k;
}
// describe: for n sequence ids writes 4 ints each (prompt length, prefill progress, current length,
// number of blocks) into meta and the block tables back to back into tables (at most cap entries).
// Returns the number of table entries written, or -1 if they did not fit; tables may be null.
int rmlx_sched_describe(void* h, void* bm, const int64_t* seqs, int n, int* meta, int* tables, int cap) {
  int used = 0;
  for (int i = 0; i < n; ++i) {
    int info[3] = {0, 0, 0};
    SC(h)->info(seqs[i], info);
    const std::vector<int>* t = BM(bm)->table(seqs[i]);
    const int nt = t ? static_cast<int>(t->size()) : 0;
    meta[4 * i] = info[0];
    meta[4 * i + 1] = info[1];
    meta[4 * i + 2] = BM(bm)->seq_len(seqs[i]);
    meta[4 * i + 3] = nt;
    if (!tables) continue;                       // the caller wants the counters only
    if (used + nt > cap) return -1;
    for (int j = 0; j < nt; ++j) tables[used + j] = (*t)[j];
    used += nt;
  }
  return used;
}
int rmlx_sched_prompt(void* h, int64_t seq, int lo, int hi, int* out) {
  return SC(h)->prompt(seq, lo, hi, out);
}
int rmlx_sched_info(void* h, int64_t seq, int* out) { return SC(h)->info(seq, out); }

}  // extern "C"
