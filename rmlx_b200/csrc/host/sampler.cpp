// Host-side token sampler and speculative-decoding verification.
//
// Order of operations as in the reference's Sampler (crates/rmlx-nn/src/sampler.rs:21-141):
// repetition penalty -> temperature (0 = greedy) -> top-k (0 = off) -> top-p (1 = off) -> softmax
// -> multinomial; greedy_verify / rejection_sample are the two acceptance rules of
// crates/rmlx-nn/src/sampler.rs:156-370. Random numbers come from a 64-bit SplitMix-seeded
// xoshiro256** generator owned by the sampler, so a seed reproduces a run whatever else the
// process does with its other generators.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <functional>
#include <numeric>
#include <thread>
#include <utility>
#include <vector>

namespace {

struct Rng {
  uint64_t s[4];
  static uint64_t splitmix(uint64_t& x) {
    uint64_t z = (x += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  explicit Rng(uint64_t seed) { for (auto& v : s) v = splitmix(seed); }
  static uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
  uint64_t next() {
    const uint64_t r = rotl(s[1] * 5, 7) * 9, t = s[1] << 17;
    s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]; s[2] ^= t; s[3] = rotl(s[3], 45);
    return r;
  }
  double uniform() { return double(next() >> 11) * (1.0 / 9007199254740992.0); }   // [0, 1)
};

struct Scratch {
  std::vector<float> work;
  std::vector<int> order;
  std::vector<std::pair<float, int>> pairs;
};

struct Sampler {
  float temperature, top_p, penalty;
  int top_k;
  Rng rng;
  Scratch own;                       // scratch of the calling thread; worker threads bring their own
  Sampler(float t, int k, float p, float pen, uint64_t seed)
      : temperature(t), top_p(p), penalty(pen), top_k(k), rng(seed) {}

  // logits after the repetition penalty, in `sc.work`
  void penalised(const float* logits, int vocab, const int* hist, int nh, Scratch& sc) const {
    std::vector<float>& work = sc.work;
    work.assign(logits, logits + vocab);
    if (penalty == 1.0f) return;
    std::vector<int> seen(hist, hist + nh);
    std::sort(seen.begin(), seen.end());
    seen.erase(std::unique(seen.begin(), seen.end()), seen.end());
    for (int t : seen) {
      if (t < 0 || t >= vocab) continue;
      work[t] = work[t] > 0.f ? work[t] / penalty : work[t] * penalty;
    }
  }

  static int argmax(const float* v, int n) {
    int best = 0;
    for (int i = 1; i < n; ++i) if (v[i] > v[best]) best = i;
    return best;
  }

  // the final sampling distribution
  void probabilities(const float* logits, int vocab, const int* hist, int nh, float* out, Scratch& sc) const {
    penalised(logits, vocab, hist, nh, sc);
    std::vector<float>& work = sc.work;
    std::vector<int>& order = sc.order;
    if (temperature == 0.f) {
      std::fill(out, out + vocab, 0.f);
      out[argmax(work.data(), vocab)] = 1.f;
      return;
    }
    const float inv_t = 1.f / temperature;
    for (auto& v : work) v *= inv_t;
    if (top_k > 0 && top_k < vocab) {
      std::vector<float> tmp(work);
      std::nth_element(tmp.begin(), tmp.begin() + (top_k - 1), tmp.end(), std::greater<float>());
      const float kth = tmp[top_k - 1];
      for (auto& v : work) if (v < kth) v = -std::numeric_limits<float>::infinity();
    }
    const float mx = *std::max_element(work.begin(), work.end());
    double sum = 0.0;
    for (int i = 0; i < vocab; ++i) { out[i] = std::exp(work[i] - mx); sum += out[i]; }
    const float inv = float(1.0 / sum);
    for (int i = 0; i < vocab; ++i) out[i] *= inv;
    if (top_p < 1.f) {
      // Nucleus: the most likely tokens whose mass BEFORE them is below p. Only the head of the
      // order is needed, so candidates (non-zero entries) are partially sorted, 1024 at first and
      // four times as many while the head's mass stays below p. Ties break by token id.
      order.clear();
      for (int i = 0; i < vocab; ++i) if (out[i] > 0.f) order.push_back(i);
      const auto before = [&](int a, int b) { return out[a] > out[b] || (out[a] == out[b] && a < b); };
      const size_t n = order.size();
      size_t m = std::min<size_t>(n, 1024), cut = n;
      double kept = 0.0;
      for (int pass = 0; pass < 2; ++pass) {
        if (pass == 0) {
          std::partial_sort(order.begin(), order.begin() + m, order.end(), before);
        } else {
          // a flat distribution: the head was not enough, sort everything once (value-index pairs
          // sort several times faster than indices compared through the probability array)
          sc.pairs.resize(n);
          for (size_t r = 0; r < n; ++r) sc.pairs[r] = {-out[order[r]], order[r]};
          std::sort(sc.pairs.begin(), sc.pairs.end());
          for (size_t r = 0; r < n; ++r) order[r] = sc.pairs[r].second;
          m = n;
        }
        double cum = 0.0;
        kept = 0.0;
        cut = m;
        bool closed = false;
        for (size_t r = 0; r < m; ++r) {
          if (!(cum < double(top_p))) { cut = r; closed = true; break; }
          cum += out[order[r]];
          kept += out[order[r]];
        }
        if (closed || m == n) break;
      }
      for (size_t r = cut; r < n; ++r) out[order[r]] = 0.f;
      const float rn = float(1.0 / kept);
      for (size_t r = 0; r < cut; ++r) out[order[r]] *= rn;
    }
  }

  int multinomial(const float* p, int n) {
    double total = 0.0;
    for (int i = 0; i < n; ++i) total += p[i];
    const double u = rng.uniform() * total;
    double cum = 0.0;
    int last = 0;
    for (int i = 0; i < n; ++i) {
      if (p[i] <= 0.f) continue;
      cum += p[i];
      last = i;
      if (u < cum) return i;
    }
    return last;                                             // rounding at the upper end
  }
};

}  // namespace

extern "C" {

void* rmlx_sampler_create(float temperature, int top_k, float top_p, float penalty, uint64_t seed) {
  if (temperature < 0.f || top_k < 0 || !(top_p > 0.f && top_p <= 1.f) || penalty <= 0.f) return nullptr;
  return new Sampler(temperature, top_k, top_p, penalty, seed);
}

void rmlx_sampler_destroy(void* h) { delete static_cast<Sampler*>(h); }

// out[vocab] = the distribution one token would be drawn from.
int rmlx_sampler_probabilities(void* h, const float* logits, int vocab, const int* hist, int nh, float* out) {
  if (!h || vocab < 1) return -1;
  Sampler* s = static_cast<Sampler*>(h);
  s->probabilities(logits, vocab, hist, nh, out, s->own);
  return 0;
}

// One token per row of logits [rows, vocab]; hist_off[rows + 1] delimits each row's history in
// hist (both may be null: no history). Returns 0, tokens in out[rows].
int rmlx_sampler_sample(void* h, const float* logits, int rows, int vocab, const int* hist,
                        const int* hist_off, int* out) {
  if (!h || vocab < 1 || rows < 0) return -1;
  Sampler* s = static_cast<Sampler*>(h);
  const auto hist_of = [&](int r, const int*& hr, int& nh) {
    hr = hist && hist_off ? hist + hist_off[r] : nullptr;
    nh = hist && hist_off ? hist_off[r + 1] - hist_off[r] : 0;
  };
  if (s->temperature == 0.f) {
    for (int r = 0; r < rows; ++r) {
      const int* hr; int nh;
      hist_of(r, hr, nh);
      s->penalised(logits + size_t(r) * vocab, vocab, hr, nh, s->own);
      out[r] = Sampler::argmax(s->own.work.data(), vocab);
    }
    return 0;
  }
  // The distributions of the rows are independent: they are shaped on up to eight threads; the
  // draws then come from the one generator in row order, so a seed gives the same tokens whatever
  // the thread count.
  std::vector<float> probs(size_t(rows) * vocab);
  const int threads = int(std::min<size_t>({size_t(rows), size_t(8), size_t(std::max(1u, std::thread::hardware_concurrency()))}));
  const auto shape_rows = [&](int t, Scratch& sc) {
    for (int r = t; r < rows; r += threads) {
      const int* hr; int nh;
      hist_of(r, hr, nh);
      s->probabilities(logits + size_t(r) * vocab, vocab, hr, nh, probs.data() + size_t(r) * vocab, sc);
    }
  };
  if (threads <= 1 || size_t(rows) * vocab < (1u << 16)) {
    for (int t = 0; t < threads; ++t) shape_rows(t, s->own);
  } else {
    std::vector<std::thread> pool;
    std::vector<Scratch> scratch(threads);
    for (int t = 1; t < threads; ++t) pool.emplace_back(shape_rows, t, std::ref(scratch[t]));
    shape_rows(0, s->own);
    for (auto& th : pool) th.join();
  }
  for (int r = 0; r < rows; ++r) out[r] = s->multinomial(probs.data() + size_t(r) * vocab, vocab);
  return 0;
}

double rmlx_sampler_uniform(void* h) { return static_cast<Sampler*>(h)->rng.uniform(); }

int rmlx_sampler_multinomial(void* h, const float* p, int n) {
  if (!h || n < 1) return -1;
  return static_cast<Sampler*>(h)->multinomial(p, n);
}

// Greedy verification: draft[i] is accepted while it equals the arg-max of target_logits[i]. Returns
// the number accepted; *next = the correcting token at the first mismatch, else the bonus token
// from row n when rows > n, else -1.
int rmlx_spec_greedy_verify(const int* draft, int n, const float* target_logits, int rows, int vocab, int* next) {
  *next = -1;
  if (n < 0 || rows < 0 || vocab < 1) return -1;
  for (int i = 0; i < n && i < rows; ++i) {
    const int best = Sampler::argmax(target_logits + size_t(i) * vocab, vocab);
    if (best != draft[i]) { *next = best; return i; }
  }
  if (rows > n) *next = Sampler::argmax(target_logits + size_t(n) * vocab, vocab);
  return n < rows ? n : rows;
}

// Rejection sampling: accept draft[i] with probability min(1, p_target / p_draft); at the first
// rejection draw the correction from normalise(max(0, p_target - p_draft)) (from p_target when that
// is empty). Returns the number accepted; *next as above (bonus drawn from target row n).
int rmlx_spec_rejection_sample(void* h, const int* draft, int n, const float* draft_probs,
                               const float* target_probs, int rows, int vocab, int* next) {
  Sampler* s = static_cast<Sampler*>(h);
  *next = -1;
  if (!h || n < 0 || rows < n || vocab < 1) return -1;      // a target row per draft token at least
  std::vector<float> resid(vocab);
  for (int i = 0; i < n; ++i) {
    const float* pt = target_probs + size_t(i) * vocab;
    const float* pd = draft_probs + size_t(i) * vocab;
    const int t = draft[i];
    if (t < 0 || t >= vocab) return -1;
    const double u = s->rng.uniform();
    if (pd[t] <= 0.f || u < std::min(1.0, double(pt[t]) / double(pd[t]))) continue;
    double total = 0.0;
    for (int v = 0; v < vocab; ++v) { resid[v] = std::max(0.f, pt[v] - pd[v]); total += resid[v]; }
    *next = total > 0.0 ? s->multinomial(resid.data(), vocab) : s->multinomial(pt, vocab);
    return i;
  }
  if (rows > n) *next = s->multinomial(target_probs + size_t(n) * vocab, vocab);
  return n;
}

}  // extern "C"
