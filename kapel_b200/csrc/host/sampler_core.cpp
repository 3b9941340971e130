// Choosing the next token on the host, in 64-bit: Kapel's order and arithmetic
// (crates/kapel-infer/src/sampling.rs:157-260,291-310). Frequency and presence penalties, the
// repetition penalty, greedy if the temperature is 0, else temperature, top_k, top_p, min_p, then a
// draw: the first index whose running total of probabilities exceeds a uniform number from the
// request's own xoshiro256** generator. Sums run in index order (in sorted order for top_p), as there.
//
// The filters never sort the whole vocabulary. After each filter only the tokens still possible are
// kept, as a list in index order, and every later pass (softmax, filter, draw) walks that list: a
// token at -inf adds exactly 0 to a sum, so the sums are the ones a walk over the whole vocabulary
// gives. top_k needs the k-th largest value only (a heap of k values over one pass); top_p sorts the
// most likely tokens in growing batches (chosen by a falling threshold) until their total reaches p,
// which gives the same kept set and the same sums as a full sort. Logits with a NaN among them take
// a plain path over the whole vocabulary. Several requests are chosen for at once on a few threads;
// each touches only its own row, sequence and generator.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace {

constexpr double NEG_INF = -std::numeric_limits<double>::infinity();

inline uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

// xoshiro256**: the next 64 bits; [0, 1) from the top 53 of them.
uint64_t next_u64(uint64_t* s) {
    const uint64_t result = rotl(s[1] * 5, 7) * 9;
    const uint64_t t = s[1] << 17;
    s[2] ^= s[0];
    s[3] ^= s[1];
    s[1] ^= s[2];
    s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl(s[3], 45);
    return result;
}
double next_uniform(uint64_t* s) { return (double)(next_u64(s) >> 11) / 9007199254740992.0; }

// The first largest; a NaN never, unless all are.
int argmax_first(const double* v, int n) {
    int best = -1;
    for (int i = 0; i < n; ++i)
        if (!std::isnan(v[i]) && (best < 0 || v[i] > v[best])) best = i;
    return best < 0 ? 0 : best;
}

// Probabilities of `l` into `p`; all zero when every logit is -inf or one is a NaN.
void softmax(const double* l, int n, double* p) {
    double m = NEG_INF;
    bool nan = false;
    for (int i = 0; i < n; ++i) {
        if (std::isnan(l[i])) nan = true;
        else if (l[i] > m) m = l[i];
    }
    if (nan || m == NEG_INF) {
        std::fill(p, p + n, 0.0);
        return;
    }
    double total = 0.0;
    for (int i = 0; i < n; ++i) {
        const double e = l[i] == NEG_INF ? 0.0 : std::exp(l[i] - m);
        p[i] = e;
        total += e;
    }
    for (int i = 0; i < n; ++i) p[i] /= total;
}

struct Settings {
    double temperature, top_p, min_p, repetition_penalty, frequency_penalty, presence_penalty;
    int top_k;             // <= 0: none
};

// Penalties, then greedy or the temperature: the certain token, or -1 to go on with the filters.
int penalties_and_temperature(double* l, int n, const Settings& s, const int* seq, int seq_len, int generated_from) {
    if (s.frequency_penalty != 0.0 || s.presence_penalty != 0.0) {
        std::vector<int> toks;
        for (int i = std::min(std::max(generated_from, 0), seq_len); i < seq_len; ++i)
            if (seq[i] >= 0 && seq[i] < n) toks.push_back(seq[i]);
        std::sort(toks.begin(), toks.end());
        for (size_t i = 0; i < toks.size();) {
            size_t j = i;
            while (j < toks.size() && toks[j] == toks[i]) ++j;
            l[toks[i]] -= (double)(j - i) * s.frequency_penalty + s.presence_penalty;
            i = j;
        }
    }
    if (s.repetition_penalty != 1.0) {
        std::vector<int> toks;
        for (int i = 0; i < seq_len; ++i)
            if (seq[i] >= 0 && seq[i] < n) toks.push_back(seq[i]);
        std::sort(toks.begin(), toks.end());
        toks.erase(std::unique(toks.begin(), toks.end()), toks.end());
        for (int t : toks) l[t] = l[t] < 0.0 ? l[t] * s.repetition_penalty : l[t] / s.repetition_penalty;
    }
    if (s.temperature <= 0.0) return argmax_first(l, n);
    for (int i = 0; i < n; ++i) l[i] /= s.temperature;

    return -1;
}

// The filters over the whole vocabulary, value by value: the path for logits with a NaN among them.
// The certain token, or -1 with the probabilities in `p`.
int filters_plain(double* l, int n, const Settings& s, double* p, std::vector<int>& idx, std::vector<double>& tmp) {
    if (s.top_k > 0 && s.top_k < n) {
        // The k-th value of the logits in descending order with NaNs first: a NaN there cuts nothing.
        tmp.clear();
        int nans = 0;
        for (int i = 0; i < n; ++i) {
            if (std::isnan(l[i])) ++nans;
            else tmp.push_back(l[i]);
        }
        if (s.top_k - 1 >= nans) {
            const size_t j = (size_t)(s.top_k - 1 - nans);
            std::nth_element(tmp.begin(), tmp.begin() + (std::ptrdiff_t)j, tmp.end(), std::greater<double>());
            const double kth = tmp[j];
            for (int i = 0; i < n; ++i)
                if (l[i] < kth) l[i] = NEG_INF;
        }
    }
    if (s.top_p < 1.0) {
        softmax(l, n, p);
        // By probability, then by index; a NaN probability last. Kept while the tokens before it
        // hold less than top_p: at least the most likely one.
        auto key = [&](int i) { return std::isnan(p[i]) ? -1.0 : p[i]; };
        auto before_than = [&](int a, int b) {
            const double ka = key(a), kb = key(b);
            return ka > kb || (ka == kb && a < b);
        };
        idx.resize((size_t)n);
        for (int i = 0; i < n; ++i) idx[(size_t)i] = i;
        int sorted = 0, cut = -1;
        int m = std::min(n, 256);
        for (;;) {
            if (m < n) std::nth_element(idx.begin() + sorted, idx.begin() + m, idx.end(), before_than);
            std::sort(idx.begin() + sorted, idx.begin() + m, before_than);
            sorted = m;
            double before = 0.0;
            for (int j = 0; j < m; ++j) {
                if (before >= s.top_p) { cut = j; break; }
                before += p[idx[(size_t)j]];
            }
            if (cut >= 0 || m == n) break;
            m = (int)std::min<long long>(n, 4ll * m);
        }
        if (cut >= 0)
            for (int j = cut; j < n; ++j) l[idx[(size_t)j]] = NEG_INF;
    }
    if (s.min_p > 0.0) {
        softmax(l, n, p);
        double top = 0.0;
        bool nan = false;
        for (int i = 0; i < n; ++i) {
            if (std::isnan(p[i])) nan = true;
            else if (p[i] > top) top = p[i];
        }
        if (!nan) {
            const double floor = s.min_p * top;
            for (int i = 0; i < n; ++i)
                if (p[i] < floor) l[i] = NEG_INF;
        }
    }
    softmax(l, n, p);
    bool any = false;
    for (int i = 0; i < n && !any; ++i) any = p[i] > 0.0;
    if (!any) return argmax_first(l, n);       // nothing left (every logit -inf or a NaN): the first largest
    return -1;
}


// What is still possible: tokens in index order with their logits and, after `softmax`, their
// probabilities. No NaN among the logits.
struct Alive {
    std::vector<int> idx;
    std::vector<double> l, p, heap;
    std::vector<char> keep_it, taken;
    std::vector<int> order;

    void keep(const std::vector<char>& keep_it) {
        size_t w = 0;
        for (size_t i = 0; i < idx.size(); ++i)
            if (keep_it[i]) { idx[w] = idx[i]; l[w] = l[i]; ++w; }
        idx.resize(w); l.resize(w);
    }
    void softmax() {
        p.assign(idx.size(), 0.0);
        double m = NEG_INF;
        for (double v : l) m = v > m ? v : m;
        if (m == NEG_INF) return;
        double total = 0.0;
        for (size_t i = 0; i < l.size(); ++i) { p[i] = std::exp(l[i] - m); total += p[i]; }
        for (double& v : p) v /= total;
    }
};

// The same filters over the list of tokens still possible. The certain token, or -1 with the list
// (and its probabilities) in `a`.
int filters_alive(const double* l, int n, const Settings& s, Alive& a) {
    a.idx.clear(); a.l.clear();
    std::vector<char>& keep_it = a.keep_it;
    int finite = 0;
    for (int i = 0; i < n; ++i) finite += l[i] != NEG_INF ? 1 : 0;
    double kth = NEG_INF;                                    // what is below this is cut by top_k
    if (s.top_k > 0 && s.top_k < n && finite >= s.top_k) {
        // the k-th largest of the logits: the smallest of a heap of the k largest seen so far
        const size_t k = (size_t)s.top_k;
        std::vector<double>& heap = a.heap;
        heap.clear();
        int i = 0;
        for (; i < n && heap.size() < k; ++i)
            if (l[i] != NEG_INF) heap.push_back(l[i]);
        std::make_heap(heap.begin(), heap.end(), std::greater<double>());
        for (; i < n; ++i)
            if (l[i] > heap.front()) {
                std::pop_heap(heap.begin(), heap.end(), std::greater<double>());
                heap.back() = l[i];
                std::push_heap(heap.begin(), heap.end(), std::greater<double>());
            }
        kth = heap.front();
    }
    const size_t room = kth == NEG_INF ? (size_t)finite : 2 * (size_t)s.top_k;
    a.idx.reserve(room); a.l.reserve(room);
    for (int i = 0; i < n; ++i)
        if (l[i] != NEG_INF && !(l[i] < kth)) { a.idx.push_back(i); a.l.push_back(l[i]); }
    if (s.top_p < 1.0) {
        a.softmax();
        const size_t m = a.idx.size();
        // positions into the list, the most likely first (then by index, which is by position); taken in
        // batches of everything at or above a falling threshold until the running total reaches top_p
        std::vector<int>& order = a.order;
        std::vector<char>& taken = a.taken;
        order.clear();
        taken.assign(m, 0);
        auto before_than = [&](int x, int y) { return a.p[(size_t)x] > a.p[(size_t)y] || (a.p[(size_t)x] == a.p[(size_t)y] && x < y); };
        double top = 0.0;
        for (double v : a.p) top = v > top ? v : top;
        double threshold = m <= 4096 ? 0.0 : top / 64.0;
        long long cut = -1;
        for (;;) {
            const size_t had = order.size();
            for (size_t i = 0; i < m; ++i)
                if (!taken[i] && a.p[i] >= threshold) { taken[i] = 1; order.push_back((int)i); }
            std::sort(order.begin() + (std::ptrdiff_t)had, order.end(), before_than);
            double before = 0.0;
            for (size_t j = 0; j < order.size(); ++j) {
                if (before >= s.top_p) { cut = (long long)j; break; }
                before += a.p[(size_t)order[j]];
            }
            if (cut >= 0 || order.size() == m) break;
            threshold = threshold > 1e-300 ? threshold / 64.0 : 0.0;
        }
        if (cut >= 0) {
            keep_it.assign(m, 0);
            for (long long j = 0; j < cut; ++j) keep_it[(size_t)order[(size_t)j]] = 1;
            a.keep(keep_it);
        }
    }
    if (s.min_p > 0.0) {
        a.softmax();
        double top = 0.0;
        for (double v : a.p) top = v > top ? v : top;
        const double floor = s.min_p * top;
        keep_it.assign(a.idx.size(), 1);
        for (size_t i = 0; i < a.p.size(); ++i) keep_it[i] = a.p[i] < floor ? 0 : 1;
        a.keep(keep_it);
    }
    a.softmax();
    for (double v : a.p)
        if (v > 0.0) return -1;
    // Nothing left: the first largest of the logits as the filters left them. What was cut is at -inf,
    // so that is the first of the list's largest, or token 0 when the list is empty.
    int best = -1;
    for (size_t i = 0; i < a.idx.size(); ++i)
        if (best < 0 || a.l[i] > a.l[(size_t)best]) best = (int)i;
    if (best >= 0 && a.l[(size_t)best] == NEG_INF) best = -1;
    return best < 0 ? 0 : a.idx[(size_t)best];
}

int draw(const double* p, int n, double u) {
    double total = 0.0;
    int last = 0;
    for (int i = 0; i < n; ++i)
        if (p[i] > 0.0) {
            total += p[i];
            last = i;
            if (u < total) return i;
        }
    return last;                               // rounding left u above the total: the last possible token
}

void widen(const void* logits, int dtype, int n, double* l) {
    if (dtype == 0) {
        const float* f = static_cast<const float*>(logits);
        for (int i = 0; i < n; ++i) l[i] = (double)f[i];
    } else {
        const double* d = static_cast<const double*>(logits);
        std::copy(d, d + n, l);
    }
}

Settings settings_of(const double* f, int top_k) { return Settings{f[0], f[1], f[2], f[3], f[4], f[5], top_k}; }

// A thread's buffers, kept between calls: the vocabulary is large and fresh memory is slow.
struct Scratch {
    std::vector<double> l, own, tmp;
    std::vector<int> idx;
    Alive a;
};

// One request; see `ks_choose`.
int choose_one(Scratch& sc, const void* logits, int dtype, int n, const double* floats, int top_k, const int* sequence, int seq_len,
               int generated_from, unsigned long long* state, double* probs, int want_draw) {
    if (n <= 0) return 0;
    const Settings s = settings_of(floats, top_k);
    std::vector<double>& l = sc.l;
    l.resize((size_t)n);
    widen(logits, dtype, n, l.data());
    int certain = penalties_and_temperature(l.data(), n, s, sequence, seq_len, generated_from);
    if (certain >= 0) return certain;
    bool nan = false;
    for (int i = 0; i < n && !nan; ++i) nan = std::isnan(l[(size_t)i]);
    if (nan) {
        double* p = probs;
        if (!p) { sc.own.resize((size_t)n); p = sc.own.data(); }
        certain = filters_plain(l.data(), n, s, p, sc.idx, sc.tmp);
        if (certain >= 0 || !want_draw) return certain;
        return draw(p, n, next_uniform(reinterpret_cast<uint64_t*>(state)));
    }
    Alive& a = sc.a;
    certain = filters_alive(l.data(), n, s, a);
    if (certain >= 0) return certain;
    if (probs) {
        std::fill(probs, probs + n, 0.0);
        for (size_t i = 0; i < a.idx.size(); ++i) probs[a.idx[i]] = a.p[i];
    }
    if (!want_draw) return -1;
    const double u = next_uniform(reinterpret_cast<uint64_t*>(state));
    double total = 0.0;
    int last = 0;
    for (size_t i = 0; i < a.idx.size(); ++i)
        if (a.p[i] > 0.0) {
            total += a.p[i];
            last = a.idx[i];
            if (u < total) return a.idx[i];
        }
    return last;                               // rounding left u above the total: the last possible token
}

}  // namespace

extern "C" {

// The generator's state from a seed: four SplitMix64 outputs.
void ks_seed(unsigned long long seed, unsigned long long* state) {
    uint64_t z = seed;
    for (int i = 0; i < 4; ++i) {
        z += 0x9E3779B97F4A7C15ull;
        uint64_t x = z;
        x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
        x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
        state[i] = x ^ (x >> 31);
    }
}

double ks_uniform(unsigned long long* state) { return next_uniform(reinterpret_cast<uint64_t*>(state)); }

// One request. `logits`: n values of `dtype` (0 float32, 1 float64), not changed. `floats`:
// temperature, top_p, min_p, repetition, frequency and presence penalty. With `probs` given and
// `want_draw` 0 nothing is drawn: the return value is the certain token, or -1 with the
// probabilities in `probs`. Otherwise a token is returned, and the generator moves on only if the
// choice was not certain.
int ks_choose(const void* logits, int dtype, int n, const double* floats, int top_k, const int* sequence, int seq_len,
              int generated_from, unsigned long long* state, double* probs, int want_draw) {
    static thread_local Scratch scratch;
    return choose_one(scratch, logits, dtype, n, floats, top_k, sequence, seq_len, generated_from, state, probs, want_draw);
}

// `count` requests at once: row i of `logits` (rows `row_stride` values apart), settings
// floats[6 i ..] and top_k[i], sequence i at sequences[i] (seq_lens[i] tokens, the generated ones from
// generated_from[i]), generator states[4 i ..]; tokens[i] receives the choice. Up to `threads`
// threads share the requests (the calling thread is one of them); calls are served one at a time.
void ks_choose_many(int count, const void* logits, long long row_stride, int dtype, int n, const double* floats, const int* top_k,
                    const int* const* sequences, const int* seq_lens, const int* generated_from, unsigned long long* states,
                    int* tokens, int threads) {
    static std::mutex one_call;
    static std::vector<std::unique_ptr<Scratch>> pool;       // a worker's buffers, kept between calls
    std::lock_guard<std::mutex> lock(one_call);
    const int workers = std::max(1, std::min(threads, count));
    while ((int)pool.size() < workers) pool.emplace_back(new Scratch());
    auto share = [&](int w) {
        for (int i = w; i < count; i += workers) {
            const char* row = static_cast<const char*>(logits) + (size_t)i * (size_t)row_stride * (dtype == 0 ? 4 : 8);
            tokens[i] = choose_one(*pool[(size_t)w], row, dtype, n, floats + 6 * (size_t)i, top_k[i], sequences[i], seq_lens[i],
                                   generated_from[i], states + 4 * (size_t)i, nullptr, 1);
        }
    };
    std::vector<std::thread> others;
    for (int w = 1; w < workers; ++w) others.emplace_back(share, w);
    share(0);
    for (std::thread& t : others) t.join();
}

}  // extern "C"
