// Random valid call sequences against the host library (the cache bookkeeping and the host sampler);
// test_host_sanitizers.py builds this file with the library's sources under AddressSanitizer, UBSan and
// ThreadSanitizer and runs it.
#include <cmath>
#include <cstdio>
#include <cstdint>
#include <limits>
#include <random>
#include <vector>
extern "C" {
int ks_choose(const void*, int, int, const double*, int, const int*, int, int, unsigned long long*, double*, int);
void ks_choose_many(int, const void*, long long, int, int, const double*, const int*, const int* const*, const int*, const int*, unsigned long long*, int*, int);
void ks_seed(unsigned long long, unsigned long long*);
void* kc_create(int, int, const int*, const int*, int);
void kc_destroy(void*);
int kc_add(void*);
int kc_remove(void*, int);
int kc_plan_prepare(void*, int, const int*, const int*, long long*);
int kc_plan_fill(void*, int, const int*, const int*, int*, int*, int*, int*, int*, int*, int*, uint8_t*, int* const*, int* const*, int, int*, int);
long long kc_commit(void*, int, const int*, const int*);
int kc_abort(void*, int, const int*);
int kc_check(void*, char*, int);
}
int main() {
    std::mt19937_64 g(7);
    auto U = [&](int lo, int hi) { return (int)(lo + g() % (uint64_t)(hi - lo + 1)); };
    // ---- sampler
    for (int it = 0; it < 3000; ++it) {
        const int n = U(1, 3000);
        std::vector<double> l((size_t)n);
        std::normal_distribution<double> d(0.0, it % 3 == 0 ? 8.0 : 1.0);
        for (auto& v : l) v = d(g);
        if (it % 5 == 0) for (int k = 0; k < n / 4 + 1; ++k) l[(size_t)U(0, n - 1)] = -std::numeric_limits<double>::infinity();
        if (it % 11 == 0) l[(size_t)U(0, n - 1)] = std::nan("");
        double f[6] = {(double)U(0, 3) * 0.6, U(0, 3) == 0 ? 1.0 : U(0, 100) / 100.0, U(0, 2) == 0 ? U(0, 100) / 100.0 : 0.0,
                       U(0, 2) == 0 ? 1.3 : 1.0, U(0, 3) == 0 ? 0.4 : 0.0, U(0, 3) == 0 ? 0.2 : 0.0};
        const int k = U(0, 3) == 0 ? 0 : U(1, n + 5);
        std::vector<int> seq((size_t)U(0, 50));
        for (auto& t : seq) t = U(-3, n + 3);
        unsigned long long st[4]; ks_seed((unsigned long long)it, st);
        std::vector<double> probs((size_t)n);
        const int tok = ks_choose(l.data(), 1, n, f, k, seq.data(), (int)seq.size(), U(0, 60), st, it % 2 ? probs.data() : nullptr, it % 3 != 0);
        if (tok < -1 || tok >= n) { printf("bad token %d of %d\n", tok, n); return 1; }
    }
    {
        const int count = 9, n = 4000;
        std::vector<float> rows((size_t)count * n);
        std::normal_distribution<float> d(0.f, 3.f);
        for (auto& v : rows) v = d(g);
        std::vector<double> f((size_t)count * 6);
        std::vector<int> tk((size_t)count), lens((size_t)count, 0), gf((size_t)count, 0), toks((size_t)count);
        std::vector<const int*> seqs((size_t)count, nullptr);
        std::vector<unsigned long long> st((size_t)count * 4);
        for (int i = 0; i < count; ++i) { double v[6] = {0.9, 0.9, 0.01, 1.0, 0.0, 0.0}; for (int j = 0; j < 6; ++j) f[(size_t)i * 6 + j] = v[j]; tk[(size_t)i] = 40; ks_seed((unsigned long long)i, &st[(size_t)i * 4]); }
        for (int rep = 0; rep < 20; ++rep) ks_choose_many(count, rows.data(), n, 0, n, f.data(), tk.data(), seqs.data(), lens.data(), gf.data(), st.data(), toks.data(), 1 + rep % 5);
    }
    // ---- cache
    for (int it = 0; it < 200; ++it) {
        const int G = U(1, 3), ps = 1 << U(2, 5), maxs = U(1, 6);
        std::vector<int> pages((size_t)G), win((size_t)G);
        for (int q = 0; q < G; ++q) { pages[(size_t)q] = U(2, 25); win[(size_t)q] = U(0, 2) == 0 ? -1 : U(1, 5 * ps); }
        void* h = kc_create(G, ps, pages.data(), win.data(), maxs);
        std::vector<int> live;
        for (int op = 0; op < 300; ++op) {
            const int what = U(0, 9);
            if (what < 2 || live.empty()) { const int s = kc_add(h); if (s > 0) live.push_back(s); }
            else if (what < 3) { const size_t i = (size_t)U(0, (int)live.size() - 1); kc_remove(h, live[i]); live.erase(live.begin() + (std::ptrdiff_t)i); }
            else {
                const int n = U(1, (int)live.size());
                std::vector<int> slots(live.begin(), live.begin() + n), counts((size_t)n);
                for (auto& c : counts) c = U(0, 4) ? 1 : U(1, 3 * ps + 1);
                long long info[7];
                if (kc_plan_prepare(h, n, slots.data(), counts.data(), info) != 0) continue;
                const int rows = (int)info[1], width = (int)(info[2] > 0 ? info[2] : 1), take = (int)info[3];
                std::vector<int> r3((size_t)3 * rows + 1), e4((size_t)4 * n), taken((size_t)4 * take + 4);
                std::vector<uint8_t> fresh((size_t)n);
                std::vector<std::vector<int>> lines((size_t)G, std::vector<int>((size_t)rows + 1)), tabs((size_t)G, std::vector<int>((size_t)n * width, -1));
                std::vector<int*> lp, tp;
                for (int q = 0; q < G; ++q) { lp.push_back(lines[(size_t)q].data()); tp.push_back(tabs[(size_t)q].data()); }
                const int got = kc_plan_fill(h, n, slots.data(), counts.data(), r3.data(), r3.data() + rows, r3.data() + 2 * rows, e4.data(), e4.data() + n,
                                             e4.data() + 2 * n, e4.data() + 3 * n, fresh.data(), lp.data(), tp.data(), width, taken.data(), take);
                if (got != take) { printf("took %d of %d\n", got, take); return 1; }
                if (U(0, 4) == 0) kc_abort(h, got, taken.data()); else kc_commit(h, n, slots.data(), counts.data());
            }
            char msg[256];
            if (kc_check(h, msg, 256)) { printf("check: %s\n", msg); return 1; }
        }
        kc_destroy(h);
    }
    printf("ok\n");
    return 0;
}
