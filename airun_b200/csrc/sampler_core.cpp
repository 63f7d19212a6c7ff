// Host side of sampling: the k largest logits of every row that the host chain samples.
//
// A request whose parameters go beyond "first maximum" and "draw at a temperature" is sampled on the
// host from its row of float32 logits (sampling/sampler.py; the reference's sampler is host code too,
// crates/airun-core/src/sample.rs:348-486, and cuts the candidates to top-k before anything that
// sorts, sample.rs:390-403).  Selecting 40 of 151,936 logits is the only step of that chain whose
// cost grows with the vocabulary, so it is done here: one pass over the row with a heap of k entries,
// rows side by side on threads.  Everything after it works on k candidates.
//
// Order of the result: the largest value first; equal values by ascending index, so the choice among
// ties does not depend on the algorithm.  NaN counts as -inf (it never wins, sample.rs:639-649).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <thread>
#include <utility>
#include <vector>

#define HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct Cand {
    float v;
    int i;
};

// "a is worse than b": a smaller value, or the same value at a later index.
inline bool worse(const Cand& a, const Cand& b) { return a.v < b.v || (a.v == b.v && a.i > b.i); }

// heap with the WORST kept candidate on top
struct WorstOnTop {
    bool operator()(const Cand& a, const Cand& b) const { return worse(b, a); }
};

void topk_row(const float* x, long long n, int k, int* out_idx, float* out_val) {
    const float ninf = -std::numeric_limits<float>::infinity();
    std::vector<Cand> heap;
    heap.reserve((size_t)k);
    long long i = 0;
    for (; i < n && (int)heap.size() < k; ++i) {
        const float v = std::isnan(x[i]) ? ninf : x[i];
        heap.push_back(Cand{v, (int)i});
    }
    std::make_heap(heap.begin(), heap.end(), WorstOnTop());
    float floor_v = heap.front().v;                 // value of the worst kept candidate
    for (; i < n; ++i) {
        const float v = x[i];
        if (!(v > floor_v)) continue;               // also false for NaN; an equal value at a later index stays out
        std::pop_heap(heap.begin(), heap.end(), WorstOnTop());
        heap.back() = Cand{v, (int)i};
        std::push_heap(heap.begin(), heap.end(), WorstOnTop());
        floor_v = heap.front().v;
    }
    std::sort(heap.begin(), heap.end(), [](const Cand& a, const Cand& b) { return worse(b, a); });
    for (size_t j = 0; j < heap.size(); ++j) {
        out_idx[j] = heap[j].i;
        out_val[j] = heap[j].v;
    }
}

}  // namespace

// x: n_rows rows of n float32 values, row r at x + r * ld.  ks[r] (1 <= ks[r] <= n) candidates of row r
// go to out_idx / out_val at r * out_ld.  Up to max_threads rows run side by side.  Returns 0, or 1
// for arguments it cannot take (nothing is written then).
HOST_EXPORT int airun_topk_rows(const float* x, long long ld, int n_rows, long long n, const int* ks, int* out_idx,
                                float* out_val, long long out_ld, int max_threads) {
    if (!x || !ks || !out_idx || !out_val || n_rows < 0 || n <= 0 || n > 2147483647LL || ld < n) return 1;
    for (int r = 0; r < n_rows; ++r)
        if (ks[r] < 1 || ks[r] > n || ks[r] > out_ld) return 1;
    auto run = [&](int r) { topk_row(x + (long long)r * ld, n, ks[r], out_idx + (long long)r * out_ld, out_val + (long long)r * out_ld); };
    const int workers = std::max(1, std::min(max_threads, n_rows));
    if (workers == 1) {
        for (int r = 0; r < n_rows; ++r) run(r);
        return 0;
    }
    std::vector<std::thread> pool;
    pool.reserve((size_t)workers);
    for (int w = 0; w < workers; ++w)
        pool.emplace_back([&, w] {
            for (int r = w; r < n_rows; r += workers) run(r);
        });
    for (std::thread& t : pool) t.join();
    return 0;
}

// ---------------------------------------------------------------------------------------------------
// The usual chain in one call: bias -> penalties -> top-k -> softmax at a fixed temperature -> min-p ->
// top-p -> draw, for the rows whose parameters ask for nothing else (sampling/sampler.py decides; DRY,
// top-n-sigma, typical, XTC, dynamic temperature, mirostat and log-probabilities stay with the Python
// chain, which is also this one's plain twin in the tests).  Every step keeps the arithmetic of that
// twin: float32 where it is float32, double where it is double, sums one after the other, so the two
// pick the same token from the same logits and generator state.  Order and formulas as the reference's
// sampler (crates/airun-core/src/sample.rs:348-486, penalties :651-705, generator :778-798).
struct ChainParams {
    double temperature, top_p, min_p, repeat, presence, frequency;
    int top_k, penalize;                 // penalize: the three penalties are on
    int n_bias;
    const int* bias_ids;
    const float* bias_vals;
};

struct ChainRow {
    float* logits;                       // [vocab], modified in place
    const long long* window;             // the last repeat_last_n tokens of the request
    long long n_window;
    const ChainParams* params;
    unsigned long long* rng_state;       // xorshift64 state, advanced by the draw
    int out;                             // the token picked
};

namespace {

inline double next_uniform(unsigned long long* state) {       // (x >> 40) / 2^24
    unsigned long long x = *state;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    *state = x;
    return (double)(x >> 40) / 16777216.0;
}

void chain_row(ChainRow& row, long long vocab) {
    const ChainParams& p = *row.params;
    float* logits = row.logits;
    for (int b = 0; b < p.n_bias; ++b)
        if (p.bias_ids[b] >= 0 && p.bias_ids[b] < vocab) logits[p.bias_ids[b]] += p.bias_vals[b];
    if (p.penalize && row.n_window > 0) {
        // once per distinct token: sorted copy of the window, runs of equal ids give the counts
        std::vector<long long> w(row.window, row.window + row.n_window);
        std::sort(w.begin(), w.end());
        for (size_t i = 0; i < w.size();) {
            size_t j = i;
            while (j < w.size() && w[j] == w[i]) ++j;
            const long long t = w[i];
            if (t >= 0 && t < vocab) {
                double l = (double)logits[t];
                if (p.repeat != 1.0) l = l > 0.0 ? l / p.repeat : l * p.repeat;
                logits[t] = (float)(l - ((double)(j - i) * p.frequency + p.presence));
            }
            i = j;
        }
    }
    long long keep = p.top_k > 0 ? std::min<long long>(std::max(p.top_k, 1), vocab) : vocab;
    std::vector<int> ids((size_t)keep);
    std::vector<float> probs((size_t)keep);
    topk_row(logits, vocab, (int)keep, ids.data(), probs.data());          // probs holds the logits for now
    const float mx = probs[0];
    const float temperature = (float)p.temperature;
    size_t n = (size_t)keep;
    float sum = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        const float scaled = (probs[i] - mx) / temperature;
        probs[i] = (float)std::exp((double)scaled);
        sum += probs[i];
    }
    for (size_t i = 0; i < n; ++i) probs[i] = probs[i] / sum;
    if (p.min_p > 0.0) {
        const float threshold = (float)p.min_p * probs[0];
        size_t k = 0;
        for (size_t i = 0; i < n; ++i) k += probs[i] >= threshold;
        n = std::max<size_t>(k, 1);
    }
    if (p.top_p < 1.0) {
        const float top_p = (float)p.top_p;
        float cumulative = 0.0f;
        size_t cut = n;
        for (size_t i = 0; i < n; ++i) {
            cumulative += probs[i];
            if (cumulative >= top_p) { cut = i + 1; break; }                 // the token that crossed the threshold stays
        }
        n = std::max<size_t>(cut, 1);
    }
    float total = 0.0f;
    for (size_t i = 0; i < n; ++i) total += probs[i];
    if (!((double)total > 0.0)) {
        if (total == total) { row.out = ids[0]; return; }                   // every survivor rounded to zero
    }
    double target = next_uniform(row.rng_state) * (double)total;
    row.out = ids[n - 1];
    for (size_t i = 0; i < n; ++i) {
        target -= (double)probs[i];
        if (target <= 0.0) { row.out = ids[i]; break; }
    }
}

}  // namespace

// One token for every row.  Returns 0, or 1 for arguments it cannot take.
HOST_EXPORT int airun_sample_chain_rows(ChainRow* rows, int n_rows, long long vocab, int max_threads) {
    if (!rows || n_rows < 0 || vocab <= 0 || vocab > 2147483647LL) return 1;
    for (int r = 0; r < n_rows; ++r)
        if (!rows[r].logits || !rows[r].params || !rows[r].rng_state || rows[r].n_window < 0 || !(rows[r].params->temperature > 0.0)) return 1;
    const int workers = std::max(1, std::min(max_threads, n_rows));
    if (workers == 1) {
        for (int r = 0; r < n_rows; ++r) chain_row(rows[r], vocab);
        return 0;
    }
    std::vector<std::thread> pool;
    pool.reserve((size_t)workers);
    for (int w = 0; w < workers; ++w)
        pool.emplace_back([&, w] {
            for (int r = w; r < n_rows; r += workers) chain_row(rows[r], vocab);
        });
    for (std::thread& t : pool) t.join();
    return 0;
}

// The same chain on each row's largest raw logits instead of the whole row (found on the device with their ids: see
// largest_logits_kernel in sampling.cu; enough of them that the chain's cut to top_k cannot reach beyond them).  The
// candidates, in ascending order of their ids, stand as a short row of their own, the window's tokens become
// positions in it (a token that is no candidate cannot be picked and is left out), and chain_row runs unchanged, so
// equal values fall as in the whole row.  ids: [n][n_cand], < 0 is padding; window: the rows' windows one after the
// other, win_off[r] .. win_off[r + 1]; params: [n] with n_bias 0; states: [n]; out: [n] token ids.
HOST_EXPORT int airun_sample_candidates(int n_rows, int n_cand, const int* ids, const float* vals, const long long* window,
                                        const long long* win_off, const ChainParams* params, unsigned long long* states,
                                        int* out, int max_threads) {
    if (n_rows < 0 || n_cand <= 0 || !ids || !vals || !win_off || !params || !states || !out) return 1;
    for (int r = 0; r < n_rows; ++r)
        if (!(params[r].temperature > 0.0) || params[r].n_bias != 0 || win_off[r + 1] < win_off[r]) return 1;
    auto one = [&](int r) {
        std::vector<std::pair<int, float>> cand;
        cand.reserve((size_t)n_cand);
        for (int i = 0; i < n_cand; ++i)
            if (ids[(size_t)r * n_cand + i] >= 0) cand.emplace_back(ids[(size_t)r * n_cand + i], vals[(size_t)r * n_cand + i]);
        if (cand.empty()) { out[r] = 0; return; }
        std::sort(cand.begin(), cand.end(), [](const std::pair<int, float>& a, const std::pair<int, float>& b) { return a.first < b.first; });
        std::vector<float> logits(cand.size());
        for (size_t i = 0; i < cand.size(); ++i) logits[i] = cand[i].second;
        std::vector<long long> positions;
        for (long long i = win_off[r]; i < win_off[r + 1]; ++i) {
            const long long t = window[i];
            size_t lo = 0, hi = cand.size();
            while (lo < hi) {
                const size_t mid = (lo + hi) / 2;
                if ((long long)cand[mid].first < t) lo = mid + 1; else hi = mid;
            }
            if (lo < cand.size() && (long long)cand[lo].first == t) positions.push_back((long long)lo);
        }
        ChainRow row{logits.data(), positions.data(), (long long)positions.size(), &params[r], &states[r], -1};
        chain_row(row, (long long)logits.size());
        out[r] = row.out >= 0 && (size_t)row.out < cand.size() ? cand[(size_t)row.out].first : 0;
    };
    // a row takes a few microseconds, starting a thread tens: threads only from 16 rows each on
    const int workers = std::max(1, std::min(max_threads, n_rows / 16));
    if (workers == 1) {
        for (int r = 0; r < n_rows; ++r) one(r);
        return 0;
    }
    std::vector<std::thread> pool;
    pool.reserve((size_t)workers);
    for (int w = 0; w < workers; ++w)
        pool.emplace_back([&, w] {
            for (int r = w; r < n_rows; r += workers) one(r);
        });
    for (std::thread& t : pool) t.join();
    return 0;
}

