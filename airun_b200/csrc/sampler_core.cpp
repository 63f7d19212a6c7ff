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
