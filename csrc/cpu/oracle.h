// CPU oracle: a C++17 restatement of the SketchML compression algorithms. Every
// sm_100a kernel of this project is tested against these functions.
//
// Reference behaviour restated (paths inside the reference project, module `sketch`):
//   sketch/quantile/HeapQuantileSketch.java:73-124,126-143,186-217,293-323 -> QuantileSketch
//   sketch/quantile/QSketchUtils.java:45-82                                -> compact / carry
//   base/Quantizer.java:39-92,119-124, quantization/QuantileQuantizer.java:27-50,
//   quantization/UniformQuantizer.java:21-44                               -> Quantizer
//   sketch/frequency/MinMaxSketch.java:27-86                               -> MinMaxSketch
//   sketch/frequency/FSketchUtils.java:30-47, GroupedMinMaxSketch.java:51-146 -> GroupedSketch
//   binary/BinaryUtils.java:6-29, DeltaBinaryEncoder.java:26-65,
//   binary/DeltaAdaptiveEncoder.java:23-146, HuffmanEncoder.java:88-166    -> encoders
//   util/Sort.java:13-58,362-379, util/Maths.java:51-67                    -> helpers
// and from module `ml`: gradient/FixedPointGradient.scala:39-75,
//   gradient/ZipGradient.scala:70-129.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <limits>
#include <map>
#include <queue>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../common/skml_common.h"

namespace skml {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// ---------------------------------------------------------------------------
// Bit streams in java.util.BitSet order: stream index i is bit (i & 63) of word
// (i >> 6); values are written most significant bit first.
// ---------------------------------------------------------------------------
struct BitStream {
    std::vector<uint64_t> words;
    void set(uint64_t i) {
        size_t w = i >> 6;
        if (w >= words.size()) words.resize(w + 1, 0);
        words[w] |= 1ull << (i & 63);
    }
    bool get(uint64_t i) const {
        size_t w = i >> 6;
        return w < words.size() && ((words[w] >> (i & 63)) & 1ull);
    }
    void put(uint64_t off, uint32_t value, int nbits) {
        for (int i = 0; i < nbits; ++i)
            if ((value >> (nbits - 1 - i)) & 1u) set(off + i);
    }
    uint32_t take(uint64_t off, int nbits) const {
        uint32_t r = 0;
        for (int i = 0; i < nbits; ++i) r = (r << 1) | (get(off + i) ? 1u : 0u);
        return r;
    }
    void pad_to_bits(uint64_t nbits) {
        size_t w = (size_t)((nbits + 63) >> 6);
        if (words.size() < w) words.resize(w, 0);
    }
    // BitSet.toLongArray() drops trailing all-zero words.
    size_t java_word_count() const {
        size_t n = words.size();
        while (n > 0 && words[n - 1] == 0) --n;
        return n;
    }
};

inline int floor_log2(uint32_t x) {
    if (x == 0) throw Error("log2 of zero: keys must be strictly increasing");
    int r = 0;
    while (x >>= 1) ++r;
    return r;
}

// ---------------------------------------------------------------------------
// Sorting / selection helpers
// ---------------------------------------------------------------------------
template <class T>
T quick_select(std::vector<T> a, size_t k) {  // k-th smallest, 1-based
    if (k < 1 || k > a.size()) throw Error("k is more than number of elements in array");
    std::nth_element(a.begin(), a.begin() + (k - 1), a.end());
    return a[k - 1];
}

template <class T>
T select_kth_largest(const std::vector<T>& a, size_t k) {
    if (k < 1 || k > a.size()) throw Error("k is more than number of elements in array");
    std::priority_queue<T, std::vector<T>, std::greater<T>> q;
    size_t i = 0;
    for (; i < k; ++i) q.push(a[i]);
    for (; i < a.size(); ++i)
        if (a[i] > q.top()) {
            q.pop();
            q.push(a[i]);
        }
    return q.top();
}

// k-way merge of ascending key lists carrying one payload each; ties go to the
// earlier list.
inline void kway_merge(const std::vector<std::vector<int32_t>>& ks,
                       const std::vector<std::vector<int32_t>>& ys, std::vector<int32_t>& k_out,
                       std::vector<int32_t>& y_out) {
    size_t total = 0;
    for (auto& v : ks) total += v.size();
    k_out.resize(total);
    y_out.resize(total);
    typedef std::pair<int32_t, size_t> Item;
    std::priority_queue<Item, std::vector<Item>, std::greater<Item>> heap;
    std::vector<size_t> cur(ks.size(), 0);
    for (size_t i = 0; i < ks.size(); ++i)
        if (!ks[i].empty()) heap.push({ks[i][0], i});
    size_t o = 0;
    while (!heap.empty()) {
        auto [key, i] = heap.top();
        heap.pop();
        k_out[o] = key;
        y_out[o] = ys[i][cur[i]];
        ++o;
        if (++cur[i] < ks[i].size()) heap.push({ks[i][cur[i]], i});
    }
}

template <class T>
std::vector<T> unique_sorted(const std::vector<T>& s) {
    std::vector<T> r;
    for (size_t i = 0; i < s.size(); ++i)
        if (i == 0 || s[i] != s[i - 1]) r.push_back(s[i]);
    return r;
}

// ---------------------------------------------------------------------------
// Mergeable quantile sketch (k items per level, level L has weight 2^(L+1)).
// offset_mode: 0 / 1 = fixed compaction offset, 2 = seeded pseudo-random.
// ---------------------------------------------------------------------------
template <class T>
class QuantileSketch {
public:
    QuantileSketch(int k = 128, uint64_t seed = 0, int offset_mode = 2, bool java_compat_max = false)
        : k_(k), seed_(seed), offset_mode_(offset_mode), java_max_(java_compat_max) {
        if (k < 1) throw Error("Invalid value of k: k should be positive");
        if (k >= 65535) throw Error("Invalid value of k: k should be smaller than 65535");
        if (k & (k - 1)) throw Error("Invalid value of k: k should be power of 2");
        reset();
    }
    void reset() {
        n_ = 0;
        draws_ = 0;
        base_.clear();
        levels_.clear();
        min_ = std::numeric_limits<T>::max();
        // The reference starts max at Double.MIN_VALUE, the smallest positive double.
        max_ = java_max_ ? std::numeric_limits<T>::denorm_min() : std::numeric_limits<T>::lowest();
    }
    void update(T v) {
        if (std::isnan(v)) throw Error("Encounter NaN value");
        max_ = std::max(max_, v);
        min_ = std::min(min_, v);
        base_.push_back(v);
        ++n_;
        if ((int)base_.size() == 2 * k_) {
            std::sort(base_.begin(), base_.end());
            std::vector<T> run = compact(base_);
            base_.clear();
            carry(0, std::move(run));
        }
    }
    void merge(const QuantileSketch& o) {
        if (o.n_ == 0) return;
        if (o.k_ != k_) throw Error("Merge sketches with different k");
        uint64_t total = n_ + o.n_;
        for (T v : o.base_) update(v);
        for (size_t l = 0; l < o.levels_.size(); ++l)
            if (!o.levels_[l].empty()) carry((int)l, o.levels_[l]);
        n_ = total;
        max_ = std::max(max_, o.max_);
        min_ = std::min(min_, o.min_);
    }
    // Samples in ascending order and their exclusive cumulative weights (last entry = n).
    void summary(std::vector<T>& samples, std::vector<uint64_t>& cum) const {
        std::vector<std::pair<T, uint64_t>> items;
        uint64_t w = 1;
        for (size_t l = 0; l < levels_.size(); ++l) {
            w *= 2;
            for (T v : levels_[l]) items.push_back({v, w});
        }
        std::vector<T> b = base_;
        std::sort(b.begin(), b.end());
        for (T v : b) items.push_back({v, 1});
        std::stable_sort(items.begin(), items.end(),
                         [](const auto& a, const auto& c) { return a.first < c.first; });
        samples.resize(items.size());
        cum.resize(items.size() + 1);
        uint64_t c = 0;
        for (size_t i = 0; i < items.size(); ++i) {
            samples[i] = items[i].first;
            cum[i] = c;
            c += items[i].second;
        }
        cum[items.size()] = c;
    }
    // q-1 split values: split i is the sample covering rank min(floor(n*(i+1)/q), n-1).
    std::vector<T> quantiles(int q) const {
        if (q <= 1) throw Error("Invalid partition number: " + std::to_string(q));
        std::vector<T> samples;
        std::vector<uint64_t> cum;
        summary(samples, cum);
        std::vector<T> splits(q - 1, std::numeric_limits<T>::quiet_NaN());
        if (samples.empty()) return splits;
        size_t index = 0;
        double frac = 1.0 / q, step = 1.0 / q;
        for (int i = 0; i + 1 < q; ++i) {
            uint64_t rank = (uint64_t)((double)n_ * frac);
            rank = std::min<uint64_t>(rank, n_ - 1);
            size_t left = index, right = cum.size() - 1;
            while (left + 1 < right) {
                size_t mid = left + ((right - left) >> 1);
                if (cum[mid] <= rank) left = mid;
                else right = mid;
            }
            splits[i] = samples[left];
            index = left;
            frac += step;
        }
        return splits;
    }
    uint64_t n() const { return n_; }
    T min_value() const { return min_; }
    T max_value() const { return max_; }
    int k() const { return k_; }
    size_t retained() const {
        size_t r = base_.size();
        for (auto& l : levels_) r += l.size();
        return r;
    }

private:
    std::vector<T> compact(const std::vector<T>& two_k) {
        int off = offset_mode_ == 2 ? (int)(skml_rand(seed_, 0x51u, draws_++, 0) & 1u) : offset_mode_;
        std::vector<T> out(k_);
        for (int j = 0; j < k_; ++j) out[j] = two_k[2 * j + off];
        return out;
    }
    void carry(int level, std::vector<T> run) {
        for (;; ++level) {
            if ((int)levels_.size() <= level) levels_.resize(level + 1);
            if (levels_[level].empty()) {
                levels_[level] = std::move(run);
                return;
            }
            std::vector<T> merged(2 * k_);
            std::merge(levels_[level].begin(), levels_[level].end(), run.begin(), run.end(),
                       merged.begin());
            levels_[level].clear();
            run = compact(merged);
        }
    }
    int k_;
    uint64_t seed_;
    int offset_mode_;
    bool java_max_;
    uint64_t n_ = 0, draws_ = 0;
    T min_, max_;
    std::vector<T> base_;
    std::vector<std::vector<T>> levels_;
};

// ---------------------------------------------------------------------------
// Quantizers
// ---------------------------------------------------------------------------
template <class T>
struct Quantizer {
    int bin_num = 0;
    int zero_idx = 0;
    T min = 0, max = 0;
    std::vector<T> splits;      // bin_num - 1 ascending split points
    std::vector<int32_t> bins;  // one bucket index per input value

    int index_of(T x) const {  // number of splits <= x
        return (int)(std::upper_bound(splits.begin(), splits.end(), x) - splits.begin());
    }
    void find_zero_idx() {
        if (min > 0) zero_idx = 0;
        else if (max < 0) zero_idx = bin_num - 1;
        else {
            int t = 0;
            while (t < bin_num - 1 && splits[t] < 0) ++t;
            zero_idx = t;
        }
    }
    std::vector<T> values() const {  // decode value of each bucket = midpoint of its edges
        std::vector<T> r(bin_num);
        if (bin_num == 1) {
            r[0] = (T)0.5 * (min + max);
            return r;
        }
        int sn = bin_num - 1;
        r[0] = (T)0.5 * (min + splits[0]);
        for (int i = 1; i < sn; ++i) r[i] = (T)0.5 * (splits[i - 1] + splits[i]);
        r[sn] = (T)0.5 * (splits[sn - 1] + max);
        return r;
    }
    void to_bins(const T* v, size_t n) {
        bins.resize(n);
        for (size_t i = 0; i < n; ++i) bins[i] = index_of(v[i]);
    }
    void times_by(T x) {
        min *= x;
        max *= x;
        for (auto& s : splits) s *= x;
    }
};

template <class T>
Quantizer<T> quantizer_from_splits(const std::vector<T>& raw_splits, T min, T max, const T* v, size_t n) {
    Quantizer<T> q;
    q.splits = unique_sorted(raw_splits);
    q.bin_num = (int)q.splits.size() + 1;
    q.min = min;
    q.max = max;
    q.find_zero_idx();
    if (v) q.to_bins(v, n);
    return q;
}

template <class T>
Quantizer<T> quantile_quantize(const T* v, size_t n, int bin_num, int k, uint64_t seed, int offset_mode,
                               bool java_compat_max) {
    if (n == 0) throw Error("cannot quantize an empty vector");
    QuantileSketch<T> sk(k, seed, offset_mode, java_compat_max);
    for (size_t i = 0; i < n; ++i) sk.update(v[i]);
    return quantizer_from_splits<T>(sk.quantiles(bin_num), sk.min_value(), sk.max_value(), v, n);
}

// Runs fn(t) for t in [0, threads) on `threads` std::threads (the calling thread takes t = 0) and
// rethrows the first exception. The reference keeps one process-wide thread pool of this size
// (common/Constants.java:19-24).
template <class F>
void run_parallel(int threads, F fn) {
    if (threads <= 1) {
        fn(0);
        return;
    }
    std::vector<std::thread> pool;
    std::vector<std::string> errors(threads);
    for (int t = 1; t < threads; ++t)
        pool.emplace_back([&, t] {
            try {
                fn(t);
            } catch (const std::exception& e) {
                errors[t] = e.what();
                if (errors[t].empty()) errors[t] = "worker thread failed";
            }
        });
    try {
        fn(0);
    } catch (const std::exception& e) {
        errors[0] = e.what();
        if (errors[0].empty()) errors[0] = "worker thread failed";
    }
    for (auto& th : pool) th.join();
    for (auto& e : errors)
        if (!e.empty()) throw Error(e);
}

// quantization/QuantileQuantizer.java:53-92 (parallelQuantize): every thread summarises a contiguous
// slice of the values in its own sketch, the sketches are merged into the first one, the splits are
// queried from the merged summary (and, unlike the reference, de-duplicated as in the serial path),
// and the bucket of every value is looked up slice by slice in parallel.
template <class T>
Quantizer<T> quantile_quantize_parallel(const T* v, size_t n, int bin_num, int k, uint64_t seed, int offset_mode,
                                        bool java_compat_max, int threads) {
    if (n == 0) throw Error("cannot quantize an empty vector");
    if (threads < 1) throw Error("parallelism must be positive");
    threads = (int)std::min<size_t>((size_t)threads, std::max<size_t>(1, n / 256));
    if (threads == 1) return quantile_quantize<T>(v, n, bin_num, k, seed, offset_mode, java_compat_max);
    std::vector<QuantileSketch<T>> parts;
    parts.reserve(threads);
    for (int t = 0; t < threads; ++t) parts.emplace_back(k, seed + 0x9E3779B97F4A7C15ull * (uint64_t)t, offset_mode, java_compat_max);
    auto slice = [&](int t, size_t& lo, size_t& hi) {
        lo = n * (size_t)t / (size_t)threads;
        hi = n * (size_t)(t + 1) / (size_t)threads;
    };
    run_parallel(threads, [&](int t) {
        size_t lo, hi;
        slice(t, lo, hi);
        for (size_t i = lo; i < hi; ++i) parts[t].update(v[i]);
    });
    for (int t = 1; t < threads; ++t) parts[0].merge(parts[t]);
    Quantizer<T> q = quantizer_from_splits<T>(parts[0].quantiles(bin_num), parts[0].min_value(), parts[0].max_value(),
                                              (const T*)nullptr, 0);
    q.bins.resize(n);
    run_parallel(threads, [&](int t) {
        size_t lo, hi;
        slice(t, lo, hi);
        for (size_t i = lo; i < hi; ++i) q.bins[i] = q.index_of(v[i]);
    });
    return q;
}

template <class T>
Quantizer<T> uniform_quantize(const T* v, size_t n, int bin_num) {
    if (n == 0) throw Error("cannot quantize an empty vector");
    Quantizer<T> q;
    q.bin_num = bin_num;
    q.min = *std::min_element(v, v + n);
    q.max = *std::max_element(v, v + n);
    T step = (q.max - q.min) / (T)bin_num;
    q.splits.resize(bin_num - 1);
    if (bin_num > 1) q.splits[0] = q.min + step;
    for (int i = 1; i < bin_num - 1; ++i) q.splits[i] = q.splits[i - 1] + step;
    q.find_zero_idx();
    q.to_bins(v, n);
    return q;
}

// ZipML-style quantizer: start from one split per sorted value and repeatedly merge
// adjacent pairs, keeping split the bin_num/2 pairs with the largest squared error.
// (The reference loses the unpaired last split of an odd round by bumping the wrong
// counter, ZipGradient.scala:111-113; here it is kept.)
template <class T>
Quantizer<T> zipml_quantize(const T* v, size_t n, int bin_num) {
    if (n == 0) throw Error("cannot quantize an empty vector");
    std::vector<T> s(v, v + n);
    std::sort(s.begin(), s.end());
    std::vector<double> r(n), t(n);
    double a = 0, b = 0;
    for (size_t i = 0; i < n; ++i) {
        a += s[i];
        b += (double)s[i] * s[i];
        r[i] = a;
        t[i] = b;
    }
    std::vector<size_t> idx(n);
    for (size_t i = 0; i < n; ++i) idx[i] = i;
    size_t split_num = n;
    while (split_num > (size_t)bin_num) {
        size_t pairs = split_num / 2;
        std::vector<double> err(pairs);
        for (size_t i = 0; i < pairs; ++i) {
            size_t L = idx[2 * i];
            size_t R = (2 * i + 2 >= split_num ? n : idx[2 * i + 2]) - 1;
            double l1 = r[R] - (L == 0 ? 0 : r[L - 1]);
            double l2 = t[R] - (L == 0 ? 0 : t[L - 1]);
            double cnt = (double)(R - L + 1), mean = l1 / cnt;
            err[i] = l2 + mean * mean * cnt - 2 * mean * l1;
        }
        size_t odd = split_num % 2;
        size_t thr_num = (size_t)std::max<long>(1, (long)bin_num / 2 - (long)odd);
        thr_num = std::min(thr_num, pairs);
        double thr = select_kth_largest(err, thr_num);
        size_t m = 0, kept = 0;
        std::vector<size_t> nidx;
        nidx.reserve(split_num);
        for (size_t i = 0; i < pairs; ++i) {
            nidx.push_back(idx[2 * i]);
            if (err[i] >= thr && kept < thr_num) {
                nidx.push_back(idx[2 * i + 1]);
                ++kept;
            }
        }
        if (odd) nidx.push_back(idx[split_num - 1]);
        m = nidx.size();
        if (m >= split_num) break;  // no progress (all errors tie): stop
        std::copy(nidx.begin(), nidx.end(), idx.begin());
        split_num = m;
    }
    std::vector<T> raw;
    for (size_t i = 1; i < split_num; ++i) raw.push_back(s[idx[i]]);
    if (raw.empty()) raw.push_back(s[0]);
    return quantizer_from_splits<T>(raw, s.front(), s.back(), v, n);
}

// ---------------------------------------------------------------------------
// Key encoders
// ---------------------------------------------------------------------------
struct EncodedKeys {
    uint32_t size = 0;
    uint32_t num_intervals = 4;
    uint32_t flag_kind = 0;
    BitStream flags, deltas;
    uint64_t flag_bits = 0, delta_bits = 0;
};

inline void check_sorted_delta(int64_t d, size_t i) {
    if (d < 0) throw Error("keys are not sorted at position " + std::to_string(i));
}

// 2 flag bits per key (bytes - 1) and the delta in 1, 2 or 4 bytes.
inline EncodedKeys delta_binary_encode(const int32_t* keys, size_t n) {
    EncodedKeys e;
    e.size = (uint32_t)n;
    e.num_intervals = 4;
    int64_t prev = 0;
    for (size_t i = 0; i < n; ++i) {
        int64_t d = (int64_t)keys[i] - prev;
        check_sorted_delta(d, i);
        int w = skml_delta_bytes((uint32_t)d);
        e.flags.put(e.flag_bits, (uint32_t)(w - 1), 2);
        e.flag_bits += 2;
        e.deltas.put(e.delta_bits, (uint32_t)d, 8 * w);
        e.delta_bits += 8 * w;
        prev = keys[i];
    }
    e.flags.pad_to_bits(e.flag_bits);
    e.deltas.pad_to_bits(e.delta_bits);
    return e;
}

inline std::vector<int32_t> delta_binary_decode(const EncodedKeys& e) {
    std::vector<int32_t> r(e.size);
    uint64_t fo = 0, dof = 0;
    uint32_t prev = 0;
    for (uint32_t i = 0; i < e.size; ++i) {
        int w = (int)e.flags.take(fo, 2) + 1;
        fo += 2;
        prev += e.deltas.take(dof, 8 * w);
        dof += 8 * w;
        r[i] = (int32_t)prev;
    }
    return r;
}

// Chooses the interval count m in {2,4,8,16} (fallback 1) and the flag kind that
// minimise the estimated bits per key, then writes flags and deltas.
inline void adaptive_choose(const double prob[32], uint32_t& num_intervals, uint32_t& flag_kind) {
    double best = 32.0;
    num_intervals = 1;
    flag_kind = 0;
    for (int m = 2; m <= 16; m *= 2) {
        int b = 32 / m;
        double sum = 0;
        for (int i = 0; i < m; ++i) {
            double ip = 0;
            for (int j = 0; j < b; ++j) ip += prob[i * b + j];
            sum += (i + 1) * ip;
        }
        double t1 = sum * b + floor_log2((uint32_t)m);
        if (t1 < best) {
            best = t1;
            num_intervals = m;
            flag_kind = 0;
        }
        double t2 = sum * (b + 1) + 1;
        if (t2 < best) {
            best = t2;
            num_intervals = m;
            flag_kind = 1;
        }
    }
}

inline EncodedKeys delta_adaptive_encode(const int32_t* keys, size_t n) {
    EncodedKeys e;
    e.size = (uint32_t)n;
    std::vector<uint32_t> delta(n);
    std::vector<int> need(n);
    double prob[32] = {0};
    int64_t prev = 0;
    for (size_t i = 0; i < n; ++i) {
        int64_t d = (int64_t)keys[i] - prev;
        check_sorted_delta(d, i);
        delta[i] = (uint32_t)d;
        need[i] = (i == 0 && d == 0) ? 1 : floor_log2((uint32_t)d) + 1;
        prob[need[i] & 31] += 1;
        prev = keys[i];
    }
    for (double& p : prob) p /= (double)std::max<size_t>(n, 1);
    adaptive_choose(prob, e.num_intervals, e.flag_kind);
    int b = 32 / (int)e.num_intervals;
    int fb = floor_log2(e.num_intervals);
    for (size_t i = 0; i < n; ++i) {
        int iv = (need[i] + b - 1) / b;
        if (!e.flag_kind) {
            e.flags.put(e.flag_bits, (uint32_t)(iv - 1), fb);
            e.flag_bits += fb;
        } else {
            e.flags.put(e.flag_bits, (1u << (iv + 1)) - 2u, iv + 1);
            e.flag_bits += iv + 1;
        }
        e.deltas.put(e.delta_bits, delta[i], b * iv);
        e.delta_bits += (uint64_t)b * iv;
    }
    e.flags.pad_to_bits(e.flag_bits);
    e.deltas.pad_to_bits(e.delta_bits);
    return e;
}

inline std::vector<int32_t> delta_adaptive_decode(const EncodedKeys& e) {
    std::vector<int32_t> r(e.size);
    int b = 32 / (int)e.num_intervals;
    int fb = floor_log2(e.num_intervals);
    uint64_t fo = 0, dof = 0;
    uint32_t prev = 0;
    for (uint32_t i = 0; i < e.size; ++i) {
        int iv;
        if (!e.flag_kind) {
            iv = (int)e.flags.take(fo, fb) + 1;
            fo += fb;
        } else {
            iv = 0;
            while (e.flags.get(fo++)) ++iv;
        }
        prev += e.deltas.take(dof, b * iv);
        dof += (uint64_t)b * iv;
        r[i] = (int32_t)prev;
    }
    return r;
}

inline std::vector<int32_t> decode_keys(const EncodedKeys& e, uint32_t encoder) {
    return encoder == SKML_KEYS_DELTA_BINARY ? delta_binary_decode(e) : delta_adaptive_decode(e);
}

// ---------------------------------------------------------------------------
// Huffman code over an int array (used for MinMaxSketch tables on the wire)
// ---------------------------------------------------------------------------
struct HuffItem {
    int32_t value;
    uint32_t bits;
    int32_t num_bits;
};
struct HuffmanCode {
    std::vector<HuffItem> items;  // ascending by value
    BitStream bits;
    uint64_t nbits = 0;
    uint32_t size = 0;
};

inline HuffmanCode huffman_encode(const int32_t* v, size_t n) {
    HuffmanCode h;
    h.size = (uint32_t)n;
    if (n == 0) return h;
    std::map<int32_t, uint64_t> freq;
    for (size_t i = 0; i < n; ++i) ++freq[v[i]];
    struct Node {
        uint64_t count;
        int left, right;
        int32_t value;
    };
    std::vector<Node> nodes;
    typedef std::pair<uint64_t, int> QI;  // (count, node id): ties resolved by creation order
    std::priority_queue<QI, std::vector<QI>, std::greater<QI>> heap;
    for (auto& kv : freq) {
        nodes.push_back({kv.second, -1, -1, kv.first});
        heap.push({kv.second, (int)nodes.size() - 1});
    }
    while (heap.size() > 1) {
        QI x = heap.top();
        heap.pop();
        QI y = heap.top();
        heap.pop();
        nodes.push_back({x.first + y.first, x.second, y.second, -1});
        heap.push({x.first + y.first, (int)nodes.size() - 1});
    }
    std::map<int32_t, HuffItem> table;
    std::function<void(int, uint32_t, int)> walk = [&](int id, uint32_t bits, int depth) {
        const Node& nd = nodes[id];
        if (nd.left < 0) {
            table[nd.value] = {nd.value, bits, depth == 0 ? 1 : depth};
            return;
        }
        if (depth >= 31) throw Error("Huffman code longer than 31 bits");
        walk(nd.left, bits << 1, depth + 1);
        walk(nd.right, (bits << 1) | 1u, depth + 1);
    };
    walk(heap.top().second, 0, 0);
    for (auto& kv : table) h.items.push_back(kv.second);
    for (size_t i = 0; i < n; ++i) {
        const HuffItem& it = table[v[i]];
        h.bits.put(h.nbits, it.bits, it.num_bits);
        h.nbits += it.num_bits;
    }
    h.bits.pad_to_bits(h.nbits);
    return h;
}

inline std::vector<int32_t> huffman_decode(const HuffmanCode& h) {
    std::vector<int32_t> r(h.size);
    if (h.size == 0) return r;
    struct Node {
        int child[2] = {-1, -1};
        bool leaf = false;
        int32_t value = 0;
    };
    std::vector<Node> nodes(1);
    for (const HuffItem& it : h.items) {
        int cur = 0;
        for (int i = it.num_bits - 1; i >= 0; --i) {
            int bit = (it.bits >> i) & 1u;
            if (nodes[cur].child[bit] < 0) {
                nodes[cur].child[bit] = (int)nodes.size();
                nodes.emplace_back();
            }
            cur = nodes[cur].child[bit];
        }
        nodes[cur].leaf = true;
        nodes[cur].value = it.value;
    }
    uint64_t idx = 0;
    int cur = 0;
    uint32_t cnt = 0;
    uint64_t limit = (uint64_t)h.bits.words.size() * 64 + 64;
    while (cnt < h.size) {
        if (idx > limit) throw Error("Huffman stream ended early");
        cur = nodes[cur].child[h.bits.get(idx++) ? 1 : 0];
        if (cur < 0) throw Error("invalid Huffman stream");
        if (nodes[cur].leaf) {
            r[cnt++] = nodes[cur].value;
            cur = 0;
        }
    }
    return r;
}

// ---------------------------------------------------------------------------
// MinMaxSketch: insert keeps the bucket closest to the zero bucket, query returns
// the furthest among the rows.
// tie_mode 0: first inserted wins a tie (sequential reference behaviour);
// tie_mode 1: the lower bucket wins (order independent; what the GPU's atomicMin does).
// ---------------------------------------------------------------------------
struct MinMaxSketch {
    int rows = 0, cols = 0, zero = 0, tie_mode = 1;
    uint8_t hash_ids[8] = {0};
    std::vector<int32_t> table;  // INT32_MAX = never written

    MinMaxSketch() {}
    MinMaxSketch(int rows_, int cols_, int zero_, const uint8_t* ids, int tie)
        : rows(rows_), cols(cols_), zero(zero_), tie_mode(tie), table((size_t)rows_ * cols_, INT32_MAX) {
        if (rows_ > 8) throw Error("Currently only 8 hash functions are available");
        for (int i = 0; i < 8; ++i) hash_ids[i] = ids[i];
    }
    int64_t dist(int32_t v) const {
        if (v == INT32_MAX) return (int64_t)1 << 40;
        int64_t d = (int64_t)v - zero;
        return d < 0 ? -d : d;
    }
    void insert(int32_t key, int32_t bin) {
        for (int i = 0; i < rows; ++i) {
            size_t idx = (size_t)i * cols + skml_hash(hash_ids[i], key, cols);
            int64_t dn = dist(bin), dc = dist(table[idx]);
            if (dn < dc || (tie_mode == 1 && dn == dc && bin < table[idx])) table[idx] = bin;
        }
    }
    int32_t query(int32_t key) const {
        int32_t res = zero;
        for (int i = 0; i < rows; ++i) {
            int32_t c = table[(size_t)i * cols + skml_hash(hash_ids[i], key, cols)];
            if (c == INT32_MAX) continue;  // never reached for a key that was inserted
            if (dist(c) > dist(res)) res = c;
        }
        return res;
    }
};

struct SketchOptions {
    int bin_num = 256, group_num = 8, row_num = 2;
    double col_ratio = 0.3;
    int key_encoder = SKML_KEYS_DELTA_BINARY;
    int cell_bits = -1;  // -1 = 8 if bin_num <= 256 else 16; 32 = raw; 0 = Huffman
    int sketch_k = 128;
    int threads = 1;   // intra-worker parallelism of the CPU library (common/Constants.java:19-24)
    uint64_t seed = 0, step = 0;
    uint32_t rank = 0, world = 1;
    int offset_mode = 2;
    int tie_mode = 1;
    bool java_compat_max = false;
    bool restart = true;
    double loss_partials[4] = {0, 0, 0, 0};
};

struct GroupedSketch {
    int group_num = 0, row_num = 0, bin_num = 0, zero = 0;
    double col_ratio = 0;
    int key_encoder = 0;
    std::vector<int> edges;
    std::vector<MinMaxSketch> sketches;  // rows == 0 for an empty group
    std::vector<EncodedKeys> keys;

    void create(const int32_t* k, const int32_t* bins, size_t n, const SketchOptions& o) {
        edges.assign(group_num, 0);
        skml_group_edges(zero, bin_num, group_num, edges.data());
        std::vector<std::vector<int32_t>> gk(group_num), gb(group_num);
        for (size_t i = 0; i < n; ++i) {
            int g = skml_group_of(bins[i], edges.data(), group_num);
            gk[g].push_back(k[i]);
            gb[g].push_back(bins[i]);
        }
        sketches.assign(group_num, MinMaxSketch());
        keys.assign(group_num, EncodedKeys());
        auto build_group = [&](int g) {
            size_t sz = gk[g].size();
            if (sz == 0) return;
            int cols = (int)std::ceil((double)sz * col_ratio);
            if (cols < 1) cols = 1;
            uint8_t ids[8];
            skml_pick_hashes(o.seed, o.step, o.rank, (uint32_t)g, row_num, ids);
            sketches[g] = MinMaxSketch(row_num, cols, zero, ids, o.tie_mode);
            for (size_t j = 0; j < sz; ++j) sketches[g].insert(gk[g][j], gb[g][j]);
            keys[g] = key_encoder == SKML_KEYS_DELTA_BINARY ? delta_binary_encode(gk[g].data(), sz)
                                                            : delta_adaptive_encode(gk[g].data(), sz);
        };
        // sketch/frequency/GroupedMinMaxSketch.java:72-101 (parallelCreate): the groups are independent,
        // so with several threads every thread builds the sketches and key codes of its share of groups
        const int threads = std::max(1, std::min(o.threads, group_num));
        run_parallel(threads, [&](int t) {
            for (int g = t; g < group_num; g += threads) build_group(g);
        });
    }
    void restore(std::vector<int32_t>& k_out, std::vector<int32_t>& b_out) const {
        std::vector<std::vector<int32_t>> ks, bs;
        for (int g = 0; g < group_num; ++g) {
            if (sketches[g].rows == 0) continue;
            std::vector<int32_t> gk = decode_keys(keys[g], (uint32_t)key_encoder);
            std::vector<int32_t> gb(gk.size());
            for (size_t j = 0; j < gk.size(); ++j) gb[j] = sketches[g].query(gk[j]);
            ks.push_back(std::move(gk));
            bs.push_back(std::move(gb));
        }
        kway_merge(ks, bs, k_out, b_out);
    }
};

// ---------------------------------------------------------------------------
// SKML container
// ---------------------------------------------------------------------------
template <class T>
struct SketchGradient {
    SkmlHeader h{};
    std::vector<T> bucket_values;
    GroupedSketch sketch;             // sparse kind
    std::vector<uint16_t> dense_codes;  // dense kind: one bucket per coordinate
};

inline int resolve_cell_bits(int requested, int bin_num) {
    if (requested < 0) return bin_num <= 256 ? 8 : 16;
    if (requested == 8 && bin_num > 256) throw Error("8-bit cells need bin_num <= 256");
    return requested;
}

// Restart points of one encoded key stream (computed by replaying the stream).
inline std::vector<SkmlRestart> build_restarts(const EncodedKeys& e, uint32_t encoder, uint32_t interval) {
    std::vector<SkmlRestart> r;
    if (interval == 0) return r;
    int b = 32 / (int)e.num_intervals;
    int fb = encoder == SKML_KEYS_DELTA_BINARY ? 2 : floor_log2(e.num_intervals);
    uint64_t fo = 0, dof = 0;
    uint32_t prev = 0;
    for (uint32_t i = 0; i < e.size; ++i) {
        if (i % interval == 0) r.push_back({prev, (uint32_t)fo, dof});
        int nbits;
        if (encoder == SKML_KEYS_DELTA_BINARY) {
            nbits = 8 * ((int)e.flags.take(fo, 2) + 1);
            fo += 2;
        } else if (!e.flag_kind) {
            nbits = b * ((int)e.flags.take(fo, fb) + 1);
            fo += fb;
        } else {
            int iv = 0;
            while (e.flags.get(fo++)) ++iv;
            nbits = b * iv;
        }
        prev += e.deltas.take(dof, nbits);
        dof += nbits;
    }
    return r;
}

struct ByteWriter {
    std::vector<uint8_t> buf;
    uint64_t reserve_aligned(uint64_t nbytes) {
        uint64_t off = skml_align16(buf.size());
        buf.resize(off + nbytes, 0);
        return off;
    }
    template <class U>
    void write_at(uint64_t off, const U* p, size_t count) {
        if (count) std::memcpy(buf.data() + off, p, count * sizeof(U));
    }
    void pad16() { buf.resize(skml_align16(buf.size()), 0); }
};

template <class T>
std::vector<uint8_t> skml_serialize(const SketchGradient<T>& g, const SketchOptions& o) {
    ByteWriter w;
    SkmlHeader h = g.h;
    h.magic = SKML_MAGIC;
    h.version = SKML_VERSION;
    h.dtype = sizeof(T) == 8 ? SKML_F64 : SKML_F32;
    w.reserve_aligned(SKML_HEADER_BYTES);
    if (h.kind != SKML_KIND_EMPTY) {
        h.off_bucket_values = w.reserve_aligned(g.bucket_values.size() * sizeof(T));
        w.write_at(h.off_bucket_values, g.bucket_values.data(), g.bucket_values.size());
    }
    if (h.kind == SKML_KIND_SPARSE) {
        const GroupedSketch& s = g.sketch;
        int G = s.group_num;
        std::vector<SkmlGroupEntry> ent(G);
        std::memset(ent.data(), 0, G * sizeof(SkmlGroupEntry));
        h.off_group_table = w.reserve_aligned((uint64_t)G * sizeof(SkmlGroupEntry));
        int cb = (int)h.cell_bits;
        // tables
        h.off_tables = skml_align16(w.buf.size());
        for (int i = 0; i < G; ++i) {
            const MinMaxSketch& m = s.sketches[i];
            ent[i].n = s.keys[i].size;
            if (m.rows == 0) continue;
            ent[i].col_num = (uint32_t)m.cols;
            std::memcpy(ent[i].hash_ids, m.hash_ids, 8);
            size_t cells = m.table.size();
            if (cb == 8 || cb == 16) {
                ent[i].table_off = w.reserve_aligned(cells * (cb / 8));
                for (size_t c = 0; c < cells; ++c) {
                    uint32_t v = m.table[c] == INT32_MAX ? (uint32_t)s.zero : (uint32_t)m.table[c];
                    if (cb == 8) w.buf[ent[i].table_off + c] = (uint8_t)v;
                    else {
                        uint16_t u = (uint16_t)v;
                        std::memcpy(&w.buf[ent[i].table_off + 2 * c], &u, 2);
                    }
                }
            } else if (cb == 32) {
                ent[i].table_off = w.reserve_aligned(cells * 4);
                w.write_at(ent[i].table_off, m.table.data(), cells);
            } else {  // Huffman section: u32 num_items, items, u32 num_words, u32 size, words
                HuffmanCode hc = huffman_encode(m.table.data(), cells);
                uint64_t bytes = 16 + hc.items.size() * 12 + hc.bits.words.size() * 8;
                ent[i].table_off = w.reserve_aligned(bytes);
                uint32_t head[4] = {(uint32_t)hc.items.size(), (uint32_t)hc.bits.words.size(), hc.size, 0};
                w.write_at(ent[i].table_off, head, 4);
                uint64_t p = ent[i].table_off + 16;
                for (auto& it : hc.items) {
                    int32_t rec[3] = {it.value, (int32_t)it.bits, it.num_bits};
                    w.write_at(p, rec, 3);
                    p += 12;
                }
                w.write_at(p, hc.bits.words.data(), hc.bits.words.size());
            }
        }
        h.off_key_flags = skml_align16(w.buf.size());
        for (int i = 0; i < G; ++i) {
            if (ent[i].n == 0) continue;
            const EncodedKeys& e = s.keys[i];
            ent[i].num_intervals = e.num_intervals;
            ent[i].flag_kind = e.flag_kind;
            ent[i].n_flag_words = (uint32_t)e.flags.words.size();
            ent[i].flag_off = w.reserve_aligned(e.flags.words.size() * 8);
            w.write_at(ent[i].flag_off, e.flags.words.data(), e.flags.words.size());
        }
        h.off_key_deltas = skml_align16(w.buf.size());
        for (int i = 0; i < G; ++i) {
            if (ent[i].n == 0) continue;
            const EncodedKeys& e = s.keys[i];
            ent[i].n_delta_words = (uint32_t)e.deltas.words.size();
            ent[i].delta_off = w.reserve_aligned(e.deltas.words.size() * 8);
            w.write_at(ent[i].delta_off, e.deltas.words.data(), e.deltas.words.size());
        }
        if (o.restart) {
            h.restart_interval = SKML_RESTART_INTERVAL;
            h.off_restart = skml_align16(w.buf.size());
            for (int i = 0; i < G; ++i) {
                if (ent[i].n == 0) continue;
                auto rs = build_restarts(s.keys[i], h.key_encoder, h.restart_interval);
                ent[i].restart_off = w.reserve_aligned(rs.size() * sizeof(SkmlRestart));
                w.write_at(ent[i].restart_off, rs.data(), rs.size());
            }
        }
        w.write_at(h.off_group_table, ent.data(), ent.size());
    } else if (h.kind == SKML_KIND_DENSE) {
        int cb = (int)h.cell_bits;
        size_t n = g.dense_codes.size();
        h.off_dense_codes = w.reserve_aligned(n * (cb / 8));
        for (size_t i = 0; i < n; ++i) {
            if (cb == 8) w.buf[h.off_dense_codes + i] = (uint8_t)g.dense_codes[i];
            else std::memcpy(&w.buf[h.off_dense_codes + 2 * i], &g.dense_codes[i], 2);
        }
    }
    w.pad16();
    h.total_bytes = w.buf.size();
    h.header_checksum = skml_header_checksum(&h);
    std::memcpy(w.buf.data(), &h, sizeof(h));
    return w.buf;
}

inline void skml_validate(const uint8_t* p, size_t len, SkmlHeader& h) {
    if (len < SKML_HEADER_BYTES) throw Error("payload shorter than its header");
    std::memcpy(&h, p, sizeof(h));
    if (h.magic != SKML_MAGIC) throw Error("bad payload magic");
    if (h.version != SKML_VERSION) throw Error("unsupported payload version");
    if (h.header_checksum != skml_header_checksum(&h)) throw Error("payload header checksum mismatch");
    if (h.total_bytes > len) throw Error("payload truncated");
    if (h.group_num > SKML_MAX_GROUPS || h.row_num > SKML_MAX_ROWS) throw Error("payload header out of range");
}

template <class T>
SketchGradient<T> skml_parse(const uint8_t* p, size_t len) {
    SketchGradient<T> g;
    skml_validate(p, len, g.h);
    const SkmlHeader& h = g.h;
    if ((h.dtype == SKML_F64) != (sizeof(T) == 8)) throw Error("payload dtype mismatch");
    auto need = [&](uint64_t off, uint64_t bytes) {
        if (off + bytes > h.total_bytes) throw Error("payload section out of bounds");
    };
    if (h.kind == SKML_KIND_EMPTY) return g;
    need(h.off_bucket_values, (uint64_t)h.bin_num * sizeof(T));
    g.bucket_values.resize(h.bin_num);
    std::memcpy(g.bucket_values.data(), p + h.off_bucket_values, h.bin_num * sizeof(T));
    if (h.kind == SKML_KIND_DENSE) {
        int cb = (int)h.cell_bits;
        need(h.off_dense_codes, h.dim * (cb / 8));
        g.dense_codes.resize(h.dim);
        for (uint64_t i = 0; i < h.dim; ++i) {
            if (cb == 8) g.dense_codes[i] = p[h.off_dense_codes + i];
            else std::memcpy(&g.dense_codes[i], p + h.off_dense_codes + 2 * i, 2);
        }
        return g;
    }
    GroupedSketch& s = g.sketch;
    s.group_num = (int)h.group_num;
    s.row_num = (int)h.row_num;
    s.bin_num = (int)h.bin_num;
    s.zero = (int)h.zero_idx;
    s.col_ratio = h.col_ratio;
    s.key_encoder = (int)h.key_encoder;
    s.edges.assign(s.group_num, 0);
    skml_group_edges(s.zero, s.bin_num, s.group_num, s.edges.data());
    need(h.off_group_table, (uint64_t)h.group_num * sizeof(SkmlGroupEntry));
    std::vector<SkmlGroupEntry> ent(h.group_num);
    std::memcpy(ent.data(), p + h.off_group_table, h.group_num * sizeof(SkmlGroupEntry));
    s.sketches.assign(s.group_num, MinMaxSketch());
    s.keys.assign(s.group_num, EncodedKeys());
    int cb = (int)h.cell_bits;
    for (int i = 0; i < s.group_num; ++i) {
        const SkmlGroupEntry& e = ent[i];
        if (e.n == 0) continue;
        MinMaxSketch m((int)h.row_num, (int)e.col_num, s.zero, e.hash_ids, 1);
        size_t cells = m.table.size();
        if (cb == 8 || cb == 16) {
            need(e.table_off, cells * (cb / 8));
            for (size_t c = 0; c < cells; ++c) {
                if (cb == 8) m.table[c] = p[e.table_off + c];
                else {
                    uint16_t u;
                    std::memcpy(&u, p + e.table_off + 2 * c, 2);
                    m.table[c] = u;
                }
            }
        } else if (cb == 32) {
            need(e.table_off, cells * 4);
            std::memcpy(m.table.data(), p + e.table_off, cells * 4);
        } else {
            need(e.table_off, 16);
            uint32_t head[4];
            std::memcpy(head, p + e.table_off, 16);
            need(e.table_off, 16 + (uint64_t)head[0] * 12 + (uint64_t)head[1] * 8);
            HuffmanCode hc;
            hc.size = head[2];
            uint64_t q = e.table_off + 16;
            for (uint32_t j = 0; j < head[0]; ++j) {
                int32_t rec[3];
                std::memcpy(rec, p + q, 12);
                hc.items.push_back({rec[0], (uint32_t)rec[1], rec[2]});
                q += 12;
            }
            hc.bits.words.resize(head[1]);
            std::memcpy(hc.bits.words.data(), p + q, (size_t)head[1] * 8);
            std::vector<int32_t> t = huffman_decode(hc);
            if (t.size() != cells) throw Error("Huffman table size mismatch");
            m.table = t;
        }
        s.sketches[i] = std::move(m);
        EncodedKeys& k = s.keys[i];
        k.size = e.n;
        k.num_intervals = e.num_intervals;
        k.flag_kind = e.flag_kind;
        need(e.flag_off, (uint64_t)e.n_flag_words * 8);
        need(e.delta_off, (uint64_t)e.n_delta_words * 8);
        k.flags.words.resize(e.n_flag_words);
        std::memcpy(k.flags.words.data(), p + e.flag_off, (size_t)e.n_flag_words * 8);
        k.deltas.words.resize(e.n_delta_words);
        std::memcpy(k.deltas.words.data(), p + e.delta_off, (size_t)e.n_delta_words * 8);
    }
    return g;
}

template <class T>
SketchGradient<T> sketch_from_quantizer(const Quantizer<T>& q, const int32_t* keys, size_t n, uint64_t dim,
                                        const SketchOptions& o) {
    SketchGradient<T> g;
    g.h.kind = SKML_KIND_SPARSE;
    g.h.step = o.step;
    g.h.rank = o.rank;
    g.h.world = o.world;
    g.h.dim = dim;
    g.h.nnz = n;
    g.h.bin_num = (uint32_t)q.bin_num;
    g.h.zero_idx = (uint32_t)q.zero_idx;
    g.h.group_num = (uint32_t)o.group_num;
    g.h.row_num = (uint32_t)o.row_num;
    g.h.col_ratio = o.col_ratio;
    g.h.key_encoder = (uint32_t)o.key_encoder;
    g.h.cell_bits = (uint32_t)resolve_cell_bits(o.cell_bits, q.bin_num);
    g.h.seed = o.seed;
    g.h.min_value = (double)q.min;
    g.h.max_value = (double)q.max;
    for (int i = 0; i < 4; ++i) g.h.loss_partials[i] = o.loss_partials[i];
    g.bucket_values = q.values();
    g.sketch.group_num = o.group_num;
    g.sketch.row_num = o.row_num;
    g.sketch.bin_num = q.bin_num;
    g.sketch.zero = q.zero_idx;
    g.sketch.col_ratio = o.col_ratio;
    g.sketch.key_encoder = o.key_encoder;
    g.sketch.create(keys, q.bins.data(), n, o);
    return g;
}

template <class T>
std::vector<uint8_t> empty_payload(uint64_t dim, const SketchOptions& o) {
    SketchGradient<T> g;
    g.h.kind = SKML_KIND_EMPTY;
    g.h.step = o.step;
    g.h.rank = o.rank;
    g.h.world = o.world;
    g.h.dim = dim;
    g.h.seed = o.seed;
    for (int i = 0; i < 4; ++i) g.h.loss_partials[i] = o.loss_partials[i];
    return skml_serialize(g, o);
}

template <class T>
std::vector<uint8_t> compress_sparse(const int32_t* keys, const T* vals, size_t n, uint64_t dim,
                                     const SketchOptions& o, const std::vector<T>* given_splits = nullptr,
                                     T given_min = 0, T given_max = 0) {
    if (o.group_num < 1 || o.group_num > SKML_MAX_GROUPS) throw Error("group_num out of range");
    if (o.row_num < 1 || o.row_num > SKML_MAX_ROWS) throw Error("row_num out of range [1, 8]");
    if (o.bin_num < 2 || o.bin_num > SKML_MAX_BINS) throw Error("bin_num out of range");
    if (n == 0) return empty_payload<T>(dim, o);
    for (size_t i = 0; i < n; ++i) {
        if (keys[i] < 0 || (uint64_t)keys[i] >= dim) throw Error("key out of range");
        if (i > 0 && keys[i] <= keys[i - 1]) throw Error("keys must be strictly increasing");
    }
    Quantizer<T> q = given_splits
                         ? quantizer_from_splits<T>(*given_splits, given_min, given_max, vals, n)
                         : quantile_quantize_parallel<T>(vals, n, o.bin_num, o.sketch_k,
                                                         skml_rand(o.seed, o.step, o.rank, 0x9u), o.offset_mode,
                                                         o.java_compat_max, o.threads);
    return skml_serialize(sketch_from_quantizer<T>(q, keys, n, dim, o), o);
}

// Dense kind: quantize all `dim` values, ship one narrow bucket code per coordinate.
template <class T>
std::vector<uint8_t> compress_dense(const T* vals, size_t dim, const SketchOptions& o,
                                    const std::vector<T>* given_splits = nullptr, T given_min = 0,
                                    T given_max = 0) {
    if (dim == 0) return empty_payload<T>(0, o);
    Quantizer<T> q = given_splits
                         ? quantizer_from_splits<T>(*given_splits, given_min, given_max, vals, dim)
                         : quantile_quantize_parallel<T>(vals, dim, o.bin_num, o.sketch_k,
                                                         skml_rand(o.seed, o.step, o.rank, 0x9u), o.offset_mode,
                                                         o.java_compat_max, o.threads);
    SketchGradient<T> g;
    g.h.kind = SKML_KIND_DENSE;
    g.h.step = o.step;
    g.h.rank = o.rank;
    g.h.world = o.world;
    g.h.dim = dim;
    g.h.nnz = dim;
    g.h.bin_num = (uint32_t)q.bin_num;
    g.h.zero_idx = (uint32_t)q.zero_idx;
    g.h.cell_bits = (uint32_t)(q.bin_num <= 256 ? 8 : 16);
    g.h.seed = o.seed;
    g.h.min_value = (double)q.min;
    g.h.max_value = (double)q.max;
    for (int i = 0; i < 4; ++i) g.h.loss_partials[i] = o.loss_partials[i];
    g.bucket_values = q.values();
    g.dense_codes.resize(dim);
    for (size_t i = 0; i < dim; ++i) g.dense_codes[i] = (uint16_t)q.bins[i];
    return skml_serialize(g, o);
}

// Decode to (keys ascending, values). Dense payloads give keys 0..dim-1.
template <class T>
void decompress(const uint8_t* p, size_t len, std::vector<int32_t>& keys, std::vector<T>& vals) {
    SketchGradient<T> g = skml_parse<T>(p, len);
    keys.clear();
    vals.clear();
    if (g.h.kind == SKML_KIND_EMPTY) return;
    if (g.h.kind == SKML_KIND_DENSE) {
        keys.resize(g.h.dim);
        vals.resize(g.h.dim);
        for (uint64_t i = 0; i < g.h.dim; ++i) {
            keys[i] = (int32_t)i;
            vals[i] = g.bucket_values.at(g.dense_codes[i]);
        }
        return;
    }
    std::vector<int32_t> bins;
    g.sketch.restore(keys, bins);
    vals.resize(keys.size());
    for (size_t i = 0; i < keys.size(); ++i) vals[i] = g.bucket_values.at((size_t)bins[i]);
}

// Scales the decode values in place (how 1/workerNum averaging is applied to a
// compressed gradient without decoding it).
inline void payload_times_by(uint8_t* p, size_t len, double x) {
    SkmlHeader h;
    skml_validate(p, len, h);
    if (h.kind == SKML_KIND_EMPTY) return;
    if (h.dtype == SKML_F64) {
        double* v = reinterpret_cast<double*>(p + h.off_bucket_values);
        for (uint32_t i = 0; i < h.bin_num; ++i) v[i] *= x;
    } else {
        float* v = reinterpret_cast<float*>(p + h.off_bucket_values);
        for (uint32_t i = 0; i < h.bin_num; ++i) v[i] = (float)(v[i] * x);
    }
    h.min_value *= x;
    h.max_value *= x;
    h.header_checksum = skml_header_checksum(&h);
    std::memcpy(p, &h, sizeof(h));
}

// ---------------------------------------------------------------------------
// Big-endian field stream in the order of the reference's writeObject methods
// (GroupedMinMaxSketch -> MinMaxSketch -> hashes -> HuffmanEncoder, key encoder).
// The JVM object-stream framing around these fields is not reproduced.
// ---------------------------------------------------------------------------
struct BigEndianWriter {
    std::vector<uint8_t> b;
    void i32(int32_t v) {
        for (int s = 24; s >= 0; s -= 8) b.push_back((uint8_t)((uint32_t)v >> s));
    }
    void i64(uint64_t v) {
        for (int s = 56; s >= 0; s -= 8) b.push_back((uint8_t)(v >> s));
    }
    void f64(double d) {
        uint64_t u;
        std::memcpy(&u, &d, 8);
        i64(u);
    }
    void boolean(bool v) { b.push_back(v ? 1 : 0); }
};

template <class T>
std::vector<uint8_t> export_java_fields(const uint8_t* p, size_t len) {
    SketchGradient<T> g = skml_parse<T>(p, len);
    BigEndianWriter w;
    if (g.h.kind != SKML_KIND_SPARSE) throw Error("only sparse payloads have a reference field stream");
    const GroupedSketch& s = g.sketch;
    static const int bkdr_seed[8] = {0, 0, 0, 31, 131, 267, 1313, 13131};
    w.i32(s.group_num);
    w.i32(s.row_num);
    w.f64(s.col_ratio);
    w.i32(s.bin_num);
    w.i32(s.zero);
    for (int i = 0; i < s.group_num; ++i) {
        const MinMaxSketch& m = s.sketches[i];
        w.boolean(m.rows != 0);  // stands for "object or null"
        if (m.rows == 0) continue;
        w.i32(m.rows);
        w.i32(m.cols);
        w.i32(m.zero);
        for (int r = 0; r < m.rows; ++r) {
            w.i32(m.cols);  // Int2IntHash.size
            if (m.hash_ids[r] >= 3) w.i32(bkdr_seed[m.hash_ids[r]]);
        }
        HuffmanCode hc = huffman_encode(m.table.data(), m.table.size());
        w.i32((int32_t)hc.items.size());
        for (auto& it : hc.items) {
            w.i32(it.value);
            w.i32((int32_t)it.bits);
            w.i32(it.num_bits);
        }
        size_t nw = hc.bits.java_word_count();
        w.i32((int32_t)nw);
        for (size_t j = 0; j < nw; ++j) w.i64(hc.bits.words[j]);
        w.i32((int32_t)hc.size);
    }
    for (int i = 0; i < s.group_num; ++i) {
        const EncodedKeys& e = s.keys[i];
        w.boolean(s.sketches[i].rows != 0);
        if (s.sketches[i].rows == 0) continue;
        w.i32((int32_t)e.size);
        if (s.key_encoder == SKML_KEYS_DELTA_ADAPTIVE) {
            w.i32((int32_t)e.num_intervals);
            w.boolean(e.flag_kind != 0);
        }
        size_t nf = e.flags.java_word_count(), nd = e.deltas.java_word_count();
        w.i32((int32_t)nf);
        for (size_t j = 0; j < nf; ++j) w.i64(e.flags.words[j]);
        w.i32((int32_t)nd);
        for (size_t j = 0; j < nd; ++j) w.i64(e.deltas.words[j]);
    }
    return w.b;
}

// Quantizer wire fields (Quantizer.java:184-203): used by the dense compressor.
template <class T>
std::vector<uint8_t> export_java_quantizer(const Quantizer<T>& q) {
    BigEndianWriter w;
    w.i32(q.bin_num);
    w.i32((int32_t)q.bins.size());
    for (auto s : q.splits) w.f64((double)s);
    w.i32(q.zero_idx);
    w.f64((double)q.min);
    w.f64((double)q.max);
    w.i32((int32_t)q.bins.size());
    for (int32_t b : q.bins) {
        if (q.bin_num <= 256) w.b.push_back((uint8_t)(int8_t)(b - 128));
        else if (q.bin_num <= 65536) {
            int16_t v = (int16_t)(b - 32768);
            w.b.push_back((uint8_t)((uint16_t)v >> 8));
            w.b.push_back((uint8_t)v);
        } else w.i32(b);
    }
    return w.b;
}

// ---------------------------------------------------------------------------
// Fixed-point baseline compressor: sign bit + (num_bits-1)-bit magnitude of
// floor(|v| / ||v||_2 * max) + Bernoulli(1/2), clamped to max.
// ---------------------------------------------------------------------------
struct FixedPointCode {
    uint32_t size = 0;
    int num_bits = 8;
    double norm = 0;
    BitStream bits;
};

template <class T>
FixedPointCode fixed_point_encode(const T* v, size_t n, int num_bits, uint64_t seed) {
    if (num_bits < 2 || num_bits >= 30) throw Error("Bit num out of range: " + std::to_string(num_bits));
    FixedPointCode c;
    c.size = (uint32_t)n;
    c.num_bits = num_bits;
    double nn = 0;
    for (size_t i = 0; i < n; ++i) nn += (double)v[i] * v[i];
    c.norm = std::sqrt(nn);
    uint32_t mx = (1u << (num_bits - 1)) - 1, sign = 1u << (num_bits - 1);
    for (size_t i = 0; i < n; ++i) {
        uint32_t sigma = (uint32_t)(skml_rand(seed, 0xF1u, i, 0) & 1u);
        uint32_t x = c.norm > 0 ? (uint32_t)std::floor(std::fabs((double)v[i]) / c.norm * mx) + sigma : 0u;
        if (x > mx) x = mx;  // the reference lets this overflow into the sign bit
        if (v[i] < 0) x |= sign;
        c.bits.put((uint64_t)i * num_bits, x, num_bits);
    }
    c.bits.pad_to_bits((uint64_t)n * num_bits);
    return c;
}

template <class T>
std::vector<T> fixed_point_decode(const FixedPointCode& c) {
    std::vector<T> r(c.size);
    uint32_t mx = (1u << (c.num_bits - 1)) - 1, sign = 1u << (c.num_bits - 1);
    for (uint32_t i = 0; i < c.size; ++i) {
        uint32_t x = c.bits.take((uint64_t)i * c.num_bits, c.num_bits);
        double v = (double)(x & mx) / mx * c.norm;
        r[i] = (T)((x & sign) ? -v : v);
    }
    return r;
}

}  // namespace skml
