// Baseline compressor "Zip" on the device: the ZipML quantizer (split points by repeated halving of
// the candidate set, keeping split the pairs whose merge would cost the largest squared error), the
// bucket codes that travel between ranks, and the inverse (code -> bucket midpoint, scatter-add of
// several ranks' lists). Nothing here reads a value back to the host: the number of non-zeros, the
// number of halving rounds and the number of buckets all stay on the device.
//
// Behaviour follows ml/gradient/ZipGradient.scala:70-129 of the reference with the one repair the CPU
// oracle shares (the unpaired last candidate of an odd round is kept; the reference bumps the wrong
// counter and loses it): sort, prefix sums of v and v^2 in double, per round the error
//   l2 + mean^2 * m - 2 * mean * l1
// of every adjacent candidate pair, the thr-th largest error as threshold, pairs at or above it
// (the first thr of them in index order) stay split. Decode value of a bucket = midpoint of its edges.
//
// The split search is one block of 1024 threads: every round is a map over the pairs, a radix select
// (12-bit digits, shared-memory histogram) and an ordered compaction, and the candidate set halves
// from round to round, so the whole search reads about two entries per value.
#include <cuda_runtime.h>
#include <stdint.h>

#include <cub/device/device_radix_sort.cuh>

#include "../common/skml_common.h"
#include "skml_api.h"

namespace {

constexpr int ZT = 1024;           // threads of the split search
constexpr int ZDIGIT = 12;         // radix-select digit
constexpr int ZBINS = 1 << ZDIGIT;
constexpr int Z_MAX_BUCKETS = 8192;     // the split and midpoint tables are staged in shared memory

struct ZScratch {
    float* sorted_in;        // values padded with +inf
    float* sorted;           // ascending
    double* r;               // prefix sums of v
    double* t;               // prefix sums of v^2
    int* idx_a;              // candidate split positions (double buffered)
    int* idx_b;
    unsigned long long* err; // order-preserving keys of the pair errors
    void* cub_temp;
    size_t cub_bytes;
};

size_t al256(size_t x) { return (x + 255) & ~(size_t)255; }

size_t cub_temp_bytes(long long n_max) {
    size_t bytes = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, bytes, (const float*)nullptr, (float*)nullptr, (int)n_max);
    return bytes;
}

size_t carve(unsigned char* base, long long n_max, ZScratch* z) {
    size_t o = 0;
    auto take = [&](size_t bytes) {
        unsigned char* p = base ? base + o : nullptr;
        o += al256(bytes);
        return p;
    };
    const size_t n = (size_t)n_max;
    float* a = reinterpret_cast<float*>(take(4 * n));
    float* b = reinterpret_cast<float*>(take(4 * n));
    double* r = reinterpret_cast<double*>(take(8 * n));
    double* t = reinterpret_cast<double*>(take(8 * n));
    int* ia = reinterpret_cast<int*>(take(4 * n));
    int* ib = reinterpret_cast<int*>(take(4 * n));
    unsigned long long* e = reinterpret_cast<unsigned long long*>(take(8 * (n / 2 + 1)));
    const size_t cb = cub_temp_bytes(n_max);
    void* ct = take(cb);
    if (z) *z = ZScratch{a, b, r, t, ia, ib, e, ct, cb};
    return o;
}

__global__ void zip_pad_kernel(const float* __restrict__ vals, const long long* __restrict__ n_ptr, long long n_max,
                               float* __restrict__ out) {
    long long n = *n_ptr;
    if (n > n_max) n = n_max;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_max; i += (long long)gridDim.x * blockDim.x)
        out[i] = i < n ? vals[i] : __int_as_float(0x7F800000);
}

// order-preserving map of a double onto an unsigned 64-bit key
__device__ __forceinline__ unsigned long long zkey(double x) {
    const unsigned long long u = (unsigned long long)__double_as_longlong(x);
    return (u >> 63) ? ~u : (u | 0x8000000000000000ull);
}

// block-wide exclusive scan of one unsigned value per thread; returns the exclusive prefix, `total` to all
__device__ __forceinline__ unsigned int zscan(unsigned int v, unsigned int* sh_warp, unsigned int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned int x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += x;
    }
    __syncthreads();  // the previous call's readers are done
    if (lane == 31) sh_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        unsigned int w = sh_warp[lane], winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int x = __shfl_up_sync(0xFFFFFFFFu, winc, o);
            if (lane >= o) winc += x;
        }
        sh_warp[lane] = winc - w;
        if (lane == 31) sh_warp[32] = winc;
    }
    __syncthreads();
    total = sh_warp[32];
    return sh_warp[warp] + inc - v;
}

// block-wide inclusive scan of one double per thread (pairwise adds in a fixed order)
__device__ __forceinline__ double zscan_double(double v, double* sh_warp, double& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    double inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc = __dadd_rn(x, inc);
    }
    __syncthreads();
    if (lane == 31) sh_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        double winc = sh_warp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double x = __shfl_up_sync(0xFFFFFFFFu, winc, o);
            if (lane >= o) winc = __dadd_rn(x, winc);
        }
        sh_warp[lane] = winc;
    }
    __syncthreads();
    total = sh_warp[31];
    return warp ? __dadd_rn(sh_warp[warp - 1], inc) : inc;
}

// meta_out: [0] buckets, [1] zero bucket, [2] halving rounds run; range_out: min, max of the values.
__global__ void __launch_bounds__(ZT, 1)
zip_splits_kernel(ZScratch z, const long long* __restrict__ n_ptr, long long n_max, int bin_num,
                  float* __restrict__ splits_out, float* __restrict__ mids_out, int* __restrict__ meta_out,
                  float* __restrict__ range_out) {
    __shared__ unsigned int hist[ZBINS];
    __shared__ unsigned long long cand[ZT];   // the last candidates of a selection, ranked directly
    __shared__ unsigned int sh_warp[33];
    __shared__ double sh_dwarp[32];
    __shared__ unsigned int sh_digit, sh_above, sh_ncand;
    __shared__ unsigned long long sh_thr;
    const int tid = threadIdx.x;
    long long n64 = *n_ptr;
    if (n64 > n_max) n64 = n_max;
    const unsigned int n = (unsigned int)n64;
    if (n == 0) {
        if (tid == 0) {
            meta_out[0] = 0;
            meta_out[1] = 0;
            meta_out[2] = 0;
        }
        return;
    }
    const float* s = z.sorted;
    // prefix sums of v and v^2, one tile of ZT values at a time (coalesced), carried from tile to tile
    {
        double carry_a = 0.0, carry_b = 0.0;
        for (unsigned int base = 0; base < n; base += ZT) {
            const unsigned int i = base + tid;
            const double v = i < n ? (double)s[i] : 0.0;
            double ta, tb;
            const double ia = zscan_double(v, sh_dwarp, ta);
            const double ib = zscan_double(__dmul_rn(v, v), sh_dwarp, tb);
            if (i < n) {
                z.r[i] = __dadd_rn(carry_a, ia);
                z.t[i] = __dadd_rn(carry_b, ib);
                z.idx_a[i] = (int)i;
            }
            carry_a = __dadd_rn(carry_a, ta);
            carry_b = __dadd_rn(carry_b, tb);
        }
    }
    __syncthreads();
    int* idx = z.idx_a;
    int* nxt = z.idx_b;
    unsigned int split_num = n, rounds = 0;
    while (split_num > (unsigned int)bin_num) {
        const unsigned int pairs = split_num / 2, odd = split_num & 1u;
        int want = bin_num / 2 - (int)odd;
        if (want < 1) want = 1;
        const unsigned int thr_num = min((unsigned int)want, pairs);
        // squared error of merging every adjacent pair of candidates
        for (unsigned int i = tid; i < pairs; i += ZT) {
            const unsigned int L = (unsigned int)idx[2 * i];
            const unsigned int R = (2 * i + 2 >= split_num ? n : (unsigned int)idx[2 * i + 2]) - 1u;
            const double l1 = __dadd_rn(z.r[R], L ? -z.r[L - 1] : 0.0);
            const double l2 = __dadd_rn(z.t[R], L ? -z.t[L - 1] : 0.0);
            const double cnt = (double)(R - L + 1u), mean = __ddiv_rn(l1, cnt);
            const double e = __dadd_rn(__dadd_rn(l2, __dmul_rn(__dmul_rn(mean, mean), cnt)), -__dmul_rn(__dmul_rn(2.0, mean), l1));
            z.err[i] = zkey(e);
        }
        __syncthreads();
        // the thr_num-th largest error: radix select, most significant digit first; once the digit that
        // holds it has at most ZT members they are gathered and ranked directly
        unsigned long long prefix = 0, mask = 0;
        unsigned int k = thr_num;
        bool found = false;
        for (int shift = 64 - ZDIGIT; shift > -ZDIGIT && !found; shift -= ZDIGIT) {
            const int sh = shift < 0 ? 0 : shift;
            const int bits = shift < 0 ? ZDIGIT + shift : ZDIGIT;
            const unsigned int dm = (1u << bits) - 1u;
            for (int i = tid; i < ZBINS; i += ZT) hist[i] = 0;
            __syncthreads();
            for (unsigned int i = tid; i < pairs; i += ZT) {
                const unsigned long long key = z.err[i];
                if ((key & mask) == prefix) atomicAdd(&hist[(unsigned int)(key >> sh) & dm], 1u);
            }
            __syncthreads();
            // thread t owns digits [4t, 4t + 4) counted from the top
            unsigned int c[4], mine = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                c[j] = hist[ZBINS - 1 - (4 * tid + j)];
                mine += c[j];
            }
            unsigned int total;
            unsigned int above = zscan(mine, sh_warp, total);
            if (above < k && k <= above + mine) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (above < k && k <= above + c[j]) {
                        sh_digit = (unsigned int)(ZBINS - 1 - (4 * tid + j));
                        sh_above = above;
                        sh_ncand = c[j];
                    }
                    above += c[j];
                }
            }
            __syncthreads();
            prefix |= (unsigned long long)sh_digit << sh;
            mask |= (unsigned long long)dm << sh;
            k -= sh_above;
            const unsigned int ncand = sh_ncand;
            __syncthreads();
            if (sh == 0) {
                found = true;   // every bit is fixed
                if (tid == 0) sh_thr = prefix;
            } else if (ncand <= ZT) {
                if (tid == 0) sh_ncand = 0;
                __syncthreads();
                for (unsigned int i = tid; i < pairs; i += ZT) {
                    const unsigned long long key = z.err[i];
                    if ((key & mask) == prefix) cand[atomicAdd(&sh_ncand, 1u)] = key;
                }
                __syncthreads();
                if ((unsigned int)tid < ncand) {
                    const unsigned long long mk = cand[tid];
                    unsigned int greater = 0, equal = 0;
                    for (unsigned int j = 0; j < ncand; ++j) {
                        greater += cand[j] > mk ? 1u : 0u;
                        equal += cand[j] == mk ? 1u : 0u;
                    }
                    if (greater < k && k <= greater + equal) sh_thr = mk;  // every such thread writes the same key
                }
                found = true;
            }
            __syncthreads();
        }
        const unsigned long long thr = sh_thr;
        // ordered compaction, one tile of ZT pairs at a time: the first thr_num pairs at or above the
        // threshold keep their second candidate
        unsigned int flagged_before = 0;
        for (unsigned int base = 0; base < pairs; base += ZT) {
            const unsigned int i = base + tid;
            const bool f = i < pairs && z.err[i] >= thr;
            unsigned int tile_total;
            const unsigned int before = flagged_before + zscan(f ? 1u : 0u, sh_warp, tile_total);
            if (i < pairs) {
                const unsigned int pos = i + min(before, thr_num);
                nxt[pos] = idx[2 * i];
                if (f && before < thr_num) nxt[pos + 1] = idx[2 * i + 1];
            }
            flagged_before += tile_total;
        }
        const unsigned int kept_total = min(flagged_before, thr_num);
        const unsigned int m = pairs + kept_total + odd;
        if (m >= split_num) break;  // no progress: stop with the current set (uniform for the block)
        if (odd && tid == 0) nxt[pairs + kept_total] = idx[split_num - 1];
        __syncthreads();
        int* sw = idx;
        idx = nxt;
        nxt = sw;
        split_num = m;
        ++rounds;
    }
    __syncthreads();
    // split values (duplicates dropped), bucket midpoints, zero bucket
    const float vmin = s[0], vmax = s[n - 1];
    const unsigned int raw = split_num > 1 ? split_num - 1 : 1u;
    // a round that cannot shrink the set any further stops the search one or two candidates early
    // (only with very few buckets): the tables hold bin_num + 2 entries for that case
    const unsigned int cap = min(raw, (unsigned int)bin_num + 1u);
    unsigned int total_distinct = 0;
    for (unsigned int base = 0; base < cap; base += ZT) {
        const unsigned int i = base + tid;
        float v = 0.f;
        bool fresh = false;
        if (i < cap) {
            v = split_num > 1 ? s[idx[i + 1]] : s[0];
            fresh = i == 0 || v != s[idx[i]];
        }
        unsigned int tile_total;
        const unsigned int pos = total_distinct + zscan(fresh ? 1u : 0u, sh_warp, tile_total);
        if (fresh) splits_out[pos] = v;
        total_distinct += tile_total;
    }
    __syncthreads();
    const unsigned int nb = total_distinct + 1u;
    for (unsigned int i = tid; i < nb; i += ZT) {
        const double left = i == 0 ? (double)vmin : (double)splits_out[i - 1];
        const double right = i + 1 == nb ? (double)vmax : (double)splits_out[i];
        mids_out[i] = (float)(0.5 * (left + right));
    }
    if (tid == 0) {
        int zero = 0;
        if (vmin > 0.f) zero = 0;
        else if (vmax < 0.f) zero = (int)nb - 1;
        else {
            while (zero < (int)nb - 1 && splits_out[zero] < 0.f) ++zero;
        }
        meta_out[0] = (int)nb;
        meta_out[1] = zero;
        meta_out[2] = (int)rounds;
        range_out[0] = vmin;
        range_out[1] = vmax;
    }
}

// bucket of every value = number of splits <= value; one or two bytes per code
__global__ void __launch_bounds__(256)
zip_code_kernel(const float* __restrict__ vals, const long long* __restrict__ n_ptr, long long n_max,
                const float* __restrict__ splits, const int* __restrict__ meta, int code_bytes,
                unsigned char* __restrict__ codes) {
    extern __shared__ float sh_splits[];
    const int nb = meta[0], ns = nb > 0 ? nb - 1 : 0;
    for (int i = threadIdx.x; i < ns; i += blockDim.x) sh_splits[i] = splits[i];
    __syncthreads();
    long long n = *n_ptr;
    if (n > n_max) n = n_max;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = vals[i];
        int lo = 0, hi = ns;  // first split > v
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (sh_splits[mid] <= v) lo = mid + 1;
            else hi = mid;
        }
        if (code_bytes == 1) codes[i] = (unsigned char)lo;
        else reinterpret_cast<unsigned short*>(codes)[i] = (unsigned short)lo;
    }
}

__global__ void __launch_bounds__(256)
zip_unpack_scatter_kernel(float* __restrict__ acc, const int* __restrict__ keys, const unsigned char* __restrict__ codes,
                          const float* __restrict__ mids, const long long* __restrict__ count, long long key_stride,
                          int code_bytes, int table_len, float* __restrict__ vals_out) {
    extern __shared__ float sh_mids[];
    for (int i = threadIdx.x; i < table_len; i += blockDim.x) sh_mids[i] = mids[i];
    __syncthreads();
    long long n = *count;
    if (n > key_stride) n = key_stride;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        unsigned int c = code_bytes == 1 ? codes[i] : reinterpret_cast<const unsigned short*>(codes)[i];
        if (c >= (unsigned int)table_len) c = table_len - 1;
        const float f = sh_mids[c];
        if (vals_out) vals_out[i] = f;
        if (acc) atomicAdd(acc + keys[i], f);
    }
}

int zip_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

}  // namespace

extern "C" long long skml_zipml_scratch_bytes(long long n_max) {
    if (n_max < 1 || n_max > 0x7FFFFFFFll) return -1;
    return (long long)carve(nullptr, n_max, nullptr);
}

extern "C" int skml_zipml_code_bytes(int bin_num) { return bin_num + 2 <= 256 ? 1 : 2; }

// entries of the split / midpoint tables of one list
extern "C" int skml_zipml_table_len(int bin_num) { return bin_num + 2; }

// vals[0..*n_ptr) -> codes (one per value), mids[bin_num + 2] (decode value of every bucket),
// meta[3] (buckets, zero bucket, rounds), range[2]. splits: bin_num + 2 floats for the split points.
extern "C" int skml_zipml_pack(const float* vals, const long long* n_ptr, long long n_max, int bin_num, void* scratch,
                               long long scratch_bytes, float* splits, float* mids, int* meta, float* range,
                               unsigned char* codes, void* stream) {
    if (bin_num < 2 || bin_num + 2 > Z_MAX_BUCKETS || n_max < 1 || n_max > 0x7FFFFFFFll) return (int)cudaErrorInvalidValue;
    ZScratch z;
    if ((long long)carve(reinterpret_cast<unsigned char*>(scratch), n_max, &z) > scratch_bytes) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    zip_pad_kernel<<<zip_sm_count() * 4, 256, 0, s>>>(vals, n_ptr, n_max, z.sorted_in);
    cudaError_t e = cub::DeviceRadixSort::SortKeys(z.cub_temp, z.cub_bytes, z.sorted_in, z.sorted, (int)n_max, 0, 32, s);
    if (e != cudaSuccess) return (int)e;
    zip_splits_kernel<<<1, ZT, 0, s>>>(z, n_ptr, n_max, bin_num, splits, mids, meta, range);
    const int cb = skml_zipml_code_bytes(bin_num);
    zip_code_kernel<<<zip_sm_count() * 4, 256, sizeof(float) * (size_t)(bin_num + 2), s>>>(vals, n_ptr, n_max, splits, meta, cb, codes);
    return (int)cudaGetLastError();
}

// One launch per list, in list order (every rank adds the lists to a coordinate in the same order).
// mids: `lists` tables of bin_num + 2 floats; codes: `lists` arrays code_stride bytes apart.
extern "C" int skml_zipml_unpack_scatter(float* acc, const int* keys, const unsigned char* codes, const float* mids,
                                         const long long* counts, long long key_stride, long long code_stride,
                                         int lists, int bin_num, float* vals_out, void* stream) {
    if (bin_num < 2 || bin_num + 2 > Z_MAX_BUCKETS) return (int)cudaErrorInvalidValue;
    const int cb = skml_zipml_code_bytes(bin_num);
    for (int l = 0; l < lists; ++l) {
        const int tl = bin_num + 2;
        zip_unpack_scatter_kernel<<<zip_sm_count() * 4, 256, sizeof(float) * (size_t)tl, (cudaStream_t)stream>>>(
            acc, keys ? keys + (long long)l * key_stride : nullptr, codes + (long long)l * code_stride,
            mids + (long long)l * tl, counts + l, key_stride, cb, tl, vals_out ? vals_out + (long long)l * key_stride : nullptr);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}
