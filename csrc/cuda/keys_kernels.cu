// DeltaAdaptive key encoder on the device (stand-alone kernels; the fused exchange writes the
// byte-aligned DeltaBinary form instead). Behaviour follows the reference's live key encoder,
// binary/DeltaAdaptiveEncoder.java:23-146:
//   bitsNeeded_i = floor(log2(delta_i)) + 1 (1 for a first key of 0), histogram over 1..31;
//   interval count m in {2, 4, 8, 16} (fallback 1) and fixed vs unary flags chosen by the estimated
//   bits per key; flag = need - 1 in log2(m) bits (fixed) or `need` ones and a zero (unary) with
//   need = ceil(bitsNeeded / (32 / m)); delta in (32 / m) * need bits; both most significant bit
//   first in two separate streams in java.util.BitSet order (stream bit p = bit (p & 31) of 32-bit
//   word p >> 5).
// The per-key bit offsets are prefix sums the caller computes between the kernels (inclusive sums
// of the width arrays), so every kernel here is a map over keys or words.
#include <cuda_runtime.h>
#include <stdint.h>

#include "skml_api.h"

namespace {

constexpr int KT = 256;

__device__ __forceinline__ int da_need(const int* keys, long long i, unsigned int* delta_out, bool* bad) {
    const long long prev = i ? (long long)keys[i - 1] : 0ll;
    const long long d = (long long)keys[i] - prev;
    if (d < 0 || (d == 0 && i > 0) || keys[i] < 0) *bad = true;
    *delta_out = (unsigned int)d;
    return d <= 0 ? 1 : 32 - __clz((unsigned int)d);
}

__global__ void __launch_bounds__(KT) da_analyze_kernel(const int* __restrict__ keys, long long n,
                                                       unsigned int* __restrict__ hist, unsigned int* __restrict__ status) {
    __shared__ unsigned int s_h[32];
    if (threadIdx.x < 32) s_h[threadIdx.x] = 0;
    __syncthreads();
    bool bad = false;
    for (long long i = (long long)blockIdx.x * KT + threadIdx.x; i < n; i += (long long)gridDim.x * KT) {
        unsigned int d;
        const int need = da_need(keys, i, &d, &bad);
        atomicAdd(&s_h[need & 31], 1u);
    }
    __syncthreads();
    if (threadIdx.x < 32 && s_h[threadIdx.x]) atomicAdd(&hist[threadIdx.x], s_h[threadIdx.x]);
    if (bad) atomicOr(status, 1u);  // keys not strictly increasing (or negative)
}

// One thread: the reference's mode search in the same double arithmetic, operation by operation
// (explicit round-to-nearest intrinsics keep the compiler from fusing multiply-adds).
__global__ void da_choose_kernel(const unsigned int* __restrict__ hist, long long n, unsigned int* __restrict__ params) {
    if (blockIdx.x || threadIdx.x) return;
    double prob[32];
    const double dn = (double)(n > 0 ? n : 1);
    for (int k = 0; k < 32; ++k) prob[k] = __ddiv_rn((double)hist[k], dn);
    double best = 32.0;
    unsigned int num = 1, kind = 0;
    for (int m = 2, lg = 1; m <= 16; m *= 2, ++lg) {
        const int b = 32 / m;
        double sum = 0.0;
        for (int i = 0; i < m; ++i) {
            double ip = 0.0;
            for (int j = 0; j < b; ++j) ip = __dadd_rn(ip, prob[i * b + j]);
            sum = __dadd_rn(sum, __dmul_rn((double)(i + 1), ip));
        }
        const double t1 = __dadd_rn(__dmul_rn(sum, (double)b), (double)lg);
        if (t1 < best) {
            best = t1;
            num = (unsigned int)m;
            kind = 0;
        }
        const double t2 = __dadd_rn(__dmul_rn(sum, (double)(b + 1)), 1.0);
        if (t2 < best) {
            best = t2;
            num = (unsigned int)m;
            kind = 1;
        }
    }
    params[0] = num;
    params[1] = kind;
}

__global__ void __launch_bounds__(KT) da_widths_kernel(const int* __restrict__ keys, long long n,
                                                      const unsigned int* __restrict__ params, int* __restrict__ flag_w,
                                                      int* __restrict__ delta_w) {
    const int m = (int)params[0], kind = (int)params[1];
    const int b = 32 / m, fb = 31 - __clz(m);
    bool bad = false;
    for (long long i = (long long)blockIdx.x * KT + threadIdx.x; i < n; i += (long long)gridDim.x * KT) {
        unsigned int d;
        const int iv = (da_need(keys, i, &d, &bad) + b - 1) / b;
        flag_w[i] = kind ? iv + 1 : fb;
        delta_w[i] = b * iv;
    }
}

// Writes `nb` (<= 32) bits of `value`, most significant first, at stream offset `off`.
__device__ __forceinline__ void put_bits(unsigned int* words, unsigned long long off, unsigned int value, int nb) {
    if (nb <= 0) return;
    const unsigned int rv = __brev(value) >> (32 - nb);  // stream order: bit j of rv is stream bit off + j
    const unsigned int sh = (unsigned int)(off & 31);
    const unsigned long long w = off >> 5;
    atomicOr(words + w, rv << sh);
    if (sh + nb > 32) atomicOr(words + w + 1, rv >> (32 - sh));
}

// Reads `nb` (<= 32) bits at stream offset `off` as a most-significant-first value. The word after
// the last one that holds data must be readable.
__device__ __forceinline__ unsigned int take_bits(const unsigned int* words, unsigned long long off, int nb) {
    if (nb <= 0) return 0u;
    const unsigned long long w = off >> 5;
    const unsigned int x = __funnelshift_r(words[w], words[w + 1], (unsigned int)(off & 31));
    return __brev(x << (32 - nb));
}

__global__ void __launch_bounds__(KT) da_pack_kernel(const int* __restrict__ keys, long long n,
                                                    const unsigned int* __restrict__ params,
                                                    const long long* __restrict__ flag_incl,
                                                    const long long* __restrict__ delta_incl, unsigned int* flag_words,
                                                    unsigned int* delta_words) {
    const int m = (int)params[0], kind = (int)params[1];
    const int b = 32 / m, fb = 31 - __clz(m);
    bool bad = false;
    for (long long i = (long long)blockIdx.x * KT + threadIdx.x; i < n; i += (long long)gridDim.x * KT) {
        unsigned int d;
        const int iv = (da_need(keys, i, &d, &bad) + b - 1) / b;
        const int fw = kind ? iv + 1 : fb, dw = b * iv;
        const unsigned int fv = kind ? ((1u << (iv + 1)) - 2u) : (unsigned int)(iv - 1);
        put_bits(flag_words, (unsigned long long)(flag_incl[i] - fw), fv, fw);
        put_bits(delta_words, (unsigned long long)(delta_incl[i] - dw), d, dw);
    }
}

// Decode, fixed flags: interval count of every key.
__global__ void __launch_bounds__(KT) da_fixed_iv_kernel(const unsigned int* __restrict__ flag_words, long long n, int fb,
                                                        int* __restrict__ iv) {
    for (long long i = (long long)blockIdx.x * KT + threadIdx.x; i < n; i += (long long)gridDim.x * KT)
        iv[i] = (int)take_bits(flag_words, (unsigned long long)i * fb, fb) + 1;
}

// Decode, unary flags: zero bits per 32-bit word (a key's flag ends at its zero bit).
__global__ void __launch_bounds__(KT) da_zero_count_kernel(const unsigned int* __restrict__ flag_words, long long flag_bits,
                                                          int* __restrict__ zeros) {
    const long long nw = (flag_bits + 31) >> 5;
    for (long long w = (long long)blockIdx.x * KT + threadIdx.x; w < nw; w += (long long)gridDim.x * KT) {
        const long long rest = flag_bits - (w << 5);
        const unsigned int valid = rest >= 32 ? 0xFFFFFFFFu : ((1u << rest) - 1u);
        zeros[w] = __popc(~flag_words[w] & valid);
    }
}

// Stream position of the i-th zero bit (= end of key i's flag).
__global__ void __launch_bounds__(KT) da_zero_pos_kernel(const unsigned int* __restrict__ flag_words, long long flag_bits,
                                                        const long long* __restrict__ zeros_incl, long long n,
                                                        long long* __restrict__ pos) {
    const long long nw = (flag_bits + 31) >> 5;
    for (long long w = (long long)blockIdx.x * KT + threadIdx.x; w < nw; w += (long long)gridDim.x * KT) {
        const long long rest = flag_bits - (w << 5);
        const unsigned int valid = rest >= 32 ? 0xFFFFFFFFu : ((1u << rest) - 1u);
        unsigned int z = ~flag_words[w] & valid;
        long long idx = zeros_incl[w] - __popc(z);
        while (z) {
            const int bit = __ffs(z) - 1;
            z &= z - 1;
            if (idx < n) pos[idx] = (w << 5) + bit;
            ++idx;
        }
    }
}

__global__ void __launch_bounds__(KT) da_extract_kernel(const unsigned int* __restrict__ delta_words, long long n,
                                                       const int* __restrict__ delta_w,
                                                       const long long* __restrict__ delta_incl,
                                                       long long* __restrict__ deltas) {
    for (long long i = (long long)blockIdx.x * KT + threadIdx.x; i < n; i += (long long)gridDim.x * KT) {
        const int dw = delta_w[i];
        deltas[i] = (long long)take_bits(delta_words, (unsigned long long)(delta_incl[i] - dw), dw);
    }
}

int grid_for(long long n) {
    long long g = (n + KT - 1) / KT;
    if (g < 1) g = 1;
    if (g > 148 * 16) g = 148 * 16;
    return (int)g;
}

}  // namespace

extern "C" int skml_da_analyze(const int* keys, long long n, unsigned int* hist32, unsigned int* params,
                               unsigned int* status, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(hist32, 0, 32 * sizeof(unsigned int), s);
    if (e != cudaSuccess) return (int)e;
    if (n > 0) da_analyze_kernel<<<grid_for(n), KT, 0, s>>>(keys, n, hist32, status);
    da_choose_kernel<<<1, 32, 0, s>>>(hist32, n, params);
    return (int)cudaGetLastError();
}

extern "C" int skml_da_widths(const int* keys, long long n, const unsigned int* params, int* flag_w, int* delta_w,
                              void* stream) {
    if (n > 0) da_widths_kernel<<<grid_for(n), KT, 0, (cudaStream_t)stream>>>(keys, n, params, flag_w, delta_w);
    return (int)cudaGetLastError();
}

extern "C" int skml_da_pack(const int* keys, long long n, const unsigned int* params, const long long* flag_incl,
                            const long long* delta_incl, unsigned int* flag_words, unsigned int* delta_words,
                            void* stream) {
    if (n > 0)
        da_pack_kernel<<<grid_for(n), KT, 0, (cudaStream_t)stream>>>(keys, n, params, flag_incl, delta_incl, flag_words,
                                                                     delta_words);
    return (int)cudaGetLastError();
}

extern "C" int skml_da_fixed_iv(const unsigned int* flag_words, long long n, int flag_bits_per_key, int* iv, void* stream) {
    if (flag_bits_per_key < 0 || flag_bits_per_key > 4) return (int)cudaErrorInvalidValue;
    if (n > 0) da_fixed_iv_kernel<<<grid_for(n), KT, 0, (cudaStream_t)stream>>>(flag_words, n, flag_bits_per_key, iv);
    return (int)cudaGetLastError();
}

extern "C" int skml_da_zero_count(const unsigned int* flag_words, long long flag_bits, int* zeros, void* stream) {
    if (flag_bits > 0)
        da_zero_count_kernel<<<grid_for((flag_bits + 31) >> 5), KT, 0, (cudaStream_t)stream>>>(flag_words, flag_bits, zeros);
    return (int)cudaGetLastError();
}

extern "C" int skml_da_zero_pos(const unsigned int* flag_words, long long flag_bits, const long long* zeros_incl,
                                long long n, long long* pos, void* stream) {
    if (flag_bits > 0)
        da_zero_pos_kernel<<<grid_for((flag_bits + 31) >> 5), KT, 0, (cudaStream_t)stream>>>(flag_words, flag_bits,
                                                                                           zeros_incl, n, pos);
    return (int)cudaGetLastError();
}

extern "C" int skml_da_extract(const unsigned int* delta_words, long long n, const int* delta_w,
                               const long long* delta_incl, long long* deltas, void* stream) {
    if (n > 0) da_extract_kernel<<<grid_for(n), KT, 0, (cudaStream_t)stream>>>(delta_words, n, delta_w, delta_incl, deltas);
    return (int)cudaGetLastError();
}
