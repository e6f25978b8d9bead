// Baseline compressor "FixedPoint" on the device: b-bit sign + magnitude codes of the values of a
// sparse gradient, packed most significant bit first in java.util.BitSet order, and the inverse
// (unpack + dequantize + scatter-add of several ranks' lists).
//
// Behaviour follows ml/gradient/FixedPointGradient.scala:39-75 of the reference:
//   code = floor(|v| / ||v||_2 * (2^(b-1) - 1)) + Bernoulli(1/2), sign in the top bit,
// with two deliberate differences that the CPU oracle shares: the Bernoulli draw comes from a
// counter-based generator (so host and device produce the same codes), and a magnitude that
// the draw pushes past the maximum saturates instead of overflowing into the sign bit.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/skml_common.h"
#include "skml_api.h"

namespace {

constexpr int FP_THREADS = 256;
constexpr int FP_PARTIALS = 1024;  // blocks of the norm pass; their partial sums are added in index order

__global__ void __launch_bounds__(FP_THREADS)
fp_norm_kernel(const float* __restrict__ vals, const long long* __restrict__ n_ptr, long long n_max,
               double* __restrict__ partials) {
    long long n = *n_ptr;
    if (n > n_max) n = n_max;
    // contiguous slice per block, fixed summation order inside it: the norm is reproducible
    const long long per = (n + gridDim.x - 1) / gridDim.x;
    const long long lo = per * blockIdx.x, hi = lo + per < n ? lo + per : n;
    double s = 0.0;
    for (long long i = lo + threadIdx.x; i < hi; i += FP_THREADS) {
        const double v = (double)vals[i];
        s += v * v;
    }
    __shared__ double sh[FP_THREADS];
    sh[threadIdx.x] = s;
    __syncthreads();
    for (int o = FP_THREADS / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) partials[blockIdx.x] = sh[0];
}

__device__ __forceinline__ double fp_total_norm(const double* partials, double* sh) {
    // every block adds the same partial sums in the same order
    double s = 0.0;
    for (int i = threadIdx.x; i < FP_PARTIALS; i += FP_THREADS) s += partials[i];
    sh[threadIdx.x] = s;
    __syncthreads();
    for (int o = FP_THREADS / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    const double r = sqrt(sh[0]);
    __syncthreads();
    return r;
}

__device__ __forceinline__ uint32_t fp_code(float v, double norm, uint32_t mx, uint32_t sign, uint64_t seed, uint64_t i) {
    const uint32_t sigma = (uint32_t)(skml_rand(seed, 0xF1u, i, 0) & 1u);
    uint32_t x = norm > 0.0 ? (uint32_t)floor(fabs((double)v) / norm * (double)mx) + sigma : 0u;
    if (x > mx) x = mx;
    if (v < 0.f) x |= sign;
    return x;
}

// One thread packs 8 values into `bits` bytes (8 * bits bits), so threads never share a byte.
__global__ void __launch_bounds__(FP_THREADS)
fp_pack_kernel(const float* __restrict__ vals, const long long* __restrict__ n_ptr, long long n_max, int bits,
               uint64_t seed, const double* __restrict__ partials, unsigned char* __restrict__ codes,
               double* __restrict__ norm_out) {
    __shared__ double sh[FP_THREADS];
    const double norm = fp_total_norm(partials, sh);
    if (blockIdx.x == 0 && threadIdx.x == 0) *norm_out = norm;
    long long n = *n_ptr;
    if (n > n_max) n = n_max;
    const uint32_t mx = (1u << (bits - 1)) - 1u, sign = 1u << (bits - 1);
    const long long octets = (n + 7) / 8;
    for (long long o = (long long)blockIdx.x * FP_THREADS + threadIdx.x; o < octets; o += (long long)gridDim.x * FP_THREADS) {
        unsigned char* dst = codes + o * bits;
        uint32_t acc = 0;   // most-significant-first bit queue
        int have = 0, out = 0;
        for (int j = 0; j < 8; ++j) {
            const long long i = o * 8 + j;
            const uint32_t x = i < n ? fp_code(vals[i], norm, mx, sign, seed, (uint64_t)i) : 0u;
            // feed the code's bits in two halves so that the 32-bit queue cannot overflow (bits < 30)
            int rest = bits;
            while (rest > 0) {
                const int take = rest > 16 ? 16 : rest;
                acc = (acc << take) | ((x >> (rest - take)) & ((1u << take) - 1u));
                have += take;
                rest -= take;
                while (have >= 8) {
                    dst[out++] = skml_brev8((uint8_t)(acc >> (have - 8)));
                    have -= 8;
                }
            }
        }
    }
}

__global__ void __launch_bounds__(FP_THREADS)
fp_unpack_scatter_kernel(float* __restrict__ acc, const int* __restrict__ keys, const unsigned char* __restrict__ codes,
                         const double* __restrict__ norms, const long long* __restrict__ counts, long long key_stride,
                         long long code_stride, int lists, int bits, float* __restrict__ vals_out) {
    const uint32_t mx = (1u << (bits - 1)) - 1u, sign = 1u << (bits - 1);
    for (int l = 0; l < lists; ++l) {
        long long n = counts[l];
        if (n > key_stride) n = key_stride;
        const double norm = norms[l];
        const int* k = keys + l * key_stride;
        const unsigned char* c = codes + l * code_stride;
        for (long long i = (long long)blockIdx.x * FP_THREADS + threadIdx.x; i < n; i += (long long)gridDim.x * FP_THREADS) {
            const unsigned long long bit0 = (unsigned long long)i * bits;
            uint32_t x = 0;
            // gather the code's bits byte by byte; stream bit p is bit (p & 7) of byte p >> 3
            int got = 0;
            unsigned long long p = bit0;
            while (got < bits) {
                const uint32_t byte = skml_brev8(c[p >> 3]);      // now most significant bit first
                const int avail = 8 - (int)(p & 7);
                const int take = bits - got < avail ? bits - got : avail;
                x = (x << take) | ((byte >> (avail - take)) & ((1u << take) - 1u));
                got += take;
                p += take;
            }
            const double v = (double)(x & mx) / (double)mx * norm;
            const float f = (float)((x & sign) ? -v : v);
            if (vals_out) vals_out[l * key_stride + i] = f;
            if (acc) atomicAdd(acc + k[i], f);
        }
    }
}

int fp_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

}  // namespace

extern "C" long long skml_fixedpoint_scratch_bytes() { return (long long)FP_PARTIALS * 8; }

extern "C" long long skml_fixedpoint_code_bytes(long long n, int bits) { return (n + 7) / 8 * bits; }

extern "C" int skml_fixedpoint_pack(const float* vals, const long long* n_ptr, long long n_max, int bits,
                                    unsigned long long seed, double* scratch, unsigned char* codes, double* norm_out,
                                    void* stream) {
    if (bits < 2 || bits >= 30) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    fp_norm_kernel<<<FP_PARTIALS, FP_THREADS, 0, s>>>(vals, n_ptr, n_max, scratch);
    fp_pack_kernel<<<fp_sm_count() * 8, FP_THREADS, 0, s>>>(vals, n_ptr, n_max, bits, seed, scratch, codes, norm_out);
    return (int)cudaGetLastError();
}

extern "C" int skml_fixedpoint_unpack_scatter(float* acc, const int* keys, const unsigned char* codes,
                                              const double* norms, const long long* counts, long long key_stride,
                                              long long code_stride, int lists, int bits, float* vals_out,
                                              void* stream) {
    if (bits < 2 || bits >= 30) return (int)cudaErrorInvalidValue;
    // one launch per list, in list order: every rank adds the lists to a coordinate in the same order
    for (int l = 0; l < lists; ++l) {
        fp_unpack_scatter_kernel<<<fp_sm_count() * 8, FP_THREADS, 0, (cudaStream_t)stream>>>(
            acc, keys + (long long)l * key_stride, codes + (long long)l * code_stride, norms + l, counts + l, key_stride,
            code_stride, 1, bits, vals_out ? vals_out + (long long)l * key_stride : nullptr);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}
