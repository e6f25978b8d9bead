// Input transport: a minibatch that crosses PCIe every step travels in a compact form and is
// expanded on the device into the CSR arrays the gradient kernels read.
//   column indices : ceil(log2(dim)) bits each, little-endian bit stream (value i at stream bits
//                    [i * bits, (i + 1) * bits), stream bit b = bit (b & 31) of 32-bit word b >> 5)
//   row pointers   : 32-bit (batch-local offsets)           -> 64-bit
//   labels         : 8-bit integers when every label is one -> fp32
// The reference keeps its rows on the executors and never ships them per step
// (ml/data/DataSet.scala:15-21); this format exists only for data that does not stay resident.
#include <cuda_runtime.h>
#include <stdint.h>

#include "skml_api.h"

namespace {

__global__ void __launch_bounds__(256)
unpack_batch_kernel(const unsigned int* __restrict__ packed, int bits, long long nnz, int* __restrict__ cols,
                    const int* __restrict__ rowptr32, long long rows, long long* __restrict__ rowptr,
                    const signed char* __restrict__ labels8, float* __restrict__ labels) {
    const long long gsz = (long long)gridDim.x * blockDim.x, gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned int mask = bits == 32 ? 0xFFFFFFFFu : ((1u << bits) - 1u);
    for (long long i = gid; i < nnz; i += gsz) {
        const unsigned long long bit = (unsigned long long)i * (unsigned int)bits;
        const unsigned long long w = bit >> 5;
        const unsigned int lo = packed[w], hi = packed[w + 1];  // the stream ends with two padding words
        cols[i] = (int)(__funnelshift_r(lo, hi, (unsigned int)(bit & 31)) & mask);
    }
    if (rowptr32)
        for (long long i = gid; i <= rows; i += gsz) rowptr[i] = (long long)rowptr32[i];
    if (labels8)
        for (long long i = gid; i < rows; i += gsz) labels[i] = (float)labels8[i];
}

// Variable-width column indices: value i takes 1..4 little-endian bytes, its width - 1 in two flag
// bits (16 values per 32-bit flag word); block_offsets[b] is the byte offset of value 1024 b. One
// block decodes 1024 values: 4 per thread (one flag byte), a block scan of the byte counts, then at
// most 16 bytes per thread fetched as aligned words.
__global__ void __launch_bounds__(256)
unpack_varbytes_kernel(const unsigned int* __restrict__ flags, const unsigned int* __restrict__ block_offsets,
                       const unsigned char* __restrict__ bytes, long long n, int* __restrict__ cols) {
    __shared__ unsigned int s_part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long nblocks = (n + 1023) / 1024;
    for (long long b = blockIdx.x; b < nblocks; b += gridDim.x) {
        const long long i0 = b * 1024 + 4 * threadIdx.x;
        unsigned int w[4] = {0, 0, 0, 0}, wsum = 0;
        if (i0 < n) {
            const unsigned int fb = (flags[i0 >> 4] >> (2 * (i0 & 15))) & 0xFFu;  // i0 is a multiple of 4
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i0 + u < n) {
                    w[u] = ((fb >> (2 * u)) & 3u) + 1u;
                    wsum += w[u];
                }
        }
        unsigned int inc = wsum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += t;
        }
        __syncthreads();  // s_part of the previous iteration has been read
        if (lane == 31) s_part[warp] = inc;
        __syncthreads();
        unsigned int base = block_offsets[b];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (k < warp) base += s_part[k];
        if (i0 < n) {
            const unsigned int byte0 = base + inc - wsum;
            const unsigned int* src = reinterpret_cast<const unsigned int*>(bytes) + (byte0 >> 2);
            unsigned int W[5];
#pragma unroll
            for (int t = 0; t < 5; ++t) W[t] = src[t];  // the stream ends with 24 bytes of padding
            unsigned int start = byte0 & 3u;
            int out[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const unsigned int wi = start >> 2, sh = 8u * (start & 3u);
                unsigned int lo = W[0], hi = W[1];
#pragma unroll
                for (int t = 1; t < 4; ++t)
                    if (wi == (unsigned int)t) { lo = W[t]; hi = W[t + 1]; }
                const unsigned int v = __funnelshift_r(lo, hi, sh);
                out[u] = (int)(w[u] >= 4 ? v : (v & ((1u << (8u * w[u])) - 1u)));
                start += w[u];
            }
            if (i0 + 3 < n) {
                *reinterpret_cast<int4*>(cols + i0) = make_int4(out[0], out[1], out[2], out[3]);
            } else {
                for (int u = 0; u < 4; ++u)
                    if (i0 + u < n) cols[i0 + u] = out[u];
            }
        }
    }
}

// Nibble-aligned variable width: value i takes 1..8 nibbles (lowest first), its width - 1 in 3 flag bits
// at bit 3 i of the flag stream; block_offsets[b] is the nibble offset of value 1024 b. Same structure
// as the byte-aligned kernel: 4 values per thread (12 flag bits), a block scan of the nibble counts,
// at most 32 nibbles per thread fetched as five aligned words.
__global__ void __launch_bounds__(256)
unpack_varnibbles_kernel(const unsigned int* __restrict__ flags, const unsigned int* __restrict__ block_offsets,
                         const unsigned int* __restrict__ words, long long n, int* __restrict__ cols) {
    __shared__ unsigned int s_part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long nblocks = (n + 1023) / 1024;
    for (long long b = blockIdx.x; b < nblocks; b += gridDim.x) {
        const long long i0 = b * 1024 + 4 * threadIdx.x;
        unsigned int w[4] = {0, 0, 0, 0}, wsum = 0;
        if (i0 < n) {
            const unsigned long long fb = 3ull * (unsigned long long)i0;
            const unsigned int f = __funnelshift_r(flags[fb >> 5], flags[(fb >> 5) + 1], (unsigned int)(fb & 31)) & 0xFFFu;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i0 + u < n) {
                    w[u] = ((f >> (3 * u)) & 7u) + 1u;
                    wsum += w[u];
                }
        }
        unsigned int inc = wsum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += t;
        }
        __syncthreads();  // s_part of the previous iteration has been read
        if (lane == 31) s_part[warp] = inc;
        __syncthreads();
        unsigned int base = block_offsets[b];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (k < warp) base += s_part[k];
        if (i0 < n) {
            const unsigned int nib0 = base + inc - wsum;
            const unsigned int* src = words + (nib0 >> 3);
            unsigned int W[5];
#pragma unroll
            for (int t = 0; t < 5; ++t) W[t] = src[t];  // the stream ends with padding words
            unsigned int start = nib0 & 7u;
            int out[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const unsigned int wi = start >> 3, sh = 4u * (start & 7u);
                unsigned int lo = W[0], hi = W[1];
#pragma unroll
                for (int t = 1; t < 4; ++t)
                    if (wi == (unsigned int)t) { lo = W[t]; hi = W[t + 1]; }
                const unsigned int v = __funnelshift_r(lo, hi, sh);
                out[u] = (int)(w[u] >= 8 ? v : (v & ((1u << (4u * w[u])) - 1u)));
                start += w[u];
            }
            if (i0 + 3 < n) {
                *reinterpret_cast<int4*>(cols + i0) = make_int4(out[0], out[1], out[2], out[3]);
            } else {
                for (int u = 0; u < 4; ++u)
                    if (i0 + u < n) cols[i0 + u] = out[u];
            }
        }
    }
}

__global__ void __launch_bounds__(256)
widen_kernel(const int* __restrict__ rowptr32, long long rows, long long* __restrict__ rowptr,
             const signed char* __restrict__ labels8, float* __restrict__ labels) {
    const long long gsz = (long long)gridDim.x * blockDim.x, gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (rowptr32)
        for (long long i = gid; i <= rows; i += gsz) rowptr[i] = (long long)rowptr32[i];
    if (labels8)
        for (long long i = gid; i < rows; i += gsz) labels[i] = (float)labels8[i];
}

// Undoes the per-row gap coding: every row's indices become the running sum of its gaps. One warp per
// row: 32 consecutive entries per step (coalesced), shuffle scan, carry into the next 32; in place.
__global__ void __launch_bounds__(256) row_prefix_kernel(const long long* __restrict__ rowptr, long long rows,
                                                        int* __restrict__ cols) {
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const long long lo = rowptr[r], hi = rowptr[r + 1];
        int carry = 0;
        for (long long base = lo; base < hi; base += 32) {
            const long long e = base + lane;
            int v = e < hi ? cols[e] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xFFFFFFFFu, v, o);
                if (lane >= o) v += t;
            }
            v += carry;
            if (e < hi) cols[e] = v;
            carry = __shfl_sync(0xFFFFFFFFu, v, 31);
        }
    }
}

}  // namespace

static int io_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

// Variable-width form of skml_unpack_batch: `bytes` must be 4-byte aligned and end with 24 bytes of
// padding; `cols` must be 16-byte aligned.
extern "C" int skml_unpack_batch_varbytes(const unsigned int* flags, const unsigned int* block_offsets,
                                          const unsigned char* bytes, long long nnz, int* cols, const int* rowptr32,
                                          long long rows, long long* rowptr, const signed char* labels8, float* labels,
                                          void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (nnz > 0) unpack_varbytes_kernel<<<io_sms() * 8, 256, 0, s>>>(flags, block_offsets, bytes, nnz, cols);
    if (rowptr32 || labels8) widen_kernel<<<io_sms() * 4, 256, 0, s>>>(rowptr32, rows, rowptr, labels8, labels);
    return (int)cudaGetLastError();
}

extern "C" int skml_unpack_batch(const unsigned int* packed, int bits, long long nnz, int* cols, const int* rowptr32,
                                 long long rows, long long* rowptr, const signed char* labels8, float* labels,
                                 void* stream) {
    if (bits < 1 || bits > 32) return (int)cudaErrorInvalidValue;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    unpack_batch_kernel<<<sms * 8, 256, 0, (cudaStream_t)stream>>>(packed, bits, nnz, cols, rowptr32, rows, rowptr,
                                                                   labels8, labels);
    return (int)cudaGetLastError();
}

// In place: cols[e] <- sum of cols[rowptr[r] .. e] for every row r (the inverse of the host's per-row
// gap coding). `rowptr` is the expanded 64-bit array of the same batch.
extern "C" int skml_row_prefix(const long long* rowptr, long long rows, int* cols, void* stream) {
    if (rows <= 0) return 0;
    long long blocks = (rows + 7) / 8;  // eight warps per block, one row per warp and step
    if (blocks > io_sms() * 16) blocks = io_sms() * 16;
    row_prefix_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(rowptr, rows, cols);
    return (int)cudaGetLastError();
}

// Nibble-aligned form of skml_unpack_batch_varbytes (`words`: the nibble stream as 32-bit words with
// six words of padding; `flags`: 3 bits per value with two words of padding).
extern "C" int skml_unpack_batch_varnibbles(const unsigned int* flags, const unsigned int* block_offsets,
                                            const unsigned int* words, long long nnz, int* cols, const int* rowptr32,
                                            long long rows, long long* rowptr, const signed char* labels8, float* labels,
                                            void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (nnz > 0) unpack_varnibbles_kernel<<<io_sms() * 8, 256, 0, s>>>(flags, block_offsets, words, nnz, cols);
    if (rowptr32 || labels8) widen_kernel<<<io_sms() * 4, 256, 0, s>>>(rowptr32, rows, rowptr, labels8, labels);
    return (int)cudaGetLastError();
}
