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

}  // namespace

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
