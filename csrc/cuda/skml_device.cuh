// Device-side building blocks shared by all sm_100a kernels of this library:
// status words, bounded waits (grid barrier, flag wait, mbarrier wait), scans,
// order-preserving float keys, 1-D bulk (TMA) copies into shared memory, and
// system-scope loads/stores used on peer-mapped memory.
//
// Every wait in this file has a clock64() budget. When it runs out the kernel
// records a status word and returns normally, so the CUDA context stays usable.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "skml_common.h"

#define SKML_BLOCK 1024
#define SKML_WARPS (SKML_BLOCK / 32)

enum SkmlStatus {
    SKML_OK = 0,
    SKML_TIMEOUT_BARRIER = 1,
    SKML_TIMEOUT_PEER = 2,
    SKML_BAD_HEADER = 3,
    SKML_CAPACITY = 4,
    SKML_BAD_INPUT = 5,
};

// status word: low 8 bits = code, bits 8..31 = detail (stage, peer, ...). First error wins.
__device__ __forceinline__ void skml_set_status(unsigned int* status, unsigned int code, unsigned int detail) {
    atomicCAS(status, 0u, code | (detail << 8));
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_v4(uint4* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---------------------------------------------------------------------------
// Table positions of one key for sketches whose rows all use the three integer mixers (BJ, Mix64,
// TW: what skml_pick_hashes draws for up to three rows). Equal to skml_hash(ids[r], key, size) for
// every row and every key, with about a third of the instructions of the general routine: the three
// mixers are computed once and handed to the rows, and `x % size` is a 32-bit reciprocal
// multiplication with one correction step (q = mulhi(x, floor(2^32 / size)) is the quotient or one
// less). Java semantics: the remainder keeps the sign of the dividend and is then moved up by size.
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned int skml_recip32(unsigned int size) {
    return size <= 1u ? 0xFFFFFFFFu : (unsigned int)((1ull << 32) / size);
}
__device__ __forceinline__ bool skml_rows_are_mixers(const unsigned char* ids, int rows) {
    bool ok = true;
    for (int r = 0; r < rows; ++r) ok = ok && ids[r] < 3;
    return ok;
}
__device__ __forceinline__ int skml_java_mod(unsigned int code, unsigned int size, unsigned int recip) {
    const bool neg = (int)code < 0;
    const unsigned int a = neg ? 0u - code : code;
    unsigned int r = a - __umulhi(a, recip) * size;
    if (r >= size) r -= size;
    return (int)(neg ? (r ? size - r : 0u) : r);
}
template <int MAXR>
__device__ __forceinline__ void skml_hash_rows_mixers(const unsigned char* ids, int rows, int key, unsigned int size,
                                                      unsigned int recip, int* out) {
    const unsigned int h0 = skml_mix_bj((unsigned int)key), h1 = skml_mix_64((unsigned int)key), h2 = skml_mix_tw((unsigned int)key);
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        if (r >= rows) continue;
        const int id = ids[r];
        out[r] = skml_java_mod(id == 0 ? h0 : (id == 1 ? h1 : h2), size, recip);
    }
}

// ---------------------------------------------------------------------------
// Grid barrier for cooperative launches. bar[0] = arrival count, bar[1] = generation.
// Returns false (on every thread of the block) when the wait budget ran out.
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool skml_grid_barrier(unsigned int* bar, unsigned int nblocks, unsigned int* status,
                                                  long long budget, unsigned int stage) {
    __shared__ int s_ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        if (nblocks > 1) {
            __threadfence();
            unsigned int gen = ld_acquire_gpu(&bar[1]);
            unsigned int prev = atomicAdd(&bar[0], 1u);
            if (prev == nblocks - 1) {
                bar[0] = 0;
                __threadfence();
                st_release_gpu(&bar[1], gen + 1);
            } else {
                long long t0 = clock64();
                unsigned int ns = 20, polls = 0;
                while (ld_acquire_gpu(&bar[1]) == gen) {
                    if (clock64() - t0 > budget) {
                        ok = 0;
                        skml_set_status(status, SKML_TIMEOUT_BARRIER, stage);
                        break;
                    }
                    // a block that reported an error has left the kernel and will never arrive
                    if ((++polls & 63u) == 0 && (ld_acquire_gpu(status) & 0xFFu) != SKML_OK) {
                        ok = 0;
                        break;
                    }
                    __nanosleep(ns);
                    if (ns < 400) ns *= 2;
                }
            }
            __threadfence();
        }
        // another block may already have failed: leave as well so nobody waits alone
        if (ok && (ld_acquire_gpu(status) & 0xFFu) != SKML_OK) ok = 0;
        s_ok = ok;
    }
    __syncthreads();
    return s_ok != 0;
}

// Waits until *flag == want (system scope). Thread 0 of the block polls.
__device__ __forceinline__ bool skml_wait_flag(const unsigned long long* flag, unsigned long long want,
                                               unsigned int* status, long long budget, unsigned int detail) {
    long long t0 = clock64();
    unsigned int ns = 32;
    while (ld_acquire_sys(flag) != want) {
        if (clock64() - t0 > budget) {
            skml_set_status(status, SKML_TIMEOUT_PEER, detail);
            return false;
        }
        __nanosleep(ns);
        if (ns < 1000) ns *= 2;
    }
    return true;
}

// ---------------------------------------------------------------------------
// Order-preserving map float -> uint32 (ascending floats give ascending keys).
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned int f2ord(float f) {
    unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float ord2f(unsigned int k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

// ---------------------------------------------------------------------------
// Block-wide exclusive scan (SKML_BLOCK threads). `total` receives the block sum.
// ---------------------------------------------------------------------------
template <class T>
__device__ __forceinline__ T block_exclusive_scan(T v, T* total) {
    __shared__ T s_warp[SKML_WARPS];
    __shared__ T s_total;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        T t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();  // protects s_warp / s_total against the previous call
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        T w = lane < (int)(blockDim.x >> 5) ? s_warp[lane] : (T)0;
        T winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            T t = __shfl_up_sync(0xFFFFFFFFu, winc, o);
            if (lane >= o) winc += t;
        }
        s_warp[lane] = winc - w;
        if (lane == 31) s_total = winc;
    }
    __syncthreads();
    if (total) *total = s_total;
    return s_warp[warp] + inc - v;
}

template <class T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// Block sum of doubles; the result is valid on thread 0.
__device__ __forceinline__ double block_sum_double(double v) {
    __shared__ double s_part[SKML_WARPS];
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = 0;
    if (threadIdx.x < 32) {
        r = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.0;
        r = warp_sum(r);
    }
    return r;
}

// ---------------------------------------------------------------------------
// mbarrier + 1-D bulk copy global -> shared (the TMA engine, no tensor map, no
// multicast). Source address, destination address and size must be multiples of 16.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned int parity) {
    unsigned int ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false when the budget ran out (the caller falls back to plain loads).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned int parity, long long budget) {
    long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > budget) return false;
    }
    return true;
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, unsigned int bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------
// In-place bitonic sort of N (power of two) unsigned keys in shared memory by the
// whole block.
// ---------------------------------------------------------------------------
template <int N>
__device__ __forceinline__ void block_bitonic_sort(unsigned int* s) {
    for (int k = 2; k <= N; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < N / 2; t += blockDim.x) {
                int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));  // index with bit j cleared
                int p = i | j;
                bool up = (i & k) == 0;
                unsigned int a = s[i], b = s[p];
                if ((a > b) == up) {
                    s[i] = b;
                    s[p] = a;
                }
            }
            __syncthreads();
        }
    }
}

// Ascending sort of 2048 unsigned keys in shared memory by a block of 1024 threads.
// Every warp keeps 64 consecutive elements in registers (two per lane), so the bitonic steps
// with partner distance <= 32 are register / shuffle exchanges without a block barrier; only
// the steps with distance >= 64 go through shared memory (20 barriers instead of 66).
__device__ __forceinline__ void block_sort_2048(unsigned int* s) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int i0 = warp * 64 + lane, i1 = i0 + 32;
    unsigned int a = s[i0], b = s[i1];
    for (int k = 2; k <= 2048; k <<= 1) {
        if (k >= 128) {
            s[i0] = a;
            s[i1] = b;
            __syncthreads();
            for (int j = k >> 1; j >= 64; j >>= 1) {
                const int t = threadIdx.x;
                const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const int p = i | j;
                const bool up = (i & k) == 0;
                const unsigned int x = s[i], y = s[p];
                if ((x > y) == up) {
                    s[i] = y;
                    s[p] = x;
                }
                __syncthreads();
            }
            a = s[i0];
            b = s[i1];
        }
        if (k >= 64) {  // distance 32: both elements live in this thread
            const bool up = (i0 & k) == 0;
            if ((a > b) == up) {
                const unsigned int t = a;
                a = b;
                b = t;
            }
        }
        for (int j = (k >> 1) < 16 ? (k >> 1) : 16; j > 0; j >>= 1) {
            const unsigned int pa = __shfl_xor_sync(0xFFFFFFFFu, a, j);
            const unsigned int pb = __shfl_xor_sync(0xFFFFFFFFu, b, j);
            const bool low = (lane & j) == 0;
            const bool up0 = (i0 & k) == 0, up1 = (i1 & k) == 0;
            a = (low == up0) ? min(a, pa) : max(a, pa);
            b = (low == up1) ? min(b, pb) : max(b, pb);
        }
        __syncwarp();
    }
    s[i0] = a;
    s[i1] = b;
    __syncthreads();
}

// Number of elements of the ascending array a[0..n) that are <= x (upper bound).
__device__ __forceinline__ int upper_bound_f(const float* a, int n, float x) {
    int lo = 0, hi = n;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (a[mid] <= x) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}
__device__ __forceinline__ int upper_bound_u(const unsigned int* a, int n, unsigned int x) {
    int lo = 0, hi = n;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (a[mid] <= x) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}
__device__ __forceinline__ int lower_bound_u(const unsigned int* a, int n, unsigned int x) {
    int lo = 0, hi = n;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (a[mid] < x) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}
