// Building blocks of the fused decode + aggregate + update kernel (decode_kernels.cu): kernel
// parameters, the (rank, group) work item, the sketch query, the one-barrier block scan and the
// decode of one 1024-key chunk.
//
// Reference behaviour restated (paths inside the reference project):
//   sketch/.../binary/DeltaBinaryEncoder.java:42-53 (key decode),
//   sketch/.../sketch/frequency/MinMaxSketch.java:64-73, GroupedMinMaxSketch.java:123-146 (query),
//   ml/.../gradient/SketchGradient.scala:57-68 (dequantize).
#pragma once
#include <math.h>

#include "skml_api.h"
#include "skml_device.cuh"

#define DEC_MAX_ITEMS (SKML_MAX_PEERS * SKML_MAX_GROUPS)
#define DEC_KPT 4        // keys of a 1024-key chunk per thread
#define DEC_THREADS (SKML_RESTART_INTERVAL / DEC_KPT)
// Blocks per SM: three blocks of 256 threads with a 36 KB table area each keep the SM's shared-memory
// carve-out at 164 KB, which leaves 92 KB of L1. The apply passes are random read-modify-writes whose
// number in flight grows with the L1 (every miss holds a line): measured on eight payloads of 433k keys,
// four blocks (28 KB of L1) took 218 us per launch, three blocks 175 us; lazy Adam 624 -> 445 us.
#ifndef DEC_BLOCKS_PER_SM
#define DEC_BLOCKS_PER_SM 3
#endif
#define DEC_HUF_MAX_ITEMS 513  // code words of one Huffman-coded table the expander accepts
// Most key ranges a block takes in the key-range-owned apply (dealt in snake order; sizes the slice
// table in shared memory). Measured at eight payloads of 433k keys: two ranges per block even out the
// blocks' finishing times (last block 38 us -> 7 us after the first) but not the SGD launch (175 us either
// way), so SGD takes one; lazy Adam, which sweeps its range 2 x ranks times, takes two (-4 %).
#ifndef DEC_OWN_RANGES
#define DEC_OWN_RANGES 2
#endif
#ifndef DEC_TAB_SMEM
#define DEC_TAB_SMEM 36864   // bytes of shared memory per block for a staged sketch table
#endif

struct DP {
    const unsigned char* payload[SKML_MAX_PEERS];
    const unsigned long long* flag[SKML_MAX_PEERS];
    int world;
    long long slot_capacity;
    unsigned long long step;
    long long dim;
    float* w;
    float* adam_m;
    float* adam_v;
    long long adam_stride;  // elements between the moments of neighbouring coordinates (4: packed {m, v, sum, -} quads)
    float* fsum;            // lazy Adam: float sum of the ranks' values per coordinate, all zero between calls
    long long fsum_stride;
    float lr, adam_scale;
    long long* acc;
    int* key_scratch;
    float* val_scratch;
    long long key_capacity;
    double* loss_out;
    float* out_sum;
    unsigned int* ctrl;
    unsigned int* status;
    long long budget;
    int max_items;
    int tab_off;     // byte offset of the staged-table area inside the dynamic shared memory (0 = none)
    unsigned char* tab_scratch;   // expanded Huffman-coded tables (null: such payloads are refused)
    long long tab_capacity;
    double* wsq;       // running sum of squares of the weights (null: not kept)
    double* reg_out;   // receives reg_lambda * sqrt(*wsq) when the launch ends
    double reg_lambda;
};

struct DecItem {  // one (rank, group) key stream
    const unsigned char* base;
    SkmlGroupEntry e;
    unsigned long long chunk_prefix, key_prefix;
    unsigned int zero, cell_bits, rows;
    unsigned int recip;       // floor(2^32 / col_num) for the mixer-only hash path
    unsigned long long off_bv;
    unsigned long long col_magic;
    int mixers;               // every row uses one of the three integer mixers (at most three rows)
    unsigned int enc;         // key encoder of the item's payload (SkmlKeyEncoder)
    const unsigned char* tab; // the sketch table as 8/16-bit bucket codes: inside the payload, or expanded from its Huffman form
    unsigned int huffman;     // the payload carries the table Huffman-coded (expanded into the scratch before the decode)
};


__device__ __forceinline__ long long to_fixed(double v, int shift) { return __double2ll_rn(ldexp(v, shift)); }
__device__ __forceinline__ double from_fixed(long long a, int shift) { return ldexp((double)a, -shift); }

// Both return new^2 - old^2 of the weight they changed (0 when they write the plain sum instead): the
// callers add these up so that the squared norm of the model is kept current without a pass over it.
__device__ __forceinline__ float apply_one(const DP& p, long long k, float g) {
    if (p.out_sum) {
        p.out_sum[k] = g;
        return 0.f;
    }
    const float old = p.w[k];
    float nw;
    if (!p.adam_v) {
        nw = old - p.lr * g;
    } else {
        const long long q = k * p.adam_stride;
        float mt = 0.9f * p.adam_m[q] + 0.1f * g;
        float vt = 0.999f * p.adam_v[q] + 0.001f * g * g;
        nw = old - p.lr * p.adam_scale * mt / (sqrtf(vt) + 1e-8f);
        p.adam_m[q] = mt;
        p.adam_v[q] = vt;
    }
    p.w[k] = nw;
    return (nw - old) * (nw + old);
}

// Linear modes: SGD step on w, or accumulation of the plain mean into out_sum.
__device__ __forceinline__ float apply_direct(const DP& p, long long k, float g) {
    if (p.out_sum) {
        p.out_sum[k] += g;
        return 0.f;
    }
    const float old = p.w[k], nw = old - p.lr * g;
    p.w[k] = nw;
    return (nw - old) * (nw + old);
}

// Query of one key in its group's sketch: the bucket value of the cell farthest from the zero bucket.
template <int MAXR>
__device__ __forceinline__ float query_one(const DP& p, const DecItem& it, unsigned int key, const unsigned char* stab) {
    const int col = (int)it.e.col_num;
    const int zero = (int)it.zero;
    int cells[MAXR];
    int pos[MAXR];
    const int rows = (int)it.rows;
    if (it.mixers) skml_hash_rows_mixers<(MAXR < 3 ? MAXR : 3)>(it.e.hash_ids, rows, (int)key, (unsigned int)col, it.recip, pos);
    else skml_hash_rows<MAXR>(it.e.hash_ids, rows, (int)key, col, it.col_magic, pos);
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {  // independent loads first
        cells[r] = zero;
        if (r < rows) {
            const unsigned int c = (unsigned int)r * (unsigned int)col + (unsigned int)pos[r];  // rows * col < 2^31 (checked in prepare)
            if (stab) {  // the group's whole table sits in shared memory
                if (it.cell_bits == 8) cells[r] = stab[c];
                else cells[r] = reinterpret_cast<const unsigned short*>(stab)[c];
            } else if (it.cell_bits == 8) {
                cells[r] = __ldcg(it.tab + c);
            } else {
                cells[r] = __ldcg(reinterpret_cast<const unsigned short*>(it.tab) + c);
            }
        }
    }
    int res = zero, best = 0;
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        int d = cells[r] - zero;
        if (d < 0) d = -d;
        if (d > best) {
            best = d;
            res = cells[r];
        }
    }
    // Bucket values (<= 16 KB per payload, read by every key) go through L1: the SM cannot hold a stale
    // line of them, because it first touches a payload after the arrival flag was acquired and L1 is
    // invalidated between dependent grids. Everything else of the payload is read once: L2 only.
    return reinterpret_cast<const float*>(it.base + it.off_bv)[res];
}

// Exclusive prefix sum over the block with ONE barrier: every warp publishes its total, every
// thread adds up the totals of the warps before it. The caller alternates `part` between calls
// so that no second barrier is needed to protect it.
__device__ __forceinline__ unsigned int dec_scan(unsigned int v, unsigned int* part) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) part[warp] = inc;
    __syncthreads();
    unsigned int base = 0;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w)
        if (w < warp) base += part[w];
    return base + inc - v;
}

// Decode of one 1024-key chunk of a (rank, group) key stream by the whole block (DEC_THREADS
// threads, DEC_KPT adjacent keys each; restart points make chunks independent): flag bits -> delta
// widths -> block scan -> delta bytes gathered from aligned words -> block scan -> keys; then the
// sketch query and the bucket value of every key. `part_a` / `part_b` are two scan scratch rows
// (DEC_THREADS / 32 words each) that the caller alternates between consecutive chunks, so that no
// extra barrier is needed between chunks. All threads of the block must call this together.
struct ChunkKeys {
    unsigned int i0;              // index inside the chunk of this thread's first key
    unsigned int cnt;             // keys in the chunk
    unsigned int first;           // index inside the list of the chunk's first key
    unsigned int keys[DEC_KPT];
    unsigned int d0;              // delta of keys[0]: keys[0] - d0 is the key before it in the list
    float bv[DEC_KPT];            // dequantized values (not yet divided by the world size)
    bool live[DEC_KPT];           // key exists and is inside [0, dim)
};

__device__ __forceinline__ void decode_chunk(const DP& p, const DecItem& it, unsigned int j, const unsigned char* stab,
                                             unsigned int* part_a, unsigned int* part_b, unsigned int* part_c,
                                             unsigned short* s_pos, ChunkKeys& o) {
    const unsigned int first = j * SKML_RESTART_INTERVAL;
    const unsigned int cnt = min((unsigned int)SKML_RESTART_INTERVAL, it.e.n - first);
    const SkmlRestart rs = *reinterpret_cast<const SkmlRestart*>(it.base + it.e.restart_off + 16ull * j);
    const unsigned int i0 = DEC_KPT * threadIdx.x;
    o.i0 = i0;
    o.cnt = cnt;
    o.first = first;
    unsigned int d[DEC_KPT];
#pragma unroll
    for (int u = 0; u < DEC_KPT; ++u) d[u] = 0;
    if (it.enc == SKML_KEYS_DELTA_BINARY) {
        unsigned int w[DEC_KPT];
        unsigned int wsum = 0;
    #pragma unroll
        for (int u = 0; u < DEC_KPT; ++u) w[u] = 0;
        if (i0 < cnt) {
            // the flags of DEC_KPT adjacent keys are 2 * DEC_KPT adjacent bits of one 32-bit word
            const unsigned long long fb = (unsigned long long)rs.flag_bit_off + 2ull * i0;
            const unsigned int word = __ldcg(reinterpret_cast<const unsigned int*>(it.base + it.e.flag_off) + (fb >> 5));
            const unsigned int b = word >> (fb & 31);
    #pragma unroll
            for (int u = 0; u < DEC_KPT; ++u) {
                if (i0 + u < cnt) {
                    const unsigned int bb = (b >> (2 * u)) & 3u;
                    unsigned int wu = (((bb & 1u) << 1) | (bb >> 1)) + 1u;  // stream order is most significant bit first
                    if (wu == 3) wu = 4;                                     // flag value 2 is never written
                    w[u] = wu;
                    wsum += wu;
                }
            }
        }
        const unsigned int boff = dec_scan(wsum, part_a);
        if (i0 < cnt) {
            const unsigned long long byte0 = (rs.delta_bit_off >> 3) + boff;
            if (byte0 + wsum <= 8ull * it.e.n_delta_words) {
                // The thread's <= 4 * DEC_KPT delta bytes sit in at most DEC_KPT + 1 aligned words.
                // Bit-reversing a little-endian word yields its four stream bytes in most-significant-
                // first order (java.util.BitSet order), so a delta is a funnel shift away.
                const unsigned int* src = reinterpret_cast<const unsigned int*>(it.base + it.e.delta_off);
                const unsigned long long w0 = byte0 >> 2, wlim = 2ull * it.e.n_delta_words;
                unsigned int W[DEC_KPT + 1];
    #pragma unroll
                for (int t = 0; t <= DEC_KPT; ++t) W[t] = (w0 + t < wlim) ? __brev(__ldcg(src + w0 + t)) : 0u;
                unsigned int start = (unsigned int)(byte0 & 3);
    #pragma unroll
                for (int u = 0; u < DEC_KPT; ++u) {
                    const unsigned int wi = start >> 2, sh = 8u * (start & 3u);
                    unsigned int hi = W[0], lo = W[1];
    #pragma unroll
                    for (int t = 1; t < DEC_KPT; ++t)
                        if (wi == (unsigned int)t) { hi = W[t]; lo = W[t + 1]; }
                    const unsigned int v = __funnelshift_l(lo, hi, sh);
                    d[u] = w[u] ? v >> (32u - 8u * w[u]) : 0u;
                    start += w[u];
                }
            }
        }
    } else {
        // delta_adaptive (binary/DeltaAdaptiveEncoder.java:114-146): b = 32 / m bits per interval; the
        // flag of a key gives its interval count iv, its delta takes b * iv bits, most significant first.
        const unsigned int m = it.e.num_intervals, b = 32u / m, fbw = 31u - (unsigned int)__clz(m);
        const unsigned int* fwords = reinterpret_cast<const unsigned int*>(it.base + it.e.flag_off);
        const unsigned long long fw_lim = 2ull * it.e.n_flag_words;
        unsigned int iv[DEC_KPT];
#pragma unroll
        for (int u = 0; u < DEC_KPT; ++u) iv[u] = 0;
        if (!it.e.flag_kind) {
            // fixed flags: iv - 1 in log2(m) bits per key (none when m = 1)
            if (i0 < cnt) {
                unsigned long long win = 0;
                if (fbw) {
                    const unsigned long long off = (unsigned long long)rs.flag_bit_off + (unsigned long long)fbw * i0;
                    const unsigned long long w0 = off >> 5;
                    const unsigned int lo = w0 < fw_lim ? __ldcg(fwords + w0) : 0u, hi = w0 + 1 < fw_lim ? __ldcg(fwords + w0 + 1) : 0u;
                    win = ((unsigned long long)lo | ((unsigned long long)hi << 32)) >> (off & 31ull);
                }
#pragma unroll
                for (int u = 0; u < DEC_KPT; ++u)
                    if (i0 + u < cnt) {
                        const unsigned int bits = fbw ? (unsigned int)(win >> (fbw * u)) & ((1u << fbw) - 1u) : 0u;
                        iv[u] = (fbw ? (__brev(bits) >> (32u - fbw)) : 0u) + 1u;
                    }
            }
        } else {
            // unary flags: iv one-bits and a zero-bit per key. The thread that holds a stretch of the chunk's
            // flag words ranks its zero bits (block scan of the counts) and notes where the key with that
            // rank ends; zero bits beyond the chunk's keys (the next chunk, padding) are ignored.
            const unsigned int sh = rs.flag_bit_off & 31u;
            const unsigned long long wbase = (unsigned long long)(rs.flag_bit_off >> 5) + 3ull * threadIdx.x;
            unsigned int zb[3], zsum = 0;
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const unsigned int word = wbase + k < fw_lim ? __ldcg(fwords + wbase + k) : 0xFFFFFFFFu;
                zb[k] = ~word;
                if (threadIdx.x == 0 && k == 0) zb[k] &= ~((1u << sh) - 1u);  // bits of the chunk before
                zsum += (unsigned int)__popc(zb[k]);
            }
            unsigned int r = dec_scan(zsum, part_c);
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                unsigned int z = zb[k];
                while (z && r < cnt) {
                    const int bit = __ffs(z) - 1;
                    z &= z - 1;
                    s_pos[r++] = (unsigned short)((3u * threadIdx.x + k) * 32u + (unsigned int)bit - sh);
                }
                r += (unsigned int)__popc(z);
            }
            __syncthreads();
#pragma unroll
            for (int u = 0; u < DEC_KPT; ++u)
                if (i0 + u < cnt) {
                    const unsigned int e = s_pos[i0 + u], st = (i0 + u) ? (unsigned int)s_pos[i0 + u - 1] + 1u : 0u;
                    iv[u] = e - st;
                }
        }
        unsigned int bsum = 0;
#pragma unroll
        for (int u = 0; u < DEC_KPT; ++u) bsum += b * iv[u];
        const unsigned int bitoff = dec_scan(bsum, part_a);
        if (i0 < cnt) {
            const unsigned int* dwords = reinterpret_cast<const unsigned int*>(it.base + it.e.delta_off);
            const unsigned long long dw_lim = 2ull * it.e.n_delta_words;
            unsigned long long off = rs.delta_bit_off + bitoff;
#pragma unroll
            for (int u = 0; u < DEC_KPT; ++u) {
                const unsigned int dw = b * iv[u];
                if (dw && dw <= 32u) {
                    const unsigned long long w0 = off >> 5;
                    const unsigned int lo = w0 < dw_lim ? __ldcg(dwords + w0) : 0u, hi = w0 + 1 < dw_lim ? __ldcg(dwords + w0 + 1) : 0u;
                    const unsigned int x = __funnelshift_r(lo, hi, (unsigned int)(off & 31ull));
                    d[u] = __brev(x << (32u - dw));
                }
                off += dw;
            }
        }
    }
    unsigned int dsum = 0;
#pragma unroll
    for (int u = 0; u < DEC_KPT; ++u) dsum += d[u];
    const unsigned int dex = dec_scan(dsum, part_b);
    o.d0 = d[0];
#pragma unroll
    for (int u = 0; u < DEC_KPT; ++u) {
        o.keys[u] = 0xFFFFFFFFu;
        o.live[u] = false;
        o.bv[u] = 0.f;
    }
    if (i0 < cnt) {
        unsigned int key = rs.prev_key + dex;
#pragma unroll
        for (int u = 0; u < DEC_KPT; ++u) {
            key += d[u];
            o.keys[u] = key;
            o.live[u] = i0 + u < cnt;
            if (o.live[u] && key >= (unsigned long long)p.dim) {
                skml_set_status(p.status, SKML_BAD_HEADER, 0x200u);
                o.live[u] = false;
                o.keys[u] = 0xFFFFFFFFu;
            }
        }
        if (it.rows <= 4) {
#pragma unroll
            for (int u = 0; u < DEC_KPT; ++u) o.bv[u] = o.live[u] ? query_one<4>(p, it, o.keys[u], stab) : 0.f;
        } else {
#pragma unroll
            for (int u = 0; u < DEC_KPT; ++u) o.bv[u] = o.live[u] ? query_one<SKML_MAX_ROWS>(p, it, o.keys[u], stab) : 0.f;
        }
    }
}

// Stages the item's sketch table in shared memory when it fits (one coalesced read instead of `rows`
// random L2 sectors per key); returns the staged copy or null. Block-wide call.
__device__ __forceinline__ const unsigned char* stage_table(const DecItem& it, unsigned char* tab_area) {
    const unsigned long long tbytes = (unsigned long long)it.rows * it.e.col_num * (it.cell_bits / 8);
    if (!tab_area || tbytes > DEC_TAB_SMEM) return nullptr;
    __syncthreads();  // the previous table's readers are done
    const uint4* src = reinterpret_cast<const uint4*>(it.tab);
    uint4* dst = reinterpret_cast<uint4*>(tab_area);
    const int nv = (int)((tbytes + 15) / 16);  // table sections are padded to 16 bytes
    for (int t = threadIdx.x; t < nv; t += blockDim.x) dst[t] = ld_cg_v4(src + t);
    __syncthreads();
    return tab_area;
}
