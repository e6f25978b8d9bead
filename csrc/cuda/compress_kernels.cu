// Fused SketchML compress + publish for sm_100a.
//
// One persistent cooperative kernel (one block per SM, 1024 threads) runs the whole
// sender side of the gradient exchange:
//   S1  mergeable quantile summary of the values (sorted shared-memory tiles, k = 128
//       samples per run, pairwise merge + keep-every-second carry chain), min / max
//   S2  weighted-rank query of the merged summaries -> q-1 raw split points
//   S3  dedupe splits, zero bucket, bucket midpoints, group edges; bucketize every value and
//       count the keys of every bucket group per warp slice
//   S4  group sizes -> payload layout; every key goes to its group's contiguous (still key-sorted)
//       staging list; grouped MinMaxSketch insert (atomicMin on packed cells)
//   S5  the groups' key lists are coded in 1024-key chunks like a plain array: delta widths, byte
//       offsets by a block scan, flag bytes, delta bytes, one restart point per chunk. A block owns a
//       contiguous run of chunks and learns its byte offset from the blocks before it (their
//       published byte counts), so no grid barrier sits inside this stage
//   S6  header and group table; sketch tables narrowed to 8/16-bit bucket codes; the finished
//       payload is stored into every peer's receive slot with 16-byte peer stores, then the
//       arrival flags are released (system scope). There is no separate all-gather.
// Grid-wide dependencies are bounded software barriers (cooperative launch guarantees
// co-residency). With `fused = 0` the same stage functions run as separate launches.
//
// Reference behaviour restated (paths inside the reference project, module `sketch`):
//   quantization/QuantileQuantizer.java:27-50, sketch/quantile/HeapQuantileSketch.java:73-143,
//   293-323, sketch/quantile/QSketchUtils.java:45-82, base/Quantizer.java:39-92,
//   sketch/frequency/FSketchUtils.java:9-47, MinMaxSketch.java:27-55,
//   GroupedMinMaxSketch.java:103-121, binary/DeltaBinaryEncoder.java:26-39, and
//   ml/gradient/SketchGradient.scala:24-48.
#include <cooperative_groups.h>
#include <stdio.h>

#include "skml_api.h"
#include "skml_device.cuh"

#define MAX_GRID 192
#define SK_K 128            // samples per run
#define TILE 2048           // values sorted at once
#define TILE_W 16           // TILE / SK_K: weight of a sample taken from a full tile
#define MAX_LEVELS 24
#define FP_SHIFT 20         // fixed-point fraction bits of sample weights
#define MAX_SAMPLE 16        // largest sampling factor of the bottom-level sampler
#define HUF_MAX_SYMS 512     // symbols per bucket group the device Huffman coder accepts
#define HUF_RESTART 128      // cells between two restart offsets of a Huffman-coded table
#define AP_STAGE_F 548       // staging words of one chunk's flag bits (<= 17 bits per key, plus a word of misalignment)
#define AP_STAGE_D 1028      // the same for its delta bits (<= 32 bits per key)

struct CP {
    const int* keys;
    const float* vals;
    const long long* meta;
    long long n_max, dim;
    int q, G, rows;
    double col_ratio;
    unsigned long long seed, step;
    unsigned int rank, world;
    const double* loss_partials;
    unsigned char* payload;
    long long slot_capacity;
    unsigned char* peer_payload[SKML_MAX_PEERS];
    unsigned long long* peer_flag[SKML_MAX_PEERS];
    unsigned int* ctrl;
    unsigned int* run_vals;
    unsigned int* run_cnt;
    unsigned long long* run_w;
    unsigned int* splits_raw;
    unsigned int* warp_cnt;          // [grid * 32 warps][SKML_MAX_GROUPS]: keys of every group in every warp slice
    unsigned int* blk_cnt;           // [grid][SKML_MAX_GROUPS]: the same per block
    unsigned long long* blk_bytes;   // [grid][SKML_MAX_GROUPS]: delta bytes of the chunks every block owns, per group
    unsigned int* blk_flag;          // [grid]: epoch in which blk_bytes was published
    unsigned int* chunk_off;         // [2 * chunks]: delta-byte offset of a chunk inside its owner's part of the group
                                     // (delta_adaptive: flag-bit and delta-bit offsets)
    unsigned long long* blk_bits;    // delta_adaptive: [grid][2 * SKML_MAX_GROUPS] flag bits / delta bits per block and group
    unsigned int* blk_done;          // delta_adaptive: [grid] epoch in which the block finished writing its chunks
    unsigned int* key_hist;          // delta_adaptive: [SKML_MAX_GROUPS][32] keys per delta width, zeroed in S1
    int key_encoder;
    int huffman;                     // sketch tables travel Huffman-coded (cell_bits = 0)
    int sample_splits;               // split points from a sample every cluster draws alike (no S2, two grid barriers fewer)
    unsigned int* cell_hist;         // Huffman: [bin_num + groups] cells per symbol, zeroed in S1
    unsigned long long* blk_tbits;   // Huffman: [grid][SKML_MAX_GROUPS] code bits per block and group
    unsigned int* tchunk_off;        // Huffman: [table chunks] bit offset of a chunk inside its owner's part of the stream
    unsigned short* bins;
    int* gkeys;                      // keys, grouped: group g's list starts at Layout::goff[g]
    unsigned int* tables;
    long long tables_cap;
    unsigned int* status;
    long long budget;
    const float* given_splits;
    int n_given;
    float given_min, given_max;
};

struct QInfo {
    int nsplits, bin_num, zero_idx, cell_bits;
    float minv, maxv;
    int edges[SKML_MAX_GROUPS];
};

struct Layout {
    unsigned int n_g[SKML_MAX_GROUPS];
    unsigned int col[SKML_MAX_GROUPS];
    unsigned int goff[SKML_MAX_GROUPS];            // start of the group's staging list (a multiple of 4 entries)
    unsigned int chunk_prefix[SKML_MAX_GROUPS + 1]; // chunks of the groups before, group-major chunk numbering
    unsigned int base_rank[SKML_MAX_GROUPS];       // keys of the group in the blocks before this one
    unsigned long long bytes_g[SKML_MAX_GROUPS];   // delta bytes of the group (block 0, for the header)
    unsigned long long flag_bits[SKML_MAX_GROUPS], delta_bits[SKML_MAX_GROUPS];  // delta_adaptive: stream lengths
    unsigned int num_iv[SKML_MAX_GROUPS], flag_kind[SKML_MAX_GROUPS];            // delta_adaptive: the groups' modes
    unsigned long long off_keys;                   // delta_adaptive: start of the per-group [flags | deltas] sections
    // Huffman-coded tables: symbol range, cells, present symbols, code bits, chunk numbering, stream / restart starts
    unsigned int sym_lo[SKML_MAX_GROUPS], nsym[SKML_MAX_GROUPS], cells[SKML_MAX_GROUPS], items[SKML_MAX_GROUPS];
    unsigned int tchunk_prefix[SKML_MAX_GROUPS + 1];
    unsigned long long tbits[SKML_MAX_GROUPS], tstream_off[SKML_MAX_GROUPS], trestart_off[SKML_MAX_GROUPS];
    unsigned long long table_off[SKML_MAX_GROUPS], flag_off[SKML_MAX_GROUPS], delta_off[SKML_MAX_GROUPS],
        restart_off[SKML_MAX_GROUPS], tab32_off[SKML_MAX_GROUPS];
    unsigned char hash_ids[SKML_MAX_GROUPS][8];
    unsigned long long col_magic[SKML_MAX_GROUPS];  // ceil(2^64 / col) for the division-free modulo
    unsigned int recip[SKML_MAX_GROUPS];            // floor(2^32 / col) for the mixer-only hash path
    int mixers;                                     // every row of every group uses an integer mixer (<= 3 rows)
    unsigned long long off_bv, off_gt, off_flags, off_restart, off_tables, off_deltas, total_bytes;
    int overflow;
};

struct WsLayout {
    long long ctrl, run_vals, run_cnt, run_w, splits_raw, warp_cnt, blk_cnt, blk_bytes, blk_flag, chunk_off, blk_bits, blk_done, key_hist, cell_hist, blk_tbits, tchunk_off, bins, gkeys, tables,
        total;
    long long tables_cap;
};

static inline long long al256(long long x) { return (x + 255) & ~255ll; }

static WsLayout ws_layout(long long n_max, long long q, long long G, long long rows, double col_ratio, long long grid) {
    WsLayout L;
    long long o = 0;
    L.ctrl = o; o += 256;
    L.run_vals = o; o += al256(grid * SK_K * 4);
    L.run_cnt = o; o += al256(grid * 4);
    L.run_w = o; o += al256(grid * 8);
    L.splits_raw = o; o += al256(q * 4);
    L.warp_cnt = o; o += al256(grid * SKML_WARPS * SKML_MAX_GROUPS * 4);
    L.blk_cnt = o; o += al256(grid * SKML_MAX_GROUPS * 4);
    L.blk_bytes = o; o += al256(grid * SKML_MAX_GROUPS * 8);
    L.blk_flag = o; o += al256(grid * 4);
    L.chunk_off = o; o += al256((n_max / SKML_RESTART_INTERVAL + SKML_MAX_GROUPS + 8) * 8);
    L.blk_bits = o; o += al256(grid * 2 * SKML_MAX_GROUPS * 8);
    L.blk_done = o; o += al256(grid * 4);
    L.key_hist = o; o += al256(SKML_MAX_GROUPS * 32 * 4);
    L.cell_hist = o; o += al256((SKML_GPU_MAX_BINS + SKML_MAX_GROUPS) * 4);
    L.blk_tbits = o; o += al256(grid * SKML_MAX_GROUPS * 8);
    L.tchunk_off = o; o += al256(((rows * ((long long)(col_ratio * (double)n_max) + 2 + G) + 64) / 1024 + SKML_MAX_GROUPS + 8) * 4);
    L.bins = o; o += al256(n_max * 2);
    L.gkeys = o; o += al256((n_max + 4 * SKML_MAX_GROUPS + 8) * 4);
    L.tables_cap = rows * ((long long)(col_ratio * (double)n_max) + 2 + G) + 64;
    L.tables = o; o += al256(L.tables_cap * 4);
    L.total = o;
    return L;
}

extern "C" long long skml_compress_workspace_bytes(long long n_max, long long bin_num, long long group_num,
                                                   long long row_num, double col_ratio, long long grid) {
    if (grid <= 0 || grid > MAX_GRID) grid = MAX_GRID;
    return ws_layout(n_max, bin_num, group_num, row_num, col_ratio, grid).total;
}

// Upper bound of the payload size for n_max non-zeros (sparse kind) or dim codes (dense kind).
static __host__ __device__ inline long long payload_bound(long long n_max, long long dim, long long bin_num, long long group_num,
                                                          long long row_num, double col_ratio) {
    long long G = group_num, R = SKML_RESTART_INTERVAL;
    long long head = SKML_HEADER_BYTES + (long long)skml_align16(4 * bin_num) + SKML_GROUP_ENTRY_BYTES * G;
    long long flags = 17 * n_max / 8 + 24 * G + 16;   // delta_adaptive with unary flags: up to 17 flag bits per key
    long long restart = 16 * (n_max / R + G) + 16 * G;
    long long cells = row_num * ((long long)(col_ratio * (double)n_max) + 2 * G);
    // two bytes per cell cover 8/16-bit codes and any Huffman stream (at most 10 bits per cell); the
    // Huffman sections add their code books (12 bytes per symbol) and one restart offset per 128 cells
    long long tables = 2 * cells + 32 * G + 12 * (bin_num + G) + cells / 32 + 96 * G;
    long long deltas = 4 * n_max + 24 * G;
    long long sparse = head + flags + restart + tables + deltas + 64;
    long long dense = head + 2 * dim + 64;
    long long cap = sparse > dense ? sparse : dense;
    return (cap + 255) & ~255ll;
}

extern "C" long long skml_payload_capacity(long long n_max, long long dim, long long bin_num, long long group_num,
                                           long long row_num, double col_ratio) {
    return payload_bound(n_max, dim, bin_num, group_num, row_num, col_ratio);
}

// ---------------------------------------------------------------------------
// shared memory carve-up (dynamic, one block per SM)
// ---------------------------------------------------------------------------
// Per-warp scratch of the Huffman code construction.
struct HufScratch {
    unsigned int w[HUF_MAX_SYMS];         // leaf weights, ascending
    unsigned int iw[HUF_MAX_SYMS];        // weights of the internal nodes, in creation order (ascending)
    unsigned short ord[HUF_MAX_SYMS];     // symbol of the i-th lightest leaf
    unsigned short pl[HUF_MAX_SYMS];      // parent (internal node) of every leaf
    unsigned short pi[HUF_MAX_SYMS];      // parent of every internal node
    unsigned char di[HUF_MAX_SYMS];       // depth of every internal node
};

// The quantile stages (S1, S2) and the coding stage (S5) never hold data at the same time, so their
// arrays share one region: the smaller the block's shared memory, the more of the SM's 256 KB is left
// as L1 for the scatter and coding passes, which keep many loads in flight.
struct SmemQuantile {
    unsigned int tile[TILE];
    unsigned int levels[MAX_LEVELS][SK_K];
    unsigned int run[SK_K];
    unsigned int merge[2 * SK_K];
    unsigned int tail[SK_K];
    unsigned long long e_acc[SK_K];
    unsigned int runs_all[MAX_GRID * SK_K];   // S2: all blocks' runs
    unsigned int runs_cnt[MAX_GRID];
    unsigned long long runs_w[MAX_GRID];
};
struct SmemCoding {
    unsigned int stage_f[4][AP_STAGE_F];            // delta_adaptive: one chunk's flag / delta bits per sub-block
    unsigned int stage_d[4][AP_STAGE_D];            // (also the staging of the Huffman table streams)
    unsigned char huf_len[SKML_GPU_MAX_BINS + SKML_MAX_GROUPS];   // Huffman: code length / code word per symbol slot
    unsigned int huf_code[SKML_GPU_MAX_BINS + SKML_MAX_GROUPS];
    HufScratch huf_scratch[8];
};

struct Smem {
    union {
        SmemQuantile qs;
        SmemCoding cs;
    };
    // stages S3..S6
    float splits[SKML_GPU_MAX_BINS];
    unsigned char grp_lut[SKML_GPU_MAX_BINS];      // bucket -> group
    QInfo qi;
    Layout lay;
    unsigned int wcnt[SKML_WARPS][SKML_MAX_GROUPS];
    unsigned int wbase[SKML_WARPS][SKML_MAX_GROUPS];
    unsigned long long my_bytes[SKML_MAX_GROUPS];   // delta bytes of the chunks this block owns, per group
    unsigned long long pre_bytes[SKML_MAX_GROUPS];  // the same, summed over the blocks before this one
    unsigned long long my_bits[2 * SKML_MAX_GROUPS], pre_bits[2 * SKML_MAX_GROUPS];  // delta_adaptive: flag / delta bits
    unsigned long long my_tbits[SKML_MAX_GROUPS], pre_tbits[SKML_MAX_GROUPS];
    unsigned int sub_part[4][8];                    // scan scratch of the four 256-thread sub-blocks
    unsigned int sub_total[4];
    unsigned long long unit_prefix[SKML_MAX_GROUPS + 1];
    int flag;
};


// 164 KB is a shared-memory carve-out step of the SM: staying under it (with the block's static shared
// memory and the 1 KB the system reserves) leaves 92 KB of L1; measured, the scatter + insert stage of
// 2.3M keys takes 69 us with that L1 and 120 us with the 28 KB that the next step (228 KB) leaves.
static_assert(sizeof(Smem) <= 162 * 1024, "the compress kernels' shared memory must stay below the 164 KB carve-out");

__device__ __forceinline__ unsigned int lanemask_lt() {
    unsigned int m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Block 0 leaves a nanosecond time stamp per stage in the control words (u64 at ctrl[16 + 2 i]);
// skml tools read them to show where a fused launch spends its time.
__device__ __forceinline__ void stage_stamp(unsigned int* ctrl, int i) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        reinterpret_cast<unsigned long long*>(ctrl)[8 + i] = t;
    }
}

// ---------------------------------------------------------------------------
// S1: quantile summary
// ---------------------------------------------------------------------------
// Merge the sorted runs a[128] and b[128] into s.qs.merge (ascending) with a bitonic merge.
__device__ __forceinline__ void merge_runs(Smem& s, const unsigned int* a, const unsigned int* b) {
    for (int t = threadIdx.x; t < SK_K; t += blockDim.x) {
        s.qs.merge[t] = a[t];
        s.qs.merge[2 * SK_K - 1 - t] = b[t];
    }
    __syncthreads();
    for (int j = SK_K; j > 0; j >>= 1) {
        for (int t = threadIdx.x; t < SK_K; t += blockDim.x) {
            int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
            unsigned int x = s.qs.merge[i], y = s.qs.merge[i | j];
            if (x > y) {
                s.qs.merge[i] = y;
                s.qs.merge[i | j] = x;
            }
        }
        __syncthreads();
    }
}

// Carry s.qs.run (weight TILE_W << level0) up the level chain.
__device__ __forceinline__ void carry_run(Smem& s, unsigned int& occupied, int level, const CP& p, unsigned long long salt) {
    while (true) {
        if (!(occupied & (1u << level))) {
            for (int t = threadIdx.x; t < SK_K; t += blockDim.x) s.qs.levels[level][t] = s.qs.run[t];
            occupied |= 1u << level;
            __syncthreads();
            return;
        }
        merge_runs(s, s.qs.levels[level], s.qs.run);
        unsigned int off = (unsigned int)(skml_rand(p.seed, p.step, ((unsigned long long)p.rank << 32) | blockIdx.x,
                                                    salt * 64 + level) & 1u);
        for (int t = threadIdx.x; t < SK_K; t += blockDim.x) s.qs.run[t] = s.qs.merge[2 * t + off];
        occupied &= ~(1u << level);
        __syncthreads();
        ++level;
        if (level >= MAX_LEVELS) return;  // unreachable for n < 2^31
    }
}

// The block's share of the values -> one run of at most SK_K samples in s.qs.tile[0, cnt) with weight w.
__device__ void summarize_slice(const CP& p, Smem& s, const float* __restrict__ vals, long long n, unsigned int& run_cnt,
                                unsigned long long& run_w) {
    run_cnt = 0;
    run_w = 0;
    // Bottom-level sampler (as in KLL sketches): of every f consecutive values one is kept at random
    // with weight f, so one 2048-sort covers f * 2048 values and enters the level chain as one run
    // of weight 16 f. f is the smallest power of two (<= MAX_SAMPLE) for which every block has one
    // sort to do; min and max still see every value.
    const long long ntiles = (n + TILE - 1) / TILE;
    int f = 1, lf = 0;
    while (f < MAX_SAMPLE && ntiles > (long long)f * gridDim.x) {
        f <<= 1;
        ++lf;
    }
    const long long ST = (long long)f * TILE;
    const long long nst = (n + ST - 1) / ST;
    const long long t0 = blockIdx.x;  // super tiles are dealt round-robin: t0, t0 + grid, ...
    if (t0 >= nst || n <= 0) return;
    unsigned int occupied = 0;
    int tail_cnt = 0;
    unsigned long long tail_w = 0;
    unsigned int kmin = 0xFFFFFFFFu, kmax = 0u;
    const unsigned long long salt0 = p.seed ^ (p.step * 0x9E3779B97F4A7C15ull) ^ ((unsigned long long)p.rank << 40);
    for (long long st = t0; st < nst; st += gridDim.x) {
        const long long base = st * ST;
        const long long m = (n - base) < ST ? (n - base) : ST;  // values of this super tile
        if (m == ST) {
            for (int t = threadIdx.x; t < TILE; t += blockDim.x) {
                const float* src = vals + base + (long long)t * f;
                const unsigned int pick = (unsigned int)(skml_splitmix64(salt0 ^ (unsigned long long)(base + t)) >> 40) & (unsigned int)(f - 1);
                unsigned int chosen = 0;
                if (f == 1) {
                    chosen = f2ord(src[0]);
                    kmin = min(kmin, chosen);
                    kmax = max(kmax, chosen);
                } else if (f == 2) {
                    const float2 q = *reinterpret_cast<const float2*>(src);
                    const unsigned int k0 = f2ord(q.x), k1 = f2ord(q.y);
                    kmin = min(kmin, min(k0, k1));
                    kmax = max(kmax, max(k0, k1));
                    chosen = pick ? k1 : k0;
                } else {
                    for (int j = 0; j < f / 4; ++j) {
                        const float4 q = reinterpret_cast<const float4*>(src)[j];
                        const unsigned int k0 = f2ord(q.x), k1 = f2ord(q.y), k2 = f2ord(q.z), k3 = f2ord(q.w);
                        kmin = min(min(kmin, k0), min(min(k1, k2), k3));
                        kmax = max(max(kmax, k0), max(max(k1, k2), k3));
                        if ((int)(pick >> 2) == j) {
                            const unsigned int r = pick & 3u;
                            chosen = r == 0 ? k0 : (r == 1 ? k1 : (r == 2 ? k2 : k3));
                        }
                    }
                }
                s.qs.tile[t] = chosen;
            }
            __syncthreads();
            if (st == t0) stage_stamp(p.ctrl, 10);
            block_sort_2048(s.qs.tile);
            if (st == t0) stage_stamp(p.ctrl, 11);
            const unsigned int off = (unsigned int)(skml_rand(p.seed, p.step, ((unsigned long long)p.rank << 32) | blockIdx.x,
                                                              0x7200u + (unsigned long long)((st - t0) / gridDim.x)) & (TILE_W - 1));
            for (int t = threadIdx.x; t < SK_K; t += blockDim.x) s.qs.run[t] = s.qs.tile[t * TILE_W + off];
            __syncthreads();
            carry_run(s, occupied, lf, p, (unsigned long long)((st - t0) / gridDim.x) + 1);
            continue;
        }
        // the last, partial super tile of the whole input: slot t samples the valid part of its f values
        const int ms = (int)((m + f - 1) / f);  // slots that hold a value
        for (int t = threadIdx.x; t < TILE; t += blockDim.x) {
            unsigned int chosen = 0xFFFFFFFFu;
            const long long g0 = base + (long long)t * f;
            if (g0 < n) {
                const int valid = (int)((n - g0) < f ? (n - g0) : f);
                const unsigned int pick = (unsigned int)((skml_splitmix64(salt0 ^ (unsigned long long)(base + t)) >> 40) % (unsigned int)valid);
                for (int j = 0; j < valid; ++j) {
                    const unsigned int k = f2ord(vals[g0 + j]);
                    kmin = min(kmin, k);
                    kmax = max(kmax, k);
                    if ((unsigned int)j == pick) chosen = k;
                }
            }
            s.qs.tile[t] = chosen;
        }
        __syncthreads();
        block_sort_2048(s.qs.tile);
        int stride = 1;
        while ((ms + stride - 1) / stride > SK_K) stride <<= 1;
        tail_cnt = (ms + stride - 1) / stride;
        const unsigned int off = stride > 1 ? (unsigned int)(skml_rand(p.seed, p.step, p.rank, 0x7100u) % stride) : 0u;
        for (int t = threadIdx.x; t < tail_cnt; t += blockDim.x) {
            int idx = t * stride + (int)off;
            if (idx > ms - 1) idx = ms - 1;
            s.qs.tail[t] = s.qs.tile[idx];
        }
        tail_w = (((unsigned long long)m) << FP_SHIFT) / (unsigned long long)tail_cnt;
        __syncthreads();
    }
    stage_stamp(p.ctrl, 12);
    // block min / max -> global (stored so that an all-zero word means "nothing yet")
    {
        unsigned int a = kmin, b = kmax;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a = min(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
            b = max(b, __shfl_xor_sync(0xFFFFFFFFu, b, o));
        }
        // one pair of atomics per block: thousands of same-address atomics would serialise in L2
        __shared__ unsigned int s_mn[SKML_WARPS], s_mx[SKML_WARPS];
        if ((threadIdx.x & 31) == 0) {
            s_mn[threadIdx.x >> 5] = a;
            s_mx[threadIdx.x >> 5] = b;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            a = s_mn[threadIdx.x];
            b = s_mx[threadIdx.x];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                a = min(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
                b = max(b, __shfl_xor_sync(0xFFFFFFFFu, b, o));
            }
            if (threadIdx.x == 0) {
                atomicMax(&p.ctrl[4], ~a);
                atomicMax(&p.ctrl[5], b);
            }
        }
    }
    stage_stamp(p.ctrl, 13);
    // collapse the levels (+ tail) into one run (the sort buffer is free now)
    int nruns = __popc(occupied) + (tail_cnt > 0 ? 1 : 0);
    unsigned int* out = s.qs.tile;
    if (nruns == 1) {
        const unsigned int* src;
        int cnt;
        unsigned long long w;
        if (tail_cnt > 0) {
            src = s.qs.tail; cnt = tail_cnt; w = tail_w;
        } else {
            int lv = __ffs(occupied) - 1;
            src = s.qs.levels[lv]; cnt = SK_K; w = ((unsigned long long)TILE_W << lv) << FP_SHIFT;
        }
        for (int t = threadIdx.x; t < cnt; t += blockDim.x) out[t] = src[t];
        run_cnt = (unsigned int)cnt;
        run_w = w;
        return;
    }
    // several runs: exclusive cumulative weight of every sample, then 128 mid-rank samples
    unsigned long long Wc = 0;
    for (int lv = 0; lv < MAX_LEVELS; ++lv)
        if (occupied & (1u << lv)) Wc += (unsigned long long)SK_K * (((unsigned long long)TILE_W << lv) << FP_SHIFT);
    Wc += (unsigned long long)tail_cnt * tail_w;
    const int total_samples = __popc(occupied) * SK_K + tail_cnt;
    for (int sidx = threadIdx.x; sidx < total_samples; sidx += blockDim.x) {
        // locate (run a, index i): occupied levels in ascending order, then the tail
        int a = -1, i = sidx, seen = 0;
        for (int lv = 0; lv < MAX_LEVELS; ++lv) {
            if (!(occupied & (1u << lv))) continue;
            if (i < SK_K) { a = lv; break; }
            i -= SK_K;
            ++seen;
        }
        const unsigned int value = a >= 0 ? s.qs.levels[a][i] : s.qs.tail[i];
        const unsigned long long wa = a >= 0 ? (((unsigned long long)TILE_W << a) << FP_SHIFT) : tail_w;
        unsigned long long e = (unsigned long long)i * wa;
        for (int lv = 0; lv < MAX_LEVELS; ++lv) {
            if (!(occupied & (1u << lv)) || lv == a) continue;
            unsigned long long wl = ((unsigned long long)TILE_W << lv) << FP_SHIFT;
            bool before = a < 0 || lv < a;  // runs earlier in the order win ties
            int c = before ? upper_bound_u(s.qs.levels[lv], SK_K, value) : lower_bound_u(s.qs.levels[lv], SK_K, value);
            e += (unsigned long long)c * wl;
        }
        if (tail_cnt > 0 && a >= 0) e += (unsigned long long)lower_bound_u(s.qs.tail, tail_cnt, value) * tail_w;
        // targets t_j = (2j+1) * Wc / 256, j = 0..127, covered iff e <= t_j < e + wa
        long long j = (long long)((e << 7) / Wc) - 1;
        if (j < 0) j = 0;
        for (; j < SK_K; ++j) {
            unsigned long long tj = ((unsigned long long)(2 * j + 1) * (Wc >> 8));
            if (tj < e) continue;
            if (tj >= e + wa) break;
            out[j] = value;
        }
        (void)seen;
    }
    run_cnt = SK_K;
    run_w = Wc / SK_K;
}

// --- thread-block cluster primitives (distributed shared memory) ---
__device__ __forceinline__ unsigned int cluster_ctarank() {
    unsigned int r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned int cluster_nctarank() {
    unsigned int r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// hardware barrier of the cluster's blocks (blocks that have exited count as arrived)
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared-memory address of `ptr` (a location in this block's shared memory) in block `rank` of the cluster
__device__ __forceinline__ unsigned int dsmem_addr(const void* ptr, unsigned int rank) {
    const unsigned int a = (unsigned int)__cvta_generic_to_shared(ptr);
    unsigned int r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ unsigned int ld_dsmem_u32(unsigned int addr) {
    unsigned int v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_dsmem_u64(unsigned int addr) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
    return v;
}

// Two weighted runs a (s.qs.tile[0, ca), weight wa) and b (s.qs.tile[SK_K, SK_K + cb), weight wb) -> SK_K samples
// at the mid ranks (2j + 1) / (2 SK_K) of their union, left in s.qs.tile[0, SK_K); returns the new weight.
__device__ unsigned long long merge_two_runs(Smem& s, unsigned int ca, unsigned long long wa, unsigned int cb,
                                             unsigned long long wb) {
    const unsigned int* a = s.qs.tile;
    const unsigned int* b = s.qs.tile + SK_K;
    const unsigned long long Wc = (unsigned long long)ca * wa + (unsigned long long)cb * wb;
    for (unsigned int sidx = threadIdx.x; sidx < ca + cb; sidx += blockDim.x) {
        const bool from_a = sidx < ca;
        const unsigned int i = from_a ? sidx : sidx - ca;
        const unsigned int value = from_a ? a[i] : b[i];
        const unsigned long long w = from_a ? wa : wb;
        // weight in front of the sample; run a wins ties
        const unsigned long long e = (unsigned long long)i * w +
            (from_a ? (unsigned long long)lower_bound_u(b, (int)cb, value) * wb : (unsigned long long)upper_bound_u(a, (int)ca, value) * wa);
        long long j = (long long)((e << 7) / Wc) - 1;
        if (j < 0) j = 0;
        for (; j < SK_K; ++j) {
            const unsigned long long tj = (unsigned long long)(2 * j + 1) * (Wc >> 8);
            if (tj < e) continue;
            if (tj >= e + w) break;
            s.qs.merge[j] = value;
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < SK_K; t += blockDim.x) s.qs.tile[t] = s.qs.merge[t];
    __syncthreads();
    return Wc / SK_K;
}

// S1: every block summarises its share of the values; the blocks of a thread-block cluster then merge
// their runs in shared memory (the cluster's first block reads the others' runs through distributed
// shared memory) and only the merged run goes to global memory, so S2 has 1 / cluster-size as many runs
// to load and to rank against. Launched without clusters the cluster is the block itself.
__device__ void stage_summary(const CP& p, Smem& s, const float* __restrict__ vals, long long n) {
    __shared__ unsigned int s_pub_cnt;
    __shared__ unsigned long long s_pub_w;
    unsigned int cnt;
    unsigned long long w;
    summarize_slice(p, s, vals, n, cnt, w);
    const unsigned int cs = cluster_nctarank(), cr = cluster_ctarank();
    if (threadIdx.x == 0) {
        s_pub_cnt = cnt;
        s_pub_w = w;
    }
    __syncthreads();
    if (cs > 1) {
        cluster_sync_all();   // every block's run, count and weight are in its shared memory
        if (cr == 0) {
            for (unsigned int r = 1; r < cs; ++r) {
                const unsigned int cb = ld_dsmem_u32(dsmem_addr(&s_pub_cnt, r));
                const unsigned long long wb = ld_dsmem_u64(dsmem_addr(&s_pub_w, r));
                if (cb == 0 || cb > SK_K) continue;   // uniform over the block
                const unsigned int src = dsmem_addr(s.qs.tile, r);
                unsigned int* dst = cnt ? s.qs.tile + SK_K : s.qs.tile;
                for (unsigned int t = threadIdx.x; t < cb; t += blockDim.x) dst[t] = ld_dsmem_u32(src + 4u * t);
                __syncthreads();
                if (cnt == 0) {
                    cnt = cb;
                    w = wb;
                } else {
                    w = merge_two_runs(s, cnt, w, cb, wb);
                    cnt = SK_K;
                }
            }
        } else {
            cnt = 0;   // this block's samples travel in the first block's run
            w = 0;
        }
        cluster_sync_all();   // nobody reads the others' shared memory any more
    }
    unsigned int* out = p.run_vals + (long long)blockIdx.x * SK_K;
    for (unsigned int t = threadIdx.x; t < cnt; t += blockDim.x) out[t] = s.qs.tile[t];
    if (threadIdx.x == 0) {
        p.run_cnt[blockIdx.x] = cnt;
        p.run_w[blockIdx.x] = w;
    }
}

// S1, sample form. Every thread-block cluster draws the SAME stratified sample of the values (one value
// per stride of n / m positions, the offset a function of (seed, step, rank)), so every block ends up with
// the same split points without a grid barrier and without S2. The two blocks of a cluster sort one half
// of a 4096-value sample each and read the other half through distributed shared memory: split t is the
// value of rank floor(m (t + 1) / q) in the union of the two sorted halves, found by a merge-path search
// over the own half and a local copy of the other. Without clusters a block sorts 2048 values alone.
// The rank error of a split is that of an m-value sample (standard deviation at most 0.8 % of n at
// m = 4096), the same order as the k = 128 summary's; inputs of up to m values are summarised exactly.
// Minimum and maximum of ALL values are taken by the count stage, which reads every value anyway.
__device__ void stage_sample_splits(const CP& p, Smem& s, const float* __restrict__ vals, long long n) {
    const unsigned int cs = cluster_nctarank(), cr = cluster_ctarank();
    const int halves = cs >= 2 ? 2 : 1;
    const long long M = (long long)TILE * halves;
    const long long m = n < M ? n : M;   // sample size
    const unsigned long long off = n > m ? skml_rand(p.seed, p.step, p.rank, 0x7300u) % (unsigned long long)n : 0ull;
    const int mine = (int)((m - (long long)(cr % halves) + halves - 1) / halves);   // samples in this block's half
    for (int t = threadIdx.x; t < TILE; t += blockDim.x) {
        const long long j = (long long)t * halves + (cr % halves);
        unsigned int key = 0xFFFFFFFFu;
        if (j < m) {
            const long long pos = n > m ? (long long)(((unsigned long long)j * (unsigned long long)n + off) / (unsigned long long)m) : j;
            key = f2ord(__ldg(vals + pos));
        }
        s.qs.tile[t] = key;
    }
    __syncthreads();
    block_sort_2048(s.qs.tile);
    __syncthreads();
    const int theirs = (int)(m - mine);
    unsigned int* const their = s.qs.runs_all;   // local copy of the other block's sorted half
    if (halves == 2) {
        cluster_sync_all();   // both halves are sorted and visible in the cluster
        const unsigned int other = dsmem_addr(s.qs.tile, (cr % halves) ^ 1u);
        for (int t = threadIdx.x; t < theirs; t += blockDim.x) their[t] = ld_dsmem_u32(other + 4u * (unsigned int)t);
        cluster_sync_all();   // nobody reads the other block's shared memory any more
    }
    __syncthreads();
    const double inv_q = 1.0 / (double)p.q;
    for (int t = threadIdx.x; t < p.q - 1; t += blockDim.x) {
        long long k = (long long)((double)m * ((double)(t + 1) * inv_q));   // target rank in the sample
        if (k > m - 1) k = m - 1;
        // i = how many of the k values before the answer come from this block's half (ties: this half first)
        int lo = (int)(k - theirs > 0 ? k - theirs : 0), hi = (int)(k < mine ? k : mine);
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            const long long j = k - mid;
            const bool ok = j >= theirs || s.qs.tile[mid - 1] <= their[j];
            if (ok) lo = mid;
            else hi = mid - 1;
        }
        const long long j = k - lo;
        const unsigned int a = lo < mine ? s.qs.tile[lo] : 0xFFFFFFFFu;
        const unsigned int b = j < theirs ? their[j] : 0xFFFFFFFFu;
        p.splits_raw[t] = a < b ? a : b;   // every block stores the same values
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------
// S2: weighted-rank query over all published runs -> splits_raw[q-1] (ordered keys)
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long rank_target(long long n, int t, double inv_q) {
    unsigned long long r = (unsigned long long)((double)n * ((double)(t + 1) * inv_q));
    if (r > (unsigned long long)(n - 1)) r = (unsigned long long)(n - 1);
    return r << FP_SHIFT;
}

__device__ void stage_query(const CP& p, Smem& s, long long n) {
    if (n <= 0) return;
    const int nb = gridDim.x;
    for (int t = threadIdx.x; t < nb; t += blockDim.x) {
        s.qs.runs_cnt[t] = p.run_cnt[t];
        s.qs.runs_w[t] = p.run_w[t];
    }
    __syncthreads();
    {
        // all published runs -> shared memory, 16 bytes per load and several loads in flight per thread
        const uint4* src = reinterpret_cast<const uint4*>(p.run_vals);
        const int nv = nb * (SK_K / 4);
        for (int t0 = threadIdx.x; t0 < nv; t0 += 4 * blockDim.x) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int t = t0 + u * blockDim.x;
                // runs that a cluster merged away are empty: nothing to fetch
                v[u] = (t < nv && (4 * t) % SK_K < (int)s.qs.runs_cnt[(4 * t) / SK_K]) ? ld_cg_v4(src + t) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int t = t0 + u * blockDim.x;
                if (t >= nv) continue;
                const int c = (4 * t) / SK_K, i = (4 * t) % SK_K, cnt = (int)s.qs.runs_cnt[c];
                s.qs.runs_all[4 * t] = i < cnt ? v[u].x : 0xFFFFFFFFu;
                s.qs.runs_all[4 * t + 1] = i + 1 < cnt ? v[u].y : 0xFFFFFFFFu;
                s.qs.runs_all[4 * t + 2] = i + 2 < cnt ? v[u].z : 0xFFFFFFFFu;
                s.qs.runs_all[4 * t + 3] = i + 3 < cnt ? v[u].w : 0xFFFFFFFFu;
            }
        }
    }
    __syncthreads();
    // total weight: every warp sums a strided share, lanes combine by shuffle (all threads need it)
    unsigned long long Wtot = 0;
    for (int c = threadIdx.x & 31; c < nb; c += 32) Wtot += (unsigned long long)s.qs.runs_cnt[c] * s.qs.runs_w[c];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) Wtot += __shfl_xor_sync(0xFFFFFFFFu, Wtot, o);
    const double inv_q = 1.0 / (double)p.q;
    const int i = threadIdx.x & (SK_K - 1), part = threadIdx.x / SK_K, parts = blockDim.x / SK_K;
    for (int c = blockIdx.x; c < nb; c += gridDim.x) {
        const int cnt = (int)s.qs.runs_cnt[c];
        if (cnt == 0) continue;  // uniform over the block
        if (threadIdx.x < SK_K) s.qs.e_acc[threadIdx.x] = 0ull;
        __syncthreads();
        if (i < cnt) {
            const unsigned int value = s.qs.runs_all[c * SK_K + i];
            unsigned long long e = 0;
            for (int c2 = part; c2 < nb; c2 += parts) {
                int cnt2 = (int)s.qs.runs_cnt[c2];
                if (cnt2 == 0) continue;
                int k;
                if (c2 == c) k = i;
                else if (c2 < c) k = upper_bound_u(s.qs.runs_all + c2 * SK_K, cnt2, value);
                else k = lower_bound_u(s.qs.runs_all + c2 * SK_K, cnt2, value);
                e += (unsigned long long)k * s.qs.runs_w[c2];
            }
            atomicAdd(&s.qs.e_acc[i], e);
        }
        __syncthreads();
        if (threadIdx.x < cnt) {
            const unsigned int value = s.qs.runs_all[c * SK_K + threadIdx.x];
            const unsigned long long e = s.qs.e_acc[threadIdx.x], w = s.qs.runs_w[c];
            const bool last = e + w >= Wtot;
            // smallest t with target >= e
            int lo = 0, hi = p.q - 1;
            while (lo < hi) {
                int mid = (lo + hi) >> 1;
                if (rank_target(n, mid, inv_q) >= e) hi = mid;
                else lo = mid + 1;
            }
            for (int t = lo; t < p.q - 1; ++t) {
                unsigned long long r = rank_target(n, t, inv_q);
                if (!last && r >= e + w) break;
                p.splits_raw[t] = value;
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// S3 prelude: unique splits, zero bucket, group edges (every block, in shared memory)
// ---------------------------------------------------------------------------
// minmax_ready = false: the minimum and maximum of the values are not known yet (sample form before the
// count stage has run); the zero bucket does not need them (see below), refresh_minmax sets them later.
__device__ void load_quantizer(const CP& p, Smem& s, bool minmax_ready = true) {
    const bool given = p.given_splits != nullptr;
    const int nraw = given ? p.n_given : p.q - 1;
    __shared__ int s_base;
    if (threadIdx.x == 0) s_base = 0;
    __syncthreads();
    for (int b = 0; b < nraw; b += blockDim.x) {
        int i = b + threadIdx.x;
        float v = 0.f, prev = 0.f;
        bool keep = false;
        if (i < nraw) {
            v = given ? p.given_splits[i] : ord2f(__ldcg(p.splits_raw + i));
            if (i > 0) prev = given ? p.given_splits[i - 1] : ord2f(__ldcg(p.splits_raw + i - 1));
            keep = i == 0 || v != prev;
        }
        unsigned int total;
        unsigned int pos = block_exclusive_scan<unsigned int>(keep ? 1u : 0u, &total);
        int base = s_base;
        if (keep) s.splits[base + pos] = v;
        __syncthreads();
        if (threadIdx.x == 0) s_base = base + (int)total;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        QInfo& q = s.qi;
        q.nsplits = s_base;
        q.bin_num = s_base + 1;
        q.cell_bits = q.bin_num <= 256 ? 8 : 16;
        if (given) {
            q.minv = p.given_min;
            q.maxv = p.given_max;
        } else if (minmax_ready) {
            q.minv = ord2f(~__ldcg(p.ctrl + 4));
            q.maxv = ord2f(__ldcg(p.ctrl + 5));
        } else {
            q.minv = q.maxv = 0.f;
        }
        // NaN or infinite gradient values cannot be bucketized (the reference's sketch throws on NaN)
        if (!isfinite(q.minv) || !isfinite(q.maxv)) skml_set_status(p.status, SKML_BAD_INPUT, 0x35u);
        // With splits taken from the data, min > 0 means every split is positive and max < 0 that every split
        // is negative, so the search below gives the first two cases' answers too; they stay for given splits.
        int z;
        if ((given || minmax_ready) && q.minv > 0.f) z = 0;
        else if ((given || minmax_ready) && q.maxv < 0.f) z = q.bin_num - 1;
        else {
            z = 0;
            while (z < q.bin_num - 1 && s.splits[z] < 0.f) ++z;
        }
        q.zero_idx = z;
        skml_group_edges(z, q.bin_num, p.G, q.edges);
    }
    __syncthreads();
}

// Sample form, after the count stage and its grid barrier: minimum and maximum of all values.
__device__ void refresh_minmax(const CP& p, Smem& s) {
    if (threadIdx.x == 0) {
        s.qi.minv = ord2f(~__ldcg(p.ctrl + 4));
        s.qi.maxv = ord2f(__ldcg(p.ctrl + 5));
        if (!isfinite(s.qi.minv) || !isfinite(s.qi.maxv)) skml_set_status(p.status, SKML_BAD_INPUT, 0x35u);
    }
    __syncthreads();
}

__device__ __forceinline__ float bucket_value(const Smem& s, int b) {
    const QInfo& q = s.qi;
    if (q.bin_num == 1) return 0.5f * (q.minv + q.maxv);
    if (b == 0) return 0.5f * (q.minv + s.splits[0]);
    if (b == q.bin_num - 1) return 0.5f * (s.splits[q.nsplits - 1] + q.maxv);
    return 0.5f * (s.splits[b - 1] + s.splits[b]);
}

// ---------------------------------------------------------------------------
// Element stages. The unit of work of S3 and S4 is a warp: warp w of block b owns one contiguous
// slice of the (key-sorted) input. S5 works on the groups' contiguous lists in 1024-key chunks.
// ---------------------------------------------------------------------------
__device__ __forceinline__ long long vslice_size(long long n) {
    const long long nv = (long long)gridDim.x * SKML_WARPS;
    long long c = (n + nv - 1) / nv;
    return (c + 31) / 32 * 32;
}

__device__ __forceinline__ void build_group_lut(const CP& p, Smem& s) {
    for (int b = threadIdx.x; b < s.qi.bin_num; b += blockDim.x) s.grp_lut[b] = (unsigned char)skml_group_of(b, s.qi.edges, p.G);
    for (int t = threadIdx.x; t < SKML_WARPS * SKML_MAX_GROUPS; t += blockDim.x) (&s.wcnt[0][0])[t] = 0;
    __syncthreads();
}

// S3: bucket of every value; keys of every group in every warp slice.
__device__ void stage_count(const CP& p, Smem& s, long long n, bool track_minmax) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int kmin = 0xFFFFFFFFu, kmax = 0u;
    build_group_lut(p, s);
    const long long sub = vslice_size(n);
    const long long vb = (long long)blockIdx.x * SKML_WARPS + warp;
    long long lo = vb * sub, hi = lo + sub;
    if (lo > n) lo = n;
    if (hi > n) hi = n;
    float nval = 0.f;
    if (lo + lane < hi) nval = p.vals[lo + lane];  // one iteration ahead: the load latency stays off the chain
    for (long long i0 = lo; i0 < hi; i0 += 32) {
        const long long i = i0 + lane;
        const bool valid = i < hi;
        const float val = nval;
        if (i + 32 < hi) nval = p.vals[i + 32];
        int g = 63;
        if (valid) {
            const int bin = upper_bound_f(s.splits, s.qi.nsplits, val);
            p.bins[i] = (unsigned short)bin;
            g = s.grp_lut[bin];
            const unsigned int k = f2ord(val);
            kmin = min(kmin, k);
            kmax = max(kmax, k);
        }
        const unsigned int peers = __match_any_sync(0xFFFFFFFFu, g);
        if (valid && (peers & lanemask_lt()) == 0) s.wcnt[warp][g] += (unsigned int)__popc(peers);  // one leader per group
        __syncwarp();
    }
    if (lane < p.G) p.warp_cnt[vb * SKML_MAX_GROUPS + lane] = s.wcnt[warp][lane];
    __syncthreads();
    if (warp < p.G) {  // the block's totals: warp g adds up group g over the 32 slices
        const unsigned int tot = warp_sum(s.wcnt[lane][warp]);
        if (lane == 0) p.blk_cnt[(long long)blockIdx.x * SKML_MAX_GROUPS + warp] = tot;
    }
    if (track_minmax) {   // sample form: the extremes of all values (one pair of atomics per block)
        __shared__ unsigned int c_mn[SKML_WARPS], c_mx[SKML_WARPS];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            kmin = min(kmin, __shfl_xor_sync(0xFFFFFFFFu, kmin, o));
            kmax = max(kmax, __shfl_xor_sync(0xFFFFFFFFu, kmax, o));
        }
        if (lane == 0) {
            c_mn[warp] = kmin;
            c_mx[warp] = kmax;
        }
        __syncthreads();
        if (warp == 0) {
            kmin = c_mn[lane];
            kmax = c_mx[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                kmin = min(kmin, __shfl_xor_sync(0xFFFFFFFFu, kmin, o));
                kmax = max(kmax, __shfl_xor_sync(0xFFFFFFFFu, kmax, o));
            }
            if (lane == 0 && kmin <= kmax) {
                atomicMax(&p.ctrl[4], ~kmin);
                atomicMax(&p.ctrl[5], kmax);
            }
        }
    }
}

// S4 prelude: group sizes, table sizes, hash rows and every section offset that does not depend on
// the key code (every block computes the same layout); this block's and its warps' starting ranks.
__device__ void layout_from_counts(const CP& p, Smem& s) {
    const int G = p.G, nb = gridDim.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    Layout& L = s.lay;
    if (warp < G) {
        const int g = warp;
        // the blocks' totals (before this block / all blocks), lanes striding over the blocks; this
        // block's own 32 slices are scanned over the lanes for the warps' starting ranks
        unsigned int before = 0, total = 0;
        for (int b = lane; b < nb; b += 32) {
            const unsigned int c = __ldcg(&p.blk_cnt[(long long)b * SKML_MAX_GROUPS + g]);
            total += c;
            if (b < (int)blockIdx.x) before += c;
        }
        const unsigned int own = __ldcg(&p.warp_cnt[((long long)blockIdx.x * SKML_WARPS + lane) * SKML_MAX_GROUPS + g]);
        total = warp_sum(total);
        before = warp_sum(before);
        unsigned int inc = own;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += t;
        }
        s.wbase[lane][g] = inc - own;
        if (lane == 0) {
            L.n_g[g] = total;
            L.base_rank[g] = before;
        }
    }
    __syncthreads();
    if (threadIdx.x < G) {  // per-group divisions and hash draws, one thread each
        const int g = threadIdx.x;
        unsigned int col = 0;
        if (L.n_g[g]) {
            col = (unsigned int)ceil((double)L.n_g[g] * p.col_ratio);
            if (col < 1) col = 1;
        }
        L.col[g] = col;
        L.col_magic[g] = col ? skml_fastmod_magic(col) : 0ull;
        L.recip[g] = skml_recip32(col);
        skml_pick_hashes(p.seed, p.step, p.rank, (unsigned int)g, p.rows, L.hash_ids[g]);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        bool mix = p.rows <= 3;
        for (int g = 0; g < G && mix; ++g) mix = skml_rows_are_mixers(L.hash_ids[g], p.rows);
        L.mixers = mix ? 1 : 0;
        const int cb = s.qi.cell_bits;
        L.off_bv = SKML_HEADER_BYTES;
        L.off_gt = L.off_bv + skml_align16(4ull * p.q);
        L.off_flags = L.off_gt + (unsigned long long)SKML_GROUP_ENTRY_BYTES * G;
        const bool adaptive = p.key_encoder == SKML_KEYS_DELTA_ADAPTIVE;
        unsigned long long o = L.off_flags;
        unsigned int go = 0, ch = 0;
        for (int g = 0; g < G; ++g) {
            L.flag_off[g] = o;
            if (L.n_g[g] && !adaptive) o += skml_align16(8ull * ((2ull * L.n_g[g] + 63) / 64));
            L.goff[g] = go;
            go += (L.n_g[g] + 3u) & ~3u;
            L.chunk_prefix[g] = ch;
            ch += (L.n_g[g] + SKML_RESTART_INTERVAL - 1) / SKML_RESTART_INTERVAL;
        }
        L.chunk_prefix[G] = ch;
        L.off_restart = o;
        for (int g = 0; g < G; ++g) {
            L.restart_off[g] = o;
            if (L.n_g[g]) o += 16ull * ((L.n_g[g] + SKML_RESTART_INTERVAL - 1) / SKML_RESTART_INTERVAL);
        }
        L.off_tables = o;
        unsigned long long t32 = 0;
        for (int g = 0; g < G; ++g) {
            const unsigned int col = L.col[g];
            L.table_off[g] = o;
            L.tab32_off[g] = t32;
            o += skml_align16((unsigned long long)p.rows * col * (cb / 8));
            t32 += (unsigned long long)p.rows * col;
        }
        L.off_deltas = o;
        L.off_keys = o;  // delta_adaptive: both key sections of every group follow the tables
        // the key code adds at most four bytes per key (delta_adaptive: 49 bits): refuse now what cannot
        // fit in the worst case
        unsigned long long worst = o;
        for (int g = 0; g < G; ++g)
            worst += skml_align16(4ull * L.n_g[g] + 8) + (adaptive ? skml_align16(17ull * L.n_g[g] / 8 + 8) : 0ull);
        L.overflow = (worst > (unsigned long long)p.slot_capacity) || (t32 + 4 > (unsigned long long)p.tables_cap);
        if (L.overflow) skml_set_status(p.status, SKML_CAPACITY, 0x30u);
    }
    __syncthreads();
}

// S4: every key goes to its group's staging list (stable, so the lists stay sorted);
// grouped MinMaxSketch insert.
__device__ void stage_scatter(const CP& p, Smem& s, long long n) {
    const int G = p.G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const Layout& L = s.lay;
    if (L.overflow) return;
    build_group_lut(p, s);  // (also clears the per-iteration counters)
    const long long sub = vslice_size(n);
    const long long vb = (long long)blockIdx.x * SKML_WARPS + warp;
    long long lo = vb * sub, hi = lo + sub;
    if (lo > n) lo = n;
    if (hi > n) hi = n;
    const int zero = s.qi.zero_idx;
    unsigned int run = 0;   // lane g: staging position of the next key of group g in this slice
    if (lane < G) run = L.goff[lane] + L.base_rank[lane] + s.wbase[warp][lane];
    int nkey = 0, nbin = 0;
    if (lo + lane < hi) {
        nkey = p.keys[lo + lane];
        nbin = p.bins[lo + lane];
    }
    for (long long i0 = lo; i0 < hi; i0 += 32) {
        const long long i = i0 + lane;
        const bool valid = i < hi;
        const int key = nkey, bin = nbin;
        if (i + 32 < hi) {
            nkey = p.keys[i + 32];
            nbin = p.bins[i + 32];
        }
        const int g = valid ? (int)s.grp_lut[bin] : 63;
        const unsigned int peers = __match_any_sync(0xFFFFFFFFu, g);
        const unsigned int lower = peers & lanemask_lt();
        const unsigned int base = __shfl_sync(0xFFFFFFFFu, run, valid ? g : 0);
        if (valid) {
            if (lower == 0) s.wcnt[warp][g] = (unsigned int)__popc(peers);
            const unsigned int dst = base + (unsigned int)__popc(lower);
            p.gkeys[dst] = key;
            const unsigned int cell = skml_pack_cell(bin, zero);
            const int col = (int)L.col[g];
            unsigned int* tab = p.tables + L.tab32_off[g];
            int pos[SKML_MAX_ROWS];
            if (L.mixers) {
                skml_hash_rows_mixers<3>(L.hash_ids[g], p.rows, key, (unsigned int)col, L.recip[g], pos);
#pragma unroll
                for (int r = 0; r < 3; ++r)
                    if (r < p.rows) atomicMin(tab + (long long)r * col + pos[r], cell);
            } else if (p.rows <= 4) {
                skml_hash_rows<4>(L.hash_ids[g], p.rows, key, col, L.col_magic[g], pos);
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (r < p.rows) atomicMin(tab + (long long)r * col + pos[r], cell);
            } else {
                skml_hash_rows<SKML_MAX_ROWS>(L.hash_ids[g], p.rows, key, col, L.col_magic[g], pos);
#pragma unroll
                for (int r = 0; r < SKML_MAX_ROWS; ++r)
                    if (r < p.rows) atomicMin(tab + (long long)r * col + pos[r], cell);
            }
        }
        __syncwarp();
        if (lane < G) {
            run += s.wcnt[warp][lane];
            s.wcnt[warp][lane] = 0;
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------
// S5: delta-binary key code of the groups' lists. Chunks of 1024 keys are numbered group-major; a
// block owns a contiguous run of them and works on four at a time (one per 256-thread sub-block,
// four adjacent keys per thread).
// ---------------------------------------------------------------------------
struct ChunkWork {
    int g;                  // group, -1 = no chunk for this sub-block
    unsigned int j;         // chunk index inside the group
    unsigned int cnt;       // keys in the chunk
    int k[4];               // this thread's keys
    unsigned int w[4];      // their delta widths in bytes (0 = no key)
    unsigned int d[4];      // their deltas
    unsigned int wsum;
    int prev0;              // key before the chunk's first key (0 at the start of a group)
};

__device__ __forceinline__ void load_chunk(const CP& p, const Layout& L, unsigned int ch, unsigned int ch_end, int G, ChunkWork& c) {
    const int t = threadIdx.x & 255, lane = threadIdx.x & 31;
    c.g = -1;
    c.wsum = 0;
    c.cnt = 0;
    c.j = 0;
    c.prev0 = 0;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        c.w[u] = 0;
        c.d[u] = 0;
        c.k[u] = 0;
    }
    if (ch >= ch_end) return;
    int g = 0;
    while (g + 1 < G && ch >= L.chunk_prefix[g + 1]) ++g;
    c.g = g;
    c.j = ch - L.chunk_prefix[g];
    const unsigned int first = c.j * SKML_RESTART_INTERVAL;
    c.cnt = min((unsigned int)SKML_RESTART_INTERVAL, L.n_g[g] - first);
    const int* list = p.gkeys + L.goff[g];
    const unsigned int i0 = 4u * t;
    int4 kk = make_int4(0, 0, 0, 0);
    if (i0 < c.cnt) kk = *reinterpret_cast<const int4*>(list + first + i0);  // goff and first are multiples of 4
    c.k[0] = kk.x; c.k[1] = kk.y; c.k[2] = kk.z; c.k[3] = kk.w;
    // the key before this thread's first key: the lane below holds it, except at a warp's start
    int prev = __shfl_up_sync(0xFFFFFFFFu, c.k[3], 1);
    if (lane == 0) prev = (first + i0 > 0 && i0 < c.cnt) ? list[first + i0 - 1] : 0;
    if (t == 0) c.prev0 = first > 0 ? list[first - 1] : 0;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        if (i0 + u < c.cnt) {
            c.d[u] = (unsigned int)(c.k[u] - prev);
            c.w[u] = (unsigned int)skml_delta_bytes(c.d[u]);
            c.wsum += c.w[u];
            prev = c.k[u];
        }
    }
}

// Exclusive scan of `v` over the 256 threads of this thread's sub-block; `total` = the sub-block's sum.
// One block barrier inside; `par` alternates between calls.
__device__ __forceinline__ unsigned int sub_scan(Smem& s, unsigned int v, unsigned int& total) {
    const int lane = threadIdx.x & 31, sw = (threadIdx.x >> 5) & 7, sb = threadIdx.x >> 8;
    unsigned int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();  // the previous call's readers are done
    if (lane == 31) s.sub_part[sb][sw] = inc;
    __syncthreads();
    unsigned int base = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const unsigned int x = s.sub_part[sb][w];
        if (w < sw) base += x;
        tot += x;
    }
    total = tot;
    return base + inc - v;
}

// Pass A: byte counts of this block's chunks -> chunk offsets inside the block's part of each group,
// the block's byte totals per group (published for the blocks after it).
__device__ void pack_measure(const CP& p, Smem& s, unsigned int my_begin, unsigned int my_end) {
    const Layout& L = s.lay;
    if (threadIdx.x < SKML_MAX_GROUPS) s.my_bytes[threadIdx.x] = 0;
    __syncthreads();
    for (unsigned int c0 = my_begin; c0 < my_end; c0 += 4) {
        ChunkWork c;
        load_chunk(p, L, c0 + (threadIdx.x >> 8), my_end, p.G, c);
        unsigned int total;
        sub_scan(s, c.wsum, total);
        if ((threadIdx.x & 255) == 0) s.sub_total[threadIdx.x >> 8] = total;
        __syncthreads();
        if (threadIdx.x == 0) {  // the four chunks of this round, in order
            for (int q = 0; q < 4 && c0 + q < my_end; ++q) {
                int g = 0;
                while (g + 1 < p.G && c0 + q >= L.chunk_prefix[g + 1]) ++g;
                p.chunk_off[c0 + q] = (unsigned int)s.my_bytes[g];
                s.my_bytes[g] += s.sub_total[q];
            }
        }
        __syncthreads();
    }
    if (threadIdx.x < SKML_MAX_GROUPS) p.blk_bytes[(long long)blockIdx.x * SKML_MAX_GROUPS + threadIdx.x] = s.my_bytes[threadIdx.x];
}

// Byte totals of the blocks before this one (they own the chunks before this block's run, so the
// sums give this block's starting offsets and the sizes of all earlier groups).
__device__ void pack_prefix(const CP& p, Smem& s, bool wait, unsigned int epoch) {
    if (threadIdx.x < SKML_MAX_GROUPS) s.pre_bytes[threadIdx.x] = 0;
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < blockIdx.x) {
        const unsigned int b = threadIdx.x;
        bool ok = true;
        if (wait) {
            const long long t0 = clock64();
            unsigned int ns = 20;
            while (ld_acquire_gpu(&p.blk_flag[b]) != epoch) {
                if (clock64() - t0 > p.budget) {
                    skml_set_status(p.status, SKML_TIMEOUT_BARRIER, 0x50u);
                    ok = false;
                    break;
                }
                __nanosleep(ns);
                if (ns < 400) ns *= 2;
            }
        }
        if (ok) {
            for (int g = 0; g < p.G; ++g) {
                const unsigned long long v = __ldcg(&p.blk_bytes[(long long)b * SKML_MAX_GROUPS + g]);
                if (v) atomicAdd(&s.pre_bytes[g], v);
            }
        } else {
            s_ok = 0;
        }
    }
    __syncthreads();
    Layout& L = s.lay;
    if (threadIdx.x == 0) {
        // section starts of the groups this block can reach: all earlier groups are complete in pre_bytes
        // (plus this block's own part of the group its run starts in)
        unsigned long long o = L.off_deltas;
        for (int g = 0; g < p.G; ++g) {
            L.delta_off[g] = o;
            const unsigned long long bytes = s.pre_bytes[g] + s.my_bytes[g];
            if (L.n_g[g]) o += skml_align16(8ull * ((bytes + 7) / 8));
        }
        if (!s_ok) L.overflow = 1;
    }
    __syncthreads();
}

// Pass B: flag bytes, delta bytes and restart points of this block's chunks.
__device__ void pack_write(const CP& p, Smem& s, unsigned int my_begin, unsigned int my_end) {
    const Layout& L = s.lay;
    if (L.overflow) return;
    const int t = threadIdx.x & 255;
    for (unsigned int c0 = my_begin; c0 < my_end; c0 += 4) {
        ChunkWork c;
        const unsigned int ch = c0 + (threadIdx.x >> 8);
        load_chunk(p, L, ch, my_end, p.G, c);
        unsigned int total;
        const unsigned int boff = sub_scan(s, c.wsum, total);
        if (c.g < 0) continue;  // (no barrier follows in this iteration)
        const int g = c.g;
        const unsigned int first = c.j * SKML_RESTART_INTERVAL, i0 = 4u * t;
        const unsigned long long chunk_off = s.pre_bytes[g] + __ldcg(&p.chunk_off[ch]);
        // flags: (w - 1) most significant bit first at stream bits 2i, 2i+1 -> one byte per four keys
        // (a group's last chunk also writes the zero padding up to the section's 16-byte end: there the
        // threads beyond the last key hold widths of zero)
        const unsigned long long flag_bytes = skml_align16(8ull * ((2ull * L.n_g[g] + 63) / 64));
        const unsigned long long fbyte = first / 4 + t;
        if (fbyte < flag_bytes) {
            unsigned int fb = 0;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const unsigned int fv = c.w[u] ? c.w[u] - 1u : 0u;
                fb |= (((fv >> 1) & 1u) | ((fv & 1u) << 1)) << (2 * u);
            }
            p.payload[L.flag_off[g] + fbyte] = (unsigned char)fb;
        }
        if (i0 < c.cnt) {
            unsigned char* dst = p.payload + L.delta_off[g] + chunk_off + boff;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                for (unsigned int j = 0; j < c.w[u]; ++j) dst[j] = skml_delta_stream_byte(c.d[u], (int)c.w[u], (int)j);
                dst += c.w[u];
            }
        }
        if (t == 0 && c.j + 1 == (L.n_g[g] + SKML_RESTART_INTERVAL - 1) / SKML_RESTART_INTERVAL) {
            // the group's last chunk: clear the padding between the last delta byte and the section's end
            const unsigned long long endb = chunk_off + total;
            for (unsigned long long a = endb; a < skml_align16(8ull * ((endb + 7) / 8)); ++a) p.payload[L.delta_off[g] + a] = 0;
        }
        if (t == 0) {
            SkmlRestart r;
            r.prev_key = (unsigned int)c.prev0;
            r.flag_bit_off = 2u * first;
            r.delta_bit_off = 8ull * chunk_off;
            *reinterpret_cast<SkmlRestart*>(p.payload + L.restart_off[g] + (unsigned long long)c.j * sizeof(SkmlRestart)) = r;
        }
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------
// S5, DeltaAdaptive key code (the reference's live encoder, binary/DeltaAdaptiveEncoder.java:23-112).
// Flags and deltas are bit streams: per group, every delta takes b * iv bits (b = 32 / m bits per
// interval, iv = intervals needed) and a flag of log2(m) bits holding iv - 1, or iv one-bits and a
// zero-bit ("unary" flags); m and the flag kind minimise the estimated bits per key over the group's
// histogram of delta widths. Chunk starts are therefore bit positions, adjacent chunks share stream
// words, and the sections' sizes depend on the data: the two sections of a group follow each other
// at the end of the payload, and the (pre-zeroed) shared words are completed with atomic ORs.
// ---------------------------------------------------------------------------
__device__ void push_bytes(const CP& p, unsigned long long lo, unsigned long long hi);

__device__ __forceinline__ int da_bits_needed(unsigned int d) { return d == 0u ? 1 : 32 - __clz(d); }

// The reference's mode search in the same double arithmetic, operation by operation (explicit
// round-to-nearest intrinsics keep the compiler from fusing multiply-adds); hist[k] = keys needing k bits.
__device__ void da_choose(const unsigned int* hist, unsigned int n, unsigned int& num, unsigned int& kind) {
    double prob[32];
    const double dn = (double)(n > 0 ? n : 1);
    for (int k = 0; k < 32; ++k) prob[k] = __ddiv_rn((double)hist[k], dn);
    double best = 32.0;
    num = 1;
    kind = 0;
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
}

// Pass 0: histogram of the delta widths of this block's chunks, per group, added to the global one.
__device__ void apack_histogram(const CP& p, Smem& s, unsigned int my_begin, unsigned int my_end) {
    const Layout& L = s.lay;
    unsigned int* hist = s.cs.stage_d[0];  // [G][32], the staging area is idle in this pass
    for (int t = threadIdx.x; t < SKML_MAX_GROUPS * 32; t += blockDim.x) hist[t] = 0;
    __syncthreads();
    for (unsigned int c0 = my_begin; c0 < my_end; c0 += 4) {
        ChunkWork c;
        load_chunk(p, L, c0 + (threadIdx.x >> 8), my_end, p.G, c);
        if (c.g >= 0) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (c.w[u]) atomicAdd(&hist[c.g * 32 + (da_bits_needed(c.d[u]) & 31)], 1u);
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < p.G * 32; t += blockDim.x)
        if (hist[t]) atomicAdd(&p.key_hist[t], hist[t]);
}

__device__ __forceinline__ unsigned long long stream_bytes(unsigned long long bits) { return skml_align16(8ull * ((bits + 63) / 64)); }

// Pass 1 prelude (every block): interval count and flag kind of every group from the complete
// histogram. The histogram also gives the exact lengths of the two bit streams of every group, so the
// whole layout of the key sections is known here, before a single key is coded.
__device__ void apack_choose(const CP& p, Smem& s) {
    Layout& L = s.lay;
    if (threadIdx.x < p.G) {
        const int g = threadIdx.x;
        unsigned int h[32];
        for (int k = 0; k < 32; ++k) h[k] = __ldcg(&p.key_hist[g * 32 + k]);
        unsigned int num = 1, kind = 0;
        da_choose(h, L.n_g[g], num, kind);
        L.num_iv[g] = num;
        L.flag_kind[g] = kind;
        const unsigned int b = 32u / num, fb = 31u - (unsigned int)__clz(num);
        unsigned long long fbits = 0, dbits = 0;
        for (unsigned int k = 0; k < 32; ++k) {
            const unsigned int need = k ? k : 32u;   // bin 0 holds the 32-bit deltas (need & 31)
            const unsigned long long iv = (need + b - 1) / b;
            fbits += (unsigned long long)h[k] * (kind ? iv + 1 : fb);
            dbits += (unsigned long long)h[k] * b * iv;
        }
        L.flag_bits[g] = fbits;
        L.delta_bits[g] = dbits;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long o = L.off_keys;
        for (int g = 0; g < p.G; ++g) {
            L.flag_off[g] = o;
            if (L.n_g[g]) o += stream_bytes(L.flag_bits[g]);
            L.delta_off[g] = o;
            if (L.n_g[g]) o += stream_bytes(L.delta_bits[g]);
        }
        L.total_bytes = o;
        if (o > (unsigned long long)p.slot_capacity) {
            L.overflow = 1;
            skml_set_status(p.status, SKML_CAPACITY, 0x37u);
        }
    }
    __syncthreads();
}

struct KeyCode {
    unsigned int fv, fw, dw;  // flag value / width, delta width (the delta value is the delta itself)
};
__device__ __forceinline__ KeyCode da_code(unsigned int d, unsigned int m, unsigned int kind) {
    const int b = 32 / (int)m, fb = 31 - __clz(m);
    const int iv = (da_bits_needed(d) + b - 1) / b;
    KeyCode k;
    k.fw = kind ? (unsigned int)(iv + 1) : (unsigned int)fb;
    k.fv = kind ? ((1u << (iv + 1)) - 2u) : (unsigned int)(iv - 1);
    k.dw = (unsigned int)(b * iv);
    return k;
}

// Writes `nb` (<= 32) bits of `value`, most significant first, at bit offset `off` of a zeroed
// shared-memory word array (stream bit p = bit (p & 31) of word p >> 5, as in java.util.BitSet).
__device__ __forceinline__ void put_bits_shared(unsigned int* words, unsigned int off, unsigned int value, unsigned int nb) {
    if (nb == 0) return;
    const unsigned int rv = __brev(value) >> (32u - nb);
    const unsigned int sh = off & 31u, w = off >> 5;
    atomicOr(&words[w], rv << sh);
    if (sh + nb > 32u) atomicOr(&words[w + 1], rv >> (32u - sh));
}

// Pass 1: flag and delta bits of this block's chunks -> chunk bit offsets inside the block's part of
// each group, the block's bit totals per group (published for the blocks after it).
__device__ void apack_measure(const CP& p, Smem& s, unsigned int my_begin, unsigned int my_end) {
    const Layout& L = s.lay;
    if (threadIdx.x < 2 * SKML_MAX_GROUPS) s.my_bits[threadIdx.x] = 0;
    __syncthreads();
    for (unsigned int c0 = my_begin; c0 < my_end; c0 += 4) {
        ChunkWork c;
        load_chunk(p, L, c0 + (threadIdx.x >> 8), my_end, p.G, c);
        unsigned int packed = 0;  // flag bits (<= 17408 per chunk) in the low half, delta bits (<= 32768) above
        if (c.g >= 0) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (c.w[u]) {
                    const KeyCode k = da_code(c.d[u], L.num_iv[c.g], L.flag_kind[c.g]);
                    packed += k.fw + (k.dw << 16);
                }
        }
        unsigned int total;
        sub_scan(s, packed, total);
        if ((threadIdx.x & 255) == 0) s.sub_total[threadIdx.x >> 8] = total;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int q = 0; q < 4 && c0 + q < my_end; ++q) {
                int g = 0;
                while (g + 1 < p.G && c0 + q >= L.chunk_prefix[g + 1]) ++g;
                p.chunk_off[2 * (c0 + q)] = (unsigned int)s.my_bits[2 * g];
                p.chunk_off[2 * (c0 + q) + 1] = (unsigned int)s.my_bits[2 * g + 1];
                s.my_bits[2 * g] += s.sub_total[q] & 0xFFFFu;
                s.my_bits[2 * g + 1] += s.sub_total[q] >> 16;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x < 2 * SKML_MAX_GROUPS) p.blk_bits[(long long)blockIdx.x * 2 * SKML_MAX_GROUPS + threadIdx.x] = s.my_bits[threadIdx.x];
}

// Bit totals of the blocks before this one -> this block's starting bit offsets inside the streams.
__device__ void apack_prefix(const CP& p, Smem& s, bool wait, unsigned int epoch) {
    if (threadIdx.x < 2 * SKML_MAX_GROUPS) s.pre_bits[threadIdx.x] = 0;
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < blockIdx.x) {
        const unsigned int b = threadIdx.x;
        bool ok = true;
        if (wait) {
            const long long t0 = clock64();
            unsigned int ns = 20;
            while (ld_acquire_gpu(&p.blk_flag[b]) != epoch) {
                if (clock64() - t0 > p.budget) {
                    skml_set_status(p.status, SKML_TIMEOUT_BARRIER, 0x52u);
                    ok = false;
                    break;
                }
                __nanosleep(ns);
                if (ns < 400) ns *= 2;
            }
        }
        if (ok) {
            for (int g = 0; g < 2 * p.G; ++g) {
                const unsigned long long v = __ldcg(&p.blk_bits[(long long)b * 2 * SKML_MAX_GROUPS + g]);
                if (v) atomicAdd(&s.pre_bits[g], v);
            }
        } else {
            s_ok = 0;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && !s_ok) s.lay.overflow = 1;
    __syncthreads();
}

// One stream segment staged in shared memory -> the payload: whole words are stored, the first and
// the last word may be shared with the neighbouring chunks and are completed with atomic ORs.
__device__ __forceinline__ void flush_stream(unsigned int* dst_words, const unsigned int* stage, unsigned long long start_bit,
                                             unsigned int nbits) {
    if (nbits == 0) return;
    const unsigned int sh = (unsigned int)(start_bit & 31ull);
    const unsigned int nw = (sh + nbits + 31u) >> 5;
    unsigned int* dst = dst_words + (start_bit >> 5);
    for (unsigned int w = threadIdx.x & 255; w < nw; w += 256) {
        const unsigned int v = stage[w];
        const bool shared_word = (w == 0 && sh != 0) || (w == nw - 1 && ((sh + nbits) & 31u) != 0);
        if (shared_word) {
            if (v) atomicOr(dst + w, v);
        } else {
            dst[w] = v;
        }
    }
}

// Pass 2: the bit streams and restart points of this block's chunks.
__device__ void apack_write(const CP& p, Smem& s, unsigned int my_begin, unsigned int my_end) {
    const Layout& L = s.lay;
    if (L.overflow) return;
    const int t = threadIdx.x & 255, sb = threadIdx.x >> 8;
    for (unsigned int c0 = my_begin; c0 < my_end; c0 += 4) {
        ChunkWork c;
        const unsigned int ch = c0 + sb;
        load_chunk(p, L, ch, my_end, p.G, c);
        KeyCode kc[4];
        unsigned int packed = 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            kc[u].fv = kc[u].fw = kc[u].dw = 0;
            if (c.g >= 0 && c.w[u]) {
                kc[u] = da_code(c.d[u], L.num_iv[c.g], L.flag_kind[c.g]);
                packed += kc[u].fw + (kc[u].dw << 16);
            }
        }
        for (int i = t; i < AP_STAGE_F; i += 256) s.cs.stage_f[sb][i] = 0;
        for (int i = t; i < AP_STAGE_D; i += 256) s.cs.stage_d[sb][i] = 0;
        unsigned int total;
        const unsigned int ex = sub_scan(s, packed, total);  // (its barriers also publish the cleared staging words)
        unsigned long long fs = 0, ds = 0;
        if (c.g >= 0) {
            fs = s.pre_bits[2 * c.g] + __ldcg(&p.chunk_off[2 * ch]);
            ds = s.pre_bits[2 * c.g + 1] + __ldcg(&p.chunk_off[2 * ch + 1]);
            unsigned int fo = (unsigned int)(fs & 31ull) + (ex & 0xFFFFu), dof = (unsigned int)(ds & 31ull) + (ex >> 16);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                put_bits_shared(s.cs.stage_f[sb], fo, kc[u].fv, kc[u].fw);
                put_bits_shared(s.cs.stage_d[sb], dof, c.d[u], kc[u].dw);
                fo += kc[u].fw;
                dof += kc[u].dw;
            }
        }
        __syncthreads();
        if (c.g >= 0) {
            flush_stream(reinterpret_cast<unsigned int*>(p.payload + L.flag_off[c.g]), s.cs.stage_f[sb], fs, total & 0xFFFFu);
            flush_stream(reinterpret_cast<unsigned int*>(p.payload + L.delta_off[c.g]), s.cs.stage_d[sb], ds, total >> 16);
            if (t == 0) {
                SkmlRestart r;
                r.prev_key = (unsigned int)c.prev0;
                r.flag_bit_off = (unsigned int)fs;
                r.delta_bit_off = ds;
                *reinterpret_cast<SkmlRestart*>(p.payload + L.restart_off[c.g] + (unsigned long long)c.j * sizeof(SkmlRestart)) = r;
            }
        }
        __syncthreads();  // the staging words are cleared again by the next round
    }
}

// The restart points and the 16-byte units of the two bit streams that hold bits of this block only
// -> the peers' slots. Units that hold a block border are sent by block 0 once every block is done.
__device__ void apush_own_chunks(const CP& p, Smem& s, unsigned int my_begin, unsigned int my_end) {
    const Layout& L = s.lay;
    if (p.world <= 1 || L.overflow || my_begin >= my_end) return;
    __syncthreads();
    for (int g = 0; g < p.G; ++g) {
        const unsigned int c0 = max(my_begin, L.chunk_prefix[g]), c1 = min(my_end, L.chunk_prefix[g + 1]);
        if (c0 >= c1) continue;
        const bool last = c1 == L.chunk_prefix[g + 1];
        push_bytes(p, L.restart_off[g] + 16ull * (c0 - L.chunk_prefix[g]), L.restart_off[g] + 16ull * (c1 - L.chunk_prefix[g]));
        for (int k = 0; k < 2; ++k) {
            const unsigned long long a = s.pre_bits[2 * g + k], b = a + s.my_bits[2 * g + k];
            const unsigned long long lo = 16ull * ((a + 127) / 128), hi = last ? stream_bytes(k ? L.delta_bits[g] : L.flag_bits[g]) : 16ull * (b / 128);
            const unsigned long long base = k ? L.delta_off[g] : L.flag_off[g];
            if (hi > lo) push_bytes(p, base + lo, base + hi);
        }
    }
}

// Block 0, after every block has written its chunks: the stream units that hold a block border.
__device__ void apush_borders(const CP& p, Smem& s) {
    const Layout& L = s.lay;
    if (p.world <= 1 || L.overflow) return;
    const unsigned int total = L.chunk_prefix[p.G];
    unsigned int per = (total + gridDim.x - 1) / gridDim.x;
    per = (per + 3u) & ~3u;
    const unsigned int b = threadIdx.x;
    if (b >= 1 && b < gridDim.x && (unsigned long long)per * b < total) {
        const unsigned int cs = per * b;
        int g = 0;
        while (g + 1 < p.G && cs >= L.chunk_prefix[g + 1]) ++g;
        if (cs != L.chunk_prefix[g]) {  // the run of block b starts inside group g
            unsigned long long a[2] = {0, 0};
            for (unsigned int q = 0; q < b; ++q) {
                a[0] += __ldcg(&p.blk_bits[(long long)q * 2 * SKML_MAX_GROUPS + 2 * g]);
                a[1] += __ldcg(&p.blk_bits[(long long)q * 2 * SKML_MAX_GROUPS + 2 * g + 1]);
            }
            for (int k = 0; k < 2; ++k) {
                if ((a[k] & 127ull) == 0) continue;
                const unsigned long long off = (k ? L.delta_off[g] : L.flag_off[g]) + 16ull * (a[k] / 128);
                const uint4 v = ld_cg_v4(reinterpret_cast<const uint4*>(p.payload + off));
                for (unsigned int r = 0; r < p.world; ++r)
                    if (r != p.rank && p.peer_payload[r]) st_v4(reinterpret_cast<uint4*>(p.peer_payload[r] + off), v);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// S5, Huffman-coded sketch tables (cell_bits = 0; the reference codes every table this way when it
// serialises a sketch: sketch/frequency/MinMaxSketch.java:88-97, binary/HuffmanEncoder.java:88-124).
// Section of one group: u32 {items, 64-bit words, cells, restart interval}; items x {i32 value,
// i32 code, i32 code length}, ascending by value; the code stream (most significant bit first in
// java.util.BitSet order); then, 16-byte aligned, one u32 stream offset per 128 cells (not in the
// reference: it lets a decoder start anywhere). The symbols of a group are the buckets of its range
// plus the "never written" cell (Integer.MAX_VALUE), at most HUF_MAX_SYMS of them. Any prefix code is
// valid on the wire (the items carry the codes); the coder builds an optimal one from the cell
// histogram and assigns canonical code words.
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned int huf_slot(const Layout& L, int g, unsigned int cell) {
    const unsigned int sidx = cell == SKML_EMPTY_CELL ? L.nsym[g] - 1u : (cell & 0xFFFFu) - L.sym_lo[g];
    return L.sym_lo[g] + (unsigned int)g + (sidx < L.nsym[g] ? sidx : L.nsym[g] - 1u);
}

// Table chunks (1024 cells of one group's table, group-major) of this block: a contiguous run.
__device__ __forceinline__ void tchunk_run(const Layout& L, int G, unsigned int& t_begin, unsigned int& t_end) {
    const unsigned int total = L.tchunk_prefix[G];
    unsigned int per = (total + gridDim.x - 1) / gridDim.x;
    per = (per + 3u) & ~3u;
    t_begin = min(total, per * blockIdx.x);
    t_end = min(total, t_begin + per);
}

struct CellWork {
    int g;
    unsigned int j, cnt;      // chunk index inside the group's table, cells in the chunk
    unsigned int cell[4];     // this thread's cells (32-bit working form)
};

__device__ __forceinline__ void load_cells(const CP& p, const Layout& L, unsigned int ch, unsigned int ch_end, int G, CellWork& c) {
    const unsigned int t = threadIdx.x & 255;
    c.g = -1;
    c.cnt = 0;
    c.j = 0;
    if (ch >= ch_end) return;
    int g = 0;
    while (g + 1 < G && ch >= L.tchunk_prefix[g + 1]) ++g;
    c.g = g;
    c.j = ch - L.tchunk_prefix[g];
    const unsigned int first = c.j * 1024u;
    c.cnt = min(1024u, L.cells[g] - first);
    const unsigned int* tab = p.tables + L.tab32_off[g] + first;
#pragma unroll
    for (int u = 0; u < 4; ++u) c.cell[u] = 4u * t + u < c.cnt ? __ldcg(tab + 4u * t + u) : SKML_EMPTY_CELL;
}

// Symbol ranges, cell counts and table chunks of the groups (every block, thread 0).
__device__ void huf_ranges(const CP& p, Smem& s) {
    Layout& L = s.lay;
    if (threadIdx.x == 0) {
        unsigned int ch = 0;
        for (int g = 0; g < p.G; ++g) {
            const int lo = g ? s.qi.edges[g - 1] : 0, hi = s.qi.edges[g];
            L.sym_lo[g] = (unsigned int)lo;
            L.nsym[g] = (unsigned int)(hi > lo ? hi - lo : 0) + 1u;
            L.cells[g] = (unsigned int)p.rows * L.col[g];
            L.tchunk_prefix[g] = ch;
            ch += (L.cells[g] + 1023u) / 1024u;
            if (L.n_g[g] && L.nsym[g] > HUF_MAX_SYMS) {
                L.overflow = 1;
                skml_set_status(p.status, SKML_BAD_INPUT, 0x38u);
            }
        }
        L.tchunk_prefix[p.G] = ch;
    }
    __syncthreads();
}

// Pass 0: histogram of the cell symbols of this block's table chunks, added to the global one.
__device__ void huf_histogram(const CP& p, Smem& s, unsigned int t_begin, unsigned int t_end) {
    const Layout& L = s.lay;
    unsigned int* hist = s.cs.huf_code;  // idle until the codes are built
    for (int t = threadIdx.x; t < SKML_GPU_MAX_BINS + SKML_MAX_GROUPS; t += blockDim.x) hist[t] = 0;
    __syncthreads();
    for (unsigned int c0 = t_begin; c0 < t_end; c0 += 4) {
        CellWork c;
        load_cells(p, L, c0 + (threadIdx.x >> 8), t_end, p.G, c);
        if (c.g >= 0) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (4u * (threadIdx.x & 255) + u < c.cnt) atomicAdd(&hist[huf_slot(L, c.g, c.cell[u])], 1u);
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < s.qi.bin_num + p.G; t += blockDim.x)
        if (hist[t]) atomicAdd(&p.cell_hist[t], hist[t]);
    __syncthreads();
}

// Optimal prefix code of every group from the complete histogram (every block; one warp per group,
// eight groups at a time), canonical code words, section sizes and the layout that follows the tables.
__device__ void huf_build(const CP& p, Smem& s) {
    Layout& L = s.lay;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    HufScratch* scratch = s.cs.huf_scratch;
    for (int t = threadIdx.x; t < SKML_GPU_MAX_BINS + SKML_MAX_GROUPS; t += blockDim.x) {
        s.cs.huf_len[t] = 0;
        s.cs.huf_code[t] = 0;
    }
    __syncthreads();
    if (warp < 8 && !L.overflow) {
        HufScratch& h = scratch[warp];
        for (int g = warp; g < p.G; g += 8) {
            const unsigned int n = L.nsym[g], base = L.sym_lo[g] + (unsigned int)g;
            if (L.n_g[g] == 0) {
                if (lane == 0) {
                    L.items[g] = 0;
                    L.tbits[g] = 0;
                }
                continue;
            }
            // rank sort of the present symbols by (count, symbol): every lane ranks its symbols
            unsigned int m = 0;
            for (unsigned int a = lane; a < n; a += 32) m += __ldcg(&p.cell_hist[base + a]) ? 1u : 0u;
            m = warp_sum(m);
            for (unsigned int a = lane; a < n; a += 32) {
                const unsigned int ca = __ldcg(&p.cell_hist[base + a]);
                if (!ca) continue;
                unsigned int r = 0;
                for (unsigned int b = 0; b < n; ++b) {
                    const unsigned int cb = __ldcg(&p.cell_hist[base + b]);
                    if (cb && (cb < ca || (cb == ca && b < a))) ++r;
                }
                h.ord[r] = (unsigned short)a;
                h.w[r] = ca;
            }
            __syncwarp();
            if (lane == 0) {
                unsigned long long bits = 0;
                if (m == 1) {
                    s.cs.huf_len[base + h.ord[0]] = 1;   // a single symbol gets the one-bit code 0
                    s.cs.huf_code[base + h.ord[0]] = 0;
                    bits = h.w[0];
                } else {
                    // two-queue construction: leaves and internal nodes are both consumed in ascending weight
                    unsigned int li = 0, ii = 0, ni = 0;
                    while (ni + 1 < m) {
                        unsigned int wsum = 0;
                        for (int k = 0; k < 2; ++k) {
                            const bool take_leaf = li < m && (ii >= ni || h.w[li] <= h.iw[ii]);
                            if (take_leaf) {
                                wsum += h.w[li];
                                h.pl[li++] = (unsigned short)ni;
                            } else {
                                wsum += h.iw[ii];
                                h.pi[ii++] = (unsigned short)ni;
                            }
                        }
                        h.iw[ni++] = wsum;
                    }
                    h.di[ni - 1] = 0;  // the root
                    for (int j = (int)ni - 2; j >= 0; --j) h.di[j] = (unsigned char)(h.di[h.pi[j]] + 1);
                    unsigned int per_len[33];
                    for (int k = 0; k < 33; ++k) per_len[k] = 0;
                    unsigned int longest = 0;
                    for (unsigned int i = 0; i < m; ++i) {
                        const unsigned int len = (unsigned int)h.di[h.pl[i]] + 1u;
                        s.cs.huf_len[base + h.ord[i]] = (unsigned char)(len < 32 ? len : 32);
                        if (len < 33) ++per_len[len];
                        longest = max(longest, len);
                        bits += (unsigned long long)h.w[i] * len;
                    }
                    if (longest > 31) {
                        L.overflow = 1;
                        skml_set_status(p.status, SKML_BAD_INPUT, 0x39u);
                    }
                    // canonical code words: lengths ascending, symbols ascending inside a length
                    unsigned int next[33], code = 0;
                    for (int k = 1; k < 33; ++k) {
                        next[k] = code;
                        code = (code + per_len[k]) << 1;
                    }
                    for (unsigned int a = 0; a < n; ++a) {
                        const unsigned int len = s.cs.huf_len[base + a];
                        if (len && len < 32) s.cs.huf_code[base + a] = next[len]++;
                    }
                }
                L.items[g] = m;
                L.tbits[g] = bits;
            }
            __syncwarp();
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long o = L.off_tables;
        for (int g = 0; g < p.G; ++g) {
            L.table_off[g] = o;
            if (L.n_g[g]) {
                const unsigned long long stream = o + 16ull + 12ull * L.items[g];
                L.tstream_off[g] = stream;
                L.trestart_off[g] = skml_align16(stream + 8ull * ((L.tbits[g] + 63) / 64));
                o = skml_align16(L.trestart_off[g] + 4ull * ((L.cells[g] + HUF_RESTART - 1) / HUF_RESTART));
            }
        }
        L.off_deltas = o;
        L.off_keys = o;
        unsigned long long worst = o;
        const bool adaptive = p.key_encoder == SKML_KEYS_DELTA_ADAPTIVE;
        for (int g = 0; g < p.G; ++g)
            worst += skml_align16(4ull * L.n_g[g] + 8) + (adaptive ? skml_align16(17ull * L.n_g[g] / 8 + 8) : 0ull);
        if (worst > (unsigned long long)p.slot_capacity && !L.overflow) {
            L.overflow = 1;
            skml_set_status(p.status, SKML_CAPACITY, 0x3Au);
        }
    }
    __syncthreads();
}

// Pass 1: code bits of this block's table chunks -> chunk offsets inside the block's part of each
// group's stream, the block's bit totals per group (published with the key counts).
__device__ void huf_measure(const CP& p, Smem& s, unsigned int t_begin, unsigned int t_end) {
    const Layout& L = s.lay;
    if (threadIdx.x < SKML_MAX_GROUPS) s.my_tbits[threadIdx.x] = 0;
    __syncthreads();
    for (unsigned int c0 = t_begin; c0 < t_end; c0 += 4) {
        CellWork c;
        load_cells(p, L, c0 + (threadIdx.x >> 8), t_end, p.G, c);
        unsigned int bits = 0;
        if (c.g >= 0) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (4u * (threadIdx.x & 255) + u < c.cnt) bits += s.cs.huf_len[huf_slot(L, c.g, c.cell[u])];
        }
        unsigned int total;
        sub_scan(s, bits, total);
        if ((threadIdx.x & 255) == 0) s.sub_total[threadIdx.x >> 8] = total;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int q = 0; q < 4 && c0 + q < t_end; ++q) {
                int g = 0;
                while (g + 1 < p.G && c0 + q >= L.tchunk_prefix[g + 1]) ++g;
                p.tchunk_off[c0 + q] = (unsigned int)s.my_tbits[g];
                s.my_tbits[g] += s.sub_total[q];
            }
        }
        __syncthreads();
    }
    if (threadIdx.x < SKML_MAX_GROUPS) p.blk_tbits[(long long)blockIdx.x * SKML_MAX_GROUPS + threadIdx.x] = s.my_tbits[threadIdx.x];
}

// Table bits of the blocks before this one (the caller has waited for their publications).
__device__ void huf_prefix(const CP& p, Smem& s) {
    if (threadIdx.x < SKML_MAX_GROUPS) s.pre_tbits[threadIdx.x] = 0;
    __syncthreads();
    if (threadIdx.x < blockIdx.x) {
        for (int g = 0; g < p.G; ++g) {
            const unsigned long long v = __ldcg(&p.blk_tbits[(long long)threadIdx.x * SKML_MAX_GROUPS + g]);
            if (v) atomicAdd(&s.pre_tbits[g], v);
        }
    }
    __syncthreads();
}

// Pass 2: code streams and restart offsets of this block's table chunks; section head and items by
// the block that owns a group's first chunk.
__device__ void huf_write(const CP& p, Smem& s, unsigned int t_begin, unsigned int t_end) {
    const Layout& L = s.lay;
    if (L.overflow) return;
    const int t = threadIdx.x & 255, sb = threadIdx.x >> 8;
    for (unsigned int c0 = t_begin; c0 < t_end; c0 += 4) {
        CellWork c;
        const unsigned int ch = c0 + sb;
        load_cells(p, L, ch, t_end, p.G, c);
        unsigned int len[4], code[4], bits = 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            len[u] = code[u] = 0;
            if (c.g >= 0 && 4u * t + u < c.cnt) {
                const unsigned int slot = huf_slot(L, c.g, c.cell[u]);
                len[u] = s.cs.huf_len[slot];
                code[u] = s.cs.huf_code[slot];
                bits += len[u];
            }
        }
        for (int i = t; i < AP_STAGE_D; i += 256) s.cs.stage_d[sb][i] = 0;
        unsigned int total;
        const unsigned int ex = sub_scan(s, bits, total);
        unsigned long long start = 0;
        if (c.g >= 0) {
            start = s.pre_tbits[c.g] + __ldcg(&p.tchunk_off[ch]);
            unsigned int off = (unsigned int)(start & 31ull) + ex;
            if (4u * t < c.cnt && ((c.j * 1024u + 4u * t) % HUF_RESTART) == 0)
                reinterpret_cast<unsigned int*>(p.payload + L.trestart_off[c.g])[(c.j * 1024u + 4u * t) / HUF_RESTART] =
                    (unsigned int)(start + ex);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                put_bits_shared(s.cs.stage_d[sb], off, code[u], len[u]);
                off += len[u];
            }
        }
        __syncthreads();
        if (c.g >= 0) {
            flush_stream(reinterpret_cast<unsigned int*>(p.payload + L.tstream_off[c.g]), s.cs.stage_d[sb], start, total);
            if (c.j == 0) {
                // this sub-block owns the group's first chunk: section head and items (ascending by value)
                const int g = c.g;
                unsigned int* head = reinterpret_cast<unsigned int*>(p.payload + L.table_off[g]);
                if (t == 0) {
                    head[0] = L.items[g];
                    head[1] = (unsigned int)((L.tbits[g] + 63) / 64);
                    head[2] = L.cells[g];
                    head[3] = HUF_RESTART;
                }
                if (t < 32) {
                    const unsigned int base = L.sym_lo[g] + (unsigned int)g, n = L.nsym[g];
                    unsigned int seen = 0;
                    for (unsigned int a0 = 0; a0 < n; a0 += 32) {
                        const unsigned int a = a0 + t;
                        const unsigned int ln = a < n ? s.cs.huf_len[base + a] : 0u;
                        const unsigned int present = __ballot_sync(0xFFFFFFFFu, ln != 0);
                        if (ln) {
                            int* rec = reinterpret_cast<int*>(head + 4) + 3 * (seen + __popc(present & ((1u << t) - 1u)));
                            rec[0] = a + 1 == n ? 0x7FFFFFFF : (int)(L.sym_lo[g] + a);
                            rec[1] = (int)s.cs.huf_code[base + a];
                            rec[2] = (int)ln;
                        }
                        seen += __popc(present);
                    }
                }
            }
        }
        __syncthreads();
    }
}

// Absolute byte range of the 16-byte units that hold only bits [a, b) of a stream starting at byte
// `base` (4-byte aligned): from the first unit boundary at or after bit a to the last one at or before b.
__device__ __forceinline__ void own_units(unsigned long long base, unsigned long long a, unsigned long long b,
                                          unsigned long long& lo, unsigned long long& hi) {
    lo = 16ull * ((8ull * base + a + 127ull) / 128ull);
    hi = 16ull * ((8ull * base + b) / 128ull);
}

// The parts of the coded tables this block wrote -> the peers' slots (units that hold a block border
// are sent by block 0 once every block is done).
__device__ void huf_push_own(const CP& p, Smem& s, unsigned int t_begin, unsigned int t_end) {
    const Layout& L = s.lay;
    if (p.world <= 1 || L.overflow || t_begin >= t_end) return;
    __syncthreads();
    for (int g = 0; g < p.G; ++g) {
        const unsigned int c0 = max(t_begin, L.tchunk_prefix[g]), c1 = min(t_end, L.tchunk_prefix[g + 1]);
        if (c0 >= c1) continue;
        const bool first = c0 == L.tchunk_prefix[g], last = c1 == L.tchunk_prefix[g + 1];
        const unsigned long long a = s.pre_tbits[g], b = a + s.my_tbits[g];
        unsigned long long lo, hi;
        own_units(L.tstream_off[g], a, b, lo, hi);
        if (first) lo = L.table_off[g];          // head, items and the stream's first bits
        if (last) hi = L.trestart_off[g];        // the stream's padding up to the restart offsets
        if (hi > lo) push_bytes(p, lo, hi);
        // restart offsets of the block's chunks (1024 / HUF_RESTART per chunk)
        const unsigned int e0 = (c0 - L.tchunk_prefix[g]) * (1024u / HUF_RESTART);
        unsigned int e1 = (c1 - L.tchunk_prefix[g]) * (1024u / HUF_RESTART);
        const unsigned int ne = (L.cells[g] + HUF_RESTART - 1) / HUF_RESTART;
        unsigned long long r1 = L.trestart_off[g] + 4ull * min(e1, ne);
        if (last) r1 = skml_align16(r1);
        push_bytes(p, L.trestart_off[g] + 4ull * e0, r1);
        (void)e1;
    }
}

// Block 0, after every block has written: the units of the table streams that hold a block border.
__device__ void huf_push_borders(const CP& p, Smem& s) {
    const Layout& L = s.lay;
    if (p.world <= 1 || L.overflow) return;
    const unsigned int total = L.tchunk_prefix[p.G];
    unsigned int per = (total + gridDim.x - 1) / gridDim.x;
    per = (per + 3u) & ~3u;
    const unsigned int b = threadIdx.x;
    if (b >= 1 && b < gridDim.x && (unsigned long long)per * b < total) {
        const unsigned int cs = per * b;
        int g = 0;
        while (g + 1 < p.G && cs >= L.tchunk_prefix[g + 1]) ++g;
        if (cs != L.tchunk_prefix[g]) {
            unsigned long long a = 0;
            for (unsigned int q = 0; q < b; ++q) a += __ldcg(&p.blk_tbits[(long long)q * SKML_MAX_GROUPS + g]);
            const unsigned long long bit = 8ull * L.tstream_off[g] + a;
            if (bit & 127ull) {
                const unsigned long long off = 16ull * (bit / 128ull);
                const uint4 v = ld_cg_v4(reinterpret_cast<const uint4*>(p.payload + off));
                for (unsigned int r = 0; r < p.world; ++r)
                    if (r != p.rank && p.peer_payload[r]) st_v4(reinterpret_cast<uint4*>(p.peer_payload[r] + off), v);
            }
        }
    }
}

__device__ __forceinline__ void chunk_run(const Layout& L, int G, unsigned int& my_begin, unsigned int& my_end) {
    const unsigned int total = L.chunk_prefix[G];
    unsigned int per = (total + gridDim.x - 1) / gridDim.x;
    per = (per + 3u) & ~3u;  // four chunks per round
    my_begin = min(total, per * blockIdx.x);
    my_end = min(total, my_begin + per);
}

// S6 prelude: every group's delta bytes from all blocks' counts -> delta section offsets, total size.
__device__ void layout_finish(const CP& p, Smem& s) {
    Layout& L = s.lay;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp < p.G) {
        unsigned long long v = 0;
        for (int b = lane; b < (int)gridDim.x; b += 32) v += __ldcg(&p.blk_bytes[(long long)b * SKML_MAX_GROUPS + warp]);
        v = warp_sum(v);
        if (lane == 0) L.bytes_g[warp] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long o = L.off_deltas;
        for (int g = 0; g < p.G; ++g) {
            L.delta_off[g] = o;
            if (L.n_g[g]) o += skml_align16(8ull * ((L.bytes_g[g] + 7) / 8));
        }
        L.total_bytes = o;
        if (o > (unsigned long long)p.slot_capacity) {
            L.overflow = 1;
            skml_set_status(p.status, SKML_CAPACITY, 0x36u);
        }
    }
    __syncthreads();
}

// Fill helpers run inside S1 (they do not depend on the summary).
__device__ void stage_prepare(const CP& p, long long n) {
    // working sketch cells start "empty"
    long long cells = (long long)p.rows * ((long long)(p.col_ratio * (double)n) + 2 + p.G);
    if (cells > p.tables_cap - 4) cells = p.tables_cap - 4;
    const long long gsz = (long long)gridDim.x * blockDim.x, gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    uint4 ones = make_uint4(~0u, ~0u, ~0u, ~0u);
    uint4* t4 = reinterpret_cast<uint4*>(p.tables);
    for (long long i = gid; i < (cells + 3) / 4; i += gsz) t4[i] = ones;
    if (p.key_encoder == SKML_KEYS_DELTA_ADAPTIVE || p.huffman) {
        // the bit streams are completed with atomic ORs where chunks meet: they start from zero
        long long bound = payload_bound(n, 0, p.q, p.G, p.rows, p.col_ratio);
        if (bound > p.slot_capacity) bound = p.slot_capacity;
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4* z4 = reinterpret_cast<uint4*>(p.payload);
        for (long long i = gid + SKML_HEADER_BYTES / 16; i < bound / 16; i += gsz) z4[i] = z;
        for (long long i = gid; i < SKML_MAX_GROUPS * 32; i += gsz) p.key_hist[i] = 0;
        for (long long i = gid; i < SKML_GPU_MAX_BINS + SKML_MAX_GROUPS; i += gsz) p.cell_hist[i] = 0;
    }
}

// Header, bucket values and group table (block 0), stored locally and into every peer's slot.
__device__ void write_header(const CP& p, Smem& s, long long n, int kind) {
    if (blockIdx.x != 0) return;
    const Layout& L = s.lay;
    const QInfo& q = s.qi;
    const bool sparse = kind == SKML_KIND_SPARSE && !L.overflow;
    if (kind != SKML_KIND_EMPTY && (kind == SKML_KIND_DENSE || sparse)) {
        float* bv = reinterpret_cast<float*>(p.payload + SKML_HEADER_BYTES);
        const int padded = (int)(skml_align16(4ull * p.q) / 4);
        for (int b = threadIdx.x; b < padded; b += blockDim.x) bv[b] = b < q.bin_num ? bucket_value(s, b) : 0.f;
    }
    if (sparse) {
        if (threadIdx.x < p.G) {
            const int g = threadIdx.x;
            SkmlGroupEntry e;
            e.n = L.n_g[g];
            e.col_num = L.col[g];
            for (int i = 0; i < 8; ++i) e.hash_ids[i] = L.n_g[g] ? L.hash_ids[g][i] : 0;
            e.table_off = L.n_g[g] ? L.table_off[g] : 0;
            e.flag_off = L.n_g[g] ? L.flag_off[g] : 0;
            e.n_flag_words = (unsigned int)((2ull * L.n_g[g] + 63) / 64);
            e.num_intervals = 4;
            e.delta_off = L.n_g[g] ? L.delta_off[g] : 0;
            e.n_delta_words = (unsigned int)((L.bytes_g[g] + 7) / 8);
            e.flag_kind = 0;
            if (p.key_encoder == SKML_KEYS_DELTA_ADAPTIVE) {
                e.n_flag_words = (unsigned int)((L.flag_bits[g] + 63) / 64);
                e.n_delta_words = (unsigned int)((L.delta_bits[g] + 63) / 64);
                e.num_intervals = L.n_g[g] ? L.num_iv[g] : 0;
                e.flag_kind = L.n_g[g] ? L.flag_kind[g] : 0;
            }
            e.restart_off = L.n_g[g] ? L.restart_off[g] : 0;
            *reinterpret_cast<SkmlGroupEntry*>(p.payload + L.off_gt + (unsigned long long)g * sizeof(SkmlGroupEntry)) = e;
        }
    }
    if (threadIdx.x == 0) {
        SkmlHeader h;
        unsigned char* hb = reinterpret_cast<unsigned char*>(&h);
        for (int i = 0; i < SKML_HEADER_BYTES; ++i) hb[i] = 0;
        h.magic = SKML_MAGIC;
        h.version = SKML_VERSION;
        h.kind = (kind == SKML_KIND_SPARSE && L.overflow) ? SKML_KIND_EMPTY : (unsigned int)kind;
        h.dtype = SKML_F32;
        h.step = p.step;
        h.rank = p.rank;
        h.world = p.world;
        h.dim = (unsigned long long)p.dim;
        h.seed = p.seed;
        if (p.loss_partials)
            for (int i = 0; i < 4; ++i) h.loss_partials[i] = p.loss_partials[i];
        h.total_bytes = SKML_HEADER_BYTES;
        if (h.kind != SKML_KIND_EMPTY) {
            h.nnz = (unsigned long long)n;
            h.bin_num = (unsigned int)q.bin_num;
            h.zero_idx = (unsigned int)q.zero_idx;
            h.cell_bits = (kind == SKML_KIND_SPARSE && p.huffman) ? 0u : (unsigned int)q.cell_bits;
            h.min_value = (double)q.minv;
            h.max_value = (double)q.maxv;
            h.off_bucket_values = SKML_HEADER_BYTES;
        }
        if (h.kind == SKML_KIND_SPARSE) {
            h.group_num = (unsigned int)p.G;
            h.row_num = (unsigned int)p.rows;
            h.col_ratio = p.col_ratio;
            h.key_encoder = (unsigned int)p.key_encoder;
            h.restart_interval = SKML_RESTART_INTERVAL;
            h.off_group_table = L.off_gt;
            h.off_key_flags = L.off_flags;
            h.off_restart = L.off_restart;
            h.off_tables = L.off_tables;
            h.off_key_deltas = L.off_deltas;
            h.total_bytes = L.total_bytes;
        } else if (h.kind == SKML_KIND_DENSE) {
            h.off_dense_codes = SKML_HEADER_BYTES + skml_align16(4ull * p.q);
            h.total_bytes = skml_align16(h.off_dense_codes + (unsigned long long)p.dim * (q.cell_bits / 8));
        }
        h.header_checksum = skml_header_checksum(&h);
        const uint4* src = reinterpret_cast<const uint4*>(&h);
        uint4* dst = reinterpret_cast<uint4*>(p.payload);
        for (int i = 0; i < SKML_HEADER_BYTES / 16; ++i) dst[i] = src[i];
    }
    // this block wrote the head of the payload (header, bucket values, group table): it also stores it
    // into the peers' slots, so that no other block has to wait for it
    __syncthreads();
    if (p.world > 1) {
        unsigned long long head = SKML_HEADER_BYTES;
        if (sparse) head = L.off_flags;
        else if (kind == SKML_KIND_DENSE) head = SKML_HEADER_BYTES + skml_align16(4ull * p.q);
        const uint4* src = reinterpret_cast<const uint4*>(p.payload);
        for (unsigned long long i = threadIdx.x; i < head / 16; i += blockDim.x) {
            const uint4 v = ld_cg_v4(src + i);
            for (unsigned int r = 0; r < p.world; ++r)
                if (r != p.rank && p.peer_payload[r]) st_v4(reinterpret_cast<uint4*>(p.peer_payload[r]) + i, v);
        }
    }
}

// ---------------------------------------------------------------------------
// S6: narrow tables, store everything into the peers' slots, release the flags
// ---------------------------------------------------------------------------
__device__ void copy_range_to_peers(const CP& p, unsigned long long lo, unsigned long long hi) {
    if (p.world <= 1 || hi <= lo) return;
    const long long gsz = (long long)gridDim.x * blockDim.x, gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long units = (long long)((hi - lo) / 16);
    const uint4* src = reinterpret_cast<const uint4*>(p.payload + lo);
    for (long long i = gid; i < units; i += gsz) {
        uint4 v = ld_cg_v4(src + i);
        for (unsigned int r = 0; r < p.world; ++r)
            if (r != p.rank && p.peer_payload[r]) st_v4(reinterpret_cast<uint4*>(p.peer_payload[r] + lo) + i, v);
    }
}

__device__ void finish_publish(const CP& p) {
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int prev = atomicAdd(&p.ctrl[2], 1u);
        s_last = prev == gridDim.x - 1;
        if (s_last) {
            p.ctrl[2] = 0;
            p.ctrl[4] = 0;  // the summary's min / max words go back to "nothing yet"
            p.ctrl[5] = 0;
        }
    }
    __syncthreads();
    // the last block to arrive raises the arrival flags, one thread per rank so that the releases (each
    // orders this GPU's earlier peer stores before its flag) run side by side instead of one after another
    if (s_last && threadIdx.x < p.world && p.peer_flag[threadIdx.x]) {
        __threadfence_system();
        st_release_sys(p.peer_flag[threadIdx.x], p.step + 1);
    }
}

// Sketch tables: 32-bit working cells -> 8/16-bit bucket codes, stored locally and into the peers' slots.
__device__ void narrow_tables(const CP& p, Smem& s) {
    const Layout& L = s.lay;
    if (L.overflow) return;
    const int G = p.G, cb = s.qi.cell_bits, per = 16 / (cb / 8);  // cells per 16-byte unit
    if (threadIdx.x == 0) {
        unsigned long long u = 0;
        for (int g = 0; g < G; ++g) {
            s.unit_prefix[g] = u;
            u += skml_align16((unsigned long long)p.rows * L.col[g] * (cb / 8)) / 16;
        }
        s.unit_prefix[G] = u;
    }
    __syncthreads();
    const long long gsz = (long long)gridDim.x * blockDim.x, gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long units = (long long)s.unit_prefix[G];
    const unsigned int zero = (unsigned int)s.qi.zero_idx;
    for (long long u = gid; u < units; u += gsz) {
        int g = 0;
        while (g + 1 < G && (unsigned long long)u >= s.unit_prefix[g + 1]) ++g;
        const long long j = u - (long long)s.unit_prefix[g];
        const long long cells = (long long)p.rows * L.col[g];
        const unsigned int* tab = p.tables + L.tab32_off[g];
        unsigned int words[4] = {0, 0, 0, 0};
        for (int t = 0; t < per; ++t) {
            long long c = j * per + t;
            unsigned int code = 0;
            if (c < cells) {
                unsigned int cell = __ldcg(tab + c);
                code = cell == SKML_EMPTY_CELL ? zero : (cell & 0xFFFFu);
            }
            if (cb == 8) words[t >> 2] |= (code & 0xFFu) << (8 * (t & 3));
            else words[t >> 1] |= (code & 0xFFFFu) << (16 * (t & 1));
        }
        uint4 v = make_uint4(words[0], words[1], words[2], words[3]);
        const unsigned long long off = L.table_off[g] + 16ull * j;
        st_v4(reinterpret_cast<uint4*>(p.payload + off), v);
        for (unsigned int r = 0; r < p.world; ++r)
            if (r != p.rank && p.peer_payload[r]) st_v4(reinterpret_cast<uint4*>(p.peer_payload[r] + off), v);
    }
}

// Bytes [lo, hi) of the local payload -> the same bytes of every peer's slot, by this block alone:
// 16-byte stores for the aligned interior, byte stores for a ragged head or tail (two blocks that
// share a 16-byte unit each store only their own bytes of it).
__device__ void push_bytes(const CP& p, unsigned long long lo, unsigned long long hi) {
    if (p.world <= 1 || hi <= lo) return;
    const unsigned long long a0 = (lo + 15ull) & ~15ull, a1 = hi & ~15ull;
    if (a0 < a1) {
        const uint4* src = reinterpret_cast<const uint4*>(p.payload + a0);
        for (unsigned long long i = threadIdx.x; i < (a1 - a0) / 16; i += blockDim.x) {
            const uint4 v = ld_cg_v4(src + i);
            for (unsigned int r = 0; r < p.world; ++r)
                if (r != p.rank && p.peer_payload[r]) st_v4(reinterpret_cast<uint4*>(p.peer_payload[r] + a0) + i, v);
        }
    }
    const unsigned long long head_end = a0 < hi ? a0 : hi, tail_begin = a1 > head_end ? a1 : head_end;
    const unsigned long long ragged = (head_end - lo) + (hi - tail_begin);
    for (unsigned long long i = threadIdx.x; i < ragged; i += blockDim.x) {
        const unsigned long long a = i < head_end - lo ? lo + i : tail_begin + (i - (head_end - lo));
        const unsigned char v = __ldcg(p.payload + a);
        for (unsigned int r = 0; r < p.world; ++r)
            if (r != p.rank && p.peer_payload[r]) p.peer_payload[r][a] = v;
    }
}

// The flag bytes, restart points and delta bytes this block wrote for its chunks -> the peers' slots.
__device__ void push_own_chunks(const CP& p, Smem& s, unsigned int my_begin, unsigned int my_end) {
    const Layout& L = s.lay;
    if (p.world <= 1 || L.overflow || my_begin >= my_end) return;
    __syncthreads();  // this block's own stores are visible to all its threads
    for (int g = 0; g < p.G; ++g) {
        const unsigned int c0 = max(my_begin, L.chunk_prefix[g]), c1 = min(my_end, L.chunk_prefix[g + 1]);
        if (c0 >= c1) continue;
        const unsigned int ja = c0 - L.chunk_prefix[g], jb = c1 - L.chunk_prefix[g];
        const bool last = c1 == L.chunk_prefix[g + 1];
        const unsigned long long flag_bytes = skml_align16(8ull * ((2ull * L.n_g[g] + 63) / 64));
        const unsigned long long f1 = min(flag_bytes, 256ull * jb);
        push_bytes(p, L.flag_off[g] + 256ull * ja, L.flag_off[g] + (last ? flag_bytes : f1));
        push_bytes(p, L.restart_off[g] + 16ull * ja, L.restart_off[g] + 16ull * jb);
        unsigned long long d0 = s.pre_bytes[g], d1 = s.pre_bytes[g] + s.my_bytes[g];
        if (last) d1 = skml_align16(8ull * ((d1 + 7) / 8));  // the zero padding written with the last chunk
        push_bytes(p, L.delta_off[g] + d0, L.delta_off[g] + d1);
    }
}

// Block 0 needs every block's byte counts for the header: bounded wait for their publications.
__device__ bool wait_all_published(const CP& p, const unsigned int* flags, unsigned int epoch) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < gridDim.x) {
        const long long t0 = clock64();
        unsigned int ns = 20;
        while (ld_acquire_gpu(&flags[threadIdx.x]) != epoch) {
            if (clock64() - t0 > p.budget) {
                skml_set_status(p.status, SKML_TIMEOUT_BARRIER, 0x51u);
                s_ok = 0;
                break;
            }
            __nanosleep(ns);
            if (ns < 400) ns *= 2;
        }
    }
    __syncthreads();
    return s_ok != 0;
}

// ---------------------------------------------------------------------------
// Kernels
// ---------------------------------------------------------------------------
#define STAGE_BARRIER(stage_id)                                                           \
    if (FUSED) {                                                                          \
        if (!skml_grid_barrier(p.ctrl, gridDim.x, p.status, p.budget, stage_id)) return; \
        stage_stamp(p.ctrl, stage_id);                                                    \
    }

// STAGE < 0: all stages in one cooperative launch; otherwise only that stage.
// ADAPTIVE / HUFFMAN: the key encoder and the table coder are compile-time choices, so that the default
// path (delta_binary keys, plain tables) carries none of the other coders' registers.
template <bool FUSED, bool ADAPTIVE, bool HUFFMAN>
__global__ void __launch_bounds__(SKML_BLOCK, 1) compress_sparse_kernel(CP p, int stage) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>(smem_raw);
    const long long kind = p.meta[1];
    if (kind == SKML_KIND_DENSE) return;  // handled by the dense kernel
    long long n = p.meta[0];
    if (n > p.n_max) {
        if (threadIdx.x == 0) skml_set_status(p.status, SKML_CAPACITY, 0x31u);
        n = 0;
    }
    if (n <= 0) {  // empty gradient: header-only payload
        if (FUSED || stage == 8) {
            if (threadIdx.x == 0) {
                s.lay.overflow = 0;
                s.qi.bin_num = 0;
            }
            __syncthreads();
            write_header(p, s, 0, SKML_KIND_EMPTY);   // block 0 stores it locally and into the peers' slots
            finish_publish(p);
        }
        return;
    }
    const bool given = p.given_splits != nullptr;
    if (FUSED) stage_stamp(p.ctrl, 0);
    // sample form of the split search: S1 ends with the splits in every block, S2 and two grid barriers drop out
    const bool sample = p.sample_splits != 0 && !given;
    if (FUSED || stage == 1) {
        stage_prepare(p, n);
        stage_stamp(p.ctrl, 8);
        if (sample) stage_sample_splits(p, s, p.vals, n);
        else if (!given) stage_summary(p, s, p.vals, n);
        stage_stamp(p.ctrl, 9);
    }
    if (sample) {
        if (FUSED) {
            stage_stamp(p.ctrl, 1);
            stage_stamp(p.ctrl, 2);
        }
    } else {
        STAGE_BARRIER(1)
        if ((FUSED || stage == 2) && !given) stage_query(p, s, n);
        STAGE_BARRIER(2)
    }
    if (FUSED || stage == 3) {
        load_quantizer(p, s, !sample);
        if (s.qi.bin_num > SKML_GPU_MAX_BINS) {
            if (threadIdx.x == 0) skml_set_status(p.status, SKML_BAD_INPUT, 0x32u);
            return;
        }
        stage_count(p, s, n, sample);
    }
    STAGE_BARRIER(3)
    if (FUSED || stage == 4) {
        if (!FUSED) load_quantizer(p, s);
        else if (sample) refresh_minmax(p, s);
        layout_from_counts(p, s);
        stage_scatter(p, s, n);
    }
    STAGE_BARRIER(4)
    // S5: key code and publication. In one cooperative launch a block waits only for the counts of the
    // blocks before it (they are resident, and never wait for a later block), and block 0 for all of them
    // before it writes the header; staged launches split the stage at those points. The delta_adaptive
    // code needs the groups' complete histograms of delta widths first: one more grid barrier.
    unsigned int my_begin = 0, my_end = 0, t_begin = 0, t_end = 0;
    constexpr bool adaptive = ADAPTIVE, huffman = HUFFMAN;
    if (FUSED || stage >= 5) {
        if (!FUSED) {
            load_quantizer(p, s);
            layout_from_counts(p, s);
        }
        chunk_run(s.lay, p.G, my_begin, my_end);
        if (huffman) {
            huf_ranges(p, s);
            tchunk_run(s.lay, p.G, t_begin, t_end);
        }
    }
    if (FUSED || stage == 5) {
        if (huffman) {
            if (!s.lay.overflow) huf_histogram(p, s, t_begin, t_end);
        } else {
            narrow_tables(p, s);   // the tables are complete since S4
        }
        if (adaptive && !s.lay.overflow) apack_histogram(p, s, my_begin, my_end);
    }
    if (FUSED && (adaptive || huffman)) {
        if (!skml_grid_barrier(p.ctrl, gridDim.x, p.status, p.budget, 0x15u)) return;
    }
    if (FUSED || stage >= 6) {
        // code tables and the layout behind the tables (every block; staged launches repeat it per stage)
        if (huffman && (FUSED || stage >= 6)) huf_build(p, s);
        if (adaptive) apack_choose(p, s);
    }
    if (FUSED || stage == 6) {
        if (adaptive) apack_measure(p, s, my_begin, my_end);
        else pack_measure(p, s, my_begin, my_end);
        if (huffman) huf_measure(p, s, t_begin, t_end);
    }
    unsigned int epoch = 0;
    if (FUSED) {
        // every block reads the same barrier generation here: it names this launch's publications
        epoch = ld_acquire_gpu(&p.ctrl[1]) + 0x40000000u;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) st_release_gpu(&p.blk_flag[blockIdx.x], epoch);
    }
    const bool borders = adaptive || huffman;  // stream words shared by two blocks are sent by block 0 at the end
    if (FUSED || stage == 7) {
        if (!FUSED) {  // the block's own counts again (shared memory does not survive a launch)
            if (threadIdx.x < SKML_MAX_GROUPS) {
                s.my_bytes[threadIdx.x] = p.blk_bytes[(long long)blockIdx.x * SKML_MAX_GROUPS + threadIdx.x];
                s.my_tbits[threadIdx.x] = p.blk_tbits[(long long)blockIdx.x * SKML_MAX_GROUPS + threadIdx.x];
            }
            if (threadIdx.x < 2 * SKML_MAX_GROUPS) s.my_bits[threadIdx.x] = p.blk_bits[(long long)blockIdx.x * 2 * SKML_MAX_GROUPS + threadIdx.x];
            __syncthreads();
        }
        if (adaptive) {
            apack_prefix(p, s, FUSED, epoch);
            apack_write(p, s, my_begin, my_end);
            apush_own_chunks(p, s, my_begin, my_end);
        } else {
            pack_prefix(p, s, FUSED, epoch);
            pack_write(p, s, my_begin, my_end);
            push_own_chunks(p, s, my_begin, my_end);
        }
        if (huffman) {
            huf_prefix(p, s);   // (the key prefix above has waited for the blocks before this one)
            huf_write(p, s, t_begin, t_end);
            huf_push_own(p, s, t_begin, t_end);
        }
        if (FUSED && borders) {
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) st_release_gpu(&p.blk_done[blockIdx.x], epoch);
        }
        if (FUSED) stage_stamp(p.ctrl, 5);
    }
    if (FUSED || stage == 8) {
        if (blockIdx.x == 0) {
            if (FUSED && !wait_all_published(p, borders ? p.blk_done : p.blk_flag, epoch)) return;
            if (adaptive) apush_borders(p, s);
            else layout_finish(p, s);
            if (huffman) huf_push_borders(p, s);
            write_header(p, s, n, SKML_KIND_SPARSE);
        }
        finish_publish(p);
        if (FUSED) stage_stamp(p.ctrl, 6);
    }
}

// Dense kind: one narrow bucket code per coordinate, written straight into the local
// payload and every peer's slot.
template <bool FUSED>
__global__ void __launch_bounds__(SKML_BLOCK, 1) compress_dense_kernel(CP p, int stage) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>(smem_raw);
    if (p.meta[1] != SKML_KIND_DENSE) return;
    const long long n = p.dim;
    const bool given = p.given_splits != nullptr;
    // sample form: the splits are in every block after S1; the extremes of the values (needed for the bucket
    // values in the header only) are collected by the code pass, and the header is written after it
    const bool sample = p.sample_splits != 0 && !given;
    if (FUSED || stage == 1) {
        if (sample) stage_sample_splits(p, s, p.vals, n);
        else if (!given) stage_summary(p, s, p.vals, n);
    }
    if (!sample) {
        STAGE_BARRIER(1)
        if ((FUSED || stage == 2) && !given) stage_query(p, s, n);
        STAGE_BARRIER(2)
    }
    if (FUSED || stage == 3) {
        load_quantizer(p, s, !sample);
        if (s.qi.bin_num > SKML_GPU_MAX_BINS) {
            if (threadIdx.x == 0) skml_set_status(p.status, SKML_BAD_INPUT, 0x33u);
            return;
        }
        if (threadIdx.x == 0) s.lay.overflow = 0;
        __syncthreads();
        const int cb = s.qi.cell_bits, per = 16 / (cb / 8);
        const unsigned long long off_codes = SKML_HEADER_BYTES + skml_align16(4ull * p.q);
        const unsigned long long total = skml_align16(off_codes + (unsigned long long)n * (cb / 8));
        if (total > (unsigned long long)p.slot_capacity) {
            if (threadIdx.x == 0) skml_set_status(p.status, SKML_CAPACITY, 0x34u);
            return;
        }
        if (!sample) write_header(p, s, n, SKML_KIND_DENSE);
        unsigned int kmin = 0xFFFFFFFFu, kmax = 0u;
        const long long units = (n + per - 1) / per;
        const long long gsz = (long long)gridDim.x * blockDim.x, gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
        for (long long u = gid; u < units; u += gsz) {
            unsigned int words[4] = {0, 0, 0, 0};
            for (int t = 0; t < per; ++t) {
                long long i = u * per + t;
                unsigned int code = 0;
                if (i < n) {
                    const float val = p.vals[i];
                    code = (unsigned int)upper_bound_f(s.splits, s.qi.nsplits, val);
                    const unsigned int k = f2ord(val);
                    kmin = min(kmin, k);
                    kmax = max(kmax, k);
                }
                if (cb == 8) words[t >> 2] |= (code & 0xFFu) << (8 * (t & 3));
                else words[t >> 1] |= (code & 0xFFFFu) << (16 * (t & 1));
            }
            uint4 v = make_uint4(words[0], words[1], words[2], words[3]);
            st_v4(reinterpret_cast<uint4*>(p.payload + off_codes) + u, v);
            for (unsigned int r = 0; r < p.world; ++r)
                if (r != p.rank && p.peer_payload[r]) st_v4(reinterpret_cast<uint4*>(p.peer_payload[r] + off_codes) + u, v);
        }
        if (sample) {   // one pair of atomics per warp
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                kmin = min(kmin, __shfl_xor_sync(0xFFFFFFFFu, kmin, o));
                kmax = max(kmax, __shfl_xor_sync(0xFFFFFFFFu, kmax, o));
            }
            if ((threadIdx.x & 31) == 0 && kmin <= kmax) {
                atomicMax(&p.ctrl[4], ~kmin);
                atomicMax(&p.ctrl[5], kmax);
            }
        }
    }
    STAGE_BARRIER(3)
    if (FUSED || stage == 4) {
        if (sample) {
            if (!FUSED) load_quantizer(p, s);   // staged launches: the extremes are complete now
            else refresh_minmax(p, s);
            if (!FUSED) {
                if (threadIdx.x == 0) s.lay.overflow = 0;
                __syncthreads();
            }
            write_header(p, s, n, SKML_KIND_DENSE);
        }
        finish_publish(p);
    }
}

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------
static int device_sms() {
    static int cached = 0;
    if (cached == 0) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cached = sms > 0 ? sms : 148;
    }
    return cached;
}

static int fill_params(const SkmlCompressArgs* a, CP& p, int& grid) {
    if (!a || !a->meta || !a->payload || !a->workspace || !a->status) return (int)cudaErrorInvalidValue;
    if (a->bin_num < 2 || a->bin_num > SKML_GPU_MAX_BINS) return (int)cudaErrorInvalidValue;
    if (a->group_num < 1 || a->group_num > SKML_MAX_GROUPS) return (int)cudaErrorInvalidValue;
    if (a->row_num < 1 || a->row_num > SKML_MAX_ROWS) return (int)cudaErrorInvalidValue;
    if (a->world < 1 || a->world > SKML_MAX_PEERS || a->rank < 0 || a->rank >= a->world) return (int)cudaErrorInvalidValue;
    if (a->n_max >= (1ll << 31) || a->dim >= (1ll << 31)) return (int)cudaErrorInvalidValue;
    if (a->key_encoder != SKML_KEYS_DELTA_BINARY && a->key_encoder != SKML_KEYS_DELTA_ADAPTIVE) return (int)cudaErrorInvalidValue;
    grid = a->grid > 0 ? (int)a->grid : device_sms();
    if (grid > MAX_GRID) grid = MAX_GRID;
    WsLayout L = ws_layout(a->n_max, a->bin_num, a->group_num, a->row_num, a->col_ratio, grid);
    if (L.total > a->workspace_bytes) return (int)cudaErrorInvalidValue;
    p.keys = a->keys;
    p.vals = a->vals;
    p.meta = a->meta;
    p.n_max = a->n_max;
    p.dim = a->dim;
    p.q = (int)a->bin_num;
    p.G = (int)a->group_num;
    p.rows = (int)a->row_num;
    p.col_ratio = a->col_ratio;
    p.seed = a->seed;
    p.step = a->step;
    p.rank = (unsigned int)a->rank;
    p.world = (unsigned int)a->world;
    p.loss_partials = a->loss_partials;
    p.payload = a->payload;
    p.slot_capacity = a->slot_capacity;
    for (int i = 0; i < SKML_MAX_PEERS; ++i) {
        p.peer_payload[i] = a->peer_payload[i];
        p.peer_flag[i] = a->peer_flag[i];
    }
    unsigned char* ws = a->workspace;
    p.ctrl = reinterpret_cast<unsigned int*>(ws + L.ctrl);
    p.run_vals = reinterpret_cast<unsigned int*>(ws + L.run_vals);
    p.run_cnt = reinterpret_cast<unsigned int*>(ws + L.run_cnt);
    p.run_w = reinterpret_cast<unsigned long long*>(ws + L.run_w);
    p.splits_raw = reinterpret_cast<unsigned int*>(ws + L.splits_raw);
    p.warp_cnt = reinterpret_cast<unsigned int*>(ws + L.warp_cnt);
    p.blk_cnt = reinterpret_cast<unsigned int*>(ws + L.blk_cnt);
    p.blk_bytes = reinterpret_cast<unsigned long long*>(ws + L.blk_bytes);
    p.blk_flag = reinterpret_cast<unsigned int*>(ws + L.blk_flag);
    p.chunk_off = reinterpret_cast<unsigned int*>(ws + L.chunk_off);
    p.blk_bits = reinterpret_cast<unsigned long long*>(ws + L.blk_bits);
    p.blk_done = reinterpret_cast<unsigned int*>(ws + L.blk_done);
    p.key_hist = reinterpret_cast<unsigned int*>(ws + L.key_hist);
    p.key_encoder = (int)a->key_encoder;
    p.huffman = a->cell_bits == 0 ? 1 : 0;
    p.sample_splits = a->quantile_summary == 1 ? 0 : 1;
    p.cell_hist = reinterpret_cast<unsigned int*>(ws + L.cell_hist);
    p.blk_tbits = reinterpret_cast<unsigned long long*>(ws + L.blk_tbits);
    p.tchunk_off = reinterpret_cast<unsigned int*>(ws + L.tchunk_off);
    p.gkeys = reinterpret_cast<int*>(ws + L.gkeys);
    p.bins = reinterpret_cast<unsigned short*>(ws + L.bins);
    p.tables = reinterpret_cast<unsigned int*>(ws + L.tables);
    p.tables_cap = L.tables_cap;
    p.status = a->status;
    p.budget = a->budget_cycles > 0 ? a->budget_cycles : 2000000000ll;
    p.given_splits = a->given_splits;
    p.n_given = (int)a->n_given;
    p.given_min = (float)a->given_min;
    p.given_max = (float)a->given_max;
    return 0;
}

// Byte offset, inside the workspace, of the q - 1 split points the last launch queried from its
// summary (order-preserving 32-bit images of the floats, before duplicates are dropped). Debug
// tooling reads them to recompute a payload on the CPU from the same splits.
extern "C" long long skml_compress_splits_offset(long long n_max, long long bin_num, long long group_num,
                                                 long long row_num, double col_ratio, long long grid) {
    long long g = grid > 0 ? grid : device_sms();
    if (g > MAX_GRID) g = MAX_GRID;
    return ws_layout(n_max, bin_num, group_num, row_num, col_ratio, g).splits_raw;
}

// Function attributes and the co-residency limit are looked up once per kernel (one process
// drives one GPU), so a steady-state launch makes a single runtime call.
static int g_last_cluster = 0;   // blocks per cluster of the most recent compress launch (0: none yet)

struct LaunchCache {
    bool ready = false;
    int max_grid = 0;
    int cluster = 1;   // blocks per thread-block cluster (2 where that many clusters fit the device at once)
};

// One launch through the extensible API: cooperative when `coop`, in clusters of `cluster` blocks.
template <class K>
static cudaError_t launch_ex(K kernel, int grid, int cluster, bool coop, const CP& p, int stage, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(SKML_BLOCK);
    cfg.dynamicSmemBytes = sizeof(Smem);
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    unsigned int na = 0;
    if (coop) {
        attrs[na].id = cudaLaunchAttributeCooperative;
        attrs[na].val.cooperative = 1;
        ++na;
    }
    if (cluster > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = (unsigned int)cluster;
        attrs[na].val.clusterDim.y = 1;
        attrs[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kernel, p, stage);
}

template <class K>
static int launch_stages(K fused_kernel, K staged_kernel, LaunchCache& cache, CP& p, int grid, bool fused, int nstages,
                         cudaStream_t stream) {
    cudaError_t e;
    if (!cache.ready) {
        e = cudaFuncSetAttribute(fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem));
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem));
        if (e != cudaSuccess) return (int)e;
        int per_sm = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_kernel, SKML_BLOCK, sizeof(Smem));
        if (per_sm < 1) return (int)cudaErrorLaunchOutOfResources;
        cache.max_grid = per_sm * device_sms();
        // pairs of blocks as clusters when the whole grid still fits the device at once that way
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(cache.max_grid & ~1);
        cfg.blockDim = dim3(SKML_BLOCK);
        cfg.dynamicSmemBytes = sizeof(Smem);
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int nclusters = 0;
        const char* knob = getenv("SKML_COMPRESS_CLUSTER");   // "1": plain blocks, no clusters
        if (knob && knob[0] == '1' && knob[1] == 0) {
            cache.cluster = 1;
        } else if (cudaOccupancyMaxActiveClusters(&nclusters, fused_kernel, &cfg) == cudaSuccess && 2 * nclusters >= (cache.max_grid & ~1) &&
            cache.max_grid >= 2)
            cache.cluster = 2;
        else
            cudaGetLastError();  // a refused query is not an error of the caller
        cache.ready = true;
    }
    if (grid > cache.max_grid) grid = cache.max_grid;
    int cluster = cache.cluster;
    if (grid < 2 * cluster) cluster = 1;   // tiny grids (tests) keep plain blocks
    if (cluster > 1) grid -= grid % cluster;
    if (fused) {
        e = launch_ex(fused_kernel, grid, cluster, true, p, -1, stream);
        if (e != cudaSuccess && cluster > 1) {
            // the device refuses cooperative clusters of this shape: plain blocks from now on
            cudaGetLastError();
            cache.cluster = cluster = 1;
            e = launch_ex(fused_kernel, grid, 1, true, p, -1, stream);
        }
        g_last_cluster = cluster;
        return (int)e;
    }
    g_last_cluster = cluster;
    for (int st = 1; st <= nstages; ++st) {
        e = launch_ex(staged_kernel, grid, st == 1 ? cluster : 1, false, p, st, stream);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

// Blocks per thread-block cluster of the most recent compress launch of this process (2 where the device
// takes the whole grid as cooperative clusters of two, 1 for plain blocks, 0 before the first launch).
extern "C" int skml_compress_cluster_size() { return g_last_cluster; }

extern "C" int skml_compress_sparse(const SkmlCompressArgs* a, void* stream) {
    CP p;
    int grid = 0;
    int rc = fill_params(a, p, grid);
    if (rc) return rc;
    static LaunchCache cache[4];
    const bool adaptive = p.key_encoder == SKML_KEYS_DELTA_ADAPTIVE, huffman = p.huffman != 0;
    const bool fused = a->fused != 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (adaptive && huffman)
        return launch_stages(compress_sparse_kernel<true, true, true>, compress_sparse_kernel<false, true, true>, cache[3], p, grid, fused, 8, st);
    if (adaptive)
        return launch_stages(compress_sparse_kernel<true, true, false>, compress_sparse_kernel<false, true, false>, cache[2], p, grid, fused, 8, st);
    if (huffman)
        return launch_stages(compress_sparse_kernel<true, false, true>, compress_sparse_kernel<false, false, true>, cache[1], p, grid, fused, 8, st);
    return launch_stages(compress_sparse_kernel<true, false, false>, compress_sparse_kernel<false, false, false>, cache[0], p, grid, fused, 8, st);
}

extern "C" int skml_compress_dense(const SkmlCompressArgs* a, void* stream) {
    CP p;
    int grid = 0;
    int rc = fill_params(a, p, grid);
    if (rc) return rc;
    static LaunchCache cache;
    return launch_stages(compress_dense_kernel<true>, compress_dense_kernel<false>, cache, p, grid, a->fused != 0, 4,
                         (cudaStream_t)stream);
}
