// Fused decode + aggregate + update for sm_100a: the receiving side of the gradient
// exchange in one persistent cooperative kernel.
//   D0  bounded wait for the arrival flags of all ranks' payloads (written by the peers'
//       compress kernels straight into this GPU's memory), header validation, work table
//   D1  per 1024-key chunk (restart points make chunks independent): flag bits -> delta
//       widths -> scan -> gather -> prefix sum = keys; grouped MinMaxSketch query
//       (furthest-from-zero over the rows); dequantize
//   Replicas must end bit-identical, so the order of the float adds per coordinate is fixed:
//   * one payload: keys are unique inside it, every value is applied by the thread that
//     decoded it (SGD step, lazy Adam step, or plain sum);
//   * several short payloads: D1 stashes (key, value) pairs; after one grid barrier every
//     block owns a key range (quantiles of the longest key list), finds its slice of every
//     (rank, group) list by binary search and applies the slices rank by rank with block
//     barriers only. Lazy Adam first sums the ranks' values per coordinate (plain floats in
//     the zeroed accumulator array), then the first rank holding the coordinate applies the
//     moment update and clears the sum;
//   * several long payloads (SGD): one decode-and-apply pass per rank, grid barrier in between;
//   * a dense-kind payload among them: per-rank passes for SGD; for Adam 64-bit fixed-point
//     accumulators (integer adds commute) and a claim pass (atomic exchange with zero).
//
// Reference behaviour restated (paths inside the reference project):
//   sketch/.../binary/DeltaBinaryEncoder.java:42-53 (key decode),
//   sketch/.../sketch/frequency/MinMaxSketch.java:64-73, GroupedMinMaxSketch.java:123-146,
//   ml/.../gradient/SketchGradient.scala:57-68, Gradient.scala:44-49 (sum over workers),
//   ml/.../algorithm/GeneralizedLinearModel.scala:150 (1/workerNum),
//   ml/.../objective/GradientDescent.scala:89-117, Adam.scala:27-77 (updates).
#include "decode_common.cuh"

// The header fields that are needed after the work table is built.
struct HdrLite {
    unsigned int kind, cell_bits, bin_num, zero_idx;
    unsigned long long off_dense_codes, off_bucket_values;
    double loss_partials[4];
};

struct DecSmem {
    HdrLite hdr[SKML_MAX_PEERS];
    int nitems;
    unsigned long long total_chunks, total_keys;
    int any_dense;
    int direct;      // linear update (SGD / plain sum): payloads applied in rank order, no accumulators
    unsigned long long rank_chunk_begin[SKML_MAX_PEERS + 1];
    unsigned long long rank_key_begin[SKML_MAX_PEERS + 1];
    int rank_item_begin[SKML_MAX_PEERS + 1];
    int ref_item;    // the (rank, group) list with the most keys: its quantiles are the blocks' key-range bounds
    int two_phase;   // several payloads: decode everything first, then ordered apply
    int adam_plain;  // Adam without fixed-point accumulators (no dense payload, and one payload or a value scratch)
    int shift;       // fixed-point: accumulator = value * 2^shift
    double inv_world;
    int ok;
    int max_items;
    int nhuf;        // items whose table arrives Huffman-coded
    DecItem items[1];  // max_items entries (dynamic shared memory)
};

// D0: wait, validate, build the work table (identically in every block).
__device__ bool decode_prepare(const DP& p, DecSmem& s) {
    // the full headers sit in the (still idle) table staging area while the work table is built
    SkmlHeader* full = reinterpret_cast<SkmlHeader*>(reinterpret_cast<unsigned char*>(&s) + p.tab_off);
    if (threadIdx.x == 0) s.ok = 1;
    __syncthreads();
    // one thread per rank polls that rank's arrival flag (bounded), so the waits overlap
    if (threadIdx.x < p.world && p.flag[threadIdx.x] &&
        !skml_wait_flag(p.flag[threadIdx.x], p.step + 1, p.status, p.budget, (unsigned int)threadIdx.x))
        s.ok = 0;
    __syncthreads();
    if (!s.ok) return false;
    // headers -> shared memory (L2 loads: the bytes were written by other GPUs)
    for (int t = threadIdx.x; t < p.world * (SKML_HEADER_BYTES / 16); t += blockDim.x) {
        int r = t / (SKML_HEADER_BYTES / 16), i = t % (SKML_HEADER_BYTES / 16);
        reinterpret_cast<uint4*>(&full[r])[i] = ld_cg_v4(reinterpret_cast<const uint4*>(p.payload[r]) + i);
    }
    __syncthreads();
    if (threadIdx.x < p.world) {
        const SkmlHeader& h = full[threadIdx.x];
        bool good = h.magic == SKML_MAGIC && h.version == SKML_VERSION && h.header_checksum == skml_header_checksum(&h) &&
                    h.step == p.step && h.rank == (unsigned int)threadIdx.x && h.dim == (unsigned long long)p.dim &&
                    h.total_bytes <= (unsigned long long)p.slot_capacity && h.dtype == SKML_F32 &&
                    h.group_num <= SKML_MAX_GROUPS && h.row_num <= SKML_MAX_ROWS && h.kind <= SKML_KIND_DENSE &&
                    (h.kind != SKML_KIND_SPARSE || ((h.off_group_table & 15ull) == 0 &&
                                                    h.off_group_table + sizeof(SkmlGroupEntry) * h.group_num <= h.total_bytes)) &&
                    (h.kind == SKML_KIND_EMPTY || (h.bin_num >= 1 && h.bin_num <= SKML_GPU_MAX_BINS && h.zero_idx < h.bin_num)) &&
                    (h.kind != SKML_KIND_SPARSE || ((h.key_encoder == SKML_KEYS_DELTA_BINARY || h.key_encoder == SKML_KEYS_DELTA_ADAPTIVE) &&
                                                    h.restart_interval == SKML_RESTART_INTERVAL &&
                                                    (h.cell_bits == 8 || h.cell_bits == 16 || (h.cell_bits == 0 && p.tab_scratch))));
        if (!good) {
            skml_set_status(p.status, SKML_BAD_HEADER, (unsigned int)threadIdx.x);
            s.ok = 0;
        }
        HdrLite& l = s.hdr[threadIdx.x];
        l.kind = h.kind;
        l.cell_bits = h.cell_bits;
        l.bin_num = h.bin_num;
        l.zero_idx = h.zero_idx;
        l.off_dense_codes = h.off_dense_codes;
        l.off_bucket_values = h.off_bucket_values;
        for (int i = 0; i < 4; ++i) l.loss_partials[i] = h.loss_partials[i];
    }
    __syncthreads();
    if (!s.ok) return false;
    // group entries: one thread per (rank, group) fetches its 64-byte entry (independent loads)
    const int gcap = p.max_items / p.world;
    for (int t = threadIdx.x; t < p.world * gcap; t += blockDim.x) {
        const int r = t / gcap, g = t % gcap;
        const SkmlHeader& h = full[r];
        DecItem& it = s.items[t];
        it.e.n = 0;
        if (h.kind == SKML_KIND_SPARSE && g < (int)h.group_num) {
            const uint4* src = reinterpret_cast<const uint4*>(p.payload[r] + h.off_group_table + g * sizeof(SkmlGroupEntry));
            unsigned long long* dst = reinterpret_cast<unsigned long long*>(&it.e);  // 8-byte aligned in DecItem
#pragma unroll
            for (int q = 0; q < (int)(sizeof(SkmlGroupEntry) / 16); ++q) {
                const uint4 v = ld_cg_v4(src + q);
                dst[2 * q] = (unsigned long long)v.x | ((unsigned long long)v.y << 32);
                dst[2 * q + 1] = (unsigned long long)v.z | ((unsigned long long)v.w << 32);
            }
            if (it.e.n) {
                const unsigned long long lim = h.total_bytes;
                const bool good = it.e.col_num > 0 && (unsigned long long)h.row_num * it.e.col_num < (1ull << 31) &&
                                  it.e.table_off + (h.cell_bits ? (unsigned long long)h.row_num * it.e.col_num * (h.cell_bits / 8) : 16ull) <= lim &&
                                  it.e.flag_off + 8ull * it.e.n_flag_words <= lim && it.e.delta_off + 8ull * it.e.n_delta_words <= lim &&
                                  it.e.restart_off + 16ull * ((it.e.n + SKML_RESTART_INTERVAL - 1) / SKML_RESTART_INTERVAL) <= lim &&
                                  (h.key_encoder == SKML_KEYS_DELTA_BINARY
                                       ? 2ull * it.e.n <= 64ull * it.e.n_flag_words
                                       : (it.e.flag_kind <= 1u && it.e.num_intervals >= 1u && it.e.num_intervals <= 16u &&
                                          (it.e.num_intervals & (it.e.num_intervals - 1u)) == 0u &&
                                          (it.e.num_intervals > 1u || it.e.flag_kind == 0u)));
                it.enc = h.key_encoder;
                it.base = p.payload[r];
                it.tab = it.base + it.e.table_off;
                it.huffman = h.cell_bits == 0 ? 1u : 0u;
                it.cell_bits = it.huffman ? (h.bin_num <= 256 ? 8u : 16u) : h.cell_bits;  // Huffman: width of the expanded table
                it.zero = h.zero_idx;
                it.rows = h.row_num;
                it.off_bv = h.off_bucket_values;
                it.col_magic = good ? skml_fastmod_magic(it.e.col_num) : 0ull;
                it.recip = skml_recip32(it.e.col_num);
                it.mixers = (h.row_num <= 3 && skml_rows_are_mixers(it.e.hash_ids, (int)h.row_num)) ? 1 : 0;
                it.chunk_prefix = good ? 0ull : 1ull;  // scratch use until the compaction below: 1 = failed validation
            }
        }
    }
    __syncthreads();
    // The work table: the non-empty (rank, group) lists moved to the front in (rank, group) order, each
    // with the number of chunks and keys in front of it. Warp 0 does it 32 slots at a time (ballot for the
    // positions, shuffle scans for the prefixes); thread 0 first looks at the per-rank header facts.
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int ni = 0, nhuf = 0;
        unsigned long long chunks = 0, keys = 0, tab_used = 0;
        int dense = 0, ref = 0;
        unsigned int ref_n = 0;
        double mx = 0.0;
        if (lane == 0) {
            for (int r = 0; r < p.world; ++r) {
                const SkmlHeader& h = full[r];
                if (h.kind == SKML_KIND_EMPTY) continue;
                mx = fmax(mx, fmax(fabs(h.min_value), fabs(h.max_value)));
                if (h.kind == SKML_KIND_DENSE) dense = 1;
                else if ((int)h.group_num > gcap) {
                    skml_set_status(p.status, SKML_BAD_HEADER, 0x300u | (unsigned int)r);
                    s.ok = 0;
                }
            }
        }
        const int nslots = p.world * gcap;
        for (int base = 0; base < nslots; base += 32) {
            const int t = base + lane;
            const bool in = t < nslots;
            const int r = in ? t / gcap : 0, g = in ? t % gcap : 0;
            const bool v = in && s.items[t].e.n != 0;
            DecItem it;
            if (v) it = s.items[t];
            const unsigned int n = v ? it.e.n : 0u;
            const bool failed = v && it.chunk_prefix != 0ull;
            const bool huf = v && it.huffman != 0u;
            unsigned long long c_inc = (n + SKML_RESTART_INTERVAL - 1) / SKML_RESTART_INTERVAL, k_inc = n;
            unsigned long long b_inc = huf ? skml_align16((unsigned long long)it.rows * it.e.col_num * (it.cell_bits / 8)) : 0ull;
            const unsigned long long c_own = c_inc, k_own = k_inc, b_own = b_inc;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long c2 = __shfl_up_sync(0xFFFFFFFFu, c_inc, o), k2 = __shfl_up_sync(0xFFFFFFFFu, k_inc, o),
                                         b2 = __shfl_up_sync(0xFFFFFFFFu, b_inc, o);
                if (lane >= o) {
                    c_inc += c2;
                    k_inc += k2;
                    b_inc += b2;
                }
            }
            const unsigned int vm = __ballot_sync(0xFFFFFFFFu, v);
            const int pos = ni + __popc(vm & ((1u << lane) - 1u));
            if (in && g == 0) {   // what lies in front of rank r's first slot
                s.rank_chunk_begin[r] = chunks + c_inc - c_own;
                s.rank_key_begin[r] = keys + k_inc - k_own;
                s.rank_item_begin[r] = pos;
            }
            __syncwarp();   // every lane holds its entry in registers: entries may now move forward
            if (v) {
                it.chunk_prefix = chunks + c_inc - c_own;
                it.key_prefix = keys + k_inc - k_own;
                if (huf) it.tab = p.tab_scratch + tab_used + b_inc - b_own;
                s.items[pos] = it;
            }
            const unsigned int fm = __ballot_sync(0xFFFFFFFFu, failed);
            if (fm) {
                const int r_bad = __shfl_sync(0xFFFFFFFFu, r, __ffs(fm) - 1);
                if (lane == 0) {
                    skml_set_status(p.status, SKML_BAD_HEADER, 0x100u | (unsigned int)r_bad);
                    s.ok = 0;
                }
            }
            // the longest list (the first of equals) gives the apply its range bounds
            unsigned int best_n = n;
            int best_pos = v ? pos : 0x7FFFFFFF;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned int on = __shfl_xor_sync(0xFFFFFFFFu, best_n, o);
                const int op = __shfl_xor_sync(0xFFFFFFFFu, best_pos, o);
                if (on > best_n || (on == best_n && op < best_pos)) {
                    best_n = on;
                    best_pos = op;
                }
            }
            if (best_n > ref_n) {
                ref_n = best_n;
                ref = best_pos;
            }
            chunks += __shfl_sync(0xFFFFFFFFu, c_inc, 31);
            keys += __shfl_sync(0xFFFFFFFFu, k_inc, 31);
            tab_used += __shfl_sync(0xFFFFFFFFu, b_inc, 31);
            ni += __popc(vm);
            nhuf += __popc(__ballot_sync(0xFFFFFFFFu, huf));
            __syncwarp();
        }
      if (lane == 0) {
        if (tab_used > (unsigned long long)p.tab_capacity) {
            skml_set_status(p.status, SKML_CAPACITY, 0x41u);
            s.ok = 0;
        }
        if (keys > (unsigned long long)p.key_capacity) {
            skml_set_status(p.status, SKML_CAPACITY, 0x40u);
            s.ok = 0;
        }
        for (int r = p.world; r <= SKML_MAX_PEERS; ++r) {
            s.rank_chunk_begin[r] = chunks;
            s.rank_key_begin[r] = keys;
            s.rank_item_begin[r] = ni;
        }
        s.ref_item = ref;
        s.nitems = ni;
        s.nhuf = nhuf;
        s.total_chunks = chunks;
        s.total_keys = keys;
        s.any_dense = dense;
        s.direct = (p.adam_v == nullptr) ? 1 : 0;
        s.adam_plain = (!s.direct && !dense && (p.world == 1 || p.val_scratch != nullptr)) ? 1 : 0;
        // Several payloads are decoded into the scratch first and applied by key range when a per-rank
        // pass would leave most blocks with one chunk or none (the pass latency then dominates). Long
        // payloads keep the blocks busy in per-rank passes and skip the scratch round trip; Adam has no
        // per-rank mode, so it always takes the scratch.
        const bool small_passes = chunks < 4ull * gridDim.x * (unsigned long long)p.world;
        s.two_phase = ((s.direct || s.adam_plain) && p.world > 1 && p.val_scratch != nullptr &&
                       (small_passes || s.adam_plain)) ? 1 : 0;
        int e = 0;
        if (mx > 0.0 && isfinite(mx)) frexp(mx, &e);
        s.shift = 60 - e;
        s.inv_world = 1.0 / (double)p.world;
      }
    }
    __syncthreads();
    return s.ok != 0;
}

// Huffman-coded sketch tables -> 8/16-bit bucket codes in the scratch, before any key is decoded
// (binary/HuffmanEncoder.java:126-166 decodes by walking a tree; here the code words, left-aligned and
// sorted, are searched with the next 32 stream bits: in a prefix code the word that matches is the
// largest one not above them). A block works on one item at a time; its threads each decode a stretch
// of cells from a restart offset (every `head[3]` cells; a table without restart offsets is decoded by
// one thread). Never-written cells (Integer.MAX_VALUE) become the zero bucket, as in the narrow form.
__device__ void expand_tables(const DP& p, DecSmem& s) {
    if (s.nhuf == 0) return;
    unsigned char* area = reinterpret_cast<unsigned char*>(&s) + p.tab_off;
    unsigned int* la = reinterpret_cast<unsigned int*>(area);                       // left-aligned code words, ascending
    unsigned short* sym = reinterpret_cast<unsigned short*>(la + DEC_HUF_MAX_ITEMS);  // their symbols (0xFFFF = never written)
    unsigned char* len = reinterpret_cast<unsigned char*>(sym + DEC_HUF_MAX_ITEMS);
    __shared__ unsigned int s_head[4];
    __shared__ int s_bad;
    // blocks are dealt to the Huffman items round-robin; the blocks of one item share its stretches
    const int H = s.nhuf, B = (int)gridDim.x;
    int seen = 0;
    for (int i = 0; i < s.nitems; ++i) {
        const DecItem& it = s.items[i];
        if (!it.huffman) continue;
        const int mine = seen++;
        int helper = 0, nhelp = 1;
        if (H <= B) {
            if ((int)blockIdx.x % H != mine) continue;
            helper = (int)blockIdx.x / H;
            nhelp = (B - mine + H - 1) / H;
        } else if (mine % B != (int)blockIdx.x) {
            continue;
        }
        const unsigned char* sec = it.base + it.e.table_off;
        __syncthreads();
        if (threadIdx.x < 4) s_head[threadIdx.x] = __ldcg(reinterpret_cast<const unsigned int*>(sec) + threadIdx.x);
        if (threadIdx.x == 0) s_bad = 0;
        __syncthreads();
        const unsigned int nitems = s_head[0], nwords = s_head[1], cells = s_head[2], interval = s_head[3];
        const unsigned long long lim = reinterpret_cast<const SkmlHeader*>(it.base)->total_bytes;
        const unsigned int want = it.rows * it.e.col_num;
        const unsigned long long stream_off = it.e.table_off + 16ull + 12ull * nitems;
        const unsigned long long restart_off = skml_align16(stream_off + 8ull * nwords);
        const unsigned int nseg = interval ? (cells + interval - 1) / interval : 1u;
        if (nitems == 0 || nitems > DEC_HUF_MAX_ITEMS || cells != want || stream_off + 8ull * nwords > lim ||
            (interval && restart_off + 4ull * nseg > lim)) {
            if (threadIdx.x == 0) skml_set_status(p.status, SKML_BAD_HEADER, 0x600u | (unsigned int)(i & 0xFF));
            continue;
        }
        // code words: rank sort by the left-aligned word
        for (unsigned int a = threadIdx.x; a < nitems; a += blockDim.x) {
            const int* rec = reinterpret_cast<const int*>(sec + 16) + 3 * a;
            const int value = __ldcg(rec), bits = __ldcg(rec + 1), nb = __ldcg(rec + 2);
            if (nb < 1 || nb > 32) {
                s_bad = 1;
                continue;
            }
            const unsigned int mine_la = (unsigned int)bits << (32 - nb);
            unsigned int r = 0;
            for (unsigned int b = 0; b < nitems; ++b) {
                const int* rb = reinterpret_cast<const int*>(sec + 16) + 3 * b;
                const int nbb = __ldcg(rb + 2);
                const unsigned int other = (nbb >= 1 && nbb <= 32) ? (unsigned int)__ldcg(rb + 1) << (32 - nbb) : 0u;
                if (other < mine_la || (other == mine_la && b < a)) ++r;
            }
            la[r] = mine_la;
            len[r] = (unsigned char)nb;
            sym[r] = value == 0x7FFFFFFF ? (unsigned short)0xFFFFu : (unsigned short)value;
        }
        __syncthreads();
        if (s_bad) {
            if (threadIdx.x == 0) skml_set_status(p.status, SKML_BAD_HEADER, 0x700u | (unsigned int)(i & 0xFF));
            continue;
        }
        const unsigned int* words = reinterpret_cast<const unsigned int*>(it.base + stream_off);
        const unsigned long long wlim = 2ull * nwords;
        const unsigned int* restart = reinterpret_cast<const unsigned int*>(it.base + restart_off);
        unsigned char* out = const_cast<unsigned char*>(it.tab);
        const unsigned int zero = it.zero;
        for (unsigned int sg = (unsigned int)helper * blockDim.x + threadIdx.x; sg < nseg; sg += (unsigned int)nhelp * blockDim.x) {
            unsigned long long pos = interval ? __ldcg(restart + sg) : 0ull;
            const unsigned int c0 = interval ? sg * interval : 0u, c1 = interval ? min(cells, c0 + interval) : cells;
            for (unsigned int c = c0; c < c1; ++c) {
                const unsigned long long w0 = pos >> 5;
                const unsigned int lo = w0 < wlim ? __ldcg(words + w0) : 0u, hi = w0 + 1 < wlim ? __ldcg(words + w0 + 1) : 0u;
                const unsigned int x = __brev(__funnelshift_r(lo, hi, (unsigned int)(pos & 31ull)));
                unsigned int a = 0, b = nitems;   // largest word <= x
                while (b - a > 1) {
                    const unsigned int mid = (a + b) >> 1;
                    if (la[mid] <= x) a = mid;
                    else b = mid;
                }
                unsigned int v = sym[a] == 0xFFFFu ? zero : sym[a];
                if (it.cell_bits == 8) out[c] = (unsigned char)v;
                else reinterpret_cast<unsigned short*>(out)[c] = (unsigned short)v;
                pos += len[a];
            }
        }
    }
    __syncthreads();
}

// D1 for sparse payloads: one 1024-key chunk per block iteration, DEC_KPT adjacent keys per
// thread (256 threads), so that every thread has several independent load chains in flight and
// several blocks share an SM.
__device__ void decode_accumulate(const DP& p, DecSmem& s, unsigned long long ch_begin, unsigned long long ch_end, float& dsq) {
    __shared__ unsigned int s_part[6][DEC_THREADS / 32];  // [3 scans x chunk parity]
    __shared__ unsigned short s_pos[SKML_RESTART_INTERVAL];  // delta_adaptive with unary flags: where every key's flag ends
    int par = 0;
    // Every block takes a contiguous run of chunks, so that consecutive chunks belong to the same
    // (rank, group) list and its sketch table, when it fits, is staged in shared memory once and
    // then queried there: three random L2 sectors per key become one coalesced read of the table.
    const unsigned long long per = (ch_end - ch_begin + gridDim.x - 1) / gridDim.x;
    const unsigned long long my_begin = ch_begin + per * blockIdx.x;
    const unsigned long long my_end = my_begin + per < ch_end ? my_begin + per : ch_end;
    unsigned char* tab_area = p.tab_off ? reinterpret_cast<unsigned char*>(&s) + p.tab_off : nullptr;
    int staged = -1, it_i = 0;
    const unsigned char* stab = nullptr;
    for (unsigned long long ch = my_begin; ch < my_end; ++ch, par ^= 1) {
        while (it_i + 1 < s.nitems && ch >= s.items[it_i + 1].chunk_prefix) ++it_i;
        const DecItem& it = s.items[it_i];
        if (it_i != staged) {
            staged = it_i;
            stab = stage_table(it, tab_area);
        }
        ChunkKeys c;
        decode_chunk(p, it, (unsigned int)(ch - it.chunk_prefix), stab, s_part[par], s_part[2 + par], s_part[4 + par], s_pos, c);
        if (c.i0 < c.cnt) {
            int* ks = p.key_scratch + it.key_prefix + c.first;
            if (s.two_phase) {
                // stash (key, value): the ordered apply passes read them back coalesced
                float* vs = p.val_scratch + it.key_prefix + c.first;
#pragma unroll
                for (int u = 0; u < DEC_KPT; ++u)
                    if (c.i0 + u < c.cnt) {
                        ks[c.i0 + u] = (int)c.keys[u];
                        vs[c.i0 + u] = c.bv[u] * (float)s.inv_world;
                    }
            } else if (s.direct) {  // single payload: keys are unique inside it, plain read-modify-write
#pragma unroll
                for (int u = 0; u < DEC_KPT; ++u)
                    if (c.live[u]) dsq += apply_direct(p, c.keys[u], c.bv[u] * (float)s.inv_world);
            } else if (s.adam_plain) {  // single payload: the decoded value is the whole gradient of its key
#pragma unroll
                for (int u = 0; u < DEC_KPT; ++u)
                    if (c.live[u] && c.bv[u] != 0.f) dsq += apply_one(p, c.keys[u], c.bv[u] * (float)s.inv_world);
            } else {
#pragma unroll
                for (int u = 0; u < DEC_KPT; ++u) {
                    if (c.i0 + u < c.cnt) ks[c.i0 + u] = (int)c.keys[u];
                    const long long fx = c.live[u] ? to_fixed((double)c.bv[u] * s.inv_world, s.shift) : 0ll;
                    if (fx) atomicAdd(reinterpret_cast<unsigned long long*>(p.acc + c.keys[u]), (unsigned long long)fx);
                }
            }
        }
        // no barrier here: the next chunk's scans use the other parity of s_part
    }
    __syncthreads();
}

// Ordered apply of one rank's stashed (key, value) pairs: keys are unique inside a payload, so the
// plain read-modify-write needs no atomics; four independent pairs per thread and iteration.
__device__ void apply_stashed(const DP& p, unsigned long long begin, unsigned long long end, float& dsq) {
    const unsigned long long gsz = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long t = begin + (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; t < end; t += 4 * gsz) {
        unsigned int k[4];
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const unsigned long long tt = t + u * gsz;
            k[u] = tt < end ? (unsigned int)__ldcg(p.key_scratch + tt) : 0xFFFFFFFFu;
            v[u] = tt < end ? __ldcg(p.val_scratch + tt) : 0.f;
        }
        float old[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float* dst = p.out_sum ? p.out_sum : p.w;
            old[u] = k[u] < (unsigned long long)p.dim ? dst[k[u]] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (k[u] < (unsigned long long)p.dim) {
                if (p.out_sum) p.out_sum[k[u]] = old[u] + v[u];
                else {
                    const float nw = old[u] - p.lr * v[u];
                    p.w[k[u]] = nw;
                    dsq += (nw - old[u]) * (nw + old[u]);
                }
            }
    }
}

// One rank's slice of the block's key range. OP 0: SGD step / plain sum; OP 1: add into the float
// accumulators; OP 2: Adam update of every coordinate whose accumulated sum is non-zero, then clear it.
// The groups of one rank hold disjoint keys, so their slices are walked as one concatenated list,
// four independent entries per thread and iteration; a block barrier ends the pass.
template <int OP>
__device__ __forceinline__ void owned_pass(const DP& p, DecSmem& s, const unsigned long long* seg_b,
                                           const unsigned long long* seg_e, int r, float& dsq) {
    const int i0 = s.rank_item_begin[r], i1 = s.rank_item_begin[r + 1];
    float* dst = OP == 0 ? (p.out_sum ? p.out_sum : p.w) : p.fsum;
    const long long ds = OP == 0 ? 1ll : p.fsum_stride;
    unsigned int total = 0;
    for (int i = i0; i < i1; ++i) total += (unsigned int)(seg_e[i] - seg_b[i]);
    for (unsigned int q = threadIdx.x; q < total; q += 4 * blockDim.x) {
        unsigned int k[4];
        float v[4], old[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            unsigned int qq = q + u * blockDim.x;
            k[u] = 0xFFFFFFFFu;
            v[u] = 0.f;
            if (qq < total) {
                int i = i0;
                unsigned int len = (unsigned int)(seg_e[i] - seg_b[i]);
                while (qq >= len) {
                    qq -= len;
                    ++i;
                    len = (unsigned int)(seg_e[i] - seg_b[i]);
                }
                const unsigned long long pos = seg_b[i] + qq;
                k[u] = (unsigned int)__ldcg(p.key_scratch + pos);
                if (OP != 2) v[u] = __ldcg(p.val_scratch + pos);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) old[u] = k[u] < (unsigned long long)p.dim ? dst[k[u] * ds] : 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (k[u] >= (unsigned long long)p.dim) continue;
            if (OP == 0) {
                const float nw = p.out_sum ? old[u] + v[u] : old[u] - p.lr * v[u];
                dst[k[u]] = nw;
                if (!p.out_sum) dsq += (nw - old[u]) * (nw + old[u]);
            } else if (OP == 1) dst[k[u] * ds] = old[u] + v[u];
            else if (old[u] != 0.f) {
                dst[k[u] * ds] = 0.f;
                dsq += apply_one(p, k[u], old[u]);
            }
        }
    }
    __syncthreads();
}

// Barrier-free ordered apply. The key space is cut into DEC_OWN_RANGES x blocks ranges at the quantiles
// of the longest key list; a block owns one range per round, dealt in snake order (round 0: range b,
// round 1: range 2B - 1 - b, ...). Low keys are the frequent ones and sit in L2 while the high ones
// miss to DRAM, so a block's ranges cost about the same in sum although single ranges differ several
// times. For each of its ranges the block finds its slice of every (rank, group) list by binary search
// in the stashed keys and applies the slices rank by rank with only a block barrier in between: all
// updates of one coordinate happen in one block, in rank order, so replicas stay bit-identical.
__device__ void apply_owned(const DP& p, DecSmem& s, float& dsq) {
    if (s.nitems == 0) return;
    unsigned long long* seg = reinterpret_cast<unsigned long long*>(&s.items[p.max_items]);  // [2 * DEC_OWN_RANGES][max_items]
    __shared__ unsigned long long s_bound[2 * DEC_OWN_RANGES];
    // SGD: one range per block (more ranges even out the blocks but do not shorten the launch: the random
    // DRAM sectors bound it in total); lazy Adam sweeps a range 2 x ranks times, and smaller ranges keep
    // its sectors in L2 between the sweeps
    const int rounds = p.adam_v ? DEC_OWN_RANGES : 1;
    if (threadIdx.x < 2 * rounds) {
        const DecItem& ref = s.items[s.ref_item];
        const unsigned long long B = gridDim.x, total = (unsigned long long)rounds * B;
        const unsigned long long round = threadIdx.x >> 1;
        const unsigned long long range = (round & 1ull) ? (round + 1ull) * B - 1ull - blockIdx.x : round * B + blockIdx.x;
        const unsigned long long j = range + (threadIdx.x & 1);   // lower / upper bound of the range
        unsigned long long v;
        if (j == 0) v = 0ull;
        else if (j >= total) v = 1ull << 32;
        else v = (unsigned long long)(unsigned int)__ldcg(p.key_scratch + ref.key_prefix + j * (unsigned long long)ref.e.n / total);
        s_bound[threadIdx.x] = v;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < 2 * rounds * s.nitems; t += blockDim.x) {
        const int item = t / (2 * rounds), which = t % (2 * rounds);
        const DecItem& it = s.items[item];
        const unsigned long long bound = s_bound[which];
        const int* list = p.key_scratch + it.key_prefix;
        unsigned int lo = 0, hi = it.e.n;
        while (lo < hi) {  // first position whose key is >= bound
            const unsigned int mid = (lo + hi) >> 1;
            if ((unsigned long long)(unsigned int)__ldcg(list + mid) < bound) lo = mid + 1;
            else hi = mid;
        }
        seg[(size_t)which * p.max_items + item] = it.key_prefix + lo;
    }
    __syncthreads();
    for (int round = 0; round < rounds; ++round) {
        const unsigned long long* seg_b = seg + (size_t)(2 * round) * p.max_items;
        const unsigned long long* seg_e = seg_b + p.max_items;
        if (p.adam_v) {
            // Adam: sum the ranks' values per coordinate in rank order (plain floats in the zeroed
            // sums), then let the first rank that holds a coordinate apply the update and clear the sum.
            for (int r = 0; r < p.world; ++r) owned_pass<1>(p, s, seg_b, seg_e, r, dsq);
            for (int r = 0; r < p.world; ++r) owned_pass<2>(p, s, seg_b, seg_e, r, dsq);
        } else {
            for (int r = 0; r < p.world; ++r) owned_pass<0>(p, s, seg_b, seg_e, r, dsq);
        }
    }
}

// D1 for dense payloads: every coordinate carries a bucket code.
__device__ void decode_accumulate_dense(const DP& p, DecSmem& s, int r_begin, int r_end, float& dsq) {
    const long long gsz = (long long)gridDim.x * blockDim.x, gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (int r = r_begin; r < r_end; ++r) {
        const HdrLite& h = s.hdr[r];
        if (h.kind != SKML_KIND_DENSE) continue;
        const unsigned char* codes = p.payload[r] + h.off_dense_codes;
        const float* bv = reinterpret_cast<const float*>(p.payload[r] + h.off_bucket_values);
        for (long long i = gid; i < p.dim; i += gsz) {
            unsigned int code = h.cell_bits == 8 ? __ldcg(codes + i) : __ldcg(reinterpret_cast<const unsigned short*>(codes) + i);
            if (code >= h.bin_num) code = h.zero_idx;
            if (s.direct) {
                dsq += apply_direct(p, i, __ldcg(bv + code) * (float)s.inv_world);
                continue;
            }
            const long long fx = to_fixed((double)__ldcg(bv + code) * s.inv_world, s.shift);
            if (fx) atomicAdd(reinterpret_cast<unsigned long long*>(p.acc + i), (unsigned long long)fx);
        }
    }
}

// D2: claim and update.
__device__ void decode_update(const DP& p, DecSmem& s, float& dsq) {
    const long long gsz = (long long)gridDim.x * blockDim.x, gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (s.any_dense) {
        for (long long i = gid; i < p.dim; i += gsz) {
            long long a = p.acc[i];
            if (a) {
                p.acc[i] = 0;
                dsq += apply_one(p, i, (float)from_fixed(a, s.shift));
            }
        }
    } else {
        // four independent claims per thread and iteration: their round trips overlap
        for (long long t = gid; t < (long long)s.total_keys; t += 4 * gsz) {
            long long k[4], a[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long tt = t + u * gsz;
                k[u] = tt < (long long)s.total_keys ? (long long)(unsigned int)p.key_scratch[tt] : p.dim;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                a[u] = k[u] < p.dim ? (long long)atomicExch(reinterpret_cast<unsigned long long*>(p.acc + k[u]), 0ull) : 0ll;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (a[u]) dsq += apply_one(p, k[u], (float)from_fixed(a[u], s.shift));
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.loss_out) {
        double l[4] = {0, 0, 0, 0};
        for (int r = 0; r < p.world; ++r)
            for (int i = 0; i < 4; ++i) l[i] += s.hdr[r].loss_partials[i];
        for (int i = 0; i < 4; ++i) p.loss_out[i] = l[i];
    }
}

// Adds the launch's change of the squared weight norm to the running sum; the last block to arrive
// turns the sum into the regularisation loss of the next batch (lambda * ||w||_2, un-squared as in
// ml/objective/Loss.scala:48-53) so that no step passes over the whole model for it.
__device__ void finish_norm(const DP& p, float dsq) {
    if (!p.wsq) return;
    __shared__ double s_red[DEC_THREADS / 32];
    double d = (double)dsq;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d += __shfl_down_sync(0xFFFFFFFFu, d, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = d;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < DEC_THREADS / 32; ++w) t += s_red[w];
        if (t != 0.0) atomicAdd(p.wsq, t);
        __threadfence();
        const unsigned int prev = atomicAdd(&p.ctrl[3], 1u);
        if (prev == gridDim.x - 1) {
            p.ctrl[3] = 0;
            __threadfence();
            const double w2 = *reinterpret_cast<volatile double*>(p.wsq);
            if (p.reg_out) p.reg_out[0] = p.reg_lambda * sqrt(w2 > 0.0 ? w2 : 0.0);
        }
    }
}

template <bool FUSED>
__global__ void __launch_bounds__(DEC_THREADS, DEC_BLOCKS_PER_SM) decode_update_kernel(DP p, int stage) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    DecSmem& s = *reinterpret_cast<DecSmem*>(smem_raw);
    float dsq = 0.f;  // this thread's share of the change of ||w||^2
    if (FUSED && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        reinterpret_cast<unsigned long long*>(p.ctrl)[8 + 4 * (int)(p.step & 1)] = t;
    }
    if (!decode_prepare(p, s)) return;
    if (s.nhuf) {  // tables that arrived Huffman-coded become plain bucket codes first
        if (FUSED || stage == 0) expand_tables(p, s);
        if (FUSED) {
            if (!skml_grid_barrier(p.ctrl, gridDim.x, p.status, p.budget, 0x2Eu)) return;
        }
    }
    if (!FUSED && stage == 0) return;
    if (FUSED && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        reinterpret_cast<unsigned long long*>(p.ctrl)[9 + 4 * (int)(p.step & 1)] = t;
    }
    if (s.direct || s.adam_plain) {
        if (s.two_phase) {
            // Phase 1 (un-fused: stage 1): every payload's keys and values, no ordering needed.
            if (FUSED || stage == 1) decode_accumulate(p, s, 0, s.total_chunks, dsq);
            if (FUSED) {
                if (!skml_grid_barrier(p.ctrl, gridDim.x, p.status, p.budget, 0x2Fu)) return;
                if (blockIdx.x == 0 && threadIdx.x == 0) {
                    unsigned long long t;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                    reinterpret_cast<unsigned long long*>(p.ctrl)[10 + 4 * (int)(p.step & 1)] = t;
                }
            }
            // Phase 2 without dense payloads (un-fused: stage 2): key-range-owned apply, no grid barrier.
            if (!s.any_dense) {
                if (FUSED || stage == 2) apply_owned(p, s, dsq);
            } else
            // Phase 2 with dense payloads (un-fused: stage r + 2): one apply pass per rank, in rank order.
            for (int r = 0; r < p.world; ++r) {
                if (FUSED || stage == r + 2) {
                    apply_stashed(p, s.rank_key_begin[r], s.rank_key_begin[r + 1], dsq);
                    if (s.any_dense) decode_accumulate_dense(p, s, r, r + 1, dsq);
                }
                if (FUSED && r + 1 < p.world) {
                    if (!skml_grid_barrier(p.ctrl, gridDim.x, p.status, p.budget, 0x30u + r)) return;
                }
            }
        } else {
            // one pass per rank; un-fused launches run pass `stage - 1` each
            for (int r = 0; r < p.world; ++r) {
                if (FUSED || stage == r + 1) {
                    decode_accumulate(p, s, s.rank_chunk_begin[r], s.rank_chunk_begin[r + 1], dsq);
                    if (s.any_dense) decode_accumulate_dense(p, s, r, r + 1, dsq);
                }
                if (FUSED && r + 1 < p.world) {
                    if (!skml_grid_barrier(p.ctrl, gridDim.x, p.status, p.budget, 0x30u + r)) return;
                }
            }
        }
        if ((FUSED || stage == 1) && blockIdx.x == 0 && threadIdx.x == 0 && p.loss_out) {
            double l[4] = {0, 0, 0, 0};
            for (int r = 0; r < p.world; ++r)
                for (int i = 0; i < 4; ++i) l[i] += s.hdr[r].loss_partials[i];
            for (int i = 0; i < 4; ++i) p.loss_out[i] = l[i];
        }
        if (FUSED && blockIdx.x == 0 && threadIdx.x == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (!s.two_phase) reinterpret_cast<unsigned long long*>(p.ctrl)[10 + 4 * (int)(p.step & 1)] = t;
            reinterpret_cast<unsigned long long*>(p.ctrl)[11 + 4 * (int)(p.step & 1)] = t;
        }
        finish_norm(p, dsq);
        if (FUSED) {
            // the last block to finish leaves the kernel's true end time (block 0's stamp above is its own)
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned int prev = atomicAdd(&p.ctrl[2], 1u);
                if (prev == gridDim.x - 1) {
                    p.ctrl[2] = 0;
                    unsigned long long t;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                    reinterpret_cast<unsigned long long*>(p.ctrl)[16 + (int)(p.step & 1)] = t;
                }
            }
        }
        return;
    }
    if (FUSED || stage == 1) {
        decode_accumulate(p, s, 0, s.total_chunks, dsq);
        if (s.any_dense) decode_accumulate_dense(p, s, 0, p.world, dsq);
    }
    if (FUSED) {
        if (!skml_grid_barrier(p.ctrl, gridDim.x, p.status, p.budget, 0x21u)) return;
    }
    if (FUSED && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        reinterpret_cast<unsigned long long*>(p.ctrl)[10 + 4 * (int)(p.step & 1)] = t;
    }
    if (FUSED || stage == 2) decode_update(p, s, dsq);
    if (FUSED && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        reinterpret_cast<unsigned long long*>(p.ctrl)[11 + 4 * (int)(p.step & 1)] = t;
    }
    finish_norm(p, dsq);
}

extern "C" long long skml_decode_workspace_bytes(long long world, long long group_num) {
    (void)world;
    (void)group_num;
    return 256;
}

extern "C" int skml_decode_update(const SkmlDecodeArgs* a, void* stream_) {
    if (!a || !a->acc || !a->key_scratch || !a->workspace || !a->status) return (int)cudaErrorInvalidValue;
    if (a->world < 1 || a->world > SKML_MAX_PEERS) return (int)cudaErrorInvalidValue;
    if (!a->out_sum && !a->w) return (int)cudaErrorInvalidValue;
    cudaStream_t stream = (cudaStream_t)stream_;
    DP p;
    for (int i = 0; i < SKML_MAX_PEERS; ++i) {
        p.payload[i] = a->payload[i];
        p.flag[i] = a->flag[i];
    }
    p.world = (int)a->world;
    p.slot_capacity = a->slot_capacity;
    p.step = a->step;
    p.dim = a->dim;
    p.w = a->w;
    p.adam_m = a->adam_m;
    p.adam_v = a->adam_v;
    p.adam_stride = a->adam_stride > 1 ? a->adam_stride : 1;
    if (p.adam_stride == 4 && a->adam_m) {
        p.fsum = a->adam_m + 2;   // packed quads {m, v, sum, -}: the three words of a coordinate share a sector
        p.fsum_stride = 4;
    } else {
        p.fsum = reinterpret_cast<float*>(a->acc);
        p.fsum_stride = 1;
    }
    p.lr = (float)a->lr;
    p.adam_scale = (float)a->adam_scale;
    p.acc = a->acc;
    p.key_scratch = a->key_scratch;
    p.val_scratch = a->val_scratch;
    p.tab_scratch = a->table_scratch;
    p.tab_capacity = a->table_capacity;
    p.wsq = a->out_sum ? nullptr : a->weight_sumsq;
    p.reg_out = a->reg_out;
    p.reg_lambda = a->reg_lambda;
    p.key_capacity = a->key_capacity;
    p.loss_out = a->loss_out;
    p.out_sum = a->out_sum;
    p.ctrl = reinterpret_cast<unsigned int*>(a->workspace);
    p.status = a->status;
    p.budget = a->budget_cycles > 0 ? a->budget_cycles : 2000000000ll;
    // the (rank, group) table lives in dynamic shared memory: world x groups entries
    long long groups = a->max_groups > 0 ? a->max_groups : SKML_MAX_GROUPS;
    if (groups > SKML_MAX_GROUPS) groups = SKML_MAX_GROUPS;
    p.max_items = (int)(a->world * groups);
    // dynamic shared memory: work table, two slice bounds per entry, then the staged-table area
    const size_t smem_items = (sizeof(DecSmem) + (size_t)p.max_items * (sizeof(DecItem) + 16 * DEC_OWN_RANGES) + 15) & ~(size_t)15;
    p.tab_off = (int)smem_items;
    const size_t smem = smem_items + DEC_TAB_SMEM;
    static int sms = 0;
    static size_t cached_smem = 0;
    static int max_grid = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        const int cap = (int)(sizeof(DecSmem) + (size_t)DEC_MAX_ITEMS * (sizeof(DecItem) + 16 * DEC_OWN_RANGES) + 16 + DEC_TAB_SMEM);
        cudaError_t e0 = cudaFuncSetAttribute(decode_update_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap);
        if (e0 == cudaSuccess)
            e0 = cudaFuncSetAttribute(decode_update_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap);
        if (e0 != cudaSuccess) {
            sms = 0;
            return (int)e0;
        }
    }
    if (cached_smem != smem) {
        int per_sm = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_update_kernel<true>, DEC_THREADS, smem);
        max_grid = per_sm * sms;
        cached_smem = smem;
    }
    int grid = a->grid > 0 ? (int)a->grid : DEC_BLOCKS_PER_SM * sms;
    cudaError_t e;
    if (a->fused) {
        if (max_grid < 1) return (int)cudaErrorLaunchOutOfResources;
        if (grid > max_grid) grid = max_grid;
        int stage = -1;
        void* args[] = {&p, &stage};
        return (int)cudaLaunchCooperativeKernel((const void*)decode_update_kernel<true>, dim3(grid), dim3(DEC_THREADS), args,
                                                smem, stream);
    }
    // stages: Adam = accumulate + claims; SGD over several payloads with a value scratch = decode +
    // one apply pass per rank; otherwise one pass per rank
    const int nst = a->adam_v ? 2 : ((a->world > 1 && a->val_scratch) ? (int)a->world + 1 : (int)a->world);
    for (int st = a->table_scratch ? 0 : 1; st <= nst; ++st) {
        decode_update_kernel<false><<<grid, DEC_THREADS, smem, stream>>>(p, st);
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

// ---------------------------------------------------------------------------
// Peer memory helpers (one process per GPU, same node).
// ---------------------------------------------------------------------------
extern "C" int skml_ipc_get_handle(void* dev_ptr, unsigned char* handle64) {
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, dev_ptr);
    if (e != cudaSuccess) return (int)e;
    memcpy(handle64, &h, sizeof(h));
    return 0;
}

extern "C" int skml_ipc_open_handle(const unsigned char* handle64, void** dev_ptr) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    return (int)cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

extern "C" int skml_ipc_close(void* dev_ptr) { return (int)cudaIpcCloseMemHandle(dev_ptr); }

// A zeroed device allocation of its own (cudaMalloc): the IPC handle of a receive region then names
// exactly that region, whatever a caching allocator does with the rest of the memory.
extern "C" int skml_region_alloc(long long bytes, void** dev_ptr) {
    if (bytes <= 0 || !dev_ptr) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaMalloc(dev_ptr, (size_t)bytes);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaMemset(*dev_ptr, 0, (size_t)bytes);
}

extern "C" int skml_region_free(void* dev_ptr) { return (int)cudaFree(dev_ptr); }

extern "C" int skml_enable_peer_access(int peer_device) {
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return 0;
    }
    return (int)e;
}
