// Definitions shared by the CPU oracle (g++) and the sm_100a kernels (nvcc):
// the SKML payload container, the eight Java-exact integer hash functions, the
// counter-based random numbers that pick hash rows and compaction offsets, and
// the bucket-group edge rule.
//
// Reference behaviour restated here (paths inside the reference project):
//   sketch/.../hash/BJHash.java:10-20, Mix64Hash.java:10-21, TWHash.java:10-20,
//   BKDRHash.java:13-21, HashFactory.java:10-37   -> skml_hash / skml_pick_hashes
//   sketch/.../sketch/frequency/FSketchUtils.java:9-28 -> skml_group_edges
//   sketch/.../sketch/frequency/GroupedMinMaxSketch.java:148-158,
//   MinMaxSketch.java:88-97, DeltaBinaryEncoder.java:67-87 -> field lists of the container
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define SKML_HD __host__ __device__ __forceinline__
#else
#define SKML_HD inline
#endif

#define SKML_MAGIC 0x4C4D4B53u /* 'S','K','M','L' little-endian */
#define SKML_VERSION 1u
#define SKML_MAX_GROUPS 32
#define SKML_MAX_ROWS 8
#define SKML_MAX_BINS 65536
#define SKML_HEADER_BYTES 256
#define SKML_GROUP_ENTRY_BYTES 64
#define SKML_RESTART_INTERVAL 1024 /* keys between two restart points of a key stream */
#define SKML_EMPTY_CELL 0xFFFFFFFFu

enum SkmlKind { SKML_KIND_EMPTY = 0, SKML_KIND_SPARSE = 1, SKML_KIND_DENSE = 2 };
enum SkmlDtype { SKML_F32 = 0, SKML_F64 = 1 };
enum SkmlKeyEncoder { SKML_KEYS_DELTA_BINARY = 0, SKML_KEYS_DELTA_ADAPTIVE = 1 };
// cell_bits: 8 or 16 = narrow bucket codes (empty cells hold zero_idx), 32 = raw
// int32 cells with the reference's Integer.MAX_VALUE sentinel, 0 = Huffman section.
enum SkmlCells { SKML_CELLS_HUFFMAN = 0, SKML_CELLS_U8 = 8, SKML_CELLS_U16 = 16, SKML_CELLS_I32 = 32 };

// Payload header, little-endian, 256 bytes. Every section offset is in bytes
// from the start of the payload and 16-byte aligned.
struct SkmlHeader {
    uint32_t magic, version;
    uint32_t kind, dtype;
    uint64_t step;
    uint32_t rank, world;
    uint64_t dim, nnz;
    uint32_t bin_num;  // effective bucket count after duplicate splits were dropped
    uint32_t zero_idx;
    uint32_t group_num, row_num;
    double col_ratio;
    uint32_t key_encoder, cell_bits;
    uint64_t seed;
    double loss_partials[4];  // batch size, objective loss sum, reg loss, spare
    double min_value, max_value;
    uint32_t restart_interval, flags;
    uint64_t total_bytes;
    uint64_t off_bucket_values, off_group_table, off_tables, off_key_flags, off_key_deltas,
        off_restart, off_dense_codes;
    uint64_t header_checksum;  // FNV-1a 64 recurrence over the 64-bit words before this field
    uint8_t pad[SKML_HEADER_BYTES - 216];
};
static_assert(sizeof(SkmlHeader) == SKML_HEADER_BYTES, "SkmlHeader must be 256 bytes");

// One entry per bucket group (fields of MinMaxSketch + key encoder writeObject).
struct SkmlGroupEntry {
    uint32_t n;            // keys in this group (0 = empty group: no sections)
    uint32_t col_num;      // ceil(n * col_ratio)
    uint8_t hash_ids[8];   // row r uses family member hash_ids[r]
    uint64_t table_off;    // row_num x col_num cells
    uint64_t flag_off;     // u64 words, java.util.BitSet bit order
    uint32_t n_flag_words;
    uint32_t num_intervals;  // delta_adaptive only (1,2,4,8,16); 4 for delta_binary
    uint64_t delta_off;
    uint32_t n_delta_words;
    uint32_t flag_kind;      // delta_adaptive only: 1 = unary flags
    uint64_t restart_off;    // ceil(n / restart_interval) x SkmlRestart, 0 if none
};
static_assert(sizeof(SkmlGroupEntry) == SKML_GROUP_ENTRY_BYTES, "SkmlGroupEntry must be 64 bytes");

// Restart point j of a group: decoding may begin at key j*restart_interval with
// `prev_key` as the running key and `delta_bit_off` / `flag_bit_off` as stream cursors.
struct SkmlRestart {
    uint32_t prev_key;
    uint32_t flag_bit_off;  // a group's flag stream is limited to 2^32 bits
    uint64_t delta_bit_off;
};
static_assert(sizeof(SkmlRestart) == 16, "SkmlRestart must be 16 bytes");

SKML_HD uint64_t skml_align16(uint64_t x) { return (x + 15ull) & ~15ull; }

SKML_HD uint64_t skml_fnv1a(const uint8_t* p, uint32_t n) {
    uint64_t h = 1469598103934665603ull;
    for (uint32_t i = 0; i < n; ++i) {
        h ^= p[i];
        h *= 1099511628211ull;
    }
    return h;
}

// Header checksum: the FNV-1a recurrence over the header's 64-bit little-endian words (not its bytes: the
// fused kernels compute it on their critical path, one dependent multiply per step, 18 steps instead of 144).
SKML_HD uint64_t skml_header_checksum(const SkmlHeader* h) {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(h);
    const uint32_t n = (uint32_t)(((const uint8_t*)&h->header_checksum - (const uint8_t*)h) / 8);
    uint64_t x = 1469598103934665603ull;
    for (uint32_t i = 0; i < n; ++i) {
        x ^= w[i];
        x *= 1099511628211ull;
    }
    return x;
}
static_assert(offsetof(SkmlHeader, header_checksum) % 8 == 0, "the checksum covers whole 64-bit words");

// ---------------------------------------------------------------------------
// Integer hashes with Java int semantics: adds, multiplies and left shifts wrap
// (done in uint32_t), `>>` is arithmetic (done on int32_t), `%` truncates toward
// zero and a negative remainder is moved up by `size`.
// ---------------------------------------------------------------------------
SKML_HD int32_t skml_sar(uint32_t c, int s) { return (int32_t)c >> s; }

SKML_HD int32_t skml_mod_size(uint32_t code, int32_t size) {
    int32_t r = (int32_t)code % size;
    return r >= 0 ? r : r + size;
}

SKML_HD uint32_t skml_mix_bj(uint32_t c) {
    c = (c + 0x7ed55d16u) + (c << 12);
    c = (c ^ 0xc761c23cu) ^ (uint32_t)skml_sar(c, 19);
    c = (c + 0x165667b1u) + (c << 5);
    c = (c + 0xd3a2646cu) ^ (c << 9);
    c = (c + 0xfd7046c5u) + (c << 3);
    c = (c ^ 0xb55a4f09u) ^ (uint32_t)skml_sar(c, 16);
    return c;
}

SKML_HD uint32_t skml_mix_64(uint32_t c) {
    c = (~c) + (c << 21);
    c = c ^ (uint32_t)skml_sar(c, 24);
    c = (c + (c << 3)) + (c << 8);
    c = c ^ (uint32_t)skml_sar(c, 14);
    c = (c + (c << 2)) + (c << 4);
    c = c ^ (uint32_t)skml_sar(c, 28);
    c = c + (c << 31);
    return c;
}

SKML_HD uint32_t skml_mix_tw(uint32_t c) {
    c = ~c + (c << 15);
    c = c ^ (uint32_t)skml_sar(c, 12);
    c = c + (c << 2);
    c = c ^ (uint32_t)skml_sar(c, 4);
    c = c * 2057u;
    c = c ^ (uint32_t)skml_sar(c, 16);
    return c;
}

SKML_HD uint32_t skml_mix_bkdr(int32_t key, uint32_t seed) {
    uint32_t c = 0;
    while (key != 0) {
        c = seed * c + (uint32_t)(key % 10);  // key % 10 keeps the sign of key, as in Java
        key /= 10;
    }
    return c;
}

// Family order of HashFactory: BJ, Mix64, TW, BKDR31, BKDR131, BKDR267, BKDR1313, BKDR13131.
SKML_HD int32_t skml_hash(int id, int32_t key, int32_t size) {
    uint32_t c;
    switch (id) {
        case 0: c = skml_mix_bj((uint32_t)key); break;
        case 1: c = skml_mix_64((uint32_t)key); break;
        case 2: c = skml_mix_tw((uint32_t)key); break;
        case 3: c = skml_mix_bkdr(key, 31u); break;
        case 4: c = skml_mix_bkdr(key, 131u); break;
        case 5: c = skml_mix_bkdr(key, 267u); break;
        case 6: c = skml_mix_bkdr(key, 1313u); break;
        default: c = skml_mix_bkdr(key, 13131u); break;
    }
    return skml_mod_size(c, size);
}

// Division-free variants for the kernels' inner loops. They return exactly what
// skml_hash returns for non-negative keys (checked against it on the CPU):
// * the decimal digits of a key are extracted once and shared by the BKDR members;
// * `x % size` uses a precomputed magic number (Lemire's fastmod: for 32-bit x and size,
//   x mod size = mulhi64(magic * x, size) with magic = floor((2^64 - 1) / size) + 1).
struct SkmlKeyDigits {
    uint64_t packed;  // digit i (least significant first) in bits [4i, 4i + 4)
    int count;
};

SKML_HD void skml_key_digits(int32_t key, SkmlKeyDigits& kd) {
    uint32_t k = key < 0 ? 0u : (uint32_t)key;
    kd.packed = 0;
    kd.count = 0;
    while (k != 0) {
        uint32_t q = k / 10u;
        kd.packed |= (uint64_t)(k - q * 10u) << (4 * kd.count);
        ++kd.count;
        k = q;
    }
}

SKML_HD uint64_t skml_fastmod_magic(uint32_t size) { return 0xFFFFFFFFFFFFFFFFull / size + 1ull; }

SKML_HD uint32_t skml_fastmod(uint32_t x, uint64_t magic, uint32_t size) {
    uint64_t low = magic * (uint64_t)x;
#if defined(__CUDA_ARCH__)
    return (uint32_t)__umul64hi(low, (uint64_t)size);
#else
    return (uint32_t)(((unsigned __int128)low * size) >> 64);
#endif
}

SKML_HD int32_t skml_hash_fast(int id, int32_t key, const SkmlKeyDigits& kd, int32_t size, uint64_t magic) {
    if (key < 0) return skml_hash(id, key, size);
    uint32_t c;
    if (id == 0) c = skml_mix_bj((uint32_t)key);
    else if (id == 1) c = skml_mix_64((uint32_t)key);
    else if (id == 2) c = skml_mix_tw((uint32_t)key);
    else {
        const uint32_t seed = id == 3 ? 31u : (id == 4 ? 131u : (id == 5 ? 267u : (id == 6 ? 1313u : 13131u)));
        c = 0;
        for (int i = 0; i < kd.count; ++i) c = seed * c + (uint32_t)((kd.packed >> (4 * i)) & 15u);
    }
    const int32_t sc = (int32_t)c;
    if (sc >= 0) return (int32_t)skml_fastmod(c, magic, (uint32_t)size);
    const uint32_t m = skml_fastmod((uint32_t)(-(int64_t)sc), magic, (uint32_t)size);  // Java: remainder keeps the sign
    return m ? size - (int32_t)m : 0;
}

// All `rows` (<= MAXR) table positions of one key at once; equal to skml_hash(ids[r], key, size)
// for every row. The BKDR members share ONE pass over the key's decimal digits: each keeps its own
// accumulator and every digit costs one divide-by-constant plus one multiply-add per row.
template <int MAXR>
SKML_HD void skml_hash_rows(const uint8_t* ids, int rows, int32_t key, int32_t size, uint64_t magic, int32_t* out) {
    if (key < 0) {
        for (int r = 0; r < MAXR; ++r)
            if (r < rows) out[r] = skml_hash(ids[r], key, size);
        return;
    }
    uint32_t c[MAXR], seed[MAXR];
    bool any = false;
#ifdef __CUDA_ARCH__
#pragma unroll
#endif
    for (int r = 0; r < MAXR; ++r) {
        const int id = r < rows ? ids[r] : 0;
        seed[r] = id < 3 ? 0u : (id == 3 ? 31u : (id == 4 ? 131u : (id == 5 ? 267u : (id == 6 ? 1313u : 13131u))));
        c[r] = 0;
        any = any || seed[r] != 0;
    }
    if (any) {
        uint32_t k = (uint32_t)key;
        while (k != 0) {
            const uint32_t q = k / 10u;
            const uint32_t d = k - q * 10u;
#ifdef __CUDA_ARCH__
#pragma unroll
#endif
            for (int r = 0; r < MAXR; ++r) c[r] = seed[r] * c[r] + d;
            k = q;
        }
    }
#ifdef __CUDA_ARCH__
#pragma unroll
#endif
    for (int r = 0; r < MAXR; ++r) {
        if (r >= rows) continue;
        const int id = ids[r];
        uint32_t h = c[r];
        if (id == 0) h = skml_mix_bj((uint32_t)key);
        else if (id == 1) h = skml_mix_64((uint32_t)key);
        else if (id == 2) h = skml_mix_tw((uint32_t)key);
        const int32_t sc = (int32_t)h;
        if (sc >= 0) {
            out[r] = (int32_t)skml_fastmod(h, magic, (uint32_t)size);
        } else {  // Java: the remainder keeps the sign of the dividend
            const uint32_t m = skml_fastmod((uint32_t)(-(int64_t)sc), magic, (uint32_t)size);
            out[r] = m ? size - (int32_t)m : 0;
        }
    }
}

// ---------------------------------------------------------------------------
// Counter-based random numbers (splitmix64): every rank derives the same value
// from (seed, step, rank, group, slot) without any shared state.
// ---------------------------------------------------------------------------
SKML_HD uint64_t skml_splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

SKML_HD uint64_t skml_rand(uint64_t seed, uint64_t a, uint64_t b, uint64_t c) {
    uint64_t h = skml_splitmix64(seed ^ 0x5851F42D4C957F2Dull);
    h = skml_splitmix64(h ^ a);
    h = skml_splitmix64(h ^ (b * 0xD6E8FEB86659FD93ull));
    h = skml_splitmix64(h ^ (c * 0xA0761D6478BD642Full));
    return h;
}

// Picks `rows` distinct members of the family of 8, driven by (seed, step, rank, group)
// (HashFactory.getRandomInt2IntHashes draws them from an unseeded java.util.Random instead, so
// every outcome here is one the reference can produce). The three integer mixers (BJ, Mix64, TW)
// are drawn first, in shuffled order, and the five BKDR members only for rows 4..8: a BKDR hash
// walks the key's decimal digits and costs about four times the instructions of a mixer in the
// insert and query kernels, where hashing is the largest single item.
SKML_HD void skml_pick_hashes(uint64_t seed, uint64_t step, uint32_t rank, uint32_t group, int rows,
                              uint8_t out[8]) {
    uint8_t ids[8] = {0, 1, 2, 3, 4, 5, 6, 7};
    for (int i = 2; i > 0; --i) {  // Fisher-Yates over the mixers ids[0..2]
        uint64_t r = skml_rand(seed, step, ((uint64_t)rank << 32) | group, (uint64_t)i);
        int j = (int)(r % (uint64_t)(i + 1));
        uint8_t t = ids[i];
        ids[i] = ids[j];
        ids[j] = t;
    }
    for (int i = 7; i > 3; --i) {  // Fisher-Yates over the BKDR members ids[3..7]
        uint64_t r = skml_rand(seed, step, ((uint64_t)rank << 32) | group, (uint64_t)i);
        int j = 3 + (int)(r % (uint64_t)(i - 2));
        uint8_t t = ids[i];
        ids[i] = ids[j];
        ids[j] = t;
    }
    for (int i = 0; i < 8; ++i) out[i] = i < rows ? ids[i] : 0;
}

// ---------------------------------------------------------------------------
// Bucket groups. edges[g] is the exclusive upper bucket of group g; group g
// covers buckets [edges[g-1], edges[g]) with edges[-1] = 0.
// ---------------------------------------------------------------------------
SKML_HD void skml_group_edges(int zero_idx, int bin_num, int group_num, int* edges) {
    if (group_num == 1) {
        edges[0] = bin_num;
        return;
    }
    if (group_num == 2) {
        edges[0] = zero_idx;
        edges[1] = bin_num;
        return;
    }
    int bpg = bin_num / group_num;
    if (bpg < 1) bpg = 1;  // more groups than buckets: the reference would divide by zero
    int e0;
    if (zero_idx < bpg) e0 = zero_idx;
    else if ((zero_idx % bpg) < (bpg / 2)) e0 = bpg + zero_idx % bpg;
    else e0 = zero_idx % bpg;
    edges[0] = e0;
    for (int i = 1; i < group_num - 1; ++i) {
        int e = edges[i - 1] + bpg;
        edges[i] = e < bin_num ? e : bin_num;
    }
    edges[group_num - 1] = bin_num;
}

SKML_HD int skml_group_of(int bin, const int* edges, int group_num) {
    int g = 0;
    while (g < group_num - 1 && edges[g] <= bin) ++g;
    return g;
}

// Packed working cell of the MinMaxSketch: (distance to the zero bucket << 16) | bucket.
// The unsigned minimum of packed cells is the bucket closest to zero, ties to the
// lower bucket, so the result does not depend on insertion order.
SKML_HD uint32_t skml_pack_cell(int bin, int zero_idx) {
    int d = bin - zero_idx;
    if (d < 0) d = -d;
    return ((uint32_t)d << 16) | (uint32_t)bin;
}

// Width in bytes of one delta in the delta-binary key code: 1, 2 or 4.
SKML_HD int skml_delta_bytes(uint32_t delta) { return delta < 256u ? 1 : (delta < 65536u ? 2 : 4); }

// Byte j (in stream order) of a `w`-byte delta. The stream stores the value most
// significant bit first at increasing java.util.BitSet indices, and BitSet index i is
// bit (i & 63) of word (i >> 6), so each stream byte is a bit-reversed value byte.
SKML_HD uint8_t skml_brev8(uint8_t b) {
#if defined(__CUDA_ARCH__)
    return (uint8_t)(__brev((unsigned int)b) >> 24);
#endif
    b = (uint8_t)(((b & 0xF0u) >> 4) | ((b & 0x0Fu) << 4));
    b = (uint8_t)(((b & 0xCCu) >> 2) | ((b & 0x33u) << 2));
    b = (uint8_t)(((b & 0xAAu) >> 1) | ((b & 0x55u) << 1));
    return b;
}
SKML_HD uint8_t skml_delta_stream_byte(uint32_t delta, int w, int j) {
    return skml_brev8((uint8_t)(delta >> (8 * (w - 1 - j))));
}
