// C ABI of libskml_cuda.so (loaded from Python with ctypes). Every function
// returns a cudaError_t value as int (0 = success) unless stated otherwise and
// launches on the given stream without synchronising.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SKML_MAX_PEERS 16
#define SKML_GPU_MAX_BINS 4096

// Arguments of the fused compress kernels. Only 8-byte fields, so the ctypes mirror
// in sketchml_b200/ops/lib.py cannot disagree about padding.
typedef struct SkmlCompressArgs {
    const int* keys;            // sorted keys (sparse kind)
    const float* vals;          // values: nnz of them (sparse) or dim of them (dense)
    const long long* meta;      // device: meta[0] = nnz, meta[1] = kind (0 empty, 1 sparse, 2 dense)
    long long n_max;            // capacity of keys / vals
    long long dim;
    long long bin_num, group_num, row_num;
    double col_ratio;
    unsigned long long seed, step;
    long long rank, world;
    const double* loss_partials;   // device, 4 doubles, may be null
    unsigned char* payload;        // this rank's slot in its own receive region
    long long slot_capacity;
    unsigned char* peer_payload[SKML_MAX_PEERS];       // this rank's slot in every rank's region (self included)
    unsigned long long* peer_flag[SKML_MAX_PEERS];     // arrival flag of that slot
    unsigned char* workspace;      // skml_compress_workspace_bytes() bytes, zero-filled once by the caller
    long long workspace_bytes;
    unsigned int* status;
    long long budget_cycles;
    const float* given_splits;     // test hook: use these split points instead of the sketch
    long long n_given;
    double given_min, given_max;
    long long fused;               // 1 = one cooperative launch, 0 = one launch per stage
    long long grid;                // 0 = one block per SM
    long long key_encoder;         // 0 = delta_binary (byte-aligned deltas), 1 = delta_adaptive (the reference's live encoder)
    long long cell_bits;           // sketch tables on the wire: -1 = 8/16-bit bucket codes, 0 = Huffman-coded (the reference's form)
    long long quantile_summary;    // 0 = split points from a 4096-value sample that every thread-block cluster
                                   // draws alike (no grid barrier, no query stage), 1 = mergeable k = 128 sketch per block,
                                   // merged per cluster and queried over all runs.
} SkmlCompressArgs;

long long skml_compress_workspace_bytes(long long n_max, long long bin_num, long long group_num, long long row_num,
                                        double col_ratio, long long grid);
long long skml_payload_capacity(long long n_max, long long dim, long long bin_num, long long group_num,
                                long long row_num, double col_ratio);
long long skml_compress_splits_offset(long long n_max, long long bin_num, long long group_num, long long row_num,
                                      double col_ratio, long long grid);
int skml_compress_sparse(const SkmlCompressArgs* args, void* stream);
// Blocks per thread-block cluster of this process's most recent compress launch (2, 1, or 0 before the first).
int skml_compress_cluster_size();
int skml_compress_dense(const SkmlCompressArgs* args, void* stream);

// Arguments of the fused decode + aggregate + update kernel.
typedef struct SkmlDecodeArgs {
    const unsigned char* payload[SKML_MAX_PEERS];     // the slots of this rank's receive region
    const unsigned long long* flag[SKML_MAX_PEERS];   // their arrival flags (null = do not wait)
    long long world;
    long long slot_capacity;
    unsigned long long step;
    long long dim;
    float* w;
    float* adam_m;
    float* adam_v;             // null for SGD
    double lr, adam_scale;     // Adam: scale = sqrt(1 - beta2^t) / (1 - beta1^t)
    long long* acc;            // dim fixed-point accumulators, all zero between calls
    int* key_scratch;          // decoded keys, capacity key_capacity
    long long key_capacity;
    double* loss_out;          // device, 4 doubles: sum over ranks of the payloads' loss partials
    float* out_sum;            // optional dense fp32 [dim]: receives the averaged decoded sum instead of updating w
    unsigned char* workspace;  // skml_decode_workspace_bytes()
    unsigned int* status;
    long long budget_cycles;
    long long fused;
    long long grid;
    long long max_groups;      // upper bound of the payloads' group count (0 = 32): sizes the work table
    float* val_scratch;        // decoded values, capacity key_capacity (null: SGD applies payload by payload)
    unsigned char* table_scratch;  // room for the sketch tables of payloads that carry them Huffman-coded (null: refused)
    long long table_capacity;      // its size in bytes
    double* weight_sumsq;          // optional device double: sum of w^2, kept current by the update (see skml_weight_norm)
    double* reg_out;               // optional device double: receives reg_lambda * sqrt(*weight_sumsq) when the launch ends
    double reg_lambda;
    long long adam_stride;         // 0 / 1: adam_m and adam_v are plain arrays; 4: both point into one array of
                                   // {m, v, sum, unused} quads (adam_v = adam_m + 1), whose third word the kernel
                                   // uses for the per-coordinate sums of lazy Adam (zero between calls)
} SkmlDecodeArgs;

long long skml_decode_workspace_bytes(long long world, long long group_num);
int skml_decode_update(const SkmlDecodeArgs* args, void* stream);

// GLM numerics
int skml_glm_grad(const long long* rowptr, const int* cols, const float* vals, const float* labels, long long row_lo,
                  long long row_cnt, long long nnz_padded, double avg_nnz, const float* w, float* g,
                  unsigned int* bitmap, int loss_id, float inv_batch, int hot, double* loss_acc, unsigned int* status,
                  long long budget, void* stream);
int skml_glm_validate(const long long* rowptr, const int* cols, const float* vals, const float* labels,
                      long long row_lo, long long row_cnt, long long nnz_padded, double avg_nnz, const float* w,
                      int loss_id, double* acc5, float* margins, unsigned int* status, long long budget, void* stream);
int skml_compact(float* g, const float* w, unsigned int* bitmap, int dim, float lambda, unsigned int* block_counts,
                 long long* meta, int* keys, float* vals, float* dense_vals, long long capacity, unsigned int* status,
                 void* stream);
long long skml_compact_blocks(int dim);
// The update entry points take `adam_stride`: elements between the moments of neighbouring coordinates (1: plain
// arrays, 4: packed quads, see SkmlDecodeArgs).
int skml_update_dense(float* w, float* m, float* v, const float* g, long long dim, float scale, int adam, float lr,
                      float adam_scale, int sparse_only, int adam_stride, void* stream);
int skml_update_sparse(float* w, float* m, float* v, const int* keys, const float* vals, const long long* n_ptr,
                       long long n_max, float scale, int adam, float lr, float adam_scale, int adam_stride, void* stream);
// Applies acc[key] * scale to the model on the coordinates of `lists` gathered key lists (list l at
// keys + l * stride, counts[l] entries) and clears those accumulator words.
int skml_update_gathered(float* w, float* m, float* v, float* acc, const int* keys, const long long* counts,
                         long long stride, int lists, float scale, int adam, float lr, float adam_scale, int adam_stride,
                         void* stream);
// sumsq_out[0] = sum of w^2 (double, fixed summation order), reg_out[0] = lambda * sqrt of it; one
// launch, `scratch` holds skml_weight_norm_scratch_bytes() bytes that are zero before the first call.
long long skml_weight_norm_scratch_bytes();
int skml_weight_norm(const float* w, long long dim, double lambda, double* sumsq_out, double* reg_out, void* scratch,
                     void* stream);
// Column sums over the row-tiled transposed index (see SkmlStepArgs.tt_*): out[c] = sum over the batch entries of
// column c of coef[row] * value + lambda * w[ucols[c]], bit-reproducible. `partial`: scratch of one float per pair.
int skml_colsum_tiled(const int* tile_pair_ptr, const int* pair_ptr, const unsigned short* lrow, const float* svals,
                      const int* pair_dst, const int* col_pair_ptr, const int* ucols, int rows, int tile_rows, int n_tiles,
                      int n_cols, const float* coef, const float* w, float lambda, float* partial, float* out, void* stream);
int skml_scatter_kv(float* acc, const int* keys, const float* vals, const long long* counts, long long stride,
                    int lists, void* stream);
int skml_gen_wstar(float* w, long long dim, double density, unsigned long long seed, void* stream);
int skml_gen_rows(int* cols, float* vals, float* labels, long long row_offset, long long rows, int dim, int k,
                  double s, int value_kind, int task, float noise, const float* wstar, unsigned long long seed,
                  void* stream);
int skml_glm_coef(const long long* rowptr, const int* cols, const float* vals, const float* labels, long long row_lo,
                  long long row_cnt, long long nnz_padded, double avg_nnz, const float* w, int loss_id,
                  float inv_batch, double* loss_acc, float* coef_out, unsigned int* status, long long budget,
                  void* stream);
int skml_colsum(const int* colptr, const int* rowidx, const float* svals, const int* ucols, const int* bins,
                const int* long_col, const int* long_e0, const int* long_e1, int n_short, int n_medium, int n_long,
                int n_cols, const float* coef, const float* w, float lambda, float* out, void* stream);
int skml_colsum_ex(const int* colptr, const int* rowidx, const float* svals, const int* ucols, const int* bins,
                   const int* long_col, const int* long_e0, const int* long_e1, int n_short, int n_medium, int n_long,
                   int n_cols, const float* coef, const float* w, float lambda, float* out, int out_is_prepared,
                   void* stream);
int skml_step_prep(double* partials, const double* partials_template, float* out, const int* long_col, int n_long,
                   void* stream);
int skml_gather_compact(const float* w, const int* ucols, int n, float* wc, void* stream);
int skml_finalize_compact(float* gc, const float* wc, float lambda, int n, float* vals, unsigned int* bitmap,
                          void* stream);
int skml_sm_count();

// DeltaAdaptive key encoder, stand-alone (csrc/cuda/keys_kernels.cu). The caller computes the
// inclusive prefix sums of the width arrays between the calls. Word buffers are 32-bit views of
// the 64-bit BitSet words, zero-filled by the caller, with one spare word at the end.
int skml_da_analyze(const int* keys, long long n, unsigned int* hist32, unsigned int* params, unsigned int* status,
                    void* stream);   // params[0] = interval count, params[1] = 1 for unary flags; status bit 0 = unsorted keys
int skml_da_widths(const int* keys, long long n, const unsigned int* params, int* flag_w, int* delta_w, void* stream);
int skml_da_pack(const int* keys, long long n, const unsigned int* params, const long long* flag_incl,
                 const long long* delta_incl, unsigned int* flag_words, unsigned int* delta_words, void* stream);
int skml_da_fixed_iv(const unsigned int* flag_words, long long n, int flag_bits_per_key, int* iv, void* stream);
int skml_da_zero_count(const unsigned int* flag_words, long long flag_bits, int* zeros, void* stream);
int skml_da_zero_pos(const unsigned int* flag_words, long long flag_bits, const long long* zeros_incl, long long n,
                     long long* pos, void* stream);
int skml_da_extract(const unsigned int* delta_words, long long n, const int* delta_w, const long long* delta_incl,
                    long long* deltas, void* stream);

// Expands a minibatch from its transport form (bit-packed column indices, 32-bit row pointers,
// 8-bit labels; the latter two optional = null) into CSR arrays. `packed` must end with two
// padding words.
int skml_unpack_batch(const unsigned int* packed, int bits, long long nnz, int* cols, const int* rowptr32,
                      long long rows, long long* rowptr, const signed char* labels8, float* labels, void* stream);
// The same for column indices in the byte-aligned variable-width form (1..4 bytes each, 2 flag bits,
// one byte offset per 1024 values).
int skml_row_prefix(const long long* rowptr, long long rows, int* cols, void* stream);
int skml_unpack_batch_varnibbles(const unsigned int* flags, const unsigned int* block_offsets, const unsigned int* words,
                                 long long nnz, int* cols, const int* rowptr32, long long rows, long long* rowptr,
                                 const signed char* labels8, float* labels, void* stream);
int skml_unpack_batch_varbytes(const unsigned int* flags, const unsigned int* block_offsets, const unsigned char* bytes,
                               long long nnz, int* cols, const int* rowptr32, long long rows, long long* rowptr,
                               const signed char* labels8, float* labels, void* stream);

// FixedPoint baseline compressor: b-bit sign + magnitude codes (2 <= bits < 30), 8 values per
// `bits` bytes, most significant bit first in java.util.BitSet order. `scratch` holds
// skml_fixedpoint_scratch_bytes() bytes; `norm_out` receives the L2 norm the codes are relative to.
long long skml_fixedpoint_scratch_bytes();
long long skml_fixedpoint_code_bytes(long long n, int bits);
int skml_fixedpoint_pack(const float* vals, const long long* n_ptr, long long n_max, int bits,
                         unsigned long long seed, double* scratch, unsigned char* codes, double* norm_out,
                         void* stream);
// Decodes `lists` code streams (list l at codes + l * code_stride, keys + l * key_stride, counts[l]
// entries, norms[l]); adds the values into acc[key] when acc is given and stores them to
// vals_out[l * key_stride + i] when vals_out is given.
int skml_fixedpoint_unpack_scatter(float* acc, const int* keys, const unsigned char* codes, const double* norms,
                                   const long long* counts, long long key_stride, long long code_stride, int lists,
                                   int bits, float* vals_out, void* stream);

// Zip baseline compressor: ZipML split search on the device (no value is read back to the host), one
// bucket code per value (skml_zipml_code_bytes(bin_num) bytes each) and a table of
// skml_zipml_table_len(bin_num) bucket midpoints per list. `scratch`: skml_zipml_scratch_bytes(n_max)
// bytes; meta: buckets, zero bucket, halving rounds; range: min, max. 2 <= bin_num <= 8190.
long long skml_zipml_scratch_bytes(long long n_max);
int skml_zipml_code_bytes(int bin_num);
int skml_zipml_table_len(int bin_num);
int skml_zipml_pack(const float* vals, const long long* n_ptr, long long n_max, int bin_num, void* scratch,
                    long long scratch_bytes, float* splits, float* mids, int* meta, float* range, unsigned char* codes,
                    void* stream);
// Decodes `lists` code arrays (list l at codes + l * code_stride, keys + l * key_stride, its table at
// mids + l * table_len, counts[l] entries); adds into acc[key] when acc is given, stores the values to
// vals_out[l * key_stride + i] when vals_out is given (keys may then be null).
int skml_zipml_unpack_scatter(float* acc, const int* keys, const unsigned char* codes, const float* mids,
                              const long long* counts, long long key_stride, long long code_stride, int lists,
                              int bin_num, float* vals_out, void* stream);

// Peer memory (one process per GPU): CUDA IPC handles of a cudaMalloc'ed region.
int skml_ipc_get_handle(void* dev_ptr, unsigned char* handle64);
int skml_ipc_open_handle(const unsigned char* handle64, void** dev_ptr);
int skml_ipc_close(void* dev_ptr);
// A zeroed cudaMalloc allocation of its own for a receive region, and its release.
int skml_region_alloc(long long bytes, void** dev_ptr);
int skml_region_free(void* dev_ptr);
int skml_enable_peer_access(int peer_device);

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
// One training step (gradient -> compaction -> fused compress -> fused decode + update) as a
// single call, so that the host spends one library call per step instead of five.
typedef struct SkmlStepArgs {
    const long long* rowptr;
    const int* cols;
    const float* vals;
    const float* labels;
    long long seg_lo[2], seg_cnt[2];   // up to two row ranges (a batch that wraps around the shard)
    long long nnz_padded;
    double avg_nnz;
    float* w;
    float* g;
    unsigned int* bitmap;
    long long loss_id;
    double inv_batch;
    long long hot;
    double* partials;                  // device, 4 doubles: batch size, loss sum, reg loss, spare
    const double* partials_template;   // device, copied into `partials` before the gradient kernel
    unsigned int* status;
    long long budget_cycles;
    double lambda;
    unsigned int* block_counts;
    long long* meta;
    int* keys;
    float* gvals;
    float* dense_vals;                 // null unless the dense kind is reachable
    long long n_max;
    long long dim;
    SkmlCompressArgs* compress;        // prepared for this step's parity; step is filled in here
    SkmlDecodeArgs* decode;
    unsigned long long step;
    double lr, adam_scale;
    double* loss_out;                  // device, 4 doubles: this step's slot of the loss ring
    // transposed-index gradient (all null / 0 = scatter + compaction path)
    const int* t_colptr;               // [t_cols + 1] entry ranges of the batch's distinct columns
    const int* t_rowidx;               // batch-local row of every entry, column-major
    const float* t_vals;               // values in the same order (null = all ones)
    const int* t_ucols;                // the distinct columns, ascending: the gradient's keys
    const int* t_bins;                 // positions of short then medium columns
    const int* t_long_col;
    const int* t_long_e0;
    const int* t_long_e1;
    long long t_short, t_medium, t_long, t_cols;
    const long long* t_meta;           // device: {t_cols, 1 (sparse kind), 0, 0}
    float* coef;                       // device scratch: one coefficient per batch row
    // local-id batch (null = not one): `cols` holds positions in l_ucols instead of feature indices
    const int* l_ucols;                // the batch's distinct columns, ascending: the gradient's keys
    const long long* l_meta;           // device: {l_ncols, 1 (sparse kind), 0, 0}
    long long l_ncols;
    float* wc;                         // device scratch [>= l_ncols]: weights of the batch's columns
    float* gc;                         // device scratch [>= l_ncols], all zero between steps: compact gradient
    void* grad_done_event;             // optional cudaEvent_t, recorded after the last kernel that reads the batch
    // row-tiled form of the transposed index (tt_pair_ptr null = the per-column form above); t_vals, t_ucols,
    // t_cols, t_meta and coef are shared with it, t_vals being in (tile, column, row) order
    const int* tt_tile_pair_ptr;       // [tt_tiles + 1] pair ranges of the row tiles
    const int* tt_pair_ptr;            // [pairs + 1] entry ranges of the (tile, column) pairs
    const unsigned short* tt_lrow;     // tile-local row of every entry
    const int* tt_pair_dst;            // [pairs] position of a pair's partial sum in (column, tile) order
    const int* tt_col_pair_ptr;        // [t_cols + 1] partial-sum ranges of the columns
    float* tt_partial;                 // device scratch [>= pairs]
    long long tt_tiles, tt_tile_rows, tt_rows;
} SkmlStepArgs;

int skml_train_step(SkmlStepArgs* args, void* stream);
#ifdef __cplusplus
}
#endif
