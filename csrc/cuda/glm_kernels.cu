// Sparse generalized-linear-model numerics for sm_100a:
//   * skml_glm_grad      : per-row margin, loss and coefficient, fused with the scatter of
//                          coefficient * feature into the dense gradient accumulator
//                          (row tiles staged into shared memory by 1-D bulk TMA copies,
//                          one warp per row, shuffle reductions, hot columns kept in
//                          shared memory, touched-coordinate bitmap)
//   * skml_compact_*     : touched bitmap -> sorted (key, value) list with L2 term and
//                          the |v| > 1e-8 filter; decides sparse vs dense kind
//   * skml_glm_validate  : margin, loss and confusion counts over a validation shard
//   * skml_update_*      : SGD / lazy-Adam updates used by the uncompressed baselines
//
// Reference behaviour restated (paths inside the reference project, module `ml`):
//   objective/GradientDescent.scala:23-51,70-87 (minibatch gradient, 1/batch, L2 on the
//   gradient's own coordinates), objective/Loss.scala:82-137 (log / hinge / square loss and
//   their negative derivatives, +-18 cut-offs), gradient/DenseDoubleGradient.scala:51-95
//   (scatter-add, countNNZ with |v| > 1e-8, toSparse, dense iff nnz > 2/3 dim),
//   util/ValidationUtil.scala:12-41, objective/Adam.scala:27-77,
//   objective/GradientDescent.scala:89-132.
#include <math.h>

#include "skml_api.h"
#include "skml_device.cuh"

#define GRAD_THREADS 512
#define GRAD_WARPS (GRAD_THREADS / 32)
#define GRAD_TILE_CAP 4096  // elements of one staged tile (cols and values each)
#define SKML_EPS 1e-8f
#define GRAD_MAX_RPT 256   // rows of one tile at most
#define GRAD_RPI 4         // rows per warp and iteration
#define GRAD_PRIV 256      // hottest columns kept once per warp

__device__ __forceinline__ float glm_loss(int loss_id, float pre, float y) {
    if (loss_id == 0) {
        float z = pre * y;
        if (z > 18.f) return __expf(-z);
        if (z < -18.f) return -z;
        return log1pf(__expf(-z));
    } else if (loss_id == 1) {
        float z = pre * y;
        return z < 1.f ? 1.f - z : 0.f;
    }
    float d = pre - y;
    return 0.5f * d * d;
}

// negative derivative of the loss with respect to the prediction
__device__ __forceinline__ float glm_grad(int loss_id, float pre, float y) {
    if (loss_id == 0) {
        float z = pre * y;
        if (z > 18.f) return y * __expf(-z);
        if (z < -18.f) return y;
        return y / (1.f + __expf(z));
    } else if (loss_id == 1) {
        return pre * y <= 1.f ? y : 0.f;
    }
    return y - pre;
}

__device__ __forceinline__ void red_add_f32(float* p, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

__device__ __forceinline__ void red_or_u32(unsigned int* p, unsigned int v) {
    asm volatile("red.global.or.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct GradSmem {
    uint64_t bar[2];
};

// MODE 0: training (scatter), MODE 1: validation (loss + confusion counts only),
// MODE 2: per-row coefficients only (the scatter is done by the transposed-index kernels)
template <int MODE>
__global__ void __launch_bounds__(GRAD_THREADS)
glm_rows_kernel(const long long* __restrict__ rowptr, const int* __restrict__ cols, const float* __restrict__ vals,
                const float* __restrict__ labels, long long row_lo, long long row_cnt, int rows_per_tile,
                long long nnz_padded, const float* __restrict__ w, float* __restrict__ g,
                unsigned int* __restrict__ bitmap, int loss_id, float inv_batch, int hot, double* __restrict__ acc,
                float* __restrict__ margins, unsigned int* status, long long budget) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // layout: [2 stages x cols][2 stages x vals, only if the shard stores values][hot floats]
    __shared__ GradSmem sb;
    __shared__ long long s_rp[GRAD_MAX_RPT + 1];
    __shared__ float s_lab[GRAD_MAX_RPT];
    int* s_cols = reinterpret_cast<int*>(smem_raw);
    float* s_vals = reinterpret_cast<float*>(smem_raw + 2 * GRAD_TILE_CAP * sizeof(int));
    const bool has_vals = vals != nullptr;
    float* s_hot = reinterpret_cast<float*>(smem_raw + (has_vals ? 4 : 2) * GRAD_TILE_CAP * sizeof(int));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int priv = hot < GRAD_PRIV ? hot : GRAD_PRIV;  // columns [0, priv): per-warp private sums
    float* s_priv = s_hot + hot;

    if (MODE == 0) {
        for (int i = threadIdx.x; i < hot; i += blockDim.x) s_hot[i] = 0.f;
        for (int i = threadIdx.x; i < priv * GRAD_WARPS; i += blockDim.x) s_priv[i] = 0.f;
    }
    if (threadIdx.x == 0) {
        mbar_init(&sb.bar[0], 1);
        mbar_init(&sb.bar[1], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const long long ntiles = (row_cnt + rows_per_tile - 1) / rows_per_tile;
    double loss_sum = 0.0;
    unsigned int tp = 0, tn = 0, fp = 0, fn = 0;
    unsigned int phase[2] = {0, 0};

    // Issues the bulk copies of one tile into `stage`; returns false when the tile does
    // not fit the staging buffer (it is then read with plain loads).
    auto tile_span = [&](long long tile, long long& a0, long long& a1) -> bool {
        long long r0 = row_lo + tile * rows_per_tile;
        long long r1 = r0 + rows_per_tile;
        if (r1 > row_lo + row_cnt) r1 = row_lo + row_cnt;
        long long e0 = rowptr[r0], e1 = rowptr[r1];
        a0 = e0 & ~3ll;
        a1 = (e1 + 3ll) & ~3ll;
        if (a1 > nnz_padded) a1 = nnz_padded;
        return (a1 - a0) <= GRAD_TILE_CAP && a1 > a0;
    };
    auto issue = [&](long long tile, int stage) {
        long long a0, a1;
        if (!tile_span(tile, a0, a1)) return;
        unsigned int bytes = (unsigned int)(a1 - a0) * 4u;
        mbar_expect_tx(&sb.bar[stage], has_vals ? 2 * bytes : bytes);
        bulk_g2s(s_cols + stage * GRAD_TILE_CAP, cols + a0, bytes, &sb.bar[stage]);
        if (has_vals) bulk_g2s(s_vals + stage * GRAD_TILE_CAP, vals + a0, bytes, &sb.bar[stage]);
    };

    long long tile = blockIdx.x;
    if (tile < ntiles && threadIdx.x == 0) issue(tile, 0);
    int stage = 0;
    for (; tile < ntiles; tile += gridDim.x, stage ^= 1) {
        long long next = tile + gridDim.x;
        if (next < ntiles && threadIdx.x == 0) issue(next, stage ^ 1);
        long long a0, a1;
        bool staged = tile_span(tile, a0, a1);
        if (staged) {
            if (!mbar_wait(&sb.bar[stage], phase[stage], budget)) {
                staged = false;  // never expected; read from global memory instead
                if (threadIdx.x == 0) skml_set_status(status, SKML_TIMEOUT_BARRIER, 0x10u);
            }
            phase[stage] ^= 1;
        }
        const int* cp = staged ? (s_cols + stage * GRAD_TILE_CAP) - a0 : cols;
        const float* vp = has_vals ? (staged ? (s_vals + stage * GRAD_TILE_CAP) - a0 : vals) : nullptr;
        long long r0 = row_lo + tile * rows_per_tile;
        long long r1 = r0 + rows_per_tile;
        if (r1 > row_lo + row_cnt) r1 = row_lo + row_cnt;
        const int nrows = (int)(r1 - r0);
        for (int t = threadIdx.x; t <= nrows; t += blockDim.x) s_rp[t] = rowptr[r0 + t];
        for (int t = threadIdx.x; t < nrows; t += blockDim.x) s_lab[t] = labels[r0 + t];
        __syncthreads();
        // GRAD_RPI rows per warp and iteration. All loads of one 32-element slice of the
        // GRAD_RPI rows are issued before any of them is consumed, so their L2 round trips overlap.
        for (int rb = warp * GRAD_RPI; rb < nrows; rb += GRAD_WARPS * GRAD_RPI) {
            long long e0[GRAD_RPI];
            int len[GRAD_RPI];
            float sum[GRAD_RPI];
            int maxlen = 0;
#pragma unroll
            for (int u = 0; u < GRAD_RPI; ++u) {
                const int rr = rb + u < nrows ? rb + u : nrows - 1;
                e0[u] = s_rp[rr];
                len[u] = rb + u < nrows ? (int)(s_rp[rr + 1] - e0[u]) : 0;
                maxlen = max(maxlen, len[u]);
                sum[u] = 0.f;
            }
            for (int off = lane; off < maxlen + lane; off += 32) {
                if (off - lane >= maxlen) break;
                int c[GRAD_RPI];
                float wv[GRAD_RPI], xv[GRAD_RPI];
#pragma unroll
                for (int u = 0; u < GRAD_RPI; ++u) {
                    const bool ok = off < len[u];
                    c[u] = ok ? cp[e0[u] + off] : -1;
                    xv[u] = (ok && vp) ? vp[e0[u] + off] : 1.f;
                }
#pragma unroll
                for (int u = 0; u < GRAD_RPI; ++u) wv[u] = c[u] >= 0 ? __ldg(w + c[u]) : 0.f;
#pragma unroll
                for (int u = 0; u < GRAD_RPI; ++u) sum[u] = fmaf(wv[u], xv[u], sum[u]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < GRAD_RPI; ++u) sum[u] += __shfl_xor_sync(0xFFFFFFFFu, sum[u], o);
            }
            // Loss and coefficient of the GRAD_RPI rows are evaluated once, by lanes 0..GRAD_RPI-1 in
            // parallel (lane u owns row rb + u); the scatter mode then broadcasts the coefficients.
            float pre_mine = sum[0];
#pragma unroll
            for (int u = 1; u < GRAD_RPI; ++u) pre_mine = lane == u ? sum[u] : pre_mine;
            float coef_mine = 0.f;
            if (lane < GRAD_RPI && rb + lane < nrows) {
                const float y = s_lab[rb + lane];
                loss_sum += (double)glm_loss(loss_id, pre_mine, y);
                if (MODE == 0 || MODE == 2) {
                    coef_mine = -glm_grad(loss_id, pre_mine, y) * inv_batch;
                    if (MODE == 2) margins[r0 - row_lo + rb + lane] = coef_mine;  // coefficient per row, no scatter
                } else {
                    const float z = pre_mine * y;
                    if (z > 0.f) {
                        if (pre_mine > 0.f) ++tp; else ++tn;
                    } else if (z < 0.f) {
                        if (pre_mine > 0.f) ++fp; else ++fn;
                    }
                    if (margins) margins[r0 - row_lo + rb + lane] = pre_mine;
                }
            }
            float coef[GRAD_RPI];
#pragma unroll
            for (int u = 0; u < GRAD_RPI; ++u) coef[u] = MODE == 0 ? __shfl_sync(0xFFFFFFFFu, coef_mine, u) : 0.f;
            if (MODE == 0) {
                for (int off = lane; off - lane < maxlen; off += 32) {
                    int c[GRAD_RPI];
                    float contrib[GRAD_RPI];
                    unsigned int seen[GRAD_RPI];
#pragma unroll
                    for (int u = 0; u < GRAD_RPI; ++u) {
                        const bool ok = off < len[u] && coef[u] != 0.f;
                        c[u] = ok ? cp[e0[u] + off] : -1;
                        contrib[u] = ok ? coef[u] * (vp ? vp[e0[u] + off] : 1.f) : 0.f;
                    }
                    // cold columns: read the bitmap words first (independent L2 loads), so that
                    // the atomicOr is only issued for bits that are not set yet
#pragma unroll
                    for (int u = 0; u < GRAD_RPI; ++u)
                        seen[u] = (bitmap && c[u] >= hot) ? *(volatile unsigned int*)(bitmap + (c[u] >> 5)) : ~0u;  // no bitmap: nothing to mark
#pragma unroll
                    for (int u = 0; u < GRAD_RPI; ++u) {
                        if (c[u] < 0) continue;
                        if (c[u] < priv) {
                            // the hottest columns: one private copy per warp. The lanes of a row hold
                            // distinct columns and a warp's shared-memory accesses are ordered, so a
                            // plain read-modify-write is exact and free of atomics.
                            s_priv[warp * priv + c[u]] += contrib[u];
                        } else if (c[u] < hot) {
                            atomicAdd(&s_hot[c[u]], contrib[u]);
                        } else {
                            red_add_f32(g + c[u], contrib[u]);
                            const unsigned int bit = 1u << (c[u] & 31);
                            if (!(seen[u] & bit)) atomicOr(bitmap + (c[u] >> 5), bit);
                        }
                    }
                    __syncwarp();
                }
            }
        }
        __syncthreads();  // everyone is done with `stage` (and s_rp / s_lab) before it is refilled
    }

    if (MODE == 0) {
        for (int i = threadIdx.x; i < priv; i += blockDim.x) {
            float t = s_hot[i];
            for (int w2 = 0; w2 < GRAD_WARPS; ++w2) t += s_priv[w2 * priv + i];
            s_hot[i] = t;
        }
        __syncthreads();
        // flush the hot columns: one red.add per non-zero entry, one atomicOr per 32 columns
        for (int base = warp * 32; base < hot; base += GRAD_WARPS * 32) {
            int i = base + lane;
            float v = i < hot ? s_hot[i] : 0.f;
            unsigned int m = __ballot_sync(0xFFFFFFFFu, v != 0.f);
            if (v != 0.f) red_add_f32(g + i, v);
            if (bitmap && lane == 0 && m) atomicOr(bitmap + (base >> 5), m);
        }
    }
    double tot = block_sum_double(loss_sum);
    if (threadIdx.x == 0 && tot != 0.0) atomicAdd(&acc[0], tot);
    if (MODE == 1) {
        double c0 = block_sum_double((double)tp), c1 = block_sum_double((double)tn);
        double c2 = block_sum_double((double)fp), c3 = block_sum_double((double)fn);
        if (threadIdx.x == 0) {
            if (c0 != 0.0) atomicAdd(&acc[1], c0);
            if (c1 != 0.0) atomicAdd(&acc[2], c1);
            if (c2 != 0.0) atomicAdd(&acc[3], c2);
            if (c3 != 0.0) atomicAdd(&acc[4], c3);
        }
    }
}

static int g_sm_count = 0;
static int sm_count() {
    if (g_sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

static int grad_launch(int mode, const long long* rowptr, const int* cols, const float* vals, const float* labels,
                       long long row_lo, long long row_cnt, long long nnz_padded, double avg_nnz, const float* w,
                       float* g, unsigned int* bitmap, int loss_id, float inv_batch, int hot, double* acc,
                       float* margins, unsigned int* status, long long budget, cudaStream_t stream) {
    if (row_cnt <= 0) return 0;
    if (hot < 0) hot = 0;
    if (hot > 16384) hot = 16384;
    hot &= ~31;
    if (mode != 0) hot = 0;
    int rpt = (int)(GRAD_TILE_CAP * 0.8 / (avg_nnz > 1.0 ? avg_nnz : 1.0));
    if (rpt < 1) rpt = 1;
    if (rpt > GRAD_MAX_RPT) rpt = GRAD_MAX_RPT;
    long long ntiles = (row_cnt + rpt - 1) / rpt;
    size_t smem = (vals ? 4 : 2) * GRAD_TILE_CAP * sizeof(int) + (size_t)hot * sizeof(float) +
                  (size_t)(hot < GRAD_PRIV ? hot : GRAD_PRIV) * GRAD_WARPS * sizeof(float);
    int per_sm = smem > 100 * 1024 ? 1 : (smem > 70 * 1024 ? 2 : 3);
    long long grid = (long long)sm_count() * per_sm;
    if (grid > ntiles) grid = ntiles;
    static bool attr_set[2] = {false, false};
    if (!attr_set[0]) {
        cudaFuncSetAttribute(glm_rows_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(glm_rows_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(glm_rows_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_set[0] = attr_set[1] = true;
    }
    if (mode == 0)
        glm_rows_kernel<0><<<(unsigned)grid, GRAD_THREADS, smem, stream>>>(
            rowptr, cols, vals, labels, row_lo, row_cnt, rpt, nnz_padded, w, g, bitmap, loss_id, inv_batch, hot, acc,
            margins, status, budget);
    else if (mode == 1)
        glm_rows_kernel<1><<<(unsigned)grid, GRAD_THREADS, smem, stream>>>(
            rowptr, cols, vals, labels, row_lo, row_cnt, rpt, nnz_padded, w, g, bitmap, loss_id, inv_batch, hot, acc,
            margins, status, budget);
    else
        glm_rows_kernel<2><<<(unsigned)grid, GRAD_THREADS, smem, stream>>>(
            rowptr, cols, vals, labels, row_lo, row_cnt, rpt, nnz_padded, w, g, bitmap, loss_id, inv_batch, hot, acc,
            margins, status, budget);
    return (int)cudaGetLastError();
}

extern "C" int skml_glm_grad(const long long* rowptr, const int* cols, const float* vals, const float* labels,
                             long long row_lo, long long row_cnt, long long nnz_padded, double avg_nnz,
                             const float* w, float* g, unsigned int* bitmap, int loss_id, float inv_batch, int hot,
                             double* loss_acc, unsigned int* status, long long budget, void* stream) {
    return grad_launch(0, rowptr, cols, vals, labels, row_lo, row_cnt, nnz_padded, avg_nnz, w, g, bitmap, loss_id,
                       inv_batch, hot, loss_acc, nullptr, status, budget, (cudaStream_t)stream);
}

extern "C" int skml_glm_validate(const long long* rowptr, const int* cols, const float* vals, const float* labels,
                                 long long row_lo, long long row_cnt, long long nnz_padded, double avg_nnz,
                                 const float* w, int loss_id, double* acc5, float* margins, unsigned int* status,
                                 long long budget, void* stream) {
    return grad_launch(1, rowptr, cols, vals, labels, row_lo, row_cnt, nnz_padded, avg_nnz, w, nullptr, nullptr,
                       loss_id, 1.f, 0, acc5, margins, status, budget, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// Compaction of the touched bitmap into a sorted sparse gradient.
// Each block owns COMPACT_WORDS consecutive bitmap words (each warp 4 groups of 32 words).
// meta[0] = nnz, meta[1] = kind (1 sparse, 2 dense, 0 empty), meta[2] = touched before filter
// ---------------------------------------------------------------------------
#define COMPACT_WPT 4
#define COMPACT_WORDS (SKML_BLOCK * COMPACT_WPT)
#define COMPACT_SPARSE_BITS 4  // words with at most this many bits are walked by one lane
#define COMPACT_DENSE_BATCH 8  // dense words whose loads are in flight together

__global__ void __launch_bounds__(SKML_BLOCK)
compact_count_kernel(float* __restrict__ g, const float* __restrict__ w, unsigned int* __restrict__ bitmap,
                     long long nwords, int dim, float lambda, unsigned int* __restrict__ block_counts) {
    // A warp owns COMPACT_WPT groups of 32 consecutive bitmap words. Words with few bits are
    // walked by their own lane; words with many bits are walked by the whole warp, one bit
    // per lane, so that the g / w accesses of dense regions are coalesced. Loads are issued in
    // batches before any of them is consumed (several memory round trips in flight per warp).
    // The filtered value g + lambda * w is stored back into g so that the write pass reads one
    // array only.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long wbase = (long long)blockIdx.x * COMPACT_WORDS + (long long)warp * (32 * COMPACT_WPT);
    unsigned int bitsv[COMPACT_WPT];
#pragma unroll
    for (int grp = 0; grp < COMPACT_WPT; ++grp) {
        const long long wi = wbase + grp * 32 + lane;
        bitsv[grp] = wi < nwords ? bitmap[wi] : 0u;
    }
    unsigned int cnt = 0;
#pragma unroll
    for (int grp = 0; grp < COMPACT_WPT; ++grp) {
        const long long gbase = wbase + grp * 32;
        const long long wi = gbase + lane;
        const unsigned int bits = bitsv[grp];
        unsigned int keep = bits;
        const int pc = __popc(bits);
        if (pc > 0 && pc <= COMPACT_SPARSE_BITS) {
            int tpos[COMPACT_SPARSE_BITS];
            bool inb[COMPACT_SPARSE_BITS];
            float gv[COMPACT_SPARSE_BITS], wv[COMPACT_SPARSE_BITS];
            unsigned int b = bits;
#pragma unroll
            for (int j = 0; j < COMPACT_SPARSE_BITS; ++j) {
                tpos[j] = b ? __ffs(b) - 1 : -1;
                b &= b - 1;
                const long long k = wi * 32 + (tpos[j] < 0 ? 0 : tpos[j]);
                inb[j] = tpos[j] >= 0 && k < dim;
                gv[j] = inb[j] ? g[k] : 0.f;
                wv[j] = inb[j] ? w[k] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < COMPACT_SPARSE_BITS; ++j) {
                if (tpos[j] < 0) continue;
                if (!inb[j]) {  // a bit beyond dim (never set by the gradient kernel): drop it
                    keep &= ~(1u << tpos[j]);
                    continue;
                }
                const long long k = wi * 32 + tpos[j];
                const float v = gv[j] + lambda * wv[j];
                if (fabsf(v) > SKML_EPS) {
                    g[k] = v;
                } else {
                    keep &= ~(1u << tpos[j]);
                    g[k] = 0.f;
                }
            }
        }
        unsigned int dense = __ballot_sync(0xFFFFFFFFu, pc > COMPACT_SPARSE_BITS);
        while (dense) {
            int jj[COMPACT_DENSE_BATCH];
            unsigned int wb[COMPACT_DENSE_BATCH];
            float gv[COMPACT_DENSE_BATCH], wv[COMPACT_DENSE_BATCH];
#pragma unroll
            for (int u = 0; u < COMPACT_DENSE_BATCH; ++u) {
                jj[u] = dense ? __ffs(dense) - 1 : -1;
                dense &= dense - 1;
                wb[u] = __shfl_sync(0xFFFFFFFFu, bits, jj[u] < 0 ? 0 : jj[u]);
                const long long k = (gbase + (jj[u] < 0 ? 0 : jj[u])) * 32 + lane;
                const bool active = jj[u] >= 0 && ((wb[u] >> lane) & 1u) && k < dim;
                gv[u] = active ? g[k] : 0.f;
                wv[u] = active ? w[k] : 0.f;
                if (!active) wb[u] &= ~(1u << lane);
            }
#pragma unroll
            for (int u = 0; u < COMPACT_DENSE_BATCH; ++u) {
                if (jj[u] < 0) continue;  // uniform over the warp
                const bool active = (wb[u] >> lane) & 1u;
                bool ok = false;
                if (active) {
                    const long long k = (gbase + jj[u]) * 32 + lane;
                    const float v = gv[u] + lambda * wv[u];
                    ok = fabsf(v) > SKML_EPS;
                    g[k] = ok ? v : 0.f;
                }
                const unsigned int kb = __ballot_sync(0xFFFFFFFFu, ok);
                if (lane == jj[u]) keep = kb;
            }
        }
        if (keep != bits) bitmap[wi] = keep;
        cnt += __popc(keep);
    }
    unsigned int total;
    block_exclusive_scan<unsigned int>(cnt, &total);
    if (threadIdx.x == 0) block_counts[blockIdx.x] = total;
}

__global__ void __launch_bounds__(SKML_BLOCK)
compact_scan_kernel(unsigned int* __restrict__ block_counts, int nblocks, int dim, int allow_dense,
                    long long* __restrict__ meta) {
    __shared__ unsigned int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < nblocks; base += SKML_BLOCK) {
        int i = base + threadIdx.x;
        unsigned int v = i < nblocks ? block_counts[i] : 0u;
        unsigned int total;
        unsigned int ex = block_exclusive_scan<unsigned int>(v, &total);
        unsigned int c = carry;
        if (i < nblocks) block_counts[i] = c + ex;
        __syncthreads();
        if (threadIdx.x == 0) carry = c + total;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        long long nnz = carry;
        meta[0] = nnz;
        long long thr = (long long)dim * 2 / 3;
        meta[1] = nnz == 0 ? 0 : ((allow_dense && nnz > thr) ? 2 : 1);
    }
}

__global__ void __launch_bounds__(SKML_BLOCK)
compact_write_kernel(float* __restrict__ g, const float* __restrict__ w, unsigned int* __restrict__ bitmap,
                     long long nwords, int dim, float lambda, const unsigned int* __restrict__ block_offsets,
                     const long long* __restrict__ meta, int* __restrict__ keys, float* __restrict__ vals,
                     float* __restrict__ dense_vals, long long capacity, unsigned int* status) {
    __shared__ unsigned int s_warp_off[SKML_WARPS];
    const int kind = (int)meta[1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long wbase = (long long)blockIdx.x * COMPACT_WORDS + (long long)warp * (32 * COMPACT_WPT);
    if (kind == 2 && dense_vals != nullptr) {
        // dense kind: every coordinate is shipped. Kept coordinates already hold g + lambda*w
        // (count pass); all others contribute lambda * w alone.
        for (int grp = 0; grp < COMPACT_WPT; ++grp) {
            const long long gbase = wbase + grp * 32;
            const long long wi = gbase + lane;
            const unsigned int bits = wi < nwords ? bitmap[wi] : 0u;
            if (wi < nwords) bitmap[wi] = 0;
            for (int j = 0; j < 32; ++j) {
                const unsigned int wb = __shfl_sync(0xFFFFFFFFu, bits, j);
                const long long k = (gbase + j) * 32 + lane;
                if (k < dim) {
                    dense_vals[k] = ((wb >> lane) & 1u) ? g[k] : lambda * w[k];
                    g[k] = 0.f;
                }
            }
        }
        return;
    }
    unsigned int words[COMPACT_WPT];
    unsigned int cnt = 0;
#pragma unroll
    for (int grp = 0; grp < COMPACT_WPT; ++grp) {
        const long long wi = wbase + grp * 32 + lane;
        words[grp] = wi < nwords ? bitmap[wi] : 0u;
        cnt += __popc(words[grp]);
    }
    const unsigned int warp_total = warp_sum(cnt);
    if (lane == 0) s_warp_off[warp] = warp_total;
    __syncthreads();
    if (warp == 0) {
        unsigned int v = s_warp_off[lane], inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            unsigned int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += t;
        }
        s_warp_off[lane] = inc - v;
    }
    __syncthreads();
    long long out = (long long)block_offsets[blockIdx.x] + s_warp_off[warp];
    bool overflow = false;
#pragma unroll
    for (int grp = 0; grp < COMPACT_WPT; ++grp) {
        const long long gbase = wbase + grp * 32;
        const long long wi = gbase + lane;
        const unsigned int bits = words[grp];
        const int pc = __popc(bits);
        unsigned int inc = (unsigned int)pc;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            unsigned int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += t;
        }
        const unsigned int ex = inc - (unsigned int)pc;
        const unsigned int grp_total = __shfl_sync(0xFFFFFFFFu, inc, 31);
        if (pc > 0 && pc <= COMPACT_SPARSE_BITS) {
            int tpos[COMPACT_SPARSE_BITS];
            float gv[COMPACT_SPARSE_BITS];
            unsigned int b = bits;
#pragma unroll
            for (int j = 0; j < COMPACT_SPARSE_BITS; ++j) {
                tpos[j] = b ? __ffs(b) - 1 : -1;
                b &= b - 1;
                gv[j] = tpos[j] >= 0 ? g[wi * 32 + tpos[j]] : 0.f;
            }
            long long pos = out + ex;
#pragma unroll
            for (int j = 0; j < COMPACT_SPARSE_BITS; ++j) {
                if (tpos[j] < 0) continue;
                const long long k = wi * 32 + tpos[j];
                if (pos < capacity) {
                    keys[pos] = (int)k;
                    vals[pos] = gv[j];
                } else {
                    overflow = true;
                }
                g[k] = 0.f;
                ++pos;
            }
        }
        unsigned int dense = __ballot_sync(0xFFFFFFFFu, pc > COMPACT_SPARSE_BITS);
        while (dense) {
            int jj[COMPACT_DENSE_BATCH];
            unsigned int wb[COMPACT_DENSE_BATCH], exj[COMPACT_DENSE_BATCH];
            float gv[COMPACT_DENSE_BATCH];
#pragma unroll
            for (int u = 0; u < COMPACT_DENSE_BATCH; ++u) {
                jj[u] = dense ? __ffs(dense) - 1 : -1;
                dense &= dense - 1;
                const int src = jj[u] < 0 ? 0 : jj[u];
                wb[u] = jj[u] < 0 ? 0u : __shfl_sync(0xFFFFFFFFu, bits, src);
                exj[u] = __shfl_sync(0xFFFFFFFFu, ex, src);
                gv[u] = ((wb[u] >> lane) & 1u) ? g[(gbase + src) * 32 + lane] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < COMPACT_DENSE_BATCH; ++u) {
                if (!((wb[u] >> lane) & 1u)) continue;
                const long long k = (gbase + jj[u]) * 32 + lane;
                const long long pos = out + exj[u] + __popc(wb[u] & ((1u << lane) - 1u));
                if (pos < capacity) {
                    keys[pos] = (int)k;
                    vals[pos] = gv[u];
                } else {
                    overflow = true;
                }
                g[k] = 0.f;
            }
        }
        if (bits) bitmap[wi] = 0;
        out += grp_total;
    }
    if (overflow) skml_set_status(status, SKML_CAPACITY, 0x20u);
}

extern "C" int skml_compact(float* g, const float* w, unsigned int* bitmap, int dim, float lambda,
                            unsigned int* block_counts, long long* meta, int* keys, float* vals, float* dense_vals,
                            long long capacity, unsigned int* status, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    long long nwords = ((long long)dim + 31) / 32;
    int nblocks = (int)((nwords + COMPACT_WORDS - 1) / COMPACT_WORDS);
    compact_count_kernel<<<nblocks, SKML_BLOCK, 0, stream>>>(g, w, bitmap, nwords, dim, lambda, block_counts);
    compact_scan_kernel<<<1, SKML_BLOCK, 0, stream>>>(block_counts, nblocks, dim, dense_vals != nullptr, meta);
    compact_write_kernel<<<nblocks, SKML_BLOCK, 0, stream>>>(g, w, bitmap, nwords, dim, lambda, block_counts, meta,
                                                            keys, vals, dense_vals, capacity, status);
    return (int)cudaGetLastError();
}

extern "C" long long skml_compact_blocks(int dim) {
    long long nwords = ((long long)dim + 31) / 32;
    return (nwords + COMPACT_WORDS - 1) / COMPACT_WORDS;
}

// ---------------------------------------------------------------------------
// Updates for the uncompressed baselines (the compressed path updates inside the
// fused decode kernel).
// opt[0] = lr, opt[1] = sqrt(1 - beta2^t) / (1 - beta1^t) for Adam.
// ---------------------------------------------------------------------------
// ms: elements between the moments of neighbouring coordinates (1: plain arrays; 4: m and v point into
// one array of per-coordinate quads, so both moments of a coordinate come with one memory sector).
__device__ __forceinline__ void apply_update(float* w, float* m, float* v, long long k, float gval, int adam,
                                             float lr, float adam_scale, long long ms) {
    if (!adam) {
        w[k] -= lr * gval;
    } else {
        const long long q = k * ms;
        float mt = 0.9f * m[q] + 0.1f * gval;
        float vt = 0.999f * v[q] + 0.001f * gval * gval;
        w[k] -= lr * adam_scale * mt / (sqrtf(vt) + 1e-8f);
        m[q] = mt;
        v[q] = vt;
    }
}

__global__ void update_dense_kernel(float* w, float* m, float* v, const float* g, long long dim, float scale,
                                    int adam, float lr, float adam_scale, int sparse_only, long long ms) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += (long long)gridDim.x * blockDim.x) {
        float gv = g[i] * scale;
        if (sparse_only && gv == 0.f) continue;
        apply_update(w, m, v, i, gv, adam, lr, adam_scale, ms);
    }
}

__global__ void update_sparse_kernel(float* w, float* m, float* v, const int* keys, const float* vals,
                                     const long long* n_ptr, long long n_max, float scale, int adam, float lr,
                                     float adam_scale, long long ms) {
    long long n = n_ptr ? *n_ptr : n_max;
    if (n > n_max) n = n_max;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        apply_update(w, m, v, keys[i], vals[i] * scale, adam, lr, adam_scale, ms);
}

extern "C" int skml_update_dense(float* w, float* m, float* v, const float* g, long long dim, float scale, int adam,
                                 float lr, float adam_scale, int sparse_only, int adam_stride, void* stream) {
    int grid = sm_count() * 8;
    update_dense_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(w, m, v, g, dim, scale, adam, lr, adam_scale,
                                                                sparse_only, adam_stride > 1 ? adam_stride : 1);
    return (int)cudaGetLastError();
}

extern "C" int skml_update_sparse(float* w, float* m, float* v, const int* keys, const float* vals,
                                  const long long* n_ptr, long long n_max, float scale, int adam, float lr,
                                  float adam_scale, int adam_stride, void* stream) {
    int grid = sm_count() * 8;
    update_sparse_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(w, m, v, keys, vals, n_ptr, n_max, scale, adam, lr,
                                                                 adam_scale, adam_stride > 1 ? adam_stride : 1);
    return (int)cudaGetLastError();
}

// Sum of squares of the model in one launch: a contiguous slice per block, the partial sums added in
// block order by the last block to finish (so the result does not depend on the schedule).
constexpr int NORM_BLOCKS = 592;

__global__ void __launch_bounds__(256) weight_norm_kernel(const float* __restrict__ w, long long dim, double lambda,
                                                          double* __restrict__ sumsq_out, double* __restrict__ reg_out,
                                                          double* __restrict__ partials, unsigned int* __restrict__ counter) {
    const long long per = ((dim + gridDim.x - 1) / gridDim.x + 3) & ~3ll;
    const long long lo = per * blockIdx.x, hi = lo + per < dim ? lo + per : dim;
    double acc = 0.0;
    for (long long i = lo + 4ll * threadIdx.x; i < hi; i += 4ll * blockDim.x) {
        if (i + 4 <= hi) {
            const float4 v = *reinterpret_cast<const float4*>(w + i);  // lo is a multiple of 4: 16-byte aligned
            acc += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
        } else {
            for (long long j = i; j < hi; ++j) acc += (double)w[j] * w[j];
        }
    }
    __shared__ double sh[256];
    __shared__ bool last;
    sh[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = sh[0];
        __threadfence();
        last = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    double t = 0.0;
    for (int b = threadIdx.x; b < (int)gridDim.x; b += 256) t += __ldcg(partials + b);
    sh[threadIdx.x] = t;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        *counter = 0;
        if (sumsq_out) sumsq_out[0] = sh[0];
        if (reg_out) reg_out[0] = lambda * sqrt(sh[0]);
    }
}

extern "C" long long skml_weight_norm_scratch_bytes() { return (NORM_BLOCKS + 2) * 8; }

extern "C" int skml_weight_norm(const float* w, long long dim, double lambda, double* sumsq_out, double* reg_out,
                                void* scratch, void* stream) {
    if (!w || !scratch || dim < 0) return (int)cudaErrorInvalidValue;
    double* partials = reinterpret_cast<double*>(scratch);
    unsigned int* counter = reinterpret_cast<unsigned int*>(partials + NORM_BLOCKS);
    weight_norm_kernel<<<NORM_BLOCKS, 256, 0, (cudaStream_t)stream>>>(w, dim, lambda, sumsq_out, reg_out, partials, counter);
    return (int)cudaGetLastError();
}

// Update from a dense accumulator on exactly the coordinates of the gathered key lists, clearing the
// accumulator on the way: the work is proportional to the number of gathered keys, not to the model
// dimension. One launch per list (keys are distinct inside a list, so a launch touches every word at
// most once); a coordinate shared by several lists is updated by the first one and found cleared
// (exactly zero, skipped) by the later ones. A sum that is exactly zero is a no-op, as in the
// `sparse_only` dense update.
__global__ void update_gathered_kernel(float* w, float* m, float* v, float* acc, const int* keys, const long long* count,
                                       long long stride, float scale, int adam, float lr, float adam_scale, long long ms) {
    long long n = *count;
    if (n > stride) n = stride;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int k = keys[i];
        const float g = acc[k];
        if (g == 0.f) continue;
        acc[k] = 0.f;
        apply_update(w, m, v, k, g * scale, adam, lr, adam_scale, ms);
    }
}

extern "C" int skml_update_gathered(float* w, float* m, float* v, float* acc, const int* keys, const long long* counts,
                                    long long stride, int lists, float scale, int adam, float lr, float adam_scale,
                                    int adam_stride, void* stream) {
    for (int l = 0; l < lists; ++l) {
        update_gathered_kernel<<<sm_count() * 8, 256, 0, (cudaStream_t)stream>>>(w, m, v, acc, keys + (long long)l * stride,
                                                                                 counts + l, stride, scale, adam, lr, adam_scale,
                                                                                 adam_stride > 1 ? adam_stride : 1);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

// Scatter-add of (key, value) lists into a dense accumulator (raw key/value all-gather
// baseline: local sum of the gathered lists).
__global__ void scatter_kv_kernel(float* acc, const int* keys, const float* vals, const long long* counts,
                                  long long stride, int lists) {
    for (int l = 0; l < lists; ++l) {
        long long n = counts[l];
        if (n > stride) n = stride;
        const int* k = keys + (long long)l * stride;
        const float* v = vals + (long long)l * stride;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
             i += (long long)gridDim.x * blockDim.x)
            atomicAdd(acc + k[i], v[i]);
    }
}

// One launch per list: inside a list every key occurs once, so its adds touch distinct words, and
// stream order fixes the order in which the lists reach a word. Every rank therefore computes the
// same floating-point sums (a single launch over all lists would let blocks run ahead into later
// lists, and three or more addends in varying order round differently).
extern "C" int skml_scatter_kv(float* acc, const int* keys, const float* vals, const long long* counts,
                               long long stride, int lists, void* stream) {
    for (int l = 0; l < lists; ++l) {
        scatter_kv_kernel<<<sm_count() * 8, 256, 0, (cudaStream_t)stream>>>(acc, keys + (long long)l * stride,
                                                                            vals + (long long)l * stride, counts + l, stride, 1);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

// ---------------------------------------------------------------------------
// Synthetic data generation on the device.
// ---------------------------------------------------------------------------
__device__ __forceinline__ double u01(uint64_t h) { return (double)(h >> 11) * (1.0 / 9007199254740992.0); }

__device__ __forceinline__ float normal_from(uint64_t h1, uint64_t h2) {
    double a = u01(h1), b = u01(h2);
    if (a < 1e-300) a = 1e-300;
    return (float)(sqrt(-2.0 * log(a)) * cospi(2.0 * b));
}

__global__ void gen_wstar_kernel(float* w, long long dim, double density, uint64_t seed) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += (long long)gridDim.x * blockDim.x) {
        bool on = density >= 1.0 || u01(skml_rand(seed, 0xA1u, (uint64_t)i, 0)) < density;
        w[i] = on ? normal_from(skml_rand(seed, 0xA2u, (uint64_t)i, 0), skml_rand(seed, 0xA3u, (uint64_t)i, 0)) : 0.f;
    }
}

extern "C" int skml_gen_wstar(float* w, long long dim, double density, unsigned long long seed, void* stream) {
    gen_wstar_kernel<<<sm_count() * 8, 256, 0, (cudaStream_t)stream>>>(w, dim, density, seed);
    return (int)cudaGetLastError();
}

// 0-based Zipf(s) rank from a uniform draw: the density x^-s on [1, dim+1) inverted in
// closed form (s == 0: uniform).
__device__ __forceinline__ int zipf_rank(double u, int dim, double s, double top_pow, double inv_a, double log_top) {
    double x;
    if (s == 0.0) x = 1.0 + u * dim;
    else if (inv_a == 0.0) x = exp(u * log_top);
    else x = pow(1.0 + u * (top_pow - 1.0), inv_a);
    long long r = (long long)x - 1;
    if (r < 0) r = 0;
    if (r >= dim) r = dim - 1;
    return (int)r;
}

#define GEN_WARPS 8
#define GEN_MAX_K 256
// One warp per row. Candidates are drawn in rounds of 32; a candidate is kept if it is
// new to the row (compared with the kept list and with lower lanes of the round).
__global__ void __launch_bounds__(GEN_WARPS * 32)
gen_rows_kernel(int* __restrict__ cols, float* __restrict__ vals, float* __restrict__ labels, long long row_offset,
                long long rows, int dim, int k, double s, int value_kind, int task, float noise,
                const float* __restrict__ wstar, uint64_t seed) {
    __shared__ int s_cols[GEN_WARPS][GEN_MAX_K];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const double a = 1.0 - s;
    const bool is_one = fabs(a) < 1e-9;
    const double inv_a = is_one ? 0.0 : 1.0 / a;
    const double top_pow = is_one ? 0.0 : pow((double)dim + 1.0, a);
    const double log_top = log((double)dim + 1.0);
    for (long long r = (long long)blockIdx.x * GEN_WARPS + warp; r < rows; r += (long long)gridDim.x * GEN_WARPS) {
        const uint64_t gid = (uint64_t)(row_offset + r);
        int have = 0;
        unsigned int round = 0;
        while (have < k && round < 4096) {
            uint64_t h = skml_rand(seed, gid, (uint64_t)round * 32 + lane, 0xC0u);
            int c = zipf_rank(u01(h), dim, s, top_pow, inv_a, log_top);
            bool fresh = true;
            for (int j = 0; j < have; ++j)
                if (s_cols[warp][j] == c) fresh = false;
            unsigned int same = __match_any_sync(0xFFFFFFFFu, c);
            if ((same & ((1u << lane) - 1u)) != 0) fresh = false;  // a lower lane drew the same column
            unsigned int m = __ballot_sync(0xFFFFFFFFu, fresh);
            int pos = have + __popc(m & ((1u << lane) - 1u));
            if (fresh && pos < k) s_cols[warp][pos] = c;
            have += __popc(m);
            if (have > k) have = k;
            ++round;
            __syncwarp();
        }
        // values, margin, label
        float sq = 0.f;
        for (int j = lane; j < k; j += 32) {
            float v = 1.f;
            if (value_kind == 1) v = (float)u01(skml_rand(seed, gid, j, 0xC1u)) + 1e-12f;
            else if (value_kind == 2) v = normal_from(skml_rand(seed, gid, j, 0xC2u), skml_rand(seed, gid, j, 0xC3u));
            sq += v * v;
        }
        sq = warp_sum(sq);
        float scale = value_kind == 1 ? rsqrtf(sq) : 1.f;
        float margin = 0.f;
        for (int j = lane; j < k; j += 32) {
            float v = 1.f;
            if (value_kind == 1) v = ((float)u01(skml_rand(seed, gid, j, 0xC1u)) + 1e-12f) * scale;
            else if (value_kind == 2) v = normal_from(skml_rand(seed, gid, j, 0xC2u), skml_rand(seed, gid, j, 0xC3u));
            int c = j < have ? s_cols[warp][j] : 0;
            cols[r * k + j] = c;
            if (vals) vals[r * k + j] = v;
            margin += wstar[c] * v;
        }
        margin = warp_sum(margin);
        if (lane == 0) {
            float y;
            float nz = noise != 0.f ? noise * normal_from(skml_rand(seed, gid, 1, 0xC4u), skml_rand(seed, gid, 2, 0xC4u)) : 0.f;
            if (task == 0) {
                float p = 1.f / (1.f + __expf(-margin));
                y = u01(skml_rand(seed, gid, 0, 0xC5u)) < (double)p ? 1.f : -1.f;
            } else if (task == 1) {
                y = margin + nz >= 0.f ? 1.f : -1.f;
            } else {
                y = margin + nz;
            }
            labels[r] = y;
        }
        __syncwarp();
    }
}

extern "C" int skml_gen_rows(int* cols, float* vals, float* labels, long long row_offset, long long rows, int dim,
                             int k, double s, int value_kind, int task, float noise, const float* wstar,
                             unsigned long long seed, void* stream) {
    if (k > GEN_MAX_K || k > dim || k < 1) return -1;
    long long blocks = (rows + GEN_WARPS - 1) / GEN_WARPS;
    long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    gen_rows_kernel<<<(unsigned)blocks, GEN_WARPS * 32, 0, (cudaStream_t)stream>>>(
        cols, vals, labels, row_offset, rows, dim, k, s, value_kind, task, noise, wstar, seed);
    return (int)cudaGetLastError();
}

extern "C" int skml_sm_count() { return sm_count(); }

// ---------------------------------------------------------------------------
// Transposed-index gradient. For a shard whose minibatches are fixed row slices, the batch's
// column-major index (distinct columns, their row lists) is built once. A step then needs the
// per-row coefficients (glm_rows_kernel<2>) and, per distinct column c of the batch,
//     value[c] = sum over the batch rows r that contain c of coef[r] * x[r][c]  +  lambda * w[c],
// which is a gather of coefficients (an L2-resident array of batch-size floats) instead of a
// scatter into the dim-sized accumulator: no atomics, no touched bitmap, no compaction, and the
// keys come out sorted because the column list is. Columns are binned by their number of
// entries when the index is built: one thread, one warp or one block per column.
// (Equivalent of ml/gradient/DenseDoubleGradient.scala:51-57 + toSparse for a known sparsity
// pattern.)
// ---------------------------------------------------------------------------
__device__ __forceinline__ float colsum_range(const int* __restrict__ rowidx, const float* __restrict__ svals,
                                              const float* __restrict__ coef, int e0, int e1, int start, int stride) {
    float acc = 0.f;
    for (int e = e0 + start; e < e1; e += stride) {
        const float c = __ldg(coef + rowidx[e]);
        acc = fmaf(c, svals ? svals[e] : 1.f, acc);
    }
    return acc;
}

// bins[0..n_short) thread per column, bins[n_short..n_short+n_medium) warp per column (bins hold
// positions into ucols / colptr). Long columns are cut into segments of a few thousand entries at
// build time: item j = (long_col[j], [long_e0[j], long_e1[j])), one block each, partial sums added
// atomically into `out` (which the caller zeroes for that reason).
__global__ void __launch_bounds__(256)
colsum_kernel(const int* __restrict__ colptr, const int* __restrict__ rowidx, const float* __restrict__ svals,
              const int* __restrict__ ucols, const int* __restrict__ bins, const int* __restrict__ long_col,
              const int* __restrict__ long_e0, const int* __restrict__ long_e1, int n_short, int n_medium, int n_long,
              int short_blocks, int medium_blocks, const float* __restrict__ coef, const float* __restrict__ w,
              float lambda, float* __restrict__ out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int b = blockIdx.x;
    if (b < short_blocks) {
        const int t = b * 256 + threadIdx.x;
        if (t < n_short) {
            const int i = bins[t];
            const float wv = __ldg(w + ucols[i]);   // issued first: this DRAM gather overlaps the coefficient chain
            out[i] = colsum_range(rowidx, svals, coef, colptr[i], colptr[i + 1], 0, 1) + lambda * wv;
        }
        return;
    }
    b -= short_blocks;
    if (b < medium_blocks) {
        const int t = b * 8 + warp;
        if (t < n_medium) {
            const int i = bins[n_short + t];
            const float wv = lane == 0 ? __ldg(w + ucols[i]) : 0.f;
            float v = colsum_range(rowidx, svals, coef, colptr[i], colptr[i + 1], lane, 32);
            v = warp_sum(v);
            if (lane == 0) out[i] = v + lambda * wv;
        }
        return;
    }
    b -= medium_blocks;
    if (b < n_long) {
        __shared__ float s_part[8];
        const int i = long_col[b];
        const int e0 = long_e0[b];
        float v = colsum_range(rowidx, svals, coef, e0, long_e1[b], threadIdx.x, 256);
        v = warp_sum(v);
        if (lane == 0) s_part[warp] = v;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.f;
            for (int k = 0; k < 8; ++k) t += s_part[k];
            if (e0 == colptr[i]) t += lambda * w[ucols[i]];  // the column's first segment carries the L2 term
            atomicAdd(out + i, t);
        }
    }
}

extern "C" int skml_glm_coef(const long long* rowptr, const int* cols, const float* vals, const float* labels,
                             long long row_lo, long long row_cnt, long long nnz_padded, double avg_nnz,
                             const float* w, int loss_id, float inv_batch, double* loss_acc, float* coef_out,
                             unsigned int* status, long long budget, void* stream) {
    return grad_launch(2, rowptr, cols, vals, labels, row_lo, row_cnt, nnz_padded, avg_nnz, w, nullptr, nullptr, loss_id,
                       inv_batch, 0, loss_acc, coef_out, status, budget, (cudaStream_t)stream);
}

// Local-id batches (streamed minibatches whose column indices were replaced on the host by their
// position in the batch's sorted list of distinct columns): the weights of those columns are
// gathered once into a compact array, the gradient is scattered into a compact accumulator, and
// the sparse gradient's values are read off it in key order. The accumulators and the touched-bit
// words of the range are cleared for the next step.
__global__ void gather_compact_kernel(const float* __restrict__ w, const int* __restrict__ ucols, int n,
                                      float* __restrict__ wc) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) wc[i] = w[ucols[i]];
}

__global__ void finalize_compact_kernel(float* __restrict__ gc, const float* __restrict__ wc, float lambda, int n,
                                        float* __restrict__ vals, unsigned int* __restrict__ bitmap) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        vals[i] = gc[i] + lambda * wc[i];
        gc[i] = 0.f;
        if (bitmap && i < (n + 31) / 32) bitmap[i] = 0u;
    }
}

extern "C" int skml_gather_compact(const float* w, const int* ucols, int n, float* wc, void* stream) {
    if (n <= 0) return 0;
    gather_compact_kernel<<<sm_count() * 8, 256, 0, (cudaStream_t)stream>>>(w, ucols, n, wc);
    return (int)cudaGetLastError();
}

extern "C" int skml_finalize_compact(float* gc, const float* wc, float lambda, int n, float* vals, unsigned int* bitmap,
                                     void* stream) {
    if (n <= 0) return 0;
    finalize_compact_kernel<<<sm_count() * 8, 256, 0, (cudaStream_t)stream>>>(gc, wc, lambda, n, vals, bitmap);
    return (int)cudaGetLastError();
}

// Start-of-step housekeeping in one small launch: the loss partials are reset from their template
// and the output slots of the long columns (the only ones the column-sum kernel accumulates into
// with atomics) are cleared.
__global__ void step_prep_kernel(double* __restrict__ partials, const double* __restrict__ partials_template,
                                 float* __restrict__ out, const int* __restrict__ long_col, int n_long) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < 4) partials[t] = partials_template[t];
    for (int i = t; i < n_long; i += gridDim.x * blockDim.x) out[long_col[i]] = 0.f;  // duplicates store the same zero
}

extern "C" int skml_step_prep(double* partials, const double* partials_template, float* out, const int* long_col,
                              int n_long, void* stream) {
    int blocks = (n_long + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 1024) blocks = 1024;
    step_prep_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(partials, partials_template, out, long_col, n_long);
    return (int)cudaGetLastError();
}

// `out_is_prepared` != 0: the long columns' slots are already zero (skml_step_prep), skip the full clear.
extern "C" int skml_colsum_ex(const int* colptr, const int* rowidx, const float* svals, const int* ucols, const int* bins,
                              const int* long_col, const int* long_e0, const int* long_e1, int n_short, int n_medium,
                              int n_long, int n_cols, const float* coef, const float* w, float lambda, float* out,
                              int out_is_prepared, void* stream);

extern "C" int skml_colsum(const int* colptr, const int* rowidx, const float* svals, const int* ucols, const int* bins,
                           const int* long_col, const int* long_e0, const int* long_e1, int n_short, int n_medium,
                           int n_long, int n_cols, const float* coef, const float* w, float lambda, float* out,
                           void* stream) {
    return skml_colsum_ex(colptr, rowidx, svals, ucols, bins, long_col, long_e0, long_e1, n_short, n_medium, n_long,
                          n_cols, coef, w, lambda, out, 0, stream);
}

extern "C" int skml_colsum_ex(const int* colptr, const int* rowidx, const float* svals, const int* ucols, const int* bins,
                              const int* long_col, const int* long_e0, const int* long_e1, int n_short, int n_medium,
                              int n_long, int n_cols, const float* coef, const float* w, float lambda, float* out,
                              int out_is_prepared, void* stream) {
    if (!out_is_prepared) {
        cudaError_t e = cudaMemsetAsync(out, 0, (size_t)n_cols * sizeof(float), (cudaStream_t)stream);
        if (e != cudaSuccess) return (int)e;
    }
    const int short_blocks = (n_short + 255) / 256, medium_blocks = (n_medium + 7) / 8;
    const long long blocks = (long long)short_blocks + medium_blocks + n_long;
    if (blocks <= 0) return 0;
    colsum_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(colptr, rowidx, svals, ucols, bins, long_col, long_e0,
                                                                     long_e1, n_short, n_medium, n_long, short_blocks,
                                                                     medium_blocks, coef, w, lambda, out);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Row-tiled form of the transposed index. The per-column gather of `coef[row]` above costs one random
// 32-byte L2 sector per batch entry. Here the batch rows are cut into tiles of `tile_rows` rows whose
// coefficients fit in shared memory (196 KB for 49,152 rows), the index is ordered by (tile, column,
// row) with 16-bit tile-local rows, and a block that owns (a share of) a tile gathers from shared
// memory. One partial sum per (tile, column) pair goes to `partial[pair_dst[p]]`, a position in
// (column, tile) order, so the second kernel adds a column's partial sums from consecutive words, in
// tile order: no atomics anywhere, the result is bit-reproducible.
// ---------------------------------------------------------------------------
constexpr int CT_SHORT = 8;   // pairs of up to this many entries are summed by one lane

template <bool HAS_VALS>
__global__ void __launch_bounds__(1024, 1)
coltile_partial_kernel(const float* __restrict__ coef, int rows, int tile_rows, const int* __restrict__ tile_pair_ptr,
                       int blocks_per_tile, const int* __restrict__ pair_ptr, const unsigned short* __restrict__ lrow,
                       const float* __restrict__ svals, const int* __restrict__ pair_dst, float* __restrict__ partial) {
    extern __shared__ __align__(16) float s_coef[];
    const int tile = blockIdx.x / blocks_per_tile, sub = blockIdx.x % blocks_per_tile;
    const int r0 = tile * tile_rows, nr = min(tile_rows, rows - r0);
    {   // the tile's coefficients (r0 is a multiple of 4 floats: 16-byte aligned rows)
        const float4* src = reinterpret_cast<const float4*>(coef + r0);
        float4* dst = reinterpret_cast<float4*>(s_coef);
        const int nv = nr / 4;
        for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = __ldg(src + i);
        for (int i = 4 * nv + threadIdx.x; i < nr; i += blockDim.x) s_coef[i] = __ldg(coef + r0 + i);
    }
    __syncthreads();
    // this block's share of the tile's pairs: cut by entries (pairs are not split), found by binary search
    const int p0 = tile_pair_ptr[tile], p1 = tile_pair_ptr[tile + 1];
    __shared__ int s_my[2];
    if (threadIdx.x < 2) {
        const long long e0 = pair_ptr[p0], e1 = pair_ptr[p1];
        const int which = sub + threadIdx.x;
        int pos;
        if (which == 0) pos = p0;
        else if (which >= blocks_per_tile) pos = p1;
        else {
            const long long target = e0 + (e1 - e0) * which / blocks_per_tile;
            int lo = p0, hi = p1;
            while (lo < hi) {   // first pair that starts at or after the target entry
                const int mid = (lo + hi) >> 1;
                if ((long long)pair_ptr[mid] < target) lo = mid + 1;
                else hi = mid;
            }
            pos = lo;
        }
        s_my[threadIdx.x] = pos;
    }
    __syncthreads();
    const int my0 = s_my[0], my1 = s_my[1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    // the warps share the block's pairs by entries too (a warp that drew the frequent columns' pairs would
    // otherwise have many times the work of the others)
    int w0 = my0, w1 = my1;
    if (lane < 2 && my1 > my0) {
        const long long e0 = pair_ptr[my0], e1 = pair_ptr[my1];
        const int which = warp + lane;
        int pos;
        if (which == 0) pos = my0;
        else if (which >= nwarps) pos = my1;
        else {
            const long long target = e0 + (e1 - e0) * which / nwarps;
            int lo = my0, hi = my1;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if ((long long)pair_ptr[mid] < target) lo = mid + 1;
                else hi = mid;
            }
            pos = lo;
        }
        if (lane == 0) w0 = pos;
        else w1 = pos;
    }
    w0 = __shfl_sync(0xFFFFFFFFu, w0, 0);
    w1 = __shfl_sync(0xFFFFFFFFu, w1, 1);
    for (int base = w0; base < w1; base += 32) {
        const int p = base + lane;
        const bool valid = p < w1;
        const int e0 = valid ? __ldg(pair_ptr + p) : 0, e1 = valid ? __ldg(pair_ptr + p + 1) : 0;
        const int len = e1 - e0;
        float acc = 0.f;
        if (valid && len <= CT_SHORT) {
            for (int e = e0; e < e1; ++e) acc = fmaf(s_coef[lrow[e]], HAS_VALS ? svals[e] : 1.f, acc);
        }
        unsigned int longs = __ballot_sync(0xFFFFFFFFu, valid && len > CT_SHORT);
        while (longs) {   // the warp sums one long pair at a time (fixed order: lane stride, shuffle tree)
            const int src = __ffs(longs) - 1;
            longs &= longs - 1;
            const int se0 = __shfl_sync(0xFFFFFFFFu, e0, src), se1 = __shfl_sync(0xFFFFFFFFu, e1, src);
            float part = 0.f, part2 = 0.f;   // two independent chains: the loads of a round overlap
            int e = se0 + lane;
            for (; e + 32 < se1; e += 64) {
                const unsigned short r0 = lrow[e], r1 = lrow[e + 32];
                part = fmaf(s_coef[r0], HAS_VALS ? svals[e] : 1.f, part);
                part2 = fmaf(s_coef[r1], HAS_VALS ? svals[e + 32] : 1.f, part2);
            }
            if (e < se1) part = fmaf(s_coef[lrow[e]], HAS_VALS ? svals[e] : 1.f, part);
            part = warp_sum(part + part2);
            if (lane == src) acc = part;
        }
        if (valid) partial[__ldg(pair_dst + p)] = acc;
    }
}

__global__ void __launch_bounds__(256)
colsum_combine_kernel(const int* __restrict__ col_pair_ptr, const float* __restrict__ partial, const int* __restrict__ ucols,
                      const float* __restrict__ w, float lambda, int n_cols, float* __restrict__ out) {
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < n_cols; c += gridDim.x * blockDim.x) {
        const int q0 = col_pair_ptr[c], q1 = col_pair_ptr[c + 1];
        float v = 0.f;
        for (int q = q0; q < q1; ++q) v += partial[q];   // tile order
        out[c] = v + lambda * __ldg(w + ucols[c]);
    }
}

extern "C" int skml_colsum_tiled(const int* tile_pair_ptr, const int* pair_ptr, const unsigned short* lrow, const float* svals,
                                 const int* pair_dst, const int* col_pair_ptr, const int* ucols, int rows, int tile_rows,
                                 int n_tiles, int n_cols, const float* coef, const float* w, float lambda, float* partial,
                                 float* out, void* stream_) {
    if (n_cols <= 0 || n_tiles <= 0) return 0;
    if (tile_rows <= 0 || tile_rows > 65536 || (tile_rows & 3) || (long long)n_tiles * tile_rows < rows) return (int)cudaErrorInvalidValue;
    cudaStream_t stream = (cudaStream_t)stream_;
    static bool ready = false;
    if (!ready) {
        cudaError_t e = cudaFuncSetAttribute(coltile_partial_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 4 - 40 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(coltile_partial_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 4 - 40 * 1024);
        if (e != cudaSuccess) return (int)e;
        ready = true;
    }
    const int tr = tile_rows < rows ? tile_rows : ((rows + 3) & ~3);
    const size_t smem = (size_t)tr * sizeof(float);
    if (smem > 65536 * 4 - 40 * 1024) return (int)cudaErrorInvalidValue;
    int bpt = sm_count() / n_tiles;
    if (bpt < 1) bpt = 1;
    const unsigned grid = (unsigned)(n_tiles * bpt);
    if (svals)
        coltile_partial_kernel<true><<<grid, 1024, smem, stream>>>(coef, rows, tile_rows, tile_pair_ptr, bpt, pair_ptr, lrow, svals,
                                                                  pair_dst, partial);
    else
        coltile_partial_kernel<false><<<grid, 1024, smem, stream>>>(coef, rows, tile_rows, tile_pair_ptr, bpt, pair_ptr, lrow, svals,
                                                                   pair_dst, partial);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    colsum_combine_kernel<<<sm_count() * 8, 256, 0, stream>>>(col_pair_ptr, partial, ucols, w, lambda, n_cols, out);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// skml_compact_noalloc: the compaction above for callers that must not allocate.
// (Declared and documented in skml_noalloc.h; it has no counterpart in the reference.)
//
// The only scratch memory of the compaction is the per-block count / offset array. Here
// it lives in a file-scope device array instead of a caller-supplied buffer, so the call
// needs no cudaMalloc, no cudaFree and no allocating library routine.
// ---------------------------------------------------------------------------
#include <stdio.h>

#include <mutex>

#include "skml_noalloc.h"

static __device__ __align__(256) unsigned int g_noalloc_block_counts[SKML_NOALLOC_MAX_BLOCKS + 64];

#define NOALLOC_MAX_DEVICES 64
static unsigned int* g_noalloc_scratch_ptr[NOALLOC_MAX_DEVICES];  // device address of the array, per device
static std::mutex g_noalloc_mutex;

// In host code the array's name is only a handle of the symbol, not a device address:
// the address is asked for once per device, with that device current.
static int noalloc_scratch(unsigned int** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_block_counts);
        if (e != cudaSuccess) return (int)e;
        g_noalloc_scratch_ptr[dev] = static_cast<unsigned int*>(p);
    }
    *out = g_noalloc_scratch_ptr[dev];
    return 0;
}

extern "C" int skml_compact_noalloc(float* g, const float* w, unsigned int* bitmap, int dim, float lambda,
                                    long long* meta, int* keys, float* vals, long long capacity,
                                    unsigned int* status, void* stream_) {
    if (dim <= 0 || !g || !w || !bitmap || !meta || !keys || !vals || !status) {
        fprintf(stderr, "skml_compact_noalloc: null pointer or non-positive dim\n");
        return SKML_NOALLOC_BAD_ARGUMENT;
    }
    if ((long long)dim > SKML_NOALLOC_MAX_DIM) {
        fprintf(stderr, "skml_compact_noalloc: dim %d exceeds the built-in scratch (at most %lld coordinates); "
                        "use skml_compact with a caller-owned block_counts buffer\n", dim, (long long)SKML_NOALLOC_MAX_DIM);
        return SKML_NOALLOC_TOO_LARGE;
    }
    unsigned int* scratch = nullptr;
    int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    long long nwords = ((long long)dim + 31) / 32;
    int nblocks = (int)((nwords + COMPACT_WORDS - 1) / COMPACT_WORDS);
    // every entry of the scratch that is read (the first nblocks) is rewritten by the count
    // kernel of this call, so nothing of an earlier call has to be cleared
    compact_count_kernel<<<nblocks, SKML_BLOCK, 0, stream>>>(g, w, bitmap, nwords, dim, lambda, scratch);
    compact_scan_kernel<<<1, SKML_BLOCK, 0, stream>>>(scratch, nblocks, dim, 0, meta);
    compact_write_kernel<<<nblocks, SKML_BLOCK, 0, stream>>>(g, w, bitmap, nwords, dim, lambda, scratch, meta, keys,
                                                            vals, nullptr, capacity, status);
    return (int)cudaGetLastError();
}
