// skml_train_step: the launch sequence of one training step behind a single C call.
// Reference: ml/algorithm/GeneralizedLinearModel.scala:116-123 (trainOneIteration =
// computeGradient + aggregateAndUpdate); here the whole iteration is five kernel launches
// (housekeeping, coefficients, column sums, fused compress, fused decode + update) issued back to
// back on one stream with no host round trip.
#include <cuda_runtime.h>

#include "skml_api.h"

// The batch arrays (rowptr, cols, vals, labels) are read by the gradient kernels only (a local-id
// batch's column list also by the compress kernel); a feeder that recycles them waits for this event.
static int batch_consumed(const SkmlStepArgs* a, cudaStream_t stream) {
    if (!a->grad_done_event) return 0;
    return (int)cudaEventRecord((cudaEvent_t)a->grad_done_event, stream);
}

extern "C" int skml_train_step(SkmlStepArgs* a, void* stream_) {
    if (!a || !a->compress || !a->decode) return (int)cudaErrorInvalidValue;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (a->t_colptr || a->tt_pair_ptr) {
        // transposed index: coefficients per row, then one gather-sum per distinct column
        const bool tiled = a->tt_pair_ptr != nullptr;
        int rc = skml_step_prep(a->partials, a->partials_template, a->gvals, a->t_long_col, tiled ? 0 : (int)a->t_long, stream_);
        if (rc) return rc;
        rc = skml_glm_coef(a->rowptr, a->cols, a->vals, a->labels, a->seg_lo[0], a->seg_cnt[0], a->nnz_padded,
                               a->avg_nnz, a->w, (int)a->loss_id, (float)a->inv_batch, a->partials + 1, a->coef,
                               a->status, a->budget_cycles, stream_);
        if (rc) return rc;
        if (tiled)
            rc = skml_colsum_tiled(a->tt_tile_pair_ptr, a->tt_pair_ptr, a->tt_lrow, a->t_vals, a->tt_pair_dst, a->tt_col_pair_ptr,
                                   a->t_ucols, (int)a->tt_rows, (int)a->tt_tile_rows, (int)a->tt_tiles, (int)a->t_cols, a->coef,
                                   a->w, (float)a->lambda, a->tt_partial, a->gvals, stream_);
        else
            rc = skml_colsum_ex(a->t_colptr, a->t_rowidx, a->t_vals, a->t_ucols, a->t_bins, a->t_long_col, a->t_long_e0,
                                a->t_long_e1, (int)a->t_short, (int)a->t_medium, (int)a->t_long, (int)a->t_cols, a->coef, a->w,
                                (float)a->lambda, a->gvals, 1, stream_);
        if (rc) return rc;
        rc = batch_consumed(a, stream);
        if (rc) return rc;
        a->compress->step = a->step;
        a->compress->keys = a->t_ucols;
        a->compress->meta = a->t_meta;
        a->compress->vals = a->gvals;
        rc = skml_compress_sparse(a->compress, stream_);
        if (rc) return rc;
        a->decode->step = a->step;
        a->decode->lr = a->lr;
        a->decode->adam_scale = a->adam_scale;
        a->decode->loss_out = a->loss_out;
        return skml_decode_update(a->decode, stream_);
    }
    cudaError_t e = cudaMemcpyAsync(a->partials, a->partials_template, 4 * sizeof(double), cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return (int)e;
    if (a->l_ucols) {
        // local-id batch: compact weights in, scatter into the compact accumulator, values out in key order
        const int n = (int)a->l_ncols;
        int rc = skml_gather_compact(a->w, a->l_ucols, n, a->wc, stream_);
        if (rc) return rc;
        for (int s = 0; s < 2; ++s) {
            if (a->seg_cnt[s] <= 0) continue;
            rc = skml_glm_grad(a->rowptr, a->cols, a->vals, a->labels, a->seg_lo[s], a->seg_cnt[s], a->nnz_padded,
                               a->avg_nnz, a->wc, a->gc, nullptr, (int)a->loss_id, (float)a->inv_batch, (int)a->hot,
                               a->partials + 1, a->status, a->budget_cycles, stream_);
            if (rc) return rc;
        }
        rc = skml_finalize_compact(a->gc, a->wc, (float)a->lambda, n, a->gvals, nullptr, stream_);  // no touched bitmap: every slot is a key
        if (rc) return rc;
        a->compress->step = a->step;
        a->compress->keys = a->l_ucols;
        a->compress->meta = a->l_meta;
        a->compress->vals = a->gvals;
        rc = skml_compress_sparse(a->compress, stream_);
        if (rc) return rc;
        rc = batch_consumed(a, stream);  // the compress kernel still reads the batch's column list and count
        if (rc) return rc;
        a->decode->step = a->step;
        a->decode->lr = a->lr;
        a->decode->adam_scale = a->adam_scale;
        a->decode->loss_out = a->loss_out;
        return skml_decode_update(a->decode, stream_);
    }
    for (int s = 0; s < 2; ++s) {
        if (a->seg_cnt[s] <= 0) continue;
        int rc = skml_glm_grad(a->rowptr, a->cols, a->vals, a->labels, a->seg_lo[s], a->seg_cnt[s], a->nnz_padded,
                               a->avg_nnz, a->w, a->g, a->bitmap, (int)a->loss_id, (float)a->inv_batch, (int)a->hot,
                               a->partials + 1, a->status, a->budget_cycles, stream_);
        if (rc) return rc;
    }
    int rc = batch_consumed(a, stream);
    if (rc) return rc;
    rc = skml_compact(a->g, a->w, a->bitmap, (int)a->dim, (float)a->lambda, a->block_counts, a->meta, a->keys,
                          a->gvals, a->dense_vals, a->n_max, a->status, stream_);
    if (rc) return rc;
    a->compress->step = a->step;
    a->compress->keys = a->keys;
    a->compress->meta = a->meta;
    a->compress->vals = a->gvals;
    rc = skml_compress_sparse(a->compress, stream_);
    if (rc) return rc;
    if (a->dense_vals) {
        a->compress->vals = a->dense_vals;
        rc = skml_compress_dense(a->compress, stream_);
        a->compress->vals = a->gvals;
        if (rc) return rc;
    }
    a->decode->step = a->step;
    a->decode->lr = a->lr;
    a->decode->adam_scale = a->adam_scale;
    a->decode->loss_out = a->loss_out;
    return skml_decode_update(a->decode, stream_);
}
