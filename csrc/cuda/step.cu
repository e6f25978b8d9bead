// skml_train_step: the launch sequence of one training step behind a single C call.
// Reference: ml/algorithm/GeneralizedLinearModel.scala:116-123 (trainOneIteration =
// computeGradient + aggregateAndUpdate); here the whole iteration is five kernel launches
// and one 32-byte device copy, issued back to back on one stream with no host round trip.
#include <cuda_runtime.h>

#include "skml_api.h"

extern "C" int skml_train_step(SkmlStepArgs* a, void* stream_) {
    if (!a || !a->compress || !a->decode) return (int)cudaErrorInvalidValue;
    cudaStream_t stream = (cudaStream_t)stream_;
    cudaError_t e = cudaMemcpyAsync(a->partials, a->partials_template, 4 * sizeof(double), cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return (int)e;
    for (int s = 0; s < 2; ++s) {
        if (a->seg_cnt[s] <= 0) continue;
        int rc = skml_glm_grad(a->rowptr, a->cols, a->vals, a->labels, a->seg_lo[s], a->seg_cnt[s], a->nnz_padded,
                               a->avg_nnz, a->w, a->g, a->bitmap, (int)a->loss_id, (float)a->inv_batch, (int)a->hot,
                               a->partials + 1, a->status, a->budget_cycles, stream_);
        if (rc) return rc;
    }
    int rc = skml_compact(a->g, a->w, a->bitmap, (int)a->dim, (float)a->lambda, a->block_counts, a->meta, a->keys,
                          a->gvals, a->dense_vals, a->n_max, a->status, stream_);
    if (rc) return rc;
    a->compress->step = a->step;
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
