/* Shared parts of the two vector ("v") benchmarks: a weighted split of the message
 * over the ranks ($ALLGATHERV_WEIGHTS / $SCATTERV_WEIGHTS, equal shares when unset;
 * every share is at least one element) and the timing loop. The oracle is the data
 * pattern regenerated per rank, as in the reference (run_codes/benchmarks/nccl/
 * allgatherv/allgatherv.c:21-38, 69-78; scatterv/scatterv.c:30-45). */
#ifndef CCB_VCOMMON_H
#define CCB_VCOMMON_H
#include "bench_runner.h"

static int v_split(int *counts, int *displs, const int *weights, int n, int total) {
    long wsum = 0;
    for (int i = 0; weights && i < n; ++i) wsum += weights[i];
    int off = 0;
    for (int i = 0; i < n; ++i) {
        long c = (weights && wsum > 0) ? (long)weights[i] * total / wsum : total / n;
        counts[i] = c < 1 ? 1 : (int)c;
        displs[i] = off;
        off += counts[i];
    }
    return off;
}

typedef int (*v_call_t)(const nccl_test_context_t *ctx, const void *d_send, void *d_recv, const int *counts,
                        const int *displs, const int *d_counts, const int *d_displs, ncclDataType_t dt);

static float v_time_loop(nccl_test_context_t *ctx, v_call_t call, const void *h_send, size_t send_bytes, void *d_send,
                         void *d_recv, void *h_recv, const void *h_ref, size_t recv_bytes, const int *counts,
                         const int *displs, const int *d_counts, const int *d_displs, ncclDataType_t dt, int validate_me,
                         validation_result_t *acc, int *bad) {
    const size_t esz = nccl_dtype_size(dt);
    nccl_barrier(ctx);
    for (int i = 0; i < ctx->config.warmup_iterations; ++i) {
        if (call(ctx, d_send, d_recv, counts, displs, d_counts, d_displs, dt)) exit(1);
        cudaStreamSynchronize(ctx->stream);
    }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float total = 0.f;
    for (int it = 0; it < ctx->config.iterations; ++it) {
        cudaMemcpy(d_send, h_send, send_bytes, cudaMemcpyHostToDevice);
        nccl_barrier(ctx);
        cudaEventRecord(e0, ctx->stream);
        if (call(ctx, d_send, d_recv, counts, displs, d_counts, d_displs, dt)) {
            fprintf(stderr, "[rank=%d] collective FAILED at iter %d, aborting\n", ctx->rank, it);
            exit(1);
        }
        cudaEventRecord(e1, ctx->stream);
        cudaEventSynchronize(e1);
        float ms;
        cudaEventElapsedTime(&ms, e0, e1);
        total += ms;
        if (validate_me) {
            cudaMemcpy(h_recv, d_recv, recv_bytes, cudaMemcpyDeviceToHost);
            validation_result_t v = validate_result(h_recv, h_ref, (int)(recv_bytes / esz), nccl_to_data_type(dt),
                                                    ctx->config.tolerance, ctx->config.metrics_mask);
            if (!v.correct) ++*bad;
            for (int m = 0; m < MAX_METRICS; ++m)
                if (ctx->config.metrics_mask & (1u << m)) acc->values[m] += v.values[m];
        }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (ctx->config.iterations > 0)
        for (int m = 0; m < MAX_METRICS; ++m)
            if (ctx->config.metrics_mask & (1u << m)) acc->values[m] /= ctx->config.iterations;
    acc->correct = *bad == 0;
    return total;
}
#endif
