/* AllGatherv benchmark through the ncclAllGatherv extension; shares weighted by
 * $ALLGATHERV_WEIGHTS. Reference: run_codes/benchmarks/nccl/allgatherv/allgatherv.c
 * (bandwidth (recv - send) bytes / t, :159-163). */
#include "vcommon.h"

static int call(const nccl_test_context_t *x, const void *s, void *r, const int *counts, const int *displs,
                const int *dc, const int *dd, ncclDataType_t dt) {
    return ncclAllGatherv(s, counts[x->rank], dt, r, counts, displs, dt, dc, dd, x->comm, x->stream);
}

int main(int argc, char **argv) {
    nccl_test_context_t ctx = nccl_test_init(argc, argv, "NCCL_AllGatherv");
    if (ctx.size < 2) {
        if (ctx.rank == 0) fprintf(stderr, "Error: Need at least 2 processes\n");
        nccl_test_fini(&ctx);
        return 1;
    }
    const int n = ctx.size;
    int nw = 0;
    int *weights = nccl_parse_env_int_array("ALLGATHERV_WEIGHTS", n, &nw);
    const ncclDataType_t dt = data_type_to_nccl(ctx.config.data_type);
    const data_type_t gdt = ctx.config.data_type;
    const size_t esz = nccl_dtype_size(dt);
    const size_t cap = ctx.config.max_message_size + (size_t)n * esz;
    void *h_send = malloc(cap), *h_recv = malloc(cap), *h_ref = malloc(cap), *d_send, *d_recv;
    int *counts = malloc(sizeof(int) * n), *displs = malloc(sizeof(int) * n), *d_counts, *d_displs;
    cudaMalloc(&d_send, cap);
    cudaMalloc(&d_recv, cap);
    cudaMalloc((void **)&d_counts, sizeof(int) * n);
    cudaMalloc((void **)&d_displs, sizeof(int) * n);
    size_iter_t it;
    size_iter_init(&it, &ctx.config);
    size_t msg;
    nccl_set_busbw_factor(0.0);
    while (size_iter_next(&it, &msg)) {
        int total = (int)(msg / esz);
        if (total < n) total = n;
        const int total_recv = v_split(counts, displs, weights, n, total);
        const size_t send_bytes = (size_t)counts[ctx.rank] * esz, recv_bytes = (size_t)total_recv * esz;
        cudaMemcpy(d_counts, counts, sizeof(int) * n, cudaMemcpyHostToDevice);
        cudaMemcpy(d_displs, displs, sizeof(int) * n, cudaMemcpyHostToDevice);
        init_buffer_pattern(h_send, counts[ctx.rank], gdt, ctx.config.pattern_type, ctx.rank);
        cudaMemcpy(d_send, h_send, send_bytes, cudaMemcpyHostToDevice);
        for (int r = 0; r < n; ++r)
            init_buffer_pattern((char *)h_ref + (size_t)displs[r] * esz, counts[r], gdt, ctx.config.pattern_type, r);
        validation_result_t acc;
        memset(&acc, 0, sizeof(acc));
        acc.num_elements = (size_t)total_recv;
        int bad = 0;
        float ms = v_time_loop(&ctx, call, h_send, send_bytes, d_send, d_recv, h_recv, h_ref, recv_bytes, counts, displs,
                               d_counts, d_displs, dt, ctx.config.validate, &acc, &bad);
        const double sec = ctx.config.iterations > 0 ? ms / ctx.config.iterations / 1e3 : 0.0;
        const double bw = sec > 0 ? (double)(recv_bytes - send_bytes) / sec / 1e9 : 0.0;
        nccl_report_results(&ctx, send_bytes, counts[ctx.rank], ms, bad, ctx.config.validate ? &acc : NULL, bw);
    }
    free(weights);
    nccl_test_fini(&ctx);
    return 0;
}
