/* Shared skeleton of the NCCL collective benchmarks: per message size load the input,
 * compute the CPU oracle, warm up, then time each call of the collective with CUDA
 * events on the benchmark's stream behind a host barrier, optionally validating every
 * iteration, and report. Mirrors the flow of the reference's drivers (representative:
 * run_codes/benchmarks/nccl/allreduce/allreduce.c:17-147) with these additions:
 * the oracle cache (-S/-R), resumption of an interrupted sweep (sizes already in the
 * CSV are skipped when CCB_RESUME=1), a per-size CSV row (-c), and nccl-tests bus
 * bandwidth beside the reference's own bandwidth definition. */
#ifndef CCB_BENCH_RUNNER_H
#define CCB_BENCH_RUNNER_H

#include <cuda_runtime.h>
#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "binary_output.h"
#include "dummy_collectives.h"
#include "nccl/nccl_extensions.h"
#include "nccl/nccl_utils.h"
#include "utils.h"
#include "validation.h"

typedef struct bench_sizes {
    size_t count;       /* elements of one "message" (what -m / -L name)  */
    size_t send_bytes;  /* bytes of the send buffer                        */
    size_t recv_bytes;  /* bytes of the receive buffer that are validated  */
} bench_sizes_t;

typedef struct bench_op {
    const char *banner;   /* "NCCL_AllReduce"                      */
    const char *name;     /* "allreduce" (CSV default, cache key)   */
    int min_ranks;
    /* buffer sizes for a message of `count` elements of `esz` bytes on n ranks */
    void (*sizes)(size_t count, size_t esz, int n, bench_sizes_t *out);
    /* enqueue the collective; return 0 on success */
    int (*call)(const nccl_test_context_t *ctx, const void *d_send, void *d_recv, size_t count, ncclDataType_t dt);
    /* expected receive buffer of THIS rank */
    void (*oracle)(const nccl_test_context_t *ctx, void *h_ref, size_t count, data_type_t dt);
    /* the reference's bandwidth definition, bytes per second */
    double (*ref_bw)(size_t msg_bytes, const bench_sizes_t *sz, int n, double sec);
    double (*bus_factor)(int n);  /* multiplies msg_bytes / t to give nccl-tests busbw */
    int validate_rank;  /* -1: every rank validates; else only this rank (-2 = last rank) */
    int dump_multi;     /* binary dump: 1 = every rank writes its chunk, 0 = single writer */
    int dump_rank;      /* single writer rank (-2 = last rank)                           */
    int in_place;       /* 1: the collective works in place on the send buffer (bcast)   */
} bench_op_t;

static inline int bench_resolve_rank(int r, int n) { return r == -2 ? n - 1 : r; }

static void bench_run_size(nccl_test_context_t *ctx, const bench_op_t *op, size_t msg_size, ncclDataType_t dt,
                           void *h_send, void *h_recv, void *h_ref, void *d_send, void *d_recv) {
    const size_t esz = nccl_dtype_size(dt);
    size_t count = msg_size / esz;
    if (count == 0) count = 1;
    const data_type_t gdt = nccl_to_data_type(dt);
    const int n = ctx->size;
    bench_sizes_t sz;
    op->sizes(count, esz, n, &sz);
    const size_t msg_bytes = count * esz;

    if (ctx->config.save_csv && getenv("CCB_RESUME")) {
        char path[600];
        if (ctx->config.csv_path[0]) snprintf(path, sizeof(path), "%s", ctx->config.csv_path);
        else snprintf(path, sizeof(path), "results/%s.csv", op->name);
        if (csv_has_size(path, msg_bytes, n)) return;
    }

    nccl_load_input(ctx, h_send, sz.send_bytes, dt);
    cudaMemcpy(d_send, h_send, sz.send_bytes, cudaMemcpyHostToDevice);
    if (!ref_cache_load(&ctx->config, op->name, n, ctx->rank, h_ref, sz.recv_bytes)) {
        op->oracle(ctx, h_ref, count, gdt);
        ref_cache_store(&ctx->config, op->name, n, ctx->rank, h_ref, sz.recv_bytes);
    }
    void *out = op->in_place ? d_send : d_recv;

    for (int i = 0; i < ctx->config.warmup_iterations; ++i) {
        if (op->in_place) cudaMemcpy(d_send, h_send, sz.send_bytes, cudaMemcpyHostToDevice);
        if (op->call(ctx, d_send, d_recv, count, dt) != 0) {
            fprintf(stderr, "[rank=%d] %s FAILED at size=%zu warm-up %d, aborting\n", ctx->rank, op->banner, msg_bytes, i);
            exit(1);
        }
        cudaStreamSynchronize(ctx->stream);
    }

    const int vrank = bench_resolve_rank(op->validate_rank, n);
    const int i_validate = ctx->config.validate && (vrank < 0 || vrank == ctx->rank);
    void *accum = ctx->config.save_binary ? calloc(1, sz.recv_bytes) : NULL;
    validation_result_t acc;
    memset(&acc, 0, sizeof(acc));
    acc.num_elements = sz.recv_bytes / esz;
    int bad_iters = 0;
    float total_ms = 0.f;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int it = 0; it < ctx->config.iterations; ++it) {
        cudaMemcpy(d_send, h_send, sz.send_bytes, cudaMemcpyHostToDevice);
        nccl_barrier(ctx);
        cudaEventRecord(e0, ctx->stream);
        if (op->call(ctx, d_send, d_recv, count, dt) != 0) {
            fprintf(stderr, "[rank=%d] %s FAILED at size=%zu iter=%d, aborting\n", ctx->rank, op->banner, msg_bytes, it);
            exit(1);
        }
        cudaEventRecord(e1, ctx->stream);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        total_ms += ms;
        if (accum || i_validate) {
            cudaMemcpy(h_recv, out, sz.recv_bytes, cudaMemcpyDeviceToHost);
            if (accum) binary_accumulate(accum, h_recv, (int)(sz.recv_bytes / esz), gdt);
        }
        if (i_validate) {
            validation_result_t v = validate_result(h_recv, h_ref, (int)(sz.recv_bytes / esz), gdt,
                                                    ctx->config.tolerance, ctx->config.metrics_mask);
            if (!v.correct) ++bad_iters;
            for (int m = 0; m < MAX_METRICS; ++m)
                if (ctx->config.metrics_mask & (1u << m)) acc.values[m] += v.values[m];
        }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (ctx->config.validate && ctx->config.iterations > 0) {
        acc.correct = bad_iters == 0;
        for (int m = 0; m < MAX_METRICS; ++m)
            if (ctx->config.metrics_mask & (1u << m)) acc.values[m] /= ctx->config.iterations;
        if (bad_iters && ctx->rank == 0)
            printf("  Validation FAILED at size %zu (%d/%d iterations failed)\n", msg_bytes, bad_iters,
                   ctx->config.iterations);
    }
    if (accum) {
        if (ctx->config.iterations > 0)
            binary_average(accum, (int)(sz.recv_bytes / esz), gdt, ctx->config.iterations);
        if (op->dump_multi) {
            write_binary_multi(ctx->config.bin_path, "reference", h_ref, sz.recv_bytes, ctx->rank, n);
            write_binary_multi(ctx->config.bin_path, "user", accum, sz.recv_bytes, ctx->rank, n);
        } else {
            const int w = bench_resolve_rank(op->dump_rank, n);
            write_binary_single(ctx->config.bin_path, "reference", h_ref, sz.recv_bytes, ctx->rank, w);
            write_binary_single(ctx->config.bin_path, "user", accum, sz.recv_bytes, ctx->rank, w);
        }
        free(accum);
    }
    const double sec = ctx->config.iterations > 0 ? (double)total_ms / ctx->config.iterations / 1e3 : 0.0;
    const double bw = sec > 0 ? op->ref_bw(msg_bytes, &sz, n, sec) / 1e9 : 0.0;
    nccl_set_busbw_factor(op->bus_factor ? op->bus_factor(n) : 0.0);
    nccl_report_results(ctx, msg_bytes, (int)count, total_ms, bad_iters, ctx->config.validate ? &acc : NULL, bw);
}

static int bench_main(int argc, char **argv, const bench_op_t *op) {
    nccl_test_context_t ctx = nccl_test_init(argc, argv, op->banner);
    /* CCB_ALLOW_SINGLE_RANK=1 lets a one-GPU host exercise the whole chain (driver, preloaded
     * wrappers, validation, CSV) with a communicator of one rank. */
    const char *single = getenv("CCB_ALLOW_SINGLE_RANK");
    const int need = (single && *single == '1') ? 1 : op->min_ranks;
    if (ctx.size < need) {
        if (ctx.rank == 0) fprintf(stderr, "Error: Need at least %d processes\n", need);
        nccl_test_fini(&ctx);
        return 1;
    }
    const ncclDataType_t dt = data_type_to_nccl(ctx.config.data_type);
    const size_t esz = nccl_dtype_size(dt);
    size_t maxcount = ctx.config.max_message_size / esz;
    if (maxcount == 0) maxcount = 1;
    bench_sizes_t mx;
    op->sizes(maxcount, esz, ctx.size, &mx);
    const size_t hb = mx.send_bytes > mx.recv_bytes ? mx.send_bytes : mx.recv_bytes;
    void *h_send = malloc(hb), *h_recv = malloc(hb), *h_ref = malloc(hb), *d_send = NULL, *d_recv = NULL;
    cudaMalloc(&d_send, mx.send_bytes > 0 ? mx.send_bytes : 1);
    cudaMalloc(&d_recv, mx.recv_bytes > 0 ? mx.recv_bytes : 1);
    if (!h_send || !h_recv || !h_ref || !d_send || !d_recv) {
        fprintf(stderr, "Error: Memory allocation failed\n");
        return 1;
    }
    size_iter_t it;
    size_iter_init(&it, &ctx.config);
    size_t s;
    while (size_iter_next(&it, &s)) bench_run_size(&ctx, op, s, dt, h_send, h_recv, h_ref, d_send, d_recv);
    free(h_send);
    free(h_recv);
    free(h_ref);
    cudaFree(d_send);
    cudaFree(d_recv);
    nccl_test_fini(&ctx);
    return 0;
}

/* common helpers for the op tables */
static double bus_allreduce(int n) { return n > 1 ? 2.0 * (n - 1) / n : 1.0; }
static double bus_nminus1_over_n(int n) { return n > 1 ? (double)(n - 1) / n : 1.0; }
static double bus_one(int n) { (void)n; return 1.0; }

#endif
