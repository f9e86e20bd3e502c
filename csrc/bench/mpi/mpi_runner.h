/* Shared skeleton of the MPI collective benchmarks. Per message size: load the input,
 * compute the reference with the un-intercepted PMPI_<collective> on a copy, warm up,
 * then time MPI_<collective> (which an LD_PRELOAD wrapper may have replaced) with
 * MPI_Wtime between two PMPI_Barriers, validating every iteration if asked. Same flow
 * as the reference's drivers (representative: run_codes/benchmarks/mpi/allreduce/
 * allreduce.c:41-140). */
#ifndef CCB_MPI_RUNNER_H
#define CCB_MPI_RUNNER_H

#include <mpi.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "binary_output.h"
#include "mpi/mpi_utils.h"
#include "utils.h"
#include "validation.h"

typedef struct {
    size_t send_bytes, recv_bytes;
} mpi_sizes_t;

typedef struct mpi_bench_op {
    const char *banner, *name;
    void (*sizes)(size_t count, size_t esz, int n, mpi_sizes_t *out);
    /* use_pmpi = 1: the reference path; 0: the (possibly intercepted) MPI_ path */
    int (*call)(const mpi_test_context_t *ctx, int use_pmpi, void *send, void *recv, int count, MPI_Datatype dt);
    double (*ref_bw)(size_t msg_bytes, const mpi_sizes_t *sz, int n, double sec);
    double (*bus_factor)(int n);
    int validate_rank; /* -1 all ranks, else one rank (-2 = last) */
    int dump_multi, dump_rank;
    int in_place;      /* result is produced in the send buffer (bcast) */
} mpi_bench_op_t;

static void mpi_bench_size(mpi_test_context_t *ctx, const mpi_bench_op_t *op, size_t msg, MPI_Datatype dt, void *u_send,
                           void *u_recv, void *r_send, void *r_recv, void *pristine) {
    int es_i = 0;
    PMPI_Type_size(dt, &es_i);
    const size_t esz = (size_t)es_i;
    size_t count = msg / esz;
    if (count == 0) count = 1;
    const int n = ctx->size;
    const data_type_t gdt = mpi_to_data_type(dt);
    mpi_sizes_t sz;
    op->sizes(count, esz, n, &sz);
    mpi_load_input(ctx, pristine, sz.send_bytes, dt);
    memcpy(u_send, pristine, sz.send_bytes);
    memcpy(r_send, pristine, sz.send_bytes);
    for (int i = 0; i < ctx->config.warmup_iterations; ++i) {
        if (op->in_place) memcpy(u_send, pristine, sz.send_bytes);
        if (op->call(ctx, 0, u_send, u_recv, (int)count, dt) != MPI_SUCCESS) {
            fprintf(stderr, "[rank=%d] %s FAILED -- aborting\n", ctx->rank, op->banner);
            exit(1);
        }
    }
    memcpy(r_send, pristine, sz.send_bytes);
    op->call(ctx, 1, r_send, r_recv, (int)count, dt);
    const void *ref = op->in_place ? r_send : r_recv;
    const int vr = op->validate_rank == -2 ? n - 1 : op->validate_rank;
    const int i_validate = ctx->config.validate && (vr < 0 || vr == ctx->rank);
    void *accum = ctx->config.save_binary ? calloc(1, sz.recv_bytes) : NULL;
    validation_result_t acc;
    memset(&acc, 0, sizeof(acc));
    acc.num_elements = sz.recv_bytes / esz;
    int bad = 0;
    double total = 0.0;
    for (int it = 0; it < ctx->config.iterations; ++it) {
        if (op->in_place) memcpy(u_send, pristine, sz.send_bytes);
        PMPI_Barrier(MPI_COMM_WORLD);
        const double t0 = MPI_Wtime();
        if (op->call(ctx, 0, u_send, u_recv, (int)count, dt) != MPI_SUCCESS) {
            fprintf(stderr, "[rank=%d] %s FAILED -- aborting\n", ctx->rank, op->banner);
            exit(1);
        }
        PMPI_Barrier(MPI_COMM_WORLD);
        total += MPI_Wtime() - t0;
        const void *out = op->in_place ? u_send : u_recv;
        if (accum) binary_accumulate(accum, out, (int)(sz.recv_bytes / esz), gdt);
        if (i_validate) {
            validation_result_t v = validate_result(out, ref, (int)(sz.recv_bytes / esz), gdt, ctx->config.tolerance, ctx->config.metrics_mask);
            if (!v.correct) ++bad;
            for (int m = 0; m < MAX_METRICS; ++m)
                if (ctx->config.metrics_mask & (1u << m)) acc.values[m] += v.values[m];
        }
    }
    if (ctx->config.validate && ctx->config.iterations > 0) {
        acc.correct = bad == 0;
        for (int m = 0; m < MAX_METRICS; ++m)
            if (ctx->config.metrics_mask & (1u << m)) acc.values[m] /= ctx->config.iterations;
    }
    if (accum) {
        if (ctx->config.iterations > 0) binary_average(accum, (int)(sz.recv_bytes / esz), gdt, ctx->config.iterations);
        if (op->dump_multi) {
            write_binary_multi(ctx->config.bin_path, "reference", ref, sz.recv_bytes, ctx->rank, n);
            write_binary_multi(ctx->config.bin_path, "user", accum, sz.recv_bytes, ctx->rank, n);
        } else {
            const int w = op->dump_rank == -2 ? n - 1 : op->dump_rank;
            write_binary_single(ctx->config.bin_path, "reference", ref, sz.recv_bytes, ctx->rank, w);
            write_binary_single(ctx->config.bin_path, "user", accum, sz.recv_bytes, ctx->rank, w);
        }
        free(accum);
    }
    const double sec = ctx->config.iterations > 0 ? total / ctx->config.iterations : 0.0;
    mpi_set_bandwidth(sec > 0 ? op->ref_bw(count * esz, &sz, n, sec) / 1e9 : 0.0, op->bus_factor ? op->bus_factor(n) : 0.0);
    mpi_report_results(ctx, count * esz, (int)count, total, bad, ctx->config.validate ? &acc : NULL);
}

static int mpi_bench_main(int argc, char **argv, const mpi_bench_op_t *op) {
    mpi_test_context_t ctx = mpi_test_init(argc, argv, op->banner);
    if (ctx.size < 2) {
        if (ctx.rank == 0) fprintf(stderr, "Error: Need at least 2 processes\n");
        mpi_test_fini(&ctx);
        return 1;
    }
    const MPI_Datatype dt = data_type_to_mpi(ctx.config.data_type);
    int es = 0;
    PMPI_Type_size(dt, &es);
    size_t maxcount = ctx.config.max_message_size / (size_t)es;
    if (maxcount == 0) maxcount = 1;
    mpi_sizes_t mx;
    op->sizes(maxcount, (size_t)es, ctx.size, &mx);
    const size_t cap = (mx.send_bytes > mx.recv_bytes ? mx.send_bytes : mx.recv_bytes) + 64;
    void *b[5];
    for (int i = 0; i < 5; ++i)
        if (!(b[i] = malloc(cap))) {
            fprintf(stderr, "Error: Memory allocation failed\n");
            return 1;
        }
    size_iter_t it;
    size_iter_init(&it, &ctx.config);
    size_t s;
    while (size_iter_next(&it, &s)) mpi_bench_size(&ctx, op, s, dt, b[0], b[1], b[2], b[3], b[4]);
    for (int i = 0; i < 5; ++i) free(b[i]);
    mpi_test_fini(&ctx);
    return 0;
}

static double mbus_allreduce(int n) { return n > 1 ? 2.0 * (n - 1) / n : 1.0; }
static double mbus_frac(int n) { return n > 1 ? (double)(n - 1) / n : 1.0; }
static double mbus_one(int n) { (void)n; return 1.0; }
#define MPI_BENCH_UNUSED (void)mbus_allreduce, (void)mbus_frac, (void)mbus_one

#endif
