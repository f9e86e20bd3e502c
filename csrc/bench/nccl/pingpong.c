/* Point-to-point ping-pong between rank 0 and every other rank in turn, each
 * ncclSend / ncclRecv timed on its own with CUDA events.
 *
 * Output contract (reference: run_codes/benchmarks/nccl/pingpong/pingpong.c:96-98,
 * 252-272): CSV header
 *   msg_size,partner,latency_us,bandwidth_gbps,send0_us,recv0_us,recvP_us,sendP_us
 * with "%.2f" values; latency = round trip / 2, bandwidth = size / round trip.
 * The reference adds the running send and receive totals into the round-trip total
 * on every iteration (:186), inflating it quadratically; here the round trip is the
 * sum of the per-iteration send and receive times. */
#include "bench_runner.h"

static float timed(cudaEvent_t e0, cudaEvent_t e1, cudaStream_t s, int is_send, void *buf, size_t count,
                   ncclDataType_t dt, int peer, ncclComm_t comm) {
    cudaEventRecord(e0, s);
    ncclResult_t r = is_send ? ncclSend(buf, count, dt, peer, comm, s) : ncclRecv(buf, count, dt, peer, comm, s);
    if (r != ncclSuccess) {
        fprintf(stderr, "pingpong: nccl%s failed: %s\n", is_send ? "Send" : "Recv", ncclGetErrorString(r));
        exit(1);
    }
    cudaEventRecord(e1, s);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    return ms;
}

int main(int argc, char **argv) {
    nccl_test_context_t ctx = nccl_test_init(argc, argv, "NCCL_PingPong");
    if (ctx.size < 2) {
        if (ctx.rank == 0) fprintf(stderr, "Error: Need at least 2 processes\n");
        nccl_test_fini(&ctx);
        return 1;
    }
    const ncclDataType_t dt = data_type_to_nccl(ctx.config.data_type);
    const size_t esz = nccl_dtype_size(dt);
    void *d_buf = NULL;
    double *d_stats = NULL;
    int *d_one = NULL;
    cudaMalloc(&d_buf, ctx.config.max_message_size ? ctx.config.max_message_size : esz);
    cudaMalloc((void **)&d_stats, 2 * sizeof(double));
    cudaMalloc((void **)&d_one, sizeof(int));
    cudaMemset(d_buf, 1, ctx.config.max_message_size ? ctx.config.max_message_size : esz);
    cudaMemset(d_one, 0, sizeof(int));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    char csv[600];
    if (ctx.config.csv_path[0]) snprintf(csv, sizeof(csv), "%s", ctx.config.csv_path);
    else snprintf(csv, sizeof(csv), "results/pingpong.csv");
    const char *header = "msg_size,partner,latency_us,bandwidth_gbps,send0_us,recv0_us,recvP_us,sendP_us";

    size_iter_t it;
    size_iter_init(&it, &ctx.config);
    size_t msg;
    while (size_iter_next(&it, &msg)) {
        size_t count = msg / esz;
        if (count == 0) count = 1;
        const size_t bytes = count * esz;
        if (ctx.rank == 0) printf("Size: %8zu bytes\n", bytes);
        for (int p = 1; p < ctx.size; ++p) {
            double send0 = 0, recv0 = 0, recvP = 0, sendP = 0;
            const int me = ctx.rank;
            if (me == 0 || me == p) {
                const int total = ctx.config.warmup_iterations + ctx.config.iterations;
                for (int i = 0; i < total; ++i) {
                    const int measured = i >= ctx.config.warmup_iterations;
                    if (me == 0) {
                        float a = timed(e0, e1, ctx.stream, 1, d_buf, count, dt, p, ctx.comm);
                        float b = timed(e0, e1, ctx.stream, 0, d_buf, count, dt, p, ctx.comm);
                        if (measured) { send0 += a; recv0 += b; }
                    } else {
                        float a = timed(e0, e1, ctx.stream, 0, d_buf, count, dt, 0, ctx.comm);
                        float b = timed(e0, e1, ctx.stream, 1, d_buf, count, dt, 0, ctx.comm);
                        if (measured) { recvP += a; sendP += b; }
                    }
                }
                /* the partner ships its two totals to rank 0 */
                if (me == p) {
                    double h[2] = {recvP, sendP};
                    cudaMemcpy(d_stats, h, sizeof(h), cudaMemcpyHostToDevice);
                    NCCLCHECK(ncclSend(d_stats, 2, ncclFloat64, 0, ctx.comm, ctx.stream));
                    cudaStreamSynchronize(ctx.stream);
                } else {
                    double h[2];
                    NCCLCHECK(ncclRecv(d_stats, 2, ncclFloat64, p, ctx.comm, ctx.stream));
                    cudaStreamSynchronize(ctx.stream);
                    cudaMemcpy(h, d_stats, sizeof(h), cudaMemcpyDeviceToHost);
                    recvP = h[0];
                    sendP = h[1];
                }
            }
            if (me == 0) {
                const int iters = ctx.config.iterations > 0 ? ctx.config.iterations : 1;
                const double s0 = send0 / iters * 1e3, r0 = recv0 / iters * 1e3;
                const double rp = recvP / iters * 1e3, sp = sendP / iters * 1e3;
                const double rt_us = s0 + r0;
                const double lat = rt_us / 2.0, bw = rt_us > 0 ? (double)bytes / (rt_us * 1e-6) / 1e9 : 0.0;
                printf("  partner %3d: latency=%10.2f us  bandwidth=%8.2f GB/s  (send0=%.2f recv0=%.2f recvP=%.2f sendP=%.2f us)\n",
                       p, lat, bw, s0, r0, rp, sp);
                if (ctx.config.save_csv)
                    nccl_csv_write(csv, header, "%zu,%d,%.2f,%.2f,%.2f,%.2f,%.2f,%.2f", bytes, p, lat, bw, s0, r0, rp, sp);
            }
            /* keep the other ranks in step between partners */
            NCCLCHECK(ncclAllReduce(d_one, d_one, 1, ncclInt32, ncclSum, ctx.comm, ctx.stream));
            cudaStreamSynchronize(ctx.stream);
        }
        if (ctx.rank == 0) printf("\n");
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(d_buf);
    cudaFree(d_stats);
    cudaFree(d_one);
    nccl_test_fini(&ctx);
    (void)bus_allreduce; (void)bus_nminus1_over_n; (void)bus_one; (void)bench_main;
    return 0;
}
