/* MPI ping-pong between rank 0 and every other rank in turn. CSV as the reference
 * (run_codes/benchmarks/mpi/pingpong/pingpong.c:72-74, 217-230): header
 *   msg_size,partner,comm_type,latency_us,bandwidth_gbps,send0_us,recv0_us,recvP_us,sendP_us
 * with comm_type intra / inter by processor name; latency = round trip / 2. */
#include <string.h>

#include "mpi_runner.h"

int main(int argc, char **argv) {
    MPI_BENCH_UNUSED;
    (void)mpi_bench_main;
    mpi_test_context_t ctx = mpi_test_init(argc, argv, "MPI_PingPong");
    if (ctx.size < 2) {
        if (ctx.rank == 0) fprintf(stderr, "Error: Need at least 2 processes\n");
        mpi_test_fini(&ctx);
        return 1;
    }
    char me[MPI_MAX_PROCESSOR_NAME] = "", *all = calloc((size_t)ctx.size, MPI_MAX_PROCESSOR_NAME);
    int len = 0;
    PMPI_Get_processor_name(me, &len);
    PMPI_Allgather(me, MPI_MAX_PROCESSOR_NAME, MPI_CHAR, all, MPI_MAX_PROCESSOR_NAME, MPI_CHAR, MPI_COMM_WORLD);
    char *buf = malloc(ctx.config.max_message_size ? ctx.config.max_message_size : 1);
    memset(buf, 1, ctx.config.max_message_size ? ctx.config.max_message_size : 1);
    char csv[600];
    if (ctx.config.csv_path[0]) snprintf(csv, sizeof(csv), "%s", ctx.config.csv_path);
    else snprintf(csv, sizeof(csv), "results/pingpong.csv");
    const char *header = "msg_size,partner,comm_type,latency_us,bandwidth_gbps,send0_us,recv0_us,recvP_us,sendP_us";
    size_iter_t it;
    size_iter_init(&it, &ctx.config);
    size_t msg;
    while (size_iter_next(&it, &msg)) {
        if (ctx.rank == 0) printf("Size: %8zu bytes\n", msg);
        for (int p = 1; p < ctx.size; ++p) {
            double t[4] = {0, 0, 0, 0}; /* send0 recv0 recvP sendP, seconds */
            if (ctx.rank == 0 || ctx.rank == p) {
                const int total = ctx.config.warmup_iterations + ctx.config.iterations;
                for (int i = 0; i < total; ++i) {
                    const int m = i >= ctx.config.warmup_iterations;
                    double a, b, c;
                    if (ctx.rank == 0) {
                        a = MPI_Wtime(); MPI_Send(buf, (int)msg, MPI_CHAR, p, 1, MPI_COMM_WORLD);
                        b = MPI_Wtime(); MPI_Recv(buf, (int)msg, MPI_CHAR, p, 2, MPI_COMM_WORLD, MPI_STATUS_IGNORE);
                        c = MPI_Wtime();
                        if (m) { t[0] += b - a; t[1] += c - b; }
                    } else {
                        a = MPI_Wtime(); MPI_Recv(buf, (int)msg, MPI_CHAR, 0, 1, MPI_COMM_WORLD, MPI_STATUS_IGNORE);
                        b = MPI_Wtime(); MPI_Send(buf, (int)msg, MPI_CHAR, 0, 2, MPI_COMM_WORLD);
                        c = MPI_Wtime();
                        if (m) { t[2] += b - a; t[3] += c - b; }
                    }
                }
                if (ctx.rank == p) PMPI_Send(&t[2], 2, MPI_DOUBLE, 0, 3, MPI_COMM_WORLD);
                else PMPI_Recv(&t[2], 2, MPI_DOUBLE, p, 3, MPI_COMM_WORLD, MPI_STATUS_IGNORE);
            }
            if (ctx.rank == 0) {
                const int iters = ctx.config.iterations > 0 ? ctx.config.iterations : 1;
                const double s0 = t[0] / iters * 1e6, r0 = t[1] / iters * 1e6, rp = t[2] / iters * 1e6, sp = t[3] / iters * 1e6;
                const double rt = s0 + r0, lat = rt / 2, bwv = rt > 0 ? (double)msg / (rt * 1e-6) / 1e9 : 0;
                const char *kind = strncmp(all, all + (size_t)p * MPI_MAX_PROCESSOR_NAME, MPI_MAX_PROCESSOR_NAME) ? "inter" : "intra";
                printf("  partner %3d (%s): latency=%10.2f us  bandwidth=%8.2f GB/s\n", p, kind, lat, bwv);
                if (ctx.config.save_csv)
                    mpi_csv_write(csv, header, "%zu,%d,%s,%.2f,%.2f,%.2f,%.2f,%.2f,%.2f", msg, p, kind, lat, bwv, s0, r0, rp, sp);
            }
            PMPI_Barrier(MPI_COMM_WORLD);
        }
    }
    free(buf);
    free(all);
    mpi_test_fini(&ctx);
    return 0;
}
