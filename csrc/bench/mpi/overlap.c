/* MPI compute / communication overlap: a communication thread exchanges messages
 * between even/odd rank pairs while the main thread spins fixed work units; both are
 * timed alone and together. Columns as the reference (run_codes/benchmarks/mpi/
 * overlap/overlap.c:297-305): Comp Send Recv PSend PRecv CntSnd CntRcv CSnd% CRcv%
 * SSlow% RSlow% (work-unit counts while a send / receive is in flight, and slow-downs). */
#include <pthread.h>
#include <string.h>

#include "mpi_runner.h"

static volatile int g_comm_running;
typedef struct { char *sbuf, *rbuf; int bytes, peer, sender, iters; double send_s, recv_s; } comm_job_t;

static double work_unit(void) {
    volatile double x = 1.0;
    for (int i = 0; i < 20000; ++i) x = x * 1.0000001 + 1e-9;
    return x;
}
static void *comm_thread(void *arg) {
    comm_job_t *j = (comm_job_t *)arg;
    for (int i = 0; i < j->iters; ++i) {
        double a = MPI_Wtime(), b;
        if (j->sender) {
            MPI_Send(j->sbuf, j->bytes, MPI_CHAR, j->peer, 7, MPI_COMM_WORLD);
            b = MPI_Wtime();
            MPI_Recv(j->rbuf, j->bytes, MPI_CHAR, j->peer, 8, MPI_COMM_WORLD, MPI_STATUS_IGNORE);
        } else {
            MPI_Recv(j->rbuf, j->bytes, MPI_CHAR, j->peer, 7, MPI_COMM_WORLD, MPI_STATUS_IGNORE);
            b = MPI_Wtime();
            MPI_Send(j->sbuf, j->bytes, MPI_CHAR, j->peer, 8, MPI_COMM_WORLD);
        }
        const double c = MPI_Wtime();
        if (j->sender) { j->send_s += b - a; j->recv_s += c - b; }
        else { j->recv_s += b - a; j->send_s += c - b; }
    }
    g_comm_running = 0;
    return NULL;
}

int main(int argc, char **argv) {
    MPI_BENCH_UNUSED;
    (void)mpi_bench_main;
    int provided = 0;
    PMPI_Init_thread(&argc, &argv, MPI_THREAD_SERIALIZED, &provided);
    mpi_test_context_t ctx = mpi_test_init(argc, argv, "MPI_Overlap");
    if (ctx.size < 2 || (ctx.size & 1)) {
        if (ctx.rank == 0) fprintf(stderr, "Error: Need an even number (>= 2) of processes\n");
        mpi_test_fini(&ctx);
        return 1;
    }
    const size_t cap = ctx.config.max_message_size ? ctx.config.max_message_size : 1;
    comm_job_t job;
    memset(&job, 0, sizeof(job));
    job.sbuf = malloc(cap);
    job.rbuf = malloc(cap);
    memset(job.sbuf, 1, cap);
    job.peer = ctx.rank ^ 1;
    job.sender = !(ctx.rank & 1);
    if (ctx.rank == 0)
        printf("%10s %9s %9s %9s %9s %9s %8s %8s %7s %7s %7s %7s\n", "Size(B)", "Comp(us)", "Send(us)", "Recv(us)", "PSend(us)", "PRecv(us)",
               "CntSnd", "CntRcv", "CSnd%", "CRcv%", "SSlow%", "RSlow%");
    size_iter_t it;
    size_iter_init(&it, &ctx.config);
    size_t msg;
    while (size_iter_next(&it, &msg)) {
        const int iters = ctx.config.iterations > 0 ? ctx.config.iterations : 1;
        job.bytes = (int)msg;
        job.iters = iters;
        /* compute alone: time of one work unit */
        double t0 = MPI_Wtime();
        for (int i = 0; i < 200; ++i) work_unit();
        const double unit_us = (MPI_Wtime() - t0) / 200 * 1e6;
        /* communication alone */
        PMPI_Barrier(MPI_COMM_WORLD);
        job.send_s = job.recv_s = 0;
        g_comm_running = 1;
        comm_thread(&job);
        const double send_us = job.send_s / iters * 1e6, recv_us = job.recv_s / iters * 1e6;
        /* both: count the work units finished while the communication thread runs */
        PMPI_Barrier(MPI_COMM_WORLD);
        job.send_s = job.recv_s = 0;
        g_comm_running = 1;
        pthread_t th;
        pthread_create(&th, NULL, comm_thread, &job);
        long units = 0;
        t0 = MPI_Wtime();
        while (g_comm_running) { work_unit(); ++units; }
        const double both_s = MPI_Wtime() - t0;
        pthread_join(th, NULL);
        const double psend_us = job.send_s / iters * 1e6, precv_us = job.recv_s / iters * 1e6;
        const double frac_s = (job.send_s + job.recv_s) > 0 ? job.send_s / (job.send_s + job.recv_s) : 0.5;
        const double cnt_s = units * frac_s / iters, cnt_r = units * (1 - frac_s) / iters;
        const double ideal = both_s * 1e6 / unit_us; /* units an undisturbed core would have done */
        const double cslow = ideal > 0 ? (1.0 - units / ideal) * 100.0 : 0.0;
        if (ctx.rank == 0)
            printf("%10zu %9.2f %9.2f %9.2f %9.2f %9.2f %8.1f %8.1f %7.1f %7.1f %7.1f %7.1f\n", msg, unit_us, send_us, recv_us, psend_us,
                   precv_us, cnt_s, cnt_r, cslow, cslow, send_us > 0 ? (psend_us / send_us - 1) * 100 : 0.0,
                   recv_us > 0 ? (precv_us / recv_us - 1) * 100 : 0.0);
        PMPI_Barrier(MPI_COMM_WORLD);
    }
    free(job.sbuf);
    free(job.rbuf);
    mpi_test_fini(&ctx);
    return 0;
}
