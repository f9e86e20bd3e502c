/* MPI_Allgatherv benchmark; shares weighted by $ALLGATHERV_WEIGHTS (reference:
 * run_codes/benchmarks/mpi/allgatherv/allgatherv.c). The message size is the TOTAL
 * gathered size; the reference result is PMPI_Allgatherv on the same input. */
#include "mpi_runner.h"
static int g_counts[64], g_displs[64], g_ready;
static void split(int n, int total) {
    int nw = 0;
    int *w = parse_env_int_array("ALLGATHERV_WEIGHTS", n, &nw);
    long ws = 0;
    for (int i = 0; w && i < n; ++i) ws += w[i];
    int off = 0;
    for (int i = 0; i < n; ++i) {
        long c = (w && ws > 0) ? (long)w[i] * total / ws : total / n;
        g_counts[i] = c < 1 ? 1 : (int)c;
        g_displs[i] = off;
        off += g_counts[i];
    }
    free(w);
    g_ready = off;
}
static void sizes(size_t c, size_t e, int n, mpi_sizes_t *o) { split(n, (int)c < n ? n : (int)c); o->send_bytes = o->recv_bytes = (size_t)g_ready * e; }
static int call(const mpi_test_context_t *x, int pm, void *s, void *r, int c, MPI_Datatype dt) {
    (void)c;
    return pm ? PMPI_Allgatherv(s, g_counts[x->rank], dt, r, g_counts, g_displs, dt, MPI_COMM_WORLD)
              : MPI_Allgatherv(s, g_counts[x->rank], dt, r, g_counts, g_displs, dt, MPI_COMM_WORLD);
}
static double bw(size_t b, const mpi_sizes_t *z, int n, double t) { (void)b; (void)n; return (double)z->recv_bytes / t; }
static const mpi_bench_op_t op = {"MPI_Allgatherv", "allgatherv", sizes, call, bw, mbus_frac, -1, 0, 0, 0};
int main(int argc, char **argv) { MPI_BENCH_UNUSED; return mpi_bench_main(argc, argv, &op); }
