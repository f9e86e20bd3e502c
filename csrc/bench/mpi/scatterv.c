/* MPI_Scatterv benchmark from root 0; shares weighted by $SCATTERV_WEIGHTS (reference:
 * run_codes/benchmarks/mpi/scatterv/scatterv.c). */
#include "mpi_runner.h"
static int g_counts[64], g_displs[64], g_total, g_max;
static void split(int n, int total) {
    int nw = 0;
    int *w = parse_env_int_array("SCATTERV_WEIGHTS", n, &nw);
    long ws = 0;
    for (int i = 0; w && i < n; ++i) ws += w[i];
    int off = 0;
    g_max = 0;
    for (int i = 0; i < n; ++i) {
        long c = (w && ws > 0) ? (long)w[i] * total / ws : total / n;
        g_counts[i] = c < 1 ? 1 : (int)c;
        g_displs[i] = off;
        off += g_counts[i];
        if (g_counts[i] > g_max) g_max = g_counts[i];
    }
    free(w);
    g_total = off;
}
static int g_rank_hint;
static void sizes(size_t c, size_t e, int n, mpi_sizes_t *o) { split(n, (int)c < n ? n : (int)c); o->send_bytes = (size_t)g_total * e; o->recv_bytes = (size_t)g_counts[g_rank_hint] * e; }
static int call(const mpi_test_context_t *x, int pm, void *s, void *r, int c, MPI_Datatype dt) {
    (void)c;
    return pm ? PMPI_Scatterv(s, g_counts, g_displs, dt, r, g_counts[x->rank], dt, 0, MPI_COMM_WORLD)
              : MPI_Scatterv(s, g_counts, g_displs, dt, r, g_counts[x->rank], dt, 0, MPI_COMM_WORLD);
}
static double bw(size_t b, const mpi_sizes_t *z, int n, double t) { (void)b; (void)n; return (double)z->recv_bytes / t; }
static const mpi_bench_op_t op = {"MPI_Scatterv", "scatterv", sizes, call, bw, mbus_one, -1, 0, 0, 0};
int main(int argc, char **argv) {
    MPI_BENCH_UNUSED;
    const char *r = getenv("OMPI_COMM_WORLD_RANK");
    g_rank_hint = r ? atoi(r) : 0;
    return mpi_bench_main(argc, argv, &op);
}
