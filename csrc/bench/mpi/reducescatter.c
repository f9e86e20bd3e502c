/* MPI_Reduce_scatter benchmark with per-rank receive counts (all equal to the message
 * here; reference: run_codes/benchmarks/mpi/reducescatter/reducescatter.c:27-57). */
#include "mpi_runner.h"
static void sizes(size_t c, size_t e, int n, mpi_sizes_t *o) { o->send_bytes = c * e * (size_t)n; o->recv_bytes = c * e; }
static int call(const mpi_test_context_t *x, int pm, void *s, void *r, int c, MPI_Datatype dt) {
    int counts[64];
    for (int i = 0; i < x->size && i < 64; ++i) counts[i] = c;
    return pm ? PMPI_Reduce_scatter(s, r, counts, dt, MPI_SUM, MPI_COMM_WORLD) : MPI_Reduce_scatter(s, r, counts, dt, MPI_SUM, MPI_COMM_WORLD);
}
static double bw(size_t b, const mpi_sizes_t *z, int n, double t) { (void)b; (void)n; return (double)z->recv_bytes / t; }
static double bus(int n) { return n > 1 ? (double)(n - 1) : 1.0; }
static const mpi_bench_op_t op = {"MPI_Reduce_scatter", "reducescatter", sizes, call, bw, bus, -1, 1, 0, 0};
int main(int argc, char **argv) { MPI_BENCH_UNUSED; return mpi_bench_main(argc, argv, &op); }
