/* MPI Bcast benchmark (reference: run_codes/benchmarks/mpi/bcast/bcast.c). */
#include "mpi_runner.h"
static void sizes(size_t c, size_t e, int n, mpi_sizes_t *o) { (void)n; o->send_bytes = o->recv_bytes = c * e; }
static int call(const mpi_test_context_t *x, int pm, void *s, void *r, int c, MPI_Datatype dt) {
    (void)x; (void)r;
    return pm ? PMPI_Bcast(s, c, dt, 0, MPI_COMM_WORLD) : MPI_Bcast(s, c, dt, 0, MPI_COMM_WORLD);
}
static double bw(size_t b, const mpi_sizes_t *z, int n, double t) { (void)z; (void)n; return (double)b / t; }
static const mpi_bench_op_t op = {"MPI_Bcast", "bcast", sizes, call, bw, mbus_one, -1, 0, -2, 1};
int main(int argc, char **argv) { MPI_BENCH_UNUSED; return mpi_bench_main(argc, argv, &op); }
