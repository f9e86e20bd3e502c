/* AllToAll benchmark through the ncclAllToAll extension: `msg` bytes per peer.
 * Reference: run_codes/benchmarks/nccl/alltoall/alltoall.c (bandwidth msg * (n-1) / t,
 * :149-151; every rank dumps its chunk). */
#include "bench_runner.h"
static void sizes(size_t c, size_t e, int n, bench_sizes_t *o) { o->count = c; o->send_bytes = o->recv_bytes = c * e * (size_t)n; }
static int call(const nccl_test_context_t *x, const void *s, void *r, size_t c, ncclDataType_t dt) {
    return ncclAllToAll(s, c, dt, r, c, dt, x->comm, x->stream);
}
static void oracle(const nccl_test_context_t *x, void *ref, size_t c, data_type_t dt) {
    dummy_alltoall(ref, x->config.input_file, dt, x->config.pattern_type, (int)c, x->size, x->rank);
}
static double bw(size_t b, const bench_sizes_t *z, int n, double t) { (void)z; return (double)b * (n - 1) / t; }
static const bench_op_t op = {"NCCL_AllToAll", "alltoall", 2, sizes, call, oracle, bw, bus_nminus1_over_n, -1, 1, 0, 0};
int main(int argc, char **argv) { (void)bus_allreduce; (void)bus_one; return bench_main(argc, argv, &op); }
