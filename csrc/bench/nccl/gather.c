/* Gather to root 0 through the ncclGather extension; `msg` bytes per rank. Reference:
 * run_codes/benchmarks/nccl/gather/gather.c (bandwidth msg / t, :147-149). */
#include "bench_runner.h"
static void sizes(size_t c, size_t e, int n, bench_sizes_t *o) { o->count = c; o->send_bytes = c * e; o->recv_bytes = c * e * (size_t)n; }
static int call(const nccl_test_context_t *x, const void *s, void *r, size_t c, ncclDataType_t dt) {
    return ncclGather(s, c, dt, r, c, dt, 0, x->comm, x->stream);
}
static void oracle(const nccl_test_context_t *x, void *ref, size_t c, data_type_t dt) {
    dummy_gather(ref, x->config.input_file, dt, x->config.pattern_type, (int)c, x->size, 0);
}
static double bw(size_t b, const bench_sizes_t *z, int n, double t) { (void)z; (void)n; return (double)b / t; }
static const bench_op_t op = {"NCCL_Gather", "gather", 2, sizes, call, oracle, bw, bus_one, 0, 0, 0, 0};
int main(int argc, char **argv) { (void)bus_allreduce; (void)bus_nminus1_over_n; return bench_main(argc, argv, &op); }
