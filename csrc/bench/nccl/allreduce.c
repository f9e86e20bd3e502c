/* ncclAllReduce(sum) benchmark. Reference: run_codes/benchmarks/nccl/allreduce/
 * allreduce.c (bandwidth printed as 2 * bytes / t, :139-146). */
#include "bench_runner.h"
static void sizes(size_t c, size_t e, int n, bench_sizes_t *o) { (void)n; o->count = c; o->send_bytes = o->recv_bytes = c * e; }
static int call(const nccl_test_context_t *x, const void *s, void *r, size_t c, ncclDataType_t dt) {
    return ncclAllReduce(s, r, c, dt, ncclSum, x->comm, x->stream) != ncclSuccess;
}
static void oracle(const nccl_test_context_t *x, void *ref, size_t c, data_type_t dt) {
    dummy_allreduce(ref, x->config.input_file, dt, x->config.pattern_type, (int)c, x->size);
}
static double bw(size_t b, const bench_sizes_t *z, int n, double t) { (void)z; (void)n; return 2.0 * (double)b / t; }
static const bench_op_t op = {"NCCL_AllReduce", "allreduce", 2, sizes, call, oracle, bw, bus_allreduce, -1, 0, 0, 0};
int main(int argc, char **argv) { (void)bus_nminus1_over_n; (void)bus_one; return bench_main(argc, argv, &op); }
