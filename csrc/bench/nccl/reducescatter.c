/* ncclReduceScatter(sum): every rank receives `msg` bytes, sends n times that.
 * Reference: run_codes/benchmarks/nccl/reducescatter/reducescatter.c (bandwidth
 * recv_bytes / t, :140-142; every rank dumps its chunk). */
#include "bench_runner.h"
static void sizes(size_t c, size_t e, int n, bench_sizes_t *o) { o->count = c; o->send_bytes = c * e * (size_t)n; o->recv_bytes = c * e; }
static int call(const nccl_test_context_t *x, const void *s, void *r, size_t c, ncclDataType_t dt) {
    return ncclReduceScatter(s, r, c, dt, ncclSum, x->comm, x->stream) != ncclSuccess;
}
static void oracle(const nccl_test_context_t *x, void *ref, size_t c, data_type_t dt) {
    dummy_reduce_scatter(ref, x->config.input_file, dt, x->config.pattern_type, (int)c, x->size, x->rank);
}
static double bw(size_t b, const bench_sizes_t *z, int n, double t) { (void)b; (void)n; return (double)z->recv_bytes / t; }
static double bus(int n) { return n > 1 ? (double)(n - 1) : 1.0; } /* msg = recv bytes: algbw = n*msg/t, busbw = algbw*(n-1)/n */
static const bench_op_t op = {"NCCL_ReduceScatter", "reducescatter", 2, sizes, call, oracle, bw, bus, -1, 1, 0, 0};
int main(int argc, char **argv) { (void)bus_allreduce; (void)bus_nminus1_over_n; (void)bus_one; return bench_main(argc, argv, &op); }
