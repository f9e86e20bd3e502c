/* perfmpi: LD_PRELOAD perf wrapper for the MPI path (first in LD_PRELOAD). Times each
 * intercepted call on the host and notes a row; offers buffers to the gendata capture.
 * Columns as the reference's userconfig/wrapper_code_examples/perf/perfmpi/perfmpi.c:
 * point-to-point -> duration, msg_bytes, intra (:62-161); MPI_Allreduce / MPI_Allgather
 * (and here also Bcast, Reduce, Alltoall, Reduce_scatter) -> duration, data_bytes
 * (:168-218); mpi_compress -> duration, input_size, output_size, compression_ratio
 * (input / output) and mpi_decompress (:221-262). Collectives capture the RECEIVE
 * buffer after the call, sends the send buffer. */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stddef.h>

#include "mpi/perf_helper_mpi.h"

#define ROW(name, t0, ...)                                                        \
    do {                                                                          \
        perf_attr_t a_[] = {__VA_ARGS__};                                         \
        perf_mpi_world_rank();                                                    \
        perf_notedown(perf_mpi_get_tls(), name, t0, (int)(sizeof(a_) / sizeof(a_[0])), a_); \
    } while (0)

int MPI_Send(const void *buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm) {
    const double t0 = perf_get_time();
    int r = PMPI_Send(buf, count, dt, dest, tag, comm);
    ROW("MPI_Send", t0, {"duration", perf_get_time() - t0}, {"msg_bytes", perf_mpi_msg_size(count, dt)}, {"intra", perf_mpi_is_intra(dest)});
    perf_gendata_dump_if_target(perf_mpi_get_tls(), "MPI_Send", buf, (size_t)perf_mpi_msg_size(count, dt));
    return r;
}
int MPI_Recv(void *buf, int count, MPI_Datatype dt, int src, int tag, MPI_Comm comm, MPI_Status *st) {
    const double t0 = perf_get_time();
    int r = PMPI_Recv(buf, count, dt, src, tag, comm, st);
    ROW("MPI_Recv", t0, {"duration", perf_get_time() - t0}, {"msg_bytes", perf_mpi_msg_size(count, dt)}, {"intra", src >= 0 ? perf_mpi_is_intra(src) : 1});
    return r;
}
int MPI_Isend(const void *buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request *req) {
    const double t0 = perf_get_time();
    int r = PMPI_Isend(buf, count, dt, dest, tag, comm, req);
    ROW("MPI_Isend", t0, {"duration", perf_get_time() - t0}, {"msg_bytes", perf_mpi_msg_size(count, dt)}, {"intra", perf_mpi_is_intra(dest)});
    perf_gendata_dump_if_target(perf_mpi_get_tls(), "MPI_Isend", buf, (size_t)perf_mpi_msg_size(count, dt));
    return r;
}
int MPI_Irecv(void *buf, int count, MPI_Datatype dt, int src, int tag, MPI_Comm comm, MPI_Request *req) {
    const double t0 = perf_get_time();
    int r = PMPI_Irecv(buf, count, dt, src, tag, comm, req);
    ROW("MPI_Irecv", t0, {"duration", perf_get_time() - t0}, {"msg_bytes", perf_mpi_msg_size(count, dt)}, {"intra", src >= 0 ? perf_mpi_is_intra(src) : 1});
    return r;
}

/* Collectives go to the NEXT definition in the preload chain (a communication wrapper
 * if there is one, else the MPI library), so that this wrapper composes with it. */
#define NEXT(name) ((__typeof__(&name))dlsym(RTLD_NEXT, #name))

int MPI_Allreduce(const void *s, void *r, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm) {
    static __typeof__(&MPI_Allreduce) next;
    if (!next) next = NEXT(MPI_Allreduce);
    const double t0 = perf_get_time();
    int rc = next ? next(s, r, count, dt, op, comm) : PMPI_Allreduce(s, r, count, dt, op, comm);
    ROW("MPI_Allreduce", t0, {"duration", perf_get_time() - t0}, {"data_bytes", perf_mpi_msg_size(count, dt)});
    perf_gendata_dump_if_target(perf_mpi_get_tls(), "MPI_Allreduce", r, (size_t)perf_mpi_msg_size(count, dt));
    return rc;
}
int MPI_Allgather(const void *s, int sc, MPI_Datatype sdt, void *r, int rc_, MPI_Datatype rdt, MPI_Comm comm) {
    static __typeof__(&MPI_Allgather) next;
    if (!next) next = NEXT(MPI_Allgather);
    int n = 1;
    PMPI_Comm_size(comm, &n);
    const double t0 = perf_get_time();
    int rc = next ? next(s, sc, sdt, r, rc_, rdt, comm) : PMPI_Allgather(s, sc, sdt, r, rc_, rdt, comm);
    ROW("MPI_Allgather", t0, {"duration", perf_get_time() - t0}, {"data_bytes", perf_mpi_msg_size(sc, sdt)});
    perf_gendata_dump_if_target(perf_mpi_get_tls(), "MPI_Allgather", r, (size_t)perf_mpi_msg_size(rc_, rdt) * (size_t)n);
    return rc;
}
int MPI_Bcast(void *buf, int count, MPI_Datatype dt, int root, MPI_Comm comm) {
    static __typeof__(&MPI_Bcast) next;
    if (!next) next = NEXT(MPI_Bcast);
    const double t0 = perf_get_time();
    int rc = next ? next(buf, count, dt, root, comm) : PMPI_Bcast(buf, count, dt, root, comm);
    ROW("MPI_Bcast", t0, {"duration", perf_get_time() - t0}, {"data_bytes", perf_mpi_msg_size(count, dt)});
    perf_gendata_dump_if_target(perf_mpi_get_tls(), "MPI_Bcast", buf, (size_t)perf_mpi_msg_size(count, dt));
    return rc;
}
int MPI_Reduce(const void *s, void *r, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm) {
    static __typeof__(&MPI_Reduce) next;
    if (!next) next = NEXT(MPI_Reduce);
    const double t0 = perf_get_time();
    int rc = next ? next(s, r, count, dt, op, root, comm) : PMPI_Reduce(s, r, count, dt, op, root, comm);
    ROW("MPI_Reduce", t0, {"duration", perf_get_time() - t0}, {"data_bytes", perf_mpi_msg_size(count, dt)});
    return rc;
}
int MPI_Alltoall(const void *s, int sc, MPI_Datatype sdt, void *r, int rc_, MPI_Datatype rdt, MPI_Comm comm) {
    static __typeof__(&MPI_Alltoall) next;
    if (!next) next = NEXT(MPI_Alltoall);
    const double t0 = perf_get_time();
    int rc = next ? next(s, sc, sdt, r, rc_, rdt, comm) : PMPI_Alltoall(s, sc, sdt, r, rc_, rdt, comm);
    ROW("MPI_Alltoall", t0, {"duration", perf_get_time() - t0}, {"data_bytes", perf_mpi_msg_size(sc, sdt)});
    return rc;
}
int MPI_Reduce_scatter(const void *s, void *r, const int rcs[], MPI_Datatype dt, MPI_Op op, MPI_Comm comm) {
    static __typeof__(&MPI_Reduce_scatter) next;
    if (!next) next = NEXT(MPI_Reduce_scatter);
    int rank = 0;
    PMPI_Comm_rank(comm, &rank);
    const double t0 = perf_get_time();
    int rc = next ? next(s, r, rcs, dt, op, comm) : PMPI_Reduce_scatter(s, r, rcs, dt, op, comm);
    ROW("MPI_Reduce_scatter", t0, {"duration", perf_get_time() - t0}, {"data_bytes", perf_mpi_msg_size(rcs[rank], dt)});
    return rc;
}

/* codec hooks: time the next definition (the compression wrapper's, or the weak identity) */
int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size) {
    static int (*next)(void *, size_t, void *, size_t *);
    if (!next) next = (int (*)(void *, size_t, void *, size_t *))dlsym(RTLD_NEXT, "mpi_compress");
    if (!next) return 1;
    const double t0 = perf_get_time();
    int rc = next(input, input_size, output, output_size);
    ROW("mpi_compress", t0, {"duration", perf_get_time() - t0}, {"input_size", (double)input_size}, {"output_size", (double)*output_size},
        {"compression_ratio", *output_size ? (double)input_size / (double)*output_size : 0.0});
    return rc;
}
int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    static int (*next)(void *, size_t, void *, size_t);
    if (!next) next = (int (*)(void *, size_t, void *, size_t))dlsym(RTLD_NEXT, "mpi_decompress");
    if (!next) return 1;
    const double t0 = perf_get_time();
    int rc = next(input, input_size, output, output_size);
    ROW("mpi_decompress", t0, {"duration", perf_get_time() - t0}, {"input_size", (double)input_size}, {"output_size", (double)output_size});
    return rc;
}
