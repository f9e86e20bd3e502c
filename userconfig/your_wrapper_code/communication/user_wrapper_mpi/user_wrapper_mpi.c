/* Starting point for your own MPI communication wrapper (communication wrapper mode 3).
 *
 * Preloaded in front of libmpi, every MPI_Xxx defined here replaces the library's; the
 * library's own implementation stays reachable as PMPI_Xxx (the MPI profiling
 * interface), so no dlsym is needed. Each hook forwards unchanged: put your algorithm
 * between the markers, e.g. mpi_compress() from the selected compression wrapper, a
 * ring of PMPI_Sendrecv, mpi_decompress(). Same role as the reference's
 * userconfig/your_wrapper_code/communication/user_wrapper_mpi/user_wrapper_mpi.c:63-177.
 *
 * Build:  python3 -m ccbench_b200.cli build-wrappers   (or scripts/build_script.sh)  */
#include <mpi.h>
#include <stdio.h>
#include <stdlib.h>

static int verbose(void) {
    static int v = -1;
    if (v < 0) v = getenv("USER_WRAPPER_VERBOSE") ? atoi(getenv("USER_WRAPPER_VERBOSE")) : 0;
    return v;
}
#define NOTE(name, n) do { if (verbose()) fprintf(stderr, "[user_wrapper_mpi] %s count=%d\n", name, (int)(n)); } while (0)

int MPI_Allreduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype datatype, MPI_Op op, MPI_Comm comm) {
    NOTE("MPI_Allreduce", count);
    /* ---- your Allreduce starts here ---- */
    return PMPI_Allreduce(sendbuf, recvbuf, count, datatype, op, comm);
    /* ---- and ends here ---- */
}

int MPI_Reduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype datatype, MPI_Op op, int root, MPI_Comm comm) {
    NOTE("MPI_Reduce", count);
    return PMPI_Reduce(sendbuf, recvbuf, count, datatype, op, root, comm);
}

int MPI_Bcast(void *buffer, int count, MPI_Datatype datatype, int root, MPI_Comm comm) {
    NOTE("MPI_Bcast", count);
    return PMPI_Bcast(buffer, count, datatype, root, comm);
}

int MPI_Allgather(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf, int recvcount, MPI_Datatype recvtype,
                  MPI_Comm comm) {
    NOTE("MPI_Allgather", sendcount);
    return PMPI_Allgather(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, comm);
}

int MPI_Alltoall(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf, int recvcount, MPI_Datatype recvtype,
                 MPI_Comm comm) {
    NOTE("MPI_Alltoall", sendcount);
    return PMPI_Alltoall(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, comm);
}

int MPI_Reduce_scatter_block(const void *sendbuf, void *recvbuf, int recvcount, MPI_Datatype datatype, MPI_Op op, MPI_Comm comm) {
    NOTE("MPI_Reduce_scatter_block", recvcount);
    return PMPI_Reduce_scatter_block(sendbuf, recvbuf, recvcount, datatype, op, comm);
}
