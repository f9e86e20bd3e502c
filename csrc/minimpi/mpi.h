/* ccb_minimpi: a single-host subset of MPI over Unix-domain sockets, for machines
 * that have no MPI installation. It exists so that the MPI side of this framework
 * (benchmark drivers, the MPI_* interposer, perf wrappers) can be built, run and
 * tested anywhere; with a real MPI present, mpicc and its mpi.h are used instead and
 * nothing of this directory is involved. Every MPI_X is a weak alias of PMPI_X, as in
 * a real MPI library, so LD_PRELOAD wrappers that define MPI_X and call PMPI_X work
 * unchanged. Ranks come from OMPI_COMM_WORLD_RANK / _SIZE (python -m
 * ccbench_b200.launch sets them). Only MPI_COMM_WORLD and contiguous basic types. */
#ifndef CCB_MINIMPI_H
#define CCB_MINIMPI_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CCB_MINIMPI 1
typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef struct ccb_mpi_request *MPI_Request;
typedef long MPI_Aint;
typedef struct { int MPI_SOURCE, MPI_TAG, MPI_ERROR; size_t ccb_bytes; } MPI_Status;

#define MPI_COMM_WORLD 0
#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_ANY_SOURCE (-1)
#define MPI_ANY_TAG (-1)
#define MPI_STATUS_IGNORE ((MPI_Status *)0)
#define MPI_STATUSES_IGNORE ((MPI_Status *)0)
#define MPI_REQUEST_NULL ((MPI_Request)0)
#define MPI_IN_PLACE ((void *)-1)
#define MPI_MAX_PROCESSOR_NAME 256
#define MPI_THREAD_SINGLE 0
#define MPI_THREAD_FUNNELED 1
#define MPI_THREAD_SERIALIZED 2
#define MPI_THREAD_MULTIPLE 3

enum { MPI_CHAR = 1, MPI_BYTE, MPI_INT, MPI_FLOAT, MPI_DOUBLE, MPI_LONG, MPI_UNSIGNED_CHAR, MPI_INT8_T, MPI_UINT8_T,
       MPI_INT32_T, MPI_INT64_T, MPI_UINT64_T, MPI_UNSIGNED, MPI_LONG_LONG };
enum { MPI_SUM = 1, MPI_PROD, MPI_MAX, MPI_MIN };

#define CCB_MPI_DECL(ret, name, args) ret MPI_##name args; ret PMPI_##name args;
CCB_MPI_DECL(int, Init, (int *argc, char ***argv))
CCB_MPI_DECL(int, Init_thread, (int *argc, char ***argv, int required, int *provided))
CCB_MPI_DECL(int, Initialized, (int *flag))
CCB_MPI_DECL(int, Finalize, (void))
CCB_MPI_DECL(int, Abort, (MPI_Comm comm, int code))
CCB_MPI_DECL(int, Comm_rank, (MPI_Comm comm, int *rank))
CCB_MPI_DECL(int, Comm_size, (MPI_Comm comm, int *size))
CCB_MPI_DECL(int, Get_processor_name, (char *name, int *len))
CCB_MPI_DECL(double, Wtime, (void))
CCB_MPI_DECL(int, Type_size, (MPI_Datatype dt, int *size))
CCB_MPI_DECL(int, Barrier, (MPI_Comm comm))
CCB_MPI_DECL(int, Send, (const void *buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm))
CCB_MPI_DECL(int, Recv, (void *buf, int count, MPI_Datatype dt, int src, int tag, MPI_Comm comm, MPI_Status *st))
CCB_MPI_DECL(int, Isend, (const void *buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request *req))
CCB_MPI_DECL(int, Irecv, (void *buf, int count, MPI_Datatype dt, int src, int tag, MPI_Comm comm, MPI_Request *req))
CCB_MPI_DECL(int, Wait, (MPI_Request *req, MPI_Status *st))
CCB_MPI_DECL(int, Waitall, (int n, MPI_Request reqs[], MPI_Status sts[]))
CCB_MPI_DECL(int, Test, (MPI_Request *req, int *flag, MPI_Status *st))
CCB_MPI_DECL(int, Probe, (int src, int tag, MPI_Comm comm, MPI_Status *st))
CCB_MPI_DECL(int, Iprobe, (int src, int tag, MPI_Comm comm, int *flag, MPI_Status *st))
CCB_MPI_DECL(int, Get_count, (const MPI_Status *st, MPI_Datatype dt, int *count))
CCB_MPI_DECL(int, Sendrecv, (const void *sbuf, int scount, MPI_Datatype sdt, int dest, int stag, void *rbuf, int rcount,
                             MPI_Datatype rdt, int src, int rtag, MPI_Comm comm, MPI_Status *st))
CCB_MPI_DECL(int, Reduce_local, (const void *in, void *inout, int count, MPI_Datatype dt, MPI_Op op))
CCB_MPI_DECL(int, Bcast, (void *buf, int count, MPI_Datatype dt, int root, MPI_Comm comm))
CCB_MPI_DECL(int, Reduce, (const void *s, void *r, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm))
CCB_MPI_DECL(int, Allreduce, (const void *s, void *r, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm))
CCB_MPI_DECL(int, Gather, (const void *s, int sc, MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, int root, MPI_Comm comm))
CCB_MPI_DECL(int, Gatherv, (const void *s, int sc, MPI_Datatype sdt, void *r, const int rcs[], const int displs[], MPI_Datatype rdt, int root, MPI_Comm comm))
CCB_MPI_DECL(int, Scatter, (const void *s, int sc, MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, int root, MPI_Comm comm))
CCB_MPI_DECL(int, Scatterv, (const void *s, const int scs[], const int displs[], MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, int root, MPI_Comm comm))
CCB_MPI_DECL(int, Allgather, (const void *s, int sc, MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, MPI_Comm comm))
CCB_MPI_DECL(int, Allgatherv, (const void *s, int sc, MPI_Datatype sdt, void *r, const int rcs[], const int displs[], MPI_Datatype rdt, MPI_Comm comm))
CCB_MPI_DECL(int, Alltoall, (const void *s, int sc, MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, MPI_Comm comm))
CCB_MPI_DECL(int, Reduce_scatter_block, (const void *s, void *r, int rc, MPI_Datatype dt, MPI_Op op, MPI_Comm comm))
CCB_MPI_DECL(int, Reduce_scatter, (const void *s, void *r, const int rcs[], MPI_Datatype dt, MPI_Op op, MPI_Comm comm))
#undef CCB_MPI_DECL

#ifdef __cplusplus
}
#endif
#endif
