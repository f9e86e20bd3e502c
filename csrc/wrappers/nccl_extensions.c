/* libnccl_extensions.so: Scatter, Gather, AllGatherv, Scatterv and AllToAll on top of
 * ncclSend / ncclRecv. The reference issues them as sequential, mostly un-grouped
 * byte-typed sends and receives (run_codes/wrappers/src/nccl/nccl_extensions.c:
 * 28-250); here every collective is ONE ncclGroupStart/End, so NCCL schedules all
 * peers at once over NVSwitch. Symbols are resolved through the dynamic linker at
 * call time, so a preloaded interposer that wraps ncclSend/ncclRecv/ncclCommUserRank
 * is honoured; the calls carry the caller's element type and count (not bytes), so that
 * such an interposer can tell floating-point payloads from the rest. */
#include <stdint.h>
#include <string.h>

#include "nccl/nccl_extensions.h"

static size_t esize(ncclDataType_t t) {
    switch (t) {
        case ncclInt8: case ncclUint8: return 1;
        case ncclFloat16: return 2;
        case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
        case ncclInt64: case ncclUint64: case ncclFloat64: return 8;
        default: return 2; /* bf16 and fp8 variants: 2 or 1; callers of these use the sizes above */
    }
}

#define TRY(x)                      \
    do {                            \
        if ((x) != ncclSuccess) {   \
            ncclGroupEnd();         \
            return 1;               \
        }                           \
    } while (0)

static int rank_size(ncclComm_t comm, int *rank, int *n) {
    return ncclCommUserRank(comm, rank) != ncclSuccess || ncclCommCount(comm, n) != ncclSuccess;
}

int ncclScatter(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
                ncclDataType_t recvtype, int root, ncclComm_t comm, cudaStream_t stream) {
    int rank, n;
    if (rank_size(comm, &rank, &n)) return 1;
    const size_t sb = sendcount * esize(sendtype), rb = recvcount * esize(recvtype);
    if (ncclGroupStart() != ncclSuccess) return 1;
    if (rank == root) {
        for (int p = 0; p < n; ++p) {
            const char *src = (const char *)sendbuf + (size_t)p * sb;
            if (p == root) {
                if (cudaMemcpyAsync(recvbuf, src, rb < sb ? rb : sb, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
                    ncclGroupEnd();
                    return 1;
                }
            } else {
                TRY(ncclSend(src, sendcount, sendtype, p, comm, stream));
            }
        }
    } else {
        TRY(ncclRecv(recvbuf, recvcount, recvtype, root, comm, stream));
    }
    return ncclGroupEnd() != ncclSuccess;
}

int ncclGather(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
               ncclDataType_t recvtype, int root, ncclComm_t comm, cudaStream_t stream) {
    int rank, n;
    if (rank_size(comm, &rank, &n)) return 1;
    const size_t sb = sendcount * esize(sendtype), rb = recvcount * esize(recvtype);
    if (ncclGroupStart() != ncclSuccess) return 1;
    if (rank == root) {
        for (int p = 0; p < n; ++p) {
            char *dst = (char *)recvbuf + (size_t)p * rb;
            if (p == root) {
                if (cudaMemcpyAsync(dst, sendbuf, sb < rb ? sb : rb, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
                    ncclGroupEnd();
                    return 1;
                }
            } else {
                TRY(ncclRecv(dst, recvcount, recvtype, p, comm, stream));
            }
        }
    } else {
        TRY(ncclSend(sendbuf, sendcount, sendtype, root, comm, stream));
    }
    return ncclGroupEnd() != ncclSuccess;
}

int ncclAllGatherv(const void *sendbuf, int sendcount, ncclDataType_t sendtype, void *recvbuf,
                   const int recvcounts[], const int displs[], ncclDataType_t recvtype, const int *d_recvcounts,
                   const int *d_displs, ncclComm_t comm, cudaStream_t stream) {
    (void)d_recvcounts;
    (void)d_displs;
    int rank, n;
    if (rank_size(comm, &rank, &n)) return 1;
    const size_t se = esize(sendtype), re = esize(recvtype);
    if (ncclGroupStart() != ncclSuccess) return 1;
    for (int p = 0; p < n; ++p) {
        char *dst = (char *)recvbuf + (size_t)displs[p] * re;
        if (p == rank) {
            if (cudaMemcpyAsync(dst, sendbuf, (size_t)sendcount * se, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
                ncclGroupEnd();
                return 1;
            }
            continue;
        }
        TRY(ncclSend(sendbuf, (size_t)sendcount, sendtype, p, comm, stream));
        TRY(ncclRecv(dst, (size_t)recvcounts[p], recvtype, p, comm, stream));
    }
    return ncclGroupEnd() != ncclSuccess;
}

int ncclScatterv(const void *sendbuf, const int sendcounts[], const int displs[], ncclDataType_t sendtype,
                 void *recvbuf, int recvcount, ncclDataType_t recvtype, int root, const int *d_sendcounts,
                 const int *d_displs, ncclComm_t comm, cudaStream_t stream) {
    (void)d_sendcounts;
    (void)d_displs;
    int rank, n;
    if (rank_size(comm, &rank, &n)) return 1;
    const size_t se = esize(sendtype);
    if (ncclGroupStart() != ncclSuccess) return 1;
    if (rank == root) {
        for (int p = 0; p < n; ++p) {
            const char *src = (const char *)sendbuf + (size_t)displs[p] * se;
            const size_t bytes = (size_t)sendcounts[p] * se;
            if (p == root) {
                if (cudaMemcpyAsync(recvbuf, src, bytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
                    ncclGroupEnd();
                    return 1;
                }
            } else if (bytes) {
                TRY(ncclSend(src, (size_t)sendcounts[p], sendtype, p, comm, stream));
            }
        }
    } else if (recvcount > 0) {
        TRY(ncclRecv(recvbuf, (size_t)recvcount, recvtype, root, comm, stream));
    }
    return ncclGroupEnd() != ncclSuccess;
}

int ncclAllToAll(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
                 ncclDataType_t recvtype, ncclComm_t comm, cudaStream_t stream) {
    int rank, n;
    if (rank_size(comm, &rank, &n)) return 1;
    const size_t sb = sendcount * esize(sendtype), rb = recvcount * esize(recvtype);
    if (ncclGroupStart() != ncclSuccess) return 1;
    for (int j = 0; j < n; ++j) {
        const int p = (rank + j) % n;
        const char *src = (const char *)sendbuf + (size_t)p * sb;
        char *dst = (char *)recvbuf + (size_t)p * rb;
        if (p == rank) {
            if (cudaMemcpyAsync(dst, src, sb < rb ? sb : rb, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
                ncclGroupEnd();
                return 1;
            }
            continue;
        }
        TRY(ncclSend(src, sendcount, sendtype, p, comm, stream));
        TRY(ncclRecv(dst, recvcount, recvtype, p, comm, stream));
    }
    return ncclGroupEnd() != ncclSuccess;
}

/* NCCL >= 2.28 has its own ncclAlltoAll (lower-case t) with a different signature;
 * this library does not define that name. */
