/* Collectives that NCCL does not offer, with the reference's signatures
 * (run_codes/wrappers/include/nccl/nccl_extensions.h): Scatter, Gather, AllGatherv,
 * Scatterv and AllToAll. They return 0 on success and 1 on failure (not a
 * ncclResult_t). libnccl_extensions.so builds them from grouped ncclSend/ncclRecv;
 * the fused interposer (libccb_nccl.so) overrides them with single-kernel versions
 * when it is preloaded first. `ncclAlltoAll` is exported as an alias of ncclAllToAll. */
#ifndef NCCL_EXTENSIONS_H
#define NCCL_EXTENSIONS_H

#include <cuda_runtime.h>
#include <nccl.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

int ncclScatter(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
                ncclDataType_t recvtype, int root, ncclComm_t comm, cudaStream_t stream);
int ncclGather(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
               ncclDataType_t recvtype, int root, ncclComm_t comm, cudaStream_t stream);
int ncclAllGatherv(const void *sendbuf, int sendcount, ncclDataType_t sendtype, void *recvbuf,
                   const int recvcounts[], const int displs[], ncclDataType_t recvtype, const int *d_recvcounts,
                   const int *d_displs, ncclComm_t comm, cudaStream_t stream);
int ncclScatterv(const void *sendbuf, const int sendcounts[], const int displs[], ncclDataType_t sendtype,
                 void *recvbuf, int recvcount, ncclDataType_t recvtype, int root, const int *d_sendcounts,
                 const int *d_displs, ncclComm_t comm, cudaStream_t stream);
int ncclAllToAll(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
                 ncclDataType_t recvtype, ncclComm_t comm, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* NCCL_EXTENSIONS_H */
