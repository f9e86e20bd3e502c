/* The library UNDER the preload chain: base_ncclXxx call the real NCCL that findso recorded in
 * bin/libs/base_so_name, whatever is interposed in front of it. A wrapper uses them when it
 * needs the untouched collective (an oracle, a fallback) and RTLD_NEXT would land in another
 * wrapper. Same names and behaviour as the reference's loader
 * (run_codes/benchmark-core/include/rccl/rccl_base.h, src/rccl/get_base_implementation.c:61-167),
 * which exists there for RCCL only; on this hardware the recorded library is NCCL.
 *
 * NCCL forks that hand out a wrapped ncclComm_t: register the real communicator once with
 * base_nccl_set_comm() and every base_ call uses it instead of the caller's. */
#ifndef CCB_NCCL_BASE_H
#define CCB_NCCL_BASE_H

#include <cuda_runtime.h>
#include <nccl.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opens the library named in `state_path` (default: $BENCH_DIR/bin/libs/base_so_name, then
 * bin/libs/base_so_name) and resolves the seven entry points. 0 on success; -1 and a line on
 * stderr otherwise. Called lazily by the first base_ call when not called before. */
int load_base_impl(const char *state_path);
void base_nccl_set_comm(ncclComm_t comm);

ncclResult_t base_ncclAllReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                                ncclComm_t comm, cudaStream_t stream);
ncclResult_t base_ncclBroadcast(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, int root,
                                ncclComm_t comm, cudaStream_t stream);
ncclResult_t base_ncclReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root,
                             ncclComm_t comm, cudaStream_t stream);
ncclResult_t base_ncclAllGather(const void *sendbuff, void *recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm,
                                cudaStream_t stream);
ncclResult_t base_ncclReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount, ncclDataType_t datatype,
                                    ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t base_ncclSend(const void *sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm,
                           cudaStream_t stream);
ncclResult_t base_ncclRecv(void *recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CCB_NCCL_BASE_H */
