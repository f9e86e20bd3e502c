/* Host-codec send/receive helpers for NCCL wrappers, with the reference's API
 * (run_codes/wrappers/nccl_compress_tools.h). A wrapper provides strong
 * nccl_compress / nccl_decompress (host buffers); the weak defaults are the identity.
 * Wire: [u64 compressed_size | payload | zero pad], always nccl_max_wire_size(n)
 * bytes so both sides post equal counts without a size hand-shake. Here
 * nccl_send_compressed / nccl_recv_decompress / nccl_exchange_compressed are weak
 * too, so a wrapper can replace the transport as well as the codec.
 * `buf`, `sendbuf` and `recvbuf` are CPU (host) buffers, as in the reference; device or
 * managed pointers are accepted as well and staged through pinned host memory. */
#ifndef NCCL_COMPRESS_TOOLS_H
#define NCCL_COMPRESS_TOOLS_H

#include <cuda_runtime.h>
#include <nccl.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

size_t nccl_type_size(ncclDataType_t dtype);
static inline size_t nccl_min_sz(size_t a, size_t b) { return a < b ? a : b; }
static inline size_t nccl_max_wire_size(size_t data_bytes) { return data_bytes + sizeof(uint64_t) + 64 + data_bytes / 16; }

int nccl_compress(void *input, size_t input_size, void *output, size_t *output_size);
int nccl_decompress(void *input, size_t input_size, void *output, size_t output_size);
int compression_enabled(void);

int nccl_send_compressed(const void *buf, size_t data_bytes, int peer, ncclComm_t comm, cudaStream_t stream);
int nccl_recv_decompress(void *buf, size_t data_bytes, int peer, ncclComm_t comm, cudaStream_t stream);
int nccl_exchange_compressed(const void *sendbuf, size_t send_bytes, void *recvbuf, size_t recv_bytes, int dst, int src,
                             ncclComm_t comm, cudaStream_t stream);
int nccl_reduce_cpu(void *dst, const void *src, size_t count, ncclDataType_t dtype, ncclRedOp_t op);

#ifdef __cplusplus
}
#endif
#endif /* NCCL_COMPRESS_TOOLS_H */
