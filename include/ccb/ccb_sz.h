/* SZ-style error-bounded lossy codec for 3-D fp32 fields ("ccb-sz v2": pre-quantise
 * under an absolute bound, 3-D Lorenzo prediction on the integers inside 32x8x8
 * tiles, per-row bit-plane packing) and its fusion with AllGather / Broadcast.
 * Fields are [nz][ny][nx] with x fastest. The format and the kernels are described
 * in csrc/kernels/ccb_sz.cu. The reference reaches SZ3 only on the CPU through
 * dlopen (userconfig/wrapper_code_examples/compression/sz3/mpi_sz3_wrapper.c). */
#ifndef CCB_SZ_H
#define CCB_SZ_H

#include <stdint.h>

#include "ccb.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Bytes a compressed buffer must provide for an nx*ny*nz field (fixed-capacity group
 * slots; the bytes actually used are reported by ccb_sz_compress). */
uint64_t ccb_sz_capacity(int nx, int ny, int nz);
/* How the last collective launch of this process went: 0 = none yet, 1 = the driver took the
 * cluster and the cooperative attribute together, 2 = it refused the pair and the kernel was
 * launched with the cluster attribute alone (grid bounded by the resident-cluster count). */
int ccb_sz_launch_path(void);
/* |in - decompress(compress(in))| <= eb for every finite element. `d_used` (device
 * memory, optional) receives the number of compressed bytes produced. */
int ccb_sz_compress(const float* in, int nx, int ny, int nz, float eb, void* out, unsigned long long* d_used,
                    ccb_stream_t stream);
int ccb_sz_decompress(const void* in, int nx, int ny, int nz, float eb, float* out, ccb_stream_t stream);
/* root < 0: AllGather (recv holds nranks fields in rank order); root >= 0: Broadcast.
 * One fused kernel: compress, store into the peers' arenas, decode on arrival.
 * `d_used`: optional device counters, one per local rank, of the compressed bytes a
 * rank sent to one destination. */
int ccb_sz_collective(ccb_comm* c, const float* const* send, float* const* recv, int nx, int ny, int nz, float eb, int root,
                      unsigned long long* d_used, ccb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
