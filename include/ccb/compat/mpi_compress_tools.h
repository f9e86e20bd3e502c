/* Compressed point-to-point helpers for MPI wrappers, with the reference's API
 * (run_codes/wrappers/mpi_compress_tools.h): tag bases per collective, a table of
 * pending non-blocking sends, and send / receive / exchange of codec output framed as
 * [int32 size | payload]. A compression wrapper provides strong mpi_compress /
 * mpi_decompress; the communication wrapper ships weak identity versions. */
#ifndef MPI_COMPRESS_TOOLS_H
#define MPI_COMPRESS_TOOLS_H

#include <mpi.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Message tags: one block of 0x100 per collective, so that a wrapper may use base, base + 1
 * (sizes) and base + 2 (payload) without colliding with another collective in flight. */
#define CCB_MPI_TAG_BLOCK(k) (0x2000 + 0x100 * (k))
#define TAG_BCAST CCB_MPI_TAG_BLOCK(0)
#define TAG_REDUCE CCB_MPI_TAG_BLOCK(1)
#define TAG_ALLREDUCE CCB_MPI_TAG_BLOCK(2)
#define TAG_GATHER CCB_MPI_TAG_BLOCK(3)
#define TAG_SCATTER CCB_MPI_TAG_BLOCK(4)
#define TAG_ALLGATHER CCB_MPI_TAG_BLOCK(5)
#define TAG_ALLTOALL CCB_MPI_TAG_BLOCK(6)
#define TAG_REDUCE_SCAT CCB_MPI_TAG_BLOCK(7)
#define TAG_ALLGATHERV CCB_MPI_TAG_BLOCK(8)
#define TAG_SCATTERV CCB_MPI_TAG_BLOCK(9)

/* ---- the codec pair: strong definitions come from a compression wrapper, the weak
 * identity pair from the communication wrapper. Both return 0 on success. ---------- */
int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size); /* in: *output_size = capacity */
int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size);
int compression_enabled(void); /* 0 when MPI_COMPRESS_DISABLE asks for pass-through */

/* ---- framed transfers: [int32 compressed size | payload] ----------------------------- */
int send_compressed(const void *buf, size_t data_size, int dest, int tag, MPI_Comm comm);
int recv_decompress(void *buf, size_t data_size, int source, int tag, MPI_Comm comm);
/* both directions at once (sizes first, then payloads, by MPI_Sendrecv) */
int exchange_compressed(const void *sendbuf, size_t send_dsize, void *recvbuf, size_t recv_dsize, int dst, int src, int tag,
                        MPI_Comm comm);

/* ---- non-blocking sends whose buffers must outlive the call --------------------------- */
void ensure_pending_capacity(int needed);
int add_pending_send(void *buf, MPI_Request req); /* takes ownership of buf */
void flush_pending(void);                          /* waits for all, frees the buffers */

/* ---- small helpers the wrappers share -------------------------------------------------- */
static inline size_t type_size(MPI_Datatype dt) {
    int bytes = 0;
    MPI_Type_size(dt, &bytes);
    return (size_t)bytes;
}
static inline int next_pow2(int x) {
    int p = 1;
    while (p < x) p += p;
    return p;
}
static inline size_t min_sz(size_t a, size_t b) { return b < a ? b : a; }

#ifdef __cplusplus
}
#endif
#endif /* MPI_COMPRESS_TOOLS_H */
