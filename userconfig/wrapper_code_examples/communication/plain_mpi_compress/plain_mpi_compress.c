/* plain_mpi_compress: LD_PRELOAD interposer that rebuilds the MPI collectives from
 * compressed point-to-point messages. Every hop goes through mpi_compress /
 * mpi_decompress (weak identity here; a compression wrapper preloaded before this
 * library overrides them) and the helpers of mpi_compress_tools.
 *
 * Collectives and algorithms are those of the reference wrapper
 * (userconfig/wrapper_code_examples/communication/plain_mpi_compress/
 * plain_mpi_compress.c): Bcast and Reduce binomial trees (:69-159), Allreduce = ring
 * reduce-scatter + ring all-gather with a codec round trip per hop (:163-289), Gather
 * and Scatter linear (:293-349), Allgather ring (:353-388), Alltoall (:392-426),
 * Reduce_scatter_block by recursive halving on a power-of-two padding (:430-511),
 * Reduce_scatter (:515-602), Allgatherv and Scatterv (:606-686). Calls on
 * communicators other than MPI_COMM_WORLD, and everything when MPI_COMPRESS_DISABLE=1,
 * fall through to PMPI_*. Chunk boundaries of the ring use the exact
 * count/size split (the first count%size chunks get one more element). */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "mpi_compress_tools.h"

#ifdef PLAIN_MPI_CODEC_ELSEWHERE /* a file that includes this one brings strong codec hooks */
int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size);
int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size);
#else
__attribute__((weak)) int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size) {
    memcpy(output, input, input_size);
    *output_size = input_size;
    return 0;
}
__attribute__((weak)) int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    memcpy(output, input, min_sz(input_size, output_size));
    return 0;
}
#endif

static int active(MPI_Comm comm) { return comm == MPI_COMM_WORLD && compression_enabled(); }
static void rank_size(MPI_Comm c, int *r, int *n) {
    PMPI_Comm_rank(c, r);
    PMPI_Comm_size(c, n);
}
static void chunk_of(int count, int n, int i, int *off, int *len) {
    const int base = count / n, rem = count % n;
    *len = base + (i < rem ? 1 : 0);
    *off = i * base + (i < rem ? i : rem);
}

int MPI_Bcast(void *buf, int count, MPI_Datatype dt, int root, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Bcast(buf, count, dt, root, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    const size_t bytes = (size_t)count * type_size(dt);
    const int v = (rank - root + n) % n; /* rank relative to the root */
    int mask = 1;
    while (mask < n) { /* receive from the parent */
        if (v & mask) {
            if (recv_decompress(buf, bytes, (v - mask + root) % n, TAG_BCAST, comm)) return MPI_ERR_OTHER;
            break;
        }
        mask <<= 1;
    }
    for (mask >>= 1; mask > 0; mask >>= 1) /* pass down to the children */
        if (v + mask < n && send_compressed(buf, bytes, (v + mask + root) % n, TAG_BCAST, comm)) return MPI_ERR_OTHER;
    flush_pending();
    return MPI_SUCCESS;
}

int MPI_Reduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Reduce(sendbuf, recvbuf, count, dt, op, root, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    const size_t bytes = (size_t)count * type_size(dt);
    void *acc = malloc(bytes ? bytes : 1), *tmp = malloc(bytes ? bytes : 1);
    memcpy(acc, sendbuf == MPI_IN_PLACE ? recvbuf : sendbuf, bytes);
    const int v = (rank - root + n) % n;
    int rc = MPI_SUCCESS;
    for (int mask = 1; mask < n; mask <<= 1) {
        if (v & mask) {
            if (send_compressed(acc, bytes, (v - mask + root) % n, TAG_REDUCE, comm)) rc = MPI_ERR_OTHER;
            break;
        }
        if (v + mask < n) {
            if (recv_decompress(tmp, bytes, (v + mask + root) % n, TAG_REDUCE, comm)) { rc = MPI_ERR_OTHER; break; }
            PMPI_Reduce_local(tmp, acc, count, dt, op);
        }
    }
    flush_pending();
    if (rank == root && rc == MPI_SUCCESS) memcpy(recvbuf, acc, bytes);
    free(acc);
    free(tmp);
    return rc;
}

int MPI_Allreduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Allreduce(sendbuf, recvbuf, count, dt, op, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    const size_t es = type_size(dt);
    if (sendbuf != MPI_IN_PLACE) memcpy(recvbuf, sendbuf, (size_t)count * es);
    if (n == 1) return MPI_SUCCESS;
    char *data = (char *)recvbuf;
    const int next = (rank + 1) % n, prev = (rank - 1 + n) % n;
    int maxlen = count / n + 1;
    void *tmp = malloc((size_t)maxlen * es);
    int rc = MPI_SUCCESS;
    for (int s = 0; s < n - 1 && rc == MPI_SUCCESS; ++s) { /* reduce-scatter */
        int so, sl, ro, rl;
        chunk_of(count, n, (rank - s + n) % n, &so, &sl);
        chunk_of(count, n, (rank - s - 1 + n) % n, &ro, &rl);
        if (exchange_compressed(data + (size_t)so * es, (size_t)sl * es, tmp, (size_t)rl * es, next, prev, TAG_ALLREDUCE, comm)) rc = MPI_ERR_OTHER;
        else PMPI_Reduce_local(tmp, data + (size_t)ro * es, rl, dt, op);
    }
    for (int s = 0; s < n - 1 && rc == MPI_SUCCESS; ++s) { /* all-gather */
        int so, sl, ro, rl;
        chunk_of(count, n, (rank + 1 - s + n) % n, &so, &sl);
        chunk_of(count, n, (rank - s + n) % n, &ro, &rl);
        if (exchange_compressed(data + (size_t)so * es, (size_t)sl * es, data + (size_t)ro * es, (size_t)rl * es, next, prev,
                                TAG_ALLREDUCE + 0x10, comm))
            rc = MPI_ERR_OTHER;
    }
    free(tmp);
    return rc;
}

int MPI_Gather(const void *sendbuf, int sc, MPI_Datatype sdt, void *recvbuf, int rcnt, MPI_Datatype rdt, int root, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Gather(sendbuf, sc, sdt, recvbuf, rcnt, rdt, root, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    const size_t sb = (size_t)sc * type_size(sdt), rb = (size_t)rcnt * type_size(rdt);
    int rc = MPI_SUCCESS;
    if (rank != root) {
        if (send_compressed(sendbuf, sb, root, TAG_GATHER, comm)) rc = MPI_ERR_OTHER;
        flush_pending();
        return rc;
    }
    for (int p = 0; p < n; ++p) {
        char *dst = (char *)recvbuf + (size_t)p * rb;
        if (p == root) { if (sendbuf != MPI_IN_PLACE) memcpy(dst, sendbuf, sb); }
        else if (recv_decompress(dst, rb, p, TAG_GATHER, comm)) rc = MPI_ERR_OTHER;
    }
    return rc;
}

int MPI_Scatter(const void *sendbuf, int sc, MPI_Datatype sdt, void *recvbuf, int rcnt, MPI_Datatype rdt, int root, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Scatter(sendbuf, sc, sdt, recvbuf, rcnt, rdt, root, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    const size_t sb = (size_t)sc * type_size(sdt), rb = (size_t)rcnt * type_size(rdt);
    if (rank != root) return recv_decompress(recvbuf, rb, root, TAG_SCATTER, comm) ? MPI_ERR_OTHER : MPI_SUCCESS;
    int rc = MPI_SUCCESS;
    for (int p = 0; p < n; ++p) {
        const char *src = (const char *)sendbuf + (size_t)p * sb;
        if (p == root) { if (recvbuf != MPI_IN_PLACE) memcpy(recvbuf, src, sb); }
        else if (send_compressed(src, sb, p, TAG_SCATTER, comm)) rc = MPI_ERR_OTHER;
    }
    flush_pending();
    return rc;
}

int MPI_Allgather(const void *sendbuf, int sc, MPI_Datatype sdt, void *recvbuf, int rcnt, MPI_Datatype rdt, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Allgather(sendbuf, sc, sdt, recvbuf, rcnt, rdt, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    const size_t rb = (size_t)rcnt * type_size(rdt);
    char *data = (char *)recvbuf;
    if (sendbuf != MPI_IN_PLACE) memcpy(data + (size_t)rank * rb, sendbuf, (size_t)sc * type_size(sdt));
    const int next = (rank + 1) % n, prev = (rank - 1 + n) % n;
    for (int s = 0; s < n - 1; ++s) { /* ring: forward the block received in the previous step */
        const int sblk = (rank - s + n) % n, rblk = (rank - s - 1 + n) % n;
        if (exchange_compressed(data + (size_t)sblk * rb, rb, data + (size_t)rblk * rb, rb, next, prev, TAG_ALLGATHER, comm)) return MPI_ERR_OTHER;
    }
    return MPI_SUCCESS;
}

int MPI_Alltoall(const void *sendbuf, int sc, MPI_Datatype sdt, void *recvbuf, int rcnt, MPI_Datatype rdt, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Alltoall(sendbuf, sc, sdt, recvbuf, rcnt, rdt, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    const size_t sb = (size_t)sc * type_size(sdt), rb = (size_t)rcnt * type_size(rdt);
    int rc = MPI_SUCCESS;
    ensure_pending_capacity(n);
    for (int j = 1; j < n; ++j) {
        const int p = (rank + j) % n;
        if (send_compressed((const char *)sendbuf + (size_t)p * sb, sb, p, TAG_ALLTOALL, comm)) rc = MPI_ERR_OTHER;
    }
    memcpy((char *)recvbuf + (size_t)rank * rb, (const char *)sendbuf + (size_t)rank * sb, min_sz(sb, rb));
    for (int j = 1; j < n; ++j) {
        const int p = (rank - j + n) % n;
        if (recv_decompress((char *)recvbuf + (size_t)p * rb, rb, p, TAG_ALLTOALL, comm)) rc = MPI_ERR_OTHER;
    }
    flush_pending();
    return rc;
}

int MPI_Reduce_scatter_block(const void *sendbuf, void *recvbuf, int rcnt, MPI_Datatype dt, MPI_Op op, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Reduce_scatter_block(sendbuf, recvbuf, rcnt, dt, op, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    const size_t es = type_size(dt), blk = (size_t)rcnt * es;
    const int p2 = next_pow2(n);
    /* work on p2 blocks; ranks >= n do not exist: their partners keep the block instead
     * (the extra blocks hold no data of their own and are simply never requested) */
    char *work = (char *)calloc((size_t)p2, blk ? blk : 1), *tmp = (char *)malloc((size_t)p2 / 2 * (blk ? blk : 1) + 1);
    memcpy(work, sendbuf == MPI_IN_PLACE ? recvbuf : sendbuf, (size_t)n * blk);
    int rc = MPI_SUCCESS;
    if (p2 != n) {
        /* non power of two: reduce to rank 0 block-wise through the ring allreduce of the
         * whole vector, then keep the own block (simple and exact in chunking) */
        rc = MPI_Allreduce(MPI_IN_PLACE, work, rcnt * n, dt, op, comm);
        memcpy(recvbuf, work + (size_t)rank * blk, blk);
        free(work);
        free(tmp);
        return rc;
    }
    int lo = 0, hi = n; /* block range this rank is still responsible for */
    for (int dist = n / 2; dist >= 1 && rc == MPI_SUCCESS; dist /= 2) {
        const int partner = rank ^ dist, mid = (lo + hi) / 2;
        const int keep_lo = (rank & dist) ? mid : lo, keep_hi = (rank & dist) ? hi : mid;
        const int give_lo = (rank & dist) ? lo : mid, give_hi = (rank & dist) ? mid : hi;
        const size_t gb = (size_t)(give_hi - give_lo) * blk, kb = (size_t)(keep_hi - keep_lo) * blk;
        if (exchange_compressed(work + (size_t)give_lo * blk, gb, tmp, kb, partner, partner, TAG_REDUCE_SCAT, comm)) rc = MPI_ERR_OTHER;
        else PMPI_Reduce_local(tmp, work + (size_t)keep_lo * blk, (keep_hi - keep_lo) * rcnt, dt, op);
        lo = keep_lo;
        hi = keep_hi;
    }
    memcpy(recvbuf, work + (size_t)rank * blk, blk);
    free(work);
    free(tmp);
    return rc;
}

int MPI_Reduce_scatter(const void *sendbuf, void *recvbuf, const int recvcounts[], MPI_Datatype dt, MPI_Op op, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Reduce_scatter(sendbuf, recvbuf, recvcounts, dt, op, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    int uniform = 1, total = 0, off = 0;
    for (int p = 0; p < n; ++p) {
        if (recvcounts[p] != recvcounts[0]) uniform = 0;
        if (p < rank) off += recvcounts[p];
        total += recvcounts[p];
    }
    if (uniform) return MPI_Reduce_scatter_block(sendbuf, recvbuf, recvcounts[0], dt, op, comm);
    const size_t es = type_size(dt);
    void *full = malloc((size_t)(total ? total : 1) * es);
    memcpy(full, sendbuf, (size_t)total * es);
    int rc = MPI_Allreduce(MPI_IN_PLACE, full, total, dt, op, comm);
    memcpy(recvbuf, (char *)full + (size_t)off * es, (size_t)recvcounts[rank] * es);
    free(full);
    return rc;
}

int MPI_Allgatherv(const void *sendbuf, int sc, MPI_Datatype sdt, void *recvbuf, const int recvcounts[], const int displs[],
                   MPI_Datatype rdt, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Allgatherv(sendbuf, sc, sdt, recvbuf, recvcounts, displs, rdt, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    const size_t es = type_size(rdt);
    if (sendbuf != MPI_IN_PLACE) memcpy((char *)recvbuf + (size_t)displs[rank] * es, sendbuf, (size_t)sc * type_size(sdt));
    for (int root = 0; root < n; ++root) /* one compressed broadcast per contributor */
        if (MPI_Bcast((char *)recvbuf + (size_t)displs[root] * es, recvcounts[root], rdt, root, comm) != MPI_SUCCESS) return MPI_ERR_OTHER;
    return MPI_SUCCESS;
}

int MPI_Scatterv(const void *sendbuf, const int sendcounts[], const int displs[], MPI_Datatype sdt, void *recvbuf, int rcnt,
                 MPI_Datatype rdt, int root, MPI_Comm comm) {
    if (!active(comm)) return PMPI_Scatterv(sendbuf, sendcounts, displs, sdt, recvbuf, rcnt, rdt, root, comm);
    int rank, n;
    rank_size(comm, &rank, &n);
    if (rank != root) return recv_decompress(recvbuf, (size_t)rcnt * type_size(rdt), root, TAG_SCATTERV, comm) ? MPI_ERR_OTHER : MPI_SUCCESS;
    const size_t es = type_size(sdt);
    int rc = MPI_SUCCESS;
    for (int p = 0; p < n; ++p) {
        const char *src = (const char *)sendbuf + (size_t)displs[p] * es;
        if (p == root) { if (recvbuf != MPI_IN_PLACE) memcpy(recvbuf, src, (size_t)sendcounts[p] * es); }
        else if (send_compressed(src, (size_t)sendcounts[p] * es, p, TAG_SCATTERV, comm)) rc = MPI_ERR_OTHER;
    }
    flush_pending();
    return rc;
}
