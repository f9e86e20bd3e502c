/* Compressed MPI point-to-point helpers. Wire format and calls follow the reference
 * (run_codes/wrappers/mpi_compress_tools.c): a message is [int32 compressed size |
 * payload] (:62-99); send_compressed posts a PMPI_Isend and parks buffer and request
 * in the pending table until flush_pending (:101-130); recv_decompress probes for the
 * size (:132-163); exchange_compressed swaps sizes, then payloads, with two
 * PMPI_Sendrecv on tag+1 / tag+2 (:165-222). Capacity bound of a compressed block:
 * n + 64 + n/16. Everything uses PMPI_* so that interposed MPI_* are not re-entered. */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "mpi_compress_tools.h"

__attribute__((weak)) int compression_enabled(void) {
    const char *e = getenv("MPI_COMPRESS_DISABLE");
    return !(e && (*e == '1' || *e == 'y' || *e == 'Y'));
}

typedef struct { void *buf; MPI_Request req; } pending_t;
static pending_t *g_pending;
static int g_npending, g_cap;

void ensure_pending_capacity(int needed) {
    if (needed <= g_cap) return;
    int cap = g_cap ? g_cap : 256;
    while (cap < needed) cap *= 2;
    g_pending = (pending_t *)realloc(g_pending, (size_t)cap * sizeof(pending_t));
    g_cap = cap;
}
int add_pending_send(void *buf, MPI_Request req) {
    ensure_pending_capacity(g_npending + 1);
    g_pending[g_npending].buf = buf;
    g_pending[g_npending].req = req;
    return g_npending++;
}
void flush_pending(void) {
    for (int i = 0; i < g_npending; ++i) {
        PMPI_Wait(&g_pending[i].req, MPI_STATUS_IGNORE);
        free(g_pending[i].buf);
    }
    g_npending = 0;
}

static size_t comp_capacity(size_t n) { return n + 64 + n / 16; }

/* [int32 size | payload] in a fresh buffer; *wire_len receives its length */
static char *pack(const void *buf, size_t n, size_t *wire_len) {
    const size_t cap = comp_capacity(n);
    char *w = (char *)malloc(sizeof(int32_t) + cap);
    if (!w) return NULL;
    size_t out = cap;
    if (!compression_enabled() || mpi_compress((void *)buf, n, w + sizeof(int32_t), &out) != 0 || out > cap) {
        memcpy(w + sizeof(int32_t), buf, n);
        out = n;
    }
    int32_t sz = (int32_t)out;
    memcpy(w, &sz, sizeof(sz));
    *wire_len = sizeof(int32_t) + out;
    return w;
}

static int unpack(char *w, size_t wire_len, void *buf, size_t n) {
    int32_t sz = 0;
    if (wire_len < sizeof(sz)) return 1;
    memcpy(&sz, w, sizeof(sz));
    if (sz < 0 || (size_t)sz + sizeof(sz) > wire_len) return 1;
    if (!compression_enabled()) {
        memcpy(buf, w + sizeof(sz), min_sz((size_t)sz, n));
        return 0;
    }
    return mpi_decompress(w + sizeof(sz), (size_t)sz, buf, n) != 0;
}

int send_compressed(const void *buf, size_t data_size, int dest, int tag, MPI_Comm comm) {
    size_t len = 0;
    char *w = pack(buf, data_size, &len);
    if (!w) return 1;
    MPI_Request req;
    if (PMPI_Isend(w, (int)len, MPI_BYTE, dest, tag, comm, &req) != MPI_SUCCESS) {
        free(w);
        return 1;
    }
    add_pending_send(w, req);
    return 0;
}

int recv_decompress(void *buf, size_t data_size, int source, int tag, MPI_Comm comm) {
    MPI_Status st;
    int len = 0;
    if (PMPI_Probe(source, tag, comm, &st) != MPI_SUCCESS) return 1;
    PMPI_Get_count(&st, MPI_BYTE, &len);
    char *w = (char *)malloc((size_t)(len > 0 ? len : 1));
    if (!w) return 1;
    int rc = PMPI_Recv(w, len, MPI_BYTE, st.MPI_SOURCE, tag, comm, MPI_STATUS_IGNORE) != MPI_SUCCESS;
    if (!rc) rc = unpack(w, (size_t)len, buf, data_size);
    free(w);
    return rc;
}

int exchange_compressed(const void *sendbuf, size_t send_dsize, void *recvbuf, size_t recv_dsize, int dst, int src, int tag,
                        MPI_Comm comm) {
    size_t slen = 0;
    char *sw = pack(sendbuf, send_dsize, &slen);
    if (!sw) return 1;
    int mine = (int)slen, theirs = 0;
    int rc = PMPI_Sendrecv(&mine, 1, MPI_INT, dst, tag + 1, &theirs, 1, MPI_INT, src, tag + 1, comm, MPI_STATUS_IGNORE) != MPI_SUCCESS;
    char *rw = rc ? NULL : (char *)malloc((size_t)(theirs > 0 ? theirs : 1));
    if (!rc && !rw) rc = 1;
    if (!rc)
        rc = PMPI_Sendrecv(sw, mine, MPI_BYTE, dst, tag + 2, rw, theirs, MPI_BYTE, src, tag + 2, comm, MPI_STATUS_IGNORE) != MPI_SUCCESS;
    if (!rc) rc = unpack(rw, (size_t)theirs, recvbuf, recv_dsize);
    free(sw);
    free(rw);
    return rc;
}
