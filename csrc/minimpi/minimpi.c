/* ccb_minimpi implementation: see mpi.h. A full mesh of non-blocking Unix stream
 * sockets (abstract names "ccbmpi.<job>.<rank>"), eager buffered sends, a progress
 * engine that is driven from every blocking call, and linear collectives built on
 * the point-to-point layer. A test substrate, not a fast MPI. */
#define _GNU_SOURCE
#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include "mpi.h"

#define COLL_TAG_BASE 0x40000000

typedef struct msg {
    int src, tag;
    size_t len;
    char *data;
    struct msg *next;
} msg_t;

typedef struct {
    int fd;
    char *out;
    size_t out_len, out_cap, out_off;
    char hdr[16];
    size_t hdr_got;
    msg_t *cur;
    size_t cur_got;
} peer_t;

struct ccb_mpi_request {
    int is_recv, done;
    void *buf;
    size_t cap;
    int src, tag;
    MPI_Status st;
};

static int g_rank, g_size = 1, g_init;
static peer_t *g_peers;
static msg_t *g_q_head, *g_q_tail;
static int g_coll_seq;

static void die(const char *what) {
    fprintf(stderr, "[minimpi rank %d] %s: %s\n", g_rank, what, strerror(errno));
    _exit(1);
}

static socklen_t make_addr(struct sockaddr_un *a, int rank) {
    const char *job = getenv("CCB_MINIMPI_JOB");
    char name[96];
    memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    int n = snprintf(name, sizeof(name), "ccbmpi.%s.%d", job ? job : "default", rank);
    memcpy(a->sun_path + 1, name, (size_t)n);
    return (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + (size_t)n);
}

static void set_nonblock(int fd) {
    fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK);
    /* Large socket buffers: a multi-megabyte message then crosses in a few system calls
     * instead of one scheduler round trip per 200 KB. The FORCE variants need privilege;
     * the plain ones are clamped by the host's limits. */
    int want = 16 << 20;
    if (setsockopt(fd, SOL_SOCKET, SO_SNDBUFFORCE, &want, sizeof(want)) != 0) setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &want, sizeof(want));
    if (setsockopt(fd, SOL_SOCKET, SO_RCVBUFFORCE, &want, sizeof(want)) != 0) setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &want, sizeof(want));
}

static size_t dt_size(MPI_Datatype dt) {
    switch (dt) {
        case MPI_CHAR: case MPI_BYTE: case MPI_UNSIGNED_CHAR: case MPI_INT8_T: case MPI_UINT8_T: return 1;
        case MPI_INT: case MPI_FLOAT: case MPI_INT32_T: case MPI_UNSIGNED: return 4;
        default: return 8;
    }
}

/* ------------------------------------------------------------------ progress */
static void flush_peer(peer_t *p) {
    while (p->out_off < p->out_len) {
        ssize_t w = send(p->fd, p->out + p->out_off, p->out_len - p->out_off, MSG_NOSIGNAL);
        if (w > 0) p->out_off += (size_t)w;
        else if (w < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) return;
        else if (w < 0 && errno == EINTR) continue;
        else die("send");
    }
    p->out_len = p->out_off = 0;
}

static void drain_peer(peer_t *p, int src) {
    for (;;) {
        if (!p->cur) {
            ssize_t r = recv(p->fd, p->hdr + p->hdr_got, sizeof(p->hdr) - p->hdr_got, 0);
            if (r > 0) p->hdr_got += (size_t)r;
            else if (r == 0) return; /* peer closed */
            else if (errno == EAGAIN || errno == EWOULDBLOCK) return;
            else if (errno == EINTR) continue;
            else die("recv");
            if (p->hdr_got < sizeof(p->hdr)) continue;
            msg_t *m = (msg_t *)calloc(1, sizeof(*m));
            int32_t tag;
            uint64_t len;
            memcpy(&tag, p->hdr, 4);
            memcpy(&len, p->hdr + 8, 8);
            m->src = src;
            m->tag = tag;
            m->len = (size_t)len;
            m->data = (char *)malloc(m->len ? m->len : 1);
            p->cur = m;
            p->cur_got = 0;
            p->hdr_got = 0;
        }
        while (p->cur_got < p->cur->len) {
            ssize_t r = recv(p->fd, p->cur->data + p->cur_got, p->cur->len - p->cur_got, 0);
            if (r > 0) p->cur_got += (size_t)r;
            else if (r == 0) return;
            else if (errno == EAGAIN || errno == EWOULDBLOCK) return;
            else if (errno == EINTR) continue;
            else die("recv");
        }
        if (g_q_tail) g_q_tail->next = p->cur;
        else g_q_head = p->cur;
        g_q_tail = p->cur;
        p->cur = NULL;
    }
}

static void progress(int wait_ms) {
    struct pollfd fds[64];
    int idx[64], n = 0;
    for (int r = 0; r < g_size; ++r) {
        if (r == g_rank) continue;
        fds[n].fd = g_peers[r].fd;
        fds[n].events = POLLIN | (g_peers[r].out_len > g_peers[r].out_off ? POLLOUT : 0);
        fds[n].revents = 0;
        idx[n++] = r;
    }
    if (n == 0) return;
    if (poll(fds, (nfds_t)n, wait_ms) <= 0) return;
    for (int i = 0; i < n; ++i) {
        if (fds[i].revents & POLLOUT) flush_peer(&g_peers[idx[i]]);
        if (fds[i].revents & (POLLIN | POLLHUP)) drain_peer(&g_peers[idx[i]], idx[i]);
    }
}

static void enqueue_send(int dest, int tag, const void *buf, size_t len) {
    if (dest == g_rank) { /* self message goes straight to the queue */
        msg_t *m = (msg_t *)calloc(1, sizeof(*m));
        m->src = g_rank;
        m->tag = tag;
        m->len = len;
        m->data = (char *)malloc(len ? len : 1);
        memcpy(m->data, buf, len);
        if (g_q_tail) g_q_tail->next = m;
        else g_q_head = m;
        g_q_tail = m;
        return;
    }
    peer_t *p = &g_peers[dest];
    const size_t need = p->out_len + 16 + len;
    if (need > p->out_cap) {
        size_t cap = p->out_cap ? p->out_cap : 65536;
        while (cap < need) cap *= 2;
        p->out = (char *)realloc(p->out, cap);
        p->out_cap = cap;
    }
    int32_t t = tag, zero = 0;
    uint64_t l = len;
    memcpy(p->out + p->out_len, &t, 4);
    memcpy(p->out + p->out_len + 4, &zero, 4);
    memcpy(p->out + p->out_len + 8, &l, 8);
    memcpy(p->out + p->out_len + 16, buf, len);
    p->out_len = need;
    flush_peer(p);
}

static msg_t *match(int src, int tag, int remove) {
    msg_t *prev = NULL;
    for (msg_t *m = g_q_head; m; prev = m, m = m->next) {
        if ((src == MPI_ANY_SOURCE || m->src == src) && (tag == MPI_ANY_TAG ? m->tag < COLL_TAG_BASE : m->tag == tag)) {
            if (remove) {
                if (prev) prev->next = m->next;
                else g_q_head = m->next;
                if (g_q_tail == m) g_q_tail = prev;
                m->next = NULL;
            }
            return m;
        }
    }
    return NULL;
}

static void recv_blocking(void *buf, size_t cap, int src, int tag, MPI_Status *st) {
    msg_t *m;
    while (!(m = match(src, tag, 1))) progress(50);
    const size_t n = m->len < cap ? m->len : cap;
    memcpy(buf, m->data, n);
    if (st) {
        st->MPI_SOURCE = m->src;
        st->MPI_TAG = m->tag;
        st->MPI_ERROR = MPI_SUCCESS;
        st->ccb_bytes = m->len;
    }
    free(m->data);
    free(m);
}

/* ---------------------------------------------------------------- lifecycle -- */
int PMPI_Init(int *argc, char ***argv) {
    (void)argc;
    (void)argv;
    if (g_init) return MPI_SUCCESS;
    const char *r = getenv("OMPI_COMM_WORLD_RANK"), *s = getenv("OMPI_COMM_WORLD_SIZE");
    if (!r) { r = getenv("PMI_RANK"); s = getenv("PMI_SIZE"); }
    if (!r) { r = getenv("RANK"); s = getenv("WORLD_SIZE"); }
    g_rank = r ? atoi(r) : 0;
    g_size = s ? atoi(s) : 1;
    if (g_size > 64) {
        fprintf(stderr, "[minimpi] at most 64 ranks\n");
        _exit(1);
    }
    g_peers = (peer_t *)calloc((size_t)g_size, sizeof(peer_t));
    for (int i = 0; i < g_size; ++i) g_peers[i].fd = -1;
    if (g_size > 1) {
        int ls = socket(AF_UNIX, SOCK_STREAM, 0);
        struct sockaddr_un a;
        socklen_t alen = make_addr(&a, g_rank);
        if (ls < 0 || bind(ls, (struct sockaddr *)&a, alen) != 0 || listen(ls, g_size) != 0) die("bind/listen");
        /* connect to every lower rank, accept from every higher rank */
        for (int p = 0; p < g_rank; ++p) {
            struct sockaddr_un pa;
            socklen_t plen = make_addr(&pa, p);
            int fd = -1;
            for (int t = 0; t < 6000; ++t) {
                fd = socket(AF_UNIX, SOCK_STREAM, 0);
                if (fd >= 0 && connect(fd, (struct sockaddr *)&pa, plen) == 0) break;
                if (fd >= 0) close(fd);
                fd = -1;
                usleep(5000);
            }
            if (fd < 0) die("connect");
            int32_t me = g_rank;
            if (send(fd, &me, 4, MSG_NOSIGNAL) != 4) die("hello");
            g_peers[p].fd = fd;
        }
        for (int k = g_rank + 1; k < g_size; ++k) {
            int fd = accept(ls, NULL, NULL);
            int32_t who = -1;
            if (fd < 0 || recv(fd, &who, 4, MSG_WAITALL) != 4 || who <= g_rank || who >= g_size) die("accept");
            g_peers[who].fd = fd;
        }
        close(ls);
        for (int p = 0; p < g_size; ++p)
            if (p != g_rank) set_nonblock(g_peers[p].fd);
    }
    g_init = 1;
    return MPI_SUCCESS;
}
int PMPI_Init_thread(int *argc, char ***argv, int required, int *provided) {
    if (provided) *provided = required < MPI_THREAD_SERIALIZED ? required : MPI_THREAD_SERIALIZED;
    return PMPI_Init(argc, argv);
}
int PMPI_Initialized(int *flag) { *flag = g_init; return MPI_SUCCESS; }
int PMPI_Finalize(void) {
    if (!g_init) return MPI_SUCCESS;
    PMPI_Barrier(MPI_COMM_WORLD);
    for (int p = 0; p < g_size; ++p)
        if (g_peers[p].fd >= 0) close(g_peers[p].fd);
    g_init = 0;
    return MPI_SUCCESS;
}
int PMPI_Abort(MPI_Comm comm, int code) { (void)comm; _exit(code ? code : 1); }
int PMPI_Comm_rank(MPI_Comm c, int *rank) { (void)c; *rank = g_rank; return MPI_SUCCESS; }
int PMPI_Comm_size(MPI_Comm c, int *size) { (void)c; *size = g_size; return MPI_SUCCESS; }
int PMPI_Get_processor_name(char *name, int *len) {
    if (gethostname(name, MPI_MAX_PROCESSOR_NAME) != 0) strcpy(name, "localhost");
    name[MPI_MAX_PROCESSOR_NAME - 1] = '\0';
    *len = (int)strlen(name);
    return MPI_SUCCESS;
}
double PMPI_Wtime(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + (double)ts.tv_nsec * 1e-9;
}
int PMPI_Type_size(MPI_Datatype dt, int *size) { *size = (int)dt_size(dt); return MPI_SUCCESS; }

/* ------------------------------------------------------------ point to point -- */
int PMPI_Send(const void *buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm) {
    (void)comm;
    enqueue_send(dest, tag, buf, (size_t)count * dt_size(dt));
    return MPI_SUCCESS;
}
int PMPI_Recv(void *buf, int count, MPI_Datatype dt, int src, int tag, MPI_Comm comm, MPI_Status *st) {
    (void)comm;
    recv_blocking(buf, (size_t)count * dt_size(dt), src, tag, st);
    return MPI_SUCCESS;
}
int PMPI_Isend(const void *buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request *req) {
    PMPI_Send(buf, count, dt, dest, tag, comm); /* buffered: complete at once */
    struct ccb_mpi_request *r = (struct ccb_mpi_request *)calloc(1, sizeof(*r));
    r->done = 1;
    *req = r;
    return MPI_SUCCESS;
}
int PMPI_Irecv(void *buf, int count, MPI_Datatype dt, int src, int tag, MPI_Comm comm, MPI_Request *req) {
    (void)comm;
    struct ccb_mpi_request *r = (struct ccb_mpi_request *)calloc(1, sizeof(*r));
    r->is_recv = 1;
    r->buf = buf;
    r->cap = (size_t)count * dt_size(dt);
    r->src = src;
    r->tag = tag;
    *req = r;
    return MPI_SUCCESS;
}
int PMPI_Wait(MPI_Request *req, MPI_Status *st) {
    if (!req || !*req) return MPI_SUCCESS;
    struct ccb_mpi_request *r = *req;
    if (r->is_recv && !r->done) recv_blocking(r->buf, r->cap, r->src, r->tag, &r->st);
    if (st && r->is_recv) *st = r->st;
    free(r);
    *req = MPI_REQUEST_NULL;
    return MPI_SUCCESS;
}
int PMPI_Waitall(int n, MPI_Request reqs[], MPI_Status sts[]) {
    for (int i = 0; i < n; ++i) PMPI_Wait(&reqs[i], sts ? &sts[i] : MPI_STATUS_IGNORE);
    return MPI_SUCCESS;
}
int PMPI_Test(MPI_Request *req, int *flag, MPI_Status *st) {
    *flag = 1;
    if (!req || !*req) return MPI_SUCCESS;
    struct ccb_mpi_request *r = *req;
    if (r->is_recv && !r->done) {
        progress(0);
        if (!match(r->src, r->tag, 0)) {
            *flag = 0;
            return MPI_SUCCESS;
        }
    }
    return PMPI_Wait(req, st);
}
int PMPI_Iprobe(int src, int tag, MPI_Comm comm, int *flag, MPI_Status *st) {
    (void)comm;
    progress(0);
    msg_t *m = match(src, tag, 0);
    *flag = m != NULL;
    if (m && st) {
        st->MPI_SOURCE = m->src;
        st->MPI_TAG = m->tag;
        st->MPI_ERROR = MPI_SUCCESS;
        st->ccb_bytes = m->len;
    }
    return MPI_SUCCESS;
}
int PMPI_Probe(int src, int tag, MPI_Comm comm, MPI_Status *st) {
    int flag = 0;
    for (;;) {
        PMPI_Iprobe(src, tag, comm, &flag, st);
        if (flag) return MPI_SUCCESS;
        progress(50);
    }
}
int PMPI_Get_count(const MPI_Status *st, MPI_Datatype dt, int *count) {
    *count = (int)(st->ccb_bytes / dt_size(dt));
    return MPI_SUCCESS;
}
int PMPI_Sendrecv(const void *sbuf, int scount, MPI_Datatype sdt, int dest, int stag, void *rbuf, int rcount, MPI_Datatype rdt,
                  int src, int rtag, MPI_Comm comm, MPI_Status *st) {
    PMPI_Send(sbuf, scount, sdt, dest, stag, comm);
    return PMPI_Recv(rbuf, rcount, rdt, src, rtag, comm, st);
}

/* ---------------------------------------------------------------- reductions -- */
#define RED(T)                                                                                     \
    do {                                                                                           \
        const T *a = (const T *)in;                                                                \
        T *b = (T *)inout;                                                                         \
        for (int i = 0; i < count; ++i) {                                                          \
            switch (op) {                                                                          \
                case MPI_SUM: b[i] = (T)(a[i] + b[i]); break;                                      \
                case MPI_PROD: b[i] = (T)(a[i] * b[i]); break;                                     \
                case MPI_MAX: b[i] = a[i] > b[i] ? a[i] : b[i]; break;                             \
                case MPI_MIN: b[i] = a[i] < b[i] ? a[i] : b[i]; break;                             \
                default: return MPI_ERR_OTHER;                                                     \
            }                                                                                      \
        }                                                                                          \
    } while (0)
int PMPI_Reduce_local(const void *in, void *inout, int count, MPI_Datatype dt, MPI_Op op) {
    switch (dt) {
        case MPI_FLOAT: RED(float); break;
        case MPI_DOUBLE: RED(double); break;
        case MPI_INT: case MPI_INT32_T: RED(int32_t); break;
        case MPI_UNSIGNED: RED(uint32_t); break;
        case MPI_LONG: case MPI_INT64_T: case MPI_LONG_LONG: RED(int64_t); break;
        case MPI_UINT64_T: RED(uint64_t); break;
        case MPI_CHAR: case MPI_INT8_T: RED(signed char); break;
        default: RED(unsigned char); break;
    }
    return MPI_SUCCESS;
}

/* --------------------------------------------------------------- collectives -- */
static int coll_tag(void) { return COLL_TAG_BASE + (g_coll_seq++ & 0xfffff); }

int PMPI_Barrier(MPI_Comm comm) {
    const int tag = coll_tag();
    char b = 0;
    if (g_rank == 0) {
        for (int p = 1; p < g_size; ++p) PMPI_Recv(&b, 1, MPI_BYTE, p, tag, comm, MPI_STATUS_IGNORE);
        for (int p = 1; p < g_size; ++p) PMPI_Send(&b, 1, MPI_BYTE, p, tag, comm);
    } else {
        PMPI_Send(&b, 1, MPI_BYTE, 0, tag, comm);
        PMPI_Recv(&b, 1, MPI_BYTE, 0, tag, comm, MPI_STATUS_IGNORE);
    }
    return MPI_SUCCESS;
}
int PMPI_Bcast(void *buf, int count, MPI_Datatype dt, int root, MPI_Comm comm) {
    const int tag = coll_tag();
    if (g_rank == root) {
        for (int p = 0; p < g_size; ++p)
            if (p != root) PMPI_Send(buf, count, dt, p, tag, comm);
    } else {
        PMPI_Recv(buf, count, dt, root, tag, comm, MPI_STATUS_IGNORE);
    }
    return MPI_SUCCESS;
}
int PMPI_Reduce(const void *s, void *r, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm) {
    const int tag = coll_tag();
    const size_t bytes = (size_t)count * dt_size(dt);
    if (g_rank != root) return PMPI_Send(s == MPI_IN_PLACE ? r : s, count, dt, root, tag, comm);
    void *tmp = malloc(bytes ? bytes : 1);
    if (s != MPI_IN_PLACE) memcpy(r, s, bytes);
    /* ranks are folded in rank order so that the result does not depend on arrival order */
    void *acc = malloc(bytes ? bytes : 1);
    int first = 1;
    for (int p = 0; p < g_size; ++p) {
        const void *contrib;
        if (p == root) contrib = r;
        else {
            PMPI_Recv(tmp, count, dt, p, tag, comm, MPI_STATUS_IGNORE);
            contrib = tmp;
        }
        if (first) { memcpy(acc, contrib, bytes); first = 0; }
        else PMPI_Reduce_local(contrib, acc, count, dt, op);
    }
    memcpy(r, acc, bytes);
    free(acc);
    free(tmp);
    return MPI_SUCCESS;
}
int PMPI_Allreduce(const void *s, void *r, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm) {
    const size_t es = dt_size(dt);
    if (g_size == 1 || (size_t)count * es < (1u << 20) || count < g_size) {
        /* small messages: fold at rank 0 in rank order (one deterministic summation order) */
        PMPI_Reduce(s, r, count, dt, op, 0, comm);
        return PMPI_Bcast(r, count, dt, 0, comm);
    }
    /* large messages: ring reduce-scatter + ring all-gather, every link busy in both
     * directions at once instead of everything funnelling through rank 0 */
    const int n = g_size, next = (g_rank + 1) % n, prev = (g_rank + n - 1) % n;
    const int tag = coll_tag();
    const int base = count / n, rem = count % n;
    int off[65];
    off[0] = 0;
    for (int c = 0; c < n; ++c) off[c + 1] = off[c] + base + (c < rem ? 1 : 0);
    if (s != MPI_IN_PLACE) memcpy(r, s, (size_t)count * es);
    void *tmp = malloc((size_t)(base + 1) * es);
    for (int step = 0; step < n - 1; ++step) {
        const int sc = ((g_rank - step) % n + n) % n, rc = ((g_rank - step - 1) % n + n) % n;
        PMPI_Sendrecv((char *)r + (size_t)off[sc] * es, off[sc + 1] - off[sc], dt, next, tag,
                      tmp, off[rc + 1] - off[rc], dt, prev, tag, comm, MPI_STATUS_IGNORE);
        PMPI_Reduce_local(tmp, (char *)r + (size_t)off[rc] * es, off[rc + 1] - off[rc], dt, op);
    }
    for (int step = 0; step < n - 1; ++step) {
        const int sc = ((g_rank + 1 - step) % n + n) % n, rc = ((g_rank - step) % n + n) % n;
        PMPI_Sendrecv((char *)r + (size_t)off[sc] * es, off[sc + 1] - off[sc], dt, next, tag,
                      (char *)r + (size_t)off[rc] * es, off[rc + 1] - off[rc], dt, prev, tag, comm, MPI_STATUS_IGNORE);
    }
    free(tmp);
    return MPI_SUCCESS;
}
int PMPI_Gatherv(const void *s, int sc, MPI_Datatype sdt, void *r, const int rcs[], const int displs[], MPI_Datatype rdt, int root, MPI_Comm comm) {
    const int tag = coll_tag();
    if (g_rank != root) return PMPI_Send(s, sc, sdt, root, tag, comm);
    for (int p = 0; p < g_size; ++p) {
        char *dst = (char *)r + (size_t)displs[p] * dt_size(rdt);
        if (p == root) memcpy(dst, s, (size_t)sc * dt_size(sdt));
        else PMPI_Recv(dst, rcs[p], rdt, p, tag, comm, MPI_STATUS_IGNORE);
    }
    return MPI_SUCCESS;
}
int PMPI_Gather(const void *s, int sc, MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, int root, MPI_Comm comm) {
    int rcs[64], displs[64];
    for (int p = 0; p < g_size; ++p) { rcs[p] = rc; displs[p] = p * rc; }
    return PMPI_Gatherv(s, sc, sdt, r, rcs, displs, rdt, root, comm);
}
int PMPI_Scatterv(const void *s, const int scs[], const int displs[], MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, int root, MPI_Comm comm) {
    const int tag = coll_tag();
    if (g_rank != root) return PMPI_Recv(r, rc, rdt, root, tag, comm, MPI_STATUS_IGNORE);
    for (int p = 0; p < g_size; ++p) {
        const char *src = (const char *)s + (size_t)displs[p] * dt_size(sdt);
        if (p == root) memcpy(r, src, (size_t)scs[p] * dt_size(sdt));
        else PMPI_Send(src, scs[p], sdt, p, tag, comm);
    }
    return MPI_SUCCESS;
}
int PMPI_Scatter(const void *s, int sc, MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, int root, MPI_Comm comm) {
    int scs[64], displs[64];
    for (int p = 0; p < g_size; ++p) { scs[p] = sc; displs[p] = p * sc; }
    return PMPI_Scatterv(s, scs, displs, sdt, r, rc, rdt, root, comm);
}
int PMPI_Allgatherv(const void *s, int sc, MPI_Datatype sdt, void *r, const int rcs[], const int displs[], MPI_Datatype rdt, MPI_Comm comm) {
    const int tag = coll_tag();
    for (int p = 0; p < g_size; ++p)
        if (p != g_rank) PMPI_Send(s, sc, sdt, p, tag, comm);
    for (int p = 0; p < g_size; ++p) {
        char *dst = (char *)r + (size_t)displs[p] * dt_size(rdt);
        if (p == g_rank) memmove(dst, s, (size_t)sc * dt_size(sdt));
        else PMPI_Recv(dst, rcs[p], rdt, p, tag, comm, MPI_STATUS_IGNORE);
    }
    return MPI_SUCCESS;
}
int PMPI_Allgather(const void *s, int sc, MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, MPI_Comm comm) {
    int rcs[64], displs[64];
    for (int p = 0; p < g_size; ++p) { rcs[p] = rc; displs[p] = p * rc; }
    return PMPI_Allgatherv(s, sc, sdt, r, rcs, displs, rdt, comm);
}
int PMPI_Alltoall(const void *s, int sc, MPI_Datatype sdt, void *r, int rc, MPI_Datatype rdt, MPI_Comm comm) {
    const int tag = coll_tag();
    const size_t sb = (size_t)sc * dt_size(sdt), rb = (size_t)rc * dt_size(rdt);
    for (int p = 0; p < g_size; ++p)
        if (p != g_rank) PMPI_Send((const char *)s + (size_t)p * sb, sc, sdt, p, tag, comm);
    for (int p = 0; p < g_size; ++p) {
        if (p == g_rank) memcpy((char *)r + (size_t)p * rb, (const char *)s + (size_t)p * sb, sb < rb ? sb : rb);
        else PMPI_Recv((char *)r + (size_t)p * rb, rc, rdt, p, tag, comm, MPI_STATUS_IGNORE);
    }
    return MPI_SUCCESS;
}
int PMPI_Reduce_scatter(const void *s, void *r, const int rcs[], MPI_Datatype dt, MPI_Op op, MPI_Comm comm) {
    int total = 0, off = 0;
    for (int p = 0; p < g_size; ++p) total += rcs[p];
    for (int p = 0; p < g_rank; ++p) off += rcs[p];
    void *full = malloc((size_t)(total ? total : 1) * dt_size(dt));
    PMPI_Allreduce(s, full, total, dt, op, comm);
    memcpy(r, (char *)full + (size_t)off * dt_size(dt), (size_t)rcs[g_rank] * dt_size(dt));
    free(full);
    return MPI_SUCCESS;
}
int PMPI_Reduce_scatter_block(const void *s, void *r, int rc, MPI_Datatype dt, MPI_Op op, MPI_Comm comm) {
    int rcs[64];
    for (int p = 0; p < g_size; ++p) rcs[p] = rc;
    return PMPI_Reduce_scatter(s, r, rcs, dt, op, comm);
}

/* MPI_X = weak alias of PMPI_X */
#define ALIAS(name) extern __typeof__(PMPI_##name) MPI_##name __attribute__((weak, alias("PMPI_" #name)));
ALIAS(Init) ALIAS(Init_thread) ALIAS(Initialized) ALIAS(Finalize) ALIAS(Abort) ALIAS(Comm_rank) ALIAS(Comm_size)
ALIAS(Get_processor_name) ALIAS(Wtime) ALIAS(Type_size) ALIAS(Barrier) ALIAS(Send) ALIAS(Recv) ALIAS(Isend) ALIAS(Irecv)
ALIAS(Wait) ALIAS(Waitall) ALIAS(Test) ALIAS(Probe) ALIAS(Iprobe) ALIAS(Get_count) ALIAS(Sendrecv) ALIAS(Reduce_local)
ALIAS(Bcast) ALIAS(Reduce) ALIAS(Allreduce) ALIAS(Gather) ALIAS(Gatherv) ALIAS(Scatter) ALIAS(Scatterv) ALIAS(Allgather)
ALIAS(Allgatherv) ALIAS(Alltoall) ALIAS(Reduce_scatter_block) ALIAS(Reduce_scatter)
