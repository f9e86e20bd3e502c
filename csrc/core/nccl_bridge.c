/* NCCL benchmark bridge (no MPI).
 *
 * File and wire formats are the reference's (run_codes/benchmark-core/src/nccl/
 * nccl_utils.c): nccl_id_file/nccl_bench_id holds the raw ncclUniqueId (:71-115),
 * nccl_id_file/nccl_barrier_addr holds "host:port\n" of rank 0's barrier socket
 * (:222-327), runtime_files/nccl_agg/s<step>_r<rank> holds three doubles
 * {avg_us, errors, bw} (:478-609), and the per-size report printed by rank 0 has the
 * same lines. Differences: files are published with write-to-temp + rename so that a
 * reader never sees a partial file; the barrier hand-shake carries a 4-byte rank
 * (the reference sends one byte, limiting it to 256 ranks); RANK / WORLD_SIZE /
 * LOCAL_RANK (torchrun) end the environment chain; with -c a result CSV row
 * (msg_size,nranks,dtype,test,time_us_avg,time_us_min,time_us_max,ref_bw,busbw,
 * errors,<metrics>) is appended per size. */
#define _GNU_SOURCE
#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <unistd.h>

#include "dummy_collectives.h"
#include "nccl/nccl_utils.h"

#define ID_DIR "nccl_id_file"
#define ID_FILE ID_DIR "/nccl_bench_id"
#define BARRIER_FILE ID_DIR "/nccl_barrier_addr"
#define AGG_DIR "runtime_files/nccl_agg"
#define WAIT_TICKS 3000 /* x 10 ms = 30 s */

static int g_rank = -1;
static double g_bus_factor = 0.0;
static char g_test_name[128] = "nccl_test";

int nccl_get_my_rank(void) { return g_rank; }
void nccl_set_busbw_factor(double f) { g_bus_factor = f; }
const char *nccl_test_name(void) { return g_test_name; }

static const char *first_env(const char *const *names) {
    for (int i = 0; names[i]; ++i) {
        const char *v = getenv(names[i]);
        if (v && *v) return v;
    }
    return NULL;
}

static void rank_from_env(int *rank, int *size, int *local) {
    static const char *const r[] = {"OMPI_COMM_WORLD_RANK", "PMI_RANK", "SLURM_PROCID", "MV2_COMM_WORLD_RANK", "RANK", NULL};
    static const char *const s[] = {"OMPI_COMM_WORLD_SIZE", "PMI_SIZE", "SLURM_NPROCS", "MV2_COMM_WORLD_SIZE", "WORLD_SIZE", NULL};
    static const char *const l[] = {"OMPI_COMM_WORLD_LOCAL_RANK", "SLURM_LOCALID", "PMI_LOCAL_RANK", "MV2_COMM_WORLD_LOCAL_RANK", "LOCAL_RANK", NULL};
    const char *v;
    *rank = (v = first_env(r)) ? atoi(v) : 0;
    *size = (v = first_env(s)) ? atoi(v) : 1;
    *local = (v = first_env(l)) ? atoi(v) : *rank;
}

static int publish_file(const char *path, const void *data, size_t n) {
    char tmp[512];
    snprintf(tmp, sizeof(tmp), "%s.tmp.%d", path, (int)getpid());
    FILE *f = fopen(tmp, "wb");
    if (!f) return -1;
    size_t w = fwrite(data, 1, n, f);
    fclose(f);
    if (w != n || rename(tmp, path) != 0) {
        remove(tmp);
        return -1;
    }
    return 0;
}

static int wait_read_file(const char *path, void *data, size_t n, size_t *got) {
    struct stat st;
    for (int t = 0; t < WAIT_TICKS; ++t) {
        if (stat(path, &st) == 0 && st.st_size > 0 && (size_t)st.st_size >= (got ? 1 : n)) {
            FILE *f = fopen(path, "rb");
            if (f) {
                size_t r = fread(data, 1, n, f);
                fclose(f);
                if (got) *got = r;
                if (got ? r > 0 : r == n) return 0;
            }
        }
        usleep(10000);
    }
    return -1;
}

static ncclComm_t make_comm(int rank, int size) {
    ncclUniqueId id;
    memset(&id, 0, sizeof(id));
    if (size == 1 || rank == 0) {
        if (rank == 0 && size > 1) printf("[nccl] Generating NCCL unique ID...\n");
        NCCLCHECK(ncclGetUniqueId(&id));
        if (size > 1) {
            mkdir(ID_DIR, 0755);
            if (publish_file(ID_FILE, &id, sizeof(id)) != 0) {
                perror("publish " ID_FILE);
                exit(1);
            }
        }
    } else {
        printf("[nccl] Waiting for NCCL unique ID from rank 0...\n");
        if (wait_read_file(ID_FILE, &id, sizeof(id), NULL) != 0) {
            fprintf(stderr, "Rank %d: timeout waiting for NCCL id\n", rank);
            exit(1);
        }
    }
    printf("[nccl] Creating NCCL communicator (%d ranks)...\n", size);
    ncclComm_t comm;
    NCCLCHECK(ncclCommInitRank(&comm, size, id, rank));
    printf("[nccl] NCCL communicator created\n");
    return comm;
}

/* ------------------------------------------------------------- TCP barrier -- */
static int send_all(int fd, const void *p, size_t n) {
    const char *c = (const char *)p;
    while (n) {
        ssize_t w = send(fd, c, n, MSG_NOSIGNAL);
        if (w <= 0) {
            if (w < 0 && errno == EINTR) continue;
            return -1;
        }
        c += w;
        n -= (size_t)w;
    }
    return 0;
}
static int recv_all(int fd, void *p, size_t n) {
    char *c = (char *)p;
    while (n) {
        ssize_t r = recv(fd, c, n, 0);
        if (r <= 0) {
            if (r < 0 && errno == EINTR) continue;
            return -1;
        }
        c += r;
        n -= (size_t)r;
    }
    return 0;
}

static void barrier_init(nccl_test_context_t *ctx) {
    for (int i = 0; i < 256; ++i) ctx->barrier_peers[i] = -1;
    ctx->barrier_listen_fd = -1;
    if (ctx->size <= 1) return;
    if (ctx->size > 256) {
        fprintf(stderr, "[nccl] barrier supports at most 256 ranks\n");
        exit(1);
    }
    int one = 1;
    if (ctx->rank == 0) {
        int ls = socket(AF_INET, SOCK_STREAM, 0);
        struct sockaddr_in a;
        memset(&a, 0, sizeof(a));
        a.sin_family = AF_INET;
        a.sin_addr.s_addr = htonl(INADDR_ANY);
        a.sin_port = 0;
        setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        if (ls < 0 || bind(ls, (struct sockaddr *)&a, sizeof(a)) != 0 || listen(ls, ctx->size) != 0) {
            perror("[nccl] barrier listen");
            exit(1);
        }
        socklen_t alen = sizeof(a);
        getsockname(ls, (struct sockaddr *)&a, &alen);
        char host[256], line[320];
        if (gethostname(host, sizeof(host)) != 0) snprintf(host, sizeof(host), "127.0.0.1");
        const char *force = getenv("CCB_BARRIER_HOST");
        int n = snprintf(line, sizeof(line), "%s:%d\n", force ? force : host, (int)ntohs(a.sin_port));
        mkdir(ID_DIR, 0755);
        if (publish_file(BARRIER_FILE, line, (size_t)n) != 0) {
            perror("publish " BARRIER_FILE);
            exit(1);
        }
        ctx->barrier_listen_fd = ls;
        for (int k = 1; k < ctx->size; ++k) {
            int fd = accept(ls, NULL, NULL);
            uint32_t r = 0;
            if (fd < 0 || recv_all(fd, &r, sizeof(r)) != 0 || ntohl(r) == 0 || ntohl(r) >= (uint32_t)ctx->size) {
                fprintf(stderr, "[nccl] barrier: bad peer hand-shake\n");
                exit(1);
            }
            setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            ctx->barrier_peers[ntohl(r)] = fd;
        }
        close(ls);
        ctx->barrier_listen_fd = -1;
    } else {
        char line[320];
        size_t got = 0;
        memset(line, 0, sizeof(line));
        if (wait_read_file(BARRIER_FILE, line, sizeof(line) - 1, &got) != 0 || !strchr(line, ':')) {
            fprintf(stderr, "Rank %d: timeout waiting for the barrier address\n", ctx->rank);
            exit(1);
        }
        char *colon = strrchr(line, ':');
        *colon = '\0';
        const int port = atoi(colon + 1);
        struct addrinfo hints, *res = NULL;
        memset(&hints, 0, sizeof(hints));
        hints.ai_family = AF_INET;
        hints.ai_socktype = SOCK_STREAM;
        char portstr[16];
        snprintf(portstr, sizeof(portstr), "%d", port);
        if (getaddrinfo(line, portstr, &hints, &res) != 0 || !res) {
            /* the container hostname may not resolve: ranks of one host talk over loopback */
            if (getaddrinfo("127.0.0.1", portstr, &hints, &res) != 0 || !res) {
                fprintf(stderr, "Rank %d: cannot resolve barrier host '%s'\n", ctx->rank, line);
                exit(1);
            }
        }
        int fd = -1;
        for (int t = 0; t < WAIT_TICKS; ++t) {
            fd = socket(AF_INET, SOCK_STREAM, 0);
            if (fd >= 0 && connect(fd, res->ai_addr, res->ai_addrlen) == 0) break;
            if (fd >= 0) close(fd);
            fd = -1;
            usleep(10000);
        }
        freeaddrinfo(res);
        if (fd < 0) {
            fprintf(stderr, "Rank %d: cannot connect to the barrier socket\n", ctx->rank);
            exit(1);
        }
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        uint32_t r = htonl((uint32_t)ctx->rank);
        send_all(fd, &r, sizeof(r));
        ctx->barrier_peers[0] = fd;
    }
}

void nccl_barrier(nccl_test_context_t *ctx) {
    if (ctx->size <= 1) return;
    char b = 1;
    if (ctx->rank == 0) {
        for (int r = 1; r < ctx->size; ++r)
            if (recv_all(ctx->barrier_peers[r], &b, 1) != 0) {
                fprintf(stderr, "[nccl] barrier: lost rank %d\n", r);
                exit(1);
            }
        for (int r = 1; r < ctx->size; ++r)
            if (send_all(ctx->barrier_peers[r], &b, 1) != 0) {
                fprintf(stderr, "[nccl] barrier: lost rank %d\n", r);
                exit(1);
            }
    } else {
        if (send_all(ctx->barrier_peers[0], &b, 1) != 0 || recv_all(ctx->barrier_peers[0], &b, 1) != 0) {
            fprintf(stderr, "[nccl] barrier: lost rank 0\n");
            exit(1);
        }
    }
}

/* ----------------------------------------------------------------- lifecycle */
nccl_test_context_t nccl_test_init(int argc, char **argv, const char *test_name) {
    nccl_test_context_t ctx;
    memset(&ctx, 0, sizeof(ctx));
    int local = 0;
    rank_from_env(&ctx.rank, &ctx.size, &local);
    g_rank = ctx.rank;
    if (test_name) snprintf(g_test_name, sizeof(g_test_name), "%s", test_name);
    char buf[16];
    snprintf(buf, sizeof(buf), "%d", ctx.rank);
    setenv("PERF_NCCL_RANK_998244353", buf, 1);

    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev < 1) {
        fprintf(stderr, "Rank %d: no CUDA device\n", ctx.rank);
        exit(1);
    }
    cudaSetDevice(local % ndev);
    barrier_init(&ctx);
    ctx.comm = make_comm(ctx.rank, ctx.size);
    cudaStreamCreate(&ctx.stream);
    nccl_barrier(&ctx);
    ctx.config = parse_arguments(argc, argv);
    if (ctx.rank == 0) {
        printf("=== %s Test ===\n", test_name ? test_name : "NCCL");
        printf("Ranks: %d\n", ctx.size);
        if (ctx.config.use_size_list) {
            printf("Message sizes (list):");
            for (int i = 0; i < ctx.config.num_sizes; ++i) printf(" %zu", ctx.config.size_list[i]);
            printf("\n");
        } else {
            printf("Message sizes: %zu to %zu (%s %d)\n", ctx.config.min_message_size, ctx.config.max_message_size,
                   ctx.config.message_size_incr_mode ? "+" : "x", ctx.config.message_size_incr);
        }
        printf("Iterations: %d (warmup: %d)\n", ctx.config.iterations, ctx.config.warmup_iterations);
        printf("Validation: %s\n", ctx.config.validate ? "enabled" : "disabled");
        if (ctx.config.input_file) printf("Input file: %s\n", ctx.config.input_file);
        printf("Tolerance: %e\n\n", ctx.config.tolerance);
    }
    return ctx;
}

void nccl_test_fini(nccl_test_context_t *ctx) {
    nccl_barrier(ctx);
    if (ctx->rank == 0) printf("=== Test Complete ===\n");
    for (int i = 0; i < 256; ++i)
        if (ctx->barrier_peers[i] >= 0) close(ctx->barrier_peers[i]);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    if (ctx->comm) ncclCommDestroy(ctx->comm);
}

void nccl_load_input(const nccl_test_context_t *ctx, void *buf, size_t msg_size, ncclDataType_t datatype) {
    dummy_load_rank_data(ctx->config.input_file, nccl_to_data_type(datatype), ctx->config.pattern_type, buf, msg_size,
                         ctx->rank, ctx->size);
}

/* ----------------------------------------------------------------- reporting */
static const char *dtype_name(data_type_t t) {
    return t == TYPE_INT ? "int" : t == TYPE_FLOAT ? "float" : t == TYPE_DOUBLE ? "double" : t == TYPE_BFLOAT16 ? "bfloat16"
           : t == TYPE_HALF ? "half" : "char";
}

void nccl_report_results(const nccl_test_context_t *ctx, size_t msg_size, int count, float total_time_ms,
                         int local_errors, const validation_result_t *metrics, double bw) {
    static int step = 0;
    const int n = ctx->size, rank = ctx->rank;
    const double avg_us = ctx->config.iterations > 0 ? (double)total_time_ms / ctx->config.iterations * 1000.0 : 0.0;
    double mn = avg_us, mx = avg_us, mean = avg_us, bmn = bw, bmx = bw, bmean = bw;
    int errors = local_errors;
    if (n > 1) {
        mkdir("runtime_files", 0755);
        mkdir(AGG_DIR, 0755);
        double mine[3] = {avg_us, (double)local_errors, bw};
        char path[256];
        snprintf(path, sizeof(path), AGG_DIR "/s%d_r%d", step, rank);
        if (publish_file(path, mine, sizeof(mine)) != 0) {
            perror("[agg] write");
            return;
        }
        double sum = 0, bsum = 0;
        errors = 0;
        for (int r = 0; r < n; ++r) {
            double d[3];
            if (r == rank) memcpy(d, mine, sizeof(d));
            else {
                snprintf(path, sizeof(path), AGG_DIR "/s%d_r%d", step, r);
                if (wait_read_file(path, d, sizeof(d), NULL) != 0) {
                    fprintf(stderr, "[agg] timeout waiting for %s\n", path);
                    return;
                }
            }
            sum += d[0];
            bsum += d[2];
            errors += (int)d[1];
            if (r == 0 || d[0] < mn) mn = d[0];
            if (r == 0 || d[0] > mx) mx = d[0];
            if (r == 0 || d[2] < bmn) bmn = d[2];
            if (r == 0 || d[2] > bmx) bmx = d[2];
        }
        mean = sum / n;
        bmean = bsum / n;
    }
    step++;
    if (rank != 0) return;
    printf("Size: %8zu bytes (%6d elements)\n", msg_size, count);
    if (n > 1) {
        printf("  User: avg=%8.2f us, min=%8.2f us, max=%8.2f us\n", mean, mn, mx);
        printf("  Bandwidth: avg=%8.2f GB/s, min=%8.2f GB/s, max=%8.2f GB/s\n", bmean, bmn, bmx);
    } else {
        printf("  User: avg=%8.2f us\n", avg_us);
        printf("  Bandwidth: %8.2f GB/s\n", bw);
    }
    if (ctx->config.validate) {
        printf("  Correct: %s\n", errors == 0 ? "YES" : "NO");
        if (metrics && ctx->config.compute_metrics && metrics->num_elements > 0)
            for (int i = 0; i < validation_registry_count() && i < MAX_METRICS; ++i)
                if (ctx->config.metrics_mask & (1u << i)) printf("  %s: %.6e\n", validation_metric_name(i), metrics->values[i]);
    }
    printf("\n");
    if (ctx->config.save_csv) {
        char path[600], header[1024], row[2048];
        if (ctx->config.csv_path[0]) snprintf(path, sizeof(path), "%s", ctx->config.csv_path);
        else snprintf(path, sizeof(path), "results/%s.csv", g_test_name);
        int h = snprintf(header, sizeof(header),
                         "msg_size,nranks,dtype,test,time_us_avg,time_us_min,time_us_max,ref_bw,busbw,errors");
        /* max time over ranks defines the bus bandwidth (slowest rank bounds the collective) */
        const double busbw = (g_bus_factor > 0 && mx > 0) ? (double)msg_size / (mx * 1e-6) / 1e9 * g_bus_factor : 0.0;
        int w = snprintf(row, sizeof(row), "%zu,%d,%s,%s,%.2f,%.2f,%.2f,%.2f,%.2f,%d", msg_size, n,
                         dtype_name(ctx->config.data_type), g_test_name, mean, mn, mx, bmean, busbw, errors);
        for (int i = 0; i < validation_registry_count() && i < MAX_METRICS; ++i)
            if (ctx->config.compute_metrics && (ctx->config.metrics_mask & (1u << i))) {
                h += snprintf(header + h, sizeof(header) - (size_t)h, ",%s", validation_metric_name(i));
                w += snprintf(row + w, sizeof(row) - (size_t)w, ",%.6e", metrics ? metrics->values[i] : 0.0);
            }
        nccl_csv_write(path, header, "%s", row);
    }
}

void nccl_csv_write(const char *path, const char *header, const char *fmt, ...) {
    if (g_rank > 0 || !path) return;
    char dir[600];
    snprintf(dir, sizeof(dir), "%s", path);
    char *slash = strrchr(dir, '/');
    if (slash) {
        *slash = '\0';
        if (dir[0]) mkdir(dir, 0755);
    }
    const int fresh = access(path, F_OK) != 0;
    FILE *f = fopen(path, "a");
    if (!f) {
        fprintf(stderr, "[csv] cannot open %s: %s\n", path, strerror(errno));
        return;
    }
    if (fresh && header) fprintf(f, "%s\n", header);
    va_list ap;
    va_start(ap, fmt);
    vfprintf(f, fmt, ap);
    va_end(ap);
    fprintf(f, "\n");
    fclose(f);
}

/* ------------------------------------------------------------------- types -- */
data_type_t nccl_to_data_type(ncclDataType_t t) {
    switch (t) {
        case ncclInt32: case ncclUint32: return TYPE_INT;
        case ncclFloat32: return TYPE_FLOAT;
        case ncclFloat64: case ncclInt64: case ncclUint64: return TYPE_DOUBLE; /* 8-byte elements, as the reference maps them */
        case ncclFloat16: return TYPE_HALF;
#if defined(__CUDA_BF16_TYPES_EXIST__) || defined(NCCL_BF16_TYPES_EXIST) || NCCL_VERSION_CODE >= 21000
        case ncclBfloat16: return TYPE_BFLOAT16;
#endif
        default: return TYPE_CHAR;
    }
}
ncclDataType_t data_type_to_nccl(data_type_t t) {
    switch (t) {
        case TYPE_INT: return ncclInt32;
        case TYPE_FLOAT: return ncclFloat32;
        case TYPE_DOUBLE: return ncclFloat64;
        case TYPE_HALF: return ncclFloat16;
#if defined(__CUDA_BF16_TYPES_EXIST__) || defined(NCCL_BF16_TYPES_EXIST) || NCCL_VERSION_CODE >= 21000
        case TYPE_BFLOAT16: return ncclBfloat16;
#endif
        default: return ncclInt8;
    }
}
size_t nccl_dtype_size(ncclDataType_t t) {
    switch (t) {
        case ncclInt8: case ncclUint8: return 1;
        case ncclFloat16: return 2;
#if defined(__CUDA_BF16_TYPES_EXIST__) || defined(NCCL_BF16_TYPES_EXIST) || NCCL_VERSION_CODE >= 21000
        case ncclBfloat16: return 2;
#endif
        case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
        case ncclInt64: case ncclUint64: case ncclFloat64: return 8;
        default: return 1;
    }
}

int *nccl_parse_env_int_array(const char *env_name, int expected_len, int *out_len) {
    if (out_len) *out_len = 0;
    const char *s = getenv(env_name);
    if (!s || !*s) return NULL;
    int cap = 16, n = 0;
    int *v = (int *)malloc((size_t)cap * sizeof(int));
    char *copy = strdup(s), *save = NULL;
    for (char *tok = strtok_r(copy, ", ", &save); tok; tok = strtok_r(NULL, ", ", &save)) {
        if (n == cap) v = (int *)realloc(v, (size_t)(cap *= 2) * sizeof(int));
        v[n++] = atoi(tok);
    }
    free(copy);
    if (expected_len > 0 && n != expected_len) {
        fprintf(stderr, "[nccl] %s: expected %d values, got %d\n", env_name, expected_len, n);
        free(v);
        return NULL;
    }
    if (out_len) *out_len = n;
    return v;
}
