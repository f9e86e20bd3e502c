/* MPI benchmark bridge. Mirrors the reference's run_codes/benchmark-core/src/mpi/
 * mpi_utils.c: mpi_test_init = PMPI_Init + device mapper + argv + banner (:31-84),
 * inputs from a file with offsets, a folder or a pattern (:166-229), the per-size
 * report with times reduced over the ranks by PMPI_Reduce (:231-263), rank-0 CSV
 * append with the header written only for a new file (:344-372). All housekeeping
 * goes through PMPI_* so that an interposed MPI_* wrapper never sees it. */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>
#include <sys/stat.h>
#include <unistd.h>

#include "dummy_collectives.h"
#include "job_device_mapper.h"
#include "mpi/mpi_utils.h"

static int g_rank;
static char g_test[128] = "mpi_test";
static double g_ref_bw, g_bus_factor;

void mpi_set_bandwidth(double ref_bw_gbs, double busbw_factor) {
    g_ref_bw = ref_bw_gbs;
    g_bus_factor = busbw_factor;
}

data_type_t mpi_to_data_type(MPI_Datatype t) {
    if (t == MPI_INT) return TYPE_INT;
    if (t == MPI_FLOAT) return TYPE_FLOAT;
    if (t == MPI_DOUBLE) return TYPE_DOUBLE;
    return TYPE_CHAR;
}
MPI_Datatype data_type_to_mpi(data_type_t t) {
    switch (t) {
        case TYPE_INT: return MPI_INT;
        case TYPE_FLOAT: return MPI_FLOAT;
        case TYPE_DOUBLE: return MPI_DOUBLE;
        default: return MPI_CHAR;
    }
}
MPI_Op parse_mpi_op(const char *name) {
    if (!name || !strcasecmp(name, "sum")) return MPI_SUM;
    if (!strcasecmp(name, "prod")) return MPI_PROD;
    if (!strcasecmp(name, "max")) return MPI_MAX;
    if (!strcasecmp(name, "min")) return MPI_MIN;
    fprintf(stderr, "Unknown op '%s' (sum, prod, max, min)\n", name);
    exit(1);
}

static void run_device_mapper(int rank, int size) {
    char path[4096];
    const char *bd = getenv("BENCH_DIR");
    snprintf(path, sizeof(path), "%s/bin/libs/libjob_device_mapper.so", bd ? bd : ".");
    void *h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    void (*init)(device_map_ctx_t *, int, int) = (void (*)(device_map_ctx_t *, int, int))dlsym(h, "device_map_init");
    void (*map)(device_map_ctx_t *) = (void (*)(device_map_ctx_t *))dlsym(h, "map_job_to_device");
    void (*flush)(device_map_ctx_t *) = (void (*)(device_map_ctx_t *))dlsym(h, "device_map_flush_to_file");
    if (init && map && flush) {
        device_map_ctx_t *ctx = (device_map_ctx_t *)calloc(1, sizeof(*ctx));
        if (ctx) {
            init(ctx, rank, size);
            map(ctx);
            flush(ctx);
            free(ctx);
        }
    }
}

mpi_test_context_t mpi_test_init(int argc, char **argv, const char *test_name) {
    mpi_test_context_t ctx;
    memset(&ctx, 0, sizeof(ctx));
    PMPI_Init(&argc, &argv);
    PMPI_Comm_rank(MPI_COMM_WORLD, &ctx.rank);
    PMPI_Comm_size(MPI_COMM_WORLD, &ctx.size);
    g_rank = ctx.rank;
    if (test_name) snprintf(g_test, sizeof(g_test), "%s", test_name);
    run_device_mapper(ctx.rank, ctx.size);
    ctx.config = parse_arguments(argc, argv);
    if (ctx.rank == 0) {
        printf("=== %s Test ===\nRanks: %d\n", test_name ? test_name : "MPI", ctx.size);
        printf("Iterations: %d (warmup: %d)\n", ctx.config.iterations, ctx.config.warmup_iterations);
        printf("Validation: %s\nTolerance: %e\n\n", ctx.config.validate ? "enabled" : "disabled", ctx.config.tolerance);
    }
    return ctx;
}

void mpi_test_fini(const mpi_test_context_t *ctx) {
    PMPI_Barrier(MPI_COMM_WORLD);
    if (ctx->rank == 0) printf("=== Test Complete ===\n");
    PMPI_Finalize();
}

void mpi_load_input(const mpi_test_context_t *ctx, void *buf, size_t msg_size, MPI_Datatype datatype) {
    dummy_load_rank_data(ctx->config.input_file, mpi_to_data_type(datatype), ctx->config.pattern_type, buf, msg_size,
                         ctx->rank, ctx->size);
}

static const char *dtype_name(data_type_t t) {
    return t == TYPE_INT ? "int" : t == TYPE_FLOAT ? "float" : t == TYPE_DOUBLE ? "double" : t == TYPE_BFLOAT16 ? "bfloat16"
           : t == TYPE_HALF ? "half" : "char";
}

void mpi_report_results(const mpi_test_context_t *ctx, size_t msg_size, int count, double total_time_user,
                        int local_errors, const validation_result_t *metrics) {
    const double mine = ctx->config.iterations > 0 ? total_time_user / ctx->config.iterations * 1e6 : 0.0;
    double mn = mine, mx = mine, sum = mine;
    int errors = local_errors;
    PMPI_Reduce(&mine, &mn, 1, MPI_DOUBLE, MPI_MIN, 0, MPI_COMM_WORLD);
    PMPI_Reduce(&mine, &mx, 1, MPI_DOUBLE, MPI_MAX, 0, MPI_COMM_WORLD);
    PMPI_Reduce(&mine, &sum, 1, MPI_DOUBLE, MPI_SUM, 0, MPI_COMM_WORLD);
    PMPI_Reduce(&local_errors, &errors, 1, MPI_INT, MPI_SUM, 0, MPI_COMM_WORLD);
    if (ctx->rank != 0) return;
    const double avg = sum / ctx->size;
    printf("Size: %8zu bytes (%6d elements)\n", msg_size, count);
    printf("  User: avg=%8.2f us, min=%8.2f us, max=%8.2f us\n", avg, mn, mx);
    if (g_ref_bw > 0) printf("  Bandwidth: %8.2f GB/s\n", g_ref_bw);
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
        else snprintf(path, sizeof(path), "results/%s.csv", g_test);
        int h = snprintf(header, sizeof(header), "msg_size,nranks,dtype,test,time_us_avg,time_us_min,time_us_max,ref_bw,busbw,errors");
        const double bus = (g_bus_factor > 0 && mx > 0) ? (double)msg_size / (mx * 1e-6) / 1e9 * g_bus_factor : 0.0;
        int w = snprintf(row, sizeof(row), "%zu,%d,%s,%s,%.2f,%.2f,%.2f,%.2f,%.2f,%d", msg_size, ctx->size,
                         dtype_name(ctx->config.data_type), g_test, avg, mn, mx, g_ref_bw, bus, errors);
        for (int i = 0; i < validation_registry_count() && i < MAX_METRICS; ++i)
            if (ctx->config.compute_metrics && (ctx->config.metrics_mask & (1u << i))) {
                h += snprintf(header + h, sizeof(header) - (size_t)h, ",%s", validation_metric_name(i));
                w += snprintf(row + w, sizeof(row) - (size_t)w, ",%.6e", metrics ? metrics->values[i] : 0.0);
            }
        mpi_csv_write(path, header, "%s", row);
    }
}

int *parse_env_int_array(const char *env_name, int expected_len, int *out_len) {
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
        fprintf(stderr, "%s: expected %d values, got %d\n", env_name, expected_len, n);
        free(v);
        return NULL;
    }
    if (out_len) *out_len = n;
    return v;
}

void mpi_csv_write(const char *path, const char *header, const char *fmt, ...) {
    if (g_rank != 0 || !path) return;
    char dir[600];
    snprintf(dir, sizeof(dir), "%s", path);
    char *slash = strrchr(dir, '/');
    if (slash) {
        *slash = '\0';
        if (dir[0]) mkdir(dir, 0755);
    }
    const int fresh = access(path, F_OK) != 0;
    FILE *f = fopen(path, "a");
    if (!f) return;
    if (fresh && header) fprintf(f, "%s\n", header);
    va_list ap;
    va_start(ap, fmt);
    vfprintf(f, fmt, ap);
    va_end(ap);
    fprintf(f, "\n");
    fclose(f);
}
