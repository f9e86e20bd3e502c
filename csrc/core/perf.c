/* perf_helper: per-function timing tables for LD_PRELOAD perf wrappers, and the
 * gendata capture of communication buffers.
 *
 * On-disk formats are those of the reference (run_codes/wrappers/src/perf_helper.c):
 *   CSV   header "func_name,<union of all columns>", values "%.6f", a cell that a
 *         function does not have (or a NaN) is left empty (:176-238); file
 *         <PERF_OUTPUT_DIR|perf_files>/<prefix>_<rank>.csv (:241-253)
 *   dump  $PERF_GENDATA_OUTPUT_DIR/<func>_<%06d occurrence>/rank_<r>.bin (:421-435)
 *   done  $PERF_GENDATA_DONE_DIR/gendata_done_<rank>, then wait up to 300 s for all
 *         ranks and _exit(0) (:437-474)
 * "duration" attributes are recorded in seconds while timestamp_us is microseconds,
 * as the analysis scripts expect. */
#define _GNU_SOURCE
#include <errno.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include "perf_helper.h"

const char *perf_output_dir(void) {
    const char *d = getenv("PERF_OUTPUT_DIR");
    return (d && *d) ? d : "perf_files";
}

static void mkdir_p(const char *path) {
    char tmp[1024];
    snprintf(tmp, sizeof(tmp), "%s", path);
    for (char *p = tmp + 1; *p; ++p)
        if (*p == '/') {
            *p = '\0';
            mkdir(tmp, 0755);
            *p = '/';
        }
    mkdir(tmp, 0755);
}

void perf_ensure_output_dir(void) { mkdir_p(perf_output_dir()); }

double perf_get_time(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + (double)ts.tv_nsec * 1e-9;
}

void perf_init(perf_state_t *s) {
    memset(s, 0, sizeof(*s));
    pthread_mutex_init(&s->lock, NULL);
    s->base_time = perf_get_time();
    s->gc_rank = -1;
    s->gc_nranks = -1;
}

void perf_destroy(perf_state_t *s) {
    pthread_mutex_lock(&s->lock);
    for (int f = 0; f < s->num_funcs; ++f) {
        perf_func_t *fn = &s->funcs[f];
        for (int c = 0; c < fn->num_cols; ++c) free(fn->col_data[c]);
        free(fn->col_data);
        fn->col_data = NULL;
    }
    s->num_funcs = 0;
    pthread_mutex_unlock(&s->lock);
    pthread_mutex_destroy(&s->lock);
}

static int find_col(perf_func_t *fn, const char *name) {
    for (int c = 0; c < fn->num_cols; ++c)
        if (!strcmp(fn->col_names[c], name)) return c;
    return -1;
}

/* New column: allocated to the table's capacity and back-filled with NaN. */
static int add_col(perf_func_t *fn, const char *name) {
    if (fn->num_cols >= PERF_COL_MAX) return -1;
    double **grown = (double **)realloc(fn->col_data, (size_t)(fn->num_cols + 1) * sizeof(double *));
    if (!grown) return -1;
    fn->col_data = grown;
    double *col = (double *)malloc((size_t)fn->entry_capacity * sizeof(double));
    if (!col) return -1;
    for (int i = 0; i < fn->entry_capacity; ++i) col[i] = NAN;
    const int c = fn->num_cols++;
    fn->col_data[c] = col;
    snprintf(fn->col_names[c], PERF_NAME_MAX, "%s", name);
    return c;
}

static perf_func_t *get_func(perf_state_t *s, const char *name) {
    for (int f = 0; f < s->num_funcs; ++f)
        if (!strcmp(s->funcs[f].name, name)) return &s->funcs[f];
    if (s->num_funcs >= PERF_MAX_FUNCS) return NULL;
    perf_func_t *fn = &s->funcs[s->num_funcs];
    memset(fn, 0, sizeof(*fn));
    snprintf(fn->name, PERF_NAME_MAX, "%s", name);
    fn->entry_capacity = PERF_INIT_CAP;
    if (add_col(fn, "timestamp_us") < 0 || add_col(fn, "call_count") < 0) return NULL;
    s->num_funcs++;
    return fn;
}

void perf_notedown(perf_state_t *s, const char *func_name, double start, int num_attrs, const perf_attr_t *attrs) {
    if (!s || !func_name) return;
    pthread_mutex_lock(&s->lock);
    perf_func_t *fn = get_func(s, func_name);
    if (!fn) {
        pthread_mutex_unlock(&s->lock);
        return;
    }
    if (fn->count >= fn->entry_capacity) {
        const int cap = fn->entry_capacity * 2;
        for (int c = 0; c < fn->num_cols; ++c) {
            double *g = (double *)realloc(fn->col_data[c], (size_t)cap * sizeof(double));
            if (!g) {
                pthread_mutex_unlock(&s->lock);
                return;
            }
            for (int i = fn->entry_capacity; i < cap; ++i) g[i] = NAN;
            fn->col_data[c] = g;
        }
        fn->entry_capacity = cap;
    }
    const int row = fn->count;
    for (int c = 0; c < fn->num_cols; ++c) fn->col_data[c][row] = NAN;
    fn->col_data[0][row] = (start - s->base_time) * 1e6;
    fn->col_data[1][row] = (double)(row + 1);
    for (int a = 0; a < num_attrs; ++a) {
        if (!attrs[a].key) continue;
        int c = find_col(fn, attrs[a].key);
        if (c < 0) c = add_col(fn, attrs[a].key);
        if (c >= 0) fn->col_data[c][row] = attrs[a].value;
    }
    fn->count++;
    s->total_records++;
    pthread_mutex_unlock(&s->lock);
}

int perf_flush_to_file(perf_state_t *s, const char *filepath) {
    if (!s || !filepath) return -1;
    pthread_mutex_lock(&s->lock);
    /* union of the column names, in order of first appearance */
    char cols[PERF_MAX_FUNCS * 4][PERF_NAME_MAX];
    int ncols = 0;
    for (int f = 0; f < s->num_funcs; ++f)
        for (int c = 0; c < s->funcs[f].num_cols; ++c) {
            int seen = 0;
            for (int k = 0; k < ncols && !seen; ++k) seen = !strcmp(cols[k], s->funcs[f].col_names[c]);
            if (!seen && ncols < PERF_MAX_FUNCS * 4) snprintf(cols[ncols++], PERF_NAME_MAX, "%s", s->funcs[f].col_names[c]);
        }
    FILE *fp = fopen(filepath, "w");
    if (!fp) {
        pthread_mutex_unlock(&s->lock);
        return -1;
    }
    fprintf(fp, "func_name");
    for (int k = 0; k < ncols; ++k) fprintf(fp, ",%s", cols[k]);
    fprintf(fp, "\n");
    for (int f = 0; f < s->num_funcs; ++f) {
        perf_func_t *fn = &s->funcs[f];
        int map[PERF_MAX_FUNCS * 4];
        for (int k = 0; k < ncols; ++k) map[k] = find_col(fn, cols[k]);
        for (int r = 0; r < fn->count; ++r) {
            fprintf(fp, "%s", fn->name);
            for (int k = 0; k < ncols; ++k) {
                if (map[k] >= 0 && !isnan(fn->col_data[map[k]][r])) fprintf(fp, ",%.6f", fn->col_data[map[k]][r]);
                else fprintf(fp, ",");
            }
            fprintf(fp, "\n");
        }
    }
    fclose(fp);
    pthread_mutex_unlock(&s->lock);
    return 0;
}

int perf_flush_to_rank_file(perf_state_t *s, int rank, const char *prefix) {
    perf_ensure_output_dir();
    char path[1024];
    snprintf(path, sizeof(path), "%s/%s_%d.csv", perf_output_dir(), prefix ? prefix : "perf", rank);
    return perf_flush_to_file(s, path);
}

/* ------------------------------------------------------------------ gendata */
static int env_int_chain(const char *const *names, int dflt) {
    for (int i = 0; names[i]; ++i) {
        const char *v = getenv(names[i]);
        if (v && *v) return atoi(v);
    }
    return dflt;
}

int perf_gendata_get_rank(void) {
    static const char *const n[] = {"OMPI_COMM_WORLD_RANK", "PMI_RANK", "SLURM_PROCID", "MV2_COMM_WORLD_RANK",
                                    "PERF_NCCL_RANK_998244353", "RANK", NULL};
    return env_int_chain(n, 0);
}
int perf_gendata_get_nranks(void) {
    static const char *const n[] = {"OMPI_COMM_WORLD_SIZE", "PMI_SIZE", "SLURM_NPROCS", "MV2_COMM_WORLD_SIZE",
                                    "WORLD_SIZE", NULL};
    return env_int_chain(n, 1);
}

/* PERF_GENDATA_TARGETS = "op:occ1,occ2;op2:occ" ; op "all" matches every function. */
int perf_gendata_load_targets(perf_state_t *s) {
    if (s->gc_loaded) return s->gc_num_entries;
    s->gc_loaded = 1;
    s->gc_num_entries = 0;
    s->gc_rank = perf_gendata_get_rank();
    s->gc_nranks = perf_gendata_get_nranks();
    const char *spec = getenv("PERF_GENDATA_TARGETS");
    if (!spec || !*spec) return 0;
    char *copy = strdup(spec), *save1 = NULL;
    for (char *ent = strtok_r(copy, ";", &save1); ent && s->gc_num_entries < 64; ent = strtok_r(NULL, ";", &save1)) {
        char *colon = strchr(ent, ':');
        if (!colon) continue;
        *colon = '\0';
        while (*ent == ' ') ++ent;
        const int e = s->gc_num_entries;
        snprintf(s->gc_ops[e], PERF_NAME_MAX, "%s", ent);
        s->gc_occ_cnt[e] = 0;
        char *save2 = NULL;
        for (char *o = strtok_r(colon + 1, ",", &save2); o && s->gc_occ_cnt[e] < 64; o = strtok_r(NULL, ",", &save2))
            s->gc_occs[e][s->gc_occ_cnt[e]++] = atoi(o);
        if (s->gc_occ_cnt[e] > 0) s->gc_num_entries++;
    }
    free(copy);
    if (s->gc_num_entries > 0) {
        /* A marker left by an earlier capture run would let the peers leave while this rank is
         * still inside a collective: every rank removes its own before its first call. */
        const char *done_dir = getenv("PERF_GENDATA_DONE_DIR");
        char mark[1024];
        snprintf(mark, sizeof(mark), "%s/gendata_done_%d", (done_dir && *done_dir) ? done_dir : "daemon_signals", s->gc_rank);
        unlink(mark);
    }
    return s->gc_num_entries;
}

static int name_matches(const char *func, const char *op) {
    if (!strcasecmp(op, "all")) return 1;
    /* "allreduce" matches MPI_Allreduce and ncclAllReduce: case-insensitive substring */
    return strcasestr(func, op) != NULL;
}

void perf_gendata_dump_if_target(perf_state_t *s, const char *func_name, const void *buf, size_t buf_size) {
    if (!s || !func_name) return;
    pthread_mutex_lock(&s->lock);
    if (!s->gc_loaded) perf_gendata_load_targets(s);
    if (s->gc_num_entries == 0) {
        pthread_mutex_unlock(&s->lock);
        return;
    }
    int fidx = -1;
    for (int f = 0; f < s->num_funcs; ++f)
        if (!strcmp(s->funcs[f].name, func_name)) fidx = f;
    if (fidx < 0) {
        perf_func_t *fn = get_func(s, func_name);
        fidx = fn ? (int)(fn - s->funcs) : -1;
    }
    if (fidx < 0) {
        pthread_mutex_unlock(&s->lock);
        return;
    }
    const int occ = ++s->gc_func_counters[fidx];
    int dumped = 0;
    for (int e = 0; e < s->gc_num_entries && !dumped; ++e) {
        if (!name_matches(func_name, s->gc_ops[e])) continue;
        for (int k = 0; k < s->gc_occ_cnt[e]; ++k) {
            if (s->gc_occs[e][k] != occ || s->gc_matched[e][k]) continue;
            s->gc_matched[e][k] = 1;
            const char *out = getenv("PERF_GENDATA_OUTPUT_DIR");
            if (!out || !*out) out = "gendata";
            char dir[1024], path[1200];
            snprintf(dir, sizeof(dir), "%s/%s_%06d", out, func_name, occ);
            mkdir_p(dir);
            snprintf(path, sizeof(path), "%s/rank_%d.bin", dir, s->gc_rank);
            FILE *fp = fopen(path, "wb");
            if (fp) {
                if (buf && buf_size) fwrite(buf, 1, buf_size, fp);
                fclose(fp);
            } else {
                fprintf(stderr, "[gendata] cannot write %s: %s\n", path, strerror(errno));
            }
            dumped = 1;
            break;
        }
    }
    int all = 1;
    for (int e = 0; e < s->gc_num_entries && all; ++e)
        for (int k = 0; k < s->gc_occ_cnt[e]; ++k)
            if (!s->gc_matched[e][k]) all = 0;
    pthread_mutex_unlock(&s->lock);
    if (!dumped || !all) return;

    /* Everything asked for has been captured: flush, mark done, wait for the peers, leave. */
    const char *done_dir = getenv("PERF_GENDATA_DONE_DIR");
    if (!done_dir || !*done_dir) done_dir = "daemon_signals";
    const char *prefix = getenv("PERF_GENDATA_CSV_PREFIX");
    perf_flush_to_rank_file(s, s->gc_rank, prefix ? prefix : "perf_function");
    mkdir_p(done_dir);
    char mark[1024];
    snprintf(mark, sizeof(mark), "%s/gendata_done_%d", done_dir, s->gc_rank);
    FILE *m = fopen(mark, "w");
    if (m) fclose(m);
    const char *limit_env = getenv("PERF_GENDATA_WAIT_SEC");
    const double limit = limit_env ? atof(limit_env) : 300.0, t0 = perf_get_time();
    for (;;) {
        int present = 0;
        for (int r = 0; r < s->gc_nranks; ++r) {
            snprintf(mark, sizeof(mark), "%s/gendata_done_%d", done_dir, r);
            present += access(mark, F_OK) == 0;
        }
        if (present >= s->gc_nranks) {
            fflush(NULL);
            _exit(0);
        }
        if (perf_get_time() - t0 > limit) {
            fprintf(stderr, "[gendata] rank %d: peers did not finish within %.0f s, continuing\n", s->gc_rank, limit);
            return;
        }
        usleep(50000);
    }
}
