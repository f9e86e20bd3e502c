/* Timing tables for LD_PRELOAD perf wrappers: one table per intercepted function,
 * one row per call, columns created on first use, flushed as CSV. Also the
 * "gendata" buffer capture. Source-compatible with the reference's
 * run_codes/wrappers/include/perf_helper.h (same struct layout and entry points). */
#ifndef PERF_HELPER_H
#define PERF_HELPER_H

#include <pthread.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PERF_MAX_FUNCS 64
#define PERF_NAME_MAX 64
#define PERF_COL_MAX 32
#define PERF_INIT_CAP 1024

/* $PERF_OUTPUT_DIR or "perf_files". */
const char *perf_output_dir(void);

typedef struct {
    const char *key;
    double value;
} perf_attr_t;

typedef struct {
    char name[PERF_NAME_MAX];
    char col_names[PERF_COL_MAX][PERF_NAME_MAX];
    int num_cols;
    double **col_data; /* [num_cols][entry_capacity] */
    int count;
    int entry_capacity;
} perf_func_t;

typedef struct {
    perf_func_t funcs[PERF_MAX_FUNCS];
    int num_funcs;
    int64_t total_records;
    double base_time; /* CLOCK_MONOTONIC seconds at perf_init */
    pthread_mutex_t lock;
    /* gendata capture state */
    int gc_loaded;
    char gc_ops[64][PERF_NAME_MAX];
    int gc_occs[64][64];
    int gc_occ_cnt[64];
    int gc_num_entries;
    int gc_func_counters[PERF_MAX_FUNCS];
    int gc_matched[64][64];
    int gc_rank;
    int gc_nranks;
} perf_state_t;

void perf_init(perf_state_t *s);
/* Column 0 "timestamp_us" = (start - base_time) * 1e6, column 1 "call_count"; every
 * attribute key becomes (or reuses) a further column; missing cells are NaN. */
void perf_notedown(perf_state_t *s, const char *func_name, double start, int num_attrs, const perf_attr_t *attrs);
int perf_flush_to_file(perf_state_t *s, const char *filepath);
int perf_flush_to_rank_file(perf_state_t *s, int rank, const char *prefix);
void perf_ensure_output_dir(void);
double perf_get_time(void);
void perf_destroy(perf_state_t *s);

int perf_gendata_load_targets(perf_state_t *s);
void perf_gendata_dump_if_target(perf_state_t *s, const char *func_name, const void *buf, size_t buf_size);
int perf_gendata_get_rank(void);
int perf_gendata_get_nranks(void);

#ifdef __cplusplus
}
#endif
#endif /* PERF_HELPER_H */
