/* rank -> (node, device type, device number) table written as perf_files/map.csv.
 * Source-compatible with the reference's
 * run_codes/benchmark-core/include/job_device_mapper.h. */
#ifndef JOB_DEVICE_MAPPER_H
#define JOB_DEVICE_MAPPER_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DEVICE_MAP_MAX_ENTRIES 4096
#define DEVICE_MAP_NODE_NAME_MAX 64
#define DEVICE_MAP_TYPE_MAX 16

typedef struct {
    int rank;
    char node[DEVICE_MAP_NODE_NAME_MAX];
    char device_type[DEVICE_MAP_TYPE_MAX]; /* "cpu" or "gpu" */
    int device_number;
} device_map_entry_t;

typedef struct {
    int rank;
    int size;
    device_map_entry_t entries[DEVICE_MAP_MAX_ENTRIES];
    int num_entries;
} device_map_ctx_t;

void device_map_init(device_map_ctx_t *ctx, int rank, int size);
int device_map_add_entry(device_map_ctx_t *ctx, const char *device_type, int device_number);
/* With MPI the entries are gathered on rank 0; without it every rank appends its own
 * rows to $PERF_OUTPUT_DIR/map.csv under a file lock. */
void device_map_flush_to_file(device_map_ctx_t *ctx);
void device_map_destroy(device_map_ctx_t *ctx);
/* Weak default does nothing; mappers (mapper_cpu, mapper_gpu_nvidia) override it. */
void map_job_to_device(device_map_ctx_t *ctx);

#ifdef __cplusplus
}
#endif
#endif /* JOB_DEVICE_MAPPER_H */
