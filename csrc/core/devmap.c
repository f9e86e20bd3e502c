/* rank -> device table, written to $PERF_OUTPUT_DIR/map.csv with the header
 * "rank,node,device_type,device_number" (reference: run_codes/benchmark-core/src/
 * job_device_mapper.c:56-123, which gathers over PMPI and therefore only works when
 * built with MPI). Here every rank appends its own rows under a file lock, so the
 * table also exists for NCCL-only runs; the header is written by whoever creates
 * the file. */
#define _GNU_SOURCE
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/file.h>
#include <sys/stat.h>
#include <unistd.h>

#include "job_device_mapper.h"
#include "perf_helper.h"

void device_map_init(device_map_ctx_t *ctx, int rank, int size) {
    memset(ctx, 0, sizeof(*ctx));
    ctx->rank = rank;
    ctx->size = size;
}

int device_map_add_entry(device_map_ctx_t *ctx, const char *device_type, int device_number) {
    if (!ctx || ctx->num_entries >= DEVICE_MAP_MAX_ENTRIES) return -1;
    device_map_entry_t *e = &ctx->entries[ctx->num_entries++];
    e->rank = ctx->rank;
    if (gethostname(e->node, sizeof(e->node)) != 0) snprintf(e->node, sizeof(e->node), "unknown");
    e->node[sizeof(e->node) - 1] = '\0';
    snprintf(e->device_type, sizeof(e->device_type), "%s", device_type ? device_type : "cpu");
    e->device_number = device_number;
    return 0;
}

void device_map_flush_to_file(device_map_ctx_t *ctx) {
    if (!ctx || ctx->num_entries == 0) return;
    perf_ensure_output_dir();
    char path[1024];
    snprintf(path, sizeof(path), "%s/map.csv", perf_output_dir());
    int fd = open(path, O_CREAT | O_RDWR | O_APPEND, 0644);
    if (fd < 0) return;
    flock(fd, LOCK_EX);
    struct stat st;
    char line[256];
    if (fstat(fd, &st) == 0 && st.st_size == 0) {
        const char *hdr = "rank,node,device_type,device_number\n";
        if (write(fd, hdr, strlen(hdr)) < 0) { /* best effort */ }
    }
    for (int i = 0; i < ctx->num_entries; ++i) {
        const device_map_entry_t *e = &ctx->entries[i];
        int n = snprintf(line, sizeof(line), "%d,%s,%s,%d\n", e->rank, e->node, e->device_type, e->device_number);
        if (write(fd, line, (size_t)n) < 0) break;
    }
    flock(fd, LOCK_UN);
    close(fd);
}

void device_map_destroy(device_map_ctx_t *ctx) {
    if (ctx) ctx->num_entries = 0;
}

__attribute__((weak)) void map_job_to_device(device_map_ctx_t *ctx) { (void)ctx; }
