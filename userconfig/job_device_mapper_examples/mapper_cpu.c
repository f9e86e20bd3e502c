/* Mapper: the CPUs this rank may run on (sched_getaffinity), one entry per CPU.
 * Named mapper_<daemon>: it is built when the daemon "cpu" is selected (reference:
 * userconfig/job_device_mapper_examples/mapper_cpu.c:25-50). */
#define _GNU_SOURCE
#include <sched.h>

#include "job_device_mapper.h"

void map_job_to_device_cpu(device_map_ctx_t *ctx) {
    cpu_set_t set;
    CPU_ZERO(&set);
    if (sched_getaffinity(0, sizeof(set), &set) != 0) return;
    for (int c = 0; c < CPU_SETSIZE; ++c)
        if (CPU_ISSET(c, &set)) device_map_add_entry(ctx, "cpu", c);
}
