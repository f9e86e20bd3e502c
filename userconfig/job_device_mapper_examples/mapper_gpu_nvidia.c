/* Mapper: the CUDA device this rank uses. cudaGetDevice is looked up at run time so
 * that the mapper library has no link-time dependency on the CUDA runtime
 * (reference: userconfig/job_device_mapper_examples/mapper_gpu_nvidia.c:26-33). */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdlib.h>

#include "job_device_mapper.h"

void map_job_to_device_gpu_nvidia(device_map_ctx_t *ctx) {
    int (*get_device)(int *) = (int (*)(int *))dlsym(RTLD_DEFAULT, "cudaGetDevice");
    int dev = -1;
    if (get_device && get_device(&dev) == 0 && dev >= 0) {
        device_map_add_entry(ctx, "gpu", dev);
        return;
    }
    const char *lr = getenv("OMPI_COMM_WORLD_LOCAL_RANK");
    if (!lr) lr = getenv("SLURM_LOCALID");
    if (!lr) lr = getenv("LOCAL_RANK");
    if (lr) device_map_add_entry(ctx, "gpu", atoi(lr));
}
