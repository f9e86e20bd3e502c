/* Host interface of the GPU burn kernel used by daemon_stress_gpu_nvidia (same role
 * as the reference's run_codes/daemons/include/daemon_gpu_burn_kernel.h). */
#ifndef DAEMON_GPU_BURN_KERNEL_H
#define DAEMON_GPU_BURN_KERNEL_H
#ifdef __cplusplus
extern "C" {
#endif
int daemon_gpu_burn_device_count(void);
/* buffer_bytes == 0 picks four times the device's L2 size (at least 256 MiB). */
void *daemon_gpu_burn_create(int device, unsigned long long buffer_bytes);
/* One finite launch of `iters` steps per thread, waited for. Returns 0 on success. */
int daemon_gpu_burn_launch(void *ctx, int iters);
void daemon_gpu_burn_destroy(void *ctx);
#ifdef __cplusplus
}
#endif
#endif
