/* GPU interference source: one host thread per visible GPU. Every cycle, with
 * probability STRESS_GPU_PERCENT % (deterministic LCG), it launches ONE finite burn
 * kernel (daemon_gpu_burn_launch, run_codes-side kernel in csrc/daemons/
 * daemon_gpu_burn_kernel.cu) of STRESS_GPU_ITERS read-modify-write steps per thread
 * over a buffer larger than L2 and waits for it; otherwise it sleeps
 * STRESS_GPU_CYCLE_GAP_US. The kernel leaves one CTA slot per SM free, so a
 * co-running collective is slowed down, never starved. STRESS_GPU_START_DELAY seconds
 * pass before the first launch. Counterpart of the reference's
 * userconfig/daemon_code_examples/daemon_stress_gpu_nvidia.c (:107-170). Nothing
 * here changes a GPU setting. */
#include <pthread.h>
#include <stdio.h>
#include <unistd.h>

#include "daemon_gpu_burn_kernel.h"
#include "daemon_loop.h"

static volatile int g_paused, g_quit;
static int g_percent = 50, g_iters = 100000, g_gap_us = 150;
static double g_delay;

static void *gpu_thread(void *arg) {
    const int dev = (int)(long)arg;
    void *ctx = daemon_gpu_burn_create(dev, 0);
    if (!ctx) {
        fprintf(stderr, "[daemon_stress_gpu] device %d: set-up failed\n", dev);
        return NULL;
    }
    unsigned int lcg = 12345u + (unsigned)dev * 977u;
    const double t_start = daemon_get_time();
    while (!g_quit) {
        if (g_paused || daemon_get_time() - t_start < g_delay) {
            usleep(20000);
            continue;
        }
        lcg = lcg * 1664525u + 1013904223u;
        if ((int)((lcg >> 8) % 100u) < g_percent) daemon_gpu_burn_launch(ctx, g_iters);
        else usleep((useconds_t)g_gap_us);
    }
    daemon_gpu_burn_destroy(ctx);
    return NULL;
}
int main(int argc, char **argv) {
    const double interval = daemon_interval_arg(argc, argv);
    const char *e;
    if ((e = getenv("STRESS_GPU_PERCENT"))) g_percent = atoi(e);
    if ((e = getenv("STRESS_GPU_ITERS"))) g_iters = atoi(e);
    if ((e = getenv("STRESS_GPU_CYCLE_GAP_US"))) g_gap_us = atoi(e);
    if ((e = getenv("STRESS_GPU_START_DELAY"))) g_delay = atof(e);
    const int n = daemon_gpu_burn_device_count();
    if (n <= 0) {
        fprintf(stderr, "[daemon_stress_gpu] no CUDA device\n");
        return 1;
    }
    pthread_t th[64];
    for (int i = 0; i < n && i < 64; ++i) pthread_create(&th[i], NULL, gpu_thread, (void *)(long)i);
    printf("[daemon_stress_gpu] %d GPU(s) at %d%% (iters %d)\n", n, g_percent, g_iters);
    daemon_setup_signal_handler();
    daemon_set_signal_file("daemon_signals/daemon_stress_gpu_nvidia.signal");
    while (!daemon_should_stop()) {
        const int w = daemon_check_signal_file();
        if (w == 2) break;
        g_paused = (w == 1);
        if (daemon_interruptible_sleep(interval < 0.2 ? interval : 0.2)) break;
    }
    g_quit = 1;
    for (int i = 0; i < n && i < 64; ++i) pthread_join(th[i], NULL);
    printf("[daemon_stress_gpu] stopped\n");
    return 0;
}
