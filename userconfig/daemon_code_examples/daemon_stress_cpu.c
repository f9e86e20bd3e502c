/* CPU interference source: one thread per online core spins for STRESS_CPU_PERCENT %
 * of every 100 ms window and sleeps the rest. Stops on SIGINT/SIGTERM or an EXIT word
 * in daemon_signals/daemon_stress_cpu.signal; PAUSE idles the threads. Counterpart of
 * the reference's userconfig/daemon_code_examples/daemon_stress_cpu.c (:28, 60-70). */
#include <pthread.h>
#include <stdio.h>
#include <time.h>
#include <unistd.h>

#include "daemon_loop.h"

static volatile int g_paused, g_quit;
static int g_percent = 50;

static void *spin(void *arg) {
    (void)arg;
    volatile double x = 1.0;
    while (!g_quit) {
        if (g_paused || g_percent <= 0) {
            usleep(100000);
            continue;
        }
        const double t0 = daemon_get_time(), busy = 0.1 * g_percent / 100.0;
        while (daemon_get_time() - t0 < busy) x = x * 1.0000001 + 1e-9;
        const double rest = 0.1 - busy;
        if (rest > 0) usleep((useconds_t)(rest * 1e6));
    }
    return NULL;
}
static void poll_all(void) {}
int main(int argc, char **argv) {
    const double interval = daemon_interval_arg(argc, argv);
    const char *p = getenv("STRESS_CPU_PERCENT");
    if (p) g_percent = atoi(p);
    if (g_percent > 100) g_percent = 100;
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    const char *lim = getenv("STRESS_CPU_THREADS");
    if (lim && atoi(lim) > 0 && atoi(lim) < n) n = atoi(lim);
    if (n < 1) n = 1;
    pthread_t *th = (pthread_t *)calloc((size_t)n, sizeof(pthread_t));
    for (long i = 0; i < n; ++i) pthread_create(&th[i], NULL, spin, NULL);
    printf("[daemon_stress_cpu] %ld thread(s) at %d%%\n", n, g_percent);
    char sig[256];
    snprintf(sig, sizeof(sig), "daemon_signals/daemon_stress_cpu.signal");
    daemon_setup_signal_handler();
    daemon_set_signal_file(sig);
    while (!daemon_should_stop()) {
        const int w = daemon_check_signal_file();
        if (w == 2) break;
        g_paused = (w == 1);
        if (daemon_interruptible_sleep(interval < 0.2 ? interval : 0.2)) break;
    }
    g_quit = 1;
    for (long i = 0; i < n; ++i) pthread_join(th[i], NULL);
    free(th);
    (void)poll_all;
    printf("[daemon_stress_cpu] stopped\n");
    return 0;
}
