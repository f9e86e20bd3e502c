/* The main loop every sampling daemon shares: poll at a fixed interval, honour the
 * signal file (PAUSE skips sampling, EXIT / FLUSH_EXIT flushes and leaves), stop on
 * SIGINT / SIGTERM. */
#ifndef CCB_DAEMON_LOOP_H
#define CCB_DAEMON_LOOP_H
#include <stdlib.h>

#include "daemon_helper.h"

static inline double daemon_interval_arg(int argc, char **argv) {
    double iv = argc > 1 ? atof(argv[1]) : 1.0;
    return iv > 0.0 ? iv : 1.0;
}

static inline void daemon_run_loop(const char *name, double interval, void (*poll_all)(void)) {
    char sig[256];
    snprintf(sig, sizeof(sig), "daemon_signals/daemon_%s.signal", name);
    daemon_setup_signal_handler();
    daemon_set_signal_file(sig);
    daemon_ensure_output_dir();
    while (!daemon_should_stop()) {
        const int word = daemon_check_signal_file();
        if (word == 2) break;
        if (word == 1) {
            if (daemon_interruptible_sleep(interval)) break;
            continue;
        }
        const double t0 = daemon_get_time();
        poll_all();
        const double used = daemon_get_time() - t0;
        if (used < interval && daemon_interruptible_sleep(interval - used)) break;
    }
}
#endif
