/* Daemon helper: sample table, signal handling, signal-file control, sysfs readers,
 * CSV flush. Behaviour of the reference's run_codes/daemons/src/daemon_helper.c:
 * time zero taken when the library is loaded so that all daemons of a node share an
 * origin (:51-66), signal file words PAUSE / EXIT / FLUSH_EXIT (:111-141), CSV
 * "timestamp_sec,<metrics>" under flock (:214-252). */
#define _GNU_SOURCE
#include <errno.h>
#include <fcntl.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/file.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include "daemon_helper.h"

static volatile sig_atomic_t g_stop;
static char g_signal_file[512];
static double g_time_zero;

double daemon_get_time(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + (double)ts.tv_nsec * 1e-9;
}
__attribute__((constructor)) static void daemon_epoch(void) { g_time_zero = daemon_get_time(); }

const char *daemon_output_dir(void) {
    const char *d = getenv("PERF_OUTPUT_DIR");
    return (d && *d) ? d : "perf_files";
}
void daemon_ensure_output_dir(void) {
    char tmp[1024];
    snprintf(tmp, sizeof(tmp), "%s", daemon_output_dir());
    for (char *p = tmp + 1; *p; ++p)
        if (*p == '/') {
            *p = '\0';
            mkdir(tmp, 0755);
            *p = '/';
        }
    mkdir(tmp, 0755);
}

void daemon_init(daemon_state_t *s, const char *device_name) {
    memset(s, 0, sizeof(*s));
    snprintf(s->device_name, sizeof(s->device_name), "%s", device_name ? device_name : "device");
    s->time_zero = g_time_zero > 0 ? g_time_zero : daemon_get_time();
}

int daemon_add_metric(daemon_state_t *s, const char *name, const char *unit) {
    if (s->num_metrics >= DAEMON_MAX_METRICS) return -1;
    daemon_metric_def_t *m = &s->metrics[s->num_metrics];
    snprintf(m->name, sizeof(m->name), "%s", name);
    snprintf(m->unit, sizeof(m->unit), "%s", unit ? unit : "");
    return s->num_metrics++;
}

daemon_sample_t *daemon_new_sample(daemon_state_t *s) {
    if (s->num_samples >= s->capacity) {
        const int cap = s->capacity ? s->capacity * 2 : DAEMON_INIT_SAMPLES;
        daemon_sample_t *g = (daemon_sample_t *)realloc(s->samples, (size_t)cap * sizeof(*g));
        if (!g) return NULL;
        s->samples = g;
        s->capacity = cap;
    }
    daemon_sample_t *sp = &s->samples[s->num_samples++];
    memset(sp, 0, sizeof(*sp));
    sp->timestamp = daemon_get_time() - s->time_zero;
    sp->count = s->num_metrics;
    return sp;
}

int daemon_flush_to_file(daemon_state_t *s, const char *filepath) {
    daemon_ensure_output_dir();
    int fd = open(filepath, O_CREAT | O_WRONLY | O_TRUNC, 0644);
    if (fd < 0) {
        fprintf(stderr, "[daemon] cannot write %s: %s\n", filepath, strerror(errno));
        return -1;
    }
    flock(fd, LOCK_EX);
    FILE *f = fdopen(fd, "w");
    if (!f) {
        close(fd);
        return -1;
    }
    fprintf(f, "timestamp_sec");
    for (int m = 0; m < s->num_metrics; ++m) fprintf(f, ",%s", s->metrics[m].name);
    fprintf(f, "\n");
    for (int i = 0; i < s->num_samples; ++i) {
        fprintf(f, "%.6f", s->samples[i].timestamp);
        for (int m = 0; m < s->num_metrics; ++m) fprintf(f, ",%.6f", s->samples[i].values[m]);
        fprintf(f, "\n");
    }
    fflush(f);
    flock(fd, LOCK_UN);
    fclose(f);
    return 0;
}

void daemon_destroy(daemon_state_t *s) {
    free(s->samples);
    s->samples = NULL;
    s->num_samples = s->capacity = 0;
}

static void on_signal(int sig) {
    (void)sig;
    g_stop = 1;
}
void daemon_setup_signal_handler(void) {
    struct sigaction sa;
    memset(&sa, 0, sizeof(sa));
    sa.sa_handler = on_signal;
    sigaction(SIGINT, &sa, NULL);
    sigaction(SIGTERM, &sa, NULL);
}
int daemon_should_stop(void) { return g_stop != 0; }

int daemon_interruptible_sleep(double seconds) {
    const double end = daemon_get_time() + seconds;
    while (!g_stop) {
        double left = end - daemon_get_time();
        if (left <= 0) break;
        if (left > 0.05) left = 0.05; /* wake often enough to notice a stop or an EXIT word */
        struct timespec ts = {(time_t)left, (long)((left - (time_t)left) * 1e9)};
        nanosleep(&ts, NULL);
        if (g_signal_file[0] && daemon_check_signal_file() == 2) return 1;
    }
    return g_stop != 0;
}

void daemon_get_hostname(char *buf, size_t size) {
    if (gethostname(buf, size) != 0) snprintf(buf, size, "unknown");
    buf[size - 1] = '\0';
    char *dot = strchr(buf, '.');
    if (dot) *dot = '\0';
}

void daemon_set_signal_file(const char *path) { snprintf(g_signal_file, sizeof(g_signal_file), "%s", path ? path : ""); }

int daemon_check_signal_file(void) {
    if (!g_signal_file[0]) return 0;
    FILE *f = fopen(g_signal_file, "r");
    if (!f) return 0;
    char word[32] = "";
    if (!fgets(word, sizeof(word), f)) word[0] = '\0';
    fclose(f);
    word[strcspn(word, "\r\n \t")] = '\0';
    if (!strcmp(word, "PAUSE")) return 1;
    if (!strcmp(word, "EXIT") || !strcmp(word, "FLUSH_EXIT")) return 2;
    return 0;
}

int daemon_read_sysfs_u64(const char *path, unsigned long long *val) {
    FILE *f = fopen(path, "r");
    if (!f) return -1;
    int ok = fscanf(f, "%llu", val) == 1;
    fclose(f);
    return ok ? 0 : -1;
}
int daemon_read_sysfs_str(const char *path, char *buf, size_t buf_size) {
    FILE *f = fopen(path, "r");
    if (!f) return -1;
    if (!fgets(buf, (int)buf_size, f)) {
        fclose(f);
        return -1;
    }
    fclose(f);
    buf[strcspn(buf, "\r\n")] = '\0';
    return 0;
}
