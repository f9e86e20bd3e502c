/* Sampling daemons: a growing table of (timestamp, metrics...) samples per device,
 * cooperative control through a signal file, CSV flush. Source-compatible with the
 * reference's run_codes/daemons/include/daemon_helper.h. */
#ifndef DAEMON_HELPER_H
#define DAEMON_HELPER_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DAEMON_MAX_METRICS 10
#define DAEMON_NAME_MAX 64
#define DAEMON_UNIT_MAX 16
#define DAEMON_INIT_SAMPLES 1024

const char *daemon_output_dir(void); /* $PERF_OUTPUT_DIR or "perf_files" */

typedef struct {
    char name[DAEMON_NAME_MAX];
    char unit[DAEMON_UNIT_MAX];
} daemon_metric_def_t;

typedef struct {
    double timestamp; /* seconds since the daemon's time zero */
    double values[DAEMON_MAX_METRICS];
    int count;
} daemon_sample_t;

typedef struct {
    char device_name[DAEMON_NAME_MAX];
    daemon_metric_def_t metrics[DAEMON_MAX_METRICS];
    int num_metrics;
    daemon_sample_t *samples;
    int num_samples;
    int capacity;
    double time_zero;
} daemon_state_t;

void daemon_init(daemon_state_t *s, const char *device_name);
int daemon_add_metric(daemon_state_t *s, const char *name, const char *unit);
daemon_sample_t *daemon_new_sample(daemon_state_t *s);
/* Header "timestamp_sec,<metric...>", values "%.6f", written under an flock. */
int daemon_flush_to_file(daemon_state_t *s, const char *filepath);
void daemon_ensure_output_dir(void);
void daemon_destroy(daemon_state_t *s);

double daemon_get_time(void);
int daemon_interruptible_sleep(double seconds); /* non-zero when a stop was requested */
void daemon_get_hostname(char *buf, size_t size);

void daemon_setup_signal_handler(void); /* SIGINT / SIGTERM request a stop */
int daemon_should_stop(void);
void daemon_set_signal_file(const char *path);
/* absent or empty file = 0 (run), "PAUSE" = 1, "EXIT" / "FLUSH_EXIT" = 2 */
int daemon_check_signal_file(void);

int daemon_read_sysfs_u64(const char *path, unsigned long long *val);
int daemon_read_sysfs_str(const char *path, char *buf, size_t buf_size);

#ifdef __cplusplus
}
#endif
#endif /* DAEMON_HELPER_H */
