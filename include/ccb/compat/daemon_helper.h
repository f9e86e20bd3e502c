/* Sampling daemons: a growing table of (timestamp, metrics...) samples per device,
 * cooperative control through a signal file, CSV flush. Source-compatible with the
 * reference's run_codes/daemons/include/daemon_helper.h. */
#ifndef DAEMON_HELPER_H
#define DAEMON_HELPER_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ limits -- */
#define DAEMON_MAX_METRICS 10      /* columns per sample */
#define DAEMON_NAME_MAX 64         /* device and metric names */
#define DAEMON_UNIT_MAX 16
#define DAEMON_INIT_SAMPLES 1024   /* first allocation of the sample table */

/* ------------------------------------------------------------------- tables -- */
typedef struct {
    char name[DAEMON_NAME_MAX];   /* CSV column */
    char unit[DAEMON_UNIT_MAX];   /* informative, not written */
} daemon_metric_def_t;

typedef struct {
    double timestamp;                   /* seconds since the daemon's time zero */
    double values[DAEMON_MAX_METRICS];  /* one per registered metric */
    int count;
} daemon_sample_t;

typedef struct {
    char device_name[DAEMON_NAME_MAX];  /* part of the CSV file name: perf_<device>_<host>.csv */
    daemon_metric_def_t metrics[DAEMON_MAX_METRICS];
    int num_metrics;
    daemon_sample_t *samples;           /* grows by doubling from DAEMON_INIT_SAMPLES */
    int num_samples;
    int capacity;
    double time_zero;                   /* taken when the library is loaded */
} daemon_state_t;

/* ----------------------------------------------------- control of the loop -- */
void daemon_setup_signal_handler(void);          /* SIGINT / SIGTERM request a stop */
int daemon_should_stop(void);
void daemon_set_signal_file(const char *path);
int daemon_check_signal_file(void);              /* 0 run (absent or empty), 1 "PAUSE", 2 "EXIT" / "FLUSH_EXIT" */
int daemon_interruptible_sleep(double seconds);  /* non-zero when a stop was requested meanwhile */
double daemon_get_time(void);

/* ------------------------------------------------------------------ samples -- */
void daemon_init(daemon_state_t *s, const char *device_name);
int daemon_add_metric(daemon_state_t *s, const char *name, const char *unit);
daemon_sample_t *daemon_new_sample(daemon_state_t *s);
void daemon_destroy(daemon_state_t *s);

/* ------------------------------------------------------------------- output -- */
const char *daemon_output_dir(void);             /* $PERF_OUTPUT_DIR or "perf_files" */
void daemon_ensure_output_dir(void);
int daemon_flush_to_file(daemon_state_t *s, const char *filepath); /* "timestamp_sec,<metric...>", "%.6f", under an flock */

/* ------------------------------------------------------------------ sources -- */
void daemon_get_hostname(char *buf, size_t size);
int daemon_read_sysfs_u64(const char *path, unsigned long long *val);
int daemon_read_sysfs_str(const char *path, char *buf, size_t buf_size);

#ifdef __cplusplus
}
#endif
#endif /* DAEMON_HELPER_H */
