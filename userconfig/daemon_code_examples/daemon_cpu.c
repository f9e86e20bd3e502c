/* CPU and memory monitor: /proc/stat deltas (aggregate and per core) and
 * /proc/meminfo. Writes perf_cpu_<host>.csv (aggregate: util %, user %, system %,
 * iowait %, mem_used MB, mem_util %) and perf_cpu_<N>_<host>.csv per core (util %).
 * Same outputs as the reference's userconfig/daemon_code_examples/daemon_cpu.c. */
#include <stdio.h>
#include <string.h>

#include "daemon_loop.h"

#define MAX_CORES 1024
typedef struct { unsigned long long user, nice, sys, idle, iowait, irq, softirq, steal; } cpu_times_t;
static daemon_state_t g_total, g_core[MAX_CORES];
static cpu_times_t g_prev_total, g_prev_core[MAX_CORES];
static int g_ncores, g_have_prev;

static int read_stat(cpu_times_t *total, cpu_times_t *cores, int max) {
    FILE *f = fopen("/proc/stat", "r");
    if (!f) return -1;
    char line[512];
    int n = 0;
    while (fgets(line, sizeof(line), f)) {
        if (strncmp(line, "cpu", 3)) break;
        cpu_times_t t;
        memset(&t, 0, sizeof(t));
        if (line[3] == ' ') {
            sscanf(line + 4, "%llu %llu %llu %llu %llu %llu %llu %llu", &t.user, &t.nice, &t.sys, &t.idle, &t.iowait, &t.irq, &t.softirq, &t.steal);
            *total = t;
        } else {
            int id;
            if (sscanf(line + 3, "%d %llu %llu %llu %llu %llu %llu %llu %llu", &id, &t.user, &t.nice, &t.sys, &t.idle, &t.iowait, &t.irq, &t.softirq, &t.steal) >= 5 && id >= 0 && id < max) {
                cores[id] = t;
                if (id + 1 > n) n = id + 1;
            }
        }
    }
    fclose(f);
    return n;
}
static double busy_pct(const cpu_times_t *a, const cpu_times_t *b, double *user, double *sys, double *iow) {
    const double idle = (double)(b->idle - a->idle) + (double)(b->iowait - a->iowait);
    const double busy = (double)(b->user - a->user) + (double)(b->nice - a->nice) + (double)(b->sys - a->sys) +
                        (double)(b->irq - a->irq) + (double)(b->softirq - a->softirq) + (double)(b->steal - a->steal);
    const double tot = idle + busy;
    if (tot <= 0) return 0.0;
    if (user) *user = 100.0 * (double)(b->user - a->user + b->nice - a->nice) / tot;
    if (sys) *sys = 100.0 * (double)(b->sys - a->sys) / tot;
    if (iow) *iow = 100.0 * (double)(b->iowait - a->iowait) / tot;
    return 100.0 * busy / tot;
}
static void read_mem(double *used_mb, double *util) {
    FILE *f = fopen("/proc/meminfo", "r");
    unsigned long long total = 0, avail = 0, v;
    char key[64];
    if (f) {
        while (fscanf(f, "%63s %llu kB\n", key, &v) == 2) {
            if (!strcmp(key, "MemTotal:")) total = v;
            else if (!strcmp(key, "MemAvailable:")) avail = v;
        }
        fclose(f);
    }
    *used_mb = (double)(total - avail) / 1024.0;
    *util = total ? 100.0 * (double)(total - avail) / (double)total : 0.0;
}
static void poll_all(void) {
    cpu_times_t tot, cores[MAX_CORES];
    memset(cores, 0, sizeof(cores));
    const int n = read_stat(&tot, cores, MAX_CORES);
    if (n < 0) return;
    if (g_have_prev) {
        double u = 0, s = 0, w = 0, used, util;
        daemon_sample_t *sp = daemon_new_sample(&g_total);
        if (sp) {
            sp->values[0] = busy_pct(&g_prev_total, &tot, &u, &s, &w);
            sp->values[1] = u; sp->values[2] = s; sp->values[3] = w;
            read_mem(&used, &util);
            sp->values[4] = used; sp->values[5] = util;
        }
        for (int c = 0; c < g_ncores && c < n; ++c) {
            daemon_sample_t *cp = daemon_new_sample(&g_core[c]);
            if (cp) cp->values[0] = busy_pct(&g_prev_core[c], &cores[c], NULL, NULL, NULL);
        }
    }
    g_prev_total = tot;
    memcpy(g_prev_core, cores, sizeof(cores));
    g_have_prev = 1;
}
int main(int argc, char **argv) {
    const double interval = daemon_interval_arg(argc, argv);
    char host[64], name[DAEMON_NAME_MAX];
    daemon_get_hostname(host, sizeof(host));
    cpu_times_t t, cores[MAX_CORES];
    g_ncores = read_stat(&t, cores, MAX_CORES);
    if (g_ncores < 0) {
        fprintf(stderr, "[daemon_cpu] cannot read /proc/stat\n");
        return 1;
    }
    snprintf(name, sizeof(name), "cpu_%s", host);
    daemon_init(&g_total, name);
    const char *m[] = {"cpu_util", "cpu_user", "cpu_system", "cpu_iowait", "mem_used", "mem_util"};
    const char *u[] = {"%", "%", "%", "%", "MB", "%"};
    for (int i = 0; i < 6; ++i) daemon_add_metric(&g_total, m[i], u[i]);
    const int per_core = getenv("DAEMON_CPU_PER_CORE") ? atoi(getenv("DAEMON_CPU_PER_CORE")) : 1;
    if (!per_core) g_ncores = 0;
    for (int c = 0; c < g_ncores; ++c) {
        snprintf(name, sizeof(name), "cpu_%d_%s", c, host);
        daemon_init(&g_core[c], name);
        daemon_add_metric(&g_core[c], "cpu_util", "%");
    }
    printf("[daemon_cpu] monitoring %d core(s) on %s, interval %.2fs\n", g_ncores, host, interval);
    daemon_run_loop("cpu", interval, poll_all);
    char path[512];
    snprintf(path, sizeof(path), "%s/perf_%s.csv", daemon_output_dir(), g_total.device_name);
    daemon_flush_to_file(&g_total, path);
    for (int c = 0; c < g_ncores; ++c) {
        snprintf(path, sizeof(path), "%s/perf_%s.csv", daemon_output_dir(), g_core[c].device_name);
        daemon_flush_to_file(&g_core[c], path);
        daemon_destroy(&g_core[c]);
    }
    daemon_destroy(&g_total);
    printf("[daemon_cpu] stopped\n");
    return 0;
}
