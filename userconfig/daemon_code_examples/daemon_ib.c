/* InfiniBand port counters from /sys/class/infiniband/<dev>/ports/<p>/counters:
 * received / transmitted MB and packets, error count, and bandwidth between samples.
 * Writes perf_ib_<dev>_<port>_<host>.csv. Counterpart of the reference's
 * userconfig/daemon_code_examples/daemon_ib.c (:66-73). DAEMON_IB_ROOT overrides the
 * sysfs root (tests). port_rcv_data / port_xmit_data count 4-byte words. */
#include <dirent.h>
#include <stdio.h>
#include <string.h>

#include "daemon_loop.h"

#define MAX_PORTS 64
typedef struct {
    daemon_state_t st;
    char dir[512];
    unsigned long long prev_rx, prev_tx;
    double prev_t;
    int have_prev;
} ib_port_t;
static ib_port_t g_ports[MAX_PORTS];
static int g_nports;

static unsigned long long ctr(const ib_port_t *p, const char *name) {
    char path[700];
    unsigned long long v = 0;
    snprintf(path, sizeof(path), "%s/%s", p->dir, name);
    daemon_read_sysfs_u64(path, &v);
    return v;
}
static void poll_all(void) {
    for (int i = 0; i < g_nports; ++i) {
        ib_port_t *p = &g_ports[i];
        const unsigned long long rx = ctr(p, "port_rcv_data") * 4ull, tx = ctr(p, "port_xmit_data") * 4ull;
        const double now = daemon_get_time();
        daemon_sample_t *sp = daemon_new_sample(&p->st);
        if (!sp) continue;
        sp->values[0] = (double)rx / 1e6;
        sp->values[1] = (double)tx / 1e6;
        sp->values[2] = (double)ctr(p, "port_rcv_packets");
        sp->values[3] = (double)ctr(p, "port_xmit_packets");
        sp->values[4] = (double)(ctr(p, "port_rcv_errors") + ctr(p, "port_xmit_discards") + ctr(p, "symbol_error"));
        if (p->have_prev && now > p->prev_t) {
            sp->values[5] = (double)(rx - p->prev_rx) / (now - p->prev_t);
            sp->values[6] = (double)(tx - p->prev_tx) / (now - p->prev_t);
        }
        p->prev_rx = rx; p->prev_tx = tx; p->prev_t = now; p->have_prev = 1;
    }
}
int main(int argc, char **argv) {
    const double interval = daemon_interval_arg(argc, argv);
    char host[64];
    daemon_get_hostname(host, sizeof(host));
    const char *root = getenv("DAEMON_IB_ROOT");
    if (!root || !*root) root = "/sys/class/infiniband";
    DIR *d = opendir(root);
    struct dirent *e;
    while (d && (e = readdir(d)) && g_nports < MAX_PORTS) {
        if (e->d_name[0] == '.') continue;
        char pdir[400];
        snprintf(pdir, sizeof(pdir), "%s/%s/ports", root, e->d_name);
        DIR *pd = opendir(pdir);
        struct dirent *pe;
        while (pd && (pe = readdir(pd)) && g_nports < MAX_PORTS) {
            if (pe->d_name[0] == '.') continue;
            ib_port_t *p = &g_ports[g_nports++];
            snprintf(p->dir, sizeof(p->dir), "%s/%s/counters", pdir, pe->d_name);
            char name[DAEMON_NAME_MAX];
            snprintf(name, sizeof(name), "ib_%.20s_%.4s_%.30s", e->d_name, pe->d_name, host);
            daemon_init(&p->st, name);
            const char *m[] = {"rcv_data", "xmit_data", "rcv_packets", "xmit_packets", "errors", "rcv_bw", "xmit_bw"};
            const char *u[] = {"MB", "MB", "pkts", "pkts", "count", "B/s", "B/s"};
            for (int k = 0; k < 7; ++k) daemon_add_metric(&p->st, m[k], u[k]);
        }
        if (pd) closedir(pd);
    }
    if (d) closedir(d);
    if (g_nports == 0) {
        fprintf(stderr, "[daemon_ib] no InfiniBand ports under %s\n", root);
        return 1;
    }
    printf("[daemon_ib] monitoring %d port(s) on %s, interval %.2fs\n", g_nports, host, interval);
    daemon_run_loop("ib", interval, poll_all);
    for (int i = 0; i < g_nports; ++i) {
        char path[512];
        snprintf(path, sizeof(path), "%s/perf_%s.csv", daemon_output_dir(), g_ports[i].st.device_name);
        daemon_flush_to_file(&g_ports[i].st, path);
        daemon_destroy(&g_ports[i].st);
    }
    printf("[daemon_ib] stopped\n");
    return 0;
}
