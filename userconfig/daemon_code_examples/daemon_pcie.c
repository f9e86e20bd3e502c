/* PCIe link monitor: current / maximum link speed (GT/s) and width of every device
 * under /sys/bus/pci/devices whose class is a display or network controller. Writes
 * perf_pcie_<bdf>_<host>.csv. Counterpart of the reference's
 * userconfig/daemon_code_examples/daemon_pcie.c (:65-77). DAEMON_PCIE_ROOT overrides
 * the sysfs root (tests); DAEMON_PCIE_ALL=1 monitors every device. */
#include <dirent.h>
#include <stdio.h>
#include <string.h>

#include "daemon_loop.h"

#define MAX_DEVS 128
typedef struct { daemon_state_t st; char dir[512]; } pcie_dev_t;
static pcie_dev_t g_devs[MAX_DEVS];
static int g_ndevs;

static double read_num(const char *dir, const char *file) {
    char path[700], buf[64];
    snprintf(path, sizeof(path), "%s/%s", dir, file);
    if (daemon_read_sysfs_str(path, buf, sizeof(buf)) != 0) return 0.0;
    return atof(buf); /* "32.0 GT/s PCIe" -> 32.0 ; "16" -> 16 */
}
static void poll_all(void) {
    for (int i = 0; i < g_ndevs; ++i) {
        daemon_sample_t *sp = daemon_new_sample(&g_devs[i].st);
        if (!sp) continue;
        sp->values[0] = read_num(g_devs[i].dir, "current_link_speed");
        sp->values[1] = read_num(g_devs[i].dir, "current_link_width");
        sp->values[2] = read_num(g_devs[i].dir, "max_link_speed");
        sp->values[3] = read_num(g_devs[i].dir, "max_link_width");
        /* usable one-direction bandwidth estimate, GB/s: GT/s * lanes * 128/130 / 8 */
        sp->values[4] = sp->values[0] * sp->values[1] * (128.0 / 130.0) / 8.0;
    }
}
int main(int argc, char **argv) {
    const double interval = daemon_interval_arg(argc, argv);
    char host[64];
    daemon_get_hostname(host, sizeof(host));
    const char *root = getenv("DAEMON_PCIE_ROOT");
    if (!root || !*root) root = "/sys/bus/pci/devices";
    const int all = getenv("DAEMON_PCIE_ALL") != NULL;
    DIR *d = opendir(root);
    struct dirent *e;
    while (d && (e = readdir(d)) && g_ndevs < MAX_DEVS) {
        if (e->d_name[0] == '.') continue;
        char dir[400], path[500], cls[32] = "";
        snprintf(dir, sizeof(dir), "%s/%s", root, e->d_name);
        snprintf(path, sizeof(path), "%s/class", dir);
        daemon_read_sysfs_str(path, cls, sizeof(cls));
        /* 0x03xxxx display, 0x12xxxx processing accelerator, 0x02xxxx network */
        const int wanted = all || !strncmp(cls, "0x03", 4) || !strncmp(cls, "0x12", 4) || !strncmp(cls, "0x02", 4);
        snprintf(path, sizeof(path), "%s/current_link_speed", dir);
        char tmp[64];
        if (!wanted || daemon_read_sysfs_str(path, tmp, sizeof(tmp)) != 0) continue;
        pcie_dev_t *p = &g_devs[g_ndevs++];
        snprintf(p->dir, sizeof(p->dir), "%s", dir);
        char name[DAEMON_NAME_MAX];
        snprintf(name, sizeof(name), "pcie_%.20s_%.30s", e->d_name, host);
        for (char *c = name; *c; ++c)
            if (*c == ':') *c = '-';
        daemon_init(&p->st, name);
        const char *m[] = {"link_speed", "link_width", "max_link_speed", "max_link_width", "link_bw"};
        const char *u[] = {"GT/s", "lanes", "GT/s", "lanes", "GB/s"};
        for (int k = 0; k < 5; ++k) daemon_add_metric(&p->st, m[k], u[k]);
    }
    if (d) closedir(d);
    if (g_ndevs == 0) {
        fprintf(stderr, "[daemon_pcie] no PCIe devices with link information under %s\n", root);
        return 1;
    }
    printf("[daemon_pcie] monitoring %d device(s) on %s, interval %.2fs\n", g_ndevs, host, interval);
    daemon_run_loop("pcie", interval, poll_all);
    for (int i = 0; i < g_ndevs; ++i) {
        char path[512];
        snprintf(path, sizeof(path), "%s/perf_%s.csv", daemon_output_dir(), g_devs[i].st.device_name);
        daemon_flush_to_file(&g_devs[i].st, path);
        daemon_destroy(&g_devs[i].st);
    }
    printf("[daemon_pcie] stopped\n");
    return 0;
}
