/* GPU monitor: one CSV per GPU, perf_gpu_<i>_<host>.csv with gpu_util, mem_util,
 * mem_used, temperature, pcie_gen, pcie_width (columns of the reference's
 * userconfig/daemon_code_examples/daemon_gpu_nvidia.c:65-96) plus sm_clock and power.
 * The reference forks `nvidia-smi` once per GPU per sample; this daemon reads the
 * same counters through NVML (libnvidia-ml.so.1, opened at run time; set
 * DAEMON_NVML_LIB to point at another library, e.g. a test double). Only read-only
 * NVML queries are used; no clock, power, persistence or compute-mode setting is
 * ever written. */
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include "daemon_loop.h"

#define MAX_GPUS 64
typedef void *nvml_dev_t;
typedef struct { unsigned int gpu, memory; } nvml_util_t;
typedef struct { unsigned long long total, free, used; } nvml_mem_t;
static struct {
    int (*Init)(void);
    int (*Shutdown)(void);
    int (*DeviceGetCount)(unsigned int *);
    int (*DeviceGetHandleByIndex)(unsigned int, nvml_dev_t *);
    int (*DeviceGetUtilizationRates)(nvml_dev_t, nvml_util_t *);
    int (*DeviceGetMemoryInfo)(nvml_dev_t, nvml_mem_t *);
    int (*DeviceGetTemperature)(nvml_dev_t, int, unsigned int *);
    int (*DeviceGetCurrPcieLinkGeneration)(nvml_dev_t, unsigned int *);
    int (*DeviceGetCurrPcieLinkWidth)(nvml_dev_t, unsigned int *);
    int (*DeviceGetClockInfo)(nvml_dev_t, int, unsigned int *);
    int (*DeviceGetPowerUsage)(nvml_dev_t, unsigned int *);
} nv;
static daemon_state_t g_state[MAX_GPUS];
static nvml_dev_t g_dev[MAX_GPUS];
static unsigned int g_ngpu;

static int load_nvml(void) {
    const char *lib = getenv("DAEMON_NVML_LIB");
    void *h = dlopen(lib && *lib ? lib : "libnvidia-ml.so.1", RTLD_NOW);
    if (!h) return -1;
#define SYM(field, name) *(void **)(&nv.field) = dlsym(h, name)
    SYM(Init, "nvmlInit_v2");
    SYM(Shutdown, "nvmlShutdown");
    SYM(DeviceGetCount, "nvmlDeviceGetCount_v2");
    SYM(DeviceGetHandleByIndex, "nvmlDeviceGetHandleByIndex_v2");
    SYM(DeviceGetUtilizationRates, "nvmlDeviceGetUtilizationRates");
    SYM(DeviceGetMemoryInfo, "nvmlDeviceGetMemoryInfo");
    SYM(DeviceGetTemperature, "nvmlDeviceGetTemperature");
    SYM(DeviceGetCurrPcieLinkGeneration, "nvmlDeviceGetCurrPcieLinkGeneration");
    SYM(DeviceGetCurrPcieLinkWidth, "nvmlDeviceGetCurrPcieLinkWidth");
    SYM(DeviceGetClockInfo, "nvmlDeviceGetClockInfo");
    SYM(DeviceGetPowerUsage, "nvmlDeviceGetPowerUsage");
#undef SYM
    if (!nv.Init || !nv.DeviceGetCount || !nv.DeviceGetHandleByIndex) return -1;
    return nv.Init() == 0 ? 0 : -1;
}

static void poll_all(void) {
    for (unsigned int i = 0; i < g_ngpu; ++i) {
        daemon_sample_t *sp = daemon_new_sample(&g_state[i]);
        if (!sp) continue;
        nvml_util_t u = {0, 0};
        nvml_mem_t m = {0, 0, 0};
        unsigned int v = 0;
        if (nv.DeviceGetUtilizationRates && nv.DeviceGetUtilizationRates(g_dev[i], &u) == 0) {
            sp->values[0] = u.gpu;
            sp->values[1] = u.memory;
        }
        if (nv.DeviceGetMemoryInfo && nv.DeviceGetMemoryInfo(g_dev[i], &m) == 0) sp->values[2] = (double)m.used / (1024.0 * 1024.0);
        if (nv.DeviceGetTemperature && nv.DeviceGetTemperature(g_dev[i], 0, &v) == 0) sp->values[3] = v;
        if (nv.DeviceGetCurrPcieLinkGeneration && nv.DeviceGetCurrPcieLinkGeneration(g_dev[i], &v) == 0) sp->values[4] = v;
        if (nv.DeviceGetCurrPcieLinkWidth && nv.DeviceGetCurrPcieLinkWidth(g_dev[i], &v) == 0) sp->values[5] = v;
        if (nv.DeviceGetClockInfo && nv.DeviceGetClockInfo(g_dev[i], 1 /* SM */, &v) == 0) sp->values[6] = v;
        if (nv.DeviceGetPowerUsage && nv.DeviceGetPowerUsage(g_dev[i], &v) == 0) sp->values[7] = v / 1000.0;
    }
}

int main(int argc, char **argv) {
    const double interval = daemon_interval_arg(argc, argv);
    char host[64];
    daemon_get_hostname(host, sizeof(host));
    if (load_nvml() != 0 || nv.DeviceGetCount(&g_ngpu) != 0 || g_ngpu == 0) {
        fprintf(stderr, "[daemon_gpu] no GPUs found (NVML unavailable)\n");
        return 1;
    }
    if (g_ngpu > MAX_GPUS) g_ngpu = MAX_GPUS;
    const char *names[] = {"gpu_util", "mem_util", "mem_used", "temperature", "pcie_gen", "pcie_width", "sm_clock", "power"};
    const char *units[] = {"%", "%", "MB", "C", "gen", "lanes", "MHz", "W"};
    for (unsigned int i = 0; i < g_ngpu; ++i) {
        char name[DAEMON_NAME_MAX];
        snprintf(name, sizeof(name), "gpu_%u_%s", i, host);
        daemon_init(&g_state[i], name);
        for (int m = 0; m < 8; ++m) daemon_add_metric(&g_state[i], names[m], units[m]);
        nv.DeviceGetHandleByIndex(i, &g_dev[i]);
    }
    printf("[daemon_gpu] monitoring %u GPU(s) on %s, interval %.2fs\n", g_ngpu, host, interval);
    daemon_run_loop("gpu_nvidia", interval, poll_all);
    for (unsigned int i = 0; i < g_ngpu; ++i) {
        char path[512];
        snprintf(path, sizeof(path), "%s/perf_%s.csv", daemon_output_dir(), g_state[i].device_name);
        daemon_flush_to_file(&g_state[i], path);
        daemon_destroy(&g_state[i]);
    }
    if (nv.Shutdown) nv.Shutdown();
    printf("[daemon_gpu] stopped\n");
    return 0;
}
