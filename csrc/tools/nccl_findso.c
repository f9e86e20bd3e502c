/* bin/nccl/findso: find the real libnccl that calls fall through to and record its
 * path in bin/libs/base_so_name (one line). Same contract as the reference's
 * run_codes/tools/nccl/findso.c:28-146: ask the dynamic linker where ncclAllReduce
 * lives (dlsym + dladdr) with sonames libnccl.so.2 / libnccl.so, then scan
 * LD_LIBRARY_PATH; paths containing "coccl" or "zccl" (NCCL forks used as wrappers)
 * and this repository's own interposer are skipped. */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include "base_impl.h"

static int excluded(const char *path) {
    return strstr(path, "coccl") || strstr(path, "zccl") || strstr(path, "libccb_nccl") || strstr(path, "nccl_extensions");
}

static int try_lib(const char *name, char *out, size_t cap) {
    void *h = dlopen(name, RTLD_LAZY | RTLD_LOCAL);
    if (!h) return 0;
    void *sym = dlsym(h, "ncclAllReduce");
    Dl_info info;
    int ok = sym && dladdr(sym, &info) && info.dli_fname && !excluded(info.dli_fname);
    if (ok) {
        char *real = realpath(info.dli_fname, NULL);
        snprintf(out, cap, "%s", real ? real : info.dli_fname);
        free(real);
    }
    dlclose(h);
    return ok;
}

int main(void) {
    char found[4096] = "";
    const char *sonames[] = {"libnccl.so.2", "libnccl.so", NULL};
    for (int i = 0; sonames[i] && !found[0]; ++i) try_lib(sonames[i], found, sizeof(found));
    const char *llp = getenv("LD_LIBRARY_PATH");
    if (!found[0] && llp) {
        char *copy = strdup(llp), *save = NULL;
        for (char *dir = strtok_r(copy, ":", &save); dir && !found[0]; dir = strtok_r(NULL, ":", &save)) {
            if (excluded(dir)) continue;
            for (int i = 0; sonames[i] && !found[0]; ++i) {
                char path[4096];
                snprintf(path, sizeof(path), "%s/%s", dir, sonames[i]);
                if (access(path, R_OK) == 0) try_lib(path, found, sizeof(found));
            }
        }
        free(copy);
    }
    if (!found[0]) {
        fprintf(stderr, "[findso] no usable libnccl found\n");
        return 1;
    }
    mkdir("bin", 0755);
    mkdir("bin/libs", 0755);
    FILE *f = fopen(BASE_SO_FILE, "w");
    if (!f) {
        perror("[findso] " BASE_SO_FILE);
        return 1;
    }
    fprintf(f, "%s\n", found);
    fclose(f);
    printf("[findso] base NCCL: %s\n", found);
    return 0;
}
