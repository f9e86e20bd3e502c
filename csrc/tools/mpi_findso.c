/* bin/mpi/findso: the MPI base implementation is reached through the PMPI_ profiling
 * names, so there is no library to locate; check that PMPI_Allreduce resolves and
 * record "builtin:pmpi" (reference: run_codes/tools/mpi/findso.c:17-53). */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdio.h>
#include <sys/stat.h>

#include "base_impl.h"

int main(void) {
    void *self = dlopen(NULL, RTLD_LAZY);
    const int have = self && dlsym(self, "PMPI_Allreduce") != NULL;
    if (!have) fprintf(stderr, "[findso] warning: PMPI_Allreduce does not resolve in this binary\n");
    mkdir("bin", 0755);
    mkdir("bin/libs", 0755);
    FILE *f = fopen(BASE_SO_FILE, "w");
    if (!f) {
        perror("[findso] " BASE_SO_FILE);
        return 1;
    }
    fprintf(f, "builtin:pmpi\n");
    fclose(f);
    printf("[findso] base MPI: builtin:pmpi\n");
    return 0;
}
