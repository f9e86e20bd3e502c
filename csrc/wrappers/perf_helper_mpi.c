/* Process-wide perf table for MPI perf wrappers (reference: run_codes/wrappers/src/
 * mpi/perf_helper_mpi.c: pthread_once state :8-20, node map by one PMPI_Allgather of
 * processor names :32-57, destructor flush to perf_function_<rank>.csv :80-102). */
#define _GNU_SOURCE
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#include "mpi/perf_helper_mpi.h"

static perf_state_t g_state;
static pthread_once_t g_once = PTHREAD_ONCE_INIT;
static char *g_names;
static int g_nranks, g_rank = -1, g_map_ready, g_flushed;
static char g_me[MPI_MAX_PROCESSOR_NAME];

static void init_once(void) { perf_init(&g_state); }
perf_state_t *perf_mpi_get_tls(void) {
    pthread_once(&g_once, init_once);
    return &g_state;
}

int perf_mpi_world_rank(void) {
    if (g_rank < 0) {
        int init = 0;
        PMPI_Initialized(&init);
        if (init) PMPI_Comm_rank(MPI_COMM_WORLD, &g_rank);
        else return perf_gendata_get_rank();
    }
    return g_rank;
}

void perf_mpi_init_node_map(void) {
    if (g_map_ready) return;
    int init = 0, len = 0;
    PMPI_Initialized(&init);
    if (!init) return;
    PMPI_Comm_size(MPI_COMM_WORLD, &g_nranks);
    memset(g_me, 0, sizeof(g_me));
    PMPI_Get_processor_name(g_me, &len);
    g_names = (char *)calloc((size_t)g_nranks, MPI_MAX_PROCESSOR_NAME);
    if (!g_names) return;
    PMPI_Allgather(g_me, MPI_MAX_PROCESSOR_NAME, MPI_CHAR, g_names, MPI_MAX_PROCESSOR_NAME, MPI_CHAR, MPI_COMM_WORLD);
    g_map_ready = 1;
}

int perf_mpi_is_intra(int rank) {
    if (!g_map_ready) perf_mpi_init_node_map();
    if (!g_map_ready || rank < 0 || rank >= g_nranks) return 1;
    return strncmp(g_names + (size_t)rank * MPI_MAX_PROCESSOR_NAME, g_me, MPI_MAX_PROCESSOR_NAME) == 0;
}

double perf_mpi_msg_size(int count, MPI_Datatype datatype) {
    int sz = 0;
    PMPI_Type_size(datatype, &sz);
    return (double)count * (double)sz;
}

void perf_mpi_flush(void) {
    if (g_flushed) return;
    g_flushed = 1;
    if (perf_mpi_get_tls()->total_records > 0) perf_flush_to_rank_file(perf_mpi_get_tls(), perf_mpi_world_rank(), "perf_function");
}
__attribute__((destructor)) static void perf_mpi_dtor(void) { perf_mpi_flush(); }

/* the table's time origin is the moment the wrapper library is loaded */
__attribute__((constructor)) static void perf_early_init(void) { perf_mpi_get_tls(); }
