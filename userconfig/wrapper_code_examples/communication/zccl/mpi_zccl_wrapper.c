/* ZCCL communication wrapper for the MPI path (LD_PRELOAD).
 *
 * Role of the reference's wrapper (userconfig/wrapper_code_examples/communication/zccl/
 * mpi_zccl_wrapper.c): MPI_Bcast, MPI_Scatter, MPI_Allreduce and MPI_Allgather on
 * MPI_FLOAT go to libZCCL's compressed collectives (:105-204):
 *   MPI_Bcast      -> MPI_Bcast_ZCCL_mt / MPI_Bcast_ZCCL
 *   MPI_Scatter    -> MPIR_Scatter_ZCCL_mt / MPIR_Scatter_ZCCL
 *   MPI_Allreduce  -> MPI_Allreduce_ZCCL_RI2_mt_oa_record / ..._st_oa_record
 *   MPI_Allgather  -> MPIR_Allgatherv_intra_ring_RI2_mt_oa_record / ..._st_oa_record
 * with (compression ratio, tolerance, block size) from ZCCL_CR (0.001), ZCCL_TOL (0.08),
 * ZCCL_BLOCK (36) and the multi-/single-thread choice from ZCCL_MODE (1 = mt, the default;
 * 0 = st) (:70-90); other types and the remaining collectives stay on MPI.
 *
 * The reference links libZCCL; this wrapper resolves those eight entry points lazily
 * (already loaded symbols first, then dlopen of libZCCL.so / libzccl.so), so it loads on
 * hosts without the library. Where ZCCL is absent the same four collectives run on the
 * in-tree compressed algorithms (ring / binomial tree over mpi_compress, compiled into this
 * library from ../plain_mpi_compress/plain_mpi_compress.c) with the in-tree error-bounded
 * codec under the absolute bound ZCCL_TOL, so a ZCCL configuration still produces
 * compressed collectives within its tolerance.
 *
 * Build: this file + csrc/wrappers/mpi_compress_tools.c (plain_mpi_compress.c and the codec
 * are included below). */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <mpi.h>
#include <stdio.h>
#include <stdlib.h>

/* ---- the in-tree fall-back: the compressed collectives under private names ------------ */
#define MPI_Bcast ccb_plain_MPI_Bcast
#define MPI_Reduce ccb_plain_MPI_Reduce
#define MPI_Allreduce ccb_plain_MPI_Allreduce
#define MPI_Gather ccb_plain_MPI_Gather
#define MPI_Scatter ccb_plain_MPI_Scatter
#define MPI_Allgather ccb_plain_MPI_Allgather
#define MPI_Alltoall ccb_plain_MPI_Alltoall
#define MPI_Reduce_scatter_block ccb_plain_MPI_Reduce_scatter_block
#define MPI_Reduce_scatter ccb_plain_MPI_Reduce_scatter
#define MPI_Allgatherv ccb_plain_MPI_Allgatherv
#define MPI_Scatterv ccb_plain_MPI_Scatterv
#define PLAIN_MPI_CODEC_ELSEWHERE
#include "../plain_mpi_compress/plain_mpi_compress.c"
#undef MPI_Bcast
#undef MPI_Reduce
#undef MPI_Allreduce
#undef MPI_Gather
#undef MPI_Scatter
#undef MPI_Allgather
#undef MPI_Alltoall
#undef MPI_Reduce_scatter_block
#undef MPI_Reduce_scatter
#undef MPI_Allgatherv
#undef MPI_Scatterv

/* strong codec hooks of this library: the error-bounded CPU codec under ZCCL_TOL */
#define SZCPU_NO_HOOKS
#include "../../compression/sz_cpu/mpi_szcpu_wrapper.c"

typedef struct { float cr, tol; int block, mt; } zccl_cfg;
static zccl_cfg zcfg_get(void) {
    zccl_cfg c = {0.001f, 0.08f, 36, 1};
    const char *e;
    if ((e = getenv("ZCCL_CR"))) c.cr = (float)atof(e);
    if ((e = getenv("ZCCL_TOL"))) c.tol = (float)atof(e);
    if ((e = getenv("ZCCL_BLOCK"))) c.block = atoi(e);
    if ((e = getenv("ZCCL_MODE"))) c.mt = atoi(e);
    return c;
}
static double fallback_bound(void) {
    const char *e = getenv("MPI_SZ3_ABS_EB"); /* an explicit codec bound wins over ZCCL_TOL */
    if (e && atof(e) > 0) return atof(e);
    const zccl_cfg c = zcfg_get();
    return c.tol > 0 ? (double)c.tol : 1e-6;
}
int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size) {
    return szcpu_compress(input, input_size, output, output_size, fallback_bound(), 0);
}
int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    return szcpu_decompress(input, input_size, output, output_size, 0);
}

/* ---- libZCCL, when it is there -------------------------------------------------------- */
typedef int (*zccl_bcast_fn)(void *, float, float, int, MPI_Aint, MPI_Datatype, int, MPI_Comm);
typedef int (*zccl_scatter_fn)(const void *, float, float, int, MPI_Aint, MPI_Datatype, void *, MPI_Aint, MPI_Datatype, int, MPI_Comm);
typedef int (*zccl_allreduce_fn)(const void *, void *, float, float, int, MPI_Aint, MPI_Datatype, MPI_Op, MPI_Comm);
typedef int (*zccl_allgatherv_fn)(const void *, MPI_Aint, MPI_Datatype, void *, const MPI_Aint *, const MPI_Aint *, MPI_Datatype,
                                  MPI_Comm, unsigned char *, float, float, int);
static struct {
    int state; /* 0 = not tried, 1 = found, -1 = absent */
    zccl_bcast_fn bcast[2];          /* [0] single-thread, [1] multi-thread */
    zccl_scatter_fn scatter[2];
    zccl_allreduce_fn allreduce[2];
    zccl_allgatherv_fn allgatherv[2];
} Z;

static void *zsym(void *h, const char *name) {
    void *p = dlsym(RTLD_DEFAULT, name);
    return p ? p : (h ? dlsym(h, name) : NULL);
}
static int have_zccl(void) {
    if (Z.state) return Z.state > 0;
    Z.state = -1;
    void *h = dlopen("libZCCL.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libzccl.so", RTLD_NOW | RTLD_GLOBAL);
    *(void **)&Z.bcast[0] = zsym(h, "MPI_Bcast_ZCCL");
    *(void **)&Z.bcast[1] = zsym(h, "MPI_Bcast_ZCCL_mt");
    *(void **)&Z.scatter[0] = zsym(h, "MPIR_Scatter_ZCCL");
    *(void **)&Z.scatter[1] = zsym(h, "MPIR_Scatter_ZCCL_mt");
    *(void **)&Z.allreduce[0] = zsym(h, "MPI_Allreduce_ZCCL_RI2_st_oa_record");
    *(void **)&Z.allreduce[1] = zsym(h, "MPI_Allreduce_ZCCL_RI2_mt_oa_record");
    *(void **)&Z.allgatherv[0] = zsym(h, "MPIR_Allgatherv_intra_ring_RI2_st_oa_record");
    *(void **)&Z.allgatherv[1] = zsym(h, "MPIR_Allgatherv_intra_ring_RI2_mt_oa_record");
    for (int i = 0; i < 2; ++i)
        if (!Z.bcast[i] || !Z.scatter[i] || !Z.allreduce[i] || !Z.allgatherv[i]) {
            fprintf(stderr, "[zccl wrapper] libZCCL not found: compressed collectives run on the built-in algorithms\n");
            return 0;
        }
    Z.state = 1;
    return 1;
}

/* ---- exported MPI entry points --------------------------------------------------------- */
int MPI_Init(int *argc, char ***argv) { /* ZCCL's multi-threaded paths use OpenMP inside MPI calls */
    int provided;
    return PMPI_Init_thread(argc, argv, MPI_THREAD_FUNNELED, &provided);
}

int MPI_Bcast(void *buffer, int count, MPI_Datatype datatype, int root, MPI_Comm comm) {
    if (datatype != MPI_FLOAT) return PMPI_Bcast(buffer, count, datatype, root, comm);
    if (!have_zccl()) return ccb_plain_MPI_Bcast(buffer, count, datatype, root, comm);
    const zccl_cfg c = zcfg_get();
    return Z.bcast[c.mt != 0](buffer, c.cr, c.tol, c.block, (MPI_Aint)count, datatype, root, comm);
}

int MPI_Scatter(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf, int recvcount, MPI_Datatype recvtype,
                int root, MPI_Comm comm) {
    if (sendtype != MPI_FLOAT || recvtype != MPI_FLOAT)
        return PMPI_Scatter(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, root, comm);
    if (!have_zccl()) return ccb_plain_MPI_Scatter(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, root, comm);
    const zccl_cfg c = zcfg_get();
    return Z.scatter[c.mt != 0](sendbuf, c.cr, c.tol, c.block, (MPI_Aint)sendcount, sendtype, recvbuf, (MPI_Aint)recvcount, recvtype,
                                root, comm);
}

int MPI_Allreduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype datatype, MPI_Op op, MPI_Comm comm) {
    if (datatype != MPI_FLOAT) return PMPI_Allreduce(sendbuf, recvbuf, count, datatype, op, comm);
    if (!have_zccl()) return ccb_plain_MPI_Allreduce(sendbuf, recvbuf, count, datatype, op, comm);
    const zccl_cfg c = zcfg_get();
    return Z.allreduce[c.mt != 0](sendbuf, recvbuf, c.cr, c.tol, c.block, (MPI_Aint)count, datatype, op, comm);
}

int MPI_Allgather(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf, int recvcount, MPI_Datatype recvtype,
                  MPI_Comm comm) {
    if (sendtype != MPI_FLOAT || recvtype != MPI_FLOAT)
        return PMPI_Allgather(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, comm);
    if (!have_zccl()) return ccb_plain_MPI_Allgather(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, comm);
    const zccl_cfg c = zcfg_get();
    /* ZCCL offers the vector form only: uniform counts, one displacement of zero */
    const MPI_Aint n = (MPI_Aint)recvcount, zero = 0;
    unsigned char *scratch = NULL;
    if (c.mt) { /* the multi-threaded ring wants a staging buffer for one compressed block */
        const size_t bytes = (size_t)recvcount * sizeof(float);
        scratch = (unsigned char *)malloc(bytes + 64 + bytes / 16);
        if (!scratch) return MPI_ERR_OTHER;
    }
    const int rc = Z.allgatherv[c.mt != 0](sendbuf, (MPI_Aint)sendcount, sendtype, recvbuf, &n, &zero, recvtype, comm, scratch, c.cr,
                                           c.tol, c.block);
    free(scratch);
    return rc;
}

/* not offered by ZCCL: plain MPI */
int MPI_Reduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype datatype, MPI_Op op, int root, MPI_Comm comm) {
    return PMPI_Reduce(sendbuf, recvbuf, count, datatype, op, root, comm);
}
int MPI_Gather(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf, int recvcount, MPI_Datatype recvtype, int root,
               MPI_Comm comm) {
    return PMPI_Gather(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, root, comm);
}
int MPI_Alltoall(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf, int recvcount, MPI_Datatype recvtype,
                 MPI_Comm comm) {
    return PMPI_Alltoall(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, comm);
}
