/* Public face of the compressed MPI collectives in plain_mpi_compress.c: the collectives
 * themselves are the MPI_* symbols the library interposes; what a codec wrapper or a test
 * may call directly is the on/off query below (MPI_COMPRESS_DISABLE=1 switches the library
 * to pass-through), plus the helpers of mpi_compress_tools.h. */
#ifndef PLAIN_MPI_COMPRESS_H
#define PLAIN_MPI_COMPRESS_H

#include "mpi_compress_tools.h"

#ifdef __cplusplus
extern "C" {
#endif

/* 1 while the collectives compress, 0 when they forward to PMPI unchanged. */
int compression_enabled(void);

#ifdef __cplusplus
}
#endif
#endif
