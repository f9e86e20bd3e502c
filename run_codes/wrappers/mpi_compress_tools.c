/* Path shim: configs written for the reference layout list this file as a source. */
#include "../../csrc/wrappers/mpi_compress_tools.c"
