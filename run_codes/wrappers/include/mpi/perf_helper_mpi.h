/* Path shim: keeps the include path of the reference layout working. */
#include "../../../../include/ccb/compat/mpi/perf_helper_mpi.h"
