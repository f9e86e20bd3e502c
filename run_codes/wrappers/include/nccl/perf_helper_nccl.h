/* Path shim: keeps the include path of the reference layout working. */
#include "../../../../include/ccb/compat/nccl/perf_helper_nccl.h"
