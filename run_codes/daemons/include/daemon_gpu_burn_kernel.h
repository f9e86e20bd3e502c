/* Path shim: keeps the include path of the reference layout working. */
#include "../../../include/ccb/compat/daemon_gpu_burn_kernel.h"
