/* Path shim: keeps the include path of the reference layout working. */
#include "../../../../include/ccb/compat/nccl/nccl_extensions.h"
