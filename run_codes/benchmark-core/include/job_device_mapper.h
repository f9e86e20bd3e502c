/* Path shim: keeps the include path of the reference layout working. */
#include "../../../include/ccb/compat/job_device_mapper.h"
