/* Path shim: configs written for the reference layout list this file as a source. */
#include "../../../csrc/daemons/daemon_helper.c"
