/* NCCL's API on another transport, as a wrapper built from source (selection mode 3).
 *
 * The reference keeps a wrapper at this path that replaces NCCL by the UCCL engine
 * (userconfig/wrapper_code_examples/communication/nccl_via_uccl/nccl_via_uccl.cu). The
 * transport of this repository inside one NVSwitch node is the peer-memory runtime: a
 * configuration that names this directory in `source_dirs` builds the NCCL-free provider,
 * csrc/interpose/ccb_nccl_standalone.c (also shipped prebuilt as
 * bin/libs/libccb_nccl_standalone.so), linked against libccb.so by the wrapper builder. */
#include "ccb/ccb.h"
#include "../../../../csrc/interpose/ccb_nccl_standalone.c"
