/* Where the path of the real (un-interposed) communication library is recorded by
 * bin/<arch>/findso. Same contract as the reference's
 * run_codes/benchmark-core/include/base_impl.h. */
#ifndef BASE_IMPL_H
#define BASE_IMPL_H
#define BASE_SO_FILE "bin/libs/base_so_name"
#ifdef __cplusplus
extern "C" {
#endif
int load_base_impl(const char *state_path);
#ifdef __cplusplus
}
#endif
#endif
