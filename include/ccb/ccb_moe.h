/* MoE token exchange with per-destination compression: dispatch (tokens -> experts)
 * and combine (expert outputs -> tokens, gate-weighted) as single fused kernels. The
 * row gather of the dispatch and the weighted top-k sum of the combine are fused into
 * the send and receive loops, so there is no separate permute or scatter pass.
 * The reference times AlltoAll only as a flat ncclAllToAll of equal blocks
 * (run_codes/benchmarks/nccl/alltoall/alltoall.c:82). */
#ifndef CCB_MOE_H
#define CCB_MOE_H

#include <stdint.h>

#include "ccb.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Rows have `hidden` elements (a multiple of 512). counts[src*n+dst] = rows src sends
 * to dst (the full matrix, identical on every rank; host memory).
 *
 * dispatch: rank r sends x[perm[send_row_off[dst] + j]] (j < counts[r][dst]) to dst;
 *   dst stores them in recv at row (sum of counts[s][dst] for s < r) + j.
 *   perm: device int32, one entry per (token, k) pair sorted by destination.
 * combine: rank r (expert side) sends the rows of `y` that came from origin q (the
 *   block starting at row sum_{s<q} counts[s][r]) back to q; origin q computes
 *   out[t] = sum_k gate[t*topk+k] * row(from rank dest_rank[t*topk+k], position pos[t*topk+k])
 *   where pos is the index of (t,k) inside the block q sent to that rank.
 * Arrays are per local rank like everywhere else. */
int ccb_moe_dispatch(ccb_comm* c, const void* const* x, void* const* recv, const int32_t* const* perm,
                     const uint64_t* counts, uint64_t hidden, int dtype, int codec, ccb_stream_t stream);
int ccb_moe_combine(ccb_comm* c, const void* const* y, void* const* out, const int32_t* const* dest_rank,
                    const int32_t* const* pos, const float* const* gate, const uint64_t* counts, uint64_t tokens,
                    int topk, uint64_t hidden, int dtype, int codec, ccb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
