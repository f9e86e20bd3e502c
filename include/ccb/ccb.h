/* Public C API of the B200 compressed-collective runtime (libccb.so).
 *
 * A communicator owns one symmetric staging arena per rank (CUDA VMM memory whose
 * handle every peer imports, so a kernel on any GPU can store into any arena over
 * NVLink) plus flag words for device-side signalling. Every collective below is ONE
 * kernel launch on the caller's stream: the codec runs in registers and the
 * compressed bytes are stored directly into the peers' arenas.
 *
 * `send`, `recv` and `ef` are arrays with one pointer per LOCAL rank: one entry in
 * the normal one-process-per-GPU case, `nranks` entries for a communicator made by
 * ccb_comm_create_local(), which plays all ranks inside a single cooperative launch
 * on one GPU (used for tests on boxes with fewer GPUs than ranks).
 *
 * Calls on one communicator must be issued in the same order on every rank and are
 * serialised on the GPU in issue order (use one stream per communicator).
 *
 * Counterpart in the reference: the LD_PRELOAD wrapper
 * userconfig/wrapper_code_examples/communication/plain_nccl_compress/
 * plain_nccl_compress.cu, which builds the same collectives from host-driven
 * ncclSend/ncclRecv hops around separate quantize / dequantize kernels. */
#ifndef CCB_H
#define CCB_H

#include <stddef.h>
#include <stdint.h>

#include "ccb_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ccb_comm ccb_comm;
typedef void* ccb_stream_t; /* a cudaStream_t */

/* One process per GPU. The CUDA device must be current. `tag` names the rendezvous
 * (abstract Unix sockets "ccb.<tag>.<rank>"); it must be the same on all ranks and
 * unique among communicators alive on the host. arena_bytes == 0 picks the default
 * (CCB_ARENA_MB or 2048 MiB). flags: bit 0 = try to set up an NVLS multicast mapping. */
int ccb_comm_create(ccb_comm** out, int rank, int nranks, const char* tag, uint64_t arena_bytes, int flags);
/* All `nranks` ranks on the current device, in one process. */
int ccb_comm_create_local(ccb_comm** out, int nranks, uint64_t arena_bytes);
int ccb_comm_destroy(ccb_comm* c);
int ccb_comm_rank(const ccb_comm* c);   /* first local rank */
int ccb_comm_nranks(const ccb_comm* c);
int ccb_comm_nlocal(const ccb_comm* c);
int ccb_comm_has_nvls(const ccb_comm* c);
uint64_t ccb_comm_arena_bytes(const ccb_comm* c);
/* Limit of every device-side wait (default CCB_TIMEOUT_MS or 10000). */
int ccb_comm_set_timeout_ms(ccb_comm* c, uint64_t ms);
/* Cap on CTAs per rank (0 = as many as fit). */
int ccb_comm_set_max_ctas(ccb_comm* c, int ctas);
/* Grids of at most `ctas` CTAs per rank are launched without the cooperative attribute
 * (0 = always cooperative, the default; also CCB_NONCOOP_CTAS). Use it together with
 * ccb_comm_set_max_ctas() for collectives that should hide behind compute on another
 * stream: a plain launch trickles into SMs as they free up instead of waiting for room
 * for the whole grid. One rank per process only; every wait stays bounded. */
int ccb_comm_set_noncooperative(ccb_comm* c, int ctas);
/* on != 0: consecutive large AllReduce / ReduceScatter calls of this communicator on one stream
 * may overlap: the first CTAs of call k + 1 start on the SMs that the CTAs of call k have left,
 * instead of after its slowest CTA (programmatic dependent launch; one rank per process). The
 * caller promises that call k + 1 neither reads what call k writes nor writes what it reads or
 * writes (gradient buckets, double-buffered outputs). Any other kernel put on the stream
 * afterwards is ordered after all of them as usual. In this mode a call uses at most 4 waves
 * (the two calls that can be on the device at once take one half of the flag rows each).
 * Off by default. */
int ccb_comm_set_call_overlap(ccb_comm* c, int on);
/* Software-pipeline depth of the two-shot kernels (0 = choose per call, at most 8). */
int ccb_comm_set_waves(ccb_comm* c, int waves);
/* The warp-specialised pipelined two-shot kernel (large AllReduce / ReduceScatter):
 * mode 0 = never, 1 = when the message is large enough (default), 2 = always;
 * link_warps = how many of a CTA's 31 data warps store over NVLink (1 to 30; 0 keeps the
 * current value, default 20; the rest decode); mc != 0 lets its second phase store once to the
 * NVLS multicast address when the communicator has one (off by default: measured slower than
 * per-peer stores at 2 and 4 GPUs). Also CCB_PIPE,
 * CCB_PIPE_LINK_WARPS, CCB_PIPE_MC, CCB_PIPE_MIN_CHUNKS in the environment. */
int ccb_comm_set_pipeline(ccb_comm* c, int mode, int link_warps, int mc);
/* Copies the CCB_STATUS_WORDS status words; returns CCB_ERR_TIMEOUT when a kernel of
 * this communicator gave up a wait (the communicator must then be destroyed). Only
 * meaningful after the stream has been synchronised. */
int ccb_comm_status(ccb_comm* c, uint32_t* words);
/* Device-side phase tracing: when on, every CTA of the two-shot kernels records
 * globaltimer nanoseconds at its phase boundaries (slots: 0 start, 1 first phase-1
 * done, 2 first phase-2 done, 3 all phase-2 done, 4 end). */
int ccb_comm_set_trace(ccb_comm* c, int on);
int ccb_comm_read_trace(ccb_comm* c, unsigned long long* out, int ctas);
/* Wire bytes a call moves per rank for `count` elements (for ratio reporting). */
uint64_t ccb_wire_bytes(int codec, int dtype, uint64_t count);

/* ---- link probe ---------------------------------------------------------------------
 * Writes `bytes` of generated data from this rank into the data area of `peer`'s arena and
 * so measures what SM-issued stores reach on the link: method 0 = 16-byte stores per lane,
 * 1 = bulk copies (TMA unit) of 512 bytes from shared memory, 2 = bulk copies of 2 KB. No
 * collective may be in flight. Time it with events on `stream`. */
int ccb_link_probe(ccb_comm* c, int method, int peer, uint64_t bytes, ccb_stream_t stream);

/* ---- point-to-point ----------------------------------------------------------------
 * Sends and receives over the peer arenas, no NCCL involved: the sender stores into a
 * mailbox in the receiver's arena, the receiver copies out. ccb_p2p launches the
 * operations of one rank (the content of one ncclGroupStart/End) as ONE kernel per 16
 * operations, so a rank may send and receive at the same time; a second transfer of the
 * same direction to the same peer starts a new kernel. Transfers between a pair must be
 * issued in the same order at both ends and on one stream (or otherwise ordered). The byte counts of a send and
 * of the matching receive must be equal; transfers between a pair are matched in issue
 * order. A send of up to two rounds (2 x 16 x lane bytes, 8 MiB with the default arena)
 * completes without its receive being posted, longer ones wait for it (bounded). */
typedef struct ccb_p2p_op {
  void* buf;
  uint64_t bytes;
  int peer;
  int is_recv;
} ccb_p2p_op;
int ccb_p2p(ccb_comm* c, const ccb_p2p_op* ops, int nops, ccb_stream_t stream);
int ccb_send(ccb_comm* c, const void* buf, uint64_t bytes, int peer, ccb_stream_t stream);
int ccb_recv(ccb_comm* c, void* buf, uint64_t bytes, int peer, ccb_stream_t stream);

/* ---- symmetric allocations -------------------------------------------------------
 * User buffers INSIDE the arena, so that collectives can work on them in place. Every
 * rank must make the same sequence of allocations (same sizes): buffers then sit at the
 * same offset everywhere. Allocation synchronises the device and shrinks the staging the
 * other collectives use; at most three quarters of the arena can be given out. */
int ccb_comm_symm_alloc(ccb_comm* c, uint64_t bytes, uint64_t* offset);
void* ccb_comm_symm_ptr(ccb_comm* c, uint64_t offset);   /* this rank's device address */
int ccb_comm_symm_free_all(ccb_comm* c);
/* Uncompressed sum of `count` elements, in place on symmetric buffers (send_off may equal
 * recv_off), reduced inside the NVSwitch: needs a communicator created with the NVLS
 * flag. No staging copies: the kernel only moves what must cross the links. */
int ccb_all_reduce_symm(ccb_comm* c, uint64_t send_off, uint64_t recv_off, uint64_t count, int dtype, ccb_stream_t stream);

/* Kernels launched by this library since it was loaded. */
uint64_t ccb_launch_count(void);
const char* ccb_last_error(void);

int ccb_all_reduce(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count, int dtype, int op,
                   int codec, int algo, float* const* ef, ccb_stream_t stream);
/* recv holds recvcount elements; send holds nranks * recvcount. */
int ccb_reduce_scatter(ccb_comm* c, const void* const* send, void* const* recv, uint64_t recvcount, int dtype,
                       int op, int codec, float* const* ef, ccb_stream_t stream);
int ccb_reduce(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count, int dtype, int op, int root,
               int codec, ccb_stream_t stream);
/* General exchange; cnt/send_off/recv_off are nranks x nranks row-major matrices:
 * cnt[src][dst] elements go from send(src) + send_off[src][dst] to recv(dst) + recv_off[dst][src]. */
int ccb_exchange(ccb_comm* c, const void* const* send, void* const* recv, const uint64_t* cnt,
                 const uint64_t* send_off, const uint64_t* recv_off, int dtype, int codec, ccb_stream_t stream);
int ccb_all_gather(ccb_comm* c, const void* const* send, void* const* recv, uint64_t sendcount, int dtype, int codec,
                   ccb_stream_t stream);
int ccb_broadcast(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count, int dtype, int root,
                  int codec, ccb_stream_t stream);
int ccb_all_to_all(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count_per_peer, int dtype,
                   int codec, ccb_stream_t stream);
int ccb_scatter(ccb_comm* c, const void* const* send, void* const* recv, uint64_t recvcount, int dtype, int root,
                int codec, ccb_stream_t stream);
int ccb_gather(ccb_comm* c, const void* const* send, void* const* recv, uint64_t sendcount, int dtype, int root,
               int codec, ccb_stream_t stream);

/* ---- stand-alone codec kernels on local memory --------------------------------
 * Wire layout of `count` elements: pad = count rounded up to 512,
 * [payload: pad elements][scales: pad / group entries], ccb_wire_bytes() bytes. */
int ccb_encode(int codec, int dtype, const void* in, uint64_t count, void* wire, ccb_stream_t stream);
int ccb_decode(int codec, int dtype, const void* wire, uint64_t count, void* out, ccb_stream_t stream);
/* inout += decode(wire) */
int ccb_decode_reduce(int codec, int dtype, const void* wire, uint64_t count, void* inout, ccb_stream_t stream);
/* The same on `nchunks` equal chunks in ONE launch: chunk c is chunk_count elements at
 * element offset c * chunk_count of the plain buffer, its wire at byte offset
 * c * wire_stride (>= ccb_wire_bytes(codec, dtype, chunk_count), a multiple of 16).
 * accumulate != 0: out[c] += decode(wire[c]). */
int ccb_encode_chunks(int codec, int dtype, const void* in, uint64_t chunk_count, uint64_t nchunks, void* wire,
                      uint64_t wire_stride, ccb_stream_t stream);
int ccb_decode_chunks(int codec, int dtype, const void* wire, uint64_t wire_stride, uint64_t chunk_count, uint64_t nchunks,
                      void* out, int accumulate, ccb_stream_t stream);
/* inout += src, element-wise in the element type. */
int ccb_accumulate(int dtype, const void* src, void* inout, uint64_t count, ccb_stream_t stream);
/* out[i] = op over p < nparts of parts[p * stride + i] for the CCB_X_* element types (integers and
 * double); op is a CCB_OP_* value or 4 for the average. Used by the NCCL-free provider, which
 * gathers the ranks' buffers and folds them locally for types the fused kernels do not carry. */
int ccb_fold(int xtype, int op, const void* parts, uint64_t stride, int nparts, uint64_t count, void* out, ccb_stream_t stream);
/* wire_out = encode(sum_k decode(wires[k])), 1 <= nwires <= 16 */
int ccb_reduce_recode(int codec, const void* const* wires, int nwires, uint64_t count, void* wire_out,
                      ccb_stream_t stream);
/* The reference wrapper's int8 wire: [f32 127/absmax per group][int8 x count]. */
int ccb_refwire_encode(int dtype, const void* in, uint64_t count, int group, void* wire, ccb_stream_t stream);
int ccb_refwire_decode(int dtype, const void* wire, uint64_t count, int group, void* out, ccb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
