/* Types and constants shared by the host runtime and the device kernels. */
#ifndef CCB_TYPES_H
#define CCB_TYPES_H

#include <stddef.h>
#include <stdint.h>

#define CCB_MAX_RANKS 8      /* one NVSwitch domain */
#define CCB_MAX_CTAS 1024    /* flag columns per (slot, source) */
#define CCB_MAX_SLOTS 16     /* flag rows: phases or ring/tree steps of one call */

/* Arena layout (identical on every rank):
 *   [0, CCB_CTRL_OFFSET)            flags  u32[CCB_MAX_SLOTS][CCB_MAX_RANKS][CCB_MAX_CTAS]
 *   [CCB_CTRL_OFFSET, CCB_DATA_OFFSET)  control words (abort epoch, barrier counters)
 *   [CCB_DATA_OFFSET, arena_bytes)  staging, split into two halves used on
 *                                   alternating calls (epoch parity)            */
#define CCB_CTRL_OFFSET (CCB_MAX_SLOTS * CCB_MAX_RANKS * CCB_MAX_CTAS * 4)
#define CCB_DATA_OFFSET (1u << 20)
#define CCB_CTRL_ABORT 0
#define CCB_CTRL_BARRIER 64 /* u32[CCB_MAX_RANKS] end-of-call acknowledgements */

/* Status words (host-mapped, written by kernels only when a wait gives up). */
#define CCB_STATUS_FLAGS 0
#define CCB_STATUS_WHERE 1
#define CCB_STATUS_EPOCH 2
#define CCB_STATUS_SEEN 3
#define CCB_STATUS_WORDS 8
/* Phase trace: CCB_TRACE_SLOTS timestamps per CTA (start, after each phase, end). */
#define CCB_TRACE_SLOTS 8
#define CCB_ST_TIMEOUT 1u
#define CCB_ST_ABORTED 2u

/* Element types of user buffers. */
enum { CCB_F32 = 0, CCB_BF16 = 1, CCB_F16 = 2 };
/* Wire codecs. */
enum {
  CCB_CODEC_NONE = 0,     /* elements travel in their own type              */
  CCB_CODEC_INT8 = 1,     /* int8, one fp32 absmax/127 scale per 128 values */
  CCB_CODEC_FP8 = 2,      /* e4m3, one ue8m0 scale byte per 32 values       */
  CCB_CODEC_INT8_G256 = 3, /* int8, group 256 (the reference wrapper default) */
  CCB_CODEC_INT4 = 4      /* int4, fp32 scale = absmax/7 per 128 values       */
};
enum { CCB_OP_SUM = 0, CCB_OP_PROD = 1, CCB_OP_MAX = 2, CCB_OP_MIN = 3 };
/* element types of ccb_fold only (the fused collectives carry CCB_F32 / CCB_F16 / CCB_BF16) */
enum { CCB_X_I8 = 16, CCB_X_U8 = 17, CCB_X_I32 = 18, CCB_X_U32 = 19, CCB_X_I64 = 20, CCB_X_U64 = 21, CCB_X_F64 = 22 };
/* AllReduce algorithms. */
enum { CCB_ALGO_AUTO = 0, CCB_ALGO_TWOSHOT = 1, CCB_ALGO_ONESHOT = 2, CCB_ALGO_RING = 3, CCB_ALGO_TREE = 4, CCB_ALGO_NVLS = 5 };

/* Result codes of the C API. */
enum {
  CCB_OK = 0,
  CCB_ERR_ARG = 1,
  CCB_ERR_CUDA = 2,
  CCB_ERR_BOOTSTRAP = 3,
  CCB_ERR_TIMEOUT = 4,   /* a device-side wait ran out; the communicator is dead */
  CCB_ERR_UNSUPPORTED = 5,
  CCB_ERR_CAPACITY = 6
};

/* What every kernel needs to know about the communicator (passed by value). */
typedef struct CommDev {
  char* arena[CCB_MAX_RANKS]; /* every rank's arena, mapped in this process  */
  char* mc_arena;             /* NVLS multicast mapping of the arenas, or 0  */
  uint32_t* status;           /* CCB_STATUS_WORDS host-mapped words          */
  unsigned long long* trace;  /* per-CTA phase timestamps (globaltimer ns), or 0 */
  uint64_t timeout_ns;
  uint64_t half_bytes;        /* size of one staging half                    */
  uint32_t epoch;             /* this call's sequence number (never 0)       */
  int nranks;
} CommDev;

/* Per-call arguments of the reduce family (AllReduce two-shot / one-shot,
 * ReduceScatter, Reduce) and of the ring and tree kernels. With nlocal > 1 one
 * launch plays `nlocal` consecutive ranks (blockIdx.y) on a single GPU. */
typedef struct ReduceArgs {
  CommDev c;
  const void* send[CCB_MAX_RANKS];
  void* recv[CCB_MAX_RANKS];
  float* ef[CCB_MAX_RANKS];   /* error-feedback residuals, count floats, or 0 */
  uint64_t count;             /* elements in the whole message                */
  uint64_t shard_elems;       /* elements per shard in the user buffers       */
  uint64_t shard_pad;         /* shard_elems rounded up to 512 (wire extent)  */
  uint64_t slot_bytes;        /* bytes of one wire slot                       */
  int rank0, nlocal;
  int op, root, mode;
  int waves;                  /* software-pipeline depth of the two-shot shape  */
  int tile_warps;             /* warps of a CTA that carry data: tile = 512 * tile_warps */
  int row_base;               /* pipelined two-shot: first flag row of this call (0, or 8 for odd epochs when calls may overlap) */
  int link_warps;             /* pipelined two-shot: warps that store over NVLink (the rest decode, one signals) */
  int use_mc;                 /* pipelined two-shot: phase 2 stores once to the NVLS multicast address */
} ReduceArgs;
enum { CCB_MODE_ALLREDUCE = 0, CCB_MODE_REDUCESCATTER = 1, CCB_MODE_REDUCE = 2 };

/* Per-call arguments of the exchange family (AllGather(v), Broadcast, Scatter(v),
 * Gather, AlltoAll(v)): rank r sends send[send_off[r][p] .. +cnt[r][p]) to peer p,
 * which lands at recv[recv_off[p][r]]. cnt[r][p] == 0 means no transfer. */
typedef struct ExchangeArgs {
  CommDev c;
  const void* send[CCB_MAX_RANKS];
  void* recv[CCB_MAX_RANKS];
  uint64_t cnt[CCB_MAX_RANKS][CCB_MAX_RANKS];      /* [src][dst] elements     */
  uint64_t send_off[CCB_MAX_RANKS][CCB_MAX_RANKS]; /* [src][dst] in src.send  */
  uint64_t recv_off[CCB_MAX_RANKS][CCB_MAX_RANKS]; /* [dst][src] in dst.recv  */
  uint64_t slot_pad;   /* wire extent of one (src,dst) slot, multiple of 512   */
  uint64_t slot_bytes;
  int rank0, nlocal;
  int ack;             /* rooted pattern: finish with an all-rank handshake     */
  int tile_warps;
} ExchangeArgs;

#endif
