// Device-side primitives shared by every fused codec+collective kernel:
// system-scope flag signalling with bounded waits, 16-element lane loads and
// stores for fp32 / bf16 / fp16, and the arena address arithmetic.
//
// Work decomposition used by all kernels in this directory:
//   lane  = 16 consecutive elements            (one 16-byte int8/fp8 wire store)
//   warp  = 512 consecutive elements           (CCB_WARP_ELEMS)
//   tile  = 512 * warps-per-CTA elements       (one CTA iteration)
// Tile t of a shard is always handled by CTA (t mod gridDim.x) on EVERY rank, so
// a receiver CTA only has to wait for the flag written by the same-numbered CTA
// of the sender: synchronisation is per CTA, never grid-wide.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ccb/ccb_types.h"

namespace ccb {

constexpr int kLaneElems = 16;
constexpr int kWarpElems = 512;
constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kTileElems = kWarpElems * kWarps;  // 8192

// ---------------------------------------------------------------- flags -----
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Flag word of (slot, src rank, CTA) inside the arena whose base is `arena`.
__device__ __forceinline__ uint32_t* flag_ptr(char* arena, int slot, int src, int cta) {
  return reinterpret_cast<uint32_t*>(arena) +
         ((size_t)slot * CCB_MAX_RANKS + src) * CCB_MAX_CTAS + cta;
}
__device__ __forceinline__ uint32_t* ctrl_ptr(char* arena, int word) {
  return reinterpret_cast<uint32_t*>(arena + CCB_CTRL_OFFSET) + word;
}

// Publish "everything this CTA stored before the preceding __syncthreads() is
// visible" to the owner of `flag`. Called by ONE thread after a __syncthreads().
// One system-scope fence followed by a relaxed store is a release pattern; a fence
// costs a round trip to every peer with stores in flight, so there is exactly one.
__device__ __forceinline__ void signal_flag(uint32_t* flag, uint32_t epoch) {
  fence_acq_rel_sys();
  st_relaxed_sys(flag, epoch);
}
// The same towards several peers at once: ONE fence, then flag (slot, src, cta) in the
// arena of every rank in `mask`. Called by ONE thread after a __syncthreads().
__device__ __forceinline__ void signal_peers(const CommDev& c, uint32_t mask, int slot, int src, int cta) {
  fence_acq_rel_sys();
  for (int p = 0; p < c.nranks; ++p)
    if ((mask >> p) & 1u) st_relaxed_sys(flag_ptr(c.arena[p], slot, src, cta), c.epoch);
}

// Bounded wait: returns true when *flag has reached `epoch` (wrap-safe compare).
// Gives up after `timeout_ns` (or 2^34 polls, whichever comes first), or as soon
// as the local abort word carries this epoch (another CTA or a peer gave up).
// A wait that gives up records where in `status` and returns false; it never traps.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch,
                                          const CommDev& c, char* my_arena, int where) {
  uint64_t t0 = 0;
  uint64_t polls = 0;
  const uint32_t* abortw = ctrl_ptr(my_arena, CCB_CTRL_ABORT);
  for (;;) {
    uint32_t v = ld_acquire_sys(flag);
    if ((int32_t)(v - epoch) >= 0) return true;
    ++polls;
    if ((polls & 0xff) == 0) {
      if (t0 == 0) t0 = globaltimer_ns();
      bool aborted = ld_relaxed_sys(abortw) == epoch;
      bool late = (globaltimer_ns() - t0) > c.timeout_ns || polls > (1ull << 34);
      if (aborted || late) {
        if (c.status) {
          atomicOr(c.status + CCB_STATUS_FLAGS, aborted ? CCB_ST_ABORTED : CCB_ST_TIMEOUT);
          if (!aborted && atomicCAS(c.status + CCB_STATUS_WHERE, 0u, (uint32_t)where | 0x80000000u) == 0u) {
            c.status[CCB_STATUS_EPOCH] = epoch;
            c.status[CCB_STATUS_SEEN] = v;
          }
        }
        return false;
      }
      __nanosleep(64);
    }
  }
}

// Tell every rank (self included) that this epoch is dead so their waits end
// promptly instead of each running out its own clock.
__device__ __forceinline__ void broadcast_abort(const CommDev& c, uint32_t epoch) {
  for (int p = 0; p < c.nranks; ++p) st_release_sys(ctrl_ptr(c.arena[p], CCB_CTRL_ABORT), epoch);
}

// Optional per-CTA phase timestamps (globaltimer, ns) for the perf columns and for
// tuning: slot k of CTA (blockIdx.y, blockIdx.x). No cost when tracing is off.
__device__ __forceinline__ void trace_mark(const CommDev& c, int k) {
  if (c.trace && threadIdx.x == 0)
    c.trace[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * CCB_TRACE_SLOTS + k] = globaltimer_ns();
}

// ------------------------------------------------------ element load/store --
template <class T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Arena data is written by other GPUs: read it past L1.
__device__ __forceinline__ uint4 ldg_cg(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_cg_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_cg8(const void* p) {
  uint2 v;
  asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ void stg8(void* p, uint2 v) {
  asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void stg_stream(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void stg(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Stores to an NVLink multicast (NVLS) address: the switch writes the value into the
// memory of every GPU bound to the multicast object; the sender's link carries it once.
__device__ __forceinline__ void mc_st16(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void mc_st8(void* p, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void mc_st4(void* p, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Load the 16 elements [idx, idx+16) of `base` as fp32; elements at or beyond
// `limit` read as 0. Vector path when the lane is fully inside and 16-byte aligned.
template <class T>
__device__ __forceinline__ void load16(const T* base, size_t idx, size_t limit, float (&v)[16]) {
  const T* p = base + idx;
  if (idx + 16 <= limit && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint4 u = ldg_stream(reinterpret_cast<const char*>(p) + 16 * k);
        v[4 * k + 0] = __uint_as_float(u.x); v[4 * k + 1] = __uint_as_float(u.y);
        v[4 * k + 2] = __uint_as_float(u.z); v[4 * k + 3] = __uint_as_float(u.w);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        uint4 u = ldg_stream(reinterpret_cast<const char*>(p) + 16 * k);
        const T* h = reinterpret_cast<const T*>(&u);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[8 * k + i] = Elem<T>::to_f(h[i]);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = (idx + i < limit) ? Elem<T>::to_f(p[i]) : 0.f;
  }
}

// The same load split in two, so that a thread can issue the loads of several lanes
// before it converts the first: the 16 elements as raw 16-byte vectors. Everything is
// written with register moves and bit operations (no pointer into the vectors), so the
// raw values stay in registers.
template <class T> struct Raw16 { uint4 q[sizeof(T)]; };
__device__ __forceinline__ uint32_t elem_bits(float x) { return __float_as_uint(x); }
__device__ __forceinline__ uint32_t elem_bits(__nv_bfloat16 x) { return __bfloat16_as_ushort(x); }
__device__ __forceinline__ uint32_t elem_bits(__half x) { return __half_as_ushort(x); }
template <class T> __device__ __forceinline__ float bits_to_f(uint32_t b);
template <> __device__ __forceinline__ float bits_to_f<float>(uint32_t b) { return __uint_as_float(b); }
template <> __device__ __forceinline__ float bits_to_f<__nv_bfloat16>(uint32_t b) { return __uint_as_float(b << 16); }
template <> __device__ __forceinline__ float bits_to_f<__half>(uint32_t b) { return __half2float(__ushort_as_half((unsigned short)b)); }

template <class T>
__device__ __forceinline__ void load16_raw(const T* base, size_t idx, size_t limit, Raw16<T>& raw) {
  const T* p = base + idx;
  if (idx + 16 <= limit && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
    for (int k = 0; k < (int)sizeof(T); ++k) raw.q[k] = ldg_stream(reinterpret_cast<const char*>(p) + 16 * k);
  } else {
    uint32_t w[4 * sizeof(T)];
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int i = 0; i < 16; ++i) w[i] = (idx + i < limit) ? elem_bits(p[i]) : 0u;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t lo = (idx + 2 * i < limit) ? elem_bits(p[2 * i]) : 0u;
        const uint32_t hi = (idx + 2 * i + 1 < limit) ? elem_bits(p[2 * i + 1]) : 0u;
        w[i] = lo | (hi << 16);
      }
    }
#pragma unroll
    for (int k = 0; k < (int)sizeof(T); ++k) raw.q[k] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
  }
}
template <class T>
__device__ __forceinline__ void raw16_to_f(const Raw16<T>& raw, float (&v)[16]) {
#pragma unroll
  for (int k = 0; k < (int)sizeof(T); ++k) {
    const uint32_t w[4] = {raw.q[k].x, raw.q[k].y, raw.q[k].z, raw.q[k].w};
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * k + i] = bits_to_f<T>(w[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[8 * k + 2 * i] = bits_to_f<T>(w[i] & 0xffffu);
        v[8 * k + 2 * i + 1] = bits_to_f<T>(w[i] >> 16);
      }
    }
  }
}

// Two fp32 values rounded to nearest even and packed into one 32-bit word (lo in the low half).
template <class T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <> __device__ __forceinline__ uint32_t pack2<float>(float lo, float) { return __float_as_uint(lo); }

template <class T>
__device__ __forceinline__ void store16(T* base, size_t idx, size_t limit, const float (&v)[16]) {
  T* p = base + idx;
  if (idx + 16 <= limit && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint4 u = make_uint4(__float_as_uint(v[4 * k]), __float_as_uint(v[4 * k + 1]),
                             __float_as_uint(v[4 * k + 2]), __float_as_uint(v[4 * k + 3]));
        stg_stream(reinterpret_cast<char*>(p) + 16 * k, u);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        // one packed conversion per pair of values
        const uint4 u = make_uint4(pack2<T>(v[8 * k], v[8 * k + 1]), pack2<T>(v[8 * k + 2], v[8 * k + 3]),
                                   pack2<T>(v[8 * k + 4], v[8 * k + 5]), pack2<T>(v[8 * k + 6], v[8 * k + 7]));
        stg_stream(reinterpret_cast<char*>(p) + 16 * k, u);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (idx + i < limit) p[i] = Elem<T>::from_f(v[i]);
  }
}

// fp32 side buffers (error-feedback residuals) use the same lane shape.
__device__ __forceinline__ void load16f_plain(const float* base, size_t idx, size_t limit, float (&v)[16]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (idx + 4 * k + 4 <= limit && (reinterpret_cast<uintptr_t>(base + idx) & 15) == 0) {
      float4 u = *reinterpret_cast<const float4*>(base + idx + 4 * k);
      v[4 * k] = u.x; v[4 * k + 1] = u.y; v[4 * k + 2] = u.z; v[4 * k + 3] = u.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * k + i] = (idx + 4 * k + i < limit) ? base[idx + 4 * k + i] : 0.f;
    }
  }
}
__device__ __forceinline__ void store16f_plain(float* base, size_t idx, size_t limit, const float (&v)[16]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (idx + 4 * k + 4 <= limit && (reinterpret_cast<uintptr_t>(base + idx) & 15) == 0) {
      *reinterpret_cast<float4*>(base + idx + 4 * k) = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (idx + 4 * k + i < limit) base[idx + 4 * k + i] = v[4 * k + i];
    }
  }
}

__device__ __forceinline__ float apply_op(int op, float a, float b) {
  switch (op) {
    case CCB_OP_PROD: return a * b;
    case CCB_OP_MAX: return fmaxf(a, b);
    case CCB_OP_MIN: return fminf(a, b);
    default: return a + b;
  }
}

}  // namespace ccb
