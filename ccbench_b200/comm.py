"""Communicator: the Python face of libccb.so.

One `Communicator` per process and GPU (`Communicator.from_torch_distributed`) or one
that plays all ranks on a single GPU inside one cooperative launch
(`Communicator.local`, for boxes with fewer GPUs than ranks). Every method is one
fused kernel launch on the current torch CUDA stream.

The reference exposes these collectives only as interposed `nccl*` symbols
(userconfig/wrapper_code_examples/communication/plain_nccl_compress/
plain_nccl_compress.cu:654-1147); the interposer of this repository calls the same C
entry points that this class wraps.
"""
from __future__ import annotations

import ctypes
import uuid
from typing import Optional, Sequence, Union

import torch

from . import constants as K
from ._lib import lib

Tensors = Union[torch.Tensor, Sequence[torch.Tensor]]

_DTYPES = {torch.float32: K.F32, torch.bfloat16: K.BF16, torch.float16: K.F16}


class CcbError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"ccb error {code}: {msg}")
        self.code = code


def _code(x, table) -> int:
    return table[x] if isinstance(x, str) else int(x)


class Communicator:
    def __init__(self, handle: int, device: torch.device):
        self._h = ctypes.c_void_p(handle)
        self.device = device
        L = lib()
        self.rank = L.ccb_comm_rank(self._h)
        self.nranks = L.ccb_comm_nranks(self._h)
        self.nlocal = L.ccb_comm_nlocal(self._h)

    # ------------------------------------------------------------ creation --
    @classmethod
    def local(cls, nranks: int, arena_bytes: int = 0, device: Optional[torch.device] = None) -> "Communicator":
        """All `nranks` ranks on one GPU; every call takes one tensor per rank."""
        device = device or torch.device("cuda", torch.cuda.current_device())
        with torch.cuda.device(device):
            h = ctypes.c_void_p()
            rc = lib().ccb_comm_create_local(ctypes.byref(h), nranks, arena_bytes)
        _check(rc)
        return cls(h.value, device)

    @classmethod
    def create(cls, rank: int, nranks: int, tag: str, arena_bytes: int = 0, nvls: bool = False,
               device: Optional[torch.device] = None) -> "Communicator":
        device = device or torch.device("cuda", torch.cuda.current_device())
        with torch.cuda.device(device):
            torch.cuda.init()
            h = ctypes.c_void_p()
            rc = lib().ccb_comm_create(ctypes.byref(h), rank, nranks, tag.encode(), arena_bytes, 1 if nvls else 0)
        _check(rc)
        return cls(h.value, device)

    @classmethod
    def from_torch_distributed(cls, group=None, arena_bytes: int = 0, nvls: bool = False) -> "Communicator":
        """Build over an initialised torch.distributed group; the group is used once,
        to agree on a rendezvous tag."""
        import torch.distributed as dist

        rank, n = dist.get_rank(group), dist.get_world_size(group)
        tag = [uuid.uuid4().hex[:16] if rank == 0 else None]
        dist.broadcast_object_list(tag, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls.create(rank, n, tag[0], arena_bytes, nvls)

    def close(self) -> None:
        if self._h:
            lib().ccb_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------- helpers --
    @property
    def has_nvls(self) -> bool:
        return bool(lib().ccb_comm_has_nvls(self._h))

    @property
    def arena_bytes(self) -> int:
        return int(lib().ccb_comm_arena_bytes(self._h))

    def set_timeout_ms(self, ms: int) -> None:
        _check(lib().ccb_comm_set_timeout_ms(self._h, ms))

    def set_max_ctas(self, ctas: int) -> None:
        _check(lib().ccb_comm_set_max_ctas(self._h, ctas))

    def set_noncooperative(self, ctas: int) -> None:
        """Grids of at most `ctas` CTAs are launched plainly instead of cooperatively (0 = never):
        for collectives overlapped with compute on another stream, with set_max_ctas()."""
        L = lib()
        L.ccb_comm_set_noncooperative.argtypes = [ctypes.c_void_p, ctypes.c_int]
        _check(L.ccb_comm_set_noncooperative(self._h, ctas))

    def set_call_overlap(self, on: bool) -> None:
        """Let consecutive large all_reduce / reduce_scatter calls on one stream overlap tail and
        head (the first CTAs of the next call start on the SMs the previous call's CTAs have
        left). Promise: consecutive calls use different tensors (buckets, double buffers)."""
        L = lib()
        L.ccb_comm_set_call_overlap.argtypes = [ctypes.c_void_p, ctypes.c_int]
        _check(L.ccb_comm_set_call_overlap(self._h, 1 if on else 0))

    def set_waves(self, waves: int) -> None:
        L = lib()
        L.ccb_comm_set_waves.argtypes = [ctypes.c_void_p, ctypes.c_int]
        _check(L.ccb_comm_set_waves(self._h, waves))

    def set_pipeline(self, mode: int = 1, link_warps: int = 0, multicast: bool = False) -> None:
        """The warp-specialised pipelined two-shot kernel: mode 0 never, 1 when the message is
        large enough, 2 always; link_warps of a CTA's 31 data warps store over NVLink (0 keeps
        the current value); multicast lets phase 2 store once through an NVLS mapping."""
        L = lib()
        L.ccb_comm_set_pipeline.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        _check(L.ccb_comm_set_pipeline(self._h, mode, link_warps, 1 if multicast else 0))

    def set_trace(self, on: bool) -> None:
        L = lib()
        L.ccb_comm_set_trace.argtypes = [ctypes.c_void_p, ctypes.c_int]
        _check(L.ccb_comm_set_trace(self._h, 1 if on else 0))

    def read_trace(self, ctas: int):
        """Phase timestamps (ns) of the last traced call as a [ctas, 8] int64 tensor."""
        L = lib()
        L.ccb_comm_read_trace.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        out = torch.zeros(ctas, 8, dtype=torch.int64)
        _check(L.ccb_comm_read_trace(self._h, out.data_ptr(), ctas))
        return out

    # ------------------------------------------------- symmetric allocations --
    def symmetric_empty(self, numel: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """A tensor INSIDE the symmetric arena (same offset on every rank when all ranks make
        the same sequence of calls). all_reduce(..., algo="nvls") on such tensors runs in place
        through the NVSwitch, without staging copies. The tensor must not outlive the communicator."""
        L = lib()
        L.ccb_comm_symm_alloc.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64)]
        L.ccb_comm_symm_ptr.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
        L.ccb_comm_symm_ptr.restype = ctypes.c_void_p
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        off = ctypes.c_uint64(0)
        _check(L.ccb_comm_symm_alloc(self._h, max(nbytes, 16), ctypes.byref(off)))
        ptr = L.ccb_comm_symm_ptr(self._h, off.value)

        class _Span:   # what torch needs to wrap foreign device memory
            __cuda_array_interface__ = {"shape": (max(nbytes, 16),), "typestr": "|u1", "data": (ptr, False), "version": 2}

        t = torch.as_tensor(_Span(), device=self.device)[:nbytes].view(dtype)
        if not hasattr(self, "_symm"):
            self._symm = {}
        self._symm[t.data_ptr()] = (off.value, nbytes)
        return t

    def symmetric_free_all(self) -> None:
        lib().ccb_comm_symm_free_all.argtypes = [ctypes.c_void_p]
        _check(lib().ccb_comm_symm_free_all(self._h))
        self._symm = {}

    def _symm_offset(self, t: torch.Tensor):
        hit = getattr(self, "_symm", {}).get(t.data_ptr())
        return hit[0] if hit and t.numel() * t.element_size() <= hit[1] else None

    def status(self) -> tuple[int, list[int]]:
        words = (ctypes.c_uint32 * 8)()
        rc = lib().ccb_comm_status(self._h, words)
        return rc, list(words)

    def _ptrs(self, t: Optional[Tensors], name: str):
        if t is None:
            return None, None
        ts = [t] if isinstance(t, torch.Tensor) else list(t)
        if len(ts) != self.nlocal:
            raise ValueError(f"{name}: expected {self.nlocal} tensor(s), got {len(ts)}")
        for x in ts:
            if not x.is_cuda or not x.is_contiguous():
                raise ValueError(f"{name}: tensors must be contiguous CUDA tensors")
        arr = (ctypes.c_void_p * self.nlocal)(*[x.data_ptr() for x in ts])
        return arr, ts

    @staticmethod
    def _stream() -> ctypes.c_void_p:
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    @staticmethod
    def _dtype(ts) -> int:
        dt = ts[0].dtype
        if dt not in _DTYPES:
            raise TypeError(f"unsupported dtype {dt}; use float32, bfloat16 or float16")
        return _DTYPES[dt]

    # --------------------------------------------------------- collectives --
    def all_reduce(self, send: Tensors, recv: Optional[Tensors] = None, *, op="sum", codec="int8", algo="auto",
                   error_feedback: Optional[Tensors] = None):
        """recv = sum over ranks of send, moved over the wire in `codec`. In place when
        recv is None. `error_feedback` is one fp32 tensor per rank of the same element
        count that carries the quantisation residual from call to call."""
        recv = send if recv is None else recv
        sp, st = self._ptrs(send, "send")
        rp, rt = self._ptrs(recv, "recv")
        ep, et = self._ptrs(error_feedback, "error_feedback")
        if et is not None and any(e.dtype != torch.float32 or e.numel() != st[0].numel() for e in et):
            raise ValueError("error_feedback must be float32 with send's element count")
        if algo == "nvls" and self.nlocal == 1 and op == "sum" and error_feedback is None:
            so, ro = self._symm_offset(st[0]), self._symm_offset(rt[0])
            if so is not None and ro is not None:   # both live in the arena: in place through the switch
                L = lib()
                L.ccb_all_reduce_symm.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int,
                                                  ctypes.c_void_p]
                _check(L.ccb_all_reduce_symm(self._h, so, ro, st[0].numel(), self._dtype(st), self._stream()))
                return recv
        if algo == "auto":   # a measured choice for this shape, when tune_all_reduce() made one
            algo = getattr(self, "_tuned", {}).get((st[0].numel(), st[0].dtype, codec), "auto")
        _check(lib().ccb_all_reduce(self._h, sp, rp, st[0].numel(), self._dtype(st), _code(op, K.OPS),
                                    _code(codec, K.CODECS), _code(algo, K.ALGOS), ep, self._stream()))
        return recv

    def tune_all_reduce(self, send: Tensors, recv: Tensors, *, codec="int8", algos=("twoshot", "ring", "oneshot"),
                        iters: int = 3, reference: Optional[torch.Tensor] = None, prefer: Optional[str] = None,
                        margin: float = 0.15, report: bool = False):
        """Times each algorithm on these very buffers (CUDA events, maximum over the ranks
        of an initialised torch.distributed group), remembers the choice for this
        (element count, dtype, codec) and returns its name; all_reduce(algo="auto") then
        uses it. Every rank must call it with the same arguments. Candidates that do not
        fit the arena (one-shot on large messages) are skipped.

        The choice is the fastest candidate, under an error cap: when `prefer` names a
        candidate (the shape with the fewest requantisations, "twoshot"), another one
        replaces it only if it is more than `margin` faster. With `reference` (the exact
        fp32 result) each candidate's relative L2 error is measured too; `report=True`
        returns (name, {algo: {"ms": ..., "rel_l2": ...}})."""
        import torch.distributed as dist

        _, st = self._ptrs(send, "send")
        _, rt = self._ptrs(recv, "recv")
        dist_up = dist.is_available() and dist.is_initialized() and self.nlocal == 1 and self.nranks > 1
        seen = {}
        for algo in algos:
            wire = wire_bytes(codec, st[0].dtype, st[0].numel())
            if algo == "oneshot" and wire * self.nranks > self.arena_bytes // 2 - (1 << 20):
                continue
            for _ in range(2):
                self.all_reduce(send, recv, codec=codec, algo=algo)
            if dist_up:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                self.all_reduce(send, recv, codec=codec, algo=algo)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device=st[0].device)
            if dist_up:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            seen[algo] = {"ms": t.item()}
            if reference is not None:
                seen[algo]["rel_l2"] = ((rt[0].float() - reference).norm() / reference.norm()).item()
        best = min(seen, key=lambda a: seen[a]["ms"]) if seen else "auto"
        if prefer in seen and best != prefer and seen[best]["ms"] > (1.0 - margin) * seen[prefer]["ms"]:
            best = prefer
        if not hasattr(self, "_tuned"):
            self._tuned = {}
        self._tuned[(st[0].numel(), st[0].dtype, codec)] = best
        return (best, seen) if report else best

    def reduce_scatter(self, send: Tensors, recv: Tensors, *, op="sum", codec="int8",
                       error_feedback: Optional[Tensors] = None):
        sp, st = self._ptrs(send, "send")
        rp, rt = self._ptrs(recv, "recv")
        ep, _ = self._ptrs(error_feedback, "error_feedback")
        if st[0].numel() != rt[0].numel() * self.nranks:
            raise ValueError("send must hold nranks * recv.numel() elements")
        _check(lib().ccb_reduce_scatter(self._h, sp, rp, rt[0].numel(), self._dtype(st), _code(op, K.OPS),
                                        _code(codec, K.CODECS), ep, self._stream()))
        return recv

    def reduce(self, send: Tensors, recv: Tensors, root: int = 0, *, op="sum", codec="int8"):
        sp, st = self._ptrs(send, "send")
        rp, _ = self._ptrs(recv, "recv")
        _check(lib().ccb_reduce(self._h, sp, rp, st[0].numel(), self._dtype(st), _code(op, K.OPS), root,
                                _code(codec, K.CODECS), self._stream()))
        return recv

    def all_gather(self, send: Tensors, recv: Tensors, *, codec="int8"):
        sp, st = self._ptrs(send, "send")
        rp, rt = self._ptrs(recv, "recv")
        if rt[0].numel() != st[0].numel() * self.nranks:
            raise ValueError("recv must hold nranks * send.numel() elements")
        _check(lib().ccb_all_gather(self._h, sp, rp, st[0].numel(), self._dtype(st), _code(codec, K.CODECS),
                                    self._stream()))
        return recv

    def broadcast(self, send: Tensors, recv: Optional[Tensors] = None, root: int = 0, *, codec="int8"):
        recv = send if recv is None else recv
        sp, st = self._ptrs(send, "send")
        rp, _ = self._ptrs(recv, "recv")
        _check(lib().ccb_broadcast(self._h, sp, rp, st[0].numel(), self._dtype(st), root, _code(codec, K.CODECS),
                                   self._stream()))
        return recv

    def all_to_all(self, send: Tensors, recv: Tensors, *, codec="fp8"):
        sp, st = self._ptrs(send, "send")
        rp, _ = self._ptrs(recv, "recv")
        if st[0].numel() % self.nranks:
            raise ValueError("send.numel() must be a multiple of nranks")
        _check(lib().ccb_all_to_all(self._h, sp, rp, st[0].numel() // self.nranks, self._dtype(st),
                                    _code(codec, K.CODECS), self._stream()))
        return recv

    def scatter(self, send: Tensors, recv: Tensors, root: int = 0, *, codec="none"):
        sp, _ = self._ptrs(send, "send")
        rp, rt = self._ptrs(recv, "recv")
        _check(lib().ccb_scatter(self._h, sp, rp, rt[0].numel(), self._dtype(rt), root, _code(codec, K.CODECS),
                                 self._stream()))
        return recv

    def gather(self, send: Tensors, recv: Tensors, root: int = 0, *, codec="none"):
        sp, st = self._ptrs(send, "send")
        rp, _ = self._ptrs(recv, "recv")
        _check(lib().ccb_gather(self._h, sp, rp, st[0].numel(), self._dtype(st), root, _code(codec, K.CODECS),
                                self._stream()))
        return recv

    def exchange(self, send: Tensors, recv: Tensors, counts, send_offsets, recv_offsets, *, codec="none"):
        """General alltoallv: counts[src][dst] elements from send(src)+send_offsets[src][dst]
        to recv(dst)+recv_offsets[dst][src]. Covers AllGatherv / Scatterv."""
        n = self.nranks
        sp, st = self._ptrs(send, "send")
        rp, _ = self._ptrs(recv, "recv")
        flat = lambda m: (ctypes.c_uint64 * (n * n))(*[int(m[i][j]) for i in range(n) for j in range(n)])
        _check(lib().ccb_exchange(self._h, sp, rp, flat(counts), flat(send_offsets), flat(recv_offsets),
                                  self._dtype(st), _code(codec, K.CODECS), self._stream()))
        return recv

    # ---- point to point over the peer arenas -------------------------------------
    def p2p(self, ops) -> None:
        """ops: iterable of ("send" | "recv", tensor, peer). All of them are launched
        together (one kernel per 16), like the content of an ncclGroupStart/End: a rank
        may send and receive at once. Tensors of any dtype, contiguous; the byte counts of a
        send and of its receive must match."""
        ops = list(ops)
        arr = (_P2pOp * len(ops))()
        for i, (kind, t, peer) in enumerate(ops):
            if kind not in ("send", "recv"):
                raise ValueError(f"p2p operation {kind!r}")
            if not t.is_cuda or not t.is_contiguous():
                raise ValueError("p2p tensors must be contiguous CUDA tensors")
            arr[i] = _P2pOp(t.data_ptr(), t.numel() * t.element_size(), int(peer), 1 if kind == "recv" else 0)
        _check(lib().ccb_p2p(self._h, arr, len(ops), self._stream()))

    def send(self, t: torch.Tensor, peer: int) -> None:
        self.p2p([("send", t, peer)])

    def recv(self, t: torch.Tensor, peer: int) -> None:
        self.p2p([("recv", t, peer)])


class _P2pOp(ctypes.Structure):
    _fields_ = [("buf", ctypes.c_void_p), ("bytes", ctypes.c_uint64), ("peer", ctypes.c_int), ("is_recv", ctypes.c_int)]


def _check(rc: int) -> None:
    if rc != K.OK:
        raise CcbError(rc, (lib().ccb_last_error() or b"").decode(errors="replace"))


def wire_bytes(codec, dtype: torch.dtype, count: int) -> int:
    return int(lib().ccb_wire_bytes(_code(codec, K.CODECS), _DTYPES[dtype], count))


def launch_count() -> int:
    return int(lib().ccb_launch_count())
