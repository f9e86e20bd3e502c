"""Hooks used by the test-suite only."""
import ctypes

import torch

from ._lib import lib
from .comm import Communicator, _check


def launch_partial_all_reduce(comm: Communicator, x: torch.Tensor, ranks_played: int) -> None:
    """Launch an AllReduce in which only the first `ranks_played` ranks of a local
    communicator take part, so the others' flags never arrive and the device-side
    waits run out their (short) limit. Nothing faults: the kernel records a time-out
    in the status words and returns."""
    L = lib()
    L.ccb_test_partial_all_reduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64,
                                              ctypes.c_int, ctypes.c_void_p]
    out = torch.empty_like(x)
    _check(L.ccb_test_partial_all_reduce(comm._h, x.data_ptr(), out.data_ptr(), x.numel(), ranks_played,
                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
