"""ccbench_b200: a Blackwell-native compressed-collective framework.

Every communication-bound path is one hand-written sm_100a kernel that fuses the
codec (int8 block-128, fp8 e4m3 with ue8m0 scales, SZ-style error-bounded) with the
collective over NVSwitch peer memory. PyTorch is the harness and the checker.
"""
from .constants import *  # noqa: F401,F403
from .comm import Communicator, CcbError  # noqa: F401

__version__ = "0.1.0"
