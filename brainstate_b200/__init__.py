"""brainstate_b200 — event-driven synaptic propagation for NVIDIA B200 (sm_100a).

A from-scratch implementation of the hot path behind ``brainstate.nn``'s
event-connection layers: the layers themselves (:mod:`brainstate_b200.nn`), the
operator layer that stands where ``brainevent`` stands in the reference
(:mod:`brainstate_b200.event`), and ``libbsx.so``, the C-ABI CUDA library that does
all the arithmetic (``include/bsx.h``).  There is no CPU fallback.
"""
from . import _lib
from . import event
from . import nn
from . import host
from .event import EventArray, FixedPostNumConn, CSR, FixedPreNumConn, CSC

__version__ = '0.1.0'
__all__ = ['event', 'nn', 'host', 'EventArray', 'FixedPostNumConn', 'CSR', 'FixedPreNumConn', 'CSC']
