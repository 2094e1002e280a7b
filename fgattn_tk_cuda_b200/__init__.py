"""B200-native (sm_100a) fine-grained threshold block-sparse attention forward path.

Layout of the package:
  csrc/      hand-written CUDA (tcgen05 / TMEM / TMA) and the extern "C" boundary
  capi.py    ctypes binding of include/fgattn_b200.h
  spattn/    the reference's Python operator interface (same names and arguments) on top of it
  synth.py   seeded synthetic workloads
"""
from . import capi, synth  # noqa: F401

__all__ = ["capi", "synth"]
