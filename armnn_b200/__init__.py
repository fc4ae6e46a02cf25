"""armnn_b200 — the B200-native compute backend for Arm NN ("B200Acc").

Contents:
  csrc/      hand-written sm_100a CUDA kernels and the C ABI (include/b200k.h) -> libb200k.so
  backend/   the C++17 Arm NN plugin (IBackendInternal & friends) that calls that C ABI
  lib.py     loader for libb200k.so (fails loudly when the library is missing)
  network.py a Python mirror of the INetwork -> Optimize -> LoadNetwork -> EnqueueWorkload flow
             driving the same C ABI, used by the tests and the benchmark
  configs.py the five benchmark configurations as seeded synthetic graphs
"""
from .lib import load_library, B200KError  # noqa: F401
