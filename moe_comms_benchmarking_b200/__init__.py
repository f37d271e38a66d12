"""B200-native MoE expert-parallel dispatch/combine framework.

Host layer in PyTorch, every communication kernel hand-written for sm_100a
(``csrc/*.cu`` -> ``lib/libmcb.so``).  Sub-packages:

* ``models``    shape presets (Nemotron-Super, DeepSeek-V3), SwiGLU experts, the MoE decode model
* ``ops``       ctypes bindings and wrappers of the CUDA kernels, plus the CPU oracle
* ``parallel``  process-group bring-up, the symmetric heap, and the dispatchers
* ``utils``     input generators, timing, CSV/plot reporting, clocks, status decoding
"""
from .config import Config, NUM_EXPERTS, TOPK, HIDDEN  # noqa: F401

__version__ = "0.1.0"
