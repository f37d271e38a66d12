"""B200-native MoE expert-parallel dispatch/combine framework.

Host layer in PyTorch, every communication kernel hand-written for sm_100a
(``csrc/*.cu`` -> ``lib/libmcb.so``).  Sub-packages:

* ``models``    shape presets (Nemotron-Super, DeepSeek-V3) and the decode engine (one captured step, replayed)
* ``ops``       ctypes bindings and launch plans of the CUDA kernels (dense collectives, all-to-all,
                routing + grouped expert GEMMs, fused norm), plus the CPU oracle
* ``parallel``  process-group bring-up, the symmetric heap, the dispatchers (dense, a2a, fused experts, NCCL
                and gloo baselines), single-GPU emulation of a multi-rank world, host-side membership
* ``utils``     input generators, timing, CSV reporting, clock sampling, NVTX tracing
"""
from .config import Config, NUM_EXPERTS, TOPK, HIDDEN  # noqa: F401

__version__ = "0.1.0"
