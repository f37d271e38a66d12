import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lib():
    """The compiled CUDA library; built on demand (nvcc cross-compiles without a GPU)."""
    from moe_comms_benchmarking_b200 import build
    from moe_comms_benchmarking_b200.ops import _ext
    build.build()
    return _ext.load()


@pytest.fixture(scope="session")
def world1(lib):
    """A one-rank NCCL process group on cuda:0 for single-GPU tests."""
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29571")
    os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"] = "0", "1", "0"
    from moe_comms_benchmarking_b200.parallel.dist import init_distributed
    group, rank, world, local_rank = init_distributed()
    yield group
    if dist.is_initialized():
        dist.destroy_process_group()


def free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]
