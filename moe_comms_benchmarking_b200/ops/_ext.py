"""ctypes binding of ``lib/libmcb.so`` (the hand-written sm_100a kernels).

The C structures of ``csrc/mcb_ctx.h`` are mirrored here field by field; ``load()`` checks
every ``sizeof`` against the library so a drifted layout fails at import time instead of
corrupting a launch.  There is no fallback: on a machine with a GPU a missing library is an
error (``require()``), so a GPU test can never pass on a silent PyTorch path.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

MAX_RANKS = 72
MAX_BLOCKS = 512
NUM_SITES = 24
STATUS_WORDS = 8
MAX_TENSORS = 4

TRANSPORT_P2P = 0
TRANSPORT_MULTIMEM = 1

SITE_META, SITE_AGV, SITE_RSV = 0, 1, 2
SITE_A2A_DISPATCH, SITE_A2A_COMBINE = 3, 4
SITE_UNIFORM_AG, SITE_UNIFORM_RS = 5, 6
SITE_NORM_IN, SITE_NORM_OUT = 7, 8
SITE_FUSED_FC1, SITE_FUSED_FC2, SITE_LAYER, SITE_TEST = 9, 10, 11, 15
SITE_AGV_LL, SITE_RSV_LL = 12, 13
SITE_A2A_GO, SITE_FC1_FUSED = 14, 16
SITE_STEP_META, SITE_STEP, SITE_STEP_CREDIT = 17, 18, 19
SITE_A2A_STEP_META, SITE_A2A_STEP, SITE_A2A_STEP_CREDIT = 20, 21, 22
LL_SITES = (SITE_AGV_LL, SITE_RSV_LL, SITE_FC1_FUSED)
STEP_STATE_WORDS = 16
STATE_STEP_SEQ, STATE_LAYER_BASE, STATE_LL_BASE, STATE_FINISHED, STATE_GATE0 = 0, 1, 2, 3, 4
MAX_GROUPS = 8

ERR_NAMES = {0: "ok", 1: "timeout", 2: "capacity", 3: "bounds", 4: "routing", 5: "gemm-timeout"}

_vp, _u64, _i32, _u32, _f32 = C.c_void_p, C.c_uint64, C.c_int32, C.c_uint32, C.c_float


class McbCtx(C.Structure):
    _fields_ = [
        ("rank", _i32), ("world", _i32), ("transport", _i32), ("reserved0", _i32),
        ("timeout_ns", _u64),
        ("heap_local", _vp), ("heap_mc", _vp), ("flags_off", _u64),
        ("epochs", _vp), ("status", _vp),
        ("heap_peer", _vp * MAX_RANKS),
    ]


class McbMetaArgs(C.Structure):
    _fields_ = [("n_local", _vp), ("counts_off", _u64), ("step_meta", _vp), ("cap", _i32),
                ("reserved0", _i32)]


class McbAgvArgs(C.Structure):
    _fields_ = [
        ("src", _vp * MAX_TENSORS), ("dst_off", _u64 * MAX_TENSORS), ("row_bytes", _u32 * MAX_TENSORS),
        ("num_tensors", _i32), ("cap", _i32), ("site", _i32), ("meta_stable", _i32),
        ("n_local", _vp), ("step_meta", _vp),
        ("ll_off", _u64), ("ll_rows", _i32), ("reserved1", _i32),
    ]


class McbRsvArgs(C.Structure):
    _fields_ = [
        ("out", _vp), ("src_off", _u64), ("row_bytes", _u32), ("dtype", _i32), ("cap", _i32),
        ("site", _i32), ("n_local", _vp), ("step_meta", _vp),
        ("ll_off", _u64), ("counts_off", _u64), ("ll_rows", _i32), ("meta_stable", _i32),
        ("ll_src_rows", _i32), ("reserved2", _i32),
    ]


class McbDenseStepArgs(C.Structure):
    _fields_ = [
        ("src", _vp * MAX_TENSORS), ("dst_off", _u64 * MAX_TENSORS), ("dst_par_stride", _u64 * MAX_TENSORS),
        ("row_bytes", _u32 * MAX_TENSORS),
        ("num_tensors", _i32), ("cap", _i32), ("num_layers", _i32), ("rsv_dtype", _i32),
        ("out", _vp), ("rsv_off", _u64), ("rsv_row_bytes", _u32), ("ll_rows", _i32),
        ("agv_ll_off", _u64), ("rsv_ll_off", _u64), ("ll_src_rows", _i32), ("groups", _i32),
        ("group_min_bytes", _u64), ("n_local", _vp), ("step_meta", _vp), ("counts_off", _u64), ("credit_off", _u64), ("state", _vp),
        ("check_errors", _vp), ("check", _i32), ("delay_every", _i32), ("delay_ns", _u32), ("fp8_hidden", _u32),
    ]


class McbA2ADispatchArgs(C.Structure):
    _fields_ = [
        ("x", _vp), ("topk_idx", _vp), ("topk_w", _vp),
        ("recv_x_off", _u64), ("recv_scale_off", _u64), ("recv_idx_off", _u64), ("recv_w_off", _u64),
        ("recv_src_off", _u64), ("recv_count_off", _u64),
        ("slot_map", _vp), ("send_count", _vp), ("n_local", _vp),
        ("hidden", _i32), ("topk", _i32), ("num_experts", _i32), ("cap", _i32), ("fp8", _i32),
        ("reserved0", _i32),
    ]


class McbA2AStepArgs(C.Structure):
    _fields_ = [
        ("x", _vp), ("topk_idx", _vp), ("topk_w", _vp), ("out", _vp), ("n_local", _vp),
        ("recv_x_off", _u64), ("recv_scale_off", _u64), ("recv_meta_off", _u64), ("y_off", _u64),
        ("x_par_stride", _u64), ("scale_par_stride", _u64), ("meta_par_stride", _u64), ("y_par_stride", _u64),
        ("meta_row_bytes", _u32), ("hidden", _i32), ("topk", _i32), ("num_experts", _i32), ("cap", _i32),
        ("fp8", _i32), ("num_layers", _i32), ("ll_rows", _i32),
        ("step_meta", _vp), ("counts_off", _u64), ("state", _vp),
        ("ll_x_off", _u64), ("ll_y_off", _u64), ("credit_off", _u64), ("ll_src_rows", _i32), ("reserved1", _i32),
    ]


class McbA2ACombineArgs(C.Structure):
    _fields_ = [("out", _vp), ("y_off", _u64), ("slot_map", _vp), ("n_local", _vp), ("hidden", _i32),
                ("cap", _i32)]


class McbNormArgs(C.Structure):
    _fields_ = [("buf_off", _u64), ("residual", _vp), ("weight", _vp), ("eps", _f32), ("hidden", _i32),
                ("tokens", _i32), ("reserved0", _i32)]


class McbGemmArgs(C.Structure):
    _fields_ = [
        ("a_base", _vp), ("a_row_bytes", _u64), ("row_index", _vp), ("row_scale", _vp),
        ("out", _vp), ("out_row_bytes", _u64),
        ("tile_expert", _vp), ("tile_row0", _vp), ("tile_rows", _vp), ("num_m_tiles", _vp),
        ("n_total", _i32), ("k_total", _i32), ("status", _vp), ("timeout_ns", _u64),
    ]


class McbRouteArgs(C.Structure):
    _fields_ = [
        ("topk_idx", _vp), ("topk_w", _vp), ("num_tokens", _vp),
        ("topk", _i32), ("expert_begin", _i32), ("num_local_experts", _i32), ("max_tokens", _i32),
        ("expert_count", _vp), ("expert_cursor", _vp), ("expert_offset", _vp),
        ("pair_token", _vp), ("pair_prob", _vp), ("pair_pos", _vp),
        ("tile_expert", _vp), ("tile_row0", _vp), ("tile_rows", _vp), ("num_m_tiles", _vp), ("sync", _vp),
        ("max_pairs", _i32), ("max_tiles", _i32), ("status", _vp), ("timeout_ns", _u64),
        ("max_rows", _vp), ("ffn_done", _vp),
    ]


class McbFfnArgs(C.Structure):
    _fields_ = [
        ("x", _vp), ("x_row_bytes", _u64), ("pair_token", _vp), ("pair_prob", _vp), ("expert_offset", _vp),
        ("max_rows", _vp), ("act", _vp), ("y", _vp), ("ffn_done", _vp),
        ("num_local_experts", _i32), ("hidden", _i32), ("intermediate", _i32), ("reserved0", _i32),
        ("status", _vp), ("timeout_ns", _u64), ("w1", _vp), ("w2", _vp),
    ]


class McbCombineArgs(C.Structure):
    _fields_ = [
        ("y", _vp), ("pair_pos", _vp), ("partial_off", _u64), ("out", _vp), ("n_local", _vp), ("step_meta", _vp),
        ("hidden", _i32), ("topk", _i32), ("cap", _i32), ("site", _i32), ("partial_par_stride", _u64),
    ]


class McbLayerArgs(C.Structure):
    """One MoE layer as one kernel parameter: the context and the argument blocks of the four
    phases (64-byte aligned as a whole)."""
    _fields_ = [
        ("ctx", McbCtx), ("agv", McbAgvArgs), ("route", McbRouteArgs), ("ffn", McbFfnArgs), ("cmb", McbCombineArgs),
        ("trace", _vp), ("reserved0", _u64),
    ]


def layer_args_size() -> int:
    """sizeof(McbLayerArgs) as the C compiler sees it (rounded up to its 64-byte alignment)."""
    return (C.sizeof(McbLayerArgs) + 63) // 64 * 64


GEMM_FC1, GEMM_FC2 = 0, 1

_STRUCTS = {
    "ctx": McbCtx, "meta_args": McbMetaArgs, "agv_args": McbAgvArgs, "rsv_args": McbRsvArgs,
    "a2a_dispatch_args": McbA2ADispatchArgs, "a2a_combine_args": McbA2ACombineArgs, "a2a_step_args": McbA2AStepArgs, "norm_args": McbNormArgs,
    "dense_step_args": McbDenseStepArgs, "gemm_args": McbGemmArgs, "ffn_args": McbFfnArgs, "route_args": McbRouteArgs, "combine_args": McbCombineArgs,
}

LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libmcb.so"
_lib = None


class ExtensionMissing(RuntimeError):
    pass


class CudaLaunchError(RuntimeError):
    pass


def available() -> bool:
    return LIB_PATH.exists()


def load():
    """Load the library once and verify the struct layouts."""
    global _lib
    if _lib is not None:
        return _lib
    from .. import build as _build
    if not _build.is_current():
        # Missing, or left over from older sources: build in place when the toolkit is there (one
        # process at a time: build() takes a file lock and links to a temporary name), otherwise
        # fail loudly.  There is no fallback path.
        try:
            _build.build()
        except Exception as e:
            if not LIB_PATH.exists():
                raise ExtensionMissing(
                    f"{LIB_PATH} is missing and could not be built ({type(e).__name__}: {e}); "
                    f"run `python -m moe_comms_benchmarking_b200.build`") from e
            raise ExtensionMissing(
                f"{LIB_PATH} was built from other sources than the ones in csrc/ and could not be rebuilt "
                f"({type(e).__name__}: {e}); run `python -m moe_comms_benchmarking_b200.build`") from e
    lib = C.CDLL(os.fspath(LIB_PATH))
    for name, struct in _STRUCTS.items():
        fn = getattr(lib, f"mcb_sizeof_{name}")
        fn.restype = C.c_int
        got, want = fn(), C.sizeof(struct)
        if got != want:
            raise ExtensionMissing(f"layout drift: sizeof({name}) is {got} in libmcb.so, {want} in ctypes")
    lib.mcb_sizeof_layer_args.restype = C.c_int
    if lib.mcb_sizeof_layer_args() != layer_args_size():
        raise ExtensionMissing(f"layout drift: sizeof(layer_args) is {lib.mcb_sizeof_layer_args()} in libmcb.so, "
                               f"{layer_args_size()} in ctypes")
    lib.mcb_error_string.restype = C.c_char_p
    lib.mcb_error_string.argtypes = [C.c_int]
    _lib = lib
    return lib


def require():
    """Like ``load`` but phrased for hot paths: never fall back, fail loudly."""
    return load()


def check(err: int, what: str) -> None:
    if err != 0:
        msg = load().mcb_error_string(err).decode()
        raise CudaLaunchError(f"{what}: CUDA error {err} ({msg})")


def ptr(t) -> int:
    """Raw device address of a tensor (0 for None)."""
    return 0 if t is None else t.data_ptr()


def stream_handle(stream=None) -> C.c_void_p:
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)
