"""ctypes binding of libb200moe.so (the C ABI declared in include/b200moe.h).

The library is the only compute path: if it is missing or does not export the
expected ABI this module raises; there is no fallback of any kind.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "libb200moe.so"
ABI_VERSION = 4

STATUS_BAD_ID = 1
STATUS_BAD_WEIGHT = 2
STATUS_TIMEOUT = 4
STATUS_EP_OVERFLOW = 8

WEIGHTS_BF16 = 0
WEIGHTS_W4G128 = 1

SCHEDULE_AUTO = 0
SCHEDULE_GENERIC = 1
SCHEDULE_TCGEN05 = 2
SCHEDULE_NAMES = {SCHEDULE_GENERIC: "generic", SCHEDULE_TCGEN05: "tcgen05"}

ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_STATE = -1, -2, -3, -4


class Shape(ctypes.Structure):
    _fields_ = [(name, ctypes.c_int32) for name in (
        "tokens", "experts", "topk", "hidden", "intermediate", "ids_are_int64", "gate_up_format",
        "down_format", "schedule", "token_tile", "use_router", "route_only", "external_dispatch", "router_bf16_weights",
        "unchained", "fused_gather", "down_tiles")] + [("reserved", ctypes.c_int32 * 1)]


WORKSPACE_BUFFERS = ("output", "counts", "offsets", "cursors", "tasks", "mapping", "ranks",
                     "grouped_input", "activated", "down_output", "status", "scratch")


class Workspace(ctypes.Structure):
    _fields_ = [(name, ctypes.c_size_t) for name in WORKSPACE_BUFFERS + ("source_rows",)] + [
        ("token_tile", ctypes.c_int32), ("schedule", ctypes.c_int32), ("launches", ctypes.c_int32),
        ("gathers", ctypes.c_int32), ("down_tiles", ctypes.c_int32), ("reserved", ctypes.c_int32)]


INPUT_BUFFERS = ("x", "router_weight", "gate_up", "gate_up_scales", "down", "down_scales", "ids",
                 "routing_weights")


class Buffers(ctypes.Structure):
    _fields_ = [(name, ctypes.c_void_p) for name in INPUT_BUFFERS + WORKSPACE_BUFFERS + (
        "valid_routes", "residual", "ep_row_dest", "ep_return_bases", "source_rows")]


class DispatchArgs(ctypes.Structure):
    """Arguments of ``b200moe_dispatch_static`` (the entry point that allocates nothing)."""
    _fields_ = [(name, ctypes.c_int32) for name in (
        "tokens", "experts", "topk", "hidden", "ids_are_int64", "token_tile")] + [
        (name, ctypes.c_void_p) for name in (
            "x", "ids", "routing_weights", "counts", "offsets", "cursors", "tasks", "ranks", "mapping",
            "grouped_input", "status")]


STATIC_DISPATCH_MAX_ROUTES = 65536
EP_MAX_RANKS = 8


class EpArgs(ctypes.Structure):
    """``B200MoeEpArgs``: expert parallelism over peer memory."""
    _fields_ = [(name, ctypes.c_int32) for name in (
        "rank", "world", "experts", "topk", "hidden", "tokens", "capacity", "token_tile", "ids_are_int64",
        "fused_return")] + [("reserved", ctypes.c_int32 * 2)] + [(name, ctypes.c_void_p) for name in (
            "x", "ids", "ranks", "counts", "expert_counts", "expert_offsets", "expert_tasks", "expert_rows",
            "expert_output", "tables", "status")] + [(name, ctypes.c_void_p * EP_MAX_RANKS) for name in (
                "recv_rows_peers", "return_rows_peers", "all_counts_peers", "flags_peers")] + [
        ("expert_chain", ctypes.c_void_p), ("expert_chain_words", ctypes.c_int32), ("reserved2", ctypes.c_int32),
        ("expert_status", ctypes.c_void_p), ("mapping", ctypes.c_void_p),
        ("row_dest_peers", ctypes.c_void_p * EP_MAX_RANKS)]


EXPORTS = {
    "b200moe_abi_version": (ctypes.c_int, []),
    "b200moe_last_error": (ctypes.c_char_p, []),
    "b200moe_plan_create": (ctypes.c_int, [ctypes.POINTER(Shape), ctypes.POINTER(ctypes.c_void_p)]),
    "b200moe_plan_workspace": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(Workspace)]),
    "b200moe_plan_bind": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(Buffers)]),
    "b200moe_forward": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "b200moe_router": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "b200moe_dispatch": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "b200moe_gate_up": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "b200moe_down": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "b200moe_combine": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "b200moe_dispatch_static": (ctypes.c_int, [ctypes.POINTER(DispatchArgs), ctypes.c_void_p]),
    "b200moe_plan_chain": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                          ctypes.POINTER(ctypes.c_int32)]),
    "b200moe_ep_table_ints": (ctypes.c_size_t, [ctypes.c_int32, ctypes.c_int32]),
    "b200moe_peer_alloc": (ctypes.c_int, [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)]),
    "b200moe_peer_free": (ctypes.c_int, [ctypes.c_void_p]),
    "b200moe_peer_export": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
    "b200moe_peer_import": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "b200moe_peer_close": (ctypes.c_int, [ctypes.c_void_p]),
    "b200moe_ep_exchange_counts": (ctypes.c_int, [ctypes.POINTER(EpArgs), ctypes.c_void_p]),
    "b200moe_ep_send_rows": (ctypes.c_int, [ctypes.POINTER(EpArgs), ctypes.c_void_p]),
    "b200moe_ep_return_rows": (ctypes.c_int, [ctypes.POINTER(EpArgs), ctypes.c_void_p]),
    "b200moe_plan_destroy": (None, [ctypes.c_void_p]),
}

_LIB = None
_LOCK = threading.Lock()


def load():
    """Load the library once; raise if it is absent or has the wrong ABI."""
    global _LIB
    with _LOCK:
        if _LIB is None:
            if not LIBRARY_PATH.is_file():
                raise RuntimeError(
                    f"{LIBRARY_PATH} is missing: build it with `python -m llm_gpu_kernels_b200.build` "
                    "(there is no fallback path)")
            lib = ctypes.CDLL(str(LIBRARY_PATH))
            for name, (restype, argtypes) in EXPORTS.items():
                fn = getattr(lib, name)  # AttributeError if the symbol is not exported
                fn.restype = restype
                fn.argtypes = argtypes
            if lib.b200moe_abi_version() != ABI_VERSION:
                raise RuntimeError("libb200moe.so has an unexpected ABI version")
            _LIB = lib
    return _LIB


def last_error() -> str:
    return load().b200moe_last_error().decode(errors="replace")


def check(code: int):
    """Map a negative return code onto the exception type the reference raises
    for the same condition (ValueError for bad arguments, RuntimeError else)."""
    if code == 0:
        return
    message = last_error()
    if code == ERR_INVALID:
        raise ValueError(message)
    raise RuntimeError(f"b200moe error {code}: {message}")
