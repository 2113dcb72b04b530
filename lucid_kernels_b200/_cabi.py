"""ctypes binding of the C ABI declared in include/lucid_b200.h.

The library is the only implementation: if it is missing, or no CUDA device is usable, calls raise.
There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading
import weakref
from typing import Dict, Tuple

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lucid_b200.so")
_lib = None
_lock = threading.Lock()

FLAG_DIAG_SOLVE = 1
FLAG_NO_SYNC = 2
FLAG_INSTRUMENT = 4
FLAG_REUSE_DIAG = 8
BWD_DV_ONLY = 0
BWD_COMBINED = 1

_I64x3 = ctypes.c_int64 * 3

EXPORTS = ("lucid_workspace_bytes", "lucid_fwd_sub", "lucid_bwd_sub", "lucid_read_status",
           "lucid_status_string", "lucid_set_wait_limit_ns", "lucid_workspace_timestamps_offset",
           "lucid_profile_next_call", "lucid_set_head_steps", "lucid_set_group_overlap", "lucid_set_dk_split", "lucid_fwd_sub_static",
           "lucid_set_fused_backward", "lucid_fwd_sub_scaled", "lucid_bwd_sub_scaled",
           "lucid_set_pair_solve", "lucid_set_pair_limits", "lucid_fwd_workspace_bytes", "lucid_stream_capture_id", "lucid_query_pair_solve", "lucid_set_solve_variant", "lucid_set_upper_in_solve", "lucid_query_upper_in_solve",
           "lucid_probe_tma_delivery", "lucid_query_chain_group")


class LucidKernelError(RuntimeError):
    pass


def lib_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load (once) and type the shared library.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(_LIB_PATH):
            raise LucidKernelError(
                f"{_LIB_PATH} not found: build it with `python -m lucid_kernels_b200.build` "
                "(there is no fallback implementation)")
        lib = ctypes.CDLL(_LIB_PATH)
        c = ctypes
        lib.lucid_workspace_bytes.restype = c.c_size_t
        lib.lucid_workspace_bytes.argtypes = [c.c_int, c.c_int, c.c_int]
        lib.lucid_fwd_workspace_bytes.restype = c.c_size_t
        lib.lucid_fwd_workspace_bytes.argtypes = [c.c_int, c.c_int, c.c_int]
        lib.lucid_stream_capture_id.restype = c.c_ulonglong
        lib.lucid_stream_capture_id.argtypes = [c.c_void_p]
        lib.lucid_set_solve_variant.restype = None
        lib.lucid_set_solve_variant.argtypes = [c.c_int]
        if os.environ.get("LUCID_B200_SOLVE_VARIANT"):
            lib.lucid_set_solve_variant(int(os.environ["LUCID_B200_SOLVE_VARIANT"]))
        lib.lucid_query_upper_in_solve.restype = c.c_int
        lib.lucid_query_upper_in_solve.argtypes = [c.c_int, c.c_int, c.c_int]
        lib.lucid_set_upper_in_solve.restype = None
        lib.lucid_set_upper_in_solve.argtypes = [c.c_int]
        if os.environ.get("LUCID_B200_UPPER_IN_SOLVE"):
            lib.lucid_set_upper_in_solve(int(os.environ["LUCID_B200_UPPER_IN_SOLVE"]))
        lib.lucid_query_pair_solve.restype = c.c_int
        lib.lucid_query_pair_solve.argtypes = [c.c_int, c.c_int, c.c_int]
        lib.lucid_set_pair_limits.restype = None
        lib.lucid_set_pair_limits.argtypes = [c.c_int, c.c_int]
        lib.lucid_workspace_timestamps_offset.restype = c.c_size_t
        lib.lucid_workspace_timestamps_offset.argtypes = [c.c_int, c.c_int, c.c_int]
        lib.lucid_fwd_sub.restype = c.c_int
        lib.lucid_fwd_sub.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, _I64x3, _I64x3, _I64x3,
                                      c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                                      c.c_void_p, c.c_size_t, c.c_void_p]
        lib.lucid_fwd_sub_static.restype = c.c_int
        lib.lucid_fwd_sub_static.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, _I64x3, _I64x3, _I64x3,
                                             c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                                             c.c_int, c.c_void_p, c.POINTER(c.c_int32)]
        lib.lucid_bwd_sub.restype = c.c_int
        lib.lucid_bwd_sub.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p,
                                      _I64x3, _I64x3, _I64x3, _I64x3, _I64x3,
                                      c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                                      c.c_void_p, c.c_size_t, c.c_void_p]
        lib.lucid_fwd_sub_scaled.restype = c.c_int
        lib.lucid_fwd_sub_scaled.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, _I64x3, _I64x3, _I64x3,
                                             c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                                             c.c_int, c.c_float, c.c_void_p, c.c_size_t, c.c_void_p]
        lib.lucid_bwd_sub_scaled.restype = c.c_int
        lib.lucid_bwd_sub_scaled.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p,
                                             _I64x3, _I64x3, _I64x3, _I64x3, _I64x3,
                                             c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                                             c.c_int, c.c_float, c.c_void_p, c.c_size_t, c.c_void_p]
        lib.lucid_read_status.restype = c.c_int
        lib.lucid_query_chain_group.restype = c.c_int
        lib.lucid_query_chain_group.argtypes = [c.c_int, c.c_int, c.c_int, c.c_int]
        lib.lucid_probe_tma_delivery.restype = c.c_int
        lib.lucid_probe_tma_delivery.argtypes = [c.c_void_p, _I64x3, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                                                 c.c_int, c.c_void_p, c.c_int, c.c_void_p]
        lib.lucid_read_status.argtypes = [c.c_void_p, c.c_void_p, c.POINTER(c.c_int32)]
        lib.lucid_status_string.restype = c.c_char_p
        lib.lucid_status_string.argtypes = [c.c_int]
        lib.lucid_set_head_steps.restype = None
        lib.lucid_set_head_steps.argtypes = [c.c_int]
        lib.lucid_set_group_overlap.restype = None
        lib.lucid_set_group_overlap.argtypes = [c.c_int]
        lib.lucid_set_dk_split.restype = None
        lib.lucid_set_dk_split.argtypes = [c.c_int]
        # LUCID_B200_GROUP_OVERLAP / LUCID_B200_HEAD_STEPS: the scheduler's experiment knobs (steps)
        if os.environ.get("LUCID_B200_GROUP_OVERLAP"):
            lib.lucid_set_group_overlap(int(os.environ["LUCID_B200_GROUP_OVERLAP"]))
        if os.environ.get("LUCID_B200_HEAD_STEPS"):
            lib.lucid_set_head_steps(int(os.environ["LUCID_B200_HEAD_STEPS"]))
        lib.lucid_set_pair_solve.restype = None
        lib.lucid_set_pair_solve.argtypes = [c.c_int]
        # LUCID_B200_PAIR_SOLVE="max_chains[,max_row_blocks]"
        if os.environ.get("LUCID_B200_PAIR_SOLVE"):
            parts = [int(x) for x in os.environ["LUCID_B200_PAIR_SOLVE"].split(",")]
            lib.lucid_set_pair_limits(parts[0], parts[1] if len(parts) > 1 else 0)
        lib.lucid_set_fused_backward.restype = None
        lib.lucid_set_fused_backward.argtypes = [c.c_int, c.c_int]
        # LUCID_B200_FUSED_BWD="max_chains[,solve_ctas]" overrides the library's default (2, automatic)
        env = os.environ.get("LUCID_B200_FUSED_BWD")
        if env:
            parts = [int(x) for x in env.split(",")]
            lib.lucid_set_fused_backward(parts[0], parts[1] if len(parts) > 1 else 0)
        lib.lucid_profile_next_call.restype = None
        lib.lucid_profile_next_call.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p]
        lib.lucid_set_wait_limit_ns.restype = None
        lib.lucid_set_wait_limit_ns.argtypes = [c.c_uint64]
        _lib = lib
    return _lib


def strides3(t: torch.Tensor):
    """Element strides {batch, sequence, head} of a (B, N, H, D) tensor."""
    return _I64x3(t.stride(0), t.stride(1), t.stride(2))


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise AssertionError("inputs must be float16 or bfloat16")


# One workspace per (device, stream, capture, problem size): the kernels of one call communicate through it,
# so two calls that may overlap on the GPU must not share one.  Calls recorded into a CUDA graph get a
# workspace of their own per capture: they run later, at replay, and must neither disturb nor trust what
# eager calls (or another graph) leave in theirs.
class _Workspace:
    __slots__ = ("buf", "diag")

    def __init__(self, buf: torch.Tensor):
        self.buf = buf
        self.diag = None          # what the diagonal-block inverses in `buf` were last prepared for


_workspaces: Dict[Tuple[int, int, int, int, int, int], _Workspace] = {}
_MAX_WORKSPACES = 64


def _entry(device: torch.device, stream_ptr: int, B: int, N: int, H: int, full: bool = True) -> _Workspace:
    """`full`: with the dK partial sums of the combined backward (64 KiB per 128 rows); a forward call asks for
    the forward's share only, and a workspace grown later for a backward call replaces it."""
    lib = load()
    cap = int(lib.lucid_stream_capture_id(stream_ptr))
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_ptr, cap, B, N, H)
    ent = _workspaces.get(key)
    nbytes = lib.lucid_workspace_bytes(B, N, H) if full else lib.lucid_fwd_workspace_bytes(B, N, H)
    if ent is None or ent.buf.numel() < nbytes:
        # torch's caching allocator hands out 512-byte aligned blocks; over-allocate to reach 1 KiB
        raw = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
        off = (-raw.data_ptr()) % 1024
        if ent is None and len(_workspaces) >= _MAX_WORKSPACES:
            # drop the oldest entry only (dict order = insertion order), with what it remembered
            _workspaces.pop(next(iter(_workspaces)))
        ent = _Workspace(raw[off:off + nbytes])
        _workspaces[key] = ent
    return ent


def workspace(device: torch.device, stream_ptr: int, B: int, N: int, H: int, full: bool = True) -> torch.Tensor:
    return _entry(device, stream_ptr, B, N, H, full).buf


# The inverses depend on k only, so a backward call that follows the forward call on the same k can skip
# recomputing them - when the caller asks for that (``reuse_diag=True``; the autograd wrapper does, because
# autograd itself refuses to run a backward whose saved k was modified).  "Same k" means the same live
# tensor object with an unchanged version counter: the address alone is not enough, because the caching
# allocator hands a freed block to the next tensor of that size.  The note lives with the workspace it
# describes, so it goes when the workspace goes.
def _diag_key(k: torch.Tensor) -> tuple:
    return (k.data_ptr(), k._version, tuple(k.shape), tuple(k.stride()), k.dtype)


def diag_is_cached(device: torch.device, stream_ptr: int, k: torch.Tensor, k_scale: float = 1.0) -> bool:
    B, N, H, _ = k.shape
    entry = _entry(device, stream_ptr, B, N, H, full=False).diag
    return entry is not None and entry[0]() is k and entry[1] == (_diag_key(k), float(k_scale))


def diag_remember(device: torch.device, stream_ptr: int, k: torch.Tensor, valid: bool, k_scale: float = 1.0) -> None:
    B, N, H, _ = k.shape
    ent = _entry(device, stream_ptr, B, N, H, full=False)
    ent.diag = (weakref.ref(k), (_diag_key(k), float(k_scale))) if valid else None


def check_rc(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = load().lucid_status_string(rc).decode()
    if rc > 0:
        msg += f" (cudaError_t {rc})"
    raise LucidKernelError(f"{what} failed: {msg}")


def read_status(ws: torch.Tensor, stream_ptr: int):
    """Synchronise the stream and return the eight status words of the last call on this workspace."""
    out = (ctypes.c_int32 * 8)()
    rc = load().lucid_read_status(ws.data_ptr(), stream_ptr, out)
    check_rc(rc, "lucid_read_status")
    return list(out)


def raise_on_device_error(ws: torch.Tensor, stream_ptr: int, what: str) -> None:
    st = read_status(ws, stream_ptr)
    if st[0] != 0:
        msg = load().lucid_status_string(st[0]).decode()
        kern = {0: "diag-prep", 1: "solve", 2: "dK"}.get(st[1], "?")
        raise LucidKernelError(
            f"{what}: {msg} [kernel={kern} chain={st[2]} row_block={st[3]} detail={st[4]} barrier={st[5]}]")


def tma_delivery_rate(t: torch.Tensor, slots: int = 4, boxes_per_sm: int = 4000) -> dict:
    """Measure how fast TMA delivers 16 KiB operand boxes of the (B, N, H, 128) tensor ``t`` from L2 into the
    shared memory of all SMs at once (``lucid_probe_tma_delivery``): the ceiling of the operand streams of the
    solve and dK kernels.  Returns bytes per clock per SM (mean over the SMs, from the SM clock counters) and
    the whole-GPU rate in TB/s (from CUDA events around a second launch; the first warms the caches)."""
    assert t.is_cuda and t.dim() == 4 and t.shape[3] == 128
    B, N, H, _ = t.shape
    lib = load()
    sms = torch.cuda.get_device_properties(t.device).multi_processor_count
    clocks = torch.zeros(sms, dtype=torch.int64, device=t.device)
    stream = torch.cuda.current_stream(t.device)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for timed in (False, True):
        if timed:
            ev0.record(stream)
        rc = lib.lucid_probe_tma_delivery(t.data_ptr(), strides3(t), B, N, H, dtype_code(t.dtype), slots,
                                          boxes_per_sm, clocks.data_ptr(), sms, stream.cuda_stream)
        check_rc(rc, "lucid_probe_tma_delivery", "lucid_query_chain_group")
        if timed:
            ev1.record(stream)
    stream.synchronize()
    c = clocks.cpu()
    if int(c.min()) <= 0:
        raise LucidKernelError("lucid_probe_tma_delivery: a wait ran out")
    ms = ev0.elapsed_time(ev1)
    total = float(sms) * boxes_per_sm * 16384
    return {"bytes_per_clk_per_sm": boxes_per_sm * 16384 / float(c.double().mean()),
            "tb_per_s": total / (ms * 1e-3) / 1e12, "ms": ms, "sms": sms, "slots": slots,
            "boxes_per_sm": boxes_per_sm}
