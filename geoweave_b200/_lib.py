"""ctypes binding of libgeoweave_b200.so.  There is no fallback: a missing library or a failing call raises."""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint, c_void_p, POINTER

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("GEOWEAVE_B200_LIB") or os.path.join(HERE, "libgeoweave_b200.so")

GW_F32, GW_BF16, GW_F16 = 0, 1, 2
GW_OK = 0
GW_ERR_TIMEOUT = -5

_DTYPES = {torch.float32: GW_F32, torch.bfloat16: GW_BF16, torch.float16: GW_F16}


class GeoWeaveError(RuntimeError):
    """A geoweave_b200 library call returned an error status."""

    def __init__(self, code: int, what: str):
        super().__init__(f"geoweave_b200: {what} (status {code})")
        self.code = code


_lock = threading.Lock()
_lib = None
_load_error: Exception | None = None

# name -> (restype, argtypes); the list mirrors include/geoweave_b200.h one to one
_I64x3 = POINTER(c_int64)
SIGNATURES = {
    "gw_strerror": (c_char_p, [c_int]),
    "gw_last_cuda_error": (c_int, []),
    "gw_abi_version": (c_int, []),
    "gw_device_cache_reset": (c_int, []),
    "gw_debug_bounded_wait_selftest": (c_int, [c_uint, c_void_p, c_void_p, c_void_p]),
    "gw_debug_indexer_profile_enable": (c_int, [c_int]),
    "gw_debug_gather_rate": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "gw_debug_gather_rate_ldg": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "gw_debug_gather_rate_ctas": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p,
                                          c_void_p]),
    "gw_indexer_topk_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "gw_debug_indexer_profile": (c_int, [c_void_p, c_int]),
    "gw_indexer_topk_launch_count": (c_int, [c_int, c_int, c_int, c_int]),
    "gw_indexer_topk_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                      c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "gw_indexer_scores": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "gw_indexer_scores_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int64, c_int,
                                      c_void_p, c_int64, c_void_p]),
    "gw_indexer_scores_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                          c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "gw_topk_exact": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "gw_merge_two_topk": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64, c_int, c_int64, c_int,
                                  c_void_p, c_void_p, c_void_p]),
    "gw_sparse_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, _I64x3, _I64x3, _I64x3, c_float, c_void_p, _I64x3, c_void_p, c_void_p,
                                   c_void_p, c_void_p]),
    "gw_project_epilogue": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                    c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                    c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "gw_group_by_key_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "gw_group_by_key": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "gw_sparse_attn_bwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "gw_sparse_attn_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_size_t, c_void_p, c_void_p]),
    "gw_indexer_topk_bwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "gw_indexer_topk_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "gw_peer_barrier": (c_int, [c_void_p, c_int, c_int, c_uint, c_int, c_void_p, c_void_p]),
    "gw_peer_exchange_create": (c_int, [c_int, c_void_p]),
    "gw_peer_exchange_destroy": (None, [c_void_p]),
    "gw_peer_exchange_run": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_uint, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                     c_int, c_void_p, c_void_p, c_void_p, c_int]),
    "gw_peer_exchange_join": (c_int, [c_void_p, c_void_p, c_int]),
    "gw_pool_sources": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "gw_expand_sources": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int64, c_int, c_int, c_int, c_void_p,
                                  c_void_p]),
    "gw_project_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                 c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
}


def load():
    """Load the shared library (once).  Raises if it has not been built: there is no other code path."""
    global _lib, _load_error
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            _load_error = FileNotFoundError(
                f"{LIB_PATH} is missing; build it with `python -m geoweave_b200.build` (needs nvcc, CUDA >= 12.8)")
            raise _load_error
        try:
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
        except Exception as exc:  # missing symbol, wrong architecture...
            _load_error = exc
            raise
        _lib = lib
        return lib


def load_error():
    return _load_error


def check(rc: int, what: str) -> None:
    if rc != GW_OK:
        lib = load()
        msg = lib.gw_strerror(rc).decode()
        if rc == -4:
            msg += f" [cudaError {lib.gw_last_cuda_error()}]"
        raise GeoWeaveError(rc, f"{what}: {msg}")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"geoweave_b200 supports float32, bfloat16 and float16 tensors, got {t.dtype}") from None


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("geoweave_b200 operates on CUDA tensors only (it has no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("all tensors must be on the same CUDA device")
    return dev


def i64x3(vals):
    return (c_int64 * 3)(*[int(v) for v in vals])


# ---------------------------------------------------------------------------------------------
# device-side status word and workspaces, one per device
# ---------------------------------------------------------------------------------------------
_status: dict = {}
_workspaces: dict = {}


def status_word(device) -> torch.Tensor:
    key = torch.device(device).index
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def check_status(device=None) -> None:
    """Synchronise and raise if a kernel recorded a device-side error (e.g. a bounded wait that ran out)."""
    devs = [torch.device(device).index] if device is not None else list(_status)
    for key in devs:
        t = _status.get(key)
        if t is None:
            continue
        code = int(t.item())
        if code != 0:
            t.zero_()
            check(code, "device-side status")


def debug_enabled() -> bool:
    return os.environ.get("GEOWEAVE_B200_DEBUG", "0") == "1"


def workspace(device, nbytes: int, tag: str = "indexer") -> torch.Tensor:
    """A cached byte buffer of at least nbytes for (device, current stream) -- grown on demand, never shrunk.

    The fused indexer's workspace holds thresholds, candidate lists and flags of the call in flight, so two calls
    whose kernels may overlap must not share one: the cache is keyed by the stream the call is enqueued on.  A
    buffer that is replaced by a larger one is handed back to the caching allocator on that same stream, which
    orders its reuse behind the kernels already enqueued.  A captured CUDA graph must own its workspace instead
    (``fused_score_topk(..., workspace=...)``): a cached buffer can be replaced after the capture.
    """
    dev = torch.device(device)
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream, tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        _workspaces.pop(key, None)
        buf = None
        buf = torch.empty(int(nbytes), dtype=torch.uint8, device=dev)
        _workspaces[key] = buf
    return buf


def clear_runtime_cache() -> None:
    """Drop cached workspaces (mirrors clear_runtime_cache of the reference's indexer module)."""
    _workspaces.clear()
