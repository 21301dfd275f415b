"""ctypes binding of libgla_b200.so (the C ABI in include/gla_b200.h).

There is no fallback: if the shared library is missing or cannot be loaded, every operator
of this package raises.  Build it with ``python -m gla_jax_b200.build``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libgla_b200.so"
_lib = None

GLA_F32, GLA_BF16 = 0, 1
IMPL_AUTO, IMPL_FP32_SIMT, IMPL_TCGEN05 = 0, 1, 2
_FAMILY = {"auto": IMPL_AUTO, "fp32": IMPL_FP32_SIMT, "simt": IMPL_FP32_SIMT, "tcgen05": IMPL_TCGEN05}
# gla_chunk_option bits of include/gla_b200.h, by the names accepted after a "+" in an impl string
OPTIONS = {"two_kernels": 0x100, "one_pass": 0x200, "no_early_start": 0x400, "all_scales": 0x800,
           "no_l2_prefetch": 0x1000, "segments": 0x2000}


class _ImplNames(dict):
    """``IMPL_BY_NAME["tcgen05+all_scales+one_pass"]`` -> family | option bits (the `impl` argument of the chunk
    entry points).  Plain family names are ordinary keys."""

    def __missing__(self, name):
        fam, *opts = str(name).split("+")
        if fam not in _FAMILY or any(o not in OPTIONS for o in opts):
            raise KeyError(f"unknown chunk implementation {name!r}: family one of {sorted(_FAMILY)}, "
                           f"options {sorted(OPTIONS)} joined by '+'")
        v = _FAMILY[fam]
        for o in opts:
            v |= OPTIONS[o]
        return v


IMPL_BY_NAME = _ImplNames(_FAMILY)

# name -> (restype, argtypes); must list every symbol include/gla_b200.h declares.
SIGNATURES = {
    "gla_status_string": (c_char_p, [c_int]),
    "gla_version": (c_char_p, []),
    "gla_last_cuda_error": (c_int, []),
    "gla_launch_count": (ctypes.c_longlong, []),
    "gla_device_wait_timeouts": (ctypes.c_uint, []),
    "gla_device_bad_offsets": (ctypes.c_uint, []),
    "gla_profile_enable": (None, [c_int]),
    "gla_profile_report": (c_size_t, [c_char_p, c_size_t]),
    "gla_cumsum": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]),
    "gla_scan": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]),
    "gla_rnn_scan": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int, c_int, c_int]),
    "gla_rnn_scan_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64]),
    "gla_rnn_scan_ws": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t]),
    "gla_recurrent_fwd": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "gla_decode_step": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_int]),
    "gla_layer_gate_fwd": (c_int, [c_void_p, c_int64, c_int, c_void_p, ctypes.c_float, c_void_p]),
    "gla_layer_gate_bwd": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, ctypes.c_float, c_void_p]),
    "gla_layer_headnorm_gate_fwd": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                            ctypes.c_float, c_void_p, c_void_p]),
    "gla_layer_headnorm_gate_bwd_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "gla_layer_headnorm_gate_bwd": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "gla_recurrent_bwd_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int]),
    "gla_recurrent_bwd": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_int, c_void_p, c_size_t]),
    "gla_chunk_saved_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int]),
    "gla_chunk_fwd_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int]),
    "gla_chunk_bwd_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int]),
    "gla_chunk_fwd": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "gla_chunk_fwd_packed": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int64, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_size_t]),
    "gla_chunk_bwd_packed": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int64, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "gla_chunk_fwd_static_max_bytes": (c_size_t, []),
    "gla_chunk_fwd_static": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "gla_chunk_bwd": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_size_t]),
    "gla_chunk_local_state": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "gla_chunk_local_dstate": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "gla_chunk_sp_fwd_local": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "gla_chunk_sp_fwd_finish": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "gla_chunk_sp_bwd_local": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "gla_chunk_sp_bwd_finish": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_size_t]),
    "gla_sp_combine": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                               c_void_p, c_int, c_int]),
    "gla_sp_combine2": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                c_void_p, c_int, c_void_p, c_void_p, c_int, c_int]),
}


class GlaError(RuntimeError):
    """A non-zero status from libgla_b200.so."""


def load() -> ctypes.CDLL:
    """Load the library once and attach the signatures; raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} not found: the CUDA library is not built (run `python -m gla_jax_b200.build`). "
            "This package has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def lib_path() -> Path:
    return _LIB_PATH


def stream_of(dev) -> int:
    """The current CUDA stream of `dev` as an integer handle for the C ABI.  The library launches on the CURRENT
    device (and looks up per-device state there), so tensors on another GPU are refused rather than launched with a
    stream of the wrong device: wrap the call in ``torch.cuda.device(tensor.device)``."""
    import torch
    cur = torch.cuda.current_device()
    if dev.index is not None and dev.index != cur:
        raise RuntimeError(f"tensors are on {dev} but the current CUDA device is cuda:{cur}; "
                           "make their device current (torch.cuda.device(...)) around the call")
    return torch.cuda.current_stream(dev).cuda_stream


_seen = {"waits": 0, "offsets": 0}


def check_device() -> None:
    """Synchronise the current device and raise GlaError if, since the previous call of this function, a bounded
    device-side wait gave up (the outputs written meanwhile are incomplete) or a packed-sequence call was given
    offsets that had to be clamped.  The entry points themselves return before their kernels run and cannot
    report either."""
    lib = load()
    waits, offs = int(lib.gla_device_wait_timeouts()), int(lib.gla_device_bad_offsets())
    new_w, new_o = waits - _seen["waits"], offs - _seen["offsets"]
    _seen["waits"], _seen["offsets"] = waits, offs
    if new_w or new_o:
        raise GlaError(f"device-side errors since the last check: {new_w} wait(s) gave up, {new_o} sequence(s) with "
                       "invalid packed offsets")


def check(status: int, what: str) -> None:
    """Raise GlaError for a non-zero status, with the library's own message."""
    if status != 0:
        lib = load()
        msg = lib.gla_status_string(status).decode()
        extra = ""
        if status == 6:
            extra = f" (cudaError {lib.gla_last_cuda_error()})"
        raise GlaError(f"{what}: {msg}{extra}")
