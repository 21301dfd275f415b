"""The scan operators of the reference's ops.py with unchanged signatures, backed by
libgla_b200.so.

    cumsum_recursive / cumsum_pallas                 ops.py:234 / ops.py:166
    rnn_recursive / rnn_pallas / binary_operator     ops.py:396 / ops.py:338 / ops.py:286

The reference needs a host-side hierarchy (``*_recursive``) because one Triton program can
scan at most 16384 / 8192 items; the CUDA kernels walk any length in one launch, so the
``*_recursive`` and ``*_pallas`` names resolve to the same kernels and the block-size
arguments are accepted and ignored.  Like the reference's, these ops are not differentiable.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

_DT = {torch.float32: _lib.GLA_F32, torch.bfloat16: _lib.GLA_BF16}


_stream = _lib.stream_of


def _need_cuda(x):
    if not x.is_cuda:
        raise RuntimeError("gla_jax_b200 operators need CUDA tensors; there is no CPU fallback")


SCAN_OPS = {"add": 0, "mul": 1, "max": 2, "min": 3, "logaddexp": 4}      # gla_scan_op of include/gla_b200.h


def scan(op: str, src, axis: int, init: Optional[torch.Tensor] = None, reverse: bool = False, out_dtype=None):
    """Inclusive associative scan of one array along ``axis`` under a named combine rule (``SCAN_OPS``), float32
    math, with ``init`` (shape = src.shape without ``axis``) combined in front of every prefix: the generic scan of
    the reference (ops.py:82-104) for the rules a precompiled library can offer."""
    _need_cuda(src)
    if op not in SCAN_OPS:
        raise NotImplementedError(f"scan: unknown combine rule {op!r}; available: {sorted(SCAN_OPS)}")
    lib = _lib.load()
    nd = src.dim()
    axis = axis if axis >= 0 else axis + nd
    pre, T, post = src.shape[:axis], src.shape[axis], src.shape[axis + 1:]
    N = 1
    for s in pre:
        N *= s
    D = 1
    for s in post:
        D *= s
    if src.dtype not in _DT:
        raise TypeError(f"unsupported dtype {src.dtype}")
    out_dtype = out_dtype or src.dtype
    x = src.contiguous()
    if init is not None:
        if tuple(init.shape) != tuple(pre) + tuple(post):
            raise ValueError(f"init must have shape {tuple(pre) + tuple(post)}, got {tuple(init.shape)}")  # ops.py:184
        init = init.to(src.dtype).contiguous()
    dst = torch.empty(src.shape, dtype=out_dtype, device=src.device)
    st = lib.gla_scan(_stream(src.device), SCAN_OPS[op], N, T, D, x.data_ptr(), None if init is None else init.data_ptr(),
                      dst.data_ptr(), int(reverse), _DT[src.dtype], _DT[out_dtype])
    _lib.check(st, "gla_scan")
    return dst


def cumsum_pallas(src, axis: int, init: Optional[torch.Tensor] = None, reverse: bool = False,
                  out_dtype=None, max_items: int = 16384, num_warps: int = 4):
    """Inclusive cumulative sum along ``axis`` in float32 with ``init`` (shape = src.shape
    without ``axis``) added to every element (reference: ops.py:166-230, kernel ops.py:152-162)."""
    del max_items, num_warps
    return scan("add", src, axis, init=init, reverse=reverse, out_dtype=out_dtype)


def cumsum_recursive(src, axis: int, init: Optional[torch.Tensor] = None, reverse: bool = False,
                     block_size_t: int = 2048):
    """Reference: ops.py:234-284.  Same kernel as ``cumsum_pallas``; no length limit."""
    del block_size_t
    return cumsum_pallas(src, axis, init=init, reverse=reverse)


def binary_operator(q_i, q_j):
    """Combine rule of the linear-RNN scan in log space (reference: ops.py:286-297)."""
    A_i, b_i = q_i
    A_j, b_j = q_j
    return A_j + A_i, torch.exp(A_j) * b_i + b_j


def rnn_pallas(log_fgate, kv, init_log_fgate: Optional[torch.Tensor] = None,
               init_kv: Optional[torch.Tensor] = None, reverse: bool = False, last_only: bool = False):
    """Inclusive scan of ``(log_fgate (T,K), kv (T,K,V))`` under ``binary_operator`` with an
    optional initial pair; returns ``(cumulative log decay (T,K), states (T,K,V))``
    (reference: ops.py:338-394, kernel ops.py:299-334).  With ``last_only`` only the final row
    (first row when reversed) is defined, as in the reference's masked store.  A leading
    batch axis on all arguments is accepted (the reference vmaps, ops.py:432,447)."""
    _need_cuda(kv)
    lib = _lib.load()
    if (init_log_fgate is None) != (init_kv is None):
        raise ValueError("init_log_fgate and init_kv must be given together")   # ops.py:351
    batched = kv.dim() == 4
    if not batched:
        log_fgate, kv = log_fgate.unsqueeze(0), kv.unsqueeze(0)
        if init_kv is not None:
            init_log_fgate, init_kv = init_log_fgate.unsqueeze(0), init_kv.unsqueeze(0)
    Bn, T, K, V = kv.shape
    if tuple(log_fgate.shape) != (Bn, T, K):
        raise ValueError(f"log_fgate must be {(T, K)}, got {tuple(log_fgate.shape[1:])}")   # ops.py:348
    if kv.dtype not in _DT:
        raise TypeError(f"unsupported dtype {kv.dtype}")
    g = log_fgate.float().contiguous()
    x = kv.contiguous()
    ig = None if init_log_fgate is None else init_log_fgate.float().contiguous()
    ikv = None if init_kv is None else init_kv.to(kv.dtype).contiguous()
    out_log = torch.zeros(Bn, T, K, dtype=torch.float32, device=kv.device)
    out_state = torch.zeros_like(x)
    # scratch for long axes with few rows (0 bytes when the plain scan serves)
    nws = 0 if last_only else lib.gla_rnn_scan_workspace_bytes(Bn, T, K, V)
    ws = torch.empty(nws, dtype=torch.uint8, device=kv.device) if nws else None
    st = lib.gla_rnn_scan_ws(_stream(kv.device), Bn, T, K, V, g.data_ptr(), x.data_ptr(),
                             None if ig is None else ig.data_ptr(), None if ikv is None else ikv.data_ptr(),
                             out_log.data_ptr(), out_state.data_ptr(), int(reverse), int(last_only), _DT[kv.dtype],
                             None if ws is None else ws.data_ptr(), nws)
    _lib.check(st, "gla_rnn_scan_ws")
    out_log = out_log.to(log_fgate.dtype)
    return (out_log, out_state) if batched else (out_log[0], out_state[0])


def rnn_recursive(log_fgate, kv, init_log_fgate: Optional[torch.Tensor] = None,
                  init_kv: Optional[torch.Tensor] = None, block_size_t: int = 256, reverse: bool = False):
    """Reference: ops.py:396-456.  Same kernel as ``rnn_pallas``; no length limit."""
    del block_size_t
    return rnn_pallas(log_fgate, kv, init_log_fgate, init_kv, reverse=reverse)


def _scan_rule(fn):
    """Name of the library's combine rule for a Python callable (or the name itself), else None."""
    import operator
    table = {"add": (torch.add, operator.add), "mul": (torch.mul, operator.mul, torch.multiply),
             "max": (torch.maximum, torch.max, max), "min": (torch.minimum, torch.min, min),
             "logaddexp": (torch.logaddexp,)}
    if isinstance(fn, str):
        return fn if fn in SCAN_OPS else None
    for name, fns in table.items():
        if any(fn is f for f in fns):
            return name
    return None


def triton_scan(fn, args, axis, init=None, reverse: bool = False):
    """Host-level counterpart of the reference's generic in-kernel scan (ops.py:82-104):
    ``out = scan(fn, args)`` along ``axis`` and then ``out = fn(init, out)`` if ``init`` is given.

    The reference traces an arbitrary combine function into Triton; a precompiled library offers named rules,
    recognised here from the callable (or given as a string):

    * on one array, any ``axis``: addition (``torch.add``, ``operator.add``, ``"add"``), multiplication (``"mul"``),
      running maximum / minimum (``torch.maximum`` / ``torch.minimum``, ``"max"`` / ``"min"``) and
      ``torch.logaddexp`` (``"logaddexp"``) -> the tiled scan kernel (``scan``);
    * ``binary_operator`` (or ``"linear_rnn"``) on a pair ``(log_fgate (..., T, K), kv (..., T, K, V))`` scanned
      along the T axis (``axis`` = 0 for unbatched arrays, 1 with a leading batch axis) -> the linear-RNN kernel,
      ``init`` being the pair ``(init_log_fgate (K), init_kv (K, V))``.

    Any other function raises ``NotImplementedError`` (there is no tracing compiler behind this library)."""
    if fn is binary_operator or fn == "linear_rnn":
        log_fgate, kv = args
        t_axis = kv.dim() - 3
        if axis not in (t_axis, t_axis - kv.dim()):
            raise ValueError(f"triton_scan(binary_operator): the scan runs along the time axis ({t_axis})")
        ig, ikv = (None, None) if init is None else init
        return rnn_pallas(log_fgate, kv, ig, ikv, reverse=reverse)
    rule = _scan_rule(fn)
    if rule is not None:
        if isinstance(args, (tuple, list)):
            raise ValueError(f"triton_scan({rule}): expected a single array")
        return scan(rule, args, axis, init=init, reverse=reverse)
    raise NotImplementedError("triton_scan: the combine function is none of the library's rules "
                              f"({sorted(SCAN_OPS)} on one array, binary_operator on a (log_fgate, kv) pair)")
