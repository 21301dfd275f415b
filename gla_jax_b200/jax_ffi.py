"""JAX adapter: the reference's operators as `jax.custom_vjp` functions over XLA FFI custom
calls into libgla_b200.so (the binding the reference's own framework would use).

NOT EXERCISED: no environment with jax/jaxlib has been available to this library, so neither this
module nor csrc/gla_xla_ffi.cc has been imported, compiled or run.  Importing it without jax
raises ImportError; nothing else in the package depends on it.  Build the handler library
with `python -m gla_jax_b200.build --with-jax` (needs jax.ffi.include_dir()).

Signatures are the reference's (gla.py:26, 405-416, 657-669; ops.py:166, 234, 338, 396); the custom-VJP
structure mirrors gla.py:362-388/441 and gla.py:628-655.  Workspaces and residual buffers are extra FFI
results sized at trace time with the C ABI's *_bytes functions (their sizes are linear in the batch).

jax.vmap (the reference maps chunk_gla over the batch with it, gla.py:1335): every ffi_call below passes
vmap_method="broadcast_all", so a mapped call reaches the handler with one more leading axis on every operand
and result, and the handlers fold all leading axes into the batch size the kernels take natively.
"""
from __future__ import annotations

import ctypes
import functools
from pathlib import Path

import jax
import jax.numpy as jnp
import numpy as np

from . import _lib

_FFI_LIB = Path(__file__).resolve().parent / "libgla_b200_xla.so"
_registered = False


def _register():
    global _registered
    if _registered:
        return
    if not _FFI_LIB.exists():
        raise RuntimeError(f"{_FFI_LIB} not built: run `python -m gla_jax_b200.build --with-jax`")
    _lib.load()                                   # the kernels themselves
    ffi_lib = ctypes.CDLL(str(_FFI_LIB))
    for name in ("GlaChunkFwd", "GlaChunkBwd", "GlaRecurrentFwd", "GlaRecurrentBwd", "GlaCumsum", "GlaRnnScan"):
        jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(ffi_lib, name)), platform="CUDA")
    _registered = True


_VMAP = "broadcast_all"


def _dt(x):
    if x.dtype == jnp.bfloat16:
        return _lib.GLA_BF16
    if x.dtype == jnp.float32:
        return _lib.GLA_F32
    raise TypeError(f"unsupported dtype {x.dtype}: float32 and bfloat16 are implemented")


def _same_dtype(*xs):
    for x in xs[1:]:
        if x.dtype != xs[0].dtype:
            raise TypeError("hidden, value, key and query must share a dtype")
    return _dt(xs[0])


def _u8(n):
    return jax.ShapeDtypeStruct((int(n),), jnp.uint8)


def _batched(hidden, *xs):
    """(T,H,D)->(1,T,H,D): the kernels take a batch axis natively; jax.vmap adds further leading axes
    (vmap_method="broadcast_all"), which the handlers fold into it."""
    if xs[0].ndim == 3:
        return True, hidden[None], tuple(x[None] for x in xs)
    return False, hidden, xs


@functools.partial(jax.custom_vjp, nondiff_argnums=(5, 6))
def _chunk(hidden_init, log_fgate, value, key, query, chunk, impl):
    return _chunk_fwd(hidden_init, log_fgate, value, key, query, chunk, impl)[0]


def _chunk_fwd(hidden_init, log_fgate, value, key, query, chunk, impl):
    _register()
    lib = _lib.load()
    B, T, H, D = value.shape
    dt = _same_dtype(value, hidden_init, key, query)
    call = jax.ffi.ffi_call(
        "GlaChunkFwd",
        (jax.ShapeDtypeStruct(hidden_init.shape, hidden_init.dtype), jax.ShapeDtypeStruct(value.shape, value.dtype),
         _u8(lib.gla_chunk_saved_bytes(B, T, H, D, chunk, dt, impl)),
         _u8(lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, chunk, dt, impl))), vmap_method=_VMAP)
    hf, out, saved, _ = call(hidden_init, log_fgate.astype(jnp.float32), value, key, query,
                             chunk=np.int64(chunk), impl=np.int64(impl))
    return (hf, out), (log_fgate, value, key, query, saved)


def _chunk_bwd(chunk, impl, res, g):
    lib = _lib.load()
    log_fgate, value, key, query, saved = res
    dhf, dout = g
    B, T, H, D = value.shape
    dt = _dt(value)
    call = jax.ffi.ffi_call(
        "GlaChunkBwd",
        (jax.ShapeDtypeStruct((B, H, D, D), value.dtype), jax.ShapeDtypeStruct(value.shape, jnp.float32),
         jax.ShapeDtypeStruct(value.shape, value.dtype), jax.ShapeDtypeStruct(value.shape, value.dtype),
         jax.ShapeDtypeStruct(value.shape, value.dtype),
         _u8(lib.gla_chunk_bwd_workspace_bytes(B, T, H, D, chunk, dt, impl))), vmap_method=_VMAP)
    dh, dg, dv, dk, dq, _ = call(log_fgate.astype(jnp.float32), value, key, query, saved, dhf.astype(value.dtype),
                                 dout.astype(value.dtype), chunk=np.int64(chunk), impl=np.int64(impl))
    return dh, dg.astype(log_fgate.dtype), dv, dk, dq


_chunk.defvjp(_chunk_fwd, _chunk_bwd)


def chunk_gla(hidden_init, log_fgate, value, key, query, chunk_size, block_size_t: int = 64, block_size_d: int = 64,
              interpret: bool = False, num_warps: int = 4, num_stages: int = 2):
    """Reference signature gla.py:657-669; tuning arguments accepted and ignored."""
    squeeze, h, (g, v, k, q) = _batched(hidden_init, log_fgate, value, key, query)
    hf, out = _chunk(h, g, v, k, q, int(chunk_size), _lib.IMPL_AUTO)
    return (hf[0], out[0]) if squeeze else (hf, out)


@functools.partial(jax.custom_vjp, nondiff_argnums=(5, 6))
def _recurrent(hidden_init, log_fgate, value, key, query, reverse, out_f32):
    return _recurrent_fwd(hidden_init, log_fgate, value, key, query, reverse, out_f32)[0]


def _recurrent_fwd(hidden_init, log_fgate, value, key, query, reverse, out_f32):
    _register()
    _same_dtype(value, hidden_init, key, query)
    call = jax.ffi.ffi_call("GlaRecurrentFwd", (jax.ShapeDtypeStruct(hidden_init.shape, hidden_init.dtype),
                                                jax.ShapeDtypeStruct(value.shape, jnp.float32 if out_f32 else value.dtype)),
                            vmap_method=_VMAP)
    hf, out = call(hidden_init, log_fgate.astype(jnp.float32), value, key, query, reverse=np.int64(reverse))
    return (hf, out), (hidden_init, log_fgate, value, key, query)


def _recurrent_bwd(reverse, out_f32, res, g):
    lib = _lib.load()
    hidden_init, log_fgate, value, key, query = res
    dhf, dout = g
    B, T, H, D = value.shape
    sds = lambda x, d=None: jax.ShapeDtypeStruct(x.shape, d or x.dtype)
    call = jax.ffi.ffi_call("GlaRecurrentBwd", (sds(hidden_init), sds(value, jnp.float32), sds(value), sds(key),
                                                sds(query), _u8(lib.gla_recurrent_bwd_workspace_bytes(B, T, H, D, _dt(value)))),
                            vmap_method=_VMAP)
    if dout.dtype not in (jnp.float32, jnp.bfloat16):
        dout = dout.astype(jnp.float32)
    dh, dg, dv, dk, dq, _ = call(hidden_init, log_fgate.astype(jnp.float32), value, key, query,
                                 dhf.astype(value.dtype), dout, reverse=np.int64(reverse))
    return dh, dg.astype(log_fgate.dtype), dv, dk, dq


_recurrent.defvjp(_recurrent_fwd, _recurrent_bwd)


def recurrent_gla(hidden_init, log_fgate, value, key, query, reverse: bool = False, max_block_size: int = 64,
                  num_warps: int = 1, num_stages: int = 1, interpret: bool = False):
    """Reference signature gla.py:405-416; tuning arguments accepted and ignored."""
    squeeze, h, (g, v, k, q) = _batched(hidden_init, log_fgate, value, key, query)
    hf, out = _recurrent(h, g, v, k, q, int(bool(reverse)), False)
    return (hf[0], out[0]) if squeeze else (hf, out)


def recurrent_gla_naive(hidden, log_fgate, value, key, query, reverse: bool = False):
    """Reference signature gla.py:26: the definitional recurrence; `out` is float32 and `hidden_final` keeps
    hidden's dtype (gla.py:43-46).  Runs the same on-chip recurrence kernel as recurrent_gla."""
    squeeze, h, (g, v, k, q) = _batched(hidden, log_fgate, value, key, query)
    hf, out = _recurrent(h, g, v, k, q, int(bool(reverse)), True)
    return (hf[0], out[0]) if squeeze else (hf, out)


# ---- scan ops of ops.py (forward only, like the reference's Pallas calls) ----------------------------------

def cumsum_pallas(src, axis: int, init=None, reverse: bool = False, out_dtype=None):
    """Reference signature ops.py:166: inclusive cumulative sum along `axis`, `init` added to every element."""
    _register()
    _dt(src)
    axis = axis % src.ndim
    x = jnp.moveaxis(src, axis, -2) if axis != src.ndim - 2 else src          # (..., T, D) with the scan axis second to last
    if axis == src.ndim - 1:
        x = src[..., None]
    lead = x.shape[:-2]
    x3 = x.reshape((-1,) + x.shape[-2:])
    odt = out_dtype or src.dtype
    i3 = jnp.zeros((0,), src.dtype) if init is None else jnp.broadcast_to(init, lead + x.shape[-1:]).reshape(-1, x.shape[-1]).astype(src.dtype)
    call = jax.ffi.ffi_call("GlaCumsum", jax.ShapeDtypeStruct(x3.shape, odt), vmap_method=_VMAP)
    y = call(x3, i3, reverse=np.int64(bool(reverse))).reshape(x.shape)
    if axis == src.ndim - 1:
        return y[..., 0]
    return jnp.moveaxis(y, -2, axis) if axis != src.ndim - 2 else y


def cumsum_recursive(src, axis: int, init=None, reverse: bool = False, out_dtype=None, block_size: int = 2048):
    """Reference signature ops.py:234; the CUDA kernel scans any length in one launch, so `block_size` is ignored."""
    del block_size
    return cumsum_pallas(src, axis, init=init, reverse=reverse, out_dtype=out_dtype)


def rnn_pallas(log_fgate, kv, init_log_fgate=None, init_kv=None, reverse: bool = False, last_only: bool = False):
    """Reference signature ops.py:338: log-space linear-RNN scan over the leading axis of (log_fgate (T, K),
    kv (T, K, V)) under ops.py:286 binary_operator; returns (cumulative log decay, states)."""
    _register()
    _dt(kv)
    if (init_log_fgate is None) != (init_kv is None):
        raise ValueError("init_log_fgate and init_kv must be given together")          # ops.py:351
    g3, kv4 = log_fgate.astype(jnp.float32)[None], kv[None]
    ig = jnp.zeros((0,), jnp.float32) if init_kv is None else init_log_fgate.astype(jnp.float32)[None]
    ikv = jnp.zeros((0,), kv.dtype) if init_kv is None else init_kv.astype(kv.dtype)[None]
    call = jax.ffi.ffi_call("GlaRnnScan", (jax.ShapeDtypeStruct(g3.shape, jnp.float32), jax.ShapeDtypeStruct(kv4.shape, kv.dtype)),
                            vmap_method=_VMAP)
    out_log, out_state = call(g3, kv4, ig, ikv, reverse=np.int64(bool(reverse)), last_only=np.int64(bool(last_only)))
    return out_log[0], out_state[0]


def rnn_recursive(log_fgate, kv, init_log_fgate=None, init_kv=None, reverse: bool = False, block_size: int = 256):
    """Reference signature ops.py:396; one launch covers any length, so `block_size` is ignored."""
    del block_size
    return rnn_pallas(log_fgate, kv, init_log_fgate, init_kv, reverse=reverse)
