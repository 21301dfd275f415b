"""JAX adapter: the reference's operators as `jax.custom_vjp` functions over XLA FFI custom
calls into libgla_b200.so (the binding the reference's own framework would use).

NOT EXERCISED where this library was developed: that image has no jax/jaxlib, so neither this
module nor csrc/gla_xla_ffi.cc has been imported, compiled or run.  Importing it without jax
raises ImportError; nothing else in the package depends on it.  Build the handler library
with `python -m gla_jax_b200.build --with-jax` (needs jax.ffi.include_dir()).

Signatures are the reference's (gla.py:405-416, 657-669); the custom-VJP structure mirrors
gla.py:362-388/441 and gla.py:628-655.  Workspaces and residual buffers are extra FFI results
sized at trace time with the C ABI's *_bytes functions.
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


def _dt(x):
    return _lib.GLA_BF16 if x.dtype == jnp.bfloat16 else _lib.GLA_F32


def _u8(n):
    return jax.ShapeDtypeStruct((int(n),), jnp.uint8)


def _batched(hidden, *xs):
    """(T,H,D)->(1,T,H,D): the kernels take the vmap axis natively; jax.vmap maps onto it
    through vmap_method='expand_dims' / 'broadcast_all' of ffi_call."""
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
    dt = _dt(value)
    call = jax.ffi.ffi_call(
        "GlaChunkFwd",
        (jax.ShapeDtypeStruct(hidden_init.shape, hidden_init.dtype), jax.ShapeDtypeStruct(value.shape, value.dtype),
         _u8(lib.gla_chunk_saved_bytes(B, T, H, D, chunk, dt, impl)),
         _u8(lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, chunk, dt, impl))))
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
         _u8(lib.gla_chunk_bwd_workspace_bytes(B, T, H, D, chunk, dt, impl))))
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


@functools.partial(jax.custom_vjp, nondiff_argnums=(5,))
def _recurrent(hidden_init, log_fgate, value, key, query, reverse):
    return _recurrent_fwd(hidden_init, log_fgate, value, key, query, reverse)[0]


def _recurrent_fwd(hidden_init, log_fgate, value, key, query, reverse):
    _register()
    call = jax.ffi.ffi_call("GlaRecurrentFwd", (jax.ShapeDtypeStruct(hidden_init.shape, hidden_init.dtype),
                                                jax.ShapeDtypeStruct(value.shape, value.dtype)))
    hf, out = call(hidden_init, log_fgate.astype(jnp.float32), value, key, query, reverse=np.int64(reverse))
    return (hf, out), (hidden_init, log_fgate, value, key, query)


def _recurrent_bwd(reverse, res, g):
    lib = _lib.load()
    hidden_init, log_fgate, value, key, query = res
    dhf, dout = g
    B, T, H, D = value.shape
    sds = lambda x, d=None: jax.ShapeDtypeStruct(x.shape, d or x.dtype)
    call = jax.ffi.ffi_call("GlaRecurrentBwd", (sds(hidden_init), sds(value, jnp.float32), sds(value), sds(key),
                                                sds(query), _u8(lib.gla_recurrent_bwd_workspace_bytes(B, T, H, D, _dt(value)))))
    dh, dg, dv, dk, dq, _ = call(hidden_init, log_fgate.astype(jnp.float32), value, key, query,
                                 dhf.astype(value.dtype), dout, reverse=np.int64(reverse))
    return dh, dg.astype(log_fgate.dtype), dv, dk, dq


_recurrent.defvjp(_recurrent_fwd, _recurrent_bwd)


def recurrent_gla(hidden_init, log_fgate, value, key, query, reverse: bool = False, max_block_size: int = 64,
                  num_warps: int = 1, num_stages: int = 1, interpret: bool = False):
    """Reference signature gla.py:405-416; tuning arguments accepted and ignored."""
    squeeze, h, (g, v, k, q) = _batched(hidden_init, log_fgate, value, key, query)
    hf, out = _recurrent(h, g, v, k, q, int(bool(reverse)))
    return (hf[0], out[0]) if squeeze else (hf, out)
