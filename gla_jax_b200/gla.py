"""The GLA operators with the reference's signatures (gla.py of zhixuan-lin/gla-jax), backed
by libgla_b200.so.

    chunk_gla(hidden_init, log_fgate, value, key, query, chunk_size, ...)   gla.py:657
    recurrent_gla(hidden_init, log_fgate, value, key, query, reverse, ...)  gla.py:405
    recurrent_gla_naive(hidden, log_fgate, value, key, query, reverse)      gla.py:26

All return ``(hidden_final, out)``.  Shapes are the reference's per-sequence shapes
``log_fgate, value, key, query : (T, H, D)``, ``hidden : (H, D, D)``; where the reference
adds a batch axis with ``jax.vmap`` (gla.py:1335), pass arrays with a leading batch axis
instead (``(B, T, H, D)`` and ``(B, H, D, D)``) — the kernels take the batch natively.

This adapter holds device memory in torch CUDA tensors and differentiates through
``torch.autograd.Function`` objects that mirror the reference's ``jax.custom_vjp`` pairs
(gla.py:362/441 and gla.py:628/655).  The JAX adapter (XLA FFI handlers plus
``jax.custom_vjp``) is ``jax_ffi.py`` / ``csrc/gla_xla_ffi.cc``; both call the same C ABI.
There is no CPU path: CPU tensors raise.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib

_DT = {torch.float32: _lib.GLA_F32, torch.bfloat16: _lib.GLA_BF16}


def _ptr(t):
    return None if t is None else t.data_ptr()


_stream = _lib.stream_of


def _prepare(hidden, log_fgate, value, key, query):
    """Validate like the reference's trace-time asserts (gla.py:118-127, 498-500) and return
    contiguous batched tensors plus whether a batch axis has to be stripped again."""
    if not value.is_cuda:
        raise RuntimeError("gla_jax_b200 operators need CUDA tensors; there is no CPU fallback")
    if value.dim() not in (3, 4):
        raise ValueError(f"value must be (T,H,D) or (B,T,H,D), got {tuple(value.shape)}")
    batched = value.dim() == 4
    if not (log_fgate.shape == value.shape == key.shape == query.shape):
        raise ValueError("log_fgate, value, key, query must have the same shape "
                         f"({tuple(log_fgate.shape)}, {tuple(value.shape)}, {tuple(key.shape)}, {tuple(query.shape)})")
    if not batched:
        hidden, log_fgate, value, key, query = (x.unsqueeze(0) for x in (hidden, log_fgate, value, key, query))
    B, T, H, D = value.shape
    if tuple(hidden.shape) != (B, H, D, D):
        raise ValueError(f"hidden must be {'(B,' if batched else '('}H,D,D) = {(B, H, D, D)}, got {tuple(hidden.shape)}")
    dt = value.dtype
    if dt not in _DT:
        raise TypeError(f"unsupported dtype {dt}: float32 and bfloat16 are implemented")
    if not (key.dtype == query.dtype == hidden.dtype == dt):
        raise TypeError("value, key, query and hidden must share one dtype")
    return (hidden.contiguous(), log_fgate.contiguous(), value.contiguous(), key.contiguous(), query.contiguous(),
            batched)


def _chunk_fwd_raw(hidden, g32, v, k, q, chunk, impl, need_grad):
    """gla_chunk_fwd on batched contiguous tensors -> (hidden_final, out, (saved,) or ())."""
    lib = _lib.load()
    B, T, H, D = v.shape
    dt = _DT[v.dtype]
    dev = v.device
    ws_n = lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, chunk, dt, impl)
    if ws_n == 0:
        raise _lib.GlaError(f"chunk_gla: unsupported configuration T={T} H={H} D={D} chunk={chunk} dtype={v.dtype}")
    saved = None
    if need_grad:
        saved = torch.empty(lib.gla_chunk_saved_bytes(B, T, H, D, chunk, dt, impl), dtype=torch.uint8, device=dev)
    ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
    hf = torch.empty_like(hidden)
    out = torch.empty_like(v)
    st = lib.gla_chunk_fwd(_stream(dev), B, T, H, D, chunk, dt, impl, _ptr(hidden), _ptr(g32), _ptr(v), _ptr(k),
                           _ptr(q), _ptr(hf), _ptr(out), _ptr(saved), _ptr(ws), ws_n)
    _lib.check(st, "gla_chunk_fwd")
    return hf, out, ((saved,) if need_grad else ())


def _chunk_bwd_raw(g32, v, k, q, residuals, dhf, dout, chunk, impl):
    """gla_chunk_bwd -> (dhidden_init, dlog_fgate (float32), dvalue, dkey, dquery)."""
    lib = _lib.load()
    (saved,) = residuals
    B, T, H, D = v.shape
    dt = _DT[v.dtype]
    dev = v.device
    ws_n = lib.gla_chunk_bwd_workspace_bytes(B, T, H, D, chunk, dt, impl)
    ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
    dh = torch.empty(B, H, D, D, dtype=v.dtype, device=dev)
    dg = torch.empty_like(g32)
    dv, dk, dq = torch.empty_like(v), torch.empty_like(k), torch.empty_like(q)
    st = lib.gla_chunk_bwd(_stream(dev), B, T, H, D, chunk, dt, impl, _ptr(g32), _ptr(v), _ptr(k), _ptr(q),
                           _ptr(saved), _ptr(dhf), _ptr(dout), _ptr(dh), _ptr(dg), _ptr(dv), _ptr(dk), _ptr(dq),
                           _ptr(ws), ws_n)
    _lib.check(st, "gla_chunk_bwd")
    return dh, dg, dv, dk, dq


class _ChunkGLA(torch.autograd.Function):
    """custom-VJP pair of chunk_gla (gla.py:628-655)."""

    @staticmethod
    def forward(ctx, hidden, g, v, k, q, chunk, impl):
        g32 = g if g.dtype == torch.float32 else g.float()
        need_grad = any(ctx.needs_input_grad[:5])
        hf, out, res = _chunk_fwd_raw(hidden, g32, v, k, q, chunk, impl, need_grad)
        ctx.save_for_backward(g32, v, k, q, *res)
        ctx.chunk, ctx.impl, ctx.g_dtype = chunk, impl, g.dtype
        return hf, out

    @staticmethod
    def backward(ctx, dhf, dout):
        g32, v, k, q, *res = ctx.saved_tensors
        B, T, H, D = v.shape
        dhf = torch.zeros(B, H, D, D, dtype=v.dtype, device=v.device) if dhf is None else dhf.to(v.dtype).contiguous()
        dout = torch.zeros_like(v) if dout is None else dout.to(v.dtype).contiguous()
        dh, dg, dv, dk, dq = _chunk_bwd_raw(g32, v, k, q, tuple(res), dhf, dout, ctx.chunk, ctx.impl)
        return dh, dg.to(ctx.g_dtype), dv, dk, dq, None, None


def chunk_gla(hidden_init, log_fgate, value, key, query, chunk_size: int,
              block_size_t: int = 64, block_size_d: int = 64, interpret: bool = False,
              num_warps: int = 4, num_stages: int = 2, impl: str = "auto") -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunk-wise GLA with multi-scale secondary chunking (reference: gla.py:657-692).

    ``block_size_t``, ``block_size_d``, ``num_warps``, ``num_stages`` and ``interpret`` are
    the reference's Triton tuning knobs; they are accepted for caller compatibility and
    ignored (the CUDA kernels fix their own tiling).  ``impl`` selects the kernel family:
    ``"auto"`` (tensor cores when the shape has a kernel), ``"tcgen05"`` or ``"fp32"``.
    """
    del block_size_t, block_size_d, interpret, num_warps, num_stages
    chunk_size = int(chunk_size)
    T = value.shape[-3]
    if chunk_size <= 0 or chunk_size & (chunk_size - 1):
        raise ValueError(f"Chunk length must be power of 2, but got {chunk_size}")   # gla.py:500
    if T % chunk_size:
        raise ValueError(f"sequence length {T} is not a multiple of chunk_size {chunk_size}")  # gla.py:674
    h, g, v, k, q, batched = _prepare(hidden_init, log_fgate, value, key, query)
    hf, out = _ChunkGLA.apply(h, g, v, k, q, chunk_size, _lib.IMPL_BY_NAME[impl])
    return (hf, out) if batched else (hf[0], out[0])


class _RecurrentGLA(torch.autograd.Function):
    """custom-VJP pair of recurrent_gla (gla.py:362-388, 441)."""

    @staticmethod
    def forward(ctx, hidden, g, v, k, q, reverse, out_fp32):
        lib = _lib.load()
        B, T, H, D = v.shape
        dt = _DT[v.dtype]
        dev = v.device
        g32 = g if g.dtype == torch.float32 else g.float()
        hf = torch.empty_like(hidden)
        out = torch.empty(v.shape, dtype=torch.float32 if out_fp32 else v.dtype, device=dev)
        st = lib.gla_recurrent_fwd(_stream(dev), B, T, H, D, dt, _ptr(hidden), _ptr(g32), _ptr(v), _ptr(k), _ptr(q),
                                   _ptr(hf), _ptr(out), _DT[out.dtype], int(reverse))
        _lib.check(st, "gla_recurrent_fwd")
        ctx.save_for_backward(hidden, g32, v, k, q)
        ctx.reverse, ctx.g_dtype = bool(reverse), g.dtype
        return hf, out

    @staticmethod
    def backward(ctx, dhf, dout):
        lib = _lib.load()
        hidden, g32, v, k, q = ctx.saved_tensors
        B, T, H, D = v.shape
        dt = _DT[v.dtype]
        dev = v.device
        dhf = torch.zeros_like(hidden) if dhf is None else dhf.to(v.dtype).contiguous()
        dout = torch.zeros_like(v) if dout is None else dout.contiguous()
        if dout.dtype not in _DT:
            dout = dout.float()
        ws_n = lib.gla_recurrent_bwd_workspace_bytes(B, T, H, D, dt)
        ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
        dh = torch.empty_like(hidden)
        dg = torch.empty_like(g32)
        dv, dk, dq = torch.empty_like(v), torch.empty_like(k), torch.empty_like(q)
        st = lib.gla_recurrent_bwd(_stream(dev), B, T, H, D, dt, _ptr(hidden), _ptr(g32), _ptr(v), _ptr(k), _ptr(q),
                                   _ptr(dhf), _ptr(dout), _DT[dout.dtype], _ptr(dh), _ptr(dg), _ptr(dv), _ptr(dk),
                                   _ptr(dq), int(ctx.reverse), _ptr(ws), ws_n)
        _lib.check(st, "gla_recurrent_bwd")
        return dh, dg.to(ctx.g_dtype), dv, dk, dq, None, None


def recurrent_gla(hidden_init, log_fgate, value, key, query, reverse: bool = False,
                  max_block_size: int = 64, num_warps: int = 1, num_stages: int = 1,
                  interpret: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exact recurrence that never writes hidden states to memory (reference: gla.py:405-439).
    ``max_block_size``, ``num_warps``, ``num_stages``, ``interpret`` are accepted and ignored."""
    del max_block_size, num_warps, num_stages, interpret
    if value.shape[-2] != key.shape[-2]:
        raise ValueError("value and key must have the same number of heads")   # gla.py:417
    h, g, v, k, q, batched = _prepare(hidden_init, log_fgate, value, key, query)
    hf, out = _RecurrentGLA.apply(h, g, v, k, q, bool(reverse), False)
    return (hf, out) if batched else (hf[0], out[0])


def recurrent_gla_naive(hidden, log_fgate, value, key, query, reverse: bool = False):
    """The definitional recurrence (reference: gla.py:26-47).  On this backend it runs the same
    on-chip recurrence kernel as ``recurrent_gla``; as in the reference ``out`` is float32
    and ``hidden_final`` keeps ``hidden``'s dtype (gla.py:43-46)."""
    h, g, v, k, q, batched = _prepare(hidden, log_fgate, value, key, query)
    hf, out = _RecurrentGLA.apply(h, g, v, k, q, bool(reverse), True)
    return (hf, out) if batched else (hf[0], out[0])


class _ChunkGLAPacked(torch.autograd.Function):
    """chunk_gla over sequences laid end to end on one time axis (gla_chunk_fwd_packed / gla_chunk_bwd_packed)."""

    @staticmethod
    def forward(ctx, hidden, g, v, k, q, cu, chunk):
        lib = _lib.load()
        T, H, D = v.shape
        nseq = hidden.shape[0]
        dt = _DT[v.dtype]
        g32 = g if g.dtype == torch.float32 else g.float()
        ws_n = lib.gla_chunk_fwd_workspace_bytes(1, T, H, D, chunk, dt, _lib.IMPL_TCGEN05)
        if ws_n == 0:
            raise _lib.GlaError(f"chunk_gla_packed: unsupported configuration T={T} H={H} D={D} chunk={chunk} dtype={v.dtype}")
        need_grad = any(ctx.needs_input_grad[:5])
        saved = torch.empty(lib.gla_chunk_saved_bytes(1, T, H, D, chunk, dt, _lib.IMPL_TCGEN05), dtype=torch.uint8,
                            device=v.device) if need_grad else None
        ws = torch.empty(ws_n, dtype=torch.uint8, device=v.device)
        hf, out = torch.empty_like(hidden), torch.empty_like(v)
        st = lib.gla_chunk_fwd_packed(_stream(v.device), T, H, D, chunk, dt, nseq, _ptr(cu), _ptr(hidden), _ptr(g32), _ptr(v),
                                      _ptr(k), _ptr(q), _ptr(hf), _ptr(out), _ptr(saved), _ptr(ws), ws_n)
        _lib.check(st, "gla_chunk_fwd_packed")
        if need_grad:
            ctx.save_for_backward(g32, v, k, q, cu, saved)
        ctx.chunk, ctx.g_dtype, ctx.nseq = chunk, g.dtype, nseq
        return hf, out

    @staticmethod
    def backward(ctx, dhf, dout):
        lib = _lib.load()
        g32, v, k, q, cu, saved = ctx.saved_tensors
        T, H, D = v.shape
        dt = _DT[v.dtype]
        dhf = torch.zeros(ctx.nseq, H, D, D, dtype=v.dtype, device=v.device) if dhf is None else dhf.to(v.dtype).contiguous()
        dout = torch.zeros_like(v) if dout is None else dout.to(v.dtype).contiguous()
        ws_n = lib.gla_chunk_bwd_workspace_bytes(1, T, H, D, ctx.chunk, dt, _lib.IMPL_TCGEN05)
        ws = torch.empty(ws_n, dtype=torch.uint8, device=v.device)
        dh = torch.empty_like(dhf)
        dg = torch.empty_like(g32)
        dv, dk, dq = torch.empty_like(v), torch.empty_like(k), torch.empty_like(q)
        st = lib.gla_chunk_bwd_packed(_stream(v.device), T, H, D, ctx.chunk, dt, ctx.nseq, _ptr(cu), _ptr(g32), _ptr(v),
                                      _ptr(k), _ptr(q), _ptr(saved), _ptr(dhf), _ptr(dout), _ptr(dh), _ptr(dg), _ptr(dv),
                                      _ptr(dk), _ptr(dq), _ptr(ws), ws_n)
        _lib.check(st, "gla_chunk_bwd_packed")
        return dh, dg.to(ctx.g_dtype), dv, dk, dq, None, None


def chunk_gla_packed(hidden_init, log_fgate, value, key, query, cu_seqlens, chunk_size: int = 128):
    """``chunk_gla`` for variable-length sequences packed end to end on one time axis.

    ``value/key/query/log_fgate`` are (T, H, D) holding ``nseq`` sequences back to back; ``cu_seqlens`` holds the
    ``nseq + 1`` token offsets (0 first, T last); ``hidden_init`` is (nseq, H, D, D).  Returns
    ``(hidden_final (nseq, H, D, D), out (T, H, D))``, equal to calling ``chunk_gla`` on each sequence;
    differentiable.  The reference has one length per call and asserts T % chunk == 0 (gla.py:499-500, 674); this
    runs on the tensor-core kernels only (bf16, D = 128).

    Offsets given as a list or CPU tensor may be ANY rising sequence: the kernels work on chunks of 128 rows that
    must not straddle two sequences, so sequences whose lengths are not multiples of 128 are first laid out with
    their tails padded to the next multiple (padding tokens have log_fgate = 0 and key = value = query = 0: no decay,
    no update, so states and gradients are those of the unpadded sequence) and the outputs are gathered back; the
    two copies are differentiable torch index operations.  Offsets given as a CUDA int32 tensor are used as they
    are, without a host round trip, and must be multiples of 128 (the kernels clamp anything else and count it in
    ``gla_device_bad_offsets``)."""
    if value.dim() != 3 or hidden_init.dim() != 4:
        raise ValueError("chunk_gla_packed: expected value (T, H, D) and hidden_init (nseq, H, D, D)")
    T, H, D = value.shape
    cu = torch.as_tensor(cu_seqlens, dtype=torch.int32) if not torch.is_tensor(cu_seqlens) else cu_seqlens.to(torch.int32)
    nseq = cu.numel() - 1
    if nseq < 1 or tuple(hidden_init.shape) != (nseq, H, D, D):
        raise ValueError("chunk_gla_packed: cu_seqlens must have nseq + 1 entries for hidden_init (nseq, H, D, D)")
    if key.shape != value.shape or query.shape != value.shape or log_fgate.shape != value.shape:
        raise ValueError("chunk_gla_packed: log_fgate, value, key, query must all be (T, H, D)")
    if not value.is_cuda:
        raise TypeError("chunk_gla_packed: CUDA tensors required (there is no CPU path)")
    idx = None
    if not cu.is_cuda:
        # offsets given on the host are checked here; a CUDA tensor is taken as is (checking it would synchronise)
        if int(cu[0]) != 0 or int(cu[-1]) != T or bool(((cu[1:] - cu[:-1]) <= 0).any()):
            raise ValueError("chunk_gla_packed: cu_seqlens must rise from 0 to T")
        if bool((cu % 128 != 0).any()):
            # ragged lengths: positions of the tokens on a time axis where every sequence starts at a multiple of 128
            lens = (cu[1:] - cu[:-1]).to(torch.int64)
            plen = (lens + 127) // 128 * 128
            pcu = torch.zeros(nseq + 1, dtype=torch.int64)
            pcu[1:] = torch.cumsum(plen, 0)
            idx = torch.cat([torch.arange(int(lens[s_]), dtype=torch.int64) + int(pcu[s_]) for s_ in range(nseq)]).to(value.device)
            Tp = int(pcu[-1])
            pad = lambda x: x.new_zeros((Tp,) + tuple(x.shape[1:])).index_copy(0, idx, x)
            log_fgate, value, key, query = pad(log_fgate), pad(value), pad(key), pad(query)
            cu = pcu.to(torch.int32)
    cu = cu.to(value.device).contiguous()
    hf, out = _ChunkGLAPacked.apply(hidden_init.contiguous(), log_fgate.contiguous(), value.contiguous(), key.contiguous(),
                                    query.contiguous(), cu, int(chunk_size))
    return (hf, out) if idx is None else (hf, out.index_select(0, idx))


def decode_step(state, log_fgate, value, key, query, out_dtype=None):
    """One token of the recurrence (reference: the loop body of gla.py:26-47) for a batch of requests.

    ``state`` (B, H, D, D) float32 CUDA tensor is updated IN PLACE
    (``S <- exp(log_fgate)[..., None] * S + key[..., None] * value[..., None, :]``); returns
    ``out = query @ S`` of shape (B, H, D) in ``out_dtype`` (default: value's dtype).  ``log_fgate``,
    ``value``, ``key``, ``query`` are (B, H, D).  T calls equal one ``recurrent_gla`` over T tokens
    (``hidden_init`` -> ``hidden_final`` chaining, gla.py:720-723).  Not differentiable (serving path)."""
    lib = _lib.load()
    if state.dtype != torch.float32 or not state.is_contiguous() or state.dim() != 4:
        raise TypeError("decode_step: state must be a contiguous float32 (B, H, D, D) tensor")
    B, H, D, D2 = state.shape
    if D != D2 or tuple(value.shape) != (B, H, D) or key.shape != value.shape or query.shape != value.shape \
            or log_fgate.shape != value.shape:
        raise ValueError("decode_step: expected state (B, H, D, D) and log_fgate, value, key, query (B, H, D)")
    if key.dtype != value.dtype or query.dtype != value.dtype:
        raise TypeError("decode_step: value, key, query must share a dtype")
    g32 = log_fgate.float().contiguous()
    v, k, q = value.contiguous(), key.contiguous(), query.contiguous()
    out = torch.empty(B, H, D, dtype=out_dtype or v.dtype, device=v.device)
    st = lib.gla_decode_step(_stream(v.device), B, H, D, _DT[v.dtype], _ptr(state), _ptr(g32), _ptr(v), _ptr(k), _ptr(q),
                             _ptr(out), _DT[out.dtype])
    _lib.check(st, "gla_decode_step")
    return out


def auto_block_size(value_dim: int, key_dim: int, num_heads: int, max_block_size: int):
    """Reference helper (gla.py:390-403) kept for callers that import it: the Triton block
    sizes it would have chosen.  The CUDA kernels do not use them."""
    assert value_dim == key_dim, "Not supported yet"
    vb = min(max_block_size, value_dim)
    kb = min(max_block_size, key_dim)
    hb = None
    for c in sorted(c for c in range(1, num_heads + 1) if num_heads % c == 0):
        if c * vb <= max_block_size and c * kb <= max_block_size:
            hb = c
        else:
            break
    assert hb is not None
    return vb, kb, hb
