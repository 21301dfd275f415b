"""A gated-linear-attention layer around ``chunk_gla``: the caller either side of the op.

The reference ships the op only (gla.py:657 ``chunk_gla``, gla.py:405 ``recurrent_gla``); this is
the smallest real caller of it, built from the published GLA layer recipe:

    q, k, v   = x Wq, (x Wk) / sqrt(D), x Wv                      (B, T, H, D)
    log_fgate = log_sigmoid((x Wg1) Wg2 + bg) / tau               float32, low-rank gate projection
    _, out    = chunk_gla(hidden, log_fgate, v, k, q, chunk_size)
    o         = rmsnorm_per_head(out) * w_norm * swish(x Wgate)
    y         = o Wo

The projections are library GEMMs (``torch.nn.functional.linear``).  The two element-wise stages
run as single CUDA passes through the C ABI (``gla_layer_gate_*``, ``gla_layer_headnorm_gate_*``),
each with a hand-written backward, so that ``log_fgate`` is produced in float32 directly from the
projection's dtype and ``out`` is read once for normalisation, weight and output gate together.
There is no CPU path: CPU tensors raise.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from .gla import _DT, _ptr, _stream, chunk_gla, recurrent_gla


def _need_cuda(t, what):
    if not t.is_cuda:
        raise RuntimeError(f"{what} needs CUDA tensors; there is no CPU fallback")
    if t.dtype not in _DT:
        raise TypeError(f"{what}: unsupported dtype {t.dtype}: float32 and bfloat16 are implemented")


class _LogForgetGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, inv_tau):
        _need_cuda(z, "log_forget_gate")
        lib = _lib.load()
        z = z.contiguous()
        g = torch.empty(z.shape, dtype=torch.float32, device=z.device)
        st = lib.gla_layer_gate_fwd(_stream(z.device), z.numel(), _DT[z.dtype], _ptr(z), float(inv_tau), _ptr(g))
        _lib.check(st, "gla_layer_gate_fwd")
        ctx.save_for_backward(z)
        ctx.inv_tau = float(inv_tau)
        return g

    @staticmethod
    def backward(ctx, dg):
        (z,) = ctx.saved_tensors
        lib = _lib.load()
        dg = dg.contiguous().float()
        dz = torch.empty_like(z)
        st = lib.gla_layer_gate_bwd(_stream(z.device), z.numel(), _DT[z.dtype], _ptr(z), _ptr(dg), ctx.inv_tau, _ptr(dz))
        _lib.check(st, "gla_layer_gate_bwd")
        return dz, None


def log_forget_gate(z: torch.Tensor, tau: float = 16.0) -> torch.Tensor:
    """``log_sigmoid(z) / tau`` in float32, whatever z's dtype: the ``log_fgate`` operand of the op."""
    return _LogForgetGate.apply(z, 1.0 / tau)


class _HeadNormGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, weight, eps):
        _need_cuda(x, "headnorm_gate")
        if gate.shape != x.shape or gate.dtype != x.dtype:
            raise ValueError("headnorm_gate: gate must have x's shape and dtype")
        D = x.shape[-1]
        if weight is not None and (tuple(weight.shape) != (D,) or weight.dtype != torch.float32):
            raise ValueError(f"headnorm_gate: weight must be float32 of shape ({D},)")
        lib = _lib.load()
        x, gate = x.contiguous(), gate.contiguous()
        rows = x.numel() // D
        y = torch.empty_like(x)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        w = None if weight is None else weight.contiguous()
        st = lib.gla_layer_headnorm_gate_fwd(_stream(x.device), rows, D, _DT[x.dtype], _ptr(x), _ptr(gate), _ptr(w),
                                             float(eps), _ptr(y), _ptr(rstd))
        _lib.check(st, "gla_layer_headnorm_gate_fwd")
        ctx.save_for_backward(x, gate, rstd, *(() if w is None else (w,)))
        ctx.has_weight = w is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gate, rstd = ctx.saved_tensors[:3]
        w = ctx.saved_tensors[3] if ctx.has_weight else None
        lib = _lib.load()
        D = x.shape[-1]
        rows = x.numel() // D
        dy = dy.contiguous()
        dx, dgate = torch.empty_like(x), torch.empty_like(gate)
        want_dw = ctx.has_weight and ctx.needs_input_grad[2]
        dw = torch.empty(D, dtype=torch.float32, device=x.device) if want_dw else None
        ws_n = lib.gla_layer_headnorm_gate_bwd_workspace_bytes(rows, D) if want_dw else 0
        ws = torch.empty(ws_n, dtype=torch.uint8, device=x.device) if want_dw else None
        st = lib.gla_layer_headnorm_gate_bwd(_stream(x.device), rows, D, _DT[x.dtype], _ptr(x), _ptr(gate), _ptr(w),
                                             _ptr(rstd), _ptr(dy), _ptr(dx), _ptr(dgate), _ptr(dw), _ptr(ws), ws_n)
        _lib.check(st, "gla_layer_headnorm_gate_bwd")
        return dx, dgate, dw, None


def headnorm_gate(x: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor] = None,
                  eps: float = 1e-5) -> torch.Tensor:
    """``rmsnorm(x over its last axis) * weight * swish(gate)`` in one pass; last axis = head size."""
    return _HeadNormGate.apply(x, gate, weight, eps)


class GLALayer(torch.nn.Module):
    """Gated linear attention layer: projections -> ``chunk_gla`` -> per-head norm, output gate, projection.

    ``forward(x, hidden=None)`` takes ``x (B, T, d_model)`` and an optional state ``(B, H, D, D)``
    and returns ``(y (B, T, d_model), hidden_final (B, H, D, D))``; the state chains across calls
    exactly as the op's ``hidden_init -> hidden_final`` does (gla.py:720-723).
    """

    def __init__(self, d_model: int, num_heads: int, head_dim: Optional[int] = None, gate_low_rank: int = 16,
                 gate_normalizer: float = 16.0, chunk_size: int = 128, eps: float = 1e-5, mode: str = "chunk",
                 device=None, dtype=torch.bfloat16):
        super().__init__()
        if mode not in ("chunk", "recurrent"):
            raise ValueError("mode must be 'chunk' or 'recurrent'")
        head_dim = d_model // num_heads if head_dim is None else head_dim
        self.d_model, self.num_heads, self.head_dim = d_model, num_heads, head_dim
        self.gate_normalizer, self.chunk_size, self.eps, self.mode = gate_normalizer, chunk_size, eps, mode
        inner = num_heads * head_dim
        kw = dict(device=device, dtype=dtype)
        self.q_proj = torch.nn.Linear(d_model, inner, bias=False, **kw)
        self.k_proj = torch.nn.Linear(d_model, inner, bias=False, **kw)
        self.v_proj = torch.nn.Linear(d_model, inner, bias=False, **kw)
        self.gate_down = torch.nn.Linear(d_model, gate_low_rank, bias=False, **kw)
        self.gate_up = torch.nn.Linear(gate_low_rank, inner, bias=True, **kw)
        self.out_gate = torch.nn.Linear(d_model, inner, bias=False, **kw)
        self.o_proj = torch.nn.Linear(inner, d_model, bias=False, **kw)
        self.norm_weight = torch.nn.Parameter(torch.ones(head_dim, device=device, dtype=torch.float32))

    def forward(self, x: torch.Tensor, hidden: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        if x.dim() != 3 or x.shape[-1] != self.d_model:
            raise ValueError(f"x must be (B, T, {self.d_model}), got {tuple(x.shape)}")
        B, T, _ = x.shape
        H, D = self.num_heads, self.head_dim
        q = self.q_proj(x).view(B, T, H, D)
        k = (self.k_proj(x) * (1.0 / math.sqrt(D))).view(B, T, H, D)
        v = self.v_proj(x).view(B, T, H, D)
        g = log_forget_gate(self.gate_up(self.gate_down(x)).view(B, T, H, D), self.gate_normalizer)
        if hidden is None:
            hidden = torch.zeros(B, H, D, D, device=x.device, dtype=x.dtype)
        if self.mode == "chunk":
            hidden_final, out = chunk_gla(hidden, g, v, k, q, chunk_size=self.chunk_size)
        else:
            hidden_final, out = recurrent_gla(hidden, g, v, k, q)
        o = headnorm_gate(out, self.out_gate(x).view(B, T, H, D), self.norm_weight, self.eps)
        return self.o_proj(o.view(B, T, H * D)), hidden_final


__all__ = ["GLALayer", "log_forget_gate", "headnorm_gate"]
