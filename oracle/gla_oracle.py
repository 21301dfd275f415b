"""CPU oracle for the gated-linear-attention (GLA) hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this module; it is
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` as the checker and as the timed CPU baseline.

PARITY UNPINNED BY THE REFERENCE: the reference (zhixuan-lin/gla-jax) ships no golden
vectors, fixtures or known-answer tests, and it cannot be imported where this file runs
(it needs jax==0.4.29 with Pallas/Triton, none of which is installed).  The oracle is
therefore pinned only by internal consistency, which ``tests/test_oracle.py`` asserts:
three independent restatements (the step recurrence, the chunk algorithm with dyadic
secondary chunking, and the hand-derived backward formulas) agree with each other and with
torch autograd to ~1e-12 in float64.

Every function cites the reference lines it restates (paths are relative to the reference
project root).  All functions are per sequence, exactly like the reference API:

    log_fgate, value, key, query : (T, H, D)      hidden : (H, D_key, D_value)

and return ``(hidden_final, out)``.  A leading batch axis is handled by ``batched``.
Everything is written with torch CPU tensors so float64, float32 and bfloat16 rounding and
autograd are all available; there is no device code here.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Optional, Tuple

import numpy as np
import torch

# --------------------------------------------------------------------------------------
# Deterministic synthetic inputs (the reference uses no dataset; its harness draws every
# tensor from N(0,1) and the gate from log_sigmoid(5 + N(0,1)), gla.py:1386-1392).  Unlike
# the harness, which reuses one PRNG key for every tensor, each tensor here has its own
# stream so that a q/k/v mix-up is caught.
# --------------------------------------------------------------------------------------

CONFIGS: Dict[str, dict] = {
    # name: B, T, H, D, chunk, dtype, gate shift, q/k/v scale, zero hidden_init
    "cfg1_cpu": dict(B=1, T=256, H=2, D=64, C=64, dtype="float32", shift=5.0, scale=1.0, zero_init=False),
    "cfg2_readme": dict(B=4, T=4096, H=6, D=128, C=128, dtype="bfloat16", shift=5.0, scale=1.0, zero_init=False),
    "cfg3_train": dict(B=32, T=8192, H=16, D=128, C=128, dtype="bfloat16", shift=5.0,
                       scale=1.0 / math.sqrt(128.0), zero_init=True),
    "cfg4_longctx": dict(B=1, T=131072, H=8, D=128, C=128, dtype="bfloat16", shift=5.0, scale=1.0, zero_init=False),
    "cfg5_sharp": dict(B=16, T=16384, H=8, D=256, C=256, dtype="bfloat16", shift=0.0, scale=1.0, zero_init=False),
}


def make_inputs(B: int, T: int, H: int, D: int, dtype=torch.float32, seed: int = 0,
                shift: float = 5.0, scale: float = 1.0, zero_init: bool = False,
                batch_axis: bool = True):
    """Seeded inputs ``(hidden_init, log_fgate, value, key, query)``.

    One generator per tensor (seed, seed+1, ...).  ``log_fgate`` is always float32
    (gla.py:1391).  With ``batch_axis=False`` (requires B == 1) the leading axis is dropped
    so the arrays have the reference's per-sequence shapes.
    """
    def normal(shape, s):
        g = torch.Generator(device="cpu").manual_seed(seed + s)
        return torch.randn(shape, generator=g, dtype=torch.float32)

    hidden = torch.zeros(B, H, D, D) if zero_init else normal((B, H, D, D), 0)
    value = normal((B, T, H, D), 1) * scale
    key = normal((B, T, H, D), 2) * scale
    query = normal((B, T, H, D), 3) * scale
    log_fgate = torch.nn.functional.logsigmoid(shift + normal((B, T, H, D), 4))
    out = [hidden.to(dtype), log_fgate.float(), value.to(dtype), key.to(dtype), query.to(dtype)]
    if not batch_axis:
        assert B == 1
        out = [x[0] for x in out]
    return tuple(out)


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """Relative L2 error ``|a-b| / |a|`` with ``a`` the trusted value (gla.py:1462)."""
    a = a.detach().double()
    b = b.detach().double()
    den = float(torch.linalg.norm(a))
    num = float(torch.linalg.norm(a - b))
    return num / den if den > 0 else num


# --------------------------------------------------------------------------------------
# 1. The definitional recurrence (gla.py:26-47).  This is the specification.
# --------------------------------------------------------------------------------------

def recurrent_gla_naive(hidden, log_fgate, value, key, query, reverse: bool = False,
                        compute_dtype=torch.float64):
    """Step recurrence ``S_t = exp(g_t)[:,None] * S_{t-1} + outer(k_t, v_t)``,
    ``o_t = sum_k q_t[k] S_t[k,:]`` (gla.py:35-37: the output is read AFTER the update, so
    token t sees itself undecayed).  State is carried in ``compute_dtype`` (float32 in the
    reference, gla.py:44); ``hidden_final`` is cast back to ``hidden.dtype`` (gla.py:46) and
    ``out`` stays in the compute dtype (the reference's is float32 by promotion).
    Differentiable by torch autograd.
    """
    T, H, D = key.shape
    S = hidden.to(compute_dtype)
    f = torch.exp(log_fgate.to(compute_dtype))
    v = value.to(compute_dtype)
    k = key.to(compute_dtype)
    q = query.to(compute_dtype)
    outs = [None] * T
    order = range(T - 1, -1, -1) if reverse else range(T)
    for t in order:
        S = f[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        outs[t] = torch.einsum("hk,hkv->hv", q[t], S)
    out = torch.stack(outs, dim=0)
    return S.to(hidden.dtype), out


def recurrent_gla_backward_formulas(hidden, log_fgate, value, key, query, dhidden_final, dout,
                                    compute_dtype=torch.float64):
    """Hand-derived gradients of the recurrence, restating the reference's custom VJP
    (gla.py:172-269 and the kernel gla.py:271-360): a forward recompute pass for
    ``dq_t = S_t dout_t`` (gla.py:306), a reverse pass ``dS = dcarry + outer(q_t, dout_t)``;
    ``dv_t = k_t dS``; ``dk_t = dS v_t``; ``dcarry = f_t * dS`` (gla.py:336-339), and
    ``dg = reverse_cumsum_T(q*dq - k*dk) + sum_v(dS_T * S_T)`` (gla.py:263).
    Returns ``(dhidden_init, dlog_fgate, dvalue, dkey, dquery)`` in ``compute_dtype``.
    """
    T, H, D = key.shape
    cd = compute_dtype
    f = torch.exp(log_fgate.to(cd))
    v, k, q = value.to(cd), key.to(cd), query.to(cd)
    do = dout.to(cd)
    S = hidden.to(cd)
    dq = torch.zeros(T, H, D, dtype=cd)
    for t in range(T):
        S = f[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        dq[t] = torch.einsum("hkv,hv->hk", S, do[t])
    S_final = S
    dc = dhidden_final.to(cd)
    dv = torch.zeros(T, H, D, dtype=cd)
    dk = torch.zeros(T, H, D, dtype=cd)
    for t in range(T - 1, -1, -1):
        dS = dc + q[t][:, :, None] * do[t][:, None, :]
        dv[t] = torch.einsum("hk,hkv->hv", k[t], dS)
        dk[t] = torch.einsum("hkv,hv->hk", dS, v[t])
        dc = f[t][:, :, None] * dS
    e = dq * q - dk * k
    dg = torch.flip(torch.cumsum(torch.flip(e, [0]), 0), [0]) + (dhidden_final.to(cd) * S_final).sum(-1)[None]
    return dc, dg, dv, dk, dq


# --------------------------------------------------------------------------------------
# 2. Scan ops of ops.py
# --------------------------------------------------------------------------------------

def cumsum(src, axis: int, init=None, reverse: bool = False, out_dtype=None, compute_dtype=torch.float32):
    """Inclusive cumulative sum along ``axis`` with ``init`` added to every element
    (ops.py:152-162 with ops.py:91-103: ``out = add(init, scan)``), optionally from the end.
    Math in ``compute_dtype`` (float32 in the reference, ops.py:159-160); result in
    ``out_dtype`` or the source dtype (ops.py:190-191).
    """
    x = src.to(compute_dtype)
    if reverse:
        x = torch.flip(torch.cumsum(torch.flip(x, [axis]), axis), [axis])
    else:
        x = torch.cumsum(x, axis)
    if init is not None:
        x = x + init.to(compute_dtype).unsqueeze(axis)
    return x.to(out_dtype or src.dtype)


def rnn_scan(log_fgate, kv, init_log_fgate=None, init_kv=None, reverse: bool = False,
             compute_dtype=torch.float32):
    """Log-space linear-RNN inclusive scan over the leading axis (ops.py:286-334, 396-456):
    combine ``(A_i, b_i) o (A_j, b_j) = (A_i + A_j, exp(A_j) b_i + b_j)``; the optional
    ``init`` pair is combined in front of every element (ops.py:103).  Returns
    ``(cumulative log decay (T,K), state (T,K,V))`` with the decay in log_fgate's dtype and
    the state in kv's dtype (ops.py:372-375).  ``reverse`` scans from the end.
    """
    T, K, V = kv.shape
    A = torch.zeros(K, dtype=compute_dtype) if init_log_fgate is None else init_log_fgate.to(compute_dtype)
    b = torch.zeros(K, V, dtype=compute_dtype) if init_kv is None else init_kv.to(compute_dtype)
    g = log_fgate.to(compute_dtype)
    x = kv.to(compute_dtype)
    out_A = torch.empty(T, K, dtype=compute_dtype)
    out_b = torch.empty(T, K, V, dtype=compute_dtype)
    order = range(T - 1, -1, -1) if reverse else range(T)
    for t in order:
        b = torch.exp(g[t])[:, None] * b + x[t]
        A = A + g[t]
        out_A[t] = A
        out_b[t] = b
    return out_A.to(log_fgate.dtype), out_b.to(kv.dtype)


# --------------------------------------------------------------------------------------
# 3. The chunk-wise algorithm with dyadic ("multi-scale") secondary chunking
# --------------------------------------------------------------------------------------

def _levels(C: int):
    """Half sizes of the dyadic levels C/2, C/4, ..., 1 (gla.py:843-852 above
    ``block_size_t``, gla.py:985-1027 below it; the structure is the same all the way down)."""
    h = C // 2
    out = []
    while h >= 1:
        out.append(h)
        h //= 2
    return out


def compute_score(lam, key, query, rnd: Callable = lambda x: x):
    """Gated causal score of one chunk (gla.py:964-1029): for every dyadic block [s, e) with
    midpoint m and anchor row a = m-1, the cross block is
    ``(q[m:e] * exp(lam[m:e]-lam[a])) @ (k[s:m] * exp(lam[a]-lam[s:m])).T`` so that every
    exponent is <= 0; the diagonal is ``sum(q*k)`` (gla.py:983) and the upper triangle is 0
    (gla.py:981).  ``lam, key, query`` are (..., C, D); returns (..., C, C).  ``rnd`` is
    applied to each weighted operand (the reference rounds them to the input dtype,
    gla.py:991-992).
    """
    C, D = lam.shape[-2:]
    P = torch.zeros(*lam.shape[:-2], C, C, dtype=lam.dtype)
    idx = torch.arange(C)
    P[..., idx, idx] = (query * key).sum(-1)
    for h in _levels(C):
        for s in range(0, C, 2 * h):
            m, e = s + h, s + 2 * h
            anchor = lam[..., m - 1:m, :]
            qw = rnd(query[..., m:e, :] * torch.exp(lam[..., m:e, :] - anchor))
            kw = rnd(key[..., s:m, :] * torch.exp(anchor - lam[..., s:m, :]))
            P[..., m:e, s:m] = qw @ kw.transpose(-1, -2)
    return P


def chunk_gla(hidden_init, log_fgate, value, key, query, chunk_size: int,
              compute_dtype=torch.float64, rnd: Optional[Callable] = None,
              return_aux: bool = False):
    """Chunk-wise GLA (gla.py:483-550, 657-692, 695-729, 792-855).

    Per head, with chunks of length C: ``lam`` = within-chunk inclusive cumsum of the gate
    (gla.py:509), ``G = lam[:, -1]`` (gla.py:512);
    intra-chunk  ``out = P @ v`` with ``P = compute_score`` (gla.py:828-852);
    inter-chunk  ``kv = (k*exp(G-lam)).T @ v`` (gla.py:705-708), states
    ``S_n = exp(G_n) S_{n-1} + kv_n`` from ``hidden_init`` (gla.py:711-723),
    ``out += (q*exp(lam)) @ S_{n-1}`` (gla.py:724-725), ``hidden_final = S_{N-1}``.

    ``rnd`` (optional) is applied at the reference's rounding points (weighted operands,
    scores, kv, stored states, per-part outputs) to emulate its bf16 behaviour; with
    ``rnd=None`` the computation is exact in ``compute_dtype``.  Differentiable by autograd.
    """
    T, H, D = key.shape
    C = chunk_size
    assert T % C == 0 and (C & (C - 1)) == 0
    N = T // C
    cd = compute_dtype
    r = rnd if rnd is not None else (lambda x: x)

    def to_chunks(x):  # (T,H,D) -> (H,N,C,D)   gla.py:673-675
        return x.to(cd).reshape(N, C, H, D).permute(2, 0, 1, 3)

    g, v, k, q = (to_chunks(x) for x in (log_fgate, value, key, query))
    lam = torch.cumsum(g, dim=-2)
    G = lam[:, :, -1, :]                                   # (H,N,D)
    P = r(compute_score(lam, k, q, r))                     # (H,N,C,C)
    intra = r(P @ v)
    k_hat = r(k * torch.exp(G[:, :, None, :] - lam))
    kv = r(k_hat.transpose(-1, -2) @ v)                    # (H,N,Dk,Dv)
    S = hidden_init.to(cd)
    states = []
    for n in range(N):
        states.append(S)
        S = torch.exp(G[:, n])[:, :, None] * S + kv[:, n]
        if n < N - 1:
            S = r(S)
    S_prev = torch.stack(states, dim=1)                    # (H,N,Dk,Dv): state entering chunk n
    q_hat = r(q * torch.exp(lam))
    inter = r(q_hat @ S_prev)
    out = r(intra + inter)
    out = out.permute(1, 2, 0, 3).reshape(T, H, D)          # gla.py:691
    hidden_final = S.to(hidden_init.dtype)
    if return_aux:
        return hidden_final, out, dict(lam=lam, G=G, P=P, S_prev=S_prev, kv=kv)
    return hidden_final, out


def chunk_gla_backward_formulas(hidden_init, log_fgate, value, key, query, chunk_size: int,
                                dhidden_final, dout, compute_dtype=torch.float64):
    """Hand-derived backward of ``chunk_gla`` restating gla.py:552-625, 731-790, 857-960 and
    the score backward gla.py:1036-1189, in the form the CUDA kernels use:

      dP      = dO V^T (lower triangle incl. diagonal)             gla.py:881,927
      dV      = P^T dO + k_hat dS_next                             gla.py:880,926,775
      dq      = sum_levels (dP_l k~_l) * wq_l + diag + (dO S_prev^T) * exp(lam)
                                                                   gla.py:892-893,1074-1076,1184,752-753
      dk      = sum_levels (dP_l^T q~_l) * wk_l + diag + (V dS_next^T) * exp(G-lam)
                                                                   gla.py:899-900,1082-1084,1183,776-778
      dstate  = q_hat^T dO ; y_n = dstate_n + exp(G_n) y_{n+1}, y_N = dhidden_final;
      dS_next(n) = y_{n+1} ; dhidden_init = y_0                    gla.py:750,759-771
      dlam    = q*dq - k*dk   (equal to the sum of the reference's per-level
                dq~*q~ - dk~*k~ terms, gla.py:894,901,1078,1086,754,780)
      dG      = sum_c(dk_hat*k_hat) + sum_v(S_prev*exp(G)*dS_next) gla.py:782
      dg      = reverse cumsum of dlam within the chunk + dG       gla.py:615-617

    Returns ``(dhidden_init, dlog_fgate, dvalue, dkey, dquery)`` in ``compute_dtype``.
    """
    T, H, D = key.shape
    C = chunk_size
    N = T // C
    cd = compute_dtype

    def to_chunks(x):
        return x.to(cd).reshape(N, C, H, D).permute(2, 0, 1, 3)

    def from_chunks(x):
        return x.permute(1, 2, 0, 3).reshape(T, H, D)

    g, v, k, q, do = (to_chunks(x) for x in (log_fgate, value, key, query, dout))
    with torch.no_grad():
        _, _, aux = chunk_gla(hidden_init, log_fgate, value, key, query, C, cd, None, True)
    lam, G, P, S_prev = aux["lam"], aux["G"], aux["P"], aux["S_prev"]
    mask = torch.tril(torch.ones(C, C, dtype=cd))
    dP = (do @ v.transpose(-1, -2)) * mask
    q_hat = q * torch.exp(lam)
    k_hat = k * torch.exp(G[:, :, None, :] - lam)
    # inter-chunk: gradient flowing into the chunk states (reverse scan over chunks)
    dstate = q_hat.transpose(-1, -2) @ do                  # (H,N,Dk,Dv)
    y = dhidden_final.to(cd)
    dS_next = [None] * N
    for n in range(N - 1, -1, -1):
        dS_next[n] = y
        y = dstate[:, n] + torch.exp(G[:, n])[:, :, None] * y
    dhidden_init = y
    dS_next = torch.stack(dS_next, dim=1)
    dv = P.transpose(-1, -2) @ do + k_hat @ dS_next
    dq = (do @ S_prev.transpose(-1, -2)) * torch.exp(lam)
    dk_hat = v @ dS_next.transpose(-1, -2)
    dk = dk_hat * torch.exp(G[:, :, None, :] - lam)
    # intra-chunk, level by level with the same anchors as the forward
    idx = torch.arange(C)
    ddiag = dP[..., idx, idx][..., None]
    dq = dq + ddiag * k
    dk = dk + ddiag * q
    for h in _levels(C):
        for s in range(0, C, 2 * h):
            m, e = s + h, s + 2 * h
            anchor = lam[..., m - 1:m, :]
            wq = torch.exp(lam[..., m:e, :] - anchor)
            wk = torch.exp(anchor - lam[..., s:m, :])
            blk = dP[..., m:e, s:m]
            dq[..., m:e, :] += (blk @ (k[..., s:m, :] * wk)) * wq
            dk[..., s:m, :] += (blk.transpose(-1, -2) @ (q[..., m:e, :] * wq)) * wk
    dlam = q * dq - k * dk
    dG = (dk_hat * k_hat).sum(-2) + (S_prev * torch.exp(G)[..., None] * dS_next).sum(-1)
    dg = torch.flip(torch.cumsum(torch.flip(dlam, [-2]), -2), [-2]) + dG[:, :, None, :]
    return dhidden_init, from_chunks(dg), from_chunks(dv), from_chunks(dk), from_chunks(dq)


# --------------------------------------------------------------------------------------
# 4. Helpers shared by tests and the CPU baseline
# --------------------------------------------------------------------------------------

def bf16_round(x: torch.Tensor) -> torch.Tensor:
    """Round to bfloat16 and back (emulates the reference's ``astype(input dtype)`` cast
    points listed in the module docstring of tests/test_oracle.py)."""
    return x.to(torch.bfloat16).to(x.dtype)


def batched(fn: Callable, *arrays, **kw):
    """Apply a per-sequence function over a leading batch axis (the reference's
    ``jax.vmap``, gla.py:1335) and stack the results."""
    outs = [fn(*[a[b] for a in arrays], **kw) for b in range(arrays[0].shape[0])]
    return tuple(torch.stack([o[i] for o in outs], 0) for i in range(len(outs[0])))


def value_and_grads(fn: Callable, hidden, log_fgate, value, key, query, dhidden_final=None, dout=None,
                    compute_dtype=torch.float64, **kw):
    """Forward plus autograd gradients w.r.t. all five inputs, for cotangents
    ``(dhidden_final, dout)``; with both ``None`` this is the harness loss
    ``hidden_final.sum() + out.sum()`` (gla.py:1336-1340).  Inputs are promoted to
    ``compute_dtype`` leaves first so the gradients are exact to that precision.
    Returns ``(hidden_final, out, (dhidden, dg, dv, dk, dq))``.
    """
    leaves = [x.detach().to(compute_dtype).requires_grad_(True) for x in (hidden, log_fgate, value, key, query)]
    hf, out = fn(*leaves, compute_dtype=compute_dtype, **kw)
    dhf = torch.ones_like(hf) if dhidden_final is None else dhidden_final.to(hf.dtype)
    do = torch.ones_like(out) if dout is None else dout.to(out.dtype)
    loss = (hf * dhf).sum() + (out * do).sum()
    grads = torch.autograd.grad(loss, leaves)
    return hf.detach(), out.detach(), tuple(g.detach() for g in grads)


def chunk_gla_cpu_fwd_bwd(hidden, log_fgate, value, key, query, chunk_size: int,
                          compute_dtype=torch.float32):
    """The timed CPU baseline: the chunk path written with plain batched tensor ops
    (the reference's jnp chunk path with its Pallas kernels replaced by plain cumsum /
    matmul, as its own ``interpret`` mode would do), forward plus autograd backward of the
    harness loss, for a batch of sequences.  Returns the five gradients.
    """
    B = key.shape[0]
    grads = []
    for b in range(B):
        _, _, g = value_and_grads(chunk_gla, hidden[b], log_fgate[b], value[b], key[b], query[b],
                                  compute_dtype=compute_dtype, chunk_size=chunk_size)
        grads.append(g)
    return grads


def to_numpy(x: torch.Tensor) -> np.ndarray:
    """Tensor -> numpy, widening bfloat16 (numpy has no native bf16)."""
    return (x.float() if x.dtype == torch.bfloat16 else x).detach().cpu().numpy()
