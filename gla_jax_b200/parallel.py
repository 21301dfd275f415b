"""Multi-GPU use of the GLA operators (no counterpart in the reference, which is single
device): batch x head sharding and sequence parallelism.

Batch x heads: every (batch, head) pair is an independent recurrence (gla.py:28, 676), so a
rank simply calls the operators on its shard; `shard_batch_heads` picks contiguous shards.

Sequence parallelism: rank r owns a contiguous time slice.  Chaining slices through
hidden_init -> hidden_final is exact (gla.py:720-723) and a slice acts on an incoming state
as S_out = exp(G_r) * S_in + S_r, the binary operator of ops.py:286-297, so

  forward   1. (G_r, S_r) = total log decay and final state of the slice from a ZERO state
            2. all-gather over ranks
            3. H_in(r) = exclusive decayed scan over ranks, seeded with hidden_init
            4. ordinary chunk_gla on the slice with hidden_init = H_in(r)
  backward  1. A_r = gradient reaching the slice's initial state for a zero final-state gradient
            2. all-gather (G_r, A_r)
            3. dH_out(r) = reverse exclusive decayed scan, seeded with dhidden_final
            4. ordinary chunk_gla backward on the slice with dhidden_final = dH_out(r)

The per-rank message is (H*D + H*D*D) float32 values (516 KB at H=8, D=128): latency-bound.
The orchestration is written against a small `ops` interface so that it runs on the CUDA
library (`CudaOps`, default) and, in CPU tests of the host logic, on any stand-in.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib


def shard_batch_heads(B: int, H: int, world: int, rank: int) -> Tuple[slice, slice]:
    """Contiguous (batch, head) shard of rank `rank`: split the batch when it divides, else the
    heads; returns (batch_slice, head_slice)."""
    if B % world == 0:
        n = B // world
        return slice(rank * n, (rank + 1) * n), slice(0, H)
    if H % world == 0:
        n = H // world
        return slice(0, B), slice(rank * n, (rank + 1) * n)
    if (B * H) % world == 0 and world % B == 0:
        per_b = world // B
        n = H // per_b
        b = rank // per_b
        j = rank % per_b
        return slice(b, b + 1), slice(j * n, (j + 1) * n)
    raise ValueError(f"cannot shard B={B}, H={H} evenly over {world} ranks")


class CudaOps:
    """The five primitives of the sequence-parallel schedule on libgla_b200.so (tensors are
    batched: (B,T,H,D) / (B,H,D,D); log_fgate float32)."""

    _DT = {torch.float32: _lib.GLA_F32, torch.bfloat16: _lib.GLA_BF16}

    def __init__(self, impl: str = "auto"):
        self.lib = _lib.load()
        self.impl = _lib.IMPL_BY_NAME[impl]

    _stream = staticmethod(_lib.stream_of)

    def local_state(self, g, v, k, chunk):
        B, T, H, D = v.shape
        dt = self._DT[v.dtype]
        n = max(self.lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, chunk, dt, self.impl),
                self.lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, chunk, dt, _lib.IMPL_FP32_SIMT))
        ws = torch.empty(n, dtype=torch.uint8, device=v.device)
        G = torch.empty(B, H, D, dtype=torch.float32, device=v.device)
        S = torch.empty(B, H, D, D, dtype=torch.float32, device=v.device)
        st = self.lib.gla_chunk_local_state(self._stream(v.device), B, T, H, D, chunk, dt, self.impl, g.data_ptr(),
                                            v.data_ptr(), k.data_ptr(), G.data_ptr(), S.data_ptr(), ws.data_ptr(), n)
        _lib.check(st, "gla_chunk_local_state")
        return G, S

    def local_dstate(self, g, q, dout, chunk):
        B, T, H, D = q.shape
        dt = self._DT[q.dtype]
        n = max(self.lib.gla_chunk_bwd_workspace_bytes(B, T, H, D, chunk, dt, self.impl),
                self.lib.gla_chunk_bwd_workspace_bytes(B, T, H, D, chunk, dt, _lib.IMPL_FP32_SIMT))
        ws = torch.empty(n, dtype=torch.uint8, device=q.device)
        A = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device)
        st = self.lib.gla_chunk_local_dstate(self._stream(q.device), B, T, H, D, chunk, dt, self.impl, g.data_ptr(),
                                             q.data_ptr(), dout.data_ptr(), A.data_ptr(), ws.data_ptr(), n)
        _lib.check(st, "gla_chunk_local_dstate")
        return A

    def combine(self, all_G, all_S, rank, init, out_dtype, reverse):
        R, B, H, D = all_G.shape
        res = torch.empty(B, H, D, D, dtype=out_dtype, device=all_G.device)
        init = init.contiguous()
        st = self.lib.gla_sp_combine(self._stream(all_G.device), R, rank, B * H, D, all_G.data_ptr(), all_S.data_ptr(),
                                     init.data_ptr(), self._DT[init.dtype], res.data_ptr(), self._DT[out_dtype],
                                     int(reverse))
        _lib.check(st, "gla_sp_combine")
        return res

    def chunk_fwd(self, h, g, v, k, q, chunk):
        """-> (hidden_final, out, residuals)"""
        from .gla import _chunk_fwd_raw
        return _chunk_fwd_raw(h, g, v, k, q, chunk, self.impl, True)

    def chunk_bwd(self, g, v, k, q, residuals, dhf, dout, chunk):
        """-> (dhidden_init, dg, dv, dk, dq)"""
        from .gla import _chunk_bwd_raw
        return _chunk_bwd_raw(g, v, k, q, residuals, dhf, dout, chunk, self.impl)


# ---- the schedule, phase by phase (each phase is rank-local; gathers happen between phases) ----

def sp_forward(ops, rank: int, all_G, all_S, hidden_init, g, v, k, q, chunk):
    """Phases 3-4 of the forward for one rank, given the gathered (G, S) of all ranks.
    Returns (hidden_final_of_whole_sequence, out_slice, residuals)."""
    R = all_G.shape[0]
    H_in = ops.combine(all_G, all_S, rank, hidden_init, hidden_init.dtype, False)
    _, out, res = ops.chunk_fwd(H_in, g, v, k, q, chunk)
    hidden_final = ops.combine(all_G, all_S, R, hidden_init, hidden_init.dtype, False)
    return hidden_final, out, res


def sp_backward(ops, rank: int, all_G, all_A, dhidden_final, g, v, k, q, residuals, dout, chunk):
    """Phases 3-4 of the backward for one rank.  Returns (dhidden_init of the whole sequence,
    dg, dv, dk, dq of the slice)."""
    dH_out = ops.combine(all_G, all_A, rank, dhidden_final, dhidden_final.dtype, True)
    _, dg, dv, dk, dq = ops.chunk_bwd(g, v, k, q, residuals, dH_out, dout, chunk)
    dhidden_init = ops.combine(all_G, all_A, -1, dhidden_final, dhidden_final.dtype, True)
    return dhidden_init, dg, dv, dk, dq


def _all_gather(t: torch.Tensor, group) -> torch.Tensor:
    """Gather one tensor per rank into a new leading axis (R, ...)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    t = t.contiguous()
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather(list(out.unbind(0)), t, group=group)
    return out


class _SeqParallelChunkGLA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden_init, g, v, k, q, chunk, group, ops):
        import torch.distributed as dist
        rank = dist.get_rank(group)
        g32 = g.float().contiguous()
        G, S = ops.local_state(g32, v, k, chunk)
        all_G, all_S = _all_gather(G, group), _all_gather(S, group)
        hf, out, res = sp_forward(ops, rank, all_G, all_S, hidden_init, g32, v, k, q, chunk)
        ctx.save_for_backward(g32, v, k, q, all_G, *res)
        ctx.chunk, ctx.group, ctx.ops, ctx.rank, ctx.g_dtype = chunk, group, ops, rank, g.dtype
        return hf, out

    @staticmethod
    def backward(ctx, dhf, dout):
        g32, v, k, q, all_G, *res = ctx.saved_tensors
        ops = ctx.ops
        dhf = dhf.to(v.dtype).contiguous()
        dout = dout.to(v.dtype).contiguous()
        A = ops.local_dstate(g32, q, dout, ctx.chunk)
        all_A = _all_gather(A, ctx.group)
        dh, dg, dv, dk, dq = sp_backward(ops, ctx.rank, all_G, all_A, dhf, g32, v, k, q, tuple(res), dout, ctx.chunk)
        return dh, dg.to(ctx.g_dtype), dv, dk, dq, None, None, None


def sequence_parallel_chunk_gla(hidden_init, log_fgate, value, key, query, chunk_size: int, group=None,
                                ops=None, impl: str = "auto"):
    """chunk_gla over a sequence split evenly across the ranks of `group`.

    Each rank passes ITS time slice of log_fgate/value/key/query, shaped (B, T/R, H, D), and the
    SAME hidden_init (B, H, D, D) (the state before the first token of the whole sequence).
    Returns (hidden_final of the whole sequence - identical on every rank, out of the slice).
    Differentiable; the cotangent of hidden_final must be the same on every rank and the
    returned gradient of hidden_init is that of the whole sequence (identical on every rank).
    """
    ops = ops or CudaOps(impl)
    return _SeqParallelChunkGLA.apply(hidden_init.contiguous(), log_fgate.contiguous(), value.contiguous(),
                                      key.contiguous(), query.contiguous(), int(chunk_size), group, ops)


def emulate_sequence_parallel(ops, R: int, hidden_init, g, v, k, q, chunk, dhidden_final=None, dout=None):
    """The same schedule with all R ranks run one after another in ONE process (the gathers
    become torch.stack): for single-GPU tests.  Takes the whole sequence, returns
    (hidden_final, out[, (dhidden_init, dg, dv, dk, dq)])."""
    T = v.shape[1]
    assert T % R == 0
    L = T // R
    sl = [slice(r * L, (r + 1) * L) for r in range(R)]
    cut = lambda x, r: x[:, sl[r]].contiguous()
    g32 = g.float()
    GS = [ops.local_state(cut(g32, r), cut(v, r), cut(k, r), chunk) for r in range(R)]
    all_G, all_S = torch.stack([x[0] for x in GS]), torch.stack([x[1] for x in GS])
    fwd = [sp_forward(ops, r, all_G, all_S, hidden_init, cut(g32, r), cut(v, r), cut(k, r), cut(q, r), chunk)
           for r in range(R)]
    hf = fwd[0][0]
    out = torch.cat([f[1] for f in fwd], dim=1)
    if dout is None:
        return hf, out
    As = [ops.local_dstate(cut(g32, r), cut(q, r), cut(dout, r), chunk) for r in range(R)]
    all_A = torch.stack(As)
    bwd = [sp_backward(ops, r, all_G, all_A, dhidden_final, cut(g32, r), cut(v, r), cut(k, r), cut(q, r), fwd[r][2],
                       cut(dout, r), chunk) for r in range(R)]
    grads = (bwd[0][0],) + tuple(torch.cat([b[i] for b in bwd], dim=1) for i in range(1, 5))
    return hf, out, grads
