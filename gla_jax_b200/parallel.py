"""Multi-GPU use of the GLA operators (no counterpart in the reference, which is single
device): batch x head sharding and sequence parallelism.

Batch x heads: every (batch, head) pair is an independent recurrence (gla.py:28, 676), so a
rank simply calls the operators on its shard; `shard_batch_heads` picks contiguous shards.

Sequence parallelism: rank r owns a contiguous time slice.  Chaining slices through
hidden_init -> hidden_final is exact (gla.py:720-723) and a slice acts on an incoming state
as S_out = exp(G_r) * S_in + S_r, the binary operator of ops.py:286-297.  The scan over chunks inside a
slice is linear in its initial state, so every rank computes its chunk states ONCE, from a zero state,
and corrects them when the true incoming state is known:

  forward   1. local: chunk states from a ZERO state (kept), total log decay G_r, final state S_r
            2. all-gather (G_r, S_r) over ranks
            3. H_in(r) = exclusive decayed scan over ranks, seeded with hidden_init
            4. finish: state entering chunk n += exp(sum_{m<n} G_m) * H_in(r); chunk kernel -> out
  backward  1. local: gradient states from a ZERO final gradient (kept), A_r = gradient reaching the slice's
               initial state
            2. all-gather A_r
            3. dH_out(r) = reverse exclusive decayed scan, seeded with dhidden_final
            4. finish: gradient state after chunk n += exp(sum_{m>n} G_m) * dH_out(r); backward chunk kernel

Shapes without the two-phase entry points (float32, head sizes other than 128) run the same schedule with
`local` = gla_chunk_local_state / gla_chunk_local_dstate and `finish` = the ordinary forward / backward.
The per-rank message is (H*D + H*D*D) float32 values (516 KB at H=8, D=128): latency-bound.
The orchestration is written against a small `ops` interface so that it runs on the CUDA
library (`CudaOps`, default) and, in CPU tests of the host logic, on any stand-in.

Failures are detected on the host: the ranks compare shapes before the first exchange of a call signature (a rank
that passes a different shape makes every rank raise SequenceParallelError instead of gathering mismatched
buffers), and a collective that does not complete within the process group's timeout (a rank that left) is
reported as SequenceParallelError on the ranks that remain.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib


class SequenceParallelError(RuntimeError):
    """The ranks of a sequence-parallel call disagree (shapes) or a collective did not complete (a rank left)."""


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
    exchange_dtype = torch.float32          # the states that cross ranks stay unrounded

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

    def combine_both(self, all_G, all_S, rank, init, total_dtype, reverse):
        """-> (state entering the slice of `rank`, float32; state leaving the last slice in scan order, `total_dtype`)
        in one launch.  all_G (R,B,H,D) / all_S (R,B,H,D,D) may be views into one packed gather: only the rank axis
        may be strided."""
        R, B, H, D = all_G.shape
        assert all_G[0].is_contiguous() and all_S[0].is_contiguous()
        entering = torch.empty(B, H, D, D, dtype=torch.float32, device=all_G.device)
        total = torch.empty(B, H, D, D, dtype=total_dtype, device=all_G.device)
        init = init.contiguous()
        st = self.lib.gla_sp_combine2(self._stream(all_G.device), R, rank, B * H, D, all_G.data_ptr(), all_G.stride(0),
                                      all_S.data_ptr(), all_S.stride(0), init.data_ptr(), self._DT[init.dtype],
                                      entering.data_ptr(), total.data_ptr(), self._DT[total_dtype], int(reverse))
        _lib.check(st, "gla_sp_combine2")
        return entering, total

    def chunk_fwd(self, h, g, v, k, q, chunk):
        """-> (hidden_final, out, residuals)"""
        from .gla import _chunk_fwd_raw
        return _chunk_fwd_raw(h, g, v, k, q, chunk, self.impl, True)

    def chunk_bwd(self, g, v, k, q, residuals, dhf, dout, chunk):
        """-> (dhidden_init, dg, dv, dk, dq)"""
        from .gla import _chunk_bwd_raw
        return _chunk_bwd_raw(g, v, k, q, residuals, dhf, dout, chunk, self.impl)

    # ---- the four phases of the schedule -----------------------------------------------------------------
    def _two_phase(self, v, chunk) -> bool:
        """Whether the library has the two-phase entry points for this shape (tensor-core path, D = 128)."""
        fam = self.impl & 0xff
        return (v.dtype == torch.bfloat16 and v.shape[-1] == 128 and chunk % 128 == 0 and
                fam in (_lib.IMPL_AUTO, _lib.IMPL_TCGEN05))

    def fwd_local(self, g, v, k, chunk):
        """-> (G (B,H,D) f32, S (B,H,D,D) f32, ctx)"""
        if not self._two_phase(v, chunk):
            G, S = self.local_state(g, v, k, chunk)
            return G, S, None
        B, T, H, D = v.shape
        impl = (self.impl & ~0xff) | _lib.IMPL_TCGEN05
        dt = self._DT[v.dtype]
        saved = torch.empty(self.lib.gla_chunk_saved_bytes(B, T, H, D, chunk, dt, impl), dtype=torch.uint8, device=v.device)
        n = self.lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, chunk, dt, impl)
        ws = torch.empty(n, dtype=torch.uint8, device=v.device)
        G = torch.empty(B, H, D, dtype=torch.float32, device=v.device)
        S = torch.empty(B, H, D, D, dtype=torch.float32, device=v.device)
        st = self.lib.gla_chunk_sp_fwd_local(self._stream(v.device), B, T, H, D, chunk, dt, impl, g.data_ptr(), v.data_ptr(),
                                             k.data_ptr(), G.data_ptr(), S.data_ptr(), saved.data_ptr(), ws.data_ptr(), n)
        _lib.check(st, "gla_chunk_sp_fwd_local")
        return G, S, (saved, ws, impl)

    def fwd_finish(self, ctx, H_in, g, v, k, q, chunk):
        """-> (out, residuals)"""
        if ctx is None:
            _, out, res = self.chunk_fwd(H_in.to(v.dtype), g, v, k, q, chunk)
            return out, res
        saved, ws, impl = ctx
        B, T, H, D = v.shape
        out = torch.empty_like(v)
        H_in = H_in.float().contiguous()
        st = self.lib.gla_chunk_sp_fwd_finish(self._stream(v.device), B, T, H, D, chunk, self._DT[v.dtype], impl, H_in.data_ptr(),
                                              g.data_ptr(), v.data_ptr(), k.data_ptr(), q.data_ptr(), out.data_ptr(),
                                              saved.data_ptr(), ws.data_ptr(), ws.numel())
        _lib.check(st, "gla_chunk_sp_fwd_finish")
        return out, (saved,)

    def bwd_local(self, g, q, dout, residuals, chunk):
        """-> (A (B,H,D,D) f32, ctx)"""
        if not self._two_phase(q, chunk):
            return self.local_dstate(g, q, dout, chunk), None
        (saved,) = residuals
        B, T, H, D = q.shape
        impl = (self.impl & ~0xff) | _lib.IMPL_TCGEN05
        dt = self._DT[q.dtype]
        n = self.lib.gla_chunk_bwd_workspace_bytes(B, T, H, D, chunk, dt, impl)
        ws = torch.empty(n, dtype=torch.uint8, device=q.device)
        A = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device)
        st = self.lib.gla_chunk_sp_bwd_local(self._stream(q.device), B, T, H, D, chunk, dt, impl, g.data_ptr(), q.data_ptr(),
                                             dout.data_ptr(), saved.data_ptr(), A.data_ptr(), ws.data_ptr(), n)
        _lib.check(st, "gla_chunk_sp_bwd_local")
        return A, (ws, impl)

    def bwd_finish(self, ctx, dH_out, g, v, k, q, residuals, dout, chunk):
        """-> (dg, dv, dk, dq)"""
        if ctx is None:
            return self.chunk_bwd(g, v, k, q, residuals, dH_out.to(v.dtype), dout, chunk)[1:]
        ws, impl = ctx
        (saved,) = residuals
        B, T, H, D = v.shape
        dg = torch.empty_like(g)
        dv, dk, dq = torch.empty_like(v), torch.empty_like(k), torch.empty_like(q)
        dH_out = dH_out.float().contiguous()
        st = self.lib.gla_chunk_sp_bwd_finish(self._stream(v.device), B, T, H, D, chunk, self._DT[v.dtype], impl, dH_out.data_ptr(),
                                              g.data_ptr(), v.data_ptr(), k.data_ptr(), q.data_ptr(), saved.data_ptr(),
                                              dout.data_ptr(), dg.data_ptr(), dv.data_ptr(), dk.data_ptr(), dq.data_ptr(),
                                              ws.data_ptr(), ws.numel())
        _lib.check(st, "gla_chunk_sp_bwd_finish")
        return dg, dv, dk, dq


# ---- the schedule, phase by phase (each phase is rank-local; gathers happen between phases) ----

def sp_forward(ops, rank: int, all_G, all_S, hidden_init, ctx, g, v, k, q, chunk):
    """Phases 3-4 of the forward for one rank, given the gathered (G, S) of all ranks and the rank's local context.
    Returns (hidden_final_of_whole_sequence, out_slice, residuals)."""
    R = all_G.shape[0]
    if hasattr(ops, "combine_both"):
        H_in, hidden_final = ops.combine_both(all_G, all_S, rank, hidden_init, hidden_init.dtype, False)
        out, res = ops.fwd_finish(ctx, H_in, g, v, k, q, chunk)
        return hidden_final, out, res
    H_in = ops.combine(all_G, all_S, rank, hidden_init, getattr(ops, "exchange_dtype", torch.float32), False)
    out, res = ops.fwd_finish(ctx, H_in, g, v, k, q, chunk)
    hidden_final = ops.combine(all_G, all_S, R, hidden_init, hidden_init.dtype, False)
    return hidden_final, out, res


def sp_backward(ops, rank: int, all_G, all_A, dhidden_final, ctx, g, v, k, q, residuals, dout, chunk):
    """Phases 3-4 of the backward for one rank.  Returns (dhidden_init of the whole sequence,
    dg, dv, dk, dq of the slice)."""
    if hasattr(ops, "combine_both"):
        dH_out, dhidden_init = ops.combine_both(all_G, all_A, rank, dhidden_final, dhidden_final.dtype, True)
        dg, dv, dk, dq = ops.bwd_finish(ctx, dH_out, g, v, k, q, residuals, dout, chunk)
        return dhidden_init, dg, dv, dk, dq
    dH_out = ops.combine(all_G, all_A, rank, dhidden_final, getattr(ops, "exchange_dtype", torch.float32), True)
    dg, dv, dk, dq = ops.bwd_finish(ctx, dH_out, g, v, k, q, residuals, dout, chunk)
    dhidden_init = ops.combine(all_G, all_A, -1, dhidden_final, dhidden_final.dtype, True)
    return dhidden_init, dg, dv, dk, dq


def _collective(fn, what):
    """Run a collective; a timeout or a peer that has gone surfaces as SequenceParallelError."""
    try:
        return fn()
    except SequenceParallelError:
        raise
    except Exception as e:          # torch.distributed raises RuntimeError / DistBackendError with backend-specific text
        raise SequenceParallelError(f"sequence-parallel {what} did not complete (a rank left or timed out): {e}") from e


def _all_gather(t: torch.Tensor, group) -> torch.Tensor:
    """Gather one tensor per rank into a new leading axis (R, ...)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    t = t.contiguous()
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    _collective(lambda: dist.all_gather_into_tensor(out, t, group=group) if t.is_cuda else dist.all_gather(list(out.unbind(0)), t, group=group),
                "all-gather")
    return out


_validated = set()


def _validate_ranks(hidden_init, v, chunk, group):
    """Every rank must pass the same slice shape, dtype and chunk size.  Compared once per (group, signature):
    one small all-gather on the first call, nothing afterwards.  A mismatch raises on EVERY rank."""
    import torch.distributed as dist
    sig = (tuple(v.shape), tuple(hidden_init.shape), str(v.dtype), int(chunk))
    key = (id(group), sig)
    if key in _validated:
        return
    code = {"torch.float32": 0, "torch.bfloat16": 1, "torch.float64": 2}.get(str(v.dtype), 9)
    mine = torch.tensor(list(v.shape) + list(hidden_init.shape) + [code, int(chunk)], dtype=torch.int64, device=v.device)
    everyone = _all_gather(mine, group).cpu()
    if not bool((everyone == everyone[0]).all()):
        raise SequenceParallelError("the ranks of a sequence-parallel call passed different shapes / dtypes / chunk sizes: "
                                    + "; ".join(f"rank {r}: {everyone[r].tolist()}" for r in range(everyone.shape[0])))
    _validated.add(key)


class _SeqParallelChunkGLA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden_init, g, v, k, q, chunk, group, ops):
        import torch.distributed as dist
        rank = dist.get_rank(group)
        _validate_ranks(hidden_init, v, chunk, group)
        g32 = g.float().contiguous()
        G, S, lctx = ops.fwd_local(g32, v, k, chunk)
        # one all-gather of a packed [G | S] record per rank; all_G / all_S are views into the gathered records
        nG = G.numel()
        packed = _all_gather(torch.cat([G.reshape(-1), S.reshape(-1).to(G.dtype)]), group)
        all_G = packed[:, :nG].unflatten(1, tuple(G.shape))
        all_S = packed[:, nG:].unflatten(1, tuple(S.shape))
        hf, out, res = sp_forward(ops, rank, all_G, all_S, hidden_init, lctx, g32, v, k, q, chunk)
        ctx.save_for_backward(g32, v, k, q, all_G, *res)
        ctx.chunk, ctx.group, ctx.ops, ctx.rank, ctx.g_dtype = chunk, group, ops, rank, g.dtype
        return hf, out

    @staticmethod
    def backward(ctx, dhf, dout):
        g32, v, k, q, all_G, *res = ctx.saved_tensors
        ops = ctx.ops
        dhf = dhf.to(v.dtype).contiguous()
        dout = dout.to(v.dtype).contiguous()
        A, lctx = ops.bwd_local(g32, q, dout, tuple(res), ctx.chunk)
        all_A = _all_gather(A, ctx.group)
        dh, dg, dv, dk, dq = sp_backward(ops, ctx.rank, all_G, all_A, dhf, lctx, g32, v, k, q, tuple(res), dout, ctx.chunk)
        return dh, dg.to(ctx.g_dtype), dv, dk, dq, None, None, None


def sequence_parallel_chunk_gla(hidden_init, log_fgate, value, key, query, chunk_size: int, group=None,
                                ops=None, impl: str = "auto"):
    """chunk_gla over a sequence split evenly across the ranks of `group`.

    Each rank passes ITS time slice of log_fgate/value/key/query, shaped (B, T/R, H, D), and the
    SAME hidden_init (B, H, D, D) (the state before the first token of the whole sequence).
    Returns (hidden_final of the whole sequence - identical on every rank, out of the slice).
    Differentiable; the cotangent of hidden_final must be the same on every rank and the
    returned gradient of hidden_init is that of the whole sequence (identical on every rank).
    Raises SequenceParallelError when the ranks disagree on shapes or a collective does not complete within the
    process group's timeout.
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
    loc = [ops.fwd_local(cut(g32, r), cut(v, r), cut(k, r), chunk) for r in range(R)]
    all_G, all_S = torch.stack([x[0] for x in loc]), torch.stack([x[1] for x in loc])
    fwd = [sp_forward(ops, r, all_G, all_S, hidden_init, loc[r][2], cut(g32, r), cut(v, r), cut(k, r), cut(q, r), chunk)
           for r in range(R)]
    hf = fwd[0][0]
    out = torch.cat([f[1] for f in fwd], dim=1)
    if dout is None:
        return hf, out
    bl = [ops.bwd_local(cut(g32, r), cut(q, r), cut(dout, r), fwd[r][2], chunk) for r in range(R)]
    all_A = torch.stack([x[0] for x in bl])
    bwd = [sp_backward(ops, r, all_G, all_A, dhidden_final, bl[r][1], cut(g32, r), cut(v, r), cut(k, r), cut(q, r), fwd[r][2],
                       cut(dout, r), chunk) for r in range(R)]
    grads = (bwd[0][0],) + tuple(torch.cat([b[i] for b in bwd], dim=1) for i in range(1, 5))
    return hf, out, grads
