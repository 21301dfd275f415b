"""CPU tests of the multi-GPU host logic (gloo, world size 2): the sequence-parallel schedule
of gla_jax_b200/parallel.py driven with an oracle-backed stand-in for the CUDA primitives, so
that the rank logic, the all-gathers and the combine algebra are covered without a GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gla_jax_b200 import parallel as P
from oracle import gla_oracle as O

CD = torch.float64


class OracleOps:
    """The five primitives of parallel.CudaOps restated with the CPU oracle (float64)."""
    exchange_dtype = CD

    def local_state(self, g, v, k, chunk):
        B, T, H, D = v.shape
        z = torch.zeros(B, H, D, D, dtype=CD)
        S = torch.stack([O.chunk_gla(z[b], g[b], v[b], k[b], torch.zeros_like(k[b]), chunk, CD)[0] for b in range(B)])
        return g.to(CD).sum(1), S

    def local_dstate(self, g, q, dout, chunk):
        B, T, H, D = q.shape
        outs = []
        for b in range(B):     # gradient w.r.t. the initial state of out = q_hat S (v = k = 0), zero dhidden_final
            with torch.enable_grad():
                h0 = torch.zeros(H, D, D, dtype=CD, requires_grad=True)
                _, out = O.recurrent_gla_naive(h0, g[b].to(CD), torch.zeros_like(q[b], dtype=CD),
                                               torch.zeros_like(q[b], dtype=CD), q[b].to(CD))
                outs.append(torch.autograd.grad((out * dout[b].to(CD)).sum(), h0)[0])
        return torch.stack(outs)

    def combine(self, all_G, all_S, rank, init, out_dtype, reverse):
        R = all_G.shape[0]
        acc = init.to(CD)
        order = range(rank) if not reverse else range(R - 1, rank, -1)
        for s in order:
            acc = torch.exp(all_G[s])[..., None] * acc + all_S[s]
        return acc.to(out_dtype)

    def chunk_fwd(self, h, g, v, k, q, chunk):
        B = v.shape[0]
        r = [O.chunk_gla(h[b], g[b], v[b], k[b], q[b], chunk, CD) for b in range(B)]
        return torch.stack([x[0] for x in r]), torch.stack([x[1] for x in r]), (h,)

    def chunk_bwd(self, g, v, k, q, residuals, dhf, dout, chunk):
        (h,) = residuals
        B = v.shape[0]
        r = [O.chunk_gla_backward_formulas(h[b], g[b], v[b], k[b], q[b], chunk, dhf[b], dout[b], CD) for b in range(B)]
        return tuple(torch.stack([x[i] for x in r]) for i in range(5))

    # the four phases of the schedule: `local` from a zero state, `finish` with the true one
    def fwd_local(self, g, v, k, chunk):
        G, S = self.local_state(g, v, k, chunk)
        return G, S, None

    def fwd_finish(self, ctx, H_in, g, v, k, q, chunk):
        _, out, res = self.chunk_fwd(H_in.to(CD), g, v, k, q, chunk)
        return out, res

    def bwd_local(self, g, q, dout, residuals, chunk):
        return self.local_dstate(g, q, dout, chunk), None

    def bwd_finish(self, ctx, dH_out, g, v, k, q, residuals, dout, chunk):
        return self.chunk_bwd(g, v, k, q, residuals, dH_out.to(CD), dout, chunk)[1:]


def _inputs(B=1, T=128, H=2, D=16):
    h, g, v, k, q = O.make_inputs(B, T, H, D, CD, seed=3, shift=1.0)
    gen = torch.Generator().manual_seed(9)
    return h, g.to(CD), v, k, q, torch.randn(B, H, D, D, generator=gen, dtype=CD), torch.randn(B, T, H, D, generator=gen, dtype=CD)


def _reference(h, g, v, k, q, dhf, do):
    hf, out, grads = O.value_and_grads(O.recurrent_gla_naive, h[0], g[0], v[0], k[0], q[0], dhf[0], do[0])
    return hf, out, grads


def test_emulated_schedule_matches_single_sequence():
    h, g, v, k, q, dhf, do = _inputs()
    hf0, out0, gr0 = _reference(h, g, v, k, q, dhf, do)
    for R in (2, 4):
        hf, out, grads = P.emulate_sequence_parallel(OracleOps(), R, h, g, v, k, q, 16, dhf, do)
        assert O.rel_l2(hf0, hf[0]) < 1e-11 and O.rel_l2(out0, out[0]) < 1e-11
        for a, b in zip(gr0, grads):
            assert O.rel_l2(a, b[0]) < 1e-10


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q_out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        h, g, v, k, q, dhf, do = _inputs()
        L = v.shape[1] // world
        sl = slice(rank * L, (rank + 1) * L)
        leaves = [x.clone().requires_grad_(True) for x in (h, g[:, sl], v[:, sl], k[:, sl], q[:, sl])]
        hf, out = P.sequence_parallel_chunk_gla(*leaves, chunk_size=16, ops=OracleOps())
        loss = (hf * dhf).sum() / world + (out * do[:, sl]).sum()      # hidden_final term shared by the ranks
        # each rank holds the same hidden_final; its cotangent must be the full dhf on every rank
        grads = torch.autograd.grad((hf * dhf).sum() + (out * do[:, sl]).sum(), leaves)
        # numpy arrays are pickled by value: no shared-memory handles that die with the child process
        q_out.put((rank, hf.detach().numpy(), out.detach().numpy(), [x.detach().numpy() for x in grads], float(loss.detach())))
    finally:
        dist.destroy_process_group()


def test_sequence_parallel_gloo_world2():
    world = 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q_out.get(timeout=60) for _ in range(world)], key=lambda x: x[0])
    res = [(r[0], torch.from_numpy(r[1]), torch.from_numpy(r[2]), [torch.from_numpy(x) for x in r[3]]) for r in res]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    h, g, v, k, q, dhf, do = _inputs()
    hf0, out0, gr0 = _reference(h, g, v, k, q, dhf, do)
    out = torch.cat([r[2] for r in res], dim=1)
    assert O.rel_l2(out0, out[0]) < 1e-11
    for r in res:
        assert O.rel_l2(hf0, r[1][0]) < 1e-11              # hidden_final identical on every rank
        assert O.rel_l2(gr0[0], r[3][0][0]) < 1e-10        # dhidden_init of the whole sequence on every rank
    for i in range(1, 5):
        full = torch.cat([r[3][i] for r in res], dim=1)
        assert O.rel_l2(gr0[i], full[0]) < 1e-10


def test_shard_batch_heads():
    for B, H, W in ((32, 16, 8), (4, 6, 2), (1, 8, 8), (2, 8, 4)):
        seen = set()
        for r in range(W):
            bs, hs = P.shard_batch_heads(B, H, W, r)
            for b in range(*bs.indices(B)):
                for h in range(*hs.indices(H)):
                    assert (b, h) not in seen
                    seen.add((b, h))
        assert len(seen) == B * H
    with pytest.raises(ValueError):
        P.shard_batch_heads(3, 5, 4, 0)


def _failure_worker(rank, world, port, q_out, mode):
    """mode 'shape': rank 1 passes a slice of another length.  mode 'leave': rank 1 takes part in the first step
    and then exits; rank 0's second step must fail within the group's timeout instead of waiting forever."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    torch.set_num_threads(1)
    h, g, v, k, q, dhf, do = _inputs()
    L = v.shape[1] // world
    sl = slice(rank * L, (rank + 1) * L)
    if mode == "shape" and rank == 1:
        sl = slice(rank * L, rank * L + L // 2)
    result = "ok"
    t0 = time.time()
    try:
        P.sequence_parallel_chunk_gla(h, g[:, sl], v[:, sl], k[:, sl], q[:, sl], chunk_size=16, ops=OracleOps())
        if mode == "leave":
            if rank == 1:
                q_out.put((rank, "left", 0.0))
                q_out.close()
                q_out.join_thread()     # the message is on its way before the process disappears
                os._exit(0)             # gone between two steps, with nothing of its own in flight
            t0 = time.time()
            P.sequence_parallel_chunk_gla(h, g[:, sl], v[:, sl], k[:, sl], q[:, sl], chunk_size=16, ops=OracleOps())
    except P.SequenceParallelError as e:
        result = "SequenceParallelError: " + str(e)[:80]
    q_out.put((rank, result, time.time() - t0))
    q_out.close()
    q_out.join_thread()
    os._exit(0)                         # no orderly shutdown of a group whose peer has gone


@pytest.mark.parametrize("mode", ["shape", "leave"])
def test_sequence_parallel_host_side_failures(mode):
    """Failures are made on the host (no device involved): a rank with a wrong shape makes EVERY rank raise; a rank
    that leaves between steps makes the remaining rank raise within the process group's timeout."""
    world = 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failure_worker, args=(r, world, port, q_out, mode)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict()
    for _ in range(world):
        r, what, dt = q_out.get(timeout=90)
        res[r] = (what, dt)
    for p in procs:
        p.join(timeout=30)
    if mode == "shape":
        assert all(w.startswith("SequenceParallelError") for w, _ in res.values()), res
    else:
        assert res[1][0] == "left"
        assert res[0][0].startswith("SequenceParallelError") and res[0][1] < 60, res
