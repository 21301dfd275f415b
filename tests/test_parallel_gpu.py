"""GPU tests of sequence parallelism: the schedule of gla_jax_b200/parallel.py on the CUDA
primitives (gla_chunk_sp_{fwd,bwd}_{local,finish} where the shape has them, else gla_chunk_local_state /
gla_chunk_local_dstate with the ordinary forward / backward; gla_sp_combine in both cases).
On one GPU the ranks run one after another in one process (no kernel waits on another rank,
the gathers are host-side stacks); with two or more GPUs a real NCCL run is added."""
import os
import socket

import pytest
import torch

from oracle import gla_oracle as O

pytestmark = pytest.mark.gpu
NAMES = ("dhidden_init", "dlog_fgate", "dvalue", "dkey", "dquery")


@pytest.mark.parametrize("dtype,D,C,R,impl,T,shift", [
    (torch.bfloat16, 128, 128, 4, "auto", 1024, 2.0),      # tensor-core kernels, 4 ranks x 256 tokens
    (torch.bfloat16, 128, 128, 2, "auto+two_kernels", 1024, 2.0),   # ... with the product + scan form of the states
    # sharp gates and 8 chunks per rank: the accumulated decay underflows after the first chunk or two, so the
    # correction of the kept states skips the rest (and every chunk takes all levels of the secondary chunking)
    (torch.bfloat16, 128, 128, 2, "auto", 2048, 0.0),
    # each rank's 16 chunks in four runs: local runs from zero, one correction pass per direction in the finish phase
    (torch.bfloat16, 128, 128, 2, "auto+segments", 4096, 2.0),
    (torch.float32, 64, 32, 2, "fp32", 1024, 2.0),
])
def test_emulated_sequence_parallel_on_one_gpu(cuda_device, dtype, D, C, R, impl, T, shift):
    from gla_jax_b200 import parallel as P
    from gla_jax_b200 import chunk_gla
    B, H = 1, 2
    h, g, v, k, q = O.make_inputs(B, T, H, D, dtype, seed=5, shift=shift)
    gen = torch.Generator().manual_seed(6)
    dhf = torch.randn(B, H, D, D, generator=gen).to(dtype)
    do = torch.randn(B, T, H, D, generator=gen).to(dtype)
    dev = cuda_device
    mv = lambda x: x.to(dev)
    hf, out, grads = P.emulate_sequence_parallel(P.CudaOps(impl), R, mv(h), mv(g), mv(v), mv(k), mv(q), C, mv(dhf), mv(do))
    torch.cuda.synchronize()
    ref = O.value_and_grads(O.recurrent_gla_naive, h[0], g[0], v[0], k[0], q[0], dhf[0], do[0])
    tf, tg = (1e-4, 1e-4) if dtype == torch.float32 else (1e-2, 2e-2)
    assert O.rel_l2(ref[0], hf[0].cpu()) < tf and O.rel_l2(ref[1], out[0].cpu()) < tf
    for n, a, b in zip(NAMES, ref[2], grads):
        assert O.rel_l2(a, b[0].cpu()) < tg, (n, O.rel_l2(a, b[0].cpu()))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _nccl_worker(rank, world, port, q_out):
    import torch.distributed as dist
    from gla_jax_b200 import parallel as P
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, T, H, D, C = 1, 2048, 2, 128, 128
        h, g, v, k, q = O.make_inputs(B, T, H, D, torch.bfloat16, seed=8)
        gen = torch.Generator().manual_seed(9)
        dhf = torch.randn(B, H, D, D, generator=gen).bfloat16()
        do = torch.randn(B, T, H, D, generator=gen).bfloat16()
        L = T // world
        sl = slice(rank * L, (rank + 1) * L)
        leaves = [x.to(dev).requires_grad_(True) for x in (h, g[:, sl], v[:, sl], k[:, sl], q[:, sl])]
        hf, out = P.sequence_parallel_chunk_gla(*leaves, chunk_size=C)
        grads = torch.autograd.grad((hf.float() * dhf.to(dev).float()).sum() + (out.float() * do[:, sl].to(dev).float()).sum(), leaves)
        torch.cuda.synchronize()
        # numpy arrays are pickled by value: no shared-memory handles that die with the child process
        q_out.put((rank, hf.detach().float().cpu().numpy(), out.detach().float().cpu().numpy(),
                   [x.detach().float().cpu().numpy() for x in grads]))
    finally:
        dist.destroy_process_group()


def test_sequence_parallel_nccl_two_gpus(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q_out.get(timeout=120) for _ in range(world)], key=lambda x: x[0])
    res = [(r[0], torch.from_numpy(r[1]), torch.from_numpy(r[2]), [torch.from_numpy(x) for x in r[3]]) for r in res]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    B, T, H, D = 1, 2048, 2, 128
    h, g, v, k, q = O.make_inputs(B, T, H, D, torch.bfloat16, seed=8)
    gen = torch.Generator().manual_seed(9)
    dhf = torch.randn(B, H, D, D, generator=gen).bfloat16()
    do = torch.randn(B, T, H, D, generator=gen).bfloat16()
    ref = O.value_and_grads(O.recurrent_gla_naive, h[0], g[0], v[0], k[0], q[0], dhf[0], do[0])
    out = torch.cat([r[2] for r in res], dim=1)
    assert O.rel_l2(ref[1], out[0]) < 1e-2
    for r in res:
        assert O.rel_l2(ref[0], r[1][0]) < 1e-2 and O.rel_l2(ref[2][0], r[3][0][0]) < 2e-2
    for i in range(1, 5):
        assert O.rel_l2(ref[2][i], torch.cat([r[3][i] for r in res], dim=1)[0]) < 2e-2
