"""GPU parity tests (pytest -m gpu): the CUDA kernels, called through the C ABI via the
Python operators, against the CPU oracle on the same seeded inputs.

Tolerances are the ones the project states (relative L2, |a-b|/|a|, gla.py:1462):
  float32: out, hidden_final and gradients <= 1e-4
  bfloat16: out, hidden_final <= 1e-2, gradients <= 2e-2
"""
import numpy as np
import pytest
import torch

from oracle import gla_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (1e-4, 1e-4), torch.bfloat16: (1e-2, 2e-2)}
NAMES = ("dhidden_init", "dlog_fgate", "dvalue", "dkey", "dquery")


def _case(B, T, H, D, dtype, seed, shift, zero_init=False):
    h, g, v, k, q = O.make_inputs(B, T, H, D, dtype, seed=seed, shift=shift, zero_init=zero_init)
    gen = torch.Generator().manual_seed(seed + 100)
    dhf = torch.randn(B, H, D, D, generator=gen).to(dtype)
    do = torch.randn(B, T, H, D, generator=gen).to(dtype)
    return h, g, v, k, q, dhf, do


def _oracle(h, g, v, k, q, dhf, do, reverse=False):
    outs = []
    for b in range(v.shape[0]):
        outs.append(O.value_and_grads(O.recurrent_gla_naive, h[b], g[b], v[b], k[b], q[b], dhf[b], do[b],
                                      reverse=reverse))
    hf = torch.stack([o[0] for o in outs])
    out = torch.stack([o[1] for o in outs])
    grads = [torch.stack([o[2][i] for o in outs]) for i in range(5)]
    return hf, out, grads


def _run_gpu(fn, dev, h, g, v, k, q, dhf, do, **kw):
    leaves = [x.to(dev).requires_grad_(True) for x in (h, g, v, k, q)]
    hf, out = fn(*leaves, **kw)
    loss = (hf.float() * dhf.to(dev).float()).sum() + (out.float() * do.to(dev).float()).sum()
    grads = torch.autograd.grad(loss, leaves)
    torch.cuda.synchronize()
    return hf.cpu(), out.cpu(), [x.cpu() for x in grads]


def _compare(ref, got, dtype, what):
    tol_f, tol_g = TOL[dtype]
    hf0, o0, g0 = ref
    hf1, o1, g1 = got
    errs = {"hidden_final": O.rel_l2(hf0, hf1), "out": O.rel_l2(o0, o1)}
    for n, a, b in zip(NAMES, g0, g1):
        errs[n] = O.rel_l2(a, b)
    bad = {n: e for n, e in errs.items() if not (e < (tol_f if n in ("hidden_final", "out") else tol_g))}
    assert not bad, f"{what}: relative L2 over tolerance: {bad} (all: {errs})"


CHUNK_CASES = [
    # B, T, H, D, C, dtype, shift, zero_init
    (1, 256, 2, 64, 64, torch.float32, 5.0, False),      # benchmark config 1
    (2, 128, 2, 32, 32, torch.float32, 0.0, False),      # sharp gates
    (1, 64, 1, 64, 64, torch.float32, 5.0, False),       # a single chunk
    (1, 128, 3, 16, 16, torch.float32, 5.0, True),       # smallest sizes, zero initial state
    (1, 256, 2, 128, 128, torch.float32, 5.0, False),
    (1, 512, 1, 256, 256, torch.float32, 0.0, False),    # config 5 head size, sharp gates
    (1, 512, 1, 256, 256, torch.bfloat16, 0.0, False),   # ... in bf16 on the float32 kernels
    (2, 256, 2, 64, 64, torch.bfloat16, 5.0, False),
    (1, 512, 2, 128, 128, torch.bfloat16, 5.0, False),   # config 2 tile shape
    (1, 256, 2, 128, 128, torch.bfloat16, 0.0, False),   # config 2 tile shape, sharp gates
]


@pytest.mark.parametrize("B,T,H,D,C,dtype,shift,zero_init", CHUNK_CASES)
def test_chunk_gla_fp32_kernels_vs_oracle(cuda_device, B, T, H, D, C, dtype, shift, zero_init):
    from gla_jax_b200 import chunk_gla
    case = _case(B, T, H, D, dtype, 0, shift, zero_init)
    ref = _oracle(*case)
    got = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=C, impl="fp32")
    _compare(ref, got, dtype, f"chunk_gla fp32 kernels {B,T,H,D,C,dtype}")


TC_CASES = [
    # B, T, H, shift, zero_init   (bf16, D = chunk = 128: the native shape of the tcgen05 kernels)
    (1, 128, 1, 5.0, False),       # one chunk
    (1, 512, 2, 5.0, False),
    (2, 512, 3, 0.0, False),       # sharp gates (benchmark config 5's gate distribution)
    (1, 256, 2, -3.0, False),      # very sharp gates: every level's weights underflow gracefully
    (2, 384, 2, 5.0, True),        # zero initial state, three chunks
]


TC_WIDE_CASES = [
    # B, T, H, D, C, shift    bf16 shapes the tensor-core kernels serve beyond D = chunk = 128:
    (1, 512, 2, 256, 256, 5.0),     # benchmark config 5's head and chunk size (a head of 256 = 2 x 2 blocks of 128)
    (1, 512, 1, 256, 256, 0.0),     # ... with its sharp gates
    (2, 256, 2, 256, 128, 0.0),
    (1, 512, 2, 128, 256, 5.0),     # a larger chunk size at head size 128 (the result does not depend on it)
]


@pytest.mark.parametrize("B,T,H,D,C,shift", TC_WIDE_CASES)
def test_chunk_gla_tcgen05_wide_heads_vs_oracle(cuda_device, B, T, H, D, C, shift):
    from gla_jax_b200 import chunk_gla, _lib
    case = _case(B, T, H, D, torch.bfloat16, 23, shift)
    ref = _oracle(*case)
    got = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=C, impl="tcgen05")
    assert _lib.load().gla_device_wait_timeouts() == 0
    _compare(ref, got, torch.bfloat16, f"chunk_gla tcgen05 {B,T,H,D,C,shift}")
    # and impl='auto' takes the same path for these shapes
    auto = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=C)
    assert torch.equal(auto[1], got[1])


@pytest.mark.parametrize("scales", ["", "+all_scales"])
@pytest.mark.parametrize("B,T,H,shift,zero_init", TC_CASES)
def test_chunk_gla_tcgen05_vs_oracle(cuda_device, B, T, H, shift, zero_init, scales):
    """Both ways of forming the intra-chunk terms: the per-chunk choice between one anchor and every level of the
    secondary chunking (mild gates, shift 5 and 2, take the single anchor; sharp ones, shift 0 and -3, all levels),
    and every level forced."""
    from gla_jax_b200 import chunk_gla, _lib
    case = _case(B, T, H, 128, torch.bfloat16, 21, shift, zero_init)
    ref = _oracle(*case)
    got = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=128, impl="tcgen05" + scales)
    assert _lib.load().gla_device_wait_timeouts() == 0
    _compare(ref, got, torch.bfloat16, f"chunk_gla tcgen05{scales} {B,T,H,shift}")


def test_one_scale_limit_is_decided_per_chunk(cuda_device):
    """A sequence whose chunks fall into all three regimes of the secondary chunking: mild gates (one anchor at the
    chunk's end), total log decay of a chunk between -60 and -140 (one anchor in the middle of the decay, state tile
    rescaled) and gates far too sharp for a single anchor (about -250 per chunk, where exp() of it underflows).
    Every chunk must take the path its own gates allow; the result must match the oracle and the all-levels path."""
    from gla_jax_b200 import chunk_gla, _lib
    B, T, H = 1, 1024, 2
    h, g, v, k, q, dhf, do = _case(B, T, H, 128, torch.bfloat16, 29, 5.0)
    g = g.clone()
    gen = torch.Generator().manual_seed(3)
    g[:, 128:256] = -2.0 + 0.5 * torch.randn(B, 128, H, 128, generator=gen).clamp(-2, 2)      # all levels
    g[:, 256:384] = -0.8 + 0.2 * torch.randn(B, 128, H, 128, generator=gen).clamp(-2, 2)      # about -102: middle anchor
    g[:, 512:640, 1, :64] = -1.9          # only some features of one head cross the second limit
    g[:, 640:768, 0, 64:] = -1.05         # -134 for half of the features of one head: middle anchor, close to its limit
    g[:, 768:896] = -0.45                 # -57.6: still the end anchor
    case = (h, g, v, k, q, dhf, do)
    ref = _oracle(*case)
    got = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=128, impl="tcgen05")
    full = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=128, impl="tcgen05+all_scales")
    assert _lib.load().gla_device_wait_timeouts() == 0
    for t in (got[0], got[1], *got[2]):
        assert torch.isfinite(t.float()).all()
    _compare(ref, got, torch.bfloat16, "mixed chunks, per-chunk choice")
    _compare(ref, full, torch.bfloat16, "mixed chunks, all levels")


STATE_PATH_CASES = [
    # B, T, H    (bf16, D = chunk = 128); the ring depths are 3 and 4, so 1..5 chunks cover every wrap case
    (1, 128, 1), (1, 256, 1), (1, 384, 2), (1, 512, 1), (1, 640, 1), (2, 1024, 3),
    (5, 256, 8),        # 160 blocks of the one-pass kernel: more than one wave of SMs
]


@pytest.mark.parametrize("B,T,H", STATE_PATH_CASES)
def test_chunk_states_one_pass_vs_product_and_scan(cuda_device, B, T, H):
    """The two ways of producing the chunk states (one-pass kernel; batched product + scan) are chosen by a
    cost estimate: force each in turn and require the same results, and parity with the oracle."""
    from gla_jax_b200 import chunk_gla, _lib
    case = _case(B, T, H, 128, torch.bfloat16, 33, 2.0, False)
    got = {}
    for mode, opt in (("1", "one_pass"), ("0", "two_kernels")):
        got[mode] = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=128, impl="tcgen05+" + opt)
    assert _lib.load().gla_device_wait_timeouts() == 0
    flat = {m: [got[m][0], got[m][1], *got[m][2]] for m in got}
    for name, a, b in zip(["hidden_final", "out", *NAMES], flat["1"], flat["0"]):
        err = O.rel_l2(b, a)
        assert err <= 4e-3, f"{name}: one-pass vs product+scan {err:.3e}"     # same bf16 operands, different summation order
    if B * T * H <= 4096:
        _compare(_oracle(*case), got["1"], torch.bfloat16, f"chunk_gla one-pass states {B,T,H}")


@pytest.mark.parametrize("B,T,H,shift", [
    (1, 2048, 2, 2.0),      # 16 chunks: four runs of four
    (2, 2176, 1, 2.0),      # 17 chunks: runs of 5, 5, 5, 2
    (1, 1152, 3, 2.0),      # 9 chunks: two runs (5 + 4)
    (1, 2048, 1, 0.0),      # sharp gates: the corrections underflow inside a run and are skipped
])
def test_chunk_states_in_runs_vs_one_walk(cuda_device, B, T, H, shift):
    """The one-pass state kernel over runs of chunks (every run from zero, corrected afterwards with the state that
    really enters it; chosen by itself for few heads and long sequences, forced here) against the single walk and
    the oracle: forward, backward, both final states."""
    import ctypes
    from gla_jax_b200 import chunk_gla, _lib
    lib = _lib.load()
    case = _case(B, T, H, 128, torch.bfloat16, 41, shift, False)
    one = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=128, impl="tcgen05+one_pass")
    lib.gla_profile_enable(1)
    runs = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=128, impl="tcgen05+segments")
    lib.gla_profile_enable(0)
    buf = ctypes.create_string_buffer(1 << 14)
    lib.gla_profile_report(buf, len(buf))
    assert b"seg_scan_kernel" in buf.value and b"sp_fix_states_kernel" in buf.value, buf.value
    assert lib.gla_device_wait_timeouts() == 0
    for name, a, b in zip(["hidden_final", "out", *NAMES], [one[0], one[1], *one[2]], [runs[0], runs[1], *runs[2]]):
        err = O.rel_l2(a, b)
        assert err <= 4e-3, f"{name}: runs vs one walk {err:.3e}"      # stored states are rounded to bf16 twice
    _compare(_oracle(*case), runs, torch.bfloat16, f"chunk_gla states in runs {B,T,H}")


def test_auto_picks_tcgen05_for_readme_shape(cuda_device):
    """impl='auto' must run the tensor-core kernels at D = chunk = 128 in bf16 (checked through
    the library's own launch profile) and the fp32 kernels elsewhere."""
    import ctypes
    from gla_jax_b200 import chunk_gla, _lib
    lib = _lib.load()
    for dtype, D, C, want in ((torch.bfloat16, 128, 128, b"tc_chunk_fwd_kernel"), (torch.float32, 64, 64, b"simt_score_kernel")):
        h, g, v, k, q = (x.to(cuda_device) for x in O.make_inputs(1, 2 * C, 2, D, dtype, seed=3))
        lib.gla_profile_enable(1)
        chunk_gla(h, g, v, k, q, chunk_size=C)
        lib.gla_profile_enable(0)
        buf = ctypes.create_string_buffer(1 << 14)
        lib.gla_profile_report(buf, len(buf))
        assert want in buf.value, buf.value


def test_tcgen05_matches_recurrent_at_readme_shape(cuda_device):
    """Full benchmark config 2 shape (B=4, H=6, D=128, T=4096, bf16), forward and backward: the
    tensor-core chunk path against recurrent_gla (exact fp32 recurrence) on the GPU, since the
    CPU oracle cannot afford this size.  Same tolerances as against the oracle."""
    from gla_jax_b200 import chunk_gla, recurrent_gla
    case = _case(4, 4096, 6, 128, torch.bfloat16, 31, 5.0)
    a = _run_gpu(recurrent_gla, cuda_device, *case)
    b = _run_gpu(chunk_gla, cuda_device, *case, chunk_size=128, impl="tcgen05")
    _compare(a, b, torch.bfloat16, "tcgen05 vs recurrent at config 2")
    # size-independent property: chaining two half-length calls equals one call (gla.py:720-723)
    h, g, v, k, q = (x.to(cuda_device) for x in case[:5])
    with torch.no_grad():
        hf, out = chunk_gla(h, g, v, k, q, chunk_size=128)
        h1, o1 = chunk_gla(h, g[:, :2048], v[:, :2048], k[:, :2048], q[:, :2048], chunk_size=128)
        h2, o2 = chunk_gla(h1, g[:, 2048:], v[:, 2048:], k[:, 2048:], q[:, 2048:], chunk_size=128)
    assert O.rel_l2(hf.cpu(), h2.cpu()) < 1e-2 and O.rel_l2(out.cpu(), torch.cat([o1, o2], 1).cpu()) < 1e-2


@pytest.mark.parametrize("B,T,H,D,dtype,shift,reverse", [
    (1, 256, 2, 64, torch.float32, 5.0, False),
    (2, 100, 3, 32, torch.float32, 0.0, False),          # T not a multiple of the time block
    (1, 128, 2, 128, torch.float32, 5.0, True),
    (1, 64, 1, 256, torch.float32, 0.0, False),
    (2, 256, 2, 128, torch.bfloat16, 5.0, False),
    (1, 128, 2, 64, torch.bfloat16, 0.0, True),
    (1, 841, 2, 32, torch.float32, 5.0, False),          # long enough that the dlog_fgate scan runs in segments
    (1, 600, 1, 64, torch.float32, 5.0, True),
])
def test_recurrent_gla_vs_oracle(cuda_device, B, T, H, D, dtype, shift, reverse):
    from gla_jax_b200 import recurrent_gla
    case = _case(B, T, H, D, dtype, 1, shift)
    ref = _oracle(*case, reverse=reverse)
    got = _run_gpu(recurrent_gla, cuda_device, *case, reverse=reverse)
    _compare(ref, got, dtype, f"recurrent_gla {B,T,H,D,dtype,reverse}")


def test_recurrent_gla_naive_returns_fp32_out(cuda_device):
    from gla_jax_b200 import recurrent_gla_naive
    case = _case(1, 128, 2, 64, torch.bfloat16, 2, 5.0)
    ref = _oracle(*case)
    got = _run_gpu(recurrent_gla_naive, cuda_device, *case, reverse=False)
    assert got[1].dtype == torch.float32 and got[0].dtype == torch.bfloat16   # gla.py:43-46
    _compare(ref, got, torch.bfloat16, "recurrent_gla_naive")


def test_per_sequence_signature(cuda_device):
    """The reference's unbatched shapes (T,H,D)/(H,D,D) work unchanged."""
    from gla_jax_b200 import chunk_gla, recurrent_gla
    h, g, v, k, q = O.make_inputs(1, 128, 2, 64, torch.float32, seed=5, batch_axis=False)
    hf0, o0 = O.recurrent_gla_naive(h, g, v, k, q)
    dev = cuda_device
    hf1, o1 = chunk_gla(h.to(dev), g.to(dev), v.to(dev), k.to(dev), q.to(dev), chunk_size=64)
    hf2, o2 = recurrent_gla(h.to(dev), g.to(dev), v.to(dev), k.to(dev), q.to(dev))
    assert tuple(o1.shape) == (128, 2, 64) and tuple(hf1.shape) == (2, 64, 64)
    for hf, o in ((hf1, o1), (hf2, o2)):
        assert O.rel_l2(hf0, hf.cpu()) < 1e-4 and O.rel_l2(o0, o.cpu()) < 1e-4


def test_golden_fixtures_on_gpu(cuda_device):
    """Committed fixtures (float64 oracle, stored float32) vs the GPU kernels."""
    from pathlib import Path
    from gla_jax_b200 import chunk_gla, recurrent_gla
    for f in sorted((Path(__file__).parent / "golden").glob("*.npz")):
        z = np.load(f)
        T, H, D, C = (int(z[n]) for n in ("T", "H", "D", "C"))
        h, g, v, k, q = O.make_inputs(1, T, H, D, torch.float32, seed=int(z["seed"]), shift=float(z["shift"]))
        dhf, do = torch.from_numpy(z["dhf"])[None], torch.from_numpy(z["dout"])[None]
        ref = (torch.from_numpy(z["hidden_final"])[None], torch.from_numpy(z["out"])[None],
               [torch.from_numpy(z[n])[None] for n in NAMES])
        got = _run_gpu(chunk_gla, cuda_device, h, g, v, k, q, dhf, do, chunk_size=C)
        _compare(ref, got, torch.float32, f"golden {f.name} chunk_gla")
        got = _run_gpu(recurrent_gla, cuda_device, h, g, v, k, q, dhf, do)
        _compare(ref, got, torch.float32, f"golden {f.name} recurrent_gla")


@pytest.mark.parametrize("N,T,D,reverse,with_init,dtype", [
    (3, 50, 7, False, True, torch.float32), (2, 4096, 96, True, True, torch.float32),
    (1, 1, 33, False, False, torch.float32), (4, 300, 64, True, False, torch.bfloat16),
    # rows of 128 columns and more take the four-columns-per-thread kernel: whole and partial column blocks,
    # lengths that are no multiple of its 128-row tile, both directions, both element types
    (2, 1000, 128, False, True, torch.float32), (3, 333, 160, True, True, torch.float32),
    (2, 515, 256, True, True, torch.bfloat16), (1, 128, 768, False, False, torch.bfloat16),
    # the float32 pipeline at its edges: exactly two tiles, one position more (reversed: a first tile of one row),
    # a last column block of four columns, more (row, column block) items than SMs
    (4, 128, 256, False, True, torch.float32), (2, 129, 128, True, False, torch.float32),
    (2, 200, 132, False, True, torch.float32), (40, 192, 512, True, True, torch.float32),
])
def test_cumsum_vs_oracle(cuda_device, N, T, D, reverse, with_init, dtype):
    from gla_jax_b200 import cumsum_recursive, cumsum_pallas
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(N, T, D, generator=gen).to(dtype)
    init = torch.randn(N, D, generator=gen).to(dtype) if with_init else None
    ref = O.cumsum(x, 1, init=init, reverse=reverse, out_dtype=torch.float32, compute_dtype=torch.float64)
    dev = cuda_device
    y = cumsum_recursive(x.to(dev), axis=1, init=None if init is None else init.to(dev), reverse=reverse)
    assert y.dtype == dtype
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert O.rel_l2(ref, y.cpu().float()) < tol
    y2 = cumsum_pallas(x.to(dev), axis=-2, init=None if init is None else init.to(dev), reverse=reverse,
                       out_dtype=torch.float32)
    assert y2.dtype == torch.float32 and O.rel_l2(ref, y2.cpu()) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_cumsum_wide_rows_from_an_unaligned_base(cuda_device):
    """Rows of 128+ columns whose base address is not 16-byte aligned fall back to the scalar kernel: same result
    as the aligned call (which takes the four-columns-per-thread kernel), bit for bit in float32 addition order
    per column."""
    from gla_jax_b200 import cumsum_recursive
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(2, 700, 128, generator=gen)
    buf = torch.empty(x.numel() + 1, device=cuda_device)
    xu = buf[1:].view(2, 700, 128)
    xu.copy_(x)
    assert xu.data_ptr() % 16 != 0 and xu.is_contiguous()
    ya, yu = cumsum_recursive(x.to(cuda_device), axis=1), cumsum_recursive(xu, axis=1)
    assert O.rel_l2(torch.cumsum(x.double(), 1), ya.cpu()) < 1e-5
    assert O.rel_l2(ya.cpu().double(), yu.cpu()) < 1e-6


def test_cumsum_inner_axis_layout(cuda_device):
    """Scan along a middle axis of a 4-d array, the layout chunk_gla uses (N, C, D) -> axis -2."""
    from gla_jax_b200 import cumsum_recursive
    x = torch.randn(2, 5, 64, 24)
    y = cumsum_recursive(x.to(cuda_device), axis=-2)
    assert O.rel_l2(torch.cumsum(x.double(), -2), y.cpu()) < 1e-5


@pytest.mark.parametrize("T,K,V,reverse,with_init,dtype", [
    (20, 5, 4, False, True, torch.float32), (32, 128, 128, True, True, torch.float32),
    (300, 16, 24, False, False, torch.float32), (64, 64, 64, False, True, torch.bfloat16),
    # long axes with few rows: cut into runs scanned by separate blocks and put together afterwards (7 runs of 143
    # and 142 positions; 5 runs with a short last one)
    (1000, 32, 32, False, True, torch.float32), (1000, 32, 32, True, True, torch.float32),
    (641, 16, 64, True, False, torch.float32), (1000, 32, 32, False, True, torch.bfloat16),
])
def test_rnn_scan_vs_oracle(cuda_device, T, K, V, reverse, with_init, dtype):
    from gla_jax_b200 import rnn_recursive, rnn_pallas
    gen = torch.Generator().manual_seed(4)
    g = -torch.rand(T, K, generator=gen)
    kv = torch.randn(T, K, V, generator=gen).to(dtype)
    ig = -torch.rand(K, generator=gen) if with_init else None
    ikv = torch.randn(K, V, generator=gen).to(dtype) if with_init else None
    A0, S0 = O.rnn_scan(g.double(), kv.double(), None if ig is None else ig.double(),
                        None if ikv is None else ikv.double(), reverse=reverse, compute_dtype=torch.float64)
    dev = cuda_device
    mv = lambda x: None if x is None else x.to(dev)
    A1, S1 = rnn_recursive(mv(g), mv(kv), mv(ig), mv(ikv), reverse=reverse)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert S1.dtype == dtype
    assert O.rel_l2(A0, A1.cpu()) < 1e-5 and O.rel_l2(S0, S1.cpu().float()) < tol
    # last_only: only the final row is defined (ops.py:330-334)
    A2, S2 = rnn_pallas(mv(g), mv(kv), mv(ig), mv(ikv), reverse=reverse, last_only=True)
    last = 0 if reverse else T - 1
    assert O.rel_l2(A0[last], A2[last].cpu()) < 1e-5 and O.rel_l2(S0[last], S2[last].cpu().float()) < tol


def test_sp_combine2_matches_two_calls_of_sp_combine(cuda_device):
    """The one-launch combine (state entering a rank's slice + state leaving the last slice, from packed [G | S]
    records addressed through rank strides) against two calls of gla_sp_combine on separate arrays."""
    from gla_jax_b200 import _lib
    lib = _lib.load()
    R, BH, D = 5, 3, 128
    gen = torch.Generator().manual_seed(21)
    nG, nS = BH * D, BH * D * D
    packed = torch.randn(R, nG + nS, generator=gen)
    packed[:, :nG] = -packed[:, :nG].abs()
    packed = packed.to(cuda_device)
    init = torch.randn(BH, D, D, generator=gen).bfloat16().to(cuda_device)
    all_G, all_S = packed[:, :nG].contiguous(), packed[:, nG:].contiguous()
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    for reverse in (0, 1):
        for rank in range(R):
            ent = torch.empty(BH, D, D, device=cuda_device)
            tot = torch.empty(BH, D, D, dtype=torch.bfloat16, device=cuda_device)
            _lib.check(lib.gla_sp_combine2(stream, R, rank, BH, D, packed.data_ptr(), nG + nS, packed.data_ptr() + 4 * nG, nG + nS,
                                           init.data_ptr(), _lib.GLA_BF16, ent.data_ptr(), tot.data_ptr(), _lib.GLA_BF16, reverse),
                       "gla_sp_combine2")
            ent0 = torch.empty_like(ent)
            tot0 = torch.empty_like(tot)
            _lib.check(lib.gla_sp_combine(stream, R, rank, BH, D, all_G.data_ptr(), all_S.data_ptr(), init.data_ptr(), _lib.GLA_BF16,
                                          ent0.data_ptr(), _lib.GLA_F32, reverse), "gla_sp_combine")
            _lib.check(lib.gla_sp_combine(stream, R, -1 if reverse else R, BH, D, all_G.data_ptr(), all_S.data_ptr(), init.data_ptr(),
                                          _lib.GLA_BF16, tot0.data_ptr(), _lib.GLA_BF16, reverse), "gla_sp_combine")
            assert torch.equal(ent, ent0) and torch.equal(tot, tot0), (reverse, rank)


def test_rnn_scan_long_axis_in_runs_matches_the_single_walk(cuda_device):
    """The segmented form of the linear-RNN scan (chosen for long axes with few rows) against the single sequential
    walk of the same library (gla_rnn_scan, no scratch), batched, both directions."""
    from gla_jax_b200 import rnn_pallas, _lib
    lib = _lib.load()
    Bn, T, K, V = 2, 2048, 16, 32
    assert lib.gla_rnn_scan_workspace_bytes(Bn, T, K, V) > 0 and lib.gla_rnn_scan_workspace_bytes(64, T, 128, 128) == 0
    gen = torch.Generator().manual_seed(12)
    g = (-0.1 * torch.rand(Bn, T, K, generator=gen)).to(cuda_device)
    kv = torch.randn(Bn, T, K, V, generator=gen).to(cuda_device)
    ig = (-torch.rand(Bn, K, generator=gen)).to(cuda_device)
    ikv = torch.randn(Bn, K, V, generator=gen).to(cuda_device)
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    for reverse in (False, True):
        A1, S1 = rnn_pallas(g, kv, ig, ikv, reverse=reverse)
        A0, S0 = torch.zeros_like(g), torch.zeros_like(kv)
        _lib.check(lib.gla_rnn_scan(stream, Bn, T, K, V, g.data_ptr(), kv.data_ptr(), ig.data_ptr(), ikv.data_ptr(),
                                    A0.data_ptr(), S0.data_ptr(), int(reverse), 0, _lib.GLA_F32), "gla_rnn_scan")
        assert O.rel_l2(A0.cpu(), A1.cpu()) < 1e-6 and O.rel_l2(S0.cpu(), S1.cpu()) < 1e-5, reverse


def test_chunk_equals_recurrent_on_gpu_full_size_slice(cuda_device):
    """Cross-check of the two GPU implementations at the README tile shape (D = C = 128) on
    a longer sequence than the oracle can afford: chunk_gla vs recurrent_gla, fp32."""
    from gla_jax_b200 import chunk_gla, recurrent_gla
    h, g, v, k, q = (x.to(cuda_device) for x in O.make_inputs(2, 2048, 2, 128, torch.float32, seed=9))
    hf1, o1 = chunk_gla(h, g, v, k, q, chunk_size=128, impl="fp32")
    hf2, o2 = recurrent_gla(h, g, v, k, q)
    assert O.rel_l2(hf2.cpu(), hf1.cpu()) < 1e-4 and O.rel_l2(o2.cpu(), o1.cpu()) < 1e-4


@pytest.mark.parametrize("B,H,D,dtype,steps,shift", [
    (2, 3, 64, torch.float32, 40, 5.0),
    (1, 2, 128, torch.float32, 24, 0.0),
    (3, 2, 128, torch.bfloat16, 32, 5.0),
    (1, 1, 256, torch.bfloat16, 16, 0.0),
    (2, 2, 32, torch.float32, 8, 5.0),
])
def test_decode_step_chain_equals_recurrence(cuda_device, B, H, D, dtype, steps, shift):
    """T calls of the single-token step from hidden_init equal the oracle's recurrence over T tokens
    (out per token and the final state), and one recurrent_gla call on the GPU."""
    from gla_jax_b200 import decode_step, recurrent_gla
    h, g, v, k, q = O.make_inputs(B, steps, H, D, dtype, seed=41, shift=shift)
    ref = [O.recurrent_gla_naive(h[b].double(), g[b].double(), v[b].double(), k[b].double(), q[b].double())
           for b in range(B)]
    ref_hf = torch.stack([r[0] for r in ref]).float()
    ref_out = torch.stack([r[1] for r in ref]).float()
    gd, vd, kd, qd = (x.to(cuda_device) for x in (g, v, k, q))
    state = h.to(cuda_device).float().contiguous()
    outs = []
    for t in range(steps):
        outs.append(decode_step(state, gd[:, t], vd[:, t], kd[:, t], qd[:, t]))
    out = torch.stack(outs, dim=1)
    torch.cuda.synchronize()
    tol = 1e-4 if dtype == torch.float32 else 1e-2
    assert O.rel_l2(ref_out, out.float().cpu()) < tol
    assert O.rel_l2(ref_hf, state.cpu()) < (1e-4 if dtype == torch.float32 else 4e-3)   # state stays float32
    hf2, out2 = recurrent_gla(h.to(cuda_device), gd, vd, kd, qd)
    assert O.rel_l2(out2.float().cpu(), out.float().cpu()) < tol


def test_decode_step_rejects_bad_arguments(cuda_device):
    from gla_jax_b200 import decode_step
    st = torch.zeros(1, 2, 64, 64, device=cuda_device)
    x = torch.zeros(1, 2, 64, device=cuda_device)
    with pytest.raises(TypeError):
        decode_step(st.half(), x, x, x, x)
    with pytest.raises(ValueError):
        decode_step(st, x, x[:, :1], x, x)
    st48 = torch.zeros(1, 1, 48, 48, device=cuda_device)
    x48 = torch.zeros(1, 1, 48, device=cuda_device)
    with pytest.raises(Exception):
        decode_step(st48, x48, x48, x48, x48)       # head size without a kernel: GLA_ERR_UNSUPPORTED


@pytest.mark.parametrize("lengths,H,shift", [
    ([128, 384, 256], 2, 5.0),
    ([512], 1, 5.0),                       # a single sequence: must equal chunk_gla
    ([256, 128, 128, 640, 128], 3, 0.0),   # sharp gates, single-chunk sequences in the mix
])
def test_chunk_gla_packed_equals_per_sequence_calls(cuda_device, lengths, H, shift):
    """Variable-length sequences packed on one time axis: forward and backward equal separate chunk_gla calls
    (the packed path always takes the one-pass state kernel, so the separate calls are pinned to it as well and the
    results must agree to the last bit or nearly), and parity with the oracle."""
    from gla_jax_b200 import chunk_gla, chunk_gla_packed, _lib
    D, T, nseq = 128, sum(lengths), len(lengths)
    cu = [0]
    for L in lengths:
        cu.append(cu[-1] + L)
    _, g, v, k, q = O.make_inputs(1, T, H, D, torch.bfloat16, seed=51, shift=shift)
    gen = torch.Generator().manual_seed(52)
    h = torch.randn(nseq, H, D, D, generator=gen).to(torch.bfloat16)
    dhf = torch.randn(nseq, H, D, D, generator=gen).to(torch.bfloat16)
    do = torch.randn(T, H, D, generator=gen).to(torch.bfloat16)
    dev = cuda_device
    leaves = [x.to(dev).requires_grad_(True) for x in (h, g[0], v[0], k[0], q[0])]
    hf, out = chunk_gla_packed(*leaves, torch.tensor(cu, dtype=torch.int32), chunk_size=128)
    loss = (hf.float() * dhf.to(dev).float()).sum() + (out.float() * do.to(dev).float()).sum()
    grads = torch.autograd.grad(loss, leaves)
    torch.cuda.synchronize()
    assert _lib.load().gla_device_wait_timeouts() == 0
    for s in range(nseq):
        sl = slice(cu[s], cu[s + 1])
        case = (h[s:s + 1], g[:, sl], v[:, sl], k[:, sl], q[:, sl], dhf[s:s + 1], do[sl].unsqueeze(0))
        ref = _run_gpu(chunk_gla, dev, *case, chunk_size=128, impl="tcgen05+one_pass")
        got = (hf[s:s + 1].cpu(), out[sl].unsqueeze(0).cpu(),
               [grads[0][s:s + 1].cpu(), grads[1][sl].unsqueeze(0).cpu(), grads[2][sl].unsqueeze(0).cpu(),
                grads[3][sl].unsqueeze(0).cpu(), grads[4][sl].unsqueeze(0).cpu()])
        for name, a, b in zip(["hidden_final", "out", *NAMES], [ref[0], ref[1], *ref[2]], [got[0], got[1], *got[2]]):
            assert O.rel_l2(a, b) <= 1e-6, f"sequence {s} {name}: packed vs separate {O.rel_l2(a, b):.3e}"
        if lengths[s] <= 256:
            _compare(_oracle(*case), got, torch.bfloat16, f"chunk_gla_packed sequence {s}")


def test_chunk_gla_packed_rejects_bad_offsets(cuda_device):
    from gla_jax_b200 import chunk_gla_packed
    H, D = 1, 128
    x = torch.zeros(256, H, D, device=cuda_device, dtype=torch.bfloat16)
    g = torch.zeros(256, H, D, device=cuda_device)
    h = torch.zeros(2, H, D, D, device=cuda_device, dtype=torch.bfloat16)
    for cu in ([0, 128, 384], [128, 256, 256], [0, 256], [0, 200, 100, 256]):
        with pytest.raises(ValueError):
            chunk_gla_packed(h, g, x, x, x, cu)


def test_chunk_gla_packed_ragged_lengths_vs_oracle(cuda_device):
    """Sequence lengths that are no multiples of the chunk length (the reference asserts T % chunk == 0,
    gla.py:499-500): tails are padded with neutral tokens inside the operator.  Forward and all five gradients of
    every sequence against the float64 oracle on the unpadded sequence."""
    from gla_jax_b200 import chunk_gla_packed
    lengths, H, D = [100, 257, 128, 31], 2, 128
    T, nseq = sum(lengths), len(lengths)
    cu = [0]
    for L in lengths:
        cu.append(cu[-1] + L)
    _, g, v, k, q = O.make_inputs(1, T, H, D, torch.bfloat16, seed=81, shift=3.0)
    gen = torch.Generator().manual_seed(82)
    h = torch.randn(nseq, H, D, D, generator=gen).to(torch.bfloat16)
    dhf = torch.randn(nseq, H, D, D, generator=gen).to(torch.bfloat16)
    do = torch.randn(T, H, D, generator=gen).to(torch.bfloat16)
    dev = cuda_device
    leaves = [x.to(dev).requires_grad_(True) for x in (h, g[0], v[0], k[0], q[0])]
    hf, out = chunk_gla_packed(*leaves, cu, chunk_size=128)
    assert tuple(out.shape) == (T, H, D)
    grads = torch.autograd.grad((hf.float() * dhf.to(dev).float()).sum() + (out.float() * do.to(dev).float()).sum(), leaves)
    torch.cuda.synchronize()
    for s_ in range(nseq):
        sl = slice(cu[s_], cu[s_ + 1])
        case = (h[s_:s_ + 1], g[:, sl], v[:, sl], k[:, sl], q[:, sl], dhf[s_:s_ + 1], do[sl].unsqueeze(0))
        got = (hf[s_:s_ + 1].cpu(), out[sl].unsqueeze(0).cpu(),
               [grads[0][s_:s_ + 1].cpu()] + [grads[i][sl].unsqueeze(0).cpu() for i in range(1, 5)])
        _compare(_oracle(*case), got, torch.bfloat16, f"ragged packed sequence {s_} (length {lengths[s_]})")


def test_triton_scan_dispatches_to_the_cuda_scans(cuda_device):
    """The host-level generic scan recognises the reference's two combine rules (ops.py:161, 318)."""
    import operator
    from gla_jax_b200 import triton_scan, binary_operator
    gen = torch.Generator().manual_seed(61)
    x = torch.randn(3, 100, 24, generator=gen)
    init = torch.randn(3, 24, generator=gen)
    got = triton_scan(operator.add, x.to(cuda_device), axis=1, init=init.to(cuda_device), reverse=True)
    ref = torch.flip(torch.cumsum(torch.flip(x.double(), [1]), 1), [1]) + init.double().unsqueeze(1)
    assert O.rel_l2(ref.float(), got.cpu()) < 1e-5
    g = torch.nn.functional.logsigmoid(torch.randn(50, 16, generator=gen))
    kv = torch.randn(50, 16, 8, generator=gen)
    ig, ikv = torch.randn(16, generator=gen).clamp(max=0), torch.randn(16, 8, generator=gen)
    out_log, out_state = triton_scan(binary_operator, (g.to(cuda_device), kv.to(cuda_device)), axis=0,
                                     init=(ig.to(cuda_device), ikv.to(cuda_device)))
    ref_log, ref_state = O.rnn_scan(g.double(), kv.double(), ig.double(), ikv.double())
    assert O.rel_l2(ref_log.float(), out_log.cpu()) < 1e-5 and O.rel_l2(ref_state.float(), out_state.cpu()) < 1e-5
    with pytest.raises(NotImplementedError):
        triton_scan(torch.atan2, x.to(cuda_device), axis=1)


@pytest.mark.parametrize("rule,ref_fn", [
    ("mul", lambda x: torch.cumprod(x, 1)),
    ("max", lambda x: torch.cummax(x, 1).values),
    ("min", lambda x: torch.cummin(x, 1).values),
    ("logaddexp", lambda x: torch.logcumsumexp(x, 1)),
])
def test_scan_library_rules(cuda_device, rule, ref_fn):
    """The other combine rules of the scan library against torch's cumulative ops in float64: a length that spans
    many tiles and is no multiple of the tile, forward and reversed, with and without an initial value, and through
    triton_scan with the matching Python callable."""
    from gla_jax_b200 import scan, triton_scan
    gen = torch.Generator().manual_seed(67)
    x = torch.randn(3, 1000, 40, generator=gen)
    if rule == "mul":
        x = 1.0 + 0.01 * x            # keep the running product in range
    init = torch.randn(3, 40, generator=gen) if rule != "mul" else 1.0 + 0.1 * torch.randn(3, 40, generator=gen)
    comb = {"mul": torch.mul, "max": torch.maximum, "min": torch.minimum, "logaddexp": torch.logaddexp}[rule]
    xd = x.double()
    for reverse in (False, True):
        base = ref_fn(torch.flip(xd, [1]) if reverse else xd)
        base = torch.flip(base, [1]) if reverse else base
        got = scan(rule, x.to(cuda_device), 1, reverse=reverse)
        assert O.rel_l2(base, got.cpu()) < 1e-5, (rule, reverse)
        got_i = scan(rule, x.to(cuda_device), 1, init=init.to(cuda_device), reverse=reverse)
        assert O.rel_l2(comb(init.double().unsqueeze(1), base), got_i.cpu()) < 1e-5, (rule, reverse, "init")
    assert torch.equal(triton_scan(comb, x.to(cuda_device), axis=1), scan(rule, x.to(cuda_device), 1))
    # the long-axis form (segments run as separate blocks) agrees with the one-pass form
    y = torch.randn(1, 20000, 16, generator=gen) * (0.001 if rule == "mul" else 1.0) + (1.0 if rule == "mul" else 0.0)
    ref = ref_fn(y.double())
    assert O.rel_l2(ref, scan(rule, y.to(cuda_device), 1).cpu()) < 1e-5
    # rows wide enough for the four-columns-per-thread kernel
    w = torch.randn(2, 300, 256, generator=gen) * (0.01 if rule == "mul" else 1.0) + (1.0 if rule == "mul" else 0.0)
    assert O.rel_l2(ref_fn(w.double()), scan(rule, w.to(cuda_device), 1).cpu()) < 1e-5


def test_early_start_gives_the_same_bits_under_graph_replay(cuda_device):
    """The forward chunk kernel is launched as a programmatic dependent of the state kernel and starts beside it
    (README shape: the state kernel fills 96 of 148 SMs).  Results must not depend on that: forward+backward
    captured in a CUDA graph and replayed 20 times gives, every time, exactly the bits of a run with the chunk
    kernel kept strictly behind the state kernel (impl option no_early_start), and no bounded wait gave up.
    Every output, dlog_fgate included, is compared bit for bit: all reductions run in a fixed order."""
    from gla_jax_b200 import chunk_gla, _lib
    lib = _lib.load()
    case = _case(4, 4096, 6, 128, torch.bfloat16, 77, 5.0)
    h, g, v, k, q, dhf, do = (x.to(cuda_device) for x in case)

    def run(impl="auto"):
        leaves = [x.clone().requires_grad_(True) for x in (h, g, v, k, q)]
        hf, out = chunk_gla(*leaves, chunk_size=128, impl=impl)
        grads = torch.autograd.grad((hf.float() * dhf.float()).sum() + (out.float() * do.float()).sum(), leaves)
        return [hf, out, *grads]

    ref = [t.clone() for t in run("auto+no_early_start")]
    torch.cuda.synchronize()
    run()                                           # warm-up outside the capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            outs = run()
    t0 = lib.gla_device_wait_timeouts()
    for _ in range(20):
        graph.replay()
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(zip(ref, outs)):
            assert torch.equal(a, b), i
    assert lib.gla_device_wait_timeouts() == t0


@pytest.mark.parametrize("B,T,H", [(64, 128, 16), (16, 512, 12)])
def test_early_start_with_more_state_blocks_than_sms(cuda_device, B, T, H):
    """The one-pass state kernel forced on shapes where its grid (4 x batch x heads blocks) is many waves: the
    dependent chunk kernel may only start once the last wave is resident.  Forward against the exact recurrence
    kernel, and no bounded wait gave up."""
    from gla_jax_b200 import chunk_gla, recurrent_gla, _lib
    lib = _lib.load()
    h, g, v, k, q = (x.to(cuda_device) for x in O.make_inputs(B, T, H, 128, torch.bfloat16, seed=3))
    t0 = lib.gla_device_wait_timeouts()
    with torch.no_grad():
        hf, out = chunk_gla(h, g, v, k, q, chunk_size=128, impl="auto+one_pass")
        hf2, out2 = recurrent_gla(h, g, v, k, q)
    torch.cuda.synchronize()
    assert O.rel_l2(hf2.cpu(), hf.cpu()) < 1e-2 and O.rel_l2(out2.cpu(), out.cpu()) < 1e-2
    assert lib.gla_device_wait_timeouts() == t0


def test_fp32_forward_without_residuals_with_chunk_larger_than_head(cuda_device):
    """chunk > D on the float32 kernels under no_grad (no residual buffer: the scores go to workspace, which must
    be sized for them) and through the entry point that brings its own scratch; the reference accepts any
    power-of-two chunk size (gla.py:499-500)."""
    from gla_jax_b200 import chunk_gla
    for D, C in ((64, 128), (32, 256), (16, 64)):
        h, g, v, k, q = O.make_inputs(2, 2 * C, 2, D, torch.float32, seed=13)
        ref_hf, ref_out = O.batched(O.recurrent_gla_naive, h, g, v, k, q)
        with torch.no_grad():
            hf, out = chunk_gla(*(x.to(cuda_device) for x in (h, g, v, k, q)), chunk_size=C, impl="fp32")
        assert O.rel_l2(ref_hf, hf.cpu()) < 1e-4 and O.rel_l2(ref_out, out.cpu()) < 1e-4, (D, C)


def test_packed_offsets_on_the_device_are_clamped_not_trusted(cuda_device):
    """Offsets handed over as a CUDA tensor are not checked on the host (that would synchronise).  Out-of-range,
    decreasing or misaligned offsets must not make the kernels leave the buffers: every access stays inside
    (canary rows around the outputs are intact), the call completes, and gla_device_bad_offsets() counts them."""
    from gla_jax_b200 import chunk_gla_packed, _lib
    lib = _lib.load()
    H, D, T = 2, 128, 512
    _, g, v, k, q = (x[0].to(cuda_device) for x in O.make_inputs(1, T, H, D, torch.bfloat16, seed=71))
    h = torch.randn(3, H, D, D, device=cuda_device).to(torch.bfloat16)
    good = torch.tensor([0, 128, 384, 512], dtype=torch.int32, device=cuda_device)
    before = lib.gla_device_bad_offsets()
    hf0, out0 = chunk_gla_packed(h, g, v, k, q, good)
    torch.cuda.synchronize()
    assert lib.gla_device_bad_offsets() == before
    for bad in ([0, 128, 100000, 512], [0, 384, 128, 512], [0, 100, 384, 512], [-256, 128, 384, 512]):
        cu = torch.tensor(bad, dtype=torch.int32, device=cuda_device)
        n0 = lib.gla_device_bad_offsets()
        with torch.no_grad():
            hf, out = chunk_gla_packed(h, g, v, k, q, cu)
        torch.cuda.synchronize()
        assert lib.gla_device_bad_offsets() > n0, bad
        assert hf.shape == hf0.shape and out.shape == out0.shape
    # the library still works afterwards and gives the same answer as before
    hf1, out1 = chunk_gla_packed(h, g, v, k, q, good)
    assert torch.equal(hf1, hf0) and torch.equal(out1, out0)


def test_tensors_on_another_device_are_refused(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from gla_jax_b200 import recurrent_gla
    other = torch.device("cuda:1")
    h, g, v, k, q = (x.to(other) for x in O.make_inputs(1, 64, 1, 32, torch.float32, seed=1))
    with pytest.raises(RuntimeError):
        recurrent_gla(h, g, v, k, q)          # the current device is cuda:0
    with torch.cuda.device(other):
        hf, out = recurrent_gla(h, g, v, k, q)
    assert out.device == other
