"""CPU tests of the oracle itself (no GPU).

The reference ships no golden vectors and cannot be imported here, so the oracle is pinned by
agreement between independent restatements in float64: the step recurrence (gla.py:26-47), the
chunk algorithm with dyadic secondary chunking (gla.py:483-550, 695-729, 792-855, 964-1029) and
the hand-derived backward formulas (gla.py:172-269, 552-625, 731-790, 857-960, 1036-1189), each
checked against torch autograd of the recurrence, plus the committed fixtures in tests/golden.
"""
import numpy as np
import pytest
import torch

from oracle import gla_oracle as O

TOL = 1e-11


def _inputs(T, H, D, shift, seed=0, zero_init=False):
    h, g, v, k, q = O.make_inputs(1, T, H, D, torch.float64, seed=seed, shift=shift, zero_init=zero_init,
                                  batch_axis=False)
    gen = torch.Generator().manual_seed(seed + 100)
    dhf = torch.randn(H, D, D, generator=gen, dtype=torch.float64)
    do = torch.randn(T, H, D, generator=gen, dtype=torch.float64)
    return h, g.double(), v, k, q, dhf, do


@pytest.mark.parametrize("T,H,D,C,shift", [(128, 2, 32, 32, 5.0), (128, 2, 32, 64, 0.0), (64, 1, 16, 64, 0.0),
                                            (96, 3, 16, 32, -2.0)])
def test_chunk_matches_recurrence_fp64(T, H, D, C, shift):
    h, g, v, k, q, dhf, do = _inputs(T, H, D, shift)
    hf0, o0, gr0 = O.value_and_grads(O.recurrent_gla_naive, h, g, v, k, q, dhf, do)
    hf1, o1, gr1 = O.value_and_grads(O.chunk_gla, h, g, v, k, q, dhf, do, chunk_size=C)
    assert O.rel_l2(hf0, hf1) < TOL and O.rel_l2(o0, o1) < TOL
    for a, b in zip(gr0, gr1):
        assert O.rel_l2(a, b) < TOL


@pytest.mark.parametrize("shift", [5.0, 0.0])
def test_backward_formulas_match_autograd(shift):
    T, H, D, C = 128, 2, 32, 32
    h, g, v, k, q, dhf, do = _inputs(T, H, D, shift)
    _, _, gr0 = O.value_and_grads(O.recurrent_gla_naive, h, g, v, k, q, dhf, do)
    gr_rec = O.recurrent_gla_backward_formulas(h, g, v, k, q, dhf, do)
    gr_chunk = O.chunk_gla_backward_formulas(h, g, v, k, q, C, dhf, do)
    for a, b, c in zip(gr0, gr_rec, gr_chunk):
        assert O.rel_l2(a, b) < TOL
        assert O.rel_l2(a, c) < TOL


def test_reverse_is_time_flip():
    T, H, D = 64, 2, 16
    h, g, v, k, q, _, _ = _inputs(T, H, D, 5.0)
    hf_r, o_r = O.recurrent_gla_naive(h, g, v, k, q, reverse=True)
    fl = lambda x: torch.flip(x, [0])
    hf_f, o_f = O.recurrent_gla_naive(h, fl(g), fl(v), fl(k), fl(q))
    assert O.rel_l2(hf_f, hf_r) < TOL and O.rel_l2(fl(o_f), o_r) < TOL


def test_chaining_is_exact():
    """hidden_final of the first half fed as hidden_init of the second half equals one call
    (gla.py:720-723): the property sequence parallelism relies on."""
    T, H, D, C = 128, 2, 16, 32
    h, g, v, k, q, _, _ = _inputs(T, H, D, 0.0)
    hf, o = O.chunk_gla(h, g, v, k, q, C)
    h1, o1 = O.chunk_gla(h, g[:64], v[:64], k[:64], q[:64], C)
    h2, o2 = O.chunk_gla(h1, g[64:], v[64:], k[64:], q[64:], C)
    assert O.rel_l2(hf, h2) < TOL and O.rel_l2(o, torch.cat([o1, o2])) < TOL


def test_anchor_exponents_nonpositive():
    """Every exponent used by the dyadic score is <= 0 (the point of the secondary chunking,
    gla.py:986-993), so sharp gates cannot overflow."""
    C, D = 64, 8
    lam = torch.cumsum(torch.nn.functional.logsigmoid(torch.randn(C, D, dtype=torch.float64) - 3.0), 0)
    for h in O._levels(C):
        for s in range(0, C, 2 * h):
            m, e = s + h, s + 2 * h
            a = lam[m - 1:m]
            assert float((lam[m:e] - a).max()) <= 0 and float((a - lam[s:m]).max()) <= 0


def test_cumsum_and_rnn_scan():
    torch.manual_seed(1)
    x = torch.randn(3, 50, 7, dtype=torch.float64)
    init = torch.randn(3, 7, dtype=torch.float64)
    y = O.cumsum(x, 1, init=init, reverse=True, compute_dtype=torch.float64)
    ref = torch.flip(torch.cumsum(torch.flip(x, [1]), 1), [1]) + init[:, None]
    assert torch.allclose(y, ref)
    T, K, V = 20, 5, 4
    g = -torch.rand(T, K, dtype=torch.float64)
    kv = torch.randn(T, K, V, dtype=torch.float64)
    ig, ikv = -torch.rand(K, dtype=torch.float64), torch.randn(K, V, dtype=torch.float64)
    A, S = O.rnn_scan(g, kv, ig, ikv, compute_dtype=torch.float64)
    # brute force with the binary operator of ops.py:286-297
    a, b = ig.clone(), ikv.clone()
    for t in range(T):
        a, b = a + g[t], torch.exp(g[t])[:, None] * b + kv[t]
        assert torch.allclose(A[t], a) and torch.allclose(S[t], b)
    A2, S2 = O.rnn_scan(g, kv, reverse=True, compute_dtype=torch.float64)
    A3, S3 = O.rnn_scan(torch.flip(g, [0]), torch.flip(kv, [0]), compute_dtype=torch.float64)
    assert torch.allclose(A2, torch.flip(A3, [0])) and torch.allclose(S2, torch.flip(S3, [0]))


def test_bf16_faithful_emulation_within_tolerance():
    """Rounding at the reference's bf16 cast points keeps the forward within the 1e-2
    relative-L2 budget against the float64 truth (calibration of the bf16 tolerance)."""
    T, H, D, C = 256, 2, 64, 64
    h, g, v, k, q = O.make_inputs(1, T, H, D, torch.bfloat16, seed=3, batch_axis=False)
    hf0, o0 = O.recurrent_gla_naive(h, g, v, k, q)
    hf1, o1 = O.chunk_gla(h, g, v, k, q, C, compute_dtype=torch.float32, rnd=O.bf16_round)
    assert O.rel_l2(o0, o1) < 1e-2 and O.rel_l2(hf0.float(), hf1.float()) < 1e-2


def test_golden_fixtures():
    """The committed fixtures (tests/golden, written by tests/golden/make_golden.py from this
    oracle in float64) still reproduce: guards the oracle against silent edits."""
    from pathlib import Path
    gdir = Path(__file__).parent / "golden"
    files = sorted(gdir.glob("*.npz"))
    assert files, "no golden fixtures committed"
    for f in files:
        z = np.load(f)
        T, H, D, C = (int(z[n]) for n in ("T", "H", "D", "C"))
        h, g, v, k, q = O.make_inputs(1, T, H, D, torch.float32, seed=int(z["seed"]), shift=float(z["shift"]),
                                      batch_axis=False)
        dhf, do = torch.from_numpy(z["dhf"]), torch.from_numpy(z["dout"])
        hf, out, grads = O.value_and_grads(O.recurrent_gla_naive, h, g, v, k, q, dhf, do)
        assert O.rel_l2(torch.from_numpy(z["hidden_final"]).double(), hf) < 1e-6
        assert O.rel_l2(torch.from_numpy(z["out"]).double(), out) < 1e-6
        for name, gr in zip(("dhidden_init", "dlog_fgate", "dvalue", "dkey", "dquery"), grads):
            assert O.rel_l2(torch.from_numpy(z[name]).double(), gr) < 1e-6
