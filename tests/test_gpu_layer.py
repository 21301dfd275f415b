"""GPU parity tests (pytest -m gpu) for the GLA layer around the op and its two element-wise CUDA stages.

The reference ships the op only, so the layer is checked against its own definition written out
in float64 on the CPU, with the oracle's recurrence (gla.py:26-47) in the middle.  Tolerances
(relative L2): float32 1e-4 throughout; bfloat16 1e-2 for outputs and 2e-2 for gradients of the
element-wise stages, 2e-2 / 4e-2 for the whole layer (its library GEMMs round q, k, v, the gates
and the output to bfloat16 on top of the op's own rounding).
"""
import math

import pytest
import torch
import torch.nn.functional as F

from oracle import gla_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,n", [(torch.float32, 1000), (torch.bfloat16, 4096 * 33 + 7)])
def test_log_forget_gate_matches_definition(cuda_device, dtype, n):
    from gla_jax_b200 import log_forget_gate
    gen = torch.Generator().manual_seed(3)
    z0 = (4.0 * torch.randn(n, generator=gen)).to(dtype)
    dg = torch.randn(n, generator=gen)
    zr = z0.double().requires_grad_(True)
    ref = F.logsigmoid(zr) / 16.0
    (dz_ref,) = torch.autograd.grad((ref * dg.double()).sum(), zr)
    z = z0.to(cuda_device).requires_grad_(True)
    g = log_forget_gate(z, 16.0)
    assert g.dtype == torch.float32 and g.shape == z.shape
    (dz,) = torch.autograd.grad((g * dg.to(cuda_device)).sum(), z)
    assert dz.dtype == dtype
    assert O.rel_l2(ref.detach(), g.cpu()) < 1e-6
    assert O.rel_l2(dz_ref, dz.cpu()) < (1e-5 if dtype == torch.float32 else 5e-3)


def _headnorm_ref(x, gate, w, eps):
    n = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    return n * w * gate * torch.sigmoid(gate)


@pytest.mark.parametrize("rows_shape,D,dtype,with_weight", [
    ((3, 50, 2), 64, torch.float32, True),
    ((2, 300, 3), 128, torch.bfloat16, True),
    ((1, 77, 1), 256, torch.bfloat16, False),
    ((5, 9, 4), 32, torch.float32, True),
    ((4, 4096, 2), 128, torch.bfloat16, True),      # more rows than one pass of the grid
])
def test_headnorm_gate_matches_definition(cuda_device, rows_shape, D, dtype, with_weight):
    from gla_jax_b200 import headnorm_gate
    gen = torch.Generator().manual_seed(11)
    shape = (*rows_shape, D)
    x0 = torch.randn(shape, generator=gen).to(dtype)
    gate0 = (2.0 * torch.randn(shape, generator=gen)).to(dtype)
    w0 = (1.0 + 0.3 * torch.randn(D, generator=gen)) if with_weight else None
    dy0 = torch.randn(shape, generator=gen).to(dtype)
    xr, gr = x0.double().requires_grad_(True), gate0.double().requires_grad_(True)
    wr = w0.double().requires_grad_(True) if with_weight else torch.ones(D, dtype=torch.float64)
    yr = _headnorm_ref(xr, gr, wr, 1e-5)
    ref = torch.autograd.grad((yr * dy0.double()).sum(), [xr, gr] + ([wr] if with_weight else []))
    x, gate = x0.to(cuda_device).requires_grad_(True), gate0.to(cuda_device).requires_grad_(True)
    w = w0.to(cuda_device).requires_grad_(True) if with_weight else None
    y = headnorm_gate(x, gate, w, 1e-5)
    got = torch.autograd.grad((y.float() * dy0.to(cuda_device).float()).sum(), [x, gate] + ([w] if with_weight else []))
    tol_f, tol_g = (1e-5, 1e-4) if dtype == torch.float32 else (1e-2, 2e-2)
    assert y.dtype == dtype and O.rel_l2(yr.detach(), y.cpu()) < tol_f
    for name, a, b in zip(("dx", "dgate", "dweight"), ref, got):
        assert O.rel_l2(a, b.cpu()) < tol_g, (name, O.rel_l2(a, b.cpu()))
    # deterministic weight gradient: a second run gives the same bits
    if with_weight:
        again = torch.autograd.grad((headnorm_gate(x, gate, w, 1e-5).float() * dy0.to(cuda_device).float()).sum(), [w])
        assert torch.equal(again[0], got[2])


def _layer_ref(layer, x, hidden, dy, dhf):
    """The layer's definition in float64 on the CPU with the oracle's recurrence; returns y, hidden_final
    and the gradients w.r.t. x, hidden and every parameter (in named_parameters order)."""
    P = {n: p.detach().cpu().double().requires_grad_(True) for n, p in layer.named_parameters()}
    xr, hr = x.detach().cpu().double().requires_grad_(True), hidden.detach().cpu().double().requires_grad_(True)
    B, T, _ = xr.shape
    H, D = layer.num_heads, layer.head_dim
    q = (xr @ P["q_proj.weight"].T).view(B, T, H, D)
    k = (xr @ P["k_proj.weight"].T).view(B, T, H, D) / math.sqrt(D)
    v = (xr @ P["v_proj.weight"].T).view(B, T, H, D)
    z = (xr @ P["gate_down.weight"].T) @ P["gate_up.weight"].T + P["gate_up.bias"]
    g = F.logsigmoid(z).view(B, T, H, D) / layer.gate_normalizer
    hf, out = zip(*(O.recurrent_gla_naive(hr[b], g[b], v[b], k[b], q[b]) for b in range(B)))
    hf, out = torch.stack(hf), torch.stack(out)
    o = _headnorm_ref(out, (xr @ P["out_gate.weight"].T).view(B, T, H, D), P["norm_weight"], layer.eps)
    y = o.reshape(B, T, H * D) @ P["o_proj.weight"].T
    loss = (y * dy.cpu().double()).sum() + (hf * dhf.cpu().double()).sum()
    grads = torch.autograd.grad(loss, [xr, hr] + list(P.values()))
    return y.detach(), hf.detach(), grads


@pytest.mark.parametrize("d_model,H,D,T,chunk,dtype,mode", [
    (64, 2, 64, 128, 64, torch.float32, "chunk"),          # float32 CUDA-core chunk path
    (256, 2, 128, 256, 128, torch.bfloat16, "chunk"),      # tensor-core chunk path
    (64, 2, 32, 96, 32, torch.float32, "recurrent"),
])
def test_gla_layer_matches_its_definition(cuda_device, d_model, H, D, T, chunk, dtype, mode):
    from gla_jax_b200 import GLALayer
    torch.manual_seed(5)
    B = 2
    layer = GLALayer(d_model, H, head_dim=D, gate_low_rank=16, chunk_size=chunk, mode=mode, device=cuda_device,
                     dtype=dtype)
    with torch.no_grad():
        layer.gate_up.bias.add_(2.0)                      # gates near 1, as trained layers have them
        layer.norm_weight.add_(0.2 * torch.randn_like(layer.norm_weight))
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(B, T, d_model, generator=gen).to(dtype).to(cuda_device).requires_grad_(True)
    hidden = (0.5 * torch.randn(B, H, D, D, generator=gen)).to(dtype).to(cuda_device).requires_grad_(True)
    dy = torch.randn(B, T, d_model, generator=gen).to(dtype).to(cuda_device)
    dhf = torch.randn(B, H, D, D, generator=gen).to(dtype).to(cuda_device)
    y, hf = layer(x, hidden)
    assert y.shape == x.shape and y.dtype == dtype and tuple(hf.shape) == (B, H, D, D)
    params = list(layer.parameters())
    got = torch.autograd.grad((y.float() * dy.float()).sum() + (hf.float() * dhf.float()).sum(), [x, hidden] + params)
    y_ref, hf_ref, ref = _layer_ref(layer, x, hidden, dy, dhf)
    tol_f, tol_g = (1e-4, 2e-4) if dtype == torch.float32 else (2e-2, 4e-2)
    assert O.rel_l2(y_ref, y.detach().cpu()) < tol_f, O.rel_l2(y_ref, y.detach().cpu())
    assert O.rel_l2(hf_ref, hf.detach().cpu()) < tol_f
    names = ["x", "hidden"] + [n for n, _ in layer.named_parameters()]
    errs = {n: O.rel_l2(a, b.cpu()) for n, a, b in zip(names, ref, got)}
    bad = {n: e for n, e in errs.items() if not e < tol_g}
    assert not bad, f"gradients over tolerance: {bad} (all: {errs})"


def test_gla_layer_state_chains_across_calls(cuda_device):
    """Two calls on the halves of a sequence, the second starting from the first's state, equal one call."""
    from gla_jax_b200 import GLALayer
    torch.manual_seed(1)
    layer = GLALayer(256, 2, head_dim=128, chunk_size=128, device=cuda_device, dtype=torch.bfloat16)
    x = torch.randn(1, 512, 256, device=cuda_device).to(torch.bfloat16)
    with torch.no_grad():
        y, hf = layer(x)
        y1, h1 = layer(x[:, :256])
        y2, h2 = layer(x[:, 256:], h1)
    assert O.rel_l2(y.cpu(), torch.cat([y1, y2], 1).cpu()) < 1e-2 and O.rel_l2(hf.cpu(), h2.cpu()) < 1e-2
