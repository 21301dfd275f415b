"""The allocation-free forward entry point, gla_chunk_fwd_static, against gla_chunk_fwd.

Collected last on purpose (file name), so a run that stops at the first failure has already
run everything else.  The entry point serves callers that cannot allocate device memory where
they call the library (a custom call under a runtime that owns the allocator, a plugin in a
serving process with a closed memory pool): it takes its scratch from a fixed 32 MiB device
array inside the library instead of from the caller.  Checked here: same results as the
ordinary entry point on two calls in a row (the array is reused and keeps the first call's
contents), for both kernel families, and a clean refusal above the fixed size.
"""
import pytest
import torch

from oracle import gla_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 1e-2}     # forward tolerances of tests/test_gpu_ops.py


def _call_pair(lib, dev, B, T, H, D, C, dtype, seed):
    from gla_jax_b200 import _lib
    dt = _lib.GLA_BF16 if dtype == torch.bfloat16 else _lib.GLA_F32
    h, g, v, k, q = (x.to(dev) for x in O.make_inputs(B, T, H, D, dtype, seed=seed))
    stream = torch.cuda.current_stream(dev).cuda_stream
    # ordinary entry point, caller-provided workspace
    ws_n = lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, C, dt, 0)
    ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
    hf0, out0 = torch.empty_like(h), torch.empty_like(v)
    st = lib.gla_chunk_fwd(stream, B, T, H, D, C, dt, 0, h.data_ptr(), g.data_ptr(), v.data_ptr(), k.data_ptr(),
                           q.data_ptr(), hf0.data_ptr(), out0.data_ptr(), None, ws.data_ptr(), ws_n)
    assert st == 0, lib.gla_status_string(st)
    # the entry point under test: inputs and outputs only
    hf1, out1 = torch.empty_like(h), torch.empty_like(v)
    st = lib.gla_chunk_fwd_static(stream, B, T, H, D, C, dt, 0, h.data_ptr(), g.data_ptr(), v.data_ptr(), k.data_ptr(),
                                  q.data_ptr(), hf1.data_ptr(), out1.data_ptr())
    assert st == 0, lib.gla_status_string(st)
    torch.cuda.synchronize()
    return (hf0.cpu(), out0.cpu()), (hf1.cpu(), out1.cpu())


@pytest.mark.parametrize("B,T,H,D,C,dtype", [
    (1, 512, 2, 128, 128, torch.bfloat16),      # tensor-core kernels
    (1, 256, 2, 64, 64, torch.float32),         # fp32 kernels
])
def test_static_entry_matches_ordinary_entry_twice(cuda_device, B, T, H, D, C, dtype):
    from gla_jax_b200 import _lib
    lib = _lib.load()
    assert lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, C, _lib.GLA_BF16 if dtype == torch.bfloat16 else 0, 0) \
        <= lib.gla_chunk_fwd_static_max_bytes()
    # two calls in a row with different inputs: the second runs on the first's leftovers
    for seed in (41, 42):
        (hf0, out0), (hf1, out1) = _call_pair(lib, cuda_device, B, T, H, D, C, dtype, seed)
        assert O.rel_l2(hf0, hf1) < TOL[dtype], (seed, O.rel_l2(hf0, hf1))
        assert O.rel_l2(out0, out1) < TOL[dtype], (seed, O.rel_l2(out0, out1))
        # and against the oracle, so that both being wrong together cannot pass
        h, g, v, k, q = O.make_inputs(B, T, H, D, dtype, seed=seed)
        hf_ref, out_ref = O.recurrent_gla_naive(h[0], g[0], v[0], k[0], q[0])
        assert O.rel_l2(out_ref, out1[0]) < TOL[dtype]
        assert O.rel_l2(hf_ref.double(), hf1[0]) < TOL[dtype]


def test_static_entry_rejects_sizes_beyond_its_array(cuda_device):
    from gla_jax_b200 import _lib
    lib = _lib.load()
    B, T, H, D, C = 4, 4096, 6, 128, 128          # needs ~76 MB of scratch: over the 32 MiB array
    assert lib.gla_chunk_fwd_workspace_bytes(B, T, H, D, C, _lib.GLA_BF16, 0) > lib.gla_chunk_fwd_static_max_bytes()
    x = torch.zeros(16, device=cuda_device)
    p = x.data_ptr()
    st = lib.gla_chunk_fwd_static(None, B, T, H, D, C, _lib.GLA_BF16, 0, p, p, p, p, p, p, p)
    assert st == 8 and b"maximum" in lib.gla_status_string(st)        # GLA_ERR_TOO_LARGE, nothing launched
    # invalid sizes are reported as such, not as "too large"
    assert lib.gla_chunk_fwd_static(None, 1, 100, 2, 64, 64, 0, 0, p, p, p, p, p, p, p) == 2
