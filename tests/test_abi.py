"""CPU checks of the drop-in boundary: the shared library builds, loads, and exports exactly
the entry points include/gla_b200.h declares; argument validation works without a GPU."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from gla_jax_b200 import build, _lib
    build.build()
    return _lib.load()


def _declared():
    text = (ROOT / "include" / "gla_b200.h").read_text()
    return sorted(set(re.findall(r"GLA_API\s+[\w\s\*]+?\b(gla_\w+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in gla_b200.h but not exported"


def test_python_signatures_cover_header():
    from gla_jax_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()


def test_status_strings(lib):
    assert lib.gla_status_string(0) == b"ok"
    for s in range(1, 9):
        assert len(lib.gla_status_string(s)) > 3
    assert b"sm_100a" in lib.gla_version()


def test_validation_without_gpu(lib):
    """Bad arguments are rejected before any launch, so these calls are safe on a CPU box."""
    p = ctypes.c_void_p(4096)
    # null pointer
    assert lib.gla_cumsum(None, 1, 8, 8, None, None, p, 0, 0, 0) == 1
    # T not a multiple of chunk / chunk not a power of two  (reference asserts gla.py:500,674)
    assert lib.gla_chunk_fwd(None, 1, 100, 2, 64, 64, 0, 0, p, p, p, p, p, p, p, None, p, 1 << 40) == 2
    assert lib.gla_chunk_fwd(None, 1, 96, 2, 64, 48, 0, 0, p, p, p, p, p, p, p, None, p, 1 << 40) == 2
    # unsupported head dim
    assert lib.gla_chunk_fwd(None, 1, 128, 2, 512, 64, 0, 0, p, p, p, p, p, p, p, None, p, 1 << 40) == 3
    # workspace too small
    assert lib.gla_chunk_fwd(None, 1, 128, 2, 64, 64, 0, 0, p, p, p, p, p, p, p, None, p, 16) == 5
    # misaligned pointer
    q = ctypes.c_void_p(4100)
    assert lib.gla_chunk_fwd(None, 1, 128, 2, 64, 64, 0, 0, q, p, p, p, p, p, p, None, p, 1 << 40) == 4
    # the tensor-core path (bf16, D = 128) stores rows with 32-byte vector stores: out must be 32-byte aligned
    o16 = ctypes.c_void_p(4096 + 16)
    assert lib.gla_chunk_fwd(None, 1, 128, 2, 128, 128, 1, 2, p, p, p, p, p, p, o16, None, p, 1 << 40) == 4
    assert lib.gla_chunk_bwd(None, 1, 128, 2, 128, 128, 1, 2, p, p, p, p, p, p, p, p, p, o16, p, p, p, 1 << 40) == 4
    # packed sequences: only the tensor-core shapes; bad sequence count
    assert lib.gla_chunk_fwd_packed(None, 256, 2, 64, 64, 1, 2, p, p, p, p, p, p, p, p, None, p, 1 << 40) == 3
    assert lib.gla_chunk_fwd_packed(None, 256, 2, 128, 128, 1, 0, p, p, p, p, p, p, p, p, None, p, 1 << 40) == 2
    # decode step: null pointer, bad dims
    assert lib.gla_decode_step(None, 1, 1, 64, 0, None, p, p, p, p, p, 0) == 1
    assert lib.gla_decode_step(None, 0, 1, 64, 0, p, p, p, p, p, p, 0) == 2
    # layer stages: null pointer, bad element count, unsupported row width, misaligned rows, missing workspace
    assert lib.gla_layer_gate_fwd(None, 8, 1, None, 1.0, p) == 1
    assert lib.gla_layer_gate_bwd(None, 0, 1, p, p, 1.0, p) == 2
    assert lib.gla_layer_headnorm_gate_fwd(None, 4, 48, 1, p, p, None, 1e-5, p, p) == 3
    assert lib.gla_layer_headnorm_gate_fwd(None, 4, 64, 1, q, p, None, 1e-5, p, p) == 4
    assert lib.gla_layer_headnorm_gate_bwd(None, 4, 64, 1, p, p, p, p, p, p, p, p, None, 0) == 5
    assert lib.gla_layer_headnorm_gate_bwd_workspace_bytes(4, 64) > 0
    # workspace sizes are positive and grow with the problem
    a = lib.gla_chunk_fwd_workspace_bytes(1, 128, 2, 64, 64, 0, 0)
    b = lib.gla_chunk_fwd_workspace_bytes(2, 128, 2, 64, 64, 0, 0)
    assert 0 < a < b
    assert lib.gla_chunk_saved_bytes(1, 128, 2, 64, 64, 0, 0) > 0
    assert lib.gla_chunk_fwd_workspace_bytes(1, 100, 2, 64, 64, 0, 0) == 0


def test_cpu_tensors_raise():
    import torch
    from gla_jax_b200 import chunk_gla
    h = torch.zeros(2, 16, 16)
    x = torch.zeros(32, 2, 16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        chunk_gla(h, x, x, x, x, 16)
    from gla_jax_b200 import headnorm_gate, log_forget_gate
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        log_forget_gate(torch.zeros(4))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        headnorm_gate(torch.zeros(2, 32), torch.zeros(2, 32))
