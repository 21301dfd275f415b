"""CPU checks of host-side logic that needs no GPU: option names of the `impl` argument, the scan rules recognised from
Python callables, size functions of the C ABI, and the table of DRAM traffic that bench.py reads from profiles/."""
import importlib.util
import operator
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from gla_jax_b200 import build, _lib
    build.build()
    return _lib.load()


def test_impl_names_carry_option_bits():
    from gla_jax_b200 import _lib
    base = _lib.IMPL_BY_NAME["tcgen05"]
    assert _lib.IMPL_BY_NAME["tcgen05+all_scales"] == base | 0x800
    assert _lib.IMPL_BY_NAME["auto+segments+no_l2_prefetch"] == _lib.IMPL_AUTO | 0x2000 | 0x1000
    assert _lib.IMPL_BY_NAME["tcgen05+one_pass+no_early_start"] == base | 0x200 | 0x400
    for bad in ("tcgen05+nonsense", "nonsense", "auto+"):
        with pytest.raises(KeyError):
            _lib.IMPL_BY_NAME[bad]


def test_scan_rules_from_callables():
    from gla_jax_b200 import ops
    assert ops._scan_rule(torch.add) == "add" and ops._scan_rule(operator.add) == "add" and ops._scan_rule("add") == "add"
    assert ops._scan_rule(torch.mul) == "mul" and ops._scan_rule(torch.maximum) == "max" and ops._scan_rule(torch.minimum) == "min"
    assert ops._scan_rule(torch.logaddexp) == "logaddexp"
    assert ops._scan_rule(torch.sub) is None and ops._scan_rule("xor") is None
    # the two-array rule of the linear RNN (ops.py:286-297) is recognised by identity
    a, b = (torch.tensor([-0.5]), torch.tensor([[1.0]])), (torch.tensor([-0.25]), torch.tensor([[2.0]]))
    A, S = ops.binary_operator(a, b)
    assert torch.allclose(A, torch.tensor([-0.75])) and torch.allclose(S, torch.exp(torch.tensor([-0.25])) * 1.0 + 2.0)


def test_size_functions_without_a_gpu(lib):
    # the long-axis form of the linear-RNN scan asks for scratch only where the plain walk has too few threads
    assert lib.gla_rnn_scan_workspace_bytes(1, 4096, 128, 128) > 0
    assert lib.gla_rnn_scan_workspace_bytes(64, 4096, 128, 128) == 0      # enough rows
    assert lib.gla_rnn_scan_workspace_bytes(1, 256, 128, 128) == 0        # short axis
    assert lib.gla_rnn_scan_workspace_bytes(0, 4096, 128, 128) == 0
    from gla_jax_b200 import _lib
    dt, impl = _lib.GLA_BF16, _lib.IMPL_BY_NAME["tcgen05"]
    small = lib.gla_chunk_fwd_workspace_bytes(1, 1024, 2, 128, 128, dt, impl)
    big = lib.gla_chunk_fwd_workspace_bytes(2, 1024, 2, 128, 128, dt, impl)
    assert 0 < small < big and big == 2 * small                            # linear in the batch
    assert lib.gla_chunk_saved_bytes(1, 1024, 2, 128, 128, dt, impl) == 8 * 2 * (128 * 128 * 2 + 128 * 4 + 128 * 128 * 2)
    assert lib.gla_chunk_fwd_static_max_bytes() == 32 << 20


def test_bench_reads_the_traffic_table():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    t = bench.load_ncu_traffic()
    assert set(t) == {"tc_chunk_bwd_kernel", "tc_chunk_fwd_kernel", "tc_state_kernel", "tc_dstate_scan_kernel"}
    total = sum(t.values())
    assert 4.2e8 < total < 1.0e9          # at least the compulsory 427.8 MB of a step, and a sane upper bound
    assert max(t, key=t.get) == "tc_chunk_bwd_kernel"
