"""gla_jax_b200 — B200-native (sm_100a) gated linear attention kernels behind the operator
API of zhixuan-lin/gla-jax (gla.py / ops.py).  All compute runs in libgla_b200.so (hand-written
CUDA behind a C ABI, include/gla_b200.h); importing this package never compiles anything and
there is no fallback if the library is absent."""
from .gla import chunk_gla, recurrent_gla, recurrent_gla_naive, auto_block_size, decode_step, chunk_gla_packed
from .layer import GLALayer, log_forget_gate, headnorm_gate
from ._lib import check_device
from .ops import cumsum_recursive, cumsum_pallas, rnn_recursive, rnn_pallas, binary_operator, triton_scan, scan

__all__ = ["chunk_gla", "recurrent_gla", "recurrent_gla_naive", "auto_block_size", "decode_step", "chunk_gla_packed", "cumsum_recursive",
           "cumsum_pallas", "rnn_recursive", "rnn_pallas", "binary_operator", "triton_scan", "scan",
           "GLALayer", "log_forget_gate", "headnorm_gate", "check_device"]
