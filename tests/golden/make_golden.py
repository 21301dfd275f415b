"""Writes the golden fixtures of tests/golden from the float64 oracle.

    python tests/golden/make_golden.py

The reference cannot run where this repository is built (it needs jax==0.4.29 with
Pallas/Triton), so the fixtures come from the oracle's restatement of its definitional
recurrence (gla.py:26-47) with autograd gradients, stored as float32.  Inputs are not stored:
they are regenerated from (seed, shift) by oracle.gla_oracle.make_inputs in float32.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import gla_oracle as O  # noqa: E402

CASES = {
    # name: T, H, D, C, seed, shift
    "cfg1_T256_H2_D64": (256, 2, 64, 64, 0, 5.0),
    "sharp_T128_H2_D32": (128, 2, 32, 32, 7, 0.0),
    "onechunk_T64_H1_D64": (64, 1, 64, 64, 11, 5.0),
}

if __name__ == "__main__":
    out_dir = Path(__file__).parent
    for name, (T, H, D, C, seed, shift) in CASES.items():
        h, g, v, k, q = O.make_inputs(1, T, H, D, torch.float32, seed=seed, shift=shift, batch_axis=False)
        gen = torch.Generator().manual_seed(seed + 100)
        dhf = torch.randn(H, D, D, generator=gen)
        do = torch.randn(T, H, D, generator=gen)
        hf, out, grads = O.value_and_grads(O.recurrent_gla_naive, h, g, v, k, q, dhf, do)
        np.savez_compressed(out_dir / f"{name}.npz", T=T, H=H, D=D, C=C, seed=seed, shift=shift,
                            dhf=dhf.numpy(), dout=do.numpy(),
                            hidden_final=hf.float().numpy(), out=out.float().numpy(),
                            dhidden_init=grads[0].float().numpy(), dlog_fgate=grads[1].float().numpy(),
                            dvalue=grads[2].float().numpy(), dkey=grads[3].float().numpy(),
                            dquery=grads[4].float().numpy())
        print("wrote", name)
