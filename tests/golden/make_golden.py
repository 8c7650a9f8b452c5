"""Generates tests/golden/cfg1_golden.npz: the fp32 CPU oracle on benchmark
config 1 (B=1, S=32, N=64, H=4, D=32; q,k,v,bias,dO ~ N(0,1); Bernoulli(0.9)
additive mask with residue 0 forced valid; seed 1001).

The reference ships no golden vectors and cannot run here (its kernel needs
ThunderKittens headers and an sm_90a GPU; its test oracle is an absent Triton
kernel), so this fixture is produced by the oracle itself and pins it against
drift, not against the reference.

    python tests/golden/make_golden.py

Stored: dbias in full; o, dq, dk, dv for S rows {0, 13, 31}; and fp64
log-sum-exp for row 0 -- a few hundred KB.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import evo_ref  # noqa: E402

ROWS = [0, 13, 31]


def main():
    torch.set_num_threads(1)          # fixed summation order
    q, k, v, mask, bias, d_o = evo_ref.make_workload("cfg1_cpu_fp32")
    r = evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o, dtype=torch.float32)
    lse = evo_ref.evo_lse_ref(q, k, mask, bias, dtype=torch.float64)
    out = {n: r[n][:, ROWS].numpy() for n in ("o", "dq", "dk", "dv")}
    out["dbias"] = r["dbias"].numpy()
    out["lse_row0"] = lse[:, 0].numpy()
    out["rows"] = np.array(ROWS)
    # input checksums: pin the generator as well
    out["input_sums"] = np.array([t.double().sum().item() for t in (q, k, v, mask, bias, d_o)])
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cfg1_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path))


if __name__ == "__main__":
    main()
