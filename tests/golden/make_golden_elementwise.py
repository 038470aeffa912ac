"""Golden vectors for the fused element-wise operators, made by RUNNING THE REFERENCE's plain
arithmetic (`_pt_complex_norm`, `_pt_mod_swish`, `_pt_mod_relu`, `_pt_cgu_gate` in
v11/triton_kernels.py) and torch autograd through it, in float64 on seeded inputs.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_elementwise.py /path/to/qllm2
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: python " + sys.argv[0] + " /path/to/qllm2   (a checkout of the reference)")
REF = sys.argv[1]
sys.path.insert(0, REF)
sys.dont_write_bytecode = True

from v11 import triton_kernels as tk  # noqa: E402

tk.set_triton_enabled(False)


def leaf(*shape, gen, scale=1.0, shift=0.0):
    return (torch.randn(*shape, generator=gen, dtype=torch.float64) * scale + shift).requires_grad_(True)


def main():
    gen = torch.Generator().manual_seed(0)
    out = {}
    # two widths: 40 channels (one partly filled vector per lane) and 776 (beyond one 128-channel sweep)
    for tag, (rows, C) in {"a": ((3, 5), 40), "b": ((1, 3), 776)}.items():
        z = leaf(*rows, C, 2, gen=gen)
        with torch.no_grad():
            z[0, 0, :4] *= 1e-3            # small magnitudes exercise the 1e-8 guards
        dout = torch.randn(*rows, C, 2, generator=gen, dtype=torch.float64)
        scale = leaf(C, gen=gen, scale=0.3, shift=1.0)
        bias = leaf(C, gen=gen, scale=0.5)
        beta = leaf(C, gen=gen, scale=0.3, shift=1.0)
        up = leaf(*rows, C, 2, gen=gen)
        cases = {
            "norm": (lambda: tk._pt_complex_norm(z, scale, 1e-6), [z, scale]),
            "swish": (lambda: tk._pt_mod_swish(z, bias, beta), [z, bias, beta]),
            "relu": (lambda: tk._pt_mod_relu(z, bias), [z, bias]),
            "gate": (lambda: tk._pt_cgu_gate(z, up), [z, up]),
        }
        for name, (fn, wrt) in cases.items():
            y = fn()
            grads = torch.autograd.grad((y * dout).sum(), wrt)
            out[f"{tag}_{name}_out"] = y.detach().numpy()
            for i, g in enumerate(grads):
                out[f"{tag}_{name}_grad{i}"] = g.numpy()
        for k_, v_ in dict(z=z, dout=dout, scale=scale, bias=bias, beta=beta, up=up).items():
            out[f"{tag}_{k_}"] = v_.detach().numpy()
    path = os.path.join(HERE, "elementwise.npz")
    np.savez_compressed(path, **{k: v.astype(np.float32) for k, v in out.items()})
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
