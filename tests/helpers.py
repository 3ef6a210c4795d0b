"""Shared helpers for the test-suite: golden fixture loading and tolerances."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Output tolerances against the float32 run of `basic` on the same values.
TOL = {
    torch.bfloat16: dict(max_abs=2e-2, mean_abs=2e-3),
    torch.float16: dict(max_abs=2e-2, mean_abs=2e-3),
    torch.float32: dict(max_abs=1e-4, mean_abs=1e-5),
}


def load(name):
    return np.load(os.path.join(GOLDEN, name), allow_pickle=False)


def from_bf16_bits(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).float()


def attention_case(z, name):
    B, H, M, N, D, dec, nb, md = [int(x) for x in z[name + "_meta"]]
    return dict(q=from_bf16_bits(z[name + "_q"]), k=from_bf16_bits(z[name + "_k"]),
                v=from_bf16_bits(z[name + "_v"]), table=from_bf16_bits(z[name + "_table"]),
                out=torch.from_numpy(z[name + "_out"]), B=B, H=H, M=M, N=N, D=D,
                unidirectional=bool(dec), nb=nb, md=md)


def check_close(got, want, dtype, what=""):
    tol = TOL[dtype]
    diff = (got.float().cpu() - want.float().cpu()).abs()
    mx, mean = diff.max().item(), diff.mean().item()
    assert mx <= tol["max_abs"] and mean <= tol["mean_abs"], (
        f"{what}: max-abs {mx:.3e} (tol {tol['max_abs']:.0e}), mean-abs {mean:.3e} "
        f"(tol {tol['mean_abs']:.0e})")
    return mx, mean


def seeded(shape, seed, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype)
