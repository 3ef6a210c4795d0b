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


TINY_T5 = dict(vocab_size=128, d_model=32, d_kv=64, num_heads=2, d_ff=64, num_layers=2, num_decoder_layers=2,
               relative_attention_num_buckets=32, relative_attention_max_distance=128)


def seed_named_parameters(model, seed=0):
    """Deterministic weights keyed by parameter name (the same names exist in the reference's
    T5ForConditionalGeneration and in turbot5_b200.t5), so both models get identical values
    without storing them."""
    import zlib
    with torch.no_grad():
        for name, p in model.named_parameters():
            g = torch.Generator().manual_seed((zlib.crc32(name.encode()) ^ seed) & 0x7fffffff)
            v = torch.randn(p.shape, generator=g)
            if name.endswith("layer_norm.weight"):
                v = 1.0 + 0.1 * v
            elif "relative_attention_bias" in name:
                v = 0.5 * v
            elif name in ("shared.weight",):
                v = 1.0 * v
            else:
                v = 0.08 * v
            p.copy_(v.to(p.dtype))
    return model


def tiny_t5_inputs():
    g = torch.Generator().manual_seed(123)
    ids = torch.randint(0, TINY_T5["vocab_size"], (2, 40), generator=g)
    dec = torch.randint(0, TINY_T5["vocab_size"], (2, 5), generator=g)
    return ids, dec


def check_grad_close(got, want, what="", rel=2e-2, floor=1e-6):
    """Gradients from 16-bit kernels against float32 autograd: the error of every element is
    bounded relative to the largest magnitude of the tensor (gradients span decades, and each
    is a sum of products of rounded factors), and the mean error by a tenth of that.  `floor`
    is the smallest magnitude taken as that scale: a bias-table gradient is a sum of thousands
    of terms of order 1e-2..1 that can cancel to exactly zero (all keys in one bucket)."""
    got, want = got.float().cpu(), want.float().cpu()
    scale = max(want.abs().max().item(), floor)
    diff = (got - want).abs()
    mx, mean = diff.max().item() / scale, diff.mean().item() / scale
    assert mx <= rel and mean <= rel / 10, f"{what}: max error {mx:.3e}, mean error {mean:.3e} of max |grad| {scale:.3e}"
    return mx, mean


def local_case(z, name):
    """q, k, v (B,H,L,D) of a block-local fixture (the module's projections are permutations)."""
    B, H, L, D, bl = [int(x) for x in z[name + "_meta"]]
    hidden = from_bf16_bits(z[name + "_hidden"])
    shape = lambda x: x.view(B, L, H, D).transpose(1, 2)
    q = shape(hidden)
    k = shape(hidden[..., torch.from_numpy(z[name + "_kperm"])])
    v = shape(hidden[..., torch.from_numpy(z[name + "_vperm"])])
    want = torch.from_numpy(z[name + "_out"]).view(B, L, H, D).transpose(1, 2)
    return q, k, v, from_bf16_bits(z[name + "_table"]), bl, want


def local_masked_case(z, name):
    """As `local_case`, plus the valid lengths of the right-padded batch."""
    q, k, v, table, bl, want = local_case(z, name)
    return q, k, v, table, bl, want, [int(x) for x in z[name + "_lens"]]
