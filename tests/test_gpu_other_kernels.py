"""RMSNorm, split-KV decoding, unpad/pad kernels and the module glue against the oracle."""
import numpy as np
import pytest
import torch

from oracle import t5_oracle as orc
from tests.helpers import attention_case, check_close, load, seeded

pytestmark = pytest.mark.gpu


def _ops():
    import turbot5_b200 as t5b
    return t5b


# ------------------------------------------------------------------ RMSNorm
def _ulp_close(got, want, dtype):
    """Equal up to rounding flips: the reference rounds twice in the weight's type (normalised
    value, then product), so a last-bit difference in rsqrt can move a result by one unit in
    the last place (rarely two, when both roundings flip)."""
    got, want = got.float().cpu(), want.float()
    if dtype == torch.float32:
        assert (got - want).abs().max().item() <= 2e-6 * max(1.0, want.abs().max().item())
        return
    bits = 8 if dtype == torch.bfloat16 else 11
    ulp = torch.pow(2.0, torch.floor(torch.log2(want.abs().clamp_min(1e-30))) - (bits - 1))
    err = (got - want).abs()
    assert not (err > ulp * 2.001).any(), "an element differs by more than two ulp"
    frac2 = (err > ulp * 1.001).float().mean().item()
    assert frac2 < 1e-4, f"{frac2:.3%} of elements differ by two ulp"
    frac = (err != 0).float().mean().item()
    assert frac < 0.02, f"{frac:.3%} of elements differ"


@pytest.mark.parametrize("tag,xdt,wdt", [("f32", torch.float32, torch.float32),
                                          ("bf16", torch.bfloat16, torch.bfloat16),
                                          ("bf16_wf32", torch.bfloat16, torch.float32),
                                          ("f16", torch.float16, torch.float16)])
def test_rmsnorm_golden(tag, xdt, wdt):
    t5b = _ops()
    z = load("rmsnorm.npz")
    x = torch.from_numpy(z[tag + "_x"]).to(xdt)
    w = torch.from_numpy(z[tag + "_w"]).to(wdt)
    y = t5b.rms_layer_norm(x.cuda(), w.cuda(), 1e-6)
    assert str(y.dtype) == str(z[tag + "_ydtype"])
    _ulp_close(y, torch.from_numpy(z[tag + "_y"]), y.dtype)


@pytest.mark.parametrize("rows,d,dt", [(16384, 768, torch.bfloat16), (64, 1024, torch.bfloat16),
                                        (100, 512, torch.float32), (7, 100, torch.bfloat16),
                                        (5, 8192, torch.bfloat16), (3, 4100, torch.float32)])
def test_rmsnorm_vs_oracle(rows, d, dt):
    t5b = _ops()
    x = (-2.3 + 0.5 * seeded((rows, d), 1)).to(dt)
    w = torch.rand((d,), generator=torch.Generator().manual_seed(2)).to(dt)
    y, rstd = t5b.rms_layer_norm(x.cuda(), w.cuda(), 1e-6, return_rstd=True)
    _ulp_close(y, orc.t5_layer_norm(x, w, 1e-6), dt)
    want_rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    assert (rstd.cpu() - want_rstd).abs().max().item() < 1e-5 * want_rstd.max().item()


def test_rmsnorm_module_and_3d_input():
    t5b = _ops()
    norm = t5b.T5LayerNorm(768, eps=1e-6).cuda().to(torch.bfloat16)
    with torch.no_grad():
        norm.weight.copy_(torch.rand(768))
    x = seeded((2, 33, 768), 3, dtype=torch.bfloat16)
    y = norm(x.cuda())
    assert y.shape == x.shape
    _ulp_close(y, orc.t5_layer_norm(x, norm.weight.detach().cpu(), 1e-6), torch.bfloat16)


# ------------------------------------------------------------------ decoding
@pytest.mark.parametrize("B,H,M,N,D,causal,dt", [
    (2, 4, 1, 1000, 64, False, torch.bfloat16),     # cross attention step, no bias
    (2, 4, 1, 129, 64, True, torch.bfloat16),       # self attention step with unidirectional bias
    (1, 2, 3, 700, 64, True, torch.bfloat16),       # short multi-token step
    (1, 2, 6, 300, 64, True, torch.bfloat16),
    (2, 2, 1, 513, 128, True, torch.bfloat16),
    (2, 2, 1, 513, 32, True, torch.float16),
    (1, 2, 1, 400, 64, True, torch.float32),
    (1, 1, 1, 1, 64, True, torch.bfloat16),
    (4, 16, 1, 8192, 64, False, torch.bfloat16),    # long cache, several splits
])
@pytest.mark.parametrize("splits", [0, 1, 5])
def test_decode_vs_oracle(B, H, M, N, D, causal, dt, splits):
    t5b = _ops()
    q, k, v = seeded((B, H, M, D), 1, dtype=dt), seeded((B, H, N, D), 2, dtype=dt), seeded((B, H, N, D), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt) if causal else None
    want = orc.attention_basic(q, k, v, table, causal=causal)
    out = t5b.flash_decoding_with_fusing_bias(q.cuda(), k.cuda(), v.cuda(), None if table is None else table.cuda(),
                                              causal=causal, sm_scale=1.0, num_splits=splits)
    check_close(out, want, dt)
    # second call on the same scratch buffer: counters were left at zero
    out2 = t5b.flash_decoding_with_fusing_bias(q.cuda(), k.cuda(), v.cuda(), None if table is None else table.cuda(),
                                               causal=causal, sm_scale=1.0, num_splits=splits)
    assert torch.equal(out, out2)


def test_decode_cache_capacity_and_per_row_lengths():
    t5b = _ops()
    dt = torch.bfloat16
    B, H, cap = 3, 2, 640
    lens = [640, 100, 333]
    q, k, v = seeded((B, H, 1, 64), 1, dtype=dt), seeded((B, H, cap, 64), 2, dtype=dt), seeded((B, H, cap, 64), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    # poison the unused tail of the cache: it must never be read into the result
    kc, vc = k.clone(), v.clone()
    for b, n in enumerate(lens):
        kc[b, :, n:] = float("nan"); vc[b, :, n:] = float("nan")
    out = t5b.flash_decoding_with_fusing_bias(q.cuda(), kc.cuda(), vc.cuda(), table.cuda(), causal=True, sm_scale=1.0,
                                              seqlens_k=torch.tensor(lens, dtype=torch.int32).cuda(), num_splits=3)
    for b, n in enumerate(lens):
        want = orc.attention_basic(q[b:b + 1], k[b:b + 1, :, :n], v[b:b + 1, :, :n], table, causal=True)
        check_close(out[b:b + 1], want, dt, f"row {b}")
    out = t5b.flash_decoding_with_fusing_bias(q.cuda(), kc.cuda(), vc.cuda(), table.cuda(), causal=True, sm_scale=1.0,
                                              kv_len=100)
    want = orc.attention_basic(q, k[:, :, :100], v[:, :, :100], table, causal=True)
    check_close(out, want, dt)


def test_decode_golden_step():
    t5b = _ops()
    c = attention_case(load("attention.npz"), "dec_step")
    dt = torch.bfloat16
    out = t5b.flash_decoding_with_fusing_bias(c["q"].to(dt).cuda(), c["k"].to(dt).cuda(), c["v"].to(dt).cuda(),
                                              c["table"].to(dt).cuda(), causal=True, sm_scale=1.0)
    check_close(out, c["out"], dt)


def test_decode_workspace_errors():
    t5b = _ops()
    dt = torch.bfloat16
    q, k = torch.zeros((1, 2, 1, 64), dtype=dt, device="cuda"), torch.zeros((1, 2, 600, 64), dtype=dt, device="cuda")
    small = torch.zeros(256, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="workspace"):
        t5b.flash_decoding_with_fusing_bias(q, k, k, None, sm_scale=1.0, num_splits=4, workspace=small)


# ------------------------------------------------------------------ unpad / pad
def test_unpad_plan_matches_reference_fixture():
    t5b = _ops()
    z = load("padding.npz")
    mask = torch.from_numpy(z["mask"]).cuda()
    plan = t5b.get_unpad_plan(mask)
    assert torch.equal(plan.cu_seqlens.cpu(), torch.from_numpy(z["cu_seqlens"]))
    dest = plan.dest.cpu()
    kept = torch.nonzero(dest >= 0).flatten()
    assert torch.equal(kept, torch.from_numpy(z["indices"]))
    assert torch.equal(dest[kept], torch.arange(kept.numel(), dtype=torch.int32))
    vals = torch.from_numpy(z["values"]).cuda()                     # (total, 2, 4) float32 = 32-byte rows
    padded = t5b.pad_rows(vals, plan)
    assert torch.equal(padded.cpu(), torch.from_numpy(z["padded"]))
    back = t5b.unpad_rows(padded, plan)
    assert torch.equal(back[:vals.shape[0]].cpu(), vals.cpu())


@pytest.mark.parametrize("mdt", [torch.bool, torch.int64, torch.int32, torch.uint8, torch.float32])
def test_unpad_plan_ragged_and_holes(mdt):
    t5b = _ops()
    g = torch.Generator().manual_seed(5)
    mask = (torch.rand((7, 1000), generator=g) > 0.3)
    mask[2] = False
    mask[4] = True
    idx, cu, mx = orc.get_unpad_data(mask.to(torch.int64))
    plan = t5b.get_unpad_plan(mask.to(mdt).cuda())
    assert torch.equal(plan.cu_seqlens.cpu(), cu)
    assert torch.equal(torch.nonzero(plan.dest.cpu() >= 0).flatten(), idx)
    x = seeded((7, 1000, 2, 8), 6, dtype=torch.bfloat16)
    packed = t5b.unpad_rows(x.cuda(), plan)
    assert torch.equal(packed[:idx.numel()].cpu(), x.reshape(7000, 2, 8)[idx])
    padded = t5b.pad_rows(packed, plan)
    assert torch.equal(padded.cpu(), orc.pad_rows(x.reshape(7000, 2, 8)[idx], idx, 7, 1000))
    assert torch.count_nonzero(packed[idx.numel():]) == 0          # unused tail is defined (zero)


# ------------------------------------------------------------------ module glue
class _Cfg:
    def __init__(self, **kw):
        self.is_decoder = False
        self.relative_attention_num_buckets = 32
        self.relative_attention_max_distance = 128
        self.d_model = 128
        self.d_kv = 64
        self.num_heads = 4
        self.dropout_rate = 0.0
        self.__dict__.update(kw)


def _make_module(cfg, dt, seed, cross=False, bias=True):
    t5b = _ops()
    mod = t5b.T5ATTENTION_TYPES["flash"](cfg, cross_attention=cross, has_relative_attention_bias=bias)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for lin in (mod.q, mod.k, mod.v, mod.o):
            lin.weight.copy_(torch.randn(lin.weight.shape, generator=g) * 0.05)
        if bias:
            mod.relative_attention_bias.weight.copy_(torch.randn((32, cfg.num_heads), generator=g) * 0.1)
    return mod.cuda().to(dt).eval()


def _oracle_layer(mod, hidden, **kw):
    f = lambda p: p.detach().float().cpu()
    table = f(mod.relative_attention_bias.weight) if mod.has_relative_attention_bias else None
    return orc.t5_attention_layer(hidden.float(), f(mod.q.weight), f(mod.k.weight), f(mod.v.weight),
                                  f(mod.o.weight), table, mod.n_heads, mod.key_value_proj_dim, **kw)


def test_module_small_fixture_fp32():
    t5b = _ops()
    z = load("layer.npz")
    cfg = _Cfg(d_model=128, d_kv=32, num_heads=4)
    mod = t5b.T5FlashAttention(cfg, has_relative_attention_bias=True)
    t = lambda k: torch.from_numpy(z[k])
    with torch.no_grad():
        mod.q.weight.copy_(t("small_wq")); mod.k.weight.copy_(t("small_wk")); mod.v.weight.copy_(t("small_wv"))
        mod.o.weight.copy_(t("small_wo")); mod.relative_attention_bias.weight.copy_(t("small_table"))
    mod = mod.cuda().eval()
    with torch.no_grad():
        out, present, pb = mod(t("small_hidden").cuda())
    assert present is None and pb is mod.relative_attention_bias.weight
    assert (out.cpu() - t("small_out")).abs().max().item() < 1e-4


def test_module_encoder_bf16_and_padding_mask():
    dt = torch.bfloat16
    cfg = _Cfg()
    mod = _make_module(cfg, dt, 1)
    hidden = seeded((3, 200, 128), 2, dtype=dt)
    with torch.no_grad():
        out = mod(hidden.cuda())[0]
    want, _ = _oracle_layer(mod, hidden)
    check_close(out, want, dt, "no mask")
    lens = [200, 37, 129]
    mask = torch.zeros((3, 200), dtype=torch.int64)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    with torch.no_grad():
        out = mod(hidden.cuda(), mask=mask.cuda())[0]
    want, _ = _oracle_layer(mod, hidden, key_padding_mask=mask)
    for b, n in enumerate(lens):
        check_close(out[b, :n], want[b, :n], dt, f"masked batch row {b}")
        assert torch.count_nonzero(out[b, n:]) == 0       # padded rows come back as zeros


def test_module_decoder_prefill_step_and_cross():
    dt = torch.bfloat16
    cfg = _Cfg(is_decoder=True)
    self_att = _make_module(cfg, dt, 3)
    cross = _make_module(cfg, dt, 4, cross=True, bias=False)
    hidden = seeded((2, 40, 128), 5, dtype=dt)
    enc = seeded((2, 300, 128), 6, dtype=dt)
    with torch.no_grad():
        out, present, _ = self_att(hidden.cuda(), use_cache=True)
    want, (wk, wv) = _oracle_layer(self_att, hidden, is_decoder=True)
    check_close(out, want, dt, "decoder prefill")
    check_close(present[0], wk, dt); check_close(present[1], wv, dt)
    # one cached decoding step
    step = seeded((2, 1, 128), 7, dtype=dt)
    with torch.no_grad():
        out1, present1, _ = self_att(step.cuda(), past_key_value=present, use_cache=True)
    want1, _ = _oracle_layer(self_att, step, is_decoder=True, past_key_value=(wk, wv))
    check_close(out1, want1, dt, "decoder step")
    assert present1[0].shape[2] == 41
    # cross attention, with and without an encoder padding mask
    with torch.no_grad():
        outc, pc, _ = cross(hidden.cuda(), key_value_states=enc.cuda(), use_cache=True)
    wantc, _ = _oracle_layer(cross, hidden, is_decoder=True, key_value_states=enc.float())
    check_close(outc, wantc, dt, "cross")
    with torch.no_grad():
        outs = cross(step.cuda(), key_value_states=enc.cuda(), past_key_value=pc)[0]
    wants, _ = _oracle_layer(cross, step, is_decoder=True, key_value_states=enc.float())
    check_close(outs, wants, dt, "cross step")
    mask = torch.ones((2, 300), dtype=torch.int64); mask[1, 120:] = 0
    with torch.no_grad():
        outm = cross(hidden.cuda(), key_value_states=enc.cuda(), mask=mask.cuda())[0]
    wantm, _ = _oracle_layer(cross, hidden, is_decoder=True, key_value_states=enc.float(), key_padding_mask=mask)
    check_close(outm, wantm, dt, "cross masked")


def test_state_dict_keys_match_hf_t5_names():
    t5b = _ops()
    mod = t5b.T5FlashAttention(_Cfg(), has_relative_attention_bias=True)
    assert set(mod.state_dict().keys()) == {"q.weight", "k.weight", "v.weight", "o.weight",
                                            "relative_attention_bias.weight"}
    assert set(t5b.T5LayerNorm(8).state_dict().keys()) == {"weight"}


def test_config5_decode_full_size_spot_heads():
    # T5-large decoding shape: batch 64, 16 heads, encoder memory 8192 (cross attention,
    # no bias) and a 128-token self-attention cache with unidirectional bias
    t5b = _ops()
    dt = torch.bfloat16
    B, H, N = 64, 16, 8192
    g = torch.Generator(device="cuda").manual_seed(0)
    k = torch.randn((B, H, N, 64), generator=g, device="cuda", dtype=torch.float32).to(dt)
    v = torch.randn((B, H, N, 64), generator=g, device="cuda", dtype=torch.float32).to(dt)
    q = torch.randn((B, H, 1, 64), generator=g, device="cuda", dtype=torch.float32).to(dt)
    out = t5b.flash_decoding_with_fusing_bias(q, k, v, None, causal=False, sm_scale=1.0)
    for b, h in ((0, 0), (17, 5), (63, 15)):
        want = orc.attention_basic(q[b:b + 1, h:h + 1].cpu(), k[b:b + 1, h:h + 1].cpu(), v[b:b + 1, h:h + 1].cpu(), None)
        check_close(out[b:b + 1, h:h + 1], want, dt, f"cross (b,h)=({b},{h})")
    table = (torch.randn((32, H), generator=g, device="cuda") * 0.1).to(dt)
    ks, vs = k[:, :, :128].contiguous(), v[:, :, :128].contiguous()
    for t_step in (1, 77, 128):
        out = t5b.flash_decoding_with_fusing_bias(q, ks, vs, table, causal=True, sm_scale=1.0, kv_len=t_step)
        want = orc.attention_basic(q[:3].cpu(), ks[:3, :, :t_step].cpu(), vs[:3, :, :t_step].cpu(), table.cpu(), causal=True)
        check_close(out[:3], want, dt, f"self step {t_step}")


@pytest.mark.parametrize("xdt,wdt", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32),
                                     (torch.bfloat16, torch.float32), (torch.float16, torch.float16)])
@pytest.mark.parametrize("rows,d", [(37, 768), (300, 512), (5, 1000)])
def test_rmsnorm_backward_vs_oracle_autograd(rows, d, xdt, wdt):
    import turbot5_b200 as t5b
    from tests.helpers import check_grad_close
    x = seeded((rows, d), 1, dtype=xdt)
    w = (1.0 + 0.2 * seeded((d,), 2)).to(wdt)
    xf, wf = x.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    # the same function on float32 copies under autograd; the reference's two roundings do not
    # change the derivative it propagates (the casts pass gradients through)
    y_ref = orc.t5_layer_norm(xf, wf)
    dy = seeded((rows, d), 3, dtype=y_ref.dtype)
    (y_ref * dy).sum().backward()
    xc, wc = x.detach().cuda().requires_grad_(True), w.detach().cuda().requires_grad_(True)
    y = t5b.rms_layer_norm(xc, wc, 1e-6)
    y.backward(dy.cuda().to(y.dtype))
    torch.cuda.synchronize()
    check_grad_close(xc.grad, xf.grad, "dx", rel=1e-4 if xdt == torch.float32 else 2e-2)
    check_grad_close(wc.grad, wf.grad, "dw", rel=1e-4 if (xdt == torch.float32 and wdt == torch.float32) else 2e-2)


def test_module_training_step_gradients_vs_oracle_layer():
    # one attention layer, encoder (with a padding mask: the packed-sequence kernels) and decoder
    # self-attention: gradients of every weight and of the input against the oracle layer under autograd
    from tests.helpers import check_grad_close
    dt = torch.bfloat16
    for is_decoder, mask_lens in ((False, None), (False, [200, 37, 129]), (True, None)):
        cfg = _Cfg(is_decoder=is_decoder)
        mod = _make_module(cfg, dt, 11).train()
        hidden = seeded((3, 200, 128), 12, dtype=dt)
        dout = seeded((3, 200, 128), 13, dtype=dt)
        mask = None
        if mask_lens is not None:
            mask = torch.zeros((3, 200), dtype=torch.int64)
            for b, n in enumerate(mask_lens):
                mask[b, :n] = 1
            dout = dout * mask[:, :, None].to(dt)        # padded rows carry no loss
        hc = hidden.cuda().requires_grad_(True)
        out = mod(hc, mask=None if mask is None else mask.cuda())[0]
        out.backward(dout.cuda())
        torch.cuda.synchronize()
        # oracle: float32 copies of the same parameters under autograd
        names = ["q", "k", "v", "o"]
        ws = {n: getattr(mod, n).weight.detach().float().cpu().requires_grad_(True) for n in names}
        table = mod.relative_attention_bias.weight.detach().float().cpu().requires_grad_(True)
        hf = hidden.float().requires_grad_(True)
        want, _ = orc.t5_attention_layer(hf, ws["q"], ws["k"], ws["v"], ws["o"], table, mod.n_heads,
                                         mod.key_value_proj_dim, is_decoder=is_decoder, key_padding_mask=mask)
        (want * dout.float()).sum().backward()
        tag = f"decoder={is_decoder} mask={mask_lens}"
        for n in names:
            check_grad_close(getattr(mod, n).weight.grad, ws[n].grad, f"{tag} d{n}.weight", rel=3e-2)
        check_grad_close(mod.relative_attention_bias.weight.grad, table.grad, f"{tag} dtable", rel=3e-2, floor=1.0)
        if mask is None:
            check_grad_close(hc.grad, hf.grad, f"{tag} dhidden", rel=3e-2)
        else:
            for b, n in enumerate(mask_lens):
                check_grad_close(hc.grad[b, :n], hf.grad[b, :n], f"{tag} dhidden row {b}", rel=3e-2)


def test_local_attention_module_matches_reference_module_fixture():
    # T5LocalFlashAttention with the fixture's permutation projections against the output of the
    # reference's T5LocalAttention module
    import numpy as np
    from tests.helpers import from_bf16_bits
    t5b = _ops()
    z = load("local.npz")
    for name in ("loc_ragged", "loc_short", "loc_long"):
        B, H, L, D, bl = [int(x) for x in z[name + "_meta"]]
        cfg = _Cfg(d_model=H * D, d_kv=D, num_heads=H, sliding_window=bl)
        mod = t5b.T5ATTENTION_TYPES["local"](cfg, has_relative_attention_bias=True)
        eye = torch.eye(H * D)
        with torch.no_grad():
            mod.q.weight.copy_(eye)
            mod.k.weight.copy_(eye[torch.from_numpy(z[name + "_kperm"])])
            mod.v.weight.copy_(eye[torch.from_numpy(z[name + "_vperm"])])
            mod.o.weight.copy_(eye)
            mod.relative_attention_bias.weight.copy_(from_bf16_bits(z[name + "_table"]))
        mod = mod.cuda().to(torch.bfloat16).eval()
        hidden = from_bf16_bits(z[name + "_hidden"]).to(torch.bfloat16)
        with torch.no_grad():
            out, present, pb = mod(hidden.cuda())
        assert present is None
        check_close(out, torch.from_numpy(z[name + "_out"]), torch.bfloat16, name)
