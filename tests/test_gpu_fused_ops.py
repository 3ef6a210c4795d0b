"""Kernels around the attention path (residual add + RMSNorm, gated GELU, merge of partial
attention results), the two-tile forward kernel, and the fused / full-width stack paths,
against the CPU oracle."""
import pytest
import torch

from oracle import t5_oracle as orc
from tests.helpers import TINY_T5, check_close, seed_named_parameters, seeded
from tests.test_gpu_other_kernels import _Cfg, _make_module, _oracle_layer, _ulp_close

pytestmark = pytest.mark.gpu


def _ops():
    import turbot5_b200 as t5b
    return t5b


# ------------------------------------------------------------------ residual add + RMSNorm
@pytest.mark.parametrize("rows,d,dt,wdt", [(1000, 768, torch.bfloat16, torch.bfloat16), (257, 512, torch.float16, torch.float16),
                                           (64, 1024, torch.bfloat16, torch.float32), (3, 2048, torch.bfloat16, torch.bfloat16),
                                           (5, 8, torch.bfloat16, torch.bfloat16)])
def test_add_rms_layer_norm_vs_oracle(rows, d, dt, wdt):
    from turbot5_b200.modules import add_rms_layer_norm
    hidden = (3.0 * seeded((rows, d), 1)).to(dt)
    branch = (0.7 * seeded((rows, d), 2) - 0.2).to(dt)
    w = torch.rand((d,), generator=torch.Generator().manual_seed(3)).to(wdt)
    h_out, normed = add_rms_layer_norm(hidden.cuda(), branch.cuda(), w.cuda(), 1e-6)
    want_h = hidden + branch                       # the residual stream, rounded to the element type
    assert torch.equal(h_out.cpu(), want_h)
    assert normed.dtype == dt
    _ulp_close(normed, orc.t5_layer_norm(want_h, w, 1e-6).to(dt), dt)
    # in place, on a 3-d view
    h3 = hidden.cuda().view(1, rows, d).clone()
    h2, n2 = add_rms_layer_norm(h3, branch.cuda().view(1, rows, d), w.cuda(), 1e-6, inplace=True)
    assert h2.data_ptr() == h3.data_ptr() and torch.equal(h2.cpu().view(rows, d), want_h)
    assert torch.equal(n2.view(rows, d), normed)


@pytest.mark.parametrize("rows,f,dt", [(1000, 2048, torch.bfloat16), (33, 256, torch.float16), (2, 8, torch.bfloat16)])
def test_gated_gelu_vs_torch(rows, f, dt):
    from turbot5_b200.modules import gated_gelu
    x = (2.5 * seeded((rows, 2 * f), 4)).to(dt)
    got = gated_gelu(x.cuda())
    want = torch.nn.functional.gelu(x[:, :f].float(), approximate="tanh").to(dt) * x[:, f:]
    assert got.shape == (rows, f) and got.dtype == dt
    err = (got.float().cpu() - want.float()).abs()
    bits = 8 if dt == torch.bfloat16 else 11
    # (in the negative tail torch's float32 0.5 * a * (1 + tanh(u)) cancels -- to exactly -0 below a = -5 --
    # while a * sigmoid(2u) keeps the true value of a few 1e-7: errors are measured against max(|want|, 1e-3))
    ulp = torch.pow(2.0, torch.floor(torch.log2(want.float().abs().clamp_min(1e-3))) - (bits - 1))
    # the activation is rounded to the element type before the product: a last-bit difference of the
    # float32 gelu can flip that rounding (one unit in the last place of the activation), which moves
    # the product by up to two units in ITS last place; such flips are rare
    worst = (err / ulp).max().item()
    assert worst <= 2.001, f"worst error {worst:.2f} ulp"
    assert (err > 1e-5).float().mean().item() < 1e-3      # beyond the cancellation noise of the negative tail


# ------------------------------------------------------------------ partial results over key slices + merge
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,cuts,off,causal", [(384, 1152, (0, 384, 1152), 384, False),
                                                 (300, 1000, (0, 77, 600, 1000), 350, False),
                                                 (256, 900, (0, 500, 900), None, True),
                                                 (100, 400, (0, 130, 400), 150, False)])
@pytest.mark.parametrize("D", [64, 32])
def test_partials_over_key_slices_merge_to_the_full_result(M, N, cuts, off, causal, dt, D):
    from turbot5_b200.attention import flash_attention_partial, merge_attention_partials
    B, H = 2, 3
    # token-major storage (the heads of a token side by side), as the sequence-parallel encoder has it
    q, k, v = (seeded((B, L_, H, D), sd, dtype=dt).transpose(1, 2) for sd, L_ in ((1, M), (2, N), (3, N)))
    table = seeded((32, H), 4, 0.1, dtype=dt)
    qpos = (N - M) if off is None else off
    want = orc.attention_basic(q, k, v, table, causal=causal, q_pos_offset=qpos)
    qc, kc, vc, tc = q.cuda(), k.cuda(), v.cuda(), table.cuda()
    parts = []
    for a, b in zip(cuts[:-1], cuts[1:]):
        o, lse = flash_attention_partial(qc, kc[:, :, a:b], vc[:, :, a:b], tc, causal=causal, sm_scale=1.0,
                                         q_pos_offset=qpos - a)
        assert o.dtype == torch.float32 and lse.shape == (B, H, M)
        parts.append((o, lse))
    out, lse = merge_attention_partials(parts, dt, return_lse=True)
    torch.cuda.synchronize()
    _ops().check_device_status()
    check_close(out, want, dt, f"merged {cuts}")
    _, lse_full = _ops().flash_attention_with_fusing_bias(qc, kc, vc, tc, causal=causal, sm_scale=1.0, q_pos_offset=qpos,
                                                          return_lse=True)
    finite = torch.isfinite(lse_full)
    assert torch.equal(finite, torch.isfinite(lse))
    # (the row sums carry the kernel's correction for the rounding of the dominant probability, up to
    # 2^-9 relative per tile, and that differs between one pass and several)
    assert (lse[finite] - lse_full[finite]).abs().max().item() < 1e-2


# ------------------------------------------------------------------ the two-tile forward kernel
CASES_2TILE = [(2, 3, 1024, 1024, False, None), (1, 2, 777, 777, False, None), (1, 2, 777, 777, True, None),
               (1, 2, 512, 1536, False, 0), (1, 2, 200, 555, True, None), (1, 2, 300, 300, False, 4000),
               (1, 2, 640, 130, True, None), (1, 1, 129, 4096, False, None)]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,M,N,causal,off", CASES_2TILE)
def test_two_tile_kernel_vs_oracle(B, H, M, N, causal, off, dt):
    t5b = _ops()
    q, k, v = seeded((B, H, M, 64), 1, dtype=dt), seeded((B, H, N, 64), 2, dtype=dt), seeded((B, H, N, 64), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = orc.attention_basic(q, k, v, table, causal=causal, q_pos_offset=off)
    out = t5b.flash_attention_with_fusing_bias(q.cuda(), k.cuda(), v.cuda(), table.cuda(), causal=causal, sm_scale=1.0,
                                               q_pos_offset=off, kernel="tcgen05_2tile")
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out, want, dt, f"two-tile {(B, H, M, N, causal, off)}")


def test_two_tile_kernel_packed_sequences():
    t5b = _ops()
    dt = torch.bfloat16
    lens = [300, 128, 1000, 257, 64, 2000]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    T = int(cu[-1])
    q, k, v = seeded((T, 4, 64), 5, dtype=dt), seeded((T, 4, 64), 6, dtype=dt), seeded((T, 4, 64), 7, dtype=dt)
    table = seeded((32, 4), 8, 0.1, dtype=dt)
    for causal in (False, True):
        want = orc.attention_basic_varlen(q, k, v, table, cu, cu, causal=causal)
        out = t5b.flash_attention_with_fusing_bias_varlen(q.cuda(), k.cuda(), v.cuda(), table.cuda(), cu.cuda(), cu.cuda(),
                                                          max(lens), max(lens), causal=causal, sm_scale=1.0,
                                                          kernel="tcgen05_2tile")
        torch.cuda.synchronize()
        t5b.check_device_status()
        check_close(out, want, dt, f"two-tile packed causal={causal}")


# ------------------------------------------------------------------ fused encoder pass
def _encoder(dt, **over):
    from turbot5_b200.t5 import T5Stack, T5StackConfig
    cfg = T5StackConfig(**{**TINY_T5, **over})
    enc = seed_named_parameters(T5Stack(cfg, torch.nn.Embedding(cfg.vocab_size, cfg.d_model), is_decoder=False), 0)
    return enc.cuda().to(dt).eval(), cfg


def test_fused_encoder_pass_equals_the_module_pass_bf16():
    enc, cfg = _encoder(torch.bfloat16, d_model=128, num_heads=4, d_ff=256, num_layers=3)
    ids = torch.randint(0, 128, (2, 300), generator=torch.Generator().manual_seed(3)).cuda()
    with torch.no_grad():
        a = enc(ids)
        b = enc.forward_fused(ids)
    # same arithmetic and rounding points; only the stacked matrix products may pick another
    # cuBLAS algorithm (a different summation order inside float32 accumulators)
    assert (a.float() - b.float()).abs().max().item() <= 0.05 * a.float().abs().max().item()
    assert (a.float() - b.float()).abs().mean().item() <= 2e-3 * a.float().abs().mean().item()
    w = {"encoder." + k: v.detach().float().cpu() for k, v in enc.state_dict().items()}
    w["shared.weight"] = enc.embed_tokens.weight.detach().float().cpu()
    want = orc.t5_stack_forward(w, {**TINY_T5, "d_model": 128, "num_heads": 4, "d_ff": 256, "num_layers": 3}, ids.cpu())
    # three layers of bf16 linears, norms and residuals against an all-float32 oracle: the fused pass
    # must be as close to it as the module pass is
    rel = lambda t: ((t.float().cpu() - want).abs().mean() / want.abs().mean()).item()
    assert rel(b) < 1e-1 and rel(b) <= 1.1 * rel(a) + 1e-3


def test_fused_encoder_pass_fp16_relu_and_embeds():
    enc, cfg = _encoder(torch.float16, d_model=128, num_heads=4, d_ff=256, feed_forward_proj="relu")
    x = (0.5 * seeded((1, 200, 128), 9)).half().cuda()
    keep = x.clone()
    with torch.no_grad():
        a = enc(inputs_embeds=x)
        b = enc.forward_fused(inputs_embeds=x)
    assert torch.equal(x, keep)            # the caller's tensor is not modified
    assert (a.float() - b.float()).abs().max().item() <= 0.05 * a.float().abs().max().item()


# ------------------------------------------------------------------ full-width (T5-base) layers
def test_t5_base_width_layers_vs_oracle():
    """d_model 768, 12 heads of 64, bf16: encoder self-attention at (2, 1024), decoder self-attention
    (2, 128) causal, and cross-attention of 128 decoder rows over 1024 encoder states.  The oracle
    rounds q, k, v and the attention output to bf16 where the bf16 module stores them (at this width
    those roundings alone move a float32 layer by more than the kernel tolerance); everything else
    is float32.  The attention core itself is then compared at the kernel tolerance, the layer
    output (one more 768-term projection) at twice that."""
    dt = torch.bfloat16
    t5b = _ops()

    def check_layer(mod, hid, what, **kw):
        with torch.no_grad():
            out = mod(hid.cuda(), **{k: (v.cuda() if torch.is_tensor(v) else v) for k, v in kw.items() if k != "is_decoder"})[0]
        okw = {k: (v.float() if k == "key_value_states" else v) for k, v in kw.items()}
        want, (kh, vh) = _oracle_layer(mod, hid, round_to=dt, **okw)
        diff = (out.float().cpu() - want).abs()
        assert diff.max().item() <= 4e-2 and diff.mean().item() <= 4e-3, (what, diff.max().item(), diff.mean().item())
        # the attention core on exactly the module's q, k, v
        f = lambda p: p.detach().float().cpu()
        B, M = hid.shape[:2]
        qh = (hid.float() @ f(mod.q.weight).t()).to(dt).view(B, M, 12, 64).transpose(1, 2)
        table = f(mod.relative_attention_bias.weight).to(dt) if mod.has_relative_attention_bias else None
        off = 0 if "key_value_states" in kw else None
        core = t5b.flash_attention_with_fusing_bias(qh.cuda(), kh.to(dt).cuda(), vh.to(dt).cuda(),
                                                    None if table is None else table.cuda(), causal=mod.causal,
                                                    sm_scale=1.0, q_pos_offset=off)
        want_core = orc.attention_basic(qh, kh.to(dt), vh.to(dt), table, causal=mod.causal, q_pos_offset=off)
        check_close(core, want_core, dt, what + " (attention core)")

    enc_att = _make_module(_Cfg(d_model=768, d_kv=64, num_heads=12), dt, 1)
    hidden = seeded((2, 1024, 768), 2, dtype=dt)
    check_layer(enc_att, hidden, "encoder layer 2x1024")
    dcfg = _Cfg(d_model=768, d_kv=64, num_heads=12, is_decoder=True)
    dec = seeded((2, 128, 768), 5, dtype=dt)
    check_layer(_make_module(dcfg, dt, 3), dec, "decoder self-attention 2x128", is_decoder=True)
    check_layer(_make_module(dcfg, dt, 4, cross=True, bias=False), dec, "cross attention 128 x 1024",
                is_decoder=True, key_value_states=hidden)


# ------------------------------------------------------------------ module paths the reference never reaches
def test_cross_attention_mask_with_equal_decoder_and_encoder_lengths():
    """The padding mask describes the encoder keys; decoder rows stay whole even when the decoder
    is exactly as long as the encoder."""
    from turbot5_b200.t5 import T5ForConditionalGeneration, T5StackConfig
    over = dict(d_model=128, num_heads=4, d_ff=256)
    model = seed_named_parameters(T5ForConditionalGeneration(T5StackConfig(**{**TINY_T5, **over})), 0)
    model = model.cuda().to(torch.bfloat16).eval()
    g = torch.Generator().manual_seed(11)
    L = 160
    ids, dec = torch.randint(0, 128, (2, L), generator=g), torch.randint(0, 128, (2, L), generator=g)
    mask = torch.ones((2, L), dtype=torch.int64)
    mask[0, 90:] = 0
    mask[1, 33:] = 0
    with torch.no_grad():
        logits = model(ids.cuda(), dec.cuda(), attention_mask=mask.cuda())
    w = {k: v.detach().float().cpu() for k, v in model.state_dict().items()}
    _, want = orc.t5_model_logits(w, {**TINY_T5, **over}, ids, dec, mask=mask)
    rel = ((logits.float().cpu() - want).abs().mean() / want.abs().mean()).item()
    assert rel < 1e-1
    # every decoder row carries a result (none was dropped as "padding")
    assert (logits.float().abs().sum(-1) > 0).all()
    cross = model.decoder.block[0].layer[1].EncDecAttention
    hid = seeded((2, L, 128), 12, dtype=torch.bfloat16)
    enc_states = seeded((2, L, 128), 13, dtype=torch.bfloat16)
    with torch.no_grad():
        out = cross(hid.cuda(), key_value_states=enc_states.cuda(), mask=mask.cuda())[0]
    want_l, _ = _oracle_layer(cross, hid, is_decoder=True, key_value_states=enc_states.float(), key_padding_mask=mask,
                              round_to=torch.bfloat16)
    diff = (out.float().cpu() - want_l).abs()       # a whole layer: twice the kernel tolerance
    assert diff.max().item() <= 4e-2 and diff.mean().item() <= 4e-3, (diff.max().item(), diff.mean().item())


def test_short_decoder_training_keeps_gradients():
    """A decoder input of a few tokens in training goes through the differentiable operator (the
    split-KV decoding kernel has no backward): the cross-attention projections and the encoder
    receive gradients."""
    dt = torch.bfloat16
    cross = _make_module(_Cfg(is_decoder=True), dt, 4, cross=True, bias=False).train()
    hid = seeded((2, 4, 128), 5, dtype=dt).cuda().requires_grad_(True)
    enc = seeded((2, 300, 128), 6, dtype=dt).cuda().requires_grad_(True)
    out = cross(hid, key_value_states=enc)[0]
    assert out.requires_grad
    out.float().pow(2).sum().backward()
    for name in ("q", "k", "v", "o"):
        g = getattr(cross, name).weight.grad
        assert g is not None and g.float().abs().sum().item() > 0, name
    assert enc.grad is not None and enc.grad.float().abs().sum().item() > 0
    with torch.no_grad():
        out_eval = cross(hid.detach(), key_value_states=enc.detach())[0]       # the decoding kernel
    check_close(out_eval, out.detach(), dt, "decode path vs dense path")


def test_fused_encoder_decoder_forward_equals_the_module_passes():
    from turbot5_b200.t5 import T5ForConditionalGeneration, T5StackConfig
    over = dict(d_model=128, num_heads=4, d_ff=256)
    model = seed_named_parameters(T5ForConditionalGeneration(T5StackConfig(**{**TINY_T5, **over})), 0)
    model = model.cuda().to(torch.bfloat16).eval()
    g = torch.Generator().manual_seed(21)
    ids, dec = torch.randint(0, 128, (2, 300), generator=g), torch.randint(0, 128, (2, 150), generator=g)
    with torch.no_grad():
        fused = model(ids.cuda(), dec.cuda())                                  # inference: both stacks fused
        enc = model.encoder(ids.cuda())
        plain = model.logits(model.decoder(dec.cuda(), encoder_hidden_states=enc))
    assert (fused.float() - plain.float()).abs().max().item() <= 0.05 * plain.float().abs().max().item()
    assert (fused.float() - plain.float()).abs().mean().item() <= 5e-3 * plain.float().abs().mean().item()
    w = {k: v.detach().float().cpu() for k, v in model.state_dict().items()}
    _, want = orc.t5_model_logits(w, {**TINY_T5, **over}, ids, dec)
    rel = lambda t: ((t.float().cpu() - want).abs().mean() / want.abs().mean()).item()
    assert rel(fused) < 1e-1 and rel(fused) <= 1.1 * rel(plain) + 1e-3
