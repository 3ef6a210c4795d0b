"""The CPU oracle against fixtures produced by the reference's own code."""
import numpy as np
import pytest
import torch

from oracle import t5_oracle as orc
from tests.helpers import attention_case, from_bf16_bits, load, local_case, local_masked_case, seeded


def test_bucket_tables_bit_exact():
    z = load("buckets.npz")
    for nb, md, bidir, lo, hi in z["settings"]:
        key = f"nb{nb}_md{md}_{'bi' if bidir else 'uni'}"
        got = orc.bucket_of_delta(range(lo, hi + 1), bool(bidir), int(nb), int(md))
        assert np.array_equal(got, z[key].astype(np.int64)), key


def test_bucket_grid_bit_exact():
    z = load("buckets.npz")
    ctx = np.arange(300)[:, None]
    mem = np.arange(280)[None, :]
    assert np.array_equal(orc.relative_position_bucket(mem - ctx, True, 32, 128), z["grid_bi"])
    assert np.array_equal(orc.relative_position_bucket(mem - ctx, False, 32, 128), z["grid_uni"])


def test_bucket_known_thresholds():
    # first distance of each bucket, keys at/before the query (32 buckets, max_distance 128)
    d = np.arange(0, 200)
    bi = orc.relative_position_bucket(-d, True, 32, 128)
    firsts = [int(d[np.argmax(bi == b)]) for b in range(16)]
    assert firsts == [0, 1, 2, 3, 4, 5, 6, 7, 8, 12, 16, 23, 32, 46, 64, 91]
    uni = orc.relative_position_bucket(-d, False, 32, 128)
    firsts = [int(d[np.argmax(uni == b)]) for b in range(32)]
    assert firsts == list(range(17)) + [19, 21, 24, 27, 31, 35, 40, 46, 52, 59, 67, 77, 87, 99, 113]
    assert np.all(orc.relative_position_bucket(d[1:], False, 32, 128) == 0)


@pytest.mark.parametrize("name", ["enc_small", "enc_ragged", "enc_long", "enc_d32", "enc_d128",
                                  "dec_cached", "dec_step", "cross_mn"])
def test_attention_cases(name):
    c = attention_case(load("attention.npz"), name)
    off = 0 if name == "cross_mn" else c["N"] - c["M"]
    bias = orc.compute_bias(c["table"], c["M"], c["N"], not c["unidirectional"], c["nb"], c["md"],
                            q_pos_offset=off)
    got = orc.naive_attention_with_bias(c["q"], c["k"], c["v"], bias)
    assert torch.equal(got, c["out"]) or (got - c["out"]).abs().max() < 1e-6
    # slabbed whole-path helper agrees too (bidirectional cases have no mask)
    if not c["unidirectional"]:
        got2 = orc.attention_basic(c["q"], c["k"], c["v"], c["table"], causal=False,
                                   num_buckets=c["nb"], max_distance=c["md"], q_pos_offset=off, slab=37)
        assert (got2 - c["out"]).abs().max() < 1e-5


def test_layer_small_and_full():
    z = load("layer.npz")
    t = lambda k: torch.from_numpy(z[k])
    out, _ = orc.t5_attention_layer(t("small_hidden"), t("small_wq"), t("small_wk"), t("small_wv"),
                                    t("small_wo"), t("small_table"), n_heads=4, d_kv=32)
    assert (out - t("small_out")).abs().max() < 1e-5
    # full-size float32 layer: batch 2, seq 512, d_model 512, 8 heads x 64, seed 0
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn((2, 512, 512), generator=g)
    ws = [torch.randn((512, 512), generator=g) * 0.05 for _ in range(3)]
    wo = torch.randn((512, 512), generator=g) * 0.05
    table = torch.randn((32, 8), generator=g) * 0.1
    sums = np.asarray([x.double().sum().item() for x in (hidden, *ws, wo, table)])
    if not np.allclose(sums, z["full_checks"], rtol=0, atol=1e-6):
        pytest.skip("torch RNG stream differs from the one that generated the fixture")
    out, _ = orc.t5_attention_layer(hidden, ws[0], ws[1], ws[2], wo, table, n_heads=8, d_kv=64)
    assert (out[:, ::16, ::16] - t("full_out_sub")).abs().max() < 1e-4


@pytest.mark.parametrize("tag,xdt,wdt", [("f32", torch.float32, torch.float32),
                                          ("bf16", torch.bfloat16, torch.bfloat16),
                                          ("bf16_wf32", torch.bfloat16, torch.float32),
                                          ("f16", torch.float16, torch.float16)])
def test_rmsnorm(tag, xdt, wdt):
    z = load("rmsnorm.npz")
    x = torch.from_numpy(z[tag + "_x"]).to(xdt)
    w = torch.from_numpy(z[tag + "_w"]).to(wdt)
    y = orc.t5_layer_norm(x, w, 1e-6)
    assert str(y.dtype) == str(z[tag + "_ydtype"])
    assert torch.equal(y.float(), torch.from_numpy(z[tag + "_y"]))


def test_padding():
    z = load("padding.npz")
    mask = torch.from_numpy(z["mask"])
    idx, cu, mx = orc.get_unpad_data(mask)
    assert torch.equal(idx, torch.from_numpy(z["indices"]))
    assert torch.equal(cu, torch.from_numpy(z["cu_seqlens"]))
    assert mx == int(z["max_seqlen"])
    padded = orc.pad_rows(torch.from_numpy(z["values"]), idx, 5, 9)
    assert torch.equal(padded, torch.from_numpy(z["padded"]))


def test_split_merge_equals_full_softmax():
    # merging per-split partials (normalised output, l, m) reproduces one softmax
    q = seeded((3, 1, 16), 5)
    k = seeded((3, 50, 16), 6)
    v = seeded((3, 50, 16), 7)
    s = torch.einsum("bqd,bkd->bqk", q, k)[:, 0]                     # (3, 50)
    full = torch.einsum("bk,bkd->bd", torch.softmax(s, -1), v)
    bounds = [0, 13, 13, 31, 50]                                      # includes an empty split
    po, pl, pm = [], [], []
    for a, b in zip(bounds[:-1], bounds[1:]):
        if a == b:
            continue
        m = s[:, a:b].max(-1).values
        p = torch.exp(s[:, a:b] - m[:, None])
        l = p.sum(-1)
        po.append(torch.einsum("bk,bkd->bd", p, v[:, a:b]) / l[:, None]); pl.append(l); pm.append(m)
    got = orc.merge_splits(torch.stack(po, 1), torch.stack(pl, 1), torch.stack(pm, 1))
    assert (got - full).abs().max() < 1e-5


def test_varlen_matches_dense_per_sequence():
    lens = [5, 17, 1, 40]
    cu = np.concatenate([[0], np.cumsum(lens)])
    T = int(cu[-1])
    q, k, v = seeded((T, 2, 16), 1), seeded((T, 2, 16), 2), seeded((T, 2, 16), 3)
    table = seeded((32, 2), 4, 0.1)
    out = orc.attention_basic_varlen(q, k, v, table, cu, cu)
    b = 3
    sl = slice(int(cu[b]), int(cu[b + 1]))
    one = orc.attention_basic(q[sl].transpose(0, 1)[None], k[sl].transpose(0, 1)[None],
                              v[sl].transpose(0, 1)[None], table)
    assert torch.equal(out[sl], one[0].transpose(0, 1))


def _tiny_reference_weights():
    """The name-seeded weights of the tiny fixture model, as a dict (built on the product's own
    module tree only to enumerate names and shapes; no kernel is involved)."""
    from tests.helpers import TINY_T5, seed_named_parameters
    from turbot5_b200.t5 import T5ForConditionalGeneration, T5StackConfig
    model = seed_named_parameters(T5ForConditionalGeneration(T5StackConfig(**TINY_T5)), 0)
    return {k: v.detach().clone() for k, v in model.state_dict().items()}, model


def test_stack_oracle_matches_reference_model_fixture():
    from tests.helpers import TINY_T5, tiny_t5_inputs
    z = load("stack.npz")
    w, model = _tiny_reference_weights()
    assert sorted(n for n, _ in model.named_parameters()) == [str(x) for x in z["param_names"]]
    ids, dec = tiny_t5_inputs()
    enc, logits = orc.t5_model_logits(w, TINY_T5, ids, dec)
    assert (enc - torch.from_numpy(z["encoder"])).abs().max() < 2e-5
    assert (logits - torch.from_numpy(z["logits"])).abs().max() < 2e-5
    mask = torch.from_numpy(z["mask"])
    enc_m, logits_m = orc.t5_model_logits(w, TINY_T5, ids, dec, mask=mask)
    valid = mask.bool()
    assert (enc_m - torch.from_numpy(z["encoder_masked"]))[valid].abs().max() < 2e-5
    assert (logits_m - torch.from_numpy(z["logits_masked"])).abs().max() < 2e-5
    # greedy decoding (recomputed without a cache) reproduces the reference's cached steps
    cur = torch.zeros((2, 1), dtype=torch.long)
    for step in range(4):
        _, lg = orc.t5_model_logits(w, TINY_T5, ids, cur)
        assert (lg[:, -1] - torch.from_numpy(z["greedy_logits"][:, step])).abs().max() < 2e-5
        cur = torch.cat([cur, lg[:, -1:].argmax(-1)], dim=1)
    assert torch.equal(cur[:, 1:], torch.from_numpy(z["greedy_tokens"]))


@pytest.mark.parametrize("name", ["g_enc", "g_cross", "g_long", "g_uni"])
def test_attention_gradients_under_autograd(name):
    # the oracle restatement under torch autograd against the reference's functions under autograd
    z = load("attention_grad.npz")
    B, H, M, N, D, dec, nb, md = [int(x) for x in z[name + "_meta"]]
    q = from_bf16_bits(z[name + "_q"]).requires_grad_(True)
    k = from_bf16_bits(z[name + "_k"]).requires_grad_(True)
    v = from_bf16_bits(z[name + "_v"]).requires_grad_(True)
    table = from_bf16_bits(z[name + "_table"]).requires_grad_(True)
    dout = from_bf16_bits(z[name + "_dout"])
    bias = orc.compute_bias(table, M, N, not dec, nb, md, q_pos_offset=0)
    out = orc.naive_attention_with_bias(q, k, v, bias)
    (out * dout).sum().backward()
    for got, key in ((q.grad, "_dq"), (k.grad, "_dk"), (v.grad, "_dv"), (table.grad, "_dtable")):
        want = torch.from_numpy(z[name + key])
        assert (got - want).abs().max().item() <= 1e-4 * max(1.0, want.abs().max().item()), (name, key)


@pytest.mark.parametrize("name", ["loc_ragged", "loc_short", "loc_even", "loc_long"])
def test_block_local_attention_oracle(name):
    q, k, v, table, bl, want = local_case(load("local.npz"), name)
    got = orc.local_attention_basic(q, k, v, table, bl)
    assert (got - want).abs().max().item() <= 2e-5


@pytest.mark.parametrize("name", ["locm_ragged", "locm_short", "locm_even", "locm_long", "locm_full"])
def test_block_local_attention_with_padding_mask_oracle(name):
    """The masked form (a sliding window over the valid keys) against the reference module driven
    with the mask its stack builds."""
    q, k, v, table, bl, want, lens = local_masked_case(load("local_masked.npz"), name)
    mask = torch.zeros((q.shape[0], q.shape[2]))
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    got = orc.local_attention_basic(q, k, v, table, bl, key_padding_mask=mask)
    for b, n in enumerate(lens):
        assert (got[b, :, :n] - want[b, :, :n]).abs().max().item() < 2e-5, name
