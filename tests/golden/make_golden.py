"""Generate the golden fixtures in this directory from the reference's own code.

Run once, in a container that has the reference source tree mounted (it is not
available on the GPU machines; the committed `.npz` files are what travels):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

The reference targets an older `transformers`; three symbols it imports (head
pruning, model-parallel device maps, ONNX config) no longer exist and are
stubbed *before* import.  None of them is on the attention path.  No reference
file is modified or copied; only outputs of its functions are stored.

Fixtures written:
  buckets.npz      bucket index for every delta in [-2*md-3, 2*md+3] for a spread
                   of (num_buckets, max_distance, bidirectional) settings, from
                   `T5Attention._relative_position_bucket`.
  attention_grad.npz  the same two functions under autograd: gradients of q, k, v and the table
  local.npz        `T5LocalAttention.forward` (block-local attention) with permutation projections
  local_masked.npz the same module with the padding mask `T5Stack` builds for it
                   (`_get_local_attention_mask`): right-padded batches
  attention.npz    small seeded q/k/v/table cases through `compute_bias` +
                   `naive_torch_attention_with_bias` (float32 math on bf16-representable
                   inputs, stored as bf16 bit patterns), incl. cached
                   decoding (last-rows slice) and unidirectional bias.
  layer.npz        `T5Attention.forward` ('basic') on a small seeded layer, and a
                   sub-sample of the full-size batch-2 x 512 x d_model-512 float32
                   layer output with input checksums (inputs are regenerated
                   from the seed by the test).
  rmsnorm.npz      `T5LayerNorm._forward` for float32 / bfloat16 weights.
  padding.npz      `_get_unpad_data` + `pad_input` on a ragged mask.
  stack.npz        the reference's whole encoder-decoder model (tiny shape, 'basic' attention,
                   weights seeded by parameter name): encoder output, logits, masked variants and
                   four greedy decoding steps through its K/V cache.
"""
import math
import os
import sys
import types

import numpy as np
import torch


def _install_shim():
    import transformers  # noqa: F401
    import transformers.pytorch_utils as pu
    if not hasattr(pu, "find_pruneable_heads_and_indices"):
        def _unavailable(*a, **k):
            raise NotImplementedError
        pu.find_pruneable_heads_and_indices = _unavailable
    m = types.ModuleType("transformers.utils.model_parallel_utils")
    m.assert_device_map = lambda *a, **k: None
    m.get_device_map = lambda *a, **k: {}
    sys.modules["transformers.utils.model_parallel_utils"] = m
    o = types.ModuleType("transformers.onnx")

    class OnnxSeq2SeqConfigWithPast:  # placeholder base class
        pass
    o.OnnxSeq2SeqConfigWithPast = OnnxSeq2SeqConfigWithPast
    sys.modules["transformers.onnx"] = o


BUCKET_SETTINGS = [
    # (num_buckets, max_distance)
    (32, 128), (32, 64), (32, 256), (64, 128), (64, 256), (16, 32), (16, 128),
    (8, 20), (24, 100), (48, 200), (128, 1024), (32, 1000), (12, 50), (4, 8), (40, 128),
]


def seeded(shape, seed, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype)


def bf16_bits(t):
    """bf16-representable float32 tensor -> uint16 bit patterns (halves the file)."""
    return t.bfloat16().view(torch.int16).numpy().view(np.uint16)


def make_local_masked(here):
    """T5LocalAttention.forward with the 5-D mask of T5Stack (src/turbot5/model/modeling.py:488-489,
    src/turbot5/model/utils.py:174-188) on right-padded batches; permutation projections as in
    local.npz.  Rows of padded queries are whatever the reference computes there (not compared)."""
    from turbot5.model.attentions import T5LocalAttention
    from turbot5.model.config import T5Config
    from turbot5.model.utils import _get_local_attention_mask
    local = {}
    # one sequence per case: the reference module itself fails on batches of several sequences with
    # several blocks (`shape_blocks` views a transposed tensor, attentions.py:575-576,596)
    specs = [("locm_ragged", 300, 128, [170]), ("locm_short", 100, 512, [37]), ("locm_even", 512, 256, [300]),
             ("locm_long", 1100, 384, [650]), ("locm_full", 700, 256, [700])]
    H, D = 2, 64
    for name, L, bl, lens in specs:
        B = len(lens)
        cfg = T5Config(d_model=H * D, d_kv=D, num_heads=H, relative_attention_num_buckets=32,
                       relative_attention_max_distance=128, is_decoder=False, dropout_rate=0.0,
                       tie_word_embeddings=False, sliding_window=bl)
        cfg.use_triton = False
        att = T5LocalAttention(cfg, has_relative_attention_bias=True).eval()
        gperm = torch.Generator().manual_seed(1600 + L)
        eye = torch.eye(H * D)
        pk_, pv_ = torch.randperm(H * D, generator=gperm), torch.randperm(H * D, generator=gperm)
        table = seeded((32, H), 1700 + L, 0.1).bfloat16().float()
        hidden = seeded((B, L, H * D), 1800 + L).bfloat16().float()
        mask2d = torch.zeros((B, L))
        for b, n in enumerate(lens):
            mask2d[b, :n] = 1
        mask5d = _get_local_attention_mask(mask2d, bl, hidden.device)
        with torch.no_grad():
            att.q.weight.copy_(eye); att.k.weight.copy_(eye[pk_]); att.v.weight.copy_(eye[pv_]); att.o.weight.copy_(eye)
            att.relative_attention_bias.weight.copy_(table)
            out = att(hidden, mask=mask5d)[0]
        local[name + "_hidden"] = bf16_bits(hidden)
        local[name + "_table"] = bf16_bits(table)
        local[name + "_kperm"] = pk_.numpy()
        local[name + "_vperm"] = pv_.numpy()
        local[name + "_out"] = out.numpy()
        local[name + "_lens"] = np.asarray(lens, dtype=np.int64)
        local[name + "_meta"] = np.asarray([B, H, L, D, bl], dtype=np.int64)
    local["names"] = np.asarray([s_[0] for s_ in specs])
    np.savez_compressed(os.path.join(here, "local_masked.npz"), **local)


def main(ref_root: str, only=None):
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(ref_root, "src"))
    _install_shim()
    torch.manual_seed(0)
    if only == "local_masked":
        make_local_masked(here)
        print("local_masked.npz written to", here)
        return
    from turbot5.model.attentions import T5Attention
    from turbot5.model.config import T5Config
    from turbot5.model.modules import T5LayerNorm
    from turbot5.model.padding import _get_unpad_data, pad_input
    from turbot5.ops.naive_attention import naive_torch_attention_with_bias

    # ---------------------------------------------------------------- buckets
    out = {}
    settings = []
    for nb, md in BUCKET_SETTINGS:
        for bidir in (True, False):
            lo, hi = -2 * md - 3, 2 * md + 3
            rel = torch.arange(lo, hi + 1, dtype=torch.long)
            b = T5Attention._relative_position_bucket(rel, bidirectional=bidir,
                                                      num_buckets=nb, max_distance=md)
            key = f"nb{nb}_md{md}_{'bi' if bidir else 'uni'}"
            out[key] = b.numpy().astype(np.int32)
            settings.append((nb, md, int(bidir), lo, hi))
    out["settings"] = np.asarray(settings, dtype=np.int64)
    # 2-D grid as compute_bias builds it, both int32 and int64 inputs
    ctx = torch.arange(300, dtype=torch.long)[:, None]
    mem = torch.arange(280, dtype=torch.long)[None, :]
    out["grid_bi"] = T5Attention._relative_position_bucket(mem - ctx, True, 32, 128).numpy().astype(np.int8)
    out["grid_uni"] = T5Attention._relative_position_bucket(mem - ctx, False, 32, 128).numpy().astype(np.int8)
    np.savez_compressed(os.path.join(here, "buckets.npz"), **out)

    # -------------------------------------------------------------- attention
    def make_att(is_decoder, H, nb, md):
        cfg = T5Config(d_model=H * 8, d_kv=8, num_heads=H, relative_attention_num_buckets=nb,
                       relative_attention_max_distance=md, is_decoder=is_decoder,
                       dropout_rate=0.0, tie_word_embeddings=False)
        cfg.is_decoder = is_decoder
        att = T5Attention(cfg, has_relative_attention_bias=True)
        return att.eval()

    cases = {}
    specs = [
        # name, B, H, M, N, D, is_decoder(unidirectional), nb, md, seed
        ("enc_small", 1, 2, 80, 80, 64, False, 32, 128, 1),
        ("enc_ragged", 1, 2, 130, 130, 64, False, 32, 128, 2),
        ("enc_long", 1, 1, 300, 300, 64, False, 32, 128, 3),
        ("enc_d32", 1, 2, 70, 70, 32, False, 32, 128, 4),
        ("enc_d128", 1, 2, 40, 40, 128, False, 16, 32, 5),
        ("dec_cached", 1, 2, 3, 41, 64, True, 32, 128, 6),    # last-rows slice
        ("dec_step", 2, 2, 1, 150, 64, True, 32, 128, 7),
        ("cross_mn", 1, 2, 17, 90, 64, False, 32, 128, 8),   # M != N, bidirectional
    ]
    for name, B, H, M, N, D, dec, nb, md, seed in specs:
        att = make_att(dec, H, nb, md)
        table = seeded((nb, H), 100 + seed, 0.1).bfloat16().float()
        with torch.no_grad():
            att.relative_attention_bias.weight.copy_(table)
            # values are bf16-representable so the same case feeds every dtype
            q = seeded((B, H, M, D), 200 + seed).bfloat16().float()
            k = seeded((B, H, N, D), 300 + seed).bfloat16().float()
            v = seeded((B, H, N, D), 400 + seed).bfloat16().float()
            # the reference builds the bias for max(M, N)... it uses
            # real_seq_length rows then keeps the last M (attentions.py:229-234)
            if name == "cross_mn":
                bias = att.compute_bias(M, N)
            else:
                bias = att.compute_bias(N, N)[:, :, -M:, :]
            o, _ = naive_torch_attention_with_bias(q, k, v, bias.clone())
        cases[name + "_q"] = bf16_bits(q)
        cases[name + "_k"] = bf16_bits(k)
        cases[name + "_v"] = bf16_bits(v)
        cases[name + "_table"] = bf16_bits(table)
        cases[name + "_out"] = o.numpy()
        cases[name + "_meta"] = np.asarray([B, H, M, N, D, int(dec), nb, md], dtype=np.int64)
    cases["names"] = np.asarray([s[0] for s in specs])
    np.savez_compressed(os.path.join(here, "attention.npz"), **cases)

    # ------------------------------------------------------------------ layer
    layer = {}

    def run_layer(B, L, d_model, H, D, seed, is_decoder=False):
        cfg = T5Config(d_model=d_model, d_kv=D, num_heads=H, relative_attention_num_buckets=32,
                       relative_attention_max_distance=128, is_decoder=is_decoder,
                       dropout_rate=0.0, tie_word_embeddings=False)
        cfg.is_decoder = is_decoder
        att = T5Attention(cfg, has_relative_attention_bias=True).eval()
        g = torch.Generator().manual_seed(seed)
        hidden = torch.randn((B, L, d_model), generator=g)
        ws = [torch.randn((H * D, d_model), generator=g) * 0.05 for _ in range(3)]
        wo = torch.randn((d_model, H * D), generator=g) * 0.05
        table = torch.randn((32, H), generator=g) * 0.1
        with torch.no_grad():
            att.q.weight.copy_(ws[0]); att.k.weight.copy_(ws[1]); att.v.weight.copy_(ws[2])
            att.o.weight.copy_(wo); att.relative_attention_bias.weight.copy_(table)
            out = att(hidden)[0]
        return hidden, ws, wo, table, out

    hidden, ws, wo, table, o = run_layer(2, 64, 128, 4, 32, seed=11)
    layer.update(small_hidden=hidden.numpy(), small_wq=ws[0].numpy(), small_wk=ws[1].numpy(),
                 small_wv=ws[2].numpy(), small_wo=wo.numpy(), small_table=table.numpy(),
                 small_out=o.numpy())
    # full-size float32 layer: batch 2, seq 512, 8 heads, d_kv 64, d_model 512, seed 0
    hidden, ws, wo, table, o = run_layer(2, 512, 512, 8, 64, seed=0)
    layer["full_out_sub"] = o[:, ::16, ::16].contiguous().numpy()
    layer["full_checks"] = np.asarray([hidden.double().sum().item(), ws[0].double().sum().item(),
                                       ws[1].double().sum().item(), ws[2].double().sum().item(),
                                       wo.double().sum().item(), table.double().sum().item()])
    np.savez_compressed(os.path.join(here, "layer.npz"), **layer)

    # ---------------------------------------------------------------- rmsnorm
    # ------------------------------------------------- attention gradients
    # the same two reference functions under autograd: d(sum(out * dout)) / d(q, k, v, table)
    grads = {}
    gspecs = [
        # name, B, H, M, N, D, unidirectional, nb, md, seed
        ("g_enc", 1, 2, 150, 150, 64, False, 32, 128, 11),
        ("g_cross", 2, 2, 70, 200, 64, False, 32, 128, 12),
        ("g_long", 1, 1, 400, 400, 64, False, 32, 128, 13),
        ("g_uni", 1, 2, 90, 90, 64, True, 32, 128, 14),      # unidirectional buckets, no mask
    ]
    for name, B, H, M, N, D, dec, nb, md, seed in gspecs:
        att = make_att(dec, H, nb, md)
        table = seeded((nb, H), 100 + seed, 0.1).bfloat16().float()
        with torch.no_grad():
            att.relative_attention_bias.weight.copy_(table)
        q = (seeded((B, H, M, D), 200 + seed) * 0.5).bfloat16().float().requires_grad_(True)
        k = (seeded((B, H, N, D), 300 + seed) * 0.5).bfloat16().float().requires_grad_(True)
        v = seeded((B, H, N, D), 400 + seed).bfloat16().float().requires_grad_(True)
        dout = seeded((B, H, M, D), 500 + seed).bfloat16().float()
        bias = att.compute_bias(M, N) if M != N else att.compute_bias(N, N)
        o, _ = naive_torch_attention_with_bias(q, k, v, bias.clone())
        (o * dout).sum().backward()
        grads[name + "_q"] = bf16_bits(q.detach())
        grads[name + "_k"] = bf16_bits(k.detach())
        grads[name + "_v"] = bf16_bits(v.detach())
        grads[name + "_table"] = bf16_bits(table)
        grads[name + "_dout"] = bf16_bits(dout)
        grads[name + "_dq"] = q.grad.numpy()
        grads[name + "_dk"] = k.grad.numpy()
        grads[name + "_dv"] = v.grad.numpy()
        grads[name + "_dtable"] = att.relative_attention_bias.weight.grad.numpy()
        grads[name + "_meta"] = np.asarray([B, H, M, N, D, int(dec), nb, md], dtype=np.int64)
    grads["names"] = np.asarray([s[0] for s in gspecs])
    np.savez_compressed(os.path.join(here, "attention_grad.npz"), **grads)

    # ------------------------------------------------- block-local attention
    # T5LocalAttention.forward with permutation matrices as q/k/v/o projections, so that the
    # module output is the attention core's output on bf16-exact q, k, v
    from turbot5.model.attentions import T5LocalAttention
    local = {}
    lspecs = [("loc_ragged", 1, 300, 128), ("loc_short", 2, 100, 512), ("loc_even", 1, 512, 256), ("loc_long", 1, 1100, 384)]
    H, D = 2, 64
    for name, B, L, bl in lspecs:
        cfg = T5Config(d_model=H * D, d_kv=D, num_heads=H, relative_attention_num_buckets=32,
                       relative_attention_max_distance=128, is_decoder=False, dropout_rate=0.0,
                       tie_word_embeddings=False, sliding_window=bl)
        cfg.use_triton = False
        att = T5LocalAttention(cfg, has_relative_attention_bias=True).eval()
        gperm = torch.Generator().manual_seed(600 + L)
        eye = torch.eye(H * D)
        pk_, pv_ = torch.randperm(H * D, generator=gperm), torch.randperm(H * D, generator=gperm)
        table = seeded((32, H), 700 + L, 0.1).bfloat16().float()
        hidden = seeded((B, L, H * D), 800 + L).bfloat16().float()
        with torch.no_grad():
            att.q.weight.copy_(eye); att.k.weight.copy_(eye[pk_]); att.v.weight.copy_(eye[pv_]); att.o.weight.copy_(eye)
            att.relative_attention_bias.weight.copy_(table)
            out = att(hidden)[0]
        local[name + "_hidden"] = bf16_bits(hidden)
        local[name + "_table"] = bf16_bits(table)
        local[name + "_kperm"] = pk_.numpy()
        local[name + "_vperm"] = pv_.numpy()
        local[name + "_out"] = out.numpy()
        local[name + "_meta"] = np.asarray([B, H, L, D, bl], dtype=np.int64)
    local["names"] = np.asarray([s_[0] for s_ in lspecs])
    np.savez_compressed(os.path.join(here, "local.npz"), **local)
    make_local_masked(here)

    rn = {}
    for tag, xdt, wdt in (("f32", torch.float32, torch.float32),
                          ("bf16", torch.bfloat16, torch.bfloat16),
                          ("bf16_wf32", torch.bfloat16, torch.float32),
                          ("f16", torch.float16, torch.float16)):
        g = torch.Generator().manual_seed(21)
        x = (-2.3 + 0.5 * torch.randn((9, 768), generator=g)).to(xdt)
        w = torch.rand((768,), generator=g).to(wdt)
        norm = T5LayerNorm(768, eps=1e-6)
        with torch.no_grad():
            norm.weight = torch.nn.Parameter(w)
            y = norm._forward(x)
        rn[tag + "_x"] = x.float().numpy()
        rn[tag + "_w"] = w.float().numpy()
        rn[tag + "_y"] = y.float().numpy()
        rn[tag + "_ydtype"] = np.asarray(str(y.dtype))
    np.savez_compressed(os.path.join(here, "rmsnorm.npz"), **rn)

    # ---------------------------------------------------------------- padding
    lens = [5, 0, 9, 3, 9]
    mask = torch.zeros((5, 9), dtype=torch.int64)
    for i, n in enumerate(lens):
        mask[i, :n] = 1
    idx, cu, mx = _get_unpad_data(mask)
    vals = seeded((int(cu[-1]), 2, 4), 31)
    padded = pad_input(vals, idx, 5, 9)
    np.savez_compressed(os.path.join(here, "padding.npz"), mask=mask.numpy(), indices=idx.numpy(),
                        cu_seqlens=cu.numpy(), max_seqlen=np.asarray(mx), values=vals.numpy(),
                        padded=padded.numpy())
    # ------------------------------------------------------------ tiny enc-dec stack
    # the reference's full model ('basic' attention on CPU) with name-seeded weights: encoder
    # output, teacher-forced logits and four greedy steps through its tuple K/V cache
    sys.path.insert(0, os.path.dirname(os.path.dirname(here)))
    from tests.helpers import TINY_T5, seed_named_parameters, tiny_t5_inputs
    from transformers.modeling_utils import PreTrainedModel
    from turbot5 import T5ForConditionalGeneration
    from turbot5.model import modeling
    _orig = PreTrainedModel.get_extended_attention_mask

    def _gem(self, attention_mask, input_shape, device=None, dtype=None):
        if isinstance(device, torch.dtype):
            dtype, device = device, None
        return _orig(self, attention_mask, input_shape, dtype=dtype)
    modeling.T5PreTrainedModel.get_extended_attention_mask = _gem
    modeling.T5PreTrainedModel.get_head_mask = lambda self, hm, n, *a: [None] * n
    cfg = T5Config(feed_forward_proj="gated-gelu", attention_type="basic", use_triton=False, dropout_rate=0.0,
                   tie_word_embeddings=False, **TINY_T5)
    model = T5ForConditionalGeneration(cfg).eval()
    model.encoder.config.attention_type = "full"      # broadcastable mask handling in the encoder stack
    seed_named_parameters(model, 0)
    ids, dec = tiny_t5_inputs()
    mask = torch.ones_like(ids)
    mask[1, 29:] = 0
    with torch.no_grad():
        enc = model.encoder(input_ids=ids)
        logits = model(input_ids=ids, decoder_input_ids=dec).logits
        enc_m = model.encoder(input_ids=ids, attention_mask=mask)
        logits_m = model(input_ids=ids, attention_mask=mask, decoder_input_ids=dec).logits
        cur = torch.zeros((2, 1), dtype=torch.long)
        pkv, toks, step_logits = None, [], []
        for _ in range(4):
            o = model(encoder_outputs=enc, decoder_input_ids=cur, past_key_values=pkv, use_cache=True)
            pkv = o.past_key_values
            step_logits.append(o.logits[:, -1])
            cur = o.logits[:, -1:].argmax(-1)
            toks.append(cur)
    np.savez_compressed(os.path.join(here, "stack.npz"), encoder=enc.last_hidden_state.numpy(),
                        logits=logits.numpy(), encoder_masked=enc_m.last_hidden_state.numpy(),
                        logits_masked=logits_m.numpy(), mask=mask.numpy(),
                        greedy_tokens=torch.cat(toks, 1).numpy(), greedy_logits=torch.stack(step_logits, 1).numpy(),
                        param_names=np.asarray(sorted(n for n, _ in model.named_parameters())))
    print("golden fixtures written to", here)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference [local_masked]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else None)
