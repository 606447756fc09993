"""End-to-end decoder on S-X8 linears: prefill against a float32 PyTorch model built from the
dequantised weights, cache consistency, and graph replay against eager stepping."""
import pytest

pytestmark = pytest.mark.gpu

SMALL = dict(layers=2, hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512, vocab=512, rope_theta=1.0e4, eps=1.0e-6)


def _reference_logits(dec, ids):
    """Float32 forward over the whole sequence with dequantised weights; last-position logits."""
    import torch
    import torch.nn.functional as F
    from sx8_quantization_b200 import ops
    from sx8_quantization_b200.decoder import _rope
    c = dec.cfg
    W = lambda t: ops.dequant_t16(t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], True).float()
    B, T = ids.shape
    D, hq, hkv = c["head_dim"], c["n_q"], c["n_kv"]
    h = W(dec.embed)[ids.reshape(-1)]
    norm = lambda z: F.rms_norm(z, (z.shape[-1],), dec.gamma, c["eps"])
    cos, sin = dec.cos[:T][None, :, None, :], dec.sin[:T][None, :, None, :]
    for L in dec.layers:
        x = norm(h)
        q = _rope((x @ W(L["q"]).t()).view(B, T, hq, D), cos, sin).transpose(1, 2)
        k = _rope((x @ W(L["k"]).t()).view(B, T, hkv, D), cos, sin).transpose(1, 2)
        v = (x @ W(L["v"]).t()).view(B, T, hkv, D).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True).transpose(1, 2).reshape(B * T, hq * D)
        h = h + a @ W(L["o"]).t()
        x = norm(h)
        h = h + (F.silu(x @ W(L["gate"]).t()) * (x @ W(L["up"]).t())) @ W(L["down"]).t()
    return norm(h.view(B, T, -1)[:, -1]) @ W(dec.lm_head).t()


@pytest.mark.parametrize("batch", [1, 2])
def test_prefill_matches_float32_model(batch):
    import torch
    from sx8_quantization_b200.decoder import SX8Decoder
    dec = SX8Decoder(SMALL, seed=3, max_seq=64, batch=batch)
    g = torch.Generator(device="cuda").manual_seed(5)
    ids = torch.randint(0, SMALL["vocab"], (batch, 24), generator=g, device="cuda")
    got = dec.prefill(ids)
    ref = _reference_logits(dec, ids)
    assert torch.isfinite(got).all()
    # fp16 activations between the linears, fp16-rounded weights inside the GEMM
    assert (got - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()


def test_cached_decode_matches_recomputed_prefill_and_graph_matches_eager():
    import torch
    from sx8_quantization_b200.decoder import SX8Decoder
    dec = SX8Decoder(SMALL, seed=4, max_seq=64, batch=1)
    g = torch.Generator(device="cuda").manual_seed(6)
    ids = torch.randint(0, SMALL["vocab"], (1, 16), generator=g, device="cuda")
    toks_eager, _ = dec.generate(ids, 8, use_graph=False)
    toks_graph, t = dec.generate(ids, 8, use_graph=True)
    assert torch.equal(toks_eager, toks_graph)
    assert t["decode_ms_per_token"] > 0
    # the logits of a cached step equal, within fp16 noise, those of a prefill over the longer prompt
    dec.prefill(ids)
    step_logits = dec._step()
    longer = torch.cat([ids, toks_eager[:, :1]], dim=1)
    full_logits = dec.prefill(longer)
    assert (step_logits - full_logits).abs().max().item() <= 2e-2 * full_logits.abs().max().item()


def test_batch_above_eight_uses_the_gemm_path():
    import torch
    from sx8_quantization_b200.decoder import SX8Decoder
    dec = SX8Decoder(SMALL, seed=5, max_seq=48, batch=12)
    g = torch.Generator(device="cuda").manual_seed(7)
    ids = torch.randint(0, SMALL["vocab"], (12, 8), generator=g, device="cuda")
    got = dec.prefill(ids)
    ref = _reference_logits(dec, ids)
    assert (got - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    toks, _ = dec.generate(ids, 4, use_graph=True)
    assert toks.shape == (12, 4)


@pytest.mark.parametrize("batch", [1, 3, 12])
def test_fused_glue_step_matches_pytorch_glue(batch):
    import torch
    from sx8_quantization_b200.decoder import SX8Decoder
    dec = SX8Decoder(SMALL, seed=6, max_seq=40, batch=batch)
    g = torch.Generator(device="cuda").manual_seed(8)
    ids = torch.randint(0, SMALL["vocab"], (batch, 20), generator=g, device="cuda")
    outs = {}
    for fused in (False, True):
        dec.fused_glue = fused
        dec.prefill(ids)
        logits = [dec._step().clone() for _ in range(3)]
        outs[fused] = torch.stack(logits)
    ref, got = outs[False], outs[True]
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()


def test_glue_kernels_against_pytorch():
    import torch
    import torch.nn.functional as F
    from sx8_quantization_b200 import ops
    from sx8_quantization_b200.decoder import _rope
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(9)
    B, H, hq, hkv, D, S = 3, 320, 8, 2, 128, 96
    h = torch.randn(B, H, generator=g, device=dev)
    y = torch.randn(B, H, generator=g, device=dev)
    gamma = torch.rand(H, generator=g, device=dev) + 0.5
    x = torch.empty(B, H, dtype=torch.float16, device=dev)
    h2 = h.clone()
    ops.glue_add_rmsnorm(h2, y, gamma, 1e-6, x)
    assert torch.allclose(h2, h + y)
    want = F.rms_norm(h + y, (H,), gamma, 1e-6)
    assert (x.float() - want).abs().max().item() <= 2e-3 * want.abs().max().item()
    # rope + cache + attention at position 37
    pos = torch.tensor([37], device=dev)
    q = torch.randn(B, hq * D, generator=g, device=dev)
    k = torch.randn(B, hkv * D, generator=g, device=dev)
    v = torch.randn(B, hkv * D, generator=g, device=dev)
    kc = torch.randn(B, hkv, S, D, generator=g, device=dev).half()
    vc = torch.randn(B, hkv, S, D, generator=g, device=dev).half()
    inv = 1.0 / (1.0e4 ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))
    ang = torch.arange(S, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q16 = torch.empty(B, hq * D, dtype=torch.float16, device=dev)
    ops.glue_rope_cache(q, k, v, pos, cos, sin, hq, hkv, D, q16, kc, vc)
    qr = _rope(q.view(B, hq, D), cos[37][None, None], sin[37][None, None]).half()
    kr = _rope(k.view(B, hkv, D), cos[37][None, None], sin[37][None, None]).half()
    kc_ref[:, :, 37] = kr
    vc_ref[:, :, 37] = v.view(B, hkv, D).half()
    assert torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)
    assert (q16.view(B, hq, D).float() - qr.float()).abs().max().item() <= 2e-3
    out = torch.empty(B, hq * D, dtype=torch.float16, device=dev)
    scale = D ** -0.5
    scratch = ops.glue_attn_scratch(B, hq, hkv, D, dev)
    for _ in range(2):   # twice: the arrival counters must come back to zero
        out.zero_()
        ops.glue_attn_decode(q16, kc, vc, pos, hq, hkv, D, scale, out, scratch)
    grp = hq // hkv
    s = torch.matmul(q16.view(B, hkv, grp, D).float(), kc[:, :, :38].float().transpose(-1, -2)) * scale
    want = torch.matmul(torch.softmax(s, -1), vc[:, :, :38].float()).reshape(B, hq * D)
    assert (out.float() - want).abs().max().item() <= 3e-3 * max(1.0, want.abs().max().item())
    # swiglu
    a, b2 = torch.randn(B, 1000, generator=g, device=dev), torch.randn(B, 1000, generator=g, device=dev)
    act = torch.empty(B, 1000, dtype=torch.float16, device=dev)
    ops.glue_silu_mul(a, b2, act)
    assert (act.float() - F.silu(a) * b2).abs().max().item() <= 2e-3 * 4


def test_captured_prefill_equals_eager_prefill():
    """The prefill replayed from its CUDA graph gives the eager prefill's bits, for a second
    prompt of the same shape too, and leaves the same cache and decode state."""
    import torch
    from sx8_quantization_b200.decoder import SX8Decoder
    dec = SX8Decoder(SMALL, seed=5, max_seq=64, batch=2)
    g = torch.Generator(device="cuda").manual_seed(8)
    for _ in range(2):
        ids = torch.randint(0, SMALL["vocab"], (2, 24), generator=g, device="cuda")
        want = dec.prefill(ids).clone()
        k_want, tok_want = dec.k_cache.clone(), dec.tok.clone()
        dec.k_cache.zero_()
        got = dec.prefill_captured(ids)
        assert torch.equal(got, want)
        assert torch.equal(dec.k_cache, k_want) and torch.equal(dec.tok, tok_want) and int(dec.pos.item()) == 24
