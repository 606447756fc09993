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
