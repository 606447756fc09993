"""The reference's own Python code running on the GPU on top of, and beside, this library.

The reference's modules come from oracle/_ref/pyc/ (byte-compiled by `python oracle/build.py
--ref` where the checkout is; sourceless, so they travel without the reference's text) or,
when that directory is absent, from the checkout's scripts/ directory.  Three things are pinned here:

  * the caller: the reference's unmodified integrate_fused_v44.SX8LinearV44
    (ref scripts/integrate_fused_v44.py:28-77) built on the drop-in modules that
    sx8_quantization_b200.launch.register() installs, forward at M = 1, M > 1 and with
    SX8_USE_WMMA=1, against the CPU oracle;
  * the float64 decoder: the reference's numba-CUDA sx8_v43_kernel / decode_tensor_gpu_fast
    (ref scripts/kernel_sx8_v43.py:14-51,109-145) against sx8_dequant_planes, sx8_dequant_t16
    and the C oracle, bit for bit;
  * the quantizer search on torch-CUDA: the reference's chunked_v6_encode / pack_levels_6bit
    (ref scripts/quantize_qwen35_4b_sx8_v43_gpu.py:22-69,148-167) with DEV = cuda against
    sx8_quantize_blocks, byte for byte.
"""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import build as obuild  # noqa: E402
from oracle import sx8_oracle as orc  # noqa: E402

TOL = 2e-3


def import_reference_caller():
    """launch.register() first, then the reference's module by its bare name."""
    pytest.importorskip("numba")
    from sx8_quantization_b200 import launch
    launch.register()
    if not obuild.install_ref_finder():
        root = obuild.ref_root()
        if root is None:
            pytest.skip("reference modules not staged (run `python oracle/build.py --ref` where the checkout is)")
        d = os.path.join(root, "scripts")
        if d not in sys.path:
            sys.path.insert(0, d)
    import integrate_fused_v44
    return integrate_fused_v44


def test_reference_caller_imports_on_top_of_the_drop_ins():
    """CPU: the unmodified module resolves every hot-path import to this package."""
    m = import_reference_caller()
    pkg = "sx8_quantization_b200."
    assert m.decode1_v44.__module__ == pkg + "sx8_decode1_v3"
    assert m.make_tensors_v44.__module__ == pkg + "sx8_decode1_v3"
    assert m.gemm_sx8_compact.__module__ == pkg + "sx8_gemm_compact"
    assert m.gemm_sx8_wmma_cached.__module__ == pkg + "sx8_fused_wmma"
    assert m.SX8EmbeddingV44.__module__ == pkg + "sx8_embed_v44"
    assert m.SX8LinearV44.__module__ == "integrate_fused_v44"            # the reference's class, not ours
    import integrate_fused
    assert integrate_fused.decode_tensor_gpu_fast.__module__ == pkg + "kernel_sx8_v43"
    assert issubclass(m.SX8LinearV44, integrate_fused.SX8Linear)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1024, 2560), (136, 1000)])
def test_reference_sx8linearv44_forward(shape, monkeypatch):
    m = import_reference_caller()
    out_f, in_f = shape
    qt, bi = orc.quantize(orc.synth_weight(out_f, in_f, 301), with_pca=True)
    w = orc.dequant_d64(qt, bi)
    bias = torch.from_numpy((np.random.default_rng(1).standard_normal(out_f) * 0.1).astype(np.float16)).cuda()
    monkeypatch.delenv("SX8_USE_WMMA", raising=False)

    def check(lin, x_np, b):
        y = lin(torch.from_numpy(x_np).cuda())
        assert y.dtype == torch.float16 and tuple(y.shape) == tuple(x_np.shape[:-1]) + (out_f,)
        ref = orc.matmul_ref(x_np.reshape(-1, in_f), w)
        if b is not None:
            ref = ref + b.float().cpu().numpy()[None, :]
        got = y.float().cpu().numpy().reshape(-1, out_f)
        assert np.isfinite(got).all()
        assert np.abs(got - ref).max() <= (TOL + 2.0 ** -10) * np.abs(ref).max()   # + the caller's y.half()

    for b in (None, bias):
        lin = m.SX8LinearV44(qt, bi, b, out_f, in_f)                # ref scripts/integrate_fused_v44.py:31-35
        check(lin, orc.synth_x(1, in_f, 11).reshape(1, 1, in_f), b)      # M == 1 -> decode1_v44
        assert lin._t44 is not None and lin._tensors is None            # only the compact tensors were built
        check(lin, orc.synth_x(64, in_f, 12).reshape(2, 32, in_f), b)    # M != 1 -> gemm_sx8_compact
        check(lin, orc.synth_x(5, in_f, 13), b)                          # 2-D input, small M
        assert lin._tensors is None
    monkeypatch.setenv("SX8_USE_WMMA", "1")
    lin = m.SX8LinearV44(qt, bi, None, out_f, in_f)
    check(lin, orc.synth_x(64, in_f, 14).reshape(1, 64, in_f), None)     # -> make_tensors(kb-major) + wmma_cached
    assert lin._tensors is not None and "_t16" in lin._tensors
    check(lin, orc.synth_x(1, in_f, 15), None)                           # M == 1 still takes decode1_v44
    # the parent class on the same drop-ins (ref scripts/integrate_fused.py:30-79)
    import integrate_fused
    lin0 = integrate_fused.SX8Linear(qt, bi, None, out_f, in_f)
    check(lin0, orc.synth_x(1, in_f, 16).reshape(1, 1, in_f), None)      # -> decode1_sx8_cached
    check(lin0, orc.synth_x(40, in_f, 17), None)                         # -> gemm_sx8_wmma_cached
    from sx8_quantization_b200 import _lib
    assert _lib.device_error_flag() == 0


def _ref_numba_decoder():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    pytest.importorskip("numba")
    mod = obuild.load_ref_py("kernel_sx8_v43", alias="ref_kernel_sx8_v43")
    if mod is None:
        pytest.skip("reference modules not staged (run `python oracle/build.py --ref` where the checkout is)")
    return mod


def _numba_decode(mod, qt, bi):
    try:
        return mod.decode_tensor_gpu_fast(qt, bi)
    except Exception as e:      # numba cannot compile for or run on this GPU: say why
        pytest.skip("the reference's numba-CUDA decoder does not run here: %r" % (e,))


@pytest.mark.gpu
def test_float64_decoder_pinned_against_the_reference_numba_kernel(golden_dir):
    """Bit-exact dequantised weights: the reference's real decoder (numba-CUDA, float64
    arithmetic by its typing rules) on this GPU against both library entry points and the C
    oracle, on the golden 48 x 80 case, on every block kind, and on BASELINE config 0."""
    from sx8_quantization_b200 import ops
    from test_exhaustive_blocks import exhaustive_case
    mod = _ref_numba_decoder()
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    g = dict(np.load(os.path.join(golden_dir, "small_case.npz")))
    small = ({"shape": (48, 80), "n_blocks": g["levels"].shape[0], "n_cb": 3, "dmin": g["dmin"], "dmax": g["dmax"],
              "config": g["config"], "levels_hi": g["levels_hi"], "levels_lo": g["levels_lo"], "coeff": g["coeff"]},
             {"n_cb": 3, "data": g["data"], "scales": g["scales"]})
    qe, be, _ = exhaustive_case()
    big = orc.quantize(orc.synth_weight(9728, 2560, 100), with_pca=True)
    for name, (qt, bi) in (("golden", small), ("exhaustive", (qe, be)), ("config0", big)):
        out_f, in_f = qt["shape"]
        with np.errstate(over="ignore"):
            W_ref = _numba_decode(mod, qt, bi)
        torch.cuda.synchronize()
        ref_bits = W_ref.view(torch.int16)
        planes = (d(qt["dmin"].view(np.uint8)), d(qt["dmax"].view(np.uint8)), d(qt["config"]),
                  d(np.asarray(qt["coeff"]).reshape(-1)), d(qt["levels_hi"]), d(qt["levels_lo"]))
        bas, sca = d(np.asarray(bi["data"], np.float32).reshape(-1, 64)), d(np.asarray(bi["scales"], np.float32).reshape(-1, 2))
        a = ops.dequant_planes(*planes, bas, sca, out_f, in_f, qt["n_cb"], True)
        wt = ops.repack_t16(*planes, out_f, qt["n_cb"])
        b = ops.dequant_t16(wt, bas, sca, out_f, in_f, qt["n_cb"], True)
        na = int((a.view(torch.int16) != ref_bits).sum().item())
        nb = int((b.view(torch.int16) != ref_bits).sum().item())
        c = torch.from_numpy(orc.dequant_d64(qt, bi)).cuda()
        nc = int((c.view(torch.int16) != ref_bits).sum().item())
        assert (na, nb, nc) == (0, 0, 0), "%s: fp16 words differing from the reference decoder: planes %d, t16 %d, C oracle %d of %d" % (
            name, na, nb, nc, out_f * in_f)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(48, 80), (1024, 2560), (9728, 2560)])
def test_quantizer_search_against_the_reference_on_torch_cuda(shape):
    """The reference quantizer runs on torch-CUDA (ref quantize_qwen35_4b_sx8_v43_gpu.py:9);
    its per-tensor loop body (ref :235-264) with DEV = cuda against sx8_quantize_blocks."""
    from sx8_quantization_b200 import ops
    ns = obuild.load_ref_quantizer(torch.device("cuda"))
    if ns is None:
        pytest.skip("reference modules not staged (run `python oracle/build.py --ref` where the checkout is)")
    out_f, in_f = shape
    w16 = torch.from_numpy(orc.synth_weight(out_f, in_f, 100)).cuda()
    W = w16.float()
    n_cb = (in_f + 31) // 32
    pad = (32 - in_f % 32) % 32
    if pad:
        W = torch.nn.functional.pad(W, (0, pad))
    blocks = W.reshape(out_f, n_cb, 32).reshape(-1, 32).contiguous()
    lv, dm, dx, cf = ns["chunked_v6_encode"](blocks)
    hi, lo = ns["pack_levels_6bit"](lv.cpu().numpy().astype(np.uint8).reshape(-1, 32))
    q = ops.quantize_blocks(w16, want_levels=True, arith="cuda")
    torch.cuda.synchronize()
    n_blk = out_f * n_cb
    mism = {
        "levels": int((q["levels"] != lv.to(torch.uint8).reshape(-1, 32)).sum().item()),
        "config": int((q["config"] != cf.to(torch.uint8)).sum().item()),
        "dmin": int((q["dmin"].view(torch.int16) != dm.half().view(torch.int16)).sum().item()),
        "dmax": int((q["dmax"].view(torch.int16) != dx.half().view(torch.int16)).sum().item()),
        "levels_hi": int((q["levels_hi"].cpu().numpy() != hi).sum()),
        "levels_lo": int((q["levels_lo"].cpu().numpy() != lo).sum()),
    }
    assert not any(mism.values()), "bytes differing from the reference on torch-CUDA (%d blocks): %r" % (n_blk, mism)
    # and the oracle's restatement of the same arithmetic
    lv_o, _, _, cf_o = orc.quant_search(orc.to_blocks(w16.cpu().numpy())[0], "cuda")
    assert np.array_equal(lv_o, lv.cpu().numpy().astype(np.uint8).reshape(-1, 32))
    assert np.array_equal(cf_o.astype(np.uint8), cf.cpu().numpy().astype(np.uint8))
    # the torch-CPU arithmetic (golden fixtures) differs from it only in a few levels per 10,000
    q_cpu = ops.quantize_blocks(w16, want_levels=True, arith="cpu")
    frac = (q_cpu["levels"] != q["levels"]).float().mean().item()
    assert frac < 1e-3


@pytest.mark.gpu
def test_reference_clone_model_fused_v44_on_a_transformers_model():
    """The reference's own end-to-end check (ref scripts/integrate_fused_v44.py:119-167:
    logits of the model with fp16 dequantised weights against the model whose Linear /
    Embedding modules were swapped by clone_model_fused_v44, accepted at max|diff| / max|ref|
    < 5e-2) restated on a small random-init Qwen3-shaped transformers model: the reference's
    unmodified clone_model_fused_v44 installs SX8LinearV44 / SX8EmbeddingV44 built on the drop-in
    modules; a 16-token prompt runs the M > 1 path (gemm_sx8_compact), a cached single-token
    step the M == 1 path (decode1_v44)."""
    transformers = pytest.importorskip("transformers")
    m = import_reference_caller()
    from transformers import Qwen3Config, Qwen3ForCausalLM
    torch.manual_seed(7)
    cfg = Qwen3Config(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=64, max_position_embeddings=128, tie_word_embeddings=False)
    ref_model = Qwen3ForCausalLM(cfg).half().eval()
    wd, bd = {}, {}
    sd = ref_model.state_dict()
    for name, p in list(ref_model.named_parameters()):
        if p.dim() < 2:
            continue
        w16 = (p.detach().float() * (0.02 / max(1e-6, p.detach().float().std().item()))).half().numpy()
        qt, bi = orc.quantize(w16, with_pca=True)
        wd[name], bd[name] = qt, bi
        sd[name] = torch.from_numpy(orc.dequant_d64(qt, bi))          # the reference model holds the decoded weights
    ref_model.load_state_dict(sd)
    import copy
    fused = copy.deepcopy(ref_model)
    ref_model = ref_model.cuda()
    fused, n_rep = m.clone_model_fused_v44(fused, wd, bd)
    assert n_rep == len(wd) == 2 * 7 + 2                                   # every Linear, the embedding and lm_head
    fused = fused.cuda().eval()
    assert type(fused.model.layers[0].self_attn.q_proj).__name__ == "SX8LinearV44"
    assert type(fused.model.embed_tokens).__module__ == "sx8_quantization_b200.sx8_embed_v44"
    ids = torch.randint(0, 1000, (1, 16), device="cuda")
    with torch.no_grad():
        a = ref_model(input_ids=ids, use_cache=True)
        b = fused(input_ids=ids, use_cache=True)
        rel = ((a.logits.float() - b.logits.float()).abs().max() / a.logits.float().abs().max()).item()
        assert rel < 2e-2, rel                                             # the reference accepts 5e-2
        nxt = a.logits[:, -1].argmax(-1, keepdim=True)
        a1 = ref_model(input_ids=nxt, past_key_values=a.past_key_values, use_cache=True)
        b1 = fused(input_ids=nxt, past_key_values=b.past_key_values, use_cache=True)
        rel1 = ((a1.logits.float() - b1.logits.float()).abs().max() / a1.logits.float().abs().max()).item()
        assert rel1 < 2e-2, rel1
    from sx8_quantization_b200 import _lib
    assert _lib.device_error_flag() == 0
