"""File formats either side of the hot path: the `.sx8v43` container and the interleaved
30-byte block_sx8 records of the GGUF files.  Fixtures were written by the reference's own
code (tests/golden/make_golden_formats.py)."""
import os

import numpy as np
import pytest

from oracle import sx8_oracle as orc
from sx8_quantization_b200 import sx8_container_v43 as cont

GATE = "model.layers.0.mlp.gate_proj.weight"
KPROJ = "model.layers.0.self_attn.k_proj.weight"


@pytest.fixture(scope="module")
def small(golden_dir):
    return dict(np.load(os.path.join(golden_dir, "small_case.npz")))


@pytest.fixture(scope="module")
def golden_file(golden_dir):
    return os.path.join(golden_dir, "small.sx8v43")


def test_container_index_matches_reference_file(golden_file, small):
    c = cont.Container(golden_file)
    assert c.names() == [GATE, KPROJ]
    assert c.meta == {"format": "sx8_v4_3", "model": "synthetic-small", "n_bases": 2}
    qt, bi = c.tensor(GATE)
    assert qt["shape"] == (48, 80) and qt["orig_shape"] is None and qt["n_blocks"] == 144 and qt["n_cb"] == 3
    for k in ("dmin", "dmax", "config", "levels_hi", "levels_lo"):
        assert np.array_equal(np.asarray(qt[k]), small[k]), k
    assert np.array_equal(np.asarray(qt["coeff"]), small["coeff"].reshape(-1))
    assert np.array_equal(bi["data"], small["data"]) and np.array_equal(bi["scales"], small["scales"])
    qt2, _ = c.tensor(KPROJ)
    assert qt2["shape"] == (16, 80) and qt2["orig_shape"] == (4, 4, 80) and qt2["n_blocks"] == 48
    assert np.array_equal(np.asarray(qt2["levels_hi"]), small["levels_hi"][:48 * 16])


def test_container_writer_is_byte_identical(golden_file, tmp_path):
    wd, bd, meta = cont.read_all(golden_file)
    # orig_shape None is written as the 2-D shape, as the reference does
    out = tmp_path / "again.sx8v43"
    cont.write_sx43({"weights": wd, "bases": bd, "meta": meta}, str(out), verbose=False)
    assert out.read_bytes() == open(golden_file, "rb").read()
    assert cont.verify_sx43({"weights": wd, "bases": bd, "meta": meta}, str(out))


def test_container_rejects_damaged_files(golden_file, tmp_path):
    raw = open(golden_file, "rb").read()
    bad = tmp_path / "bad_magic.sx8v43"
    bad.write_bytes(b"SX42FILE" + raw[8:])
    with pytest.raises(cont.ContainerError):
        cont.Container(str(bad))
    short = tmp_path / "short.sx8v43"
    short.write_bytes(raw[:len(raw) // 2])
    with pytest.raises(cont.ContainerError):
        cont.Container(str(short))
    ver = tmp_path / "ver.sx8v43"
    ver.write_bytes(raw[:8] + b"\x07" + raw[9:])
    with pytest.raises(cont.ContainerError):
        cont.Container(str(ver))
    evil = tmp_path / "meta.sx8v43"       # metadata that is code, not a literal: refused, not run
    payload = b"__import__('os').getcwd()"
    import struct
    evil.write_bytes(raw[:9] + struct.pack("<I", len(payload)) + payload + raw[13 + struct.unpack("<I", raw[9:13])[0]:])
    with pytest.raises(cont.ContainerError):
        cont.Container(str(evil))


def test_oracle_blocks_match_reference_blockify(golden_dir, golden_file):
    want = np.load(os.path.join(golden_dir, "small_blocks.npz"))["blocks"]
    qt, _ = cont.Container(golden_file).tensor(GATE)
    got = orc.blocks_from_planes(qt)
    assert got.shape == (144, 30) and np.array_equal(got, want)
    back = orc.planes_from_blocks(want, (48, 80))
    for k in ("dmin", "dmax", "config", "levels_hi", "levels_lo", "coeff"):
        assert np.array_equal(np.asarray(back[k]).reshape(-1).view(np.uint8), np.asarray(qt[k]).reshape(-1).view(np.uint8)), k


# ------------------------------------------------------------------------------- GPU
@pytest.mark.gpu
def test_gpu_blocks_roundtrip_and_repack(golden_dir, golden_file):
    import torch
    from sx8_quantization_b200 import ops
    want = np.load(os.path.join(golden_dir, "small_blocks.npz"))["blocks"]
    qt, bi = cont.Container(golden_file).tensor(GATE)
    dev = torch.device("cuda:0")
    pl = {k: torch.from_numpy(np.array(qt[k])).to(dev) for k in ("dmin", "dmax", "config", "coeff", "levels_hi", "levels_lo")}
    blocks = ops.blocks_from_planes(pl["dmin"], pl["dmax"], pl["config"], pl["coeff"], pl["levels_hi"], pl["levels_lo"])
    assert np.array_equal(blocks.cpu().numpy(), want)
    back = ops.planes_from_blocks(torch.from_numpy(want).to(dev))
    for k in pl:
        assert torch.equal(back[k].view(torch.uint8).reshape(-1), pl[k].view(torch.uint8).reshape(-1)), k
    t16_a = ops.repack_t16(pl["dmin"], pl["dmax"], pl["config"], pl["coeff"], pl["levels_hi"], pl["levels_lo"], 48, 3)
    t16_b = ops.repack_t16_blocks(blocks, 48, 3)
    assert torch.equal(t16_a, t16_b)
    assert np.array_equal(t16_a.cpu().numpy().reshape(-1), orc.to_t16(qt).reshape(-1))


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(256, 2560), (100, 1000)])
def test_gpu_blocks_seeded(shape):
    import torch
    from sx8_quantization_b200 import ops
    n, k = shape
    qt, bi = orc.quantize(orc.synth_weight(n, k, seed=31))
    dev = torch.device("cuda:0")
    pl = {kk: torch.from_numpy(np.ascontiguousarray(qt[kk]).reshape(-1)).to(dev)
          for kk in ("dmin", "dmax", "config", "coeff", "levels_hi", "levels_lo")}
    blocks = ops.blocks_from_planes(pl["dmin"], pl["dmax"], pl["config"], pl["coeff"], pl["levels_hi"], pl["levels_lo"])
    assert np.array_equal(blocks.cpu().numpy(), orc.blocks_from_planes(qt))
    assert torch.equal(ops.repack_t16_blocks(blocks, n, qt["n_cb"]),
                       ops.repack_t16(pl["dmin"], pl["dmax"], pl["config"], pl["coeff"], pl["levels_hi"], pl["levels_lo"], n, qt["n_cb"]))
    back = ops.planes_from_blocks(blocks)
    for kk in pl:
        assert torch.equal(back[kk].view(torch.uint8).reshape(-1), pl[kk].view(torch.uint8).reshape(-1)), kk


@pytest.mark.gpu
def test_gpu_load_container_to_device(golden_file, small):
    import torch
    from sx8_quantization_b200 import ops
    ts = cont.load_to_device(golden_file, device="cuda:0")
    assert sorted(ts) == [GATE, KPROJ]
    c = cont.Container(golden_file)
    for name in (GATE, KPROJ):
        qt, bi = c.tensor(name)
        t = ts[name]
        assert np.array_equal(t["wt16"].cpu().numpy().reshape(-1), orc.to_t16(qt).reshape(-1))
        assert np.array_equal(t["bases"].cpu().numpy(), bi["data"])
        w_ref = orc.dequant_d64(qt, bi)
        w = ops.dequant_t16(t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], True)
        assert np.array_equal(w.cpu().numpy().view(np.uint16), w_ref.view(np.uint16))
    t = ts[GATE]
    x = torch.from_numpy(orc.synth_x(2, 80, seed=5)).to("cuda:0")
    y = ops.gemv(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"]).cpu().numpy()
    qt, bi = c.tensor(GATE)
    ref = orc.matmul_ref(orc.synth_x(2, 80, seed=5), orc.dequant_d64(qt, bi))
    assert np.abs(y - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max())
