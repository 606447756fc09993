"""Generate the golden fixtures under tests/golden/ by running the REFERENCE's own
code on CPU.  Run where the reference checkout is (its path comes from SX8_REF); the
fixtures it writes are committed, the reference is not.

What is imported from the reference, unmodified:
  * scripts/quantize_qwen35_4b_sx8_v43_gpu.py -- the script touches a GPU and a model
    path at import, so its four pure functions (v6_encode_6bit_gpu, chunked_v6_encode,
    pca_correct_gpu, pack_levels_6bit; lines 22-167) are taken out of its syntax tree
    and executed with DEV = cpu and the module constants it defines at lines 6-8.
  * scripts/prepare_v44.py -- imported as a module (to_v44, extract_levels_v43/v44,
    decode_v44_numpy).

Outputs:
  small_case.npz      a 48 x 80 matrix (K padded to 96) with special rows; every
                      reference output stored in full.
  checksums.json      sha256 of every reference output for seeded matrices up to the
                      BASELINE config-0 size (9728 x 2560); tests regenerate the
                      matrix from the seed and compare digests.

    python tests/golden/make_golden.py
"""
import ast
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import sx8_oracle as orc  # noqa: E402  (synthetic generators only)

from oracle import build as _ob  # noqa: E402

REF = _ob.ref_root()   # $SX8_REF, else the path BASELINE.json records
if not REF:
    sys.exit("set SX8_REF to the reference checkout")


def load_ref_quantizer():
    src = open(os.path.join(REF, "scripts", "quantize_qwen35_4b_sx8_v43_gpu.py")).read()
    tree = ast.parse(src)
    want = {"v6_encode_6bit_gpu", "chunked_v6_encode", "pca_correct_gpu", "pack_levels_6bit"}
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in want]
    assert len(body) == 4
    ns = dict(torch=torch, np=np, DEV=torch.device("cpu"), B=32, L63=63, N_BASES=4,
              MAX_BLOCKS_PER_CHUNK=3_000_000)
    exec(compile(ast.Module(body=body, type_ignores=[]), "ref_quantizer", "exec"), ns)
    return ns


def load_ref_prepare():
    sys.path.insert(0, os.path.join(REF, "scripts"))
    import prepare_v44
    return prepare_v44


def ref_quantize(ns, w16, with_pca=True):
    """The reference's per-tensor loop body (quantize...py:235-272) on CPU."""
    out_f, in_f = w16.shape
    W = torch.from_numpy(w16.astype(np.float32))
    n_cb = (in_f + 31) // 32
    pad = (32 - in_f % 32) % 32
    if pad:
        W = torch.nn.functional.pad(W, (0, pad))
    blocks = W.reshape(out_f, n_cb, 32).reshape(-1, 32).contiguous()
    lv, dm, dx, cf = ns["chunked_v6_encode"](blocks)
    if with_pca:
        coeff, bl, sl = ns["pca_correct_gpu"](lv, dm, dx, cf, blocks, n_cb)
        data = np.array([b.flatten() for b in bl], dtype=np.float32)
        scales = np.array(sl, dtype=np.float32)
    else:
        coeff = np.zeros((blocks.shape[0], 1), np.uint8)
        data = np.zeros((n_cb, 64), np.float32)
        scales = np.zeros((n_cb, 2), np.float32)
    lv_cpu = lv.numpy().astype(np.uint8).reshape(-1, 32)
    hi, lo = ns["pack_levels_6bit"](lv_cpu)
    qt = {"shape": (out_f, in_f), "orig_shape": (out_f, in_f), "n_blocks": blocks.shape[0],
          "n_cb": n_cb, "dmin": dm.numpy().astype(np.float16), "dmax": dx.numpy().astype(np.float16),
          "config": cf.numpy().astype(np.uint8), "levels_hi": hi, "levels_lo": lo, "coeff": coeff}
    bi = {"n_cb": n_cb, "data": data, "scales": scales}
    raw = {"levels": lv_cpu, "dmin32": dm.numpy(), "dmax32": dx.numpy(), "config32": cf.numpy()}
    return qt, bi, raw


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def small_matrix():
    w = orc.synth_weight(48, 80, seed=11).astype(np.float32)
    w[3, :] = 0.0                      # all-zero row: dmin == dmax == 0
    w[4, :] = 0.0123                   # constant row: degenerate range
    w[5, :32] = np.linspace(-1, 1, 32)  # wide block
    w[6, 40:48] = 3.0                  # outlier sub-block (quarter strategies)
    w[7, :] = -np.abs(w[7, :])         # all-negative
    w[8, :] = np.abs(w[8, :])          # all-positive
    w[9, ::2] = 6.0e-8                 # fp16 subnormal spacing
    w[9, 1::2] = 0.0
    w[10, :] = 60000.0 * np.sign(w[10, :] + 1e-9)  # near fp16 max
    return w.astype(np.float16)


def main():
    ns = load_ref_quantizer()
    pv = load_ref_prepare()

    # ---- small case, everything stored
    w = small_matrix()
    qt, bi, raw = ref_quantize(ns, w)
    v6 = pv.to_v44(qt, bi, hdr_aligned=False)
    v8 = pv.to_v44(qt, bi, hdr_aligned=True)
    lv43 = pv.extract_levels_v43(qt)
    lv44 = pv.extract_levels_v44(v6)
    x = orc.synth_x(1, 96, seed=12, scale=0.5)[0].astype(np.float32)
    cols = np.array([0, 3, 4, 5, 6, 9, 10, 47])
    y_cols = np.array([pv.decode_v44_numpy(v6, x, int(n)) for n in cols], dtype=np.float64)
    np.savez_compressed(
        os.path.join(HERE, "small_case.npz"),
        w=w, levels=raw["levels"], dmin32=raw["dmin32"], dmax32=raw["dmax32"],
        config32=raw["config32"], dmin=qt["dmin"], dmax=qt["dmax"], config=qt["config"],
        levels_hi=qt["levels_hi"], levels_lo=qt["levels_lo"], coeff=qt["coeff"],
        data=bi["data"], scales=bi["scales"], hdr6=v6["hdr"], hdr8=v8["hdr"],
        levels44=v6["levels"], lv43=lv43, lv44=lv44, x=x, cols=cols, y_cols=y_cols)

    # ---- seeded matrices, digests only
    cases = [("tiny_64x256", 64, 256, 21), ("kv_slice_256x2560", 256, 2560, 22),
             ("odd_k_128x1000", 128, 1000, 23), ("config0_gate_9728x2560", 9728, 2560, 100)]
    out = {}
    for name, n, k, seed in cases:
        w = orc.synth_weight(n, k, seed)
        qt, bi, raw = ref_quantize(ns, w, with_pca=False)
        v6 = pv.to_v44(qt, bi)
        out[name] = {
            "out_f": n, "in_f": k, "seed": seed, "w": sha(w), "levels": sha(raw["levels"]),
            "dmin": sha(qt["dmin"]), "dmax": sha(qt["dmax"]), "config": sha(qt["config"]),
            "levels_hi": sha(qt["levels_hi"]), "levels_lo": sha(qt["levels_lo"]),
            "hdr6": sha(v6["hdr"]), "levels44": sha(v6["levels"]),
            "strategy_hist": np.bincount(((qt["config"][:, None] >> np.array([0, 2, 4, 6])) & 3).ravel(),
                                         minlength=4).tolist(),
        }
        print(name, out[name]["strategy_hist"])
    json.dump({"torch": torch.__version__, "numpy": np.__version__, "cases": out},
              open(os.path.join(HERE, "checksums.json"), "w"), indent=1)


if __name__ == "__main__":
    main()
