"""Generate the file-format fixtures under tests/golden/ with the REFERENCE's own code
(run where the reference checkout is; its path comes from SX8_REF):

  small.sx8v43        two tensors of small_case.npz written by the reference's
                      scripts/sx8_container_v43.py:write_sx43 (from a temporary pkl).
  small_blocks.npz    the same tensor as interleaved 30-byte block_sx8 records, made by
                      blockify_vec of scripts/convert_pkl_to_gguf_sx8.py (the function is
                      taken out of the script's syntax tree: the script imports a GGUF
                      writer that is not part of the reference).

    python tests/golden/make_golden_formats.py
"""
import ast
import os
import pickle
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import build as _ob  # noqa: E402

REF = _ob.ref_root()   # $SX8_REF, else the path BASELINE.json records
if not REF:
    sys.exit("set SX8_REF to the reference checkout")


def tensors_from_small_case():
    g = np.load(os.path.join(HERE, "small_case.npz"))
    n_cb = 3
    qt = {"shape": (48, 80), "orig_shape": (48, 80), "n_blocks": 48 * n_cb, "n_cb": n_cb,
          "dmin": g["dmin"], "dmax": g["dmax"], "config": g["config"], "levels_hi": g["levels_hi"],
          "levels_lo": g["levels_lo"], "coeff": g["coeff"]}
    bi = {"n_cb": n_cb, "data": g["data"], "scales": g["scales"]}
    # a second tensor: the first 16 rows, stored with a 3-D original shape as the
    # reference does for reshaped tensors
    nb = 16 * n_cb
    qt2 = {"shape": (16, 80), "orig_shape": (4, 4, 80), "n_blocks": nb, "n_cb": n_cb,
           "dmin": g["dmin"][:nb].copy(), "dmax": g["dmax"][:nb].copy(), "config": g["config"][:nb].copy(),
           "levels_hi": g["levels_hi"][:nb * 16].copy(), "levels_lo": g["levels_lo"][:nb * 8].copy(),
           "coeff": g["coeff"][:nb].copy()}
    return {"model.layers.0.mlp.gate_proj.weight": (qt, bi), "model.layers.0.self_attn.k_proj.weight": (qt2, bi)}


def main():
    sys.path.insert(0, os.path.join(REF, "scripts"))
    import sx8_container_v43 as ref_container
    tensors = tensors_from_small_case()
    meta = {"format": "sx8_v4_3", "model": "synthetic-small", "n_bases": 2}
    with tempfile.TemporaryDirectory() as td:
        pkl = os.path.join(td, "small.pkl")
        pickle.dump({"weights": {k: v[0] for k, v in tensors.items()},
                     "bases": {k: v[1] for k, v in tensors.items()}, "meta": meta}, open(pkl, "wb"))
        out = os.path.join(HERE, "small.sx8v43")
        ref_container.write_sx43(pkl, out, verbose=False)
        assert ref_container.verify_sx43(pkl, out)

    src = open(os.path.join(REF, "scripts", "convert_pkl_to_gguf_sx8.py")).read()
    fn = [n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "blockify_vec"]
    ns = {"np": np}
    exec(compile(ast.Module(body=fn, type_ignores=[]), "ref_blockify", "exec"), ns)
    qt = tensors["model.layers.0.mlp.gate_proj.weight"][0]
    np.savez_compressed(os.path.join(HERE, "small_blocks.npz"), blocks=ns["blockify_vec"](qt))
    print("wrote small.sx8v43 (%d bytes), small_blocks.npz" % os.path.getsize(os.path.join(HERE, "small.sx8v43")))


if __name__ == "__main__":
    main()
