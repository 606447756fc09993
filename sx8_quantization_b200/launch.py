"""Run an unmodified script of the reference on top of this library.

The reference's callers (scripts/infer_sx8.py, integrate_fused_v44.py,
bench_decode_v44_v2.py) put their own scripts/ directory first on sys.path and
`import sx8_decode1_v3` etc. by bare name.  Registering this package's drop-in modules
under those names in sys.modules before the script starts makes every such import
resolve here.

    python -m sx8_quantization_b200.launch /path/to/reference/scripts/infer_sx8.py [args...]
"""
import importlib
import runpy
import sys

DROP_IN = ("sx8_decode1_v3", "sx8_gemm_compact", "sx8_fused_wmma", "sx8_embed_v44", "kernel_sx8_v43",
           "sx8_container_v43")


def register():
    for name in DROP_IN:
        sys.modules[name] = importlib.import_module("sx8_quantization_b200." + name)
    return [sys.modules[n] for n in DROP_IN]


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit(__doc__)
    register()
    sys.argv = argv
    runpy.run_path(argv[0], run_name="__main__")


if __name__ == "__main__":
    main()
