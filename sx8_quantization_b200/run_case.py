"""Run ONE kernel of the library on one synthetic tensor and print its CUDA-event time:

    python -m sx8_quantization_b200.run_case gemm --N 9728 --K 2560 --M 2048
    python -m sx8_quantization_b200.run_case gemv --N 151936 --K 2560 --M 1

Meant for profilers (one shape, a handful of launches, a few hundred MB on the device) and
for quick A/B timing of a launch-shape change.  The weight is the seeded synthetic
distribution N(0, 0.02) with 0.1 % outliers, quantised on the device with PCA."""
import argparse
import json

import torch

from . import _lib, ops, quantizer


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemv", "gemm", "embed", "dequant", "quantize"])
    ap.add_argument("--N", type=int, default=9728)
    ap.add_argument("--K", type=int, default=2560)
    ap.add_argument("--M", type=int, default=1, help="batch rows (gemv <= 8; gemm any; embed: rows gathered)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default="f16", choices=["f16", "f32"], help="gemm output type")
    ap.add_argument("--seed", type=int, default=3)
    a = ap.parse_args(argv)
    dev = torch.device("cuda:0")
    N, K, M = a.N, a.K, a.M
    w = quantizer.synth_weight_gpu(N, K, a.seed, device=dev)
    g = torch.Generator(device=dev).manual_seed(a.seed + 1)
    if a.kernel == "quantize":
        fn = lambda: ops.quantize_blocks(w)
        units, unit = N * ((K + 31) // 32), "blocks"
    else:
        t = quantizer.quantize_tensor(w, with_pca=True)
        del w
        n_cb = t["n_cb"]
        x = torch.randn(M, K, generator=g, device=dev).half()
        if a.kernel == "gemv":
            y = torch.empty(M, N, dtype=torch.float32, device=dev)
            fn = lambda: ops.gemv(x, t["wt16"], t["bases"], t["scales"], N, K, n_cb, out=y)
            units, unit = N * n_cb * 30, "packed bytes"
        elif a.kernel == "gemm":
            od = torch.float16 if a.out == "f16" else torch.float32
            y = torch.empty(M, N, dtype=od, device=dev)
            fn = lambda: ops.gemm(x, t["wt16"], t["bases"], t["scales"], N, K, n_cb, out_dtype=od, out=y)
            units, unit = 2 * M * N * K, "flop"
        elif a.kernel == "embed":
            ids = torch.randint(0, N, (M,), generator=g, device=dev, dtype=torch.int32)
            fn = lambda: ops.embed(ids, t["wt16"], t["bases"], t["scales"], K, N, n_cb)
            units, unit = M, "rows"
        else:
            fn = lambda: ops.dequant_t16(t["wt16"], t["bases"], t["scales"], N, K, n_cb, True)
            units, unit = N * n_cb * 30, "packed bytes"
    for _ in range(a.warmup):
        fn()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    us = e0.elapsed_time(e1) * 1e3 / a.iters
    flag = _lib.device_error_flag()
    print(json.dumps({"kernel": a.kernel, "N": N, "K": K, "M": M, "us_per_call": round(us, 2),
                      "per_second": units / (us * 1e-6), "unit": unit + "/s", "device_error_flag": flag}))
    if flag:
        raise SystemExit("device error flag 0x%x" % flag)


if __name__ == "__main__":
    main()
