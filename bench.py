"""Benchmark of the S-X8 v4.3 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1  workload `gemv_sweep_qwen3_4b` (BASELINE config 1): one step = the decode GEMVs of
       a whole Qwen3-4B-shaped model (36 distinct layers x {q,k,v,o,gate,up,down} +
       lm_head, 3.77 GB of packed weights -- larger than L2, so no flush is needed) at
       batch 1, 2, 4 and 8, replayed from CUDA graphs with programmatic dependent
       launch.  metric = packed weight bytes streamed per second (GB/s).
N > 1  workload `tp_decode_llama70b` (BASELINE config 4): Llama-70B-shaped layers as
       column/row tensor-parallel S-X8 linears with an NCCL all-reduce after the two
       row-parallel projections; strong scaling; same metric, aggregated over ranks.

The JSON line carries `roofline` (HBM bound, measured peak from MEASURED_PEAKS.json),
`cpu_baseline` (the oracle's dequant + matmul on the host cores, bounded sample),
`e2e` (same sweep through the drop-in Python wrapper with pinned host buffers, copies
inside the timed region) and `clocks` (nvidia-smi samples during the timed region).
`--impl reference` times the reference's CPU path (oracle port) on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only without MEASURED_PEAKS.json
BATCHES = (1, 2, 4, 8)
# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes for one gemv launch (ncu, lm_head)
NCU_TRAFFIC_RATIO = 1.012


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi samples (read-only query) taken while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0, period_ms=100):
        self.samples = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", str(period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.monotonic(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self, t0, t1):
        rows = [s for t, s in self.samples if t0 <= t <= t1 + 0.15]
        if not rows:
            rows = [s for _, s in self.samples[-2:]]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            f = [x.strip() for x in r.split(",")]
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except Exception:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------- model set-up

def build_model(family, n_layers, device, seed0=1000, with_pca=True, shard=None):
    """Random-init weights of `family`, quantised on the device.  shard = (rank, world):
    quantise the full matrix, then keep this rank's column or row shard (so that shards
    are byte-identical to slices of the single-GPU tensors)."""
    import torch
    from sx8_quantization_b200 import quantizer, tp
    layers = []
    for li in range(n_layers):
        mats = {}
        for pi, (name, N, K, style) in enumerate(family["proj"]):
            w = quantizer.synth_weight_gpu(N, K, seed0 + li * 16 + pi, device)
            t = quantizer.quantize_tensor(w, with_pca=with_pca)
            del w
            if shard is not None and shard[1] > 1:
                t = tp.shard_tensor(t, style, shard[0], shard[1])
            mats[name] = t
        layers.append(mats)
    torch.cuda.synchronize()
    return layers


def build_lm_head(family, device, seed, with_pca=True, shard=None):
    from sx8_quantization_b200 import quantizer, tp
    w = quantizer.synth_weight_gpu(family["vocab"], family["hidden"], seed, device)
    t = quantizer.quantize_tensor(w, with_pca=with_pca)
    del w
    if shard is not None and shard[1] > 1:
        t = tp.shard_tensor(t, "col", shard[0], shard[1])
    return t


def tensor_bytes(t):
    """Algorithmic packed bytes: 30 per block (the T16 blob pads N to a multiple of 16)."""
    return 30 * t["N"] * t["n_cb"]


# ------------------------------------------------------------------------- N = 1

def run_single(args):
    import numpy as np
    import torch
    from sx8_quantization_b200 import ops, model_shapes as ms
    from sx8_quantization_b200 import sx8_decode1_v3 as drop_in
    fam = ms.QWEN3_4B
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n_layers = args.layers if args.layers > 0 else fam["layers"]
    layers = build_model(fam, n_layers, dev, with_pca=True)
    head = build_lm_head(fam, dev, 999, with_pca=True)
    mats = [(name, L[name]) for L in layers for name, _, _, _ in fam["proj"]] + [("lm_head", head)]
    bytes_pass = sum(tensor_bytes(t) for _, t in mats)
    g = torch.Generator(device=dev).manual_seed(5)
    xs = {}
    for M in BATCHES:
        for K in sorted({t["K"] for _, t in mats}):
            xs[(M, K)] = torch.randn(M, K, generator=g, device=dev).half()
    ys = {(M, t["N"]): torch.empty(M, t["N"], dtype=torch.float32, device=dev) for M in BATCHES for _, t in mats}
    ws = ops.Workspace.get(dev, max(t["n_cb"] for _, t in mats) * 512)

    def one_pass(M, flags):
        for _, t in mats:
            ops.gemv(xs[(M, t["K"])], t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                     out=ys[(M, t["N"])], flags=flags, workspace=ws)

    flags = 0 if args.no_pdl else ops.SX8_F_PDL
    st = torch.cuda.Stream(device=dev)
    graphs = {}
    with torch.cuda.stream(st):
        for M in BATCHES:
            one_pass(M, flags)
        st.synchronize()
        if not args.no_graph:
            for M in BATCHES:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=st):
                    one_pass(M, flags)
                graphs[M] = gr

    def step():
        for M in BATCHES:
            if graphs:
                graphs[M].replay()
            else:
                one_pass(M, flags)

    sampler = ClockSampler(0)
    with torch.cuda.stream(st):
        for _ in range(args.warmup):
            step()
        st.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(BATCHES) + 1)]
        per_batch = {M: 0.0 for M in BATCHES}
        torch.cuda.synchronize()
        t0 = time.monotonic()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(st)
        marks = []
        for k in range(args.steps):
            if k == args.steps - 1:   # per-batch split on the last step only (events are cheap but not free)
                ev[0].record(st)
            for i, M in enumerate(BATCHES):
                if graphs:
                    graphs[M].replay()
                else:
                    one_pass(M, flags)
                if k == args.steps - 1:
                    ev[i + 1].record(st)
        e1.record(st)
        st.synchronize()
        torch.cuda.synchronize()
        t1 = time.monotonic()
    total_ms = e0.elapsed_time(e1)
    for i, M in enumerate(BATCHES):
        per_batch[M] = ev[i].elapsed_time(ev[i + 1])
    ms_per_step = total_ms / args.steps
    bytes_step = bytes_pass * len(BATCHES)
    value = bytes_step / (ms_per_step * 1e-3) / 1e9
    clocks = sampler.summary(t0, t1)

    # ---- per-shape kernel rate, each shape rotating over its distinct per-layer copies
    per_shape = {}
    with torch.cuda.stream(st):
        for name, N, K, _ in fam["proj"] + [("lm_head", fam["vocab"], fam["hidden"], "col")]:
            group = [t for nm, t in mats if nm == name]
            reps = max(1, (256 << 20) // max(1, sum(tensor_bytes(t) for t in group)))
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=st):
                for _ in range(reps):
                    for t in group:
                        ops.gemv(xs[(1, K)], t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                                 out=ys[(1, N)], flags=flags, workspace=ws)
            gr.replay(); st.synchronize()
            a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
            a.record(st)
            for _ in range(5):
                gr.replay()
            b.record(st); st.synchronize()
            n_launch = 5 * reps * len(group)
            us = a.elapsed_time(b) * 1e3 / n_launch
            per_shape[name] = {"N": N, "K": K, "us_per_launch": round(us, 3),
                               "GBps": round(tensor_bytes(group[0]) / us / 1e3, 1),
                               "resident_copies": len(group)}

    # ---- the same pass with the projections that share their input fused into one launch
    #      (q|k|v and gate|up: 4 launches per layer instead of 7), batch 1
    fused = None
    if not args.no_extras:
        mq = [ops.MultiGemv([L["q"], L["k"], L["v"]], 1, dev) for L in layers]
        mg = [ops.MultiGemv([L["gate"], L["up"]], 1, dev) for L in layers]

        def fused_pass():
            for L, a, b in zip(layers, mq, mg):
                a(xs[(1, L["q"]["K"])], flags=flags, workspace=ws)
                t = L["o"]
                ops.gemv(xs[(1, t["K"])], t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                         out=ys[(1, t["N"])], flags=flags, workspace=ws)
                b(xs[(1, L["gate"]["K"])], flags=flags, workspace=ws)
                t = L["down"]
                ops.gemv(xs[(1, t["K"])], t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                         out=ys[(1, t["N"])], flags=flags, workspace=ws)
            t = head
            ops.gemv(xs[(1, t["K"])], t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                     out=ys[(1, t["N"])], flags=flags, workspace=ws)

        with torch.cuda.stream(st):
            fused_pass(); st.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=st):
                fused_pass()
            for _ in range(3):
                gr.replay()
            st.synchronize()
            a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
            a.record(st)
            for _ in range(20):
                gr.replay()
            b.record(st); st.synchronize()
        fms = a.elapsed_time(b) / 20
        fused = {"ms_per_pass": round(fms, 4), "GBps": round(bytes_pass / (fms * 1e-3) / 1e9, 1),
                 "launches_per_layer": 4, "frac_of_hbm": round(bytes_pass / (fms * 1e-3) / 1e9 / peaks()[0], 4)}

    # ---- the other rows of the hot path (BASELINE configs 2 and 4): prefill GEMM, quantizer,
    #      embedding rows, full-tensor decode -- short device-timed loops, reported as extras
    extras = {} if args.no_extras else other_kernels(dev, layers[0], head, fam)

    # ---- e2e: the drop-in wrapper with pinned host buffers, copies inside the timed region
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    xh = {k: v.cpu().pin_memory() for k, v in xs.items()}
    yh = {k: torch.empty(v.shape, dtype=torch.float32).pin_memory() for k, v in ys.items()}
    xd = {k: torch.empty_like(v) for k, v in xs.items()}
    h2d = sum(xs[(M, t["K"])].numel() * 2 for M in BATCHES for _, t in mats)
    d2h = sum(M * t["N"] * 4 for M in BATCHES for _, t in mats)

    def e2e_step():
        for M in BATCHES:
            for _, t in mats:
                x = xd[(M, t["K"])]
                x.copy_(xh[(M, t["K"])], non_blocking=True)
                Y, _ = drop_in.decode1_v44(x, {"n_cb": t["n_cb"], "shape": (t["N"], t["K"])}, None, None,
                                           t["wt16"], t["bases"], t["scales"], 6)
                yh[(M, t["N"])].copy_(Y, non_blocking=True)
        torch.cuda.synchronize()

    e2e_step()
    a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(e2e_steps):
        e2e_step()
    b.record(); torch.cuda.synchronize()
    e2e_ms = a.elapsed_time(b) / e2e_steps
    e2e_val = bytes_step / (e2e_ms * 1e-3) / 1e9
    sampler.stop()

    peak, peak_kind = peaks()
    n_gemv = len(mats) * len(BATCHES)
    from sx8_quantization_b200 import _lib
    flag = _lib.device_error_flag()
    line = {
        "metric": "sx8_decode_gemv_weight_GBps", "value": round(value, 1), "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 x u6 -> f32 accumulate",
        "data": "synthetic (random-init N(0,0.02) + 0.1% x10 outliers, quantised on the device)",
        "config": {"workload": "gemv_sweep_qwen3_4b", "layers": n_layers, "batches": list(BATCHES),
                   "matrices_per_pass": len(mats), "packed_bytes_per_pass": bytes_pass,
                   "l2": "inputs larger than L2 (%.2f GB of distinct packed weights per pass)" % (bytes_pass / 1e9),
                   "cuda_graph": not args.no_graph, "pdl": not args.no_pdl},
        "per_batch_GBps": {str(M): round(bytes_pass / (per_batch[M] * 1e-3) / 1e9, 1) for M in BATCHES},
        "tok_per_s_equiv_batch1": round(1e3 / per_batch[1], 1) if n_layers == fam["layers"] else None,
        "per_shape_batch1": per_shape,
        "gpu_launches": n_gemv * args.steps,
        "device_error_flag": flag,
        "roofline": {"bound": "hbm", "achieved": round(value, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(value / peak, 4),
                     "traffic": int(NCU_TRAFFIC_RATIO * bytes_pass / len(mats)),
                     "note": "achieved = packed weight bytes / wall time of the whole graph-replayed step "
                             "(every gemv kernel and the launch gaps between them included), of %s peak; traffic = "
                             "DRAM bytes per average launch: the ncu capture of the lm_head launch read+wrote "
                             "%.3f x its algorithmic bytes, scaled by bytes to the average launch of the step"
                             % (peak_kind, NCU_TRAFFIC_RATIO)},
        "e2e": {"value": round(e2e_val, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(e2e_ms, 3), "steps": e2e_steps,
                "api": "sx8_decode1_v3.decode1_v44 with pinned host x and y"},
        "clocks": clocks,
        "fused_projections_batch1": fused,
        "other_kernels": extras,
        "e2e_decoder_qwen3_4b": None if (args.no_extras or args.no_decoder) else decoder_e2e(dev),
    }
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(budget_s=args.cpu_seconds)
    print(json.dumps(line))


def _time_us(fn, iters=10, warm=3):
    import torch
    for _ in range(warm):
        fn()
    a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record(); torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def decoder_e2e(dev, prompt=512, new=256):
    """BASELINE config 3: random-init Qwen3-4B-shaped decoder, every linear and the embedding
    in S-X8; a prompt of uniform random ids, then greedy decode with the step in one CUDA
    graph, at batch 1 (GEMV path) and batch 32 (tensor-core GEMM path)."""
    import torch
    from sx8_quantization_b200.decoder import SX8Decoder, QWEN3_4B_DECODER
    out = {"prompt_tokens": prompt, "new_tokens": new, "glue": "decode step: sx8_glue kernels (nine launches per layer); prefill: PyTorch"}
    for batch in (1, 32):
        dec = SX8Decoder(QWEN3_4B_DECODER, device=dev, seed=9, max_seq=prompt + new, batch=batch)
        g = torch.Generator(device=dev).manual_seed(1234)
        ids = torch.randint(0, QWEN3_4B_DECODER["vocab"], (batch, prompt), generator=g, device=dev)
        dec.generate(ids, 8)                       # warm-up: allocations, graph capture
        toks, t = dec.generate(ids, new)
        out["batch%d" % batch] = {
            "prefill_ms": round(t["prefill_ms"], 2), "prefill_tok_per_s": round(batch * prompt / t["prefill_ms"] * 1e3, 1),
            "decode_ms_per_step": round(t["decode_ms_per_token"], 4),
            "decode_tok_per_s": round(batch / t["decode_ms_per_token"] * 1e3, 1),
            "weight_GBps_decode": round(dec.packed_bytes / (t["decode_ms_per_token"] * 1e-3) / 1e9, 1),
            "distinct_tokens": int(toks.unique().numel())}
        del dec
        torch.cuda.empty_cache()
    return out


def other_kernels(dev, layer0, head, fam):
    """Prefill GEMM on the gate projection (M = 128 .. 8192, f16 out), quantizer search,
    embedding gather and full-tensor decode; fractions are of the measured peaks."""
    import torch
    from sx8_quantization_b200 import ops, quantizer
    out = {}
    pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"bf16_tflops": 1590.0, "hbm_gbs": FALLBACK_HBM_GBS}
    t = layer0["gate"]
    g = torch.Generator(device=dev).manual_seed(77)
    gem = {}
    for M in (128, 512, 2048, 8192):
        x = torch.randn(M, t["K"], generator=g, device=dev).half()
        y = torch.empty(M, t["N"], dtype=torch.float16, device=dev)
        us = _time_us(lambda: ops.gemm(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                                       out_dtype=torch.float16, out=y))
        tf = 2.0 * M * t["N"] * t["K"] / us / 1e6
        gem[str(M)] = {"us": round(us, 1), "TFLOPs": round(tf, 1), "frac_of_bf16_burst": round(tf / pk["bf16_tflops"], 3)}
        del x, y
    out["prefill_gemm_gate_9728x2560"] = gem
    w = quantizer.synth_weight_gpu(t["N"], t["K"], 4242, dev)
    us = _time_us(lambda: ops.quantize_blocks(w))
    n_blk = t["N"] * t["n_cb"]
    out["quantizer_search"] = {"us": round(us, 1), "Mblocks_per_s": round(n_blk / us, 1),
                               "GBps_in_plus_out": round(n_blk * (64 + 29) / us / 1e3, 1),
                               "frac_of_hbm": round(n_blk * (64 + 29) / us / 1e3 / pk["hbm_gbs"], 3)}
    us = _time_us(lambda: quantizer.quantize_tensor(w, with_pca=True), iters=3, warm=1)
    out["quantizer_full_with_pca"] = {"us": round(us, 1), "Mblocks_per_s": round(n_blk / us, 1)}
    del w
    ids = torch.randint(0, head["N"], (512,), generator=g, device=dev)
    o = torch.empty(512, head["K"], dtype=torch.float16, device=dev)
    us = _time_us(lambda: ops.embed(ids, head["wt16"], head["bases"], head["scales"], head["K"], head["N"],
                                    head["n_cb"], out=o))
    out["embed_512_rows"] = {"us": round(us, 1), "GBps": round(512 * head["K"] * (30 / 32 + 2) / us / 1e3, 1)}
    us = _time_us(lambda: ops.dequant_t16(t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], True))
    out["dequant_gate"] = {"us": round(us, 1), "GBps": round(n_blk * (30 + 64) / us / 1e3, 1),
                           "frac_of_hbm": round(n_blk * (30 + 64) / us / 1e3 / pk["hbm_gbs"], 3)}
    return out


# ------------------------------------------------------------------------- CPU legs

_CPU_CACHE = {}


def cpu_baseline(budget_s=12.0):
    """The reference's CPU-runnable comparator (ref scripts/sx8_decode1_v3.py:130-131):
    full-tensor dequantisation followed by X.float() @ W.float().t(), timed on the host
    cores with the oracle port.  Sample: the gate projection (9728 x 2560), batch 1."""
    import numpy as np
    import torch
    from oracle import sx8_oracle as orc
    from sx8_quantization_b200 import model_shapes as ms
    N, K = 9728, 2560
    torch.set_num_threads(os.cpu_count() or 1)
    if "case" not in _CPU_CACHE:
        w = orc.synth_weight(N, K, 100)
        _CPU_CACHE["case"] = orc.quantize(w, with_pca=False)
    qt, bi = _CPU_CACHE["case"]
    x = torch.from_numpy(orc.synth_x(1, K, 3))
    ts = []
    t_end = time.monotonic() + budget_s
    while len(ts) < 3 or (time.monotonic() < t_end and len(ts) < 50):
        t0 = time.perf_counter()
        W = torch.from_numpy(orc.dequant_d64(qt, bi))
        y = x.float() @ W.float().t()
        ts.append(time.perf_counter() - t0)
    med = sorted(ts)[len(ts) // 2]
    return {"value": round(ms.packed_bytes(N, K) / med / 1e9, 4), "unit": "GB/s", "cores": os.cpu_count(),
            "kind": "port", "threads": orc.num_threads(),
            "sample": "gate projection 9728x2560, batch 1, dequant (C oracle, OpenMP) + torch fp32 matmul, "
                      "median of %d calls, %.1f ms per call" % (len(ts), med * 1e3)}


def run_reference(args):
    """--impl reference: the reference's CPU path on the host cores (oracle port; the
    reference has no CPU inference path of its own, its comparator is dequant + matmul)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ts = []
    for i in range(args.warmup + args.steps):
        c = cpu_baseline(budget_s=1.0)
        if i >= args.warmup:
            ts.append(c["value"])
    v = sum(ts) / len(ts)
    c["value"] = round(v, 4)
    n = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    print(json.dumps({
        "impl": "reference", "metric": "sx8_decode_gemv_weight_GBps", "value": round(v, 4), "unit": "GB/s",
        "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(30 * 9728 * 80 / (v * 1e9) * 1e3, 3),   # one call of the sample (gate projection)
        "higher_is_better": True,
        "scaling": "weak" if n == 1 else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gemv_sweep_qwen3_4b" if n == 1 else "tp_decode_llama70b",
                   "sample": c["sample"]},
        "cpu_baseline": c,
        "e2e": {"value": round(v, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------- N > 1

def run_tp(args, rank, world, local_rank):
    """Llama-70B-shaped tensor-parallel decode: q,k,v (column) -> o (row, all-reduce) ->
    gate, up (column) -> down (row, all-reduce) per layer; every rank streams its shard.
    Strong scaling: the model is fixed, the shard shrinks with N."""
    import torch
    import torch.distributed as dist
    from sx8_quantization_b200 import ops, tp, model_shapes as ms
    fam = ms.LLAMA_70B
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    n_layers = args.layers if args.layers > 0 else 4
    # --emulate-world W on one GPU: time rank 0's shard of a W-way split without any exchange
    shard_world = args.emulate_world if (world == 1 and args.emulate_world > 1) else world
    layers = build_model(fam, n_layers, dev, with_pca=True, shard=(rank, shard_world))
    batches = (1, 8)
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    bytes_rank = sum(tensor_bytes(t) for L in layers for t in L.values())
    xs, ys = {}, {}
    for M in batches:
        for L in layers[:1]:
            for name, t in L.items():
                xs[(M, name)] = torch.randn(M, t["K"], generator=g, device=dev).half()
                ys[(M, name)] = torch.zeros(M, t["N"], dtype=torch.float32, device=dev)
    ws = ops.Workspace.get(dev, max(t["n_cb"] for L in layers for t in L.values()) * 512)
    flags = 0 if args.no_pdl else ops.SX8_F_PDL
    exchange = None
    if world > 1 and args.allreduce == "fused":
        try:
            exchange = tp.PeerExchange(8 * fam["hidden"], dev)
        except Exception as e:
            if rank == 0:
                print("peer exchange unavailable, using NCCL:", repr(e)[:300], file=sys.stderr)
            exchange = None

    def one_pass(M):
        for L in layers:
            for name, _, _, style in fam["proj"]:
                t = L[name]
                if style == "row" and world > 1:
                    tp.linear(xs[(M, name)], t, out=ys[(M, name)], flags=flags, exchange=exchange)
                else:
                    ops.gemv(xs[(M, name)], t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                             out=ys[(M, name)], flags=flags, workspace=ws)

    st = torch.cuda.Stream(device=dev)
    graphs = {}
    with torch.cuda.stream(st):
        for M in batches:
            one_pass(M)
        st.synchronize()
        if not args.no_graph:
            try:
                for M in batches:
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr, stream=st):
                        one_pass(M)
                    graphs[M] = gr
            except Exception as e:  # NCCL capture unavailable: run eagerly and say so
                graphs = {}
                if rank == 0:
                    print("graph capture failed, running eagerly:", repr(e)[:200], file=sys.stderr)

    def step():
        for M in batches:
            if graphs:
                graphs[M].replay()
            else:
                one_pass(M)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    with torch.cuda.stream(st):
        for _ in range(args.warmup):
            step()
        st.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.monotonic()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        eb = torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for k in range(args.steps):
            if graphs:
                graphs[batches[0]].replay()
            else:
                one_pass(batches[0])
            if k == args.steps - 1:
                eb.record(st)
            if graphs:
                graphs[batches[1]].replay()
            else:
                one_pass(batches[1])
        e1.record(st)
        st.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t1 = time.monotonic()
    ms_local = e0.elapsed_time(e1) / args.steps

    # ---- e2e: the same pass through the public tp.linear call, activations coming from pinned
    #      host memory every step and the last projection's result read back
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    xh = {k: v.cpu().pin_memory() for k, v in xs.items()}
    last = fam["proj"][-1][0]
    yh = {M: torch.empty(M, layers[0][last]["N"], dtype=torch.float32).pin_memory() for M in batches}
    h2d = sum(v.numel() * 2 for v in xs.values()) * n_layers
    d2h = sum(v.numel() * 4 for v in yh.values())

    def e2e_step():
        for M in batches:
            for L in layers:
                for name, _, _, style in fam["proj"]:
                    xs[(M, name)].copy_(xh[(M, name)], non_blocking=True)
                    y = tp.linear(xs[(M, name)], L[name], out=ys[(M, name)], flags=flags, exchange=exchange)
            yh[M].copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    e2e_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(e2e_steps):
        e2e_step()
    b.record(); torch.cuda.synchronize()
    e2e_ms = a.elapsed_time(b) / e2e_steps

    tm = torch.tensor([ms_local, e2e_ms], device=dev, dtype=torch.float64)
    tb = torch.tensor([float(bytes_rank)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(tb, op=dist.ReduceOp.SUM)
    ms_per_step = float(tm[0].item())
    e2e_ms = float(tm[1].item())
    bytes_step = float(tb.item()) * len(batches)
    value = bytes_step / (ms_per_step * 1e-3) / 1e9
    if rank == 0:
        clocks = sampler.summary(t0, t1)
        sampler.stop()
        peak, peak_kind = peaks()
        n_gemv = n_layers * len(fam["proj"]) * len(batches)
        full_layer = ms.layer_bytes(fam)
        from sx8_quantization_b200 import _lib
        line = {
            "metric": "sx8_decode_gemv_weight_GBps", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 x u6 -> f32 accumulate", "data": "synthetic (random-init, quantised on the device)",
            "config": {"workload": "tp_decode_llama70b", "layers": n_layers, "batches": list(batches),
                       "parallelism": "tp%d" % world if shard_world == world else "rank 0 of tp%d, no exchange" % shard_world,
                       "allreduce": ("fused into the GEMV epilogue over peer memory (fp32, rank-ordered sum)"
                                     if exchange is not None else "nccl fp32 sum") + " after o and down",
                       "packed_bytes_per_layer": full_layer,
                       "l2": "per-rank weights %.0f MB (> L2 when above 126 MB)" % (bytes_rank / 1e6),
                       "cuda_graph": bool(graphs), "pdl": not args.no_pdl},
            "tok_per_s_80_layers_equiv": round(1e3 / (ms_per_step / len(batches)) * n_layers / fam["layers"], 2),
            "gpu_launches": n_gemv * args.steps,
            "device_error_flag": _lib.device_error_flag(),
            "roofline": {"bound": "hbm", "achieved": round(value / world, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(value / world / peak, 4), "traffic": None,
                         "note": "per-GPU packed weight bytes / step wall time incl. all-reduces, of %s peak" % peak_kind},
            "e2e": {"value": round(bytes_step / (e2e_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 3),
                    "steps": e2e_steps, "api": "tp.linear per projection, pinned host activations, NCCL all-reduce"},
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    # Tear-down: drop the captured graphs (they hold NCCL kernels) before leaving, and leave
    # with a hard exit after a last barrier -- destroying the NCCL communicator while graphs
    # that captured its collectives are still alive can block forever.
    graphs.clear()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def _watchdog(seconds):
    """Abort the process if the whole run takes longer than `seconds` (a hung collective or
    tear-down must not hold the GPUs)."""
    import signal

    def _die(signum, frame):
        sys.stderr.write("bench.py: watchdog expired after %d s, aborting\n" % seconds)
        sys.stderr.flush()
        os._exit(3)

    signal.signal(signal.SIGALRM, _die)
    signal.alarm(int(seconds))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "gemv_sweep_qwen3_4b", "tp_decode_llama70b"])
    ap.add_argument("--layers", type=int, default=0, help="distinct layers resident (0 = workload default)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the GEMM / quantizer / embed / dequant extras")
    ap.add_argument("--no-decoder", action="store_true", help="skip the end-to-end decoder leg")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="single GPU: run rank 0's shard of a W-way tensor-parallel split, no exchange")
    ap.add_argument("--allreduce", default="fused", choices=["fused", "nccl"],
                    help="row-parallel reduction: fused peer-memory exchange or NCCL")
    ap.add_argument("--max-seconds", type=int, default=900, help="watchdog for the whole run")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    _watchdog(args.max_seconds)
    if args.impl == "reference":
        return run_reference(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = args.workload
    if wl == "auto":
        wl = "gemv_sweep_qwen3_4b" if world == 1 and args.gpus == 1 else "tp_decode_llama70b"
    if wl == "gemv_sweep_qwen3_4b":
        if rank == 0:
            run_single(args)
    else:
        run_tp(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
