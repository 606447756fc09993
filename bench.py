"""Benchmark of the S-X8 v4.3 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --case gemv|gemm|embed|dequant|quantize --N .. --K .. --M ..   (one kernel, one shape)

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

    # ---- reference kernels on this GPU, beside ours
    refk = None
    if not args.no_extras:
        try:
            refk = ref_kernels_same_box(dev, fam, per_shape, extras.get("prefill_gemm", {}).get("gate_up_9728x2560", {}))
        except Exception as e:  # the checker's kernels are optional evidence, never part of the product path
            refk = {"unavailable": repr(e)[:300]}

    # ---- e2e: the same sweep through the drop-in API (sx8_decode1_v3.decode1_v44, one call per
    #      projection, eager launches), a decode step's data flow: every step its activations
    #      come from pinned host memory (one copy per distinct input) and the step's result --
    #      the lm_head logits of every batch -- is read back into pinned host memory.  The
    #      projections' outputs stay on the device, as they do between the layers of a decoder.
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    xh = {k: v.cpu().pin_memory() for k, v in xs.items()}
    xd = {k: torch.empty_like(v) for k, v in xs.items()}
    yh = {M: torch.empty(M, head["N"], dtype=torch.float32).pin_memory() for M in BATCHES}
    h2d = sum(v.numel() * 2 for v in xs.values())
    d2h = sum(v.numel() * 4 for v in yh.values())
    stubs = [({"n_cb": t["n_cb"], "shape": (t["N"], t["K"])}, t) for _, t in mats]

    def e2e_step():
        for k in xd:
            xd[k].copy_(xh[k], non_blocking=True)
        for M in BATCHES:
            for q_, t in stubs:
                Y, _ = drop_in.decode1_v44(xd[(M, t["K"])], q_, None, None, t["wt16"], t["bases"], t["scales"], 6)
            yh[M].copy_(Y, non_blocking=True)        # the last matrix of a pass is lm_head
        torch.cuda.synchronize()

    e2e_step()
    e2e_step()
    # This path is bound by the host (1012 eager calls per step), and the GPU boxes' host cores are
    # shared: three rounds, the fastest one reported, all three kept in the line.
    e2e_rounds = []
    for _ in range(3):
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(e2e_steps):
            e2e_step()
        b.record(); torch.cuda.synchronize()
        e2e_rounds.append(a.elapsed_time(b) / e2e_steps)
    e2e_ms = min(e2e_rounds)
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
        "config": workload_config("gemv_sweep_qwen3_4b", args, 1),
        "launch": {"cuda_graph": not args.no_graph, "pdl": not args.no_pdl},
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
                "ms_per_step": round(e2e_ms, 3), "steps": e2e_steps, "rounds_ms_per_step": [round(v, 3) for v in e2e_rounds],
                "api": "sx8_decode1_v3.decode1_v44 per projection (eager, torch binding); per step: activations from "
                       "pinned host memory, lm_head logits of every batch back to pinned host memory",
                "binding": "torch extension" if _lib.ext() is not None else "ctypes"},
        "clocks": clocks,
        "fused_projections_batch1": fused,
        "other_kernels": extras,
        "ref_kernels_same_box": refk,
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
    """Prefill GEMM over every distinct projection shape of the family at M = 128 .. 8192 (f16
    out, BASELINE config 2), quantizer search, embedding gather and full-tensor decode;
    fractions are of the measured peaks."""
    import torch
    from sx8_quantization_b200 import ops, quantizer
    out = {}
    pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                                                         "hbm_gbs": FALLBACK_HBM_GBS}
    g = torch.Generator(device=dev).manual_seed(77)
    gem = {}
    def gemm_row(name, t):
        row = {}
        for M in (128, 512, 2048, 8192):
            x = torch.randn(M, t["K"], generator=g, device=dev).half()
            y = torch.empty(M, t["N"], dtype=torch.float16, device=dev)
            us = _time_us(lambda: ops.gemm(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                                           out_dtype=torch.float16, out=y), iters=5 if name == "lm_head" else 10)
            tf = 2.0 * M * t["N"] * t["K"] / us / 1e6
            row[str(M)] = {"us": round(us, 1), "TFLOPs": round(tf, 1), "frac_of_bf16_burst": round(tf / pk["bf16_tflops"], 3),
                           "frac_of_bf16_sustained": round(tf / pk.get("bf16_tflops_sustained", pk["bf16_tflops"]), 3)}
            if M == 128:   # the crossover: also as a fraction of HBM (packed weights + x + y)
                by = tensor_bytes(t) + 2 * M * t["K"] + 2 * M * t["N"]
                row[str(M)]["frac_of_hbm"] = round(by / us / 1e3 / pk["hbm_gbs"], 3)
            del x, y
        gem["%s_%dx%d" % (name, t["N"], t["K"])] = row

    for name, t in [("q", layer0["q"]), ("k_v", layer0["k"]), ("o", layer0["o"]), ("gate_up", layer0["gate"]),
                    ("down", layer0["down"])]:
        gemm_row(name, t)
    # projections that share their input, one launch (sx8_gemm_multi): q|k|v and gate|up
    fused = {}
    for name, ts in (("q_k_v", [layer0["q"], layer0["k"], layer0["v"]]), ("gate_up", [layer0["gate"], layer0["up"]])):
        mg = ops.MultiGemm(ts)
        row = {}
        for M in (128, 512, 2048, 8192):
            x = torch.randn(M, ts[0]["K"], generator=g, device=dev).half()
            outs = [torch.empty(M, t["N"], dtype=torch.float16, device=dev) for t in ts]
            us = _time_us(lambda: mg(x, out_dtype=torch.float16, outs=outs))
            us_sep = _time_us(lambda: [ops.gemm(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                                                out_dtype=torch.float16, out=o) for t, o in zip(ts, outs)])
            tf = 2.0 * M * sum(t["N"] for t in ts) * ts[0]["K"] / us / 1e6
            row[str(M)] = {"us": round(us, 1), "us_separate_launches": round(us_sep, 1), "TFLOPs": round(tf, 1),
                           "frac_of_bf16_burst": round(tf / pk["bf16_tflops"], 3)}
            del x, outs
        fused[name] = row
    gemm_row("lm_head", head)   # last: its 6 ms launches at M = 8192 run into the power cap and would colour what follows
    out["prefill_gemm"] = gem
    out["prefill_gemm_fused"] = fused
    t = layer0["gate"]
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


def ref_kernels_same_box(dev, fam, our_per_shape, our_gemm):
    """The reference's own CUDA kernels, compiled unmodified for this GPU into oracle/_ref
    (checker side; the package never loads them), timed beside this library's on the same
    shapes: decode1_v44_combined (ref cuda/sx8_decode1_v3.cu:223-246) at M = 1 on the
    projections of the sweep, rotating over more distinct copies than L2 holds, and gemm_compact
    (ref cuda/sx8_gemm_compact.cu:171-194) / fused_forward (ref cuda/sx8_fused_wmma.cu:134-154)
    on the gate projection.  None when oracle/_ref was not built."""
    import torch
    from oracle import build as obuild
    from sx8_quantization_b200 import ops, quantizer
    d1 = obuild.load_ref("ref_sx8_decode1_v3")
    if d1 is None:
        return None
    out = {"decode1_v44_combined_batch1": {}, "note": "reference kernels built with nvcc -O3 for sm_100 from the reference's "
           "sources, launched through their own pybind entry points; same CUDA-event timing, graph replay and "
           "copy rotation as per_shape_batch1"}
    g = torch.Generator(device=dev).manual_seed(5)
    st = torch.cuda.Stream(device=dev)

    def v44_of(N, K, seed):
        t = quantizer.quantize_tensor(quantizer.synth_weight_gpu(N, K, seed, dev), with_pca=True, keep_planes=True)
        p = t["planes"]
        hdr, lev = ops.repack_v44(p["dmin"], p["dmax"], p["config"], p["coeff"], p["levels_hi"], p["levels_lo"], N, t["n_cb"], 6)
        return t, hdr, lev

    for name, N, K, _ in fam["proj"] + [("lm_head", fam["vocab"], fam["hidden"], "col")]:
        if name in ("v", "up"):
            continue
        n_cb = K // 32
        nbytes = 30 * N * n_cb
        copies = 1 if nbytes > (200 << 20) else max(2, (300 << 20) // nbytes)
        sets = []
        for c in range(copies):
            t, hdr, lev = v44_of(N, K, 7000 + c)
            sets.append((hdr, lev, t["bases"], t["scales"]))
            del t
        x = torch.randn(K, generator=g, device=dev).half()
        Z = torch.empty(n_cb, 2, device=dev)
        Y = torch.empty(N, device=dev)
        with torch.cuda.stream(st):
            for hdr, lev, b, s_ in sets[:2]:
                d1.decode1_v44_combined(x, hdr, lev, b, s_, n_cb, 6, Z, Y)
            st.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=st):
                for hdr, lev, b, s_ in sets:
                    d1.decode1_v44_combined(x, hdr, lev, b, s_, n_cb, 6, Z, Y)
            gr.replay(); st.synchronize()
            a = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
            a.record(st)
            for _ in range(5):
                gr.replay()
            e.record(st); st.synchronize()
        us = a.elapsed_time(e) * 1e3 / (5 * len(sets))
        ours = our_per_shape.get(name, {}).get("us_per_launch")
        out["decode1_v44_combined_batch1"][name] = {
            "N": N, "K": K, "ref_us_per_call": round(us, 3), "ref_GBps": round(nbytes / us / 1e3, 1),
            "ours_us_per_launch": ours, "speedup": round(us / ours, 2) if ours else None, "resident_copies": len(sets),
            "ref_launches_per_call": 2}
        del sets
        torch.cuda.empty_cache()
    # prefill kernels on the gate projection
    gc = obuild.load_ref("ref_sx8_gemm_compact")
    wm = obuild.load_ref("ref_sx8_fused_wmma")
    N, K = 9728, 2560
    n_cb = K // 32
    t, hdr, lev = v44_of(N, K, 7100)
    p = t["planes"]
    kbm = lambda a, per: a.reshape(N, n_cb, per).transpose(0, 1).contiguous().reshape(-1)
    planar = (kbm(p["dmin"].view(torch.uint8), 2).view(torch.float16), kbm(p["dmax"].view(torch.uint8), 2).view(torch.float16),
              kbm(p["config"], 1), kbm(p["coeff"], 1), kbm(p["levels_hi"], 16), kbm(p["levels_lo"], 8),
              t["bases"].reshape(-1).contiguous(), t["scales"].reshape(-1).contiguous())
    gem = {}
    for M in (128, 2048):
        x = torch.randn(M, K, generator=g, device=dev).half()
        row = {}
        if gc is not None:
            def f_compact():
                Zb = gc.compute_z44_batch(x, t["bases"], t["scales"], n_cb)
                return gc.gemm_compact(x, hdr, lev, Zb, n_cb, 6)
            us = _time_us(f_compact, iters=5, warm=2)
            row["gemm_compact_us"] = round(us, 1)
            row["gemm_compact_TFLOPs"] = round(2.0 * M * N * K / us / 1e6, 2)
        if wm is not None:
            torch.cuda.synchronize()
            us = _time_us(lambda: wm.fused_forward(x, *planar, n_cb), iters=5, warm=2)   # launches on the legacy default stream
            row["fused_wmma_us"] = round(us, 1)
            row["fused_wmma_TFLOPs"] = round(2.0 * M * N * K / us / 1e6, 2)
        ours = our_gemm.get(str(M), {}).get("us")
        row["ours_us"] = ours
        if ours:
            best = min(v for k, v in row.items() if k.endswith("_us") and k != "ours_us" and v)
            row["speedup_vs_best_ref"] = round(best / ours, 1)
        gem[str(M)] = row
    out["prefill_gate_9728x2560"] = gem
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


def cpu_dequant_matmul(orc, qt, bi, x):
    """One call of the reference's CPU comparator: full-tensor decode, then the fp32 matmul."""
    import torch
    W = torch.from_numpy(orc.dequant_d64(qt, bi))
    return x.float() @ W.float().t()


def run_reference(args):
    """--impl reference: the reference's own CPU-runnable path for this workload -- its
    comparator Y = X.float() @ decode(W).float().t() (ref scripts/sx8_decode1_v3.py:130-131),
    decode by the oracle's C port of the reference decoder (OpenMP, all host cores), matmul by
    torch on all host cores -- timed on the workload the other arm names.  A step is a bounded
    sample of that workload: every distinct matrix shape of the model once (one layer's seven
    projections, and lm_head for the sweep) at every batch size of the workload; no decoded
    weight is kept between calls, as on the reference's fused path.  Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import torch
    from oracle import sx8_oracle as orc
    from sx8_quantization_b200 import model_shapes as ms
    n = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    torch.set_num_threads(os.cpu_count() or 1)
    if n == 1:
        fam, batches, wl = ms.QWEN3_4B, BATCHES, "gemv_sweep_qwen3_4b"
        shapes = [(nm, N, K) for nm, N, K, _ in fam["proj"]] + [("lm_head", fam["vocab"], fam["hidden"])]
    else:
        fam, batches, wl = ms.LLAMA_70B, TP_BATCHES, "tp_decode_llama70b"
        shapes = [(nm, N, K) for nm, N, K, _ in fam["proj"]]
    mats = []
    for i, (nm, N, K) in enumerate(shapes):
        qt, bi = orc.quantize(orc.synth_weight(N, K, 100 + i), with_pca=False)
        mats.append((nm, N, K, qt, bi))
    xs = {(M, K): torch.from_numpy(orc.synth_x(M, K, 3 + M)) for M in batches for K in {k for _, _, k in shapes}}
    bytes_step = sum(ms.packed_bytes(N, K) for _, N, K, _, _ in mats) * len(batches)

    def step():
        for M in batches:
            for _, N, K, qt, bi in mats:
                cpu_dequant_matmul(orc, qt, bi, xs[(M, K)])

    ts = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        step()
        if i >= args.warmup:
            ts.append(time.perf_counter() - t0)
    sec = sum(ts) / len(ts)
    v = bytes_step / sec / 1e9
    sample = ("per step: %s at batch %s, %d calls of C-oracle decode (OpenMP, %d threads) + torch fp32 matmul, "
              "%.2f s; the full workload repeats these shapes over %d layers" %
              (", ".join(nm for nm, *_ in mats), "/".join(str(b) for b in batches), len(mats) * len(batches),
               orc.num_threads(), sec, fam["layers"]))
    c = {"value": round(v, 4), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port", "threads": orc.num_threads(),
         "sample": sample}
    print(json.dumps({
        "impl": "reference", "metric": "sx8_decode_gemv_weight_GBps", "value": round(v, 4), "unit": "GB/s",
        "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 2),
        "higher_is_better": True, "scaling": "weak" if n == 1 else "strong", "vs_baseline": None,
        "dtype": "f64 decode -> f16 W, f32 matmul", "data": "synthetic",
        "config": workload_config(wl, args, n),
        "cpu_baseline": c,
        "e2e": {"value": round(v, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(wl, args, world):
    """The `config` object of a workload: the same for both arms."""
    from sx8_quantization_b200 import model_shapes as ms
    if wl == "gemv_sweep_qwen3_4b":
        fam = ms.QWEN3_4B
        n_layers = args.layers if args.layers > 0 else fam["layers"]
        bytes_pass = n_layers * ms.layer_bytes(fam) + ms.packed_bytes(fam["vocab"], fam["hidden"])
        return {"workload": wl, "layers": n_layers, "batches": list(BATCHES),
                "matrices_per_pass": n_layers * len(fam["proj"]) + 1, "packed_bytes_per_pass": bytes_pass,
                "l2": "inputs larger than L2 (%.2f GB of distinct packed weights per pass)" % (bytes_pass / 1e9)}
    fam = ms.LLAMA_70B
    n_layers = args.layers if args.layers > 0 else TP_LAYERS
    return {"workload": wl, "layers": n_layers, "batches": list(TP_BATCHES), "parallelism": "tp%d" % world,
            "packed_bytes_per_layer": ms.layer_bytes(fam),
            "l2": "per-rank weights %.0f MB of distinct layers (> L2)" % (n_layers * ms.layer_bytes(fam) / world / 1e6)}


# ------------------------------------------------------------------------- N > 1

TP_BATCHES = (1, 16)
TP_LAYERS = 16
TP_PREFILL = 2048


def _graph_time(fn, st, steps, warm=3):
    """CUDA-graph capture of fn() on stream st, then the mean replay time in ms (device events)."""
    import torch
    with torch.cuda.stream(st):
        fn(); fn()
        st.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            fn()
        for _ in range(warm):
            gr.replay()
        st.synchronize()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        a.record(st)
        for _ in range(steps):
            gr.replay()
        b.record(st)
        st.synchronize()
    return a.elapsed_time(b) / steps, gr


def run_tp(args, rank, world, local_rank):
    """BASELINE config 4: Llama-70B-shaped layers as column/row tensor-parallel S-X8 linears.
    A step is one decode pass through the resident layers and the vocabulary-sharded lm_head
    at batch 1 and at batch 16 (tp.TPStack: column-parallel outputs feed the row-parallel
    linears, two summed reductions per layer, logit shards gathered).  Strong scaling: the
    model is fixed, the shard shrinks with N; rank 0 also times the unsharded stack (tp1) in
    the same process.  Secondary figures: a 2048-token prefill pass through the GEMM + NCCL,
    and the quantizer's throughput on the 70B shapes."""
    import torch
    import torch.distributed as dist
    from sx8_quantization_b200 import ops, tp, quantizer, _lib, model_shapes as ms
    fam = ms.LLAMA_70B
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    n_layers = args.layers if args.layers > 0 else TP_LAYERS
    H, V = fam["hidden"], fam["vocab"]
    flags = 0 if args.no_pdl else ops.SX8_F_PDL
    st = torch.cuda.Stream(device=dev)

    # ---- quantise the full matrices, keep this rank's shard (rank 0 keeps the full tensors too)
    t_q0 = time.monotonic()
    quant_blocks = 0
    layers, full_layers = [], []
    for li in range(n_layers):
        sh, fu = {}, {}
        for pi, (name, N, K, style) in enumerate(fam["proj"]):
            w = quantizer.synth_weight_gpu(N, K, 1000 + li * 16 + pi, dev)
            t = quantizer.quantize_tensor(w, with_pca=True)
            del w
            quant_blocks += N * t["n_cb"]
            sh[name] = tp.shard_tensor(t, style, rank, world) if world > 1 else tp.shard_tensor(t, style, 0, 1)
            if rank == 0 and world > 1 and not args.no_tp1:
                fu[name] = tp.shard_tensor(t, style, 0, 1)
        layers.append(sh)
        full_layers.append(fu)
    w = quantizer.synth_weight_gpu(V, H, 999, dev)
    t_head = quantizer.quantize_tensor(w, with_pca=True)
    del w
    head = tp.shard_tensor(t_head, "col", rank, world) if world > 1 else tp.shard_tensor(t_head, "col", 0, 1)
    full_head = tp.shard_tensor(t_head, "col", 0, 1) if (rank == 0 and world > 1 and not args.no_tp1) else None
    torch.cuda.synchronize()
    build_s = time.monotonic() - t_q0

    # ---- quantizer throughput on the 70B shapes (search + PCA + layout, one tensor at a time)
    quant = {}
    for name, N, K in (("q_8192x8192", 8192, 8192), ("gate_28672x8192", 28672, 8192)):
        w = quantizer.synth_weight_gpu(N, K, 4242, dev)
        us_s = _time_us(lambda: ops.quantize_blocks(w), iters=3, warm=1)
        us_f = _time_us(lambda: quantizer.quantize_tensor(w, with_pca=True), iters=2, warm=1)
        nb = N * (K // 32)
        quant[name] = {"search_Mblocks_per_s": round(nb / us_s, 1), "search_GBps_fp16_in": round(nb * 64 / us_s / 1e3, 1),
                       "full_with_pca_Mblocks_per_s": round(nb / us_f, 1), "full_GBps_fp16_in": round(nb * 64 / us_f / 1e3, 1)}
        del w
    quant["note"] = ("per GPU; ranks quantise disjoint tensors of a model independently, so N GPUs give N times this; "
                     "building this run's %d layers + lm_head (%.1f M blocks incl. weight generation) took %.1f s per rank"
                     % (n_layers, quant_blocks / 1e6, build_s))
    torch.cuda.empty_cache()

    exchange = None
    if world > 1 and args.allreduce != "nccl":
        try:
            exchange = tp.PeerExchange(max(TP_BATCHES) * H, dev)
        except Exception as e:
            if rank == 0:
                print("peer exchange unavailable, using NCCL:", repr(e)[:300], file=sys.stderr)
    g = torch.Generator(device=dev).manual_seed(5)           # same activations on every rank
    x0 = {M: torch.randn(M, H, generator=g, device=dev).half() for M in TP_BATCHES + (TP_PREFILL,)}

    # ---- correctness of the row-parallel reduction, before anything is timed: the o projection of
    #      layer 0 three ways (fused exchange, NCCL, unsharded on rank 0), and one whole decode step
    #      sharded vs unsharded
    tp_check = None
    if world > 1:
        t_sh = layers[0]["o"]
        k0, k1 = t_sh["k_range"]
        xg = torch.randn(8, fam["proj"][3][2], generator=g, device=dev).half()
        xl = xg[:, k0:k1].contiguous()
        y_nccl = tp.linear(xl, t_sh, flags=0).clone()
        y_fused = tp.linear(xl, t_sh, flags=0, exchange=exchange).clone() if exchange is not None else None
        y_pull = None
        if exchange is not None:    # the pull protocol: partial into the own slot, one kernel sums + residual + norm
            part = exchange.partial_out(8, t_sh["N"])
            tp.linear(xl, t_sh, out=part, flags=0, reduce=False)
            h0 = torch.zeros(8, t_sh["N"], device=dev)
            exchange.reduce_norm(h0, torch.ones(t_sh["N"], device=dev), 1e-5, torch.empty(8, t_sh["N"], dtype=torch.float16, device=dev))
            y_pull = h0          # residual was zero: h holds the sum
            exchange.partial_out(8, t_sh["N"]).zero_()   # keep the number of pull calls even (two halves)
            exchange.reduce_norm(torch.zeros_like(h0), torch.ones(t_sh["N"], device=dev), 1e-5,
                                 torch.empty(8, t_sh["N"], dtype=torch.float16, device=dev))
            exchange.next()      # and of push calls
        y_full = torch.empty_like(y_nccl)
        if rank == 0:
            if full_layers[0]:
                tf = full_layers[0]["o"]
                y_full = ops.gemv(xg, tf["wt16"], tf["bases"], tf["scales"], tf["N"], tf["K"], tf["n_cb"]).clone()
            else:
                y_full.copy_(y_nccl)
        dist.broadcast(y_full, 0)
        sc = y_full.abs().max()
        rel = lambda a: float(((a - y_full).abs().max() / sc).item())
        chk = torch.tensor([rel(y_nccl), rel(y_fused) if y_fused is not None else 0.0,
                            float(((y_fused - y_nccl).abs().max() / sc).item()) if y_fused is not None else 0.0,
                            rel(y_pull) if y_pull is not None else 0.0],
                           device=dev, dtype=torch.float64)
        dist.all_reduce(chk, op=dist.ReduceOp.MAX)
        tp_check = {"nccl_vs_unsharded": chk[0].item(), "push_vs_unsharded": chk[1].item() if exchange is not None else None,
                    "push_vs_nccl": chk[2].item() if exchange is not None else None,
                    "pull_vs_unsharded": chk[3].item() if exchange is not None else None,
                    "what": "o projection of layer 0, batch 8: max |diff| / max |y| over all ranks; push = GEMV epilogue "
                            "stores into the peers' slots, pull = all-reduce + residual + RMSNorm kernel reading the peers' partials"}

    def make_stack(M, lay, hd, ex, how="nccl"):
        return tp.TPStack(lay, hd, H, M, dev, exchange=ex, flags=flags, reduce=how if ex is not None else "nccl")

    def time_stack(stack, M, steps):
        stack.reset(x0[M])
        def fn():
            stack.step()
        return _graph_time(fn, st, steps)

    # ---- tp1 on rank 0 alone (same layers, same process), before the sharded runs
    tp1 = {}
    if world > 1 and rank == 0 and not args.no_tp1:
        for M in TP_BATCHES:
            s1 = make_stack(M, full_layers, full_head, None)
            s1.world = 1
            ms1, gr = time_stack(s1, M, max(3, args.steps // 2))
            tp1[M] = ms1
            del gr, s1
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()

    # ---- choose the reduction: NCCL, or one of the two peer-memory exchanges, whichever replays
    #      faster (trial at every batch size of the step, max over ranks)
    choice, trial = {M: "nccl" for M in TP_BATCHES}, {}
    if world > 1 and exchange is not None:
        modes = ["nccl", "pull", "push"] if args.allreduce == "auto" else [{"fused": "pull"}.get(args.allreduce, args.allreduce)]
        for M in TP_BATCHES:
            trial[str(M)] = {}
            for how in modes:
                if how == "push" and M > 8:
                    continue
                sT = make_stack(M, layers, head, None if how == "nccl" else exchange, how)
                m_, gr = time_stack(sT, M, 5)
                tt = torch.tensor([m_], device=dev, dtype=torch.float64)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                trial[str(M)][how] = round(float(tt.item()), 4)
                del gr, sT
            choice[M] = min(trial[str(M)], key=trial[str(M)].get)
    stacks = {M: make_stack(M, layers, head, None if choice[M] == "nccl" else exchange, choice[M]) for M in TP_BATCHES}
    graphs = {}
    for M in TP_BATCHES:
        stacks[M].reset(x0[M])
        _, graphs[M] = _graph_time(lambda M=M: stacks[M].step(), st, 1, warm=1)
    bytes_rank = stacks[TP_BATCHES[0]].packed_bytes

    sampler = ClockSampler(local_rank) if rank == 0 else None
    with torch.cuda.stream(st):
        for _ in range(args.warmup):
            for M in TP_BATCHES:
                graphs[M].replay()
        st.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.monotonic()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        eb = [torch.cuda.Event(enable_timing=True) for _ in range(len(TP_BATCHES) + 1)]
        e0.record(st)
        for k in range(args.steps):
            last = k == args.steps - 1
            if last:
                eb[0].record(st)
            for i, M in enumerate(TP_BATCHES):
                graphs[M].replay()
                if last:
                    eb[i + 1].record(st)
        e1.record(st)
        st.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t1 = time.monotonic()
    ms_local = e0.elapsed_time(e1) / args.steps
    per_batch_ms = [eb[i].elapsed_time(eb[i + 1]) for i in range(len(TP_BATCHES))]

    # ---- 2048-token prefill pass: GEMM linears, NCCL all-reduce after o and down, no lm_head
    pre = make_stack(TP_PREFILL, layers, None, None)
    pre.reset(x0[TP_PREFILL])
    pre.step(); pre.step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(3):
        pre.step()
    b.record(); torch.cuda.synchronize()
    prefill_ms = a.elapsed_time(b) / 3
    del pre

    # ---- e2e: the same step through the public API (tp.TPStack.step, eager), the step's input
    #      activations coming from pinned host memory and the gathered logits read back
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    xh = {M: x0[M].cpu().pin_memory() for M in TP_BATCHES}
    vloc = head["N"]
    yh = {M: torch.empty(world, M, vloc, dtype=torch.float32).pin_memory() for M in TP_BATCHES}
    h2d = sum(v.numel() * 2 for v in xh.values())
    d2h = sum(v.numel() * 4 for v in yh.values())

    def e2e_step():
        for M in TP_BATCHES:
            s_ = stacks[M]
            s_.h.zero_()
            s_.x.copy_(xh[M], non_blocking=True)
            out = s_.step()
            yh[M].view(-1).copy_(out.view(-1), non_blocking=True)
        torch.cuda.synchronize()

    e2e_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    # host-bound path on shared host cores: three rounds, each the max over ranks, the fastest round reported
    e2e_rounds = []
    for _ in range(3):
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(e2e_steps):
            e2e_step()
        b.record(); torch.cuda.synchronize()
        e2e_rounds.append(a.elapsed_time(b) / e2e_steps)

    tm = torch.tensor([ms_local, prefill_ms] + e2e_rounds + per_batch_ms, device=dev, dtype=torch.float64)
    tb = torch.tensor([float(bytes_rank)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(tb, op=dist.ReduceOp.SUM)
    ms_per_step, prefill_ms = float(tm[0].item()), float(tm[1].item())
    e2e_rounds = [float(v) for v in tm[2:5].tolist()]
    e2e_ms = min(e2e_rounds)
    per_batch_ms = [float(v) for v in tm[5:].tolist()]
    bytes_step = float(tb.item()) * len(TP_BATCHES)
    value = bytes_step / (ms_per_step * 1e-3) / 1e9
    flag = _lib.device_error_flag()
    if exchange is not None and flag & 0xC and rank == 0:
        print("WARNING: a tensor-parallel exchange wait timed out (device error word 0x%x): results invalid" % flag,
              file=sys.stderr)
    if rank == 0:
        clocks = sampler.summary(t0, t1)
        sampler.stop()
        peak, peak_kind = peaks()
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
            os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"bf16_tflops": 1590.0}
        launches_per_pass = {M: (n_layers * (7 if M <= 8 else 10) + 1) for M in TP_BATCHES}
        layer_flops = 2.0 * TP_PREFILL * sum(N * K for _, N, K, _ in fam["proj"])
        strong = None
        if tp1:
            t1ms = sum(tp1[M] for M in TP_BATCHES)
            strong = {"tp1_ms_per_step": round(t1ms, 4), "speedup": round(t1ms / ms_per_step, 3),
                      "efficiency": round(t1ms / ms_per_step / world, 3),
                      "tp1_ms_by_batch": {str(M): round(tp1[M], 4) for M in TP_BATCHES},
                      "note": "tp1 = the same layers and lm_head unsharded, timed on rank 0 alone in this process "
                              "before the sharded run"}
        cfg = workload_config("tp_decode_llama70b", args, world)
        names = {"nccl": "NCCL fp32 all-reduce, then residual + RMSNorm",
                 "pull": "one kernel: every rank reads the peers' partials over NVLink, rank-ordered fp32 sum + residual + RMSNorm",
                 "push": "GEMV epilogue stores tiles into the peers' slots, small kernel sums them, then residual + RMSNorm"}
        launch = {"allreduce": {str(M): names[choice[M]] for M in TP_BATCHES}, "allreduce_choice": {str(M): choice[M] for M in TP_BATCHES},
                  "allreduce_trial_ms": trial or None, "logits": "all-gather (NCCL)", "cuda_graph": True, "pdl": not args.no_pdl}
        line = {
            "metric": "sx8_decode_gemv_weight_GBps", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 x u6 -> f32 accumulate", "data": "synthetic (random-init, quantised on the device)",
            "config": cfg,
            "launch": launch,
            "decode": {str(M): {"ms_per_step": round(per_batch_ms[i], 4),
                                "tok_per_s_%d_layers" % n_layers: round(M / per_batch_ms[i] * 1e3, 1),
                                "tok_per_s_80_layers_equiv": round(M / per_batch_ms[i] * 1e3 * n_layers / fam["layers"], 2)}
                       for i, M in enumerate(TP_BATCHES)},
            "prefill_2048": {"ms_per_pass": round(prefill_ms, 3), "layers": n_layers,
                             "tok_per_s_80_layers_equiv": round(TP_PREFILL / prefill_ms * 1e3 * n_layers / fam["layers"], 1),
                             "TFLOPs_aggregate": round(layer_flops * n_layers / prefill_ms / 1e9, 1),
                             "frac_of_bf16_burst_per_gpu": round(layer_flops * n_layers / prefill_ms / 1e9 / world / pk["bf16_tflops"], 3),
                             "allreduce": "nccl fp32, 2 x %d MB per layer" % (TP_PREFILL * H * 4 >> 20)},
            "quantizer_70b_shapes": quant,
            "strong_scaling": strong,
            "tp_check_max_rel": tp_check,
            "gpu_launches": sum(launches_per_pass.values()) * args.steps,
            "device_error_flag": flag,
            "roofline": {"bound": "hbm", "achieved": round(value / world, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(value / world / peak, 4), "traffic": None,
                         "note": "per-GPU packed weight bytes / step wall time incl. reductions and glue kernels, of %s peak" % peak_kind},
            "e2e": {"value": round(bytes_step / (e2e_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 3),
                    "steps": e2e_steps, "rounds_ms_per_step": [round(v, 3) for v in e2e_rounds],
                    "api": "tp.TPStack.step (eager), input activations from pinned host memory, "
                                               "gathered logits back to pinned host memory; reduction: " + "/".join(choice[M] for M in TP_BATCHES)},
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


def run_case(args):
    """--case: ONE kernel of the library on one synthetic tensor, a handful of launches, and its
    CUDA-event time -- the command profilers are pointed at."""
    import torch
    from sx8_quantization_b200 import _lib, ops, quantizer
    dev = torch.device("cuda:0")
    N, K, M = args.N, args.K, args.M
    if args.case == "decoder":   # a short eager run of the 4B-shaped decoder: --N layers, --M batch, --K prompt tokens
        from sx8_quantization_b200.decoder import SX8Decoder, QWEN3_4B_DECODER
        cfg = dict(QWEN3_4B_DECODER, layers=N)
        dec = SX8Decoder(cfg, device=dev, seed=9, max_seq=K + 64, batch=M)
        ids = torch.randint(0, cfg["vocab"], (M, K), generator=torch.Generator(device=dev).manual_seed(1), device=dev)
        toks, t = dec.generate(ids, args.iters, use_graph=False)
        print(json.dumps({"case": "decoder", "layers": N, "batch": M, "prompt": K, "new_tokens": args.iters,
                          "prefill_ms": round(t["prefill_ms"], 3), "decode_ms_per_token": round(t["decode_ms_per_token"], 4),
                          "device_error_flag": _lib.device_error_flag()}))
        return
    w = quantizer.synth_weight_gpu(N, K, 3, device=dev)
    g = torch.Generator(device=dev).manual_seed(4)
    if args.case == "quantize":
        fn = lambda: ops.quantize_blocks(w)
        units, unit = N * ((K + 31) // 32), "blocks"
    elif args.case == "quantize_pca":   # search + PCA stage + device layout
        fn = lambda: quantizer.quantize_tensor(w, with_pca=True)
        units, unit = N * ((K + 31) // 32), "blocks"
    else:
        t = quantizer.quantize_tensor(w, with_pca=True)
        del w
        n_cb = t["n_cb"]
        x = torch.randn(M, K, generator=g, device=dev).half()
        if args.case == "gemv":
            y = torch.empty(M, N, dtype=torch.float32, device=dev)
            fn = lambda: ops.gemv(x, t["wt16"], t["bases"], t["scales"], N, K, n_cb, out=y)
            units, unit = N * n_cb * 30, "packed bytes"
        elif args.case == "gemm":
            y = torch.empty(M, N, dtype=torch.float16, device=dev)
            fn = lambda: ops.gemm(x, t["wt16"], t["bases"], t["scales"], N, K, n_cb, out_dtype=torch.float16, out=y)
            units, unit = 2 * M * N * K, "flop"
        elif args.case == "embed":
            ids = torch.randint(0, N, (M,), generator=g, device=dev)
            fn = lambda: ops.embed(ids, t["wt16"], t["bases"], t["scales"], K, N, n_cb)
            units, unit = M, "rows"
        else:
            fn = lambda: ops.dequant_t16(t["wt16"], t["bases"], t["scales"], N, K, n_cb, True)
            units, unit = N * n_cb * 30, "packed bytes"
    us = _time_us(fn, iters=args.iters, warm=args.warmup)
    flag = _lib.device_error_flag()
    print(json.dumps({"case": args.case, "N": N, "K": K, "M": M, "us_per_call": round(us, 2),
                      "per_second": units / (us * 1e-6), "unit": unit + "/s", "device_error_flag": flag}))


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
    ap.add_argument("--allreduce", default="auto", choices=["auto", "pull", "push", "fused", "nccl"],
                    help="row-parallel reduction: peer-memory exchange (pull = all-reduce + RMSNorm kernel, push = from "
                         "the GEMV epilogue), NCCL, or whichever replays faster")
    ap.add_argument("--no-tp1", action="store_true", help="N > 1: skip the unsharded run on rank 0")
    ap.add_argument("--case", default=None, choices=["gemv", "gemm", "embed", "dequant", "quantize", "quantize_pca", "decoder"],
                    help="time one kernel on one synthetic tensor (for profilers)")
    ap.add_argument("--N", type=int, default=9728)
    ap.add_argument("--K", type=int, default=2560)
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--max-seconds", type=int, default=900, help="watchdog for the whole run")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    _watchdog(args.max_seconds)
    if args.case:
        args.warmup = min(args.warmup, 3)
        return run_case(args)
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
