"""End-to-end random-init dense decoder on S-X8 linears: prefill through the tensor-core
GEMM, greedy decode through the GEMV with the whole step captured in one CUDA graph (static
KV cache, position held in a device tensor).

Every linear (q, k, v, o, gate, up, down, lm_head) and the embedding table are S-X8 v4.3
tensors in the T16 device layout, quantised on the device from seeded random weights
(N(0, 0.02) + 0.1 % outliers); projections that share their input run as one multi-matrix
GEMV launch (q|k|v, gate|up).  The glue between the linears -- RMSNorm, RoPE, attention
over the cache, SwiGLU -- is not part of the S-X8 path (the reference takes it from the host
framework, ref scripts/integrate_fused_v44.py:85-116 swaps only the nn.Linear / nn.Embedding
modules of a transformers model).  Prefill uses PyTorch for it; a decode step uses the four
sx8_glue_* kernels (nine launches per layer) or, with fused_glue=False, plain PyTorch.

Default shapes follow Qwen3-4B (36 layers, hidden 2560, 32 query / 8 key-value heads of
128, SwiGLU 9728, vocabulary 151936); the per-head q/k norms of that family are left out."""
import math

import torch
import torch.nn.functional as F

from . import ops, quantizer
from ._lib import SX8_F_PDL

QWEN3_4B_DECODER = dict(layers=36, hidden=2560, n_q=32, n_kv=8, head_dim=128, ffn=9728, vocab=151936,
                        rope_theta=1.0e6, eps=1.0e-6)


def _rope(x, cos, sin):
    """x (..., d) with the half-split convention: [x1*cos - x2*sin, x2*cos + x1*sin]."""
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


class SX8Decoder:
    def __init__(self, cfg=None, device="cuda:0", seed=0, max_seq=768, batch=1, with_pca=True, fused_glue=True):
        self.cfg = dict(QWEN3_4B_DECODER if cfg is None else cfg)
        c = self.cfg
        self.dev = torch.device(device)
        self.B, self.S = int(batch), int(max_seq)
        H, D = c["hidden"], c["head_dim"]
        self.nq, self.nkv = c["n_q"] * D, c["n_kv"] * D

        def make(n, k, s):
            w = quantizer.synth_weight_gpu(n, k, s, device=self.dev)
            t = quantizer.quantize_tensor(w, with_pca=with_pca)
            del w
            return t

        s = seed * 100003
        self.embed = make(c["vocab"], H, s + 1)
        self.lm_head = make(c["vocab"], H, s + 2)
        self.layers = []
        for l in range(c["layers"]):
            b = s + 10 + 8 * l
            self.layers.append({"q": make(self.nq, H, b), "k": make(self.nkv, H, b + 1), "v": make(self.nkv, H, b + 2),
                                "o": make(H, self.nq, b + 3), "gate": make(c["ffn"], H, b + 4),
                                "up": make(c["ffn"], H, b + 5), "down": make(H, c["ffn"], b + 6)})
        self.gamma = torch.ones(H, device=self.dev)          # every RMSNorm weight (random-init model: ones)
        # static KV cache (layers, batch, kv heads, positions, head_dim), fp16
        self.k_cache = torch.zeros(c["layers"], self.B, c["n_kv"], self.S, D, dtype=torch.float16, device=self.dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (c["rope_theta"] ** (torch.arange(0, D, 2, device=self.dev, dtype=torch.float32) / D))
        ang = torch.arange(self.S, device=self.dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()            # (S, D/2)
        self.scale = 1.0 / math.sqrt(D)
        # decode state (device-resident so that one captured graph serves every step)
        self.tok = torch.zeros(self.B, dtype=torch.long, device=self.dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.dev)
        self.steps = torch.arange(self.S, device=self.dev)
        self.multi = None
        if self.B <= 8:
            self.multi = [(ops.MultiGemv([L["q"], L["k"], L["v"]], self.B, self.dev),
                           ops.MultiGemv([L["gate"], L["up"]], self.B, self.dev)) for L in self.layers]
        # projections that share their input as one tensor-core launch (prefill; decode above 8 rows)
        self.multi_gemm = [(ops.MultiGemm([L["q"], L["k"], L["v"]]), ops.MultiGemm([L["gate"], L["up"]])) for L in self.layers]
        self.graph = None
        self.fused_glue = bool(fused_glue)
        f16, f32 = dict(dtype=torch.float16, device=self.dev), dict(dtype=torch.float32, device=self.dev)
        B = self.B
        self.buf = {"h": torch.empty(B, H, **f32), "x": torch.empty(B, H, **f16), "q16": torch.empty(B, self.nq, **f16),
                    "a": torch.empty(B, self.nq, **f16), "act": torch.empty(B, c["ffn"], **f16),
                    "o": torch.empty(B, H, **f32), "d": torch.empty(B, H, **f32),
                    "q": torch.empty(B, self.nq, **f32), "k": torch.empty(B, self.nkv, **f32),
                    "v": torch.empty(B, self.nkv, **f32), "g": torch.empty(B, c["ffn"], **f32),
                    "u": torch.empty(B, c["ffn"], **f32), "logits": torch.empty(B, c["vocab"], **f32)}
        self.attn_scratch = ops.glue_attn_scratch(B, c["n_q"], c["n_kv"], D, self.dev)
        self.packed_bytes = sum(t["wt16"].numel() for L in self.layers for t in L.values()) + self.lm_head["wt16"].numel()

    # ------------------------------------------------------------------ pieces
    def _norm(self, h):
        return F.rms_norm(h, (h.shape[-1],), self.gamma, self.cfg["eps"]).half()

    def _linear(self, x, t, out_dtype=torch.float32):
        """x (M, K) f16 -> (M, N): GEMV up to 8 rows, tensor-core GEMM above."""
        if x.shape[0] <= 8:
            y = ops.gemv(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], flags=SX8_F_PDL)
            return y if out_dtype == torch.float32 else y.half()
        return ops.gemm(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], out_dtype=out_dtype)

    def _embed(self, ids):
        e = self.embed
        return ops.embed(ids, e["wt16"], e["bases"], e["scales"], e["K"], e["N"], e["n_cb"])

    # ------------------------------------------------------------------ prefill
    def prefill(self, ids):
        """ids (B, T) long.  Fills the cache for positions 0..T-1, sets the decode state to
        (argmax of the last position, T) and returns the last-position logits (B, vocab)."""
        c = self.cfg
        B, T = ids.shape
        if B != self.B or T > self.S:
            raise ops.SX8Error("prompt (%d, %d) does not fit the decoder (batch %d, max_seq %d)" % (B, T, self.B, self.S))
        D, hq, hkv = c["head_dim"], c["n_q"], c["n_kv"]
        h = self._embed(ids.reshape(-1)).float()                                    # (B*T, H) residual stream, f32
        cos, sin = self.cos[:T], self.sin[:T]                                       # (T, D/2)
        for l, L in enumerate(self.layers):
            x = self._norm(h)
            q, k, v = self.multi_gemm[l][0](x, out_dtype=torch.float16)
            q, k, v = q.view(B, T, hq, D), k.view(B, T, hkv, D), v.view(B, T, hkv, D)
            q = _rope(q.float(), cos[None, :, None, :], sin[None, :, None, :]).half().transpose(1, 2)
            k = _rope(k.float(), cos[None, :, None, :], sin[None, :, None, :]).half().transpose(1, 2)
            v = v.transpose(1, 2)
            self.k_cache[l, :, :, :T] = k
            self.v_cache[l, :, :, :T] = v
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)   # (B, hq, T, D)
            a = a.transpose(1, 2).reshape(B * T, hq * D)
            h = h + self._linear(a, L["o"])
            x = self._norm(h)
            g, u = self.multi_gemm[l][1](x, out_dtype=torch.float16)
            h = h + self._linear(F.silu(g) * u, L["down"])
        last = self._norm(h.view(B, T, -1)[:, -1])
        logits = self._linear(last, self.lm_head)
        self.tok.copy_(logits.argmax(-1))
        self.pos.fill_(T)
        return logits

    # ------------------------------------------------------------------ one decode step
    def _lin_into(self, x, t, out):
        """x (B, K) f16 -> out (B, N) f32, preallocated."""
        if x.shape[0] <= 8:
            return ops.gemv(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], out=out, flags=SX8_F_PDL)
        return ops.gemm(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], out_dtype=torch.float32, out=out)

    def _step_fused(self):
        """One decode step with the sx8_glue_* kernels between the linears."""
        c, b = self.cfg, self.buf
        D, hq, hkv = c["head_dim"], c["n_q"], c["n_kv"]
        b["h"].copy_(self._embed(self.tok))
        y = None
        for l, L in enumerate(self.layers):
            ops.glue_add_rmsnorm(b["h"], y, self.gamma, c["eps"], b["x"])
            if self.multi is not None:
                q, k, v = self.multi[l][0](b["x"], flags=SX8_F_PDL)
            else:
                q, k, v = self.multi_gemm[l][0](b["x"], outs=[b["q"], b["k"], b["v"]])
            ops.glue_rope_cache(q, k, v, self.pos, self.cos, self.sin, hq, hkv, D, b["q16"], self.k_cache[l], self.v_cache[l])
            ops.glue_attn_decode(b["q16"], self.k_cache[l], self.v_cache[l], self.pos, hq, hkv, D, self.scale, b["a"],
                                 self.attn_scratch)
            self._lin_into(b["a"], L["o"], b["o"])
            ops.glue_add_rmsnorm(b["h"], b["o"], self.gamma, c["eps"], b["x"])
            if self.multi is not None:
                g, u = self.multi[l][1](b["x"], flags=SX8_F_PDL)
            else:
                g, u = self.multi_gemm[l][1](b["x"], outs=[b["g"], b["u"]])
            ops.glue_silu_mul(g, u, b["act"])
            y = self._lin_into(b["act"], L["down"], b["d"])
        ops.glue_add_rmsnorm(b["h"], y, self.gamma, c["eps"], b["x"])
        logits = self._lin_into(b["x"], self.lm_head, b["logits"])
        self.tok.copy_(logits.argmax(-1))
        self.pos.add_(1)
        return logits

    def _step(self):
        """Consumes self.tok at position self.pos; writes the next token and advances."""
        if self.fused_glue:
            return self._step_fused()
        c = self.cfg
        B, D, hq, hkv = self.B, c["head_dim"], c["n_q"], c["n_kv"]
        grp = hq // hkv
        h = self._embed(self.tok).float()                                           # (B, H)
        cos = self.cos.index_select(0, self.pos)                                    # (1, D/2)
        sin = self.sin.index_select(0, self.pos)
        future = (self.steps > self.pos)[None, None, None, :]                       # positions not written yet
        for l, L in enumerate(self.layers):
            x = self._norm(h)
            if self.multi is not None:
                q, k, v = self.multi[l][0](x, flags=SX8_F_PDL)
            else:
                q, k, v = self.multi_gemm[l][0](x)
            q = _rope(q.view(B, hq, D), cos[:, None, :], sin[:, None, :]).half()
            k = _rope(k.view(B, hkv, D), cos[:, None, :], sin[:, None, :]).half()
            self.k_cache[l].index_copy_(2, self.pos, k.unsqueeze(2))
            self.v_cache[l].index_copy_(2, self.pos, v.view(B, hkv, 1, D).half())
            s = torch.matmul(q.view(B, hkv, grp, D), self.k_cache[l].transpose(-1, -2)).float() * self.scale
            p = torch.softmax(s.masked_fill(future, float("-inf")), dim=-1).half()  # (B, hkv, grp, S)
            a = torch.matmul(p, self.v_cache[l]).reshape(B, hq * D)
            h = h + self._linear(a, L["o"])
            x = self._norm(h)
            if self.multi is not None:
                g, u = self.multi[l][1](x, flags=SX8_F_PDL)
            else:
                g, u = self.multi_gemm[l][1](x)
            h = h + self._linear((F.silu(g) * u).half(), L["down"])
        logits = self._linear(self._norm(h), self.lm_head)
        self.tok.copy_(logits.argmax(-1))
        self.pos.add_(1)
        return logits

    def capture(self):
        """Capture one decode step in a CUDA graph (call after prefill; the state tensors keep
        their addresses).  The capture itself runs the step zero times: the warm-up steps
        before it are undone by restoring token and position."""
        tok0, pos0 = self.tok.clone(), self.pos.clone()
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self._step()
        torch.cuda.current_stream(self.dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._logits = self._step()
        self.tok.copy_(tok0)
        self.pos.copy_(pos0)
        return self.graph

    def prefill_captured(self, ids):
        """prefill() replayed from a CUDA graph (one graph per prompt shape, captured on first
        use): the glue between the linears is some forty framework kernels per layer, and at
        small batch the host cannot issue them as fast as the GPU runs them."""
        if not hasattr(self, "_pf_graphs"):
            self._pf_graphs = {}
        key = tuple(ids.shape)
        ent = self._pf_graphs.get(key)
        if ent is None:
            static_ids = ids.clone()
            side = torch.cuda.Stream(self.dev)
            side.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(side):
                self.prefill(static_ids)            # warm-up: workspaces and allocator pools
            torch.cuda.current_stream(self.dev).wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                logits = self.prefill(static_ids)
            ent = self._pf_graphs[key] = (g, static_ids, logits)
        g, static_ids, logits = ent
        static_ids.copy_(ids)
        g.replay()
        return logits

    def generate(self, ids, n_new, use_graph=True):
        """Greedy decode.  Returns (tokens (B, n_new) long on the device, timings dict in ms)."""
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        if ids.shape[1] + n_new > self.S:
            raise ops.SX8Error("prompt + new tokens exceed max_seq")
        if use_graph and tuple(ids.shape) not in getattr(self, "_pf_graphs", {}):
            self.prefill_captured(ids)           # capture outside the timed region
        torch.cuda.synchronize(self.dev)
        e[0].record()
        if use_graph:
            self.prefill_captured(ids)
        else:
            self.prefill(ids)
        e[1].record()
        out = torch.empty(self.B, n_new, dtype=torch.long, device=self.dev)
        if use_graph and self.graph is None:
            self.capture()
        torch.cuda.synchronize(self.dev)
        e[2].record()
        for i in range(n_new):
            out[:, i].copy_(self.tok)
            if use_graph:
                self.graph.replay()
            else:
                self._step()
        e[3].record()
        torch.cuda.synchronize(self.dev)
        return out, {"prefill_ms": e[0].elapsed_time(e[1]), "decode_ms_per_token": e[2].elapsed_time(e[3]) / max(1, n_new)}
