"""Tensor-parallel S-X8 linears: one process per GPU, torch.distributed (NCCL) for the
exchange.  The reference has no multi-GPU code; this is the sharding its format
implies:

  column-parallel (q, k, v, gate, up, lm_head): shard the output rows N in multiples
      of 16.  The T16 blob is tile-major, so a row shard is one contiguous byte range;
      bases/scales are replicated.
  row-parallel (o, down): shard K on 32-weight block boundaries.  A kb range is a
      strided slice per tile, re-materialised contiguously per rank at load, together
      with the matching rows of bases/scales; every rank produces a partial y (its own
      PCA term included) and the partials are summed with one all-reduce.

Tensors are quantised before slicing, so shards are byte-identical to slices of the
single-GPU tensors (the PCA bases of a kb depend on all N rows)."""
import torch

from . import ops


def shard_bounds(total, rank, world, quantum):
    """Contiguous near-equal split of `total` units in multiples of `quantum`."""
    units = total // quantum
    if units * quantum != total:
        raise ops.SX8Error("size %d is not a multiple of %d" % (total, quantum))
    base, rem = divmod(units, world)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return lo * quantum, hi * quantum


def shard_tensor(t, style, rank, world):
    """t: dict from quantizer.quantize_tensor.  Returns this rank's shard (same dict
    format, plus "style" and the global sizes)."""
    if world == 1:
        out = dict(t)
        out["style"] = style
        return out
    N, K, n_cb = t["N"], t["K"], t["n_cb"]
    blob = t["wt16"].reshape(-1, n_cb, 480)          # (tiles, kb, unit)
    if style == "col":
        n0, n1 = shard_bounds(N, rank, world, 16)
        return {"wt16": blob[n0 // 16:n1 // 16].contiguous().reshape(-1, 480), "bases": t["bases"],
                "scales": t["scales"], "N": n1 - n0, "K": K, "n_cb": n_cb, "style": "col", "n_range": (n0, n1),
                "global": (N, K)}
    if style == "row":
        kb0, kb1 = shard_bounds(n_cb, rank, world, 1)
        k0, k1 = kb0 * 32, min(K, kb1 * 32)
        return {"wt16": blob[:, kb0:kb1].contiguous().reshape(-1, 480), "bases": t["bases"][kb0:kb1].contiguous(),
                "scales": t["scales"][kb0:kb1].contiguous(), "N": N, "K": k1 - k0, "n_cb": kb1 - kb0,
                "style": "row", "k_range": (k0, k1), "global": (N, K)}
    raise ops.SX8Error("unknown tensor-parallel style %r" % (style,))


class PeerExchange:
    """Symmetric exchange buffers of a tensor-parallel group: every rank maps every other rank's
    buffer (torch symmetric memory over NVLink peer access).  NVLink multicast is not used
    (plain peer loads and stores only).  Two protocols share the buffers:

      * sx8_gemv_allreduce (next()): the GEMV epilogue pushes its partial tiles into slot `rank`
        of every peer's buffer and a small kernel sums the slots;
      * sx8_glue_allreduce_add_rmsnorm (reduce_norm()): a rank writes its partial into slot 0 of
        its OWN buffer (partial_out()), and the consumer kernel -- residual add + RMSNorm -- pulls
        all partials from the peers' memory and sums them.

    Calls alternate between two halves of the buffers; all ranks must make the same calls in the
    same order.  A CUDA graph that captures exchange calls must contain an even number of them
    per protocol, so that a replay starts with the half it was captured with.

    After a bounded wait inside either kernel ran out (bit 2 or 3 of the device error word, see
    check()), the ranks are out of step: the exchange must be rebuilt on all ranks."""

    def __init__(self, max_elems, device, group=None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        self.group = group if group is not None else torch.distributed.group.WORLD
        self.world = torch.distributed.get_world_size(self.group)
        self.rank = torch.distributed.get_rank(self.group)
        if self.world > 8:
            raise ops.SX8Error("at most 8 ranks")
        self.slot_elems = int(max_elems)
        self.data = symm_mem.empty(2 * self.world * self.slot_elems, dtype=torch.float32, device=device)
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=device)
        self.data.zero_()
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self._hd = symm_mem.rendezvous(self.data, group=self.group)
        self._hf = symm_mem.rendezvous(self.flags, group=self.group)
        torch.distributed.barrier(self.group)
        self._desc = []
        for par in (0, 1):
            self._desc.append(self._make(par))
        self.calls = 0
        self.pull_calls = 0

    def _make(self, parity):
        from . import _lib
        d = _lib.Peers()
        for q in range(self.world):
            d.data[q] = int(self._hd.buffer_ptrs[q])
            d.flags[q] = int(self._hf.buffer_ptrs[q])
        d.slot_elems = self.slot_elems
        d.rank, d.world, d.parity = self.rank, self.world, parity
        return d

    def next(self):
        d = self._desc[self.calls & 1]
        self.calls += 1
        return d

    # ---- pull protocol (sx8_glue_allreduce_add_rmsnorm)
    def partial_out(self, M, N):
        """The (M, N) f32 view a row-parallel linear writes its partial into for the next
        reduce_norm() call: slot 0 of the current half of this rank's own buffer."""
        if M * N > self.slot_elems:
            raise ops.SX8Error("partial (%d, %d) exceeds the exchange slot (%d elements)" % (M, N, self.slot_elems))
        off = (self.pull_calls & 1) * self.world * self.slot_elems
        return self.data[off:off + M * N].view(M, N)

    def reduce_norm(self, h, gamma, eps, x_out):
        """h += sum over ranks of the partials written through partial_out(); x_out = rmsnorm(h)."""
        d = self._desc[self.pull_calls & 1]
        self.pull_calls += 1
        return ops.glue_allreduce_add_rmsnorm(d, h, gamma, eps, x_out)

    def check(self):
        """Raise if a bounded wait of either exchange kernel ever ran out on this device (the sums
        of that call were taken without the late rank's data, and later calls are out of step)."""
        from . import _lib
        flag = _lib.device_error_flag()
        if flag & 0xC:
            raise ops.SX8Error("tensor-parallel exchange timed out waiting for a peer (device error word 0x%x): "
                               "results since then are invalid; rebuild the PeerExchange on all ranks" % flag)
        return flag


def linear(x, t, out=None, flags=0, group=None, reduce=True, exchange=None):
    """y = x @ W^T for a (possibly sharded) S-X8 tensor.  x: (M, K_local) f16.  For a
    row-parallel shard the fp32 partial is summed over ranks: through `exchange` (a
    PeerExchange: the GEMV stores into peer memory and a small kernel reduces) when given and
    M <= 8, else with an NCCL all-reduce in place; reduce=False skips it.  M <= 8 runs the
    decode GEMV, larger M the GEMM."""
    M = x.shape[0]
    row = reduce and t.get("style") == "row" and torch.distributed.is_initialized() \
        and torch.distributed.get_world_size(group) > 1
    if row and exchange is not None and M <= 8 and M * t["N"] <= exchange.slot_elems:
        return ops.gemv_allreduce(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"],
                                  exchange.next(), out=out, flags=flags)
    if M <= 8:
        y = ops.gemv(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], out=out, flags=flags)
    else:
        y = ops.gemm(x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], out_dtype=torch.float32,
                     out=out)
    if row:
        torch.distributed.all_reduce(y, group=group)
    return y


class TPStack:
    """A stack of Llama-shaped decoder layers as tensor-parallel S-X8 linears, one rank's part:
    per layer  x -> q|k|v (column) -> o (row, summed over ranks) -> residual + RMSNorm ->
    gate|up (column) -> SiLU(gate)*up -> down (row, summed) -> residual + RMSNorm, then a
    vocabulary-sharded lm_head whose logit shards are gathered.  Column-parallel outputs feed
    the row-parallel linears directly, so every rank only ever holds its own slice of the
    q / ffn activations.  Attention over a KV cache is not part of the S-X8 path and is stood
    in for by a cast of the local q slice (the o projection then reads (M, n_q/world) values
    as it would after attention).

    M <= 8 runs the decode GEMV (q|k|v and gate|up as one launch each), larger M the GEMM.
    layers: list of dicts name -> this rank's shard (shard_tensor); head: column shard or None.
    How the partial sums of o and down are combined (reduce=):
      "nccl"  all-reduce by NCCL, then sx8_glue_add_rmsnorm;
      "pull"  (needs exchange) the linear writes its partial into this rank's exchange slot and
              ONE kernel, sx8_glue_allreduce_add_rmsnorm, pulls all ranks' partials over NVLink,
              sums them and applies residual + RMSNorm;
      "push"  (needs exchange, M <= 8) sx8_gemv_allreduce pushes tiles into the peers' slots from
              the GEMV epilogue and a small kernel sums them, then sx8_glue_add_rmsnorm."""

    def __init__(self, layers, head, hidden, M, device, group=None, exchange=None, flags=0, eps=1e-5, reduce=None):
        self.layers, self.head, self.M, self.dev = layers, head, int(M), device
        self.group, self.exchange, self.flags, self.eps = group, exchange, flags, eps
        self.reduce = reduce if reduce is not None else ("push" if exchange is not None else "nccl")
        if self.reduce != "nccl" and exchange is None:
            raise ops.SX8Error("reduce=%r needs a PeerExchange" % (self.reduce,))
        if self.reduce == "pull" and M * hidden > exchange.slot_elems:
            self.reduce = "nccl"            # the partial does not fit the exchange slot
        self.world = torch.distributed.get_world_size(group) if torch.distributed.is_initialized() else 1
        o = layers[0]["o"]
        if o.get("global") is None or o["global"][1] == o["K"]:     # unsharded tensors: one rank's whole model
            self.world = 1
        f16, f32 = dict(dtype=torch.float16, device=device), dict(dtype=torch.float32, device=device)
        L0 = layers[0]
        self.h = torch.zeros(M, hidden, **f32)                     # residual stream
        self.x = torch.zeros(M, hidden, **f16)                     # normalised input of the next linear
        self.gamma = torch.ones(hidden, **f32)
        self.attn = torch.empty(M, L0["o"]["K"], **f16)
        self.act = torch.empty(M, L0["down"]["K"], **f16)
        self.y_o = torch.empty(M, hidden, **f32)
        self.y_d = torch.empty(M, hidden, **f32)
        self.multi = None
        if M <= 8:
            self.multi = [(ops.MultiGemv([L["q"], L["k"], L["v"]], M, device), ops.MultiGemv([L["gate"], L["up"]], M, device))
                          for L in layers]
        else:   # one tensor-core launch per group where the shard widths allow it (sx8_gemm_multi)
            self.qkv = [torch.empty(M, L0[n]["N"], **f32) for n in ("q", "k", "v")]
            self.gu = [torch.empty(M, L0[n]["N"], **f32) for n in ("gate", "up")]
            self.multi_gemm = [(ops.MultiGemm([L["q"], L["k"], L["v"]]), ops.MultiGemm([L["gate"], L["up"]])) for L in layers]
        self.logits_local = torch.empty(M, head["N"], **f32) if head is not None else None
        self.logits = None
        if head is not None and self.world > 1:
            self.logits = torch.empty(self.world, M, head["N"], **f32)
        self.packed_bytes = sum(30 * t["N"] * t["n_cb"] for L in layers for t in L.values()) + \
            (30 * head["N"] * head["n_cb"] if head is not None else 0)

    def _row_norm(self, x, t, out):
        """Row-parallel linear, sum over ranks, h += sum, self.x = rmsnorm(h)."""
        if self.world > 1 and self.reduce == "pull":
            part = self.exchange.partial_out(self.M, t["N"])
            linear(x, t, out=part, flags=self.flags, group=self.group, reduce=False)
            self.exchange.reduce_norm(self.h, self.gamma, self.eps, self.x)
            return
        linear(x, t, out=out, flags=self.flags, group=self.group,
               exchange=self.exchange if (self.world > 1 and self.reduce == "push") else None, reduce=self.world > 1)
        ops.glue_add_rmsnorm(self.h, out, self.gamma, self.eps, self.x)

    def step(self):
        """One pass over all layers from the current self.x / self.h; leaves the gathered logits
        (world, M, vocab/world) in self.logits (self.logits_local when world == 1)."""
        M = self.M
        for i, L in enumerate(self.layers):
            if self.multi is not None:
                q, _, _ = self.multi[i][0](self.x, flags=self.flags)
            else:
                q, _, _ = self.multi_gemm[i][0](self.x, outs=self.qkv)
            self.attn.copy_(q)                                        # stand-in for attention over the cache
            self._row_norm(self.attn, L["o"], self.y_o)
            if self.multi is not None:
                g, u = self.multi[i][1](self.x, flags=self.flags)
            else:
                g, u = self.multi_gemm[i][1](self.x, outs=self.gu)
            ops.glue_silu_mul(g, u, self.act)
            self._row_norm(self.act, L["down"], self.y_d)
        if self.head is not None:
            t = self.head
            if M <= 8:
                ops.gemv(self.x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], out=self.logits_local,
                         flags=self.flags)
            else:
                ops.gemm(self.x, t["wt16"], t["bases"], t["scales"], t["N"], t["K"], t["n_cb"], out=self.logits_local)
            if self.logits is not None:
                torch.distributed.all_gather_into_tensor(self.logits, self.logits_local, group=self.group)
                return self.logits
        return self.logits_local

    def reset(self, x0):
        """Start of a sequence of steps: residual stream zero, first input x0 (M, hidden) f16."""
        self.h.zero_()
        self.x.copy_(x0)
