"""Tensor-parallel host logic on CPU: shard bounds, shard byte-identity against the
oracle's own T16 blobs, and a world_size-2 gloo run in which every rank computes its
partial with the CPU oracle and the all-reduce reproduces the unsharded result."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sx8_oracle as orc
from sx8_quantization_b200 import tp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_cover_and_align():
    for total, world, q in [(1024, 8, 16), (9728, 8, 16), (28672, 8, 16), (304, 8, 1), (80, 3, 1), (48, 4, 16)]:
        spans = [tp.shard_bounds(total, r, world, q) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c
        assert all(a % q == 0 and b % q == 0 for a, b in spans)
    with pytest.raises(Exception):
        tp.shard_bounds(100, 0, 2, 16)


def _tensor(N, K, seed):
    w = orc.synth_weight(N, K, seed)
    qt, bi = orc.quantize(w)
    t = {"wt16": torch.from_numpy(orc.to_t16(qt)).reshape(-1, 480), "bases": torch.from_numpy(bi["data"]),
         "scales": torch.from_numpy(bi["scales"]), "N": N, "K": K, "n_cb": qt["n_cb"]}
    return w, qt, bi, t


def _sub_qt(qt, bi, n0, n1, kb0, kb1):
    """Slice of the file planes: rows n0:n1, block columns kb0:kb1."""
    N, n_cb = qt["shape"][0], qt["n_cb"]
    def cut(a, per):
        return np.ascontiguousarray(np.asarray(a).reshape(N, n_cb, per)[n0:n1, kb0:kb1]).reshape(-1)
    q = {"shape": (n1 - n0, (kb1 - kb0) * 32), "n_cb": kb1 - kb0, "n_blocks": (n1 - n0) * (kb1 - kb0),
         "dmin": cut(qt["dmin"], 1), "dmax": cut(qt["dmax"], 1), "config": cut(qt["config"], 1),
         "coeff": cut(qt["coeff"], 1), "levels_hi": cut(qt["levels_hi"], 16), "levels_lo": cut(qt["levels_lo"], 8)}
    b = {"n_cb": kb1 - kb0, "data": bi["data"][kb0:kb1], "scales": bi["scales"][kb0:kb1]}
    return q, b


@pytest.mark.parametrize("world", [2, 4])
def test_shards_are_byte_identical_to_slices(world):
    w, qt, bi, t = _tensor(64, 256, 3)
    for rank in range(world):
        c = tp.shard_tensor(t, "col", rank, world)
        n0, n1 = c["n_range"]
        q, _ = _sub_qt(qt, bi, n0, n1, 0, qt["n_cb"])
        assert np.array_equal(c["wt16"].numpy().reshape(-1), orc.to_t16(q))
        r = tp.shard_tensor(t, "row", rank, world)
        k0, k1 = r["k_range"]
        q, b = _sub_qt(qt, bi, 0, 64, k0 // 32, k1 // 32)
        assert np.array_equal(r["wt16"].numpy().reshape(-1), orc.to_t16(q))
        assert np.array_equal(r["bases"].numpy(), b["data"])


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w, qt, bi, t = _tensor(64, 256, 3)
    x = orc.synth_x(2, 256, 9)
    # row-parallel: each rank owns a K range and all-reduces its partial
    r = tp.shard_tensor(t, "row", rank, world)
    k0, k1 = r["k_range"]
    q, b = _sub_qt(qt, bi, 0, 64, k0 // 32, k1 // 32)
    part = torch.from_numpy(orc.matmul_ref(x[:, k0:k1], orc.dequant_d64(q, b)))
    dist.all_reduce(part)
    # column-parallel: each rank owns rows of W; gather the pieces
    c = tp.shard_tensor(t, "col", rank, world)
    n0, n1 = c["n_range"]
    q, b = _sub_qt(qt, bi, n0, n1, 0, qt["n_cb"])
    piece = torch.from_numpy(orc.matmul_ref(x, orc.dequant_d64(q, b)))
    pieces = [torch.empty_like(piece) for _ in range(world)]
    dist.all_gather(pieces, piece)
    if rank == 0:
        full = orc.matmul_ref(x, orc.dequant_d64(qt, bi))
        np.save(out, np.stack([part.numpy(), torch.cat(pieces, dim=1).numpy(), full]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_row_and_column_parallel(tmp_path):
    out = str(tmp_path / "res.npy")
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    row, col, full = np.load(out)
    assert np.allclose(row, full, rtol=0, atol=1e-4 * np.abs(full).max())
    assert np.array_equal(col, full)
