"""Projection shapes of the two decoder families the benchmark configurations name
(dense decoder, GQA attention, SwiGLU MLP).  Each entry: name -> (out_features N,
in_features K, tensor-parallel style: "col" shards N, "row" shards K + all-reduce)."""

QWEN3_4B = {
    "hidden": 2560, "layers": 36, "vocab": 151936,
    "proj": [("q", 4096, 2560, "col"), ("k", 1024, 2560, "col"), ("v", 1024, 2560, "col"),
             ("o", 2560, 4096, "row"), ("gate", 9728, 2560, "col"), ("up", 9728, 2560, "col"),
             ("down", 2560, 9728, "row")],
}

LLAMA_70B = {
    "hidden": 8192, "layers": 80, "vocab": 128256,
    "proj": [("q", 8192, 8192, "col"), ("k", 1024, 8192, "col"), ("v", 1024, 8192, "col"),
             ("o", 8192, 8192, "row"), ("gate", 28672, 8192, "col"), ("up", 28672, 8192, "col"),
             ("down", 8192, 28672, "row")],
}


def packed_bytes(N, K):
    """Algorithmic bytes of one packed matrix: 30 bytes per 32 weights
    (ref scripts/sx8_decode1_v3.py:168 with hdr_bytes = 6)."""
    return 30 * N * ((K + 31) // 32)


def layer_bytes(family):
    return sum(packed_bytes(n, k) for _, n, k, _ in family["proj"])
