"""Drop-in for the reference's scripts/sx8_embed_v44.py (ref :40-72): an nn.Module that
decodes only the rows of the active tokens into a preallocated fp16 buffer."""
import torch
import torch.nn as nn

from . import ops


class SX8EmbeddingV44(nn.Module):
    def __init__(self, qt, bases_info, hdr_bytes=6):
        super().__init__()
        self.qt = qt
        self.bases_info = bases_info
        self.N = int(qt["shape"][0])
        self.K = int(qt["shape"][1])
        self.n_cb = int(qt["n_cb"])
        self.hdr_bytes = 6  # the reference always builds the 6-byte header here (ref :56-57)
        self._t = None
        self._out = None

    def _load(self, device):
        if self._t is None:
            from .sx8_decode1_v3 import make_tensors_v44
            self._t = make_tensors_v44(self.qt, self.bases_info, hdr_aligned=False, device=device)
            self._hdr, self._lvl, self._bas, self._sca = self._t
            self.qt = None
            self.bases_info = None

    def forward(self, ids):
        dev = ids.device if ids.is_cuda else torch.device("cuda", torch.cuda.current_device())
        self._load(dev)
        ids = ids.to(dev)
        T = ids.numel()
        if self._out is None or self._out.shape[0] < T:
            self._out = torch.empty(T, self.K, dtype=torch.float16, device=dev)
        out = self._out[:T]
        ops.embed(ids, self._lvl, self._bas, self._sca, self.K, self.N, self.n_cb, out=out)
        return out.reshape(*ids.shape, self.K)
