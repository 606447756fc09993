"""Drop-in for the decode entry points of the reference's scripts/kernel_sx8_v43.py
(ref :54-82 decode_tensor_gpu, :109-145 decode_tensor_gpu_fast): the full-tensor
decode to fp16, bit-identical arithmetic (float64 decode, float32 rounding, fp16
cast), run by libsx8b200.so instead of a numba kernel."""
import numpy as np
import torch

from . import ops

DEV = torch.device("cuda")
N_BASES = 2
BYTES_PER_BLOCK = 30


def _up(a, dtype, device):
    return torch.from_numpy(np.ascontiguousarray(np.asarray(a).reshape(-1), dtype=dtype).view(np.uint8)).to(device)


def decode_tensor_gpu_fast(qt, bases_info, out=None, device=None):
    out_f, in_f = qt["shape"]
    n_cb = int(qt["n_cb"])
    if out is not None and tuple(out.shape) != (out_f, in_f):
        raise ValueError(f"out shape {tuple(out.shape)} != {(out_f, in_f)}")
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    W = ops.dequant_planes(_up(qt["dmin"], np.float16, dev), _up(qt["dmax"], np.float16, dev),
                           _up(qt["config"], np.uint8, dev), _up(qt["coeff"], np.uint8, dev),
                           _up(qt["levels_hi"], np.uint8, dev), _up(qt["levels_lo"], np.uint8, dev),
                           _up(bases_info["data"], np.float32, dev).view(torch.float32),
                           _up(bases_info["scales"], np.float32, dev).view(torch.float32),
                           int(out_f), int(in_f), n_cb, True)
    orig = qt.get("orig_shape")
    if orig is not None and tuple(orig) != (out_f, in_f):
        W = W.reshape(tuple(orig))
    if out is not None:
        out.copy_(W)
        return out
    return W


def decode_tensor_gpu(qt, bases_info):
    return decode_tensor_gpu_fast(qt, bases_info)
