"""`.sx8v43` container: index, read, write, and load straight into the device layout.

Byte format (little endian), identical to ref scripts/sx8_container_v43.py:12-43:

    "SX43FILE" | u8 version=1 | u32 len | repr(sorted(meta.items())) |
    u32 n_tensors | per tensor, sorted by name:
        u32 len | name | u32 out_f | u32 in_f | u8 n_dims | u32 orig_shape[n_dims] |
        u32 n_blocks | u32 n_cb |
        dmin f16[nb] | dmax f16[nb] | config u8[nb] | levels_hi u8[16 nb] |
        levels_lo u8[8 nb] | coeff u8[nb] |
        u32 n_cb | bases f32[n_cb*64] | scales f32[n_cb*2]

Differences from the reference module of the same name (same public functions
`write_sx43`, `verify_sx43`, `read_all`):
  * the file is memory-mapped and indexed once; tensors are numpy views, nothing is read
    until touched (the reference reads every plane with f.read);
  * the metadata is parsed with ast.literal_eval, not eval;
  * `load_to_device` goes file -> pinned staging -> device planes -> T16 blob
    (sx8_repack_t16 on the GPU).  The reference's load path decodes every tensor with a
    numba kernel and builds kb-major host copies first (ref scripts/eval_common.py:111-123,
    scripts/integrate_fused.py:51-58, scripts/prepare_v44.py:35-79)."""
import ast
import pickle
import struct

import numpy as np

MAGIC = b"SX43FILE"
VERSION = 1
BYTES_PER_BLOCK = 30

_PLANES = (("dmin", 2, np.float16), ("dmax", 2, np.float16), ("config", 1, np.uint8),
           ("levels_hi", 16, np.uint8), ("levels_lo", 8, np.uint8), ("coeff", 1, np.uint8))


class ContainerError(ValueError):
    pass


def _as_dict(src):
    if isinstance(src, (str, bytes)):
        with open(src, "rb") as f:
            return pickle.load(f)
    return src


def write_sx43(pkl_path, out_path, verbose=True):
    """pkl_path: path of a pkl {"weights","bases","meta"} (as the reference) or that dict."""
    d = _as_dict(pkl_path)
    wd, bd, meta = d["weights"], d["bases"], d["meta"]
    n_blk_tot = 0
    with open(out_path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<B", VERSION))
        mb = repr(sorted(meta.items())).encode()
        f.write(struct.pack("<I", len(mb)))
        f.write(mb)
        f.write(struct.pack("<I", len(wd)))
        for name in sorted(wd):
            qt, bi = wd[name], bd[name]
            nb, ncb = int(qt["n_blocks"]), int(qt["n_cb"])
            nbytes = name.encode()
            f.write(struct.pack("<I", len(nbytes)))
            f.write(nbytes)
            sh = qt["shape"]
            os_ = qt.get("orig_shape") or sh
            f.write(struct.pack("<II", sh[0], sh[1]))
            f.write(struct.pack("<B", len(os_)))
            f.write(struct.pack("<%dI" % len(os_), *os_))
            f.write(struct.pack("<II", nb, ncb))
            for key, per, dt in _PLANES:
                a = np.ascontiguousarray(np.asarray(qt[key]).reshape(-1)).astype(dt, copy=False)
                if a.size != nb * (per // a.itemsize):
                    raise ContainerError("%s: plane %s has %d elements, expected %d" %
                                         (name, key, a.size, nb * (per // a.itemsize)))
                f.write(a.tobytes())
            f.write(struct.pack("<I", int(bi["n_cb"])))
            f.write(np.ascontiguousarray(bi["data"], dtype=np.float32).tobytes())
            f.write(np.ascontiguousarray(bi["scales"], dtype=np.float32).tobytes())
            n_blk_tot += nb
    if verbose:
        print("wrote %s: %d tensors, %d blocks (%.3f GB at 30 B/block)" %
              (out_path, len(wd), n_blk_tot, n_blk_tot * BYTES_PER_BLOCK / 1e9))
    return out_path


class Entry:
    """One tensor of an indexed container: sizes and the byte offset of each plane."""
    __slots__ = ("name", "shape", "orig_shape", "n_blocks", "n_cb", "planes_offset", "bases_offset",
                 "scales_offset", "bases_n_cb")

    def plane_offsets(self):
        off, out = self.planes_offset, {}
        for key, per, _ in _PLANES:
            out[key] = (off, self.n_blocks * per)
            off += self.n_blocks * per
        return out


class Container:
    """Memory-mapped `.sx8v43` file.  `entries[name]` is an Entry; `tensor(name)` returns the
    reference-format dicts (qt, bases_info) as views of the mapping."""

    def __init__(self, path):
        self.path = path
        self.mm = np.memmap(path, dtype=np.uint8, mode="r")
        self.entries = {}
        self.meta = {}
        self._index()

    def _index(self):
        mm = self.mm
        size = mm.size

        def take(off, n):
            if off + n > size:
                raise ContainerError("%s: truncated at byte %d" % (self.path, off))
            return bytes(mm[off:off + n]), off + n

        raw, off = take(0, 8)
        if raw != MAGIC:
            raise ContainerError("%s: not an SX43FILE container" % self.path)
        raw, off = take(off, 1)
        if raw[0] != VERSION:
            raise ContainerError("%s: container version %d, this reader handles %d" % (self.path, raw[0], VERSION))
        raw, off = take(off, 4)
        raw, off = take(off, struct.unpack("<I", raw)[0])
        try:
            self.meta = dict(ast.literal_eval(raw.decode()))
        except (ValueError, SyntaxError) as e:
            raise ContainerError("%s: metadata is not a literal list of pairs (%s)" % (self.path, e))
        raw, off = take(off, 4)
        for _ in range(struct.unpack("<I", raw)[0]):
            e = Entry()
            raw, off = take(off, 4)
            raw, off = take(off, struct.unpack("<I", raw)[0])
            e.name = raw.decode()
            raw, off = take(off, 8)
            e.shape = struct.unpack("<II", raw)
            raw, off = take(off, 1)
            n_os = raw[0]
            raw, off = take(off, 4 * n_os)
            e.orig_shape = struct.unpack("<%dI" % n_os, raw)
            raw, off = take(off, 8)
            e.n_blocks, e.n_cb = struct.unpack("<II", raw)
            if e.n_blocks != e.shape[0] * e.n_cb or e.n_cb != (e.shape[1] + 31) // 32:
                raise ContainerError("%s: %s has n_blocks=%d n_cb=%d for shape %s" %
                                     (self.path, e.name, e.n_blocks, e.n_cb, e.shape))
            e.planes_offset = off
            off += e.n_blocks * BYTES_PER_BLOCK
            raw, off = take(off, 4)
            e.bases_n_cb = struct.unpack("<I", raw)[0]
            e.bases_offset = off
            off += e.bases_n_cb * 64 * 4
            e.scales_offset = off
            off += e.bases_n_cb * 2 * 4
            if off > size:
                raise ContainerError("%s: truncated inside %s" % (self.path, e.name))
            self.entries[e.name] = e

    def tensor(self, name):
        e = self.entries[name]
        qt = {"shape": tuple(e.shape), "orig_shape": tuple(e.orig_shape) if tuple(e.orig_shape) != tuple(e.shape) else None,
              "n_blocks": e.n_blocks, "n_cb": e.n_cb}
        for key, (off, nbytes) in e.plane_offsets().items():
            dt = np.float16 if key in ("dmin", "dmax") else np.uint8
            qt[key] = self.mm[off:off + nbytes].view(dt)
        n = e.bases_n_cb
        bi = {"n_cb": n, "data": self.mm[e.bases_offset:e.bases_offset + n * 256].view(np.float32).reshape(n, 64),
              "scales": self.mm[e.scales_offset:e.scales_offset + n * 8].view(np.float32).reshape(n, 2)}
        return qt, bi

    def names(self):
        return list(self.entries)


def read_all(sx43_path):
    """(wd, bd, meta) in the reference's dict format (ref scripts/sx8_container_v43.py:88-118);
    the arrays are views of a memory mapping."""
    c = Container(sx43_path)
    wd, bd = {}, {}
    for name in c.names():
        wd[name], bd[name] = c.tensor(name)
    return wd, bd, dict(c.meta)


def verify_sx43(pkl_path, sx43_path):
    """True when every array in the container equals the pkl's (ref :45-86)."""
    d = _as_dict(pkl_path)
    wd, bd, _ = read_all(sx43_path)
    if sorted(wd) != sorted(d["weights"]):
        return False
    for name, qt in d["weights"].items():
        got, bi, want_bi = wd[name], bd[name], d["bases"][name]
        for key, _, dt in _PLANES:
            if not np.array_equal(np.asarray(got[key]).reshape(-1), np.asarray(qt[key]).reshape(-1).astype(dt, copy=False)):
                return False
        if not (np.array_equal(bi["data"], np.asarray(want_bi["data"], dtype=np.float32)) and
                np.array_equal(bi["scales"], np.asarray(want_bi["scales"], dtype=np.float32))):
            return False
    return True


def load_to_device(sx43_path, names=None, device="cuda"):
    """Load tensors of a container into the device layout used by every kernel of this
    library: {name: {"wt16", "bases", "scales", "N", "K", "n_cb"}}.

    Per tensor: the six planes are one contiguous 30*n_blocks-byte range of the file; it is
    copied into one of two pinned staging buffers (so the host copy of tensor i+1 overlaps the
    transfer and repack of tensor i), sent to the device plane by plane, and repacked to T16 by
    sx8_repack_t16.  No host-side transposes, no decode at load."""
    import torch
    from . import ops
    dev = torch.device(device)
    c = Container(sx43_path)
    want = list(names) if names is not None else c.names()
    if not want:
        return {}
    max_nb = max(c.entries[n].n_blocks for n in want)
    stage = [torch.empty(max_nb * BYTES_PER_BLOCK, dtype=torch.uint8).pin_memory() for _ in range(2)]
    done = [None, None]
    out = {}
    with torch.cuda.device(dev):
        for i, name in enumerate(want):
            e = c.entries[name]
            nb = e.n_blocks
            sb = stage[i & 1]
            if done[i & 1] is not None:
                done[i & 1].synchronize()          # the transfer that last used this buffer
            sb[:nb * BYTES_PER_BLOCK].numpy()[:] = c.mm[e.planes_offset:e.planes_offset + nb * BYTES_PER_BLOCK]
            planes, off = {}, 0
            for key, per, _ in _PLANES:
                t = torch.empty(nb * per, dtype=torch.uint8, device=dev)
                t.copy_(sb[off:off + nb * per], non_blocking=True)
                planes[key] = t
                off += nb * per
            ev = torch.cuda.Event()
            ev.record()
            done[i & 1] = ev
            n = e.bases_n_cb
            bases = torch.from_numpy(np.array(c.mm[e.bases_offset:e.bases_offset + n * 256]).view(np.float32).reshape(n, 64)).to(dev)
            scales = torch.from_numpy(np.array(c.mm[e.scales_offset:e.scales_offset + n * 8]).view(np.float32).reshape(n, 2)).to(dev)
            wt16 = ops.repack_t16(planes["dmin"].view(torch.float16), planes["dmax"].view(torch.float16), planes["config"],
                                  planes["coeff"], planes["levels_hi"], planes["levels_lo"], e.shape[0], e.n_cb)
            out[name] = {"wt16": wt16, "bases": bases, "scales": scales, "N": e.shape[0], "K": e.shape[1],
                         "n_cb": e.n_cb, "orig_shape": tuple(e.orig_shape)}
        torch.cuda.synchronize(dev)
    return out
