"""A constants file without pickle: the dict that `exact.consts.build` / `int8.consts.build` return, stored as a JSON
header plus raw little-endian tensor bytes.

The reference keeps its constants as a `torch.save` file, i.e. Python pickle, which must not be loaded from an
untrusted source (docs/REPRODUCING.md:43-45 of the reference). Here loading only parses JSON and views bytes.

Layout: 8 bytes magic `BXCONST1`, 8 bytes little-endian header length H, H bytes of JSON, then the data section,
every tensor at a 64-byte aligned offset relative to the start of the data section. Header:
  {"tensors": {name: {"dtype": "int8", "shape": [..], "offset": o, "nbytes": n}}, "values": {name: json value},
   "sha256": digest of the data section}
`values` holds the non-tensor entries (config dict, layer count, integer scalars)."""

import hashlib
import json
import mmap
import struct

import numpy as np
import torch

MAGIC = b"BXCONST1"
ALIGN = 64
_DTYPES = {"int8": (torch.int8, np.int8), "int16": (torch.int16, np.int16), "int32": (torch.int32, np.int32),
           "int64": (torch.int64, np.int64), "uint8": (torch.uint8, np.uint8), "bool": (torch.bool, np.bool_),
           "float32": (torch.float32, np.float32), "float64": (torch.float64, np.float64)}
_NAMES = {t: k for k, (t, _) in _DTYPES.items()}


def _plain(v):
    """A JSON value for a non-tensor entry (numpy / torch scalars become Python numbers)."""
    if isinstance(v, dict):
        return {str(k): _plain(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    if isinstance(v, (np.integer,)):
        return int(v)
    if isinstance(v, (np.floating,)):
        return float(v)
    if isinstance(v, (bool, int, float, str)) or v is None:
        return v
    raise TypeError(f"constants entry of type {type(v).__name__} has no JSON form")


def save(c, path):
    """Write the constants dict c to path. Tensors may live on any device; they are stored contiguous."""
    tensors, values, off = {}, {}, 0
    order = []
    for k, v in c.items():
        if torch.is_tensor(v):
            if v.dtype not in _NAMES:
                raise TypeError(f"{k}: dtype {v.dtype} is not storable")
            n = v.numel() * v.element_size()
            tensors[k] = {"dtype": _NAMES[v.dtype], "shape": list(v.shape), "offset": off, "nbytes": n}
            order.append(k)
            off += (n + ALIGN - 1) // ALIGN * ALIGN
        else:
            values[k] = _plain(v)
    h = hashlib.sha256()
    pad = bytes(ALIGN)
    with open(path, "wb") as f:
        f.write(MAGIC + bytes(8))                                   # header length patched below
        body = []
        for k in order:
            b = c[k].detach().contiguous().cpu().numpy().tobytes()
            b += pad[: (-len(b)) % ALIGN]
            h.update(b)
            body.append(b)
        head = json.dumps({"tensors": tensors, "values": values, "sha256": h.hexdigest()}, sort_keys=True).encode()
        head += b" " * ((-(16 + len(head))) % ALIGN)                 # the data section starts on a 64-byte boundary
        f.write(head)
        for b in body:
            f.write(b)
        f.seek(8)
        f.write(struct.pack("<Q", len(head)))


def load(path, device="cpu", verify=True):
    """Read a constants file -> dict (tensors on `device`). verify: recompute the data section's SHA-256."""
    with open(path, "rb") as f:
        pre = f.read(16)
        if len(pre) != 16 or pre[:8] != MAGIC:
            raise ValueError("not a constants file")
        (hl,) = struct.unpack("<Q", pre[8:])
        if hl > 1 << 28:
            raise ValueError("header too large")
        head = json.loads(f.read(hl).decode())
        base = 16 + hl
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    size = len(mm) - base
    if verify and hashlib.sha256(memoryview(mm)[base:]).hexdigest() != head.get("sha256"):
        raise ValueError("constants file: data section does not match its SHA-256")
    c = dict(head.get("values", {}))
    for k, t in head["tensors"].items():
        if t["dtype"] not in _DTYPES:
            raise ValueError(f"{k}: unknown dtype {t['dtype']}")
        tdt, ndt = _DTYPES[t["dtype"]]
        shape = [int(x) for x in t["shape"]]
        n = int(np.prod(shape, dtype=np.int64)) * np.dtype(ndt).itemsize if shape else np.dtype(ndt).itemsize
        off = int(t["offset"])
        if n != int(t["nbytes"]) or off < 0 or off % ALIGN or off + n > size or min(shape, default=0) < 0:
            raise ValueError(f"{k}: bad extent")
        a = np.frombuffer(mm, dtype=ndt, count=n // np.dtype(ndt).itemsize, offset=base + off).reshape(shape)
        c[k] = torch.from_numpy(a.copy()).to(tdt).to(device)
    return c
