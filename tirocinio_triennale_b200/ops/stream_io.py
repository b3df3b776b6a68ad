"""The compressed stream as an on-disk format for float32 tensors.

A ``.hcz`` file is a 64-byte little-endian header followed by the stream bytes exactly as the codec
produced them (the reference has no file format of its own: its drivers dump raw floats,
HomComp/src/main_allred.cu:120-128; here the stream doubles as a compressed-tensor container):

    offset  size  field
    0       8     magic  b"HCZSTRM1"
    8       8     n            number of float32 values
    16      8     stream_bytes length of the stream that follows
    24      4     eb           absolute error bound (float32)
    28      4     mode         0 outlier, 1 plain, 2 vec
    32      4     ndim, then up to 6 x uint32 dims (row-major shape; 0-filled)
    60      4     reserved

``save_tensor`` / ``load_tensor`` work on CPU tensors through the portable codec and on CUDA
tensors through the sm_100a codec; files written by one are read by the other (same bytes).
``save_state`` / ``load_state`` store a whole ``state_dict``: float32 tensors above a size threshold
go in compressed, everything else through ``torch.save``.
"""
from __future__ import annotations

import io
import os
import struct
import zipfile

import numpy as np
import torch

from . import cpu_codec

MAGIC = b"HCZSTRM1"
HEADER = struct.Struct("<8sQQfII6II")
_MODES = {"outlier": 0, "plain": 1, "vec": 2}
_MODE_NAMES = {v: k for k, v in _MODES.items()}


def pack_header(n: int, stream_bytes: int, eb: float, mode: str, shape) -> bytes:
    shape = tuple(int(d) for d in shape)
    if len(shape) > 6:
        shape = (int(np.prod(shape)),)
    dims = shape + (0,) * (6 - len(shape))
    return HEADER.pack(MAGIC, n, stream_bytes, eb, _MODES[mode], len(shape), *dims, 0)


def unpack_header(raw: bytes):
    magic, n, nbytes, eb, mode, ndim, *rest = HEADER.unpack(raw[: HEADER.size])
    if magic != MAGIC:
        raise ValueError("not a compressed-stream file")
    if mode not in _MODE_NAMES or ndim > 6:
        raise ValueError("corrupt header")
    return n, nbytes, eb, _MODE_NAMES[mode], tuple(rest[:ndim])


def _compress(t: torch.Tensor, eb: float, mode: str) -> np.ndarray:
    flat = t.detach().reshape(-1)
    if flat.is_cuda:
        from .codec import Codec

        codec = Codec(flat.numel(), device=flat.device)
        out, size = codec.compress(flat.contiguous(), eb, mode=mode)
        return out[: int(size.item())].cpu().numpy()
    return cpu_codec.cpu_compress(flat.contiguous().numpy().astype(np.float32, copy=False), eb, mode=mode)


def _decompress(stream: np.ndarray, n: int, eb: float, mode: str, device) -> torch.Tensor:
    device = torch.device(device)
    if device.type == "cuda":
        from .codec import Codec

        codec = Codec(n, device=device)
        # own copy (the file buffer is read-only) with the slack that the kernel's 16-byte aligned
        # bulk copies may read past the last payload byte
        padded = np.zeros(stream.size + 64, dtype=np.uint8)
        padded[: stream.size] = stream
        s = torch.from_numpy(padded).to(device)
        out = codec.decompress(s, n, eb, mode=mode, stream_bytes=stream.size)
        st = codec.status()
        if st != 0:  # e.g. 2: the body is shorter than its rate bytes imply (cut-off or corrupted file)
            raise ValueError("corrupt stream: the device decoder reported status %d" % st)
        return out
    return torch.from_numpy(cpu_codec.cpu_decompress(stream, n, eb, mode=mode))


def dumps_tensor(t: torch.Tensor, eb: float, mode: str = "outlier") -> bytes:
    if t.dtype != torch.float32:
        raise ValueError("expected a float32 tensor")
    stream = _compress(t, eb, mode)
    return pack_header(t.numel(), stream.size, eb, mode, t.shape) + stream.tobytes()


def loads_tensor(raw: bytes, device="cpu") -> torch.Tensor:
    n, nbytes, eb, mode, shape = unpack_header(raw)
    body = np.frombuffer(raw, dtype=np.uint8, count=nbytes, offset=HEADER.size)
    if body.size != nbytes:
        raise ValueError("truncated file")
    out = _decompress(body, n, eb, mode, device)
    return out.reshape(shape) if int(np.prod(shape)) == n else out


def save_tensor(path, t: torch.Tensor, eb: float, mode: str = "outlier") -> int:
    """Writes ``t`` (float32, CPU or CUDA) to ``path``; returns the file size in bytes."""
    raw = dumps_tensor(t, eb, mode)
    tmp = str(path) + ".tmp%d" % os.getpid()
    with open(tmp, "wb") as f:
        f.write(raw)
    os.replace(tmp, path)
    return len(raw)


def load_tensor(path, device="cpu") -> torch.Tensor:
    with open(path, "rb") as f:
        return loads_tensor(f.read(), device)


def save_state(path, state: dict, eb: float, min_elems: int = 4096, mode: str = "outlier") -> dict:
    """``state_dict`` -> one zip: float32 tensors of at least ``min_elems`` values as streams with
    absolute error bound ``eb``, the rest (small tensors, other dtypes, python values) verbatim.
    Returns {"raw_bytes", "file_bytes"} of the compressed part."""
    plain, stats = {}, {"raw_bytes": 0, "file_bytes": 0}
    tmp = str(path) + ".tmp%d" % os.getpid()
    with zipfile.ZipFile(tmp, "w", zipfile.ZIP_STORED) as z:
        for i, (k, v) in enumerate(state.items()):
            if torch.is_tensor(v) and v.dtype == torch.float32 and v.numel() >= min_elems:
                raw = dumps_tensor(v, eb, mode)
                z.writestr("t%06d.hcz" % i, raw)
                plain[k] = ("__hcz__", "t%06d.hcz" % i)
                stats["raw_bytes"] += 4 * v.numel()
                stats["file_bytes"] += len(raw)
            else:
                plain[k] = v.detach().cpu() if torch.is_tensor(v) else v
        buf = io.BytesIO()
        torch.save(plain, buf)
        z.writestr("rest.pt", buf.getvalue())
    os.replace(tmp, path)
    return stats


def load_state(path, device="cpu") -> dict:
    out = {}
    with zipfile.ZipFile(path, "r") as z:
        # tensors, python scalars and the ("__hcz__", member) marker tuples only: nothing that needs pickle code
        plain = torch.load(io.BytesIO(z.read("rest.pt")), map_location="cpu", weights_only=True)
        for k, v in plain.items():
            if isinstance(v, tuple) and len(v) == 2 and v[0] == "__hcz__":
                out[k] = loads_tensor(z.read(v[1]), device)
            else:
                out[k] = v.to(device) if torch.is_tensor(v) else v
    return out
