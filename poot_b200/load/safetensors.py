"""safetensors reader (memory-mapped, duplicate-key-refusing header) and writer.

File = u64 little-endian header length, a JSON object ``{name: {dtype, shape, data_offsets}, "__metadata__": ..}``,
then the tensor bytes.  The reader checks what a hostile file can get wrong: header length against the file size,
duplicate keys (the JSON standard leaves them undefined), offsets that overlap, leave gaps or overrun the data
section, and a byte count that disagrees with dtype x shape (crates/poot-load/src/safetensors.rs:295-371).
Sharded checkpoints are merged through ``model.safetensors.index.json``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from ..quant.weights import PackedWeight, WeightStore
from ..tensor import SAFETENSORS_NAMES, DType

MAX_HEADER = 100 * 1024 * 1024
_DT_TO_FORMAT = {DType.F32: "F32", DType.F16: "F16", DType.BF16: "BF16"}
_NAMES = {v: k for k, v in SAFETENSORS_NAMES.items()}


class SafetensorsError(ValueError):
    pass


def _no_duplicates(pairs):
    d = {}
    for k, v in pairs:
        if k in d:
            raise SafetensorsError(f"duplicate key {k!r} in the header")
        d[k] = v
    return d


def read_header(path: str) -> Tuple[Dict[str, Any], int, mmap.mmap]:
    f = open(path, "rb")
    size = os.fstat(f.fileno()).st_size
    if size < 8:
        raise SafetensorsError("file too small")
    mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    (n,) = struct.unpack_from("<Q", mm, 0)
    if n > MAX_HEADER or 8 + n > size:
        raise SafetensorsError(f"header length {n} overruns the file")
    try:
        header = json.loads(bytes(mm[8:8 + n]).decode("utf-8"), object_pairs_hook=_no_duplicates)
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"header is not valid JSON: {e}") from None
    if not isinstance(header, dict):
        raise SafetensorsError("header is not a JSON object")
    return header, 8 + n, mm


def read_tensors(path: str) -> Dict[str, Tuple[DType, Tuple[int, ...], np.ndarray]]:
    header, start, mm = read_header(path)
    raw = np.frombuffer(mm, dtype=np.uint8)
    data_len = raw.size - start
    out, spans = {}, []
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dt, shape, (lo, hi) = SAFETENSORS_NAMES[info["dtype"]], tuple(int(s) for s in info["shape"]), info["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"tensor {name!r}: malformed entry") from None
        n = 1
        for s in shape:
            if s < 0:
                raise SafetensorsError(f"tensor {name!r}: negative extent")
            n *= s
        if not (0 <= lo <= hi <= data_len) or hi - lo != n * dt.size:
            raise SafetensorsError(f"tensor {name!r}: offsets [{lo}, {hi}) do not match {dt} x {shape}")
        spans.append((lo, hi, name))
        out[name] = (dt, shape, raw[start + lo:start + hi])
    spans.sort()
    pos = 0
    for lo, hi, name in spans:
        if lo != pos:
            raise SafetensorsError(f"tensor {name!r}: data section has a gap or an overlap at byte {lo}")
        pos = hi
    out["__mmap__"] = mm  # keep the mapping alive with the views
    return out


def as_numpy(dt: DType, shape, raw: np.ndarray) -> np.ndarray:
    return raw.view(dt.storage_numpy).reshape(shape)


def load_weight_store(path: str, check: bool = True) -> WeightStore:
    """A file, or a directory with ``model.safetensors`` / an index of shards."""
    files: List[str]
    if os.path.isdir(path):
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                files = sorted({os.path.join(path, v) for v in json.load(f)["weight_map"].values()})
        else:
            files = sorted(os.path.join(path, n) for n in os.listdir(path) if n.endswith(".safetensors"))
    else:
        files = [path]
    if not files:
        raise SafetensorsError(f"no safetensors files under {path!r}")
    store = WeightStore()
    store.source = path
    store._maps = []
    for fp in files:
        ts = read_tensors(fp)
        store._maps.append(ts.pop("__mmap__"))
        for name, (dt, shape, raw) in ts.items():
            fmt = _DT_TO_FORMAT.get(dt)
            if fmt is not None:
                store.add(PackedWeight(name, fmt, shape, raw))
            else:   # operand of a planar quantised format (int32 qweight, fp8 weight, scales ...): keep typed
                store.add(PackedWeight(name, "F32", shape, raw, planar={"__raw__": as_numpy(dt, shape, raw)}))
    return store.publish(check=False)


def write_safetensors(path: str, tensors: Dict[str, Tuple[DType, np.ndarray]], metadata: Optional[Dict[str, str]] = None) -> None:
    header: Dict[str, Any] = {}
    if metadata:
        header["__metadata__"] = metadata
    off, blobs = 0, []
    for name, (dt, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        header[name] = {"dtype": _NAMES[dt], "shape": list(arr.shape), "data_offsets": [off, off + raw.nbytes]}
        off += raw.nbytes
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj)
        for b in blobs:
            f.write(b.tobytes())
