"""GGUF v3 container: reader, weight loading and a small writer for tests.

Mirrors the host-side loader the reference keeps next to its quantized kernels
(GgufFile / GgufTensorInfo, src/KokkosDNN_GGUF.hpp:385-774; load_quant_weight, :864-885;
the synthetic writer its tests use, src/KokkosDNN_GGUF_Synthetic.hpp:49-173):

  header    magic "GGUF", version u32 (3), n_tensors u64, n_kv u64
  metadata  per KV: key string, value-type u32, value
  infos     per tensor: name string, n_dims u32, dims u64[n_dims] (ggml order: dims[0]
            varies fastest), ggml type u32, offset u64 from the start of the data section
  data      starts at the next 32-byte boundary; raw packed payloads

Strings are a u64 length plus bytes. Everything is little-endian. The file is memory-mapped
read-only; every tensor's byte range is validated while parsing, so payload() cannot run
past the mapping. Errors are RuntimeError, as the reference's std::runtime_error.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass, field
from typing import Any, Dict, List, Sequence, Tuple

import numpy as np

ALIGN = 32
VERSION = 3
# ggml type id -> (elements per block, bytes per block); src/KokkosDNN_GGUF.hpp:68-138
TYPE_INFO: Dict[int, Tuple[int, int]] = {
    0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 36),
    10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292),
    24: (1, 1), 25: (1, 2), 26: (1, 4), 30: (1, 2),
}
COMPUTE_TYPES = (8, 12, 13, 14)          # Q8_0, Q4_K, Q5_K, Q6_K: what the kernels of this library take
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
T_STRING, T_ARRAY = 8, 9


@dataclass
class GgufTensorInfo:
    name: str
    dims: List[int]            # ggml order: dims[0] is the fastest-varying extent
    dtype: int
    offset: int                # bytes from the start of the data section
    nbytes: int = 0
    numel: int = 0

    @property
    def n_dims(self) -> int:
        return len(self.dims)

    def rows(self) -> int:
        """Row-major matrix view: a 2-D tensor is stored as dims = {cols, rows}; a 1-D tensor is one row."""
        return 0 if not self.dims else (1 if len(self.dims) == 1 else self.dims[1])

    def cols(self) -> int:
        return self.dims[0] if self.dims else 0


class _Cursor:
    def __init__(self, buf, size: int):
        self.buf, self.size, self.pos = buf, size, 0

    def take(self, n: int, what: str) -> bytes:
        if n < 0 or self.pos + n > self.size:
            raise RuntimeError(f"GgufFile: truncated {what}")
        out = self.buf[self.pos:self.pos + n]
        self.pos += n
        return out

    def scalar(self, fmt: str, what: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt), what))[0]

    def string(self, what: str) -> str:
        n = self.scalar("<Q", what)
        return bytes(self.take(n, what)).decode("utf-8", errors="replace")


@dataclass
class GgufFile:
    path: str
    version: int = 0
    data_start: int = 0
    tensors: List[GgufTensorInfo] = field(default_factory=list)
    kv: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        try:
            self._fh = open(self.path, "rb")
        except OSError as ex:
            raise RuntimeError(f"GgufFile: cannot open '{self.path}'") from ex
        self._fh.seek(0, 2)
        self.size = self._fh.tell()
        if self.size < 24:
            raise RuntimeError(f"GgufFile: file too small '{self.path}'")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        self._index: Dict[str, int] = {}
        self._parse()

    # ---- parsing ---------------------------------------------------------------------
    def _value(self, c: _Cursor, vtype: int, key: str):
        if vtype in _SCALARS:
            return c.scalar(_SCALARS[vtype], f"value of '{key}'")
        if vtype == T_STRING:
            return c.string(f"string value of '{key}'")
        if vtype == T_ARRAY:
            etype = c.scalar("<I", f"array type of '{key}'")
            n = c.scalar("<Q", f"array length of '{key}'")
            if etype in _SCALARS and etype != 7:       # packed numeric array: one bulk read
                fmt = _SCALARS[etype]
                raw = c.take(n * struct.calcsize(fmt), f"array of '{key}'")
                return np.frombuffer(raw, dtype=np.dtype(fmt)).copy()
            return [self._value(c, etype, key) for _ in range(n)]
        raise RuntimeError(f"GgufFile: bad metadata type {vtype}")

    def _parse(self) -> None:
        c = _Cursor(self._map, self.size)
        if bytes(c.take(4, "magic")) != b"GGUF":
            raise RuntimeError("GgufFile: bad magic (not a GGUF file)")
        self.version = c.scalar("<I", "version")
        if self.version != VERSION:
            raise RuntimeError(f"GgufFile: unsupported version {self.version} (want 3)")
        n_tensors = c.scalar("<Q", "tensor count")
        n_kv = c.scalar("<Q", "metadata count")
        for _ in range(n_kv):
            key = c.string("metadata key")
            self.kv[key] = self._value(c, c.scalar("<I", "metadata type"), key)
        for _ in range(n_tensors):
            name = c.string("tensor name")
            n_dims = c.scalar("<I", "n_dims")
            if n_dims == 0 or n_dims > 4:
                raise RuntimeError(f"GgufFile: bad n_dims {n_dims} for '{name}'")
            dims = [c.scalar("<Q", "dims") for _ in range(n_dims)]
            dtype = c.scalar("<I", "tensor dtype")
            if dtype not in TYPE_INFO:
                raise RuntimeError(f"GgufFile: tensor '{name}' has unknown dtype {dtype}")
            numel = 1
            for d in dims:
                numel *= d
            blk, bsz = TYPE_INFO[dtype]
            if numel % blk:
                raise RuntimeError(f"GgufFile: tensor '{name}' numel not a multiple of block length")
            info = GgufTensorInfo(name, dims, dtype, c.scalar("<Q", "tensor offset"), numel // blk * bsz, numel)
            self._index[name] = len(self.tensors)
            self.tensors.append(info)
        self.data_start = (c.pos + ALIGN - 1) & ~(ALIGN - 1)
        if self.data_start > self.size:
            raise RuntimeError("GgufFile: header runs past EOF")
        for t in self.tensors:
            if self.data_start + t.offset + t.nbytes > self.size:
                raise RuntimeError(f"GgufFile: tensor '{t.name}' payload out of range")

    # ---- access ----------------------------------------------------------------------
    def has_tensor(self, name: str) -> bool:
        return name in self._index

    def tensor(self, name: str) -> GgufTensorInfo:
        if name not in self._index:
            raise RuntimeError(f"GgufFile: tensor not found '{name}'")
        return self.tensors[self._index[name]]

    def payload(self, info: GgufTensorInfo) -> np.ndarray:
        """Read-only uint8 view of the packed payload (zero-copy over the mapping)."""
        start = self.data_start + info.offset
        return np.frombuffer(self._map, dtype=np.uint8, count=info.nbytes, offset=start)

    def get(self, key: str, kind: type):
        if key not in self.kv or not isinstance(self.kv[key], kind):
            raise RuntimeError(f"GgufFile: {kind.__name__} KV not found '{key}'")
        return self.kv[key]

    def close(self) -> None:
        self._map.close()
        self._fh.close()


def _row_bytes(dtype: int, cols: int) -> int:
    blk, bsz = TYPE_INFO[dtype]
    return cols // blk * bsz


def _weights_ready(t):
    """Packed weights must be complete before the kernel that precedes their first use starts (the library's
    kernels request weight bytes ahead of their stream dependency): finish the upload / repack here."""
    import torch
    if t.is_cuda:
        torch.cuda.current_stream(t.device).synchronize()
    return t


def load_quant_weight(kd, file: GgufFile, info: GgufTensorInfo, device="cuda"):
    """One 1-D / 2-D tensor's packed payload on the device as a QuantWeight
    (load_quant_weight, src/KokkosDNN_GGUF.hpp:864-885): dims {cols, rows} -> [rows, cols]."""
    import torch
    if info.n_dims not in (1, 2):
        raise RuntimeError("load_quant_weight: only 1-D/2-D supported")
    if info.dtype not in COMPUTE_TYPES:
        raise RuntimeError(f"load_quant_weight: unsupported dtype {info.dtype}")
    rows, cols = info.rows(), info.cols()
    if rows * _row_bytes(info.dtype, cols) != info.nbytes:
        raise RuntimeError(f"load_quant_weight: size mismatch for '{info.name}'")
    data = _weights_ready(torch.from_numpy(np.array(file.payload(info))).to(device))
    return kd.QuantWeight(data, info.dtype, rows, cols)


def load_expert_weights(kd, file: GgufFile, info: GgufTensorInfo, device="cuda") -> list:
    """A stacked expert tensor, dims {cols, rows, experts} in ggml order (expert is the slowest extent,
    models/lfm2_5/KokkosDNN_LFM25Weights.cpp:135-172): one device allocation, one QuantWeight view per
    expert, ready for make_quant_weight_table."""
    import torch
    if info.n_dims != 3:
        raise RuntimeError("load_expert_weights: expected a 3-D {cols, rows, experts} tensor")
    if info.dtype not in COMPUTE_TYPES:
        raise RuntimeError(f"load_expert_weights: unsupported dtype {info.dtype}")
    cols, rows, experts = info.dims
    per = rows * _row_bytes(info.dtype, cols)
    if per * experts != info.nbytes:
        raise RuntimeError(f"load_expert_weights: size mismatch for '{info.name}'")
    stride = (per + 255) & ~255       # every expert starts on a 256-byte boundary, whatever the block size
    host = torch.from_numpy(np.array(file.payload(info))).view(experts, per)
    data = torch.zeros(experts * stride, dtype=torch.uint8, device=device)
    data.view(experts, stride)[:, :per].copy_(host)
    _weights_ready(data)
    return [kd.QuantWeight(data[e * stride:e * stride + per], info.dtype, rows, cols) for e in range(experts)]


def tensor_to_float(kd, file: GgufFile, info: GgufTensorInfo, device="cuda"):
    """A whole tensor as fp32 on `device`, shaped [numel / cols, cols] (dequant_tensor_to_float,
    src/KokkosDNN_GGUF.hpp:778-846). F32 / F16 / BF16 widen exactly on any device; the packed types go to the
    GPU packed and are expanded there by dequant_to_dense, whose fp32 output equals the reference's block
    formulas bit for bit -- they need a CUDA device."""
    import torch
    cols = info.cols()
    rows = info.numel // cols if cols else 0
    raw = file.payload(info)
    if info.dtype == 0:
        return torch.from_numpy(np.array(raw).view(np.float32)).view(rows, cols).to(device)
    if info.dtype == 1:
        return torch.from_numpy(np.array(raw).view(np.float16)).view(rows, cols).to(device).float()
    if info.dtype == 30:
        return torch.from_numpy(np.array(raw).view(np.int16)).view(torch.bfloat16).view(rows, cols).to(device).float()
    if info.dtype not in COMPUTE_TYPES:
        raise RuntimeError(f"tensor_to_float: unsupported dtype {info.dtype}")
    if torch.device(device).type != "cuda":
        raise RuntimeError("tensor_to_float: packed types are expanded on the GPU; pass a CUDA device")
    w = kd.QuantWeight(torch.from_numpy(np.array(raw)).to(device), info.dtype, rows, cols)
    out = torch.empty(rows, cols, dtype=torch.float32, device=device)
    _weights_ready(w.data)
    kd.dequant_to_dense(w, out)
    return _weights_ready(out)


# ---- writer (tests, synthetic checkpoints) ----------------------------------------------
def _pack_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _pack_value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I", 7) + struct.pack("<?", v)
    if isinstance(v, int):
        return struct.pack("<I", 4) + struct.pack("<I", v) if 0 <= v < 2 ** 32 else struct.pack("<I", 11) + struct.pack("<q", v)
    if isinstance(v, float):
        return struct.pack("<I", 6) + struct.pack("<f", v)
    if isinstance(v, str):
        return struct.pack("<I", T_STRING) + _pack_string(v)
    if isinstance(v, (list, tuple)) and v and all(isinstance(e, str) for e in v):
        return struct.pack("<IIQ", T_ARRAY, T_STRING, len(v)) + b"".join(_pack_string(e) for e in v)
    if isinstance(v, (list, tuple, np.ndarray)):
        a = np.asarray(v)
        code = {np.dtype("float32"): 6, np.dtype("int32"): 5, np.dtype("uint32"): 4, np.dtype("int64"): 11,
                np.dtype("uint8"): 0, np.dtype("bool"): 7}.get(a.dtype)
        if code is None:
            a, code = a.astype(np.int32), 5
        return struct.pack("<IIQ", T_ARRAY, code, a.size) + a.tobytes()
    raise TypeError(f"write_gguf: cannot encode {type(v).__name__}")


def write_gguf(path: str, kv: Dict[str, Any], tensors: Sequence[Tuple[str, Sequence[int], int, np.ndarray]]) -> None:
    """Writes a GGUF v3 file. `tensors`: (name, dims in ggml order, ggml type id, packed payload bytes)."""
    head = b"GGUF" + struct.pack("<IQQ", VERSION, len(tensors), len(kv))
    for key, v in kv.items():
        head += _pack_string(key) + _pack_value(v)
    offsets, off = [], 0
    for _, _, _, payload in tensors:
        offsets.append(off)
        off = (off + int(np.asarray(payload).nbytes) + ALIGN - 1) & ~(ALIGN - 1)
    for (name, dims, dtype, _), o in zip(tensors, offsets):
        head += _pack_string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", dtype, o)
    with open(path, "wb") as fh:
        fh.write(head)
        fh.write(b"\0" * (-len(head) % ALIGN))
        for (_, _, _, payload), o in zip(tensors, offsets):
            raw = np.ascontiguousarray(payload).view(np.uint8).reshape(-1).tobytes()
            fh.write(raw)
            fh.write(b"\0" * (-len(raw) % ALIGN))
