"""Minimal safetensors reader, the host-side mirror of src/weights/safetensors.ts.

Layout of a file: 8-byte little-endian header length, a JSON header, the raw tensor bytes. Same functions,
same validation rules and the same error texts as the reference (``parseSafetensorsHeader`` :39-82,
``parseSafetensors`` :84-110, ``tensorCount`` :113, ``requireTensor`` :119, ``expectTensor`` :127-142,
``f16BitsToF32`` :144-153, ``readTensorBytes`` :155-162, ``readTensorF32`` :164-198, ``dtypeByteSize``
:200-222). Tensors are returned as numpy views of the file buffer wherever the reference copies; a
``bytes``, ``bytearray``, ``memoryview`` or ``numpy.memmap`` all work as the buffer.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass

import numpy as np

ENTRY_KEY_SKIP = "__metadata__"

_DTYPE_BYTES = {"F64": 8, "I64": 8, "F32": 4, "I32": 4, "F16": 2, "BF16": 2, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1}


class SafetensorsError(ValueError):
    """What the reference signals with ``throw new Error('safetensors: …')``."""


@dataclass
class SafetensorEntry:
    dtype: str
    shape: list
    data_offsets: tuple


@dataclass
class SafetensorFile:
    buffer: np.ndarray  # uint8 view of the whole file
    data_start: int
    header: dict


def dtype_byte_size(dtype: str) -> int:
    try:
        return _DTYPE_BYTES[dtype]
    except KeyError:
        raise SafetensorsError(f"safetensors: 未知 dtype {dtype}") from None


def _number(v) -> float:
    """JavaScript's ``Number(v)`` for the values a JSON header can hold."""
    if isinstance(v, bool):
        return float(v)
    if isinstance(v, (int, float)):
        return float(v)
    if v is None:
        return 0.0
    if isinstance(v, str):
        try:
            return float(v) if v.strip() else 0.0
        except ValueError:
            return math.nan
    return math.nan


def parse_safetensors_header(header_bytes) -> dict:
    """Parses the JSON header; checks only that every entry is self-consistent (not that it fits a file), so a
    header fetched alone can be inspected (src/weights/safetensors.ts:39-82)."""
    try:
        parsed = json.loads(bytes(header_bytes).decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as err:
        raise SafetensorsError(f"safetensors: header JSON 解析失败：{err}") from None
    if not isinstance(parsed, dict):
        raise SafetensorsError("safetensors: header 不是 JSON object")
    header = {}
    for name, item in parsed.items():
        if name == ENTRY_KEY_SKIP:
            continue
        if not isinstance(item, dict):
            raise SafetensorsError(f"safetensors: {name} 条目非法")
        if not isinstance(item.get("dtype"), str):
            raise SafetensorsError(f"safetensors: {name} 缺少 dtype")
        if not isinstance(item.get("shape"), list):
            raise SafetensorsError(f"safetensors: {name} 缺少 shape")
        offs = item.get("data_offsets")
        if not isinstance(offs, list) or len(offs) != 2:
            raise SafetensorsError(f"safetensors: {name} data_offsets 非法")
        start, end = (_number(v) for v in offs)
        if not math.isfinite(start) or not math.isfinite(end) or start < 0 or end < start:
            raise SafetensorsError(f"safetensors: {name} data_offsets 数值非法")
        header[name] = SafetensorEntry(item["dtype"], [int(_number(v)) for v in item["shape"]], (int(start), int(end)))
    return header


def parse_safetensors(buffer) -> SafetensorFile:
    """Parses a whole file image and checks the header length and every tensor's end against its size
    (src/weights/safetensors.ts:84-110)."""
    buf = np.frombuffer(buffer, dtype=np.uint8) if not isinstance(buffer, np.ndarray) else buffer.view(np.uint8).reshape(-1)
    if buf.size < 8:
        raise SafetensorsError("safetensors: buffer 过短")
    header_len = int(buf[0:4].view("<u4")[0])
    if int(buf[4:8].view("<u4")[0]) != 0:
        raise SafetensorsError("safetensors: header 长度超过 4GiB，当前不支持")
    data_start = 8 + header_len
    if header_len <= 0 or data_start > buf.size:
        raise SafetensorsError(f"safetensors: header 长度非法 headerLen={header_len} bufferSize={buf.size}")
    header = parse_safetensors_header(buf[8:data_start])
    for name, entry in header.items():
        if data_start + entry.data_offsets[1] > buf.size:
            raise SafetensorsError(f"safetensors: {name} 数据越界 end={entry.data_offsets[1]}")
    return SafetensorFile(buf, data_start, header)


def tensor_count(entry: SafetensorEntry) -> int:
    """Number of elements; an empty shape is a scalar."""
    n = 1
    for d in entry.shape:
        n *= d
    return n


def require_tensor(file: SafetensorFile, name: str) -> SafetensorEntry:
    entry = file.header.get(name)
    if entry is None:
        raise SafetensorsError(f"safetensors: 缺少 tensor {name}")
    return entry


def expect_tensor(file: SafetensorFile, name: str, dtype: str, shape) -> SafetensorEntry:
    """Checks dtype and shape up front so that a file of another model fails early."""
    entry = require_tensor(file, name)
    if entry.dtype != dtype:
        raise SafetensorsError(f"safetensors: {name} dtype={entry.dtype}，期望 {dtype}")
    if list(entry.shape) != list(shape):
        raise SafetensorsError(f"safetensors: {name} shape=[{','.join(map(str, entry.shape))}]，"
                               f"期望 [{','.join(map(str, shape))}]")
    return entry


def f16_bits_to_f32(bits) -> np.ndarray:
    """IEEE binary16 bit patterns to f32 values, exactly (subnormals, infinities and NaN included)."""
    return np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)


def read_tensor_bytes(file: SafetensorFile, name: str) -> np.ndarray:
    """The tensor's raw bytes (a view: the reference makes a shallow copy only to dodge alignment)."""
    entry = require_tensor(file, name)
    start = file.data_start + entry.data_offsets[0]
    return file.buffer[start:start + tensor_count(entry) * dtype_byte_size(entry.dtype)]


def read_tensor_f32(file: SafetensorFile, name: str) -> np.ndarray:
    """Reads a tensor back as f32. F32 / F16 / BF16 / U8 / I8, like the reference."""
    entry = require_tensor(file, name)
    raw = read_tensor_bytes(file, name)
    if entry.dtype == "F32":
        return raw.view("<f4").astype(np.float32)
    if entry.dtype == "F16":
        return f16_bits_to_f32(raw.view("<u2"))
    if entry.dtype == "BF16":
        return (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)
    if entry.dtype == "U8":
        return raw.astype(np.float32)
    if entry.dtype == "I8":
        return raw.view(np.int8).astype(np.float32)
    raise SafetensorsError(f"readTensorF32: 不支持的 dtype {entry.dtype}（{name}）")


def build_safetensors(tensors: dict, metadata: dict | None = None) -> bytes:
    """Serialises ``{name: (dtype, shape, array-or-bytes)}`` into a safetensors image (what the reference's tests
    do by hand, src/tests/qwen/weights.ts:7-41); used to write synthetic checkpoints."""
    header = {} if metadata is None else {ENTRY_KEY_SKIP: metadata}
    blobs, offset = [], 0
    for name, (dtype, shape, data) in tensors.items():
        raw = data if isinstance(data, (bytes, bytearray)) else np.ascontiguousarray(data).tobytes()
        expect = dtype_byte_size(dtype)
        for d in shape:
            expect *= d
        if len(raw) != expect:
            raise SafetensorsError(f"safetensors: {name} 有 {len(raw)} 字节，shape/dtype 需要 {expect}")
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * (-len(hb) % 8)  # writers pad the header so that the data start is 8-byte aligned
    return len(hb).to_bytes(8, "little") + hb + b"".join(blobs)
