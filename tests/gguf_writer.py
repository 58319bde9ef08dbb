"""A small GGUF writer for the tests (test-side only): header, metadata and tensor infos laid
out as the reference's parser reads them (crates/oxillama-gguf/src/parser.rs:34-212,
header.rs:22-95), dimensions in the order its fixtures use (dims[0] = out_features,
crates/oxillama-gguf/src/test_utils.rs:183-199)."""
import struct

import numpy as np

VT = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10,
      "i64": 11, "f64": 12}
FMT = {"u8": "<B", "i8": "<b", "u16": "<H", "i16": "<h", "u32": "<I", "i32": "<i", "f32": "<f", "bool": "<B",
       "u64": "<Q", "i64": "<q", "f64": "<d"}


def _s(text, version):
    b = text.encode()
    return struct.pack("<Q" if version >= 3 else "<I", len(b)) + b


def _value(kind, v, version):
    if kind == "str":
        return _s(v, version)
    if kind == "arr":
        ek, items = v
        out = struct.pack("<I", VT[ek]) + struct.pack("<Q" if version >= 3 else "<I", len(items))
        return out + b"".join(_value(ek, it, version) for it in items)
    return struct.pack(FMT[kind], v)


def write_gguf(path, tensors, metadata=(), version=3, alignment=None):
    """tensors: [(name, dims, type_id, bytes)]; metadata: [(key, kind, value)].  Returns
    {name: absolute offset of the tensor's data}."""
    metadata = list(metadata)
    if alignment is not None:
        metadata.append(("general.alignment", "u32", alignment))
    align = alignment or 32
    cnt = "<Q" if version >= 3 else "<I"
    head = struct.pack("<I", 0x46554747) + struct.pack("<I", version) + struct.pack(cnt, len(tensors)) + \
        struct.pack(cnt, len(metadata))
    for key, kind, v in metadata:
        head += _s(key, version) + struct.pack("<I", VT[kind]) + _value(kind, v, version)
    offs, rel = [], 0
    for name, dims, type_id, data in tensors:
        offs.append(rel)
        rel += -(-len(data) // align) * align
    for (name, dims, type_id, data), off in zip(tensors, offs):
        head += _s(name, version) + struct.pack("<I", len(dims))
        for d in dims:
            head += struct.pack("<Q" if version >= 3 else "<I", d)
        head += struct.pack("<I", type_id) + (struct.pack("<Q", off) if version >= 2 else struct.pack("<I", off))
    data_off = -(-len(head) // align) * align
    out = {}
    with open(path, "wb") as f:
        f.write(head + b"\0" * (data_off - len(head)))
        for (name, dims, type_id, data), off in zip(tensors, offs):
            out[name] = data_off + off
            blob = np.ascontiguousarray(data, dtype=np.uint8).tobytes()
            f.write(blob + b"\0" * (-len(blob) % align))
    return out
