"""CPU restatement of what the reference's weight loader makes of a safetensors file
(Infer-engine/src/safetensors.c:57-181).  TEST INFRASTRUCTURE ONLY.

File format: 8-byte little-endian header length, a JSON object, then the tensor bytes; a tensor's
``data_offsets`` are relative to the first byte after the header.  The reference walks the header in textual
order and, per entry:
  * ``__metadata__`` and values that are not objects are skipped (:88-95);
  * dtype names map to tags BF16 -> 1, F32 -> 0, F16 -> 2, U8 -> 3, F8_E4M3 -> 4 (:48-55, types.h:8-12); an entry
    with any other dtype creates no tensor (:141);
  * at most 4 dims of the shape are kept, as C ints (:116-126);
  * nbytes = data_offsets[1] - data_offsets[0]; an entry with no bytes AND no dims counts the dtype's size
    instead (:143-146); the bytes read are nbytes, or 4 when that is 0 (:148-158);
  * at most 2048 entries (:76).
"""
from __future__ import annotations

import json
import struct

DTYPE_TAGS = {"F32": 0, "BF16": 1, "F16": 2, "U8": 3, "F8_E4M3": 4}
DTYPE_SIZE = {0: 4, 1: 2, 2: 2, 3: 1, 4: 1}
MAX_DIMS, MAX_WEIGHTS = 4, 2048


def load_index(path: str):
    """Entries the reference would create, in order: dicts with name, dtype (tag), shape, nbytes, file_offset."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = f.read(hlen).decode("utf-8")
    pairs = json.loads(header, object_pairs_hook=list)         # keep textual order (and duplicates)
    out = []
    for name, val in pairs:
        if len(out) >= MAX_WEIGHTS:
            break
        if name == "__metadata__" or not isinstance(val, list):
            continue
        fields = dict(val)
        tag = DTYPE_TAGS.get(fields.get("dtype"), -1)
        if tag < 0:
            continue
        shape = [int(d) for d in fields.get("shape", [])][:MAX_DIMS]
        off0, off1 = fields.get("data_offsets", [0, 0])
        nbytes = off1 - off0
        if nbytes == 0 and len(shape) == 0:
            nbytes = DTYPE_SIZE[tag]
        out.append({"name": name, "dtype": tag, "shape": shape, "nbytes": nbytes, "file_offset": 8 + hlen + off0})
    return out


def tensor_bytes(path: str, entry) -> bytes:
    with open(path, "rb") as f:
        f.seek(entry["file_offset"])
        return f.read(entry["nbytes"])


def write_file(path: str, tensors, metadata=None):
    """Write a safetensors file from (name, dtype string, shape, raw bytes) tuples, in the given order, the data
    region packed without padding (as the format's writers do)."""
    header = {}
    if metadata is not None:
        header["__metadata__"] = metadata
    blob = bytearray()
    for name, dtype, shape, raw in tensors:
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    js = json.dumps(header, separators=(",", ":")).encode("utf-8")
    js += b" " * ((8 - len(js) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        f.write(bytes(blob))
