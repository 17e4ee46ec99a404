"""Reads the committed golden fixtures (safetensors layout: u64 header length, JSON header, raw bytes)."""
import json
import struct
from pathlib import Path

import numpy as np

from homura_b200.host import BF16, BOOL, F16, F32, F64, I8, I16, I32, I64, STORAGE, U8

GOLDEN = Path(__file__).resolve().parent / "golden"
CODES = {"BOOL": BOOL, "U8": U8, "I8": I8, "I16": I16, "I32": I32, "I64": I64, "F16": F16, "BF16": BF16, "F32": F32,
         "F64": F64}


class Golden:
    def __init__(self, name: str):
        data = (GOLDEN / name).read_bytes()
        n = struct.unpack("<Q", data[:8])[0]
        self.header = json.loads(data[8:8 + n])
        self.body = data[8 + n:]
        self.metadata = self.header.pop("__metadata__", {})

    def cases(self):
        return sorted({k.split("/")[0] for k in self.header})

    def names(self, case: str):
        return sorted(k.split("/", 1)[1] for k in self.header if k.split("/")[0] == case)

    def get(self, key: str):
        """(dtype code, shape, raw elements as a numpy array of the storage dtype)."""
        info = self.header[key]
        dt = CODES[info["dtype"]]
        a, b = info["data_offsets"]
        raw = np.frombuffer(self.body[a:b], dtype=STORAGE[dt]).reshape(info["shape"]).copy()
        return dt, tuple(info["shape"]), raw
