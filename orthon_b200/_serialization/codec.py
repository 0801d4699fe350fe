"""Closed, tagged value vocabulary: null / bool / int / float (non-finite as strings) / str /
list / tuple / dict (item list, string keys) / tensor.  Tensors are raw little-endian logical
row-major bytes with shape, dtype, byte count and SHA-256.
(reference project: python/orthon/_serialization/codec.py:13-155, tensor.py:8-68)"""
import hashlib
import math

from .. import _C
from .format import fail

_DTYPE_SIZES = {"float32": 4, "float64": 8, "float16": 2, "bfloat16": 2, "int32": 4, "int64": 8,
                "uint8": 1, "int8": 1, "bool": 1}


def _no_grad():
    import orthon_b200 as ob
    return ob.no_grad()


class Encoder:
    def __init__(self):
        self.payloads = []  # ordered (member name, bytes)

    def _tensor(self, t):
        with _no_grad():
            data = _C._tensor_to_bytes(t)  # host snapshot in logical order
        name = "tensors/%06d.bin" % len(self.payloads)
        self.payloads.append((name, data))
        return {"k": "tensor", "shape": [int(d) for d in t.shape], "dtype": t.dtype, "nbytes": len(data),
                "sha256": hashlib.sha256(data).hexdigest(), "payload": name}

    def encode(self, value, where):
        if value is None:
            return {"k": "null"}
        if isinstance(value, bool):
            return {"k": "bool", "v": value}
        if isinstance(value, int):
            return {"k": "int", "v": value}
        if isinstance(value, float):
            if math.isnan(value):
                return {"k": "float", "v": "nan"}
            if math.isinf(value):
                return {"k": "float", "v": "inf" if value > 0 else "-inf"}
            return {"k": "float", "v": value}
        if isinstance(value, str):
            return {"k": "str", "v": value}
        if isinstance(value, _C.Tensor):
            return self._tensor(value)
        if isinstance(value, (list, tuple)):
            kind = "list" if isinstance(value, list) else "tuple"
            return {"k": kind, "v": [self.encode(v, f"{where}[{i}]") for i, v in enumerate(value)]}
        if isinstance(value, dict):
            items = []
            for key, v in value.items():
                if not isinstance(key, str):
                    raise TypeError(f"checkpoint: {where}: dictionary keys must be str, got {type(key)!r}")
                items.append([key, self.encode(v, f"{where}.{key}")])
            return {"k": "dict", "v": items}
        raise TypeError(f"checkpoint: {where}: unsupported value type {type(value)!r}")


class Decoder:
    def __init__(self, read_payload):
        self._read = read_payload
        self._seen = set()

    def _tensor(self, node, where):
        shape, dtype, nbytes = node.get("shape"), node.get("dtype"), node.get("nbytes")
        digest, payload = node.get("sha256"), node.get("payload")
        if (not isinstance(shape, list) or not all(type(d) is int and d >= 0 for d in shape)
                or dtype not in _DTYPE_SIZES or type(nbytes) is not int or nbytes < 0 or not isinstance(digest, str)
                or len(digest) != 64):
            fail(f"{where}: malformed tensor record")
        count = 1
        for d in shape:
            count *= d
        if count * _DTYPE_SIZES[dtype] != nbytes:
            fail(f"{where}: tensor byte count does not match shape and dtype")
        if payload in self._seen:
            fail(f"{where}: payload {payload} is referenced more than once")
        self._seen.add(payload)
        data = self._read(payload, nbytes, where)
        if hashlib.sha256(data).hexdigest() != digest:
            fail(f"{where}: payload checksum mismatch")
        return _C._tensor_from_bytes(data, shape, dtype)

    def decode(self, node, where):
        if not isinstance(node, dict) or "k" not in node:
            fail(f"{where}: malformed value record")
        kind = node["k"]
        if kind == "null":
            return None
        if kind == "bool":
            if type(node.get("v")) is not bool:
                fail(f"{where}: malformed bool")
            return node["v"]
        if kind == "int":
            if type(node.get("v")) is not int:
                fail(f"{where}: malformed int")
            return node["v"]
        if kind == "float":
            v = node.get("v")
            if isinstance(v, str):
                if v not in ("inf", "-inf", "nan"):
                    fail(f"{where}: malformed float tag")
                return float(v)
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                fail(f"{where}: malformed float")
            return float(v)
        if kind == "str":
            if not isinstance(node.get("v"), str):
                fail(f"{where}: malformed str")
            return node["v"]
        if kind in ("list", "tuple"):
            if not isinstance(node.get("v"), list):
                fail(f"{where}: malformed {kind}")
            out = [self.decode(v, f"{where}[{i}]") for i, v in enumerate(node["v"])]
            return out if kind == "list" else tuple(out)
        if kind == "dict":
            if not isinstance(node.get("v"), list):
                fail(f"{where}: malformed dict")
            out = {}
            for item in node["v"]:
                if not isinstance(item, list) or len(item) != 2 or not isinstance(item[0], str):
                    fail(f"{where}: malformed dict item")
                if item[0] in out:
                    fail(f"{where}: duplicate dictionary key {item[0]!r}")
                out[item[0]] = self.decode(item[1], f"{where}.{item[0]}")
            return out
        if kind == "tensor":
            return self._tensor(node, where)
        fail(f"{where}: unknown value tag {kind!r}")
