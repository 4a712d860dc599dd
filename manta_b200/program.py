"""ctypes front end of the host executor (``include/manta_b200_host.h``): the Python twin of what a Go caller gets
from ``Runtime.Load`` / ``Program.Run`` (runtime/runtime.go:43-119 of the reference).

Tensors follow the reference's convention (runtime/backend/tensor.go:11-19): a dtype label plus float32 data for
f16 / f32 / q4 / q8, int32 for i32, int64 for i64.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import POINTER, byref, c_char_p, c_int, c_int64, c_void_p

import numpy as np

from . import native
from .native import MantaError


class TensorArg(ctypes.Structure):
    _fields_ = [("name", c_char_p), ("dtype", c_char_p), ("rank", c_int), ("shape", POINTER(c_int64)), ("data", c_void_p)]


def _np_dtype(label: str):
    return {"i32": np.int32, "i64": np.int64}.get(label, np.float32)


class Tensor:
    """backend.Tensor: NewTensorF16 / NewTensorQ4 / NewTensorI64 ... are ``Tensor(label, shape, values)``."""

    def __init__(self, dtype: str, shape, values):
        self.dtype = dtype
        self.array = np.ascontiguousarray(np.asarray(values, dtype=_np_dtype(dtype)).reshape(shape))

    @property
    def shape(self):
        return list(self.array.shape)


_configured = False


def _lib():
    global _configured
    lib = native.load()
    if not _configured:
        E = POINTER(c_char_p)
        lib.manta_b200_program_load.argtypes = [c_void_p, c_char_p, POINTER(c_void_p), E]
        lib.manta_b200_program_bind_weight.argtypes = [c_void_p, POINTER(TensorArg), E]
        lib.manta_b200_program_plan.argtypes = [c_void_p, c_char_p, POINTER(c_void_p), E]
        lib.manta_b200_program_run.argtypes = [c_void_p, c_char_p, POINTER(TensorArg), c_int, POINTER(c_void_p), E]
        lib.manta_b200_program_destroy.argtypes = [c_void_p, E]
        lib.manta_b200_program_memory_plan.argtypes = [c_void_p, c_int64, c_int, c_int, c_int, POINTER(c_void_p), E]
        lib.manta_b200_program_apply_memory_plan.argtypes = [c_void_p, c_char_p, E]
        lib.manta_b200_program_memory_plan.restype = c_int
        lib.manta_b200_program_apply_memory_plan.restype = c_int
        lib.manta_b200_result_json.argtypes = [c_void_p]
        lib.manta_b200_result_json.restype = c_char_p
        lib.manta_b200_result_tensor.argtypes = [c_void_p, c_char_p, c_char_p, POINTER(TensorArg), E]
        lib.manta_b200_result_free.argtypes = [c_void_p]
        lib.manta_b200_result_free.restype = None
        for n in ("manta_b200_program_load", "manta_b200_program_bind_weight", "manta_b200_program_plan",
                  "manta_b200_program_run", "manta_b200_program_destroy", "manta_b200_result_tensor"):
            getattr(lib, n).restype = c_int
        _configured = True
    return lib


def _arg(name: str, t: Tensor, keep: list) -> TensorArg:
    shape = (c_int64 * max(len(t.shape), 1))(*t.shape)
    nb, db = name.encode(), t.dtype.encode()
    keep.extend([shape, nb, db, t.array])
    return TensorArg(nb, db, len(t.shape), shape, t.array.ctypes.data_as(c_void_p))


class Output:
    """backend.Value of a result: data (numpy array or a dict for a candidate_pack) plus producer and metadata."""

    def __init__(self, kind, data, producer, inputs, metadata, dtype=None):
        self.kind, self.data, self.producer, self.inputs, self.metadata, self.dtype = kind, data, producer, inputs, metadata, dtype


class Result:
    def __init__(self, outputs, trace, metadata):
        self.outputs, self.trace, self.metadata = outputs, trace, metadata


class Program:
    """A loaded plan on one device runtime (``rt`` may be None for plan inspection without a GPU)."""

    def __init__(self, rt, module_json):
        lib = _lib()
        text = module_json if isinstance(module_json, str) else json.dumps(module_json)
        self.handle = None
        h = c_void_p()
        native.call("manta_b200_program_load", rt.handle if rt is not None else None, text.encode(), byref(h))
        self.handle, self.rt, self._lib = h, rt, lib

    def bind_weight(self, name: str, tensor: Tensor):
        keep = []
        a = _arg(name, tensor, keep)
        native.call("manta_b200_program_bind_weight", self.handle, byref(a))

    def plan(self, entry: str):
        out = c_void_p()
        native.call("manta_b200_program_plan", self.handle, entry.encode(), byref(out))
        text = ctypes.cast(out, c_char_p).value.decode()
        self._lib.manta_b200_free_cstring(out)
        return json.loads(text)

    def memory_plan(self, device_budget_bytes: int = 0, shared_host_weights: bool = False, shards: int = 1,
                    accounting: str = "device") -> dict:
        """NewMemoryPlan over the bound weights; accounting "logical" reproduces the reference's byte counts."""
        out = c_void_p()
        native.call("manta_b200_program_memory_plan", self.handle, c_int64(device_budget_bytes), c_int(1 if shared_host_weights else 0),
                    c_int(shards), c_int(0 if accounting == "logical" else 1), byref(out))
        text = ctypes.cast(out, c_char_p).value.decode()
        self._lib.manta_b200_free_cstring(out)
        return json.loads(text)

    def apply_memory_plan(self, plan: dict):
        native.call("manta_b200_program_apply_memory_plan", self.handle, json.dumps(plan).encode())

    def run(self, entry: str, inputs: dict) -> Result:
        keep = []
        arr = (TensorArg * max(len(inputs), 1))()
        for i, (name, t) in enumerate(inputs.items()):
            arr[i] = _arg(name, t, keep)
        res = c_void_p()
        native.call("manta_b200_program_run", self.handle, entry.encode(), arr, c_int(len(inputs)), byref(res))
        try:
            desc = json.loads(self._lib.manta_b200_result_json(res).decode())
            outputs = {}
            for name, o in desc["outputs"].items():
                if o["kind"] == "candidate_pack":
                    data = {f: self._tensor(res, name, f) for f in ("ids", "scores", "docs")}
                    data["docs_dtype"] = self._dtype(res, name, "docs")
                    outputs[name] = Output(o["kind"], data, o["producer"], o["inputs"], o["metadata"])
                else:
                    outputs[name] = Output(o["kind"], self._tensor(res, name, ""), o["producer"], o["inputs"], o["metadata"], o.get("dtype"))
            return Result(outputs, desc["trace"], desc["metadata"])
        finally:
            self._lib.manta_b200_result_free(res)

    def _view(self, res, name, field):
        v = TensorArg()
        native.call("manta_b200_result_tensor", res, name.encode(), field.encode(), byref(v))
        return v

    def _dtype(self, res, name, field):
        return self._view(res, name, field).dtype.decode()

    def _tensor(self, res, name, field):
        v = self._view(res, name, field)
        shape = [v.shape[i] for i in range(v.rank)]
        dt = _np_dtype(v.dtype.decode())
        n = int(np.prod(shape)) if shape else 1
        if n == 0:
            return np.zeros(shape, dt)
        buf = (ctypes.c_char * (n * np.dtype(dt).itemsize)).from_address(v.data)
        return np.frombuffer(buf, dtype=dt).reshape(shape).copy()

    def close(self):
        if self.handle is not None:
            # a program whose runtime is already closed cannot release its resident sets through it: the handle is
            # dropped (the runtime's destruction has freed the device)
            if self.rt is None or getattr(self.rt, "handle", None) is not None:
                native.call("manta_b200_program_destroy", self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


__all__ = ["Program", "Tensor", "Result", "Output", "MantaError"]
