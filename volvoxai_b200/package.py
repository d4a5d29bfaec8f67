"""Host-side mirror of the package loader (include/vxb200_package.h): open a model package
(graph.json + SafeTensors files), compile it onto a device context, run forward passes with NumPy
arrays in and out.  Counterpart of loading a model and compiling it for a backend in the reference
(VxModelSource -> compile -> context_execute, native/include/volvoxai_backend.h:168-259)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

_NP = {_lib.DT_F32: np.float32, _lib.DT_I8: np.int8, _lib.DT_U8: np.uint8, _lib.DT_I32: np.int32}


class PackageError(RuntimeError):
    def __init__(self, code: int):
        self.code = code
        super().__init__(f"libvxb200 returned {code}: {_lib.last_error()}")


class Package:
    """A validated package on the host.  Raises PackageError(0) when the package holds an operator,
    a dtype or metadata this route does not serve (the host then keeps it on its own routes)."""

    def __init__(self, graph_path: str, weight_paths: list[str]):
        self._L = _lib.load()
        paths = (C.c_char_p * max(1, len(weight_paths)))(*[p.encode() for p in weight_paths])
        h = C.c_void_p(0)
        rc = self._L.vxb_package_open(graph_path.encode(), paths, len(weight_paths), C.byref(h))
        if rc != 1:
            raise PackageError(rc)
        self.handle = h

    def _io(self, is_output: int):
        out = []
        for i in range(self._L.vxb_package_io_count(self.handle, is_output)):
            rank = self._L.vxb_package_io_rank(self.handle, is_output, i)
            out.append({"name": self._L.vxb_package_io_name(self.handle, is_output, i).decode(),
                        "dtype": _NP[self._L.vxb_package_io_dtype(self.handle, is_output, i)],
                        "shape": tuple(int(self._L.vxb_package_io_dim(self.handle, is_output, i, a)) for a in range(rank)),
                        "bytes": int(self._L.vxb_package_io_bytes(self.handle, is_output, i))})
        return out

    @property
    def inputs(self):
        return self._io(0)

    @property
    def outputs(self):
        return self._io(1)

    @property
    def node_ops(self) -> list[str]:
        return [self._L.vxb_package_node_op(self.handle, i).decode() for i in range(self._L.vxb_package_node_count(self.handle))]

    def close(self) -> None:
        if getattr(self, "handle", None):
            self._L.vxb_package_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Program:
    """A package compiled onto a context: weights repacked once, intermediate tensors on the device."""

    def __init__(self, ctx, package: Package):
        self._L = package._L
        self.ctx = ctx
        self._inputs, self._outputs = package.inputs, package.outputs
        h = C.c_void_p(0)
        rc = self._L.vxb_program_compile(ctx.handle, package.handle, C.byref(h))
        if rc != 1:
            raise PackageError(rc)
        self.handle = h

    @property
    def device_bytes(self) -> int:
        return int(self._L.vxb_program_device_bytes(self.handle))

    @property
    def route_evidence(self) -> str:
        return self._L.vxb_program_route_evidence(self.handle).decode()

    def execute_raw(self, inputs: list[np.ndarray], outputs: list[np.ndarray]) -> int:
        """The C entry as it is: 1 / 0 / -1, outputs written in place."""
        ip = (C.c_void_p * len(inputs))(*[a.ctypes.data for a in inputs])
        ib = (C.c_size_t * len(inputs))(*[a.nbytes for a in inputs])
        op = (C.c_void_p * len(outputs))(*[a.ctypes.data for a in outputs])
        ob = (C.c_size_t * len(outputs))(*[a.nbytes for a in outputs])
        return int(self._L.vxb_program_execute(self.handle, ip, ib, len(inputs), op, ob, len(outputs)))

    def __call__(self, *inputs: np.ndarray) -> list[np.ndarray]:
        ins = [np.ascontiguousarray(a, spec["dtype"]) for a, spec in zip(inputs, self._inputs)]
        outs = [np.empty(spec["shape"], spec["dtype"]) for spec in self._outputs]
        rc = self.execute_raw(ins, outs)
        if rc != 1:
            raise PackageError(rc)
        return outs

    def close(self) -> None:
        if getattr(self, "handle", None):
            self._L.vxb_program_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
