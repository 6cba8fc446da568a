"""A stand-in for the Fortran / C host program: holds column-major arrays and calls the library's C ABI the way a
fortisc-rewritten host does (mom6_zb/host_fissioned.fir:732-740):

    call fortis_gather(arrays...) ; call mlp_forward_batched() ; do k: call fortis_scatter(k, arrays...)

Arrays may be numpy arrays (host memory, Fortran order) or torch CUDA tensors (device-resident, used in place).
"""
import ctypes
import json

import numpy as np

from . import lib as _lib


def _ptr(a):
    if isinstance(a, np.ndarray):
        if not (a.flags.f_contiguous or a.flags.c_contiguous):
            raise ValueError("host arrays must be contiguous")
        return a.ctypes.data
    if hasattr(a, "data_ptr"):        # torch tensor (device or host)
        return a.data_ptr()
    if isinstance(a, int):
        return a
    raise TypeError("unsupported array type %r" % type(a))


class Host:
    def __init__(self):
        self.L = _lib.load()
        self._keep = []          # host arrays handed to the library stay alive until reset(): it pins them by address

    # ---- configuration -----------------------------------------------------------------------------------------
    def reset(self):
        self.L.fortis_reset()
        self._keep = []

    def configure(self, gather=None, scatter=None, loop=None, kdist=None, lift2d=None):
        for key, obj in (("gather", gather), ("scatter", scatter), ("loop", loop), ("kdist", kdist), ("lift2d", lift2d)):
            if obj is None:
                continue
            text = obj if isinstance(obj, str) else json.dumps(obj)
            if self.L.fortis_configure(key.encode(), text.encode()) != 0:
                raise _lib.FortisError(self.L.fortis_last_error_message().decode())

    def load_model(self, blob: bytes):
        buf = ctypes.create_string_buffer(blob, len(blob))
        if self.L.fortis_load_model_mem(ctypes.cast(buf, ctypes.c_void_p), len(blob)) != 0:
            raise _lib.FortisError(self.L.fortis_last_error_message().decode())

    def option(self, key, value):
        if self.L.fortis_set_option(key.encode(), str(value).encode()) != 0:
            raise _lib.FortisError(self.L.fortis_last_error_message().decode())

    def set_vector(self, name, data):
        a = np.ascontiguousarray(data)
        elt = {np.dtype(np.float32): 0, np.dtype(np.float64): 1}[a.dtype]
        if self.L.fortis_set_vector(name.encode(), a.ctypes.data, a.size, elt) != 0:
            raise _lib.FortisError(self.L.fortis_last_error_message().decode())

    def check(self):
        _lib.check(self.L)

    # ---- the three calls of a lifted host ----------------------------------------------------------------------
    def _vp(self, arrays):
        self._keep.extend(a for a in arrays if isinstance(a, np.ndarray) and not any(a is k for k in self._keep))
        return (ctypes.c_void_p * len(arrays))(*[_ptr(a) for a in arrays])

    def _ip(self, ints):
        return (ctypes.c_int * max(1, len(ints)))(*ints)

    def gather(self, arrays, args=()):
        self.L.fortis_gatherv(self._ip(list(args)), len(args), self._vp(arrays), len(arrays))
        self.check()

    def forward_batched(self, x=None, y=None):
        self.L.mlp_forward_batched(_ptr(x) if x is not None else None, _ptr(y) if y is not None else None)
        self.check()

    def scatter(self, arrays, args=(1,)):
        self.L.fortis_scatterv(self._ip(list(args)), len(args), self._vp(arrays), len(arrays))
        self.check()

    def step(self, gather_arrays, scatter_arrays, args=()):
        if args:
            self.L.fortis_stepvi(self._ip(list(args)), len(args), self._vp(gather_arrays), len(gather_arrays),
                                 self._vp(scatter_arrays), len(scatter_arrays))
        else:
            self.L.fortis_stepv(self._vp(gather_arrays), len(gather_arrays), self._vp(scatter_arrays), len(scatter_arrays))
        self.check()

    def forward(self, x, y):
        self._keep.extend(a for a in (x, y) if isinstance(a, np.ndarray))
        self.L.mlp_forward(_ptr(x), _ptr(y))
        self.check()

    # ---- helpers -----------------------------------------------------------------------------------------------
    def sync(self):
        self.L.fortis_sync()

    def stream(self):
        return self.L.mgpuStreamCreate()

    def model_output(self, rows, nout):
        """Copy of the device model-output buffer as (rows, nout) float32."""
        p = self.L.fortis_model_output()
        self.check()
        out = np.empty((rows, nout), dtype=np.float32)
        if self.L.fortis_copy_to_host(out.ctypes.data, p, out.nbytes) != 0:
            raise _lib.FortisError(self.L.fortis_last_error_message().decode())
        return out

    def model_input(self, rows, nin):
        """Copy of the device model-input buffer; a pending gather is run as its own kernel first."""
        p = self.L.fortis_model_input()
        self.check()
        out = np.empty((rows, nin), dtype=np.float32)
        if self.L.fortis_copy_to_host(out.ctypes.data, p, out.nbytes) != 0:
            raise _lib.FortisError(self.L.fortis_last_error_message().decode())
        return out

    def checksum(self, a):
        out = ctypes.c_double(0.0)
        if isinstance(a, np.ndarray):
            elt = {np.dtype(np.float32): 0, np.dtype(np.float64): 1}[a.dtype]
            n = a.size
        else:
            import torch
            elt = {torch.float32: 0, torch.float64: 1}[a.dtype]
            n = a.numel()
        if self.L.fortis_checksum(_ptr(a), n, elt, ctypes.byref(out)) != 0:
            raise _lib.FortisError(self.L.fortis_last_error_message().decode())
        return out.value

    def step_checksum(self):
        out = ctypes.c_double(0.0)
        self.L.fortis_step_checksum(ctypes.byref(out))
        return out.value
