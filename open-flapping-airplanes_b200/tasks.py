"""Task-level host interface: device buffers and explicit phase lists run through the persistent scheduler
(ofa_run_phases). This is how the per-task parity tests drive single kernels, the way the reference's standalone test
programs launch one task set at a time (llm/gemm/test_gemm.cu, llm/attention/test_attention.cu,
llm/elementwise/test_elementwise.cu)."""
import ctypes as C

import numpy as np

from . import capi


class OfaError(RuntimeError):
    def __init__(self, code, msg, status=None):
        super().__init__(f"ofa error {code}: {msg}")
        self.code, self.status = code, status


def to_bf16_bits(a):
    """float32 array -> uint16 bf16 bit patterns, round-to-nearest-even (NaN preserved)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    out = ((u + r) >> 16).astype(np.uint16)
    nan = np.isnan(a)
    if nan.any():
        out[nan] = 0x7FC0
    return out


def from_bf16_bits(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_round(a):
    return from_bf16_bits(to_bf16_bits(a)).reshape(np.shape(a))


class DeviceBuffer:
    """A device allocation made through the C ABI; `dtype` is 'bf16', np.float32, np.int32 ... Zero-filled."""

    def __init__(self, shape, dtype):
        self.shape = tuple(np.atleast_1d(shape).tolist()) if not isinstance(shape, tuple) else shape
        self.dtype = dtype
        self.itemsize = 2 if dtype == "bf16" else np.dtype(dtype).itemsize
        self.nbytes = int(np.prod(self.shape)) * self.itemsize
        self.ptr = C.c_void_p()
        rc = capi.load().ofa_dev_alloc(C.byref(self.ptr), max(1, self.nbytes))
        if rc != capi.OK:
            raise OfaError(rc, "device allocation failed")

    @classmethod
    def from_host(cls, arr, dtype=None):
        arr = np.asarray(arr)
        dt = dtype if dtype is not None else arr.dtype
        buf = cls(arr.shape, dt)
        buf.upload(arr)
        return buf

    def upload(self, arr):
        host = to_bf16_bits(arr) if self.dtype == "bf16" else np.ascontiguousarray(arr, dtype=self.dtype)
        assert host.nbytes == self.nbytes, (host.nbytes, self.nbytes)
        rc = capi.load().ofa_h2d(self.ptr, host.ctypes.data_as(C.c_void_p), self.nbytes)
        if rc != capi.OK:
            raise OfaError(rc, "H2D copy failed")

    def download(self):
        host = np.empty(self.shape, dtype=np.uint16 if self.dtype == "bf16" else self.dtype)
        rc = capi.load().ofa_d2h(host.ctypes.data_as(C.c_void_p), self.ptr, self.nbytes)
        if rc != capi.OK:
            raise OfaError(rc, "D2H copy failed")
        return from_bf16_bits(host).reshape(self.shape) if self.dtype == "bf16" else host

    def at(self, elem_offset):
        return C.c_void_p(self.ptr.value + elem_offset * self.itemsize)

    def free(self):
        if self.ptr and self.ptr.value:
            capi.load().ofa_dev_free(self.ptr)
            self.ptr = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, DeviceBuffer):
        return x.ptr.value
    if isinstance(x, C.c_void_p):
        return x.value
    return int(x)


def phase(kind, ptrs=(), n=0, i0=0, i1=0, i2=0):
    ph = capi.Phase()
    ph.kind = kind
    for k, p in enumerate(ptrs):
        ph.p[k] = _ptr(p)
    ph.n, ph.i0, ph.i1, ph.i2 = n, i0, i1, i2
    return ph


def gemm_phase(layout, epi, M, N, K, A, lda, B, ldb, Cc, ldc, aux=None, ldaux=0, accumulate=0, nsub=0):
    ph = capi.Phase()
    ph.kind, ph.layout, ph.epi, ph.accumulate = capi.TK_GEMM, layout, epi, accumulate
    ph.M, ph.N, ph.K, ph.lda, ph.ldb, ph.ldc, ph.ldaux, ph.nsub = M, N, K, lda, ldb, ldc, ldaux, nsub
    ph.p[0], ph.p[1], ph.p[2], ph.p[3] = _ptr(A), _ptr(B), _ptr(Cc), _ptr(aux)
    return ph


def run_phases(dtype, dims, phases, repeats=1, adam=None):
    """dims = dict(vocab, d_model, n_layer, n_head, ctx_len, batch). Returns the CUDA-event time of the launch in ms."""
    lib = capi.load()
    d = capi.Dims(dims["vocab"], dims["d_model"], dims.get("n_layer", 1), dims["n_head"], dims["ctx_len"], dims["batch"])
    arr = (capi.Phase * len(phases))(*phases)
    ms = C.c_float(0)
    st = capi.Status()
    ad = (C.c_float * 6)(*adam) if adam is not None else None
    rc = lib.ofa_run_phases(dtype, C.byref(d), arr, len(phases), repeats, ad, C.byref(ms), C.byref(st))
    if rc != capi.OK:
        raise OfaError(rc, lib.ofa_last_error(None).decode(), st)
    return ms.value
