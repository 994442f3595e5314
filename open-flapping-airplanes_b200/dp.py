"""Data-parallel driver: bucketed gradient all-reduce over NCCL, ordered against the persistent megakernel by device flags
only. The reference is single-GPU (no collective anywhere in it); this is the multi-GPU plumbing of this library.

Per rank, the megakernel raises ready[b] = s+1 (a 1-task phase of its graph) once every gradient of bucket b of step s is
written, and holds that bucket's AdamW phases behind a bounded wait for done[b] >= s+1. This module enqueues, for every
step and bucket of a launch, on one communication stream and BEFORE the launch:
    cuStreamWaitValue32(ready[b] >= s+1)  ->  all_reduce(bucket b, sum, in place)  ->  cuStreamWriteValue32(done[b] = s+1)
so no host thread sits in the loop while the kernel runs. The sum is not divided here: AdamW folds 1/world into its read of
the gradient. NCCL's blocks run on the SMs the megakernel leaves unoccupied (the reserved partition), so the number of NCCL
channels must not exceed what fits there: `configure_nccl_env()` caps it before the process group is created.
"""
import ctypes as C
import os

import numpy as np


def configure_nccl_env(reserved_sms=8):
    """Call before torch.distributed.init_process_group. Keeps NCCL's resident blocks within the reserved SM partition."""
    os.environ.setdefault("NCCL_MAX_CTAS", str(max(1, reserved_sms)))
    os.environ.setdefault("NCCL_MIN_CTAS", "1")


def bucket_schedule(buckets, nsteps):
    """Order in which (step, bucket) pairs are communicated: step-major, buckets in the order their gradients become ready
    (the library lists them in that order: head first, embeddings last)."""
    return [(s, b) for s in range(nsteps) for b in range(len(buckets))]


def allreduce_buckets_host(dist, flat, buckets, nsteps=1):
    """The communication the device-flag schedule performs, without the flags: sum-all-reduce every bucket of `flat` in
    place, in schedule order. Works on CPU tensors over gloo (used by the CPU tests) and defines what the GPU path must equal."""
    for _, b in bucket_schedule(buckets, nsteps):
        off, cnt = buckets[b]
        dist.all_reduce(flat[off:off + cnt])
    return flat


def buckets_partition_params(buckets, num_params):
    """True when the buckets are disjoint and cover [0, num_params) exactly."""
    spans = sorted(buckets)
    pos = 0
    for off, cnt in spans:
        if off != pos or cnt <= 0:
            return False
        pos = off + cnt
    return pos == num_params


class _DevArray:
    """Minimal __cuda_array_interface__ wrapper so torch can view library-owned device memory without a copy."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (int(ptr), False), "version": 3, "strides": None}


class DataParallel:
    def __init__(self, mk, dist, stream=None):
        import torch
        from cuda.bindings import driver as cu
        self.torch, self.cu, self.mk, self.dist = torch, cu, mk, dist
        self.buckets = mk.buckets()
        if not self.buckets:
            raise RuntimeError("the context was not created with ext_sync=1")
        n = mk.num_params
        gptr = mk.grad_buffer_ptr()
        if mk.cfg.grad_bf16:
            raw = torch.as_tensor(_DevArray(gptr, n, "<i2"), device="cuda")      # bf16 has no array-interface code: view int16 as bf16
            self.grad = raw.view(torch.bfloat16)
        else:
            self.grad = torch.as_tensor(_DevArray(gptr, n, "<f4"), device="cuda")
        self.ready_ptr, self.done_ptr = mk.ext_flags_ptrs()
        self.stream = stream if stream is not None else torch.cuda.Stream()
        self._zeros = np.zeros(64, dtype=np.int32)

    def _check(self, res):
        err = res[0] if isinstance(res, tuple) else res
        if int(err) != 0:
            raise RuntimeError(f"CUDA driver call failed: {err}")

    def enqueue(self, nsteps):
        """Queue the whole launch's communication. The previous launch must have finished (its flags are cleared here)."""
        from . import capi
        capi.load().ofa_h2d(C.c_void_p(self.ready_ptr), self._zeros.ctypes.data_as(C.c_void_p), self._zeros.nbytes)
        torch, cu = self.torch, self.cu
        h = cu.CUstream(self.stream.cuda_stream)
        geq = cu.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_GEQ
        with torch.cuda.stream(self.stream):
            for s, b in bucket_schedule(self.buckets, nsteps):
                off, cnt = self.buckets[b]
                self._check(cu.cuStreamWaitValue32(h, self.ready_ptr + 4 * b, s + 1, geq))
                self.dist.all_reduce(self.grad[off:off + cnt])
                self._check(cu.cuStreamWriteValue32(h, self.done_ptr + 4 * b, s + 1, 0))

    def finish(self):
        self.stream.synchronize()
