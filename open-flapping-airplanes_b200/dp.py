"""Data-parallel driver: bucketed gradient all-reduce over NCCL, ordered against the persistent megakernel by device flags
only. The reference is single-GPU (no collective anywhere in it); this is the multi-GPU plumbing of this library.

Per rank, the megakernel raises ready[b] = g+1 (a 1-task phase of its graph; g = global step index since the context was
created) once every gradient of bucket b of that step is written, and holds the bucket's AdamW phases behind a bounded wait
for done[b] >= g+1. For every step and bucket of a launch this module enqueues on one communication stream
    cuStreamWaitValue32(ready[b] >= g+1)  ->  all_reduce(bucket b, sum, in place)  ->  cuStreamWriteValue32(done[b] = g+1)
so no host thread sits in the loop while the kernel runs. The sum is not divided here: AdamW folds 1/world into its read of
the gradient.

Two rules keep this free of false dependencies:
  * enqueue AFTER the launch (`mk.launch(n); dp.enqueue(n)`): a stream-wait that sits at the head of a hardware queue blocks
    every stream mapped to that queue, and it must never be able to block the launch of the kernel that will satisfy it;
    `configure_env()` also raises CUDA_DEVICE_MAX_CONNECTIONS so that streams rarely share a queue;
  * NCCL's blocks run on the SMs the megakernel leaves unoccupied (the reserved partition), so the number of NCCL channels
    must not exceed what fits there: `configure_env()` caps it before the process group is created.
If the communication side never answers, the device-side wait expires and the launch returns OFA_DEVICE_ABORT.
"""
import os

import numpy as np


def configure_env(reserved_sms=8):
    """Call before the first CUDA call of the process and before torch.distributed.init_process_group."""
    os.environ.setdefault("NCCL_MAX_CTAS", str(max(1, reserved_sms)))
    os.environ.setdefault("NCCL_MIN_CTAS", "1")
    os.environ.setdefault("NCCL_CGA_CLUSTER_SIZE", "0")     # no thread-block clusters: a cluster needs several free SMs of one GPC at once
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")


configure_nccl_env = configure_env


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
        if self.grad.data_ptr() != gptr:
            raise RuntimeError("torch copied the gradient buffer instead of aliasing it")
        self.ready_ptr, self.done_ptr = mk.ext_flags_ptrs()
        self.stream = stream if stream is not None else torch.cuda.Stream()
        # first collective on the communication stream now: communicator set-up and its allocations must not happen while
        # a persistent kernel is resident
        with torch.cuda.stream(self.stream):
            warm = torch.zeros(1024, device="cuda", dtype=self.grad.dtype)
            dist.all_reduce(warm)
        self.stream.synchronize()

    def _check(self, res):
        err = res[0] if isinstance(res, tuple) else res
        if int(err) != 0:
            raise RuntimeError(f"CUDA driver call failed: {err}")

    def enqueue(self, nsteps, first_step=None):
        """Queue the communication of a launch of `nsteps` steps. Call right AFTER mk.launch(nsteps)."""
        torch, cu = self.torch, self.cu
        base = self.mk.steps_done if first_step is None else first_step
        h = cu.CUstream(self.stream.cuda_stream)
        geq = cu.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_GEQ
        with torch.cuda.stream(self.stream):
            for s, b in bucket_schedule(self.buckets, nsteps):
                off, cnt = self.buckets[b]
                self._check(cu.cuStreamWaitValue32(h, self.ready_ptr + 4 * b, base + s + 1, geq))
                self.dist.all_reduce(self.grad[off:off + cnt])
                self._check(cu.cuStreamWriteValue32(h, self.done_ptr + 4 * b, base + s + 1, 0))

    def finish(self):
        self.stream.synchronize()
