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

The reverse case - a rank's kernel stops early (a bounded device wait expired, or the host called ofa_abort) - would leave that
rank's queued stream waits without the `ready` values they wait for, and every peer's all-reduce waiting for this rank.
`DataParallel.wait()` handles it: the failing rank raises every ready flag to the last queued target (`cancel()`), so its queue
drains and the collectives complete with data nobody will use; afterwards the ranks exchange their status, so that every rank
raises, not only the one whose kernel stopped. `finish()` gives up after a timeout instead of blocking for good.

`NativeDataParallel` offers the same calls on top of the library's own C++ queue (ofa_dp_*: an NCCL communicator of its own,
looked up with dlopen), for hosts that have no torch.distributed; `DataParallel` reuses the process group the host already has.

The queue itself sits behind a small interface (wait for a flag value, all-reduce a span, write a flag value, raise the ready
flags out of band, drain with a timeout). `CudaFlagQueue` implements it with stream memory operations; `HostFlagQueue` runs
the same operations on a host thread over a numpy flag array, so the cancel and status logic is tested among CPU ranks (gloo).
"""
import os
import time

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


class DataParallelAborted(RuntimeError):
    """A rank's kernel stopped before the end of the launch; raised on EVERY rank of the group after the queues have drained."""


class CudaFlagQueue:
    """The communication queue on a CUDA stream: stream memory operations on the library's device flags around NCCL calls."""

    def __init__(self, mk, dist, stream=None):
        import torch
        from cuda.bindings import driver as cu
        self.torch, self.cu, self.dist = torch, cu, dist
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
        self.side = torch.cuda.Stream()                  # out-of-band flag writes (cancel) must not queue behind the waits they release
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

    def wait_ready(self, b, value):
        self._check(self.cu.cuStreamWaitValue32(self.cu.CUstream(self.stream.cuda_stream), self.ready_ptr + 4 * b, value,
                                                self.cu.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_GEQ))

    def all_reduce(self, off, cnt):
        with self.torch.cuda.stream(self.stream):
            self.dist.all_reduce(self.grad[off:off + cnt])

    def write_done(self, b, value):
        self._check(self.cu.cuStreamWriteValue32(self.cu.CUstream(self.stream.cuda_stream), self.done_ptr + 4 * b, value, 0))

    def raise_ready(self, nbuckets, value):
        h = self.cu.CUstream(self.side.cuda_stream)
        for b in range(nbuckets):
            self._check(self.cu.cuStreamWriteValue32(h, self.ready_ptr + 4 * b, value, 0))

    def drain(self, timeout_s):
        t0 = time.monotonic()
        while not self.stream.query():
            if timeout_s is not None and time.monotonic() - t0 > timeout_s:
                return False
            time.sleep(0.0005)
        return True

    def exchange_failed(self, failed):
        t = self.torch.tensor([1 if failed else 0], device="cuda", dtype=self.torch.int32)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return bool(t.item())


class HostFlagQueue:
    """The same queue on the host: a worker thread executes the operations in order over a numpy flag array (ready[0:32],
    done[32:64]) and a CPU gradient tensor, with torch.distributed (gloo) as the collective. Stands in for the device flags
    and the stream in CPU tests; the "kernel" of such a test is whoever writes ready[] and reads done[]."""

    def __init__(self, grad, dist, poll_s=0.0005):
        import threading
        self.grad, self.dist, self.poll_s = grad, dist, poll_s
        self.flags = np.zeros(64, dtype=np.int32)
        self.ops, self.lock, self.stop = [], threading.Lock(), False
        self.idle = threading.Event(); self.idle.set()
        self.th = threading.Thread(target=self._run, daemon=True); self.th.start()

    def _run(self):
        while not self.stop:
            with self.lock:
                op = self.ops.pop(0) if self.ops else None
                if op is None:
                    self.idle.set()
            if op is None:
                time.sleep(self.poll_s); continue
            kind = op[0]
            if kind == "wait":
                while self.flags[op[1]] < op[2] and not self.stop:
                    time.sleep(self.poll_s)
            elif kind == "reduce":
                self.dist.all_reduce(self.grad[op[1]:op[1] + op[2]])
            else:
                self.flags[32 + op[1]] = op[2]

    def _push(self, op):
        with self.lock:
            self.idle.clear(); self.ops.append(op)

    def wait_ready(self, b, value):
        self._push(("wait", b, value))

    def all_reduce(self, off, cnt):
        self._push(("reduce", off, cnt))

    def write_done(self, b, value):
        self._push(("write", b, value))

    def raise_ready(self, nbuckets, value):
        for b in range(nbuckets):
            self.flags[b] = max(int(self.flags[b]), value)

    def drain(self, timeout_s):
        return self.idle.wait(timeout_s)

    def exchange_failed(self, failed):
        import torch
        t = torch.tensor([1 if failed else 0], dtype=torch.int32)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return bool(t.item())

    def close(self):
        self.stop = True


class DataParallel:
    def __init__(self, mk, dist, stream=None, queue=None):
        self.mk, self.dist = mk, dist
        self.buckets = mk.buckets()
        if not self.buckets:
            raise RuntimeError("the context was not created with ext_sync=1")
        self.q = queue if queue is not None else CudaFlagQueue(mk, dist, stream)
        self.last_target = 0                             # highest flag value any queued wait is waiting for

    @property
    def stream(self):
        return self.q.stream

    @property
    def grad(self):
        return self.q.grad

    def enqueue(self, nsteps, first_step=None):
        """Queue the communication of a launch of `nsteps` steps. Call right AFTER mk.launch(nsteps)."""
        base = self.mk.steps_done if first_step is None else first_step
        for s, b in bucket_schedule(self.buckets, nsteps):
            off, cnt = self.buckets[b]
            self.q.wait_ready(b, base + s + 1)
            self.q.all_reduce(off, cnt)
            self.q.write_done(b, base + s + 1)
        self.last_target = max(self.last_target, base + nsteps)

    def cancel(self):
        """Release every queued wait of this rank: its kernel will not raise the remaining ready flags (it stopped early), so
        the host raises them to the last queued target. The collectives behind them then run on whatever the buckets hold; the
        step they belong to is lost, which `wait()` reports on every rank."""
        self.q.raise_ready(len(self.buckets), self.last_target)

    def finish(self, timeout_s=120.0):
        """Wait until the queue is empty. Returns False when it is not after `timeout_s` seconds (None = no limit)."""
        return self.q.drain(timeout_s)

    def wait(self, timeout_ms=600000, comm_timeout_s=120.0, kernel_wait=None):
        """mk.wait + finish for a data-parallel launch, with the failure path: if this rank's kernel stopped early its queue is
        cancelled first; then all ranks learn whether any of them failed and raise together (the failing rank its own error,
        the others DataParallelAborted). `kernel_wait` replaces mk.wait in tests."""
        err = None
        try:
            (kernel_wait or (lambda: self.mk.wait(timeout_ms)))()
        except Exception as e:                           # OfaError from ofa_wait: device abort, timeout, CUDA error
            err = e
            self.cancel()
        drained = self.finish(comm_timeout_s)
        if not drained and err is None:
            err = DataParallelAborted(f"the communication queue did not drain within {comm_timeout_s} s")
        if drained:
            any_failed = self.q.exchange_failed(err is not None)
        else:
            any_failed = True                            # this rank cannot take part in a collective any more
        if err is not None:
            raise err
        if any_failed:
            raise DataParallelAborted("another rank's kernel stopped early: the gradients of this launch are not valid")


def torch_nccl_library():
    """Path of the NCCL that ships with torch (nvidia-nccl wheel), or None: what OFA_NCCL_LIB should point to when the
    process has no other NCCL."""
    try:
        import nvidia.nccl as pkg
        for base in list(getattr(pkg, "__path__", [])):
            cand = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(cand):
                return cand
    except Exception:
        pass
    return None


class NativeDataParallel:
    """DataParallel's surface (enqueue / cancel / finish / wait) on the library's C++ communication side. The only thing it
    needs from the host is the rendezvous: `exchange(id_bytes_or_None) -> id_bytes` hands rank 0's 128-byte id to every
    rank (default: torch.distributed's object broadcast)."""

    def __init__(self, mk, rank, world, exchange=None):
        import ctypes as C
        from . import capi
        self.mk, self.C, self.capi, self.lib = mk, C, capi, mk.lib
        self.buckets = mk.buckets()
        if not self.buckets:
            raise RuntimeError("the context was not created with ext_sync=1")
        if "OFA_NCCL_LIB" not in os.environ and torch_nccl_library():
            os.environ["OFA_NCCL_LIB"] = torch_nccl_library()
        ident, why = None, ""
        if rank == 0:
            buf = C.create_string_buffer(128)
            if self.lib.ofa_dp_unique_id(buf) == capi.OK:
                ident = buf.raw
            else:
                why = self.lib.ofa_last_error(None).decode()      # the other ranks still get their answer below: nobody waits for good
        if exchange is None:
            import torch.distributed as dist
            box = [ident, why]
            dist.broadcast_object_list(box, src=0)
            ident, why = box
        else:
            ident = exchange(ident)
        if ident is None:
            raise RuntimeError("ofa_dp_unique_id failed on rank 0: " + why)
        mk._chk(self.lib.ofa_dp_init(mk.h, C.c_char_p(ident), rank, world))

    def enqueue(self, nsteps):
        self.mk._chk(self.lib.ofa_dp_enqueue(self.mk.h, nsteps))

    def cancel(self):
        self.lib.ofa_dp_cancel(self.mk.h)

    def finish(self, timeout_s=120.0):
        return self.lib.ofa_dp_finish(self.mk.h, -1 if timeout_s is None else int(timeout_s * 1000)) == self.capi.OK

    def wait(self, timeout_ms=600000, comm_timeout_s=120.0):
        from .host import OfaError
        st = self.capi.Status()
        rc = self.lib.ofa_dp_wait(self.mk.h, timeout_ms, int(comm_timeout_s * 1000), self.C.byref(st))
        if rc == self.capi.OK:
            return
        msg = self.lib.ofa_last_error(self.mk.h).decode()
        if rc == self.capi.DEVICE_ABORT and "another rank" in msg:
            raise DataParallelAborted(msg)
        raise OfaError(rc, "timeout" if rc == self.capi.TIMEOUT and not msg else msg, st)

    def close(self):
        self.lib.ofa_dp_shutdown(self.mk.h)
