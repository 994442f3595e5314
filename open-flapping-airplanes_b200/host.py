"""Model-level host interface: the calls main() of the reference program makes (llm/b200/megakernel/ofa.cu:394-766),
as a Python class over the C ABI: configure, load weights and tokens, one persistent launch, wait with a bound, read
losses / timings / decoded tokens back."""
import ctypes as C

import numpy as np

from . import capi
from .tasks import OfaError

PARAM_ORDER_DOC = "wte, wpe, [lm_head], per layer {g1, Wqkv, Wo, g2, Wup, Wdn}, gf  (all W[in,out] row-major)"


def default_config(preset):
    cfg = capi.Config()
    rc = capi.load().ofa_default_config(C.byref(cfg), preset.encode())
    if rc != capi.OK:
        raise OfaError(rc, f"unknown preset {preset!r}")
    return cfg


def flat_from_named(w, n_layer, tied):
    """dict name -> fp32 array in the reference's naming (llm/baseline/common.py:39-54: wte, wpe, L00_Wqkv, ... gamma_f,
    plus lm_head when untied) -> one flat fp32 vector in the library's layout."""
    parts = [w["wte"], w["wpe"]]
    if not tied:
        parts.append(w["lm_head"])
    for l in range(n_layer):
        p = f"L{l:02d}_"
        parts += [w[p + "gamma1"], w[p + "Wqkv"], w[p + "Wo"], w[p + "gamma2"], w[p + "Wup"], w[p + "Wdown"]]
    parts.append(w["gamma_f"])
    return np.concatenate([np.asarray(x, dtype=np.float32).reshape(-1) for x in parts])


class Megakernel:
    def __init__(self, cfg):
        self.lib = capi.load()
        self.cfg = cfg
        self.h = C.c_void_p()
        rc = self.lib.ofa_create(C.byref(cfg), C.byref(self.h))
        if rc != capi.OK:
            raise OfaError(rc, self.lib.ofa_last_error(None).decode())

    # ---- helpers
    def _chk(self, rc, status=None):
        if rc != capi.OK:
            raise OfaError(rc, self.lib.ofa_last_error(self.h).decode(), status)

    def close(self):
        if self.h:
            self.lib.ofa_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def num_params(self):
        return self.lib.ofa_num_params(self.h)

    def param_span(self, name):
        off, cnt = C.c_size_t(), C.c_size_t()
        self._chk(self.lib.ofa_param_span(self.h, name.encode(), C.byref(off), C.byref(cnt)))
        return off.value, cnt.value

    # ---- weights / tokens
    def load_weights(self, flat):
        flat = np.ascontiguousarray(flat, dtype=np.float32)
        self._chk(self.lib.ofa_load_weights(self.h, flat.ctypes.data_as(C.c_void_p), flat.size))

    def _read(self, fn, n=None):
        n = self.num_params if n is None else n
        out = np.empty(n, dtype=np.float32)
        self._chk(fn(self.h, out.ctypes.data_as(C.c_void_p), n))
        return out

    def read_weights(self):
        return self._read(self.lib.ofa_read_weights)

    def read_grads(self):
        return self._read(self.lib.ofa_read_grads)

    def read_adam(self):
        return self._read(self.lib.ofa_read_adam_m), self._read(self.lib.ofa_read_adam_v)

    def load_adam_state(self, m, v, step_base):
        m = np.ascontiguousarray(m, dtype=np.float32); v = np.ascontiguousarray(v, dtype=np.float32)
        self._chk(self.lib.ofa_load_adam_state(self.h, m.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p), m.size, step_base))

    def set_tokens(self, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        self._chk(self.lib.ofa_set_tokens(self.h, t.ctypes.data_as(C.c_void_p), t.size))

    def set_starts(self, starts):
        if starts is None:
            self._chk(self.lib.ofa_set_starts(self.h, None, 0)); return
        s = np.ascontiguousarray(starts, dtype=np.uint32)
        assert s.ndim == 2 and s.shape[1] == self.cfg.batch
        self._chk(self.lib.ofa_set_starts(self.h, s.ctypes.data_as(C.c_void_p), s.shape[0]))

    # ---- run
    def launch(self, nsteps):
        self._chk(self.lib.ofa_launch(self.h, nsteps))

    def wait(self, timeout_ms=600000):
        st = capi.Status()
        rc = self.lib.ofa_wait(self.h, timeout_ms, C.byref(st))
        if rc != capi.OK:
            raise OfaError(rc, "timeout" if rc == capi.TIMEOUT else self.lib.ofa_last_error(self.h).decode(), st)

    def abort(self):
        return self.lib.ofa_abort(self.h)

    def run(self, nsteps, timeout_ms=600000):
        self.launch(nsteps); self.wait(timeout_ms)
        return self.lib.ofa_last_launch_ms(self.h)

    @property
    def steps_done(self):
        return self.lib.ofa_steps_done(self.h)

    @property
    def last_launch_ms(self):
        return self.lib.ofa_last_launch_ms(self.h)

    def live(self):
        l = capi.LiveT()
        self._chk(self.lib.ofa_live(self.h, C.byref(l)))
        return {"steps": l.steps, "loss": l.loss, "decode_steps": l.decode_steps}

    def losses(self, n=None):
        n = self.steps_done if n is None else n
        out = np.empty(n, dtype=np.float32)
        if n:
            self._chk(self.lib.ofa_read_losses(self.h, out.ctypes.data_as(C.c_void_p), n))
        return out

    def step_times_ns(self, n):
        out = np.empty(n, dtype=np.uint64)
        self._chk(self.lib.ofa_read_step_times(self.h, out.ctypes.data_as(C.c_void_p), n))
        return out

    def phases(self):
        res = []
        for i in range(self.lib.ofa_num_phases(self.h)):
            name = C.create_string_buffer(64); kind, nt, busy = C.c_int(), C.c_int(), C.c_ulonglong()
            self._chk(self.lib.ofa_phase_info(self.h, i, name, 64, C.byref(kind), C.byref(nt), C.byref(busy)))
            wait = C.c_ulonglong()
            self._chk(self.lib.ofa_phase_wait_ns(self.h, i, C.byref(wait)))
            res.append({"name": name.value.decode(), "kind": kind.value, "ntasks": nt.value, "busy_ns": busy.value, "wait_ns": wait.value})
        return res

    def phase_windows(self):
        """(first task start, last task end) in %globaltimer ns of every training phase in the last step of the last launch"""
        res = []
        for i in range(self.lib.ofa_num_phases(self.h)):
            a, b = C.c_ulonglong(), C.c_ulonglong()
            self._chk(self.lib.ofa_phase_window(self.h, i, C.byref(a), C.byref(b)))
            res.append((a.value, b.value))
        return res

    def block_busy_ns(self, nblocks=296):
        out = np.zeros(2 * nblocks, dtype=np.uint64)
        self._chk(self.lib.ofa_read_block_busy(self.h, out.ctypes.data_as(C.c_void_p), out.size))
        return out.reshape(nblocks, 2)

    def block_wait_ns(self, nblocks=296):
        """rows: dependency wait, claim, hand-off to the block, completion signalling (ns per block, training job)"""
        out = np.zeros(6 * nblocks, dtype=np.uint64)
        self._chk(self.lib.ofa_read_block_busy(self.h, out.ctypes.data_as(C.c_void_p), out.size))
        return out[2 * nblocks:].reshape(4, nblocks)

    def block_info(self, nblocks=296):
        """(smid, role) per block of the last launch; role 1 serving, 2 reserved, 3 training, 4 idle"""
        out = np.zeros(nblocks, dtype=np.int32)
        self._chk(self.lib.ofa_read_block_info(self.h, out.ctypes.data_as(C.c_void_p), out.size))
        return out & 0xFFFF, out >> 16

    def decode_trace(self):
        out = np.zeros(64, dtype=np.uint64)
        self._chk(self.lib.ofa_read_decode_trace(self.h, out.ctypes.data_as(C.c_void_p), 64))
        return out

    def decode_phases(self):
        res, i = [], 0
        while True:
            name = C.create_string_buffer(64); nt, busy = C.c_int(), C.c_ulonglong()
            if self.lib.ofa_decode_phase_info(self.h, i, name, 64, C.byref(nt), C.byref(busy)) != capi.OK:
                return res
            res.append({"name": name.value.decode(), "ntasks": nt.value, "busy_ns": busy.value}); i += 1

    def phase_deps(self, phase, job=0):
        ph = (C.c_int * 64)(); de = (C.c_int * 64)()
        n = self.lib.ofa_phase_deps(self.h, job, phase, ph, de, 64)
        if n < 0:
            raise OfaError(capi.BAD_ARGUMENT, "no such phase")
        return [(ph[i], de[i]) for i in range(min(n, 64))]

    def phase_dep_grain(self, phase):
        """(rb_map of the phase, [1 if the dependency is waited for per 128-token row block else 0, ...] in phase_deps order)"""
        rb = C.c_int(); gr = (C.c_int * 64)()
        n = self.lib.ofa_phase_dep_grain(self.h, phase, C.byref(rb), gr, 64)
        if n < 0:
            raise OfaError(capi.BAD_ARGUMENT, "no such phase")
        return rb.value, [gr[i] for i in range(min(n, 64))]

    # ---- decode
    @property
    def decode_steps(self):
        return self.lib.ofa_decode_steps(self.h)

    def decode_tokens(self, cap=None):
        cap = self.cfg.decode_out_cap if cap is None else cap
        out = np.empty(cap, dtype=np.int32)
        n = self.lib.ofa_read_decode_tokens(self.h, out.ctypes.data_as(C.c_void_p), cap)
        if n < 0:
            raise OfaError(n, self.lib.ofa_last_error(self.h).decode())
        return out[:n]

    def decode_logits(self):
        out = np.empty(self.cfg.vocab, dtype=np.float32)
        self._chk(self.lib.ofa_read_decode_logits(self.h, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def read_buffer(self, name, shape, dtype):
        """dtype: 'bf16' or a numpy dtype. Returns float32 for bf16."""
        from .tasks import from_bf16_bits
        host = np.empty(shape, dtype=np.uint16 if dtype == "bf16" else dtype)
        self._chk(self.lib.ofa_read_buffer(self.h, name.encode(), host.ctypes.data_as(C.c_void_p), host.nbytes))
        return from_bf16_bits(host).reshape(shape) if dtype == "bf16" else host

    # ---- data-parallel hooks
    def buckets(self):
        res = []
        for b in range(self.lib.ofa_num_buckets(self.h)):
            off, cnt = C.c_size_t(), C.c_size_t()
            self._chk(self.lib.ofa_bucket_span(self.h, b, C.byref(off), C.byref(cnt)))
            res.append((off.value, cnt.value))
        return res

    def grad_buffer_ptr(self):
        return self.lib.ofa_grad_buffer(self.h)

    def ext_flags_ptrs(self):
        return self.lib.ofa_ext_ready_flags(self.h), self.lib.ofa_ext_done_flags(self.h)
