"""ctypes view of include/ofa_b200.h. The library is loaded from csrc/ (in-tree); a missing library is an error, never a
fallback: there is no CPU path in this package."""
import ctypes as C
import os

from . import build as _build

_lib = None


class Config(C.Structure):
    _fields_ = [
        ("vocab", C.c_int), ("d_model", C.c_int), ("n_layer", C.c_int), ("n_head", C.c_int), ("ctx_len", C.c_int), ("batch", C.c_int),
        ("valid_vocab", C.c_int), ("tied_head", C.c_int), ("dtype", C.c_int), ("mode", C.c_int),
        ("sched_steps", C.c_int), ("warmup", C.c_int), ("constant_lr", C.c_int),
        ("lr_max", C.c_float), ("lr_min", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float), ("weight_decay", C.c_float),
        ("data_seed", C.c_ulonglong),
        ("infer_sms", C.c_int), ("reserved_sms", C.c_int), ("train_sms", C.c_int), ("use_decode", C.c_int),
        ("n_prompt", C.c_int), ("prompt", C.c_int * 32), ("answer_len", C.c_int), ("temperature", C.c_float), ("decode_seed", C.c_ulonglong),
        ("decode_out_cap", C.c_int), ("dp_world", C.c_int), ("grad_bf16", C.c_int), ("ext_sync", C.c_int), ("bucket_bytes", C.c_int), ("attn_legacy", C.c_int), ("adam_interleave", C.c_int), ("head_dx_splitk", C.c_int),
        ("gemm_nsub", C.c_int), ("timeout_s", C.c_double), ("device", C.c_int), ("sched_profile", C.c_int),
    ]


class Status(C.Structure):
    _fields_ = [("code", C.c_int), ("dev_code", C.c_int), ("phase", C.c_int), ("task", C.c_int), ("block", C.c_int), ("aux", C.c_int)]


class LiveT(C.Structure):
    _fields_ = [("steps", C.c_uint), ("loss", C.c_float), ("decode_steps", C.c_uint)]


class Phase(C.Structure):
    _fields_ = [
        ("kind", C.c_int), ("layout", C.c_int), ("epi", C.c_int), ("accumulate", C.c_int),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("lda", C.c_int), ("ldb", C.c_int), ("ldc", C.c_int), ("ldaux", C.c_int), ("nsub", C.c_int),
        ("p", C.c_void_p * 10), ("n", C.c_size_t), ("i0", C.c_int), ("i1", C.c_int), ("i2", C.c_int),
    ]


class Dims(C.Structure):
    _fields_ = [("vocab", C.c_int), ("d_model", C.c_int), ("n_layer", C.c_int), ("n_head", C.c_int), ("ctx_len", C.c_int), ("batch", C.c_int)]


# every symbol include/ofa_b200.h declares: name -> (restype, argtypes)
PROTOTYPES = {
    "ofa_default_config": (C.c_int, [C.POINTER(Config), C.c_char_p]),
    "ofa_create": (C.c_int, [C.POINTER(Config), C.POINTER(C.c_void_p)]),
    "ofa_destroy": (None, [C.c_void_p]),
    "ofa_last_error": (C.c_char_p, [C.c_void_p]),
    "ofa_num_params": (C.c_size_t, [C.c_void_p]),
    "ofa_param_span": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "ofa_load_weights": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_read_weights": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_read_grads": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_read_adam_m": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_read_adam_v": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_load_adam_state": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]),
    "ofa_set_tokens": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_set_starts": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_launch": (C.c_int, [C.c_void_p, C.c_int]),
    "ofa_wait": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(Status)]),
    "ofa_abort": (C.c_int, [C.c_void_p]),
    "ofa_steps_done": (C.c_int, [C.c_void_p]),
    "ofa_last_launch_ms": (C.c_float, [C.c_void_p]),
    "ofa_live": (C.c_int, [C.c_void_p, C.POINTER(LiveT)]),
    "ofa_read_losses": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_read_step_times": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_num_phases": (C.c_int, [C.c_void_p]),
    "ofa_phase_window": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong)]),
    "ofa_phase_wait_ns": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_ulonglong)]),
    "ofa_phase_info": (C.c_int, [C.c_void_p, C.c_int, C.c_char_p, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_ulonglong)]),
    "ofa_read_block_busy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_read_decode_trace": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_read_block_info": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_decode_phase_info": (C.c_int, [C.c_void_p, C.c_int, C.c_char_p, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.c_ulonglong)]),
    "ofa_phase_deps": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int]),
    "ofa_phase_dep_grain": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int]),
    "ofa_decode_steps": (C.c_int, [C.c_void_p]),
    "ofa_read_decode_tokens": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_read_decode_logits": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_read_buffer": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t]),
    "ofa_num_buckets": (C.c_int, [C.c_void_p]),
    "ofa_bucket_span": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "ofa_grad_buffer": (C.c_void_p, [C.c_void_p]),
    "ofa_ext_ready_flags": (C.c_void_p, [C.c_void_p]),
    "ofa_ext_done_flags": (C.c_void_p, [C.c_void_p]),
    "ofa_dp_unique_id": (C.c_int, [C.c_void_p]),
    "ofa_dp_init": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "ofa_dp_enqueue": (C.c_int, [C.c_void_p, C.c_int]),
    "ofa_dp_cancel": (C.c_int, [C.c_void_p]),
    "ofa_dp_finish": (C.c_int, [C.c_void_p, C.c_int]),
    "ofa_dp_wait": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(Status)]),
    "ofa_dp_shutdown": (None, [C.c_void_p]),
    "ofa_dev_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "ofa_dev_free": (C.c_int, [C.c_void_p]),
    "ofa_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ofa_ln_bwd_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "ofa_noalloc_max_rows": (C.c_int, []),
    "ofa_noalloc_last_error": (C.c_char_p, []),
    "ofa_debug_set_task_shuffle": (None, [C.c_uint]),
    "ofa_run_phases": (C.c_int, [C.c_int, C.POINTER(Dims), C.POINTER(Phase), C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(Status)]),
}

OK, TIMEOUT, DEVICE_ABORT, CUDA_ERROR, BAD_CONFIG, BAD_ARGUMENT, NOT_LAUNCHED = range(7)
DTYPE_BF16, DTYPE_F32 = 0, 1
MODE_TRAIN, MODE_FORWARD, MODE_NO_OPT, MODE_DECODE_ONLY = 0, 1, 2, 3
(TK_DATA, TK_EMBED, TK_LN_FWD, TK_GEMM, TK_ATT_FWD, TK_ATT_PREP, TK_ATT_BWD, TK_CE, TK_CE_MEAN, TK_LN_BWD, TK_LN_DG, TK_EMB_WTE,
 TK_EMB_WPE, TK_ADAMW, TK_BARRIER) = range(15)
GEMM_NN, GEMM_NT, GEMM_TN = 0, 1, 2
EPI_STORE, EPI_RES, EPI_GELU, EPI_DGELU, EPI_F32, EPI_DR, EPI_LSE = range(7)
OUT_RESTART = 1 << 24
OUT_FORCED = OUT_RESTART + 1


def lib_path():
    return _build.LIB


def load():
    """Load csrc/libofa_b200.so (building it first if nvcc is present and it is missing or stale) and bind every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("OFA_B200_LIB")        # a prebuilt library elsewhere (a host application's own build, an A/B variant)
    if not path:
        if not os.path.exists(_build.LIB) or _build.needs_build():
            _build.build()
        path = _build.LIB
    lib = C.CDLL(path)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)      # AttributeError = the library does not export what the header declares
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
