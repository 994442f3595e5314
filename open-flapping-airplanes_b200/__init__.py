"""B200-native persistent megakernel (GPT training + live-weight decode) behind the C ABI of include/ofa_b200.h.

The directory name contains a hyphen, so import it with importlib.import_module("open-flapping-airplanes_b200")
(tests/conftest.py and bench.py do exactly that and call the result `ofa`).
"""
from . import build as build_mod
from . import capi
from . import dp
from . import files
from .host import Megakernel, OfaError, default_config, flat_from_named, PARAM_ORDER_DOC
from .tasks import DeviceBuffer, run_phases, gemm_phase, phase, bf16_round, to_bf16_bits, from_bf16_bits

build = build_mod.build

__all__ = ["build", "capi", "dp", "Megakernel", "OfaError", "default_config", "flat_from_named", "DeviceBuffer", "run_phases",
           "gemm_phase", "phase", "bf16_round", "to_bf16_bits", "from_bf16_bits", "PARAM_ORDER_DOC"]
