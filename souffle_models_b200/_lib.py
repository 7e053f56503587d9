"""ctypes binding of libsouffle_b200.so (the C ABI declared in include/souffle_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

STATUS_NAMES = {0: "OK", 1: "BAD_SHAPE", 2: "BAD_POINTER", 3: "BAD_DEVICE", 4: "NOT_CORESIDENT",
                5: "CUDA_ERROR", 6: "DEVICE_TIMEOUT", 7: "BAD_ARGUMENT"}


class SouffleError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"souffle_b200 error {code} ({STATUS_NAMES.get(code, '?')}): {message}")
        self.code = code


class BertDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "seq", "heads", "head_dim", "ffn", "n_layers", "variant",
                                         "keep_probs")] + [("eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("bn_qkv", "bn_fc1", "bn_proj", "split_proj", "bn_fc2", "split_fc2",
                                         "max_ctas", "timeout_ms", "profile", "bm_qkv", "bm_fc1", "bm_proj",
                                         "bm_fc2", "debug_max_slots", "debug_skip_arrival", "autotune", "pair_mma")]


class BertLayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("qkv_w", "qkv_b", "proj_w", "proj_b", "ln1_g", "ln1_b", "fc1_w",
                                          "fc1_b", "fc2_w", "fc2_b", "ln2_g", "ln2_b")]


class SwinDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "res", "dim", "heads", "window", "shift", "mlp_ratio")] + \
               [("eps", C.c_float), ("timeout_ms", C.c_int32), ("n_blocks", C.c_int32), ("shift_alt", C.c_int32)]


class SwinMerge(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("norm_g", "norm_b", "reduction_w")]


class SwinWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("ln1_g", "ln1_b", "qkv_w", "qkv_b", "rel_bias", "proj_w", "proj_b", "ln2_g",
                                          "ln2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b")]


class LstmDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("layers", "hidden", "steps", "ref_input_delay", "timeout_ms")]


# name -> (restype, argtypes); must list every symbol include/souffle_b200.h declares
SIGNATURES = {
    "souffle_last_error": (C.c_char_p, []),
    "souffle_abi_version": (C.c_int, []),
    "souffle_bert_plan_create": (C.c_int, [C.POINTER(BertDesc), C.POINTER(BertLayerWeights), C.POINTER(C.c_void_p)]),
    "souffle_bert_plan_destroy": (C.c_int, [C.c_void_p]),
    "souffle_bert_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "souffle_bert_forward_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "souffle_bert_forward_host_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "souffle_bert_plan_buffer": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]),
    "souffle_bert_plan_copy_buffer": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]),
    "souffle_bert_plan_status": (C.c_int, [C.c_void_p]),
    "souffle_bert_plan_read_profile": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "souffle_bert_plan_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "souffle_bert_plan_uses_pairs": (C.c_int, [C.c_void_p]),
    "souffle_bert_packed_weights": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(BertLayerWeights),
                                              C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]),
    "souffle_bert_plan_stage_info": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int)]),
    "souffle_lstm_plan_create": (C.c_int, [C.POINTER(LstmDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "souffle_lstm_plan_destroy": (C.c_int, [C.c_void_p]),
    "souffle_lstm_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "souffle_lstm_plan_status": (C.c_int, [C.c_void_p]),
    "souffle_lstm_launch_mode": (C.c_int, []),
    "souffle_lstm_forward_static": (C.c_int, [C.POINTER(LstmDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p]),
    "souffle_lstm_static_status": (C.c_int, [C.c_void_p]),
    "souffle_workspace_forget": (C.c_int, [C.c_void_p]),
    "souffle_gemm_workspace_bytes": (C.c_size_t, []),
    "souffle_gemm_f16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                   C.c_void_p, C.c_size_t, C.c_void_p]),
    "souffle_swin_mlp_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "souffle_swin_mlp_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                           C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p]),
    "souffle_layernorm_forward": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_void_p, C.c_int32, C.c_int32, C.c_float, C.c_void_p, C.c_size_t,
                                            C.c_void_p]),
    "souffle_swin_block_plan_create": (C.c_int, [C.POINTER(SwinDesc), C.POINTER(SwinWeights), C.POINTER(C.c_void_p)]),
    "souffle_swin_stage_plan_create": (C.c_int, [C.POINTER(SwinDesc), C.POINTER(SwinWeights), C.POINTER(SwinMerge),
                                                 C.POINTER(C.c_void_p)]),
    "souffle_swin_block_plan_destroy": (C.c_int, [C.c_void_p]),
    "souffle_swin_block_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "souffle_swin_block_plan_status": (C.c_int, [C.c_void_p]),
    "souffle_se_module_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "souffle_se_module_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                            C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p]),
    "souffle_workspace_status": (C.c_int, [C.c_void_p, C.c_void_p]),
}

_lib = None


def lib_path() -> str:
    return os.environ.get("SOUFFLE_B200_LIB", _build.LIB_PATH)


def load() -> C.CDLL:
    """Loads the library (building it in-tree first if the sources are newer)."""
    global _lib
    if _lib is None:
        path = lib_path()
        if path == _build.LIB_PATH and _build.is_stale():
            _build.build()
        if not os.path.exists(path):
            raise SouffleError(3, f"native library not found at {path}; run python -m souffle_models_b200.build")
        lib = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise SouffleError(code, load().souffle_last_error().decode())
