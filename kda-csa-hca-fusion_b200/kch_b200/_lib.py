"""ctypes binding of libkch_b200.so (the C ABI declared in include/kch_b200.h).

PyTorch is used only for device memory and streams: tensors are passed as raw device pointers.
There is no CPU fallback: a missing library or a CPU tensor raises.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

KCH_F32, KCH_BF16, KCH_FP8_E4M3, KCH_INT8 = 0, 1, 2, 3
ACT_SILU, ACT_SIGMOID, ACT_NEG_SOFTPLUS, ACT_SILU_L2NORM = 1, 2, 3, 4

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkch_b200.so")

_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float


class AttendArgs(C.Structure):
    _fields_ = [("q", _vp), ("q_dtype", _i), ("q_ld", _i64), ("q_normalize", _i),
                ("B", _i), ("T", _i), ("nh", _i), ("c", _i),
                ("comp", _vp), ("comp_dtype", _i), ("comp_ld", _i64), ("comp_batch_rows", _i64), ("n_comp", _i),
                ("comp_norms", _vp), ("comp_scales", _vp),
                ("sel_indices", _vp), ("topk", _i), ("m", _i), ("t0", _i64), ("n_visible", _i),
                ("win", _vp), ("win_dtype", _i), ("win_ld", _i64), ("win_batch_rows", _i64),
                ("sliding_window", _i), ("win_mode", _i), ("win_len", _i),
                ("sink", _vp), ("sink_dtype", _i), ("scale", _f), ("out", _vp), ("out_dtype", _i), ("win_t0", _i)]


class Epilogue(C.Structure):
    _fields_ = [("n_segments", _i), ("seg_end", _i * 8), ("seg_act", _i * 8), ("seg_param", _f * 8), ("group", _i)]


class CacheAppendArgs(C.Structure):
    _fields_ = [("B", _i), ("c", _i), ("c_I", _i), ("m", _i), ("win", _i), ("dtype", _i),
                ("Ca", _vp), ("Cb", _vp), ("Za", _vp), ("Zb", _vp), ("K_idx", _vp), ("Z_idx", _vp),
                ("ld_c", _i64), ("ld_i", _i64),
                ("acc_Ca", _vp), ("acc_Cb", _vp), ("acc_Za", _vp), ("acc_Zb", _vp), ("acc_K_idx", _vp), ("acc_Z_idx", _vp),
                ("acc_len", _i), ("prev_Cb", _vp), ("prev_Zb", _vp), ("has_prev", _i),
                ("Ba", _vp), ("Bb", _vp), ("B_idx", _vp),
                ("comp", _vp), ("comp_kind", _i), ("comp_scales", _vp), ("comp_norms", _vp),
                ("kcomp", _vp), ("kcomp_norms", _vp), ("capacity", _i64), ("n_blocks", _i),
                ("ring", _vp), ("ring_pos", _i), ("normalize", _i), ("counters", _vp)]


class AttendDecodeArgs(C.Structure):
    _fields_ = [("q", _vp), ("q_dtype", _i), ("q_ld", _i64), ("q_normalize", _i),
                ("B", _i), ("nh", _i), ("c", _i),
                ("comp", _vp), ("comp_dtype", _i), ("capacity", _i64), ("comp_norms", _vp), ("comp_scales", _vp),
                ("sel_indices", _vp), ("topk", _i), ("m", _i),
                ("win", _vp), ("win_dtype", _i), ("sliding_window", _i),
                ("sink", _vp), ("sink_dtype", _i), ("scale", _f),
                ("out", _vp), ("out_dtype", _i),
                ("counters", _vp), ("workspace", _vp), ("workspace_bytes", _i64)]


# indices into a cache's device counters (include/kch_b200.h KCH_CTR_*)
CTR_ACC_LEN, CTR_N_BLOCKS, CTR_RING_N, CTR_HAS_PREV, CTR_TOKENS, CTR_ARRIVALS, CTR_WORDS = 0, 1, 2, 3, 4, 5, 8
STATUS_CACHE_CAPACITY = 64
STATUS_SELFTEST_WAIT = 0x5E1F
STATUS_PEER_GATHER = 0x9A7E


# name -> (restype, argtypes); must list every symbol declared in include/kch_b200.h
PROTOTYPES = {
    "kch_abi_version": (_i, []),
    "kch_last_error": (C.c_char_p, []),
    "kch_device_status": (C.c_uint, [_i]),
    "kch_launch_count": (C.c_longlong, [_i]),
    "kch_selftest_bounded_wait": (_i, [C.c_uint, _vp, _vp]),
    "kch_layernorm": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _f, _i, _i, _vp]),
    "kch_short_conv": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "kch_linear": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _i64, _i64, _i64, _i64, _i, _vp]),
    "kch_linear_ex": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _i64, _i64, _i64, _i64, _i, C.POINTER(Epilogue), _vp]),
    "kch_linear_kslabs": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i64, _i64, _i64, _i, _vp]),
    "kch_peer_gather_flag_words": (_i64, [_i]),
    "kch_peer_allgather": (_i, [_vp, _i64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _i, _i, _vp]),
    "kch_activation": (_i, [_vp, _vp, _i64, _i, _i, _f, _i, _i, _i64, _i64, _vp]),
    "kch_rownorm": (_i, [_vp, _i64, _vp, _vp, _i64, _i, _i, _i, _vp]),
    "kch_kda_recurrent": (_i, [_vp] * 8 + [_i] * 6 + [_f, _f, _i, _i64, _i64, _i64, _i64, _vp]),
    "kch_kda_chunk_workspace_bytes": (_i64, [_i] * 6),
    "kch_kda_chunk": (_i, [_vp] * 8 + [_i] * 7 + [_f, _f, _i, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    "kch_kda_chunk_gate_supported": (_i, [_i, _i, _i, _f, _i]),
    "kch_kda_chunk_gate": (_i, [_vp] * 8 + [_i] * 7 + [_f, _f, _f, _i, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    "kch_compress_kv": (_i, [_vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i64, _i64, _i64, _i, _i, _vp]),
    "kch_compress_kv_overlapped": (_i, [_vp] * 8 + [_i64, _vp, _i, _i64, _i, _i, _i64, _i64, _i64, _i, _i, _vp]),
    "kch_indexer_workspace_bytes": (_i64, [_i, _i, _i, _i, _i]),
    "kch_indexer_topk": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i64, _i, _i, _i64, _vp, _i64, _vp]),
    "kch_indexer_workspace_bytes_ex": (_i64, [_i, _i, _i, _i]),
    "kch_indexer_topk_ex": (_i, [_vp, _i, _i64, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i64, _i, _i, _i64, _vp,
                                 _i64, _vp]),
    "kch_indexer_topk_static_capacity": (_i64, []),
    "kch_indexer_topk_static": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i64, _i, _i64, _vp]),
    "kch_attend": (_i, [C.POINTER(AttendArgs), _vp]),
    "kch_cache_append_token": (_i, [C.POINTER(CacheAppendArgs), _vp]),
    "kch_cache_append_token_advance": (_i, [C.POINTER(CacheAppendArgs), _vp]),
    "kch_quantize_rows": (_i, [_vp, _i64, _vp, _vp, _vp, _i64, _i, _i, _i, _vp]),
    "kch_cache_advance": (_i, [_vp, _i, _vp]),
    "kch_decode_indexer_workspace_bytes": (_i64, [_i, _i64]),
    "kch_decode_indexer_topk": (_i, [_vp, _i, _i64, _vp, _i, _vp, _vp, _i, _i64, _vp, _i, _i64, _i, _i, _i, _i, _f, _i, _vp,
                                     _vp, _i64, _vp]),
    "kch_short_conv_step": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "kch_layernorm_short_conv": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "kch_layernorm_short_conv_step": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "kch_attend_decode_splits": (_i, [_i]),
    "kch_attend_decode_workspace_bytes": (_i64, [_i, _i, _i]),
    "kch_attend_decode": (_i, [C.POINTER(AttendDecodeArgs), _vp]),
}

_lib = None


def load():
    """Load the shared library (once).  Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"kch_b200: {LIB_PATH} is missing - build it with `python kda-csa-hca-fusion_b200/build.py`; "
            "there is no fallback path")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(rc: int):
    if rc == 0:
        return
    msg = load().kch_last_error().decode("utf-8", "replace")
    if rc < 0:
        raise ValueError(msg)
    raise RuntimeError(f"kch_b200: {msg}")


def dtype_tag(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return KCH_F32
    if dt == torch.bfloat16:
        return KCH_BF16
    raise TypeError(f"kch_b200 kernels take float32 or bfloat16 tensors, got {dt}")


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def require_cuda(*tensors, fn="kch_b200"):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(f"{fn}: backend 'b200' requires CUDA tensors (got a {t.device} tensor); "
                               "there is no CPU fallback")


def device_status(reset=False) -> int:
    return int(load().kch_device_status(1 if reset else 0))


def raise_on_device_status(where: str) -> None:
    """Synchronise the current device and raise if a bounded device-side wait has expired since the last check.

    The status word is sticky on purpose: after one wait gives up, every later wait returns at its first poll, so
    kernels drain instead of spinning, but they also leave their outputs unwritten.  Callers that keep a process
    alive across requests should call this (or `device_status(reset=True)`) at their own synchronisation points;
    the package does so in `HostPipeline.run` and `HybridDecoding.export_state`."""
    import torch
    torch.cuda.synchronize()
    st = device_status(reset=True)
    if st:
        raise RuntimeError(f"kch_b200 ({where}): a device-side bounded wait expired (status 0x{st:x}); results since "
                           f"the previous check are not valid.  The status word has been cleared.")

