"""KDA operators on the B200 kernels, with the reference signatures.

Mirrors ``naive_recurrent_kda`` (ops_kda.py:175-267), ``naive_chunk_kda`` (ops_kda.py:464-494) and the
backend dispatcher ``kda_forward`` (ops_kda_backend.py:158-251) of 183600/kda-csa-hca-fusion: same
argument names, same validation messages and exception types, same return contract (output in
``v.dtype``, state in fp32 unless ``state_dtype``).
"""
from __future__ import annotations

import math
import warnings

import torch

from . import _lib

_VALID_BACKENDS = {"b200"}


def _validate_inputs(q, k, v, g, beta, fn_name):
    # shape / device / dtype contract of ops_kda.py:28-83
    for name, t, rank in (("q", q, 4), ("k", k, 4), ("v", v, 4), ("g", g, 4), ("beta", beta, 3)):
        if t.dim() != rank:
            expect = ("[B, T, H, K]" if name in ("q", "k") else "[B, T, HV, V]" if name == "v"
                      else "[B, T, HV, K]" if name == "g" else "[B, T, HV]")
            raise ValueError(f"{fn_name}: {name} must have rank {rank} but got rank {t.dim()} "
                             f"(shape={tuple(t.shape)}). Expected shape: {expect}")
    B, T = q.shape[0], q.shape[1]
    for name, t in (("k", k), ("v", v), ("g", g), ("beta", beta)):
        if t.shape[0] != B or t.shape[1] != T:
            raise ValueError(f"{fn_name}: {name}.shape[0:2]={tuple(t.shape[0:2])} does not match "
                             f"q.shape[0:2]=({B}, {T}). All inputs must share the same batch (B) and "
                             f"sequence (T) dimensions.")
    for name, t in (("k", k), ("v", v), ("g", g), ("beta", beta)):
        if t.device != q.device:
            raise ValueError(f"{fn_name}: {name}.device={t.device} does not match q.device={q.device}. "
                             f"All inputs must be on the same device.")
    for name, t in (("k", k), ("v", v), ("g", g), ("beta", beta)):
        if t.dtype != q.dtype:
            raise ValueError(f"{fn_name}: {name}.dtype={t.dtype} does not match q.dtype={q.dtype}. "
                             f"All inputs must share the same dtype (cast before calling if needed).")


def _validate_shapes(q, k, v, g, beta, fn_name, chunk_size=None):
    # ops_kda.py:86-125
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[-1]
    if H < 1:
        raise ValueError(f"{fn_name}: H={H} must be >= 1 (would cause ZeroDivisionError in HV // H)")
    if K < 1:
        raise ValueError(f"{fn_name}: K={K} must be >= 1")
    if V < 1:
        raise ValueError(f"{fn_name}: V={V} must be >= 1")
    if chunk_size is not None and chunk_size < 1:
        raise ValueError(f"{fn_name}: chunk_size={chunk_size} must be >= 1")
    if HV % H != 0:
        raise ValueError(f"{fn_name}: HV={HV} must be divisible by H={H} (GVA factor)")
    if g.shape[2] != HV:
        raise ValueError(f"{fn_name}: g.shape[2]={g.shape[2]} must equal HV={HV} "
                         f"(g must be [B, T, HV, K], got {tuple(g.shape)})")
    if g.shape[-1] != K:
        raise ValueError(f"{fn_name}: g.shape[-1]={g.shape[-1]} must equal K={K} "
                         f"(g must be [B, T, HV, K], got {tuple(g.shape)})")
    if beta.shape[2] != HV:
        raise ValueError(f"{fn_name}: beta.shape[2]={beta.shape[2]} must equal HV={HV} "
                         f"(beta must be [B, T, HV], got {tuple(beta.shape)})")


def _token_stride(x):
    """``(tensor, elements between consecutive tokens)`` for a ``[B,T,H,K]`` / ``[B,T,HV]`` operand whose heads are
    dense within a token (e.g. a column slice of a fused projection); anything else is made contiguous."""
    inner = 1
    ok = True
    for d in range(x.dim() - 1, 1, -1):
        ok = ok and (x.shape[d] == 1 or x.stride(d) == inner)
        inner *= x.shape[d]
    B, T = x.shape[0], x.shape[1]
    if ok and T > 0 and B > 0:
        # one token per sequence: the token stride is whatever separates the batch entries
        ld = x.stride(1) if T > 1 else (x.stride(0) if B > 1 else inner)
        if ld >= inner and (B == 1 or x.stride(0) == T * ld) and ld % 8 == 0 and x.data_ptr() % 16 == 0:
            return x, ld
    x = x.contiguous()
    return x, inner


def _scale_value(scale, K):
    if scale is None:
        return K ** -0.5
    if isinstance(scale, torch.Tensor):
        return float(scale)          # the hybrid layer passes its 0-dim `scale` buffer (ops_fused.py:602)
    return float(scale)


def _run(fn_name, q, k, v, g, beta, scale, initial_state, output_final_state, g_clamp_min, state_dtype,
         chunk_size, state_out=None, gate_scale=None):
    _validate_inputs(q, k, v, g, beta, fn_name)
    _validate_shapes(q, k, v, g, beta, fn_name, chunk_size)
    _lib.require_cuda(q, fn=fn_name)
    lib = _lib.load()
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[-1]
    tag = _lib.dtype_tag(v.dtype)
    (q, ld_q), (k, ld_k), (v, ld_v), (g, ld_g), (beta, ld_b) = (_token_stride(x) for x in (q, k, v, g, beta))
    if ld_q != ld_k:
        q, k = q.contiguous(), k.contiguous()
        ld_q = ld_k = H * K
    S0 = None
    if initial_state is not None:
        S0 = initial_state.to(device=q.device, dtype=torch.float32).contiguous()
        if tuple(S0.shape) != (B, HV, K, V):
            raise ValueError(f"{fn_name}: initial_state.shape={tuple(S0.shape)} must be (B, HV, K, V)="
                             f"({B}, {HV}, {K}, {V})")
    o = torch.empty(B, T, HV, V, dtype=v.dtype, device=q.device)
    S = None
    if output_final_state:
        if state_out is not None:
            # caller-owned fp32 state buffer; may be the same memory as `initial_state` (decode updates in place)
            if (state_out.dtype != torch.float32 or tuple(state_out.shape) != (B, HV, K, V)
                    or not state_out.is_contiguous() or state_out.device != q.device):
                raise ValueError(f"{fn_name}: state_out must be a contiguous fp32 ({B}, {HV}, {K}, {V}) tensor on "
                                 f"{q.device}")
            S = state_out
        else:
            S = torch.empty(B, HV, K, V, dtype=torch.float32, device=q.device)
    gmin = float(g_clamp_min) if g_clamp_min > -math.inf else -math.inf
    sc = _scale_value(scale, K)
    with torch.cuda.device(q.device):
        if chunk_size is None:
            _lib.check(lib.kch_kda_recurrent(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g), _lib.ptr(beta),
                                             _lib.ptr(S0), _lib.ptr(o), _lib.ptr(S), B, T, H, HV, K, V, sc, gmin,
                                             tag, ld_q, ld_v, ld_g, ld_b, _lib.stream()))
        else:
            nbytes = lib.kch_kda_chunk_workspace_bytes(B, T, HV, K, V, int(chunk_size))
            ws = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=q.device)
            if gate_scale is not None:
                _lib.check(lib.kch_kda_chunk_gate(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g), _lib.ptr(beta),
                                                  _lib.ptr(S0), _lib.ptr(o), _lib.ptr(S), B, T, H, HV, K, V,
                                                  int(chunk_size), sc, gmin, float(gate_scale), tag, ld_q, ld_v, ld_g,
                                                  ld_b, _lib.ptr(ws), int(nbytes), _lib.stream()))
            else:
                _lib.check(lib.kch_kda_chunk(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g), _lib.ptr(beta),
                                             _lib.ptr(S0), _lib.ptr(o), _lib.ptr(S), B, T, H, HV, K, V, int(chunk_size),
                                             sc, gmin, tag, ld_q, ld_v, ld_g, ld_b, _lib.ptr(ws), int(nbytes),
                                             _lib.stream()))
    if S is not None and state_dtype is not None:
        S = S.to(state_dtype)
    return o, S


def naive_recurrent_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, *,
                        g_clamp_min: float = -10.0, state_dtype=None, state_out=None):
    """Token-by-token KDA.  q,k ``[B,T,H,K]``; v ``[B,T,HV,V]``; g ``[B,T,HV,K]``; beta ``[B,T,HV]``;
    ``initial_state [B,HV,K,V]``.  Returns ``(o [B,T,HV,V] in v.dtype, final state or None)``.
    ``state_out`` (not in the reference) names an fp32 buffer to receive the final state; it may be the
    ``initial_state`` tensor itself, which makes a decode step update its state in place."""
    return _run("naive_recurrent_kda", q, k, v, g, beta, scale, initial_state, output_final_state,
                g_clamp_min, state_dtype, None, state_out)


def chunk_gate_supported(K, V, chunk_size, g_clamp_min, dtype):
    """Can ``naive_chunk_kda`` take the gate's pre-activation (``_gate_scale``) for this geometry?"""
    if dtype != torch.bfloat16:
        return False
    gmin = float(g_clamp_min) if g_clamp_min > -math.inf else -math.inf
    return bool(_lib.load().kch_kda_chunk_gate_supported(int(K), int(V), int(chunk_size), gmin, _lib.KCH_BF16))


def naive_chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                    chunk_size: int = 64, *, g_clamp_min: float = -10.0, state_dtype=None, _gate_scale=None):
    """Chunk-parallel KDA; equals :func:`naive_recurrent_kda` up to fp32 round-off.  Chunks larger
    than 64 tokens (or than K) are processed as smaller chunks: the same mathematics in a different
    summation order.  ``_gate_scale`` (not in the reference): ``g`` is the pre-activation of the layer's gate and
    the kernel applies ``-softplus(g) * _gate_scale`` itself (see :func:`chunk_gate_supported`)."""
    return _run("naive_chunk_kda", q, k, v, g, beta, scale, initial_state, output_final_state,
                g_clamp_min, state_dtype, int(chunk_size), gate_scale=_gate_scale)


def validate_kda_backend(backend: str) -> str:
    if backend not in _VALID_BACKENDS:
        raise ValueError(f"kda_backend={backend!r} must be one of {sorted(_VALID_BACKENDS)}.")
    return backend


def kda_forward(q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False,
                chunk_size: int = 64, use_chunk: bool = False, g_clamp_min: float = -10.0,
                backend: str = "b200", state_out=None, gate_scale=None):
    """Dispatcher with the keyword contract of ``ops_kda_backend.kda_forward``; only ``backend='b200'``
    exists here (no Triton, no FLA, no CPU path)."""
    validate_kda_backend(backend)
    if not isinstance(g_clamp_min, (int, float)) or isinstance(g_clamp_min, bool):
        raise TypeError(f"g_clamp_min must be a real number, got {g_clamp_min!r}")
    if math.isnan(float(g_clamp_min)):
        raise ValueError("g_clamp_min must not be NaN")
    if not q.is_cuda:
        raise RuntimeError("KDA backend 'b200' requires CUDA tensors; use kda_backend='reference' "
                           "for CPU experiments.")
    if use_chunk:
        return naive_chunk_kda(q, k, v, g, beta, scale=scale, initial_state=initial_state,
                               output_final_state=output_final_state, chunk_size=chunk_size,
                               g_clamp_min=g_clamp_min, _gate_scale=gate_scale)
    if gate_scale is not None:
        raise ValueError("kda_forward: gate_scale is only meaningful with use_chunk=True")
    return naive_recurrent_kda(q, k, v, g, beta, scale=scale, initial_state=initial_state,
                               output_final_state=output_final_state, g_clamp_min=g_clamp_min, state_out=state_out)


def warn_if_nonfinite(o, fn_name):
    """Same advisory as ops_kda.py:151-172 (a device->host sync; the operators do not call it)."""
    if not torch.isfinite(o).all():
        warnings.warn(f"{fn_name}: output contains NaN/Inf; q/k must be L2-normalised and g_clamp_min "
                      f"must not be disabled.", stacklevel=2)
