"""The hybrid KDA / CSA / HCA stack on the B200 kernels.

Mirrors ``HybridConfig`` (ops_fused.py:65-313), ``KDAHybridLayer`` (316-609), ``CSAHybridLayer``
(612-713), ``HCAHybridLayer`` (716-739), ``HybridKCHAttention`` (742-1131) and the decode wiring
``HybridDecoding`` (run_decoding.py:601-851) of 183600/kda-csa-hca-fusion.  Parameter names are the
reference's ``state_dict`` names, so a reference checkpoint loads unchanged.  Forward only.

Every projection of a layer that reads the same input runs as ONE GEMM over row-concatenated weights
(the reference already does this for the six CSA projections, ops_csa.py:841-850); each output column
is the same dot product as in the separate call, so values do not change.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from . import _lib
from .csa import attend, fuse_rows, indexer_topk, linear, mma_attention_eligible, naive_csa, rownorm
from .decoding_cache import CSADecodingCache, HCADecodingCache
from .hca import naive_hca
from .kda import chunk_gate_supported, kda_forward, validate_kda_backend
from .tp import gather_heads, out_projection, out_projection_rows, row_span  # noqa: F401


@dataclass
class HybridConfig:
    d_model: int = 256
    n_heads_qk: int = 4
    n_heads_v: int = 4
    head_dim_k: int = 64
    head_dim_v: int = 64
    kda_chunk_size: int = 64
    kda_backend: str = "b200"
    csa_m: int = 16
    csa_topk: int = 8
    csa_nh: int = 4
    csa_c: int = 64
    csa_dc: int = 128
    csa_nIh: int = 2
    csa_cI: int = 32
    csa_sliding_window: int = 16
    hca_m2: int = 64
    hca_nh: int = 4
    hca_c: int = 64
    hca_dc: int = 128
    hca_sliding_window: int = 16
    n_kda: int = 3
    n_csa: int = 1
    n_hca: int = 1
    kda_decay_scale: float = 0.1
    init_std: float = 0.02
    dropout: float = 0.0

    def __post_init__(self):
        if not isinstance(self.dropout, (int, float)) or isinstance(self.dropout, bool):
            raise TypeError(f"HybridConfig.dropout={self.dropout!r} must be a float, "
                            f"got {type(self.dropout).__name__}.")
        if math.isnan(self.dropout) or math.isinf(self.dropout) or not 0.0 <= self.dropout <= 1.0:
            raise ValueError(f"HybridConfig.dropout={self.dropout!r} must be a finite value in [0, 1].")
        if self.dropout != 0.0:
            raise NotImplementedError("HybridConfig.dropout != 0 is a training option; this is a forward path")
        validate_kda_backend(self.kda_backend)
        for name in ("n_heads_qk", "n_heads_v"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v < 1:
                raise ValueError(f"{name}={v!r} must be a positive int")
        if self.n_heads_v % self.n_heads_qk != 0:
            raise ValueError(f"n_heads_v={self.n_heads_v} must be divisible by n_heads_qk={self.n_heads_qk} "
                             f"(KDA GVA factor G = HV // H must be an integer).")
        for name in ("d_model", "head_dim_k", "head_dim_v", "csa_m", "csa_c", "csa_dc", "csa_cI", "csa_nIh",
                     "hca_m2", "hca_c", "hca_dc", "csa_nh", "hca_nh"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool):
                raise ValueError(f"HybridConfig.{name}={v!r} must be a positive int.")
            if v < 1:
                raise ValueError(f"HybridConfig.{name}={v} must be >= 1.")
        if not isinstance(self.kda_chunk_size, int):
            raise ValueError(f"HybridConfig.kda_chunk_size={self.kda_chunk_size!r} must be an int")
        for name in ("n_kda", "n_csa", "n_hca", "csa_topk", "csa_sliding_window", "hca_sliding_window"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool):
                raise ValueError(f"HybridConfig.{name}={v!r} must be a non-negative int.")
            if v < 0:
                raise ValueError(f"HybridConfig.{name}={v} must be >= 0.")
        if self.n_kda + self.n_csa + self.n_hca == 0:
            raise ValueError("HybridConfig: at least one of n_kda, n_csa, n_hca must be non-zero")
        if not isinstance(self.kda_decay_scale, (int, float)) or not math.isfinite(self.kda_decay_scale) \
                or self.kda_decay_scale < 0:
            raise ValueError(f"HybridConfig.kda_decay_scale={self.kda_decay_scale!r} must be a finite value >= 0")


def layernorm(x, weight, bias, eps=1e-5):
    """LayerNorm in fp32, output in ``x.dtype`` (``_Fp32LayerNorm``, ops_fused.py:42-60)."""
    lib = _lib.load()
    _lib.require_cuda(x, fn="layernorm")
    x = x.contiguous()
    d = x.shape[-1]
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(lib.kch_layernorm(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(y), x.numel() // d, d,
                                     float(eps), _lib.dtype_tag(x.dtype), _lib.dtype_tag(weight.dtype),
                                     _lib.stream()))
    return y


def short_conv(x, weight, bias, lookback=None):
    """Causal depthwise kernel-3 conv over time; x ``[B,T,d]``, weight ``[d,1,3]``, lookback ``[B,2,d]``."""
    lib = _lib.load()
    B, T, d = x.shape
    x = x.contiguous()
    w = weight.reshape(d, 3).to(x.dtype).contiguous()
    b = bias.to(x.dtype).contiguous()
    lb = None if lookback is None else lookback.to(x.dtype).contiguous()
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(lib.kch_short_conv(_lib.ptr(x), _lib.ptr(lb), _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), B, T, d,
                                      _lib.dtype_tag(x.dtype), _lib.stream()))
    return y


def layernorm_short_conv_ok(x, lookback):
    B, T, d = x.shape
    return (x.is_cuda and x.dtype == torch.bfloat16 and T >= 2 and d % 256 == 0 and d <= 2048
            and (lookback is None or (lookback.dtype == x.dtype and tuple(lookback.shape) == (B, 2, d))))


def layernorm_short_conv(x, ln_weight, ln_bias, eps, weight, bias, lookback=None):
    """``short_conv(layernorm(x))`` in one pass; returns ``(y, last two normalised rows [B,2,d])``."""
    lib = _lib.load()
    B, T, d = x.shape
    x = x.contiguous()
    w = weight.reshape(d, 3).to(x.dtype).contiguous()
    b = bias.to(x.dtype).contiguous()
    lb = None if lookback is None else lookback.contiguous()
    lw, lbias = ln_weight.contiguous(), ln_bias.contiguous()
    y = torch.empty_like(x)
    new_lb = torch.empty(B, 2, d, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.kch_layernorm_short_conv(_lib.ptr(x), _lib.ptr(lw), _lib.ptr(lbias), float(eps), _lib.ptr(lb),
                                                _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), _lib.ptr(new_lb), B, T, d,
                                                _lib.dtype_tag(x.dtype), _lib.dtype_tag(lw.dtype), _lib.stream()))
    return y, new_lb


def short_conv_step(x, weight, bias, lookback):
    """One-token conv step: x ``[B,1,d]``; ``lookback [B,2,d]`` (same dtype, contiguous) slides by one token in place."""
    lib = _lib.load()
    B, T, d = x.shape
    if T != 1 or lookback.dtype != x.dtype or not lookback.is_contiguous() or tuple(lookback.shape) != (B, 2, d):
        raise ValueError("short_conv_step: needs x [B,1,d] and a contiguous lookback [B,2,d] of the same dtype")
    x = x.contiguous()
    w = weight.reshape(d, 3).to(x.dtype).contiguous()
    b = bias.to(x.dtype).contiguous()
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(lib.kch_short_conv_step(_lib.ptr(x), _lib.ptr(lookback), _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), B, d,
                                           _lib.dtype_tag(x.dtype), _lib.stream()))
    return y


def layernorm_short_conv_step_ok(x, lookback):
    B, T, d = x.shape
    return (x.is_cuda and T == 1 and x.dtype == torch.bfloat16 and d % 256 == 0 and d <= 2048
            and lookback is not None and lookback.dtype == x.dtype and lookback.is_contiguous()
            and tuple(lookback.shape) == (B, 2, d))


def layernorm_short_conv_step(x, ln_weight, ln_bias, eps, weight, bias, lookback):
    """``short_conv_step(layernorm(x))`` in one launch; ``lookback`` (normalised rows) slides in place."""
    lib = _lib.load()
    B, T, d = x.shape
    x = x.contiguous()
    w = weight.reshape(d, 3).to(x.dtype).contiguous()
    b = bias.to(x.dtype).contiguous()
    lw, lbias = ln_weight.contiguous(), ln_bias.contiguous()
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(lib.kch_layernorm_short_conv_step(_lib.ptr(x), _lib.ptr(lw), _lib.ptr(lbias), float(eps),
                                                     _lib.ptr(lookback), _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), B, d,
                                                     _lib.dtype_tag(x.dtype), _lib.dtype_tag(lw.dtype), _lib.stream()))
    return y


def activation(x, act, *, param=0.0, group=1):
    """Activation with the reference's rounding points on a ``[..., cols]`` view (row-strided ok)."""
    lib = _lib.load()
    cols = x.shape[-1]
    lead = x.shape[:-1]
    x2 = x.reshape(-1, cols) if x.is_contiguous() else x
    if x2.dim() == 3:
        # [B,T,cols] slice of a wider contiguous [B,T,W]: rows are uniformly W apart
        if x2.stride(-1) == 1 and (x2.shape[0] == 1 or x2.stride(0) == x2.shape[1] * x2.stride(1)):
            rows, ldx = x2.shape[0] * x2.shape[1], x2.stride(1)
        else:
            x2 = x2.contiguous().reshape(-1, cols)
            rows, ldx = x2.shape[0], cols
    else:
        if x2.dim() != 2:
            x2 = x2.contiguous().reshape(-1, cols)
        rows, ldx = x2.shape[0], (x2.stride(0) if x2.shape[0] > 1 else cols)
    y = torch.empty(rows, cols, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.kch_activation(_lib.ptr(x2), _lib.ptr(y), rows, cols, act, float(param), int(group),
                                      _lib.dtype_tag(x.dtype), ldx, cols, _lib.stream()))
    return y.reshape(*lead, cols)


class _FusedWeights:
    """Row-concatenated copy of several weight matrices, rebuilt when the sources move or change dtype."""

    def __init__(self):
        self._key = None
        self._w = None

    def get(self, *weights):
        key = tuple((w.data_ptr(), w.dtype, w.device, w._version) for w in weights)
        if key != self._key:
            self._w = fuse_rows(*weights)
            self._key = key
        return self._w


class KDAHybridLayer(nn.Module):
    """KDA sub-layer: short conv, projections + activations, the delta-rule operator, ``o_proj``."""

    def __init__(self, cfg: HybridConfig):
        super().__init__()
        self.cfg = cfg
        d, H, K, V = cfg.d_model, cfg.n_heads_qk, cfg.head_dim_k, cfg.head_dim_v
        self.q_proj = nn.Linear(d, H * K, bias=False)
        self.k_proj = nn.Linear(d, H * K, bias=False)
        self.v_proj = nn.Linear(d, cfg.n_heads_v * V, bias=False)
        self.g_down = nn.Linear(d, K, bias=False)
        self.g_up = nn.Linear(K, cfg.n_heads_v * K, bias=False)
        self.beta = nn.Linear(d, cfg.n_heads_v, bias=False)
        self.o_proj = nn.Linear(cfg.n_heads_v * V, d, bias=False)
        self.short_conv = nn.Conv1d(d, d, kernel_size=3, padding=0, groups=d, bias=True)
        self.register_buffer("scale", torch.tensor(K ** -0.5), persistent=False)
        self._conv_lookback = None
        self._fused = _FusedWeights()
        self._scale_cache = None
        self.tp = None              # TPContext when heads are sharded across GPUs

    def _scale_value(self):
        """The `scale` buffer as a Python float, read from the device once per dtype / device (the buffer is
        cast with the module, so the value is the one the reference passes, ops_fused.py:602)."""
        key = (self.scale.dtype, self.scale.device)
        if self._scale_cache is None or self._scale_cache[0] != key:
            self._scale_cache = (key, float(self.scale))
        return self._scale_cache[1]

    def reset_conv_state(self):
        self._conv_lookback = None

    def forward(self, x, state=None, residual=None, state_out=None, lookback_in_place=False, norm=None):
        o, new_state, lb = self.forward_functional(x, state, self._conv_lookback, residual=residual,
                                                   state_out=state_out, lookback_in_place=lookback_in_place, norm=norm)
        self._conv_lookback = lb
        return o, new_state

    def project(self, x, conv_lookback, lookback_in_place=False, norm=None, raw_gate=False):
        """conv + fused projection + activations -> (q, k, v, g, beta, new_lookback).  With
        ``lookback_in_place`` a one-token call slides ``conv_lookback`` where it lies and returns it.
        ``norm``: the sub-layer's pre-norm when ``x`` is the un-normalised residual stream; LayerNorm and the
        convolution then run as one kernel where the shape allows."""
        cfg = self.cfg
        B, T, d = x.shape
        H, HV, K, V = cfg.n_heads_qk, cfg.n_heads_v, cfg.head_dim_k, cfg.head_dim_v
        lb = conv_lookback
        if lb is not None and lb.shape[0] != B:
            lb = None
        fused_norm = norm is not None and layernorm_short_conv_ok(x, lb)
        fused_step = (norm is not None and not fused_norm and lookback_in_place
                      and layernorm_short_conv_step_ok(x, lb) and norm.weight.dtype == norm.bias.dtype)
        if norm is not None and not (fused_norm or fused_step):
            x = norm(x)
        if fused_step:
            xc = layernorm_short_conv_step(x, norm.weight, norm.bias, norm.eps, self.short_conv.weight,
                                           self.short_conv.bias, lb)
            new_lb = lb
        elif fused_norm:
            xc, new_lb = layernorm_short_conv(x, norm.weight, norm.bias, norm.eps, self.short_conv.weight,
                                              self.short_conv.bias, lb)
        elif (lookback_in_place and T == 1 and lb is not None and lb.dtype == x.dtype and lb.is_contiguous()
                and tuple(lb.shape) == (B, 2, d)):
            xc = short_conv_step(x, self.short_conv.weight, self.short_conv.bias, lb)
            new_lb = lb
        else:
            xc = short_conv(x, self.short_conv.weight, self.short_conv.bias, lb)
            if T >= 2:
                new_lb = x[:, -2:].clone()
            else:
                prev = lb if lb is not None else x.new_zeros(B, 2, d)
                new_lb = torch.cat([prev.to(x.dtype), x], dim=1)[:, -2:].clone()
        W = self._fused.get(self.q_proj.weight, self.k_proj.weight, self.v_proj.weight, self.g_down.weight,
                            self.beta.weight)
        # one GEMM for q|k|v|g_down|beta with the activations of ops_fused.py:571-581 applied in its epilogue
        # (silu + per-head L2 norm, silu, none, sigmoid); q, k, v, beta stay column slices of its output
        n_used = 2 * H * K + HV * V + K + HV
        segs = [(H * K, _lib.ACT_SILU_L2NORM, 0.0), (H * K, _lib.ACT_SILU_L2NORM, 0.0), (HV * V, _lib.ACT_SILU, 0.0),
                (K, 0, 0.0), (HV + (W.shape[0] - n_used), _lib.ACT_SIGMOID, 0.0)]
        proj = linear(xc, W, epilogue=segs, group=K)
        q, k, v, gd, beta = proj[..., :n_used].split([H * K, H * K, HV * V, K, HV], dim=-1)
        if raw_gate:     # the chunk kernel applies -softplus(.) * decay_scale when it loads the gate
            g = linear(gd, self.g_up.weight)
        else:
            g = linear(gd, self.g_up.weight, epilogue=[(HV * K, _lib.ACT_NEG_SOFTPLUS, cfg.kda_decay_scale)])
        return (q.unflatten(-1, (H, K)), k.unflatten(-1, (H, K)), v.unflatten(-1, (HV, V)),
                g.view(B, T, HV, K), beta, new_lb)

    def forward_functional(self, x, state, conv_lookback, *, detach_lookback=True, residual=None, state_out=None,
                           lookback_in_place=False, norm=None):
        cfg = self.cfg
        B, T, _ = x.shape
        HV, V = cfg.n_heads_v, cfg.head_dim_v
        use_chunk = cfg.kda_chunk_size >= 1 and T >= cfg.kda_chunk_size
        raw_gate = use_chunk and cfg.kda_decay_scale > 0 and chunk_gate_supported(
            cfg.head_dim_k, cfg.head_dim_v, cfg.kda_chunk_size, -10.0, x.dtype)
        q, k, v, g, beta, new_lb = self.project(x, conv_lookback, lookback_in_place, norm, raw_gate)
        o, new_state = kda_forward(q, k, v, g, beta, scale=self._scale_value(), initial_state=state,
                                   output_final_state=True, chunk_size=cfg.kda_chunk_size, use_chunk=use_chunk,
                                   backend=cfg.kda_backend, state_out=None if use_chunk else state_out,
                                   gate_scale=cfg.kda_decay_scale if raw_gate else None)
        out = out_projection(o.reshape(B, T, HV * V), self.tp, self.o_proj.weight, residual=residual)
        return out, new_state, new_lb


def _rows_mode(tp):
    return tp is not None and tp.world > 1 and tp.attn_shard == "rows"


def _forward_by_rows(layer, x, residual):
    """CSA / HCA sub-layer with its QUERY ROWS sharded: this rank runs the operator for its contiguous run of the
    flattened ``[B*T]`` rows (whole sequences, or a slice of one sequence against that sequence's prefix), the runs
    are all-gathered along the row axis and ``o_proj`` (+ residual) follows on every rank."""
    B, T, _ = x.shape
    r0, per = row_span(B * T, layer.tp)
    if per % T == 0:
        b0 = r0 // T
        o = layer.core(x[b0:b0 + per // T])
    elif T % per == 0:
        b, lo = r0 // T, r0 % T
        o = layer.core(x[b:b + 1], q_rows=(lo, lo + per))
    else:
        raise ValueError(f"tensor parallelism by rows: {B} x {T} rows do not split over {layer.tp.world} ranks into "
                         f"whole sequences or equal slices of a sequence")
    return out_projection_rows(o, layer.tp, layer.o_proj.weight, residual, lead=(B, T))


class CSAHybridLayer(nn.Module):
    """CSA sub-layer (compression + lightning indexer + sparse MQA + window + sink) and ``o_proj``."""

    def __init__(self, cfg: HybridConfig):
        super().__init__()
        self.cfg = cfg
        d, c = cfg.d_model, cfg.csa_c
        self.W_aKV = nn.Linear(d, c, bias=False)
        self.W_bKV = nn.Linear(d, c, bias=False)
        self.W_aZ = nn.Linear(d, c, bias=False)
        self.W_bZ = nn.Linear(d, c, bias=False)
        self.Ba = nn.Parameter(torch.randn(cfg.csa_m, c) * cfg.init_std)
        self.Bb = nn.Parameter(torch.randn(cfg.csa_m, c) * cfg.init_std)
        self.W_DQ = nn.Linear(d, cfg.csa_dc, bias=False)
        self.W_UQ = nn.Linear(cfg.csa_dc, c * cfg.csa_nh, bias=False)
        self.W_IUQ = nn.Linear(cfg.csa_dc, cfg.csa_cI * cfg.csa_nIh, bias=False)
        self.W_w = nn.Linear(d, cfg.csa_nIh, bias=False)
        self.W_KV_idx = nn.Linear(d, cfg.csa_cI, bias=False)
        self.W_Z_idx = nn.Linear(d, cfg.csa_cI, bias=False)
        self.B_idx = nn.Parameter(torch.randn(cfg.csa_m, cfg.csa_cI) * cfg.init_std)
        self.sink = nn.Parameter(torch.zeros(cfg.csa_nh))
        self.o_proj = nn.Linear(c * cfg.csa_nh, d, bias=False)
        self.use_ste = True
        self.tp = None
        self._fused = _FusedWeights()
        self._fused_q = _FusedWeights()

    def q_weight(self):
        return self._fused_q.get(self.W_UQ.weight, self.W_IUQ.weight)

    def fused_weight(self):
        return self._fused.get(self.W_aKV.weight, self.W_bKV.weight, self.W_aZ.weight, self.W_bZ.weight,
                               self.W_KV_idx.weight, self.W_Z_idx.weight, self.W_DQ.weight, self.W_w.weight)

    def core(self, x, *, return_projections=False, q_rows=None):
        cfg = self.cfg
        return naive_csa(x, self.W_aKV.weight, self.W_bKV.weight, self.W_aZ.weight, self.W_bZ.weight, self.Ba,
                         self.Bb, self.W_DQ.weight, self.W_UQ.weight, self.W_IUQ.weight, self.W_w.weight,
                         self.W_KV_idx.weight, self.W_Z_idx.weight, self.B_idx, m=cfg.csa_m, topk=cfg.csa_topk,
                         nh=cfg.csa_nh, nIh=cfg.csa_nIh, c=cfg.csa_c, c_I=cfg.csa_cI, dc=cfg.csa_dc,
                         sliding_window=cfg.csa_sliding_window, sink_logits=self.sink, use_ste=False,
                         normalize_qk=True, return_projections=return_projections,
                         _fused_weight=self.fused_weight(), _fused_q_weight=self.q_weight(), _q_rows=q_rows)

    def forward(self, x, state=None, residual=None):
        if _rows_mode(self.tp):
            return _forward_by_rows(self, x, residual), None
        return out_projection(self.core(x), self.tp, self.o_proj.weight, residual=residual), None


class HCAHybridLayer(nn.Module):
    """HCA sub-layer (heavy compression + dense MQA + window + sink) and ``o_proj``."""

    def __init__(self, cfg: HybridConfig):
        super().__init__()
        self.cfg = cfg
        d, c = cfg.d_model, cfg.hca_c
        self.W_KV = nn.Linear(d, c, bias=False)
        self.W_Z = nn.Linear(d, c, bias=False)
        self.B_pos = nn.Parameter(torch.randn(cfg.hca_m2, c) * cfg.init_std)
        self.W_DQ = nn.Linear(d, cfg.hca_dc, bias=False)
        self.W_UQ = nn.Linear(cfg.hca_dc, c * cfg.hca_nh, bias=False)
        self.sink = nn.Parameter(torch.zeros(cfg.hca_nh))
        self.o_proj = nn.Linear(c * cfg.hca_nh, d, bias=False)
        self.tp = None
        self._fused = _FusedWeights()

    def fused_weight(self):
        return self._fused.get(self.W_KV.weight, self.W_Z.weight, self.W_DQ.weight)

    def core(self, x, *, return_projections=False, q_rows=None):
        cfg = self.cfg
        return naive_hca(x, self.W_KV.weight, self.W_Z.weight, self.B_pos, self.W_DQ.weight, self.W_UQ.weight,
                         m2=cfg.hca_m2, nh=cfg.hca_nh, c=cfg.hca_c, dc=cfg.hca_dc,
                         sliding_window=cfg.hca_sliding_window, sink_logits=self.sink,
                         return_projections=return_projections, _fused_weight=self.fused_weight(), _q_rows=q_rows)

    def forward(self, x, state=None, residual=None):
        if _rows_mode(self.tp):
            return _forward_by_rows(self, x, residual), None
        return out_projection(self.core(x), self.tp, self.o_proj.weight, residual=residual), None


class _Fp32LayerNorm(nn.LayerNorm):
    def forward(self, x):
        return layernorm(x, self.weight, self.bias, self.eps)


class HybridKCHAttention(nn.Module):
    """Pre-norm residual stack of KDA / CSA / HCA sub-layers in the repeating ``[KDA*n_kda, CSA*n_csa,
    HCA*n_hca]`` order: ``x = x + layer(LayerNorm(x))``."""

    LAYER_TYPES = ("kda", "csa", "hca")

    def __init__(self, cfg: HybridConfig, total_layers: int = 5):
        super().__init__()
        self.cfg = cfg
        if not isinstance(total_layers, int) or total_layers < 0:
            raise ValueError(f"total_layers={total_layers!r} must be a non-negative int")
        self.total_layers = total_layers
        self.layout = self._build_layout()
        make = {"kda": KDAHybridLayer, "csa": CSAHybridLayer, "hca": HCAHybridLayer}
        self.layers = nn.ModuleList([make[k](cfg) for k in self.layout])
        self.norms = nn.ModuleList([_Fp32LayerNorm(cfg.d_model) for _ in self.layout])
        self.n_kda_layers = sum(1 for k in self.layout if k == "kda")
        self._kda_state = None

    def _build_layout(self):
        unit = ["kda"] * self.cfg.n_kda + ["csa"] * self.cfg.n_csa + ["hca"] * self.cfg.n_hca
        layout = []
        while len(layout) < self.total_layers:
            layout.extend(unit)
        return layout[:self.total_layers]

    def layout_str(self):
        return "-".join(s.upper() for s in self.layout)

    def reset_state(self):
        self._kda_state = None
        for layer in self.layers:
            if isinstance(layer, KDAHybridLayer):
                layer.reset_conv_state()

    @torch.no_grad()
    def forward(self, x):
        kda_layers = [l for l in self.layers if isinstance(l, KDAHybridLayer)]
        o, new_state, new_lbs = self.forward_functional(x, self._kda_state, [l._conv_lookback for l in kda_layers])
        self._kda_state = new_state
        for layer, lb in zip(kda_layers, new_lbs):
            layer._conv_lookback = lb
        return o

    @torch.no_grad()
    def forward_functional(self, x, kda_state, conv_lookbacks, *, detach_state=True, detach_lookback=True):
        """``(x [B,T,d], stacked KDA state [n_kda,B,HV,K,V] | None, lookbacks) -> (y, new state, new lookbacks)``."""
        stacked = kda_state
        if stacked is not None and stacked.shape[1] != x.shape[0]:
            stacked = None
        if stacked is not None:
            if stacked.shape[0] != self.n_kda_layers:
                raise ValueError(f"HybridKCHAttention.forward_functional: stacked KDA state has {stacked.shape[0]} "
                                 f"layers but the model has {self.n_kda_layers} KDA layers.")
            states = list(stacked.to(x.device).unbind(0))
        else:
            states = [None] * self.n_kda_layers
        lookbacks = list(conv_lookbacks)
        if len(lookbacks) != self.n_kda_layers:
            raise ValueError(f"HybridKCHAttention.forward_functional: conv_lookbacks has length {len(lookbacks)} "
                             f"but the model has {self.n_kda_layers} KDA layers.")
        ki = 0
        new_lbs = []
        for layer, norm, kind in zip(self.layers, self.norms, self.layout):
            if kind == "kda":
                # the pre-norm goes into the layer: LayerNorm + short conv are one kernel there
                x, st, lb = layer.forward_functional(x, states[ki], lookbacks[ki], residual=x, norm=norm)
                states[ki] = st
                new_lbs.append(lb)
                ki += 1
            else:
                x, _ = layer(norm(x), None, residual=x)
        new_state = torch.stack(states, dim=0) if self.n_kda_layers > 0 else None
        return x, new_state, new_lbs


class HybridDecoding(nn.Module):
    """Decode-time wiring of the stack: a multi-token call runs the full-sequence operators and fills the
    per-layer caches from the same projections (a later multi-token call continues the sequence: chunked
    prefill); a one-token call appends to the caches and attends through them; KDA layers carry their
    recurrent state and conv lookback."""

    def __init__(self, cfg: HybridConfig | None = None, total_layers: int = 5, *, model=None, kv_quant=None,
                 reserve_tokens: int = 0, use_cuda_graph: bool = False):
        super().__init__()
        if model is None:
            model = HybridKCHAttention(cfg, total_layers)
        self.model = model
        self.cfg = model.cfg
        self.kv_quant = kv_quant
        self.reserve_tokens = reserve_tokens
        # one-token steps are replayed from a captured CUDA graph once a first step has run eagerly; every
        # per-token quantity the kernels need is on the device (cache counters), so the launch arguments are static
        self.use_cuda_graph = use_cuda_graph
        # with heads sharded over several GPUs the per-layer all-gather (NCCL) is captured with the step; every
        # rank captures and replays the same sequence of collectives
        self.graph_collectives = True
        self._caches = {}
        self._graph = None
        self._eager_token_steps = 0

    def reset(self):
        self.model.reset_state()
        self._caches = {}
        self._graph = None

    def export_state(self):
        """The whole decode session as a dict: stacked KDA state, conv lookbacks and every layer cache
        (``CSADecodingCache.export_state`` / ``HCADecodingCache.export_state``).  Tensors stay on their device;
        move them with ``torch.save`` / ``.cpu()`` as needed."""
        model = self.model
        dev = next(model.parameters()).device
        if dev.type == "cuda":
            with torch.cuda.device(dev):
                _lib.raise_on_device_status("HybridDecoding.export_state")      # never checkpoint a broken session
        return {
            "layout": list(model.layout),
            "kda_state": None if model._kda_state is None else model._kda_state.clone(),
            "conv_lookbacks": [None if l._conv_lookback is None else l._conv_lookback.clone()
                               for l in model.layers if isinstance(l, KDAHybridLayer)],
            "caches": {i: c.export_state() for i, c in self._caches.items()},
        }

    def import_state(self, st):
        model, cfg = self.model, self.cfg
        if list(st["layout"]) != list(model.layout):
            raise ValueError(f"HybridDecoding.import_state: layout {st['layout']} does not match {list(model.layout)}")
        self.reset()
        dev = next(model.parameters()).device
        if st["kda_state"] is not None:
            model._kda_state = st["kda_state"].to(dev).clone()
        kda_layers = [l for l in model.layers if isinstance(l, KDAHybridLayer)]
        for layer, lb in zip(kda_layers, st["conv_lookbacks"]):
            layer._conv_lookback = None if lb is None else lb.to(dev).clone()
        for i, cst in st["caches"].items():
            layer = model.layers[i]
            dtype = getattr(torch, cst["dtype"].split(".")[-1])
            if isinstance(layer, CSAHybridLayer):
                cache = CSADecodingCache(cst["B"], cfg.csa_c, cfg.csa_cI, cfg.csa_m, cfg.csa_sliding_window, dev, dtype,
                                         kv_quant=cst["kv_quant"])
            else:
                cache = HCADecodingCache(cst["B"], cfg.hca_c, cfg.hca_m2, cfg.hca_sliding_window, dev, dtype,
                                         kv_quant=cst["kv_quant"])
            cache.import_state(cst)
            self._caches[i] = cache
        self.kv_quant = next((c["kv_quant"] for c in st["caches"].values()), self.kv_quant)

    def _cache(self, i, layer, h):
        cfg, B = self.cfg, h.shape[0]
        cache = self._caches.get(i)
        if cache is None or cache.B != B or cache.device != h.device or cache.dtype != h.dtype:
            if isinstance(layer, CSAHybridLayer):
                cache = CSADecodingCache(B, cfg.csa_c, cfg.csa_cI, cfg.csa_m, cfg.csa_sliding_window, h.device, h.dtype,
                                         kv_quant=self.kv_quant)
                if self.reserve_tokens:
                    cache.reserve(self.reserve_tokens // cfg.csa_m + 1)
            else:
                cache = HCADecodingCache(B, cfg.hca_c, cfg.hca_m2, cfg.hca_sliding_window, h.device, h.dtype,
                                         kv_quant=self.kv_quant)
                if self.reserve_tokens:
                    cache.reserve(self.reserve_tokens // cfg.hca_m2 + 1)
            self._caches[i] = cache
        return cache

    # ---- a later chunk of a sequence (multi-token call on caches that already hold tokens) -----------------------
    # Not in the reference, whose caches only attend one token at a time (ops_decoding_cache.py:831-836).  The
    # chunk's rows are appended first, then its queries run through the full-sequence kernels against everything
    # the cache holds: visibility n < (t0 + t + 1) // m with t0 = tokens before the chunk, window keys = the tail
    # of the ring followed by the chunk's own keys.  Same values as feeding the chunk token by token.
    @staticmethod
    def _ring_tail(cache, win):
        if cache._sw is None or win <= 1 or cache._sw.n_valid == 0:
            return None
        # a copy: while the ring is not full `get()` is a view of its storage, and the append that follows the
        # call overwrites slots of that storage when the chunk wraps around
        return cache._sw.get()[:, -(win - 1):].clone()

    def _csa_chunk(self, layer, cache, h):
        cfg = self.cfg
        B, T, _ = h.shape
        c, cI, dc, nIh, nh, m, win = (cfg.csa_c, cfg.csa_cI, cfg.csa_dc, cfg.csa_nIh, cfg.csa_nh, cfg.csa_m,
                                      cfg.csa_sliding_window)
        t0 = cache.n_tokens_seen
        proj = linear(h, layer.fused_weight())
        Ca, Cb, Za, Zb, K_idx, Z_idx, cQ, w_idx = proj[..., :4 * c + 2 * cI + dc + nIh].split(
            [c, c, c, c, cI, cI, dc, nIh], dim=-1)
        qq = linear(cQ, layer.q_weight())
        q, q_idx = qq[..., :nh * c + nIh * cI].split([nh * c, nIh * cI], dim=-1)
        prev = self._ring_tail(cache, win)
        cache.append_step(Ca, Cb, Za, Zb, K_idx, Z_idx, layer.Ba, layer.Bb, layer.B_idx)
        nb = cache.n_blocks
        indices = None
        if cfg.csa_topk > 0 and nb > 0:
            kn = (cache._kcomp[:, :nb].float() / cache._kcomp_norms[:, :nb].unsqueeze(-1)).contiguous()
            indices = indexer_topk(q_idx.unflatten(-1, (nIh, cI)), kn, w_idx, cfg.csa_topk, m=m, t0=t0,
                                   normalize_qk=True, sorted_output=False, k_prenormalized=True)
        kdt = torch.bfloat16 if mma_attention_eligible(h.dtype, c, nh, True, 1.0) else torch.float32
        comp_n = rownorm(cache.C_comp, True, kdt) if (cfg.csa_topk > 0 and nb > 0) else None
        local, P = None, 0
        if win > 0:
            local = rownorm(Ca, True, kdt)
            if prev is not None:
                P = prev.shape[1]
                local = torch.cat([prev.to(kdt), local], dim=1)
        return attend(q, comp_n, nh=nh, c=c, sel=indices, m=m, t0=t0, q_normalize=True, win=local, sliding_window=win,
                      sink=layer.sink, scale=1.0, out_dtype=h.dtype, win_t0=P)

    def _hca_chunk(self, layer, cache, h):
        cfg = self.cfg
        c, dc, nh, m2, win = cfg.hca_c, cfg.hca_dc, cfg.hca_nh, cfg.hca_m2, cfg.hca_sliding_window
        t0 = cache.n_tokens_seen
        proj = linear(h, layer.fused_weight())
        C, Z, cQ = proj[..., :2 * c + dc].split([c, c, dc], dim=-1)
        q = linear(cQ, layer.W_UQ.weight)
        prev = self._ring_tail(cache, win)
        cache.append_step(C, Z, layer.B_pos)
        nb = cache.n_blocks
        kdt = torch.bfloat16 if mma_attention_eligible(h.dtype, c, nh, True, 1.0) else torch.float32
        comp_n = rownorm(cache.C_comp, True, kdt) if nb > 0 else None
        local, P = None, 0
        if win > 0:
            local = rownorm(C, True, kdt)
            if prev is not None:
                P = prev.shape[1]
                local = torch.cat([prev.to(kdt), local], dim=1)
        return attend(q, comp_n, nh=nh, c=c, sel=None, m=m2, t0=t0, q_normalize=True, win=local, sliding_window=win,
                      sink=layer.sink, scale=1.0, out_dtype=h.dtype, win_t0=P)

    def _local_rows(self, layer, h):
        """Rows mode of the head-sharded stack: this rank's sequences of the batch (the caches of a CSA / HCA layer
        then hold those sequences only)."""
        if not _rows_mode(layer.tp):
            return h
        B = h.shape[0]
        if B % layer.tp.world != 0:
            raise ValueError(f"decode with CSA / HCA sharded by rows needs the batch ({B}) to divide over "
                             f"{layer.tp.world} ranks: a sequence's cache lives on one rank")
        per = B // layer.tp.world
        return h[layer.tp.rank * per:(layer.tp.rank + 1) * per]

    def _project_out(self, layer, o_core, residual, B, T):
        if _rows_mode(layer.tp):
            return out_projection_rows(o_core, layer.tp, layer.o_proj.weight, residual, lead=(B, T))
        return out_projection(o_core, layer.tp, layer.o_proj.weight, residual=residual)

    def _csa(self, i, layer, h, residual):
        cfg = self.cfg
        B_all = h.shape[0]
        h = self._local_rows(layer, h)
        B, T, _ = h.shape
        cache = self._cache(i, layer, h)
        if T > 1 and cache.n_tokens_seen > 0:
            o_core = self._csa_chunk(layer, cache, h)
        elif T > 1:
            o_core, proj = layer.core(h, return_projections=True)
            cache.append_step(*proj, layer.Ba, layer.Bb, layer.B_idx)
        else:
            c, cI, dc, nIh, nh = cfg.csa_c, cfg.csa_cI, cfg.csa_dc, cfg.csa_nIh, cfg.csa_nh
            proj = linear(h, layer.fused_weight())
            Ca, Cb, Za, Zb, K_idx, Z_idx, cQ, w_idx = proj[..., :4 * c + 2 * cI + dc + nIh].split(
                [c, c, c, c, cI, cI, dc, nIh], dim=-1)
            qq = linear(cQ, layer.q_weight())
            q, q_idx = qq[..., :nh * c + nIh * cI].split([nh * c, nIh * cI], dim=-1)
            cache.append_step(Ca, Cb, Za, Zb, K_idx, Z_idx, layer.Ba, layer.Bb, layer.B_idx)
            if cache._decode_attend_ok(nh):
                # the decode kernels read the projection slices where they lie, normalise the query themselves
                # and write the layer dtype: the same arithmetic as the chain below without its glue launches
                o = cache.forward_step(q.unflatten(-1, (nh, c)), q_idx.unflatten(-1, (nIh, cI)), w_idx, topk=cfg.csa_topk,
                                       nh=nh, nIh=nIh, scale=1.0, sink_logits=layer.sink, use_ste=False,
                                       normalize_qk=True, _q_normalize=True, _out_dtype=h.dtype)
                o_core = o.reshape(B, 1, nh * c)
            else:
                qn = rownorm(q.contiguous().view(B, 1, nh, c), True)
                o = cache.forward_step(qn, q_idx.contiguous().view(B, 1, nIh, cI).float(), w_idx.float(),
                                       topk=cfg.csa_topk, nh=nh, nIh=nIh, scale=1.0, sink_logits=layer.sink,
                                       use_ste=False, normalize_qk=True)
                o_core = o.reshape(B, 1, nh * c).to(h.dtype)
        return self._project_out(layer, o_core, residual, B_all, T)

    def _hca(self, i, layer, h, residual):
        cfg = self.cfg
        B_all = h.shape[0]
        h = self._local_rows(layer, h)
        B, T, _ = h.shape
        cache = self._cache(i, layer, h)
        if T > 1 and cache.n_tokens_seen > 0:
            o_core = self._hca_chunk(layer, cache, h)
        elif T > 1:
            o_core, (C, Z) = layer.core(h, return_projections=True)
            cache.append_step(C, Z, layer.B_pos)
        else:
            c, dc, nh = cfg.hca_c, cfg.hca_dc, cfg.hca_nh
            proj = linear(h, layer.fused_weight())
            C, Z, cQ = proj[..., :2 * c + dc].split([c, c, dc], dim=-1)
            q = linear(cQ, layer.W_UQ.weight)
            cache.append_step(C, Z, layer.B_pos)
            if cache._decode_attend_ok(nh):
                o = cache.forward_step(q.view(B, 1, nh, c), nh=nh, scale=1.0, sink_logits=layer.sink, _q_normalize=True,
                                       _out_dtype=h.dtype)
                o_core = o.reshape(B, 1, nh * c)
            else:
                qn = rownorm(q.view(B, 1, nh, c), True)
                o = cache.forward_step(qn, nh=nh, scale=1.0, sink_logits=layer.sink)
                o_core = o.reshape(B, 1, nh * c).to(h.dtype)
        return self._project_out(layer, o_core, residual, B_all, T)

    # ---- CUDA-graph replay of one-token steps ------------------------------------------------------------------
    def _graph_signature(self, x):
        """What a captured step depends on besides the data: the addresses of every state tensor it updates in
        place.  None when a step cannot be replayed (no state yet, or a geometry served by host-counter kernels)."""
        model, cfg = self.model, self.cfg
        st = model._kda_state
        if model.n_kda_layers and (st is None or st.shape[1] != x.shape[0] or st.dtype != torch.float32
                                   or not st.is_contiguous() or cfg.kda_chunk_size == 1):
            return None
        sig = [x.shape[0], x.dtype, 0 if st is None else st.data_ptr()]
        for i, (layer, kind) in enumerate(zip(model.layers, model.layout)):
            if layer.tp is not None and layer.tp.world > 1 and not self.graph_collectives:
                return None                                    # the head all-gather is launched eagerly
            if kind == "kda":
                lb = layer._conv_lookback
                if lb is None or lb.shape[0] != x.shape[0] or lb.dtype != x.dtype:
                    return None
                sig.append(lb.data_ptr())
                continue
            cache = self._caches.get(i)
            nh = cfg.csa_nh if kind == "csa" else cfg.hca_nh
            b_local = x.shape[0] // layer.tp.world if _rows_mode(layer.tp) else x.shape[0]
            if cache is None or cache.B != b_local or cache._comp is None or not cache._decode_attend_ok(nh):
                return None
            if kind == "csa" and (cfg.csa_nIh > 64 or cfg.csa_nIh * cfg.csa_cI > 1024 or cfg.csa_topk < 1):
                return None
            if cache._n_blocks + 1 > cache._comp.shape[1]:
                cache.reserve(2 * cache._comp.shape[1])        # grow outside the graph; forces a re-capture
            sig.extend([cache._comp.data_ptr(), cache._ctr.data_ptr(), cache._n_blocks >= 0])
        return tuple(sig)

    def _host_counters(self):
        return [(c._acc_len, c._n_blocks, c._n_tokens_seen, getattr(c, "_has_prev", None),
                 None if c._sw is None else c._sw._n) for c in self._caches.values()]

    def _restore_host_counters(self, saved):
        for c, (acc, nb, nt, hp, rn) in zip(self._caches.values(), saved):
            c._acc_len, c._n_blocks, c._n_tokens_seen = acc, nb, nt
            if hp is not None:
                c._has_prev = hp
            if rn is not None:
                c._sw._n = rn

    def _graph_step(self, x, sig):
        if self._graph is None or self._graph[0] != sig:
            # capture records the launches without running them: the host counters the Python path advanced
            # are put back, the device state is untouched, and the first replay below performs the step
            x_static = x.clone()
            saved = self._host_counters()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                y_static = self._forward_eager(x_static)
            self._restore_host_counters(saved)
            self._graph = (sig, graph, x_static, y_static)
        _, graph, x_static, y_static = self._graph
        x_static.copy_(x)
        graph.replay()
        for i, cache in self._caches.items():
            cache._advance(cache.m if hasattr(cache, "m") else cache.m2)
        return y_static.clone()

    @torch.no_grad()
    def forward(self, x):
        B, T, _ = x.shape
        if T == 1 and self.use_cuda_graph and self._eager_token_steps >= 1:
            sig = self._graph_signature(x)
            if sig is not None:
                return self._graph_step(x, sig)
        if T == 1:
            self._eager_token_steps += 1       # every kernel of the step is loaded before a capture is attempted
        return self._forward_eager(x)

    @torch.no_grad()
    def _forward_eager(self, x):
        model = self.model
        B, T, _ = x.shape
        stacked = model._kda_state
        if stacked is not None and stacked.shape[1] == B:
            states = list(stacked.unbind(0))
        else:
            states = [None] * model.n_kda_layers
            stacked = None
        # a one-token step on an existing fp32 state updates it where it lies (no copy of the 3 x B x HV x K x V state)
        in_place = (T == 1 and stacked is not None and stacked.dtype == torch.float32 and stacked.is_contiguous()
                    and stacked.device == x.device and model.cfg.kda_chunk_size != 1)
        ki = 0
        for i, (layer, norm, kind) in enumerate(zip(model.layers, model.norms, model.layout)):
            if T == 0:
                continue
            if kind == "kda":
                # in place: the state and the conv lookback keep their addresses from token to token
                x, st = layer(x, states[ki], residual=x, state_out=states[ki] if in_place else None,
                              lookback_in_place=in_place, norm=norm)
                states[ki] = st
                ki += 1
            elif kind == "csa":
                x = self._csa(i, layer, norm(x), x)
            else:
                x = self._hca(i, layer, norm(x), x)
        if T > 0 and not in_place:
            model._kda_state = torch.stack(states, dim=0) if model.n_kda_layers > 0 else None
        return x
