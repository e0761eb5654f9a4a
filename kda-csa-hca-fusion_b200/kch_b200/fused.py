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
from .csa import attend, fuse_rows, linear, naive_csa, rownorm
from .decoding_cache import CSADecodingCache, HCADecodingCache
from .hca import naive_hca
from .kda import kda_forward, validate_kda_backend
from .tp import gather_heads


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
        self.tp = None              # TPContext when heads are sharded across GPUs

    def reset_conv_state(self):
        self._conv_lookback = None

    def forward(self, x, state=None, residual=None):
        o, new_state, lb = self.forward_functional(x, state, self._conv_lookback, residual=residual)
        self._conv_lookback = lb
        return o, new_state

    def project(self, x, conv_lookback):
        """conv + fused projection + activations -> (q, k, v, g, beta, new_lookback)."""
        cfg = self.cfg
        B, T, d = x.shape
        H, HV, K, V = cfg.n_heads_qk, cfg.n_heads_v, cfg.head_dim_k, cfg.head_dim_v
        lb = conv_lookback
        if lb is not None and lb.shape[0] != B:
            lb = None
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
        g = linear(gd, self.g_up.weight, epilogue=[(HV * K, _lib.ACT_NEG_SOFTPLUS, cfg.kda_decay_scale)])
        return (q.unflatten(-1, (H, K)), k.unflatten(-1, (H, K)), v.unflatten(-1, (HV, V)),
                g.view(B, T, HV, K), beta, new_lb)

    def forward_functional(self, x, state, conv_lookback, *, detach_lookback=True, residual=None):
        cfg = self.cfg
        B, T, _ = x.shape
        HV, V = cfg.n_heads_v, cfg.head_dim_v
        q, k, v, g, beta, new_lb = self.project(x, conv_lookback)
        use_chunk = cfg.kda_chunk_size >= 1 and T >= cfg.kda_chunk_size
        o, new_state = kda_forward(q, k, v, g, beta, scale=self.scale, initial_state=state,
                                   output_final_state=True, chunk_size=cfg.kda_chunk_size, use_chunk=use_chunk,
                                   backend=cfg.kda_backend)
        o = gather_heads(o.reshape(B, T, HV * V), self.tp)
        out = linear(o, self.o_proj.weight, residual=residual)
        return out, new_state, new_lb


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

    def core(self, x, *, return_projections=False):
        cfg = self.cfg
        return naive_csa(x, self.W_aKV.weight, self.W_bKV.weight, self.W_aZ.weight, self.W_bZ.weight, self.Ba,
                         self.Bb, self.W_DQ.weight, self.W_UQ.weight, self.W_IUQ.weight, self.W_w.weight,
                         self.W_KV_idx.weight, self.W_Z_idx.weight, self.B_idx, m=cfg.csa_m, topk=cfg.csa_topk,
                         nh=cfg.csa_nh, nIh=cfg.csa_nIh, c=cfg.csa_c, c_I=cfg.csa_cI, dc=cfg.csa_dc,
                         sliding_window=cfg.csa_sliding_window, sink_logits=self.sink, use_ste=False,
                         normalize_qk=True, return_projections=return_projections,
                         _fused_weight=self.fused_weight(), _fused_q_weight=self.q_weight())

    def forward(self, x, state=None, residual=None):
        return linear(gather_heads(self.core(x), self.tp), self.o_proj.weight, residual=residual), None


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

    def core(self, x, *, return_projections=False):
        cfg = self.cfg
        return naive_hca(x, self.W_KV.weight, self.W_Z.weight, self.B_pos, self.W_DQ.weight, self.W_UQ.weight,
                         m2=cfg.hca_m2, nh=cfg.hca_nh, c=cfg.hca_c, dc=cfg.hca_dc,
                         sliding_window=cfg.hca_sliding_window, sink_logits=self.sink,
                         return_projections=return_projections, _fused_weight=self.fused_weight())

    def forward(self, x, state=None, residual=None):
        return linear(gather_heads(self.core(x), self.tp), self.o_proj.weight, residual=residual), None


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
            h = norm(x)
            if kind == "kda":
                x, st, lb = layer.forward_functional(h, states[ki], lookbacks[ki], residual=x)
                states[ki] = st
                new_lbs.append(lb)
                ki += 1
            else:
                x, _ = layer(h, None, residual=x)
        new_state = torch.stack(states, dim=0) if self.n_kda_layers > 0 else None
        return x, new_state, new_lbs


class HybridDecoding(nn.Module):
    """Decode-time wiring of the stack: a multi-token call runs the full-sequence operators and fills the
    per-layer caches from the same projections; a one-token call appends to the caches and attends
    through them; KDA layers carry their recurrent state and conv lookback."""

    def __init__(self, cfg: HybridConfig | None = None, total_layers: int = 5, *, model=None, kv_quant=None,
                 reserve_tokens: int = 0):
        super().__init__()
        if model is None:
            model = HybridKCHAttention(cfg, total_layers)
        self.model = model
        self.cfg = model.cfg
        self.kv_quant = kv_quant
        self.reserve_tokens = reserve_tokens
        self._caches = {}

    def reset(self):
        self.model.reset_state()
        self._caches = {}

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

    def _csa(self, i, layer, h, residual):
        cfg = self.cfg
        B, T, _ = h.shape
        cache = self._cache(i, layer, h)
        if T > 1:
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
            qn = rownorm(q.contiguous().view(B, 1, nh, c), True)
            o = cache.forward_step(qn, q_idx.contiguous().view(B, 1, nIh, cI).float(), w_idx.float(), topk=cfg.csa_topk,
                                   nh=nh, nIh=nIh, scale=1.0, sink_logits=layer.sink, use_ste=False, normalize_qk=True)
            o_core = o.reshape(B, 1, nh * c).to(h.dtype)
        return linear(gather_heads(o_core, layer.tp), layer.o_proj.weight, residual=residual)

    def _hca(self, i, layer, h, residual):
        cfg = self.cfg
        B, T, _ = h.shape
        cache = self._cache(i, layer, h)
        if T > 1:
            o_core, (C, Z) = layer.core(h, return_projections=True)
            cache.append_step(C, Z, layer.B_pos)
        else:
            c, dc, nh = cfg.hca_c, cfg.hca_dc, cfg.hca_nh
            proj = linear(h, layer.fused_weight())
            C, Z, cQ = proj[..., :2 * c + dc].split([c, c, dc], dim=-1)
            q = linear(cQ, layer.W_UQ.weight)
            cache.append_step(C, Z, layer.B_pos)
            qn = rownorm(q.view(B, 1, nh, c), True)
            o = cache.forward_step(qn, nh=nh, scale=1.0, sink_logits=layer.sink)
            o_core = o.reshape(B, 1, nh * c).to(h.dtype)
        return linear(gather_heads(o_core, layer.tp), layer.o_proj.weight, residual=residual)

    @torch.no_grad()
    def forward(self, x):
        model = self.model
        B, T, _ = x.shape
        stacked = model._kda_state
        if stacked is not None and stacked.shape[1] == B:
            states = list(stacked.unbind(0))
        else:
            states = [None] * model.n_kda_layers
        ki = 0
        for i, (layer, norm, kind) in enumerate(zip(model.layers, model.norms, model.layout)):
            if T == 0:
                continue
            h = norm(x)
            if kind == "kda":
                x, st = layer(h, states[ki], residual=x)
                states[ki] = st
                ki += 1
            elif kind == "csa":
                x = self._csa(i, layer, h, x)
            else:
                x = self._hca(i, layer, h, x)
        if T > 0:
            model._kda_state = torch.stack(states, dim=0) if model.n_kda_layers > 0 else None
        return x
