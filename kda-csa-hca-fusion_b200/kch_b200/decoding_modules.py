"""Single-operator decode modules with the reference's names and parameters.

Mirrors ``KDAAttnDecoding`` (run_decoding.py:234-379), ``CSAAttnDecoding`` (382-522) and ``HCAAttnDecoding``
(525-598) of 183600/kda-csa-hca-fusion: one attention operator plus its output projection, no pre-norm and no
residual, a multi-token call prefills (and fills the cache from the same projections), a one-token call decodes
incrementally.  Same ``state_dict`` keys as the reference modules, so their weights load unchanged.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib
from .csa import fuse_rows, linear, naive_csa, rownorm
from .decoding_cache import CSADecodingCache, HCADecodingCache
from .fused import activation, short_conv
from .hca import naive_hca
from .kda import kda_forward


class KDAAttnDecoding(nn.Module):
    """KDA with its O(1) recurrent state and the short-conv lookback carried across calls; always the
    token-recurrent operator (``use_chunk=False``), as in the reference's decode benchmark."""

    def __init__(self, d_model, H=2, K=16, V=16):
        super().__init__()
        self.q = nn.Linear(d_model, H * K, bias=False)
        self.k = nn.Linear(d_model, H * K, bias=False)
        self.v = nn.Linear(d_model, H * V, bias=False)
        self.g_down = nn.Linear(d_model, K, bias=False)
        self.g_up = nn.Linear(K, H * K, bias=False)
        self.beta = nn.Linear(d_model, H, bias=False)
        self.o = nn.Linear(H * V, d_model, bias=False)
        self.short_conv = nn.Conv1d(d_model, d_model, kernel_size=3, padding=0, groups=d_model, bias=True)
        self.decay_scale = 0.1
        self.kda_backend = "b200"
        self.H, self.K, self.V = H, K, V
        self._state = None
        self._conv_lookback = None

    def reset(self):
        self._state = None
        self._conv_lookback = None

    @torch.no_grad()
    def forward(self, x):
        B, T, d = x.shape
        H, K, V = self.H, self.K, self.V
        lb = self._conv_lookback
        if lb is not None and (lb.shape[0] != B or lb.dtype != x.dtype):
            lb = None
        xc = short_conv(x, self.short_conv.weight, self.short_conv.bias, lb)
        if T >= 2:
            self._conv_lookback = x[:, -2:].clone()
        else:
            prev = lb if lb is not None else x.new_zeros(B, 2, d)
            self._conv_lookback = torch.cat([prev, x], dim=1)[:, -2:].clone()
        q = activation(linear(xc, self.q.weight), _lib.ACT_SILU_L2NORM, group=K).view(B, T, H, K)
        k = activation(linear(xc, self.k.weight), _lib.ACT_SILU_L2NORM, group=K).view(B, T, H, K)
        v = activation(linear(xc, self.v.weight), _lib.ACT_SILU).view(B, T, H, V)
        g = activation(linear(linear(xc, self.g_down.weight), self.g_up.weight), _lib.ACT_NEG_SOFTPLUS,
                       param=self.decay_scale).view(B, T, H, K)
        beta = activation(linear(xc, self.beta.weight), _lib.ACT_SIGMOID)
        state = self._state
        if state is not None and state.shape[0] != B:
            state = None
        o, self._state = kda_forward(q, k, v, g, beta, scale=K ** -0.5, initial_state=state, output_final_state=True,
                                     use_chunk=False, backend=self.kda_backend)
        return linear(o.reshape(B, T, H * V), self.o.weight)


class CSAAttnDecoding(nn.Module):
    def __init__(self, d_model, m=4, topk=2, nh=2, c=8, dc=8, nIh=1, c_I=4, sliding_window=4, use_ste=False):
        super().__init__()
        self.d_model = d_model
        self.m, self.topk, self.nh, self.c = m, topk, nh, c
        self.dc, self.nIh, self.c_I = dc, nIh, c_I
        self.sliding_window = sliding_window
        self.use_ste = use_ste
        d = d_model
        self.W_aKV = nn.Linear(d, c, bias=False)
        self.W_bKV = nn.Linear(d, c, bias=False)
        self.W_aZ = nn.Linear(d, c, bias=False)
        self.W_bZ = nn.Linear(d, c, bias=False)
        self.Ba = nn.Parameter(torch.randn(m, c) * 0.02)
        self.Bb = nn.Parameter(torch.randn(m, c) * 0.02)
        self.W_DQ = nn.Linear(d, dc, bias=False)
        self.W_UQ = nn.Linear(dc, c * nh, bias=False)
        self.W_IUQ = nn.Linear(dc, c_I * nIh, bias=False)
        self.W_w = nn.Linear(d, nIh, bias=False)
        self.W_KV_idx = nn.Linear(d, c_I, bias=False)
        self.W_Z_idx = nn.Linear(d, c_I, bias=False)
        self.B_idx = nn.Parameter(torch.randn(m, c_I) * 0.02)
        self.sink = nn.Parameter(torch.zeros(nh))
        self.o_proj = nn.Linear(c * nh, d, bias=False)
        self._cache = None

    def reset(self):
        self._cache = None

    def _ensure_cache(self, B, device, dtype):
        if self._cache is None or self._cache.B != B or self._cache.device != device or self._cache.dtype != dtype:
            self._cache = CSADecodingCache(B, self.c, self.c_I, self.m, self.sliding_window, device, dtype)

    @torch.no_grad()
    def forward(self, x):
        B, T, _ = x.shape
        self._ensure_cache(B, x.device, x.dtype)
        cache = self._cache
        c, cI, dc, nh, nIh = self.c, self.c_I, self.dc, self.nh, self.nIh
        if T > 1:
            o, proj = naive_csa(x, self.W_aKV.weight, self.W_bKV.weight, self.W_aZ.weight, self.W_bZ.weight, self.Ba,
                                self.Bb, self.W_DQ.weight, self.W_UQ.weight, self.W_IUQ.weight, self.W_w.weight,
                                self.W_KV_idx.weight, self.W_Z_idx.weight, self.B_idx, m=self.m, topk=self.topk, nh=nh,
                                nIh=nIh, c=c, c_I=cI, dc=dc, sliding_window=self.sliding_window, sink_logits=self.sink,
                                use_ste=False, normalize_qk=True, return_projections=True)
            cache.append_step(*proj, self.Ba, self.Bb, self.B_idx)
            return linear(o, self.o_proj.weight)
        W = fuse_rows(self.W_aKV.weight, self.W_bKV.weight, self.W_aZ.weight, self.W_bZ.weight, self.W_KV_idx.weight,
                      self.W_Z_idx.weight, self.W_DQ.weight, self.W_w.weight)
        proj = linear(x, W)
        Ca, Cb, Za, Zb, K_idx, Z_idx, cQ, w_idx = proj[..., :4 * c + 2 * cI + dc + nIh].split(
            [c, c, c, c, cI, cI, dc, nIh], dim=-1)
        q = linear(cQ, self.W_UQ.weight).view(B, 1, nh, c)
        q_idx = linear(cQ, self.W_IUQ.weight).view(B, 1, nIh, cI)
        cache.append_step(Ca, Cb, Za, Zb, K_idx, Z_idx, self.Ba, self.Bb, self.B_idx)
        o = cache.forward_step(rownorm(q, True), q_idx.float(), w_idx.float(), topk=self.topk, nh=nh, nIh=nIh, scale=1.0,
                               sink_logits=self.sink, use_ste=False, normalize_qk=True)
        return linear(o.reshape(B, 1, nh * c).to(x.dtype), self.o_proj.weight)


class HCAAttnDecoding(nn.Module):
    def __init__(self, d_model, m2=4, nh=2, c=8, dc=8, sliding_window=4):
        super().__init__()
        self.d_model = d_model
        self.m2, self.nh, self.c, self.dc = m2, nh, c, dc
        self.sliding_window = sliding_window
        d = d_model
        self.W_KV = nn.Linear(d, c, bias=False)
        self.W_Z = nn.Linear(d, c, bias=False)
        self.B_pos = nn.Parameter(torch.randn(m2, c) * 0.02)
        self.W_DQ = nn.Linear(d, dc, bias=False)
        self.W_UQ = nn.Linear(dc, c * nh, bias=False)
        self.sink = nn.Parameter(torch.zeros(nh))
        self.o_proj = nn.Linear(c * nh, d, bias=False)
        self._cache = None

    def reset(self):
        self._cache = None

    def _ensure_cache(self, B, device, dtype):
        if self._cache is None or self._cache.B != B or self._cache.device != device or self._cache.dtype != dtype:
            self._cache = HCADecodingCache(B, self.c, self.m2, self.sliding_window, device, dtype)

    @torch.no_grad()
    def forward(self, x):
        B, T, _ = x.shape
        self._ensure_cache(B, x.device, x.dtype)
        cache = self._cache
        c, dc, nh = self.c, self.dc, self.nh
        if T > 1:
            o, (C, Z) = naive_hca(x, self.W_KV.weight, self.W_Z.weight, self.B_pos, self.W_DQ.weight, self.W_UQ.weight,
                                  m2=self.m2, nh=nh, c=c, dc=dc, sliding_window=self.sliding_window,
                                  sink_logits=self.sink, return_projections=True)
            cache.append_step(C, Z, self.B_pos)
            return linear(o, self.o_proj.weight)
        proj = linear(x, fuse_rows(self.W_KV.weight, self.W_Z.weight, self.W_DQ.weight))
        C, Z, cQ = proj[..., :2 * c + dc].split([c, c, dc], dim=-1)
        q = linear(cQ, self.W_UQ.weight).view(B, 1, nh, c)
        cache.append_step(C, Z, self.B_pos)
        o = cache.forward_step(rownorm(q, True), nh=nh, scale=1.0, sink_logits=self.sink)
        return linear(o.reshape(B, 1, nh * c).to(x.dtype), self.o_proj.weight)
