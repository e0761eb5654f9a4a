"""Seeded synthetic inputs for the KDA / CSA / HCA hot path.

Everything is drawn on the CPU from ``torch.Generator().manual_seed(seed)`` in fp32 and cast
afterwards, so a CPU checker and the GPU kernels see identical bits (a CUDA generator produces
a different stream).  Shapes and value distributions follow the benchmark configurations:
unit-norm q/k, ``g = -softplus(N(0,1))``, ``beta = sigmoid(N(0,1))``, weights ``N(0, 0.02)``,
hidden states ``N(0,1)``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


def kda_inputs(seed, B, T, H, K, V, HV=None, dtype=torch.float32, with_state=False):
    """q,k ``[B,T,H,K]`` unit norm; v ``[B,T,HV,V]``; g ``[B,T,HV,K]`` <= 0; beta ``[B,T,HV]``.
    Draw order q, k, v, g, beta (then the optional initial state)."""
    HV = H if HV is None else HV
    g_ = _gen(seed)
    q = F.normalize(torch.randn(B, T, H, K, generator=g_), dim=-1)
    k = F.normalize(torch.randn(B, T, H, K, generator=g_), dim=-1)
    v = torch.randn(B, T, HV, V, generator=g_)
    g = -F.softplus(torch.randn(B, T, HV, K, generator=g_))
    beta = torch.sigmoid(torch.randn(B, T, HV, generator=g_))
    out = [x.to(dtype) for x in (q, k, v, g, beta)]
    if with_state:
        out.append(torch.randn(B, HV, K, V, generator=g_) * 0.1)
    return out


CSA_WEIGHT_ORDER = ("W_aKV", "W_bKV", "W_aZ", "W_bZ", "Ba", "Bb", "W_DQ", "W_UQ", "W_IUQ", "W_w",
                    "W_KV_idx", "W_Z_idx", "B_idx")


def csa_inputs(seed, B, T, d, *, nh, c, dc, nIh, c_I, m, dtype=torch.bfloat16, random_sink=False,
               std=0.02):
    """Weights in the order of the ``naive_csa`` signature, then ``sink``, then ``H``."""
    g_ = _gen(seed)

    def W(o, i):
        return torch.randn(o, i, generator=g_) * std

    w = dict(W_aKV=W(c, d), W_bKV=W(c, d), W_aZ=W(c, d), W_bZ=W(c, d), Ba=W(m, c), Bb=W(m, c),
             W_DQ=W(dc, d), W_UQ=W(c * nh, dc), W_IUQ=W(c_I * nIh, dc), W_w=W(nIh, d),
             W_KV_idx=W(c_I, d), W_Z_idx=W(c_I, d), B_idx=W(m, c_I))
    sink = torch.randn(nh, generator=g_) if random_sink else torch.zeros(nh)
    H = torch.randn(B, T, d, generator=g_)
    w = {k: v.to(dtype) for k, v in w.items()}
    return w, sink.to(dtype), H.to(dtype)


def hca_inputs(seed, B, T, d, *, nh, c, dc, m2, dtype=torch.bfloat16, random_sink=False, std=0.02):
    g_ = _gen(seed)

    def W(o, i):
        return torch.randn(o, i, generator=g_) * std

    w = dict(W_KV=W(c, d), W_Z=W(c, d), B_pos=W(m2, c), W_DQ=W(dc, d), W_UQ=W(c * nh, dc))
    sink = torch.randn(nh, generator=g_) if random_sink else torch.zeros(nh)
    H = torch.randn(B, T, d, generator=g_)
    w = {k: v.to(dtype) for k, v in w.items()}
    return w, sink.to(dtype), H.to(dtype)


def hybrid_layout(n_kda, n_csa, n_hca, total_layers):
    unit = ["kda"] * n_kda + ["csa"] * n_csa + ["hca"] * n_hca
    out = []
    while len(out) < total_layers:
        out.extend(unit)
    return out[:total_layers]


def hybrid_params(seed, cfg, total_layers=5, dtype=torch.bfloat16, std=0.02, random_sink=False):
    """Random-init parameters of the hybrid stack, keyed by the ``state_dict`` names of the
    module tree (``layers.{i}.q_proj.weight``, ``norms.{i}.weight`` ...).  Every matrix is
    ``N(0, std)``; the short-conv taps and bias are ``U(-1/sqrt(3), 1/sqrt(3))`` (the default
    initialisation of a depthwise kernel-3 convolution); norms are (1, 0); sinks are 0."""
    g_ = _gen(seed)
    d = cfg.d_model
    H, HV, K, V = cfg.n_heads_qk, cfg.n_heads_v, cfg.head_dim_k, cfg.head_dim_v
    p = {}

    def W(o, i):
        return torch.randn(o, i, generator=g_) * std

    for i, kind in enumerate(hybrid_layout(cfg.n_kda, cfg.n_csa, cfg.n_hca, total_layers)):
        L = f"layers.{i}."
        if kind == "kda":
            p[L + "q_proj.weight"] = W(H * K, d)
            p[L + "k_proj.weight"] = W(H * K, d)
            p[L + "v_proj.weight"] = W(HV * V, d)
            p[L + "g_down.weight"] = W(K, d)
            p[L + "g_up.weight"] = W(HV * K, K)
            p[L + "beta.weight"] = W(HV, d)
            p[L + "o_proj.weight"] = W(d, HV * V)
            bound = 1.0 / math.sqrt(3.0)
            p[L + "short_conv.weight"] = (torch.rand(d, 1, 3, generator=g_) * 2 - 1) * bound
            p[L + "short_conv.bias"] = (torch.rand(d, generator=g_) * 2 - 1) * bound
        elif kind == "csa":
            c, cI = cfg.csa_c, cfg.csa_cI
            p[L + "W_aKV.weight"] = W(c, d)
            p[L + "W_bKV.weight"] = W(c, d)
            p[L + "W_aZ.weight"] = W(c, d)
            p[L + "W_bZ.weight"] = W(c, d)
            p[L + "Ba"] = W(cfg.csa_m, c)
            p[L + "Bb"] = W(cfg.csa_m, c)
            p[L + "W_DQ.weight"] = W(cfg.csa_dc, d)
            p[L + "W_UQ.weight"] = W(c * cfg.csa_nh, cfg.csa_dc)
            p[L + "W_IUQ.weight"] = W(cI * cfg.csa_nIh, cfg.csa_dc)
            p[L + "W_w.weight"] = W(cfg.csa_nIh, d)
            p[L + "W_KV_idx.weight"] = W(cI, d)
            p[L + "W_Z_idx.weight"] = W(cI, d)
            p[L + "B_idx"] = W(cfg.csa_m, cI)
            p[L + "sink"] = torch.randn(cfg.csa_nh, generator=g_) if random_sink else torch.zeros(cfg.csa_nh)
            p[L + "o_proj.weight"] = W(d, c * cfg.csa_nh)
        else:
            c = cfg.hca_c
            p[L + "W_KV.weight"] = W(c, d)
            p[L + "W_Z.weight"] = W(c, d)
            p[L + "B_pos"] = W(cfg.hca_m2, c)
            p[L + "W_DQ.weight"] = W(cfg.hca_dc, d)
            p[L + "W_UQ.weight"] = W(c * cfg.hca_nh, cfg.hca_dc)
            p[L + "sink"] = torch.randn(cfg.hca_nh, generator=g_) if random_sink else torch.zeros(cfg.hca_nh)
            p[L + "o_proj.weight"] = W(d, c * cfg.hca_nh)
        p[f"norms.{i}.weight"] = torch.ones(d)
        p[f"norms.{i}.bias"] = torch.zeros(d)
    return {k: v.to(dtype) for k, v in p.items()}


def hidden_states(seed, B, T, d, dtype=torch.bfloat16):
    return torch.randn(B, T, d, generator=_gen(seed)).to(dtype)


def fill_decode_state(dec, B, context, extra_tokens, dev, seed):
    """Put the decode wrapper in the state it has after `context` tokens without running a prefill:
    compressed rows, scoring copies, norms, accumulators, rings and KDA states filled with seeded random
    values of the right scale, counters set.  The step cost does not depend on the values."""
    from .fused import CSAHybridLayer, HCAHybridLayer
    g = torch.Generator(device=dev).manual_seed(seed)
    model, cfg = dec.model, dec.cfg
    dec.reset()
    h = torch.empty(B, 1, cfg.d_model, dtype=torch.bfloat16, device=dev)
    for i, layer in enumerate(model.layers):
        if not isinstance(layer, (CSAHybridLayer, HCAHybridLayer)):
            continue
        cache = dec._cache(i, layer, dec._local_rows(layer, h))    # rows-sharded layers cache this rank's sequences only
        B = cache.B
        m = cache.m if isinstance(layer, CSAHybridLayer) else cache.m2
        nb = context // m
        cache.reserve(nb + extra_tokens // m + 2)
        for s0 in range(0, nb, 4096):                 # bounded temporaries
            n = min(4096, nb - s0)
            cache._store_rows(torch.randn(B, n, cache.c, device=dev, generator=g), s0)
        if isinstance(layer, CSAHybridLayer):
            k = torch.randn(B, nb, cache.c_I, device=dev, generator=g).to(cache.dtype)
            cache._kcomp[:, :nb] = k
            cache._kcomp_norms[:, :nb] = k.float().norm(dim=-1).clamp_min(1e-12)
            for p in cache._prev:
                p.copy_(torch.randn(p.shape, device=dev, generator=g))
            cache._has_prev = True
        for a in cache._acc:
            a.copy_(torch.randn(a.shape, device=dev, generator=g))
        cache._acc_len = context % m
        cache._n_blocks = nb
        cache._n_tokens_seen = context
        if cache._sw is not None:
            w = torch.randn(cache._sw._buf.shape, device=dev, generator=g)
            cache._sw._buf.copy_(w / w.norm(dim=-1, keepdim=True))
            cache._sw._n = context
        cache._sync_counters()
    B = h.shape[0]
    HV, K, V = cfg.n_heads_v, cfg.head_dim_k, cfg.head_dim_v
    model._kda_state = 0.02 * torch.randn(model.n_kda_layers, B, HV, K, V, device=dev, generator=g)
    for layer in model.layers:
        if hasattr(layer, "_conv_lookback"):
            layer._conv_lookback = torch.randn(B, 2, cfg.d_model, device=dev, generator=g).to(torch.bfloat16)
