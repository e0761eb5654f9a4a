"""Case tables shared by the golden-vector generator and the tests.

Sizes are chosen so the reference finishes each case in seconds and the stored outputs stay small;
they include the edge shapes the reference's own suite exercises: T not a multiple of the chunk /
compression factor, grouped value heads, an initial state, top-k larger than the number of blocks,
no window, no sink, un-normalised scoring.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch

F32, BF16 = torch.float32, torch.bfloat16

KDA_CASES = {
    # name: geometry
    "gva_pad_state": dict(seed=11, B=2, T=150, H=2, HV=4, K=32, V=48, chunk=64, dtype=F32, state=True),
    "k128": dict(seed=12, B=1, T=256, H=2, HV=2, K=128, V=128, chunk=64, dtype=F32, state=False),
    "bf16_small_chunk": dict(seed=13, B=2, T=70, H=2, HV=2, K=64, V=64, chunk=16, dtype=BF16, state=True),
    "short": dict(seed=14, B=1, T=5, H=1, HV=1, K=16, V=16, chunk=64, dtype=F32, state=False),
}

_csa_small = dict(B=2, T=70, d=64, nh=2, c=16, dc=16, nIh=2, c_I=8, m=4, topk=6, win=8, sink=True,
                  random_sink=True, normalize_qk=True, std=0.3)
CSA_CASES = {
    "small_f32": dict(seed=21, dtype=F32, **_csa_small),
    "small_bf16": dict(seed=22, dtype=BF16, **_csa_small),
    "no_norm_no_sink": dict(seed=23, dtype=F32, **{**_csa_small, "sink": False, "normalize_qk": False}),
    "topk_all_no_win": dict(seed=24, dtype=F32, **{**_csa_small, "topk": 40, "win": 0}),
    "prod_dims_bf16": dict(seed=25, B=1, T=512, d=256, nh=4, c=128, dc=128, nIh=4, c_I=64, m=4, topk=32,
                           win=128, sink=True, random_sink=False, normalize_qk=True, dtype=BF16),
}

_hca_small = dict(B=2, T=70, d=64, nh=2, c=16, dc=16, m2=8, win=8, sink=True, random_sink=True, std=0.3)
HCA_CASES = {
    "small_f32": dict(seed=31, dtype=F32, **_hca_small),
    "small_bf16": dict(seed=32, dtype=BF16, **_hca_small),
    "no_sink_no_win": dict(seed=33, dtype=F32, **{**_hca_small, "sink": False, "win": 0}),
    "prod_dims_bf16": dict(seed=34, B=1, T=640, d=256, nh=4, c=128, dc=128, m2=128, win=128, sink=True,
                           random_sink=False, dtype=BF16),
}

CACHE_CASES = {
    "f32": dict(seed=41, B=2, T=37, c=16, c_I=8, m=4, m2=8, win=8, nh=2, nIh=2, topk=100, dtype=F32),
    "bf16": dict(seed=42, B=2, T=37, c=16, c_I=8, m=4, m2=8, win=8, nh=2, nIh=2, topk=100, dtype=BF16),
    "bf16_sparse": dict(seed=43, B=1, T=45, c=32, c_I=16, m=4, m2=8, win=4, nh=2, nIh=2, topk=3, dtype=BF16),
}

_hyb_cfg = dict(d_model=64, n_heads_qk=2, n_heads_v=4, head_dim_k=16, head_dim_v=16, kda_chunk_size=16,
                csa_m=4, csa_topk=16, csa_nh=2, csa_c=16, csa_dc=16, csa_nIh=2, csa_cI=8, csa_sliding_window=8,
                hca_m2=8, hca_nh=2, hca_c=16, hca_dc=16, hca_sliding_window=8, n_kda=3, n_csa=1, n_hca=1)
HYBRID_CASES = {
    "f32": dict(seed=51, B=2, T=50, layers=5, dtype=F32, cfg=_hyb_cfg),
    "bf16": dict(seed=52, B=2, T=50, layers=5, dtype=BF16, cfg=_hyb_cfg),
}

DECODE_CASE = dict(seed=61, B=2, d_model=64, prefill=21, steps=7, csa_topk=100, dtype=F32)

# single-operator decode modules (run_decoding.py:234-598): constructor arguments per kind
STANDALONE_CASE = dict(seed=83, B=2, d_model=32, prefill=13, steps=9, dtype=F32,
                       kda=dict(H=2, K=8, V=8),
                       csa=dict(m=4, topk=100, nh=2, c=8, dc=8, nIh=1, c_I=4, sliding_window=4),
                       hca=dict(m2=4, nh=2, c=8, dc=8, sliding_window=4))


def np32(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float32).cpu().numpy()


def checksum(*tensors) -> np.ndarray:
    """Eight bytes of SHA-256 over the fp32 bits of the inputs (detects generator drift)."""
    h = hashlib.sha256()
    for t in tensors:
        h.update(np.ascontiguousarray(np32(t)).tobytes())
    return np.frombuffer(h.digest()[:8], dtype=np.uint8).copy()


def make_cache_stream(c):
    """Per-token projections fed to the decode caches: values rounded to the cache dtype."""
    g = torch.Generator().manual_seed(c["seed"])
    B, T, dt = c["B"], c["T"], c["dtype"]

    def r(*s, std=1.0):
        return (torch.randn(*s, generator=g) * std).to(dt)

    st = {n: r(B, T, c["c"]) for n in ("Ca", "Cb", "Za", "Zb")}
    st["K_idx"], st["Z_idx"] = r(B, T, c["c_I"]), r(B, T, c["c_I"])
    st["Ba"], st["Bb"] = r(c["m"], c["c"], std=0.3), r(c["m"], c["c"], std=0.3)
    st["B_idx"] = r(c["m"], c["c_I"], std=0.3)
    st["B_pos"] = r(c["m2"], c["c"], std=0.3)
    st["q"] = r(B, T, c["nh"], c["c"])
    st["q_idx"] = r(B, T, c["nIh"], c["c_I"])
    st["w_idx"] = r(B, T, c["nIh"])
    st["sink"] = r(c["nh"])
    return st
