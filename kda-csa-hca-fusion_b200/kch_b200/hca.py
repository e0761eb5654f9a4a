"""HCA operator on the B200 kernels, with the reference signature.

Mirrors ``naive_hca`` (ops_hca.py:30-201) of 183600/kda-csa-hca-fusion: heavy single-branch
compression (ratio m2), dense MQA over every visible compressed block, a sliding window over the
normalised per-token keys and an attention sink, all under one softmax.
"""
from __future__ import annotations

import torch

from . import _lib
from .csa import attend, csa_compress_kv, fuse_rows, linear, mma_attention_eligible, rownorm


def naive_hca(H, W_KV, W_Z, B_pos, W_DQ, W_UQ, *, m2: int, nh: int, c: int, dc: int, scale: float = 1.0,
              sliding_window: int = 0, sink_logits=None, return_projections: bool = False, W_KV_local=None,
              _fused_weight=None, _q_rows=None):
    """``[B,T,d] -> [B,T,nh*c]`` in ``H.dtype``.  ``_fused_weight`` (optional) is ``[W_KV;W_Z;W_DQ]``
    (plus ``W_KV_local`` when used) concatenated once by the layer object.  ``_q_rows = (lo, hi)`` (sharding by
    query rows): only the queries ``lo..hi-1`` are attended, against the keys of tokens ``0..hi-1``; returns
    ``[B, hi-lo, nh*c]``."""
    B_, T, d = H.shape
    if m2 < 1:
        raise ValueError(f"heavy compression factor m2={m2} must be >= 1")
    if nh < 1:
        raise ValueError(f"nh={nh} must be >= 1")
    if c < 1:
        raise ValueError(f"c={c} must be >= 1")
    if dc < 1:
        raise ValueError(f"dc={dc} must be >= 1")
    if sliding_window < 0:
        raise ValueError(f"sliding_window={sliding_window} must be >= 0 (0 disables the branch)")
    if not torch.is_floating_point(H):
        raise TypeError(f"naive_hca: H must be a floating-point tensor, got dtype={H.dtype}")
    if W_KV.shape != (c, d):
        raise ValueError(f"naive_hca: W_KV.shape={tuple(W_KV.shape)} must equal (c, d)=({c}, {d})")
    if W_Z.shape != (c, d):
        raise ValueError(f"naive_hca: W_Z.shape={tuple(W_Z.shape)} must equal (c, d)=({c}, {d})")
    if W_DQ.shape != (dc, d):
        raise ValueError(f"naive_hca: W_DQ.shape={tuple(W_DQ.shape)} must equal (dc, d)=({dc}, {d})")
    if W_UQ.shape != (c * nh, dc):
        raise ValueError(f"naive_hca: W_UQ.shape={tuple(W_UQ.shape)} must equal (c*nh, dc)=({c*nh}, {dc})")
    if B_pos.shape != (m2, c):
        raise ValueError(f"naive_hca: B_pos.shape={tuple(B_pos.shape)} must equal (m2, c)=({m2}, {c})")
    if sink_logits is not None and sink_logits.shape != (nh,):
        raise ValueError(f"naive_hca: sink_logits.shape={tuple(sink_logits.shape)} must equal (nh,)=({nh},)")
    if W_KV_local is not None and W_KV_local.shape != (c, d):
        raise ValueError(f"naive_hca: W_KV_local.shape={tuple(W_KV_local.shape)} must equal (c, d)=({c}, {d})")
    _lib.require_cuda(H, fn="naive_hca")
    device = H.device
    if T == 0:
        out_empty = torch.zeros(B_, 0, nh * c, dtype=H.dtype, device=device)
        if return_projections:
            return out_empty, (torch.zeros(B_, 0, c, dtype=H.dtype, device=device),
                               torch.zeros(B_, 0, c, dtype=H.dtype, device=device))
        return out_empty
    q_lo = 0
    if _q_rows is not None:
        q_lo, q_hi = int(_q_rows[0]), int(_q_rows[1])
        if not 0 <= q_lo < q_hi <= T:
            raise ValueError(f"naive_hca: _q_rows={_q_rows} must satisfy 0 <= lo < hi <= T={T}")
        if return_projections:
            raise ValueError("naive_hca: _q_rows and return_projections cannot be combined")
        H, T = H[:, :q_hi], q_hi
    original_T = T
    pad = (-T) % m2
    if pad:
        H = torch.nn.functional.pad(H, (0, 0, 0, pad))
        T += pad
    if _fused_weight is None:
        parts = [W_KV, W_Z, W_DQ] + ([W_KV_local] if W_KV_local is not None else [])
        _fused_weight = fuse_rows(*parts)
    proj = linear(H, _fused_weight)
    if W_KV_local is not None:
        C, Z, cQ, C_loc = proj[..., :3 * c + dc].split([c, c, dc, c], dim=-1)
    else:
        C, Z, cQ = proj[..., :2 * c + dc].split([c, c, dc], dim=-1)
        C_loc = C
    C_comp = csa_compress_kv(C, Z, B_pos, m2)
    kdt = torch.bfloat16 if mma_attention_eligible(H.dtype, c, nh, True, scale) else torch.float32
    C_comp_n = rownorm(C_comp, True, kdt)
    q = linear(cQ[:, q_lo:] if q_lo else cQ, W_UQ)
    local = rownorm(C_loc, True, kdt) if sliding_window > 0 else None
    out = attend(q, C_comp_n, nh=nh, c=c, sel=None, m=m2, t0=q_lo, q_normalize=True, win=local,
                 sliding_window=sliding_window, sink=sink_logits, scale=scale, out_dtype=H.dtype, win_t0=q_lo)
    out_final = out[:, :original_T - q_lo]
    if return_projections:
        return out_final, (C[:, :original_T], Z[:, :original_T])
    return out_final
