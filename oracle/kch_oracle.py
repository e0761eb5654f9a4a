"""CPU oracle for the KDA / CSA / HCA hybrid-attention forward path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it is
used by the tests, by the smoke check and by the CPU-baseline leg of the benchmark
as the *checker* (and the timed CPU arm), never as a product code path.

What it is: an independent restatement, in plain dense tensor algebra on the CPU,
of the algorithms of the reference project 183600/kda-csa-hca-fusion.  Each function
cites the reference lines it follows.  The reference does all of its arithmetic in
PyTorch CPU tensor ops (an un-vendored dependency, pinned ``torch>=2.2,<2.7`` in its
``pyproject.toml:45``); this file uses the same array library for storage, matmul
and bf16 rounding so that rounding points coincide, but shares no code with the
reference: loops are query-tiled so that shapes the reference cannot materialise
(its ``[B,T,topk,c]`` gather, ``ops_csa.py:970``) still run.

Pinning: ``tests/golden/make_golden.py`` runs the *reference itself* on seeded inputs
and stores its outputs; ``tests/test_oracle_golden.py`` checks every function here
against those stored outputs.  The FP8/INT8 block-scaled cache variant has no
counterpart in the reference: for it, parity is unpinned (oracle by construction:
quantise -> dequantise -> the pinned bf16 path).

Top-k tie rule (the reference leaves it to ``torch.topk``, whose tie order is
implementation-defined, see ``ops_decoding_cache.py:62-87``): equal logits are
ordered by ascending block index; the CUDA kernels follow the same rule.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

NEG_INF = float("-inf")


# --------------------------------------------------------------------------------------
# small helpers
# --------------------------------------------------------------------------------------
def _cdtype(t: torch.Tensor) -> torch.dtype:
    return torch.float64 if t.dtype == torch.float64 else torch.float32


def l2_normalize(x: torch.Tensor, eps: float = 1e-12) -> torch.Tensor:
    """``x / max(||x||_2, eps)`` along the last axis (``F.normalize`` semantics)."""
    n = x.pow(2).sum(-1, keepdim=True).sqrt().clamp_min(eps)
    return x / n


# --------------------------------------------------------------------------------------
# KDA  (reference: ops_kda.py)
# --------------------------------------------------------------------------------------
def recurrent_kda(q, k, v, g, beta, scale=None, initial_state=None, g_clamp_min=-10.0):
    """Token-by-token gated delta rule (``ops_kda.py:222-258``).

    q,k ``[B,T,H,K]``; v ``[B,T,HV,V]``; g ``[B,T,HV,K]``; beta ``[B,T,HV]``.
    Returns ``(o [B,T,HV,V] in v.dtype, S [B,HV,K,V] in fp32/fp64)``.
    """
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    G = HV // H
    cd = _cdtype(v)
    if scale is None:
        scale = K ** -0.5
    scale = float(scale)
    qf = q.to(cd).repeat_interleave(G, dim=2) * scale
    kf = k.to(cd).repeat_interleave(G, dim=2)
    vf, gf, bf = v.to(cd), g.to(cd), beta.to(cd)
    if g_clamp_min > -math.inf:
        gf = gf.clamp(min=float(g_clamp_min))
    S = torch.zeros(B, HV, K, V, dtype=cd)
    if initial_state is not None:
        S = S + initial_state.to(cd)
    o = torch.zeros(B, T, HV, V, dtype=cd)
    for t in range(T):
        S = S * gf[:, t].exp().unsqueeze(-1)                       # decay rows of S
        pred = (kf[:, t].unsqueeze(-1) * S).sum(-2)                # k^T S   [B,HV,V]
        delta = bf[:, t].unsqueeze(-1) * (vf[:, t] - pred)
        S = S + kf[:, t].unsqueeze(-1) * delta.unsqueeze(-2)
        o[:, t] = (qf[:, t].unsqueeze(-1) * S).sum(-2)
    return o.to(v.dtype), S


def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, chunk_size=64,
              g_clamp_min=-10.0):
    """Chunked WY form (``ops_kda.py:375-424`` prepare, ``509-535`` chain).

    Inside a chunk of C tokens, with gamma the per-channel running sum of g:
      A[i,j]   = beta_i sum_k k_i k_j exp(gamma_i-gamma_j)   (i>j)
      Tm       = (I + A)^-1 diag(beta)
      w, u     = Tm (exp(gamma) * k),  Tm v
      Aqk[i,j] = sum_k q_i k_j exp(gamma_i-gamma_j)          (i>=j)
      vt = u - w S;  o = (q*exp(gamma)) S + Aqk vt
      S  = exp(gamma_last) * S + (exp(gamma_last-gamma) * k)^T vt
    """
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    G = HV // H
    C = int(chunk_size)
    cd = _cdtype(v)
    if scale is None:
        scale = K ** -0.5
    scale = float(scale)
    S = torch.zeros(B, HV, K, V, dtype=cd)
    if initial_state is not None:
        S = S + initial_state.to(cd)
    if T == 0:
        return torch.zeros(B, 0, HV, V, dtype=v.dtype), S
    pad = (-T) % C
    Tp = T + pad

    def prep(x, rep):
        x = x.to(cd)
        if pad:
            x = torch.cat([x, x.new_zeros(B, pad, *x.shape[2:])], dim=1)
        if rep:
            x = x.repeat_interleave(G, dim=2)
        return x

    qf = prep(q, True) * scale
    kf = prep(k, True)
    vf = prep(v, False)
    gf = g.to(cd)
    if g_clamp_min > -math.inf:
        gf = gf.clamp(min=float(g_clamp_min))
    gf = prep(gf, False)
    bf = prep(beta, False)
    o = torch.zeros(B, Tp, HV, V, dtype=cd)
    eye = torch.eye(C, dtype=cd)
    strict_lower = torch.tril(torch.ones(C, C, dtype=torch.bool), diagonal=-1)
    lower = torch.tril(torch.ones(C, C, dtype=torch.bool), diagonal=0)
    for n in range(Tp // C):
        sl = slice(n * C, (n + 1) * C)
        qc = qf[:, sl].transpose(1, 2)              # [B,HV,C,K]
        kc = kf[:, sl].transpose(1, 2)
        vc = vf[:, sl].transpose(1, 2)              # [B,HV,C,V]
        gam = gf[:, sl].transpose(1, 2).cumsum(-2)  # [B,HV,C,K]
        bc = bf[:, sl].transpose(1, 2)              # [B,HV,C]
        diff = (gam.unsqueeze(-2) - gam.unsqueeze(-3)).clamp(max=50.0).exp()   # [.,i,j,K]
        kk = (kc.unsqueeze(-2) * kc.unsqueeze(-3) * diff).sum(-1)              # [.,i,j]
        A = (kk * bc.unsqueeze(-1)).masked_fill(~strict_lower, 0.0)
        # forward substitution for (I + A)^-1, one row at a time
        Tm = eye.expand(B, HV, C, C).clone()
        for i in range(1, C):
            Tm[..., i, :] = Tm[..., i, :] - (A[..., i, :i].unsqueeze(-1) * Tm[..., :i, :]).sum(-2)
        Tm = Tm * bc.unsqueeze(-2)
        w = Tm @ (gam.exp() * kc)
        u = Tm @ vc
        Aqk = (qc.unsqueeze(-2) * kc.unsqueeze(-3) * diff).sum(-1).masked_fill(~lower, 0.0)
        vt = u - w @ S
        o[:, sl] = ((qc * gam.exp()) @ S + Aqk @ vt).transpose(1, 2)
        glast = gam[..., -1:, :]
        S = S * glast.squeeze(-2).exp().unsqueeze(-1) + ((glast - gam).exp() * kc).transpose(-1, -2) @ vt
    return o[:, :T].to(v.dtype), S


# --------------------------------------------------------------------------------------
# compression  (reference: ops_csa.py:198-305)
# --------------------------------------------------------------------------------------
def compress_kv(C, Z, B_pos, m):
    """Per block of m tokens and per channel: softmax_m(Z+B_pos) . C  (``ops_csa.py:225-234``)."""
    B, T, c = C.shape
    if m < 1:
        raise ValueError(f"compression factor m={m} must be >= 1")
    if T % m:
        raise ValueError(f"T={T} must be divisible by m={m}")
    cd = _cdtype(C)
    Cb = C.to(cd).reshape(B, T // m, m, c)
    lg = Z.to(cd).reshape(B, T // m, m, c) + B_pos.to(cd)
    p = torch.softmax(lg, dim=2)
    return (p * Cb).sum(2)


def compress_kv_overlapped(Ca, Cb, Za, Zb, Ba, Bb, m):
    """Block i mixes its own m a-branch tokens with the m b-branch tokens of block i-1
    under ONE softmax over the 2m logits (``ops_csa.py:262-305``)."""
    B, T, c = Ca.shape
    if m < 1:
        raise ValueError(f"compression factor m={m} must be >= 1")
    if T % m:
        raise ValueError(f"T={T} must be divisible by m={m}")
    cd = _cdtype(Ca)
    n = T // m
    if T == 0:
        return torch.zeros(B, 0, c, dtype=cd)
    ca = Ca.to(cd).reshape(B, n, m, c)
    la = Za.to(cd).reshape(B, n, m, c) + Ba.to(cd)
    cb = torch.zeros(B, n, m, c, dtype=cd)
    lb = torch.full((B, n, m, c), NEG_INF, dtype=cd)
    if n > 1:
        cb[:, 1:] = Cb.to(cd).reshape(B, n, m, c)[:, :-1]
        lb[:, 1:] = Zb.to(cd).reshape(B, n, m, c)[:, :-1] + Bb.to(cd)
    p = torch.softmax(torch.cat([la, lb], dim=2), dim=2)
    return (p[:, :, :m] * ca).sum(2) + (p[:, :, m:] * cb).sum(2)


# --------------------------------------------------------------------------------------
# lightning indexer + top-k  (reference: ops_csa.py:503-554)
# --------------------------------------------------------------------------------------
def indexer_logits(q_idx, k_idx, w_idx, normalize_qk, scale=None):
    """``sum_h w[t,h] * relu(q[t,h] . k[n] * scale)``  -> ``[B,T,n]`` (no mask)."""
    cd = _cdtype(q_idx)
    qf, kf = q_idx.to(cd), k_idx.to(cd)
    if scale is None:
        scale = 1.0 if normalize_qk else q_idx.shape[-1] ** -0.5
    if normalize_qk:
        qf, kf = l2_normalize(qf), l2_normalize(kf)
    s = torch.relu(torch.einsum("bthd,bnd->bhtn", qf, kf) * scale)
    if w_idx is None:
        return s.sum(1)
    return torch.einsum("bhtn,bth->btn", s, w_idx.to(cd))


def topk_lowest_index(logits, k):
    """Top-k of each row, descending by value, ties by ascending index; -inf -> -1."""
    n = logits.shape[-1]
    S = min(k, n)
    vals, idx = torch.sort(logits, dim=-1, descending=True, stable=True)
    vals, idx = vals[..., :S], idx[..., :S]
    idx = idx.masked_fill(torch.isinf(vals) & (vals < 0), -1)
    if k > S:
        idx = torch.cat([idx, idx.new_full((*idx.shape[:-1], k - S), -1)], dim=-1)
    return idx


def lightning_indexer(q_idx, k_idx, w_idx, topk, *, m=None, t0=0, normalize_qk=False,
                      scale=None, n_visible=None, return_logits=False):
    """Indices ``[B,T,topk]`` (int64, -1 padded).  Causality: block b visible to the query
    at absolute position t iff ``b < (t+1)//m`` (``ops_csa.py:179-195``); ``t0`` is the
    absolute position of the first query row; ``n_visible`` overrides (decode)."""
    B, T = q_idx.shape[:2]
    n = k_idx.shape[1]
    if topk == 0:
        return torch.zeros(B, T, 0, dtype=torch.long)
    lg = indexer_logits(q_idx, k_idx, w_idx, normalize_qk, scale)
    if n_visible is not None:
        vis = torch.as_tensor(n_visible).reshape(-1, 1).expand(T, 1)
    elif m is not None:
        vis = ((torch.arange(T) + t0 + 1) // m).reshape(T, 1)
    else:
        vis = None
    if vis is not None:
        lg = lg.masked_fill(torch.arange(n).reshape(1, n) >= vis, NEG_INF)
    idx = topk_lowest_index(lg, topk)
    return (idx, lg) if return_logits else idx


# --------------------------------------------------------------------------------------
# joint softmax over [selected compressed entries U window entries] with optional sink
# (reference: ops_csa.py:1126-1155, ops_hca.py:165-192)
# --------------------------------------------------------------------------------------
def joint_attend(q, keys_a, valid_a, keys_w, valid_w, sink, scale):
    """q ``[N,nh,c]``; keys_a ``[N,Ka,c]`` with valid_a ``[N,Ka]``; keys_w ``[N,Kw,c]`` with
    valid_w ``[N,Kw]``; values are the keys.  ``p_j = e^{s_j}/(sum_i e^{s_i} + e^{sink})``.
    Rows with no valid entry give 0."""
    keys = torch.cat([keys_a, keys_w], dim=1)
    valid = torch.cat([valid_a, valid_w], dim=1)
    N, nh, c = q.shape
    if keys.shape[1] == 0:
        return torch.zeros(N, nh, c, dtype=q.dtype)
    s = torch.einsum("nhd,nkd->nhk", q, keys) * scale
    s = s.masked_fill(~valid.unsqueeze(1), NEG_INF)
    mx = s.amax(-1, keepdim=True)
    mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    if sink is not None:
        mx = torch.maximum(mx, sink.to(q.dtype).reshape(1, nh, 1))
    e = (s - mx).exp()
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + (sink.to(q.dtype).reshape(1, nh, 1) - mx).exp()
    p = e / den
    p = p.masked_fill(~valid.any(-1).reshape(N, 1, 1), 0.0)
    return torch.einsum("nhk,nkd->nhd", p, keys)


def _window_keys(local, t_lo, t_hi, win):
    """Window rows for queries t_lo..t_hi-1 of one batch element: ``[n,win,c]`` + validity."""
    T, c = local.shape
    pos = torch.arange(t_lo, t_hi).reshape(-1, 1) - (win - 1) + torch.arange(win).reshape(1, -1)
    valid = pos >= 0
    return local[pos.clamp(min=0)], valid


# --------------------------------------------------------------------------------------
# CSA / HCA full forward  (reference: ops_csa.py:576-1184, ops_hca.py:30-201)
# --------------------------------------------------------------------------------------
def _query_tiles(T, tile, query_rows):
    """(lo, hi) tiles of at most ``tile`` queries covering ``[0,T)`` or the given ranges."""
    spans = [(0, T)] if query_rows is None else [(max(0, lo), min(T, hi)) for lo, hi in query_rows]
    return [(t, min(hi, t + tile)) for lo, hi in spans for t in range(lo, hi, tile)]


def csa_forward(H, W_aKV, W_bKV, W_aZ, W_bZ, Ba, Bb, W_DQ, W_UQ, W_IUQ, W_w, W_KV_idx,
                W_Z_idx, B_idx, *, m, topk, nh, nIh, c, c_I, dc, scale=None, sliding_window=0,
                sink_logits=None, normalize_qk=False, tile=256, indices_override=None,
                return_aux=False, query_rows=None):
    """CSA forward; same rounding points as the reference (each projection output is stored
    in H.dtype; everything after is fp32).  Query-tiled.  ``query_rows`` (list of ``(lo, hi)``)
    restricts the indexer + attention stage to those query ranges (other output rows stay 0),
    so that a few tiles of a long sequence can be checked without paying for all of them."""
    B, T, d = H.shape
    if T == 0:
        return torch.zeros(B, 0, nh * c, dtype=H.dtype)
    T0 = T
    pad = (-T) % m
    if pad:
        H = torch.cat([H, H.new_zeros(B, pad, d)], dim=1)
        T += pad
    n = T // m
    Wcat = torch.cat([W_aKV, W_bKV, W_aZ, W_bZ, W_KV_idx, W_Z_idx], dim=0)
    Ca, Cb, Za, Zb, K_idx, Z_idx = F.linear(H, Wcat).split([c, c, c, c, c_I, c_I], dim=-1)
    C_comp = compress_kv_overlapped(Ca, Cb, Za, Zb, Ba, Bb, m)
    K_IComp = compress_kv(K_idx, Z_idx, B_idx, m)
    cQ = F.linear(H, W_DQ)
    q_idx = F.linear(cQ, W_IUQ).reshape(B, T, nIh, c_I)
    w_idx = F.linear(H, W_w)
    cd = _cdtype(H)
    q = F.linear(cQ, W_UQ).reshape(B, T, nh, c).to(cd)
    if normalize_qk:
        q = l2_normalize(q)
        Cn = l2_normalize(C_comp)
        local = l2_normalize(Ca.to(cd))
    else:
        Cn = C_comp.to(cd)
        local = Ca.to(cd)
    if scale is None:
        scale = 1.0 if normalize_qk else c ** -0.5
    out = torch.zeros(B, T, nh, c, dtype=cd)
    all_idx = torch.full((B, T, topk), -1, dtype=torch.long)
    for b in range(B):
        for t_lo, t_hi in _query_tiles(T, tile, query_rows):
            if indices_override is not None:
                idx = indices_override[b:b + 1, t_lo:t_hi]
            else:
                idx = lightning_indexer(q_idx[b:b + 1, t_lo:t_hi], K_IComp[b:b + 1],
                                        w_idx[b:b + 1, t_lo:t_hi], topk, m=m, t0=t_lo,
                                        normalize_qk=normalize_qk)
            all_idx[b, t_lo:t_hi] = idx[0]
            idx = idx[0]
            va = idx >= 0
            ka = Cn[b][idx.clamp(min=0)] if topk > 0 else torch.zeros(t_hi - t_lo, 0, c, dtype=cd)
            if sliding_window > 0:
                kw, vw = _window_keys(local[b], t_lo, t_hi, sliding_window)
            else:
                kw = torch.zeros(t_hi - t_lo, 0, c, dtype=cd)
                vw = torch.zeros(t_hi - t_lo, 0, dtype=torch.bool)
            out[b, t_lo:t_hi] = joint_attend(q[b, t_lo:t_hi], ka, va, kw, vw, sink_logits, scale)
    res = out.reshape(B, T, nh * c).to(H.dtype)[:, :T0]
    if return_aux:
        return res, dict(Ca=Ca[:, :T0], Cb=Cb[:, :T0], Za=Za[:, :T0], Zb=Zb[:, :T0],
                         K_idx=K_idx[:, :T0], Z_idx=Z_idx[:, :T0], C_comp=C_comp, K_IComp=K_IComp,
                         q_idx=q_idx, w_idx=w_idx, indices=all_idx, cQ=cQ)
    return res


def hca_forward(H, W_KV, W_Z, B_pos, W_DQ, W_UQ, *, m2, nh, c, dc, scale=1.0,
                sliding_window=0, sink_logits=None, W_KV_local=None, tile=512,
                return_aux=False, query_rows=None):
    """HCA forward (``ops_hca.py:117-201``): dense MQA over every visible compressed block.
    ``query_rows``: as in ``csa_forward``."""
    B, T, d = H.shape
    if T == 0:
        return torch.zeros(B, 0, nh * c, dtype=H.dtype)
    T0 = T
    pad = (-T) % m2
    if pad:
        H = torch.cat([H, H.new_zeros(B, pad, d)], dim=1)
        T += pad
    n = T // m2
    C = F.linear(H, W_KV)
    Z = F.linear(H, W_Z)
    cd = _cdtype(H)
    C_comp = compress_kv(C, Z, B_pos, m2)
    Cn = l2_normalize(C_comp)
    cQ = F.linear(H, W_DQ)
    q = l2_normalize(F.linear(cQ, W_UQ).reshape(B, T, nh, c).to(cd))
    loc_raw = C if W_KV_local is None else F.linear(H, W_KV_local)
    local = l2_normalize(loc_raw.to(cd))
    out = torch.zeros(B, T, nh, c, dtype=cd)
    for b in range(B):
        for t_lo, t_hi in _query_tiles(T, tile, query_rows):
            nq = t_hi - t_lo
            vis = ((torch.arange(t_lo, t_hi) + 1) // m2).reshape(-1, 1)
            va = torch.arange(n).reshape(1, -1) < vis
            ka = Cn[b].unsqueeze(0).expand(nq, n, c)
            if sliding_window > 0:
                kw, vw = _window_keys(local[b], t_lo, t_hi, sliding_window)
            else:
                kw = torch.zeros(nq, 0, c, dtype=cd)
                vw = torch.zeros(nq, 0, dtype=torch.bool)
            out[b, t_lo:t_hi] = joint_attend(q[b, t_lo:t_hi], ka, va, kw, vw, sink_logits, scale)
    res = out.reshape(B, T, nh * c).to(H.dtype)[:, :T0]
    if return_aux:
        return res, dict(C=C[:, :T0], Z=Z[:, :T0], C_comp=C_comp)
    return res


# --------------------------------------------------------------------------------------
# block-scaled 8-bit storage of compressed rows (no counterpart in the reference)
# --------------------------------------------------------------------------------------
FP8_MAX = 448.0
QBLOCK = 64


def quantize_rows(x, kind):
    """Per 64-element block: fp32 scale = max|x|/qmax (1.0 for an all-zero block);
    payload = round(x/scale) to e4m3 (``kind='fp8'``) or int8 (``kind='int8'``).
    Returns (payload, scales ``[..., c/64]``)."""
    xs = x.float().reshape(*x.shape[:-1], -1, QBLOCK)
    amax = xs.abs().amax(-1, keepdim=True)
    qmax = FP8_MAX if kind == "fp8" else 127.0
    scale = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
    y = xs / scale
    if kind == "fp8":
        payload = y.to(torch.float8_e4m3fn)
    else:
        payload = torch.clamp(torch.round(y), -127, 127).to(torch.int8)
    return payload.reshape(x.shape), scale.squeeze(-1)


def dequantize_rows(payload, scale):
    xs = payload.float().reshape(*payload.shape[:-1], -1, QBLOCK)
    return (xs * scale.unsqueeze(-1)).reshape(payload.shape)


# --------------------------------------------------------------------------------------
# decode caches  (reference: ops_decoding_cache.py)
# --------------------------------------------------------------------------------------
class CSACacheOracle:
    """State of ``CSADecodingCache`` (``ops_decoding_cache.py:407-1070``) held as dense
    tensors.  Completed block rows are stored rounded to ``dtype`` (``754-762``) and
    re-normalised in fp32 at every use (``919-924``); the window ring holds
    ``dtype(normalize(fp32(Ca)))`` (``725-730``) and is used as stored (``1022-1027``).
    ``kv_quant`` in {None,'fp8','int8'} additionally passes the stored rows through the
    block-scaled 8-bit format."""

    def __init__(self, B, c, c_I, m, win, dtype, kv_quant=None):
        self.B, self.c, self.c_I, self.m, self.win, self.dtype = B, c, c_I, m, win, dtype
        self.kv_quant = kv_quant
        self.tokens = 0
        self.acc = [torch.zeros(B, 0, w, dtype=dtype) for w in (c, c, c, c, c_I, c_I)]
        self.prev_Cb = None
        self.prev_Zb = None
        self.C_comp = torch.zeros(B, 0, c, dtype=dtype)
        self.K_IComp = torch.zeros(B, 0, c_I, dtype=dtype)
        self.window = torch.zeros(B, 0, c, dtype=dtype)

    def _store(self, rows):
        rows = rows.to(self.dtype)
        if self.kv_quant:
            rows = dequantize_rows(*quantize_rows(rows, self.kv_quant)).to(torch.float32)
        return rows

    def append(self, Ca, Cb, Za, Zb, K_idx, Z_idx, Ba, Bb, B_idx):
        new = [x.to(self.dtype) for x in (Ca, Cb, Za, Zb, K_idx, Z_idx)]
        Tn = Ca.shape[1]
        m = self.m
        if self.win > 0:
            w = l2_normalize(new[0].float()).to(self.dtype)
            self.window = torch.cat([self.window, w], dim=1)[:, -self.win:]
        self.acc = [torch.cat([a, x], dim=1) for a, x in zip(self.acc, new)]
        self.tokens += Tn
        nfull = self.acc[0].shape[1] // m
        if nfull:
            blk = [a[:, :nfull * m] for a in self.acc]
            self.acc = [a[:, nfull * m:].clone() for a in self.acc]
            # prepend the previous block's b-branch so the shifted overlap lines up
            if self.prev_Cb is None:
                rows = compress_kv_overlapped(blk[0], blk[1], blk[2], blk[3], Ba, Bb, m)
            else:
                z = torch.zeros_like(self.prev_Cb)
                rows = compress_kv_overlapped(
                    torch.cat([z, blk[0]], 1), torch.cat([self.prev_Cb, blk[1]], 1),
                    torch.cat([z, blk[2]], 1), torch.cat([self.prev_Zb, blk[3]], 1), Ba, Bb, m)[:, 1:]
            krows = compress_kv(blk[4], blk[5], B_idx, m)
            st = self._store(rows)
            self.C_comp = torch.cat([self.C_comp.to(st.dtype), st], dim=1)
            self.K_IComp = torch.cat([self.K_IComp, krows.to(self.dtype)], dim=1)
            self.prev_Cb = blk[1][:, -m:].clone()
            self.prev_Zb = blk[3][:, -m:].clone()

    def step(self, q, q_idx, w_idx, *, topk, sink_logits=None, scale=None, normalize_qk=True,
             return_indices=False, indices_override=None):
        """q ``[B,1,nh,c]`` fp32 (already normalised when normalize_qk), q_idx ``[B,1,nIh,c_I]``,
        w_idx ``[B,1,nIh]``  ->  fp32 ``[B,1,nh,c]``.  ``indices_override [B,1,k]`` replaces the indexer's
        selection (to check the attention on a selection that differs only by a near-tie)."""
        B, _, nh, c = q.shape
        t = self.tokens - 1
        nvis = min((t + 1) // self.m, self.C_comp.shape[1])
        if scale is None:
            scale = 1.0 if normalize_qk else c ** -0.5
        out = torch.zeros(B, 1, nh, c)
        Cn = self.C_comp.float()
        if normalize_qk:
            Cn = l2_normalize(Cn)
        if indices_override is not None:
            idx = indices_override.long()
        elif Cn.shape[1] > 0 and topk > 0:
            idx = lightning_indexer(q_idx.float(), self.K_IComp.float(), w_idx.float(), topk,
                                    n_visible=nvis, normalize_qk=normalize_qk)
        else:
            idx = torch.zeros(B, 1, 0, dtype=torch.long)
        for b in range(B):
            ib = idx[b, 0]
            ka = Cn[b][ib.clamp(min=0)].unsqueeze(0)
            va = (ib >= 0).unsqueeze(0)
            kw = self.window[b].float().unsqueeze(0)
            vw = torch.ones(1, kw.shape[1], dtype=torch.bool)
            out[b, 0] = joint_attend(q[b, 0].float().unsqueeze(0), ka, va, kw, vw, sink_logits, scale)[0]
        return (out, idx) if return_indices else out


class HCACacheOracle:
    """State of ``HCADecodingCache`` (``ops_decoding_cache.py:1077-1395``)."""

    def __init__(self, B, c, m2, win, dtype, kv_quant=None):
        self.B, self.c, self.m2, self.win, self.dtype = B, c, m2, win, dtype
        self.kv_quant = kv_quant
        self.tokens = 0
        self.acc = [torch.zeros(B, 0, c, dtype=dtype) for _ in range(2)]
        self.C_comp = torch.zeros(B, 0, c, dtype=dtype)
        self.window = torch.zeros(B, 0, c, dtype=dtype)

    def append(self, C, Z, B_pos):
        new = [x.to(self.dtype) for x in (C, Z)]
        if self.win > 0:
            w = l2_normalize(new[0].float()).to(self.dtype)
            self.window = torch.cat([self.window, w], dim=1)[:, -self.win:]
        self.acc = [torch.cat([a, x], dim=1) for a, x in zip(self.acc, new)]
        self.tokens += C.shape[1]
        nfull = self.acc[0].shape[1] // self.m2
        if nfull:
            blk = [a[:, :nfull * self.m2] for a in self.acc]
            self.acc = [a[:, nfull * self.m2:].clone() for a in self.acc]
            rows = compress_kv(blk[0], blk[1], B_pos, self.m2).to(self.dtype)
            if self.kv_quant:
                rows = dequantize_rows(*quantize_rows(rows, self.kv_quant))
            self.C_comp = torch.cat([self.C_comp.to(rows.dtype), rows], dim=1)

    def step(self, q, *, sink_logits=None, scale=None, normalize_qk=True):
        B, _, nh, c = q.shape
        t = self.tokens - 1
        n = self.C_comp.shape[1]
        nvis = min((t + 1) // self.m2, n)
        if scale is None:
            scale = 1.0 if normalize_qk else c ** -0.5
        Cn = self.C_comp.float()
        if normalize_qk:
            Cn = l2_normalize(Cn)
        out = torch.zeros(B, 1, nh, c)
        for b in range(B):
            ka = Cn[b].unsqueeze(0)
            va = (torch.arange(n) < nvis).unsqueeze(0)
            kw = self.window[b].float().unsqueeze(0)
            vw = torch.ones(1, kw.shape[1], dtype=torch.bool)
            out[b, 0] = joint_attend(q[b, 0].float().unsqueeze(0), ka, va, kw, vw, sink_logits, scale)[0]
        return out


# --------------------------------------------------------------------------------------
# layer glue  (reference: ops_fused.py)
# --------------------------------------------------------------------------------------
def layernorm_fp32(x, weight, bias, eps=1e-5):
    """LayerNorm evaluated in fp32, result cast back (``ops_fused.py:52-60``)."""
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    y = (xf - mu) * torch.rsqrt(var + eps) * weight.float() + bias.float()
    return y.to(x.dtype)


def short_conv(x, weight, bias, lookback=None):
    """Causal depthwise conv, kernel 3, over time (``ops_fused.py:505-527``).
    x ``[B,T,d]``; weight ``[d,1,3]``; lookback ``[B,2,d]`` or None (zeros)."""
    B, T, d = x.shape
    lb = x.new_zeros(B, 2, d) if lookback is None else lookback.to(x.dtype)
    xp = torch.cat([lb, x], dim=1).float()
    w = weight.float().reshape(d, 3)
    y = xp[:, 0:T] * w[:, 0] + xp[:, 1:T + 1] * w[:, 1] + xp[:, 2:T + 2] * w[:, 2] + bias.float()
    new_lb = torch.cat([lb, x], dim=1)[:, -2:].clone()
    return y.to(x.dtype), new_lb


def kda_layer_inputs(p, x_conv, H, HV, K, V, decay_scale=0.1):
    """Projections and activations of ``KDAHybridLayer`` in the input dtype
    (``ops_fused.py:571-581``)."""
    B, T, _ = x_conv.shape
    q = F.normalize(F.silu(F.linear(x_conv, p["q_proj.weight"])).view(B, T, H, K), dim=-1)
    k = F.normalize(F.silu(F.linear(x_conv, p["k_proj.weight"])).view(B, T, H, K), dim=-1)
    v = F.silu(F.linear(x_conv, p["v_proj.weight"])).view(B, T, HV, V)
    g = -F.softplus(F.linear(F.linear(x_conv, p["g_down.weight"]), p["g_up.weight"])).view(B, T, HV, K) * decay_scale
    beta = torch.sigmoid(F.linear(x_conv, p["beta.weight"]))
    return q, k, v, g, beta


@dataclass
class HybridSpec:
    """Geometry of the stack (field names follow ``HybridConfig``, ``ops_fused.py:65-92``)."""
    d_model: int = 256
    n_heads_qk: int = 4
    n_heads_v: int = 4
    head_dim_k: int = 64
    head_dim_v: int = 64
    kda_chunk_size: int = 64
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
    layout: list = field(default_factory=list)

    def build_layout(self, total_layers):
        unit = ["kda"] * self.n_kda + ["csa"] * self.n_csa + ["hca"] * self.n_hca
        out = []
        while len(out) < total_layers:
            out.extend(unit)
        self.layout = out[:total_layers]
        return self.layout


def hybrid_forward(spec: HybridSpec, params: dict, x, kda_states=None, lookbacks=None,
                   csa_indices=None, trace=None):
    """Pre-norm residual stack ``x = x + layer(LN(x))`` (``ops_fused.py:1075-1091``).
    ``params`` uses the reference's ``state_dict`` names (``layers.i.q_proj.weight`` ...).
    Returns (y, list of KDA states, list of conv lookbacks).  ``trace`` (a list) receives one
    dict per layer: its input ``x_in``, the operator output before ``o_proj`` (``core``) and
    the residual stream after the layer (``x_out``)."""
    B, T, d = x.shape
    s = spec
    states, lbs = [], []
    ki = 0
    for i, kind in enumerate(s.layout):
        p = {k[len(f"layers.{i}."):]: v for k, v in params.items() if k.startswith(f"layers.{i}.")}
        h = layernorm_fp32(x, params[f"norms.{i}.weight"], params[f"norms.{i}.bias"])
        if kind == "kda":
            xc, lb = short_conv(h, p["short_conv.weight"], p["short_conv.bias"],
                                None if lookbacks is None else lookbacks[ki])
            q, k, v, g, beta = kda_layer_inputs(p, xc, s.n_heads_qk, s.n_heads_v, s.head_dim_k,
                                                s.head_dim_v, s.kda_decay_scale)
            sc = float(torch.tensor(s.head_dim_k ** -0.5).to(x.dtype))
            st0 = None if kda_states is None else kda_states[ki]
            if s.kda_chunk_size >= 1 and T >= s.kda_chunk_size:
                o, st = chunk_kda(q, k, v, g, beta, sc, st0, s.kda_chunk_size)
            else:
                o, st = recurrent_kda(q, k, v, g, beta, sc, st0)
            core = o.reshape(B, T, -1)
            o = F.linear(core, p["o_proj.weight"])
            states.append(st)
            lbs.append(lb)
            ki += 1
        elif kind == "csa":
            o = csa_forward(h, p["W_aKV.weight"], p["W_bKV.weight"], p["W_aZ.weight"], p["W_bZ.weight"],
                            p["Ba"], p["Bb"], p["W_DQ.weight"], p["W_UQ.weight"], p["W_IUQ.weight"],
                            p["W_w.weight"], p["W_KV_idx.weight"], p["W_Z_idx.weight"], p["B_idx"],
                            m=s.csa_m, topk=s.csa_topk, nh=s.csa_nh, nIh=s.csa_nIh, c=s.csa_c,
                            c_I=s.csa_cI, dc=s.csa_dc, sliding_window=s.csa_sliding_window,
                            sink_logits=p["sink"], normalize_qk=True,
                            indices_override=None if csa_indices is None else csa_indices.get(i))
            core = o
            o = F.linear(o, p["o_proj.weight"])
        else:
            o = hca_forward(h, p["W_KV.weight"], p["W_Z.weight"], p["B_pos"], p["W_DQ.weight"],
                            p["W_UQ.weight"], m2=s.hca_m2, nh=s.hca_nh, c=s.hca_c, dc=s.hca_dc,
                            sliding_window=s.hca_sliding_window, sink_logits=p["sink"])
            core = o
            o = F.linear(o, p["o_proj.weight"])
        x_in, x = x, x + o
        if trace is not None:
            trace.append(dict(kind=kind, x_in=x_in, core=core, x_out=x))
    return x, states, lbs


class HybridDecodeOracle:
    """Layer-by-layer decode wiring (``run_decoding.py:601-851``): a multi-token call runs the
    full-sequence operators and fills the caches from the same projections; a one-token call
    appends to the caches and attends through them; KDA layers carry state + conv lookback."""

    def __init__(self, spec: HybridSpec, params: dict, kv_quant=None):
        self.spec, self.params, self.kv_quant = spec, params, kv_quant
        self.reset()

    def reset(self):
        self.states = {}
        self.lookbacks = {}
        self.caches = {}

    def _p(self, i):
        pre = f"layers.{i}."
        return {k[len(pre):]: v for k, v in self.params.items() if k.startswith(pre)}

    def forward(self, x):
        s = self.spec
        B, T, d = x.shape
        for i, kind in enumerate(s.layout):
            p = self._p(i)
            h = layernorm_fp32(x, self.params[f"norms.{i}.weight"], self.params[f"norms.{i}.bias"])
            if kind == "kda":
                xc, lb = short_conv(h, p["short_conv.weight"], p["short_conv.bias"], self.lookbacks.get(i))
                q, k, v, g, beta = kda_layer_inputs(p, xc, s.n_heads_qk, s.n_heads_v, s.head_dim_k,
                                                    s.head_dim_v, s.kda_decay_scale)
                sc = float(torch.tensor(s.head_dim_k ** -0.5).to(x.dtype))
                if s.kda_chunk_size >= 1 and T >= s.kda_chunk_size:
                    o, st = chunk_kda(q, k, v, g, beta, sc, self.states.get(i), s.kda_chunk_size)
                else:
                    o, st = recurrent_kda(q, k, v, g, beta, sc, self.states.get(i))
                self.states[i], self.lookbacks[i] = st, lb
                o = o.reshape(B, T, -1)
            elif kind == "csa":
                if i not in self.caches:
                    self.caches[i] = CSACacheOracle(B, s.csa_c, s.csa_cI, s.csa_m, s.csa_sliding_window,
                                                    x.dtype, self.kv_quant)
                cache = self.caches[i]
                kw = dict(m=s.csa_m, topk=s.csa_topk, nh=s.csa_nh, nIh=s.csa_nIh, c=s.csa_c, c_I=s.csa_cI,
                          dc=s.csa_dc, sliding_window=s.csa_sliding_window, sink_logits=p["sink"],
                          normalize_qk=True)
                W = [p[n] for n in ("W_aKV.weight", "W_bKV.weight", "W_aZ.weight", "W_bZ.weight", "Ba", "Bb",
                                    "W_DQ.weight", "W_UQ.weight", "W_IUQ.weight", "W_w.weight",
                                    "W_KV_idx.weight", "W_Z_idx.weight", "B_idx")]
                if T > 1:
                    o, aux = csa_forward(h, *W, return_aux=True, **kw)
                    cache.append(aux["Ca"], aux["Cb"], aux["Za"], aux["Zb"], aux["K_idx"], aux["Z_idx"],
                                 p["Ba"], p["Bb"], p["B_idx"])
                else:
                    Wcat = torch.cat([W[0], W[1], W[2], W[3], W[10], W[11]], dim=0)
                    Ca, Cb, Za, Zb, K_idx, Z_idx = F.linear(h, Wcat).split(
                        [s.csa_c] * 4 + [s.csa_cI] * 2, dim=-1)
                    cQ = F.linear(h, W[6])
                    q = F.linear(cQ, W[7]).reshape(B, 1, s.csa_nh, s.csa_c)
                    q_idx = F.linear(cQ, W[8]).reshape(B, 1, s.csa_nIh, s.csa_cI)
                    w_idx = F.linear(h, W[9])
                    cache.append(Ca, Cb, Za, Zb, K_idx, Z_idx, p["Ba"], p["Bb"], p["B_idx"])
                    oo = cache.step(l2_normalize(q.float()), q_idx.float(), w_idx.float(),
                                    topk=s.csa_topk, sink_logits=p["sink"], scale=1.0)
                    o = oo.reshape(B, 1, -1).to(x.dtype)
            else:
                if i not in self.caches:
                    self.caches[i] = HCACacheOracle(B, s.hca_c, s.hca_m2, s.hca_sliding_window, x.dtype,
                                                    self.kv_quant)
                cache = self.caches[i]
                if T > 1:
                    o, aux = hca_forward(h, p["W_KV.weight"], p["W_Z.weight"], p["B_pos"], p["W_DQ.weight"],
                                         p["W_UQ.weight"], m2=s.hca_m2, nh=s.hca_nh, c=s.hca_c, dc=s.hca_dc,
                                         sliding_window=s.hca_sliding_window, sink_logits=p["sink"],
                                         return_aux=True)
                    cache.append(aux["C"], aux["Z"], p["B_pos"])
                else:
                    C = F.linear(h, p["W_KV.weight"])
                    Z = F.linear(h, p["W_Z.weight"])
                    q = F.linear(F.linear(h, p["W_DQ.weight"]), p["W_UQ.weight"]).reshape(B, 1, s.hca_nh, s.hca_c)
                    cache.append(C, Z, p["B_pos"])
                    oo = cache.step(l2_normalize(q.float()), sink_logits=p["sink"], scale=1.0)
                    o = oo.reshape(B, 1, -1).to(x.dtype)
            x = x + F.linear(o, p["o_proj.weight"])
        return x


class StandaloneDecodeOracle:
    """The single-operator decode modules ``KDAAttnDecoding`` / ``CSAAttnDecoding`` / ``HCAAttnDecoding``
    (``run_decoding.py:234-598``): operator + output projection, no pre-norm, no residual.  ``p`` holds the
    module's ``state_dict``; ``cfg`` its constructor arguments."""

    def __init__(self, kind, p, **cfg):
        self.kind, self.p, self.cfg = kind, p, cfg
        self.state = self.lookback = self.cache = None

    def forward(self, x):
        p, c = self.p, self.cfg
        B, T, _ = x.shape
        if self.kind == "kda":
            H, K, V = c["H"], c["K"], c["V"]
            xc, self.lookback = short_conv(x, p["short_conv.weight"], p["short_conv.bias"], self.lookback)
            pp = {"q_proj.weight": p["q.weight"], "k_proj.weight": p["k.weight"], "v_proj.weight": p["v.weight"],
                  "g_down.weight": p["g_down.weight"], "g_up.weight": p["g_up.weight"], "beta.weight": p["beta.weight"]}
            q, k, v, g, beta = kda_layer_inputs(pp, xc, H, H, K, V, 0.1)
            o, self.state = recurrent_kda(q, k, v, g, beta, K ** -0.5, self.state)
            return F.linear(o.reshape(B, T, H * V), p["o.weight"])
        if self.kind == "csa":
            if self.cache is None:
                self.cache = CSACacheOracle(B, c["c"], c["c_I"], c["m"], c["sliding_window"], x.dtype)
            W = [p[n] for n in ("W_aKV.weight", "W_bKV.weight", "W_aZ.weight", "W_bZ.weight", "Ba", "Bb", "W_DQ.weight",
                                "W_UQ.weight", "W_IUQ.weight", "W_w.weight", "W_KV_idx.weight", "W_Z_idx.weight", "B_idx")]
            if T > 1:
                o, aux = csa_forward(x, *W, m=c["m"], topk=c["topk"], nh=c["nh"], nIh=c["nIh"], c=c["c"], c_I=c["c_I"],
                                     dc=c["dc"], sliding_window=c["sliding_window"], sink_logits=p["sink"],
                                     normalize_qk=True, return_aux=True)
                self.cache.append(aux["Ca"], aux["Cb"], aux["Za"], aux["Zb"], aux["K_idx"], aux["Z_idx"], p["Ba"], p["Bb"],
                                  p["B_idx"])
            else:
                Wcat = torch.cat([W[0], W[1], W[2], W[3], W[10], W[11]], dim=0)
                Ca, Cb, Za, Zb, K_idx, Z_idx = F.linear(x, Wcat).split([c["c"]] * 4 + [c["c_I"]] * 2, dim=-1)
                cQ = F.linear(x, W[6])
                q = F.linear(cQ, W[7]).reshape(B, 1, c["nh"], c["c"])
                q_idx = F.linear(cQ, W[8]).reshape(B, 1, c["nIh"], c["c_I"])
                w_idx = F.linear(x, W[9])
                self.cache.append(Ca, Cb, Za, Zb, K_idx, Z_idx, p["Ba"], p["Bb"], p["B_idx"])
                o = self.cache.step(l2_normalize(q.float()), q_idx.float(), w_idx.float(), topk=c["topk"],
                                    sink_logits=p["sink"], scale=1.0).reshape(B, 1, -1).to(x.dtype)
            return F.linear(o, p["o_proj.weight"])
        if self.cache is None:
            self.cache = HCACacheOracle(B, c["c"], c["m2"], c["sliding_window"], x.dtype)
        if T > 1:
            o, aux = hca_forward(x, p["W_KV.weight"], p["W_Z.weight"], p["B_pos"], p["W_DQ.weight"], p["W_UQ.weight"],
                                 m2=c["m2"], nh=c["nh"], c=c["c"], dc=c["dc"], sliding_window=c["sliding_window"],
                                 sink_logits=p["sink"], return_aux=True)
            self.cache.append(aux["C"], aux["Z"], p["B_pos"])
        else:
            C = F.linear(x, p["W_KV.weight"])
            Z = F.linear(x, p["W_Z.weight"])
            q = F.linear(F.linear(x, p["W_DQ.weight"]), p["W_UQ.weight"]).reshape(B, 1, c["nh"], c["c"])
            self.cache.append(C, Z, p["B_pos"])
            o = self.cache.step(l2_normalize(q.float()), sink_logits=p["sink"], scale=1.0).reshape(B, 1, -1).to(x.dtype)
        return F.linear(o, p["o_proj.weight"])

