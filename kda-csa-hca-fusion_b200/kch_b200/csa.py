"""CSA operators on the B200 kernels, with the reference signatures.

Mirrors ``csa_compress_kv`` (ops_csa.py:198-234), ``csa_compress_kv_overlapped`` (237-305),
``csa_lightning_indexer`` (330-573) and ``naive_csa`` (576-1184) of 183600/kda-csa-hca-fusion.
Forward only: the straight-through surrogate of the reference (ops_csa.py:1033-1099) exists for
training and is not part of this path; asking for it with gradients enabled raises.
"""
from __future__ import annotations

import torch

from . import _lib


def _as_rows(t):
    """Return (tensor, ld, batch_stride_rows) such that element [b,t,d] lives at
    base + (b*batch_stride_rows + t)*ld + d; copies only when the view cannot be expressed."""
    B, T, c = t.shape
    if T == 0 or B == 0:
        t = t.contiguous()
        return t, c, T
    ok = (t.stride(-1) == 1 or c == 1)
    ld = t.stride(1) if T > 1 else max(c, t.stride(1))
    if ok and ld >= c and (B == 1 or (t.stride(0) % ld == 0 and t.stride(0) >= T * ld)):
        return t, ld, (t.stride(0) // ld if B > 1 else T)
    t = t.contiguous()
    return t, c, T


def linear(x, W, residual=None, epilogue=None, group=1):
    """``F.linear(x, W)`` (+ residual) through the C ABI.  x ``[..., K]`` (last dim dense), W ``[N, K]``.
    ``epilogue``: list of ``(width, act, param)`` column segments covering all N output columns, applied with
    the rounding points of the unfused chain (``group`` = head width of the silu+L2-norm activation)."""
    _lib.require_cuda(x, W, fn="linear")
    lib = _lib.load()
    K = x.shape[-1]
    N = W.shape[0]
    if W.shape[1] != K:
        raise ValueError(f"linear: weight shape {tuple(W.shape)} does not match input features {K}")
    if W.dtype != x.dtype:
        raise ValueError(f"linear: weight dtype {W.dtype} does not match input dtype {x.dtype}")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1 and K > 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    lda = x2.stride(0) if M > 1 else K
    if W.stride(-1) != 1:
        W = W.contiguous()
    out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    r2, ldr = None, 0
    if residual is not None:
        r2 = residual.reshape(-1, N)
        if r2.stride(-1) != 1:
            r2 = r2.contiguous()
        ldr = r2.stride(0) if M > 1 else N
    ep = None
    if epilogue:
        ep = _lib.Epilogue()
        ep.n_segments, ep.group = len(epilogue), int(group)
        end = 0
        for i, (width, act, param) in enumerate(epilogue):
            end += int(width)
            ep.seg_end[i], ep.seg_act[i], ep.seg_param[i] = end, int(act), float(param)
        if end != N:
            raise ValueError(f"linear: epilogue segments cover {end} columns, the weight has {N} rows")
    with torch.cuda.device(x.device):
        _lib.check(lib.kch_linear_ex(_lib.ptr(x2), _lib.ptr(W), _lib.ptr(out), _lib.ptr(r2), M, N, K, lda,
                                     W.stride(0), N, ldr, _lib.dtype_tag(x.dtype), ep, _lib.stream()))
    return out.reshape(*lead, N)


def linear_kslabs(a_slabs, W, residual=None):
    """``F.linear(cat(a_slabs, dim=-1), W)`` (+ residual) without forming the concatenation: ``a_slabs``
    ``[n_slabs, M, K / n_slabs]`` contiguous bf16 (the rank-major buffer an all-gather of per-GPU head slices leaves
    behind), W ``[N, K]``.  Returns ``[M, N]``."""
    _lib.require_cuda(a_slabs, W, fn="linear_kslabs")
    lib = _lib.load()
    n_slabs, M, kl = a_slabs.shape
    N, K = W.shape
    if K != n_slabs * kl:
        raise ValueError(f"linear_kslabs: weight has {K} input features, the slabs hold {n_slabs} x {kl}")
    if a_slabs.dtype != torch.bfloat16 or W.dtype != torch.bfloat16:
        raise ValueError("linear_kslabs: bf16 operands only")
    a_slabs = a_slabs.contiguous()
    if W.stride(-1) != 1:
        W = W.contiguous()
    out = torch.empty(M, N, dtype=a_slabs.dtype, device=a_slabs.device)
    r2, ldr = None, 0
    if residual is not None:
        r2 = residual.reshape(-1, N)
        if r2.stride(-1) != 1:
            r2 = r2.contiguous()
        ldr = r2.stride(0) if M > 1 else N
    with torch.cuda.device(a_slabs.device):
        _lib.check(lib.kch_linear_kslabs(_lib.ptr(a_slabs), _lib.ptr(W), _lib.ptr(out), _lib.ptr(r2), M, N, K, n_slabs,
                                         W.stride(0), N, ldr, _lib.KCH_BF16, _lib.stream()))
    return out


def fuse_rows(*weights):
    """Row-concatenate weight matrices and zero-pad the row count to a multiple of 8, so that every column
    slice of the fused projection output keeps a 16-byte-aligned row stride (TMA-readable in place)."""
    w = torch.cat([x.detach() for x in weights], dim=0)
    pad = (-w.shape[0]) % 8
    if pad:
        w = torch.cat([w, w.new_zeros(pad, w.shape[1])], dim=0)
    return w.contiguous()


def rownorm(x, normalize=True, out_dtype=torch.float32):
    """``F.normalize(x.float(), dim=-1)`` of a ``[..., c]`` tensor, evaluated in fp32 and stored as
    ``out_dtype`` (row-strided 3-D views are read in place)."""
    if not normalize:
        return x.to(out_dtype)
    lib = _lib.load()
    c = x.shape[-1]
    lead = x.shape[:-1]
    if x.is_contiguous() or x.dim() != 3:
        x3 = x.contiguous().reshape(1, -1, c)
    else:
        x3 = x
    x3, ld, bsr = _as_rows(x3)
    if bsr != x3.shape[1]:
        x3, ld = x3.contiguous(), c
    rows = x3.shape[0] * x3.shape[1]
    y = torch.empty(rows, c, dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.kch_rownorm(_lib.ptr(x3), ld, _lib.ptr(y), None, rows, c, _lib.dtype_tag(x.dtype),
                                   _lib.dtype_tag(out_dtype), _lib.stream()))
    return y.reshape(*lead, c)


def csa_compress_kv(C, Z, B_pos, m: int):
    """``[B,T,c] -> [B,T//m,c]`` fp32: per block and channel ``softmax_m(Z + B_pos) . C``."""
    B, T, c = C.shape
    if m < 1:
        raise ValueError(f"compression factor m={m} must be >= 1")
    if T % m != 0:
        raise ValueError(f"T={T} must be divisible by m={m}")
    _lib.require_cuda(C, Z, B_pos, fn="csa_compress_kv")
    lib = _lib.load()
    C2, ld, bsr = _as_rows(C)
    Z2, ldz, bsrz = _as_rows(Z)
    if (ldz, bsrz) != (ld, bsr):
        C2, Z2 = C.contiguous(), Z.contiguous()
        ld, bsr = c, T
    Bp = B_pos.contiguous()
    n = T // m
    out = torch.empty(B, n, c, dtype=torch.float32, device=C.device)
    with torch.cuda.device(C.device):
        _lib.check(lib.kch_compress_kv(_lib.ptr(C2), _lib.ptr(Z2), _lib.ptr(Bp), _lib.ptr(out), B, T, c, m, ld, bsr,
                                       n * c, _lib.dtype_tag(C.dtype), _lib.dtype_tag(Bp.dtype), _lib.stream()))
    return out


def csa_compress_kv_overlapped(Ca, Cb, Za, Zb, Ba, Bb, m: int, *, prev_Cb=None, prev_Zb=None):
    """Two-branch overlapped compression.  ``prev_Cb/prev_Zb [B,m,c]`` (an extension used by the decode
    caches) give the b-branch of the block before block 0; without them block 0 has no b-branch."""
    B, T, c = Ca.shape
    if m < 1:
        raise ValueError(f"compression factor m={m} must be >= 1")
    if T % m != 0:
        raise ValueError(f"T={T} must be divisible by m={m}")
    if T == 0:
        return Ca.new_zeros(B, 0, c)
    _lib.require_cuda(Ca, Cb, Za, Zb, fn="csa_compress_kv_overlapped")
    lib = _lib.load()
    views = [_as_rows(x) for x in (Ca, Cb, Za, Zb)]
    if len({(v[1], v[2]) for v in views}) != 1:
        views = [(x.contiguous(), c, T) for x in (Ca, Cb, Za, Zb)]
    ld, bsr = views[0][1], views[0][2]
    Ba_, Bb_ = Ba.contiguous(), Bb.contiguous()
    if Bb_.dtype != Ba_.dtype:
        Bb_ = Bb_.to(Ba_.dtype)
    pc = pz = None
    if prev_Cb is not None:
        pc, pz = prev_Cb.to(Ca.dtype).contiguous(), prev_Zb.to(Ca.dtype).contiguous()
    n = T // m
    out = torch.empty(B, n, c, dtype=torch.float32, device=Ca.device)
    with torch.cuda.device(Ca.device):
        _lib.check(lib.kch_compress_kv_overlapped(
            _lib.ptr(views[0][0]), _lib.ptr(views[1][0]), _lib.ptr(views[2][0]), _lib.ptr(views[3][0]),
            _lib.ptr(Ba_), _lib.ptr(Bb_), _lib.ptr(pc), _lib.ptr(pz), c, _lib.ptr(out), B, T, c, m, ld, bsr, n * c,
            _lib.dtype_tag(Ca.dtype), _lib.dtype_tag(Ba_.dtype), _lib.stream()))
    return out


def indexer_topk(q_idx, k_idx, w_idx, topk, *, m=0, t0=0, n_visible=-1, normalize_qk=False, scale=None,
                 sorted_output=True, k_prenormalized=False, k_batch_stride=0):
    """Kernel-level entry: int32 indices ``[B,T,topk]``.  Visibility ``n < (t0+t+1)//m`` (``m>0``),
    ``n < n_visible`` (``n_visible>=0``) or unrestricted."""
    lib = _lib.load()
    B, T, HI, DI = q_idx.shape
    n = k_idx.shape[1]
    if scale is None:
        scale = 1.0 if normalize_qk else DI ** -0.5
    dev = q_idx.device
    idx = torch.empty(B, T, topk, dtype=torch.int32, device=dev)
    if B == 0 or T == 0 or topk == 0:
        return idx
    # bf16 queries of the production width are scored as they lie (a strided slice of the fused projection is
    # fine): exact tensor-core operands, their norm divides the dot product inside the kernel
    raw_q = (q_idx.dtype == torch.bfloat16 and DI == 64 and normalize_qk and n > 0 and q_idx.stride(-1) == 1
             and q_idx.stride(2) == DI and q_idx.stride(1) % 8 == 0 and q_idx.data_ptr() % 16 == 0
             and (B == 1 or q_idx.stride(0) == T * q_idx.stride(1)))
    if raw_q:
        kn = k_idx if k_prenormalized else rownorm(k_idx, True).contiguous()
        wf = None if w_idx is None else w_idx.float().contiguous()
        nbytes = int(lib.kch_indexer_workspace_bytes_ex(B, T, n, _lib.KCH_BF16))
        ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.kch_indexer_topk_ex(_lib.ptr(q_idx), _lib.KCH_BF16, q_idx.stride(1), 1, _lib.ptr(kn),
                                               _lib.ptr(wf), _lib.ptr(idx), B, T, n, HI, DI, int(topk), float(scale),
                                               int(m), int(t0), int(n_visible), 1 if sorted_output else 0,
                                               int(k_batch_stride), _lib.ptr(ws), nbytes, _lib.stream()))
        return idx
    qn = rownorm(q_idx.contiguous(), normalize_qk).contiguous()
    if k_prenormalized:
        kn = k_idx                      # fp32, rows dense, batch entries k_batch_stride elements apart
    elif normalize_qk:
        kn = rownorm(k_idx, True).contiguous()
    else:
        kn = k_idx.float().contiguous()
    wf = None if w_idx is None else w_idx.float().contiguous()
    nbytes = int(lib.kch_indexer_workspace_bytes(B, T, n, HI, DI))
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.kch_indexer_topk(_lib.ptr(qn), _lib.ptr(kn), _lib.ptr(wf), _lib.ptr(idx), B, T, n, HI, DI,
                                        int(topk), float(scale), int(m), int(t0), int(n_visible),
                                        1 if sorted_output else 0, int(k_batch_stride), _lib.ptr(ws), nbytes,
                                        _lib.stream()))
    return idx


def csa_lightning_indexer(q_idx, k_idx, w_idx, topk: int, scale=None, causal_block_mask=None,
                          return_soft_weights: bool = False, *, ste_mode: str = "topk_columns",
                          normalize_qk: bool = False, m: int | None = None, t0: int = 0):
    """Top-k over compressed indexer keys; returns int64 indices ``[B,T,topk]`` (-1 padded).

    The reference passes causality as a dense boolean ``[T,n_blocks]`` mask built by
    ``_causal_block_mask`` (ops_csa.py:179-195).  The kernel evaluates the same rule ``b < (t+1)//m``
    arithmetically, so pass ``m`` (and ``t0``) instead; a mask tensor is still accepted when it is of
    that form (each row a prefix of ones), which covers every call site of the reference.
    """
    if topk < 0:
        raise ValueError(f"topk={topk} must be >= 0 (0 selects zero blocks)")
    if q_idx.shape[-1] < 1:
        raise ValueError(f"q_idx.shape[-1]={q_idx.shape[-1]} must be >= 1 "
                         f"(indexer key dimension c_I must be positive)")
    if ste_mode not in ("topk_columns", "full_softmax", "aux_contrastive"):
        raise ValueError(f"ste_mode={ste_mode!r} must be one of 'topk_columns', 'full_softmax', or "
                         f"'aux_contrastive'.")
    if ste_mode == "aux_contrastive":
        raise NotImplementedError("ste_mode='aux_contrastive' is reserved for a future implementation")
    if return_soft_weights:
        raise NotImplementedError("return_soft_weights=True (the training-time straight-through surrogate) "
                                  "is outside the forward path of the b200 backend")
    _lib.require_cuda(q_idx, k_idx, fn="csa_lightning_indexer")
    B, T = q_idx.shape[:2]
    n = k_idx.shape[1]
    if topk == 0:
        return torch.zeros(B, T, 0, dtype=torch.long, device=q_idx.device)
    if causal_block_mask is None and m is None:
        idx = indexer_topk(q_idx, k_idx, w_idx, topk, normalize_qk=normalize_qk, scale=scale)
    elif m is not None:
        idx = indexer_topk(q_idx, k_idx, w_idx, topk, m=m, t0=t0, normalize_qk=normalize_qk, scale=scale)
    else:
        cbm = causal_block_mask
        if cbm.dim() != 2 or cbm.shape[-1] != n:
            raise ValueError(f"causal_block_mask must be [T, n_blocks]=[{T}, {n}], got {tuple(cbm.shape)}")
        nvis = cbm.sum(-1)
        prefix = torch.arange(n, device=cbm.device)[None, :] < nvis[:, None]
        if not bool((prefix == cbm.bool()).all()):
            raise NotImplementedError("csa_lightning_indexer(b200): causal_block_mask rows must be prefixes "
                                      "of visible blocks (the block-causal rule b < (t+1)//m)")
        nv = nvis.tolist()
        if len(nv) == 1:
            idx = indexer_topk(q_idx, k_idx, w_idx, topk, n_visible=int(nv[0]), normalize_qk=normalize_qk,
                               scale=scale)
        else:
            # recover m from the staircase: the visible count of row t is min((t+1)//m, n_blocks)
            first = next((t for t, x in enumerate(nv) if x > 0), None)
            m_rec = len(nv) + 1 if first is None else first + 1
            if [min((t + 1) // m_rec, n) for t in range(len(nv))] != nv:
                raise NotImplementedError("csa_lightning_indexer(b200): mask is not of the form (t+1)//m")
            idx = indexer_topk(q_idx, k_idx, w_idx, topk, m=m_rec, normalize_qk=normalize_qk, scale=scale)
    return idx.long()


def mma_attention_eligible(dtype, c, nh, normalize_qk, scale):
    """Geometry served by the tensor-core attention kernel: bf16, c=128, <=16 heads, cosine scoring."""
    return dtype == torch.bfloat16 and c == 128 and nh <= 16 and bool(normalize_qk) and abs(float(scale)) <= 16.0


def attend(q, comp, *, nh, c, sel=None, m=0, t0=0, n_visible=-1, q_normalize=False, comp_norms=None,
           comp_scales=None, comp_kind=None, win=None, sliding_window=0, win_mode=0, win_len=0, sink=None,
           scale=1.0, out_dtype=torch.float32, win_t0=0):
    """Kernel-level joint-softmax attention.  q ``[B,T,nh*c]`` view (row-strided ok); comp ``[B,n,c]``
    contiguous or None; win ``[B,Tw,c]`` (row-strided ok) or None."""
    lib = _lib.load()
    B, T = q.shape[0], q.shape[1]
    a = _lib.AttendArgs()
    q3, qld, qbsr = _as_rows(q.reshape(B, T, nh * c))
    if qbsr != T:
        q3 = q3.contiguous()
        qld = nh * c
    a.q, a.q_dtype, a.q_ld, a.q_normalize = q3.data_ptr(), _lib.dtype_tag(q3.dtype), qld, int(q_normalize)
    a.B, a.T, a.nh, a.c = B, T, nh, c
    keep = [q3]
    if comp is not None and comp.shape[1] > 0:
        comp = comp if comp.is_contiguous() else comp.contiguous()
        keep.append(comp)
        a.comp = comp.data_ptr()
        a.comp_dtype = comp_kind if comp_kind is not None else _lib.dtype_tag(comp.dtype)
        a.comp_ld, a.comp_batch_rows, a.n_comp = c, comp.shape[1], comp.shape[1]
        if comp_norms is not None:
            keep.append(comp_norms)
            a.comp_norms = comp_norms.data_ptr()
        if comp_scales is not None:
            keep.append(comp_scales)
            a.comp_scales = comp_scales.data_ptr()
    else:
        a.comp, a.n_comp = None, 0
    if sel is not None:
        sel = sel.to(torch.int32).contiguous()
        keep.append(sel)
        a.sel_indices, a.topk = sel.data_ptr(), sel.shape[-1]
    a.m, a.t0, a.n_visible = int(m), int(t0), int(n_visible)
    if win is not None and sliding_window > 0:
        w3, wld, wbsr = _as_rows(win)
        keep.append(w3)
        a.win, a.win_dtype, a.win_ld, a.win_batch_rows = w3.data_ptr(), _lib.dtype_tag(w3.dtype), wld, wbsr
        a.sliding_window, a.win_mode, a.win_len = int(sliding_window), int(win_mode), int(win_len)
        a.win_t0 = int(win_t0)
    if sink is not None:
        sink = sink.contiguous()
        keep.append(sink)
        a.sink, a.sink_dtype = sink.data_ptr(), _lib.dtype_tag(sink.dtype)
    a.scale = float(scale)
    out = torch.empty(B, T, nh * c, dtype=out_dtype, device=q.device)
    a.out, a.out_dtype = out.data_ptr(), _lib.dtype_tag(out_dtype)
    with torch.cuda.device(q.device):
        _lib.check(lib.kch_attend(a, _lib.stream()))
    return out


def naive_csa(H, W_aKV, W_bKV, W_aZ, W_bZ, Ba, Bb, W_DQ, W_UQ, W_IUQ, W_w, W_KV_idx, W_Z_idx, B_idx, *,
              m: int, topk: int, nh: int, nIh: int, c: int, c_I: int, dc: int, scale=None,
              sliding_window: int = 0, sink_logits=None, use_ste: bool = True, ste_mode: str = "topk_columns",
              normalize_qk: bool = False, fuse_projections: bool = True, return_projections: bool = False,
              _fused_weight=None, _fused_q_weight=None, _return_indices: bool = False, _aux: dict | None = None,
              _q_rows=None):
    """Full CSA forward: ``[B,T,d] -> [B,T,nh*c]`` in ``H.dtype``; weights in ``nn.Linear`` layout.

    ``_fused_weight`` (optional) is the row-concatenation ``[W_aKV;W_bKV;W_aZ;W_bZ;W_KV_idx;W_Z_idx;
    W_DQ;W_w]`` prepared once by the layer object so the eight input projections run as one GEMM.
    ``_aux`` (a dict, for stage-by-stage checks) receives the intermediate tensors exactly as the kernels saw
    them: ``q_idx``, ``w_idx``, ``K_IComp``, ``C_comp``, ``q`` (padded length).
    ``_q_rows = (lo, hi)`` (sharding by query rows): only the queries ``lo..hi-1`` are scored and attended, against
    the keys of tokens ``0..hi-1`` (``H`` may be longer, the rest is not read); returns ``[B, hi-lo, nh*c]``.
    """
    B_, T, d = H.shape
    if m < 1:
        raise ValueError(f"compression factor m={m} must be >= 1")
    if topk < 0:
        raise ValueError(f"topk={topk} must be >= 0 (0 disables sparse selection)")
    if nh < 1:
        raise ValueError(f"nh={nh} must be >= 1")
    if c < 1:
        raise ValueError(f"c={c} must be >= 1")
    if dc < 1:
        raise ValueError(f"dc={dc} must be >= 1")
    if c_I < 1:
        raise ValueError(f"c_I={c_I} must be >= 1 (indexer key dim)")
    if nIh < 1:
        raise ValueError(f"nIh={nIh} must be >= 1 (indexer head count)")
    if sliding_window < 0:
        raise ValueError(f"sliding_window={sliding_window} must be >= 0 (0 disables the branch)")
    if use_ste and torch.is_grad_enabled() and H.requires_grad:
        raise NotImplementedError("naive_csa(b200): use_ste=True with gradients enabled is the training path; "
                                  "call under torch.no_grad() or pass use_ste=False")
    _lib.require_cuda(H, fn="naive_csa")
    device = H.device
    if T == 0:
        out_empty = torch.zeros(B_, 0, nh * c, dtype=H.dtype, device=device)
        if return_projections:
            z = lambda w: torch.zeros(B_, 0, w, dtype=H.dtype, device=device)  # noqa: E731
            return out_empty, (z(c), z(c), z(c), z(c), z(c_I), z(c_I))
        return out_empty
    for name, w in (("W_aKV", W_aKV), ("W_bKV", W_bKV), ("W_aZ", W_aZ), ("W_bZ", W_bZ),
                    ("W_KV_idx", W_KV_idx), ("W_Z_idx", W_Z_idx)):
        if w.device != H.device:
            raise ValueError(f"naive_csa: {name}.device={w.device} does not match H.device={H.device}. "
                             f"All weights must be on the same device as the input.")
        if w.dtype != H.dtype:
            raise ValueError(f"naive_csa: {name}.dtype={w.dtype} does not match H.dtype={H.dtype}. "
                             f"All weights must share the input's dtype (cast before calling if needed).")
        if w.shape[1] != d:
            raise ValueError(f"naive_csa: {name}.shape={tuple(w.shape)} — second dim (in_features) must "
                             f"equal d={d} (H.shape[-1]).")
    q_lo = 0
    if _q_rows is not None:
        q_lo, q_hi = int(_q_rows[0]), int(_q_rows[1])
        if not 0 <= q_lo < q_hi <= T:
            raise ValueError(f"naive_csa: _q_rows={_q_rows} must satisfy 0 <= lo < hi <= T={T}")
        if return_projections:
            raise ValueError("naive_csa: _q_rows and return_projections cannot be combined")
        H, T = H[:, :q_hi], q_hi
    original_T = T
    pad = (-T) % m
    if pad:
        H = torch.nn.functional.pad(H, (0, 0, 0, pad))
        T += pad
    n_blocks = T // m
    if _fused_weight is None:
        _fused_weight = fuse_rows(W_aKV, W_bKV, W_aZ, W_bZ, W_KV_idx, W_Z_idx, W_DQ, W_w)
    proj = linear(H, _fused_weight)                                     # [B,T,4c+2cI+dc+nIh (+pad)]
    Ca, Cb, Za, Zb, K_idx_raw, Z_idx, cQ, w_idx = proj[..., :4 * c + 2 * c_I + dc + nIh].split(
        [c, c, c, c, c_I, c_I, dc, nIh], dim=-1)
    C_comp = csa_compress_kv_overlapped(Ca, Cb, Za, Zb, Ba, Bb, m)      # [B,n,c] fp32
    K_IComp = csa_compress_kv(K_idx_raw, Z_idx, B_idx, m)               # [B,n,cI] fp32
    W_q = _fused_q_weight if _fused_q_weight is not None else torch.cat([W_UQ, W_IUQ], dim=0)
    if q_lo:                                                            # the query side for this rank's rows only
        cQ, w_idx = cQ[:, q_lo:], w_idx[:, q_lo:]
    qq = linear(cQ, W_q)                                                # [B,Tq,nh*c + nIh*cI]
    q, q_idx = qq[..., :nh * c + nIh * c_I].split([nh * c, nIh * c_I], dim=-1)
    q_idx = q_idx.unflatten(-1, (nIh, c_I))                             # a view of the fused projection
    indices = None
    if topk > 0:
        indices = indexer_topk(q_idx, K_IComp, w_idx, topk, m=m, t0=q_lo, normalize_qk=normalize_qk,
                               sorted_output=False)
    if _aux is not None:
        _aux.update(q_idx=q_idx, w_idx=w_idx, K_IComp=K_IComp, C_comp=C_comp, q=q)
    if scale is None:
        scale = 1.0 if normalize_qk else c ** -0.5
    # production geometry in bf16: unit keys are kept in bf16 for the tensor-core attention kernel
    kdt = torch.bfloat16 if mma_attention_eligible(H.dtype, c, nh, normalize_qk, scale) else torch.float32
    C_comp_n = rownorm(C_comp, normalize_qk, kdt)
    local = None
    if sliding_window > 0:
        local = rownorm(Ca, normalize_qk, kdt) if normalize_qk else Ca
    out = attend(q, C_comp_n if topk > 0 else None, nh=nh, c=c, sel=indices, m=m, t0=q_lo, q_normalize=normalize_qk,
                 win=local, sliding_window=sliding_window, sink=sink_logits, scale=scale, out_dtype=H.dtype,
                 win_t0=q_lo)
    out_final = out[:, :original_T - q_lo]
    res = [out_final]
    if return_projections:
        res.append(tuple(x[:, :original_T] for x in (Ca, Cb, Za, Zb, K_idx_raw, Z_idx)))
    if _return_indices:
        res.append(None if indices is None else indices[:, :original_T])
    return res[0] if len(res) == 1 else tuple(res)
