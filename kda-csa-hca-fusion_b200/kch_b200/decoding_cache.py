"""Incremental decode caches on the B200 kernels, with the reference step API.

Mirrors ``CSADecodingCache`` (ops_decoding_cache.py:407-1070), ``HCADecodingCache`` (1077-1395) and the
window ring (251-400) of 183600/kda-csa-hca-fusion.  All state lives in preallocated device tensors;
the counters stay on the host as in the reference (one counter set per cache: every sequence of the
batch advances in lock-step).  ``kv_quant='fp8'|'int8'`` stores the compressed rows block-scaled in
8 bits (one fp32 scale per 64 elements), which the reference does not have.

Storage roundings reproduced from the reference: completed rows are rounded to the cache dtype when
stored (754-762) and re-normalised in fp32 at use (919-924) — here the fp32 norm of the stored row is
kept next to it; the ring holds ``dtype(normalize(fp32(Ca)))`` (725-730) and is used as stored.
"""
from __future__ import annotations

import torch

from . import _lib
from .csa import attend, csa_compress_kv, csa_compress_kv_overlapped, indexer_topk, rownorm

_QUANT = {None: None, "fp8": _lib.KCH_FP8_E4M3, "int8": _lib.KCH_INT8}


def _validate_cache_dtype(dtype):
    try:
        is_float = torch.empty((), dtype=dtype).is_floating_point()
    except (TypeError, RuntimeError) as exc:
        raise TypeError(f"cache dtype must be a floating torch.dtype, got {dtype!r}") from exc
    if not is_float:
        raise TypeError(f"cache dtype must be floating-point, got {dtype!r}")
    if dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"the b200 caches store float32 or bfloat16, got {dtype!r}")


class _SlidingWindowRingBuffer:
    """Last ``win`` keys per sequence, written at slot ``n_written % win``."""

    def __init__(self, B, win, c, device, dtype):
        if win < 1:
            raise ValueError(f"_SlidingWindowRingBuffer: win={win} must be >= 1")
        self.B, self.win, self.c = B, win, c
        self.device, self.dtype = torch.device(device), dtype
        self._buf = torch.zeros(B, win, c, device=self.device, dtype=dtype)
        self._n = 0

    def reset(self):
        self._buf.zero_()
        self._n = 0

    @property
    def n_valid(self):
        return min(self._n, self.win)

    def get(self):
        """Contents in causal order (oldest first): ``[B, n_valid, c]``."""
        if self._n <= self.win:
            return self._buf[:, :self._n]
        h = self._n % self.win
        return torch.cat([self._buf[:, h:], self._buf[:, :h]], dim=1)

    def append(self, x):
        """x ``[B,T_new,c]`` already in storage form."""
        Tn = x.shape[1]
        x = x[:, -self.win:].to(self.dtype)
        k = x.shape[1]
        pos = (torch.arange(self._n + Tn - k, self._n + Tn, device=self.device) % self.win)
        self._buf.index_copy_(1, pos, x)
        self._n += Tn


def _row_norms(x):
    """fp32 ``max(||row||, 1e-12)`` of ``x [B,n,c]`` (the divisor the kernels use for a stored row)."""
    lib = _lib.load()
    B, n, c = x.shape
    x = x.contiguous()
    out = torch.empty(B, n, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.kch_rownorm(_lib.ptr(x), c, None, _lib.ptr(out), B * n, c, _lib.dtype_tag(x.dtype), _lib.KCH_F32,
                                   _lib.stream()))
    return out


class _CacheBase:
    # The counters live twice: Python ints (the reference's interface) and an int32 vector on the device that
    # the one-token kernels read, so that a decode step has no host argument that changes between tokens.
    def _init_counters(self):
        self._ctr = torch.zeros(_lib.CTR_WORDS, dtype=torch.int32, device=self.device)
        self._ws_attn = None
        self._ws_idx = None

    def _sync_counters(self):
        """Host counters -> device mirror (after reset, a bulk append or any direct edit of the counters)."""
        vals = [0] * _lib.CTR_WORDS
        vals[_lib.CTR_ACC_LEN] = self._acc_len
        vals[_lib.CTR_N_BLOCKS] = self._n_blocks
        vals[_lib.CTR_RING_N] = 0 if self._sw is None else self._sw._n
        vals[_lib.CTR_HAS_PREV] = int(getattr(self, "_has_prev", False))
        vals[_lib.CTR_TOKENS] = self._n_tokens_seen
        self._ctr.copy_(torch.tensor(vals, dtype=torch.int32))

    def _advance(self, m):
        """The host half of one appended token (the device half is kch_cache_advance)."""
        if self._sw is not None:
            self._sw._n += 1
        self._n_tokens_seen += 1
        if self._acc_len + 1 == m:
            self._n_blocks += 1
            self._acc_len = 0
            if hasattr(self, "_has_prev"):
                self._has_prev = True
        else:
            self._acc_len += 1

    # ---- state export / import (not in the reference: checkpoint / resume of a long decode session) ----------
    def export_state(self):
        """Everything needed to continue decoding elsewhere: a dict of tensors (clones, trimmed to the rows in
        use) and Python counters.  ``import_state`` of a cache built with the same constructor arguments
        restores it exactly."""
        nb = self._n_blocks
        st = {
            "kind": type(self).__name__, "B": self.B, "c": self.c, "win": self.win, "dtype": str(self.dtype),
            "kv_quant": self.kv_quant, "n_blocks": nb, "acc_len": self._acc_len, "n_tokens_seen": self._n_tokens_seen,
            "acc": [a.clone() for a in self._acc],
            "comp": None if self._comp is None else self._comp[:, :nb].clone(),
            "scales": None if self._scales is None else self._scales[:, :nb].clone(),
            "norms": None if self._norms is None else self._norms[:, :nb].clone(),
            "ring": None if self._sw is None else self._sw._buf.clone(),
            "ring_n": 0 if self._sw is None else self._sw._n,
        }
        if hasattr(self, "_prev"):
            st.update(prev=[p.clone() for p in self._prev], has_prev=self._has_prev,
                      kcomp=None if self._kcomp is None else self._kcomp[:, :nb].clone(),
                      kcomp_norms=None if self._kcomp_norms is None else self._kcomp_norms[:, :nb].clone())
        return st

    def import_state(self, st):
        if st["kind"] != type(self).__name__ or st["B"] != self.B or st["c"] != self.c or st["win"] != self.win \
                or st["dtype"] != str(self.dtype) or st["kv_quant"] != self.kv_quant:
            raise ValueError(f"{type(self).__name__}.import_state: the state was exported from a cache with a "
                             f"different geometry ({st['kind']}, B={st['B']}, c={st['c']}, win={st['win']}, "
                             f"{st['dtype']}, kv_quant={st['kv_quant']})")
        self.reset()
        nb = int(st["n_blocks"])
        if nb:
            self._grow(nb)
            self._comp[:, :nb] = st["comp"].to(self.device)
            self._norms[:, :nb] = st["norms"].to(self.device)
            if self._scales is not None:
                self._scales[:, :nb] = st["scales"].to(self.device)
            if hasattr(self, "_prev"):
                self._kcomp[:, :nb] = st["kcomp"].to(self.device)
                self._kcomp_norms[:, :nb] = st["kcomp_norms"].to(self.device)
        for a, src in zip(self._acc, st["acc"]):
            a.copy_(src)
        if hasattr(self, "_prev"):
            for p_, src in zip(self._prev, st["prev"]):
                p_.copy_(src)
            self._has_prev = bool(st["has_prev"])
        if self._sw is not None:
            self._sw._buf.copy_(st["ring"])
            self._sw._n = int(st["ring_n"])
        self._n_blocks, self._acc_len, self._n_tokens_seen = nb, int(st["acc_len"]), int(st["n_tokens_seen"])
        self._sync_counters()

    def _decode_attend_ok(self, nh):
        return self.c == 128 and nh <= 16

    def _attend_decode(self, q, sel, topk, m, nh, scale, sink, normalize_qk, q_normalize=False, out_dtype=None):
        """One-token attention over the cache storage with the split kernel; geometry from the device counters.
        ``q`` may be a row-strided view (a slice of a fused projection) in fp32 or bf16."""
        lib = _lib.load()
        B = self.B
        q2 = q.reshape(B, nh * self.c) if q.is_contiguous() else q.flatten(1)
        if q2.dim() != 2 or q2.stride(-1) != 1 or (B > 1 and q2.stride(0) < nh * self.c):
            q2 = q2.contiguous().view(B, nh * self.c)
        out_dtype = torch.float32 if out_dtype is None else out_dtype
        need = int(lib.kch_attend_decode_workspace_bytes(B, nh, self.c))
        if self._ws_attn is None or self._ws_attn.numel() < need:
            self._ws_attn = torch.empty(need, dtype=torch.uint8, device=self.device)
        out = torch.empty(B, nh * self.c, dtype=out_dtype, device=self.device)
        a = _lib.AttendDecodeArgs()
        a.q, a.q_dtype, a.q_normalize = q2.data_ptr(), _lib.dtype_tag(q2.dtype), int(q_normalize)
        a.q_ld = q2.stride(0) if B > 1 else nh * self.c
        a.B, a.nh, a.c = B, nh, self.c
        if self._comp is not None:
            a.comp = self._comp.data_ptr()
            a.comp_dtype = self._kind if self._kind is not None else _lib.dtype_tag(self.dtype)
            a.capacity = self._comp.shape[1]
            a.comp_norms = self._norms.data_ptr() if normalize_qk else None
            a.comp_scales = None if self._scales is None else self._scales.data_ptr()
            if sel is not None:
                a.sel_indices, a.topk = sel.data_ptr(), int(topk)
        a.m = int(m)
        if self._sw is not None:
            a.win, a.win_dtype, a.sliding_window = self._sw._buf.data_ptr(), _lib.dtype_tag(self._sw.dtype), self.win
        if sink is not None:
            sk = sink if sink.is_contiguous() else sink.contiguous()
            a.sink, a.sink_dtype = sk.data_ptr(), _lib.dtype_tag(sk.dtype)
        a.scale = float(scale)
        a.out, a.out_dtype = out.data_ptr(), _lib.dtype_tag(out_dtype)
        a.counters = self._ctr.data_ptr()
        a.workspace, a.workspace_bytes = self._ws_attn.data_ptr(), self._ws_attn.numel()
        with torch.cuda.device(self.device):
            _lib.check(lib.kch_attend_decode(a, _lib.stream()))
        return out

    def _alloc_rows(self, cap):
        B, c, dev = self.B, self.c, self.device
        if self._kind is None:
            comp = torch.empty(B, cap, c, dtype=self.dtype, device=dev)
            scales = None
        else:
            comp = torch.empty(B, cap, c, dtype=torch.uint8, device=dev)
            scales = torch.empty(B, cap, c // 64, dtype=torch.float32, device=dev)
        norms = torch.ones(B, cap, dtype=torch.float32, device=dev)
        return comp, scales, norms

    def _grow(self, required):
        old = 0 if self._comp is None else self._comp.shape[1]
        if required <= old:
            return
        cap = max(required, max(1, old * 2))
        comp, scales, norms = self._alloc_rows(cap)
        nb = self._n_blocks
        if nb:
            comp[:, :nb] = self._comp[:, :nb]
            norms[:, :nb] = self._norms[:, :nb]
            if scales is not None:
                scales[:, :nb] = self._scales[:, :nb]
        self._comp, self._scales, self._norms = comp, scales, norms
        self._grow_extra(cap, nb)

    def _grow_extra(self, cap, nb):
        pass

    def reserve(self, n_blocks):
        """Pre-size the compressed-row storage (avoids reallocation during a long decode)."""
        self._grow(int(n_blocks))

    def _store_rows(self, rows_f32, start):
        """rows ``[B,nb,c]`` fp32 -> storage at block offset ``start`` (+ norms of the stored rows)."""
        lib = _lib.load()
        B, nb, c = rows_f32.shape
        r = rows_f32.to(self.dtype)
        tmp_norm = torch.empty(B, nb, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            if self._kind is None:
                self._comp[:, start:start + nb] = r
                _lib.check(lib.kch_rownorm(_lib.ptr(r), c, None, _lib.ptr(tmp_norm), B * nb, c,
                                           _lib.dtype_tag(self.dtype), _lib.KCH_F32, _lib.stream()))
            else:
                payload = torch.empty(B, nb, c, dtype=torch.uint8, device=self.device)
                sc = torch.empty(B, nb, c // 64, dtype=torch.float32, device=self.device)
                _lib.check(lib.kch_quantize_rows(_lib.ptr(r), c, _lib.ptr(payload), _lib.ptr(sc), _lib.ptr(tmp_norm),
                                                 B * nb, c, self._kind, _lib.dtype_tag(self.dtype), _lib.stream()))
                self._comp[:, start:start + nb] = payload
                self._scales[:, start:start + nb] = sc
        self._norms[:, start:start + nb] = tmp_norm

    def _dequant(self, nb):
        if self._comp is None:
            return None
        if self._kind is None:
            return self._comp[:, :nb]
        raw = self._comp[:, :nb]
        if self._kind == _lib.KCH_FP8_E4M3:
            vals = raw.view(torch.float8_e4m3fn).float()
        else:
            vals = raw.view(torch.int8).float()
        B, n, c = vals.shape
        return (vals.reshape(B, n, c // 64, 64) * self._scales[:, :nb].unsqueeze(-1)).reshape(B, n, c).to(self.dtype)

    def _attend(self, q, sel, nvis, nh, scale, sink, normalize_qk):
        nb = self._n_blocks
        win_len = 0 if self._sw is None else self._sw.n_valid
        return attend(q, None if nb == 0 else self._comp, nh=nh, c=self.c, sel=sel, n_visible=nvis,
                      q_normalize=False, comp_norms=self._norms if (normalize_qk and nb) else None,
                      comp_scales=self._scales, comp_kind=self._kind if self._kind is not None else None,
                      win=None if self._sw is None else self._sw._buf, sliding_window=self.win, win_mode=1,
                      win_len=win_len, sink=sink, scale=scale, out_dtype=torch.float32)


class CSADecodingCache(_CacheBase):
    """Decode cache of a CSA layer: partial-block accumulator, compressed rows + indexer keys,
    sliding-window ring.  ``append_step`` then ``forward_step`` per token."""

    def __init__(self, B, c, c_I, m, win, device, dtype, *, kv_quant=None):
        if B < 1:
            raise ValueError(f"B={B} must be >= 1")
        if c < 1:
            raise ValueError(f"c={c} must be >= 1")
        if c_I < 1:
            raise ValueError(f"c_I={c_I} must be >= 1")
        if m < 1:
            raise ValueError(f"m={m} must be >= 1")
        if win < 0:
            raise ValueError(f"win={win} must be >= 0 (0 disables SW)")
        if kv_quant not in _QUANT:
            raise ValueError(f"kv_quant={kv_quant!r} must be None, 'fp8' or 'int8'")
        if kv_quant is not None and c % 64 != 0:
            raise ValueError(f"kv_quant needs c={c} to be a multiple of 64 (one scale per 64 elements)")
        self.B, self.c, self.c_I, self.m, self.win = B, c, c_I, m, win
        _validate_cache_dtype(dtype)
        self.device, self.dtype = torch.device(device), dtype
        if self.device.type != "cuda":
            raise RuntimeError("CSADecodingCache(b200) requires a CUDA device; there is no CPU fallback")
        self.kv_quant, self._kind = kv_quant, _QUANT[kv_quant]
        self._normalize_qk = True
        self.reset()

    def reset(self):
        B, m, c, cI, dev, dt = self.B, self.m, self.c, self.c_I, self.device, self.dtype
        self._acc = [torch.zeros(B, m, w, dtype=dt, device=dev) for w in (c, c, c, c, cI, cI)]
        self._acc_len = 0
        self._prev = [torch.zeros(B, m, c, dtype=dt, device=dev) for _ in range(2)]
        self._has_prev = False
        self._comp = self._scales = self._norms = None
        self._kcomp = self._kcomp_norms = None
        self._sw = _SlidingWindowRingBuffer(B, self.win, c, dev, dt) if self.win > 0 else None
        self._n_tokens_seen = 0
        self._n_blocks = 0
        self._init_counters()

    def _grow_extra(self, cap, nb):
        k = torch.empty(self.B, cap, self.c_I, dtype=self.dtype, device=self.device)
        kn = torch.ones(self.B, cap, dtype=torch.float32, device=self.device)
        if nb:
            k[:, :nb] = self._kcomp[:, :nb]
            kn[:, :nb] = self._kcomp_norms[:, :nb]
        self._kcomp, self._kcomp_norms = k, kn
        self._ws_idx = None

    # ---- properties of the reference object --------------------------------------------------------
    @property
    def n_tokens_seen(self):
        return self._n_tokens_seen

    @property
    def n_blocks(self):
        return self._n_blocks

    @property
    def accumulator_len(self):
        return self._acc_len

    @property
    def C_comp(self):
        return self._dequant(self._n_blocks)

    @property
    def K_IComp(self):
        return None if self._kcomp is None else self._kcomp[:, :self._n_blocks]

    @property
    def sw_buffer(self):
        return self._sw

    def to(self, device=None, dtype=None):
        if dtype is not None and dtype != self.dtype:
            raise NotImplementedError("CSADecodingCache(b200).to(dtype=...): rebuild the cache in the new dtype")
        if device is not None and torch.device(device) != self.device:
            raise NotImplementedError("CSADecodingCache(b200).to(device=...): caches are bound to their GPU")
        return self

    # ---- append ---------------------------------------------------------------------------------------
    def append_step(self, Ca_new, Cb_new, Za_new, Zb_new, K_idx_new, Z_idx_new, Ba, Bb, B_idx):
        B, T_new, c = Ca_new.shape
        if B != self.B:
            raise ValueError(f"CSADecodingCache.append_step: batch size {B} does not match cache's B={self.B}. "
                             f"Call reset() between sequences with different batch sizes.")
        if c != self.c:
            raise ValueError(f"CSADecodingCache.append_step: c={c} does not match cache's c={self.c}.")
        if K_idx_new.shape[-1] != self.c_I:
            raise ValueError(f"CSADecodingCache.append_step: c_I={K_idx_new.shape[-1]} does not match "
                             f"cache's c_I={self.c_I}.")
        for name, t in (("Cb_new", Cb_new), ("Za_new", Za_new), ("Zb_new", Zb_new), ("K_idx_new", K_idx_new),
                        ("Z_idx_new", Z_idx_new)):
            if t.shape[1] != T_new:
                raise ValueError(f"CSADecodingCache.append_step: {name}.shape[1]={t.shape[1]} does not match "
                                 f"Ca_new.shape[1]={T_new}. All inputs must share the same T_new.")
        if T_new == 0:
            return []
        new = [x.to(device=self.device, dtype=self.dtype) for x in (Ca_new, Cb_new, Za_new, Zb_new, K_idx_new, Z_idx_new)]
        biases = [x.to(device=self.device, dtype=self.dtype).contiguous() for x in (Ba, Bb, B_idx)]
        first_new = self._n_blocks
        if T_new == 1:
            self._append_one(new, biases)
        else:
            self._append_many(new, biases)
        return list(range(first_new, self._n_blocks))

    def _append_one(self, new, biases):
        lib = _lib.load()
        m = self.m
        self._grow(self._n_blocks + 1)      # the kernel learns on the device whether this token closes a block
        a = _lib.CacheAppendArgs()
        a.B, a.c, a.c_I, a.m, a.win, a.dtype = self.B, self.c, self.c_I, m, self.win, _lib.dtype_tag(self.dtype)
        rows = [x[:, 0] for x in new]
        rows = [r if r.stride(-1) == 1 else r.contiguous() for r in rows]
        ldc = {r.stride(0) if self.B > 1 else self.c for r in rows[:4]}
        ldi = {r.stride(0) if self.B > 1 else self.c_I for r in rows[4:]}
        if len(ldc) != 1 or len(ldi) != 1:
            rows = [r.contiguous() for r in rows]
            ldc, ldi = {self.c}, {self.c_I}
        a.Ca, a.Cb, a.Za, a.Zb, a.K_idx, a.Z_idx = (r.data_ptr() for r in rows)
        a.ld_c, a.ld_i = ldc.pop(), ldi.pop()
        a.acc_Ca, a.acc_Cb, a.acc_Za, a.acc_Zb, a.acc_K_idx, a.acc_Z_idx = (x.data_ptr() for x in self._acc)
        a.acc_len = self._acc_len
        a.prev_Cb, a.prev_Zb, a.has_prev = self._prev[0].data_ptr(), self._prev[1].data_ptr(), int(self._has_prev)
        a.Ba, a.Bb, a.B_idx = (x.data_ptr() for x in biases)
        if self._comp is not None:
            a.comp = self._comp.data_ptr()
            a.comp_scales = None if self._scales is None else self._scales.data_ptr()
            a.comp_norms = self._norms.data_ptr()
            a.kcomp, a.kcomp_norms = self._kcomp.data_ptr(), self._kcomp_norms.data_ptr()
            a.capacity = self._comp.shape[1]
        a.comp_kind = self._kind if self._kind is not None else _lib.dtype_tag(self.dtype)
        a.n_blocks = self._n_blocks
        if self._sw is not None:
            a.ring, a.ring_pos = self._sw._buf.data_ptr(), self._sw._n % self.win
        a.normalize = int(self._normalize_qk)
        a.counters = self._ctr.data_ptr()
        with torch.cuda.device(self.device):
            _lib.check(lib.kch_cache_append_token_advance(a, _lib.stream()))   # the last CTA advances the device counters
        self._advance(m)

    def _append_many(self, new, biases):
        m, T_new = self.m, new[0].shape[1]
        if self._sw is not None:
            tail = new[0][:, -self.win:]
            keys = rownorm(tail, True).to(self.dtype) if self._normalize_qk else tail
            self._sw._n += T_new - tail.shape[1]
            self._sw.append(keys)
        staged = [torch.cat([a[:, :self._acc_len], x], dim=1) for a, x in zip(self._acc, new)]
        total = staged[0].shape[1]
        nb = total // m
        if nb:
            self._grow(self._n_blocks + nb)
            full = [s[:, :nb * m].contiguous() for s in staged]
            rows = csa_compress_kv_overlapped(full[0], full[1], full[2], full[3], biases[0], biases[1], m,
                                              prev_Cb=self._prev[0] if self._has_prev else None,
                                              prev_Zb=self._prev[1] if self._has_prev else None)
            self._store_rows(rows, self._n_blocks)
            krows = csa_compress_kv(full[4], full[5], biases[2], m).to(self.dtype)
            self._kcomp[:, self._n_blocks:self._n_blocks + nb] = krows
            self._kcomp_norms[:, self._n_blocks:self._n_blocks + nb] = _row_norms(krows)
            self._prev[0].copy_(full[1][:, -m:])
            self._prev[1].copy_(full[3][:, -m:])
            self._has_prev = True
            self._n_blocks += nb
        rest = total - nb * m
        for a, s in zip(self._acc, staged):
            if rest:
                a[:, :rest] = s[:, nb * m:]
        self._acc_len = rest
        self._n_tokens_seen += T_new
        self._sync_counters()

    # ---- attend -----------------------------------------------------------------------------------------
    def forward_step(self, q, q_idx, w_idx, *, topk, nh, nIh, scale=None, sink_logits=None, use_ste=True,
                     ste_mode="topk_columns", normalize_qk=True, _return_indices=False, _q_normalize=False,
                     _out_dtype=None):
        B, T_new = q.shape[0], q.shape[1]
        if T_new != 1:
            raise ValueError(f"CSADecodingCache.forward_step: T_new={T_new} must be 1. For multi-token chunks, "
                             f"call append_step + forward_step in a loop (or use naive_csa on the full chunk and "
                             f"populate the cache via the prefill path).")
        if B != self.B:
            raise ValueError(f"CSADecodingCache.forward_step: batch size {B} does not match cache's B={self.B}.")
        if q.shape[2] != nh:
            raise ValueError(f"q.shape[2]={q.shape[2]} does not match nh={nh}.")
        if q_idx.shape[2] != nIh:
            raise ValueError(f"q_idx.shape[2]={q_idx.shape[2]} does not match nIh={nIh}.")
        if q.device != self.device:
            raise ValueError(f"CSADecodingCache.forward_step: q.device={q.device} does not match cache's "
                             f"device={self.device}. Call cache.to(device=q.device) or move q to the cache's device.")
        if use_ste and torch.is_grad_enabled() and q.requires_grad:
            raise NotImplementedError("forward_step(b200): the straight-through surrogate is a training path")
        t = self._n_tokens_seen - 1
        core_scale = (1.0 if normalize_qk else self.c ** -0.5) if scale is None else float(scale)
        nb = self._n_blocks
        nvis = min((t + 1) // self.m, nb)
        sel = None
        if topk > 0 and self._kcomp is not None and nIh <= 64 and nIh * self.c_I <= 1024:
            # stored keys + their norms are scored in place; row count and visible prefix come from the device counters
            sel = self._indexer_decode(q_idx, w_idx, topk, normalize_qk)
        elif nb > 0 and topk > 0:
            sel = indexer_topk(q_idx.float(), self._kcomp[:, :nb].float().contiguous(), w_idx.float(), topk,
                               n_visible=nvis, normalize_qk=normalize_qk, sorted_output=False)
        elif topk > 0:
            sel = torch.full((B, 1, topk), -1, dtype=torch.int32, device=self.device)
        if topk == 0:
            out = self._attend_no_comp(q, nh, core_scale, sink_logits)
        elif self._decode_attend_ok(nh) and self._comp is not None:
            out = self._attend_decode(q, sel, topk, self.m, nh, core_scale, sink_logits, normalize_qk,
                                      q_normalize=_q_normalize, out_dtype=_out_dtype)
        else:
            if _q_normalize:
                q = rownorm(q.contiguous(), True)
            out = self._attend(q.float(), sel, nvis, nh, core_scale, sink_logits, normalize_qk)
            if _out_dtype is not None:
                out = out.to(_out_dtype)
        out = out.reshape(B, 1, nh, self.c)
        return (out, sel) if _return_indices else out

    def _indexer_decode(self, q_idx, w_idx, topk, normalize_qk):
        lib = _lib.load()
        B, _, HI, DI = q_idx.shape
        cap = self._kcomp.shape[1]
        need = int(lib.kch_decode_indexer_workspace_bytes(B, cap))
        if self._ws_idx is None or self._ws_idx.numel() < need:
            self._ws_idx = torch.empty(need, dtype=torch.uint8, device=self.device)
        def rows(x, width):          # [B, width] view with unit inner stride (a projection slice is fine as it is)
            x2 = x.reshape(B, width) if x.is_contiguous() else x.flatten(1)
            if x2.dtype not in (torch.float32, torch.bfloat16):
                x2 = x2.float()
            if x2.stride(-1) != 1 or (B > 1 and x2.stride(0) < width):
                x2 = x2.contiguous()
            return x2, (x2.stride(0) if B > 1 else width)
        qf, q_ld = rows(q_idx, HI * DI)
        wf, w_ld = (None, 0) if w_idx is None else rows(w_idx, HI)
        idx = torch.empty(B, 1, topk, dtype=torch.int32, device=self.device)
        scale = 1.0 if normalize_qk else DI ** -0.5
        with torch.cuda.device(self.device):
            _lib.check(lib.kch_decode_indexer_topk(
                _lib.ptr(qf), _lib.dtype_tag(qf.dtype), q_ld, _lib.ptr(self._kcomp), _lib.dtype_tag(self.dtype),
                _lib.ptr(self._kcomp_norms), _lib.ptr(wf), 0 if wf is None else _lib.dtype_tag(wf.dtype), w_ld,
                _lib.ptr(idx), B, cap, HI, DI, int(topk), int(normalize_qk), scale, self.m, self._ctr.data_ptr(),
                _lib.ptr(self._ws_idx), self._ws_idx.numel(), _lib.stream()))
        return idx

    def _attend_no_comp(self, q, nh, scale, sink):
        win_len = 0 if self._sw is None else self._sw.n_valid
        return attend(q.float(), None, nh=nh, c=self.c, sel=None, n_visible=0, q_normalize=False,
                      win=None if self._sw is None else self._sw._buf, sliding_window=self.win, win_mode=1,
                      win_len=win_len, sink=sink, scale=scale, out_dtype=torch.float32)


class HCADecodingCache(_CacheBase):
    """Decode cache of an HCA layer: partial-block accumulator, compressed rows, window ring."""

    def __init__(self, B, c, m2, win, device, dtype, *, kv_quant=None):
        if B < 1:
            raise ValueError(f"B={B} must be >= 1")
        if c < 1:
            raise ValueError(f"c={c} must be >= 1")
        if m2 < 1:
            raise ValueError(f"m2={m2} must be >= 1")
        if win < 0:
            raise ValueError(f"win={win} must be >= 0 (0 disables SW)")
        if kv_quant not in _QUANT:
            raise ValueError(f"kv_quant={kv_quant!r} must be None, 'fp8' or 'int8'")
        if kv_quant is not None and c % 64 != 0:
            raise ValueError(f"kv_quant needs c={c} to be a multiple of 64 (one scale per 64 elements)")
        self.B, self.c, self.m2, self.win = B, c, m2, win
        _validate_cache_dtype(dtype)
        self.device, self.dtype = torch.device(device), dtype
        if self.device.type != "cuda":
            raise RuntimeError("HCADecodingCache(b200) requires a CUDA device; there is no CPU fallback")
        self.kv_quant, self._kind = kv_quant, _QUANT[kv_quant]
        self._normalize_qk = True
        self.reset()

    def reset(self):
        B, m, c, dev, dt = self.B, self.m2, self.c, self.device, self.dtype
        self._acc = [torch.zeros(B, m, c, dtype=dt, device=dev) for _ in range(2)]
        self._acc_len = 0
        self._comp = self._scales = self._norms = None
        self._sw = _SlidingWindowRingBuffer(B, self.win, c, dev, dt) if self.win > 0 else None
        self._n_tokens_seen = 0
        self._n_blocks = 0
        self._init_counters()

    @property
    def n_tokens_seen(self):
        return self._n_tokens_seen

    @property
    def n_blocks(self):
        return self._n_blocks

    @property
    def accumulator_len(self):
        return self._acc_len

    @property
    def C_comp(self):
        return self._dequant(self._n_blocks)

    @property
    def sw_buffer(self):
        return self._sw

    def to(self, device=None, dtype=None):
        if dtype is not None and dtype != self.dtype:
            raise NotImplementedError("HCADecodingCache(b200).to(dtype=...): rebuild the cache in the new dtype")
        if device is not None and torch.device(device) != self.device:
            raise NotImplementedError("HCADecodingCache(b200).to(device=...): caches are bound to their GPU")
        return self

    def append_step(self, C_new, Z_new, B_pos):
        B, T_new, c = C_new.shape
        if B != self.B:
            raise ValueError(f"HCADecodingCache.append_step: batch size {B} does not match cache's B={self.B}. "
                             f"Call reset() between sequences with different batch sizes.")
        if c != self.c:
            raise ValueError(f"HCADecodingCache.append_step: c={c} does not match cache's c={self.c}.")
        if Z_new.shape[1] != T_new:
            raise ValueError(f"HCADecodingCache.append_step: Z_new.shape[1]={Z_new.shape[1]} does not match "
                             f"C_new.shape[1]={T_new}.")
        if T_new == 0:
            return []
        new = [x.to(device=self.device, dtype=self.dtype) for x in (C_new, Z_new)]
        bias = B_pos.to(device=self.device, dtype=self.dtype).contiguous()
        first_new = self._n_blocks
        if T_new == 1:
            self._append_one(new, bias)
        else:
            self._append_many(new, bias)
        return list(range(first_new, self._n_blocks))

    def _append_one(self, new, bias):
        lib = _lib.load()
        m = self.m2
        self._grow(self._n_blocks + 1)
        a = _lib.CacheAppendArgs()
        a.B, a.c, a.c_I, a.m, a.win, a.dtype = self.B, self.c, 0, m, self.win, _lib.dtype_tag(self.dtype)
        rows = [x[:, 0] for x in new]
        rows = [r if r.stride(-1) == 1 else r.contiguous() for r in rows]
        lds = {r.stride(0) if self.B > 1 else self.c for r in rows}
        if len(lds) != 1:
            rows = [r.contiguous() for r in rows]
            lds = {self.c}
        a.Ca, a.Za = rows[0].data_ptr(), rows[1].data_ptr()
        a.ld_c = lds.pop()
        a.acc_Ca, a.acc_Za = self._acc[0].data_ptr(), self._acc[1].data_ptr()
        a.acc_len = self._acc_len
        a.Ba = bias.data_ptr()
        if self._comp is not None:
            a.comp = self._comp.data_ptr()
            a.comp_scales = None if self._scales is None else self._scales.data_ptr()
            a.comp_norms = self._norms.data_ptr()
            a.capacity = self._comp.shape[1]
        a.comp_kind = self._kind if self._kind is not None else _lib.dtype_tag(self.dtype)
        a.n_blocks = self._n_blocks
        if self._sw is not None:
            a.ring, a.ring_pos = self._sw._buf.data_ptr(), self._sw._n % self.win
        a.normalize = int(self._normalize_qk)
        a.counters = self._ctr.data_ptr()
        with torch.cuda.device(self.device):
            _lib.check(lib.kch_cache_append_token_advance(a, _lib.stream()))   # the last CTA advances the device counters
        self._advance(m)

    def _append_many(self, new, bias):
        m, T_new = self.m2, new[0].shape[1]
        if self._sw is not None:
            tail = new[0][:, -self.win:]
            keys = rownorm(tail, True).to(self.dtype) if self._normalize_qk else tail
            self._sw._n += T_new - tail.shape[1]
            self._sw.append(keys)
        staged = [torch.cat([a[:, :self._acc_len], x], dim=1) for a, x in zip(self._acc, new)]
        total = staged[0].shape[1]
        nb = total // m
        if nb:
            self._grow(self._n_blocks + nb)
            full = [s[:, :nb * m].contiguous() for s in staged]
            self._store_rows(csa_compress_kv(full[0], full[1], bias, m), self._n_blocks)
            self._n_blocks += nb
        rest = total - nb * m
        for a, s in zip(self._acc, staged):
            if rest:
                a[:, :rest] = s[:, nb * m:]
        self._acc_len = rest
        self._n_tokens_seen += T_new
        self._sync_counters()

    def forward_step(self, q, *, nh, scale=None, sink_logits=None, normalize_qk=True, _q_normalize=False,
                     _out_dtype=None):
        B, T_new = q.shape[0], q.shape[1]
        if T_new != 1:
            raise ValueError(f"HCADecodingCache.forward_step: T_new={T_new} must be 1.")
        if B != self.B:
            raise ValueError(f"HCADecodingCache.forward_step: batch size {B} does not match cache's B={self.B}.")
        if q.shape[2] != nh:
            raise ValueError(f"q.shape[2]={q.shape[2]} does not match nh={nh}.")
        if q.device != self.device:
            raise ValueError(f"HCADecodingCache.forward_step: q.device={q.device} does not match cache's "
                             f"device={self.device}. Call cache.to(device=q.device) or move q to the cache's device.")
        core_scale = (1.0 if normalize_qk else self.c ** -0.5) if scale is None else float(scale)
        t = self._n_tokens_seen - 1
        nvis = min((t + 1) // self.m2, self._n_blocks)
        if self._decode_attend_ok(nh) and self._comp is not None:
            out = self._attend_decode(q, None, 0, self.m2, nh, core_scale, sink_logits, normalize_qk,
                                      q_normalize=_q_normalize, out_dtype=_out_dtype)
        else:
            if _q_normalize:
                q = rownorm(q.contiguous(), True)
            out = self._attend(q.float(), None, nvis, nh, core_scale, sink_logits, normalize_qk)
            if _out_dtype is not None:
                out = out.to(_out_dtype)
        return out.reshape(B, 1, nh, self.c)
