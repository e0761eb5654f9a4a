"""Tensor parallelism by heads over the GPUs of one node (one process per GPU).

The reference has no distributed code.  The path shards naturally by head: KDA heads are independent
(ops_kda.py:226-258), CSA / HCA query heads share one KV head but are otherwise independent
(ops_csa.py:1102, ops_hca.py:145).  Rank r of N owns heads ``[r*h/N, (r+1)*h/N)``: it holds the matching
row slices of ``q/k/v/g_up/beta`` (KDA) and ``W_UQ`` / ``sink`` (CSA, HCA); LayerNorm, conv, ``g_down``,
the shared KV / indexer projections, compression, the indexer and ``o_proj`` are replicated.  Per layer
there is exactly one exchange: an all-gather of the head outputs ``[B,T,(h/N)*c] -> [B,T,h*c]`` before
``o_proj``.
"""
from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist


@dataclasses.dataclass
class TPContext:
    rank: int
    world: int
    group: object = None
    # how the CSA / HCA layers are divided.  "heads": query heads, like KDA (every rank scores and attends for all
    # queries with its share of the heads).  "rows": the flattened query rows [B*T] in equal contiguous runs (whole
    # sequences while world <= B, else a slice of one sequence): the indexer, the top-k and the gather of selected
    # rows cost the same whatever the head count, so only this axis divides them.  One all-gather per layer either way.
    attn_shard: str = "heads"
    # optional PeerGather: decode-sized all-gathers by plain peer stores instead of the library collective
    peer: object = None


class PeerGather:
    """Decode-sized all-gather over peer-mapped memory (``kch_peer_allgather``): every rank stores its slab into every
    peer's gather buffer over NVLink and the ranks meet on flags, in one launch of one CTA -- a fraction of the
    latency of a library collective for the 256 KiB a decode step gathers per layer.  The buffer and the flags live
    in one allocation of torch's symmetric-memory allocator (CUDA VMM, mapped on every rank by ``rendezvous``).
    Calls must be made by all ranks in the same order; the result of ``gather`` is a view of the buffer and stays
    valid until the next call."""

    def __init__(self, ctx, max_slab_bytes, device):
        import ctypes

        import torch.distributed._symmetric_memory as symm

        from . import _lib
        self._lib = _lib
        lib = _lib.load()
        self.rank, self.world = ctx.rank, ctx.world
        self.flag_bytes = 256 * ((4 * int(lib.kch_peer_gather_flag_words(ctx.world)) + 255) // 256)
        self.max_slab = (int(max_slab_bytes) + 15) // 16 * 16
        group = ctx.group if ctx.group is not None else dist.group.WORLD
        self.mem = symm.empty(self.flag_bytes + ctx.world * self.max_slab, dtype=torch.uint8, device=device)
        self.mem.zero_()
        self.hdl = symm.rendezvous(self.mem, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=ctx.group)                    # every rank's flags are zero before anyone's first store
        ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self._flags = (ctypes.c_void_p * ctx.world)(*ptrs)
        self._bufs = (ctypes.c_void_p * ctx.world)(*[p + self.flag_bytes for p in ptrs])

    def fits(self, flat):
        return flat.numel() * flat.element_size() <= self.max_slab and (flat.numel() * flat.element_size()) % 16 == 0

    def gather(self, flat):
        """``flat [rows, width]`` contiguous on this rank -> ``[world, rows, width]`` (rank-major), a view of the buffer."""
        _lib = self._lib
        nbytes = flat.numel() * flat.element_size()
        with torch.cuda.device(flat.device):
            _lib.check(_lib.load().kch_peer_allgather(_lib.ptr(flat), nbytes, self._bufs, self._flags, self.rank,
                                                      self.world, _lib.stream()))
        out = self.mem[self.flag_bytes:self.flag_bytes + self.world * nbytes].view(flat.dtype)
        return out.view(self.world, flat.shape[0], flat.shape[1])


def enable_peer_gather(ctx, max_slab_bytes, device):
    """Give ``ctx`` a ``PeerGather`` for slabs of up to ``max_slab_bytes``; returns False (and leaves the library
    collective in place) when the symmetric-memory allocator is not usable on this system."""
    try:
        ctx.peer = PeerGather(ctx, max_slab_bytes, device)
        return True
    except Exception as exc:                               # no peer mapping available: keep NCCL
        import warnings
        warnings.warn(f"kch_b200: peer-store all-gather unavailable ({exc!r}); using the NCCL all-gather")
        ctx.peer = None
        return False


def local_config(cfg, world, attn_shard="heads"):
    """The per-rank geometry: head counts divided by the world size (CSA / HCA heads only when they are the
    sharded axis of those layers)."""
    names = ("n_heads_qk", "n_heads_v") + (("csa_nh", "hca_nh") if attn_shard == "heads" else ())
    for name in names:
        if getattr(cfg, name) % world != 0:
            raise ValueError(f"tensor parallelism: {name}={getattr(cfg, name)} must be divisible by the "
                             f"world size {world}")
    div = world if attn_shard == "heads" else 1
    return dataclasses.replace(cfg, n_heads_qk=cfg.n_heads_qk // world, n_heads_v=cfg.n_heads_v // world,
                               csa_nh=cfg.csa_nh // div, hca_nh=cfg.hca_nh // div)


def _rows(w, rank, world):
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n].clone()


def shard_state_dict(params, layout, rank, world, attn_shard="heads"):
    """Slice a full ``state_dict`` for one rank.  Head-major row blocks of the per-head projections are
    cut; everything else (including every ``o_proj``) is kept whole."""
    out = {}
    attn = ("W_UQ.weight", "sink") if attn_shard == "heads" else ()
    per_head = {"kda": ("q_proj.weight", "k_proj.weight", "v_proj.weight", "g_up.weight", "beta.weight"),
                "csa": attn, "hca": attn}
    for key, val in params.items():
        parts = key.split(".")
        if parts[0] == "layers":
            kind = layout[int(parts[1])]
            name = ".".join(parts[2:])
            out[key] = _rows(val, rank, world) if name in per_head[kind] else val
        else:
            out[key] = val
    return out


def gather_heads(o_local, ctx: TPContext):
    """All-gather of per-rank head outputs along the feature axis: ``[..., h_local*c] -> [..., h*c]``."""
    if ctx is None or ctx.world == 1:
        return o_local
    lead = o_local.shape[:-1]
    kl = o_local.shape[-1]
    flat = o_local.reshape(-1, kl).contiguous()
    rows = flat.shape[0]
    buf = torch.empty(ctx.world * rows, kl, dtype=flat.dtype, device=flat.device)    # rank-major concatenation
    dist.all_gather_into_tensor(buf, flat, group=ctx.group)
    return buf.view(ctx.world, rows, kl).permute(1, 0, 2).reshape(*lead, ctx.world * kl)


def row_span(n_rows, ctx: TPContext):
    """``(first row, row count)`` of this rank's contiguous run of ``n_rows`` flattened query rows."""
    if n_rows % ctx.world != 0:
        raise ValueError(f"tensor parallelism by rows: {n_rows} query rows do not divide over {ctx.world} ranks")
    per = n_rows // ctx.world
    return ctx.rank * per, per


def gather_rows(o_rows, ctx: TPContext, lead=None):
    """All-gather of per-rank row runs ``[rows / world, width]`` along the row axis: rank order is row order, so the
    result is the plain ``[rows, width]`` matrix (viewed as ``[*lead, width]`` when ``lead`` is given)."""
    flat = o_rows.reshape(-1, o_rows.shape[-1]).contiguous()
    if ctx.peer is not None and ctx.peer.fits(flat):
        buf = ctx.peer.gather(flat).view(ctx.world * flat.shape[0], flat.shape[1])
    else:
        buf = torch.empty(ctx.world * flat.shape[0], flat.shape[1], dtype=flat.dtype, device=flat.device)
        dist.all_gather_into_tensor(buf, flat, group=ctx.group)
    return buf if lead is None else buf.view(*lead, flat.shape[1])


def out_projection_rows(o_rows, ctx: TPContext, W, residual=None, lead=None):
    """``o_proj`` of a layer whose QUERY ROWS are sharded: every rank projects ITS rows (+ its rows of the residual),
    then the projected rows are all-gathered along the row axis -- the same bytes on the wire as gathering the head
    outputs first, and the projection costs a 1/world share instead of being repeated on every rank."""
    from .csa import linear
    flat = o_rows.reshape(-1, o_rows.shape[-1])
    per = flat.shape[0]
    res = None
    if residual is not None:
        res = residual.reshape(-1, residual.shape[-1])[ctx.rank * per:(ctx.rank + 1) * per]
    y = linear(flat, W, residual=res)
    out = gather_rows(y, ctx, lead)
    if ctx.peer is not None and ctx.peer.fits(y):
        out = out.clone()          # a view of the peer buffer, which the next layer's gather overwrites: this one lives on
    return out


def out_projection(o_local, ctx: TPContext, W, residual=None):
    """``o_proj`` of a layer whose heads are sharded: all-gather of the per-rank head outputs ``[..., h_local*c]``,
    then ``F.linear(cat over ranks, W)`` (+ residual) on every rank.  The gather lands rank-major
    (``[world, rows, h_local*c]``); the GEMM walks those slabs along its K loop (``kch_linear_kslabs``), so the
    gathered tensor is never permuted into ``[rows, h*c]``."""
    from .csa import linear, linear_kslabs
    if ctx is None or ctx.world == 1:
        return linear(o_local, W, residual=residual)
    lead = o_local.shape[:-1]
    kl = o_local.shape[-1]
    slab_ok = (o_local.dtype == torch.bfloat16 and W.dtype == torch.bfloat16 and kl % 64 == 0 and W.shape[0] >= 32
               and W.data_ptr() % 16 == 0 and W.stride(0) % 8 == 0)
    if not slab_ok:
        return linear(gather_heads(o_local, ctx), W, residual=residual)
    flat = o_local.reshape(-1, kl).contiguous()
    rows = flat.shape[0]
    if ctx.peer is not None and ctx.peer.fits(flat):
        slabs = ctx.peer.gather(flat)
    else:
        buf = torch.empty(ctx.world * rows, kl, dtype=flat.dtype, device=flat.device)
        dist.all_gather_into_tensor(buf, flat, group=ctx.group)
        slabs = buf.view(ctx.world, rows, kl)
    y = linear_kslabs(slabs, W, residual=residual)
    return y.reshape(*lead, W.shape[0])


def build_tp_model(cfg, params, total_layers, ctx: TPContext, device, dtype):
    """A ``HybridKCHAttention`` holding rank ``ctx.rank``'s shard of ``params`` (full ``state_dict``)."""
    import torch.nn as nn

    from .fused import HybridKCHAttention

    if ctx.attn_shard not in ("heads", "rows"):
        raise ValueError(f"TPContext.attn_shard={ctx.attn_shard!r} must be 'heads' or 'rows'")
    lcfg = local_config(cfg, ctx.world, ctx.attn_shard)
    model = HybridKCHAttention(lcfg, total_layers)
    for layer, kind in zip(model.layers, model.layout):
        full_in = {"kda": cfg.n_heads_v * cfg.head_dim_v, "csa": cfg.csa_nh * cfg.csa_c,
                   "hca": cfg.hca_nh * cfg.hca_c}[kind]
        layer.o_proj = nn.Linear(full_in, cfg.d_model, bias=False)
        layer.tp = ctx
    local = shard_state_dict(params, model.layout, ctx.rank, ctx.world, ctx.attn_shard)
    model.load_state_dict(local, strict=True)
    return model.to(dtype).to(device).eval()
