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


def local_config(cfg, world):
    """The per-rank geometry: head counts divided by the world size."""
    for name in ("n_heads_qk", "n_heads_v", "csa_nh", "hca_nh"):
        if getattr(cfg, name) % world != 0:
            raise ValueError(f"tensor parallelism: {name}={getattr(cfg, name)} must be divisible by the "
                             f"world size {world}")
    return dataclasses.replace(cfg, n_heads_qk=cfg.n_heads_qk // world, n_heads_v=cfg.n_heads_v // world,
                               csa_nh=cfg.csa_nh // world, hca_nh=cfg.hca_nh // world)


def _rows(w, rank, world):
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n].clone()


def shard_state_dict(params, layout, rank, world):
    """Slice a full ``state_dict`` for one rank.  Head-major row blocks of the per-head projections are
    cut; everything else (including every ``o_proj``) is kept whole."""
    out = {}
    per_head = {"kda": ("q_proj.weight", "k_proj.weight", "v_proj.weight", "g_up.weight", "beta.weight"),
                "csa": ("W_UQ.weight", "sink"), "hca": ("W_UQ.weight", "sink")}
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
    buf = torch.empty(ctx.world * rows, kl, dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(buf, flat, group=ctx.group)
    y = linear_kslabs(buf.view(ctx.world, rows, kl), W, residual=residual)
    return y.reshape(*lead, W.shape[0])


def build_tp_model(cfg, params, total_layers, ctx: TPContext, device, dtype):
    """A ``HybridKCHAttention`` holding rank ``ctx.rank``'s shard of ``params`` (full ``state_dict``)."""
    import torch.nn as nn

    from .fused import HybridKCHAttention

    lcfg = local_config(cfg, ctx.world)
    model = HybridKCHAttention(lcfg, total_layers)
    for layer, kind in zip(model.layers, model.layout):
        full_in = {"kda": cfg.n_heads_v * cfg.head_dim_v, "csa": cfg.csa_nh * cfg.csa_c,
                   "hca": cfg.hca_nh * cfg.hca_c}[kind]
        layer.o_proj = nn.Linear(full_in, cfg.d_model, bias=False)
        layer.tp = ctx
    local = shard_state_dict(params, model.layout, ctx.rank, ctx.world)
    model.load_state_dict(local, strict=True)
    return model.to(dtype).to(device).eval()
