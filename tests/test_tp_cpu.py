"""Tensor-parallel host logic on CPU ranks (gloo, world size 2): the per-rank weight shards and the
all-gather of head outputs reproduce the unsharded layer.  The arithmetic here is the CPU oracle's (the
CUDA kernels need a GPU); what is under test is `kch_b200.tp`: which rows each rank owns and how the
gathered head outputs are laid out before `o_proj`."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CFG = dict(d_model=32, n_heads_qk=2, n_heads_v=4, head_dim_k=8, head_dim_v=8, kda_chunk_size=8, csa_m=4, csa_topk=64,
           csa_nh=4, csa_c=8, csa_dc=8, csa_nIh=2, csa_cI=4, csa_sliding_window=4, hca_m2=8, hca_nh=2, hca_c=8,
           hca_dc=8, hca_sliding_window=4)


def _worker(rank, world, port, out):
    for p in (os.path.join(ROOT, "kda-csa-hca-fusion_b200"), ROOT):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import torch.nn.functional as F

        import kch_b200
        from kch_b200 import synthetic as syn
        from kch_b200.tp import TPContext, gather_heads, local_config, shard_state_dict
        from oracle import kch_oracle as orc
        cfg = kch_b200.HybridConfig(**CFG)
        layout = syn.hybrid_layout(cfg.n_kda, cfg.n_csa, cfg.n_hca, 5)
        params = syn.hybrid_params(5, cfg, 5, dtype=torch.float32, random_sink=True)
        x = syn.hidden_states(6, 2, 24, cfg.d_model, torch.float32)
        ctx = TPContext(rank, world, None)
        lcfg = local_config(cfg, world)
        local = shard_state_dict(params, layout, rank, world)
        res = {}
        # --- KDA layer 0: local heads -> gather -> o_proj equals the full layer
        pf = {k[len("layers.0."):]: v for k, v in params.items() if k.startswith("layers.0.")}
        pl = {k[len("layers.0."):]: v for k, v in local.items() if k.startswith("layers.0.")}
        xc, _ = orc.short_conv(x, pf["short_conv.weight"], pf["short_conv.bias"])
        q, k, v, g, beta = orc.kda_layer_inputs(pf, xc, cfg.n_heads_qk, cfg.n_heads_v, cfg.head_dim_k, cfg.head_dim_v)
        o_full, _ = orc.chunk_kda(q, k, v, g, beta, chunk_size=8)
        y_full = F.linear(o_full.reshape(2, 24, -1), pf["o_proj.weight"])
        ql, kl, vl, gl, bl = orc.kda_layer_inputs(pl, xc, lcfg.n_heads_qk, lcfg.n_heads_v, cfg.head_dim_k, cfg.head_dim_v)
        o_loc, _ = orc.chunk_kda(ql, kl, vl, gl, bl, chunk_size=8)
        o_gath = gather_heads(o_loc.reshape(2, 24, -1), ctx)
        assert o_gath.shape == (2, 24, cfg.n_heads_v * cfg.head_dim_v)
        res["kda"] = float((F.linear(o_gath, pl["o_proj.weight"]) - y_full).abs().max())
        # --- CSA layer 3: W_UQ / sink sharded, everything else replicated
        pf = {k[len("layers.3."):]: v for k, v in params.items() if k.startswith("layers.3.")}
        pl = {k[len("layers.3."):]: v for k, v in local.items() if k.startswith("layers.3.")}

        def csa(p, nh):
            return orc.csa_forward(x, p["W_aKV.weight"], p["W_bKV.weight"], p["W_aZ.weight"], p["W_bZ.weight"], p["Ba"],
                                   p["Bb"], p["W_DQ.weight"], p["W_UQ.weight"], p["W_IUQ.weight"], p["W_w.weight"],
                                   p["W_KV_idx.weight"], p["W_Z_idx.weight"], p["B_idx"], m=cfg.csa_m, topk=cfg.csa_topk,
                                   nh=nh, nIh=cfg.csa_nIh, c=cfg.csa_c, c_I=cfg.csa_cI, dc=cfg.csa_dc,
                                   sliding_window=cfg.csa_sliding_window, sink_logits=p["sink"], normalize_qk=True)
        full = csa(pf, cfg.csa_nh)
        gath = gather_heads(csa(pl, lcfg.csa_nh), ctx)
        res["csa"] = float((gath - full).abs().max())
        # --- HCA layer 4
        pf = {k[len("layers.4."):]: v for k, v in params.items() if k.startswith("layers.4.")}
        pl = {k[len("layers.4."):]: v for k, v in local.items() if k.startswith("layers.4.")}

        def hca(p, nh):
            return orc.hca_forward(x, p["W_KV.weight"], p["W_Z.weight"], p["B_pos"], p["W_DQ.weight"], p["W_UQ.weight"],
                                   m2=cfg.hca_m2, nh=nh, c=cfg.hca_c, dc=cfg.hca_dc,
                                   sliding_window=cfg.hca_sliding_window, sink_logits=p["sink"])
        res["hca"] = float((gather_heads(hca(pl, lcfg.hca_nh), ctx) - hca(pf, cfg.hca_nh)).abs().max())
        # --- rows mode of CSA / HCA: this rank's contiguous run of the flattened [B*T] query rows, gathered along rows
        from kch_b200.tp import gather_rows, row_span
        rctx = TPContext(rank, world, None, attn_shard="rows")
        rl = shard_state_dict(params, layout, rank, world, "rows")
        res["rows_w_uq_full"] = tuple(rl["layers.3.W_UQ.weight"].shape) == tuple(params["layers.3.W_UQ.weight"].shape) \
            and local_config(cfg, world, "rows").csa_nh == cfg.csa_nh and local_config(cfg, world, "rows").n_heads_v * world == cfg.n_heads_v
        pf3 = {k[len("layers.3."):]: v for k, v in params.items() if k.startswith("layers.3.")}
        pf4 = {k[len("layers.4."):]: v for k, v in params.items() if k.startswith("layers.4.")}
        for name, xb in (("whole", x), ("slice", x[:1])):          # 2 sequences over 2 ranks; 1 sequence cut in two
            Bx, Tx = xb.shape[0], xb.shape[1]
            r0, per = row_span(Bx * Tx, rctx)
            if per % Tx == 0:
                xs, rows = xb[r0 // Tx:r0 // Tx + per // Tx], None
            else:
                xs, rows = xb[r0 // Tx:r0 // Tx + 1], [(r0 % Tx, r0 % Tx + per)]
            def csa_rows(p, xi, qr):
                y = orc.csa_forward(xi, p["W_aKV.weight"], p["W_bKV.weight"], p["W_aZ.weight"], p["W_bZ.weight"], p["Ba"],
                                    p["Bb"], p["W_DQ.weight"], p["W_UQ.weight"], p["W_IUQ.weight"], p["W_w.weight"],
                                    p["W_KV_idx.weight"], p["W_Z_idx.weight"], p["B_idx"], m=cfg.csa_m, topk=cfg.csa_topk,
                                    nh=cfg.csa_nh, nIh=cfg.csa_nIh, c=cfg.csa_c, c_I=cfg.csa_cI, dc=cfg.csa_dc,
                                    sliding_window=cfg.csa_sliding_window, sink_logits=p["sink"], normalize_qk=True,
                                    query_rows=qr)
                return y if qr is None else y[:, qr[0][0]:qr[0][1]]
            def hca_rows(p, xi, qr):
                y = orc.hca_forward(xi, p["W_KV.weight"], p["W_Z.weight"], p["B_pos"], p["W_DQ.weight"], p["W_UQ.weight"],
                                    m2=cfg.hca_m2, nh=cfg.hca_nh, c=cfg.hca_c, dc=cfg.hca_dc,
                                    sliding_window=cfg.hca_sliding_window, sink_logits=p["sink"], query_rows=qr)
                return y if qr is None else y[:, qr[0][0]:qr[0][1]]
            g3 = gather_rows(csa_rows(pf3, xs, rows), rctx, lead=(Bx, Tx))
            g4 = gather_rows(hca_rows(pf4, xs, rows), rctx, lead=(Bx, Tx))
            res[f"rows_csa_{name}"] = float((g3 - csa_rows(pf3, xb, None)).abs().max())
            res[f"rows_hca_{name}"] = float((g4 - hca_rows(pf4, xb, None)).abs().max())
        # o_proj and the norms are replicated, per-head weights are halved
        res["o_proj_full"] = tuple(local["layers.0.o_proj.weight"].shape) == tuple(params["layers.0.o_proj.weight"].shape)
        res["q_rows"] = local["layers.0.q_proj.weight"].shape[0] * world == params["layers.0.q_proj.weight"].shape[0]
        out[rank] = res
    finally:
        dist.destroy_process_group()


def test_head_sharding_and_gather_world2():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert len(out) == world
    for rank in range(world):
        r = out[rank]
        assert r["kda"] <= 1e-5 and r["csa"] <= 1e-5 and r["hca"] <= 1e-5, r
        assert r["o_proj_full"] and r["q_rows"] and r["rows_w_uq_full"]
        for name in ("whole", "slice"):
            assert r[f"rows_csa_{name}"] <= 1e-6 and r[f"rows_hca_{name}"] <= 1e-6, r


def test_local_config_rejects_indivisible_heads():
    import kch_b200
    from kch_b200.tp import local_config
    cfg = kch_b200.HybridConfig(**CFG)
    with pytest.raises(ValueError, match="n_heads_qk"):
        local_config(cfg, 4)
    assert local_config(cfg, 2).n_heads_v == 2
