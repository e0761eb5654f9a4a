"""One seeded case per kernel family, run as a child process so that an environment switch (read once per process by
the library) selects the alternate kernel:  python tests/alt_kernel_case.py <kind> <out.pt>."""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "kda-csa-hca-fusion_b200"))


def run(kind, dev="cuda:0"):
    import kch_b200  # noqa: F401
    from kch_b200 import synthetic as syn
    from kch_b200.csa import attend, linear
    g = torch.Generator().manual_seed(77)
    if kind == "attend":
        B, T, nh, c, m, topk, win = 2, 300, 16, 128, 4, 64, 128
        q = torch.randn(B, T, nh * c, generator=g).bfloat16().to(dev)
        comp = torch.nn.functional.normalize(torch.randn(B, T // m, c, generator=g), dim=-1).bfloat16().to(dev)
        wk = torch.nn.functional.normalize(torch.randn(B, T, c, generator=g), dim=-1).bfloat16().to(dev)
        sink = (torch.randn(nh, generator=g) * 0.5).to(dev)
        sel = torch.full((B, T, topk), -1, dtype=torch.int32)
        for b in range(B):
            for t in range(T):
                nv = (t + 1) // m
                k = min(nv, topk)
                if k:
                    sel[b, t, :k] = torch.randperm(nv, generator=g)[:k].to(torch.int32)
        sparse = attend(q, comp, nh=nh, c=c, sel=sel.to(dev), m=m, q_normalize=True, win=wk, sliding_window=win,
                        sink=sink, scale=1.0, out_dtype=torch.bfloat16)
        dense = attend(q, comp, nh=nh, c=c, sel=None, m=m, q_normalize=True, win=wk, sliding_window=win,
                       sink=sink, scale=1.0, out_dtype=torch.bfloat16)
        return torch.stack([sparse.float().cpu(), dense.float().cpu()])
    if kind == "kda":
        q, k, v, gg, beta, S0 = syn.kda_inputs(301, 2, 300, 2, 128, 128, 4, torch.bfloat16, with_state=True)
        o, s = kch_b200.naive_chunk_kda(*(x.to(dev) for x in (q, k, v, gg, beta)), initial_state=S0.to(dev),
                                        output_final_state=True, chunk_size=64)
        return torch.cat([o.float().cpu().flatten(), s.float().cpu().flatten()])
    if kind == "kda_long":      # 256 chunks: the chain length of the benchmark's order, slow-decay gate
        q, k, v, gg, beta, S0 = syn.kda_inputs(302, 1, 16384, 4, 128, 128, 4, torch.bfloat16, with_state=True)
        gg = (gg.float() * 0.1).bfloat16()
        o, s = kch_b200.naive_chunk_kda(*(x.to(dev) for x in (q, k, v, gg, beta)), initial_state=S0.to(dev),
                                        output_final_state=True, chunk_size=64)
        return torch.cat([o.float().cpu().flatten(), s.float().cpu().flatten()])
    if kind == "linear":
        x = torch.randn(1000, 2048, generator=g).bfloat16().to(dev)
        w = (torch.randn(772, 2048, generator=g) * 0.05).bfloat16().to(dev)
        r = torch.randn(1000, 772, generator=g).bfloat16().to(dev)
        return linear(x, w, residual=r).float().cpu()
    if kind == "select":        # odd number of rows, rows shorter than top-k, ties (relu zeros): exact indices
        from kch_b200.csa import indexer_topk
        B, T, HI, DI, m, topk = 1, 1531, 4, 64, 1, 256
        qi = torch.randn(B, T, HI, DI, generator=g).bfloat16().to(dev)
        ki = torch.randn(B, T // m, DI, generator=g).to(dev)
        wi = (torch.randn(B, T, HI, generator=g) * 0.1).to(dev)
        idx = indexer_topk(qi, ki, wi, topk, m=m, normalize_qk=True, sorted_output=False)
        return idx.sort(dim=-1).values.float().cpu()
    if kind == "decode_step":   # one-token steps of the small stack: indexer, KDA step, decode GEMMs, attention
        cfg = kch_b200.HybridConfig(d_model=256, n_heads_qk=2, n_heads_v=2, head_dim_k=128, head_dim_v=128, kda_chunk_size=64,
                                    csa_m=4, csa_topk=64, csa_nh=4, csa_c=128, csa_dc=64, csa_nIh=2, csa_cI=64,
                                    csa_sliding_window=16, hca_m2=16, hca_nh=4, hca_c=128, hca_dc=64, hca_sliding_window=16)
        model = kch_b200.HybridKCHAttention(cfg, 5)
        model.load_state_dict(syn.hybrid_params(91, cfg, 5, dtype=torch.bfloat16), strict=True)
        model = model.bfloat16().to(dev).eval()
        x = syn.hidden_states(92, 3, 120, cfg.d_model, torch.bfloat16).to(dev)
        dec = kch_b200.HybridDecoding(model=model, use_cuda_graph=False)
        dec.reset()
        ys = [dec(x[:, :70])]
        for t in range(70, 120):
            ys.append(dec(x[:, t:t + 1]))
        return torch.cat(ys, 1).float().cpu()
    raise ValueError(kind)


if __name__ == "__main__":
    from kch_b200 import _lib
    out = run(sys.argv[1])
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "a bounded device-side wait expired"
    torch.save(out, sys.argv[2])
