"""Single-kernel micro-benchmarks (CUDA-event timed) for profiling one kernel of the path in isolation.

    python -m kch_b200.microbench linear --M 16384 --N 2048 --K 2048
    python -m kch_b200.microbench kda_chunk --B 1 --T 4096 --H 16
    python -m kch_b200.microbench csa_attend --B 1 --T 4096 --topk 1024
    python -m kch_b200.microbench compress --B 4 --T 32768
    python -m kch_b200.microbench indexer --B 1 --T 4096
    python -m kch_b200.microbench decode --B 64 --T 131072 --iters 4 [--kv-quant fp8]

Each prints one JSON line with the average launch time and the achieved algorithmic rate.  Inputs are
seeded synthetic tensors of the benchmark geometry (K=V=c=128, 16 heads, m=4, 4x64 indexer).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)


_PROFILE = False


def _time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if _PROFILE:        # `ncu --profile-from-start off` then sees the timed iterations only
        torch.cuda.profiler.start()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    if _PROFILE:
        torch.cuda.profiler.stop()
    return a.elapsed_time(b) / iters


def main():
    import kch_b200
    from kch_b200 import csa, synthetic as syn

    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["linear", "kda_chunk", "kda_recurrent", "csa_attend", "hca_attend", "compress",
                                       "indexer", "decode"])
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=2048)
    ap.add_argument("--K", type=int, default=2048)
    ap.add_argument("--B", type=int, default=1)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--H", type=int, default=16)
    ap.add_argument("--topk", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--fp32-queries", action="store_true", help="indexer: fp32 queries (the mma.sync logits kernel)")
    ap.add_argument("--gate-scale", type=float, default=0.1, help="kda: multiplies the synthetic log-decay")
    ap.add_argument("--kv-quant", default=None, choices=[None, "fp8", "int8"])
    ap.add_argument("--graph", action="store_true", help="decode: replay the step from a CUDA graph")
    ap.add_argument("--profile", action="store_true", help="bracket the timed iterations with cudaProfilerStart/Stop")
    a = ap.parse_args()
    global _PROFILE
    _PROFILE = a.profile
    dev = "cuda:0"
    g = torch.Generator().manual_seed(1)
    out = {"kernel": a.kernel}
    if a.kernel == "linear":
        x = torch.randn(a.M, a.K, generator=g).bfloat16().to(dev)
        w = (torch.randn(a.N, a.K, generator=g) * 0.02).bfloat16().to(dev)
        ms = _time(lambda: csa.linear(x, w), a.iters, a.warmup)
        fl = 2.0 * a.M * a.N * a.K
        out.update(M=a.M, N=a.N, K=a.K, ms=ms, tflops=fl / ms / 1e9, algorithmic_bytes=2.0 * (a.M * a.K + a.N * a.K + a.M * a.N))
    elif a.kernel in ("kda_chunk", "kda_recurrent"):
        q, k, v, gg, beta = (t.to(dev) for t in syn.kda_inputs(0, a.B, a.T, a.H, 128, 128, dtype=torch.bfloat16))
        gg = (gg.float() * a.gate_scale).bfloat16()     # 0.1: the decay range of the layer's gate (-0.1 softplus)
        if a.kernel == "kda_chunk":
            fn = lambda: kch_b200.naive_chunk_kda(q, k, v, gg, beta, output_final_state=True)  # noqa: E731
        else:
            fn = lambda: kch_b200.naive_recurrent_kda(q, k, v, gg, beta, output_final_state=True)  # noqa: E731
        ms = _time(fn, a.iters, a.warmup)
        fl = a.B * a.T * a.H * (6.0 * 128 * 128 + 3 * 64 * 128 + 64 * 64)
        out.update(B=a.B, T=a.T, H=a.H, ms=ms, tflops=fl / ms / 1e9, tokens_per_s=a.B * a.T / ms * 1e3)
    elif a.kernel in ("csa_attend", "hca_attend"):
        nh, c, m = 16, 128, (4 if a.kernel == "csa_attend" else 128)
        n = a.T // m
        q = torch.randn(a.B, a.T, nh * c, generator=g).bfloat16().to(dev)
        comp = csa.rownorm(torch.randn(a.B, n, c, generator=g).to(dev), True, torch.bfloat16)
        win = csa.rownorm(torch.randn(a.B, a.T, c, generator=g).to(dev), True, torch.bfloat16)
        sink = torch.zeros(nh, dtype=torch.bfloat16, device=dev)
        sel = None
        if a.kernel == "csa_attend":
            # a valid selection per query: the first min(topk, visible) blocks, the rest -1
            ar = torch.arange(a.topk, device=dev).view(1, 1, -1).expand(a.B, a.T, -1)
            vis = ((torch.arange(a.T, device=dev) + 1) // m).view(1, -1, 1)
            sel = torch.where(ar < vis, ar, torch.full_like(ar, -1)).to(torch.int32).contiguous()
        fn = lambda: csa.attend(q, comp, nh=nh, c=c, sel=sel, m=m, q_normalize=True, win=win, sliding_window=128,  # noqa: E731
                                sink=sink, scale=1.0, out_dtype=torch.bfloat16)
        ms = _time(fn, a.iters, a.warmup)
        t = torch.arange(a.T, dtype=torch.float64)
        ent = (torch.minimum((t + 1) // m, torch.tensor(float(a.topk if sel is not None else n))) +
               torch.minimum(t + 1, torch.tensor(128.0))).sum().item() * a.B
        out.update(B=a.B, T=a.T, ms=ms, entries=ent, tflops=ent * 4.0 * nh * c / ms / 1e9,
                   gather_gbs=ent * c * 2 / ms / 1e6)
    elif a.kernel == "compress":
        c, m = 128, 4
        t4 = [torch.randn(a.B, a.T, c, generator=g).bfloat16().to(dev) for _ in range(4)]
        Ba, Bb = [(torch.randn(m, c, generator=g) * 0.02).bfloat16().to(dev) for _ in range(2)]
        ms = _time(lambda: kch_b200.csa_compress_kv_overlapped(*t4, Ba, Bb, m), a.iters, a.warmup)
        by = a.B * a.T * c * 2 * 4 + a.B * (a.T // m) * c * 4
        out.update(B=a.B, T=a.T, ms=ms, algorithmic_bytes=by, gbs=by / ms / 1e6)
    elif a.kernel == "indexer":
        HI, DI, m = 4, 64, 4
        n = a.T // m
        qi = torch.randn(a.B, a.T, HI, DI, generator=g).to(dev)
        if not a.fp32_queries:      # as in the layer: bf16 query rows, scored by the tcgen05 logits kernel
            qi = qi.bfloat16()
        ki = torch.randn(a.B, n, DI, generator=g).to(dev)
        wi = (torch.randn(a.B, a.T, HI, generator=g) * 0.1).to(dev)
        ms = _time(lambda: csa.indexer_topk(qi, ki, wi, a.topk, m=m, normalize_qk=True, sorted_output=False),
                   a.iters, a.warmup)
        vis = float(((torch.arange(a.T, dtype=torch.float64) + 1) // m).sum()) * a.B
        out.update(B=a.B, T=a.T, ms=ms, tflops=vis * 2 * HI * DI / ms / 1e9)
    elif a.kernel == "decode":
        # one-token steps of the 5-layer stack (d_model 2048) on caches filled as after --T tokens
        cfg = kch_b200.HybridConfig(d_model=2048, n_heads_qk=16, n_heads_v=16, head_dim_k=128, head_dim_v=128,
                                    kda_chunk_size=64, csa_m=4, csa_topk=a.topk, csa_nh=16, csa_c=128, csa_dc=128,
                                    csa_nIh=4, csa_cI=64, csa_sliding_window=128, hca_m2=128, hca_nh=16, hca_c=128,
                                    hca_dc=128, hca_sliding_window=128)
        model = kch_b200.HybridKCHAttention(cfg, 5)
        model.load_state_dict(syn.hybrid_params(3, cfg, 5, dtype=torch.bfloat16), strict=True)
        model = model.bfloat16().to(dev).eval()
        dec = kch_b200.HybridDecoding(model=model, kv_quant=a.kv_quant, use_cuda_graph=a.graph)
        syn.fill_decode_state(dec, a.B, a.T, a.iters + a.warmup, torch.device(dev), 11)
        x = torch.randn(a.B, 1, 2048, generator=g).bfloat16().to(dev)
        ms = _time(lambda: dec(x), a.iters, a.warmup)
        out.update(B=a.B, context=a.T, kv_quant=a.kv_quant, graph=dec._graph is not None, us_per_step=ms * 1e3,
                   us_per_token=ms * 1e3 / a.B)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
