"""GPU parity: the CUDA kernels (through the C ABI) against the CPU oracle and the golden vectors
produced by the reference.  Tolerances: fp32 inputs 2e-5 (the reference's own fp32 tolerance is 1e-5,
run_correctness.py:59-77); bf16 inputs max-abs 2e-3 on operator outputs (north-star bound); top-k is
compared as the exact multiset of selected logits (tie order is unpinned upstream)."""
import numpy as np
import pytest
import torch

from golden_cases import (CACHE_CASES, CSA_CASES, DECODE_CASE, STANDALONE_CASE, HCA_CASES, HYBRID_CASES, KDA_CASES,
                          make_cache_stream, np32)
from kch_b200 import synthetic as syn
from oracle import kch_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32_TOL, BF16_TOL = 2e-5, 2e-3


def md(a, b):
    a = a.detach().float().cpu().numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
    b = b.detach().float().cpu().numpy() if isinstance(b, torch.Tensor) else np.asarray(b)
    assert a.shape == b.shape, (a.shape, b.shape)
    return float(np.abs(a - b).max()) if a.size else 0.0


def tol(dt):
    return F32_TOL if dt == torch.float32 else BF16_TOL


@pytest.fixture(scope="module")
def kch():
    import kch_b200
    from kch_b200 import _lib
    _lib.load()
    yield kch_b200
    assert _lib.device_status() == 0, "a bounded device-side wait expired"


# ---------------------------------------------------------------------------------------------- linear
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 772, 256), (1000, 6288, 2048), (64, 40, 64), (7, 16, 24)])
def test_linear_bf16(kch, M, N, K):
    from kch_b200.csa import linear
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    r = torch.randn(M, N, generator=g).bfloat16()
    ref = (x.float() @ w.float().T)
    y = linear(x.to(DEV), w.to(DEV)).cpu()
    # one rounding to bf16 of an fp32-accumulated product: at most 1 ulp from the fp32 reference rounded
    ulp = ref.abs() * 2 ** -7          # (fp32 summation order differs: allow 1e-4 absolute near zero)
    assert ((y.float() - ref).abs() <= ulp + 1e-4).all()
    y2 = linear(x.to(DEV), w.to(DEV), residual=r.to(DEV)).cpu()
    ref2 = (y.float() + r.float()).bfloat16()
    assert md(y2, ref2) == 0.0


@pytest.mark.parametrize("M,N,K", [(64, 2048, 2048), (37, 776, 2048), (1, 384, 2048), (64, 1024, 128), (64, 6288, 2048)])
def test_linear_decode_batch_split_k(kch, M, N, K):
    """A decode batch (at most 64 rows) runs one tile per cluster with the K loop divided over its CTAs; the sum of the
    partial tiles, the fused activations and the residual must match the single-CTA kernel that a taller batch of
    the same rows takes (fp32 summation order differs: rare one-ulp flips of the bf16 rounding only)."""
    from kch_b200 import _lib
    from kch_b200.csa import linear
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(200, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    r = torch.randn(200, N, generator=g).bfloat16().to(DEV)
    ref = x[:M].float() @ w.float().T
    y = linear(x[:M], w)
    assert ((y.float() - ref).abs() <= ref.abs() * 2 ** -7 + 1e-4).all()
    assert torch.equal(linear(x[:M], w, residual=r[:M]), (y.float() + r[:M].float()).bfloat16())
    tall = linear(x, w)[:M]
    assert (y != tall).float().mean() <= 0.01 and md(y, tall) <= float(ref.abs().max()) * 2 ** -7
    if N == 6288:       # the KDA projection's epilogue: silu + per-head L2 norm | silu | none | sigmoid
        segs = [(2048, _lib.ACT_SILU_L2NORM, 0.0), (2048, _lib.ACT_SILU_L2NORM, 0.0), (2048, _lib.ACT_SILU, 0.0),
                (128, 0, 0.0), (16, _lib.ACT_SIGMOID, 0.0)]
        ye = linear(x[:M], w, epilogue=segs, group=128)
        te = linear(x, w, epilogue=segs, group=128)[:M]
        assert (ye != te).float().mean() <= 0.01 and md(ye, te) <= 3.2e-2
        import torch.nn.functional as F
        q_ref = F.normalize(F.silu(ref[:, :2048]).view(M, 16, 128), dim=-1).view(M, 2048)
        assert md(ye[:, :2048], q_ref) <= 4e-3
        assert md(ye[:, 6272:], torch.sigmoid(ref[:, 6272:])) <= 4e-3


@pytest.mark.parametrize("M,N,slabs,kl", [(300, 256, 2, 128), (1000, 2048, 8, 256), (64, 2048, 4, 512)])
def test_linear_kslabs_equals_linear_of_concatenation(kch, M, N, slabs, kl):
    """The output projection over a rank-major all-gather buffer: same bits as F.linear of the concatenated heads."""
    from kch_b200.csa import linear, linear_kslabs
    g = torch.Generator().manual_seed(M + N + slabs)
    a = torch.randn(slabs, M, kl, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, slabs * kl, generator=g) * 0.05).bfloat16().to(DEV)
    r = torch.randn(M, N, generator=g).bfloat16().to(DEV)
    cat = a.permute(1, 0, 2).reshape(M, slabs * kl).contiguous()
    assert torch.equal(linear_kslabs(a, w), linear(cat, w))
    assert torch.equal(linear_kslabs(a, w, residual=r), linear(cat, w, residual=r))
    with pytest.raises(ValueError, match="multiple of 64"):
        linear_kslabs(a[..., :40].contiguous(), w[:, :slabs * 40].contiguous())


def test_linear_f32_and_strided(kch):
    from kch_b200.csa import linear
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 50, 96, generator=g)
    w = torch.randn(33, 64, generator=g) * 0.1
    xs = x[..., 16:80]
    y = linear(xs.to(DEV), w.to(DEV)).cpu()
    assert md(y, xs @ w.T) <= 1e-4
    xb, wb = x.bfloat16().to(DEV)[..., 16:80], w.bfloat16().to(DEV)
    yb = linear(xb, wb).cpu()
    assert md(yb, (xb.cpu().float() @ wb.cpu().float().T).bfloat16()) <= 2e-2


@pytest.mark.parametrize("d", [64, 512, 2048])
def test_glue_kernels(kch, d):
    """LayerNorm / short conv / activations (scalar and vectorised paths) against the oracle's formulas."""
    import torch.nn.functional as F
    from kch_b200 import _lib
    from kch_b200.fused import activation, layernorm, short_conv
    g = torch.Generator().manual_seed(d)
    B, T = 2, 37
    x = (torch.randn(B, T, d, generator=g) * 2).bfloat16()
    w, b = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16(), (0.1 * torch.randn(d, generator=g)).bfloat16()
    y = layernorm(x.to(DEV), w.to(DEV), b.to(DEV))
    assert md(y, orc.layernorm_fp32(x, w, b)) <= 4e-2            # 1 bf16 ulp at |y| ~ 4
    assert (y.cpu().float() - orc.layernorm_fp32(x, w, b).float()).abs().mean() <= 2e-4
    cw, cb = (torch.randn(d, 1, 3, generator=g) * 0.5).bfloat16(), (torch.randn(d, generator=g) * 0.5).bfloat16()
    lb = torch.randn(B, 2, d, generator=g).bfloat16()
    for look in (None, lb):
        yc = short_conv(x.to(DEV), cw.to(DEV), cb.to(DEV), None if look is None else look.to(DEV))
        ref, _ = orc.short_conv(x, cw, cb, look)
        assert (yc.cpu().float() - ref.float()).abs().max() <= 6.3e-2 and \
            ((yc.cpu() != ref).float().mean() <= 0.02)               # same fp32 formula: rare rounding flips only
    if d % 256 == 0:
        # the decode step's single launch: bit-identical to LayerNorm followed by the one-token conv step
        from kch_b200.fused import layernorm_short_conv_step, short_conv_step
        x1 = x[:, :1].contiguous().to(DEV)
        lb_a, lb_b = lb.to(DEV).clone(), lb.to(DEV).clone()
        for _ in range(3):                                         # three steps: the lookback slides in place
            ya = short_conv_step(layernorm(x1, w.to(DEV), b.to(DEV)), cw.to(DEV), cb.to(DEV), lb_a)
            yb = layernorm_short_conv_step(x1, w.to(DEV), b.to(DEV), 1e-5, cw.to(DEV), cb.to(DEV), lb_b)
            assert torch.equal(ya, yb) and torch.equal(lb_a, lb_b)
            x1 = (x1.float() * 0.5 + 1.0).bfloat16()
    xs = x.to(DEV)
    assert md(activation(xs, _lib.ACT_SILU), F.silu(x)) <= 3.2e-2
    assert md(activation(xs, _lib.ACT_SIGMOID), torch.sigmoid(x)) <= 4e-3
    assert md(activation(xs, _lib.ACT_NEG_SOFTPLUS, param=0.1), -F.softplus(x) * 0.1) <= 4e-3
    grp = 128 if d % 128 == 0 else 16
    qn = activation(xs, _lib.ACT_SILU_L2NORM, group=grp).cpu()
    ref = F.normalize(F.silu(x).view(B, T, d // grp, grp), dim=-1).view(B, T, d)
    assert md(qn, ref) <= 4e-3 and ((qn != ref).float().mean() <= 0.02)
    # strided input (column slice of a wider tensor)
    wide = torch.randn(B, T, d + 64, generator=g).bfloat16().to(DEV)
    sl = wide[..., 32:32 + d]
    assert md(activation(sl, _lib.ACT_SILU), F.silu(sl.cpu())) <= 3.2e-2


# ---------------------------------------------------------------------------------------------- KDA
@pytest.mark.parametrize("name", list(KDA_CASES))
def test_kda(kch, golden, name):
    c = KDA_CASES[name]
    q, k, v, g, beta, S0 = syn.kda_inputs(c["seed"], c["B"], c["T"], c["H"], c["K"], c["V"], c["HV"], c["dtype"],
                                          with_state=True)
    S0 = S0 if c["state"] else None
    dq, dk, dv, dg, db = (x.to(DEV) for x in (q, k, v, g, beta))
    dS = None if S0 is None else S0.to(DEV)
    o_r, s_r = kch.naive_recurrent_kda(dq, dk, dv, dg, db, initial_state=dS, output_final_state=True)
    o_c, s_c = kch.naive_chunk_kda(dq, dk, dv, dg, db, initial_state=dS, output_final_state=True,
                                   chunk_size=c["chunk"])
    assert o_r.dtype == c["dtype"] and s_r.dtype == torch.float32
    to = 1e-2 if c["dtype"] == torch.bfloat16 else F32_TOL       # bf16 output rounding: 1 ulp at |o|~2
    assert md(o_r, golden[f"kda/{name}/o_rec"]) <= to
    assert md(s_r, golden[f"kda/{name}/s_rec"]) <= F32_TOL
    assert md(o_c, golden[f"kda/{name}/o_chunk"]) <= to
    assert md(s_c, golden[f"kda/{name}/s_chunk"]) <= F32_TOL
    o0, s0 = orc.recurrent_kda(q, k, v, g, beta, initial_state=S0)
    assert md(o_r, o0) <= to and md(s_r, s0) <= F32_TOL


def test_kda_config1_full_size(kch):
    """BASELINE config 1: B=1, T=1024, H=4, K=V=128, chunk 64, fp32, seed 0: chunk == recurrent."""
    q, k, v, g, beta = (x.to(DEV) for x in syn.kda_inputs(0, 1, 1024, 4, 128, 128))
    o1, s1 = kch.naive_chunk_kda(q, k, v, g, beta, output_final_state=True, chunk_size=64)
    o2, s2 = kch.naive_recurrent_kda(q, k, v, g, beta, output_final_state=True)
    assert md(o1, o2) <= 1e-5 and md(s1, s2) <= 1e-5
    o0, s0 = orc.recurrent_kda(*(x.cpu() for x in (q, k, v, g, beta)))
    assert md(o2, o0) <= 1e-5 and md(s2, s0) <= 1e-5


@pytest.mark.parametrize("B,T,H,HV,state", [(2, 300, 2, 4, True), (1, 64, 1, 1, False), (1, 1000, 2, 2, True)])
def test_kda_chunk_tensor_core_path(kch, B, T, H, HV, state):
    """bf16, K=V=128, chunk 64 takes the tensor-core kernels (two-term bf16 split, fp32 accumulation):
    state within fp32-level round-off of the oracle, output within one bf16 rounding of it."""
    q, k, v, g, beta, S0 = syn.kda_inputs(40 + T, B, T, H, 128, 128, HV, torch.bfloat16, with_state=True)
    S0 = S0 if state else None
    o_ref, s_ref = orc.chunk_kda(q, k, v, g, beta, initial_state=S0, chunk_size=64)
    o, s = kch.naive_chunk_kda(*(x.to(DEV) for x in (q, k, v, g, beta)), initial_state=None if S0 is None else S0.to(DEV),
                               output_final_state=True, chunk_size=64)
    assert o.dtype == torch.bfloat16 and s.dtype == torch.float32
    assert md(s, s_ref) <= 2e-4, md(s, s_ref)
    d = (o.float().cpu() - o_ref.float()).abs()
    assert bool((d <= o_ref.float().abs() * 2 ** -7 + 2e-3).all()), float(d.max())
    # the token recurrence on the same inputs agrees as well
    o2, s2 = kch.naive_recurrent_kda(*(x.to(DEV) for x in (q, k, v, g, beta)),
                                     initial_state=None if S0 is None else S0.to(DEV), output_final_state=True)
    assert md(s, s2) <= 2e-4
    # the slow-decay regime of the model (g = -0.1 softplus) and a hard-decay regime near the clamp
    for gscale in (0.1, 6.0):
        g2 = (g.float() * gscale).bfloat16()
        o_ref, s_ref = orc.chunk_kda(q, k, v, g2, beta, initial_state=S0, chunk_size=64)
        o, s = kch.naive_chunk_kda(*(x.to(DEV) for x in (q, k, v, g2, beta)),
                                   initial_state=None if S0 is None else S0.to(DEV), output_final_state=True)
        assert md(s, s_ref) <= 5e-4, (gscale, md(s, s_ref))
        d = (o.float().cpu() - o_ref.float()).abs()
        assert bool((d <= o_ref.float().abs() * 2 ** -7 + 3e-3).all()), (gscale, float(d.max()))


def test_kda_edges(kch):
    q, k, v, g, beta = (x.to(DEV) for x in syn.kda_inputs(3, 2, 0, 2, 16, 16))
    S0 = torch.randn(2, 2, 16, 16, device=DEV)
    for fn in (kch.naive_recurrent_kda, kch.naive_chunk_kda):
        o, s = fn(q, k, v, g, beta, initial_state=S0, output_final_state=True)
        assert o.shape == (2, 0, 2, 16) and md(s, S0) == 0.0
    q, k, v, g, beta = (x.to(DEV) for x in syn.kda_inputs(3, 1, 9, 2, 16, 16))
    o, s = kch.naive_recurrent_kda(q, k, v, g, beta, output_final_state=True, state_dtype=torch.float64)
    assert s.dtype == torch.float64
    o2, none = kch.naive_recurrent_kda(q, k, v, g, beta)
    assert none is None and md(o, o2) == 0.0
    with pytest.raises(ValueError, match="beta"):
        kch.naive_recurrent_kda(q, k, v, g, beta[..., :1])
    with pytest.raises(ValueError, match="chunk_size"):
        kch.naive_chunk_kda(q, k, v, g, beta, chunk_size=0)
    with pytest.raises(ValueError, match="dtype"):
        kch.naive_recurrent_kda(q, k, v.bfloat16(), g, beta)
    with pytest.raises(RuntimeError):
        kch.kda_forward(q.cpu(), k.cpu(), v.cpu(), g.cpu(), beta.cpu())


# ---------------------------------------------------------------------------------------------- CSA
def _csa_kwargs(c, sink):
    return dict(m=c["m"], topk=c["topk"], nh=c["nh"], nIh=c["nIh"], c=c["c"], c_I=c["c_I"], dc=c["dc"],
                sliding_window=c["win"], sink_logits=sink if c["sink"] else None, normalize_qk=c["normalize_qk"])


def _multiset_equal(lg, idx_a, idx_b, rtol=1e-6):
    """Rows of selected logits (sorted) agree; index -1 maps to -inf."""
    n = lg.shape[-1]
    lgp = torch.cat([lg, torch.full_like(lg[..., :1], float("-inf"))], -1)
    sa = torch.gather(lgp, -1, torch.where(idx_a < 0, n, idx_a)).sort(-1).values
    sb = torch.gather(lgp, -1, torch.where(idx_b < 0, n, idx_b)).sort(-1).values
    ok = (sa == sb) | torch.isclose(sa, sb, rtol=rtol, atol=1e-7)
    return ok.all(-1)


@pytest.mark.parametrize("name", list(CSA_CASES))
def test_csa(kch, golden, name):
    c = CSA_CASES[name]
    w, sink, H = syn.csa_inputs(c["seed"], c["B"], c["T"], c["d"], nh=c["nh"], c=c["c"], dc=c["dc"], nIh=c["nIh"],
                                c_I=c["c_I"], m=c["m"], dtype=c["dtype"], random_sink=c["random_sink"],
                                std=c.get("std", 0.02))
    W = [w[n] for n in syn.CSA_WEIGHT_ORDER]
    kw = _csa_kwargs(c, sink)
    dkw = dict(kw, sink_logits=None if kw["sink_logits"] is None else sink.to(DEV))
    aux_k = {}
    out, proj, idx = kch.naive_csa(H.to(DEV), *[x.to(DEV) for x in W], use_ste=False, return_projections=True,
                                   _return_indices=True, _aux=aux_k, **dkw)
    assert out.dtype == c["dtype"] and out.shape == (c["B"], c["T"], c["nh"] * c["c"])
    T, m = c["T"], c["m"]
    nb = (T + m - 1) // m
    o_ref, aux = orc.csa_forward(H, *W, return_aux=True, **kw)
    # stage 1: projections (bf16 GEMM: at most 1 ulp apart from the CPU GEMM)
    for mine, key in zip(proj, ("Ca", "Cb", "Za", "Zb", "K_idx", "Z_idx")):
        assert md(mine, aux[key]) <= (1e-5 if c["dtype"] == torch.float32 else 2e-2)
    # stage 2: top-k.  fp32: the kernel's picks against the oracle's own pipeline (identical inputs up to fp32
    # round-off).  bf16: the oracle's projections differ from the kernel's by single bf16 roundings, so the selection
    # is checked on exactly the tensors the indexer kernels read: index sets equal wherever the boundary gap exceeds
    # 1e-6 relative, selected-logit multisets equal everywhere.
    idx = idx.cpu().long()
    if c["dtype"] == torch.float32:
        _, lg = orc.lightning_indexer(aux["q_idx"][:, :T], aux["K_IComp"][:, :nb], aux["w_idx"][:, :T], c["topk"], m=m,
                                      normalize_qk=c["normalize_qk"], return_logits=True)
        ref_idx = aux["indices"][:, :T]
    else:
        ref_idx, lg = orc.lightning_indexer(aux_k["q_idx"][:, :T].float().cpu(), aux_k["K_IComp"][:, :nb].float().cpu(),
                                            aux_k["w_idx"][:, :T].float().cpu(), c["topk"], m=m,
                                            normalize_qk=c["normalize_qk"], return_logits=True)
    assert ((idx >= 0).sum(-1) == (ref_idx >= 0).sum(-1)).all()
    agree = _multiset_equal(lg, idx, ref_idx, rtol=1e-6)
    assert bool(agree.all()), float(agree.float().mean())
    if lg.shape[-1] > c["topk"]:
        sv = lg.sort(-1, descending=True).values
        a_, b_ = sv[..., c["topk"] - 1], sv[..., c["topk"]]
        clear = ((lg > float("-inf")).sum(-1) <= c["topk"]) | ((a_ - b_).abs() > 1e-6 * a_.abs().clamp_min(1e-30))
        same = (idx.sort(-1).values == ref_idx.sort(-1).values).all(-1)
        assert bool(same[clear].all()), int((~same[clear]).sum())
    # stage 3: outputs against the oracle evaluated on the kernel's selection
    idx_pad = torch.full((c["B"], aux["indices"].shape[1], c["topk"]), -1, dtype=torch.long)
    idx_pad[:, :T] = idx
    o_or = orc.csa_forward(H, *W, indices_override=idx_pad, **kw)
    assert md(out, o_or) <= tol(c["dtype"])
    if c["dtype"] == torch.float32 and bool(agree.all()):
        ref_idx = torch.from_numpy(golden[f"csa/{name}/indices"].astype(np.int64))
        same = (idx.sort(-1).values == ref_idx.sort(-1).values).all(-1)      # rows with the reference's own picks
        d = np.abs(np32(out) - golden[f"csa/{name}/out"]).reshape(c["B"], T, -1).max(-1)
        assert (d[same.numpy()] <= F32_TOL).all()


def test_csa_stage_topk_exact_on_reference_projections(kch, golden):
    """Feed identical fp32 indexer inputs to the kernel and the oracle: index SETS must be bit-exact
    wherever the boundary gap exceeds 1e-6 relative (north-star rule)."""
    g = torch.Generator().manual_seed(77)
    B, T, HI, DI, m, topk = 2, 512, 4, 64, 4, 48
    n = T // m
    q = torch.randn(B, T, HI, DI, generator=g)
    k = torch.randn(B, n, DI, generator=g)
    w = torch.randn(B, T, HI, generator=g) * 0.1
    ref, lg = orc.lightning_indexer(q, k, w, topk, m=m, normalize_qk=True, return_logits=True)
    mine = kch.csa_lightning_indexer(q.to(DEV), k.to(DEV), w.to(DEV), topk, m=m, normalize_qk=True).cpu()
    assert mine.dtype == torch.long and mine.shape == ref.shape
    sv = lg.sort(-1, descending=True).values
    nvis = ((torch.arange(T) + 1) // m).clamp(max=n)
    clear = torch.ones(B, T, dtype=torch.bool)
    rows = nvis > topk
    a, b = sv[:, :, topk - 1], sv[:, :, topk]
    clear[:, rows] = ((a - b).abs() > 1e-6 * a.abs().clamp_min(1e-30))[:, rows]
    same = (mine.sort(-1).values == ref.sort(-1).values).all(-1)
    assert same[clear].all()
    assert _multiset_equal(lg, mine, ref).all()
    # descending order of the returned picks, as torch.topk gives
    picked = torch.gather(torch.cat([lg, torch.full_like(lg[..., :1], float("-inf"))], -1), -1,
                          torch.where(mine < 0, n, mine))
    assert (picked[..., :-1] >= picked[..., 1:]).all()


def test_csa_edges(kch):
    c = CSA_CASES["small_f32"]
    w, sink, H = syn.csa_inputs(1, 1, 10, c["d"], nh=c["nh"], c=c["c"], dc=c["dc"], nIh=c["nIh"], c_I=c["c_I"], m=c["m"],
                                dtype=torch.float32, std=0.3)
    W = [w[n].to(DEV) for n in syn.CSA_WEIGHT_ORDER]
    kw = dict(m=c["m"], nh=c["nh"], nIh=c["nIh"], c=c["c"], c_I=c["c_I"], dc=c["dc"], normalize_qk=True, use_ste=False)
    Wc = [w[n] for n in syn.CSA_WEIGHT_ORDER]
    ckw = {k: v for k, v in kw.items() if k != "use_ste"}
    # T = 0
    o = kch.naive_csa(H[:, :0].to(DEV), *W, topk=4, sliding_window=4, **kw)
    assert o.shape == (1, 0, c["nh"] * c["c"])
    # topk = 0 with a window; topk = 0 without anything -> zeros; T < m
    o = kch.naive_csa(H.to(DEV), *W, topk=0, sliding_window=4, **kw)
    assert md(o, orc.csa_forward(H, *Wc, topk=0, sliding_window=4, **ckw)) <= F32_TOL
    o = kch.naive_csa(H.to(DEV), *W, topk=0, sliding_window=0, **kw)
    assert float(o.abs().max()) == 0.0
    o = kch.naive_csa(H[:, :3].to(DEV), *W, topk=4, sliding_window=0, sink_logits=sink.to(DEV), **kw)
    assert float(o.abs().max()) == 0.0      # no block closes before T=m and no window: nothing to attend
    with pytest.raises(ValueError, match="c_I"):
        kch.naive_csa(H.to(DEV), *W, topk=1, **dict(kw, c_I=0))
    with pytest.raises(ValueError, match="topk"):
        kch.naive_csa(H.to(DEV), *W, topk=-1, **kw)
    with pytest.raises(ValueError, match="W_aKV"):
        kch.naive_csa(H.to(DEV), W[0].bfloat16(), *W[1:], topk=1, **kw)
    with pytest.raises(ValueError, match="divisible"):
        kch.csa_compress_kv(H[:, :10].to(DEV), H[:, :10].to(DEV), torch.zeros(4, c["d"], device=DEV), 4)


def test_compress_matches_oracle(kch):
    g = torch.Generator().manual_seed(9)
    for dt in (torch.float32, torch.bfloat16):
        B, T, c, m = 3, 64, 40, 4
        t = [torch.randn(B, T, c, generator=g).to(dt) for _ in range(4)]
        Ba, Bb = [(torch.randn(m, c, generator=g) * 0.3).to(dt) for _ in range(2)]
        a = kch.csa_compress_kv_overlapped(*[x.to(DEV) for x in t], Ba.to(DEV), Bb.to(DEV), m)
        assert a.dtype == torch.float32
        assert md(a, orc.compress_kv_overlapped(*t, Ba, Bb, m)) <= 2e-6
        b = kch.csa_compress_kv(t[0].to(DEV), t[2].to(DEV), Ba.to(DEV), m)
        assert md(b, orc.compress_kv(t[0], t[2], Ba, m)) <= 2e-6
    e = kch.csa_compress_kv_overlapped(*[x[:, :0].to(DEV) for x in t], Ba.to(DEV), Bb.to(DEV), m)
    assert e.shape == (B, 0, c)


# ---------------------------------------------------------------------------------------------- HCA
@pytest.mark.parametrize("name", list(HCA_CASES))
def test_hca(kch, golden, name):
    c = HCA_CASES[name]
    w, sink, H = syn.hca_inputs(c["seed"], c["B"], c["T"], c["d"], nh=c["nh"], c=c["c"], dc=c["dc"], m2=c["m2"],
                                dtype=c["dtype"], random_sink=c["random_sink"], std=c.get("std", 0.02))
    out, (C, Z) = kch.naive_hca(H.to(DEV), *[w[n].to(DEV) for n in ("W_KV", "W_Z", "B_pos", "W_DQ", "W_UQ")],
                                m2=c["m2"], nh=c["nh"], c=c["c"], dc=c["dc"], sliding_window=c["win"],
                                sink_logits=sink.to(DEV) if c["sink"] else None, return_projections=True)
    assert out.dtype == c["dtype"] and C.shape == (c["B"], c["T"], c["c"])
    assert md(out, golden[f"hca/{name}/out"]) <= tol(c["dtype"])


def test_hca_errors(kch):
    c = HCA_CASES["small_f32"]
    w, sink, H = syn.hca_inputs(1, 1, 16, c["d"], nh=c["nh"], c=c["c"], dc=c["dc"], m2=c["m2"], dtype=torch.float32)
    a = [w[n].to(DEV) for n in ("W_KV", "W_Z", "B_pos", "W_DQ", "W_UQ")]
    kw = dict(m2=c["m2"], nh=c["nh"], c=c["c"], dc=c["dc"])
    with pytest.raises(ValueError, match="W_UQ"):
        kch.naive_hca(H.to(DEV), *a[:4], a[4][:-1], **kw)
    with pytest.raises(TypeError):
        kch.naive_hca(H.to(DEV).long(), *a, **kw)
    with pytest.raises(ValueError, match="sink_logits"):
        kch.naive_hca(H.to(DEV), *a, sink_logits=torch.zeros(c["nh"] + 1, device=DEV), **kw)
    assert kch.naive_hca(H[:, :0].to(DEV), *a, **kw).shape == (1, 0, c["nh"] * c["c"])


@pytest.mark.parametrize("T", [200, 512])
def test_csa_stage_topk_exact_with_bf16_queries(kch, T):
    """bf16 queries are scored in place as exact tensor-core operands (T = 512: the tcgen05 kernel with 128-query
    tiles; T = 200: the mma.sync kernel), keys as three bf16 terms: the picks must still be exact wherever the
    boundary gap exceeds 1e-6 relative.  The queries are a strided column slice, as in the layer."""
    g = torch.Generator().manual_seed(79)
    B, HI, DI, m, topk = 2, 4, 64, 4, 24
    n = T // m
    wide = torch.randn(B, T, 40 + HI * DI, generator=g).to(torch.bfloat16)
    q = wide[..., 40:].unflatten(-1, (HI, DI))
    k = torch.randn(B, n, DI, generator=g)
    w = torch.randn(B, T, HI, generator=g) * 0.1
    ref, lg = orc.lightning_indexer(q.float(), k, w, topk, m=m, normalize_qk=True, return_logits=True)
    from kch_b200 import csa as csa_mod
    wide_d = wide.to(DEV)
    qd = wide_d[..., 40:].unflatten(-1, (HI, DI))
    mine = csa_mod.indexer_topk(qd, k.to(DEV), w.to(DEV), topk, m=m, normalize_qk=True, sorted_output=True).cpu().long()
    sv = lg.sort(-1, descending=True).values
    nvis = ((torch.arange(T) + 1) // m).clamp(max=n)
    clear = torch.ones(B, T, dtype=torch.bool)
    rows = nvis > topk
    a, b = sv[:, :, topk - 1], sv[:, :, topk]
    clear[:, rows] = ((a - b).abs() > 1e-6 * a.abs().clamp_min(1e-30))[:, rows]
    same = (mine.sort(-1).values == ref.sort(-1).values).all(-1)
    assert same[clear].all(), (~same[clear]).sum()
    assert _multiset_equal(lg, mine, ref).all()
    assert kch._lib.device_status() == 0


# ---------------------------------------------------------------------------------------------- caches
@pytest.mark.parametrize("name", list(CACHE_CASES))
@pytest.mark.parametrize("bulk_prefix", [0, 13])
def test_decode_caches(kch, golden, name, bulk_prefix):
    """Token-by-token append + attend against the reference's caches; `bulk_prefix` tokens are first
    appended in one multi-token call (the prefill path), which must leave the same state."""
    c = CACHE_CASES[name]
    st = {k: v.to(DEV) for k, v in make_cache_stream(c).items()}
    cc = kch.CSADecodingCache(c["B"], c["c"], c["c_I"], c["m"], c["win"], DEV, c["dtype"])
    hc = kch.HCADecodingCache(c["B"], c["c"], c["m2"], c["win"], DEV, c["dtype"])
    names = ("Ca", "Cb", "Za", "Zb", "K_idx", "Z_idx")
    o_csa, o_hca = [], []
    t0 = 0
    if bulk_prefix:
        sl = slice(0, bulk_prefix)
        new_blocks = cc.append_step(*[st[n][:, sl] for n in names], st["Ba"], st["Bb"], st["B_idx"])
        assert new_blocks == list(range(bulk_prefix // c["m"]))
        hc.append_step(st["Ca"][:, sl], st["Za"][:, sl], st["B_pos"])
        t0 = bulk_prefix
    for t in range(t0, c["T"]):
        sl = slice(t, t + 1)
        cc.append_step(*[st[n][:, sl] for n in names], st["Ba"], st["Bb"], st["B_idx"])
        hc.append_step(st["Ca"][:, sl], st["Za"][:, sl], st["B_pos"])
        qn = torch.nn.functional.normalize(st["q"][:, sl].float(), dim=-1)
        o_csa.append(cc.forward_step(qn, st["q_idx"][:, sl].float(), st["w_idx"][:, sl].float(), topk=c["topk"],
                                     nh=c["nh"], nIh=c["nIh"], scale=1.0, sink_logits=st["sink"], use_ste=False))
        o_hca.append(hc.forward_step(qn, nh=c["nh"], scale=1.0, sink_logits=st["sink"]))
    assert cc.n_tokens_seen == c["T"] and cc.n_blocks == c["T"] // c["m"] and cc.accumulator_len == c["T"] % c["m"]
    st_tol = 1e-6 if c["dtype"] == torch.float32 else 8e-3     # 1 bf16 ulp of a stored row
    assert md(cc.C_comp, golden[f"cache/{name}/C_comp"]) <= st_tol
    assert md(cc.K_IComp, golden[f"cache/{name}/K_IComp"]) <= st_tol
    assert md(hc.C_comp, golden[f"cache/{name}/hca_C_comp"]) <= st_tol
    o_tol = F32_TOL if c["dtype"] == torch.float32 else BF16_TOL
    assert md(torch.cat(o_hca, 1), golden[f"cache/{name}/hca"][:, t0:]) <= o_tol
    if c["topk"] >= c["T"] // c["m"]:
        assert md(torch.cat(o_csa, 1), golden[f"cache/{name}/csa"][:, t0:]) <= o_tol
    else:
        d = np.abs(np32(torch.cat(o_csa, 1)) - golden[f"cache/{name}/csa"][:, t0:]).max(axis=(2, 3))
        assert (d <= o_tol).mean() >= 0.85
    ring = cc.sw_buffer.get()
    assert ring.shape == (c["B"], min(c["T"], c["win"]), c["c"])


@pytest.mark.parametrize("kind", ["fp8", "int8"])
def test_quantised_cache_against_oracle(kch, kind):
    """Block-scaled 8-bit compressed rows: parity is unpinned upstream (the reference has no such mode);
    the oracle quantises and dequantises the same rows."""
    c = dict(seed=71, B=2, T=41, c=64, c_I=16, m=4, m2=8, win=8, nh=2, nIh=2, topk=100, dtype=torch.bfloat16)
    stc = make_cache_stream(c)
    st = {k: v.to(DEV) for k, v in stc.items()}
    cc = kch.CSADecodingCache(c["B"], c["c"], c["c_I"], c["m"], c["win"], DEV, c["dtype"], kv_quant=kind)
    hc = kch.HCADecodingCache(c["B"], c["c"], c["m2"], c["win"], DEV, c["dtype"], kv_quant=kind)
    oc = orc.CSACacheOracle(c["B"], c["c"], c["c_I"], c["m"], c["win"], c["dtype"], kv_quant=kind)
    oh = orc.HCACacheOracle(c["B"], c["c"], c["m2"], c["win"], c["dtype"], kv_quant=kind)
    names = ("Ca", "Cb", "Za", "Zb", "K_idx", "Z_idx")
    for t in range(c["T"]):
        sl = slice(t, t + 1)
        cc.append_step(*[st[n][:, sl] for n in names], st["Ba"], st["Bb"], st["B_idx"])
        hc.append_step(st["Ca"][:, sl], st["Za"][:, sl], st["B_pos"])
        oc.append(*[stc[n][:, sl] for n in names], stc["Ba"], stc["Bb"], stc["B_idx"])
        oh.append(stc["Ca"][:, sl], stc["Za"][:, sl], stc["B_pos"])
        qn = torch.nn.functional.normalize(st["q"][:, sl].float(), dim=-1)
        a = cc.forward_step(qn, st["q_idx"][:, sl].float(), st["w_idx"][:, sl].float(), topk=c["topk"], nh=c["nh"],
                            nIh=c["nIh"], scale=1.0, sink_logits=st["sink"], use_ste=False)
        b = hc.forward_step(qn, nh=c["nh"], scale=1.0, sink_logits=st["sink"])
        ra = oc.step(qn.cpu(), stc["q_idx"][:, sl].float(), stc["w_idx"][:, sl].float(), topk=c["topk"],
                     sink_logits=stc["sink"], scale=1.0)
        rb = oh.step(qn.cpu(), sink_logits=stc["sink"], scale=1.0)
        assert md(a, ra) <= 1e-4 and md(b, rb) <= 1e-4, t
    assert md(cc.C_comp.float(), oc.C_comp.float()) <= 1e-2

@pytest.mark.parametrize("kind", [None, "fp8", "int8"])
def test_split_decode_attention_against_oracle(kch, kind):
    """Production geometry (c = 128, 16 heads): the one-token path runs the split-softmax decode kernel and the
    matrix-vector indexer, both driven by the cache's device counters; top-k is smaller than the visible prefix."""
    c = dict(seed=73, B=3, T=150, c=128, c_I=64, m=4, m2=8, win=16, nh=16, nIh=4, topk=12, dtype=torch.bfloat16)
    stc = make_cache_stream(c)
    st = {k: v.to(DEV) for k, v in stc.items()}
    cc = kch.CSADecodingCache(c["B"], c["c"], c["c_I"], c["m"], c["win"], DEV, c["dtype"], kv_quant=kind)
    hc = kch.HCADecodingCache(c["B"], c["c"], c["m2"], c["win"], DEV, c["dtype"], kv_quant=kind)
    oc = orc.CSACacheOracle(c["B"], c["c"], c["c_I"], c["m"], c["win"], c["dtype"], kv_quant=kind)
    oh = orc.HCACacheOracle(c["B"], c["c"], c["m2"], c["win"], c["dtype"], kv_quant=kind)
    names = ("Ca", "Cb", "Za", "Zb", "K_idx", "Z_idx")
    bulk = 37                                          # a bulk prefix first: the counters must be mirrored to the device
    cc.append_step(*[st[n][:, :bulk] for n in names], st["Ba"], st["Bb"], st["B_idx"])
    hc.append_step(st["Ca"][:, :bulk], st["Za"][:, :bulk], st["B_pos"])
    for t in range(bulk):
        sl = slice(t, t + 1)
        oc.append(*[stc[n][:, sl] for n in names], stc["Ba"], stc["Bb"], stc["B_idx"])
        oh.append(stc["Ca"][:, sl], stc["Za"][:, sl], stc["B_pos"])
    worst = 0.0
    for t in range(bulk, c["T"]):
        sl = slice(t, t + 1)
        cc.append_step(*[st[n][:, sl] for n in names], st["Ba"], st["Bb"], st["B_idx"])
        hc.append_step(st["Ca"][:, sl], st["Za"][:, sl], st["B_pos"])
        oc.append(*[stc[n][:, sl] for n in names], stc["Ba"], stc["Bb"], stc["B_idx"])
        oh.append(stc["Ca"][:, sl], stc["Za"][:, sl], stc["B_pos"])
        qn = torch.nn.functional.normalize(st["q"][:, sl].float(), dim=-1)
        a, sel = cc.forward_step(qn, st["q_idx"][:, sl].float(), st["w_idx"][:, sl].float(), topk=c["topk"], nh=c["nh"],
                                 nIh=c["nIh"], scale=1.0, sink_logits=st["sink"], use_ste=False, _return_indices=True)
        b = hc.forward_step(qn, nh=c["nh"], scale=1.0, sink_logits=st["sink"])
        ra, rsel = oc.step(qn.cpu(), stc["q_idx"][:, sl].float(), stc["w_idx"][:, sl].float(), topk=c["topk"],
                           sink_logits=stc["sink"], scale=1.0, return_indices=True)
        rb = oh.step(qn.cpu(), sink_logits=stc["sink"], scale=1.0)
        assert md(b, rb) <= 1e-4, t
        same = all(set(sel[i, 0].tolist()) - {-1} == set(rsel[i, 0].tolist()) - {-1} for i in range(c["B"]))
        if same:
            worst = max(worst, md(a, ra))
        else:                                          # a near-tie at the selection boundary: rerun the oracle on our set
            ra2 = oc.step(qn.cpu(), stc["q_idx"][:, sl].float(), stc["w_idx"][:, sl].float(), topk=c["topk"],
                          sink_logits=stc["sink"], scale=1.0, indices_override=sel.cpu())
            worst = max(worst, md(a, ra2))
    assert worst <= 1e-4
    assert cc.n_tokens_seen == c["T"] and cc.n_blocks == c["T"] // c["m"]
    ctr = cc._ctr.cpu().tolist()
    assert ctr[:5] == [c["T"] % c["m"], c["T"] // c["m"], c["T"], 1, c["T"]]
    assert kch._lib.device_status() == 0


@pytest.mark.parametrize("quant", [None, "fp8"])
def test_hybrid_decode_graph_replay_matches_eager(kch, quant):
    """One-token steps replayed from a captured CUDA graph give the same bits as the same kernels launched from
    Python, across block closings of both caches and one growth of the cache storage."""
    cfgd = dict(d_model=256, n_heads_qk=2, n_heads_v=2, head_dim_k=128, head_dim_v=128, kda_chunk_size=64, csa_m=4,
                csa_topk=8, csa_nh=4, csa_c=128, csa_dc=64, csa_nIh=2, csa_cI=64, csa_sliding_window=16, hca_m2=16,
                hca_nh=4, hca_c=128, hca_dc=64, hca_sliding_window=16)
    cfg, model, _ = _load_model(kch, cfgd, 5, 91, torch.bfloat16)
    B, prefill, steps = 2, 70, 45
    x = syn.hidden_states(92, B, prefill + steps, cfg.d_model, torch.bfloat16).to(DEV)
    outs = {}
    for mode in (False, True):
        dec = kch.HybridDecoding(model=model, use_cuda_graph=mode, kv_quant=quant)
        dec.reset()
        ys = [dec(x[:, :prefill])]
        for t in range(steps):
            ys.append(dec(x[:, prefill + t:prefill + t + 1]))
        outs[mode] = torch.cat(ys, 1).float()
        if mode:
            assert dec._graph is not None
        caches = list(dec._caches.values())
        assert all(cch.n_tokens_seen == prefill + steps for cch in caches)
        assert all(cch._ctr.cpu().tolist()[4] == prefill + steps for cch in caches)
    assert torch.isfinite(outs[True]).all()
    assert torch.equal(outs[True], outs[False])
    assert kch._lib.device_status() == 0


# ---------------------------------------------------------------------------------------------- stack
def _load_model(kch, cfgd, layers, seed, dtype):
    cfg = kch.HybridConfig(**cfgd)
    model = kch.HybridKCHAttention(cfg, total_layers=layers)
    params = syn.hybrid_params(seed, cfg, layers, dtype=torch.float32, random_sink=True)
    model.load_state_dict(params, strict=True)
    return cfg, model.to(dtype).to(DEV).eval(), params


@pytest.mark.parametrize("name", list(HYBRID_CASES))
def test_hybrid_stack(kch, golden, name):
    c = HYBRID_CASES[name]
    cfg, model, _ = _load_model(kch, c["cfg"], c["layers"], c["seed"], c["dtype"])
    assert model.layout_str() == "KDA-KDA-KDA-CSA-HCA"
    x = syn.hidden_states(c["seed"] + 100, c["B"], c["T"], cfg.d_model, c["dtype"])
    y = model(x.to(DEV))
    t = 5e-5 if c["dtype"] == torch.float32 else 6e-2     # bf16 residual stream: 1 ulp at |x|~4 is 3e-2
    assert md(y, golden[f"hybrid/{name}/y"]) <= t
    assert md(model._kda_state, golden[f"hybrid/{name}/state"]) <= (5e-5 if c["dtype"] == torch.float32 else 2e-2)
    if c["dtype"] == torch.bfloat16:
        frac = (np.abs(np32(y) - golden[f"hybrid/{name}/y"]) <= 2e-3 + 2 ** -8 * np.abs(golden[f"hybrid/{name}/y"])).mean()
        assert frac >= 0.95, frac


def test_hybrid_decode(kch, golden):
    c = DECODE_CASE
    v = golden["decode/cfg"]
    names = ["d_model", "n_heads_qk", "n_heads_v", "head_dim_k", "head_dim_v", "csa_m", "csa_topk", "csa_nh", "csa_c",
             "csa_dc", "csa_nIh", "csa_cI", "csa_sliding_window", "hca_m2", "hca_nh", "hca_c", "hca_dc",
             "hca_sliding_window"]
    cfgd = dict(kda_chunk_size=0, **{n: int(x) for n, x in zip(names, v)})
    cfg, model, _ = _load_model(kch, cfgd, 5, c["seed"], c["dtype"])
    dec = kch.HybridDecoding(model=model)
    x = syn.hidden_states(c["seed"] + 100, c["B"], c["prefill"] + c["steps"], cfg.d_model, c["dtype"]).to(DEV)
    ys = [dec(x[:, :c["prefill"]])]
    for t in range(c["steps"]):
        ys.append(dec(x[:, c["prefill"] + t:c["prefill"] + t + 1]))
    assert md(torch.cat(ys, 1), golden["decode/y"]) <= 5e-5


def test_host_pipeline_matches_direct_passes(kch):
    """Overlapped upload / compute / download of several host batches gives exactly the passes run one by one."""
    cfgd = dict(d_model=256, n_heads_qk=2, n_heads_v=2, head_dim_k=128, head_dim_v=128, kda_chunk_size=64, csa_m=4,
                csa_topk=8, csa_nh=4, csa_c=128, csa_dc=64, csa_nIh=2, csa_cI=64, csa_sliding_window=16, hca_m2=16,
                hca_nh=4, hca_c=128, hca_dc=64, hca_sliding_window=16)
    cfg, model, _ = _load_model(kch, cfgd, 5, 95, torch.bfloat16)
    xs = [syn.hidden_states(96 + i, 2, 300, cfg.d_model, torch.bfloat16).pin_memory() for i in range(4)]
    ys = [torch.empty_like(x).pin_memory() for x in xs]
    kch.HostPipeline(model, DEV).run(xs, ys)
    torch.cuda.synchronize()
    for x, y in zip(xs, ys):
        model.reset_state()
        ref = model(x.to(DEV)).cpu()
        assert torch.equal(ref, y)


@pytest.mark.parametrize("quant", [None, "fp8"])
def test_decode_state_export_import_round_trip(kch, quant):
    """A session exported after some steps and imported into a fresh wrapper continues bit for bit."""
    cfgd = dict(d_model=256, n_heads_qk=2, n_heads_v=2, head_dim_k=128, head_dim_v=128, kda_chunk_size=64, csa_m=4,
                csa_topk=8, csa_nh=4, csa_c=128, csa_dc=64, csa_nIh=2, csa_cI=64, csa_sliding_window=16, hca_m2=16,
                hca_nh=4, hca_c=128, hca_dc=64, hca_sliding_window=16)
    cfg, model, _ = _load_model(kch, cfgd, 5, 97, torch.bfloat16)
    x = syn.hidden_states(98, 2, 130, cfg.d_model, torch.bfloat16).to(DEV)
    a = kch.HybridDecoding(model=model, kv_quant=quant)
    a.reset()
    a(x[:, :90])
    for t in range(90, 110):
        a(x[:, t:t + 1])
    st = a.export_state()
    st = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in st.items()}          # e.g. through host memory
    ref = [a(x[:, t:t + 1]).float() for t in range(110, 130)]
    b = kch.HybridDecoding(model=model, kv_quant=quant)
    b.import_state(st)
    got = [b(x[:, t:t + 1]).float() for t in range(110, 130)]
    assert all(torch.equal(r, g) for r, g in zip(ref, got))
    assert all(c.n_tokens_seen == 130 for c in b._caches.values())


@pytest.mark.parametrize("quant", [None, "int8"])
def test_chunked_prefill_matches_token_by_token(kch, quant):
    """Later multi-token calls continue a sequence through the caches (chunked prefill): same outputs as feeding
    the same tokens one at a time, and the same state afterwards."""
    cfgd = dict(d_model=256, n_heads_qk=2, n_heads_v=2, head_dim_k=128, head_dim_v=128, kda_chunk_size=64, csa_m=4,
                csa_topk=64, csa_nh=4, csa_c=128, csa_dc=64, csa_nIh=2, csa_cI=64, csa_sliding_window=16, hca_m2=16,
                hca_nh=4, hca_c=128, hca_dc=64, hca_sliding_window=16)
    cfg, model, _ = _load_model(kch, cfgd, 5, 101, torch.bfloat16)
    x = syn.hidden_states(102, 2, 230, cfg.d_model, torch.bfloat16).to(DEV)
    cuts = [40, 97, 225]                                   # chunks of 57 (recurrent KDA) and 128 (chunked KDA) tokens
    a = kch.HybridDecoding(model=model, kv_quant=quant)
    a.reset()
    ya = [a(x[:, :cuts[0]])] + [a(x[:, t:t + 1]) for t in range(cuts[0], 230)]
    ya = torch.cat(ya, 1).float()
    b = kch.HybridDecoding(model=model, kv_quant=quant)
    b.reset()
    yb = [b(x[:, :cuts[0]]), b(x[:, cuts[0]:cuts[1]]), b(x[:, cuts[1]:cuts[2]])]
    assert all(c.n_tokens_seen == cuts[2] for c in b._caches.values())
    yb += [b(x[:, t:t + 1]) for t in range(cuts[2], 230)]  # and decoding goes on from the chunk-filled caches
    yb = torch.cat(yb, 1).float()
    d = (ya - yb).abs()
    assert float(d.max()) <= 6.3e-2 and float(d.mean()) <= 2e-3, (float(d.max()), float(d.mean()))   # bf16 residual stream
    for ca, cb in zip(a._caches.values(), b._caches.values()):
        assert ca.n_blocks == cb.n_blocks and ca.accumulator_len == cb.accumulator_len
        assert md(ca.C_comp.float(), cb.C_comp.float()) <= 2e-2
    assert kch._lib.device_status() == 0


@pytest.mark.parametrize("kind", ["kda", "csa", "hca"])
def test_standalone_decode_modules_against_reference(kch, golden, kind):
    """The single-operator decode modules load the reference modules' state_dict unchanged and reproduce their
    outputs (prefill of 13 tokens, then 9 one-token steps)."""
    from golden_cases import STANDALONE_CASE as c
    from kch_b200 import decoding_modules as dm
    cls = {"kda": dm.KDAAttnDecoding, "csa": dm.CSAAttnDecoding, "hca": dm.HCAAttnDecoding}[kind]
    mod = cls(c["d_model"], **c[kind])
    pre = f"standalone/{kind}/param/"
    sd = {k[len(pre):]: torch.from_numpy(golden[k]) for k in golden.files if k.startswith(pre)}
    mod.load_state_dict(sd, strict=True)
    mod = mod.to(DEV).eval()
    x = syn.hidden_states(c["seed"] + 100, c["B"], c["prefill"] + c["steps"], c["d_model"], c["dtype"]).to(DEV)
    ys = [mod(x[:, :c["prefill"]])]
    for t in range(c["steps"]):
        ys.append(mod(x[:, c["prefill"] + t:c["prefill"] + t + 1]))
    assert md(torch.cat(ys, 1), golden[f"standalone/{kind}/y"]) <= 5e-5



@pytest.mark.parametrize("kind,env,atol", [("attend", {"KCH_ATTEND": "t"}, 1e-3), ("attend", {"KCH_ATTEND": "l"}, 1e-3),
                                           ("kda", {"KCH_KDA_SCAN": "m"}, 2e-3), ("kda_long", {"KCH_KDA_SCAN": "m"}, 4e-3),
                                           ("kda", {"KCH_KDA_PREPARE": "m"}, 2e-3), ("kda_long", {"KCH_KDA_PREPARE": "m"}, 4e-3),
                                           ("linear", {"KCH_GEMM": "1"}, 0.0), ("select", {"KCH_SELECT": "s"}, 0.0),
                                           ("decode_step", {"KCH_KDA_DECODE": "o"}, 0.0),
                                           ("decode_step", {"KCH_INDEXER_DECODE": "m", "KCH_GEMM_DECODE": "0"}, 6.3e-2)])
def test_alternate_kernels_agree_with_defaults(kch, tmp_path, kind, env, atol):
    """The kernels behind an environment switch (tcgen05 attention core, mma.sync KDA scan and prepare stage, one-CTA-per-tile
    GEMM, staged select, the general KDA kernel / mma.sync indexer / general GEMM for one-token steps)
    compute the same case as the default ones: the library reads the switch once, so the alternate runs in a child.
    Tolerance 0 where both kernels are built to return the same bits; the decode-step case with another GEMM and
    indexer differs by bf16 roundings of the residual stream (|x| ~ 4)."""
    import os
    import subprocess
    import sys
    import alt_kernel_case
    ref = alt_kernel_case.run(kind)
    out = tmp_path / f"{kind}.pt"
    child_env = dict(os.environ, **env)
    subprocess.run([sys.executable, alt_kernel_case.__file__, kind, str(out)], check=True, env=child_env, timeout=300)
    alt = torch.load(out)
    assert alt.shape == ref.shape and bool(torch.isfinite(alt).all())
    assert md(alt, ref) <= atol, md(alt, ref)
