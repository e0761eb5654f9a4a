"""The CPU oracle against outputs of the reference itself (tests/golden/reference_outputs.npz)."""
import numpy as np
import pytest
import torch

from golden_cases import (CACHE_CASES, CSA_CASES, DECODE_CASE, HCA_CASES, HYBRID_CASES, KDA_CASES,
                          STANDALONE_CASE, checksum, make_cache_stream, np32)
from kch_b200 import synthetic as syn
from oracle import kch_oracle as orc

F32_TOL = 2e-5          # reference's own fp32 "match" tolerance is 1e-5 (run_correctness.py:59-77)
BF16_TOL = 2e-3         # north-star output tolerance for bf16 inputs


def maxdiff(a, b):
    return float(np.max(np.abs(np32(a) - np.asarray(b)))) if np.asarray(b).size else 0.0


def tol(dtype):
    return F32_TOL if dtype == torch.float32 else BF16_TOL


@pytest.mark.parametrize("name", list(KDA_CASES))
def test_kda(golden, name):
    c = KDA_CASES[name]
    q, k, v, g, beta, S0 = syn.kda_inputs(c["seed"], c["B"], c["T"], c["H"], c["K"], c["V"], c["HV"], c["dtype"],
                                          with_state=True)
    assert (checksum(q, k, v, g, beta) == golden[f"kda/{name}/in_sum"]).all()
    S0 = S0 if c["state"] else None
    o, s = orc.recurrent_kda(q, k, v, g, beta, initial_state=S0)
    o2, s2 = orc.chunk_kda(q, k, v, g, beta, initial_state=S0, chunk_size=c["chunk"])
    t = 1e-2 if c["dtype"] == torch.bfloat16 else F32_TOL
    assert maxdiff(o, golden[f"kda/{name}/o_rec"]) <= t
    assert maxdiff(s, golden[f"kda/{name}/s_rec"]) <= F32_TOL
    assert maxdiff(o2, golden[f"kda/{name}/o_chunk"]) <= t
    assert maxdiff(s2, golden[f"kda/{name}/s_chunk"]) <= F32_TOL


def _csa_kwargs(c, sink):
    return dict(m=c["m"], topk=c["topk"], nh=c["nh"], nIh=c["nIh"], c=c["c"], c_I=c["c_I"], dc=c["dc"],
                sliding_window=c["win"], sink_logits=sink if c["sink"] else None, normalize_qk=c["normalize_qk"])


@pytest.mark.parametrize("name", list(CSA_CASES))
def test_csa(golden, name):
    c = CSA_CASES[name]
    w, sink, H = syn.csa_inputs(c["seed"], c["B"], c["T"], c["d"], nh=c["nh"], c=c["c"], dc=c["dc"], nIh=c["nIh"],
                                c_I=c["c_I"], m=c["m"], dtype=c["dtype"], random_sink=c["random_sink"],
                                std=c.get("std", 0.02))
    assert (checksum(H, *w.values()) == golden[f"csa/{name}/in_sum"]).all()
    W = [w[n] for n in syn.CSA_WEIGHT_ORDER]
    out, aux = orc.csa_forward(H, *W, return_aux=True, **_csa_kwargs(c, sink))
    T, m = c["T"], c["m"]
    nb = (T + m - 1) // m
    # compression is deterministic fp32 arithmetic on identical bf16/fp32 projections
    assert maxdiff(aux["C_comp"][:, :nb], golden[f"csa/{name}/C_comp"]) <= 1e-6
    assert maxdiff(aux["K_IComp"][:, :nb], golden[f"csa/{name}/K_IComp"]) <= 1e-6
    # top-k: the multiset of selected logits must match exactly (tie order is unpinned upstream)
    ref_idx = torch.from_numpy(golden[f"csa/{name}/indices"].astype(np.int64))
    Tm = nb * m
    _, lg = orc.lightning_indexer(aux["q_idx"][:, :T], aux["K_IComp"][:, :nb], aux["w_idx"][:, :T], c["topk"], m=m,
                                  normalize_qk=c["normalize_qk"], return_logits=True)
    mine = aux["indices"][:, :T]
    assert ((ref_idx >= 0).sum(-1) == (mine >= 0).sum(-1)).all()
    pad = torch.full_like(lg[..., :1], float("-inf"))
    lgp = torch.cat([lg, pad], -1)
    sel_ref = torch.gather(lgp, -1, torch.where(ref_idx < 0, lg.shape[-1], ref_idx)).sort(-1).values
    sel_me = torch.gather(lgp, -1, torch.where(mine < 0, lg.shape[-1], mine)).sort(-1).values
    close = torch.isclose(sel_ref, sel_me, rtol=1e-6, atol=1e-7) | (sel_ref == sel_me)
    assert close.all()
    # outputs, evaluated on the reference's own selection so that tie order cannot matter
    idx_pad = torch.full((c["B"], aux["indices"].shape[1], c["topk"]), -1, dtype=torch.long)
    idx_pad[:, :T] = ref_idx
    out2 = orc.csa_forward(H, *W, indices_override=idx_pad, **_csa_kwargs(c, sink))
    assert maxdiff(out2, golden[f"csa/{name}/out"]) <= tol(c["dtype"])
    assert out.shape == out2.shape


@pytest.mark.parametrize("name", list(HCA_CASES))
def test_hca(golden, name):
    c = HCA_CASES[name]
    w, sink, H = syn.hca_inputs(c["seed"], c["B"], c["T"], c["d"], nh=c["nh"], c=c["c"], dc=c["dc"], m2=c["m2"],
                                dtype=c["dtype"], random_sink=c["random_sink"], std=c.get("std", 0.02))
    assert (checksum(H, *w.values()) == golden[f"hca/{name}/in_sum"]).all()
    out = orc.hca_forward(H, w["W_KV"], w["W_Z"], w["B_pos"], w["W_DQ"], w["W_UQ"], m2=c["m2"], nh=c["nh"], c=c["c"],
                          dc=c["dc"], sliding_window=c["win"], sink_logits=sink if c["sink"] else None)
    assert maxdiff(out, golden[f"hca/{name}/out"]) <= tol(c["dtype"])


@pytest.mark.parametrize("name", list(CACHE_CASES))
def test_decode_caches(golden, name):
    c = CACHE_CASES[name]
    st = make_cache_stream(c)
    cc = orc.CSACacheOracle(c["B"], c["c"], c["c_I"], c["m"], c["win"], c["dtype"])
    hc = orc.HCACacheOracle(c["B"], c["c"], c["m2"], c["win"], c["dtype"])
    o_csa, o_hca = [], []
    for t in range(c["T"]):
        sl = slice(t, t + 1)
        cc.append(*[st[n][:, sl] for n in ("Ca", "Cb", "Za", "Zb", "K_idx", "Z_idx")], st["Ba"], st["Bb"], st["B_idx"])
        hc.append(st["Ca"][:, sl], st["Za"][:, sl], st["B_pos"])
        qn = orc.l2_normalize(st["q"][:, sl].float())
        o_csa.append(cc.step(qn, st["q_idx"][:, sl].float(), st["w_idx"][:, sl].float(), topk=c["topk"],
                             sink_logits=st["sink"], scale=1.0))
        o_hca.append(hc.step(qn, sink_logits=st["sink"], scale=1.0))
    assert maxdiff(cc.C_comp, golden[f"cache/{name}/C_comp"]) == 0.0 or c["dtype"] == torch.float32
    assert maxdiff(cc.C_comp, golden[f"cache/{name}/C_comp"]) <= 1e-6 + (4e-3 if c["dtype"] != torch.float32 else 0)
    assert maxdiff(cc.K_IComp, golden[f"cache/{name}/K_IComp"]) <= 1e-6 + (4e-3 if c["dtype"] != torch.float32 else 0)
    assert maxdiff(hc.C_comp, golden[f"cache/{name}/hca_C_comp"]) <= 1e-6 + (4e-3 if c["dtype"] != torch.float32 else 0)
    assert maxdiff(torch.cat(o_hca, 1), golden[f"cache/{name}/hca"]) <= F32_TOL
    if c["topk"] >= c["T"] // c["m"]:          # select-all: tie order cannot matter
        assert maxdiff(torch.cat(o_csa, 1), golden[f"cache/{name}/csa"]) <= F32_TOL
    else:                                      # sparse: rows may differ only through tied logits
        d = np.abs(np32(torch.cat(o_csa, 1)) - golden[f"cache/{name}/csa"]).max(axis=(2, 3))
        assert (d <= F32_TOL).mean() >= 0.9


@pytest.mark.parametrize("name", list(HYBRID_CASES))
def test_hybrid_stack(golden, name):
    c = HYBRID_CASES[name]
    spec = orc.HybridSpec(**c["cfg"])
    spec.build_layout(c["layers"])
    params = {k: v.to(c["dtype"]) for k, v in
              syn.hybrid_params(c["seed"], spec, c["layers"], dtype=torch.float32, random_sink=True).items()}
    x = syn.hidden_states(c["seed"] + 100, c["B"], c["T"], spec.d_model, c["dtype"])
    y, states, _ = orc.hybrid_forward(spec, params, x)
    t = 5e-5 if c["dtype"] == torch.float32 else 6e-2   # bf16 residual stream: 1 ulp at |x|~4 is 3e-2
    assert maxdiff(y, golden[f"hybrid/{name}/y"]) <= t
    assert maxdiff(torch.stack(states), golden[f"hybrid/{name}/state"]) <= (5e-5 if c["dtype"] == torch.float32 else 2e-2)


def test_hybrid_decode(golden):
    c = DECODE_CASE
    v = golden["decode/cfg"]
    names = ["d_model", "n_heads_qk", "n_heads_v", "head_dim_k", "head_dim_v", "csa_m", "csa_topk", "csa_nh", "csa_c",
             "csa_dc", "csa_nIh", "csa_cI", "csa_sliding_window", "hca_m2", "hca_nh", "hca_c", "hca_dc",
             "hca_sliding_window"]
    spec = orc.HybridSpec(kda_chunk_size=0, **{n: int(x) for n, x in zip(names, v)})
    spec.build_layout(5)
    params = syn.hybrid_params(c["seed"], spec, 5, dtype=torch.float32, random_sink=True)
    x = syn.hidden_states(c["seed"] + 100, c["B"], c["prefill"] + c["steps"], spec.d_model, c["dtype"])
    dec = orc.HybridDecodeOracle(spec, params)
    ys = [dec.forward(x[:, :c["prefill"]])]
    for t in range(c["steps"]):
        ys.append(dec.forward(x[:, c["prefill"] + t:c["prefill"] + t + 1]))
    y = torch.cat(ys, 1)
    # csa_topk >= number of blocks (select-all), as in the reference's own cache tests, so that
    # tie order in top-k cannot matter
    assert maxdiff(y, golden["decode/y"]) <= 5e-5


@pytest.mark.parametrize("kind", ["kda", "csa", "hca"])
def test_standalone_decode_modules(golden, kind):
    """KDAAttnDecoding / CSAAttnDecoding / HCAAttnDecoding of the reference (run_decoding.py:234-598), parameters as
    its constructors drew them (stored next to the outputs)."""
    c = STANDALONE_CASE
    pre = f"standalone/{kind}/param/"
    p = {k[len(pre):]: torch.from_numpy(golden[k]) for k in golden.files if k.startswith(pre)}
    x = syn.hidden_states(c["seed"] + 100, c["B"], c["prefill"] + c["steps"], c["d_model"], c["dtype"])
    dec = orc.StandaloneDecodeOracle(kind, p, **c[kind])
    ys = [dec.forward(x[:, :c["prefill"]])]
    for t in range(c["steps"]):
        ys.append(dec.forward(x[:, c["prefill"] + t:c["prefill"] + t + 1]))
    assert maxdiff(torch.cat(ys, 1), golden[f"standalone/{kind}/y"]) <= 5e-5

