"""Generate the golden vectors under tests/golden/ by running the REFERENCE itself.

Run once, where the reference checkout is importable:

    python tests/golden/make_golden.py --reference /path/to/kda-csa-hca-fusion

Inputs come from the seeded generators in ``kch_b200.synthetic`` (so they are not stored; a
checksum of each input set is stored instead to detect generator drift); outputs of the
reference's public functions are stored as fp32 arrays (bf16 values up-cast exactly).
"""
from __future__ import annotations

import argparse
import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "kda-csa-hca-fusion_b200"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

from golden_cases import (CACHE_CASES, CSA_CASES, DECODE_CASE, HCA_CASES, HYBRID_CASES,  # noqa: E402
                          KDA_CASES, STANDALONE_CASE, checksum, make_cache_stream, np32)
from kch_b200 import synthetic as syn  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("KCH_REFERENCE_DIR"),
                    help="checkout of 183600/kda-csa-hca-fusion (or set KCH_REFERENCE_DIR)")
    args = ap.parse_args()
    if not args.reference or not os.path.isdir(args.reference):
        ap.error("pass --reference <checkout of the reference> or set KCH_REFERENCE_DIR")
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    warnings.simplefilter("ignore")
    import ops_csa
    import ops_decoding_cache as odc
    import ops_fused
    import ops_hca
    import ops_kda
    import run_decoding

    torch.set_grad_enabled(False)
    out = {}

    # ---- KDA: recurrent and chunk forms ------------------------------------------------
    for name, c in KDA_CASES.items():
        q, k, v, g, beta, S0 = syn.kda_inputs(c["seed"], c["B"], c["T"], c["H"], c["K"], c["V"], c["HV"],
                                              c["dtype"], with_state=True)
        S0 = S0 if c["state"] else None
        out[f"kda/{name}/in_sum"] = checksum(q, k, v, g, beta)
        o_r, s_r = ops_kda.naive_recurrent_kda(q, k, v, g, beta, initial_state=S0, output_final_state=True)
        o_c, s_c = ops_kda.naive_chunk_kda(q, k, v, g, beta, initial_state=S0, output_final_state=True,
                                           chunk_size=c["chunk"])
        out[f"kda/{name}/o_rec"], out[f"kda/{name}/s_rec"] = np32(o_r), np32(s_r)
        out[f"kda/{name}/o_chunk"], out[f"kda/{name}/s_chunk"] = np32(o_c), np32(s_c)

    # ---- CSA: compression, indexer, full operator --------------------------------------
    for name, c in CSA_CASES.items():
        w, sink, H = syn.csa_inputs(c["seed"], c["B"], c["T"], c["d"], nh=c["nh"], c=c["c"], dc=c["dc"],
                                    nIh=c["nIh"], c_I=c["c_I"], m=c["m"], dtype=c["dtype"],
                                    random_sink=c["random_sink"], std=c.get("std", 0.02))
        out[f"csa/{name}/in_sum"] = checksum(H, *w.values())
        kw = dict(m=c["m"], topk=c["topk"], nh=c["nh"], nIh=c["nIh"], c=c["c"], c_I=c["c_I"], dc=c["dc"],
                  sliding_window=c["win"], sink_logits=sink if c["sink"] else None,
                  normalize_qk=c["normalize_qk"], use_ste=False, return_projections=True)
        o, proj = ops_csa.naive_csa(H, *[w[n] for n in syn.CSA_WEIGHT_ORDER], **kw)
        out[f"csa/{name}/out"] = np32(o)
        Ca, Cb, Za, Zb, K_idx, Z_idx = proj
        # Re-run the indexer exactly as naive_csa does internally (on the sequence right-padded to a
        # multiple of m), so that torch.topk sees the same tensor lengths and breaks ties the same way.
        T, m = c["T"], c["m"]
        pad = (-T) % m
        Fl = torch.nn.functional
        Hp = Fl.pad(H, (0, 0, 0, pad))
        Tp = T + pad
        proj_p = [Fl.linear(Hp, w[n]) for n in ("W_aKV", "W_bKV", "W_aZ", "W_bZ", "W_KV_idx", "W_Z_idx")]
        out[f"csa/{name}/C_comp"] = np32(ops_csa.csa_compress_kv_overlapped(*proj_p[:4], w["Ba"], w["Bb"], m))
        KI = ops_csa.csa_compress_kv(proj_p[4], proj_p[5], w["B_idx"], m)
        out[f"csa/{name}/K_IComp"] = np32(KI)
        cQ = Fl.linear(Hp, w["W_DQ"])
        q_idx = Fl.linear(cQ, w["W_IUQ"]).view(c["B"], Tp, c["nIh"], c["c_I"])
        w_idx = Fl.linear(Hp, w["W_w"])
        cbm = ops_csa._causal_block_mask(Tp, Tp // m, m, "cpu")
        idx = ops_csa.csa_lightning_indexer(q_idx, KI, w_idx, c["topk"], causal_block_mask=cbm,
                                            normalize_qk=c["normalize_qk"])
        out[f"csa/{name}/indices"] = idx[:, :T].numpy().astype(np.int32)

    # ---- HCA ---------------------------------------------------------------------------
    for name, c in HCA_CASES.items():
        w, sink, H = syn.hca_inputs(c["seed"], c["B"], c["T"], c["d"], nh=c["nh"], c=c["c"], dc=c["dc"],
                                    m2=c["m2"], dtype=c["dtype"], random_sink=c["random_sink"],
                                    std=c.get("std", 0.02))
        out[f"hca/{name}/in_sum"] = checksum(H, *w.values())
        o = ops_hca.naive_hca(H, w["W_KV"], w["W_Z"], w["B_pos"], w["W_DQ"], w["W_UQ"], m2=c["m2"], nh=c["nh"],
                              c=c["c"], dc=c["dc"], sliding_window=c["win"],
                              sink_logits=sink if c["sink"] else None)
        out[f"hca/{name}/out"] = np32(o)

    # ---- decode caches, token by token ---------------------------------------------------
    for name, c in CACHE_CASES.items():
        st = make_cache_stream(c)
        dt = c["dtype"]
        cc = odc.CSADecodingCache(c["B"], c["c"], c["c_I"], c["m"], c["win"], "cpu", dt)
        hc = odc.HCADecodingCache(c["B"], c["c"], c["m2"], c["win"], "cpu", dt)
        o_csa, o_hca = [], []
        for t in range(c["T"]):
            sl = slice(t, t + 1)
            cc.append_step(*[st[n][:, sl] for n in ("Ca", "Cb", "Za", "Zb", "K_idx", "Z_idx")],
                           st["Ba"], st["Bb"], st["B_idx"])
            hc.append_step(st["Ca"][:, sl], st["Za"][:, sl], st["B_pos"])
            qn = torch.nn.functional.normalize(st["q"][:, sl].float(), dim=-1)
            o_csa.append(cc.forward_step(qn, st["q_idx"][:, sl].float(), st["w_idx"][:, sl].float(),
                                         topk=c["topk"], nh=c["nh"], nIh=c["nIh"], scale=1.0,
                                         sink_logits=st["sink"], use_ste=False, normalize_qk=True))
            o_hca.append(hc.forward_step(qn, nh=c["nh"], scale=1.0, sink_logits=st["sink"]))
        out[f"cache/{name}/csa"] = np32(torch.cat(o_csa, 1))
        out[f"cache/{name}/hca"] = np32(torch.cat(o_hca, 1))
        out[f"cache/{name}/C_comp"] = np32(cc.C_comp)
        out[f"cache/{name}/K_IComp"] = np32(cc.K_IComp)
        out[f"cache/{name}/hca_C_comp"] = np32(hc.C_comp)

    # ---- hybrid stack ---------------------------------------------------------------------
    for name, c in HYBRID_CASES.items():
        cfg = ops_fused.HybridConfig(**c["cfg"])
        model = ops_fused.HybridKCHAttention(cfg, total_layers=c["layers"])
        params = syn.hybrid_params(c["seed"], cfg, c["layers"], dtype=torch.float32, random_sink=True)
        missing = model.load_state_dict(params, strict=True)
        model = model.to(c["dtype"]).eval()
        x = syn.hidden_states(c["seed"] + 100, c["B"], c["T"], cfg.d_model, c["dtype"])
        y = model(x)
        out[f"hybrid/{name}/y"] = np32(y)
        out[f"hybrid/{name}/state"] = np32(model._kda_state)

    # ---- hybrid decode (prefill + single-token steps) ---------------------------------------
    c = DECODE_CASE
    dec = run_decoding.HybridDecoding(d_model=c["d_model"], total_layers=5, csa_topk=c["csa_topk"])
    cfg = dec.cfg
    params = syn.hybrid_params(c["seed"], cfg, 5, dtype=torch.float32, random_sink=True)
    dec.model.load_state_dict(params, strict=True)
    dec = dec.to(c["dtype"]).eval()
    x = syn.hidden_states(c["seed"] + 100, c["B"], c["prefill"] + c["steps"], cfg.d_model, c["dtype"])
    ys = [dec(x[:, :c["prefill"]])]
    for t in range(c["steps"]):
        ys.append(dec(x[:, c["prefill"] + t:c["prefill"] + t + 1]))
    out["decode/y"] = np32(torch.cat(ys, 1))
    out["decode/cfg"] = np.array([cfg.d_model, cfg.n_heads_qk, cfg.n_heads_v, cfg.head_dim_k, cfg.head_dim_v,
                                  cfg.csa_m, cfg.csa_topk, cfg.csa_nh, cfg.csa_c, cfg.csa_dc, cfg.csa_nIh,
                                  cfg.csa_cI, cfg.csa_sliding_window, cfg.hca_m2, cfg.hca_nh, cfg.hca_c,
                                  cfg.hca_dc, cfg.hca_sliding_window], dtype=np.int64)

    # ---- single-operator decode modules: parameters as the reference's constructors drew them ----------
    c = STANDALONE_CASE
    x = syn.hidden_states(c["seed"] + 100, c["B"], c["prefill"] + c["steps"], c["d_model"], c["dtype"])
    os.environ["KDA_BACKEND"] = "reference"
    for kind, cls in (("kda", run_decoding.KDAAttnDecoding), ("csa", run_decoding.CSAAttnDecoding),
                      ("hca", run_decoding.HCAAttnDecoding)):
        torch.manual_seed(c["seed"])
        mod = cls(c["d_model"], **c[kind]).to(c["dtype"]).eval()
        if kind != "kda":
            mod.sink.data = torch.randn(mod.sink.shape, generator=torch.Generator().manual_seed(c["seed"] + 1))
        for k_, v_ in mod.state_dict().items():
            out[f"standalone/{kind}/param/{k_}"] = np32(v_)
        ys = [mod(x[:, :c["prefill"]])]
        for t in range(c["steps"]):
            ys.append(mod(x[:, c["prefill"] + t:c["prefill"] + t + 1]))
        out[f"standalone/{kind}/y"] = np32(torch.cat(ys, 1))

    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, "%.1f KiB" % (os.path.getsize(path) / 1024), len(out), "arrays")


if __name__ == "__main__":
    main()
