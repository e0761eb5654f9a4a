"""The drop-in claim on hardware: after `kch_b200.install()` the REFERENCE's own modules and runners execute on
the B200 kernels.

Needs the reference importable: an offline install under baseline/_ref (git-ignored; `pip install --no-index
--no-deps --target baseline/_ref <checkout>`), or a checkout named by KCH_REFERENCE_DIR.  Skipped otherwise.

  * `ops_fused.HybridKCHAttention(HybridConfig(kda_backend="b200"))` on CUDA against (a) the same reference module
    on the CPU with `kda_backend="reference"` -- the reference itself -- and (b) this package's module tree;
  * `run_decoding.HybridDecoding` (KDA_BACKEND=b200) prefill + one-token steps against the reference on the CPU;
  * the reference's `run_benchmark.main()` and `run_decoding.bench_decoding` with KDA_BACKEND=b200: rows come
    back without errors and with the row schema the reference documents (README.md:213-223).
"""
import json
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"

CFG = dict(d_model=256, n_heads_qk=2, n_heads_v=2, head_dim_k=128, head_dim_v=128, kda_chunk_size=64, csa_m=4,
           csa_topk=64, csa_nh=4, csa_c=128, csa_dc=64, csa_nIh=2, csa_cI=64, csa_sliding_window=16, hca_m2=16,
           hca_nh=4, hca_c=128, hca_dc=64, hca_sliding_window=16)


def _ref_dir():
    ref = os.environ.get("KCH_REFERENCE_DIR") or os.path.join(ROOT, "baseline", "_ref")
    return ref if os.path.isfile(os.path.join(ref, "ops_fused.py")) else None


@pytest.fixture()
def installed(monkeypatch):
    ref = _ref_dir()
    if ref is None:
        pytest.skip("the reference is not installed (baseline/_ref) and KCH_REFERENCE_DIR is not set")
    sys.dont_write_bytecode = True
    monkeypatch.syspath_prepend(ref)
    monkeypatch.setenv("KDA_BACKEND", "b200")
    import kch_b200
    done = kch_b200.install()
    yield kch_b200, done
    kch_b200.uninstall()
    from kch_b200 import _lib
    assert _lib.device_status() == 0


def _stats(a, b):
    d = (a.detach().float().cpu() - b.detach().float().cpu()).abs()
    return float(d.max()), float(d.mean())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reference_stack_runs_on_the_kernels(installed, dtype):
    kch, done = installed
    import ops_fused
    from kch_b200 import _lib, synthetic as syn
    assert {"ops_kda_backend.kda_forward", "ops_fused.kda_forward", "ops_fused.naive_csa", "ops_fused.naive_hca"} <= set(done)
    params = syn.hybrid_params(21, kch.HybridConfig(**CFG), 5, dtype=torch.float32, random_sink=True)
    x = syn.hidden_states(22, 2, 200, CFG["d_model"], dtype)

    ref_cpu = ops_fused.HybridKCHAttention(ops_fused.HybridConfig(kda_backend="reference", **CFG), 5)
    ref_cpu.load_state_dict(params, strict=True)
    ref_cpu = ref_cpu.to(dtype).eval()
    with torch.no_grad():
        y_ref = ref_cpu(x)

    ref_gpu = ops_fused.HybridKCHAttention(ops_fused.HybridConfig(kda_backend="b200", **CFG), 5)
    ref_gpu.load_state_dict(params, strict=True)
    ref_gpu = ref_gpu.to(dtype).to(DEV).eval()
    lib = _lib.load()
    lib.kch_launch_count(1)
    with torch.no_grad():
        y_gpu = ref_gpu(x.to(DEV))
    assert int(lib.kch_launch_count(0)) >= 10                     # the reference's module launched this library's kernels

    mine = kch.HybridKCHAttention(kch.HybridConfig(**CFG), 5)
    mine.load_state_dict(params, strict=True)
    mine = mine.to(dtype).to(DEV).eval()
    y_mine = mine(x.to(DEV))

    if dtype == torch.float32:
        # top-k = 64 of at most 50 blocks: every visible block is selected, so no tie can change the result
        assert _stats(y_gpu, y_ref)[0] <= 5e-5
        assert _stats(y_mine, y_gpu)[0] <= 5e-5
        assert _stats(ref_gpu._kda_state, ref_cpu._kda_state)[0] <= 5e-5
    else:
        for a, b in ((y_gpu, y_ref), (y_mine, y_gpu)):
            mx, mean = _stats(a, b)
            assert mx <= 6.3e-2 and mean <= 2e-3, (mx, mean)      # bf16 residual stream, |x| ~ 4


def test_reference_hybrid_decoding_runs_on_the_kernels(installed):
    kch, done = installed
    import run_decoding
    assert {"run_decoding.CSADecodingCache", "run_decoding.HCADecodingCache", "run_decoding.naive_csa"} <= set(done)
    torch.manual_seed(0)
    ref = run_decoding.HybridDecoding(d_model=64, total_layers=5, csa_topk=100).eval()
    assert ref.cfg.kda_backend == "b200"
    sd = {k: v.clone() for k, v in ref.state_dict().items()}
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 40, 64, generator=g)

    def run(model, dev):
        model.reset()
        with torch.no_grad():
            ys = [model(x[:, :21].to(dev))]
            for t in range(21, 40):
                ys.append(model(x[:, t:t + 1].to(dev)))
        return torch.cat(ys, 1).float().cpu()

    y_gpu = run(ref.to(DEV), DEV)
    assert type(ref._csa_caches[0]).__module__.startswith("kch_b200")     # the rebound cache classes were used
    kch.uninstall()
    os.environ["KDA_BACKEND"] = "reference"
    torch.manual_seed(0)
    cpu = run_decoding.HybridDecoding(d_model=64, total_layers=5, csa_topk=100).eval()
    cpu.load_state_dict(sd, strict=True)
    y_cpu = run(cpu, "cpu")
    assert float((y_gpu - y_cpu).abs().max()) <= 5e-5


def test_reference_runners_produce_their_rows(installed, tmp_path, monkeypatch):
    kch, done = installed
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("BENCH_LENGTHS", "128,320")
    monkeypatch.setenv("BENCH_REPEATS", "2")
    import run_benchmark
    kch.install()                                                 # the runner was imported after the first install()
    assert run_benchmark.main() == 0
    rows = json.load(open(tmp_path / "results" / "exp2_benchmark.json"))
    assert len(rows) == 2 * 8 and not any("error" in r for r in rows)
    for r in rows:
        assert {"T", "op", "time_ms", "peak_mem_MB", "device", "repeats", "compute_boundary", "n_layers", "note"} <= set(r)
        assert r["device"].startswith("cuda") and r["time_ms"] > 0
        if r["op"] in ("kda_rec", "kda_chunk", "kda_rec_hybrid", "kda_chunk_hybrid", "hybrid"):
            assert r["kda_backend"] == "b200"
    import run_decoding
    dev = torch.device(DEV)
    for name, factory in (("kda", run_decoding.KDAAttnDecoding), ("csa", run_decoding.CSAAttnDecoding),
                          ("hca", run_decoding.HCAAttnDecoding), ("hybrid", run_decoding.HybridDecoding)):
        torch.manual_seed(0)
        r = run_decoding.bench_decoding(factory(64), 64, 128, 6, dev, repeats=2)
        assert {"prefill_ms", "mean_decode_ms_per_token", "median_decode_ms_per_token", "peak_mem_MB"} <= set(r), (name, r)
        assert r["mean_decode_ms_per_token"] > 0
