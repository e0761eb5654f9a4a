"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol the header
declares, host validation rejects bad arguments with the reference's exception types before any
launch, CPU tensors are refused (no fallback), and the backend installer is reversible."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    src = open(os.path.join(ROOT, "include", "kch_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(kch_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from kch_b200 import _lib
    lib = _lib.load()
    syms = _header_symbols()
    assert len(syms) >= 18
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/kch_b200.h but not exported"
        assert s in _lib.PROTOTYPES, f"{s} has no ctypes prototype"
    assert sorted(_lib.PROTOTYPES) == syms
    assert lib.kch_abi_version() == 1


def test_argument_errors_come_back_as_codes_without_a_gpu():
    from kch_b200 import _lib
    lib = _lib.load()
    # every one of these is rejected on the host before any CUDA call
    rc = lib.kch_compress_kv(None, None, None, None, 1, 10, 8, 0, 8, 10, 0, 0, 0, None)
    assert rc < 0 and b"m=0" in lib.kch_last_error()
    rc = lib.kch_compress_kv(None, None, None, None, 1, 10, 8, 4, 8, 10, 0, 0, 0, None)
    assert rc < 0 and b"divisible" in lib.kch_last_error()
    rc = lib.kch_kda_recurrent(*([None] * 8), 1, 4, 2, 3, 8, 8, 1.0, -10.0, 0, 0, 0, 0, 0, None)
    assert rc < 0 and b"HV=3" in lib.kch_last_error()
    rc = lib.kch_indexer_topk(None, None, None, None, 1, 4, 4, 2, 0, 3, 1.0, 4, 0, -1, 0, 0, None, 0, None)
    assert rc < 0 and b"c_I" in lib.kch_last_error()
    rc = lib.kch_linear(None, None, None, None, 4, 4, 4, 2, 4, 4, 0, 0, None)
    assert rc < 0 and b"lda" in lib.kch_last_error()
    with pytest.raises(ValueError, match="lda"):
        _lib.check(rc)
    assert lib.kch_kda_chunk_workspace_bytes(4, 32768, 16, 128, 128, 64) > 0
    assert lib.kch_indexer_workspace_bytes(1, 4096, 1024, 4, 32) == 4096 * 1024 * 4
    assert lib.kch_indexer_workspace_bytes(1, 4096, 1024, 4, 64) > 4096 * 1024 * 4


def test_cpu_tensors_are_refused_not_silently_computed():
    import kch_b200
    q = torch.randn(1, 4, 2, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        kch_b200.naive_recurrent_kda(q, q, q, q, torch.rand(1, 4, 2))
    with pytest.raises(RuntimeError, match="CUDA"):
        kch_b200.kda_forward(q, q, q, q, torch.rand(1, 4, 2))
    H = torch.randn(1, 8, 16)
    W = torch.randn(4, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        kch_b200.naive_hca(H, W, W, torch.zeros(4, 4), torch.randn(4, 16), torch.randn(8, 4), m2=4, nh=2, c=4, dc=4)
    with pytest.raises(RuntimeError, match="CUDA"):
        kch_b200.CSADecodingCache(1, 8, 4, 4, 4, "cpu", torch.float32)


def test_validation_matches_reference_types_and_names():
    import kch_b200
    q = torch.randn(1, 4, 2, 8)
    with pytest.raises(ValueError, match="rank"):
        kch_b200.naive_recurrent_kda(q[0], q, q, q, torch.rand(1, 4, 2))
    with pytest.raises(ValueError, match="beta"):
        kch_b200.naive_chunk_kda(q, q, q, q, torch.rand(1, 4, 3))
    with pytest.raises(ValueError, match="kda_backend"):
        kch_b200.kda_forward(q, q, q, q, torch.rand(1, 4, 2), backend="fla")
    with pytest.raises(TypeError):
        kch_b200.kda_forward(q, q, q, q, torch.rand(1, 4, 2), g_clamp_min="x")
    with pytest.raises(ValueError, match="m=0"):
        kch_b200.csa_compress_kv(torch.zeros(1, 4, 4), torch.zeros(1, 4, 4), torch.zeros(1, 4), 0)
    with pytest.raises(ValueError, match="topk"):
        kch_b200.csa_lightning_indexer(torch.zeros(1, 2, 1, 4), torch.zeros(1, 2, 4), None, -1)
    with pytest.raises(NotImplementedError):
        kch_b200.csa_lightning_indexer(torch.zeros(1, 2, 1, 4), torch.zeros(1, 2, 4), None, 1, ste_mode="aux_contrastive")
    with pytest.raises(ValueError, match="n_heads_v"):
        kch_b200.HybridConfig(n_heads_qk=3, n_heads_v=4)
    with pytest.raises(ValueError, match="kda_backend"):
        kch_b200.HybridConfig(kda_backend="triton")
    with pytest.raises(ValueError, match="win"):
        kch_b200.CSADecodingCache(1, 8, 4, 4, -1, "cuda", torch.float32)
    with pytest.raises(TypeError):
        kch_b200.HCADecodingCache(1, 8, 4, 4, "cuda", torch.int32)


def test_module_tree_uses_reference_state_dict_names():
    import kch_b200
    from kch_b200 import synthetic as syn
    cfg = kch_b200.HybridConfig(d_model=32, n_heads_qk=2, n_heads_v=2, head_dim_k=8, head_dim_v=8, csa_c=8, csa_dc=8,
                                csa_cI=4, csa_nh=2, hca_c=8, hca_dc=8, hca_nh=2, csa_m=4, hca_m2=8)
    model = kch_b200.HybridKCHAttention(cfg, total_layers=5)
    assert model.layout == ["kda", "kda", "kda", "csa", "hca"]
    params = syn.hybrid_params(1, cfg, 5, dtype=torch.float32)
    assert set(params) == set(model.state_dict())
    model.load_state_dict(params, strict=True)


def test_install_is_reversible_when_reference_is_importable():
    import sys
    # a checkout named by the environment, else the offline install of the reference under baseline/_ref
    ref = os.environ.get("KCH_REFERENCE_DIR") or os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref, "ops_fused.py")):
        pytest.skip("the reference is not installed (baseline/_ref) and KCH_REFERENCE_DIR is not set")
    sys.path.insert(0, ref)
    try:
        import kch_b200
        import ops_fused
        import ops_kda_backend
        before = (ops_kda_backend.kda_forward, ops_fused.naive_csa, ops_fused.naive_hca)
        done = kch_b200.install()
        assert "ops_kda_backend.kda_forward" in done and "ops_fused.naive_csa" in done
        assert "ops_csa.naive_csa" in done and "ops_hca.naive_hca" in done and "ops_fused.kda_forward" in done
        assert ops_kda_backend.validate_kda_backend("b200") == "b200"
        cfg = ops_fused.HybridConfig(kda_backend="b200")
        assert cfg.kda_backend == "b200"
        # CPU tensors still reach the reference implementation through the rebound globals
        q = torch.nn.functional.normalize(torch.randn(1, 4, 2, 8), dim=-1)
        o, _ = ops_kda_backend.kda_forward(q, q, q, -torch.rand(1, 4, 2, 8), torch.rand(1, 4, 2), backend="reference")
        assert o.shape == (1, 4, 2, 8)
        with pytest.raises(RuntimeError, match="CUDA"):
            ops_kda_backend.kda_forward(q, q, q, -torch.rand(1, 4, 2, 8), torch.rand(1, 4, 2), backend="b200")
        kch_b200.uninstall()
        assert (ops_kda_backend.kda_forward, ops_fused.naive_csa, ops_fused.naive_hca) == before
        with pytest.raises(ValueError):
            ops_kda_backend.validate_kda_backend("b200")
    finally:
        sys.path.remove(ref)


def test_ring_tail_does_not_alias_the_ring_storage():
    """The window keys a chunked prefill takes from the ring before appending its own chunk must survive that
    append: while the ring is not yet full its contents are a view of the storage, and a chunk that wraps around
    overwrites the very slots the view shows."""
    from types import SimpleNamespace
    from kch_b200.decoding_cache import _SlidingWindowRingBuffer
    from kch_b200.fused import HybridDecoding
    for first, second in ((6, 6), (1, 9), (3, 20)):
        ring = _SlidingWindowRingBuffer(1, 8, 2, "cpu", torch.float32)
        rows = torch.arange(1, first + second + 1, dtype=torch.float32).view(1, -1, 1).expand(1, -1, 2)
        ring.append(rows[:, :first])
        tail = HybridDecoding._ring_tail(SimpleNamespace(_sw=ring), 8)
        want = rows[:, max(0, first - 7):first].clone()
        ring.append(rows[:, first:])
        assert torch.equal(tail, want), (first, second, tail[0, :, 0].tolist())
        assert torch.equal(ring.get(), rows[:, -8:])


def test_projection_slices_are_read_in_place():
    """Column slices of a fused projection reach the KDA kernels without a copy, also for a single token per
    sequence (where PyTorch reports an arbitrary stride for the size-1 time axis)."""
    from kch_b200.kda import _token_stride
    for B, T in ((64, 1), (1, 1), (2, 5), (1, 7)):
        proj = torch.zeros(B, T, 6288, dtype=torch.bfloat16)
        q, k, v, gd, beta = proj.split([2048, 2048, 2048, 128, 16], dim=-1)
        for t, inner in ((q.unflatten(-1, (16, 128)), 2048), (v.unflatten(-1, (16, 128)), 2048), (beta, 16)):
            t2, ld = _token_stride(t)
            assert t2.data_ptr() == t.data_ptr()
            assert ld == (6288 if B * T > 1 else inner)
    odd = torch.zeros(2, 3, 100, dtype=torch.bfloat16)[..., 1:65].unflatten(-1, (2, 32))   # misaligned start
    t2, ld = _token_stride(odd)
    assert t2.is_contiguous() and ld == 64


def test_new_entry_points_validate_on_the_host():
    from kch_b200 import _lib
    lib = _lib.load()
    rc = lib.kch_cache_advance(None, 4, None)
    assert rc < 0 and b"counters" in lib.kch_last_error()
    assert lib.kch_attend_decode_splits(64) >= 1 and lib.kch_attend_decode_splits(1) <= 32
    assert lib.kch_attend_decode_workspace_bytes(64, 16, 128) == 64 * lib.kch_attend_decode_splits(64) * 16 * 130 * 4
    assert lib.kch_decode_indexer_workspace_bytes(64, 32770) == 64 * 32772 * 4
    a = _lib.AttendDecodeArgs()
    a.B, a.nh, a.c = 4, 16, 64
    rc = lib.kch_attend_decode(a, None)
    assert rc < 0 and b"c == 128" in lib.kch_last_error()
    rc = lib.kch_decode_indexer_topk(None, 0, 0, None, 1, None, None, 0, 0, None, 2, 16, 4, 64, 0, 1, 1.0, 4, None, None, 0, None)
    assert rc < 0 and b"topk" in lib.kch_last_error()
    rc = lib.kch_layernorm_short_conv(None, None, None, 1e-5, None, None, None, None, None, 1, 8, 100, 1, 1, None)
    assert rc < 0 and b"d=100" in lib.kch_last_error()
    rc = lib.kch_indexer_topk_ex(None, 2, 64, 0, None, None, None, 1, 4, 4, 1, 64, 4, 1.0, 4, 0, -1, 0, 0, None, 0, None)
    assert rc < 0 and b"q_dtype" in lib.kch_last_error()
    assert lib.kch_kda_chunk_gate_supported(128, 128, 64, -10.0, _lib.KCH_BF16) == 1
    assert lib.kch_kda_chunk_gate_supported(64, 128, 64, -10.0, _lib.KCH_BF16) == 0
    assert lib.kch_kda_chunk_gate_supported(128, 128, 64, -10.0, _lib.KCH_F32) == 0


def test_bench_accounting():
    import importlib.util
    spec = importlib.util.spec_from_file_location("kch_bench", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    fpt = bench.algorithmic_flops_per_token(bench.C4, 32768)
    assert abs(fpt - 145.86e6) / 145.86e6 < 1e-3
    nbytes = bench.decode_state_bytes(bench.C4, 64, 131072, 2)
    assert 0.80e9 < nbytes < 0.90e9          # indexer keys counted at their stored width (bf16 + fp32 norm per row)
    assert bench.decode_state_bytes(bench.C4, 64, 131072, 1.0625) < nbytes
