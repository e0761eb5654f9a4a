"""Tensor parallelism on real GPUs (needs >= 2): the head-sharded stack with one NCCL all-gather per layer
reproduces the single-GPU stack.  Runs as child processes, one per GPU."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CFG = dict(d_model=256, n_heads_qk=4, n_heads_v=4, head_dim_k=128, head_dim_v=128, kda_chunk_size=64, csa_m=4,
           csa_topk=1024, csa_nh=4, csa_c=128, csa_dc=64, csa_nIh=2, csa_cI=64, csa_sliding_window=16, hca_m2=16,
           hca_nh=4, hca_c=128, hca_dc=64, hca_sliding_window=16)


def _worker(rank, world, port, out):
    for p in (os.path.join(ROOT, "kda-csa-hca-fusion_b200"), ROOT):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import kch_b200
        from kch_b200 import _lib, synthetic as syn
        from kch_b200.tp import TPContext, build_tp_model
        cfg = kch_b200.HybridConfig(**CFG)
        params = syn.hybrid_params(9, cfg, 5, dtype=torch.bfloat16, random_sink=True)
        x = syn.hidden_states(10, 2, 200, cfg.d_model, torch.bfloat16).to(dev)
        tp = build_tp_model(cfg, params, 5, TPContext(rank, world, None), dev, torch.bfloat16)
        y_tp = tp(x)
        full = kch_b200.HybridKCHAttention(cfg, 5)
        full.load_state_dict(params, strict=True)
        full = full.bfloat16().to(dev).eval()
        y = full(x)
        # top-k = all blocks here, so sharding cannot change the selection; only bf16 rounding order differs
        d = (y_tp.float() - y.float()).abs()
        st = (tp._kda_state - full._kda_state[:, :, rank * 2:(rank + 1) * 2]).abs().max()
        torch.cuda.synchronize()
        out[rank] = (float(d.max()), float(d.mean()), float(st), int(_lib.device_status()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_tp2_matches_single_gpu():
    world = 2
    port = 29700 + (os.getpid() % 1000)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    for rank in range(world):
        dmax, dmean, st, status = out[rank]
        assert status == 0
        assert dmax <= 6.3e-2 and dmean <= 2e-3, (rank, dmax, dmean)      # bf16 residual stream, |x| ~ 4
        assert st <= 1e-3, (rank, st)
