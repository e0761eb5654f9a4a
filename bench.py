"""Benchmark of the hot path: hybrid-layer prefill tokens/s.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --gpus 1 --steps 2 --warmup 1      # CPU arm (oracle port)

Workload ("hybrid_prefill_c4"): the 5-layer KDA-KDA-KDA-CSA-HCA stack, d_model 2048, 16 heads x 128,
KDA chunk 64, CSA m=4 / top-k 1024 / 4x64 indexer / window 128 / sink, HCA ratio 128 / window 128 / sink,
bf16, batch 4 x T=32768 of synthetic N(0,1) hidden states, random-init N(0,0.02) weights.  One step is
one forward pass over the whole batch.  With N > 1 the total work stays fixed (strong scaling) and every layer is
tensor parallel with one all-gather per layer: the KDA layers by heads (16/N heads per GPU), the CSA / HCA layers by
query rows (`--tp-attn rows`, the default: their indexer, top-k and row gathers cost the same whatever the head count,
so only the row axis divides them) or by heads as well (`--tp-attn heads`); the mode that was not asked for is timed in
the same run and reported as `tp_variant`.  The sequences of a batch are independent as well; `--dp-sequences` deals
them out to the GPUs first (replicas with no exchange on the data path) -- an extra, not the configuration of the metric.

The JSON line carries: the device-timed value, `e2e` (host buffers, H2D + D2H inside the timed region,
through the public module API), `roofline` for the dominant kernel (the tcgen05 GEMM) measured with CUDA
events around every launch of it during the timed steps, `cpu_baseline` (the CPU oracle port timed on a
bounded sample on this box's cores), the clocks seen under load and the kernel-launch count.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "kda-csa-hca-fusion_b200"), ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "hybrid_prefill_tokens_per_s"
UNIT = "tokens/s"

C4 = dict(d_model=2048, n_heads_qk=16, n_heads_v=16, head_dim_k=128, head_dim_v=128, kda_chunk_size=64, csa_m=4,
          csa_topk=1024, csa_nh=16, csa_c=128, csa_dc=128, csa_nIh=4, csa_cI=64, csa_sliding_window=128, hca_m2=128,
          hca_nh=16, hca_c=128, hca_dc=128, hca_sliding_window=128, n_kda=3, n_csa=1, n_hca=1)
LAYERS = 5
SEED = 3
# dram__bytes_read.sum + dram__bytes_write.sum of one o_proj-shaped launch (M = 131072, N = K = 2048, no residual):
# 546.1 MB + 512.6 MB from one ncu capture at the full size, where A and C (537 MB each) cannot sit in the 126 MB L2;
# the algorithmic bytes of that launch, 2 (MK + NK + MN), are 1082 MB
NCU_GEMM_DRAM_BYTES_M131072 = 1058.7e6


def algorithmic_flops_per_token(cfg, T):
    """Closed-form forward FLOPs per token of one sequence of length T (multiply-add = 2), counted the way
    the reference's analytic model does (run_kv_cache.py:286-496): dense projections, the KDA recurrence
    and chunk terms, causal indexer entries, selected / dense compressed entries and window entries (score
    and value products), o_proj."""
    d, H, HV, K, V, C = (cfg[k] for k in ("d_model", "n_heads_qk", "n_heads_v", "head_dim_k", "head_dim_v",
                                          "kda_chunk_size"))
    kda = 2 * d * (2 * H * K + HV * V + K + HV) + 2 * K * HV * K + 2 * 3 * d      # projections + conv
    kda += 6 * HV * K * V + HV * (3 * C * K + C * C)                               # recurrence + chunk terms
    kda += 2 * HV * V * d                                                          # o_proj
    m, c, cI, nIh, nh, dc, topk, win = (cfg[k] for k in ("csa_m", "csa_c", "csa_cI", "csa_nIh", "csa_nh", "csa_dc",
                                                          "csa_topk", "csa_sliding_window"))
    nb = T // m
    csa = 2 * d * (4 * c + 2 * cI + dc + nIh) + 2 * dc * (nh * c + nIh * cI)
    vis = sum((t + 1) // m for t in range(0, T, max(1, T // 4096))) / len(range(0, T, max(1, T // 4096)))
    sel = sum(min((t + 1) // m, topk) for t in range(0, T, max(1, T // 4096))) / len(range(0, T, max(1, T // 4096)))
    wn = sum(min(t + 1, win) for t in range(0, T, max(1, T // 4096))) / len(range(0, T, max(1, T // 4096)))
    csa += 2 * nIh * cI * vis + 4 * nh * c * (sel + wn) + 2 * nh * c * d
    m2, c2, nh2, dc2, win2 = (cfg[k] for k in ("hca_m2", "hca_c", "hca_nh", "hca_dc", "hca_sliding_window"))
    vis2 = sum((t + 1) // m2 for t in range(0, T, max(1, T // 4096))) / len(range(0, T, max(1, T // 4096)))
    wn2 = sum(min(t + 1, win2) for t in range(0, T, max(1, T // 4096))) / len(range(0, T, max(1, T // 4096)))
    hca = 2 * d * (2 * c2 + dc2) + 2 * dc2 * nh2 * c2 + 4 * nh2 * c2 * (vis2 + wn2) + 2 * nh2 * c2 * d
    del nb
    return cfg["n_kda"] * kda + cfg["n_csa"] * csa + cfg["n_hca"] * hca


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs (one streaming nvidia-smi
    process, a line every 50 ms, started before and terminated after the region)."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self._proc, self._t, self._mark = index, [], None, None, 0

    def mark(self):
        """Call when the timed region starts: earlier samples (idle clocks) are left out of the summary."""
        self._mark = len(self.samples)

    def _run(self):
        try:
            for line in self._proc.stdout:
                f = [x.strip() for x in line.strip().split(",")]
                if len(f) >= 7:
                    self.samples.append(f)
        except Exception:
            pass

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                           "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE,
                                          stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
            time.sleep(0.15)          # first sample lands before the region starts
        except Exception:
            self._proc = None
        return self

    def __exit__(self, *a):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except Exception:
                self._proc.kill()
            if self._t is not None:
                self._t.join(timeout=5)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        if len(self.samples) > self._mark:
            self.samples = self.samples[self._mark:]
            self._mark = 0
        sm = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        reasons = []
        for i, name in ((3, "hw_slowdown"), (4, "hw_thermal_slowdown"), (5, "sw_thermal_slowdown"), (6, "sw_power_cap")):
            if any(s[i].lower().startswith("active") for s in self.samples):
                reasons.append(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": float(self.samples[0][1]),
                "power_w_max": max(float(s[2]) for s in self.samples), "samples": len(self.samples),
                "reasons": reasons}


class GemmProbe:
    """CUDA events around every kch_linear launch during the timed steps (the dominant kernel)."""

    def __init__(self):
        self.calls = []
        self.enabled = False

    def wrap(self, fn):
        def linear(x, W, residual=None, **kw):
            if not self.enabled:
                return fn(x, W, residual, **kw)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            y = fn(x, W, residual, **kw)
            b.record()
            M = x.numel() // x.shape[-1]
            self.calls.append((a, b, 2.0 * M * W.shape[0] * W.shape[1], M, W.shape[0], W.shape[1],
                               bool(kw.get("epilogue")), residual is not None))
            return y
        return linear

    def wrap_kslabs(self, fn):
        def linear_kslabs(a_slabs, W, residual=None):
            if not self.enabled:
                return fn(a_slabs, W, residual)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            y = fn(a_slabs, W, residual)
            b.record()
            M = a_slabs.shape[1]
            self.calls.append((a, b, 2.0 * M * W.shape[0] * W.shape[1], M, W.shape[0], W.shape[1], False,
                               residual is not None))
            return y
        return linear_kslabs

    def summary(self):
        ms = sum(a.elapsed_time(b) for a, b, *_ in self.calls)
        fl = sum(c[2] for c in self.calls)
        return ms, fl, len(self.calls)

    def by_shape(self):
        """Per distinct (M, N, K, fused epilogue, residual): launches, average ms, TFLOP/s."""
        agg = {}
        for a, b, fl, M, N, K, ep, res in self.calls:
            e = agg.setdefault((M, N, K, ep, res), [0, 0.0, 0.0])
            e[0] += 1
            e[1] += a.elapsed_time(b)
            e[2] += fl
        return [{"M": k[0], "N": k[1], "K": k[2], "fused_epilogue": k[3], "residual": k[4], "launches": v[0],
                 "ms_avg": v[1] / v[0], "tflops": v[2] / (v[1] / 1e3) / 1e12 if v[1] > 0 else 0.0}
                for k, v in sorted(agg.items(), key=lambda kv: -kv[1][1])]


def cpu_baseline_sample():
    """The CPU arm (the installed reference, else the oracle port) on the host cores, on a bounded sample: one
    sequence of T=4096 of the same geometry, one pass after none (about 10-20 s)."""
    T = 4096
    step, kind = cpu_arm(T)
    t0 = time.perf_counter()
    step()
    dt = time.perf_counter() - t0
    what = "the reference's own HybridKCHAttention" if kind == "reference" else "oracle port"
    return {"value": T / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{what}, same stack, B=1 T={T} bf16, one pass, {dt:.1f} s"}


def decode_state_bytes(cfg, B, context, kv_bytes, world=1):
    """Bytes one GPU of `world` must move in a decode step at this context (the algorithmic floor of the step; with
    heads sharded, the KDA states and the per-head weight rows divide by `world`, the rest is replicated): the three KDA
    states read and written in fp32, the CSA indexer keys as stored (bf16 row + one fp32 norm per row), the
    selected CSA rows, every HCA row, both windows, and the weights once."""
    HV, K, V = cfg["n_heads_v"], cfg["head_dim_k"], cfg["head_dim_v"]
    kda = cfg["n_kda"] * B * HV * K * V * 4 * 2 // world
    nb, nb2 = context // cfg["csa_m"], context // cfg["hca_m2"]
    idx = B * nb * (cfg["csa_cI"] * 2 + 4)
    sel = B * min(nb, cfg["csa_topk"]) * cfg["csa_c"] * kv_bytes
    hca = B * nb2 * cfg["hca_c"] * kv_bytes
    win = B * (cfg["csa_sliding_window"] * cfg["csa_c"] + cfg["hca_sliding_window"] * cfg["hca_c"]) * 2
    d = cfg["d_model"]
    w_kda = d * ((2 * cfg["n_heads_qk"] * K + HV * V + HV) // world + K) + K * HV * K // world + HV * V * d
    w_csa = d * (4 * cfg["csa_c"] + 2 * cfg["csa_cI"] + cfg["csa_dc"] + cfg["csa_nIh"]) + cfg["csa_dc"] * (
        cfg["csa_nh"] * cfg["csa_c"] // world + cfg["csa_nIh"] * cfg["csa_cI"]) + cfg["csa_nh"] * cfg["csa_c"] * d
    w_hca = d * (2 * cfg["hca_c"] + cfg["hca_dc"]) + cfg["hca_dc"] * cfg["hca_nh"] * cfg["hca_c"] // world + \
        cfg["hca_nh"] * cfg["hca_c"] * d
    weights = 2 * (cfg["n_kda"] * w_kda + cfg["n_csa"] * w_csa + cfg["n_hca"] * w_hca)
    return kda + idx + sel + hca + win + weights


def decode_bench(model, cfg_dict, B, context, steps, warmup, dev, peak_gbs, world=1, peer_gather=True):
    """One-token decode steps through `HybridDecoding` at a long context, bf16 and FP8 compressed rows.  With
    `world` > 1 every rank steps its head shard of the same batch (the compressed-KV, indexer and window caches are
    replicated, the KDA states sharded) and the step time is the maximum over the ranks; the roofline fraction is
    then taken against the bytes ONE GPU must move (its share of the states and per-head weights, all of the rest)."""
    import torch.distributed as dist

    import kch_b200
    from kch_b200.synthetic import fill_decode_state
    out = {"batch": B, "context": context, "steps": steps, "warmup": warmup, "n_gpus": world}
    if world > 1:
        # the per-layer all-gather of a decode step (256 KiB over all ranks) by plain peer stores where the
        # symmetric-memory allocator is usable, else the NCCL collective
        from kch_b200.tp import enable_peer_gather
        ctx = next((l.tp for l in model.layers if getattr(l, "tp", None) is not None), None)
        if ctx is not None and ctx.peer is None and peer_gather:
            enable_peer_gather(ctx, B * cfg_dict["d_model"] * 2, dev)
        out["allgather"] = "peer_store" if (ctx is not None and ctx.peer is not None) else "nccl"
    x = torch.randn(B, 1, cfg_dict["d_model"], device=dev, generator=torch.Generator(device=dev).manual_seed(5)
                    ).to(torch.bfloat16)
    for name, quant, kvb in (("bf16", None, 2), ("fp8", "fp8", 1.0625)):
        dec = kch_b200.HybridDecoding(model=model, kv_quant=quant, use_cuda_graph=True)
        fill_decode_state(dec, B, context, steps + warmup, dev, 11)
        for _ in range(warmup):
            dec(x)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            y = dec(x)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / steps
        if world > 1:
            t = torch.tensor([us], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item())
        nbytes = decode_state_bytes(cfg_dict, B, context, kvb, world)
        out[name] = {"us_per_step": us, "us_per_token": us / B, "tokens_per_s": B / (us * 1e-6),
                     "algorithmic_bytes_per_step_per_gpu": nbytes, "achieved_gbs_per_gpu": nbytes / (us * 1e-6) / 1e9,
                     "frac_of_hbm_peak": nbytes / (us * 1e-6) / 1e9 / peak_gbs,
                     "finite": bool(torch.isfinite(y.float()).all()), "cuda_graph": dec._graph is not None}
        dec.reset()
        del dec
        torch.cuda.empty_cache()
    model.reset_state()
    return out


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _host_cores():
    """The cores this process may use (torchrun exports OMP_NUM_THREADS=1 to its ranks; the CPU arm takes the host)."""
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def cpu_arm(T):
    """(step function, kind) of the CPU arm on one sequence of T tokens of the benchmark geometry: the installed
    reference when baseline/_ref holds it, else the oracle port."""
    from kch_b200 import synthetic as syn
    x = syn.hidden_states(SEED, 1, T, C4["d_model"], torch.bfloat16)
    if os.path.isfile(os.path.join(REF_DIR, "ops_fused.py")):
        sys.dont_write_bytecode = True
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        try:
            import ops_fused
            cfg = ops_fused.HybridConfig(kda_backend="reference", **C4)
            model = ops_fused.HybridKCHAttention(cfg, LAYERS)
            model.load_state_dict(syn.hybrid_params(SEED, cfg, LAYERS, dtype=torch.bfloat16), strict=True)
            model = model.bfloat16().eval()

            def step():
                model.reset_state()
                with torch.no_grad():
                    return model(x)
            return step, "reference"
        except Exception as exc:                                  # an incomplete install: say so and use the port
            sys.stderr.write(f"baseline/_ref is present but not usable ({exc!r}); timing the oracle port\n")
    from oracle import kch_oracle as orc
    spec = orc.HybridSpec(**C4)
    spec.build_layout(LAYERS)
    params = syn.hybrid_params(SEED, spec, LAYERS, dtype=torch.bfloat16)

    def step():
        with torch.no_grad():
            return orc.hybrid_forward(spec, params, x)
    return step, "port"


def run_reference(args):
    """CPU arm: the reference's own PyTorch path on the host cores.  When the reference is installed under
    baseline/_ref (an offline `pip install --target`, git-ignored) its unmodified `ops_fused.HybridKCHAttention`
    with `kda_backend="reference"` is what runs (`kind: "reference"`); otherwise the oracle port of the same
    stack (`kind: "port"`).  Each step is a bounded sample of the workload: one sequence of the same geometry at a
    length the monolithic reference can hold (its CSA gather is T x top-k x c fp32), so that the run ends in minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(max(1, _host_cores()))
    T = 4096 if args.steps + args.warmup <= 8 else 2048
    step, kind = cpu_arm(T)
    times = []
    with torch.no_grad():
        for i in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            step()
            if i >= args.warmup:
                times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    val = T / (ms / 1e3)
    what = ("the reference's own ops_fused.HybridKCHAttention (kda_backend='reference')" if kind == "reference"
            else "oracle port of the reference path")
    sample = f"{what}, B=1 T={T} per step (bounded sample of B=4 T=32768), {torch.get_num_threads()} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "hybrid_prefill_c4", "B": 4, "T": 32768, "layers": LAYERS, **C4},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_b200(args):
    import torch.distributed as dist

    import kch_b200
    from kch_b200 import _lib, csa as csa_mod, fused as fused_mod, hca as hca_mod, synthetic as syn
    from kch_b200.tp import TPContext, build_tp_model

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (launch with torch.distributed.run); "
                         f"WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, T = args.batch, args.seq_len
    cfg = kch_b200.HybridConfig(**C4)
    params = syn.hybrid_params(SEED, cfg, LAYERS, dtype=torch.bfloat16)
    # N GPUs: the sequences of the batch are independent, so they are dealt out first (dp ranks, no exchange on
    # the data path); GPUs beyond the batch size split the heads of their sequences (tp ranks, one all-gather
    # of head outputs per layer inside each tp group).  The total work stays that of one B x T batch.
    dp = 1
    while dp * 2 <= world and B % (dp * 2) == 0 and world % (dp * 2) == 0 and args.dp_sequences:
        dp *= 2
    tp = world // dp
    dp_rank, tp_rank = rank // tp, rank % tp
    tp_group = None
    if tp > 1 and dp > 1:
        for g in range(dp):                                   # every rank creates every group, in the same order
            grp = dist.new_group(list(range(g * tp, (g + 1) * tp)))
            if g == dp_rank:
                tp_group = grp
    allgather = None
    if tp > 1:
        ctx = TPContext(tp_rank, tp, tp_group, args.tp_attn)
        model = build_tp_model(cfg, params, LAYERS, ctx, dev, torch.bfloat16)
        allgather = "nccl"
        if not args.no_peer_gather:
            # the per-layer all-gather by plain peer stores into symmetric memory (one slab of B*T/tp rows, or of
            # h/tp heads, per rank: the same bytes either way) where that allocator is usable, else NCCL
            from kch_b200.tp import enable_peer_gather
            if enable_peer_gather(ctx, (B // dp) * T * cfg.d_model * 2 // tp, dev):
                allgather = "peer_store"
    else:
        model = kch_b200.HybridKCHAttention(cfg, LAYERS)
        model.load_state_dict(params, strict=True)
        model = model.bfloat16().to(dev).eval()
    del params
    B_local = B // dp
    x_host = syn.hidden_states(SEED, B, T, cfg.d_model, torch.bfloat16)[dp_rank * B_local:(dp_rank + 1) * B_local]
    x_host = x_host.contiguous().pin_memory()
    x = x_host.to(dev)

    probe = GemmProbe()
    wrapped = probe.wrap(csa_mod.linear)
    for mod in (csa_mod, hca_mod, fused_mod):
        mod.linear = wrapped
    csa_mod.linear_kslabs = probe.wrap_kslabs(csa_mod.linear_kslabs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        model.reset_state()
        return model(x)

    for _ in range(args.warmup):
        step()
    barrier()
    lib = _lib.load()
    lib.kch_launch_count(1)
    probe.enabled = rank == 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        clocks.mark()
        ev0.record()
        for _ in range(args.steps):
            y = step()
        ev1.record()
        barrier()
    probe.enabled = False
    launches = int(lib.kch_launch_count(0))
    ms_total = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms = ms_total / args.steps
    tokens = B * T
    value = tokens / (ms / 1e3)

    # end to end through the public host-buffer API: every step uploads its input from pinned host memory and
    # downloads its output; HostPipeline overlaps those copies with the neighbouring steps' kernels
    y_host = torch.empty(B_local, T, cfg.d_model, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(1, args.steps)
    # (under tensor parallelism each rank uploads and downloads its 1/tp run of the rows; the runs are all-gathered on the
    # device, so the host moves one copy of the batch per step, not one per GPU)
    pipe = kch_b200.HostPipeline(model, dev, tp=ctx if (tp > 1 and dp == 1) else None)
    pipe.run([x_host], [y_host])
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pipe.run([x_host] * e2e_steps, [y_host] * e2e_steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    # the same without overlap (upload, pass, download in sequence), for reference
    e0.record()
    xd = x_host.to(dev, non_blocking=True)
    model.reset_state()
    y_host.copy_(model(xd), non_blocking=True)
    e1.record()
    barrier()
    e2e_serial_ms = e0.elapsed_time(e1)
    del xd
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    decode = None
    if not args.no_decode and (dp == 1 or world == 1):          # every rank steps its head shard
        del x, y, pipe
        torch.cuda.empty_cache()
        decode = decode_bench(model, C4, args.decode_batch, args.decode_context, args.decode_steps, 8, dev,
                              float(peaks.get("hbm_gbs", 6650.0)), world, not args.no_peer_gather)
    layout_str = model.layout_str()
    variant = None
    if tp > 1 and dp == 1 and not args.no_variant:
        # the same steps with the CSA / HCA layers divided the other way (device-timed only; an extra, not the metric)
        other = "rows" if args.tp_attn == "heads" else "heads"
        del model
        torch.cuda.empty_cache()
        params = syn.hybrid_params(SEED, cfg, LAYERS, dtype=torch.bfloat16)
        vctx = TPContext(tp_rank, tp, tp_group, other)
        model = build_tp_model(cfg, params, LAYERS, vctx, dev, torch.bfloat16)
        if not args.no_peer_gather:
            from kch_b200.tp import enable_peer_gather
            enable_peer_gather(vctx, (B // dp) * T * cfg.d_model * 2 // tp, dev)
        del params
        xv = x_host.to(dev)
        for _ in range(args.warmup):
            model.reset_state()
            model(xv)
        barrier()
        v0, v1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        v0.record()
        for _ in range(args.steps):
            model.reset_state()
            yv = model(xv)
        v1.record()
        barrier()
        t = torch.tensor([v0.elapsed_time(v1) / args.steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        vms = float(t.item())
        variant = {"parallelism": f"tp{tp}_heads" if other == "heads" else f"tp{tp}_kda_heads_attn_rows",
                   "ms_per_step": vms, "value": tokens / (vms / 1e3), "unit": UNIT,
                   "finite": bool(torch.isfinite(yv.float()).all())}
        del xv, yv
        if not args.no_decode and args.decode_batch % tp == 0:
            torch.cuda.empty_cache()
            vd = decode_bench(model, C4, args.decode_batch, args.decode_context, args.decode_steps, 8, dev,
                              float(peaks.get("hbm_gbs", 6650.0)), world, not args.no_peer_gather)
            variant["decode"] = {k: ({kk: vv for kk, vv in v.items() if kk in ("us_per_step", "us_per_token", "finite", "cuda_graph")}
                                     if isinstance(v, dict) else v) for k, v in vd.items()}
    status = _lib.device_status()
    if rank == 0:
        peak_tf = float(peaks.get("bf16_tflops_sustained", 1400.0))
        peak_src = "measured (MEASURED_PEAKS.json bf16_tflops_sustained)" if peaks else "fallback 1.4 PFLOP/s sustained"
        gemm_ms, gemm_flops, gemm_calls = probe.summary()
        achieved = gemm_flops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else 0.0
        fpt = algorithmic_flops_per_token(C4, T)
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "hybrid_prefill_c4", "B": B, "T": T, "layers": LAYERS, "layout": layout_str,
                       "parallelism": ("single_gpu" if world == 1 else (f"dp{dp}_sequences" if tp == 1 else (
                           (f"tp{tp}_heads" if args.tp_attn == "heads" else f"tp{tp}_kda_heads_attn_rows") if dp == 1
                           else f"dp{dp}_sequences_x_tp{tp}_heads"))), "allgather": allgather,
                       "l2": "inputs larger than L2 (537 MB hidden states)", **C4},
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": UNIT,
                    "h2d_bytes_per_step": x_host.numel() * 2 * (dp if (tp > 1 and dp == 1) or tp == 1 else world),
                    "d2h_bytes_per_step": y_host.numel() * 2 * (dp if (tp > 1 and dp == 1) or tp == 1 else world),
                    "steps": e2e_steps, "ms_per_step": e2e_ms,
                    "api": "kch_b200.HostPipeline.run (pinned host in / out, copies overlapped with the passes)",
                    "ms_per_step_without_overlap": e2e_serial_ms},
            "gpu_launches": launches,
            "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel (all dense projections)",
                         "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                         "peak_source": peak_src, "traffic": NCU_GEMM_DRAM_BYTES_M131072 * (B * T / 131072.0),
                         "traffic_note": "DRAM bytes (read + write) of one N=2048 K=2048 launch, ncu capture at M=131072 "
                                         "(this batch); the algorithmic bytes of that launch, 2(MK + NK + MN), are 1082 MB",
                         "launches": gemm_calls,
                         "flops_per_step": gemm_flops / max(1, args.steps), "ms_per_step": gemm_ms / max(1, args.steps),
                         "shapes": probe.by_shape()},
            "layer_roofline": {"flops_per_token": fpt, "achieved_tflops": value * fpt / 1e12,
                               "frac_of_tensor_peak": value * fpt / 1e12 / peak_tf},
            "clocks": clocks.summary(), "device_status": status,
        }
        if decode is not None:
            out["decode"] = decode
        if variant is not None:
            out["tp_variant"] = variant
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline_sample()
        print(json.dumps(out))
    if world > 1:
        # the decode legs captured NCCL all-gathers into CUDA graphs; tearing the process group down after that does
        # not return on this stack, so every rank meets once more and leaves without it
        sys.stdout.flush()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--dp-sequences", action="store_true",
                    help="N > 1: deal the sequences of the batch out to the GPUs first (replicas), heads only beyond")
    ap.add_argument("--tp-only", action="store_true", help="accepted for compatibility: tensor parallelism is the default")
    ap.add_argument("--tp-attn", default="rows", choices=["heads", "rows"],
                    help="N > 1: how the CSA / HCA layers are divided: the query rows (default: their indexer, top-k and "
                         "gathers do not shrink with the head count), or query heads like KDA; KDA is always by heads, "
                         "and either way there is one all-gather per layer.  The other mode is timed too (tp_variant)")
    ap.add_argument("--no-peer-gather", action="store_true",
                    help="N > 1: keep the NCCL all-gather (default: plain peer stores into symmetric memory when available)")
    ap.add_argument("--no-variant", action="store_true", help="N > 1: skip the extra timing of the other --tp-attn mode")
    ap.add_argument("--decode-batch", type=int, default=64)
    ap.add_argument("--decode-context", type=int, default=131072)
    ap.add_argument("--decode-steps", type=int, default=256)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
