#!/usr/bin/env python
"""bench.py — prefill throughput of the B200-native Krasis hot path (driver contract: one JSON line on stdout).

  python bench.py [--gpus N --steps K --warmup W] [--impl reference] [--config qcn|qwen35|v2lite|q235b]

Workload (default = BASELINE.json configs[3], the configuration the metric is quoted on): the WHOLE Qwen3-Coder-Next
prefill — embedding gather -> 48 x (RMSNorm, Gated DeltaNet or gated GQA attention with an FP8 paged KV cache, fused
add + RMSNorm, router, 512-expert top-10 INT4 g128 MoE, INT8 gated shared expert) -> final norm -> INT8 lm_head — of one
8192-token prompt, with synthetic weights of the real shapes (krasis_b200.model.SyntheticWeights; no checkpoints exist in
this environment).  --config selects the other BASELINE configurations (DeepSeek-V2-Lite: MLA + first dense layer + INT4
shared experts; Qwen3.5-35B-A3B; Qwen3-235B at 4096 tokens).  A "step" is one such prefill.

  value     tokens/s, inputs resident in HBM, device-timed with CUDA events around K steps, max over ranks.  Per-kernel
            and per-component profiling is OFF inside this region.
  e2e       the same prefill through the public API (KrasisModel.forward) with HOST buffers: pinned token ids copied in,
            last-token logits copied out, every step, wall clock, max over ranks.
  roofline  for the kernel class with the LARGEST measured share of the step; the per-kernel table comes from a separate
            profiled pass (CUDA events around every launch, kb2_kernel_profile_*) that is not part of `value`.
  cpu_baseline / --impl reference   the reference's CPU expert path (C/AVX2 port, oracle/cpu_moe.c) on the host cores.

N > 1 (torchrun, one rank per GPU): the residual stream is token-sharded, attention head-parallel (all-gather in,
reduce-scatter out), experts sliced by rank like the reference (python/krasis/gpu_prefill.py:353-359) with an all-gather of
the routed rows and a reduce-scatter of the partial sums — NCCL over NVLink behind the C ABI (kb2_comm_*).  One prompt is
split over the GPUs: scaling = "strong".
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "prefill tokens/sec @8K ctx, Qwen3-Coder-Next Q4"
DEFAULT_TOKENS = {"qcn": 8192, "qwen35": 8192, "v2lite": 8192, "q235b": 4096}
BASELINE_CONFIG = {"qcn": "configs[3] Qwen3-Coder-Next int4gpu", "qwen35": "configs[2] Qwen3.5-35B-A3B int4gpu",
                   "v2lite": "configs[1] DeepSeek-V2-Lite int4gpu", "q235b": "configs[4] Qwen3-235B-A22B int4gpu (prefill half)"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf_sustained=d["bf16_tflops_sustained"],
                    source="measured (MEASURED_PEAKS.json)")
    return dict(hbm_gbs=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback (B200_PROFILING.md)")


def host_threads():
    """Threads this process may really use: affinity mask capped by the cgroup CPU quota."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        q, per = open("/sys/fs/cgroup/cpu.max").read().split()
        if q != "max":
            n = max(1, min(n, int(int(q) / int(per))))
    except Exception:
        pass
    return n


class ClockSampler(threading.Thread):
    """nvidia-smi clocks / throttle reasons during the timed region (B200_PROFILING.md recipe)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        super().__init__(daemon=True)
        self.gpu, self.rows, self._halt = gpu_index, [], threading.Event()

    def run(self):
        while not self._halt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.gpu)], capture_output=True, text=True, timeout=5).stdout
                for line in out.strip().splitlines():
                    self.rows.append([c.strip() for c in line.split(",")])
            except Exception:
                pass
            self._halt.wait(0.2)

    def stop(self):
        self._halt.set()
        self.join(timeout=6)
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit())
        reasons = set()
        for r in self.rows:
            if len(r) >= 8:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        mx = max((float(r[2]) for r in self.rows if len(r) >= 8 and r[2].replace(".", "").isdigit()), default=None)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def preset(args):
    from dataclasses import replace
    from krasis_b200.model import PRESETS
    cfg = PRESETS[args.config]
    if args.layers:
        cfg = replace(cfg, num_hidden_layers=args.layers)
    return cfg


# --------------------------------------------------------------------------------------------- CPU arm

def cpu_sample_gguf(cfg, budget_s=15.0, threads=0):
    """BASELINE configs[0]: the reference's CPU path on native GGUF blocks (moe_forward_gguf, src/moe.rs:990-1110): Q4_K
    gate/up and — because K = moe_intermediate_size = 1408 is not a multiple of 256 for DeepSeek-V2-Lite — Q8_0 down
    (SURVEY.md §8d C1), random blocks with sane fp16 scales, one weight set cycled over the MoE layer passes."""
    import numpy as np
    from oracle import cpu_ref, gguf_blocks as G
    H, I, E, k, L = cfg.hidden_size, cfg.moe_intermediate_size, cfg.n_routed_experts, cfg.num_experts_per_tok, cfg.num_moe_layers
    rng = np.random.default_rng(0xDEADBEEF)
    t13 = G.GGML_Q4_K
    t2 = G.GGML_Q4_K if I % 256 == 0 else G.GGML_Q8_0
    gate = G.random_blocks(rng, t13, E * I, H).reshape(E, I, -1)
    up = G.random_blocks(rng, t13, E * I, H).reshape(E, I, -1)
    down = G.random_blocks(rng, t2, E * H, I).reshape(E, H, -1)
    avail = host_threads()
    nthreads = threads or min(avail, 64)

    def run(n_tok):
        x = rng.normal(0, 1, (n_tok, H)).astype(np.float32)
        x /= np.sqrt((x ** 2).mean(axis=1, keepdims=True))
        xb = ((x.view(np.uint32) + 0x8000) >> 16).astype(np.uint16)
        ids = np.stack([rng.choice(E, k, replace=False) for _ in range(n_tok)]).astype(np.int32)
        w = rng.dirichlet(np.ones(k), n_tok).astype(np.float32)
        t0 = time.perf_counter()
        for _ in range(L):
            cpu_ref.moe_forward_gguf(gate, up, down, t13, t2, H, I, xb, ids, w, nthreads=nthreads)
        return time.perf_counter() - t0

    run(1)
    t1 = run(4) / 4
    n_tok = int(max(2, min(2048, budget_s / max(t1, 1e-4))))
    dt = run(n_tok)
    return dict(value=n_tok / dt, unit="tokens/s", cores=nthreads, host_threads_available=avail, kind="port",
                sample=f"{n_tok} tokens x {L} MoE layer passes, {cfg.name} expert geometry (H{H} I{I} E{E} top-{k}), native GGUF blocks "
                       f"({G.NAMES[t13]} gate/up, {G.NAMES[t2]} down), one random weight set cycled; C/AVX2 port of moe_forward_gguf "
                       f"(src/moe.rs:990-1110, src/gguf_kernels.rs:271-425,690-756) ({dt:.1f}s); routed-expert blocks only"), n_tok, dt


def cpu_sample(cfg, budget_s=15.0, n_weight_sets=2, threads=0, fmt="int4"):
    if fmt == "gguf":
        return cpu_sample_gguf(cfg, budget_s=budget_s, threads=threads)
    return _cpu_sample_int4(cfg, budget_s, n_weight_sets, threads)


def _cpu_sample_int4(cfg, budget_s=15.0, n_weight_sets=2, threads=0):
    """Time the C/AVX2 port of the reference's CPU expert path (moe_forward_unified, src/moe.rs:572-715) on a bounded
    token sample of the SAME workload geometry (one pass per MoE layer per token).  Weights: n_weight_sets layers of random
    packed INT4 cycled over the layer passes; routing: uniform without replacement + Dirichlet(1) weights
    (tests/bench_engine_isolated.py:88-92)."""
    import numpy as np
    from oracle import cpu_ref
    H, I, E, k, L = cfg.hidden_size, cfg.moe_intermediate_size, cfg.n_routed_experts, cfg.num_experts_per_tok, cfg.num_moe_layers
    rng = np.random.default_rng(0xDEADBEEF)
    sets = []
    for _ in range(n_weight_sets):
        w13 = rng.integers(0, 2 ** 32, (E, H // 8, 2 * I), dtype=np.uint64).astype(np.uint32)
        w2 = rng.integers(0, 2 ** 32, (E, I // 8, H), dtype=np.uint64).astype(np.uint32)
        s13 = ((rng.uniform(0.004, 0.012, (E, H // 128, 2 * I)).astype(np.float32).view(np.uint32) + 0x8000) >> 16).astype(np.uint16)
        s2 = ((rng.uniform(0.004, 0.012, (E, I // 128, H)).astype(np.float32).view(np.uint32) + 0x8000) >> 16).astype(np.uint16)
        sets.append((w13, s13, w2, s2))
    avail = host_threads()

    def run(n_tok):
        x = rng.normal(0, 1, (n_tok, H)).astype(np.float32)
        x /= np.sqrt((x ** 2).mean(axis=1, keepdims=True))
        xb = ((x.view(np.uint32) + 0x8000) >> 16).astype(np.uint16)
        ids = np.stack([rng.choice(E, k, replace=False) for _ in range(n_tok)]).astype(np.int32)
        w = rng.dirichlet(np.ones(k), n_tok).astype(np.float32)
        t0 = time.perf_counter()
        for l in range(L):
            cpu_ref.moe_forward_int4(*sets[l % n_weight_sets], xb, ids, w, nthreads=nthreads)
        return time.perf_counter() - t0

    # "all the host threads it can use": the flattened dispatch has k*H/.. work items per phase (src/moe.rs:727-740), so more
    # threads than that only add barrier cost; pick the fastest of a few thread counts on a 2-token probe and say which.
    nthreads = threads or avail
    run(1)                                                # warms the thread pool, first-touches the weights
    if not threads:
        best = None
        for cand in sorted({c for c in (8, 16, 32, 64, avail) if c <= avail}):
            nthreads = cand
            t = run(2) / 2
            if best is None or t < best[0]:
                best = (t, cand)
        nthreads = best[1]
    t1 = run(4) / 4                                       # calibration
    n_tok = int(max(2, min(4096, budget_s / max(t1, 1e-4))))
    dt = run(n_tok)
    return dict(value=n_tok / dt, unit="tokens/s", cores=nthreads, host_threads_available=avail, kind="port",
                sample=f"{n_tok} tokens x {L} MoE layer passes, {cfg.name} expert geometry (H{H} I{I} E{E} top-{k}), {n_weight_sets} random "
                       f"weight sets cycled; C/AVX2 port of src/moe.rs:572-715 + src/kernel/avx2.rs:1066-1206 ({dt:.1f}s); routed-expert "
                       f"MoE blocks only (the reference's CPU expert path) — attention is not in the CPU sample"), n_tok, dt


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = preset(args)
    per_step = max(3.0, min(20.0, 60.0 / max(1, args.steps + args.warmup)))
    vals = []
    for i in range(args.warmup + args.steps):
        r, n_tok, dt = cpu_sample(cfg, budget_s=per_step, fmt=args.cpu_format)
        if i >= args.warmup:
            vals.append((r, n_tok, dt))
    tot_tok = sum(v[1] for v in vals)
    tot_t = sum(v[2] for v in vals)
    cb = dict(vals[-1][0])
    cb["value"] = tot_tok / tot_t
    line = {"impl": "reference", "metric": METRIC, "value": tot_tok / tot_t, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * tot_t / max(1, args.steps),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int16xint4->f32",
            "data": "synthetic", "config": workload_config(args, cfg, 1),
            "cpu_baseline": cb,
            "e2e": {"value": tot_tok / tot_t, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(args, cfg, n):
    n_lin = sum(cfg.layer_type(i) == "linear_attention" for i in range(cfg.num_hidden_layers))
    att = ("MLA (FP8 latent cache)" if cfg.is_mla else f"gated GQA {cfg.num_attention_heads}/{cfg.num_key_value_heads}/{cfg.gqa_head_dim}"
           if cfg.gated_attention else f"GQA {cfg.num_attention_heads}/{cfg.num_key_value_heads}/{cfg.gqa_head_dim}")
    if not cfg.shared_width:
        shared = "no shared expert"
    elif cfg.shared_expert_gate:
        shared = "INT8 gated shared expert"
    else:
        shared = "INT4 fused shared experts (manager-owned)" if n == 1 else "INT8 shared experts"
    return {"workload": f"{args.config}_full_prefill: {cfg.name} architecture, {cfg.num_hidden_layers} layers ({n_lin} Gated-DeltaNet, "
                        f"{cfg.num_hidden_layers - n_lin} {att}, {cfg.first_k_dense_replace} dense-MLP), {cfg.n_routed_experts}-expert "
                        f"top-{cfg.num_experts_per_tok} INT4 g128 MoE (H{cfg.hidden_size} I{cfg.moe_intermediate_size}) + {shared}, final norm + "
                        f"INT8 lm_head, {args.tokens}-token prompt",
            "baseline_config": BASELINE_CONFIG[args.config],
            "tokens": args.tokens, "layers": cfg.num_hidden_layers,
            "parallelism": (f"tp{n}+ep{n}: token-sharded residual stream, head-parallel attention (all-gather / reduce-scatter), "
                            f"experts sliced by rank (all-gather rows, reduce-scatter partial sums), NCCL behind the C ABI") if n > 1 else "single",
            "l2_policy": "inputs larger than L2: every layer streams its own expert weights (0.3-1.2 GB per layer) from HBM",
            "kv_cache": "FP8 E4M3 paged (16 tokens/page)"}


# --------------------------------------------------------------------------------------------- roofline bookkeeping

def algorithmic_work(cfg, M, R):
    """Algorithmic FLOPs (tensor-bound classes) or bytes (HBM-bound classes) per STEP of each kernel class, on one rank
    (DESIGN.md §4 states the per-unit figures).  Returns {class: (bound, work_per_step)}."""
    H, I, k, E = cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts_per_tok, cfg.n_routed_experts
    L = cfg.num_hidden_layers
    n_moe = cfg.num_moe_layers
    types = [cfg.layer_type(i) for i in range(L)]
    n_gdn, n_mla = types.count("linear_attention"), types.count("mla")
    n_gqa = L - n_gdn - n_mla
    nk, nv, dk, dv = cfg.linear_num_key_heads // R, cfg.linear_num_value_heads // R, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    kd, vd = nk * dk, nv * dv
    nh, d = cfg.num_attention_heads // R, cfg.gqa_head_dim
    nkv = max(1, cfg.num_key_value_heads // R)
    nch = (M + 63) // 64
    Ml = M // R
    w = {}
    w["grouped_gemm<gate_up+silu_mul>"] = ("tensor", n_moe * 2.0 * M * k * H * 2 * I / R)
    w["grouped_gemm<down>"] = ("tensor", n_moe * 2.0 * M * k * I * H / R)
    if cfg.shared_width and not cfg.shared_expert_gate and R == 1:      # manager-owned INT4 shared experts run the same kernels
        w["grouped_gemm<gate_up+silu_mul>"] = ("tensor", w["grouped_gemm<gate_up+silu_mul>"][1] + n_moe * 2.0 * M * H * 2 * cfg.shared_width)
        w["grouped_gemm<down>"] = ("tensor", w["grouped_gemm<down>"][1] + n_moe * 2.0 * M * cfg.shared_width * H)
    w["router_gemm"] = ("tensor", n_moe * 2.0 * Ml * H * E)
    # Gated DeltaNet, per (head, 64-token chunk): kcd.S, q.S, k^T.v (2*64*dk*dv each) + intra.v (2*64*64*dv); prepare: k.k^T,
    # q.k^T (2*64*64*dk each) + the unit-lower-triangular solve with dk+dv right-hand sides (64*64*(dk+dv))
    w["gdn_chunk_scan"] = ("tensor", n_gdn * nv * nch * (3 * 2.0 * 64 * dk * dv + 2.0 * 64 * 64 * dv))
    w["gdn_chunk_prepare"] = ("tensor", n_gdn * nv * nch * (2 * 2.0 * 64 * 64 * dk + 64.0 * 64 * (dk + dv)))
    w["gdn_prep(conv+l2norm+gates)"] = ("hbm", n_gdn * M * 2.0 * ((2 * kd + 2 * vd) + (2 * kd + vd)))         # read qkvz, write q,k,v
    w["gdn_post(gated_rmsnorm)"] = ("hbm", n_gdn * M * 2.0 * 3 * vd)                                           # core + z in, normed out
    if cfg.is_mla:
        qd = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
        w["fmha"] = ("tensor", n_mla * 2.0 * M * M / 2 * nh * (qd + cfg.v_head_dim))
    else:
        w["fmha"] = ("tensor", n_gqa * 4.0 * M * M / 2 * nh * d)
    dense = n_gdn * (2.0 * M * H * (2 * kd + 2 * vd) + 2.0 * M * H * 2 * nv + 2.0 * M * vd * H)
    if cfg.is_mla:
        lora, qd = cfg.kv_lora_rank, cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
        dense += n_mla * (2.0 * M * H * (lora + cfg.qk_rope_head_dim) + 2.0 * M * H * nh * qd + 2.0 * M * lora * nh * 256 + 2.0 * M * nh * 128 * H)
    else:
        dense += n_gqa * (2.0 * M * H * nh * d * (2 if cfg.gated_attention else 1) + 2 * 2.0 * M * H * nkv * d + 2.0 * M * nh * d * H)
    w["dense_gemm<bf16>"] = ("tensor", dense)
    i8 = 2.0 * H * cfg.vocab_size                                                                               # lm_head on the last token
    if cfg.shared_width and (cfg.shared_expert_gate or R > 1):
        i8 += n_moe * 2.0 * Ml * H * 3 * cfg.shared_width
    i8 += cfg.first_k_dense_replace * 2.0 * Ml * H * 3 * cfg.intermediate_size
    w["dense_gemm<int8>"] = ("tensor", i8)
    w["combine"] = ("hbm", n_moe * (M * k * H * 2.0 / R * 1.0 + M * H * 2.0 * 2))
    w["binning(count+scan+scatter)"] = ("hbm", n_moe * (M * H * 2.0 + M * k * H * 2.0 / R))
    w["rmsnorm"] = ("hbm", (2 * L + 1) * Ml * H * 2.0 * 4)                                                      # x, residual in; x, residual out
    w["kv_gather(fp8->bf16)"] = ("hbm", (n_gqa * M * nkv * d * 2 * 3.0) if not cfg.is_mla else n_mla * M * (cfg.kv_lora_rank + 64) * 3.0)
    return w


def load_traffic():
    """ncu DRAM bytes per launch, per kernel class, from the committed capture summary (profiles/kernel_traffic.json)."""
    p = os.path.join(ROOT, "profiles", "kernel_traffic.json")
    try:
        return json.load(open(p))
    except Exception:
        return {}


# --------------------------------------------------------------------------------------------- GPU arm

def run_full_model(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from krasis_b200 import capi
    from krasis_b200.model import KrasisModel

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    comm = None
    if world > 1:
        from krasis_b200.parallel import Communicator
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        torch.cuda.set_device(local)
        comm = Communicator.from_torch_distributed(local)       # NCCL behind the C ABI; torch.distributed only carried the id
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = preset(args)
    M = args.tokens
    model = KrasisModel(cfg, device=local, max_tokens=M, rank=rank, num_ranks=world, comm=comm)
    eng = model.engine
    g = torch.Generator().manual_seed(42)
    tok_host = torch.randint(0, cfg.vocab_size, (M,), generator=g, dtype=torch.int32).pin_memory()
    pos = torch.arange(M, dtype=torch.int32, device=dev)
    tok = tok_host.to(dev)
    logits_host = torch.empty((1, cfg.vocab_size), dtype=torch.float32).pin_memory()

    use_graph = not args.no_graph

    def step():
        if use_graph:
            return model.forward_graphed(tok, pos)        # captured on the first warm-up step; eager fallback inside
        return model.forward(tok, pos, model.new_sequence())

    def eager_step():
        return model.forward(tok, pos, model.new_sequence())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world > 1:
            t = torch.tensor([x], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return x

    for _ in range(args.warmup):
        step()
    barrier()
    # ---- timed region: no per-kernel events, no component spans
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    graphed = use_graph and model._graphs.get(M) not in (None, False)
    l0 = capi.total_launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms = max_over_ranks(ev0.elapsed_time(ev1))
    launches = capi.total_launches() - l0          # 0 when the steps were graph replays: counted from the eager profiled pass below
    clocks = sampler.stop() if sampler else None
    ms_per_step = ms / args.steps
    value = M / (ms_per_step * 1e-3)

    # ---- end to end: pinned host token ids -> device, forward, last-token logits -> pinned host, every step
    def e2e_step():
        tk = tok_host.to(dev, non_blocking=True)
        lg = model.forward_graphed(tk, pos) if use_graph else model.forward(tk, pos, model.new_sequence())
        logits_host.copy_(lg, non_blocking=True)
        torch.cuda.synchronize()
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    dt = max_over_ranks((time.perf_counter() - t0) / args.steps)
    e2e = {"value": M / dt, "unit": "tokens/s", "h2d_bytes_per_step": M * 4, "d2h_bytes_per_step": cfg.vocab_size * 4,
           "ms_per_step": dt * 1e3,
           "entry": ("KrasisModel.forward_graphed(token_ids, positions): pinned host token ids in, CUDA-graph replay of the prefill step, last-token logits out"
                     if graphed else "KrasisModel.forward(token_ids, positions, seq_states): pinned host token ids in, last-token logits out")}

    # ---- separate profiled pass (not part of `value`): CUDA events around every kernel launch + per-component spans
    prof_steps = max(1, min(2, args.steps))
    capi.kernel_profile(True)
    model.timing_start()
    barrier()
    l1 = capi.total_launches()
    for _ in range(prof_steps):
        eager_step()
    if graphed:
        launches = (capi.total_launches() - l1) // prof_steps * args.steps      # a replay launches exactly what the captured eager step did
    kprof = {n: (t / prof_steps, c // prof_steps) for n, (t, c) in capi.kernel_profile_collect().items()}
    comp = {kk: v / prof_steps for kk, v in model.timing_collect().items()}
    capi.kernel_profile(False)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    pk = peaks()
    work = algorithmic_work(cfg, M, world)
    traffic = load_traffic()
    table = {}
    for name, (t_ms, n) in sorted(kprof.items(), key=lambda kv: -kv[1][0]):
        row = {"ms_per_step": t_ms, "launches_per_step": n}
        if name in work and t_ms > 0:
            bound, amount = work[name]
            row["bound"] = bound
            if bound == "tensor":
                row["achieved_tflops"] = amount / (t_ms * 1e-3) / 1e12
                row["frac_of_peak"] = row["achieved_tflops"] / pk["tf_sustained"]
            else:
                row["achieved_gbs"] = amount / (t_ms * 1e-3) / 1e9
                row["frac_of_peak"] = row["achieved_gbs"] / pk["hbm_gbs"]
        table[name] = row
    top = next(iter(table)) if table else None
    roofline = None
    if top:
        r = table[top]
        tensor = r.get("bound", "tensor") == "tensor"
        ach = r.get("achieved_tflops" if tensor else "achieved_gbs")
        roofline = {"kernel": top, "bound": "tensor" if tensor else "hbm", "achieved": ach,
                    "peak": pk["tf_sustained"] if tensor else pk["hbm_gbs"], "unit": "TFLOP/s" if tensor else "GB/s",
                    "frac": r.get("frac_of_peak"),
                    "traffic": traffic.get(top, {}).get("dram_bytes_per_launch") if world == 1 and M == DEFAULT_TOKENS[args.config] else None,
                    "traffic_source": traffic.get(top, {}).get("source"),
                    "peak_source": pk["source"] + (", sustained figure (kernel timed inside a long step)" if tensor else ""),
                    "selection": "kernel class with the largest summed device time in the profiled pass",
                    "share_of_profiled_step": r["ms_per_step"] / max(1e-9, sum(x["ms_per_step"] for x in table.values())),
                    "avg_launch_ms": r["ms_per_step"] / max(1, r["launches_per_step"]),
                    "algorithmic_per_step": work.get(top, (None, None))[1],
                    "per_kernel": table, "component_ms_per_step": comp}
    cnt = eng.last_expert_counts().astype(np.float64)          # routing load of the last MoE layer of the last step
    if roofline:
        roofline["last_layer_tokens_per_expert"] = {"mean": float(cnt.mean()), "max": float(cnt.max()), "p50": float(np.median(cnt)),
                                                    "below_32": int((cnt < 32).sum()), "above_192": int((cnt > 192).sum())}
    cpu_b = None
    if not args.no_cpu_baseline:
        cpu_b, _, _ = cpu_sample(cfg, budget_s=args.cpu_budget, fmt=args.cpu_format)
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int4 experts x bf16 activations (fp32 acc), bf16 attention, fp8 KV, int8 shared expert / lm_head",
            "data": "synthetic", "config": workload_config(args, cfg, world), "clocks": clocks, "e2e": e2e,
            "gpu_launches": int(launches), "cuda_graph": bool(graphed), "roofline": roofline, "cpu_baseline": cpu_b}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="qcn", choices=["qcn", "qwen35", "v2lite", "q235b"],
                    help="BASELINE configuration: qcn (default, the one the metric is quoted on), qwen35, v2lite, q235b")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling runs)")
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying the captured step")
    ap.add_argument("--cpu-format", default="int4", choices=["int4", "gguf"],
                    help="CPU arm: int4 = moe_forward_unified on INT4 g128 (default); gguf = moe_forward_gguf on native Q4_K/Q8_0 blocks "
                         "(BASELINE configs[0]: --config v2lite --impl reference --cpu-format gguf --tokens 2048)")
    ap.add_argument("--arch", default="moe", choices=["moe", "vofelix", "megolorn", "gurozen", "zaronex"],
                    help="moe (default): the BASELINE workload above; vofelix: prefill / decode throughput of the ragged-batch model at "
                         "real layer sizes beside the Gated-DeltaNet and MLA blocks at equal size (1 GPU); megolorn: the same for the "
                         "differential-attention / routed-expert model beside Vofelix and the GQA block at equal size; gurozen: the same for "
                         "the capped-attention / channel-decay delta rule / squared-relu expert model beside the Megolorn and Vofelix blocks; "
                         "zaronex: the same for the depth-averaged model of side-by-side mixers (pooled-block attention, gated linear "
                         "attention, selective scan, latent attention) beside the Gurozen and Vofelix blocks, with its new kernels alone")
    args = ap.parse_args()
    if args.arch == "vofelix":
        from krasis_b200.bench_seq import run as run_seq
        run_seq(args, peaks())
        return
    if args.arch == "megolorn":
        from krasis_b200.bench_seq import run_megolorn
        run_megolorn(args, peaks())
        return
    if args.arch == "gurozen":
        from krasis_b200.bench_seq import run_gurozen
        run_gurozen(args, peaks())
        return
    if args.arch == "zaronex":
        from krasis_b200.bench_seq import run_zaronex
        run_zaronex(args, peaks())
        return
    args.tokens = args.tokens or DEFAULT_TOKENS[args.config]
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_full_model(args)


if __name__ == "__main__":
    main()
