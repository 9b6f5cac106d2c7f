"""Throughput of the ragged-batch models (Vofelix, Megolorn, Gurozen, Zaronex) at layer sizes of real models, beside the framework's closest existing blocks at
equal size: prefill tokens/s (one prompt, whole and in portions), decode tokens/s (several live requests, one token each per step),
and per-mixer times — the gated delta mixer against the Gated-DeltaNet block, windowed latent attention against the MLA block.
Random weights; device timing with CUDA events after warm-up; the weights of a step exceed the L2 cache."""
import json

import torch


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def bench_config(width=2048, window=1024, vocab=32768):
    """Qwen3-Next's linear-attention geometry for the delta mixer, DeepSeek-V2-Lite's MLA geometry for latent attention."""
    delta = {"heads": 32, "kv_heads": 16, "dim": 128, "vdim": 128, "conv": 4}
    latent = {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5, "mask": {"size": window},
              "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    layers = [_layer("delta", delta), _layer("delta", delta, ff=4 * width), _layer("latent_attention", latent, ff=4 * width),
              _layer("delta", delta)]
    return {"architecture": "Vofelix", "vocab": vocab, "width": width, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-5},
            "token_side": {"dim": 256}, "loop": {"start": 1, "stop": 3, "times": 2}, "layers": layers}, delta, latent


def _time(fn, warmup, steps):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run(args, peaks):
    from . import seqops as ops
    from .build import build_seq
    build_seq()
    from .scheduler import Scheduler
    from .vofelix import VofelixConfig, VofelixModel
    dev = torch.device("cuda", 0)
    tokens = args.tokens or 4096
    raw, delta, latent = bench_config()
    cfg = VofelixConfig.from_dict(raw)
    model = VofelixModel.random(cfg, seed=0, dtype=torch.bfloat16, device=0)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (tokens,), generator=g).tolist()
    out = {"metric": "vofelix_prefill_tokens_per_s", "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
           "higher_is_better": True, "dtype": "bf16", "data": "synthetic (random weights and token ids)", "vs_baseline": None,
           "config": {"model": "vofelix width 2048: 4 layers (3 delta 32/16 heads x 128, 1 latent 16 heads 128+64 / rank 512, window 1024), "
                               "span 1..3 run twice = 6 layer runs, ff 8192, side 256", "prompt_tokens": tokens,
                      "l2": "weights of one step (about 0.4 GB) exceed L2"}}

    # ---- prefill: the whole prompt in one step, then in portions of 512
    launches0 = ops.total_launches()

    def prefill(portion):
        s = Scheduler(model, max_tokens=tokens + 64, max_requests=4)
        at = 0
        while at < tokens:
            n = min(portion, tokens - at)
            lg = s.step([("p", prompt[at:at + n], [n - 1] if at + n == tokens else [])])
            at += n
        s.finish("p")
        return lg
    ms = _time(lambda: prefill(tokens), args.warmup, args.steps)
    out.update(value=round(tokens / ms * 1e3, 1), ms_per_step=round(ms, 3))
    ms_p = _time(lambda: prefill(512), 1, max(1, args.steps // 2))
    out["prefill_portions_512"] = {"tokens_per_s": round(tokens / ms_p * 1e3, 1), "ms": round(ms_p, 3)}

    # ---- decode: 4 live requests with `ctx` tokens each, one token per request per step
    ctx = 2048
    s = Scheduler(model, max_tokens=4 * (ctx + 256), max_requests=4, cuda_graphs=not getattr(args, 'no_graph', False))
    for r in range(4):
        s.step([(r, prompt[:ctx], [])])
    nxt = [[1], [2], [3], [4]]
    ms_d = _time(lambda: s.step([(r, nxt[r], [0]) for r in range(4)]), args.warmup, 16)
    out["decode"] = {"live_requests": 4, "context": ctx, "tokens_per_s": round(4 / ms_d * 1e3, 1), "ms_per_step": round(ms_d, 3),
                     "cuda_graph": bool(s.cuda_graphs and any(v not in (None, False) for v in s._graphs.values()))}
    out["gpu_launches"] = ops.total_launches() - launches0

    # ---- end to end through the generation entry point: pinned host tables in, sampled ids out every step
    s = Scheduler(model, max_tokens=tokens + 256, max_requests=4)
    s.generate([prompt], max_new_tokens=8, step_tokens=tokens)                 # warm-up of the same call
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    h2d0, steps0 = s.h2d_bytes, s.steps_run
    t0.record()
    s.generate([prompt], max_new_tokens=8, step_tokens=tokens)
    t1.record()
    torch.cuda.synchronize()
    out["e2e"] = {"value": round((tokens + 8) / t0.elapsed_time(t1) * 1e3, 1), "unit": "tokens/s (prompt + 8 generated, Scheduler.generate)",
                  "h2d_bytes_per_step": (s.h2d_bytes - h2d0) // max(s.steps_run - steps0, 1), "d2h_bytes_per_step": 8}

    # ---- per-mixer times beside the closest blocks of the MoE prefill models at equal size
    mix = {}
    W = cfg.width
    h = (torch.randn(tokens, W, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    tb = ops.StepTables([(prompt, 0, 0, list(range((tokens + 63) // 64)))], dev)
    model.make_caches(tokens + 64, 4)
    dl = model.layers[0]["mixer"]
    tail, state = model._run_state[0]
    mix["delta_mixer_ms"] = round(_time(lambda: dl.forward(h, tb, tail, state), 2, 5), 3)
    la = model.layers[2]["mixer"]
    ckv, kr = model.kv_cache.get_layer_caches(0)
    mix["latent_attention_window_1024_ms"] = round(_time(lambda: la.forward(h, tb, ckv, kr, 64), 1, 3), 3)
    try:
        from types import SimpleNamespace
        from .build import build
        build()
        from .attention import GatedDeltaNetAttention, MLAAttention, MLAPagedKVCache, SequenceKVState
        from .model import SyntheticWeights, HybridMoEConfig
        hc = HybridMoEConfig(hidden_size=W, linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128,
                             linear_value_head_dim=128, linear_conv_kernel_dim=4, num_attention_heads=16, kv_lora_rank=512,
                             qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, rope_theta=10000.0, rms_norm_eps=1e-5)
        src = SyntheticWeights(hc, dev, 0)
        ac = SimpleNamespace(**{f: getattr(hc, f) for f in hc.__dataclass_fields__})
        gdn = GatedDeltaNetAttention(ac, 0, src.attention(0, "linear_attention"), dev, max_tokens=tokens)

        def gdn_step():
            gdn.reset_state()
            gdn.forward(h)
        mix["gated_deltanet_block_ms"] = round(_time(gdn_step, 2, 5), 3)
        mla = MLAAttention(ac, 0, src.attention(0, "mla"), dev, max_tokens=tokens, max_kv_len=tokens)
        kv = MLAPagedKVCache(1, 512, 64, dev, max_pages=tokens // 16 + 2)
        pos = torch.arange(tokens, dtype=torch.int32, device=dev)

        def mla_step():
            st = SequenceKVState(kv)
            mla.forward(h, pos, kv, st, 0, num_new_tokens=tokens)
            st.free()
        mix["mla_block_full_causal_ms"] = round(_time(mla_step, 2, 5), 3)
    except Exception as exc:       # noqa: BLE001 — the comparison is optional; the new design's numbers stand without it
        mix["comparison_unavailable"] = f"{type(exc).__name__}: {exc}"
    out["mixers_at_equal_size"] = mix
    out["peaks"] = peaks
    print(json.dumps(out))


# ------------------------------------------------------------------------------------------------ Megolorn
def megolorn_config(width=2048, chunk=2048, vocab=32768, experts=62, identity=2, top=6, expert_ff=1024):
    """16 query heads x 2 maps x 128 over 2 key/value heads with 256-wide values: the score and value products of the GQA block of
    Qwen3-Next (16 heads x 256 over 2 key/value heads) with the value product doubled.  Every other layer reads the previous layer's
    keys and values and carries routed experts (64 router outputs in 8 groups, 4 kept, top 6) with a shared expert."""
    att = {"heads": 16, "kv_heads": 2, "dim": 128, "vdim": 256, "diff": 0.5, "scale": 128 ** -0.5, "mask": {"size": chunk},
           "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 4.0}}}
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": 2 * expert_ff},
           "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": 8, "keep": 4}}}
    dense = {"kind": "dense", "ff": 4 * width, "limit": 7.0}
    layers = []
    for i in range(2):
        layers.append({"type": "attention", "mixer": dict(att), "mlp": dense})
        layers.append({"type": "attention", "mixer": dict(att, kv_from=2 * i), "mlp": moe})
    return {"architecture": "Megolorn", "vocab": vocab, "width": width, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-5}, "layers": layers}


def run_megolorn(args, peaks):
    from . import seqops as ops
    from .build import build, build_seq
    build_seq()
    build()                                          # the tcgen05 GEMM and attention core serve long bfloat16 steps
    from .megolorn import MegolornConfig, MegolornModel
    from .scheduler import Scheduler
    dev = torch.device("cuda", 0)
    tokens = args.tokens or 4096
    raw = megolorn_config()
    cfg = MegolornConfig.from_dict(raw)
    model = MegolornModel.random(cfg, seed=0, dtype=torch.bfloat16, device=0)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (tokens,), generator=g).tolist()
    out = {"metric": "megolorn_prefill_tokens_per_s", "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
           "higher_is_better": True, "dtype": "bf16", "data": "synthetic (random weights and token ids)", "vs_baseline": None,
           "config": {"model": "megolorn width 2048: 4 layers, differential attention 16 heads x 2 maps x 128 / 2 kv heads / values 256, "
                               "chunk 2048; layers 1 and 3 read the keys and values of layers 0 and 2; dense ff 8192 / 62 experts + 2 identity, "
                               "top 6, expert ff 1024, shared ff 2048", "prompt_tokens": tokens,
                      "l2": "weights of one step (about 1.8 GB) exceed L2"}}
    launches0 = ops.total_launches()

    def prefill(portion):
        s = Scheduler(model, max_tokens=tokens + 64, max_requests=4)
        at = 0
        while at < tokens:
            n = min(portion, tokens - at)
            lg = s.step([("p", prompt[at:at + n], [n - 1] if at + n == tokens else [])])
            at += n
        s.finish("p")
        return lg
    ms = _time(lambda: prefill(tokens), args.warmup, args.steps)
    out.update(value=round(tokens / ms * 1e3, 1), ms_per_step=round(ms, 3))
    ms_p = _time(lambda: prefill(512), 1, max(1, args.steps // 2))
    out["prefill_portions_512"] = {"tokens_per_s": round(tokens / ms_p * 1e3, 1), "ms": round(ms_p, 3)}

    ctx = 2048
    s = Scheduler(model, max_tokens=4 * (ctx + 256), max_requests=4, cuda_graphs=not getattr(args, 'no_graph', False))
    for r in range(4):
        s.step([(r, prompt[:ctx], [])])
    nxt = [[1], [2], [3], [4]]
    ms_d = _time(lambda: s.step([(r, nxt[r], [0]) for r in range(4)]), args.warmup, 16)
    out["decode"] = {"live_requests": 4, "context": ctx, "tokens_per_s": round(4 / ms_d * 1e3, 1), "ms_per_step": round(ms_d, 3),
                     "cuda_graph": bool(s.cuda_graphs and any(v not in (None, False) for v in s._graphs.values()))}
    out["gpu_launches"] = ops.total_launches() - launches0

    s = Scheduler(model, max_tokens=tokens + 256, max_requests=4)
    s.generate([prompt], max_new_tokens=8, step_tokens=tokens)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    h2d0, steps0 = s.h2d_bytes, s.steps_run
    t0.record()
    s.generate([prompt], max_new_tokens=8, step_tokens=tokens)
    t1.record()
    torch.cuda.synchronize()
    out["e2e"] = {"value": round((tokens + 8) / t0.elapsed_time(t1) * 1e3, 1), "unit": "tokens/s (prompt + 8 generated, Scheduler.generate)",
                  "h2d_bytes_per_step": (s.h2d_bytes - h2d0) // max(s.steps_run - steps0, 1), "d2h_bytes_per_step": 8}

    # ---- per-block times, prefill and decode, beside the closest blocks at equal size
    blk = {}
    W = cfg.width
    h = (torch.randn(tokens, W, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    tb = ops.StepTables([(prompt, 0, 0, list(range((tokens + 63) // 64)))], dev)
    model.make_caches(tokens + 64, 4)
    att = model.layers[0]["mixer"]
    kc, vc = model.kv_cache.get_layer_caches(0)
    blk["differential_attention_block_ms"] = round(_time(lambda: att.forward(h, tb, kc, vc, 64), 2, 5), 3)
    att.tc_min_portion = 1 << 30
    hs = h[:512].contiguous()
    tbs = ops.StepTables([(prompt[:512], 0, 0, list(range(8)))], dev)
    blk["differential_attention_block_plain_kernel_512_tokens_ms"] = round(_time(lambda: att.forward(hs, tbs, kc, vc, 64), 1, 3), 3)
    att.tc_min_portion = 128
    blk["dense_ff_8192_ms"] = round(_time(lambda: model.layers[0]["mlp"].forward(h), 2, 5), 3)
    moe = model.layers[1]["mlp"]
    blk["routed_experts_block_ms"] = round(_time(lambda: moe.forward(h), 2, 5), 3)
    h4 = h[:4].contiguous()
    tb4 = ops.StepTables([([1], ctx, r, list(range(r * 40, r * 40 + 33))) for r in range(4)], dev)
    blk["decode_4_tokens_attention_ms"] = round(_time(lambda: att.forward(h4, tb4, kc, vc, 64), 3, 20), 4)
    blk["decode_4_tokens_routed_experts_ms"] = round(_time(lambda: moe.forward(h4), 3, 20), 4)
    blk["decode_4_tokens_dense_ff_ms"] = round(_time(lambda: model.layers[0]["mlp"].forward(h4), 3, 20), 4)
    try:
        from types import SimpleNamespace
        from .attention import GQAAttention, PagedKVCache, SequenceKVState
        from .model import HybridMoEConfig, SyntheticWeights
        hc = HybridMoEConfig(hidden_size=W, num_attention_heads=16, num_key_value_heads=2, gqa_head_dim=256, rope_theta=1000000.0,
                             rms_norm_eps=1e-6)
        src = SyntheticWeights(hc, dev, 0)
        ac = SimpleNamespace(**{f: getattr(hc, f) for f in hc.__dataclass_fields__}, rotary_dim=hc.rotary_dim)
        gqa = GQAAttention(ac, 0, src.attention(0, "full_attention"), dev, max_tokens=tokens)
        kv = PagedKVCache.from_config(ac, 1, dev, max_pages=tokens // 16 + 2)
        pos = torch.arange(tokens, dtype=torch.int32, device=dev)

        def gqa_step():
            st = SequenceKVState(kv)
            gqa.forward(h, pos, kv, st, 0, num_new_tokens=tokens)
            st.free()
        blk["gqa_block_16x256_full_causal_ms"] = round(_time(gqa_step, 2, 5), 3)
    except Exception as exc:       # noqa: BLE001 — the comparison is optional; the new design's numbers stand without it
        blk["comparison_unavailable"] = f"{type(exc).__name__}: {exc}"
    out["blocks_at_equal_size"] = blk
    out["peaks"] = peaks
    print(json.dumps(out))


# ------------------------------------------------------------------------------------------------ Gurozen
def gurozen_config(width=2048, vocab=32768, experts=64, top=6, expert_ff=1024):
    """Attention 16 heads x 128 over 2 key/value heads (the score product of Qwen3-Next's GQA block at half the value width), the
    channel-decay delta rule at Qwen3-Next's linear-attention geometry (32 / 16 heads x 128), 64 squared-relu experts in 8 groups
    (4 kept, top 6) with a gated shared expert; layers 1 and 2 run twice."""
    att = {"heads": 16, "kv_heads": 2, "dim": 128, "vdim": 128, "conv": 4, "scale": 128 ** -0.5, "softcap": 50.0,
           "rot": {"base": 1000000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 8.0, "original": 8192}}}
    delta = {"heads": 32, "kv_heads": 16, "dim": 128, "vdim": 128, "conv": 4}
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": 2 * expert_ff},
           "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": 8, "keep": 4}}}
    dense = {"kind": "dense", "ff": 4 * width}
    layers = [{"type": "attention", "mixer": att, "mlp": dense}, {"type": "channel_delta", "mixer": delta, "mlp": moe},
              {"type": "attention", "mixer": att, "mlp": moe}, {"type": "channel_delta", "mixer": delta, "mlp": dense}]
    return {"architecture": "Gurozen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.7, "logit_scale": 0.25,
            "loop": {"start": 1, "stop": 3, "times": 2}, "layers": layers}


def run_gurozen(args, peaks):
    from . import seqops as ops
    from .build import build, build_seq
    build_seq()
    build()                                          # the tcgen05 GEMM and attention core serve long bfloat16 steps
    from .gurozen import GurozenConfig, GurozenModel
    from .scheduler import Scheduler
    dev = torch.device("cuda", 0)
    tokens = args.tokens or 4096
    raw = gurozen_config()
    cfg = GurozenConfig.from_dict(raw)
    model = GurozenModel.random(cfg, seed=0, dtype=torch.bfloat16, device=0)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (tokens,), generator=g).tolist()
    out = {"metric": "gurozen_prefill_tokens_per_s", "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
           "higher_is_better": True, "dtype": "bf16", "data": "synthetic (random weights and token ids)", "vs_baseline": None,
           "config": {"model": "gurozen width 2048: 4 layers (attention 16 heads x 128 / 2 kv heads, conv 4, cap 50; channel-decay delta rule "
                               "32 / 16 heads x 128, conv 4), layers 1..2 run twice = 6 layer runs; dense ff 8192 / 64 squared-relu experts in 8 "
                               "groups, top 6, expert ff 1024, gated shared ff 2048", "prompt_tokens": tokens,
                      "l2": "weights of one step (about 1.3 GB) exceed L2"}}
    launches0 = ops.total_launches()

    def prefill(portion):
        s = Scheduler(model, max_tokens=tokens + 64, max_requests=4)
        at = 0
        while at < tokens:
            n = min(portion, tokens - at)
            lg = s.step([("p", prompt[at:at + n], [n - 1] if at + n == tokens else [])])
            at += n
        s.finish("p")
        return lg
    ms = _time(lambda: prefill(tokens), args.warmup, args.steps)
    out.update(value=round(tokens / ms * 1e3, 1), ms_per_step=round(ms, 3))
    ms_p = _time(lambda: prefill(512), 1, max(1, args.steps // 2))
    out["prefill_portions_512"] = {"tokens_per_s": round(tokens / ms_p * 1e3, 1), "ms": round(ms_p, 3)}

    ctx = 2048
    s = Scheduler(model, max_tokens=4 * (ctx + 256), max_requests=4, cuda_graphs=not getattr(args, 'no_graph', False))
    for r in range(4):
        s.step([(r, prompt[:ctx], [])])
    nxt = [[1], [2], [3], [4]]
    ms_d = _time(lambda: s.step([(r, nxt[r], [0]) for r in range(4)]), args.warmup, 16)
    out["decode"] = {"live_requests": 4, "context": ctx, "tokens_per_s": round(4 / ms_d * 1e3, 1), "ms_per_step": round(ms_d, 3),
                     "cuda_graph": bool(s.cuda_graphs and any(v not in (None, False) for v in s._graphs.values()))}
    out["gpu_launches"] = ops.total_launches() - launches0

    s = Scheduler(model, max_tokens=tokens + 256, max_requests=4)
    s.generate([prompt], max_new_tokens=8, step_tokens=tokens)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    h2d0, steps0 = s.h2d_bytes, s.steps_run
    t0.record()
    s.generate([prompt], max_new_tokens=8, step_tokens=tokens)
    t1.record()
    torch.cuda.synchronize()
    out["e2e"] = {"value": round((tokens + 8) / t0.elapsed_time(t1) * 1e3, 1), "unit": "tokens/s (prompt + 8 generated, Scheduler.generate)",
                  "h2d_bytes_per_step": (s.h2d_bytes - h2d0) // max(s.steps_run - steps0, 1), "d2h_bytes_per_step": 8}

    # ---- per-block times, prefill and decode, beside the closest blocks of the other designs at equal size
    blk = {}
    W = cfg.width
    h = (torch.randn(tokens, W, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    pages = list(range((tokens + 63) // 64))
    tb = ops.StepTables([(prompt, 0, 0, pages)], dev)
    model.make_caches(tokens + 64, 4)
    att, dl = model.layers[0]["mixer"], model.layers[1]["mixer"]
    kc, vc = model.kv_cache.get_layer_caches(0)
    blk["attention_block_ms"] = round(_time(lambda: att.forward(h, tb, kc, vc, 64, tail=model._run_state[0]), 2, 5), 3)
    tail, state = model._run_state[1]
    blk["channel_delta_mixer_ms"] = round(_time(lambda: dl.forward(h, tb, tail, state), 2, 5), 3)
    blk["dense_ff_8192_ms"] = round(_time(lambda: model.layers[0]["mlp"].forward(h), 2, 5), 3)
    moe = model.layers[1]["mlp"]
    blk["routed_experts_block_ms"] = round(_time(lambda: moe.forward(h), 2, 5), 3)
    h4 = h[:4].contiguous()
    tb4 = ops.StepTables([([1], ctx, r, list(range(r * 40, r * 40 + 33))) for r in range(4)], dev)
    blk["decode_4_tokens_attention_ms"] = round(_time(lambda: att.forward(h4, tb4, kc, vc, 64, tail=model._run_state[0]), 3, 20), 4)
    blk["decode_4_tokens_channel_delta_ms"] = round(_time(lambda: dl.forward(h4, tb4, tail, state), 3, 20), 4)
    blk["decode_4_tokens_routed_experts_ms"] = round(_time(lambda: moe.forward(h4), 3, 20), 4)
    try:                                             # the closest blocks: Megolorn's attention and experts, Vofelix's delta mixer
        from .attention import HeadKVCache, RecurrentStatePool
        from .megolorn import MegolornConfig, MegolornModel
        from .vofelix import VofelixConfig, VofelixModel
        mraw = megolorn_config(experts=64, identity=0)
        mraw["layers"] = mraw["layers"][:2]
        mraw["layers"][0]["mixer"]["vdim"] = mraw["layers"][1]["mixer"]["vdim"] = 128
        mm = MegolornModel.random(MegolornConfig.from_dict(mraw), seed=0, dtype=torch.bfloat16, device=0)
        matt, mmoe = mm.layers[0]["mixer"], mm.layers[1]["mlp"]
        mkv = HeadKVCache([matt.cache_dims()], dev, max_pages=len(pages) + 1, dtype=torch.bfloat16, page_size=64)
        mk, mv = mkv.get_layer_caches(0)
        blk["megolorn_attention_block_2_maps_ms"] = round(_time(lambda: matt.forward(h, tb, mk, mv, 64), 2, 5), 3)
        blk["megolorn_routed_experts_block_ms"] = round(_time(lambda: mmoe.forward(h), 2, 5), 3)
        blk["megolorn_decode_4_tokens_routed_experts_ms"] = round(_time(lambda: mmoe.forward(h4), 3, 20), 4)
        vraw, _, _ = bench_config()
        vraw["layers"] = vraw["layers"][:1]
        vraw["loop"] = {"start": 0, "stop": 0, "times": 1}
        vm = VofelixModel.random(VofelixConfig.from_dict(vraw), seed=0, dtype=torch.bfloat16, device=0)
        vd = vm.layers[0]["mixer"]
        vt, vs = vd.register_state(RecurrentStatePool(4, dev))
        blk["vofelix_delta_mixer_ms"] = round(_time(lambda: vd.forward(h, tb, vt, vs), 2, 5), 3)
        blk["vofelix_decode_4_tokens_delta_ms"] = round(_time(lambda: vd.forward(h4, tb4, vt, vs), 3, 20), 4)
    except Exception as exc:       # noqa: BLE001 — the comparison is optional; the new design's numbers stand without it
        blk["comparison_unavailable"] = f"{type(exc).__name__}: {exc}"
    out["blocks_at_equal_size"] = blk
    out["peaks"] = peaks
    print(json.dumps(out))


def zaronex_config(width=2048, vocab=32768, window=1024):
    """Latent attention at DeepSeek-V2-Lite's MLA geometry with a query latent of 1536; grouped-query attention 16 heads x 128 over 2
    key/value heads (Gurozen's benchmark geometry) with a window of 1024, pooled blocks of 64 and sinks; gated linear attention with the
    state size of Qwen3-Next's linear-attention block (32 heads, 128 x 128); selective scan with an inner width of twice the model's,
    16 states per channel."""
    latent = {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "q_rank": 1536, "scale": 192 ** -0.5,
              "mask": {"size": window}, "rot": {"base": 10000.0, "dims": 64}}
    left1 = {"heads": 16, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": window, "pool": 64},
             "rot": {"base": 1000000.0, "dims": 64}}
    left2 = {"heads": 16, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": window},
             "rot": {"base": 1000000.0, "dims": 64, "scaling": {"factor": 8.0}}}
    gla = {"heads": 32, "dim": 128, "vdim": 128, "tau": 16.0}
    scan = {"inner": 2 * width, "state": 16, "dt_rank": 128, "conv": 4}
    dense = {"kind": "dense", "ff": 4 * width}
    layers = [{"type": "latent_attention", "mixer": latent, "mlp": dense},
              {"type": "parallel", "mixer": {"left": left1, "right": gla}, "mlp": dense},
              {"type": "parallel_2", "mixer": {"left": left2, "right": scan}, "mlp": dense},
              {"type": "parallel", "mixer": {"left": left1, "right": gla}, "mlp": None}]
    return {"architecture": "Zaronex", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": layers}


def run_zaronex(args, peaks):
    from . import seqops as ops
    from .build import build, build_seq
    build_seq()
    build()                                          # the tcgen05 GEMM and attention core serve long bfloat16 steps
    from .attention import RecurrentStatePool
    from .scheduler import Scheduler
    from .zaronex import ZaronexConfig, ZaronexModel
    dev = torch.device("cuda", 0)
    tokens = args.tokens or 4096
    raw = zaronex_config()
    cfg = ZaronexConfig.from_dict(raw)
    model = ZaronexModel.random(cfg, seed=0, dtype=torch.bfloat16, device=0)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (tokens,), generator=g).tolist()
    out = {"metric": "zaronex_prefill_tokens_per_s", "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
           "higher_is_better": True, "dtype": "bf16", "data": "synthetic (random weights and token ids)", "vs_baseline": None,
           "config": {"model": "zaronex width 2048: 4 layers (latent attention 16 heads 128+64 / rank 512, query rank 1536, window 1024; "
                               "parallel: attention 16 heads x 128 / 2 kv heads, window 1024, pooled blocks of 64, sinks, beside gated linear "
                               "attention 32 heads 128 x 128; parallel_2: attention with rotated values beside a selective scan of 4096 "
                               "channels x 16 states), depth-averaged stream, dense ff 8192", "prompt_tokens": tokens,
                      "l2": "weights of one step (about 0.6 GB) exceed L2"}}
    launches0 = ops.total_launches()

    def prefill(portion):
        s = Scheduler(model, max_tokens=tokens + 64, max_requests=4)
        at = 0
        while at < tokens:
            n = min(portion, tokens - at)
            lg = s.step([("p", prompt[at:at + n], [n - 1] if at + n == tokens else [])])
            at += n
        s.finish("p")
        return lg
    ms = _time(lambda: prefill(tokens), args.warmup, args.steps)
    out.update(value=round(tokens / ms * 1e3, 1), ms_per_step=round(ms, 3))
    ms_p = _time(lambda: prefill(512), 1, max(1, args.steps // 2))
    out["prefill_portions_512"] = {"tokens_per_s": round(tokens / ms_p * 1e3, 1), "ms": round(ms_p, 3)}

    ctx = 2048
    s = Scheduler(model, max_tokens=4 * (ctx + 256), max_requests=4, cuda_graphs=not getattr(args, 'no_graph', False))
    for r in range(4):
        s.step([(r, prompt[:ctx], [])])
    nxt = [[1], [2], [3], [4]]
    ms_d = _time(lambda: s.step([(r, nxt[r], [0]) for r in range(4)]), args.warmup, 16)
    out["decode"] = {"live_requests": 4, "context": ctx, "tokens_per_s": round(4 / ms_d * 1e3, 1), "ms_per_step": round(ms_d, 3),
                     "cuda_graph": bool(s.cuda_graphs and any(v not in (None, False) for v in s._graphs.values()))}
    out["gpu_launches"] = ops.total_launches() - launches0

    s = Scheduler(model, max_tokens=tokens + 256, max_requests=4)
    s.generate([prompt], max_new_tokens=8, step_tokens=tokens)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    h2d0, steps0 = s.h2d_bytes, s.steps_run
    t0.record()
    s.generate([prompt], max_new_tokens=8, step_tokens=tokens)
    t1.record()
    torch.cuda.synchronize()
    out["e2e"] = {"value": round((tokens + 8) / t0.elapsed_time(t1) * 1e3, 1), "unit": "tokens/s (prompt + 8 generated, Scheduler.generate)",
                  "h2d_bytes_per_step": (s.h2d_bytes - h2d0) // max(s.steps_run - steps0, 1), "d2h_bytes_per_step": 8}

    # ---- per-block times, prefill and decode, beside the closest blocks of the other designs at equal size
    blk = {}
    W = cfg.width
    h = (torch.randn(tokens, W, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    pages = list(range((tokens + 63) // 64))
    tb = ops.StepTables([(prompt, 0, 0, pages)], dev)
    model.make_caches(max(tokens, 4 * 40 * 64) + 64, 4)
    kvc = model.kv_cache
    lat, par, par2 = model.layers[0]["mixer"], model.layers[1]["mixer"], model.layers[2]["mixer"]
    h4 = h[:4].contiguous()
    tb4 = ops.StepTables([([1], ctx, r, list(range(r * 40, r * 40 + 33))) for r in range(4)], dev)

    def both(name, fn_of):                           # fn_of(h, tables) -> callable
        blk[name + "_ms"] = round(_time(fn_of(h, tb), 2, 5), 3)
        blk["decode_4_tokens_" + name + "_ms"] = round(_time(fn_of(h4, tb4), 3, 20), 4)
    both("latent_attention_block", lambda hh, t: (lambda: lat.forward(hh, t, *kvc.get_layer_caches(0), 64)))
    both("pooled_sink_attention_block", lambda hh, t: (lambda: par.left.forward(hh, t, *kvc.get_layer_caches(1), 64, pooled=kvc.get_pooled_caches(1))))
    both("gated_linear_attention_mixer", lambda hh, t: (lambda: par.right.forward(hh, t, model._state[1])))
    both("rotated_value_attention_block", lambda hh, t: (lambda: par2.left.forward(hh, t, *kvc.get_layer_caches(2), 64)))
    both("selective_scan_mixer", lambda hh, t: (lambda: par2.right.forward(hh, t, *model._state[2])))
    blk["dense_ff_8192_ms"] = round(_time(lambda: model.layers[0]["mlp"].forward(h), 2, 5), 3)

    # ---- the new kernels alone: time, algorithmic bytes and flops, fraction of the measured copy bandwidth / of the fp32 FMA rate
    kern = {}
    fma_tflops = 148 * 128 * 2 * 1.965e9 / 1e12      # fp32 FMA lanes x 2 flops x max SM clock: the ceiling of a recurrence on CUDA cores
    cs = torch.cuda.current_stream(dev).cuda_stream
    lib = ops.load()

    def kernel(name, fn, nbytes, flops=0.0, reps=(2, 8)):
        ms_k = _time(fn, *reps)
        e = {"ms": round(ms_k, 4), "GB_per_s": round(nbytes / ms_k / 1e6, 1), "of_measured_hbm": round(nbytes / ms_k / 1e6 / peaks["hbm_gbs"], 3)}
        if flops:
            e.update(TFLOP_per_s=round(flops / ms_k / 1e9, 2), of_fp32_fma_ceiling=round(flops / ms_k / 1e9 / fma_tflops, 3))
        kern[name] = e
    for label, T_, tbl in (("prefill_4096", tokens, tb), ("decode_4", 4, tb4)):
        S_ = tbl.S
        H, dk, dv = par.right.H, par.right.dk, par.right.dv
        proj = torch.randn(T_, par.right.w_in.shape[0], device=dev) * 0.3
        dec = torch.randn(T_, H * dk, device=dev)
        o = torch.empty(T_, H * dv, device=dev)
        gsc = torch.empty(T_, H * dk, device=dev)
        st = model._state[1]
        state_bytes = 2 * S_ * H * dk * dv * 4
        kernel(f"gla_scan_{label}", lambda: ops.check(lib.kb2_seq_gla(proj.data_ptr(), proj.stride(0), 0, H * dk, 2 * H * dk, dec.data_ptr(), H * dk,
                                                                         par.right.a2_b.data_ptr(), 16.0, dk ** -0.5, T_, S_, H, dk, dv, st.data_ptr(),
                                                                         tbl.cu.data_ptr(), tbl.slots.data_ptr(), gsc.data_ptr(), o.data_ptr(), cs)),
               T_ * (3 * H * dk + 2 * H * dv) * 4 + state_bytes, flops=4.0 * T_ * H * dk * dv)
        C, N, R = par2.right.C, par2.right.N, par2.right.R
        xc, dtin, zz = torch.randn(T_, C, device=dev), torch.randn(T_, C, device=dev), torch.randn(T_, 2 * C, device=dev)
        xp = torch.randn(T_, R + 2 * N, device=dev)
        y = torch.empty(T_, C, dtype=torch.bfloat16, device=dev)
        tl, sst = model._state[2]
        kernel(f"selective_scan_{label}", lambda: ops.check(lib.kb2_seq_selective_scan(xc.data_ptr(), C, dtin.data_ptr(), C, par2.right.dt_b.data_ptr(),
                                                                                        xp.data_ptr(), R + 2 * N, R, zz.data_ptr(), 2 * C, C,
                                                                                        par2.right.A_log.data_ptr(), par2.right.D.data_ptr(), T_, S_, C,
                                                                                        N, sst.data_ptr(), tbl.cu.data_ptr(), tbl.slots.data_ptr(),
                                                                                        y.data_ptr(), 1, cs)),
               T_ * (3 * C * 4 + C * 2 + 2 * N * 4) + 2 * S_ * C * N * 4 + C * N * 4, flops=6.0 * T_ * C * N)
        nst = len(model.layers) + 1
        stack = torch.randn(nst, T_, W, device=dev)
        x, yv = torch.randn(T_, W, device=dev), torch.randn(T_, W, device=dev)
        hb = torch.empty(T_, W, dtype=torch.bfloat16, device=dev)
        coef = model.layers[-1]["dwa"]
        kernel(f"depth_mix_{nst}_results_{label}", lambda: ops.check(lib.kb2_seq_depth_mix(stack.data_ptr(), stack.stride(0), nst, coef.data_ptr(), x.data_ptr(),
                                                                                            yv.data_ptr(), model.final_norm.data_ptr(), hb.data_ptr(), 1,
                                                                                            T_, W, 1e-6, cs)),
               T_ * W * (4 * (nst - 1) + 4 + 4 + 4 + 4 + 2))
        a_, b_ = torch.randn(T_, W, device=dev), torch.randn(T_, W, device=dev)
        kernel(f"branch_merge_{label}", lambda: ops.branch_merge(a_, b_, par.w_left, par.w_right, 1e-6), T_ * W * 12)
        kernel(f"residual_scale_rms_{label} (like kernel of the other designs)",
               lambda: ops.residual_scale_rms(x, yv, 1.0, norm=model.final_norm, out_dtype=torch.bfloat16, eps=1e-6), T_ * W * 14)
    try:                                             # the closest blocks: Gurozen's attention and channel-decay delta rule, Vofelix's latent attention
        from .attention import HeadKVCache
        from .gurozen import GurozenConfig, GurozenModel
        from .vofelix import VofelixConfig, VofelixModel
        graw = gurozen_config()
        graw["layers"] = [graw["layers"][0], dict(graw["layers"][1], mlp=None)]
        graw["loop"] = {"start": 0, "stop": 0, "times": 0}
        gm = GurozenModel.random(GurozenConfig.from_dict(graw), seed=0, dtype=torch.bfloat16, device=0)
        gm.make_caches(max(tokens, 4 * 40 * 64) + 64, 4)
        gatt, gdl = gm.layers[0]["mixer"], gm.layers[1]["mixer"]
        gk, gv = gm.kv_cache.get_layer_caches(0)
        gtail, gstate = gm._run_state[1]
        blk["gurozen_attention_block_ms"] = round(_time(lambda: gatt.forward(h, tb, gk, gv, 64, tail=gm._run_state[0]), 2, 5), 3)
        blk["gurozen_decode_4_tokens_attention_ms"] = round(_time(lambda: gatt.forward(h4, tb4, gk, gv, 64, tail=gm._run_state[0]), 3, 20), 4)
        blk["gurozen_channel_delta_mixer_ms"] = round(_time(lambda: gdl.forward(h, tb, gtail, gstate), 2, 5), 3)
        blk["gurozen_decode_4_tokens_channel_delta_ms"] = round(_time(lambda: gdl.forward(h4, tb4, gtail, gstate), 3, 20), 4)
        for label, T_, tbl in (("prefill_4096", tokens, tb), ("decode_4", 4, tb4)):      # the like kernel of the recurrences, alone
            H, Hk, dk, dv = gdl.H, gdl.Hk, gdl.dk, gdl.dv
            conv = torch.randn(T_, gdl.C, device=dev) * 0.3
            beta, dec, gate = torch.randn(T_, H, device=dev), torch.randn(T_, H * dk, device=dev), torch.randn(T_, H * dv, device=dev)
            scratch = torch.empty(2 * T_ * Hk * dk + T_ * H + T_ * H * dk + T_ * H * dv + 16, device=dev)
            od = torch.empty(T_, H * dv, dtype=torch.bfloat16, device=dev)
            kernel(f"delta_rule_ch_{label} (like kernel: Gurozen)",
                   lambda: ops.check(lib.kb2_seq_delta_rule_ch(conv.data_ptr(), gdl.C, beta.data_ptr(), H, dec.data_ptr(), H * dk, gate.data_ptr(), H * dv, 1,
                                                               T_, tbl.S, H, Hk, dk, dv, gdl.A_log.data_ptr(), gdl.dt_bias.data_ptr(), gdl.norm.data_ptr(),
                                                               1e-6, gstate.data_ptr(), tbl.cu.data_ptr(), tbl.slots.data_ptr(), scratch.data_ptr(),
                                                               od.data_ptr(), 1, cs)),
                   T_ * (gdl.C + H + H * dk + H * dv) * 4 + T_ * H * dv * 2 + 2 * tbl.S * H * dk * dv * 4, flops=8.0 * T_ * H * dk * dv)
        vraw, _, vlat = bench_config()
        vraw["layers"] = [_layer("latent_attention", vlat)]
        vraw["loop"] = {"start": 0, "stop": 0, "times": 1}
        vm = VofelixModel.random(VofelixConfig.from_dict(vraw), seed=0, dtype=torch.bfloat16, device=0)
        vl = vm.layers[0]["mixer"]
        vkv = HeadKVCache([vl.cache_dims()], dev, max_pages=max(len(pages), 4 * 40) + 1, dtype=torch.bfloat16, page_size=64)
        vc_, vk_ = vkv.get_layer_caches(0)
        blk["vofelix_latent_attention_block_ms"] = round(_time(lambda: vl.forward(h, tb, vc_, vk_, 64), 2, 5), 3)
        blk["vofelix_decode_4_tokens_latent_attention_ms"] = round(_time(lambda: vl.forward(h4, tb4, vc_, vk_, 64), 3, 20), 4)
    except Exception as exc:       # noqa: BLE001 — the comparison is optional; the new design's numbers stand without it
        blk["comparison_unavailable"] = f"{type(exc).__name__}: {exc}"
    out["blocks_at_equal_size"] = blk
    out["kernels"] = kern
    out["peaks"] = peaks
    print(json.dumps(out))
