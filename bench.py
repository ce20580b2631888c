"""Benchmark of the engine on one B200: decode tokens per second at batch 8 (and 1
and 64), prefill of one 2,048-token prompt, at Llama-3.2-1B size with random
weights and uniform random prompt ids.

    python bench.py --gpus 1 --steps K --warmup W      -> one JSON line
    python bench.py --impl reference ...               -> the reference arm (or why it is unavailable)

A "step" is one decode step of the whole batch.  ``value`` is device-timed
(CUDA events around K steps fed from the device); ``e2e`` is the same through
``Engine.step`` with host tokens in and out every step.  Weights (2.5 GB) are
larger than L2, so every step streams them from HBM: no L2 flush is needed.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PROMPT_LEN = 2048
POOL_CONTEXT = 4096
PAGE = 16


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, t0, t1):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            if not (t0 - 0.05 <= t <= t1 + 0.15):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def model_numbers(cfg):
    d, L, H, Hk, hd, I, V = (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads,
                             cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size)
    per_layer = (H * hd + 2 * Hk * hd) * d + d * H * hd + 3 * I * d
    linear_params = L * per_layer
    head_params = V * d
    weight_bytes = 2 * (linear_params + head_params) + 2 * 2 * L * d + 2 * d       # bf16; norms are small
    kv_bytes_per_token = 2 * L * Hk * hd * 2
    return dict(linear_params=linear_params, head_params=head_params, weight_bytes=weight_bytes,
                kv_bytes_per_token=kv_bytes_per_token)


def prefill_flops(cfg, n):
    m = model_numbers(cfg)
    attn = cfg.num_hidden_layers * 4 * cfg.num_attention_heads * cfg.head_dim * (n * (n + 1) // 2)
    return 2 * n * m["linear_params"] + attn + 2 * m["head_params"]


def run_ours(args):
    import numpy as np
    import torch

    from inf_engine_b200 import Engine, Request, SamplingConfig, StepEntry, kernels
    from inf_engine_b200.config import get_preset
    from inf_engine_b200.sampling import pack_rows, request_key
    from inf_engine_b200.weights import write_random_model

    cfg = get_preset(args.model)
    n_layers_full = cfg.num_hidden_layers
    if args.layers:
        import dataclasses
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers)
    pk = peaks()
    torch.cuda.set_device(0)
    t_build = time.perf_counter()
    with tempfile.TemporaryDirectory(prefix="bench_model_") as tmp:
        write_random_model(cfg, args.seed, tmp)
        engine = Engine.from_dir(tmp, dtype="bfloat16", n_total_blocks=args.pool_requests * POOL_CONTEXT // PAGE, block_size=PAGE,
                                 max_requests=max(64, args.pool_requests), max_tokens_per_step=8192, chunk=2048)
    t_build = time.perf_counter() - t_build
    runner = engine.runner
    V = cfg.vocab_size
    rng = np.random.default_rng(args.seed)
    nums = model_numbers(cfg)
    clocks = ClockSampler()
    clocks.start()

    def prompt():
        return rng.integers(0, V, PROMPT_LEN).tolist()

    # ---------------------------------------------------------------- prefill
    def prefill_once():
        runner.open("p")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        toks = prompt()
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepEntry("p", toks, [PROMPT_LEN - 1])])
        e1.record()
        torch.cuda.synchronize()
        runner.close("p")
        return e0.elapsed_time(e1)

    if args.only == "decode":
        pre_ms = [float("nan")]
    else:
        for _ in range(3):
            prefill_once()
        pre_ms = sorted(prefill_once() for _ in range(args.prefill_reps))
    pre = pre_ms[len(pre_ms) // 2]
    prefill = {"value": PROMPT_LEN / pre * 1e3, "unit": "tok/s", "tokens": PROMPT_LEN, "ms": pre,
               "frac": prefill_flops(cfg, PROMPT_LEN) / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12),
               "peak_tflops": pk["bf16_tflops"], "peak_source": pk["source"]}

    # ----------------------------------------------------------------- decode
    greedy = SamplingConfig()

    def decode_device(batch, steps, warmup):
        """Device-timed decode: K steps, each fed the ids the step before sampled, no host read inside."""
        rids = [f"d{batch}_{i}" for i in range(batch)]
        for rid in rids:
            runner.open(rid)
        for i in range(0, batch, 4):                      # prompts, four at a time
            runner.step([StepEntry(r, prompt(), []) for r in rids[i:i + 4]])
        rows = pack_rows([greedy] * batch, [request_key(i, 0) for i in range(batch)], V)
        ids = torch.as_tensor(rng.integers(0, V, batch), dtype=torch.int32).cuda()
        entries = [StepEntry(r, [0], [0]) for r in rids]
        for _ in range(warmup):
            _, ids = runner.step_and_sample(entries, rows, device_tokens=ids)
        gc.collect()          # a full collection of the host's garbage inside the timed steps would stall the launches
        torch.cuda.synchronize()
        ctx0 = runner.length(rids[0])
        n0 = kernels.LAUNCHES
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            _, ids = runner.step_and_sample(entries, rows, device_tokens=ids)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        ms = e0.elapsed_time(e1)
        launches = kernels.LAUNCHES - n0
        for rid in rids:
            runner.close(rid)
        mean_ctx = ctx0 + steps / 2
        bytes_step = nums["weight_bytes"] + batch * mean_ctx * nums["kv_bytes_per_token"]
        return dict(tok_s=batch * steps / ms * 1e3, ms_per_step=ms / steps, launches=launches, t0=t0, t1=t1,
                    bytes_step=bytes_step, ctx=(ctx0, ctx0 + steps))

    def decode_e2e(batch, steps, warmup):
        """Through Engine.step: host tokens in (one pinned copy a step), sampled ids out (one read a step)."""
        reqs = [Request(1000 + i, prompt(), max_new_tokens=warmup + steps + 8) for i in range(batch)]
        for r in reqs:
            assert engine.submit(r), r.error
        while any(len(r.generated) < 1 for r in reqs):
            engine.step()
        for _ in range(warmup):
            engine.step()
        gc.collect()
        torch.cuda.synchronize()
        n_before = sum(len(r.generated) for r in reqs)
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        n_tok = sum(len(r.generated) for r in reqs) - n_before
        while engine.has_work:
            engine.step()
        engine.completed.clear()
        b = next(iter(runner.graphs._buckets.values()))
        key = [k for k in runner.graphs._buckets if k[0] >= batch]
        h2d = min(runner.graphs._buckets[k].n for k in key) * 4 if key else 0
        return dict(tok_s=n_tok / (t1 - t0), h2d=h2d, d2h=4 * batch)

    if args.only == "prefill":
        clocks.stop()
        print(json.dumps({"impl": "ours", "only": "prefill", "prefill": prefill, "config": {"model": args.model, "layers": cfg.num_hidden_layers}}))
        return 0
    main = decode_device(args.batch, args.steps, args.warmup)
    if args.only == "decode":
        clocks.stop()
        print(json.dumps({"impl": "ours", "only": "decode", "value": main["tok_s"], "ms_per_step": main["ms_per_step"],
                          "config": {"model": args.model, "layers": cfg.num_hidden_layers, "global_batch": args.batch}}))
        return 0
    e2e = decode_e2e(args.batch, args.steps, args.warmup)
    points = {}
    for b in (1, 64):
        if b <= args.pool_requests:
            points[f"decode_b{b}"] = decode_device(b, args.steps, args.warmup)["tok_s"]
    clocks.stop()
    clk = clocks.summary(main["t0"], main["t1"])
    # the other two configurations of the baseline: continuous batching at their sizes, wall clock
    workloads = {}
    if not args.no_workloads:
        del engine, runner
        gc.collect()
        torch.cuda.empty_cache()
        for key, model, n_req, lo, hi, new, temps in WORKLOADS:
            for rec in measure_workload(model, n_req, lo, hi, new, temps, args.seed):
                workloads[key + ("" if rec["temperature"] == 0 else f"_t{rec['temperature']}")] = {
                    k: rec[k] for k in ("seconds", "generated_tok_s", "total_tok_s", "steps", "preemptions",
                                        "ttft_s_p50", "tpot_s_mean")}

    achieved = main["bytes_step"] / (main["ms_per_step"] * 1e-3) / 1e9
    out = {
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B size, random weights)",
        "value": main["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random prompt ids", "impl": "ours",
        "config": {
            "model": args.model, "layers": cfg.num_hidden_layers, "layers_of_model": n_layers_full,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "seq_len": PROMPT_LEN, "context_start": main["ctx"][0],
            "context_end": main["ctx"][1], "pool_context": POOL_CONTEXT, "page_size": PAGE,
            "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights 2.5 GB per step)",
            "decode": "cuda graph per batch bucket, sampling in graph",
        },
        "e2e": {"value": e2e["tok_s"], "unit": "tok/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"]},
        "points": points,
        "workloads": workloads,
        "clocks": clk,
        "build_s": t_build,
    }
    print(json.dumps(out))
    return 0


# BASELINE.json's other two configurations: (key, preset, requests, shortest and longest prompt, new tokens, temperatures)
WORKLOADS = [("llama-3.2-3b_32req_128-4096_128new", "llama-3.2-3b", 32, 128, 4096, 128, (0.0,)),
             ("smollm2-1.7b_64req_64-2048_256new", "smollm2-1.7b", 64, 64, 2048, 256, (0.0, 0.8))]


def measure_workload(model, n_req, lo, hi, new, temperatures, seed=0, layers=0):
    """Continuous batching through ``Engine.run_offline``: N requests with seeded uniform-random prompts of
    MIN..MAX tokens, NEW generated tokens each (no end-of-sequence id, so every request runs its full length),
    wall clock around the whole run; every run is made twice and the second one counts (the first one also captures
    the decode graphs).  One engine serves every temperature; returns one record per temperature."""
    import dataclasses

    import numpy as np
    import torch

    from inf_engine_b200 import Engine, Request, SamplingConfig
    from inf_engine_b200.config import get_preset

    cfg = get_preset(model)
    n_layers_full = cfg.num_hidden_layers
    if layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=layers)
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, n_req)
    n_blocks = int(sum(int(n) + new for n in lens)) // PAGE + 4 * n_req + 64
    torch.cuda.set_device(0)
    engine = Engine.from_random(cfg, seed=seed, dtype="bfloat16", n_total_blocks=n_blocks, block_size=PAGE,
                                max_requests=max(64, n_req), max_tokens_per_step=2048, eos_token=-1)
    out = []
    for temperature in temperatures:
        sampling = SamplingConfig(mode="temperature", temperature=temperature, seed=1) if temperature > 0 else SamplingConfig()

        def once():
            requests = [Request(i, rng.integers(0, cfg.vocab_size, int(n)).tolist(), new, sampling=sampling)
                        for i, n in enumerate(lens)]
            engine.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0}
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = engine.run_offline(requests)
            torch.cuda.synchronize()
            seconds = time.perf_counter() - t0
            engine.completed.clear()
            return seconds, sum(len(v) for v in res.values()), Engine.latency_stats(requests)

        once()
        seconds, generated, lat = once()
        prompt_tokens = int(lens.sum())
        out.append({"seconds": seconds, "generated": generated, "generated_tok_s": generated / seconds,
                    "total_tok_s": (generated + prompt_tokens) / seconds, "prompt_tokens": prompt_tokens,
                    "steps": engine.stats["steps"], "preemptions": engine.stats["preemptions"],
                    "temperature": temperature, "ttft_s_p50": lat["ttft_s"]["p50"], "tpot_s_mean": lat["tpot_s"]["mean"],
                    "layers": cfg.num_hidden_layers, "layers_of_model": n_layers_full})
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return out


def run_workload(args):
    """``--workload N:MIN:MAX:NEW[:TEMPERATURE]`` with ``--model``: one continuous-batching run (see measure_workload);
    BASELINE.json's other two workloads are ``--model smollm2-1.7b --workload 64:64:2048:256`` and
    ``--model llama-3.2-3b --workload 32:128:4096:128``; the default run prints both under ``workloads``."""
    parts = args.workload.split(":")
    if len(parts) not in (4, 5):
        print("--workload wants N:MIN:MAX:NEW or N:MIN:MAX:NEW:TEMPERATURE")
        return 2
    n_req, lo, hi, new = (int(x) for x in parts[:4])
    temperature = float(parts[4]) if len(parts) == 5 else 0.0
    rec = measure_workload(args.model, n_req, lo, hi, new, (temperature,), args.seed, args.layers)[0]
    print(json.dumps({"impl": "ours", "workload": args.workload, **rec, "dtype": "bf16",
                      "data": "synthetic: seeded random weights, uniform random prompt ids",
                      "config": {"model": args.model, "layers": rec["layers"], "layers_of_model": rec["layers_of_model"],
                                 "requests": n_req, "prompt_min": lo, "prompt_max": hi, "new_tokens": new,
                                 "temperature": temperature, "page_size": PAGE, "max_tokens_per_step": 2048}}))
    return 0


# ---------------------------------------------------------------- another family beside the Llama decoder
# ``--family barerax``: prefill and decode of a Barerax model (three delta-rule layers to one attention layer, LayerNorm,
# PolyNorm feed-forward, hashed bigram embedding) at sizes that resemble a real model's layers, beside a Llama model of
# equal width, depth, head geometry and parameter count, and every kernel of the new family beside the like kernel
# of the Llama path, each against its roofline.  The default workload and its JSON line are not touched by this.
FAMILY_SIZES = {"w1024": dict(width=1024, heads=16, kv=4, inter=4096), "w2048": dict(width=2048, heads=32, kv=8, inter=8192)}
FAMILY_LAYERS, FAMILY_VOCAB, FAMILY_HD = 4, 32768, 64


def _family_configs(size):
    from inf_engine_b200.config import parse_config_dict
    z = FAMILY_SIZES[size]
    w, H, G, inter = z["width"], z["heads"], z["kv"], z["inter"]
    ff = inter * 3 // 2                                   # two matrices of ff against three of inter: equal parameters
    mlp = {"kind": "dense", "ff": ff}
    delta = {"type": "general_delta", "mixer": {"heads": H, "dim": FAMILY_HD, "decay_rank": 64}, "mlp": mlp}
    att = {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": FAMILY_HD, "vdim": FAMILY_HD, "scale": FAMILY_HD ** -0.5,
                                          "bias_max": 1024, "rel_buckets": 32}, "mlp": mlp}
    layers = [att if i % 4 == 3 else delta for i in range(FAMILY_LAYERS)]
    brx = parse_config_dict({"architecture": "Barerax", "vocab": FAMILY_VOCAB, "width": w, "norm": {"eps": 1e-5},
                             "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}}, "layers": layers})
    llama = parse_config_dict(dict(architectures=["LlamaForCausalLM"], num_hidden_layers=FAMILY_LAYERS, hidden_size=w,
                                   num_attention_heads=H, num_key_value_heads=G, head_dim=FAMILY_HD, intermediate_size=inter,
                                   vocab_size=FAMILY_VOCAB, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
                                   max_position_embeddings=8192, hidden_act="silu"))
    return brx, llama


def _kipezen_configs(size):
    """A Kipezen model of the size's width (three delta layers to one parallel layer; 16 experts of which a token runs
    two, and a shared one: as many ACTIVE feed-forward parameters as the dense models beside it) and the Barerax model
    of equal width, depth and heads, the closest family the engine had."""
    from inf_engine_b200.config import parse_config_dict
    z = FAMILY_SIZES[size]
    w, H, G, inter = z["width"], z["heads"], z["kv"], z["inter"]
    mlp = {"kind": "moe", "expert": {"ff": inter // 4}, "shared": {"ff": inter // 2},
           "router": {"experts": 16, "top": 2, "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
    delta = {"type": "delta", "mixer": {"heads": H, "kv_heads": G, "dim": FAMILY_HD, "vdim": FAMILY_HD, "conv": 4}, "mlp": mlp}
    par = {"type": "parallel", "mlp": mlp,
           "mixer": {"left": {"heads": H, "kv_heads": G, "dim": FAMILY_HD, "vdim": FAMILY_HD, "scale": FAMILY_HD ** -0.5,
                              "rot": {"base": 10000.0, "dims": FAMILY_HD // 2}, "mask": {"size": 1024, "keep_first": 4}},
                     "right": {"width": w, "blocks": w // 256, "conv": 4}, "left_scale": 1.0, "right_scale": 1.0}}
    layers = [par if i % 4 == 3 else delta for i in range(FAMILY_LAYERS)]
    kpz = parse_config_dict({"architecture": "Kipezen", "vocab": FAMILY_VOCAB, "width": w, "norm": {"eps": 1e-5}, "layers": layers})
    return kpz, _family_configs(size)[0]


def _fovunex_configs(size):
    """A Fovunex model of the size's width (a recurrence, differential attention in chunks of 1,024 positions with
    values twice as large as a map, a recurrence, latent attention over rows of 192 compressed and 64 rotated numbers;
    gated residual sums; a clamped feed-forward of three matrices) and the Kipezen model of equal width, depth and head
    geometry, the closest family the engine had (rotated attention under a mask beside a gated recurrence with a float32
    state)."""
    from inf_engine_b200.config import parse_config_dict
    z = FAMILY_SIZES[size]
    w, H, G, inter = z["width"], z["heads"], z["kv"], z["inter"]
    mlp = {"kind": "dense", "ff": inter, "limit": 7.0}
    gru = {"type": "mingru", "mixer": {"width": w}, "mlp": mlp}
    diff = {"type": "attention", "mlp": mlp,
            "mixer": {"heads": H // 2, "kv_heads": G // 2, "dim": FAMILY_HD, "vdim": 2 * FAMILY_HD, "scale": FAMILY_HD ** -0.5,
                      "diff": 0.8, "rot": {"base": 10000.0, "dims": FAMILY_HD // 2}, "mask": {"size": FOVUNEX_CHUNK}}}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": H, "dim": FAMILY_HD, "rot_dim": FOVUNEX_ROT, "vdim": FAMILY_HD, "kv_rank": FOVUNEX_RANK,
                     "scale": (FAMILY_HD + FOVUNEX_ROT) ** -0.5,
                     "rot": {"base": 10000.0, "dims": FOVUNEX_ROT,
                             "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}}
    fvx = parse_config_dict({"architecture": "Fovunex", "vocab": FAMILY_VOCAB, "width": w, "norm": {"eps": 1e-5},
                             "embedding": {"scale": float(w) ** 0.5}, "layers": [gru, diff, gru, lat]})
    return fvx, _kipezen_configs(size)[0]


FOVUNEX_CHUNK, FOVUNEX_RANK, FOVUNEX_ROT = 1024, 192, 64


def _gavatar_configs(size):
    """A Gavatar model of the size's width (a matrix memory, attention with weights mixed across heads under a window of
    1,024 keys, a matrix memory, latent attention over compressed rows of 192 numbers with a sink under the same window;
    every layer with 16 experts of which a token runs four: as many ACTIVE feed-forward parameters as the dense models)
    and the Kipezen model of equal width, depth and head geometry, the closest family the engine had (a routed mixture of
    experts, windowed attention, a gated recurrence with a float32 matrix state per head)."""
    from inf_engine_b200.config import parse_config_dict
    z = FAMILY_SIZES[size]
    w, H, G, inter = z["width"], z["heads"], z["kv"], z["inter"]
    mlp = {"kind": "moe", "expert": {"ff": inter // 4}, "router": {"experts": 16, "top": 4}}
    mem = {"type": "mlstm", "mixer": {"heads": H, "dim": FAMILY_HD, "vdim": FAMILY_HD, "gate_cap": 15.0}, "mlp": mlp}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": H, "kv_heads": G, "dim": FAMILY_HD, "vdim": FAMILY_HD, "scale": FAMILY_HD ** -0.5,
                     "mask": {"size": GAVATAR_WINDOW}}}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": H, "dim": FAMILY_HD, "vdim": FAMILY_HD, "q_rank": w // 2, "kv_rank": GAVATAR_RANK,
                     "scale": FAMILY_HD ** -0.5, "mask": {"size": GAVATAR_WINDOW}}}
    gav = parse_config_dict({"architecture": "Gavatar", "vocab": FAMILY_VOCAB, "width": w, "norm": {"eps": 1e-5},
                             "embedding": {"scale": float(w) ** 0.5}, "layers": [mem, att, mem, lat]})
    return gav, _kipezen_configs(size)[0]


GAVATAR_WINDOW, GAVATAR_RANK = 1024, 192


def _weight_bytes(runner):
    seen, n = set(), 0
    import torch
    stack = [runner.model]
    while stack:
        o = stack.pop()
        if id(o) in seen:
            continue
        seen.add(id(o))
        if isinstance(o, torch.Tensor):
            n += o.numel() * o.element_size()
        elif isinstance(o, (list, tuple)):
            stack.extend(o)
        elif hasattr(o, "__dict__") and type(o).__module__.startswith("inf_engine_b200.parts"):
            stack.extend(v for k, v in vars(o).items() if k not in ("rt", "spec", "_views", "_prev_token"))
    return n


def run_family(args):
    import numpy as np
    import torch

    from inf_engine_b200 import Engine, StepEntry, SamplingConfig, kernels
    from inf_engine_b200.sampling import pack_rows, request_key

    if args.family not in ("barerax", "kipezen", "fovunex", "gavatar"):
        print(f"--family {args.family}: unknown (known: barerax, kipezen, fovunex, gavatar)")
        return 2
    pk = peaks()
    torch.cuda.set_device(0)
    rng = np.random.default_rng(args.seed)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")        # larger than L2; written between timed launches
    clocks = ClockSampler()
    clocks.start()
    t_all0 = time.perf_counter()

    def timed(fn, reps=9, warm=3):
        """Median device time (ms) of ``fn`` alone, L2 flushed before every timed launch."""
        for _ in range(warm):
            fn()
        out = []
        for _ in range(reps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            out.append(e0.elapsed_time(e1))
        return sorted(out)[len(out) // 2]

    def model_numbers_of(cfg, batch):
        engine = Engine.from_random(cfg, seed=args.seed, dtype="bfloat16", n_total_blocks=(batch + 1) * POOL_CONTEXT // PAGE,
                                    block_size=PAGE, max_requests=max(16, batch), max_tokens_per_step=8192, chunk=2048)
        runner = engine.runner
        V = runner.spec.vocab_size

        def prefill_once():
            runner.open("p")
            toks = rng.integers(0, V, PROMPT_LEN).tolist()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            n0 = kernels.LAUNCHES
            e0.record()
            runner.step([StepEntry("p", toks, [PROMPT_LEN - 1])])
            e1.record()
            torch.cuda.synchronize()
            runner.close("p")
            return e0.elapsed_time(e1), kernels.LAUNCHES - n0
        for _ in range(3):
            prefill_once()
        runs = sorted(prefill_once() for _ in range(5))
        pre_ms, pre_launches = runs[len(runs) // 2]
        rids = [f"d{i}" for i in range(batch)]
        for rid in rids:
            runner.open(rid)
        for i in range(0, batch, 4):
            runner.step([StepEntry(r, rng.integers(0, V, PROMPT_LEN).tolist(), []) for r in rids[i:i + 4]])
        rows = pack_rows([SamplingConfig()] * batch, [request_key(i, 0) for i in range(batch)], V)
        ids = torch.as_tensor(rng.integers(0, V, batch), dtype=torch.int32).cuda()
        entries = [StepEntry(r, [0], [0]) for r in rids]
        for _ in range(max(args.warmup, 3)):
            _, ids = runner.step_and_sample(entries, rows, device_tokens=ids)
        torch.cuda.synchronize()
        n0 = kernels.LAUNCHES
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            _, ids = runner.step_and_sample(entries, rows, device_tokens=ids)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        launches = (kernels.LAUNCHES - n0) // args.steps
        wb = _weight_bytes(runner)
        cache_b = runner.cache.storage_bytes()
        for rid in rids:
            runner.close(rid)
        out = {"prefill_tok_s": PROMPT_LEN / pre_ms * 1e3, "prefill_ms": pre_ms, "prefill_launches": pre_launches,
               "decode_tok_s": batch / ms * 1e3, "decode_ms_per_step": ms, "decode_launches_per_step": launches,
               "weight_bytes": wb, "decode_weight_stream_frac": wb / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]}
        del engine, runner
        gc.collect()
        torch.cuda.empty_cache()
        return out

    def kernel_table(size):
        """Every kernel of the family alone, beside the like kernel of the Llama path, at 2,048 tokens of one request
        (prefill) and at 8 requests of one token over 2,048 keys (decode).  frac: of the HBM peak for what only moves
        bytes, of the bf16 tensor peak for attention over a prompt."""
        z = FAMILY_SIZES[size]
        W, H, G, hd, inter = z["width"], z["heads"], z["kv"], FAMILY_HD, z["inter"]
        ff = inter * 3 // 2
        N, dev, bf = PROMPT_LEN, "cuda", torch.bfloat16
        g = torch.Generator(device=dev).manual_seed(1)
        rnd = lambda *shape: (torch.randn(*shape, device=dev, generator=g) * 0.5)
        i32 = lambda v: torch.as_tensor(v, dtype=torch.int32, device=dev)
        rows = []

        def add(name, like, nbytes, ms, ms_like, nbytes_like=None, flops=None):
            rec = {"kernel": name, "like": like, "ms": ms, "like_ms": ms_like}
            if flops is None:
                rec["frac_of_hbm"] = nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]
                rec["like_frac_of_hbm"] = (nbytes_like or nbytes) / (ms_like * 1e-3) / 1e9 / pk["hbm_gbs"] if ms_like else None
            else:
                rec["frac_of_bf16"] = flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"]
                rec["like_frac_of_bf16"] = flops / (ms_like * 1e-3) / 1e12 / pk["bf16_tflops"] if ms_like else None
            rows.append(rec)

        # norms: residual in and out (float32) + delta in + normed out (bfloat16)
        res, delta, out = rnd(N, W), rnd(N, W).to(bf), torch.empty(N, W, device=dev, dtype=bf)
        gain, bias = rnd(W).to(bf), rnd(W).to(bf)
        add("layernorm(+residual sum)", "rmsnorm(+residual sum)", N * W * (4 + 4 + 2 + 2),
            timed(lambda: kernels.layernorm(res, delta, gain, bias, out, 1e-5)),
            timed(lambda: kernels.rmsnorm(res, delta, gain, out, 1e-5)))
        # activation of the feed-forward
        z_up, h = rnd(N, ff).to(bf), torch.empty(N, ff, device=dev, dtype=bf)
        gu, h2 = rnd(N, 2 * inter).to(bf), torch.empty(N, inter, device=dev, dtype=bf)
        add("polynorm(+up bias)", "silu_mul", N * ff * 4, timed(lambda: kernels.polynorm(z_up, rnd(ff).to(bf), rnd(4).to(bf), h, 1e-5)),
            timed(lambda: kernels.silu_mul(gu, h2, interleaved=True)), N * inter * 6)
        # embedding
        table, bigram = rnd(FAMILY_VOCAB, W).to(bf), rnd(65522, W).to(bf)
        ids, pos = i32(rng.integers(0, FAMILY_VOCAB, N)), torch.arange(N, dtype=torch.int32, device=dev)
        state = torch.zeros(4, dtype=torch.int32, device=dev)
        add("embed + hashed bigram", "embed_gather", N * W * (2 + 2 + 4),
            timed(lambda: kernels.embed_bigram(ids, pos, i32([0, N]), i32([0]), 1, table, bigram, state, res, 65521, 1000003, 31)),
            timed(lambda: kernels.embed_gather(ids, table, res)), N * W * (2 + 4))
        # q/k head norm + cache write against rotation + cache write
        B = 8
        n_pages = B * N // PAGE                              # room for 8 requests of 2,048 keys
        qkv = rnd(N, (H + 2 * G) * hd).to(bf)
        q, kx, v = qkv[:, :H * hd], qkv[:, H * hd:(H + G) * hd], qkv[:, (H + G) * hd:]
        kpool = torch.zeros(n_pages, G, PAGE, hd, device=dev, dtype=bf)
        vpool = torch.zeros_like(kpool)
        slot_map = torch.arange(N, dtype=torch.int32, device=dev)
        cos, sin = torch.ones(N, hd // 2, device=dev), torch.zeros(N, hd // 2, device=dev)
        qg = (1 + 0.1 * rnd(hd)).to(bf)
        nb = N * (H + 2 * G) * hd * 2 * 2
        add("q/k head norm + cache write", "rotation + cache write", nb,
            timed(lambda: kernels.headnorm_kv_write(q, kx, v, qg, qg, 1e-5, slot_map, kpool, vpool, H, G, hd, hd, PAGE)),
            timed(lambda: kernels.rope_kv_write(q, kx, v, cos, sin, pos, slot_map, kpool, vpool, H, G, hd, PAGE)))
        # attention over a prompt of 2,048 tokens
        from inf_engine_b200.parts.attention import PagedAttention
        from inf_engine_b200.parts import Runtime
        from inf_engine_b200.engine.batch import KVGroupContext, StepContext
        brx, llama = _family_configs(size)
        rt = Runtime(dev, bf)

        def attention_part(spec_layer, names):
            spec = spec_layer.mixer
            tensors = {n: (rnd(*e.shape) * 0.1).to(bf) for n, e in PagedAttention.expected_tensors(spec).items()}
            return PagedAttention(spec, tensors, rt)

        def context(q_lens, before):
            ctx = StepContext(rt, PAGE)
            R, n = len(q_lens), sum(q_lens)
            ctx.n_tokens, ctx.n_requests, ctx.n_logits = n, R, 0
            starts = [0]
            for ql in q_lens:
                starts.append(starts[-1] + ql)
            per = n_pages // R
            ctx.q_start, ctx.ctx_before = i32(starts), i32(before)
            ctx.positions = i32([b + t for ql, b in zip(q_lens, before) for t in range(ql)])
            ctx.slots = i32(list(range(R)))
            table_ = torch.arange(per * R, dtype=torch.int32, device=dev).view(R, per)
            sm = i32([(r * per + (b + t) // PAGE) * PAGE + (b + t) % PAGE for r, (ql, b) in enumerate(zip(q_lens, before)) for t in range(ql)])
            ctx.kv = [KVGroupContext(sm, table_)]
            ctx.host = {"q_lens": list(q_lens), "ctx_before": list(before), "q_start": starts}
            ctx.max_q_len, ctx.max_seq_len = max(q_lens), max(b + ql for ql, b in zip(q_lens, before))
            ctx.keys_cap = ctx.max_seq_len
            return ctx

        from inf_engine_b200.parts import CacheView
        att_b = attention_part(brx.model_spec().layers[3], None)
        att_l = attention_part(llama.model_spec().layers[0], None)
        view = CacheView("kv", 0, kpool, vpool, None, True)
        flops = 4 * H * hd * (N * (N + 1) // 2)
        ctx_p = context([N], [0])
        qkv_p = rnd(N, (H + 2 * G) * hd).to(bf)
        add("attention, prompt (head norms, temperature, distance bias)", "attention, prompt (rotation)", 0,
            timed(lambda: att_b._rotate_write_attend(qkv_p.clone(), ctx_p, view), reps=5),
            timed(lambda: att_l._rotate_write_attend(qkv_p.clone(), ctx_p, view), reps=5), flops=flops)
        ctx_d = context([1] * B, [N - 1] * B)                # 8 requests of 2,048 keys, one new token each
        qkv_d = rnd(B, (H + 2 * G) * hd).to(bf)
        kv_bytes = B * N * G * hd * 2 * 2
        add("attention, decode b8 x 2,048 keys", "attention, decode (fused rotation)", kv_bytes,
            timed(lambda: att_b._rotate_write_attend(qkv_d.clone(), ctx_d, view)),
            timed(lambda: att_l._rotate_write_attend(qkv_d.clone(), ctx_d, view)))
        # the delta rule: five projections in (bfloat16), w_pre (float32), output (bfloat16); state in and out
        Wd = H * hd
        proj, w_pre = rnd(N, 5 * Wd + 64).to(bf), rnd(N, Wd)
        vec = rnd(Wd).to(bf)
        st = torch.zeros(16, H, hd, hd, device=dev)
        mixed = torch.empty(N, Wd, device=dev, dtype=bf)
        views = [proj[:, i * Wd:(i + 1) * Wd] for i in range(5)]
        run_delta = lambda n, qs, sl, R: kernels.delta_rule(views[0][:n], views[1][:n], views[2][:n], views[4][:n], views[3][:n], w_pre[:n],
                                                             vec, vec, vec, st, mixed[:n], qs, sl, R, H, hd, 0.6, 1e-6, 1e-5)
        qs1, sl1 = i32([0, N]), i32([0])
        qs8, sl8 = torch.arange(B + 1, dtype=torch.int32, device=dev), torch.arange(B, dtype=torch.int32, device=dev)
        ms_p = timed(lambda: run_delta(N, qs1, sl1, 1), reps=5)
        ms_d = timed(lambda: run_delta(B, qs8, sl8, B))
        rows.append({"kernel": "delta rule, prompt of 2,048 tokens (one request)", "like": None, "ms": ms_p,
                     "frac_of_hbm": (N * Wd * (5 * 2 + 4 + 2) + 2 * H * hd * hd * 4) / (ms_p * 1e-3) / 1e9 / pk["hbm_gbs"],
                     "note": "a token-by-token scan: latency of %d dependent steps, not bytes, bounds it" % N})
        rows.append({"kernel": "delta rule, decode b8", "like": "attention, decode (fused rotation)", "ms": ms_d,
                     "frac_of_hbm": (B * 2 * H * hd * hd * 4) / (ms_d * 1e-3) / 1e9 / pk["hbm_gbs"],
                     "like_ms": rows[-2]["like_ms"], "like_frac_of_hbm": rows[-2]["like_frac_of_hbm"]})
        return rows

    def kipezen_kernel_table(size):
        """Every kernel that the Kipezen family added, alone, beside the like kernel of the closest family (Barerax, or
        the Llama path where Barerax has none), at 2,048 tokens of one request and at 8 requests of one token."""
        z = FAMILY_SIZES[size]
        W, H, G, hd, inter = z["width"], z["heads"], z["kv"], FAMILY_HD, z["inter"]
        N, B, dev, bf = PROMPT_LEN, 8, "cuda", torch.bfloat16
        g = torch.Generator(device=dev).manual_seed(1)
        rnd = lambda *shape: (torch.randn(*shape, device=dev, generator=g) * 0.5)
        i32 = lambda v: torch.as_tensor(v, dtype=torch.int32, device=dev)
        rows = []

        def add(name, like, ms, ms_like, nbytes=None, nbytes_like=None, flops=None, flops_like=None, note=None):
            rec = {"kernel": name, "like": like, "ms": ms, "like_ms": ms_like}
            if nbytes is not None:
                rec["frac_of_hbm"] = nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]
                if ms_like:
                    rec["like_frac_of_hbm"] = (nbytes_like or nbytes) / (ms_like * 1e-3) / 1e9 / pk["hbm_gbs"]
            if flops is not None:
                rec["frac_of_bf16"] = flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"]
                if ms_like:
                    rec["like_frac_of_bf16"] = (flops_like or flops) / (ms_like * 1e-3) / 1e12 / pk["bf16_tflops"]
            if note:
                rec["note"] = note
            rows.append(rec)

        qs1, sl1 = i32([0, N]), i32([0])
        qs8, sl8 = torch.arange(B + 1, dtype=torch.int32, device=dev), torch.arange(B, dtype=torch.int32, device=dev)
        # the norm of a sublayer's output into the residual (and the next sublayer's input) | RMSNorm + residual sum
        res, y, nxt = rnd(N, W), rnd(N, W).to(bf), torch.empty(N, W, device=dev, dtype=bf)
        gain = (1 + 0.1 * rnd(W))
        add("output norm into the residual (+ next input)", "rmsnorm(+residual sum)",
            timed(lambda: kernels.outnorm_accumulate(res, y, gain, 1e-5, nxt)),
            timed(lambda: kernels.rmsnorm(res, y, gain.to(bf), nxt, 1e-5)), N * W * (4 + 4 + 2 + 2))
        # short convolution with state over q | k | v of a delta layer | SiLU(gate) * up (an elementwise pass)
        C = 2 * G * hd + H * hd
        xin, cw, cout = rnd(N, C + 2 * H + H * hd).to(bf), rnd(C, 4).to(bf), torch.empty(N, C, device=dev, dtype=bf)
        cstate = torch.zeros(16, 3, C, device=dev, dtype=bf)
        gu, h2 = rnd(N, 2 * inter).to(bf), torch.empty(N, inter, device=dev, dtype=bf)
        add("short convolution + SiLU, prompt", "silu_mul",
            timed(lambda: kernels.causal_conv(xin[:, :C], cw, None, cstate, cout, qs1, sl1, 1, activation="silu")),
            timed(lambda: kernels.silu_mul(gu, h2, interleaved=True)), N * C * 4, N * inter * 6)
        add("short convolution + SiLU, decode b8", None,
            timed(lambda: kernels.causal_conv(xin[:B, :C], cw, None, cstate, cout[:B], qs8, sl8, B, activation="silu")), None,
            B * C * (2 + 2 + 2 * 3 * 2))
        # the gated delta rule | the generalized delta rule of Barerax
        Wd = H * hd
        q_, k_, v_ = cout[:, :G * hd], cout[:, G * hd:2 * G * hd], cout[:, 2 * G * hd:]
        gate, b_pre, a_pre = xin[:, C:C + Wd], xin[:, C + Wd:C + Wd + H], xin[:, C + Wd + H:C + Wd + 2 * H]
        a_log, dt_b, og = rnd(H).to(bf), rnd(H).to(bf), (1 + 0.1 * rnd(hd)).to(bf)
        st = torch.zeros(16, H, hd, hd, device=dev)
        mixed = torch.empty(N, Wd, device=dev, dtype=bf)
        run_gd = lambda n, qs, sl, R: kernels.gated_delta(q_[:n], k_[:n], v_[:n], b_pre[:n], a_pre[:n], gate[:n], a_log, dt_b, og, st,
                                                          mixed[:n], qs, sl, R, H, G, hd, hd, 1e-6, 1e-5)
        proj, w_pre, vec = rnd(N, 5 * Wd + 64).to(bf), rnd(N, Wd), rnd(Wd).to(bf)
        views = [proj[:, i * Wd:(i + 1) * Wd] for i in range(5)]
        run_brx = lambda n, qs, sl, R: kernels.delta_rule(views[0][:n], views[1][:n], views[2][:n], views[4][:n], views[3][:n], w_pre[:n],
                                                           vec, vec, vec, st, mixed[:n], qs, sl, R, H, hd, 0.6, 1e-6, 1e-5)
        add("gated delta rule, prompt of 2,048 tokens (one request)", "generalized delta rule, prompt",
            timed(lambda: run_gd(N, qs1, sl1, 1), reps=5), timed(lambda: run_brx(N, qs1, sl1, 1), reps=5),
            N * (2 * G * hd + 3 * Wd) * 2 + 2 * H * hd * hd * 4, N * Wd * (5 * 2 + 4 + 2) + 2 * H * hd * hd * 4,
            note="a token-by-token scan: the chain of %d dependent steps bounds it, not bytes" % N)
        add("gated delta rule, decode b8", "generalized delta rule, decode",
            timed(lambda: run_gd(B, qs8, sl8, B)), timed(lambda: run_brx(B, qs8, sl8, B)), B * 2 * H * hd * hd * 4)
        # whole-row norm + pair rotation + cache write | head norm + cache write of Barerax
        n_pages = B * N // PAGE
        qkv = rnd(N, (H + 2 * G) * hd).to(bf)
        q, kx, v = qkv[:, :H * hd], qkv[:, H * hd:(H + G) * hd], qkv[:, (H + G) * hd:]
        kpool = torch.zeros(n_pages, G, PAGE, hd, device=dev, dtype=bf)
        vpool = torch.zeros_like(kpool)
        slot_map, pos = torch.arange(N, dtype=torch.int32, device=dev), torch.arange(N, dtype=torch.int32, device=dev)
        qb, kb, vb, qg, kg = rnd(H * hd).to(bf), rnd(G * hd).to(bf), rnd(G * hd).to(bf), (1 + 0.1 * rnd(H * hd)).to(bf), (1 + 0.1 * rnd(G * hd)).to(bf)
        inv_freq = (10000.0 ** (-2.0 * torch.arange(hd // 4, dtype=torch.float64) / (hd // 2))).to(dev)
        hg = (1 + 0.1 * rnd(hd)).to(bf)
        add("biases + whole-row norm + pair rotation + cache write", "q/k head norm + cache write",
            timed(lambda: kernels.rownorm_rotate_write(q, kx, v, qb, kb, vb, qg, kg, 1e-5, inv_freq, hd // 2, pos, slot_map, kpool, vpool,
                                                       H, G, hd, hd, PAGE)),
            timed(lambda: kernels.headnorm_kv_write(q, kx, v, hg, hg, 1e-5, slot_map, kpool, vpool, H, G, hd, hd, PAGE)),
            N * (H + 2 * G) * hd * 2 * 2)
        # attention with a window and kept first keys | attention with a distance bias (Barerax)
        from inf_engine_b200.parts.attention import PagedAttention
        from inf_engine_b200.parts import CacheView, Runtime
        from inf_engine_b200.engine.batch import KVGroupContext, StepContext
        kpz, brx = _kipezen_configs(size)
        rt = Runtime(dev, bf)

        def attention_part(spec):
            tensors = {n: ((1 + 0.1 * rnd(*e.shape)) if e.init == "gain" else rnd(*e.shape) * 0.1).to(bf)
                       for n, e in PagedAttention.expected_tensors(spec).items()}
            return PagedAttention(spec, tensors, rt)

        def context(q_lens, before):
            ctx = StepContext(rt, PAGE)
            R, n = len(q_lens), sum(q_lens)
            ctx.n_tokens, ctx.n_requests, ctx.n_logits = n, R, 0
            starts = [0]
            for ql in q_lens:
                starts.append(starts[-1] + ql)
            per = n_pages // R
            ctx.q_start, ctx.ctx_before = i32(starts), i32(before)
            ctx.positions = i32([b + t for ql, b in zip(q_lens, before) for t in range(ql)])
            ctx.slots = i32(list(range(R)))
            table_ = torch.arange(per * R, dtype=torch.int32, device=dev).view(R, per)
            sm = i32([(r * per + (b + t) // PAGE) * PAGE + (b + t) % PAGE for r, (ql, b) in enumerate(zip(q_lens, before)) for t in range(ql)])
            ctx.kv = [KVGroupContext(sm, table_)]
            ctx.host = {"q_lens": list(q_lens), "ctx_before": list(before), "q_start": starts}
            ctx.max_q_len, ctx.max_seq_len = max(q_lens), max(b + ql for ql, b in zip(q_lens, before))
            ctx.keys_cap = ctx.max_seq_len
            return ctx

        att_k = attention_part(kpz.model_spec().layers[3].mixer.branches[0])
        att_b = attention_part(brx.model_spec().layers[3].mixer)
        view = CacheView("kv", 0, kpool, vpool, None, True)
        window = 1024
        pairs_b = N * (N + 1) // 2
        pairs_k = pairs_b - (N - window) * (N - window + 1) // 2 + 4 * (N - window - 4)
        ctx_p = context([N], [0])
        qkv_p = rnd(N, (H + 2 * G) * hd).to(bf)
        add("attention, prompt (window of 1,024 + 4 kept keys)", "attention, prompt (distance bias, every key)",
            timed(lambda: att_k._rotate_write_attend(qkv_p.clone(), ctx_p, view), reps=5),
            timed(lambda: att_b._rotate_write_attend(qkv_p.clone(), ctx_p, view), reps=5),
            flops=4 * H * hd * pairs_k, flops_like=4 * H * hd * pairs_b)
        ctx_d = context([1] * B, [N - 1] * B)
        qkv_d = rnd(B, (H + 2 * G) * hd).to(bf)
        add("attention, decode b8 x 2,048 keys (1,028 visible)", "attention, decode (distance bias, every key)",
            timed(lambda: att_k._rotate_write_attend(qkv_d.clone(), ctx_d, view)),
            timed(lambda: att_b._rotate_write_attend(qkv_d.clone(), ctx_d, view)),
            B * (window + 4) * G * hd * 2 * 2, B * N * G * hd * 2 * 2)
        # the recurrent block: block-diagonal gates (float32 products) and the scan
        nb_ = W // 256
        u, ypre = rnd(N, W).to(bf), rnd(N, W).to(bf)
        ag, gates = rnd(nb_, 256, 256).to(bf), torch.empty(N, 2 * W, device=dev)
        lam, rb = rnd(W).to(bf), rnd(W).to(bf)
        sst, rout = torch.zeros(16, W, device=dev), torch.empty(N, W, device=dev, dtype=bf)
        ms = timed(lambda: kernels.gemm_simt_batched(u, ag, gates[:, :W]))
        rows.append({"kernel": "block-diagonal gate product, prompt (float32 on CUDA cores)", "like": None, "ms": ms,
                     "tflops_f32": 2 * N * W * 256 / (ms * 1e-3) / 1e12})
        add("linear recurrent unit scan, prompt of 2,048 tokens (one request)", "generalized delta rule, prompt",
            timed(lambda: kernels.linear_recurrence(u, ypre, gates[:, :W], gates[:, W:], rb, rb, lam, sst, rout, qs1, sl1, 1, 8.0), reps=5),
            rows[3]["like_ms"], N * W * (2 + 2 + 4 + 4 + 2), N * Wd * (5 * 2 + 4 + 2),
            note="a scan over tokens, a channel a thread")
        add("linear recurrent unit scan, decode b8", "generalized delta rule, decode",
            timed(lambda: kernels.linear_recurrence(u[:B], ypre[:B], gates[:B, :W], gates[:B, W:], rb, rb, lam, sst, rout[:B], qs8, sl8, B, 8.0)),
            rows[4]["like_ms"], B * W * (2 + 2 + 4 + 4 + 2 + 8), B * 2 * H * hd * hd * 4)
        # the routed experts: route + sort, the two grouped products | the dense gate/up product of the Llama path
        E, top, ffe = 16, 2, inter // 4
        x = rnd(N, W).to(bf)
        logits = rnd(N, E + 1) * 2
        ids, wts, gt = torch.empty(N, top, dtype=torch.int32, device=dev), torch.empty(N, top, device=dev), torch.empty(N, device=dev)
        sorted_pairs = torch.empty(N * top, dtype=torch.int32, device=dev)
        tiles = torch.empty(kernels.moe_max_tiles(N * top, E), 4, dtype=torch.int32, device=dev)
        def route_sort():
            kernels.moe_route(logits, None, ids, wts, gt, E, top, 4, 2, 2.5, 1e-20, gate_col=E)
            kernels.moe_sort(ids, E, sorted_pairs, tiles)
        ms = timed(route_sort)
        rows.append({"kernel": "route + sort, 2,048 tokens x 2 of 16 experts", "like": None, "ms": ms})
        gate_up, down = (rnd(E, 2 * ffe, W) * 0.1).to(bf), (rnd(E, W, ffe) * 0.1).to(bf)
        hid, yp = torch.empty(N * top, ffe, device=dev, dtype=bf), torch.empty(N * top, W, device=dev)
        dense_w, dense_out = (rnd(2 * inter, W) * 0.1).to(bf), torch.empty(N, inter, device=dev, dtype=bf)
        like_ms = timed(lambda: kernels.gemm_tcgen05(x, dense_w, dense_out, "silu_mul"))
        add("experts' gate/up product with SiLU, prompt (2 of 16 experts a token)", "dense gate/up product with SiLU (tcgen05)",
            timed(lambda: kernels.moe_gemm(x, gate_up, hid, sorted_pairs, tiles, top, gather=True, scatter=False, epi="silu_mul")),
            like_ms, flops=2 * N * top * 2 * ffe * W, flops_like=2 * N * 2 * inter * W)
        add("experts' down product, prompt", "dense gate/up product with SiLU (tcgen05)",
            timed(lambda: kernels.moe_gemm(hid, down, yp, sorted_pairs, tiles, top, gather=False, scatter=True)),
            like_ms, flops=2 * N * top * ffe * W, flops_like=2 * N * 2 * inter * W)
        # decode: 8 tokens choose 2 of 16 experts; what must move is the chosen experts' weights
        ids8 = ids[:B].contiguous()
        sp8, tl8 = torch.empty(B * top, dtype=torch.int32, device=dev), torch.empty(kernels.moe_max_tiles(B * top, E), 4, dtype=torch.int32, device=dev)
        kernels.moe_sort(ids8, E, sp8, tl8)
        n_chosen = len(set(ids8.flatten().tolist()))
        add("experts' gate/up product with SiLU, decode b8", "dense gate/up with SiLU, decode (streaming product)",
            timed(lambda: kernels.moe_gemm(x[:B], gate_up, hid[:B * top], sp8, tl8, top, gather=True, scatter=False, epi="silu_mul")),
            timed(lambda: kernels.gemm_stream(x[:B], dense_w, dense_out[:B], B, "silu_mul")),
            n_chosen * 2 * ffe * W * 2, 2 * inter * W * 2)
        return rows

    def fovunex_kernel_table(size):
        """Every kernel that the Fovunex family added, alone, beside the like kernel of the closest family (Kipezen, or
        the Llama path where Kipezen has none), at 2,048 tokens of one request and at 8 requests of one token over
        2,048 keys."""
        from inf_engine_b200.engine.batch import KVGroupContext, StepContext
        from inf_engine_b200.parts import CacheView, Runtime
        from inf_engine_b200.parts.attention import PagedAttention
        from inf_engine_b200.parts.latent import attend_float32
        z = FAMILY_SIZES[size]
        W, H, G, hd, inter = z["width"], z["heads"], z["kv"], FAMILY_HD, z["inter"]
        N, B, dev, bf = PROMPT_LEN, 8, "cuda", torch.bfloat16
        g = torch.Generator(device=dev).manual_seed(1)
        rnd = lambda *shape: (torch.randn(*shape, device=dev, generator=g) * 0.5)
        i32 = lambda v: torch.as_tensor(v, dtype=torch.int32, device=dev)
        rows = []

        def add(name, like, ms, ms_like, nbytes=None, nbytes_like=None, flops=None, flops_like=None, note=None):
            rec = {"kernel": name, "like": like, "ms": ms, "like_ms": ms_like}
            if nbytes is not None:
                rec["frac_of_hbm"] = nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]
                if ms_like:
                    rec["like_frac_of_hbm"] = (nbytes_like or nbytes) / (ms_like * 1e-3) / 1e9 / pk["hbm_gbs"]
            if flops is not None:
                rec["frac_of_bf16"] = flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"]
                if ms_like:
                    rec["like_frac_of_bf16"] = (flops_like or flops) / (ms_like * 1e-3) / 1e12 / pk["bf16_tflops"]
            if note:
                rec["note"] = note
            rows.append(rec)

        rt = Runtime(dev, bf)
        n_pages = B * N // PAGE
        qs1, sl1 = i32([0, N]), i32([0])
        qs8, sl8 = torch.arange(B + 1, dtype=torch.int32, device=dev), torch.arange(B, dtype=torch.int32, device=dev)

        def context(q_lens, before):
            ctx = StepContext(rt, PAGE)
            R, n = len(q_lens), sum(q_lens)
            ctx.n_tokens, ctx.n_requests, ctx.n_logits = n, R, 0
            starts = [0]
            for ql in q_lens:
                starts.append(starts[-1] + ql)
            per = n_pages // R
            ctx.q_start, ctx.ctx_before = i32(starts), i32(before)
            ctx.positions = i32([b + t for ql, b in zip(q_lens, before) for t in range(ql)])
            ctx.slots = i32(list(range(R)))
            table_ = torch.arange(per * R, dtype=torch.int32, device=dev).view(R, per)
            sm = i32([(r * per + (b + t) // PAGE) * PAGE + (b + t) % PAGE for r, (ql, b) in enumerate(zip(q_lens, before)) for t in range(ql)])
            ctx.kv = [KVGroupContext(sm, table_)]
            ctx.host = {"q_lens": list(q_lens), "ctx_before": list(before), "q_start": starts}
            ctx.max_q_len, ctx.max_seq_len = max(q_lens), max(b + ql for ql, b in zip(q_lens, before))
            ctx.keys_cap = ctx.max_seq_len
            return ctx

        ctx_p, ctx_d = context([N], [0]), context([1] * B, [N - 1] * B)
        # the gated sum into the residual | the norm of a sublayer's output into the residual (Kipezen)
        res, y, gpre, gb = rnd(N, W), rnd(N, W).to(bf), rnd(N, W).to(bf), rnd(W).to(bf)
        nxt, gain = torch.empty(N, W, device=dev, dtype=bf), (1 + 0.1 * rnd(W))
        add("gated sum into the residual", "output norm into the residual (+ next input)",
            timed(lambda: kernels.gated_residual_add(res, y, gpre, gb)),
            timed(lambda: kernels.outnorm_accumulate(res, y, gain, 1e-5, nxt)), N * W * (4 + 4 + 2 + 2), N * W * (4 + 4 + 2 + 2))
        # the clamped activation of the feed-forward | SiLU(gate) * up (the Llama path's elementwise pass)
        gu, h2 = rnd(N, 2 * inter).to(bf), torch.empty(N, inter, device=dev, dtype=bf)
        add("clamped gate * sigmoid(1.702 gate) * (up + 1)", "silu_mul",
            timed(lambda: kernels.glu_act(gu, h2, "clamped_swish", interleaved=True, alpha=1.702, limit=7.0, up_offset=1.0)),
            timed(lambda: kernels.silu_mul(gu, h2, interleaved=True)), N * inter * 6)
        # the minGRU scan | the linear recurrent unit's scan (Kipezen)
        zug, zb = rnd(N, 3 * W).to(bf), rnd(W).to(bf)
        sst, rout = torch.zeros(16, W, device=dev), torch.empty(N, W, device=dev, dtype=bf)
        u, ypre, gates, lam = rnd(N, W).to(bf), rnd(N, W).to(bf), rnd(N, 2 * W), rnd(W).to(bf)
        scan = lambda n, qs, sl, R: kernels.mingru_scan(zug[:n, :W], zug[:n, W:2 * W], zug[:n, 2 * W:], zb, zb, sst, rout[:n], qs, sl, R,
                                                        max_q_len=n // R)
        lru = lambda n, qs, sl, R: kernels.linear_recurrence(u[:n], ypre[:n], gates[:n, :W], gates[:n, W:], zb, zb, lam, sst, rout[:n],
                                                             qs, sl, R, 8.0)
        add("minGRU scan, prompt of 2,048 tokens (one request)", "linear recurrent unit scan, prompt",
            timed(lambda: scan(N, qs1, sl1, 1), reps=5), timed(lambda: lru(N, qs1, sl1, 1), reps=5),
            N * W * (3 * 2 + 2), N * W * (2 + 2 + 4 + 4 + 2), note="the request's tokens cut into runs that are scanned side by side")
        add("minGRU scan, decode b8", "linear recurrent unit scan, decode",
            timed(lambda: scan(B, qs8, sl8, B)), timed(lambda: lru(B, qs8, sl8, B)),
            B * W * (3 * 2 + 2 + 8), B * W * (2 + 2 + 4 + 4 + 2 + 8))
        # differential attention: H/2 heads of two maps of 64 over values of 128; G/2 key heads of two maps
        Hd, Gd, dv = H // 2, G // 2, 2 * hd
        qkv = rnd(N, (H + G) * hd + Gd * dv).to(bf)
        q, kx, v = qkv[:, :H * hd], qkv[:, H * hd:(H + G) * hd], qkv[:, (H + G) * hd:]
        kpool = torch.zeros(n_pages, G, PAGE, hd, device=dev, dtype=bf)
        vpool = torch.zeros(n_pages, Gd, PAGE, dv, device=dev, dtype=bf)
        hg = (1 + 0.1 * rnd(hd)).to(bf)
        inv_freq = (10000.0 ** (-2.0 * torch.arange(hd // 4, dtype=torch.float64) / (hd // 2))).to(dev)
        # Kipezen's like kernels work on H heads of 64 over G key heads, keys and values of 64
        qkv_k = rnd(N, (H + 2 * G) * hd).to(bf)
        q_k, k_k, v_k = qkv_k[:, :H * hd], qkv_k[:, H * hd:(H + G) * hd], qkv_k[:, (H + G) * hd:]
        kpool_k, vpool_k = torch.zeros(n_pages, G, PAGE, hd, device=dev, dtype=bf), torch.zeros(n_pages, G, PAGE, hd, device=dev, dtype=bf)
        qb, kb, vb = rnd(H * hd).to(bf), rnd(G * hd).to(bf), rnd(G * hd).to(bf)
        qg, kg = (1 + 0.1 * rnd(H * hd)).to(bf), (1 + 0.1 * rnd(G * hd)).to(bf)
        like_prepare = timed(lambda: kernels.rownorm_rotate_write(q_k, k_k, v_k, qb, kb, vb, qg, kg, 1e-5, inv_freq, hd // 2, ctx_p.positions,
                                                                  ctx_p.kv[0].slot_mapping, kpool_k, vpool_k, H, G, hd, hd, PAGE))
        add("map norms + rotation in halves + cache write (differential)", "biases + whole-row norm + pair rotation + cache write",
            timed(lambda: kernels.head_prepare(q, H, hd, kx, G, hd, ctx_p.positions, ctx_p.kv[0].slot_mapping, kpool, PAGE, q_gain=hg,
                                               q_norm_dims=hd, k_gain=hg, k_norm_dims=hd, eps=1e-5, inv_freq=inv_freq, rot_dims=hd // 2,
                                               v=v, vpool=vpool, n_v_heads=Gd, v_head_dim=dv)),
            like_prepare, N * ((H + G) * hd * 2 + Gd * dv) * 2 * 1.0 + N * G * hd * 2, N * (H + 2 * G) * hd * 2 * 2)
        kpz = _kipezen_configs(size)[0]
        spec_k = kpz.model_spec().layers[3].mixer.branches[0]
        tensors = {n: ((1 + 0.1 * rnd(*e.shape)) if e.init == "gain" else rnd(*e.shape) * 0.1).to(bf)
                   for n, e in PagedAttention.expected_tensors(spec_k).items()}
        att_k = PagedAttention(spec_k, tensors, rt)
        view_k = CacheView("kv", 0, kpool_k, vpool_k, None, True)
        out_k = torch.empty(N, H * hd, device=dev, dtype=bf)
        like_att = lambda ctx, n: att_k._attend(q_k[:n], out_k[:n], view_k, ctx, ctx.kv[0], head_scale=att_k.head_scale)
        window = 1024
        pairs_all = N * (N + 1) // 2
        pairs_k = pairs_all - (N - window) * (N - window + 1) // 2 + 4 * (N - window - 4)
        like_prompt, like_decode = timed(lambda: like_att(ctx_p, N), reps=5), timed(lambda: like_att(ctx_d, B))
        like_prompt_flops, like_decode_bytes = 4 * H * hd * pairs_k, B * (window + 4) * G * hd * 2 * 2
        maps = torch.empty(N, H * dv, device=dev, dtype=bf)
        diff_att = lambda ctx, n: attend_float32(q[:n], maps[:n], kpool, vpool, ctx, ctx.kv[0], H, G, hd, dv, hd ** -0.5, FOVUNEX_CHUNK,
                                                  n_v_heads=Gd)
        pairs_c = (N // FOVUNEX_CHUNK) * FOVUNEX_CHUNK * (FOVUNEX_CHUNK + 1) // 2
        add("attention, prompt (two maps a head, chunks of 1,024, float32 scores)", "attention, prompt (window of 1,024 + 4 kept keys)",
            timed(lambda: diff_att(ctx_p, N), reps=5), like_prompt, flops=2 * H * (hd + dv) * pairs_c, flops_like=like_prompt_flops)
        add("attention, decode b8 x 2,048 keys (two maps a head, 1,024 visible)", "attention, decode (1,028 visible)",
            timed(lambda: diff_att(ctx_d, B)), like_decode, B * FOVUNEX_CHUNK * (G * hd + Gd * dv) * 2, like_decode_bytes)
        gate_, dout = rnd(N, Hd * dv).to(bf), torch.empty(N, Hd * dv, device=dev, dtype=bf)
        add("maps' difference + head norm + output gate", "silu_mul",
            timed(lambda: kernels.diff_combine(maps, gate_, dout, Hd, Gd, dv, 0.7, 1e-5, 0.2)), rows[1]["like_ms"],
            N * Hd * dv * (2 * 2 + 2 + 2), N * inter * 6)
        # latent attention: H heads of 64 + 64 rotated over one cached row of 192 + 64 a token
        kr, r = FOVUNEX_RANK, FOVUNEX_ROT
        qd, rd = hd + r, kr + r
        ql, row = rnd(N, H * qd).to(bf), rnd(N, rd).to(bf)
        lpool = torch.zeros(n_pages, 1, PAGE, rd, device=dev, dtype=bf)
        lg = (1 + 0.1 * rnd(kr)).to(bf)
        inv_l = (10000.0 ** (-2.0 * torch.arange(r // 2, dtype=torch.float64) / r)).to(dev)
        add("compressed-row norm + rotation of neighbours + cache write (latent)", "biases + whole-row norm + pair rotation + cache write",
            timed(lambda: kernels.head_prepare(ql, H, qd, row, 1, rd, ctx_p.positions, ctx_p.kv[0].slot_mapping, lpool, PAGE, k_gain=lg,
                                               k_norm_dims=kr, eps=1e-5, inv_freq=inv_l, rot_dims=r, q_rot_off=hd, k_rot_off=kr,
                                               neighbours=True, mult=1.1)),
            like_prepare, N * (H * qd * 2 + rd * 2) * 2, N * (H + 2 * G) * hd * 2 * 2)
        absorb, qc = (rnd(H, qd, rd) * 0.1).to(bf), torch.empty(N, H * rd, device=dev, dtype=bf)
        ag, gts = rnd(W // 256, 256, 256).to(bf), torch.empty(N, W, device=dev)
        like_hg = timed(lambda: kernels.gemm_simt_batched(u, ag, gts))
        from inf_engine_b200.parts.latent import heads_product
        like_tf = 2 * N * W * 256 / (like_hg * 1e-3) / 1e12
        expand, mixed, heads = (rnd(H, kr, hd) * 0.1).to(bf), torch.empty(N, H * kr, device=dev, dtype=bf), torch.empty(N, H * hd, device=dev, dtype=bf)
        for what, run, flops_row in (
                ("queries into the compressed space, a product a head", lambda n, f: f(ql[:n], qd, absorb, qc[:n], rd), 2 * H * qd * rd),
                ("values out of the compressed space, a product a head", lambda n, f: f(mixed[:n], kr, expand, heads[:n], hd), 2 * H * kr * hd)):
            # a prompt portion: the library's batched product on tensor cores; decode tokens: this package's kernel
            rec = {"kernel": what + ", prompt (library batched product)", "like": "block-diagonal gate product, prompt (float32 on CUDA cores)",
                   "ms": timed(lambda: run(N, heads_product)), "like_ms": like_hg, "like_tflops_f32": like_tf}
            rec["tflops"] = N * flops_row / (rec["ms"] * 1e-3) / 1e12
            rec["frac_of_bf16"] = rec["tflops"] / pk["bf16_tflops"]
            rows.append(rec)
            rec = {"kernel": what + ", prompt, this package's kernel (float32 on CUDA cores; what the 32-bit path runs)", "like": rec["like"],
                   "ms": timed(lambda: run(N, kernels.heads_gemm)), "like_ms": like_hg, "like_tflops_f32": like_tf}
            rec["tflops_f32"] = N * flops_row / (rec["ms"] * 1e-3) / 1e12
            rows.append(rec)
            ms = timed(lambda: run(B, heads_product))
            rows.append({"kernel": what + ", decode b8", "like": "none", "ms": ms, "like_ms": 0.0,
                         "frac_of_hbm": H * (flops_row // (2 * H)) * 2 / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]})
        lat_att = lambda ctx, n: attend_float32(qc[:n], mixed[:n], lpool, lpool, ctx, ctx.kv[0], H, 1, rd, kr, qd ** -0.5, None,
                                                n_v_heads=1, v_row=rd)
        add("attention, prompt (latent: %d heads over one row of %d, every key)" % (H, rd), "attention, prompt (window of 1,024 + 4 kept keys)",
            timed(lambda: lat_att(ctx_p, N), reps=5), like_prompt, flops=2 * H * (rd + kr) * pairs_all, flops_like=like_prompt_flops)
        add("attention, decode b8 x 2,048 keys (latent)", "attention, decode (1,028 visible)",
            timed(lambda: lat_att(ctx_d, B)), like_decode, B * N * rd * 2, like_decode_bytes)
        return rows

    def gavatar_kernel_table(size):
        """Every kernel that the Gavatar family added, alone, beside the like kernel of the closest family (Kipezen), at
        2,048 tokens of one request and at 8 requests of one token over 2,048 keys."""
        from inf_engine_b200.engine.batch import KVGroupContext, StepContext
        from inf_engine_b200.parts import CacheView, Runtime
        from inf_engine_b200.parts.attention import PagedAttention
        from inf_engine_b200.parts.latent import attend_float32, heads_product
        z = FAMILY_SIZES[size]
        W, H, G, hd, inter = z["width"], z["heads"], z["kv"], FAMILY_HD, z["inter"]
        N, B, dev, bf = PROMPT_LEN, 8, "cuda", torch.bfloat16
        g = torch.Generator(device=dev).manual_seed(1)
        rnd = lambda *shape: (torch.randn(*shape, device=dev, generator=g) * 0.5)
        i32 = lambda v: torch.as_tensor(v, dtype=torch.int32, device=dev)
        rows = []

        def add(name, like, ms, ms_like, nbytes=None, nbytes_like=None, flops=None, flops_like=None, note=None):
            rec = {"kernel": name, "like": like, "ms": ms, "like_ms": ms_like}
            if nbytes is not None:
                rec["frac_of_hbm"] = nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]
                if ms_like:
                    rec["like_frac_of_hbm"] = (nbytes_like or nbytes) / (ms_like * 1e-3) / 1e9 / pk["hbm_gbs"]
            if flops is not None:
                rec["frac_of_bf16"] = flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"]
                if ms_like:
                    rec["like_frac_of_bf16"] = (flops_like or flops) / (ms_like * 1e-3) / 1e12 / pk["bf16_tflops"]
            if note:
                rec["note"] = note
            rows.append(rec)

        rt = Runtime(dev, bf)
        n_pages = B * N // PAGE
        qs1, sl1 = i32([0, N]), i32([0])
        qs8, sl8 = torch.arange(B + 1, dtype=torch.int32, device=dev), torch.arange(B, dtype=torch.int32, device=dev)

        def context(q_lens, before):
            ctx = StepContext(rt, PAGE)
            R, n = len(q_lens), sum(q_lens)
            ctx.n_tokens, ctx.n_requests, ctx.n_logits = n, R, 0
            starts = [0]
            for ql in q_lens:
                starts.append(starts[-1] + ql)
            per = n_pages // R
            ctx.q_start, ctx.ctx_before = i32(starts), i32(before)
            ctx.positions = i32([b + t for ql, b in zip(q_lens, before) for t in range(ql)])
            ctx.slots = i32(list(range(R)))
            table_ = torch.arange(per * R, dtype=torch.int32, device=dev).view(R, per)
            sm = i32([(r * per + (b + t) // PAGE) * PAGE + (b + t) % PAGE for r, (ql, b) in enumerate(zip(q_lens, before)) for t in range(ql)])
            ctx.kv = [KVGroupContext(sm, table_)]
            ctx.host = {"q_lens": list(q_lens), "ctx_before": list(before), "q_start": starts}
            ctx.max_q_len, ctx.max_seq_len = max(q_lens), max(b + ql for ql, b in zip(q_lens, before))
            ctx.keys_cap = ctx.max_seq_len
            return ctx

        ctx_p, ctx_d = context([N], [0]), context([1] * B, [N - 1] * B)
        window = GAVATAR_WINDOW
        pairs_all = N * (N + 1) // 2
        pairs_w = pairs_all - (N - window) * (N - window + 1) // 2
        # elementwise passes of the stream | the like passes of the closest families
        res, y = rnd(N, W), rnd(N, W).to(bf)
        nxt, gain = torch.empty(N, W, device=dev, dtype=bf), (1 + 0.1 * rnd(W))
        silu_in, silu_out = rnd(N, 2 * W).to(bf), torch.empty(N, W, device=dev, dtype=bf)
        like_silu = timed(lambda: kernels.silu_mul(silu_in, silu_out, interleaved=True))
        add("scaled embedding + sinusoidal position vector", "scale of the embedding (Fovunex)",
            timed(lambda: kernels.scale_add_sinusoid(res, ctx_p.positions, 1.0, 10000.0)), timed(lambda: kernels.scale_rows(res, 1.0)),
            N * W * 8, N * W * 8)
        h_in, h_out, mu, last = rnd(N, W).to(bf), torch.empty(N, W, device=dev, dtype=bf), rnd(W).to(bf), torch.zeros(16, W, device=dev, dtype=bf)
        add("token shift of the mixer's input, prompt", "silu_mul over rows of the same width",
            timed(lambda: kernels.token_shift(h_in, h_out, mu, last, qs1, i32([0]), sl1, 1)), like_silu, N * W * 6, N * W * 6)
        add("token shift of the mixer's input, decode b8", "silu_mul, 8 rows",
            timed(lambda: kernels.token_shift(h_in[:B], h_out[:B], mu, last, qs8, i32([N - 1] * B), sl8, B)),
            timed(lambda: kernels.silu_mul(silu_in[:B], silu_out[:B], interleaved=True)), B * W * 8, B * W * 6)
        add("norm of a sublayer's output into the residual (the block's second norm)", "the same kernel in Kipezen",
            timed(lambda: kernels.outnorm_accumulate(res, y, gain, 1e-5, None)), timed(lambda: kernels.outnorm_accumulate(res, y, gain, 1e-5, nxt)),
            N * W * (4 + 4 + 2), N * W * (4 + 4 + 2 + 2))
        # attention with mixed heads: biases, head norms of q, k and v, cache write | Kipezen's prepare kernel
        qkv = rnd(N, (H + 2 * G) * hd).to(bf)
        q, kx, v = qkv[:, :H * hd], qkv[:, H * hd:(H + G) * hd], qkv[:, (H + G) * hd:]
        kpool = torch.zeros(n_pages, G, PAGE, hd, device=dev, dtype=bf)
        vpool = torch.zeros(n_pages, 1, PAGE, G * hd, device=dev, dtype=bf)
        vpool_k = torch.zeros(n_pages, G, PAGE, hd, device=dev, dtype=bf)
        qb, kb, vb = rnd(H * hd).to(bf), rnd(G * hd).to(bf), rnd(G * hd).to(bf)
        qg, kg = (1 + 0.1 * rnd(H * hd)).to(bf), (1 + 0.1 * rnd(G * hd)).to(bf)
        inv_freq = (10000.0 ** (-2.0 * torch.arange(hd // 4, dtype=torch.float64) / (hd // 2))).to(dev)
        like_prepare = timed(lambda: kernels.rownorm_rotate_write(q, kx, v, qb, kb, vb, qg, kg, 1e-5, inv_freq, hd // 2, ctx_p.positions,
                                                                  ctx_p.kv[0].slot_mapping, kpool, vpool_k, H, G, hd, hd, PAGE))
        add("biases + head norms of q, k and v + cache write", "biases + whole-row norm + pair rotation + cache write",
            timed(lambda: kernels.qkv_prepare(q, H, kx, G, hd, v, G, hd, ctx_p.kv[0].slot_mapping, kpool, vpool, PAGE, 1e-5, q_bias=qb,
                                              k_bias=kb, v_bias=vb, q_norm=True, k_norm=True, v_norm=True, pool_v_heads=1)),
            like_prepare, N * (H + 2 * G) * hd * 2 * 2, N * (H + 2 * G) * hd * 2 * 2)
        kpz = _kipezen_configs(size)[0]
        spec_k = kpz.model_spec().layers[3].mixer.branches[0]
        tensors = {n: ((1 + 0.1 * rnd(*e.shape)) if e.init == "gain" else rnd(*e.shape) * 0.1).to(bf)
                   for n, e in PagedAttention.expected_tensors(spec_k).items()}
        att_k = PagedAttention(spec_k, tensors, rt)
        view_k = CacheView("kv", 0, kpool, vpool_k, None, True)
        out_k = torch.empty(N, H * hd, device=dev, dtype=bf)
        like_att = lambda ctx, n: att_k._attend(q[:n], out_k[:n], view_k, ctx, ctx.kv[0], head_scale=att_k.head_scale)
        pairs_k = pairs_w + 4 * (N - window - 4)
        like_prompt, like_decode = timed(lambda: like_att(ctx_p, N), reps=5), timed(lambda: like_att(ctx_d, B))
        like_prompt_flops, like_decode_bytes = 4 * H * hd * pairs_k, B * (window + 4) * G * hd * 2 * 2
        slice_heads = max(1, min(G, 256 // hd))
        values = vpool.view(n_pages, PAGE, G * hd)
        talk, gate_ = rnd(H, H), rnd(N, H * hd).to(bf)
        unmixed, tout = torch.empty(N, H * slice_heads * hd, device=dev, dtype=bf), torch.empty(N, H * hd, device=dev, dtype=bf)

        def talking(ctx, n, combine=True):
            for c0 in range(0, G, slice_heads):
                nc = min(slice_heads, G - c0)
                attend_float32(q[:n], unmixed[:n, :H * nc * hd], kpool, values[:, :, c0 * hd:], ctx, ctx.kv[0], H, G, hd, nc * hd, 0.125,
                               None, n_v_heads=1, v_row=G * hd, window=window)
                if combine:
                    kernels.talk_combine(unmixed[:n, :H * nc * hd], talk, gate_[:n], tout[:n], H, G, hd, first_v_head=c0, slice_v_heads=nc)
        # what the mechanism asks for: scores and weights of every head at every pair, the H x H mix, one value head a head
        useful = 2 * H * (2 * hd + H) * pairs_w
        add("attention with weights mixed across heads, prompt (window 1,024; every head over all value heads, then the mix)",
            "attention, prompt (window of 1,024 + 4 kept keys)", timed(lambda: talking(ctx_p, N), reps=5), like_prompt,
            flops=useful, flops_like=like_prompt_flops,
            note="useful FLOPs (scores, the mix, one value head a head); the launches do %.1f times that: every head meets all %d value heads"
                 % (2 * H * (-(-G // slice_heads) * hd + G * hd) * pairs_w / useful, G))
        add("attention with weights mixed across heads, decode b8 x 2,048 keys (1,024 visible)", "attention, decode (1,028 visible)",
            timed(lambda: talking(ctx_d, B)), like_decode, B * window * 2 * G * hd * 2, like_decode_bytes)
        add("mix of the heads' results + output gate (one launch a slice of value heads)", "silu_mul",
            timed(lambda: kernels.talk_combine(unmixed, talk, gate_, tout, H, G, hd, first_v_head=0, slice_v_heads=slice_heads)), like_silu,
            N * (H * slice_heads * hd + 2 * H * hd // (G // slice_heads)) * 2, N * W * 6)
        # latent attention with a sink under a window | Kipezen's windowed attention
        kr = GAVATAR_RANK
        cq, row = rnd(N, W // 2).to(bf), rnd(N, kr).to(bf)
        lpool = torch.zeros(n_pages, 1, PAGE, kr, device=dev, dtype=bf)
        cg, lg = (1 + 0.1 * rnd(W // 2)).to(bf), (1 + 0.1 * rnd(kr)).to(bf)
        add("norms of both compressed vectors + cache write (latent)", "biases + whole-row norm + pair rotation + cache write",
            timed(lambda: kernels.head_prepare(cq, 1, W // 2, row, 1, kr, ctx_p.positions, ctx_p.kv[0].slot_mapping, lpool, PAGE, q_gain=cg,
                                               q_norm_dims=W // 2, k_gain=lg, k_norm_dims=kr, eps=1e-5)),
            like_prepare, N * (W // 2 * 2 + kr * 2) * 2, N * (H + 2 * G) * hd * 2 * 2)
        ql, qc = rnd(N, H * hd).to(bf), torch.empty(N, H * kr, device=dev, dtype=bf)
        mixed, heads = torch.empty(N, H * kr, device=dev, dtype=bf), torch.empty(N, H * hd, device=dev, dtype=bf)
        sink = rnd(H)
        lat_att = lambda ctx, n: attend_float32(qc[:n], mixed[:n], lpool, lpool, ctx, ctx.kv[0], H, 1, kr, kr, hd ** -0.5, None,
                                                n_v_heads=1, v_row=kr, window=window, sink=sink)
        add("attention, prompt (latent: %d heads over one row of %d, window 1,024, a sink)" % (H, kr),
            "attention, prompt (window of 1,024 + 4 kept keys)", timed(lambda: lat_att(ctx_p, N), reps=5), like_prompt,
            flops=2 * H * 2 * kr * pairs_w, flops_like=like_prompt_flops)
        add("attention, decode b8 x 2,048 keys (latent, 1,024 visible)", "attention, decode (1,028 visible)",
            timed(lambda: lat_att(ctx_d, B)), like_decode, B * window * kr * 2, like_decode_bytes)
        hgate = rnd(N, H).to(bf)
        add("a head's output times sigmoid of its gate", "silu_mul", timed(lambda: kernels.gate_mul(heads, hgate, group=hd)), like_silu,
            N * H * hd * 4, N * W * 6)
        # the matrix memory | the gated delta rule of Kipezen (the same head geometry: a float32 matrix of 64 x 64 a head)
        Wd = H * hd
        proj = rnd(N, 4 * Wd).to(bf)
        mq, mk, mv, mg = (proj[:, i * Wd:(i + 1) * Wd] for i in range(4))
        zg, ib, fb = rnd(N, 2 * H) * 3, rnd(H).to(bf), (3 + rnd(H)).to(bf)
        words = kernels.mlstm_state_floats(hd, hd)
        mst, mo = torch.zeros(16, H, words, device=dev), torch.empty(N, Wd, device=dev)
        run_mm = lambda n, qs, sl, R: kernels.mlstm_scan(mq[:n], mk[:n], mv[:n], zg[:n], ib, fb, 15.0, mst, mo[:n], qs, sl, R, H, hd, hd)
        b_pre, a_pre = rnd(N, H).to(bf), rnd(N, H).to(bf)
        a_log, dt_b, og = rnd(H).to(bf), rnd(H).to(bf), (1 + 0.1 * rnd(hd)).to(bf)
        gst, gmixed = torch.zeros(16, H, hd, hd, device=dev), torch.empty(N, Wd, device=dev, dtype=bf)
        run_gd = lambda n, qs, sl, R: kernels.gated_delta(mq[:n, :G * hd], mk[:n, :G * hd], mv[:n], b_pre[:n], a_pre[:n], mg[:n], a_log, dt_b,
                                                          og, gst, gmixed[:n], qs, sl, R, H, G, hd, hd, 1e-6, 1e-5)
        add("matrix memory, prompt of 2,048 tokens (one request)", "gated delta rule, prompt",
            timed(lambda: run_mm(N, qs1, sl1, 1), reps=5), timed(lambda: run_gd(N, qs1, sl1, 1), reps=5),
            N * (3 * Wd * 2 + Wd * 4) + 2 * H * words * 4, N * (2 * G * hd + 3 * Wd) * 2 + 2 * H * hd * hd * 4,
            note="a token-by-token scan: the chain of %d dependent steps bounds it, not bytes" % N)
        add("matrix memory, decode b8", "gated delta rule, decode", timed(lambda: run_mm(B, qs8, sl8, B)), timed(lambda: run_gd(B, qs8, sl8, B)),
            B * 2 * H * words * 4, B * 2 * H * hd * hd * 4)
        ogain = (1 + 0.1 * rnd(Wd)).to(bf)
        add("matrix memory: head norm, gain and output gate", "silu_mul", timed(lambda: kernels.mlstm_finish(mo, ogain, mg, gmixed, H, hd, 1e-5)),
            like_silu, N * Wd * (4 + 2 + 2), N * W * 6)
        # the router of the largest logits | Kipezen's router (sigmoid scores in groups)
        E = 16
        logits = rnd(N, E + 1) * 2
        rb = rnd(E)
        ids4, wts4 = torch.empty(N, 4, dtype=torch.int32, device=dev), torch.empty(N, 4, device=dev)
        ids2, wts2, gt = torch.empty(N, 2, dtype=torch.int32, device=dev), torch.empty(N, 2, device=dev), torch.empty(N, device=dev)
        add("router: 4 largest of 16 logits, softmax over the chosen", "router: sigmoid scores, 2 of 16 from 2 of 4 groups",
            timed(lambda: kernels.moe_route(logits[:, :E], rb, ids4, wts4, None, E, 4, 1, 1, 1.0, 0.0, score="softmax_top")),
            timed(lambda: kernels.moe_route(logits, None, ids2, wts2, gt, E, 2, 4, 2, 2.5, 1e-20, gate_col=E)),
            N * (E * 4 + 4 * 8), N * (E * 4 + 2 * 8 + 4))
        return rows

    sizes = {}
    if args.family in ("kipezen", "fovunex", "gavatar") and args.family_step:
        # one step launched kernel by kernel (no graphs) between cudaProfilerStart / Stop, for a launch list:
        #   ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off --csv --log-file L \
        #       python bench.py --family kipezen --family-sizes w2048 --family-step decode
        import tempfile
        from inf_engine_b200 import ModelRunner
        from inf_engine_b200.weights import write_random_model
        size = (args.family_sizes or "w2048").split(",")[0]
        kpz, _ = {"kipezen": _kipezen_configs, "fovunex": _fovunex_configs, "gavatar": _gavatar_configs}[args.family](size)
        with tempfile.TemporaryDirectory() as tmp:
            write_random_model(kpz, args.seed, tmp)
            r = ModelRunner.from_dir(tmp, dtype="bfloat16", page_size=PAGE, n_pages=(args.batch + 1) * POOL_CONTEXT // PAGE,
                                     max_requests=max(16, args.batch), use_graphs=False)
        V = r.spec.vocab_size
        rids = [f"d{i}" for i in range(args.batch)]
        for rid in rids:
            r.open(rid)
        for i in range(0, args.batch, 4):
            r.step([StepEntry(x, rng.integers(0, V, PROMPT_LEN).tolist(), []) for x in rids[i:i + 4]])
        for _ in range(2):
            r.step([StepEntry(x, [5], [0]) for x in rids])
        r.open("p")
        r.step([StepEntry("p", rng.integers(0, V, PROMPT_LEN).tolist(), [PROMPT_LEN - 1])])
        r.close("p")
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStart()
        if args.family_step == "decode":
            r.step([StepEntry(x, [7], [0]) for x in rids])
        else:
            r.open("p")
            r.step([StepEntry("p", rng.integers(0, V, PROMPT_LEN).tolist(), [PROMPT_LEN - 1])])
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
        clocks.stop()
        print(json.dumps({"impl": "ours", "family": args.family, "step": args.family_step, "size": size, "launches": kernels.LAUNCHES}))
        return 0
    if args.family == "gavatar":
        for size in (args.family_sizes.split(",") if args.family_sizes else list(FAMILY_SIZES)):
            gav, kpz = _gavatar_configs(size)
            rec = {"gavatar": model_numbers_of(gav, args.batch), "kipezen": model_numbers_of(kpz, args.batch)}
            rec["kernels"] = gavatar_kernel_table(size)
            sizes[size] = rec
        clocks.stop()
        print(json.dumps({"impl": "ours", "family": "gavatar", "dtype": "bf16", "n_gpus": 1, "steps": args.steps,
                          "warmup": max(args.warmup, 3),
                          "data": "synthetic: seeded random weights, uniform random prompt ids",
                          "config": {"layers": FAMILY_LAYERS, "pattern": "matrix memory, attention with mixed heads, matrix memory, latent attention",
                                     "vocab": FAMILY_VOCAB, "head_dim": FAMILY_HD, "prompt": PROMPT_LEN, "decode_batch": args.batch,
                                     "page_size": PAGE, "window": GAVATAR_WINDOW, "kv_rank": GAVATAR_RANK,
                                     "experts": "16, 4 a token",
                                     "l2": "a 256 MB buffer is written before every timed kernel; model steps stream their weights",
                                     "sizes": FAMILY_SIZES},
                          "peaks": pk, "sizes": sizes, "clocks": clocks.summary(t_all0, time.perf_counter())}))
        return 0
    if args.family == "fovunex":
        for size in (args.family_sizes.split(",") if args.family_sizes else list(FAMILY_SIZES)):
            fvx, kpz = _fovunex_configs(size)
            rec = {"fovunex": model_numbers_of(fvx, args.batch), "kipezen": model_numbers_of(kpz, args.batch)}
            rec["kernels"] = fovunex_kernel_table(size)
            sizes[size] = rec
        clocks.stop()
        print(json.dumps({"impl": "ours", "family": "fovunex", "dtype": "bf16", "n_gpus": 1, "steps": args.steps,
                          "warmup": max(args.warmup, 3),
                          "data": "synthetic: seeded random weights, uniform random prompt ids",
                          "config": {"layers": FAMILY_LAYERS, "pattern": "minGRU, differential attention, minGRU, latent attention",
                                     "vocab": FAMILY_VOCAB, "head_dim": FAMILY_HD, "prompt": PROMPT_LEN, "decode_batch": args.batch,
                                     "page_size": PAGE, "chunk": FOVUNEX_CHUNK, "kv_rank": FOVUNEX_RANK, "rot_dim": FOVUNEX_ROT,
                                     "l2": "a 256 MB buffer is written before every timed kernel; model steps stream their weights",
                                     "sizes": FAMILY_SIZES},
                          "peaks": pk, "sizes": sizes, "clocks": clocks.summary(t_all0, time.perf_counter())}))
        return 0
    if args.family == "kipezen":
        for size in (args.family_sizes.split(",") if args.family_sizes else list(FAMILY_SIZES)):
            kpz, brx = _kipezen_configs(size)
            rec = {"kipezen": model_numbers_of(kpz, args.batch), "barerax": model_numbers_of(brx, args.batch)}
            rec["kernels"] = kipezen_kernel_table(size)
            sizes[size] = rec
        clocks.stop()
        print(json.dumps({"impl": "ours", "family": "kipezen", "dtype": "bf16", "n_gpus": 1, "steps": args.steps,
                          "warmup": max(args.warmup, 3),
                          "data": "synthetic: seeded random weights, uniform random prompt ids",
                          "config": {"layers": FAMILY_LAYERS, "pattern": "delta, delta, delta, parallel", "vocab": FAMILY_VOCAB,
                                     "head_dim": FAMILY_HD, "prompt": PROMPT_LEN, "decode_batch": args.batch, "page_size": PAGE,
                                     "experts": "16, 2 a token from 2 of 4 groups, and a shared one",
                                     "l2": "a 256 MB buffer is written before every timed kernel; model steps stream their weights",
                                     "sizes": FAMILY_SIZES},
                          "peaks": pk, "sizes": sizes, "clocks": clocks.summary(t_all0, time.perf_counter())}))
        return 0
    for size in (args.family_sizes.split(",") if args.family_sizes else list(FAMILY_SIZES)):
        brx, llama = _family_configs(size)
        rec = {"barerax": model_numbers_of(brx, args.batch), "llama": model_numbers_of(llama, args.batch)}
        rec["kernels"] = kernel_table(size)
        sizes[size] = rec
    clocks.stop()
    print(json.dumps({"impl": "ours", "family": "barerax", "dtype": "bf16", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3),
                      "data": "synthetic: seeded random weights, uniform random prompt ids",
                      "config": {"layers": FAMILY_LAYERS, "pattern": "delta, delta, delta, attention", "vocab": FAMILY_VOCAB,
                                 "head_dim": FAMILY_HD, "prompt": PROMPT_LEN, "decode_batch": args.batch, "page_size": PAGE,
                                 "l2": "a 256 MB buffer is written before every timed kernel; model steps stream their weights",
                                 "sizes": FAMILY_SIZES},
                      "peaks": pk, "sizes": sizes, "clocks": clocks.summary(t_all0, time.perf_counter())}))
    return 0


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _reference_package():
    """The reference's ``engine`` package, unmodified, under ``baseline/_ref`` (git-ignored).  It has no setup.py or
    pyproject.toml, so ``pip install --target baseline/_ref`` refuses it; it is pure Python over torch and runs from a
    plain copy of its folder, which is made here when a checkout of the reference lies beside this repository."""
    if not os.path.isfile(os.path.join(REF_DIR, "engine", "llama_paged_engine.py")):
        src = os.environ.get("INF_ENGINE_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
        if not os.path.isfile(os.path.join(src, "engine", "llama_paged_engine.py")):
            return f"no copy of the reference's engine package under baseline/_ref and no checkout at {src}"
        import shutil
        os.makedirs(REF_DIR, exist_ok=True)
        shutil.copytree(os.path.join(src, "engine"), os.path.join(REF_DIR, "engine"))
    return None


def run_reference(args):
    """The reference arm: the UNMODIFIED reference (``baseline/_ref/engine``) through its own public API and stock
    path: ``LlamaModel`` over a ``LlamaWeights`` dictionary of seeded random bfloat16 tensors (built as its own
    tests build one, tests/test_paged_cache.py:42-72) at its ``LLAMA_3_2_1B`` preset (engine/config.py:77-89),
    ``LlamaPagedEngine(model, n_total_blocks, block_size)`` with its defaults (engine/llama_paged_engine.py:129-166),
    prompts through ``submit`` and ``step`` (:169-174, :418-442).  Nothing of this repository's package is imported in
    this process.  Same metric, batch, prompt length, pool and page size as the other arm."""
    why = _reference_package()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    sys.path.insert(0, REF_DIR)
    try:
        import numpy as np
        import torch
        from engine.config import LLAMA_3_2_1B, LLAMA_3_2_3B, SMOLLM2_1_7B
        from engine.llama_model import LlamaModel
        from engine.llama_paged_engine import LlamaPagedEngine, LlamaRequest
        from engine.llama_weights import LlamaWeights
    except Exception as e:                                   # noqa: BLE001 - whatever keeps it from importing
        print(json.dumps({"impl": "reference", "unavailable": f"the reference does not import here: {e!r}"[:300]}))
        return 0
    presets = {"llama-3.2-1b": LLAMA_3_2_1B, "llama-3.2-3b": LLAMA_3_2_3B, "smollm2-1.7b": SMOLLM2_1_7B}
    if args.model not in presets:
        print(json.dumps({"impl": "reference", "unavailable": f"the reference has no preset for {args.model}"}))
        return 0
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device"}))
        return 0
    cfg = presets[args.model]
    n_layers_full = cfg.n_layer
    if args.layers:
        import dataclasses
        cfg = dataclasses.replace(cfg, n_layer=args.layers)
    pk = peaks()
    dev = "cuda:0"
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev).manual_seed(args.seed)
    d, hq, hk, f, V = cfg.d_model, cfg.n_head * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim, cfg.intermediate_size, cfg.vocab_size

    def mat(*shape):
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    def gain():
        return (1.0 + (torch.rand(d, generator=g, device=dev) * 0.2 - 0.1)).to(torch.bfloat16)

    tensors = {"model.embed_tokens.weight": mat(V, d), "model.norm.weight": gain()}
    for i in range(cfg.n_layer):
        p = f"model.layers.{i}."
        tensors.update({p + "input_layernorm.weight": gain(), p + "post_attention_layernorm.weight": gain(),
                        p + "self_attn.q_proj.weight": mat(hq, d), p + "self_attn.k_proj.weight": mat(hk, d),
                        p + "self_attn.v_proj.weight": mat(hk, d), p + "self_attn.o_proj.weight": mat(d, hq),
                        p + "mlp.gate_proj.weight": mat(f, d), p + "mlp.up_proj.weight": mat(f, d),
                        p + "mlp.down_proj.weight": mat(d, f)})
    if not cfg.tie_word_embeddings:
        tensors["lm_head.weight"] = mat(V, d)
    model = LlamaModel(LlamaWeights(tensors, cfg), cfg)
    engine = LlamaPagedEngine(model, n_total_blocks=args.pool_requests * POOL_CONTEXT // PAGE, block_size=PAGE)
    rng = np.random.default_rng(args.seed)
    clocks = ClockSampler()
    clocks.start()

    def prompt():
        return rng.integers(0, V, PROMPT_LEN).tolist()

    # prefill: one 2,048-token request that is done after its first token, so step() is its prefill and nothing else
    def prefill_once():
        engine.submit(LlamaRequest(req_id=-1, prompt_ids=prompt(), max_new_tokens=1))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step()
        e1.record()
        torch.cuda.synchronize()
        engine.completed.clear()
        return e0.elapsed_time(e1)

    for _ in range(3):
        prefill_once()
    pre_ms = sorted(prefill_once() for _ in range(args.prefill_reps))
    pre = pre_ms[len(pre_ms) // 2]
    L, H, hd = cfg.n_layer, cfg.n_head, cfg.head_dim
    linear_params = L * ((hq + 2 * hk) * d + d * hq + 3 * f * d)
    flops = 2 * PROMPT_LEN * linear_params + L * 4 * H * hd * (PROMPT_LEN * (PROMPT_LEN + 1) // 2) + 2 * V * d
    prefill = {"value": PROMPT_LEN / pre * 1e3, "unit": "tok/s", "tokens": PROMPT_LEN, "ms": pre,
               "frac": flops / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12), "peak_tflops": pk["bf16_tflops"],
               "peak_source": pk["source"], "note": "flops of the wanted logit row only; the reference computes every row's"}

    def decode(batch, steps, warmup):
        reqs = [LlamaRequest(req_id=i, prompt_ids=prompt(), max_new_tokens=warmup + steps + 8) for i in range(batch)]
        for r in reqs:
            assert engine.submit(r)
        engine.step()                                         # admits and prefills all of them, one decode step
        assert len(engine._active) == batch, "the reference did not admit the whole batch"
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        ctx0 = len(reqs[0].prompt_ids) + len(reqs[0].generated)
        n_before = sum(len(r.generated) for r in reqs)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            engine.step()                                     # reads the sampled ids on the host every step
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        n_tok = sum(len(r.generated) for r in reqs) - n_before
        ms = e0.elapsed_time(e1)
        while engine.has_work:
            engine.step()
        engine.completed.clear()
        return dict(tok_s=n_tok / ms * 1e3, e2e=n_tok / (t1 - t0), ms_per_step=ms / steps, t0=t0, t1=t1,
                    ctx=(ctx0, ctx0 + steps))

    args.warmup = max(args.warmup, 3)
    main = decode(args.batch, args.steps, args.warmup)
    points = {}
    for b in (1, 64):
        if b <= args.pool_requests and not args.no_points:
            # fewer steps: the reference's cache gathers block by block in Python, a second a step at batch 64
            points[f"decode_b{b}"] = decode(b, max(4, args.steps // 16), 3)["tok_s"]
    clocks.stop()
    weight_bytes = 2 * (linear_params + V * d)
    bytes_step = weight_bytes + args.batch * (main["ctx"][0] + args.steps / 2) * (2 * L * hk * 2)
    achieved = bytes_step / (main["ms_per_step"] * 1e-3) / 1e9
    print(json.dumps({
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B size, random weights)", "impl": "reference",
        "value": main["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random prompt ids",
        "config": {"model": args.model, "layers": cfg.n_layer, "layers_of_model": n_layers_full, "hidden": d,
                   "heads": cfg.n_head, "kv_heads": cfg.n_kv_heads, "head_dim": hd, "intermediate": f, "vocab": V,
                   "global_batch": args.batch, "seq_len": PROMPT_LEN, "context_start": main["ctx"][0],
                   "context_end": main["ctx"][1], "pool_context": POOL_CONTEXT, "page_size": PAGE,
                   "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights 2.5 GB per step)",
                   "decode": "the reference's defaults: eager steps, enable_cuda_graphs=False"},
        "e2e": {"value": main["e2e"], "unit": "tok/s", "h2d_bytes_per_step": 8 * args.batch,
                "d2h_bytes_per_step": 8 * args.batch,
                "note": "the reference builds its step tensors from Python lists and reads int64 ids back (.tolist())"},
        "gpu_launches": 0, "launch_note": "library kernels only (torch); none of this repository's",
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"]},
        "points": points, "clocks": clocks.summary(main["t0"], main["t1"]),
    }))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3.2-1b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--prefill-reps", type=int, default=7)
    ap.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                    help="measure one part only (short runs for profiling); the JSON line then lacks the rest")
    ap.add_argument("--pool-requests", type=int, default=64, help="requests of 4,096 tokens the cache pool is made for")
    ap.add_argument("--no-points", action="store_true", help="leave out the batch-1 and batch-64 points")
    ap.add_argument("--no-workloads", action="store_true",
                    help="leave out the two continuous-batching workloads at the other models' sizes")
    ap.add_argument("--family", default=None, metavar="NAME",
                    help="instead of the default workload: prefill and decode of another model family (barerax, kipezen, fovunex, gavatar) at sizes like "
                         "a real model's layers, beside the closest earlier model of equal size, and its kernels beside the like ones")
    ap.add_argument("--family-sizes", default=None, help="comma-separated subset of the family's sizes (w1024,w2048)")
    ap.add_argument("--family-step", default=None, choices=["decode", "prefill"],
                    help="with --family kipezen, fovunex or gavatar: run one such step kernel by kernel between cudaProfilerStart/Stop (for a launch list) and exit")
    ap.add_argument("--workload", default=None, metavar="N:MIN:MAX:NEW[:TEMP]",
                    help="instead of the step measurements: N requests through Engine.run_offline (continuous batching)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.family:
        args.steps = min(args.steps, 64)
        return run_family(args)
    if args.workload:
        return run_workload(args)
    args.warmup = max(args.warmup, 3)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
