#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens/s (headline: batch 8),
prefill tokens/s at 2,048 tokens, decode at batch 1 and 64, each with its
fraction of the measured roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

The model has the layer sizes of the 4B benchmark configuration (the qwen3-4b preset) with random
bfloat16 weights made on the device; prompts are seeded random token ids.  A
"step" is one decode step of the whole batch.  Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from kipp_b200.config.presets import load_preset  # noqa: E402

# the 4B benchmark configuration (Qwen3-4B-shaped): the sizes and the weight seed are the preset's
QWEN3_4B, _INIT_4B = load_preset("qwen3-4b")
WEIGHT_SEED = int(_INIT_4B["seed"])
CONTEXT = 8192            # the 4B benchmark configuration's context length
POINT_PROMPT = 2048       # ... decode at batch 1/8/64 with 2,048-token prompts
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs.  It is
    started before the warm-up (nvidia-smi needs a moment to come up); each sample
    carries nvidia-smi's own timestamp, and only samples between mark_start() and
    mark_end() count.  A timed region shorter than the sampling period may hold
    none: then the samples of the warm-up just before it (the same load) stand
    in, and "window" says so."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int = 0):
        self.proc = None
        self.t_begin = datetime.datetime.now()
        self.t_start = self.t_end = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def mark_start(self) -> None:
        self.t_start = datetime.datetime.now()

    def mark_end(self) -> None:
        self.t_end = datetime.datetime.now()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        samples = []
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                when = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
                samples.append((when, float(parts[1]), float(parts[2]),
                                [n for n, v in zip(self.NAMES, parts[3:7]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        t0, t1 = self.t_start or self.t_begin, self.t_end or datetime.datetime.now()
        window = "timed region"
        chosen = [x for x in samples if t0 <= x[0] <= t1]
        if not chosen:
            window = "warm-up and timed region (the timed region is shorter than the sampling period)"
            chosen = [x for x in samples if self.t_begin <= x[0] <= t1]
        sm = [x[1] for x in chosen]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(x[2] for x in chosen) if chosen else None,
                "reasons": sorted({r for x in chosen for r in x[3]}), "samples": len(chosen), "window": window}


def reference_arm(args) -> int:
    """The reference's own CUDA path on the same workload: see baseline/reference_arm.py."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm as ref
    except Exception as e:                                   # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"baseline/reference_arm.py cannot be imported: {e}"}))
        return 0
    config = QWEN3_4B if args.preset == "qwen3-4b" else load_preset(args.preset)[0]
    return ref.main(args, dict(config), WEIGHT_SEED, POINT_PROMPT, PREFILL_TOKENS)


def median_mad(values: list) -> tuple[float, float]:
    """Median and median absolute deviation (the reference's policy for its own
    benchmark figures, tools/bench.py:260-268)."""
    m = statistics.median(values)
    return m, statistics.median(abs(v - m) for v in values)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None,
                    help="run fewer layers than the configuration has (named in the record)")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64 and the prefill")
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--repeats", type=int, default=5, help="timed runs of --steps steps each; the median counts")
    ap.add_argument("--preset", default="qwen3-4b", help="another preset's sizes (the record names them)")
    ap.add_argument("--own-length-splits", action="store_true",
                    help="decode attention splits from each token's own context only")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from kipp_b200.config import config_from_dict
    from kipp_b200.engine import StepEntry
    from kipp_b200.engine.llm import LLM

    pk, pk_src = peaks()
    cfg = dict(QWEN3_4B if args.preset == "qwen3-4b" else load_preset(args.preset)[0])
    seed = WEIGHT_SEED if args.preset == "qwen3-4b" else int(load_preset(args.preset)[1]["seed"])
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    config = config_from_dict(cfg)
    K, W, B, R = args.steps, args.warmup, args.batch, max(args.repeats, 1)
    span = R * K + W + 2 + 4                 # the timed steps and four more for the kernel shares
    batches = [B] if args.skip_points else sorted({1, 8, B, 64})
    cache_tokens = max([B * (args.context + PAGE)] +
                       [b * (POINT_PROMPT + span + PAGE) for b in batches if b != B])
    llm = LLM(config, dtype="bfloat16", kv_block_size=PAGE, kv_tokens=cache_tokens, ctx=args.context,
              max_requests=max(batches), max_batch_tokens=max(PREFILL_TOKENS, max(batches)),
              chunk=PREFILL_TOKENS, seed=seed, own_length_splits=args.own_length_splits)
    eng = llm.engine
    dev = eng.runtime.device
    stream = eng.stream                      # the engine's stream: the timing events are recorded there
    g = torch.Generator().manual_seed(1234)

    def prompt(n):
        return torch.randint(0, config.vocab_size, (n,), generator=g).tolist()

    weight_bytes = eng.weight_bytes()
    kv_bytes_token = eng.cache_bytes_per_token()

    # ---- prefill of one 2,048-token prompt ------------------------------------------
    prefill = None
    if not args.skip_points:
        toks = prompt(PREFILL_TOKENS)
        # Back to back the 1 kW power cap pulls the clock down after the first few runs
        # (sw_power_cap), so two figures are taken: runs with an idle gap before each
        # (the step as a request meets it: "ms"), and runs back to back ("ms_sustained").
        def prefill_runs(count: int, gap: float, tag: str) -> list:
            out = []
            for i in range(count):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize(dev)
                if gap:
                    time.sleep(gap)
                a.record(stream)
                eng.step([StepEntry((tag, i), toks, [PREFILL_TOKENS - 1])])
                b.record(stream)
                torch.cuda.synchronize(dev)
                eng.finish((tag, i))
                out.append(a.elapsed_time(b))
            return out
        prefill_runs(3, 0.0, "warm")                       # warm-up; the third run is captured as a graph
        times = prefill_runs(R, 0.3, "gap")
        sustained = prefill_runs(R + 3, 0.0, "chain")[3:]
        ms, ms_mad = median_mad(times)
        ms_sus, _ = median_mad(sustained)
        c = config
        gemm_params = c.num_hidden_layers * (c.hidden_size * (c.q_dim + 2 * c.kv_dim) +
                                             c.q_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
        T = PREFILL_TOKENS
        flops = 2.0 * T * gemm_params + 2.0 * c.hidden_size * c.vocab_size \
            + c.num_hidden_layers * 2.0 * T * (T + 1) * c.head_dim * c.num_attention_heads
        prefill = {"value": round(T / (ms / 1e3), 1), "tokens": T, "ms": round(ms, 3), "ms_mad": round(ms_mad, 3),
                   "runs": len(times),
                   "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                   "flops": flops, "peak_tflops": pk["bf16_tflops"], "peak_source": pk_src,
                   "ms_sustained": round(ms_sus, 3), "peak_tflops_sustained": pk["bf16_tflops_sustained"],
                   "frac_sustained": round(flops / (ms_sus / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                   "note": "ms: runs with an idle gap before each, against the burst peak; ms_sustained: back to "
                           "back under the power cap, against the sustained peak"}

    # ---- decode ------------------------------------------------------------------------
    def fill(batch: int, context: int, tag: str) -> list:
        """``batch`` live requests holding ``context`` tokens each (real prefill)."""
        rids = [(tag, i) for i in range(batch)]
        for rid in rids:
            toks = prompt(context)
            for a in range(0, context, PREFILL_TOKENS):
                eng.step([StepEntry(rid, toks[a:a + PREFILL_TOKENS], [])])
        return rids

    def decode_run(rids: list, steps: int, warmup: int, repeats: int, sample_clocks: bool):
        """Greedy decode of all ``rids``: ``warmup`` steps, then ``repeats`` timed runs of
        ``steps`` steps each, device-timed on the engine's stream.  The argmax of a step is
        fed to the next one on the device (Engine.decode_burst, which the generation loop
        uses for greedy requests): the host launches and waits for no token.  (The
        end-to-end figure below has the host in every step.)  Returns the median
        milliseconds per step, its median absolute deviation, clocks, kernel launches."""
        next_tokens = prompt(len(rids))
        sampler = ClockSampler() if sample_clocks else None
        ring = eng.decode_burst(rids, next_tokens, warmup)
        next_tokens = ring[-1].tolist()
        torch.cuda.synchronize(dev)
        launches0 = eng.kernel_launches()
        if sampler:
            sampler.mark_start()
        per_step = []
        for _ in range(repeats):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(dev)
            a.record(stream)
            ring = eng.decode_burst(rids, next_tokens, steps)
            b.record(stream)
            torch.cuda.synchronize(dev)
            assert ring.shape[0] == steps and int(ring.min()) >= 0
            next_tokens = ring[-1].tolist()
            per_step.append(a.elapsed_time(b) / steps)
        if sampler:
            sampler.mark_end()
        clocks = sampler.stop() if sampler else None
        ms, mad = median_mad(per_step)
        return ms, mad, clocks, (eng.kernel_launches() - launches0) // repeats

    headline_ctx = args.context - span
    rids = fill(B, headline_ctx, "head")
    ms_step, ms_mad, clocks, launches = decode_run(rids, K, W, R, True)
    ctx_mid = headline_ctx + W + R * K / 2.0
    step_bytes = weight_bytes + B * ctx_mid * kv_bytes_token
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    # Where the step's time goes: four steps without graphs, an event after every launch
    # (Engine.profile_start/stop); shares of the time between the events, by kernel.
    eng.profile_start()
    ring = eng.decode_burst(rids, prompt(len(rids)), 4)
    spent = eng.profile_stop()
    total_spent = sum(spent.values()) or 1.0
    shares = {k: round(v / total_spent, 3) for k, v in sorted(spent.items(), key=lambda kv: -kv[1])[:8]}
    for r in rids:
        eng.finish(r)
    eng.runtime.check_status()

    points = {}
    if not args.skip_points:
        for b in sorted({1, 8, 64}):
            rr = fill(b, POINT_PROMPT, f"p{b}")
            steps_b = min(K, 32)
            ms_b, mad_b, _, _ = decode_run(rr, steps_b, 3, R, False)
            ctx_b = POINT_PROMPT + 3 + R * steps_b / 2.0
            gbs = (weight_bytes + b * ctx_b * kv_bytes_token) / (ms_b / 1e3) / 1e9
            points[f"decode_b{b}"] = round(b / (ms_b / 1e3), 1)
            points[f"decode_b{b}_ms"] = round(ms_b, 4)
            points[f"decode_b{b}_ms_mad"] = round(mad_b, 4)
            points[f"decode_b{b}_hbm_frac"] = round(gbs / pk["hbm_gbs"], 4)
            for r in rr:
                eng.finish(r)

    # ---- end to end through the Python entry point: host token ids in and out --------
    from kipp_b200.engine.scheduler import Request
    sched = llm.new_scheduler()
    # requests finish their prompts one after the other; each keeps decoding until
    # all of them have decoded together for K steps
    e2e_span = K + W + 2
    prefill_steps = B * (-(-(args.context - e2e_span) // PREFILL_TOKENS))
    e2e_new = K + 4 + prefill_steps
    e2e_ctx = args.context - e2e_new - 1
    for i in range(B):
        sched.add(Request(id=("e2e", i), prompt=prompt(e2e_ctx), max_new_tokens=e2e_new))
    llm.run(sched, record_steps=True)
    dec = [s for s in llm.step_log if s["decode_only"] and s["sampled"] == B][2:2 + K]
    e2e_s = sum(s["seconds"] for s in dec)
    e2e = {"value": round(sum(s["sampled"] for s in dec) / e2e_s, 1) if dec else None,
           "unit": "tokens/s",
           "h2d_bytes_per_step": int(statistics.median(s["h2d_bytes"] for s in dec)) if dec else 0,
           "d2h_bytes_per_step": int(statistics.median(s["d2h_bytes"] for s in dec)) if dec else 0,
           "steps": len(dec)}

    model_name = "Qwen3-4B-shaped" if args.preset == "qwen3-4b" else args.preset + "-shaped"
    record = {
        "metric": f"decode tokens/s, {model_name} bf16, batch {B} (prefill and batch 1/8/64 after 2,048-token prompts beside it)",
        "value": round(B / (ms_step / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": K,
        "warmup": W, "ms_per_step": round(ms_step, 4), "ms_per_step_mad": round(ms_mad, 4), "repeats": R,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": f"synthetic: random weights N(0,0.02) seed {seed}, seeded random token ids",
        "config": {"model": model_name, "layers": config.num_hidden_layers,
                   "layers_full": layers_full, "hidden": config.hidden_size,
                   "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                   "head_dim": config.head_dim, "intermediate": config.intermediate_size,
                   "vocab": config.vocab_size, "tied": config.tie_word_embeddings,
                   "global_batch": B, "seq_len": args.context, "decode_context": int(ctx_mid),
                   "points_prompt": POINT_PROMPT, "kv_block": PAGE, "parallelism": "none (1 GPU)",
                   "l2": "inputs larger than L2 (weights + cache read once per step)",
                   "weight_gb": round(weight_bytes / 1e9, 3),
                   "value_loop": "median of the repeats; argmax fed back on the device, tokens read at the end (the loop "
                                 "generation takes for greedy requests); e2e has the host in every step"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                     "bytes_per_step": int(step_bytes), "peak_source": pk_src,
                     "kernel_shares": shares,
                     "kernel_shares_note": "four steps without graphs, CUDA events between the launches"},
        "points": points,
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
