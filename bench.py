"""Decode and prefill throughput of the library on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

The default run has the layer sizes of a Llama-3.1-8B (32 layers, hidden 4096,
32 heads over 8 kv heads of 128, feed-forward 14336, vocabulary 128256, llama3
rope scaling) with random bfloat16 weights, a batch of 8 and a context of 8192.
A step is one decode step of the whole batch; `value` is decoded tokens a
second, timed with CUDA events over exactly K steps after W warm-up steps.
One JSON line goes to standard output. The test names follow the `pp`/`tg`
split of MythEclipse/llm's bench (apps/cli/src/bench.rs:10-12): prefill alone,
and decoding alone on a cache that is already filled.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
import threading
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FULL_LAYERS = 32
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    """Measured peaks if the file beside this script has them (keys searched at any depth:
    hbm_gbs, bf16_tflops, bf16_tflops_sustained), else the fallback figures."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for k, v in node.items():
                        if isinstance(v, (int, float)) and not isinstance(v, bool) and k in FALLBACK_PEAKS:
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
                elif isinstance(node, list):
                    for v in node:
                        walk(v)
            walk(raw)
            if flat.get("hbm_gbs", 0) > 0 and flat.get("bf16_tflops", 0) > 0:
                return {**FALLBACK_PEAKS, **flat}, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.process, self.thread = [], None, None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        def read():
            for line in self.process.stdout:
                self.samples.append([f.strip() for f in line.split(",")])
        self.thread = threading.Thread(target=read, daemon=True)
        self.thread.start()

    def mark(self):
        return len(self.samples)

    def stop(self):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self, begin=0, end=None):
        rows = [r for r in self.samples[begin:end] if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            rows = [r for r in self.samples if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(rows[0][1]), "reasons": reasons}


def reference_arm():
    """MythEclipse/llm is a Rust workspace (Cargo.toml, no setup.py or pyproject.toml):
    pip cannot install it and there is no Rust toolchain in this image."""
    print(json.dumps({"impl": "reference",
                      "unavailable": "MythEclipse/llm is a Rust workspace without Python packaging; "
                                     "pip install of its source tree fails (no setup.py or pyproject.toml) "
                                     "and no cargo/rustc is installed"}))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours")
    parser.add_argument("--layers", type=int, default=FULL_LAYERS,
                        help="run fewer layers than the 32 of the configuration (same layer sizes)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=8192)
    parser.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--no-prefill", action="store_true")
    parser.add_argument("--e2e-context", type=int, default=None,
                        help="context of the run through the entry point (default: --context)")
    parser.add_argument("--dtype", default="bfloat16")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built (single-GPU library)")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    import llm_b200
    from llm_b200 import ops
    from llm_b200.api import parse_dtype
    from llm_b200.config import config_from_dict
    from llm_b200.engine import Engine, Entry, random_model

    torch.cuda.set_device(0)
    device = "cuda:0"
    dtype = parse_dtype(args.dtype)
    from llm_b200.shapes import shape
    raw = shape("llama-3.1-8b", args.layers)
    config = config_from_dict(raw)
    peak, peak_source = peaks()
    model = random_model(config, seed=0, dtype=dtype, device=device)
    weight_bytes = model.weight_bytes()
    kv_bytes_per_token = (2 * config.num_key_value_heads * config.head_dim * args.layers
                          * (2 if dtype == torch.bfloat16 else 4))
    clocks = ClockSampler()
    clocks.start()

    def filled_engine(batch, context, steps_ahead):
        """An engine whose `batch` sequences already hold `context - steps_ahead - 1`
        positions of synthetic keys and values."""
        per_seq = (context + 63) // 64 * 64
        engine = Engine(model, max_tokens=batch * per_seq, max_seq_len=context, max_slots=batch)
        for group in engine.cache.groups:
            flat = group.storage.view(-1)
            chunk = 1 << 26
            for at in range(0, flat.numel(), chunk):
                part = flat[at:at + chunk]
                part.copy_(torch.randn(part.numel(), device=device, dtype=torch.float32).mul_(0.5))
        slots = engine.acquire(batch)
        start = context - steps_ahead - 1
        for s in slots:
            engine.cache.reserve(s, start)
            engine.cache.set_length(s, start)
        return engine, slots, start

    def time_decode(batch, context, steps, warmup):
        engine, slots, start = filled_engine(batch, context, steps + warmup)
        gen = torch.Generator().manual_seed(batch)
        feed = torch.randint(0, config.vocab_size, (steps + warmup, batch), generator=gen).tolist()
        for k in range(warmup):
            engine.step([Entry(s, [t], [0]) for s, t in zip(slots, feed[k])])
        torch.cuda.synchronize()
        launches_before = ops.launch_count()
        mark = clocks.mark()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for k in range(warmup, warmup + steps):
            engine.step([Entry(s, [t], [0]) for s, t in zip(slots, feed[k])])
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        mean_context = start + warmup + (steps + 1) / 2
        moved = weight_bytes + batch * mean_context * kv_bytes_per_token
        engine.release(slots)
        result = {"ms": ms, "tok_s": batch * 1e3 / ms, "bytes": moved,
                  "launches": ops.launch_count() - launches_before, "clock_mark": (mark, clocks.mark())}
        del engine
        torch.cuda.empty_cache()
        return result

    main_run = time_decode(args.batch, args.context, args.steps, args.warmup)

    # prefill of 2,048 tokens, one sequence, logits at the last place
    c = config

    def time_prefill(n_prefill=2048, repeats=3):
        engine = Engine(model, max_tokens=n_prefill + 64, max_seq_len=n_prefill + 64, max_slots=1)
        prompt = torch.randint(0, config.vocab_size, (n_prefill,),
                               generator=torch.Generator().manual_seed(1)).tolist()
        times = []
        for k in range(3 + repeats):
            (slot,) = engine.acquire()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin.record()
            engine.step([Entry(slot, prompt, [n_prefill - 1])])
            end.record()
            torch.cuda.synchronize()
            if k >= 3:
                times.append(begin.elapsed_time(end))
            engine.release([slot])
        prefill_ms = sum(times) / len(times)
        linear_flops = 2 * n_prefill * args.layers * (
            c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
            + c.num_attention_heads * c.head_dim * c.hidden_size
            + 3 * c.hidden_size * c.intermediate_size)
        # causal: every query sees half of the keys on average
        attention_flops = 2 * n_prefill * n_prefill * c.head_dim * c.num_attention_heads * args.layers
        head_flops = 2 * c.hidden_size * c.vocab_size
        flops = linear_flops + attention_flops + head_flops
        del engine
        torch.cuda.empty_cache()
        return {"value": round(n_prefill * 1e3 / prefill_ms, 1), "tokens": n_prefill,
                "ms": round(prefill_ms, 3),
                "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)}

    prefill = None if args.no_prefill else time_prefill()

    points = {}
    if not args.no_points:
        for b in (1, 64):
            r = time_decode(b, args.context, max(8, args.steps // 4), 3)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)

    e2e = None
    if not args.no_e2e:
        # the same decode metric through the Python entry point: host token ids in
        # (pinned, copied every step with the step's index arrays), sampled ids out
        llm = llm_b200.LLM(model, context=args.context, batch=args.batch)
        e2e_steps = args.steps
        prompt_len = (args.e2e_context or args.context) - e2e_steps - 1
        prompts = [torch.randint(0, config.vocab_size, (prompt_len,),
                                 generator=torch.Generator().manual_seed(100 + i)).tolist()
                   for i in range(args.batch)]
        llm.generate(prompts, max_tokens=4, temperature=0.0, stop_tokens=[])      # warm-up
        results = llm.generate(prompts, max_tokens=e2e_steps, temperature=0.0, stop_tokens=[],
                               details=True)
        decode_s = max(r.decode_ms for r in results) * 1e-3
        generated = sum(r.generated_tokens - 1 for r in results)
        table_ints = sum(llm.engine.cache.table_width(g) for g in range(len(llm.engine.cache.groups)))
        e2e = {"value": round(generated / decode_s, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": 4 * args.batch * (7 + table_ints),
               "d2h_bytes_per_step": 4 * args.batch, "prompt_tokens": prompt_len}
    clocks.stop()

    line = {
        "metric": f"decode tokens/s, Llama-3.1-8B shape {'bf16' if dtype == torch.bfloat16 else 'fp32'}, "
                  f"batch {args.batch}, context {args.context}",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if dtype == torch.bfloat16 else "fp32", "data": "synthetic",
        "config": {
            "model": "llama-3.1-8b-shape", "layers": args.layers, "layers_full": FULL_LAYERS,
            "hidden": c.hidden_size, "heads": c.num_attention_heads,
            "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
            "intermediate": c.intermediate_size, "vocab": c.vocab_size,
            "rope_theta": c.rope_theta, "rope_scaling": "llama3 factor 8 low 1 high 4 orig 8192",
            "rms_norm_eps": c.rms_norm_eps, "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "none (1 GPU)", "weights": "random N(0,0.02) seed 0",
            "l2": "inputs larger than L2 (weights read once a step)",
            "peaks": peak_source, "cache_page": 64,
        },
        "e2e": e2e, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9, 1),
                     "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9 / peak["hbm_gbs"], 4)},
        "points": points,
        "gpu_launches": main_run["launches"],
        "clocks": clocks.summary(*main_run["clock_mark"]),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
