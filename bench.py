"""Decode and prefill throughput of the library on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]
    python bench.py --workload llama-2-7b | llama-3.2-1b | 8b-decode512

The default run has the layer sizes of a Llama-3.1-8B (32 layers, hidden 4096,
32 heads over 8 kv heads of 128, feed-forward 14336, vocabulary 128256, llama3
rope scaling) with random bfloat16 weights, a batch of 8 and a context of 8192.
A step is one decode step of the whole batch; `value` is decoded tokens a
second, timed with CUDA events over exactly K steps after W warm-up steps.
One JSON line goes to standard output. `--workload` runs one of the other workloads of the
baseline instead and prints its own line: a Llama-2-7B shape with 16 prompts of 64 to 2,048
tokens and 128 new tokens each, a Llama-3.2-1B shape with 64 prompts of 1 to 8,192 tokens and
256 new tokens at temperature 0.7 (both through `LLM.generate`, host ids in and out), and the
Llama-3.1-8B shape decoding 256 tokens after prompts of 512 at batch 1, 8 and 64. The test names follow the `pp`/`tg`
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


# ----------------------------------------------------------------------------- the other workloads

def _generate_workload(args, shape_name, model_label, n_prompts, low, high, new_tokens, context, sampling, note):
    """`n_prompts` prompts with lengths uniform in [low, high], `new_tokens` new tokens each, through
    LLM.generate: tokens a second over the decode steps (host ids in and out), the bytes a decode
    step has to read at the mean context and their fraction of the copy rate."""
    import time

    import torch
    import llm_b200
    from llm_b200.config import config_from_dict
    from llm_b200.engine import random_model
    from llm_b200.shapes import shape

    torch.cuda.set_device(0)
    config = config_from_dict(shape(shape_name))
    peak, peak_source = peaks()
    model = random_model(config, seed=0)
    gen = torch.Generator().manual_seed(0)
    lengths = torch.randint(low, high + 1, (n_prompts,), generator=gen).tolist()
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    llm = llm_b200.LLM(model, context=context, batch=n_prompts)
    llm.generate([p[:8] for p in prompts[:2]], max_tokens=4, temperature=0.0, stop_tokens=[])
    clocks = ClockSampler()
    clocks.start()
    runs = []
    for repeat in range(max(1, min(args.steps, 3))):
        started = time.perf_counter()
        results = llm.generate(prompts, max_tokens=new_tokens, stop_tokens=[], details=True, **sampling)
        total_s = time.perf_counter() - started
        decode_s = max(r.decode_ms for r in results) * 1e-3
        runs.append({"decode_tok_s": sum(r.generated_tokens - 1 for r in results) / decode_s,
                     "prefill_tok_s": sum(lengths) / (results[0].prefill_ms * 1e-3),
                     "total_s": total_s, "ttft_ms": results[0].ttft_ms, "decode_s": decode_s})
    clocks.stop()
    llm.engine.cache.check()
    best = max(runs, key=lambda r: r["decode_tok_s"])
    mean = sum(r["decode_tok_s"] for r in runs) / len(runs)
    spread = (sum((r["decode_tok_s"] - mean) ** 2 for r in runs) / len(runs)) ** 0.5
    kv_bytes_per_token = 2 * config.num_key_value_heads * config.head_dim * config.num_hidden_layers * 2
    mean_context = sum(lengths) / n_prompts + new_tokens / 2
    step_bytes = model.weight_bytes() + n_prompts * mean_context * kv_bytes_per_token
    step_s = best["decode_s"] / (new_tokens - 1)
    print(json.dumps({
        "metric": f"decode tokens/s through LLM.generate, {model_label} shape bf16, {note}",
        "value": round(mean, 1), "stddev": round(spread, 1), "repeats": len(runs), "unit": "tokens/s",
        "n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "prefill_tokens_per_s": round(best["prefill_tok_s"], 1), "ttft_ms": round(best["ttft_ms"], 1),
        "total_s": round(best["total_s"], 3), "prompt_tokens": sum(lengths), "new_tokens": new_tokens,
        "config": {"model": model_label, "layers": config.num_hidden_layers, "hidden": config.hidden_size,
                   "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                   "head_dim": config.head_dim, "intermediate": config.intermediate_size,
                   "vocab": config.vocab_size, "global_batch": n_prompts, "context": context,
                   "prompt_lengths": f"uniform in [{low}, {high}]", "weights": "random N(0,0.02) seed 0",
                   "peaks": peak_source},
        "roofline": {"bound": "hbm", "bytes_per_step": int(step_bytes),
                     "achieved": round(step_bytes / step_s / 1e9, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(step_bytes / step_s / 1e9 / peak["hbm_gbs"], 4)},
        "clocks": clocks.summary()}))
    return 0


def workload_llama_2_7b(args):
    return _generate_workload(args, "llama-2-7b", "llama-2-7b", 16, 64, 2048, 128, 4096,
                              dict(temperature=0.0), "16 prompts of 64 to 2,048 tokens, 128 new tokens, greedy")


def workload_llama_3_2_1b(args):
    return _generate_workload(args, "llama-3.2-1b", "llama-3.2-1b", 64, 1, 8192, 256, 8192 + 256,
                              dict(temperature=0.7), "64 prompts of 1 to 8,192 tokens, 256 new tokens at temperature 0.7")


def workload_8b_decode512(args):
    """Llama-3.1-8B shape: prompts of 512 tokens and 256 new tokens at batch 1, 8 and 64, through
    LLM.generate (the baseline's own decode workload; the default run decodes at a full context)."""
    import torch
    import llm_b200
    from llm_b200.config import config_from_dict
    from llm_b200.engine import random_model
    from llm_b200.shapes import shape

    torch.cuda.set_device(0)
    config = config_from_dict(shape("llama-3.1-8b", args.layers))
    peak, peak_source = peaks()
    model = random_model(config, seed=0)
    kv_bytes_per_token = 2 * config.num_key_value_heads * config.head_dim * args.layers * 2
    clocks = ClockSampler()
    clocks.start()
    points = {}
    for batch in (1, 8, 64):
        llm = llm_b200.LLM(model, context=1024, batch=batch)
        gen = torch.Generator().manual_seed(batch)
        prompts = [torch.randint(0, config.vocab_size, (512,), generator=gen).tolist() for _ in range(batch)]
        llm.generate(prompts, max_tokens=8, temperature=0.0, stop_tokens=[])
        results = llm.generate(prompts, max_tokens=256, temperature=0.0, stop_tokens=[], details=True)
        decode_s = max(r.decode_ms for r in results) * 1e-3
        step_bytes = model.weight_bytes() + batch * 640 * kv_bytes_per_token
        points[f"b{batch}"] = {"decode_tok_s": round(batch * 255 / decode_s, 1),
                               "prefill_tok_s": round(batch * 512 / (results[0].prefill_ms * 1e-3), 1),
                               "hbm_frac": round(step_bytes / (decode_s / 255) / 1e9 / peak["hbm_gbs"], 3)}
        del llm
        torch.cuda.empty_cache()
    clocks.stop()
    print(json.dumps({
        "metric": "decode tokens/s through LLM.generate, Llama-3.1-8B shape bf16, prompts 512, 256 new tokens",
        "value": points["b8"]["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic", "points": points,
        "config": {"model": "llama-3.1-8b-shape", "layers": args.layers, "layers_full": FULL_LAYERS,
                   "prompt": 512, "new_tokens": 256, "weights": "random N(0,0.02) seed 0", "peaks": peak_source},
        "clocks": clocks.summary()}))
    return 0


WORKLOADS = {"llama-2-7b": workload_llama_2_7b, "llama-3.2-1b": workload_llama_3_2_1b,
             "8b-decode512": workload_8b_decode512}



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
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                        help="run one of the baseline's other workloads and print its line")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built (single-GPU library)")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.workload:
        return WORKLOADS[args.workload](args)

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
            # (the prefill before these ran at the power cap; the clock comes back over some tenths of a
            # second, so the warm-up here is a quarter of a second of steps)
            r = time_decode(b, args.context, max(16, args.steps // 2), 80 if b == 1 else 20)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / peak["hbm_gbs"], 3)
        # the baseline's own decode workload: prompts of 512 tokens, 256 new tokens (contexts 512 to 768)
        for b in (1, 8, 64):
            r = time_decode(b, 768, 252, 3)
            points[f"p512_n256_b{b}"] = round(r["tok_s"], 1)
            points[f"p512_n256_b{b}_hbm_frac"] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / peak["hbm_gbs"], 3)

    e2e = None
    if not args.no_e2e:
        # the same decode metric through the Python entry point: host token ids in
        # (pinned, copied every step with the step's index arrays), sampled ids out.
        # 256 tokens are generated after prompts that fill the context up to them; the
        # prefill of those prompts runs at the power cap and leaves the clock low for the
        # first steps, so the steps after the first 64 are also reported on their own.
        import time
        llm = llm_b200.LLM(model, context=args.context, batch=args.batch)
        e2e_new = 256
        prompt_len = (args.e2e_context or args.context) - e2e_new - 1
        prompts = [torch.randint(0, config.vocab_size, (prompt_len,),
                                 generator=torch.Generator().manual_seed(100 + i)).tolist()
                   for i in range(args.batch)]
        llm.generate(prompts, max_tokens=4, temperature=0.0, stop_tokens=[])      # warm-up
        stamps = []
        mark = clocks.mark()
        replays_before = llm.engine.graph_replays
        results = llm.generate(prompts, max_tokens=e2e_new, temperature=0.0, stop_tokens=[], details=True,
                               on_token=lambda index, token: stamps.append(time.perf_counter()) if index == 0 else None)
        e2e_clock = clocks.summary(mark, clocks.mark())
        decode_s = max(r.decode_ms for r in results) * 1e-3
        generated = sum(r.generated_tokens - 1 for r in results)
        steady_s = stamps[-1] - stamps[64]
        steady_steps = len(stamps) - 1 - 64
        gaps = sorted((b - a) * 1e3 for a, b in zip(stamps[64:], stamps[65:]))
        table_ints = sum(llm.engine.cache.table_width(g) for g in range(len(llm.engine.cache.groups)))
        e2e = {"value": round(generated / decode_s, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": 4 * args.batch * (7 + table_ints),
               "d2h_bytes_per_step": 4 * args.batch, "prompt_tokens": prompt_len, "new_tokens": e2e_new,
               "steady_value": round(args.batch * steady_steps / steady_s, 1),
               "steady_ms_per_step": round(steady_s / steady_steps * 1e3, 4), "steady_after_steps": 64,
               "steady_step_ms_p10": round(gaps[len(gaps) // 10], 3), "steady_step_ms_p50": round(gaps[len(gaps) // 2], 3),
               "steady_step_ms_p90": round(gaps[len(gaps) * 9 // 10], 3),
               "graph_replays": llm.engine.graph_replays - replays_before,
               "sm_mhz": e2e_clock["sm_mhz"],
               "ms_x_ghz": round(steady_s / steady_steps * 1e3 * (e2e_clock["sm_mhz"] or 0) / 1e3, 3)}
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
    main_clock = line["clocks"]
    line["ms_x_ghz"] = round(main_run["ms"] * (main_clock["sm_mhz"] or 0) / 1e3, 3)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
