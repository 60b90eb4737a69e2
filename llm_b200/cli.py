"""Command line of the library, in the manner of MythEclipse/llm's `llm-cli`.

    python -m llm_b200 [--model DIR] [--context 4096] [--max-tokens 256] [--temperature 0.7] ID ...
    python -m llm_b200 bench [-m DIR | --random SHAPE] [-c 4096] [-p 512] [-n 128] [-b 1] [-r 5] [-o json]
    python -m llm_b200 inspect DIR
    python -m llm_b200 random (--shape NAME | --config FILE) --out DIR [--seed S]

The first form completes a prompt given as token ids and prints the generated
ids and the run's statistics (apps/cli/src/main.rs:55-76: the same flags and
defaults; text and tokenizers are outside this library). `bench` keeps the
flags of apps/cli/src/bench.rs:45-71 (-m, -c, -p, -n, -r, -o with comma lists)
and its two tests: `pp<N>` times the prefill of N tokens and nothing else,
`tg<N>` prefills a 16-token prompt and times only the decoding of N tokens
(bench.rs:10-12,27); `-b` adds the batch size; every test runs once uncounted before its `-r`
repetitions. `inspect` prints the model's
geometry, checks the checkpoint's tensors and names the kernel variant each
product and attention shape gets (apps/cli/src/inspect.rs:16-131).
"""
from __future__ import annotations

import json
import statistics
import sys
import time

DEFAULT_CONTEXT = 4096
DEFAULT_MAX_TOKENS = 256
TG_PROMPT = 16


def _value(args, flag):
    if not args:
        raise SystemExit(f"{flag} needs a value")
    return args.pop(0)


def _int_list(text, flag):
    try:
        return [int(p) for p in text.split(",")]
    except ValueError:
        raise SystemExit(f"bad list for {flag}: {text}") from None


def main(argv=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    if not args or args[0] in ("-h", "--help", "help"):
        print(__doc__.strip())
        return 0 if args else 2
    if args and args[0] == "bench":
        return bench(args[1:])
    if args and args[0] == "random":
        return random_folder(args[1:])
    if args and args[0] == "inspect":
        if len(args) < 2:
            raise SystemExit("inspect needs a model folder")
        return inspect(args[1])
    return complete(args)


def complete(args) -> int:
    model, context, max_tokens, temperature, dtype = None, DEFAULT_CONTEXT, DEFAULT_MAX_TOKENS, 0.7, "bfloat16"
    seed, prompt = None, []
    while args:
        a = args.pop(0)
        if a == "--model":
            model = _value(args, a)
        elif a == "--context":
            context = int(_value(args, a))
        elif a == "--max-tokens":
            max_tokens = int(_value(args, a))
        elif a == "--temperature":
            temperature = float(_value(args, a))
        elif a == "--dtype":
            dtype = _value(args, a)
        elif a == "--seed":
            seed = int(_value(args, a))
        else:
            prompt += _int_list(a, "the prompt")
    if model is None or not prompt:
        raise SystemExit("usage: python -m llm_b200 --model DIR [--context N] [--max-tokens N] "
                         "[--temperature T] [--dtype bfloat16|float32] [--seed S] TOKEN_ID ...")
    import llm_b200
    llm = llm_b200.LLM(model, dtype=dtype, context=context, batch=1)
    options = {} if seed is None else {"seed": seed}
    (result,) = llm.generate([prompt], max_tokens=max_tokens, temperature=temperature, details=True,
                             on_token=lambda i, t: print(t, end=" ", flush=True), **options)
    print()
    print(f"[{result.prompt_tokens} prompt tokens, {result.generated_tokens} generated, "
          f"ttft {result.ttft_ms:.0f} ms, {result.tokens_per_second:.1f} tok/s, "
          f"stop: {result.stop_reason}]", file=sys.stderr)
    return 0


def bench(args) -> int:
    model_dir, random_shape, context, dtype = None, None, DEFAULT_CONTEXT, "bfloat16"
    prompts, gens, batches, reps, as_json, layers = [512], [128], [1], 5, False, None
    while args:
        a = args.pop(0)
        if a in ("-m", "--model"):
            model_dir = _value(args, a)
        elif a == "--random":
            random_shape = _value(args, a)
        elif a == "--layers":
            layers = int(_value(args, a))
        elif a in ("-c", "--context"):
            context = int(_value(args, a))
        elif a in ("-p", "--prompt"):
            prompts = _int_list(_value(args, a), a)
        elif a in ("-n", "--gen"):
            gens = _int_list(_value(args, a), a)
        elif a in ("-b", "--batch"):
            batches = _int_list(_value(args, a), a)
        elif a in ("-r", "--reps"):
            reps = int(_value(args, a))
        elif a in ("-o", "--output"):
            as_json = _value(args, a).lower() == "json"
        elif a == "--dtype":
            dtype = _value(args, a)
        else:
            raise SystemExit(f"unknown bench flag {a}")
    if (model_dir is None) == (random_shape is None):
        raise SystemExit("bench needs -m DIR or --random SHAPE (one of them)")
    import torch

    from .api import parse_dtype
    from .config import config_from_dict
    from .engine import (Engine, Entry, GenerationRequest, generate, load_model, random_model)
    from .sampling import SamplingParams
    from .cache import round_up
    from .shapes import shape
    if model_dir:
        model, name = load_model(model_dir, parse_dtype(dtype)), model_dir
    else:
        model = random_model(config_from_dict(shape(random_shape, layers)), 0, parse_dtype(dtype))
        name = random_shape + (f" ({layers} layers)" if layers else "")
    vocab = model.spec.vocab
    filler = torch.randint(0, vocab, (max(prompts + [TG_PROMPT]),),
                           generator=torch.Generator().manual_seed(0)).tolist()
    rows = []
    for batch in batches:
        per_seq = round_up(context)
        engine = Engine(model, max_tokens=batch * per_seq, max_seq_len=context, max_slots=batch)
        for n in prompts:
            samples = []
            for rep in range(reps + 1):            # the first run is not counted: it plans the scratch
                slots = engine.acquire(batch)
                torch.cuda.synchronize()
                started = time.perf_counter()
                engine.step([Entry(s, filler[:n], [n - 1]) for s in slots])
                torch.cuda.synchronize()
                if rep:
                    samples.append(batch * n / (time.perf_counter() - started))
                engine.release(slots)
            rows.append((f"pp{n}", batch, samples))
        for n in (g for g in gens if g > 0):
            samples = []
            for rep in range(reps + 1):            # the first run is not counted: it captures the graphs
                requests = [GenerationRequest(filler[:TG_PROMPT], n + 1, SamplingParams(temperature=0.0))
                            for _ in range(batch)]
                results = generate(engine, requests)
                decode_s = max(r.decode_ms for r in results) * 1e-3
                if rep:
                    samples.append(batch * n / decode_s if decode_s > 0 else 0.0)
            rows.append((f"tg{n}", batch, samples))
        scratch_identity = engine.workspace.plan_for(batch).identity()
        scratch_bytes, graphs = engine.workspace.bytes(), engine.use_graphs
        del engine
        torch.cuda.empty_cache()
    out = []
    for test, batch, samples in rows:
        mean = statistics.fmean(samples)
        spread = statistics.stdev(samples) if len(samples) > 1 else 0.0
        out.append({"test": test, "batch": batch, "backend": "B200 sm_100a", "avg_ts": mean,
                    "stddev_ts": spread})
    if as_json:
        print(json.dumps(out))
    else:
        print(f"| model | backend | batch | test | t/s |\n|---|---|---|---|---|")
        for r in out:
            print(f"| {name} {dtype} | {r['backend']} | {r['batch']} | {r['test']} | "
                  f"{r['avg_ts']:.2f} ± {r['stddev_ts']:.2f} |")
        used = torch.cuda.max_memory_allocated() / 2 ** 30
        print(f"\ndevice memory peak {used:.2f} GiB; weights read per decode step "
              f"{model.weight_bytes() / 2 ** 30:.2f} GiB")
        from .ops.build import build_identity, nvcc_version
        print(f"build {build_identity()} (nvcc {nvcc_version()}, sm_100a); kernel plan "
              f"{model.plan_identity()}; scratch plan {scratch_identity} ({scratch_bytes / 2 ** 20:.1f} MiB); "
              f"decode steps {'replayed from CUDA graphs' if graphs else 'launched one by one'}")
    return 0


def random_folder(args) -> int:
    """python -m llm_b200 random (--shape NAME | --config FILE) --out DIR [--seed S] [--layers L]
    [--dtype bfloat16|float32] [--std 0.02]: write config.json and model.safetensors with random
    weights (the fixture writer of MythEclipse/llm, scripts/make_tiny_moe.py, as a command)."""
    name, config_file, out, seed, layers, dtype, std = None, None, None, 0, None, "bfloat16", 0.02
    while args:
        a = args.pop(0)
        if a == "--shape":
            name = _value(args, a)
        elif a == "--config":
            config_file = _value(args, a)
        elif a == "--out":
            out = _value(args, a)
        elif a == "--seed":
            seed = int(_value(args, a))
        elif a == "--layers":
            layers = int(_value(args, a))
        elif a == "--dtype":
            dtype = _value(args, a)
        elif a == "--std":
            std = float(_value(args, a))
        else:
            raise SystemExit(f"unknown flag {a}")
    if out is None or (name is None) == (config_file is None):
        raise SystemExit("usage: python -m llm_b200 random (--shape NAME | --config FILE) --out DIR "
                         "[--seed S] [--layers L] [--dtype bfloat16|float32] [--std 0.02]")
    from . import native
    from .api import parse_dtype
    from .config import config_from_dict
    from .shapes import shape
    from .weights import write_random_model
    raw = shape(name, layers) if name else native.read_json(open(config_file, "rb").read(), config_file)
    if config_file and layers is not None:
        raw["num_hidden_layers"] = layers
    folder = write_random_model(out, config_from_dict(raw), seed, parse_dtype(dtype), std=std)
    print(folder)
    return 0


def inspect(folder) -> int:
    import torch

    from .config import load_config
    from .engine.model import DecoderModel
    from .errors import LlmError
    from .ops import tactics
    from .weights import check_names, open_checkpoint
    config = load_config(folder)
    spec = config.model_spec()
    model = DecoderModel(spec)
    expected = model.parameters()
    print(f"architecture  {spec.architecture}")
    for key, value in config.to_dict().items():
        if key not in ("architectures", "model_type"):
            print(f"{key:28s}{value}")
    params = sum(int(torch.tensor(p.shape).prod()) for p in expected.values())
    print(f"{'parameters':28s}{params:,} in {len(expected)} tensors")
    kv, states = model.cache_requests()
    per_token = sum(2 * r.n_kv_heads * r.head_dim * 2 for r in kv if r is not None)
    print(f"{'cache per token (bfloat16)':28s}{per_token / 1024:.1f} KiB")
    try:
        files = open_checkpoint(folder)
        check_names(expected, {n: f.shape(n) for n, f in files.items()}, str(folder))
        kinds = sorted({str(f.dtype(n)).replace('torch.', '') for n, f in files.items()})
        print(f"{'checkpoint':28s}all tensors present, stored as {', '.join(kinds)}")
        verdict = "runnable"
    except LlmError as error:
        print(f"checkpoint problem:\n{error}")
        verdict = "not runnable"
    for label, family, shape in model.kernel_shapes(torch.bfloat16):
        print(tactics.explain(family, **shape) + f"   [{label}]")
    from .ops.build import build_identity, nvcc_version
    print(f"{'kernel plan':28s}{model.plan_identity(torch.bfloat16)}")
    print(f"{'build':28s}{build_identity()} (nvcc {nvcc_version()}, sm_100a)")
    print(verdict)
    return 0 if verdict == "runnable" else 1
