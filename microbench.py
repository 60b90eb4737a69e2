"""Time one kernel of the library alone, at a given shape.

    python microbench.py linear --m 8 --n 6144 --k 4096 [--variant gemm_skinny]
    python microbench.py attention_decode --batch 8 --context 8192
    python microbench.py attention_prefill --tokens 2048
    python microbench.py rmsnorm --m 8 --k 4096
    python microbench.py sample --batch 8 --n 128256 [--temperature 0.7]
    LLMB_NVCC_FLAGS=-DLLMB_TRACE python microbench.py linear --m 8 --n 6144 --k 4096 --timeline
    LLMB_NVCC_FLAGS=-DLLMB_TRACE python microbench.py attention_prefill --tokens 2048 --timeline

Each call is timed inside a CUDA graph of `--reps` back-to-back launches (so that
the host's launch cost is not in the number), with CUDA events, after warm-up.
Weights rotate over enough copies to exceed L2, so every launch streams from
HBM. `--once` runs a single plain launch after warm-up instead (for a profiler).
Default sizes are those of a Llama-3.1-8B layer. The per-kernel table that
MythEclipse/llm prints with LLM_PROFILE=1 (apps/engine/src/cuda/mod.rs:1917-1972)
is the precedent; this tool isolates one kernel instead of wrapping every launch.
`--timeline` (tcgen05 product and decode attention, a build with -DLLMB_TRACE) prints when
the blocks of the last launch passed the phases the kernel stamps with the GPU's global timer;
for attention_prefill it prints the SM clock cycles that a softmax thread and the product thread
spend in each phase of a key block (the phases are too short for the global timer's steps).
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))

from llm_b200.ops import attention, linear, rmsnorm, rope_cache_write, swiglu, tactics  # noqa: E402

DEV = "cuda:0"


def time_in_graph(fn, reps: int, rounds: int = 10) -> float:
    """Microseconds per call of fn, from `rounds` replays of a graph of `reps` calls."""
    fn()
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(rounds):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / (rounds * reps) * 1e3


def run(fn, args, work_bytes=0.0, work_flops=0.0, label=""):
    if args.once:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        fn()
        torch.cuda.synchronize()
        print(f"{label}: one launch done")
        return
    us = time_in_graph(fn, args.reps)
    line = f"{label}: {us:.1f} us"
    if work_bytes:
        line += f", {work_bytes / us / 1e6:.2f} TB/s"
    if work_flops:
        line += f", {work_flops / us / 1e6:.1f} TFLOP/s"
    print(line)


PHASES = {
    "gemm_tc": ["block started", "set-up done", "predecessor complete", "first tiles landed",
                "last product issued", "partial written and fenced", "counter answered",
                "summed and stored (last arriver)"],
    "attention_decode": ["block started", "predecessor complete", "first pages landed", "keys done",
                         "partial written"],
}


def timeline(fn, label: str, library: str = "gemm_tc") -> int:
    """Back-to-back launches of fn, then the global-timer stamps of the last one, in microseconds
    after its first block started: earliest, median and latest block for every phase."""
    import ctypes
    from llm_b200.ops.build import load_library
    lib = load_library(library)
    read = getattr(lib, f"llmb_{library}_trace")
    rows, slots = 296, 12
    stamps = (ctypes.c_ulonglong * (rows * slots))()
    for _ in range(20):
        fn()
    torch.cuda.synchronize()
    if read(stamps, 1) != 0:
        print("this build has no stamps: set LLMB_NVCC_FLAGS=-DLLMB_TRACE", file=sys.stderr)
        return 1
    for _ in range(3):                       # the chain that is measured: the last of three launches
        fn()
    torch.cuda.synchronize()
    read(stamps, 0)
    table = torch.tensor(list(stamps), dtype=torch.float64).view(rows, slots)
    table = table[table[:, 0] > 0]
    # every block of every launch overwrites its row: what is left belongs to the last launch,
    # except phases that only some blocks reach (they may be older): those are cut at the start
    start = table[:, 0].min()
    print(f"{label}: {table.shape[0]} blocks; microseconds after the first block started")
    for slot, name in enumerate(PHASES[library]):
        column = table[:, slot]
        column = column[column >= start]
        if column.numel():
            relative = (column - start) / 1e3
            print(f"  {name:34s}{relative.min():8.2f}{relative.median():8.2f}{relative.max():8.2f}"
                  f"   ({column.numel()} blocks)")
    return 0


def phase_sums(fn, label: str) -> int:
    """attention_prefill, a build with -DLLMB_TRACE: mean SM clock cycles per key block that a softmax
    thread and the product thread of a block spend in each phase (over the launch's first 296 blocks)."""
    import ctypes
    from llm_b200.ops.build import load_library
    lib = load_library("attention_prefill_tc")
    rows, slots = 296, 12
    sums = (ctypes.c_ulonglong * (rows * slots))()
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    if lib.llmb_attention_prefill_tc_trace(sums, 1) != 0:
        print("this build has no phase sums: set LLMB_NVCC_FLAGS=-DLLMB_TRACE", file=sys.stderr)
        return 1
    fn()
    torch.cuda.synchronize()
    lib.llmb_attention_prefill_tc_trace(sums, 0)
    table = torch.tensor(list(sums), dtype=torch.float64).view(rows, slots)
    table = table[table[:, slots - 1] > 0]
    key_blocks = table[:, slots - 1].sum()
    names = ["softmax thread: waiting for S", "  reading S, the row's maximum", None,
             "  waiting for O, rescaling", "  exponentials, writing P", "  releasing P",
             "product thread: waiting for P", "  waiting for V", "  issuing P V", "  waiting for K, issuing Q K^T",
             "  the first two Q K^T"]
    print(f"{label}: {table.shape[0]} blocks, {int(key_blocks)} key blocks; mean SM cycles per key block")
    for slot, name in enumerate(names):
        if name:
            print(f"  {name:36s}{float(table[:, slot].sum() / key_blocks):9.0f}")
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("op", choices=["linear", "attention_decode", "attention_prefill", "rmsnorm",
                                  "swiglu", "rope", "sample"])
    p.add_argument("--m", type=int, default=8, help="rows (tokens)")
    p.add_argument("--n", type=int, default=6144)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=8192)
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--variant", default=None, help="force a kernel variant by disabling higher ranks")
    p.add_argument("--residual", action="store_true", help="linear: add into a 32-bit residual")
    p.add_argument("--norm", action="store_true", help="linear: with a folded norm (32 partial sums a row)")
    p.add_argument("--emit", action="store_true", help="linear (with --residual): leave the next norm's input")
    p.add_argument("--rope", action="store_true",
                   help="linear: the q/k/v product with rotation and cache write (n = (heads + 2 kv heads) * head dim)")
    p.add_argument("--glu", action="store_true", help="linear: the gated epilogue (n = 2 x the feed-forward width)")
    p.add_argument("--yardstick", action="store_true",
                   help="linear: also time torch.matmul (cuBLAS) on the same operands in the same harness: a "
                        "yardstick only, the library never calls it")
    p.add_argument("--temperature", type=float, default=0.0,
                   help="sample: 0 is greedy; above it the default chain (top-k 40, top-p 0.75, min-p 0.25, "
                        "repeat penalty 1.1 over the last 64) runs")
    p.add_argument("--reps", type=int, default=20)
    p.add_argument("--once", action="store_true")
    p.add_argument("--timeline", action="store_true",
                   help="linear, attention_decode: phases of the last launch's blocks; attention_prefill: cycles "
                        "per key block and phase (builds with -DLLMB_TRACE)")
    args = p.parse_args(argv)
    torch.manual_seed(0)
    bf16 = torch.bfloat16

    if args.op == "linear":
        if args.variant:
            table = tactics.rows("linear")
            wanted = [r for r in table if r.name == args.variant][0]
            for row in table:
                if row.rank > wanted.rank:
                    tactics.disable(row.name)
        m, n, k = args.m, args.n, args.k
        copies = 1 if args.once else max(2, int(300e6 / (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=DEV, dtype=bf16) * 0.02 for _ in range(copies)]
        x = torch.randn(m, k, device=DEV, dtype=bf16)
        res = torch.zeros(m, n, device=DEV, dtype=torch.float32) if args.residual else None
        out = None if args.residual else torch.empty(m, n, device=DEV, dtype=bf16)
        turn = [0]

        import llm_b200.ops as ops
        norm = emit = rope = None
        if args.norm:
            norm = ops.FoldedNorm(x, torch.rand(m, ops.SUMSQ_LD, device=DEV) * k / 32, 32, 1e-5, k)
        if args.emit:
            emit = ops.Emit(torch.empty(m, n, device=DEV, dtype=bf16), torch.empty(m, ops.SUMSQ_LD, device=DEV))
        if args.rope:
            hq, hkv, d = args.heads, args.kv_heads, args.head_dim
            assert n == (hq + 2 * hkv) * d, "--n must be (heads + 2 kv heads) * head dim"
            if m <= 64:                      # a decode step: m sequences, each at its context's last position
                pages = (args.context + 63) // 64
                kc = torch.zeros(m * pages, hkv, 64, d, device=DEV, dtype=bf16)
                vc = torch.zeros_like(kc)
                rope = ops.RopeWrite(torch.rand(args.context, d, device=DEV),
                                     torch.full((m,), args.context - 1, dtype=torch.int32, device=DEV),
                                     torch.arange(m, dtype=torch.int32, device=DEV),
                                     torch.arange(m * pages, dtype=torch.int32, device=DEV).view(m, pages), pages,
                                     kc, vc, hq, hkv, d)
            else:                            # a prefill: one sequence of m tokens
                pages = (m + 63) // 64
                kc = torch.zeros(pages, hkv, 64, d, device=DEV, dtype=bf16)
                vc = torch.zeros_like(kc)
                rope = ops.RopeWrite(torch.rand(m, d, device=DEV), torch.arange(m, dtype=torch.int32, device=DEV),
                                     torch.zeros(m, dtype=torch.int32, device=DEV),
                                     torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages), pages,
                                     kc, vc, hq, hkv, d)
        if args.glu:
            out = torch.empty(m, n // 2, device=DEV, dtype=bf16)

        def fn():
            linear(x, ws[turn[0] % copies], residual=res, out=out, norm=norm, emit=emit, rope=rope, glu=args.glu)
            turn[0] += 1
        args.reps = max(args.reps, copies * 2) if not args.once else args.reps
        name = tactics.choose_linear(m, n, k, bf16, bf16, k)
        if args.timeline:
            return timeline(fn, f"linear {name} M={m} N={n} K={k}")
        run(fn, args, n * k * 2, 2.0 * m * n * k, f"linear {name} M={m} N={n} K={k}")
        if args.yardstick and not args.once:
            plain_out = torch.empty(m, n, device=DEV, dtype=bf16)

            def library():
                torch.matmul(x, ws[turn[0] % copies].t(), out=plain_out)
                turn[0] += 1
            run(library, args, n * k * 2, 2.0 * m * n * k, f"torch.matmul (cuBLAS) M={m} N={n} K={k}")
    elif args.op in ("attention_decode", "attention_prefill"):
        hq, hkv, d = args.heads, args.kv_heads, args.head_dim
        decode = args.op == "attention_decode"
        batch = args.batch if decode else 1
        ctx = args.context if decode else args.tokens
        pages_per = (ctx + 63) // 64
        n_pages = batch * pages_per
        kc = torch.randn(n_pages, hkv, 64, d, device=DEV, dtype=bf16)
        vc = torch.randn(n_pages, hkv, 64, d, device=DEV, dtype=bf16)
        table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(batch, pages_per)
        lens = torch.full((batch,), ctx, dtype=torch.int32, device=DEV)
        if decode:
            qkv = torch.randn(batch, (hq + 2 * hkv) * d, device=DEV, dtype=bf16)
            pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=DEV)
            seq = torch.arange(batch, dtype=torch.int32, device=DEV)
            fn = lambda: attention(qkv, kc, vc, table, pages_per, pos, seq, hq, hkv, d, d ** -0.5, 0,
                                   decode=True, seq_lens=lens, max_len=ctx)
            if args.timeline:
                return timeline(fn, f"attention_decode batch={batch} context={ctx} heads={hq}/{hkv} D={d}",
                                "attention_decode")
            run(fn, args, batch * ctx * hkv * d * 2 * 2, 0.0,
                f"attention_decode batch={batch} context={ctx} heads={hq}/{hkv} D={d}")
        else:
            qkv = torch.randn(ctx, (hq + 2 * hkv) * d, device=DEV, dtype=bf16)
            pos = torch.arange(ctx, dtype=torch.int32, device=DEV)
            seq = torch.zeros(ctx, dtype=torch.int32, device=DEV)
            cu = torch.tensor([0, ctx], dtype=torch.int32, device=DEV)
            fn = lambda: attention(qkv, kc, vc, table, pages_per, pos, seq, hq, hkv, d, d ** -0.5, 0,
                                   seq_lens=lens, max_len=ctx, cu_seqlens=cu, max_new=ctx)
            args.reps = min(args.reps, 5)
            if args.timeline:
                return phase_sums(fn, f"attention_prefill tokens={ctx} heads={hq}/{hkv} D={d}")
            run(fn, args, 0.0, 2.0 * 2.0 * ctx * ctx / 2 * d * hq,
                f"attention_prefill tokens={ctx} heads={hq}/{hkv} D={d} (causal flops)")
    elif args.op == "sample":
        from llm_b200.sampling import BatchSampler, SamplingParams
        vocab, rows = args.n, list(range(args.batch))
        sampler = BatchSampler([SamplingParams(temperature=args.temperature)] * args.batch, vocab, DEV)
        base = torch.randn(args.batch, vocab, device=DEV)
        logits = base.clone()

        def fn():
            logits.copy_(base)                      # the penalty changes logits in place
            sampler.sample(logits, rows)
        run(fn, args, 0.0, 0.0, f"sample (with a copy of the logits) rows={args.batch} vocab={vocab} "
                                f"temperature={args.temperature}")
    elif args.op == "rmsnorm":
        x = torch.randn(args.m, args.k, device=DEV)
        g = torch.ones(args.k, device=DEV)
        run(lambda: rmsnorm(x, g, 1e-5, bf16), args, args.m * args.k * 6, 0.0, f"rmsnorm {args.m}x{args.k}")
    elif args.op == "swiglu":
        gu = torch.randn(args.m, 2 * args.n, device=DEV, dtype=bf16)
        run(lambda: swiglu(gu), args, args.m * args.n * 6, 0.0, f"swiglu {args.m}x{args.n}")
    elif args.op == "rope":
        hq, hkv, d, b = args.heads, args.kv_heads, args.head_dim, args.batch
        pages_per = (args.context + 63) // 64
        kc = torch.zeros(b * pages_per, hkv, 64, d, device=DEV, dtype=bf16)
        vc = torch.zeros_like(kc)
        table = torch.arange(b * pages_per, dtype=torch.int32, device=DEV).view(b, pages_per)
        qkv = torch.randn(b, (hq + 2 * hkv) * d, device=DEV, dtype=bf16)
        pos = torch.full((b,), args.context - 1, dtype=torch.int32, device=DEV)
        seq = torch.arange(b, dtype=torch.int32, device=DEV)
        angles = torch.randn(args.context, d, device=DEV)
        run(lambda: rope_cache_write(qkv, angles, pos, seq, table, pages_per, kc, vc, hq, hkv, d), args,
            0.0, 0.0, f"rope_cache_write batch={b}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
