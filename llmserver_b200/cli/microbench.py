"""Kernel microbenchmarks, in the manner of the reference's bench_gemm.py, bench_attention.py and
bench_prefill_attention.py: each workload is timed inside a CUDA graph, and buffers are rotated over more
than the L2 cache (126 MB on B200) so that every launch reads from HBM (bench_gemm.py:5-6,59).  The same
workloads are what ``ncu`` is pointed at for the summaries under ``profiles/``.

    python -m llmserver_b200.cli.microbench gemm --rows 8 --out-features 4096 --in-features 4096
    python -m llmserver_b200.cli.microbench attention-decode --batch 64 --context 3072
    python -m llmserver_b200.cli.microbench attention-prefill --tokens 2048 [--context 32768]
    python -m llmserver_b200.cli.microbench decode-step --batch 8 --layers 4 [--eager]
    python -m llmserver_b200.cli.microbench prefill-step --tokens 2048 --layers 4
    python -m llmserver_b200.cli.microbench decode-timeline --batch 8 --layers 8

Head sizes and counts default to the Qwen3-8B shape (32 / 8 heads of 128, pages of 16 tokens).
``--eager`` launches kernels one by one instead of replaying a graph (what a profiler wants to see);
``--profile-range`` brackets the measured launches with cudaProfilerStart/Stop for ``ncu --profile-from-start off``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _graph_time(run_all, launches: int, repeats: int = 5) -> float:
    """Microseconds per launch of ``run_all`` (which issues ``launches`` launches) replayed from a graph."""
    import torch

    run_all()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_all()
    graph.replay()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(repeats):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / repeats / launches * 1e3


class _Range:
    def __init__(self, on: bool):
        self.on = on

    def __enter__(self):
        import torch
        if self.on:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()

    def __exit__(self, *exc):
        import torch
        torch.cuda.synchronize()
        if self.on:
            torch.cuda.profiler.stop()


def bench_gemm(args) -> dict:
    import torch
    from ..ops import gemm_bf16
    from ..ops.library import call, stream_handle

    rows, cols, inner = args.rows, args.out_features, args.in_features
    weight_bytes = cols * inner * 2
    copies = max(2, int(300e6 // weight_bytes) + 1)
    weights = [(torch.randn(cols, inner, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(rows, inner, device="cuda").to(torch.bfloat16)
    outs = [torch.empty(rows, cols, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    flag = gemm_bf16.error_flag(torch.device("cuda", torch.cuda.current_device()))

    def ours():
        for weight, out in zip(weights, outs):
            call("llm_gemm_small_m", x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, cols, inner, cols, 0,
                 args.split, *gemm_bf16.NO_SCALE, flag.data_ptr(), stream_handle())

    def library():
        for weight, out in zip(weights, outs):
            torch.matmul(x, weight.t(), out=out)

    result = {"workload": "gemm", "rows": rows, "out_features": cols, "in_features": inner, "weight_MB": weight_bytes / 1e6}
    if rows <= 64 and gemm_bf16.small_m_supported(rows, cols, inner):
        if args.eager:
            with _Range(args.profile_range):
                ours()
        else:
            micro = _graph_time(ours, copies)
            result.update(tcgen05_us=round(micro, 2), tcgen05_TBps=round(weight_bytes / micro / 1e6, 3))
        gemm_bf16.check_errors()
    if not args.eager:
        micro = _graph_time(library, copies)
        result.update(cublas_us=round(micro, 2), cublas_TBps=round(weight_bytes / micro / 1e6, 3),
                      cublas_TFLOPs=round(2.0 * rows * cols * inner / micro / 1e6, 1))
    return result


class _Batch:
    """The fields of a step batch that the attention wrappers read."""

    def __init__(self, contexts, q_lens):
        import torch
        self.q_lens, self.context_lens = list(q_lens), list(contexts)
        self.n_seqs, self.n_tokens = len(q_lens), sum(q_lens)
        starts = [0]
        for count in q_lens:
            starts.append(starts[-1] + count)
        self.q_start = torch.tensor(starts, dtype=torch.int32, device="cuda")
        self.context_len = torch.tensor(contexts, dtype=torch.int32, device="cuda")
        self.scratch = {}


def bench_attention(args, prefill: bool) -> dict:
    import torch
    from ..ops import attention_bf16

    heads, kv_heads, dim, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    if not attention_bf16.supported(dim, heads, kv_heads):
        return {"workload": "attention-prefill" if prefill else "attention-decode", "heads": heads, "kv_heads": kv_heads, "head_dim": dim,
                "unsupported": "the tensor-core kernels do not take these sizes; the engine runs the generic kernel for them"}
    if prefill:
        contexts, q_lens = [max(args.context or 0, args.tokens)], [args.tokens]
    else:
        contexts, q_lens = [args.context] * args.batch, [1] * args.batch
    batch = _Batch(contexts, q_lens)
    blocks = -(-contexts[0] // page)
    pages = len(contexts) * blocks + 1
    kv_bytes = len(contexts) * contexts[0] * kv_heads * dim * 2 * 2
    layers = max(2, int(300e6 // max(kv_bytes, 1)) + 1) if not prefill else 3
    layers = min(layers, 12)
    caches = [(torch.randn(pages, kv_heads, page, dim, device="cuda", dtype=torch.bfloat16),
               torch.randn(pages, kv_heads, page, dim, device="cuda", dtype=torch.bfloat16)) for _ in range(layers)]
    if args.shuffle_pages:      # pages of a request scattered over the pool, as after a long run of a server
        order = torch.randperm(len(contexts) * blocks, generator=torch.Generator().manual_seed(0))
        tables = order.to(torch.int32).view(len(contexts), blocks).cuda()
    else:
        tables = torch.arange(len(contexts) * blocks, device="cuda", dtype=torch.int32).view(len(contexts), blocks)
    stride = (heads + 2 * kv_heads) * dim
    qkv = torch.randn(batch.n_tokens, stride, device="cuda", dtype=torch.bfloat16)

    def run():
        for k_pages, v_pages in caches:
            attention_bf16.try_attention(qkv, stride, batch, tables, k_pages, v_pages, heads, kv_heads, dim, dim ** -0.5, 0)

    result = {"workload": "attention-prefill" if prefill else "attention-decode", "heads": heads, "kv_heads": kv_heads,
              "head_dim": dim, "page_size": page, "plan": list(attention_bf16.plan(batch, heads // kv_heads, kv_heads))}
    if args.eager:
        run()
        with _Range(args.profile_range):
            run()
        return result
    micro = _graph_time(run, layers)
    if prefill:
        before = contexts[0] - args.tokens          # keys every row of the portion sees, plus the causal triangle
        flops = 4.0 * heads * dim * (args.tokens * before + args.tokens * (args.tokens + 1) / 2)
        result.update(tokens=args.tokens, context=contexts[0], us=round(micro, 1), causal_TFLOPs=round(flops / micro / 1e6, 1))
    else:
        result.update(batch=args.batch, context=args.context, us=round(micro, 1), kv_MB=round(kv_bytes / 1e6, 1),
                      TBps=round(kv_bytes / micro / 1e6, 3))
    return result


def bench_step(args, prefill: bool) -> dict:
    """One model step of the 8B layer sizes with ``--layers`` layers (decode at ``--context`` or a prompt)."""
    import torch

    from .. import ops
    from .harness import Harness

    harness = Harness(args.layers, 1 if prefill else args.batch)
    if prefill:
        def once():
            for request_id in list(harness.step_function.computed):
                harness.step_function.release(request_id)
            harness.step_function.admit("p")
            harness.step_function.run([("p", harness.tokens(args.tokens), [args.tokens - 1])])
        once()
        once()
        with _Range(args.profile_range):
            once()
        return {"workload": "prefill-step", "layers": args.layers, "tokens": args.tokens}
    ids = harness.place(args.batch, args.context)
    tokens = harness.tokens(args.batch)

    def once():
        logits = harness.step_function.run([(request_id, [token], [0]) for request_id, token in zip(ids, tokens)])
        ops.sample(logits)
    for _ in range(4):
        once()
    with _Range(args.profile_range):
        once()
    return {"workload": "decode-step", "layers": args.layers, "batch": args.batch, "context": args.context, "mode": "eager"}


def decode_timeline(args) -> dict:
    """When every kernel of one replayed decode step starts and ends (CUPTI activity records through torch.profiler;
    no profiler replay, kernels overlap as they do in serving).  ``after`` is how long after the kernel before it
    ENDED a kernel ended: the step's time is the sum of that column, so it shows what each kernel adds to the step."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    from ..sampling import SamplingRow
    from .harness import Harness

    harness = Harness(args.layers, args.batch)
    harness.time_decode(args.batch, 4, 3)
    harness.time_decode(args.batch, 8, 3)        # the graph exists now; the requests sit near the mean context
    ids = list(harness.step_function.computed)[:args.batch]
    rows = [SamplingRow() for _ in ids]

    def step():
        return harness.step_function.run_and_sample([(request_id, [1], [0]) for request_id in ids], rows)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as recorded:
        step()
        torch.cuda.synchronize()
    events = sorted((event for event in recorded.events() if event.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda event: event.time_range.start)
    first = next(index for index, event in enumerate(events) if "Memcpy" not in event.name and "memcpy" not in event.name)
    events = events[first:]
    origin, last_end, lines = events[0].time_range.start, events[0].time_range.start, []
    for event in events:
        begin, end = event.time_range.start - origin, event.time_range.end - origin
        name = event.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0].split("<")[0]
        lines.append({"kernel": name, "start_us": round(begin, 2), "end_us": round(end, 2),
                      "after": round(max(0.0, event.time_range.end - last_end), 2)})
        last_end = max(last_end, event.time_range.end)
    if not args.json_only:
        for line in lines:
            print(f"{line['kernel']:44s} start {line['start_us']:9.2f}  end {line['end_us']:9.2f}  adds {line['after']:7.2f}", file=sys.stderr)
    per_kernel = {}
    for line in lines:
        per_kernel[line["kernel"]] = round(per_kernel.get(line["kernel"], 0.0) + line["after"], 2)
    return {"workload": "decode-timeline", "layers": args.layers, "batch": args.batch, "kernels": len(lines),
            "step_us": round(last_end - origin, 2), "adds_us_by_kernel": per_kernel}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="workload", required=True)

    def common(p):
        p.add_argument("--eager", action="store_true")
        p.add_argument("--profile-range", action="store_true")
        p.add_argument("--heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=128)
        p.add_argument("--page-size", type=int, default=16)
        p.add_argument("--shuffle-pages", action="store_true", help="scatter each request's pages over the pool")

    gemm = sub.add_parser("gemm")
    common(gemm)
    gemm.add_argument("--rows", type=int, default=8)
    gemm.add_argument("--out-features", type=int, default=4096)
    gemm.add_argument("--in-features", type=int, default=4096)
    gemm.add_argument("--split", type=int, default=0, help="split of K across a cluster (0: the kernel's default)")
    decode = sub.add_parser("attention-decode")
    common(decode)
    decode.add_argument("--batch", type=int, default=8)
    decode.add_argument("--context", type=int, default=3072)
    prefill = sub.add_parser("attention-prefill")
    common(prefill)
    prefill.add_argument("--tokens", type=int, default=2048)
    prefill.add_argument("--context", type=int, default=0, help="tokens the request holds after the portion (default: the portion is the whole prompt)")
    step = sub.add_parser("decode-step")
    common(step)
    step.add_argument("--batch", type=int, default=8)
    step.add_argument("--context", type=int, default=3072)
    step.add_argument("--layers", type=int, default=4)
    timeline = sub.add_parser("decode-timeline")
    common(timeline)
    timeline.add_argument("--batch", type=int, default=8)
    timeline.add_argument("--layers", type=int, default=8)
    timeline.add_argument("--json-only", action="store_true", help="no line per kernel on standard error")
    prompt = sub.add_parser("prefill-step")
    common(prompt)
    prompt.add_argument("--tokens", type=int, default=2048)
    prompt.add_argument("--layers", type=int, default=4)
    args = parser.parse_args(argv)
    os.environ["PATH"] = os.path.dirname(sys.executable) + os.pathsep + os.environ.get("PATH", "")
    if args.workload == "gemm":
        result = bench_gemm(args)
    elif args.workload == "attention-decode":
        result = bench_attention(args, prefill=False)
    elif args.workload == "attention-prefill":
        result = bench_attention(args, prefill=True)
    elif args.workload == "decode-timeline":
        result = decode_timeline(args)
    else:
        result = bench_step(args, prefill=args.workload == "prefill-step")
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
