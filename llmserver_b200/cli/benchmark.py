"""Command-line benchmark in the manner of the reference's ``benchmark_cuda.py``: token-id prompts,
exactly n forced tokens per request, greedy.

    python -m llmserver_b200.cli.benchmark --model DIR [--prompt-tokens 128,1024] [--batch-sizes 1,8,32]
           [--output-tokens 128] [--repeats 3] [--dtype bfloat16] [--block-size 16]
           [--max-num-batched-tokens 16384] [--json] [--out-dir DIR]
    python -m llmserver_b200.cli.benchmark --random-config config.json --seed 0 ...
    python -m llmserver_b200.cli.benchmark --shape 14b --mixed-requests 32 --mixed-prompt-range 128,2048 \
           --output-tokens 256 --max-num-batched-tokens 8192 --json
    python -m llmserver_b200.cli.benchmark --shape 32b --mixed-requests 16 --mixed-prompt-range 4096,4096 \
           --shared-prefix-tokens 2048 --output-tokens 4096 --max-num-batched-tokens 8192 --json

Option names and meanings follow benchmark_cuda.py:477-496 where the reference has them
(``--model``, ``--prompt-tokens``, ``--batch-sizes``, ``--output-tokens``, ``--repeats``, ``--dtype``,
``--block-size``, ``--max-num-batched-tokens``, ``--json``, ``--out-dir``); ``--random-config`` and
``--seed`` are this engine's random-weights mode.  Method (benchmark_cuda.py:8-13,228-231): TTFT is the
time to produce one token for the whole batch; decode tokens/s = batch * (n - 1) / (total - TTFT); the
median over the repeats is reported; every run gets fresh uniform-random prompts so that no cached prefix
carries over; cache pages = batch * ceil((prompt + output) / block) + 8 (benchmark_cuda.py:107-111).

``--shape`` gives seeded random weights of one of the dense Qwen3 sizes the reference publishes numbers for.
``--mixed-requests`` queues that many requests at once and serves them by continuous batching; with
``--shared-prefix-tokens`` every second request begins with the same tokens and cached prefixes are on (the
reference's ``--matrix-prefix-modes cold,warm``, benchmark.py:340-364, asks the same question).  A scenario's result
carries a ``roofline`` block: the bytes every step has to read (all weights once, the cache of the requests it runs)
and its FLOPs, the time the slower of the two would take at the measured peaks summed over the steps, and the
fraction of the measured time that is.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time


def _int_list(text: str):
    return [int(part) for part in text.split(",") if part]


def run_once(engine, prompts, output_tokens: int) -> float:
    import torch

    torch.cuda.synchronize()
    started = time.perf_counter()
    for prompt in prompts:
        engine.add_request(prompt_token_ids=prompt, max_new_tokens=output_tokens, ignore_eos=True)
    while engine.step():
        pass
    torch.cuda.synchronize()
    return time.perf_counter() - started


def run_scenario(args, model, generator) -> dict:
    """``--mixed-requests``: all requests queued at once, served by continuous batching; the median run of
    ``--repeats`` is reported with its bytes, FLOPs and roofline."""
    import random
    import torch

    from ..engine.engine import Engine
    from .harness import attention_flops, cache_bytes_per_token, linear_flops_per_token, read_peaks, weight_bytes

    vocab = model.spec.vocab_size
    rng = random.Random(args.seed)
    low, high = args.mixed_prompt_range
    lengths = [rng.randint(low, high) for _ in range(args.mixed_requests)]
    slots = args.max_batch_size or args.mixed_requests
    longest = high + args.output_tokens
    shared = args.shared_prefix_tokens
    engine = Engine(model, max_new_tokens=args.output_tokens, max_batch_size=slots,
                    max_num_batched_tokens=args.max_num_batched_tokens,
                    kv_cache_num_blocks=slots * -(-longest // args.block_size) + 8, kv_cache_block_size=args.block_size,
                    ignore_eos=True, prefix_caching=shared > 0, cuda_graphs=not args.no_cuda_graphs, max_context=longest)

    def fresh_prompts():
        common = torch.randint(0, vocab, (shared,), generator=generator).tolist()
        prompts = []
        for index, length in enumerate(lengths):
            own = torch.randint(0, vocab, (length,), generator=generator).tolist()
            prompts.append(common + own[shared:] if shared and index % 2 == 1 and length > shared else own)
        return prompts

    run_once(engine, [prompt[:64] for prompt in fresh_prompts()[:min(4, len(lengths))]], 4)      # warm-up
    engine.warmup()
    runs = []
    for _ in range(args.repeats):
        before = dict(engine.stats)
        engine.record_steps, engine.step_log = True, []
        torch.cuda.synchronize()
        started = time.perf_counter()
        requests = [engine.add_request(prompt_token_ids=prompt, max_new_tokens=args.output_tokens, ignore_eos=True)
                    for prompt in fresh_prompts()]
        while engine.step():
            pass
        torch.cuda.synchronize()
        seconds = time.perf_counter() - started
        runs.append((seconds, list(engine.step_log), {key: engine.stats[key] - before[key] for key in before}, requests, started))
    engine.record_steps = False
    seconds, log, stats, requests, started = sorted(runs, key=lambda run: run[0])[len(runs) // 2]
    # bytes and FLOPs of the run, step by step, and the time the slower of the two needs at the measured peaks
    config, layers = model.config, len(model.spec.layers)
    peaks, peak_source = read_peaks()
    weights, per_token = weight_bytes(config, layers), cache_bytes_per_token(config, layers)
    linear, head = linear_flops_per_token(config, layers), 2 * config.vocab_size * config.hidden_size
    total_bytes = total_flops = floor = 0.0
    hbm_bound = 0
    for decode_rows, prompt_tokens, logit_rows, cached_tokens, pairs in log:
        step_bytes = weights + per_token * cached_tokens
        step_flops = linear * (decode_rows + prompt_tokens) + attention_flops(config, layers, pairs) + head * logit_rows
        by_hbm, by_tensor = step_bytes / (peaks["hbm_gbs"] * 1e9), step_flops / (peaks["bf16_tflops_sustained"] * 1e12)
        floor += max(by_hbm, by_tensor)
        hbm_bound += by_hbm >= by_tensor
        total_bytes += step_bytes
        total_flops += step_flops
    ttft = [request.first_token_at - request.created_at for request in requests]
    row = {"mixed_requests": args.mixed_requests, "prompt_tokens_total": sum(lengths), "output_tokens": args.output_tokens,
           "token_budget": args.max_num_batched_tokens, "max_batch_size": slots, "seconds": round(seconds, 4), "steps": stats["steps"],
           "output_tokens_per_s": round(args.mixed_requests * args.output_tokens / seconds, 1),
           "all_tokens_per_s": round((sum(lengths) + args.mixed_requests * args.output_tokens) / seconds, 1),
           "preemptions": stats["preemptions"], "prefix_tokens": stats["prefix_tokens"],
           "prefill_tokens_computed": stats["prefill_tokens"],
           "roofline": {"bytes": total_bytes, "flops": total_flops, "floor_s": round(floor, 4), "frac": round(floor / seconds, 4),
                        "steps_bound_by_hbm": hbm_bound, "steps_bound_by_tensor": len(log) - hbm_bound,
                        "peaks": f"{peak_source}: {peaks['hbm_gbs']:.0f} GB/s, {peaks['bf16_tflops_sustained']:.0f} TFLOP/s sustained"},
           "step_profile_ms": {key: round(value, 3) for key, value in engine.step_profile().items()},
           "ttft_s_mean": round(sum(ttft) / len(ttft), 4)}
    if shared:
        sharing = [value for index, value in enumerate(ttft) if index % 2 == 1]
        others = [value for index, value in enumerate(ttft) if index % 2 == 0]
        row.update(shared_prefix_tokens=shared, ttft_s_mean_sharing=round(sum(sharing) / len(sharing), 4),
                   ttft_s_mean_not_sharing=round(sum(others) / len(others), 4))
        # one request alone on the idle engine: a prompt whose beginning is cached against one that is all new
        prompts = fresh_prompts()
        run_once(engine, [prompts[1]], 1)                     # leaves the common beginning in the cache
        again = list(prompts[1][:shared]) + torch.randint(0, vocab, (len(prompts[1]) - shared,), generator=generator).tolist()
        row["ttft_s_alone_prefix_cached"] = round(run_once(engine, [again], 1), 4)
        row["ttft_s_alone_all_new"] = round(run_once(engine, [torch.randint(0, vocab, (len(again),), generator=generator).tolist()], 1), 4)
    return row


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", help="folder with config.json and model.safetensors")
    parser.add_argument("--random-config", help="config.json of a model to be given seeded random weights on the device")
    parser.add_argument("--shape", choices=["8b", "14b", "32b"], help="seeded random weights of this dense Qwen3 size")
    parser.add_argument("--layers", type=int, default=0, help="with --shape: fewer layers than the size has (layer sizes stay)")
    parser.add_argument("--shared-prefix-tokens", type=int, default=0,
                        help="with --mixed-requests: every second request begins with the same tokens, and cached prefixes are on")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--prompt-tokens", type=_int_list, default=[128, 1024])
    parser.add_argument("--batch-sizes", type=_int_list, default=[1, 8, 32])
    parser.add_argument("--output-tokens", type=int, default=128)
    parser.add_argument("--repeats", type=int, default=3)
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--max-num-batched-tokens", type=int, default=16384)
    parser.add_argument("--no-cuda-graphs", action="store_true")
    parser.add_argument("--mixed-requests", type=int, default=0,
                        help="instead of the grid: this many requests with uniform-random prompt lengths, all queued at once "
                             "and served by continuous batching (prompt portions and decode tokens share each step)")
    parser.add_argument("--mixed-prompt-range", type=_int_list, default=[128, 2048], help="shortest,longest prompt of --mixed-requests")
    parser.add_argument("--max-batch-size", type=int, default=0, help="request slots for --mixed-requests (default: all of them)")
    parser.add_argument("--json", action="store_true", help="print the results as JSON")
    parser.add_argument("--out-dir", help="also write results.json there")
    args = parser.parse_args(argv)
    if sum(map(bool, (args.model, args.random_config, args.shape))) != 1:
        parser.error("give exactly one of --model, --random-config and --shape")
    os.environ["PATH"] = os.path.dirname(sys.executable) + os.pathsep + os.environ.get("PATH", "")

    import torch

    from ..config.registry import architecture_of
    from ..engine.engine import Engine
    from ..models import load_model, random_model

    load_started = time.perf_counter()
    if args.model:
        model = load_model(args.model, args.dtype, args.device)
    else:
        if args.shape:
            from .harness import SHAPES
            raw = dict(SHAPES[args.shape])
            if args.layers:
                raw["num_hidden_layers"] = args.layers
        else:
            with open(args.random_config) as handle:
                raw = json.load(handle)
        model = random_model(architecture_of(raw).config_class.from_dict(raw), args.seed, args.dtype, args.device)
    torch.cuda.synchronize()
    load_seconds = time.perf_counter() - load_started
    vocab = model.spec.vocab_size
    generator = torch.Generator().manual_seed(args.seed)
    results = []
    if args.mixed_requests:
        results.append(run_scenario(args, model, generator))
        if not args.json:
            print(results[-1], flush=True)
        args.prompt_tokens = []
    for prompt_tokens in args.prompt_tokens:
        for batch in args.batch_sizes:
            longest = prompt_tokens + args.output_tokens
            engine = Engine(model, max_new_tokens=args.output_tokens, max_batch_size=batch,
                            max_num_batched_tokens=max(args.max_num_batched_tokens, batch),
                            kv_cache_num_blocks=batch * -(-longest // args.block_size) + 8,
                            kv_cache_block_size=args.block_size, ignore_eos=True, prefix_caching=False,
                            cuda_graphs=not args.no_cuda_graphs, max_context=longest)

            def fresh():
                return [torch.randint(0, vocab, (prompt_tokens,), generator=generator).tolist() for _ in range(batch)]

            run_once(engine, fresh(), min(4, args.output_tokens))      # warm-up (benchmark_cuda.py:208)
            ttfts, totals = [], []
            for _ in range(args.repeats):
                ttfts.append(run_once(engine, fresh(), 1))
                totals.append(run_once(engine, fresh(), args.output_tokens))
            ttft, total = statistics.median(ttfts), statistics.median(totals)
            decode = batch * (args.output_tokens - 1) / (total - ttft) if args.output_tokens > 1 and total > ttft else None
            row = {"prompt_tokens": prompt_tokens, "batch_size": batch, "output_tokens": args.output_tokens,
                   "ttft_ms": round(ttft * 1e3, 3), "total_ms": round(total * 1e3, 3),
                   "decode_tokens_per_s": None if decode is None else round(decode, 1),
                   "generation_tokens_per_s": round(batch * args.output_tokens / total, 1)}
            results.append(row)
            if not args.json:
                print(f"prompt {prompt_tokens:6d}  batch {batch:4d}  TTFT {row['ttft_ms']:9.2f} ms  "
                      f"decode {row['decode_tokens_per_s']} tok/s  total {row['total_ms']:.1f} ms", flush=True)
            del engine
            torch.cuda.empty_cache()
    report = {"model": args.model or args.random_config, "dtype": args.dtype, "load_seconds": round(load_seconds, 2),
              "block_size": args.block_size, "repeats": args.repeats, "results": results}
    if args.json:
        print(json.dumps(report))
    if args.out_dir:
        os.makedirs(args.out_dir, exist_ok=True)
        with open(os.path.join(args.out_dir, "results.json"), "w") as handle:
            json.dump(report, handle, indent=2)
    return 0


if __name__ == "__main__":
    sys.exit(main())
