#!/usr/bin/env python3
"""Runs the unmodified reference (AshvinSehgal/LLMServer, a copy of its files under ``baseline/_ref``) on the headline
benchmark: decode steps of a batch at a given mean context, through its own loader and its own ``Engine``.

This process imports nothing of llmserver_b200: only the reference's modules and what they import themselves.  It is
started by ``bench.py --impl reference`` with a model folder (config.json, generation_config.json, model.safetensors)
that holds seeded random weights of the benchmark's shape.

The path is the reference's stock one (benchmark_cuda.py:86-137): ``model_loader(folder, device, dtype)``,
``Engine(model, tokenizer, ..., kv_cache_block_size=16, ignore_eos=True)`` with its paged decode and CUDA graphs on,
``add_request(None, prompt_token_ids=...)``, ``while engine.step()``.  Prompts are prefilled for real; then W warm-up
decode steps and K timed ones.  ``value`` is device time (CUDA events around each ``engine.step()``); ``e2e`` is wall
clock over the same steps (each step sends the tokens to the device and reads the sampled tokens back).

Prints one JSON line; on any failure a line with ``unavailable`` and the error's own words.
"""
import argparse
import json
import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.path.join(HERE, "_ref")


class IdTokenizer:
    """The engine is driven with token ids; it still wants an object with these attributes (tests/test_engine.py:11-25)."""
    bos_token_id, pad_token_id, eos_token_id = 1, 0, 2

    def __call__(self, prompt):
        raise RuntimeError("the benchmark passes token ids, not text")

    def decode(self, token_ids, skip_special_tokens=True, clean_up_tokenization_spaces=False):
        return ""


def run(args):
    import math
    import torch
    sys.path.insert(0, REFERENCE)
    from utils.model_loader import model_loader
    from utils.engine import Engine
    from utils.request import RequestStatus

    device = torch.device("cuda")
    started = time.perf_counter()
    model = model_loader(args.model, device=device, dtype=torch.bfloat16)
    load_s = time.perf_counter() - started
    config = model.config
    prompt_len = max(1, args.context_mean - args.steps // 2 - args.warmup)
    max_length = prompt_len + args.warmup + args.steps + 64
    blocks = args.batch * math.ceil(max(max_length, args.context) / args.block_size) + 8      # benchmark_cuda.py:107
    engine = Engine(model, IdTokenizer(), max_new_tokens=args.warmup + args.steps + 48, max_batch_size=args.batch,
                    max_num_batched_tokens=max(8192, args.batch), kv_cache_num_blocks=blocks, kv_cache_block_size=args.block_size,
                    stream_text=False, max_completed_requests=0, ignore_eos=True, paged_context_limit=max(8192, max_length),
                    paged_decode=True, cuda_graphs=True)
    generator = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, config.vocab_size, (prompt_len,), generator=generator).tolist() for _ in range(args.batch)]
    requests = [engine.add_request(None, prompt_token_ids=prompt) for prompt in prompts]
    started = time.perf_counter()
    guard = 0
    while any(request.status != RequestStatus.DECODING for request in requests):
        engine.step()
        guard += 1
        if guard > 10000:
            raise RuntimeError("the prompts never finished")
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - started
    for _ in range(args.warmup):
        engine.step()
    torch.cuda.synchronize()
    before = sum(len(request.generated_token_ids) for request in requests)
    events = []
    wall = time.perf_counter()
    for _ in range(args.steps):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        engine.step()
        end.record()
        events.append((begin, end))
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall
    generated = sum(len(request.generated_token_ids) for request in requests) - before
    if generated != args.batch * args.steps:
        raise RuntimeError(f"the timed steps produced {generated} tokens, not {args.batch} x {args.steps}")
    device_ms = sum(begin.elapsed_time(end) for begin, end in events)
    return {
        "ms_per_step": device_ms / args.steps, "value": args.batch * args.steps / (device_ms / 1e3),
        "e2e": {"value": args.batch * args.steps / wall, "unit": "tokens/s", "ms_per_step": wall * 1e3 / args.steps,
                "h2d_bytes_per_step": args.batch * 8 * 2, "d2h_bytes_per_step": args.batch * 8},
        "mean_context": prompt_len + args.warmup + (args.steps + 1) / 2, "load_s": round(load_s, 1),
        "prefill_s": round(prefill_s, 2), "graphs": engine.graph_runner is not None, "paged_decode": bool(engine.paged_decode),
    }


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--model", required=True)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--context-mean", type=int, default=3072)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--block-size", type=int, default=16)
    args = parser.parse_args()
    try:
        result = run(args)
    except BaseException as error:      # the caller prints this as the reason the reference arm is unavailable
        lines = traceback.format_exception_only(type(error), error)
        frames = traceback.extract_tb(error.__traceback__)
        where = f" ({os.path.basename(frames[-1].filename)}:{frames[-1].lineno})" if frames else ""
        print(json.dumps({"unavailable": (lines[-1].strip() + where)[:600]}))
        return 0
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
