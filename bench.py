#!/usr/bin/env python3
"""Headline benchmark: decode tokens per second of the Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

One "step" is one decode step of the whole batch.  The default run builds the 8B shape (36 layers,
width 4096, 32/8 heads of 128, intermediate 12288, vocabulary 151936) with seeded random bfloat16
weights, puts ``--batch`` requests (default 8) at a context whose mean over the timed steps is 3072
(2048-token prompts decoded to 4096), and times K decode steps with CUDA events after W warm-up steps.
It prints ONE JSON line: ``value`` is decoded tokens per second on the device, ``e2e`` the same through
``llmserver_b200.Engine`` with host token ids in and sampled ids out, ``prefill`` a 2048-token prompt
in one step, ``roofline`` the decode step's bytes over its time against the measured copy bandwidth,
``points`` decode at batch 1 and 64.  Inputs larger than L2: every step streams all weights (16 GB).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from llmserver_b200.cli.harness import (CONTEXT, MEAN_DECODE_CONTEXT, PAGE_SIZE, PROMPT, QWEN3_8B, ClockSampler,  # noqa: E402
                                        Harness, decode_bytes, prefill_flops, read_peaks)


def reference_arm(args) -> int:
    """Runs the unmodified reference (a copy of its files under baseline/_ref) on the same metric and configuration, in
    a process of its own that imports nothing of this package: ``baseline/reference_arm.py`` drives the reference's
    ``model_loader`` and ``Engine`` over a model folder with seeded random weights of the benchmark's shape, which is
    written here first.  Whatever stops it is printed as ``unavailable`` in its own words."""
    import shutil
    import subprocess
    import tempfile

    line = {"impl": "reference", "metric": "decode tok/s (Qwen3-8B shape, batch 8, context 4096)", "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids"}

    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:700]}))
        return 0

    reference = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(reference, "utils", "engine.py")):
        return unavailable("baseline/_ref does not hold the reference's files: pip cannot install AshvinSehgal/LLMServer (it has "
                           "neither setup.py nor pyproject.toml), so it runs from a plain copy of its files, which is missing here")
    if args.gpus != 1:
        return unavailable("the reference's engine is measured on one GPU, like this one")
    import torch
    import llmserver_b200.models  # noqa: F401  (registers the architecture)
    from llmserver_b200.config import Qwen3Config
    from llmserver_b200.weights import write_model_folder
    if not torch.cuda.is_available():
        return unavailable("no CUDA device is visible")
    raw = dict(QWEN3_8B, num_hidden_layers=args.layers, bos_token_id=1, eos_token_id=2, pad_token_id=0)
    free = {path: shutil.disk_usage(path).free for path in ("/dev/shm", tempfile.gettempdir()) if os.path.isdir(path)}
    need = 2.2 * (args.layers * 0.2e9 + 1.3e9) + (1 << 30)
    places = [path for path, room in free.items() if room > need]
    if not places:
        return unavailable(f"no room for the {need / 1e9:.0f} GB model folder the reference's loader reads: free space {free}")
    folder = tempfile.mkdtemp(prefix="llmserver_b200_ref_", dir=places[0])
    try:
        write_model_folder(Qwen3Config.from_dict(raw), folder, 0, torch.bfloat16, device="cuda:0")
        with open(os.path.join(folder, "config.json")) as handle:
            config_json = json.load(handle)
        config_json.update(bos_token_id=1, eos_token_id=2, pad_token_id=0, torch_dtype="bfloat16")
        with open(os.path.join(folder, "config.json"), "w") as handle:
            json.dump(config_json, handle)
        with open(os.path.join(folder, "generation_config.json"), "w") as handle:
            json.dump({"bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0}, handle)
        torch.cuda.empty_cache()
        command = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--model", folder, "--batch", str(args.batch),
                   "--steps", str(args.steps), "--warmup", str(max(args.warmup, 3)), "--context-mean", str(MEAN_DECODE_CONTEXT),
                   "--context", str(CONTEXT), "--block-size", str(PAGE_SIZE)]
        environment = dict(os.environ, HF_HUB_OFFLINE="1", TRANSFORMERS_OFFLINE="1", PYTHONPATH=reference)
        try:
            done = subprocess.run(command, capture_output=True, text=True, timeout=1500, env=environment, cwd=reference)
        except subprocess.TimeoutExpired:
            return unavailable("the reference did not finish within 1500 s")
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    result = None
    for text in reversed(done.stdout.strip().splitlines()):
        try:
            result = json.loads(text)
            break
        except ValueError:
            continue
    if result is None:
        tail = (done.stderr or done.stdout).strip().splitlines()[-3:]
        return unavailable(f"the reference's process ended with code {done.returncode}: " + " | ".join(tail))
    if "unavailable" in result:
        return unavailable("the reference failed on this box: " + result["unavailable"])
    config = Qwen3Config.from_dict(raw)
    line.update(value=round(result["value"], 1), ms_per_step=round(result["ms_per_step"], 4),
                e2e={key: (round(value, 1) if isinstance(value, float) else value) for key, value in result["e2e"].items()},
                config={"model": "Qwen3-8B shape", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
                        "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                        "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": config.vocab_size,
                        "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT,
                        "decode_context_mean": round(result["mean_context"]), "page_size": PAGE_SIZE, "parallelism": "none (1 GPU)",
                        "path": "utils.model_loader + utils.engine.Engine, paged decode, CUDA graphs"},
                reference={key: result[key] for key in ("load_s", "prefill_s", "graphs", "paged_decode") if key in result})
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"],
                        help="fewer layers than the 8B shape's 36 (layer sizes stay); the record names both numbers")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--skip-points", action="store_true", help="skip the batch-1 and batch-64 points")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (the engine has no multi-GPU path)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    import torch

    os.environ["PATH"] = os.path.dirname(sys.executable) + os.pathsep + os.environ.get("PATH", "")
    peaks, peak_source = read_peaks()
    harness = Harness(args.layers, max(args.batch, 1 if args.skip_points else 64))
    config = harness.config
    harness.time_decode(args.batch, 4, 3)      # untimed: lets the library choose its kernels
    with ClockSampler() as clocks:
        main_run = harness.time_decode(args.batch, args.steps, args.warmup)
    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            if batch == args.batch:
                points[f"decode_b{batch}"] = round(main_run["tokens_per_s"], 1)
                continue
            points[f"decode_b{batch}"] = round(harness.time_decode(batch, min(args.steps, 32), 3)["tokens_per_s"], 1)
    prefill_ms = harness.time_prefill(PROMPT)
    flops = prefill_flops(config, args.layers, PROMPT)
    e2e = harness.time_e2e(args.batch, args.steps, args.warmup)
    bytes_per_step = decode_bytes(config, args.layers, args.batch, main_run["mean_context"])
    achieved = bytes_per_step / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tok/s (Qwen3-8B shape, batch 8, context 4096)", "value": round(main_run["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
                   "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                   "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": config.vocab_size,
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT,
                   "decode_context_mean": round(main_run["mean_context"]), "page_size": PAGE_SIZE, "parallelism": "none (1 GPU)",
                   "l2": "inputs larger than L2: each step streams all weights", "peaks": peak_source},
        "clocks": clocks.summary(),
        "e2e": {key: (round(value, 1) if isinstance(value, float) else value) for key, value in e2e.items()},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": round(PROMPT / (prefill_ms / 1e3), 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
