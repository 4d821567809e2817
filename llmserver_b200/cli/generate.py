"""Generates from token ids and prints the generated ids.

    python -m llmserver_b200.cli.generate --model DIR --prompt-ids 1,2,3 [--prompt-ids 7,8 ...]
           [--max-new-tokens 32] [--temperature 0.0] [--seed 0] [--ignore-eos] [--dtype bfloat16]
           [--block-size 16] [--max-batch-size 8] [--max-num-batched-tokens 8192] [--json]
    python -m llmserver_b200.cli.generate --random-config config.json --seed 0 --prompt-ids ...

The engine works on token ids (it has no tokenizer), so prompts are comma-separated ids, one ``--prompt-ids`` per
request, or one request per line of ``--prompt-file``.  All requests are queued at once and served by the same
``Engine`` that the Python entry point gives (continuous batching, greedy or seeded temperature sampling); one line
per request is printed, the generated ids separated by commas, in the order of the requests.  The reference prints
what it generated at the end of its benchmark and serves text through ``server.py`` (benchmark.py:338-490); this is
the token-id counterpart.  Option names follow the reference's engine (``max_new_tokens``, ``max_batch_size``,
``max_num_batched_tokens``, ``ignore_eos``; block size as ``--block-size`` in benchmark_cuda.py:490).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _ids(text: str):
    try:
        return [int(part) for part in text.replace(" ", "").split(",") if part]
    except ValueError as error:
        raise argparse.ArgumentTypeError(f"token ids are integers separated by commas: {error}") from error


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", help="folder with config.json and model.safetensors")
    parser.add_argument("--random-config", help="config.json of a model to be given seeded random weights on the device")
    parser.add_argument("--prompt-ids", type=_ids, action="append", default=[], help="one request: its prompt's token ids")
    parser.add_argument("--prompt-file", help="a file with one request per line (comma-separated ids)")
    parser.add_argument("--max-new-tokens", type=int, default=32)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--seed", type=int, default=0, help="seed of the weights (--random-config) and of the sampler; request i samples with seed + i")
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--max-batch-size", type=int, default=8)
    parser.add_argument("--max-num-batched-tokens", type=int, default=8192)
    parser.add_argument("--no-cuda-graphs", action="store_true")
    parser.add_argument("--json", action="store_true", help="print one JSON object with the ids, finish reasons and engine statistics")
    args = parser.parse_args(argv)
    if bool(args.model) == bool(args.random_config):
        parser.error("give exactly one of --model and --random-config")
    prompts = list(args.prompt_ids)
    if args.prompt_file:
        with open(args.prompt_file) as handle:
            prompts += [_ids(line) for line in handle if line.strip()]
    if not prompts or any(not prompt for prompt in prompts):
        parser.error("give at least one prompt, and no empty one (--prompt-ids 1,2,3)")
    os.environ["PATH"] = os.path.dirname(sys.executable) + os.pathsep + os.environ.get("PATH", "")

    from ..config.registry import architecture_of
    from ..engine.engine import Engine
    from ..models import load_model, random_model

    if args.model:
        model = load_model(args.model, args.dtype, args.device)
    else:
        with open(args.random_config) as handle:
            raw = json.load(handle)
        model = random_model(architecture_of(raw).config_class.from_dict(raw), args.seed, args.dtype, args.device)
    longest = max(len(prompt) for prompt in prompts) + args.max_new_tokens
    engine = Engine(model, max_new_tokens=args.max_new_tokens, max_batch_size=args.max_batch_size,
                    max_num_batched_tokens=args.max_num_batched_tokens, kv_cache_block_size=args.block_size,
                    ignore_eos=args.ignore_eos, cuda_graphs=not args.no_cuda_graphs, max_context=longest)
    requests = [engine.add_request(prompt_token_ids=prompt, temperature=args.temperature, seed=args.seed + index)
                for index, prompt in enumerate(prompts)]
    while engine.step():
        pass
    if args.json:
        print(json.dumps({"generated": [request.generated_token_ids for request in requests],
                          "finish_reasons": [request.finish_reason.value for request in requests],
                          "stats": {key: value for key, value in engine.stats.items() if not key.endswith("_s")},
                          "step_profile_ms": {key: round(value, 4) for key, value in engine.step_profile().items()}}))
    else:
        for request in requests:
            print(",".join(str(token) for token in request.generated_token_ids))
    return 0


if __name__ == "__main__":
    sys.exit(main())
