"""Generation through the Python entry point on the GPU, against the plain implementation."""
import numpy as np
import pytest
import torch

import plain_model
from helpers import TOLERANCE, plain_folder, plain_logits, tokens_for
from tiny_configs import TINY

pytestmark = pytest.mark.gpu


def plain_greedy(folder, prompt, count):
    config, weights = plain_folder(folder)
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(plain_model.greedy(plain_model.forward(config, weights, tokens)[-1]))
    return tokens[len(prompt):]


def assert_tokens_are_argmax_of_plain(folder, prompt, generated, dtype, temperature=0.0, seed=0):
    """Every generated token must (nearly) maximise the plain implementation's score for its own prefix:
    logits for greedy, logits / T + Gumbel noise for sampling.  'Nearly' is the logit tolerance of the dtype."""
    logits = plain_logits(folder, list(prompt) + list(generated))
    for index, token in enumerate(generated):
        row = torch.from_numpy(logits[len(prompt) - 1 + index])
        slack = TOLERANCE[dtype] * row.abs().max().item() * 2
        if temperature > 0:
            scores = plain_model.gumbel_scores(row, temperature, seed, index)
            slack /= temperature
        else:
            scores = row.double()
        assert scores[token] >= scores.max() - slack, f"token {index} ({token}) is not the best choice"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tiny_a_three_requests_greedy(tiny_folders, dtype):
    """3 requests with prompts of 5 / 9 / 13 tokens, 8 greedy tokens each, pages of 4 tokens."""
    from llmserver_b200 import Engine
    folder = tiny_folders["a"]
    prompts = [tokens_for(256, length, 50 + length) for length in (5, 9, 13)]
    engine = Engine(folder, max_new_tokens=8, max_batch_size=4, max_num_batched_tokens=64, kv_cache_num_blocks=24,
                    kv_cache_block_size=4, ignore_eos=True, dtype=dtype)
    generated = engine.generate(prompts)
    assert all(len(tokens) == 8 for tokens in generated)
    for prompt, tokens in zip(prompts, generated):
        assert_tokens_are_argmax_of_plain(folder, prompt, tokens, dtype)
        if dtype == "float32":
            assert tokens == plain_greedy(folder, prompt, 8)
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity()     # every page came back


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tiny_b_chunks_mixed_with_decode_shared_prefix_and_temperature(tiny_folders, dtype):
    """4 requests with prompts of 1 / 7 / 17 / 37 tokens, the first 16 tokens shared by two of them,
    prefilled in portions of 6 beside decoding requests, 12 tokens each at temperature 0.8, pages of 8."""
    from llmserver_b200 import Engine
    folder = tiny_folders["b"]
    shared = tokens_for(509, 16, 1)
    prompts = [tokens_for(509, 1, 2), tokens_for(509, 7, 3), shared + tokens_for(509, 1, 4), shared + tokens_for(509, 21, 5)]
    engine = Engine(folder, max_new_tokens=12, max_batch_size=4, max_num_batched_tokens=16, prefill_chunk_size=6,
                    kv_cache_num_blocks=40, kv_cache_block_size=8, ignore_eos=True, dtype=dtype)
    requests = [engine.add_request(prompt_token_ids=prompt, temperature=0.8, seed=100 + index)
                for index, prompt in enumerate(prompts[:3])]
    # the fourth request arrives once the third one's prompt is in the cache, so it finds the shared pages
    while requests[2].status.value != "Decoding":
        engine.step()
    requests.append(engine.add_request(prompt_token_ids=prompts[3], temperature=0.8, seed=103))
    while engine.step():
        pass
    for index, (prompt, request) in enumerate(zip(prompts, requests)):
        assert len(request.generated_token_ids) == 12
        assert_tokens_are_argmax_of_plain(folder, prompt, request.generated_token_ids, dtype, 0.8, 100 + index)
    # the second request with the shared beginning took the first one's two complete pages over
    assert engine.stats["prefill_tokens"] == sum(len(p) for p in prompts) - 16
    engine.cache.check_invariants()
    # sampled tokens do not depend on the batch: each request alone gives the same tokens (32-bit logits
    # are bit-identical however the work is cut)
    if dtype == "float32":
        for index, prompt in enumerate(prompts):
            alone = Engine(engine.model, max_new_tokens=12, max_batch_size=1, max_num_batched_tokens=64,
                           kv_cache_num_blocks=16, kv_cache_block_size=8, ignore_eos=True)
            request = alone.add_request(prompt_token_ids=prompt, temperature=0.8, seed=100 + index)
            while alone.step():
                pass
            assert request.generated_token_ids == requests[index].generated_token_ids


def test_running_out_of_pages_preempts_and_changes_no_token(tiny_folders):
    from llmserver_b200 import Engine
    folder = tiny_folders["c"]
    prompts = [tokens_for(301, length, 70 + length) for length in (30, 21, 44, 9)]
    roomy = Engine(folder, max_new_tokens=40, max_batch_size=4, max_num_batched_tokens=32, kv_cache_num_blocks=128,
                   kv_cache_block_size=4, ignore_eos=True, dtype="float32")
    expected = roomy.generate(prompts)
    assert roomy.stats["preemptions"] == 0
    tight = Engine(roomy.model, max_new_tokens=40, max_batch_size=4, max_num_batched_tokens=32, kv_cache_num_blocks=48,
                   kv_cache_block_size=4, ignore_eos=True)
    assert tight.generate(prompts) == expected
    assert tight.stats["preemptions"] > 0
    tight.cache.check_invariants()
    assert tight.cache.available() == tight.cache.capacity()
    for prompt, tokens in zip(prompts, expected):
        assert_tokens_are_argmax_of_plain(folder, prompt, tokens, "float32")


def test_eos_stops_a_request(tiny_folders):
    from llmserver_b200 import Engine
    folder = tiny_folders["a"]
    prompt = tokens_for(256, 6, 9)
    free_run = plain_greedy(folder, prompt, 10)
    engine = Engine(folder, max_new_tokens=10, max_batch_size=2, kv_cache_num_blocks=16, kv_cache_block_size=4,
                    dtype="float32", eos_token_ids=[free_run[3]])
    stop = free_run.index(free_run[3])
    assert engine.generate([prompt]) == [free_run[:stop + 1]]


def test_the_first_tokens_of_a_sequence(tiny_folders):
    """Prompts of one and two tokens: the first positions have no history, pages are nearly empty."""
    from llmserver_b200 import Engine
    for name in ("a", "b", "c"):
        folder = tiny_folders[name]
        vocab = TINY[name][0]["vocab_size"]
        engine = Engine(folder, max_new_tokens=5, max_batch_size=3, kv_cache_num_blocks=12, kv_cache_block_size=16,
                        ignore_eos=True, dtype="float32")
        prompts = [[vocab - 1], [0, 1], [5]]
        for prompt, tokens in zip(prompts, engine.generate(prompts)):
            assert tokens == plain_greedy(folder, prompt, 5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuda_graph_decode_gives_the_same_tokens(tiny_folders, dtype):
    """Decode steps replayed from CUDA graphs against the same steps launched one by one."""
    from llmserver_b200 import Engine
    folder = tiny_folders["d"]
    prompts = [tokens_for(400, length, 90 + length) for length in (33, 5, 71)]
    outputs = {}
    for graphs in (False, True):
        engine = Engine(folder, max_new_tokens=40, max_batch_size=4, max_num_batched_tokens=128, kv_cache_num_blocks=64,
                        kv_cache_block_size=16, ignore_eos=True, dtype=dtype, cuda_graphs=graphs, max_context=256)
        # different lengths: the batch shrinks from 3 to 2 to 1, so padded buckets (4, 2, 1) are replayed
        requests = [engine.add_request(prompt_token_ids=prompt, max_new_tokens=limit)
                    for prompt, limit in zip(prompts, (40, 22, 31))]
        while engine.step():
            pass
        outputs[graphs] = [request.generated_token_ids for request in requests]
        assert [len(tokens) for tokens in outputs[graphs]] == [40, 22, 31]
        assert (engine.step_function.graph_steps > 20) == graphs
        if graphs:
            assert set(engine.step_function.graphs.graphs) >= {4, 2}
        engine.cache.check_invariants()
        assert engine.cache.available() == engine.cache.capacity()
    if dtype == "float32":
        assert outputs[True] == outputs[False]
    for prompt, tokens in zip(prompts, outputs[True]):
        assert_tokens_are_argmax_of_plain(folder, prompt, tokens, dtype)


def test_random_serving_schedule_changes_no_token(tiny_folders):
    """Thirty requests of random lengths arrive over time into a small cache (preemptions), with shared
    beginnings (prefix pages), a small token budget (portions beside decode tokens), CUDA graphs of several
    buckets, greedy and sampled: in 32-bit every request must produce exactly the tokens it produces alone."""
    import random
    from llmserver_b200 import Engine
    folder = tiny_folders["b"]      # one cache group without a window: shared prefixes are on
    rng = random.Random(3)
    common = tokens_for(509, 48, 500)
    jobs = []
    for index in range(30):
        prompt = tokens_for(509, rng.randint(1, 90), 600 + index)
        if index % 3 == 0:
            prompt = common[:rng.choice([16, 32, 48])] + prompt
        jobs.append(dict(prompt=prompt, new=rng.randint(1, 40), temperature=rng.choice([0.0, 0.0, 0.7]), seed=900 + index,
                         arrives=rng.randint(0, 60)))
    engine = Engine(folder, max_new_tokens=64, max_batch_size=6, max_num_batched_tokens=48, prefill_chunk_size=20,
                    kv_cache_num_blocks=13, kv_cache_block_size=16, ignore_eos=True, dtype="float32", max_context=256)
    requests, step = {}, 0
    while len(requests) < len(jobs) or engine.scheduler.waiting or engine.scheduler.running:
        for index, job in enumerate(jobs):
            if index not in requests and job["arrives"] <= step:
                requests[index] = engine.add_request(prompt_token_ids=job["prompt"], max_new_tokens=job["new"],
                                                     temperature=job["temperature"], seed=job["seed"])
        engine.step()
        step += 1
        assert step < 5000
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity()
    assert engine.stats["preemptions"] > 0 and engine.step_function.graph_steps > 0
    assert engine.stats["prefix_tokens"] > 0, "prefixes were meant to be shared"
    alone = Engine(engine.model, max_new_tokens=64, max_batch_size=1, max_num_batched_tokens=256, kv_cache_num_blocks=24,
                   kv_cache_block_size=16, ignore_eos=True, prefix_caching=False, cuda_graphs=False, max_context=256)
    for index, job in enumerate(jobs):
        request = alone.add_request(prompt_token_ids=job["prompt"], max_new_tokens=job["new"], temperature=job["temperature"],
                                    seed=job["seed"])
        while alone.step():
            pass
        assert requests[index].generated_token_ids == request.generated_token_ids, f"request {index} differs"
        assert len(request.generated_token_ids) == job["new"]


def test_random_serving_schedule_in_bfloat16_at_head_dim_128(tiny_folders):
    """The serving path's own kernels (tcgen05 prompt attention, TMA decode attention, the tcgen05 product for few rows)
    under a random schedule: requests of random lengths arrive over time into a small cache of two groups (one layer
    has a window of 150), portions run beside decode tokens, decode steps replay graphs of several buckets, requests
    are preempted.  Every token must be the plain implementation's choice for its own prefix, within the logit
    tolerance, greedy and sampled."""
    import random
    from llmserver_b200 import Engine
    folder, vocab = tiny_folders["e"], 333
    rng = random.Random(11)
    jobs = [dict(prompt=tokens_for(vocab, rng.randint(1, 260), 700 + index), new=rng.randint(1, 48),
                 temperature=rng.choice([0.0, 0.0, 0.8]), seed=40 + index, arrives=rng.randint(0, 40)) for index in range(18)]
    engine = Engine(folder, max_new_tokens=64, max_batch_size=5, max_num_batched_tokens=96, prefill_chunk_size=70,
                    kv_cache_num_blocks=44, kv_cache_block_size=16, ignore_eos=True, dtype="bfloat16", max_context=320)
    requests, step = {}, 0
    while len(requests) < len(jobs) or engine.scheduler.waiting or engine.scheduler.running:
        for index, job in enumerate(jobs):
            if index not in requests and job["arrives"] <= step:
                requests[index] = engine.add_request(prompt_token_ids=job["prompt"], max_new_tokens=job["new"],
                                                     temperature=job["temperature"], seed=job["seed"])
        engine.step()
        step += 1
        assert step < 5000
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity()
    assert engine.stats["preemptions"] > 0 and engine.step_function.graph_steps > 0
    for index, job in enumerate(jobs):
        tokens = requests[index].generated_token_ids
        assert len(tokens) == job["new"]
        assert_tokens_are_argmax_of_plain(folder, job["prompt"], tokens, "bfloat16", job["temperature"], job["seed"])


def run_alone(model, prompt, new_tokens, temperature=0.0, seed=0, block=16):
    from llmserver_b200 import Engine
    alone = Engine(model, max_new_tokens=new_tokens, max_batch_size=1, max_num_batched_tokens=512, kv_cache_num_blocks=40,
                   kv_cache_block_size=block, ignore_eos=True, prefix_caching=False, cuda_graphs=False, max_context=512)
    request = alone.add_request(prompt_token_ids=prompt, temperature=temperature, seed=seed)
    while alone.step():
        pass
    return request.generated_token_ids


@pytest.mark.parametrize("name,dtype", [("b", "float32"), ("e", "bfloat16")])
def test_a_request_put_out_between_replayed_steps_reads_its_new_pages(tiny_folders, name, dtype):
    """Three requests decode through the graph of four rows; the youngest is put out, waits at the head of the queue,
    has its cache rebuilt in other pages beside the two others' decode tokens, and returns to the same row beside the
    same neighbours.  The replayed step must read its new pages: a graph that recognised rows by request id kept the
    old ones, read pages that now belong to nobody and wrote the new token's keys into them."""
    from llmserver_b200 import Engine
    folder, vocab = tiny_folders[name], TINY[name][0]["vocab_size"]
    prompts = [tokens_for(vocab, length, 300 + length) for length in (23, 40, 31)]
    engine = Engine(folder, max_new_tokens=36, max_batch_size=4, max_num_batched_tokens=128, kv_cache_num_blocks=40,
                    kv_cache_block_size=16, ignore_eos=True, dtype=dtype, prefix_caching=False, max_context=256)
    requests = [engine.add_request(prompt_token_ids=prompt) for prompt in prompts]
    while engine.step_function.graph_steps < 4:
        assert engine.step()
    before = engine.step_function.graph_steps
    old_pages = [list(engine.cache.table(requests[2].request_id, group)) for group in range(len(engine.cache.groups))]
    # other requests come and go in between, so that the freed pages are taken and the free list moves on
    engine.put_out(requests[2])
    filler = engine.add_request(prompt_token_ids=tokens_for(vocab, 50, 77), max_new_tokens=1)
    engine.scheduler.waiting.rotate(1)        # the filler first: it takes the pages the victim gave back
    engine.step()
    assert len(filler.generated_token_ids) == 1
    while requests[2].status.value != "Decoding":
        engine.step()
    new_pages = [list(engine.cache.table(requests[2].request_id, group)) for group in range(len(engine.cache.groups))]
    assert new_pages != old_pages
    while engine.step():
        pass
    assert engine.step_function.graph_steps > before + 5 and requests[2].times_put_out == 1
    for prompt, request in zip(prompts, requests):
        assert len(request.generated_token_ids) == 36
        if dtype == "float32":
            assert request.generated_token_ids == run_alone(engine.model, prompt, 36)
        assert_tokens_are_argmax_of_plain(folder, prompt, request.generated_token_ids, dtype)
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity()


def test_a_tight_cache_puts_the_youngest_out_under_graphs_and_changes_no_token(tiny_folders):
    """Three requests that together outgrow the cache, graphs on: the youngest gives way, the others go on through the
    graph of two rows, it returns later; every request's tokens are those it produces alone."""
    from llmserver_b200 import Engine
    folder = tiny_folders["b"]
    prompts = [tokens_for(509, length, 400 + length) for length in (20, 27, 30)]
    engine = Engine(folder, max_new_tokens=48, max_batch_size=4, max_num_batched_tokens=96, kv_cache_num_blocks=12,
                    kv_cache_block_size=16, ignore_eos=True, dtype="float32", prefix_caching=False, max_context=128)
    requests = [engine.add_request(prompt_token_ids=prompt) for prompt in prompts]
    while engine.step():
        pass
    assert engine.stats["preemptions"] > 0 and engine.step_function.graph_steps > 20
    assert requests[0].times_put_out == 0
    for prompt, request in zip(prompts, requests):
        assert request.generated_token_ids == run_alone(engine.model, prompt, 48)
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity()


def test_warmup_leaves_nothing_to_tune_or_capture_and_the_step_profile_adds_up(tiny_folders):
    from llmserver_b200 import Engine
    from llmserver_b200.ops import gemm_bf16
    folder = tiny_folders["e"]
    engine = Engine(folder, max_new_tokens=12, max_batch_size=4, max_num_batched_tokens=96, kv_cache_num_blocks=40,
                    kv_cache_block_size=16, ignore_eos=True, dtype="bfloat16", max_context=256)
    report = engine.warmup()
    assert report["graphs"] == [1, 2, 4]
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity() and not engine.cache.requests
    tuned, captured = gemm_bf16.tunings(), dict(engine.step_function.graphs.graphs)
    prompts = [tokens_for(333, length, 800 + length) for length in (9, 33, 60, 17)]
    generated = engine.generate(prompts)
    assert gemm_bf16.tunings() == tuned, "a product was tuned inside a step after warmup()"
    assert engine.step_function.graphs.graphs == captured, "a graph was captured inside a step after warmup()"
    assert engine.step_function.graph_steps >= 8
    for prompt, tokens in zip(prompts, generated):
        assert_tokens_are_argmax_of_plain(folder, prompt, tokens, "bfloat16")
    profile = engine.step_profile()
    parts = sum(profile[name] for name in ("schedule", "pack_copy", "launch", "read_back", "accept"))
    assert 0 < parts <= profile["step"] * 1.001
    with pytest.raises(RuntimeError):
        engine.add_request(prompt_token_ids=[1, 2, 3])
        engine.warmup()


def test_the_generate_command_prints_the_ids_the_engine_generates(tiny_folders):
    import json
    import os
    import subprocess
    import sys
    folder = tiny_folders["a"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompts = [tokens_for(256, 6, 21), tokens_for(256, 11, 22)]
    command = [sys.executable, "-m", "llmserver_b200.cli.generate", "--model", folder, "--dtype", "float32", "--block-size", "4",
               "--max-new-tokens", "7", "--ignore-eos"]
    for prompt in prompts:
        command += ["--prompt-ids", ",".join(str(token) for token in prompt)]
    done = subprocess.run(command, capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = done.stdout.strip().splitlines()
    assert [[int(token) for token in line.split(",")] for line in lines] == [plain_greedy(folder, prompt, 7) for prompt in prompts]
    done = subprocess.run(command + ["--json", "--temperature", "0.7", "--seed", "5"], capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    report = json.loads(done.stdout.strip().splitlines()[-1])
    assert [len(tokens) for tokens in report["generated"]] == [7, 7] and report["finish_reasons"] == ["length", "length"]
    for index, (prompt, tokens) in enumerate(zip(prompts, report["generated"])):
        assert_tokens_are_argmax_of_plain(folder, prompt, tokens, "float32", 0.7, 5 + index)


def test_two_processes_with_the_same_plan_file_give_the_same_bfloat16_logits(tiny_folders, tmp_path):
    """The choice among the variants of a matrix product (which fixes the order of its partial sums) is measured per
    process unless it is read from a file: the first process measures and writes the file, two more read it and must
    agree bit for bit."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = tiny_folders["e"]
    plan = str(tmp_path / "gemm_plan.txt")
    script = (
        "import sys, hashlib, torch\n"
        "from llmserver_b200.models import load_model\n"
        "from llmserver_b200.cache import CacheManager\n"
        "from llmserver_b200.engine.step import StepFunction\n"
        "from llmserver_b200.ops import gemm_bf16\n"
        "model = load_model(sys.argv[1], 'bfloat16', 'cuda:0')\n"
        "cache = CacheManager(model.cache_needs(), 16, 40, num_slots=4, prefix_sharing=False)\n"
        "cache.materialize(model.runtime.device, model.runtime.dtype)\n"
        "step = StepFunction(model, cache)\n"
        "digest = hashlib.sha256()\n"
        "for name, count in (('a', 37), ('b', 5), ('c', 64)):\n"
        "    step.admit(name)\n"
        "    logits = step.run([(name, [(7 * i + len(name)) % 333 for i in range(count)], list(range(count)))])\n"
        "    digest.update(logits.cpu().numpy().tobytes())\n"
        "for round_index in range(4):\n"
        "    logits = step.run([(name, [round_index], [0]) for name in 'abc'])\n"
        "    digest.update(logits.cpu().numpy().tobytes())\n"
        "print('DIGEST', digest.hexdigest(), gemm_bf16.tunings())\n")
    results = []
    for _ in range(3):
        done = subprocess.run([sys.executable, "-c", script, folder], capture_output=True, text=True, cwd=root, timeout=600,
                              env=dict(os.environ, LLMSERVER_B200_GEMM_PLAN=plan, PYTHONPATH=root))
        assert done.returncode == 0, done.stderr[-2000:]
        line = [text for text in done.stdout.splitlines() if text.startswith("DIGEST")][-1].split()
        results.append((line[1], int(line[2])))
    assert os.path.isfile(plan) and results[0][1] > 0, "the first process was meant to measure and write the plan"
    assert results[1][1] == 0 and results[2][1] == 0, "a process that reads the plan measured again"
    assert results[1][0] == results[2][0] == results[0][0], "the same plan gave other logits"


@pytest.mark.parametrize("name", ["a", "c", "e"])
def test_few_rows_run_without_norm_kernels_and_agree_with_the_stand_alone_norms(tiny_folders, monkeypatch, name):
    """Up to 16 rows in bfloat16 the residual add and the norms run inside the products (two launches fewer per layer
    and per sub-layer boundary); the same step with the stand-alone kernels gives the same logits up to bfloat16
    rounding, and both match the plain implementation."""
    from helpers import assert_close, plain_logits, tokens_for
    from llmserver_b200 import ops
    from llmserver_b200.cache import CacheManager
    from llmserver_b200.engine.step import StepFunction
    from llmserver_b200.models import load_model
    folder = tiny_folders[name]
    model = load_model(folder, "bfloat16", "cuda:0")
    cache = CacheManager(model.cache_needs(), 8, 24, num_slots=2, prefix_sharing=False)
    cache.materialize(model.runtime.device, model.runtime.dtype)
    step = StepFunction(model, cache)
    tokens = tokens_for(model.spec.vocab_size, 13, 77)
    results, norm_calls = {}, {}
    real_add_rmsnorm = ops.add_rmsnorm
    calls = []

    def counted(*args, **kwargs):
        calls.append(1)
        return real_add_rmsnorm(*args, **kwargs)

    monkeypatch.setattr(ops, "add_rmsnorm", counted)
    for rows in (ops.STREAM_ROWS, 0):
        monkeypatch.setattr(ops, "STREAM_ROWS", rows)
        step.admit("r")
        step.run([("r", tokens[:9], [8])])
        del calls[:]
        logits = step.run([("r", tokens[9:], [0, 1, 2, 3])])
        norm_calls[rows] = len(calls)
        results[rows] = logits.float().cpu().numpy()
        step.release("r")
    layers = len(model.spec.schedule)
    # stand-alone: two per layer and the final norm; inside the products: the first layer's input and the final norm
    assert norm_calls == {16: 2, 0: 2 * layers + 1}, norm_calls
    want = plain_logits(folder, tokens)[9:]
    assert_close(results[16], want, "bfloat16", "norms inside the products")
    assert_close(results[0], want, "bfloat16", "stand-alone norms")
    assert_close(results[16], results[0], "bfloat16", "the two against each other")
