"""Trace replay on the GPU against the plain implementation: the same requests whole, with the last
32 tokens decoded one by one, in portions of changing size, and mixed with other requests in a pool
so small that pages are used again; in 32-bit and in bfloat16, on three tiny configurations."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import traces
from helpers import assert_close, plain_logits, tokens_for
from tiny_configs import TINY

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["a", "b", "c", "d", "e"]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_in_process(folder, dtype, records, max_tokens, page_size=16):
    from llmserver_b200.engine.replay import TraceReplayer

    replayer = TraceReplayer(folder, dtype, max_tokens, page_size)
    out = {}
    for record in records:
        logits = replayer.run_step(record)
        if logits is not None:
            out[record["step"]] = logits
    replayer.cache.check_invariants()
    assert not replayer.cache.requests, "requests left in the cache after the trace ended"
    for group in replayer.cache.groups:
        assert group.pool.num_available == group.pool.num_pages, "pages were lost"
    return out, replayer


def compare(got, records, requests, folder, dtype, what):
    want = traces.expected_rows(records, requests, lambda name: plain_logits(folder, requests[name]))
    assert set(got) == set(want), f"{what}: steps with logits differ"
    worst = 0.0
    for step in sorted(want):
        worst = max(worst, assert_close(got[step], want[step], dtype, f"{what} step {step}"))
    return worst


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests(tiny_folders, name, dtype):
    vocab = TINY[name][0]["vocab_size"]
    for length, page_size in ((1, 16), (2, 16), (5, 4), (67, 8), (300, 16)):
        tokens = tokens_for(vocab, length, 100 + length)
        records = traces.whole("r", tokens)
        got, _ = run_in_process(tiny_folders[name], dtype, records, traces.rounded(length), page_size)
        compare(got, records, {"r": tokens}, tiny_folders[name], dtype, f"{name} whole {length}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_tail_decoded_one_by_one(tiny_folders, name, dtype):
    vocab = TINY[name][0]["vocab_size"]
    tokens = tokens_for(vocab, 203, 7)
    records = traces.tail_decoded("r", tokens, 32)
    got, _ = run_in_process(tiny_folders[name], dtype, records, traces.rounded(len(tokens)))
    compare(got, records, {"r": tokens}, tiny_folders[name], dtype, f"{name} tail decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_changing_size(tiny_folders, name, dtype):
    vocab = TINY[name][0]["vocab_size"]
    tokens = tokens_for(vocab, 181, 11)
    records = traces.portions("r", tokens, [7, 2, 5, 3, 2, 16, 33, 2, 64, 1, 17])
    got, _ = run_in_process(tiny_folders[name], dtype, records, traces.rounded(len(tokens)), page_size=8)
    compare(got, records, {"r": tokens}, tiny_folders[name], dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_requests_reuse_pages(tiny_folders, name, dtype):
    vocab = TINY[name][0]["vocab_size"]
    lengths = {"r0": 150, "r1": 97, "r2": 40, "r3": 211, "r4": 64, "r5": 18, "r6": 129}
    requests = {key: tokens_for(vocab, length, 31 + index) for index, (key, length) in enumerate(lengths.items())}
    records, peak = traces.mixed(requests, seed=5)
    got, replayer = run_in_process(tiny_folders[name], dtype, records, peak)
    compare(got, records, requests, tiny_folders[name], dtype, f"{name} mixed")
    pool = replayer.cache.groups[0].pool
    assert pool.allocations > pool.num_pages, "the trace was meant to reuse pages"


@pytest.mark.parametrize("kernel,pairing", [("tcgen05-128", True), ("tcgen05-256", False), ("tcgen05-256", True)])
def test_prompt_kernels_through_replay(tiny_folders, kernel, pairing):
    """The other ways prompt portions can run (the 256-row kernel, which serving uses from 8192 rows on; row tiles
    handed out in mirror pairs, which it does when there are enough of them), driven through the same traces."""
    from llmserver_b200.ops import attention_bf16
    name, dtype = "e", "bfloat16"
    vocab = TINY[name][0]["vocab_size"]
    attention_bf16.PREFILL_KERNEL, attention_bf16.FORCE_PAIRING = kernel, pairing
    try:
        tokens = tokens_for(vocab, 300, 11)
        records = traces.portions("r", tokens, [7, 2, 70, 3, 130, 16, 33])
        got, _ = run_in_process(tiny_folders[name], dtype, records, traces.rounded(len(tokens)), page_size=8)
        compare(got, records, {"r": tokens}, tiny_folders[name], dtype, f"portions ({kernel})")
        lengths = {"r0": 150, "r1": 97, "r2": 40, "r3": 211, "r4": 64}
        requests = {key: tokens_for(vocab, length, 31 + index) for index, (key, length) in enumerate(lengths.items())}
        records, peak = traces.mixed(requests, seed=5)
        got, _ = run_in_process(tiny_folders[name], dtype, records, peak)
        compare(got, records, requests, tiny_folders[name], dtype, f"mixed ({kernel})")
    finally:
        attention_bf16.PREFILL_KERNEL, attention_bf16.FORCE_PAIRING = "tcgen05", None


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tiny_folders, dtype):
    vocab = TINY["c"][0]["vocab_size"]
    tokens = tokens_for(vocab, 420, 3)
    records = traces.tail_decoded("r", tokens, tail=412)
    got, _ = run_in_process(tiny_folders["c"], dtype, records, traces.rounded(len(tokens)))
    compare(got, records, {"r": tokens}, tiny_folders["c"], dtype, "long decoding")


def test_float32_logits_do_not_depend_on_the_cut(tiny_folders):
    """In 32-bit every kernel sums in an order that depends on the token's position only, so the
    logits of a position are bit-identical however the request was cut and batched."""
    vocab = TINY["b"][0]["vocab_size"]
    tokens = tokens_for(vocab, 120, 19)
    other = tokens_for(vocab, 75, 20)
    whole, _ = run_in_process(tiny_folders["b"], "float32", traces.whole("r", tokens), 128)
    cut = traces.portions("r", tokens, [3, 2, 40, 1, 1, 9])
    pieces, _ = run_in_process(tiny_folders["b"], "float32", cut, 128, page_size=4)
    stacked = np.concatenate([pieces[step] for step in sorted(pieces)])
    assert np.array_equal(stacked, whole[0])
    records, peak = traces.mixed({"r": tokens, "o": other}, seed=2)
    mixed, _ = run_in_process(tiny_folders["b"], "float32", records, peak)
    want = traces.expected_rows(records, {"r": tokens, "o": other},
                                lambda name: whole[0] if name == "r" else np.zeros((len(other), vocab), np.float32))
    fed = {}
    for record in records:
        row = 0
        for entry in record["entries"]:
            for place in entry["want"]:
                if entry["id"] == "r":
                    assert np.array_equal(mixed[record["step"]][row], want[record["step"]][row])
                row += 1


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("c", "bfloat16")])
def test_trace_run_program(tiny_folders, tmp_path, name, dtype):
    """The program itself, as a user runs it: JSON lines in, ``done`` lines and .f32 files out."""
    vocab = TINY[name][0]["vocab_size"]
    requests = {"x": tokens_for(vocab, 90, 1), "y": tokens_for(vocab, 33, 2), "z": tokens_for(vocab, 130, 3)}
    records, peak = traces.mixed(requests, seed=9, max_live=2)
    out_dir = tmp_path / "out"
    process = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", tiny_folders[name],
                              "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(peak)],
                             input="\n".join(json.dumps(record) for record in records) + "\n",
                             capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    assert [line for line in process.stdout.splitlines() if line.startswith("done ")] == [f"done {r['step']}" for r in records]
    got = {}
    for record in records:
        path = out_dir / f"{record['step']}.f32"
        wanted = sum(len(entry["want"]) for entry in record["entries"])
        assert path.exists() == (wanted > 0)
        if wanted:
            got[record["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
    compare(got, records, requests, tiny_folders[name], dtype, f"trace_run {name}")
