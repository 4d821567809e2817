"""What the benchmarks share: the model shapes of the published configurations, the measured peaks, a clock
sampler, the bytes and FLOPs of a step, and a harness that holds a model, a cache and a step function on the device.

``bench.py`` at the root of the repository (the headline line), ``cli/benchmark.py`` (the reference's own method and
the serving scenarios) and ``cli/microbench.py`` (single kernels and steps for the profiler) all build on this module.
"""
from __future__ import annotations

import json
import os
import threading
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

def _qwen3(layers: int, hidden: int, heads: int, intermediate: int) -> dict:
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=hidden,
                intermediate_size=intermediate, num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=8,
                head_dim=128, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=40960, hidden_act="silu", attention_bias=False, use_sliding_window=False)


# the dense Qwen3 sizes the reference publishes numbers for (docs/results.md); random weights stand in for checkpoints
SHAPES = {"8b": _qwen3(36, 4096, 32, 12288), "14b": _qwen3(40, 5120, 40, 17408), "32b": _qwen3(64, 5120, 64, 25600)}
QWEN3_8B = SHAPES["8b"]
CONTEXT = 4096          # prompts of 2048 tokens decoded to 4096
PROMPT = 2048
MEAN_DECODE_CONTEXT = (CONTEXT + PROMPT) // 2
PAGE_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                raw = json.load(handle)
            peaks = {key: float(raw[key]) for key in FALLBACK_PEAKS if key in raw}
            if "hbm_gbs" in peaks and "bf16_tflops" in peaks:
                peaks.setdefault("bf16_tflops_sustained", peaks["bf16_tflops"])
                return peaks, "measured"
        except (OSError, ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs (reads only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int = 0, period: float = 0.1):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period, self.index = period, index
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: report nothing rather than fail the benchmark
            self.nvml = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
                mask = self.nvml.nvmlDeviceGetCurrentClocksEventReasons(self.handle) if hasattr(
                    self.nvml, "nvmlDeviceGetCurrentClocksEventReasons") else self.nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        ordered = sorted(self.samples)
        return {"sm_mhz": ordered[len(ordered) // 2] if ordered else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def weight_bytes(config, layers: int) -> float:
    """Bytes of every weight a step reads (the embedding table, of which a step reads a few rows, left out)."""
    hidden, inter, dim = config.hidden_size, config.intermediate_size, config.head_dim
    heads, kv_heads = config.num_attention_heads, config.num_key_value_heads
    per_layer = ((heads + 2 * kv_heads) * dim * hidden + hidden * heads * dim + 3 * hidden * inter + 2 * hidden + 2 * dim) * 2
    return layers * per_layer + config.vocab_size * hidden * 2 + hidden * 2


def cache_bytes_per_token(config, layers: int) -> float:
    """Bytes of keys and values one cached token holds over all layers."""
    return 2 * config.num_key_value_heads * config.head_dim * 2 * layers


def decode_bytes(config, layers: int, batch: int, context: int) -> float:
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live requests."""
    return weight_bytes(config, layers) + cache_bytes_per_token(config, layers) * batch * context


def linear_flops_per_token(config, layers: int) -> float:
    hidden, inter, dim = config.hidden_size, config.intermediate_size, config.head_dim
    heads, kv_heads = config.num_attention_heads, config.num_key_value_heads
    return 2 * layers * ((heads + 2 * kv_heads) * dim * hidden + hidden * heads * dim + 3 * hidden * inter)


def attention_flops(config, layers: int, query_key_pairs: float) -> float:
    """QK^T and PV for ``query_key_pairs`` (query token, visible key) pairs, all heads and layers."""
    return 2 * 2 * config.num_attention_heads * config.head_dim * query_key_pairs * layers


def prefill_flops(config, layers: int, tokens: int) -> float:
    hidden, inter, dim = config.hidden_size, config.intermediate_size, config.head_dim
    heads, kv_heads = config.num_attention_heads, config.num_key_value_heads
    linear = 2 * tokens * ((heads + 2 * kv_heads) * dim * hidden + hidden * heads * dim + 3 * hidden * inter)
    attention = 2 * 2 * heads * dim * tokens * (tokens + 1) / 2      # QK^T and PV over the causal half
    return layers * (linear + attention) + 2 * config.vocab_size * hidden   # logits of the last token only


class Harness:
    """Model, cache and step function sized for the largest batch, reused by every measurement."""

    def __init__(self, layers: int, max_batch: int, seed: int = 0, shape: str = "8b"):
        import torch
        from llmserver_b200.cache import CacheManager
        from llmserver_b200.config import Qwen3Config
        from llmserver_b200.engine.step import StepFunction
        from llmserver_b200.models import random_model

        self.torch = torch
        raw = dict(SHAPES[shape], num_hidden_layers=layers)
        self.config = Qwen3Config.from_dict(raw)
        self.layers = layers
        self.model = random_model(self.config, seed, "bfloat16", "cuda:0")
        pages = max_batch * (CONTEXT // PAGE_SIZE) + 8     # the reference benchmark's sizing rule
        self.cache = CacheManager(self.model.cache_needs(), PAGE_SIZE, pages, num_slots=max_batch, prefix_sharing=False)
        self.cache.materialize(self.model.runtime.device, self.model.runtime.dtype)
        for group in self.cache.groups:     # contents do not change the timing; avoid an all-zero cache anyway
            group.storage.normal_(0.0, 0.5)
        self.step_function = StepFunction(self.model, self.cache)
        self.generator = torch.Generator().manual_seed(seed)

    def tokens(self, count: int):
        return self.torch.randint(0, self.config.vocab_size, (count,), generator=self.generator).tolist()

    def place(self, batch: int, context: int):
        """Puts ``batch`` requests at ``context`` cached tokens each (pages allocated, contents as they are)."""
        for request_id in list(self.step_function.computed):
            self.step_function.release(request_id)
        ids = [f"b{index}" for index in range(batch)]
        for request_id in ids:
            self.step_function.admit(request_id)
            self.cache.ensure(request_id, context)
            self.step_function.computed[request_id] = context
        return ids

    def time_decode(self, batch: int, steps: int, warmup: int):
        torch = self.torch
        from llmserver_b200 import ops
        start_context = max(1, MEAN_DECODE_CONTEXT - steps // 2 - warmup)
        ids = self.place(batch, start_context)
        from llmserver_b200.sampling import SamplingRow
        if self.step_function.graphs is None:
            self.step_function.enable_graphs(CONTEXT, 64)
        tokens = self.tokens(batch)
        events = []
        launches_before = None
        rows = [SamplingRow() for _ in ids]
        for step in range(warmup + steps):
            if step == warmup:
                torch.cuda.synchronize()
                launches_before = ops.launch_count()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            # one decode step: batch in (one copy), forward, sampling, tokens out (one copy)
            tokens = self.step_function.run_and_sample([(request_id, [token], [0]) for request_id, token in zip(ids, tokens)], rows)
            end.record()
            if step >= warmup:
                events.append((begin, end))
        torch.cuda.synchronize()
        launches = ops.launch_count() - launches_before
        if self.step_function.graph_steps:      # replayed steps launch the captured kernels: count them per step
            launches = steps * self.launches_per_step(batch)
        self.step_function.check_errors()
        times = [begin.elapsed_time(end) for begin, end in events]
        total_ms = sum(times)
        mean_context = start_context + warmup + (steps + 1) / 2
        return {"ms_per_step": total_ms / steps, "tokens_per_s": batch * steps / (total_ms / 1e3),
                "launches": launches, "mean_context": mean_context}

    def launches_per_step(self, batch: int) -> int:
        """Kernels of this package in one decode step, counted on an eager step of the same shape."""
        from llmserver_b200 import ops
        ids = list(self.step_function.computed)[:batch]
        graphs, self.step_function.graphs = self.step_function.graphs, None
        before = ops.launch_count()
        self.step_function.run([(request_id, [0], [0]) for request_id in ids])
        count = ops.launch_count() - before + 1     # + the sampling kernel
        self.step_function.graphs = graphs
        return count

    def time_prefill(self, tokens: int, repeats: int = 3):
        torch = self.torch
        best = None
        for _ in range(repeats + 1):     # the first run warms up
            for request_id in list(self.step_function.computed):
                self.step_function.release(request_id)
            self.step_function.admit("p")
            prompt = self.tokens(tokens)
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            self.step_function.run([("p", prompt, [tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            elapsed = begin.elapsed_time(end)
            best = elapsed if best is None else min(best, elapsed)
        self.step_function.release("p")
        return best

    def time_e2e(self, batch: int, steps: int, warmup: int):
        """The same decode through the public entry point: host token ids in, sampled ids out; every
        step copies its batch from pinned host memory and reads the sampled tokens back."""
        torch = self.torch
        from llmserver_b200.engine.engine import Engine
        from llmserver_b200.engine.request import RequestStatus

        for request_id in list(self.step_function.computed):
            self.step_function.release(request_id)
        prompt_len = max(1, MEAN_DECODE_CONTEXT - steps // 2 - warmup)
        # the engine shares the model and the cache that are already on the device
        # requests that finish their prompt first decode while the others still prefill: leave room for that
        prefill_steps = -(-batch * prompt_len // max(8192, batch)) + 2
        engine = Engine(self.model, max_new_tokens=warmup + steps + prefill_steps + 8, max_batch_size=batch,
                        max_num_batched_tokens=max(8192, batch), ignore_eos=True, cache=self.cache,
                        step_function=self.step_function)
        requests = [engine.add_request(prompt_token_ids=self.tokens(prompt_len)) for _ in range(batch)]
        while any(request.status != RequestStatus.DECODING for request in requests):
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        before = sum(len(request.generated_token_ids) for request in requests)
        stats_before = dict(engine.stats)
        started = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - started
        generated = sum(len(request.generated_token_ids) for request in requests) - before
        if generated != batch * steps:
            raise RuntimeError(f"the timed steps produced {generated} tokens, not {batch} x {steps}")
        h2d = engine.step_function.last_batch_bytes
        for request in requests:
            engine.cancel_request(request.request_id)
        # where a step's host time goes (mean over the engine's steps; read_back is the wait for the device)
        phases = {name: 1e3 * (engine.stats[name + "_s"] - stats_before[name + "_s"]) / steps
                  for name in ("schedule", "pack_copy", "launch", "read_back", "accept")}
        return {"value": batch * steps / elapsed, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": batch * 4, "ms_per_step": elapsed * 1e3 / steps,
                "host_phases_ms": ", ".join(f"{name} {phases[name]:.3f}" for name in ("schedule", "pack_copy", "launch", "read_back", "accept"))}


