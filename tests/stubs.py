"""A stub model for scheduler and engine tests without a GPU: it follows the DecoderModel interface,
keeps no weights, and returns logits that make the greedy token a known function of the input."""
import torch

from llmserver_b200.cache import KVPagesNeed
from llmserver_b200.config.spec import ModelSpec, PartSpec
from llmserver_b200.parts import Runtime

VOCAB = 50


class StubModel:
    """Next token = (last token of the row + 1 + position) % VOCAB: depends on the token and on how
    many tokens precede it, so a wrong position or a token fed twice shows in the output."""

    def __init__(self, max_positions=None, eos=()):
        self.runtime = Runtime(torch.float32, torch.device("cpu"))
        self.spec = ModelSpec(architecture="Stub", vocab_size=VOCAB, hidden_size=4, layers=[], schedule=[], positions={},
                              final_norm=PartSpec.of("none"), max_positions=max_positions, eos_token_ids=tuple(eos))
        self.batches = []

    def cache_needs(self):
        return [KVPagesNeed(1, 2, None)]

    def bind_cache(self, cache):
        self.cache = cache

    def step(self, batch):
        self.batches.append(batch)
        logits = torch.zeros((batch.n_logits, VOCAB))
        for out_row, token_row in enumerate(batch.logit_rows.tolist()):
            token = int(batch.token_ids[token_row])
            position = int(batch.positions[token_row])
            logits[out_row, (token + 1 + position) % VOCAB] = 1.0
        return logits


def expected_generation(prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append((tokens[-1] + 1 + len(tokens) - 1) % VOCAB)
    return tokens[len(prompt):]


class ArgmaxSampler:
    def __call__(self, logits, rows):
        return torch.argmax(logits, dim=-1).tolist()
