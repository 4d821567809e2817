"""Builders of replay traces: the same requests cut into steps in different ways."""
import random

ROUND = 64


def rounded(count):
    return -(-count // ROUND) * ROUND


def whole(request_id, tokens, step=0):
    return [{"step": step, "entries": [{"id": request_id, "tokens": list(tokens), "want": list(range(len(tokens)))}],
             "end": [request_id]}]


def tail_decoded(request_id, tokens, tail=32, first_step=0):
    """Most of the sequence in one step, the last ``tail`` tokens one by one."""
    head = max(1, len(tokens) - tail)
    records = [{"step": first_step, "entries": [{"id": request_id, "tokens": list(tokens[:head]), "want": list(range(head))}], "end": []}]
    for index in range(head, len(tokens)):
        records.append({"step": first_step + len(records), "entries": [{"id": request_id, "tokens": [tokens[index]], "want": [0]}], "end": []})
    records[-1]["end"] = [request_id]
    return records


def portions(request_id, tokens, sizes, first_step=0):
    """Portions of changing size (cycled), logits wanted everywhere."""
    records, at, turn = [], 0, 0
    while at < len(tokens):
        size = min(sizes[turn % len(sizes)], len(tokens) - at)
        records.append({"step": first_step + len(records),
                        "entries": [{"id": request_id, "tokens": list(tokens[at:at + size]), "want": list(range(size))}], "end": []})
        at += size
        turn += 1
    records[-1]["end"] = [request_id]
    return records


def mixed(requests, seed, max_live=4, sizes=(1, 1, 2, 3, 5, 8, 17, 31), decode_tail=12):
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others; a
    request may sit out a step; requests end and new ones start, so pages are given back and reused.

    ``requests``: dict id -> tokens.  Returns (records, max_tokens) where max_tokens is the peak of
    the sum over live requests of their token counts rounded up to 64."""
    rng = random.Random(seed)
    waiting = list(requests)
    live, fed = [], {}
    records, peak = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            name = waiting.pop(0)
            live.append(name)
            fed[name] = 0
        entries, ended = [], []
        for name in list(live):
            tokens = requests[name]
            left = len(tokens) - fed[name]
            if rng.random() < 0.15 and len(live) > 1:
                continue  # sits this step out
            size = 1 if left <= decode_tail else min(rng.choice(sizes), left - decode_tail) or 1
            piece = tokens[fed[name]:fed[name] + size]
            want = list(range(size)) if rng.random() < 0.7 else sorted(rng.sample(range(size), max(1, size // 2)))
            entries.append({"id": name, "tokens": list(piece), "want": want})
            fed[name] += size
            if fed[name] == len(tokens):
                ended.append(name)
        if not entries:
            continue
        peak = max(peak, sum(rounded(fed[name]) for name in live))
        records.append({"step": len(records), "entries": entries, "end": ended})
        for name in ended:
            live.remove(name)
    return records, peak


def expected_rows(records, requests, logits_of):
    """For each step with wanted places: the rows the plain implementation gives, in trace order.
    ``logits_of(name)`` returns [T, V] for the request's whole token list."""
    import numpy as np

    fed = {}
    out = {}
    for record in records:
        rows = []
        for entry in record["entries"]:
            start = fed.get(entry["id"], 0)
            for place in entry.get("want", []):
                rows.append(logits_of(entry["id"])[start + place])
            fed[entry["id"]] = start + len(entry["tokens"])
        for name in record.get("end", []):
            fed.pop(name, None)
        if rows:
            out[record["step"]] = np.stack(rows)
    return out
