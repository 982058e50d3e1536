"""Ways of cutting the same requests into steps, shared by the replay tests."""
import random


def whole(requests):
    """Each request alone and whole."""
    steps = []
    for rid, tokens in requests.items():
        steps.append({"entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [rid]})
    return steps


def tail_one_by_one(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"entries": [{"id": rid, "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(tokens)):
            steps.append({"entries": [{"id": rid, "tokens": [tokens[i]], "want": [0]}], "end": [rid] if i == len(tokens) - 1 else []})
    return steps


def changing_portions(requests, sizes=(5, 2, 17, 3, 2, 30, 9, 2, 64, 1, 13)):
    """Portions of changing size, down to two tokens (and one)."""
    steps = []
    for rid, tokens in requests.items():
        i = k = 0
        while i < len(tokens):
            take = min(sizes[k % len(sizes)], len(tokens) - i)
            last = i + take == len(tokens)
            steps.append({"entries": [{"id": rid, "tokens": tokens[i:i + take], "want": list(range(take))}],
                          "end": [rid] if last else []})
            i += take
            k += 1
    return steps


def mixed(requests, max_tokens, page, seed=0, max_live=4):
    """Up to ``max_live`` live requests: portions of some beside single tokens of others, some left
    out of a step, new ones admitted as old ones end, under a pool of ``max_tokens`` tokens so that
    pages are used again."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live = {}  # id -> next index
    steps = []

    def rounded(n):
        return (n + 63) // 64 * 64

    while pending or live:
        held = sum(rounded(len(requests[r])) for r in live)
        while pending and len(live) < max_live and held + rounded(len(pending[0][1])) <= max_tokens:
            rid, tokens = pending.pop(0)
            live[rid] = 0
            held += rounded(len(tokens))
        entries, end = [], []
        for rid in list(live):
            tokens, i = requests[rid], live[rid]
            if rng.random() < 0.2 and len(live) > 1:
                continue  # left out of this step
            decoding = i > len(tokens) * 0.6
            take = 1 if decoding and rng.random() < 0.8 else rng.choice([1, 2, 2, 3, 7, 16, 33])
            take = min(take, len(tokens) - i)
            entries.append({"id": rid, "tokens": tokens[i:i + take], "want": list(range(take))})
            live[rid] = i + take
            if live[rid] == len(tokens):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def collect(steps, outputs):
    """outputs[i]: array [wanted, vocab] of step i (or None) -> {id: list of rows in request order}."""
    rows = {}
    for step, out in zip(steps, outputs):
        k = 0
        for e in step["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(out[k])
                k += 1
    return rows
