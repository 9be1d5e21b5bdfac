"""Builders of replay traces for the tests: the same requests cut into steps in different
ways.  A trace is a list of step records in the format ``bin/trace_run`` reads."""

from __future__ import annotations

import random


def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone, the whole sequence in one step."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def tail_one_by_one(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(0, len(toks) - tail)
        if head:
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": [rid] if i == len(toks) - 1 else []})
    return steps


def portions(requests: dict[str, list[int]], sizes=(7, 2, 16, 3, 2, 33, 5, 1, 9)) -> list[dict]:
    """Each request alone, in portions of changing size, down to two tokens (and one)."""
    steps = []
    for k, (rid, toks) in enumerate(requests.items()):
        pos, i = 0, k
        while pos < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - pos)
            i += 1
            last = pos + n == len(toks)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[pos : pos + n], "want": list(range(n))}], "end": [rid] if last else []})
            pos += n
    return steps


def mixed(requests: dict[str, list[int]], prompt_lens: dict[str, int], max_live: int = 4, seed: int = 0) -> list[dict]:
    """Up to ``max_live`` requests live at once: portions of some prompts beside single decoded
    tokens of others in the same step; now and then a request sits a step out; finished
    requests end and later ones take their pages."""
    rng = random.Random(seed)
    waiting = list(requests)
    live: dict[str, int] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            toks, pos = requests[rid], live[rid]
            if len(live) > 1 and rng.random() < 0.15:
                continue  # left out of this step
            if pos < prompt_lens[rid]:
                n = min(rng.choice([2, 3, 5, 8, 13, 21]), prompt_lens[rid] - pos)
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[pos : pos + n], "want": list(range(n))})
            live[rid] = pos + n
            if live[rid] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def last_only(steps: list[dict]) -> list[dict]:
    """The same steps asking for the logits of each entry's last token alone (a step of many
    tokens is replayed as a captured graph only when it wants no more rows than it has sequences)."""
    return [{**s, "entries": [{**e, "want": [len(e["tokens"]) - 1]} for e in s["entries"]]} for s in steps]


def many_decoders(requests: dict[str, list[int]], prompt_lens: dict[str, int], live: int, seed: int = 0, join_p: float = 0.6) -> list[dict]:
    """Steps of many single decoded tokens: ``live`` requests are admitted (their prompts whole, a
    few per step), then every live request decodes one token per step; requests are of different
    lengths, so they leave at different times, and when one has left another joins, its prompt
    beside the decoded tokens of the others, so that the number of sequences moves across the
    sizes a step is padded to.  Logits are wanted for the last token of every entry."""
    rng = random.Random(seed)
    waiting = list(requests)
    pos: dict[str, int] = {}
    steps: list[dict] = []

    def emit(entries, end):
        steps.append({"step": len(steps), "entries": entries, "end": end})

    def advance(rid, n):
        toks, p = requests[rid], pos[rid]
        pos[rid] = p + n
        return {"id": rid, "tokens": toks[p : p + n], "want": [n - 1]}

    first = [waiting.pop(0) for _ in range(min(live, len(waiting)))]
    for i in range(0, len(first), 5):  # prompts, five requests a step
        group = first[i : i + 5]
        for rid in group:
            pos[rid] = 0
        emit([advance(rid, prompt_lens[rid]) for rid in group], [])
    while pos:
        entries, end = [], []
        for rid in list(pos):
            entries.append(advance(rid, 1))
            if pos[rid] == len(requests[rid]):
                end.append(rid)
                del pos[rid]
        joiners = 0
        while waiting and len(entries) < live and rng.random() < join_p and joiners < 2:
            rid = waiting.pop(0)
            pos[rid] = 0
            entries.append(advance(rid, prompt_lens[rid]))
            joiners += 1
        emit(entries, end)
    return steps


def tokens_needed(steps: list[dict], page: int = 64) -> int:
    """Most tokens live requests hold at any time, each request rounded up to ``page``."""
    held: dict[str, int] = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // page) * page for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def wanted_places(steps: list[dict]) -> list[list[tuple[str, int]]]:
    """Per step, the (request, absolute position) of every wanted row, in output order."""
    pos: dict[str, int] = {}
    out = []
    for s in steps:
        rows = []
        for e in s["entries"]:
            start = pos.get(e["id"], 0)
            rows.extend((e["id"], start + i) for i in e.get("want", []))
            pos[e["id"]] = start + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
        out.append(rows)
    return out


def staggered(requests: dict[str, list[int]], prompt_lens: dict[str, int], sizes=(2048, 1024, 3000, 4096)) -> list[dict]:
    """Requests join one after the other: the newcomer's prompt comes in portions of changing
    size while the earlier ones decode one token a step beside it; when every prompt is in, all
    decode together until their tokens are used up.  Logits are wanted for the last token of
    every entry.  Made for long prompts: few steps, each with a long reach into the cache."""
    steps: list[dict] = []
    pos: dict[str, int] = {}
    turn = 0

    def decoders(end):
        entries = []
        for rid in list(pos):
            toks, p = requests[rid], pos[rid]
            if p >= prompt_lens[rid] and p < len(toks):
                entries.append({"id": rid, "tokens": [toks[p]], "want": [0]})
                pos[rid] = p + 1
                if pos[rid] == len(toks):
                    end.append(rid)
        return entries

    for rid, toks in requests.items():
        p = 0
        while p < prompt_lens[rid]:
            end: list[str] = []
            entries = decoders(end)
            n = min(sizes[turn % len(sizes)], prompt_lens[rid] - p)
            turn += 1
            entries.append({"id": rid, "tokens": toks[p : p + n], "want": [n - 1]})
            p += n
            pos[rid] = p
            steps.append({"step": len(steps), "entries": entries, "end": end})
            for r in end:
                del pos[r]
    while pos:
        end = []
        entries = decoders(end)
        steps.append({"step": len(steps), "entries": entries, "end": end})
        for r in end:
            del pos[r]
    return steps
