"""Builders of replay traces: the same requests cut in different ways.

A trace is a list of step records as `bin/trace_run` reads them. Each builder also returns,
per written step, which (request, position) every output row is, so that a test can compare
each row with the plain implementation's logits at that position.
"""

from __future__ import annotations


class TraceBuilder:
    def __init__(self):
        self.steps: list[dict] = []
        self.rows: dict[int, list[tuple[str, int]]] = {}
        self.fed: dict[str, int] = {}

    def step(self, entries: list[tuple[str, list[int], list[int]]], end=()) -> None:
        """entries: (request id, its next tokens, wanted places among them)."""
        n = len(self.steps)
        record = {"step": n, "entries": [], "end": list(end)}
        rows = []
        for rid, tokens, want in entries:
            start = self.fed.get(rid, 0)
            record["entries"].append({"id": rid, "tokens": list(tokens), "want": list(want)})
            rows += [(rid, start + w) for w in want]
            self.fed[rid] = start + len(tokens)
        for rid in end:
            self.fed.pop(rid, None)
        self.steps.append(record)
        if rows:
            self.rows[n] = rows


def whole(requests: dict[str, list[int]]) -> TraceBuilder:
    """Each request alone and whole: one step, every position wanted."""
    tb = TraceBuilder()
    for rid, ids in requests.items():
        tb.step([(rid, ids, list(range(len(ids))))], end=[rid])
    return tb


def prefill_then_decode(requests: dict[str, list[int]], n_decode: int = 32) -> TraceBuilder:
    """Most of a request in one step, the last `n_decode` tokens one by one."""
    tb = TraceBuilder()
    for rid, ids in requests.items():
        head = max(1, len(ids) - n_decode)
        tb.step([(rid, ids[:head], list(range(head)))])
        for i in range(head, len(ids)):
            tb.step([(rid, [ids[i]], [0])], end=[rid] if i == len(ids) - 1 else [])
        if head == len(ids):
            tb.step([], end=[rid])
    return tb


def portions(requests: dict[str, list[int]], sizes=(48, 7, 2, 16, 3, 2, 29, 5)) -> TraceBuilder:
    """Portions of changing size, down to two tokens; every position wanted."""
    tb = TraceBuilder()
    for rid, ids in requests.items():
        at, k = 0, 0
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            if len(ids) - at - n == 1:  # never leave a single token for a "portion": take it too
                n += 1
            last = at + n == len(ids)
            tb.step([(rid, ids[at: at + n], list(range(n)))], end=[rid] if last else [])
            at += n
            k += 1
    return tb


def mixed(requests: dict[str, list[int]], max_live: int = 4, chunk_sizes=(24, 5, 2, 11, 40, 3),
          n_decode: int = 12) -> TraceBuilder:
    """Up to `max_live` requests at a time: portions of some beside single decoded tokens of
    others; a request that ends frees its pages and the next one starts in them."""
    tb = TraceBuilder()
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live[rid] = {"ids": ids, "at": 0}
        entries, ended = [], []
        for rid, st in live.items():
            ids, at = st["ids"], st["at"]
            left = len(ids) - at
            if left <= n_decode:  # the tail of a request goes one token at a time
                n = 1
            else:
                n = min(chunk_sizes[k % len(chunk_sizes)], left - n_decode)
                k += 1
            if k % 7 == 3 and len(live) > 1 and left > n_decode:
                continue  # this request sits the step out and goes on later
            entries.append((rid, ids[at: at + n], list(range(n))))
            st["at"] = at + n
            if st["at"] == len(ids):
                ended.append(rid)
        k += 1
        tb.step(entries, end=ended)
        for rid in ended:
            del live[rid]
    return tb


def with_last_only(tb: TraceBuilder) -> TraceBuilder:
    """The same steps with only each entry's last token wanted: the one logit row per entry that
    generation computes, and so what a step that runs as a CUDA graph can return."""
    out = TraceBuilder()
    for record in tb.steps:
        out.step([(e["id"], e["tokens"], [len(e["tokens"]) - 1]) for e in record["entries"]], end=record["end"])
    return out


def peak_pages(tb: TraceBuilder, page_size: int) -> int:
    """The most pages that the live requests hold at the same time: a request holds
    ceil(tokens fed so far / page_size) pages from its first step to the step that ends it."""
    fed: dict[str, int] = {}
    peak = 0
    for record in tb.steps:
        for entry in record["entries"]:
            fed[entry["id"]] = fed.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-n // page_size) for n in fed.values()))
        for rid in record["end"]:
            fed.pop(rid, None)
    return peak


def max_live(tb: TraceBuilder) -> int:
    live: set[str] = set()
    most = 0
    for record in tb.steps:
        live |= {e["id"] for e in record["entries"]}
        most = max(most, len(live))
        live -= set(record["end"])
    return most


def page_traffic(tb: TraceBuilder, page_size: int, num_pages: int) -> dict[int, list[str]]:
    """Which requests hold each page, in order, when the trace runs over the cache manager with a
    pool of `num_pages` pages (no GPU): page -> its owners one after the other."""
    from research_2_b200.cache import CacheManager, GroupSpec

    cache = CacheManager([GroupSpec(page_size, 0, num_pages)], max(1, max_live(tb)), 1 << 20)
    slots: dict[str, int] = {}
    fed: dict[str, int] = {}
    owners: dict[int, list[str]] = {}
    for record in tb.steps:
        for entry in record["entries"]:
            rid = entry["id"]
            if rid not in slots:
                slots[rid] = min(set(range(cache.max_requests)) - set(slots.values()))
                cache.open(slots[rid])
                fed[rid] = 0
            cache.reserve(slots[rid], fed[rid], fed[rid] + len(entry["tokens"]))
            fed[rid] += len(entry["tokens"])
            for page in cache.table(slots[rid]):
                if page and (page not in owners or owners[int(page)][-1] != rid):
                    owners.setdefault(int(page), []).append(rid)
        for rid in record["end"]:
            if rid in slots:
                cache.close(slots.pop(rid))
                del fed[rid]
    return owners
