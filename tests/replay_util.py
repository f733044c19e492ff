"""Builds traces (steps of entries) in the four schedule families and collects the logits
the engine returns per (request, position)."""
import random
from typing import Dict, List, Sequence, Tuple

import torch


def whole(reqs: Dict[str, List[int]]):
    """Each request alone and whole, one step each, every row wanted."""
    recs = []
    for s, (rid, toks) in enumerate(reqs.items()):
        recs.append({"step": s, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                     "end": [rid]})
    return recs


def tail_decoded(reqs: Dict[str, List[int]], tail: int = 32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    recs, s = [], 0
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        recs.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                     "end": []})
        s += 1
        for i in range(head, len(toks)):
            recs.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                         "end": [rid] if i == len(toks) - 1 else []})
            s += 1
        if head == len(toks):
            recs[-1]["end"] = [rid]
    return recs


def portions(reqs: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 16, 3, 2, 31, 5, 2, 64, 2, 9)):
    """Each request alone, cut into portions of changing size, down to two tokens."""
    recs, s = [], 0
    for rid, toks in reqs.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            last = i + n == len(toks)
            recs.append({"step": s, "entries": [{"id": rid, "tokens": toks[i:i + n], "want": list(range(n))}],
                         "end": [rid] if last else []})
            i += n
            s += 1
    return recs


def mixed(reqs: Dict[str, List[int]], max_live: int = 4, seed: int = 0, prefill_frac: float = 0.6):
    """Up to ``max_live`` requests at a time; each first receives ``prefill_frac`` of its
    tokens in portions of random size, then the rest one token a step; portions of some
    requests run beside single tokens of others; a request may sit out a step; a new
    request starts when one ends."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: Dict[str, Tuple[List[int], int]] = {}
    recs, s = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = (toks, 0)
        entries, end = [], []
        for rid in list(live):
            toks, done = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # sits this step out
            split = max(1, int(len(toks) * prefill_frac))
            if done < split:
                n = min(rng.choice([2, 3, 5, 8, 13, 21, 40]), split - done)
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[done:done + n], "want": list(range(n))})
            done += n
            live[rid] = (toks, done)
            if done == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            recs.append({"step": s, "entries": entries, "end": end})
            s += 1
    return recs


def batch_decode(reqs: Dict[str, List[int]], decode_tokens: int, prefill_group: int = 4,
                 portion: int = 24):
    """All requests live at once: their heads go in as prompt portions, ``prefill_group``
    requests a step, then the last ``decode_tokens`` tokens of every request one a step with
    all requests in the same step (a decode step of len(reqs) rows)."""
    recs, s = [], 0
    ids = list(reqs)
    heads = {r: max(1, len(reqs[r]) - decode_tokens) for r in ids}
    for g in range(0, len(ids), prefill_group):
        grp, done = ids[g:g + prefill_group], {}
        while any(done.get(r, 0) < heads[r] for r in grp):
            entries = []
            for r in grp:
                d = done.get(r, 0)
                if d < heads[r]:
                    n = min(portion, heads[r] - d)
                    entries.append({"id": r, "tokens": reqs[r][d:d + n], "want": list(range(n))})
                    done[r] = d + n
            recs.append({"step": s, "entries": entries, "end": []})
            s += 1
    pos = dict(heads)
    while any(pos[r] < len(reqs[r]) for r in ids):
        entries, end = [], []
        for r in ids:
            if pos[r] < len(reqs[r]):
                entries.append({"id": r, "tokens": [reqs[r][pos[r]]], "want": [0]})
                pos[r] += 1
                if pos[r] == len(reqs[r]):
                    end.append(r)
        recs.append({"step": s, "entries": entries, "end": end})
        s += 1
    return recs


def run_records(runner, records, replayer=None, **replayer_args) -> Dict[str, Dict[int, torch.Tensor]]:
    """Runs records in-process through the replay code of the package; returns
    {request: {position: logits row (float32, CPU)}}."""
    from paged_batch_engine_b200.engine.replay import TraceReplayer
    rp = replayer if replayer is not None else TraceReplayer(runner, **replayer_args)
    progress: Dict[str, int] = {}
    out: Dict[str, Dict[int, torch.Tensor]] = {}
    for rec in records:
        logits = rp.run_record(rec)
        rows = logits.float().cpu() if logits is not None else None
        i = 0
        for e in rec["entries"]:
            base = progress.get(e["id"], 0)
            for w in e.get("want", []):
                out.setdefault(e["id"], {})[base + w] = rows[i]
                i += 1
            progress[e["id"]] = base + len(e["tokens"])
        for rid in rec.get("end", []):
            progress.pop(rid, None)
    return out


def max_error(got: Dict[str, Dict[int, torch.Tensor]], want: Dict[str, torch.Tensor]):
    """(largest |difference|, where it is, largest |reference logit|)."""
    worst, where, scale = 0.0, None, 0.0
    for rid, rows in got.items():
        for pos, row in rows.items():
            d = (row - want[rid][pos]).abs().max().item()
            if not (d <= worst):          # also catches NaN
                worst, where = d, (rid, pos)
        scale = max(scale, want[rid].abs().max().item())
    return worst, where, scale


def first_wrong(got, want, tol):
    """The first (request, position) beyond the tolerance: where to start asking what is
    special about the place (a page's edge, the start of a portion, a page used again)."""
    for rid in got:
        for pos in sorted(got[rid]):
            if not ((got[rid][pos] - want[rid][pos]).abs().max().item() <= tol):
                return rid, pos
    return None


def pool_tokens_needed(records, round_to: int = 64) -> int:
    """The most tokens that live requests hold at any time, each request's count rounded
    up to a multiple of ``round_to``: the smallest pool a trace may be given."""
    held, worst = {}, 0
    for rec in records:
        for e in rec["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for rid in rec.get("end", []):
            held.pop(rid, None)
    return worst
