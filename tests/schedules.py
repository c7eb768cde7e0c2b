"""Ways of cutting the same requests into steps.  A schedule is a list of steps; a step is
(entries, end) with entries = [(request id, first token index, number of tokens)]."""


def whole(reqs):
    """Each request alone and whole."""
    return [([(rid, 0, len(toks))], [rid]) for rid, toks in reqs.items()]


def last_one_by_one(reqs, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in reqs.items():
        n = len(toks)
        head = max(1, n - tail)
        steps.append(([(rid, 0, head)], []))
        for p in range(head, n):
            steps.append(([(rid, p, 1)], [rid] if p == n - 1 else []))
        if head == n:
            steps[-1] = (steps[-1][0], [rid])
    return steps


def changing_portions(reqs, sizes=(7, 2, 13, 1, 5, 3, 29, 2, 16, 4, 64, 2, 11)):
    """Each request alone, in portions of changing size, down to two tokens and one."""
    steps = []
    for rid, toks in reqs.items():
        p, i = 0, 0
        while p < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - p)
            i += 1
            steps.append(([(rid, p, n)], [rid] if p + n == len(toks) else []))
            p += n
    return steps


def mixed(reqs, max_live=4, sizes=(9, 2, 17, 1, 6, 3, 24, 2, 12, 5), decode_tail=6):
    """Up to ``max_live`` requests at a time; each is fed in portions of changing size and its last
    ``decode_tail`` tokens one at a time, so portions of some stand beside single tokens of others; when
    one ends the next is admitted and takes over its pages."""
    waiting = list(reqs.items())
    live, steps, i = {}, [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0]
        entries, end = [], []
        for k, (rid, st) in enumerate(list(live.items())):
            toks, p = st
            if (len(steps) + k) % 5 == 4 and len(live) > 1:
                continue                       # a request may be left out of a step and go on later
            left = len(toks) - p
            n = 1 if left <= decode_tail else min(sizes[i % len(sizes)], left - decode_tail)
            i += 1
            entries.append((rid, p, n))
            st[1] = p + n
            if st[1] == len(toks):
                end.append(rid)
        for rid in end:
            del live[rid]
        if entries:
            steps.append((entries, end))
    return steps


def peak_tokens(reqs, steps, round_to=64):
    """Most tokens live requests hold at any time, each rounded up to a multiple of ``round_to``."""
    held, peak = {}, 0
    for entries, end in steps:
        for rid, p, n in entries:
            held[rid] = p + n
        peak = max(peak, sum(-(-v // round_to) * round_to for v in held.values()))
        for rid in end:
            held.pop(rid, None)
    return peak
