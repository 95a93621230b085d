"""What the replay tests share: how a trace is run through the replayer, the plain implementation's exact and
bfloat16-rounded logits, and the comparison that decides whether the engine's logits are right."""
from __future__ import annotations

import torch

import plain_qwen3 as plain

# float32: the engine against the plain implementation, both in 32-bit on the same weights: 1e-4, the reference's own
# bound for its CPU engine (plugins/tests/test_qwen3_cpu.py:24). bfloat16 has no fixed bound: the yardstick is how far
# the plain implementation itself moves when its intermediate results are rounded to bfloat16 where the reference's
# pipeline rounds them (`plain.rounding`). The engine may differ from the exact logits by at most twice that in the
# largest element and 1.5 times that on average, the way the reference's judge holds an engine to twice the distance
# of a plain bfloat16 run (judge/README.md:64-67).
TOLERANCE = 1e-4
BF16_MAX, BF16_MEAN = 2.0, 1.5


def exact_and_rounded(config, weights, ids):
    exact = plain.forward(config, weights, ids)
    with plain.rounding(torch.bfloat16):
        return exact, plain.forward(config, weights, ids)


def run(replayer, steps):
    """{(request id, position): logits row} over all steps of a trace."""
    got, at = {}, {}
    for number, (entries, end) in enumerate(steps):
        record = {"step": number, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}
                                              for rid, toks in entries], "end": end}
        logits = replayer.step(record)
        rows = logits.float().cpu() if logits is not None else None
        k = 0
        for rid, toks in entries:
            for _ in toks:
                got[(rid, at.get(rid, 0))] = rows[k]
                at[rid] = at.get(rid, 0) + 1
                k += 1
        for rid in end:
            at.pop(rid, None)
        replayer.built.cache.check()
    return got


def compare(got, want, dtype):
    """`got`: {(request, position): logits row}; `want`: {request: (exact logits, plain bfloat16 logits)}. float32:
    every element within TOLERANCE and every arg max the same. bfloat16: request by request, the engine's largest and
    mean distance from the exact logits against those of the plain bfloat16 run over the same positions (a bound over
    all requests at once would let a wrong row pass under another row's rounding)."""
    by_request: dict = {}
    for (rid, pos), row in got.items():
        by_request.setdefault(rid, []).append((pos, row))
    for rid, rows in by_request.items():
        exact = want[rid][0]
        ours = torch.stack([(row - exact[pos]).abs() for pos, row in rows])
        if dtype == "float32":
            assert ours.max() <= TOLERANCE, f"{rid}: largest logit difference {float(ours.max())}"
            for pos, row in rows:
                assert int(row.argmax()) == int(exact[pos].argmax()), (rid, pos)
            continue
        floor = torch.stack([(want[rid][1][pos] - exact[pos]).abs() for pos, _ in rows])
        assert ours.max() <= BF16_MAX * floor.max(), \
            f"{rid}: largest difference {float(ours.max())}, plain bfloat16 {float(floor.max())}"
        assert ours.mean() <= BF16_MEAN * floor.mean(), \
            f"{rid}: mean difference {float(ours.mean())}, plain bfloat16 {float(floor.mean())}"


def portions(ids, sizes):
    out, at, i = [], 0, 0
    while at < len(ids):
        n = min(sizes[i % len(sizes)], len(ids) - at)
        out.append(ids[at:at + n])
        at, i = at + n, i + 1
    return out




def mixed_trace(prompts):
    """Four requests r0 .. r3 (70, 133, 37 and 96 tokens) live at once in 448 tokens of pool (7 pages of 64): r1, r2
    and r3 arrive in portions while r0 decodes; when r0 ends, r3 grows into a page that r0 gave back."""
    p = prompts
    steps = [
        ([("r0", p["r0"][:38]), ("r1", p["r1"][:50])], []),
        ([("r0", p["r0"][38:39]), ("r1", p["r1"][50:90]), ("r2", p["r2"][:2])], []),
    ]
    at = {"r0": 39, "r1": 90, "r2": 2, "r3": 0}
    while at["r0"] < len(p["r0"]):                    # r0 decodes; r1, r2 and r3 bring small portions beside it
        entries, end = [], []
        for rid, n in (("r0", 1), ("r1", 3), ("r2", 2), ("r3", 2)):
            if at[rid] < len(p[rid]):
                entries.append((rid, p[rid][at[rid]:at[rid] + n]))
                at[rid] = min(len(p[rid]), at[rid] + n)
                if at[rid] == len(p[rid]):
                    end.append(rid)
        steps.append((entries, end))
    assert at["r3"] == 62                                            # four live requests filled all seven pages
    while any(at[rid] < len(p[rid]) for rid in ("r1", "r2", "r3")):   # r3 arrives in r0's pages; the others decode
        entries, end = [], []
        for rid, n in (("r1", 1), ("r2", 1), ("r3", 29)):
            if at[rid] < len(p[rid]):
                entries.append((rid, p[rid][at[rid]:at[rid] + n]))
                at[rid] = min(len(p[rid]), at[rid] + n)
                if at[rid] == len(p[rid]):
                    end.append(rid)
        steps.append((entries, end))
    return steps
