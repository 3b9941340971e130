"""A plain sampler for the tests: Kapel's rules in Python lists and `math`, one value at a time,
sharing no code with the package (whose host sampler is C++).

From crates/kapel-infer/src/sampling.rs: the order of the steps :157-238, the draw :241-260, the first
largest without NaNs :291-299, the softmax in 64-bit with sums in index order :302-310. One rule is
this engine's own: a NaN among the logits makes the softmax all zeros, so the choice falls back to
the first largest that is no NaN ("a NaN never").
"""
import math

NEG_INF = float("-inf")


def plain_argmax(values):
    best = None
    for i, v in enumerate(values):
        if not math.isnan(v) and (best is None or v > values[best]):
            best = i
    return 0 if best is None else best


def plain_softmax(logits):
    if any(math.isnan(v) for v in logits):
        return [0.0] * len(logits)
    m = max(logits, default=NEG_INF)
    if m == NEG_INF:
        return [0.0] * len(logits)
    exps = [0.0 if v == NEG_INF else math.exp(v - m) for v in logits]
    total = 0.0
    for e in exps:
        total += e
    return [e / total for e in exps]


def plain_distribution(logits, temperature=0.0, top_k=None, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
                       frequency_penalty=0.0, presence_penalty=0.0, sequence=(), generated_from=0):
    """(token, None) when the choice is certain, else (None, probabilities)."""
    l = [float(v) for v in logits]
    n = len(l)
    if frequency_penalty != 0.0 or presence_penalty != 0.0:
        counts = {}
        for t in sequence[min(generated_from, len(sequence)):]:
            counts[t] = counts.get(t, 0) + 1
        for t, c in counts.items():
            if 0 <= t < n:
                l[t] -= c * frequency_penalty + presence_penalty
    if repetition_penalty != 1.0:
        for t in set(sequence):
            if 0 <= t < n:
                l[t] = l[t] * repetition_penalty if l[t] < 0 else l[t] / repetition_penalty
    if temperature <= 0.0:
        return plain_argmax(l), None
    l = [v / temperature for v in l]
    if top_k is not None and 0 < top_k < n:
        # descending with NaNs first, as a total order puts them (sampling.rs:197-199)
        ordered = sorted(l, key=lambda v: (0, 0.0) if math.isnan(v) else (1, -v))
        kth = ordered[top_k - 1]
        l = [NEG_INF if v < kth else v for v in l]
    if top_p < 1.0:
        probs = plain_softmax(l)
        order = sorted(range(n), key=lambda i: (-probs[i], i))
        before = 0.0
        for i in order:
            if before >= top_p:
                l[i] = NEG_INF
            before += probs[i]
    if min_p > 0.0:
        probs = plain_softmax(l)
        floor = min_p * max(probs)
        l = [NEG_INF if p < floor else v for v, p in zip(l, probs)]
    probs = plain_softmax(l)
    if not any(p > 0.0 for p in probs):
        return plain_argmax(l), None
    return None, probs


def plain_draw(probs, u):
    total, last = 0.0, 0
    for i, p in enumerate(probs):
        if p > 0.0:
            total += p
            last = i
            if u < total:
                return i
    return last
