"""Independent float64 numpy restatement of the sampler specification (test helper).

Written from the specification, not from the C oracle: plain sorts and cumulative sums in
float64.  It is the second implementation of the one spec; where its decision differs from
the oracle's the row must be one the oracle flags as near a cutoff (or a tie in float64).
"""
import numpy as np


def bf16_to_f32(h):
    return (h.astype(np.uint32) << np.uint32(16)).view(np.float32)


def prepare(logits, p, mask=None, history=None):
    z = logits.astype(np.float32).copy()
    V = z.size
    rep = np.float32(p.get("repetition_penalty", 0.0))
    f = np.float32(p.get("frequency_penalty", 0.0))
    pr = np.float32(p.get("presence_penalty", 0.0))
    rep_on = rep not in (0.0, 1.0)
    add_on = (f != 0) or (pr != 0)
    if history is not None and (rep_on or add_on):
        ids, cnt = np.unique(history[(history >= 0) & (history < V)], return_counts=True)
        for t, c in zip(ids, cnt):
            v = z[t]
            if rep_on:
                v = np.float32(v / rep) if v > 0 else np.float32(v * rep)
            if add_on:
                pen = np.float32(np.float32(f * np.float32(c)) + pr)
                v = np.float32(v - pen)
            z[t] = v
    if mask is not None:
        bits = np.unpackbits(mask.view(np.uint8), bitorder="little")[:V].astype(bool)
        z[~bits] = -np.inf
    return z


def sample_row(logits, p, u, mask=None, history=None, segments=1):
    """Returns (token, prob, kept ids in rank order, lse) in float64 arithmetic."""
    z = prepare(logits, p, mask, history)
    V = z.size
    if np.isnan(z).any():
        return -1, 0.0, [], np.nan
    m = z.max()
    if m == np.inf or m == -np.inf:
        return -1, 0.0, [], np.nan
    greedy = bool(p.get("greedy", False)) or p.get("temperature", 0.0) == 0.0
    inv_T = 1.0 if greedy else 1.0 / float(np.float32(p["temperature"]))
    zd = z.astype(np.float64)
    lse = m * inv_T + np.log(np.exp((zd - m) * inv_T).sum())
    if greedy:
        t = int(np.argmax(z))
        return t, 1.0, [t], lse
    order = np.lexsort((np.arange(V), -zd))  # value desc, index asc
    order = order[np.isfinite(zd[order])]
    k = int(p.get("top_k", 0))
    if k > 0:
        if segments > 1:
            seg = V // segments
            sel = []
            for g in range(segments):
                lo, hi = g * seg, (V if g == segments - 1 else (g + 1) * seg)
                o = order[(order >= lo) & (order < hi)][:k]
                sel.append(o)
            sel = np.concatenate(sel)
            order = sel[np.lexsort((sel, -zd[sel]))]
        else:
            order = order[:k]
    w = np.exp((zd[order] - m) * inv_T)
    a = float(np.float32(p.get("min_p", 0.0)))
    if a > 0:
        keep = w >= a
        order, w = order[keep], w[keep]
    P = float(np.float32(p.get("top_p", 0.0)))
    if 0 < P < 1:
        c = np.cumsum(w)
        n = int(np.searchsorted(c, P * c[-1], side="left")) + 1
        n = min(max(n, 1), len(order))
        order, w = order[:n], w[:n]
    idx = np.argsort(order)
    oi, wi = order[idx], w[idx]
    c = np.cumsum(wi)
    tgt = float(u) * c[-1]
    pos = int(np.searchsorted(c, tgt, side="right"))
    pos = min(pos, len(oi) - 1)
    return int(oi[pos]), float(wi[pos] / c[-1]), [int(t) for t in order], lse
