"""A plain, slow implementation of the Malapel decoder for the tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 by default.  It
shares no code with ``leone_b200``: it takes the raw ``config.json`` mapping and a dict of
tensors under the checkpoint's names.  Notation: ``h`` is a mixer's or feed-forward's input
``[T, width]``; ``W["foo"]`` is the tensor ``<layer>.mix.foo`` or ``<layer>.mlp.foo``.

The design: the token rows are RMS-normed right after the table (``x0``).  Layers are pre-norm,
``x <- x + mixer(norm1(x))`` then ``x <- x + ff(norm2(x))``, with norm weights stored as their
distance from one.  A span of layers may be run several times in a row with the same weights
(``loop``); before the first layer of every pass the stream is replaced by ``W_in [x; x0]``.
Three attention mixers share projections, grouped key/value heads, separate key and value
widths and a partial half-split rotation, and differ in what a query may see and how scores
become weights: chunks with a softmax that has a silent extra member of score 0, everything
before with an ordinary softmax, a sliding window with an independent sigmoid per key.  The
feed-forward is a clamped gated layer or a mixture of ungated squared-ReLU experts chosen from
the best groups of a softmax router.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


# -- small functions ---------------------------------------------------------------------------
def rms(x, eps):
    """x divided by its root mean square, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_one(x, w, eps):
    """The layer norm of the design: the stored weight is the gain's distance from one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def linear(x, w):
    return x @ w.t()


def relu_squared(z):
    r = torch.clamp(z, min=0)
    return r * r


# -- rotation ----------------------------------------------------------------------------------
def rotate_half_split(x, positions, dims, base, angle_dtype=torch.float32):
    """``x``: [T, heads, dim].  Of the first ``dims`` elements of a head, element i (< dims/2) is
    paired with element i + dims/2; the pair turns by ``position * base^(-2i/dims)``.  Elements
    from ``dims`` on pass unchanged."""
    half = dims // 2
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64).to(angle_dtype)
    ang = torch.as_tensor(positions).to(angle_dtype)[:, None] * f[None, :]
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# -- what a query sees ---------------------------------------------------------------------------
def seen_causal(positions):
    p = torch.as_tensor(positions)
    return p[:, None] >= p[None, :]


def seen_chunked(positions, size):
    """Keys at or before the query that lie in the query's chunk; chunks count from position 0."""
    p = torch.as_tensor(positions)
    return (p[:, None] >= p[None, :]) & ((p[:, None] // size) == (p[None, :] // size))


def seen_window(positions, size):
    """The query itself and the size - 1 positions before it."""
    p = torch.as_tensor(positions)
    gap = p[:, None] - p[None, :]
    return (gap >= 0) & (gap < size)


# -- how scores become weights -------------------------------------------------------------------
def weights_softmax(scores, seen):
    s = scores.masked_fill(~seen, float("-inf"))
    return torch.softmax(s, dim=-1)


def weights_softmax_with_silent_zero(scores, seen):
    """exp(s_j) / (1 + sum exp(s_j)): one more member of score 0 that carries no value."""
    s = scores.masked_fill(~seen, float("-inf"))
    top = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - top)
    return e / (torch.exp(-top) + e.sum(dim=-1, keepdim=True))


def weights_sigmoid(scores, seen, bias):
    """Every seen key on its own: sigmoid(score + bias of the head); nothing is normalised."""
    return torch.sigmoid(scores + bias[:, None, None]) * seen


# -- the attention mixers ------------------------------------------------------------------------
def attention_mixer(h, W, m, kind, eps, positions=None, angle_dtype=torch.float32):
    """``kind``: 'attention' (chunks, whole-projection q/k norms, silent zero), 'attention_2'
    (causal, softmax) or 'attention_3' (window, sigmoid with a per-head bias)."""
    t_len = h.shape[0]
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = list(range(t_len)) if positions is None else positions
    q, k, v = linear(h, W["q"]), linear(h, W["k"]), linear(h, W["v"])
    if kind == "attention":
        # one norm over the whole projection, before the heads are split and before rotation
        q = norm_plain(q, W["q.norm"], eps)
        k = norm_plain(k, W["k.norm"], eps)
    q, k, v = q.view(t_len, heads, dim), k.view(t_len, groups, dim), v.view(t_len, groups, vdim)
    rot = m["rot"]
    q = rotate_half_split(q, positions, rot["dims"], rot["base"], angle_dtype)
    k = rotate_half_split(k, positions, rot["dims"], rot["base"], angle_dtype)
    per = heads // groups
    k = k.repeat_interleave(per, dim=1)
    v = v.repeat_interleave(per, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * m["scale"]
    if kind == "attention":
        w = weights_softmax_with_silent_zero(scores, seen_chunked(positions, m["mask"]["size"])[None])
    elif kind == "attention_2":
        w = weights_softmax(scores, seen_causal(positions)[None])
    elif kind == "attention_3":
        w = weights_sigmoid(scores, seen_window(positions, m["mask"]["size"])[None], W["pb"].to(h.dtype))
    else:
        raise ValueError(kind)
    out = torch.einsum("hts,shv->thv", w, v).reshape(t_len, heads * vdim)
    return linear(out, W["o"])


# -- feed-forwards -----------------------------------------------------------------------------
def dense_ff(h, W, limit):
    """g = min(W_gate h, limit); u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(linear(h, W["gate"]), max=limit)
    u = torch.clamp(linear(h, W["up"]), min=-limit, max=limit)
    return linear(g * torch.sigmoid(1.702 * g) * (u + 1.0), W["down"])


def router_choice(h, W, router):
    """(chosen experts [T, top], their weights [T, top]).  Scores are a softmax over all experts;
    experts form ``groups.count`` runs of neighbours, a run is worth its best score, only the
    ``groups.keep`` best runs may be chosen from; weights are the chosen scores times ``scale``."""
    s = torch.softmax(linear(h, W["router"]), dim=-1)
    experts, top = router["experts"], router["top"]
    allowed = torch.ones_like(s, dtype=torch.bool)
    g = router.get("groups")
    if g:
        count, keep = g["count"], g["keep"]
        worth = s.view(-1, count, experts // count).max(dim=-1).values
        best = torch.topk(worth, keep, dim=-1).indices
        ok = torch.zeros_like(worth, dtype=torch.bool).scatter_(1, best, True)
        allowed = ok.repeat_interleave(experts // count, dim=1)
    val, idx = torch.topk(s.masked_fill(~allowed, -1.0), top, dim=-1)
    return idx, val * router.get("scale", 1.0)


def moe_ff(h, W, mlp):
    idx, wt = router_choice(h, W, mlp["router"])
    out = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t].tolist(), wt[t]):
            out[t] += w * linear(relu_squared(linear(h[t][None], W[f"e{e}.up"])), W[f"e{e}.down"])[0]
    return out


# -- the model ---------------------------------------------------------------------------------
def part_tensors(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def run_order(cfg):
    """[(layer index, first of a pass?)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def layer_forward(x, layer, tensors, i, eps, positions=None, angle_dtype=torch.float32):
    mix = part_tensors(tensors, f"l{i}.mix.")
    x = x + attention_mixer(norm_around_one(x, tensors[f"l{i}.norm1"], eps), mix, layer["mixer"], layer["type"], eps,
                            positions, angle_dtype)
    mlp = layer.get("mlp")
    if mlp is not None:
        h2 = norm_around_one(x, tensors[f"l{i}.norm2"], eps)
        ff = part_tensors(tensors, f"l{i}.mlp.")
        x = x + (dense_ff(h2, ff, mlp["limit"]) if mlp["kind"] == "dense" else moe_ff(h2, ff, mlp))
    return x


class PlainMalapel:
    def __init__(self, cfg, tensors, dtype=DT, angle_dtype=torch.float32):
        self.cfg = cfg
        self.t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.dtype = dtype
        self.angle_dtype = angle_dtype
        self._memo = {}

    def residuals(self, tokens):
        """The residual stream after every layer run, [runs, T, width]."""
        eps = self.cfg["norm"]["eps"]
        x0 = norm_around_one(self.t["embed"][torch.as_tensor(tokens, dtype=torch.long)], self.t["embed.norm"], eps)
        x = x0
        out = []
        for i, first in run_order(self.cfg):
            if first:
                x = linear(torch.cat([x, x0], dim=-1), self.t["loop.in"])
            x = layer_forward(x, self.cfg["layers"][i], self.t, i, eps, angle_dtype=self.angle_dtype)
            out.append(x)
        return torch.stack(out)

    def logits(self, tokens):
        key = tuple(tokens)
        if key not in self._memo:
            x = self.residuals(tokens)[-1]
            x = norm_around_one(x, self.t["final.norm"], self.cfg["norm"]["eps"])
            self._memo[key] = linear(x, self.t["head"])
        return self._memo[key]
