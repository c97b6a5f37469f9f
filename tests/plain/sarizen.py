"""A plain, slow implementation of the Sarizen decoder for the tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 by default.  It
shares no code with ``leone_b200``: it takes the raw ``config.json`` mapping and a dict of
tensors under the checkpoint's names.  Notation: ``h`` is a mixer's or feed-forward's input
``[T, width]``; ``W["foo"]`` is the tensor ``<layer>.mix.foo`` or ``<layer>.mlp.foo``.

The design: every layer is ``x <- x + mixer(norm1(x)) + ff(norm2(x))`` (both branches read the
same ``x``); mixers are a gated linear attention with a per-head decaying state ("lightning")
and a latent attention whose cache is one normed latent vector plus one shared rotated key part
per token, with a sliding window, a per-head softmax sink and a per-head output gate; the
feed-forward is dense with a squared-ReLU or a mixture of gated experts with a sigmoid router
whose scores scale the experts' inputs.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def bf16_round(t):
    return t.to(torch.float32).to(torch.bfloat16).to(t.dtype)


# -- small functions ---------------------------------------------------------------------------
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    r = torch.clamp(z, min=0)
    return r * r


def linear(x, w):
    return x @ w.t()


# -- rotary with YaRN --------------------------------------------------------------------------
def yarn_frequencies(dims, base, scaling, dtype=DT):
    """Per pair i (0 <= i < dims/2): the frequency after YaRN's blend, and the factor that
    multiplies both cos and sin.  ``scaling`` None: plain frequencies, factor 1."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if scaling is None:
        return torch.tensor(f, dtype=dtype), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=dtype), 0.1 * math.log(factor) + 1.0


def rotate_adjacent(x, positions, freqs, magnitude, angle_dtype=torch.float32):
    """``x``: [T, ..., dims]; pair i is elements (2i, 2i+1); angle = position * freq_i.  Angles
    are formed in ``angle_dtype`` (the design computes positions and angles in 32-bit)."""
    pos = torch.as_tensor(positions).to(angle_dtype)
    ang = pos[:, None] * freqs.to(angle_dtype)[None, :]
    cos = (torch.cos(ang) * magnitude).to(x.dtype)
    sin = (torch.sin(ang) * magnitude).to(x.dtype)
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * cos - v * sin
    out[..., 1::2] = v * cos + u * sin
    return out


# -- mixers ------------------------------------------------------------------------------------
def lightning_mixer(h, W, m, eps, state=None):
    """Gated linear attention.  Per head: S_t = decay * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with
    q, k, v = silu of their projections; heads are concatenated, RMS-normed together, multiplied by
    sigmoid(W_g h) and projected.  Returns (output, final state [heads, dim, vdim])."""
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    t_len = h.shape[0]
    q = silu(linear(h, W["q"])).view(t_len, heads, dim)
    k = silu(linear(h, W["k"])).view(t_len, heads, dim)
    v = silu(linear(h, W["v"])).view(t_len, heads, vdim)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    s = torch.zeros(heads, dim, vdim, dtype=h.dtype) if state is None else state.clone()
    outs = []
    for t in range(t_len):
        s = decay[:, None, None] * s + k[t][:, :, None] * v[t][:, None, :]
        outs.append(torch.einsum("hdv,hd->hv", s, q[t]))
    o = torch.stack(outs).reshape(t_len, heads * vdim)
    o = rms_norm(o, W["norm"], eps) * torch.sigmoid(linear(h, W["g"]))
    return linear(o, W["o"]), s


def latent_attention_mixer(h, W, m, eps, positions=None, angle_dtype=torch.float32):
    """Attention through a latent: the cache would hold, per token, the normed latent c and one
    rotated key part shared by all heads; keys and values of a head are W_uk c and W_uv c."""
    heads, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    t_len = h.shape[0]
    positions = list(range(t_len)) if positions is None else positions
    q = linear(h, W["q"]).view(t_len, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    dkv = linear(h, W["dkv"])
    c = rms_norm(dkv[:, :rank], W["dkv.norm"], eps)
    k_rot = dkv[:, rank:]
    rot = m["rot"]
    freqs, magnitude = yarn_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
    rd = rot["dims"]
    q_rot = torch.cat([rotate_adjacent(q_rot[..., :rd], positions, freqs, magnitude, angle_dtype), q_rot[..., rd:]], -1)
    k_rot = torch.cat([rotate_adjacent(k_rot[..., :rd], positions, freqs, magnitude, angle_dtype), k_rot[..., rd:]], -1)
    k_plain = linear(c, W["uk"]).view(t_len, heads, dim)
    value = linear(c, W["uv"]).view(t_len, heads, vdim)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thr,sr->hts", q_rot, k_rot)) * m["scale"]
    pos = torch.as_tensor(positions)
    gap = pos[:, None] - pos[None, :]
    seen = gap >= 0
    window = (m.get("mask") or {}).get("size")
    if window:
        seen = seen & (gap < window)
    scores = scores.masked_fill(~seen[None], float("-inf"))
    sink = W["sink"].to(h.dtype)
    top = torch.maximum(scores.max(dim=-1).values, sink[:, None])
    e = torch.exp(scores - top[..., None])
    weights = e / (e.sum(dim=-1) + torch.exp(sink[:, None] - top))[..., None]
    out = torch.einsum("hts,shv->thv", weights, value)
    out = out * torch.sigmoid(linear(h, W["g"]))[:, :, None]
    return linear(out.reshape(t_len, heads * vdim), W["o"])


# -- feed-forwards -----------------------------------------------------------------------------
def dense_ff(h, W):
    return linear(relu_squared(linear(h, W["up"])), W["down"])


def gated_expert(h, W, prefix):
    return linear(silu(linear(h, W[prefix + "gate"])) * linear(h, W[prefix + "up"]), W[prefix + "down"])


def router_choice(h, W, top):
    """(chosen experts [T, top], their sigmoid scores [T, top])."""
    s = torch.sigmoid(linear(h, W["router"]))
    score, chosen = torch.topk(s, top, dim=-1)
    return chosen, score


def moe_ff(h, W, mlp):
    """sum over the chosen experts of expert(score * h), plus the shared expert on h."""
    chosen, score = router_choice(h, W, mlp["router"]["top"])
    out = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), score[t]):
            out[t] += gated_expert((w * h[t])[None], W, f"e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + gated_expert(h, W, "shared.")
    return out


# -- the model ---------------------------------------------------------------------------------
def part_tensors(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer_forward(x, layer, tensors, i, eps, positions=None, angle_dtype=torch.float32, round_act=None):
    ra = round_act or (lambda t: t)
    mix = part_tensors(tensors, f"l{i}.mix.")
    h1 = ra(rms_norm(x, tensors[f"l{i}.norm1"], eps))
    if layer["type"] == "lightning":
        a, _ = lightning_mixer(h1, mix, layer["mixer"], eps)
    elif layer["type"] == "latent_attention":
        a = latent_attention_mixer(h1, mix, layer["mixer"], eps, positions, angle_dtype)
    else:
        raise ValueError(layer["type"])
    out = x + a
    mlp = layer.get("mlp")
    if mlp is not None:
        h2 = ra(rms_norm(x, tensors[f"l{i}.norm2"], eps))
        ff = part_tensors(tensors, f"l{i}.mlp.")
        out = out + (dense_ff(h2, ff) if mlp["kind"] == "dense" else moe_ff(h2, ff, mlp))
    return out


class PlainSarizen:
    def __init__(self, cfg, tensors, dtype=DT, angle_dtype=torch.float32):
        self.cfg = cfg
        self.t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.dtype = dtype
        self.angle_dtype = angle_dtype
        self._memo = {}

    def residuals(self, tokens):
        """The residual stream after every layer, [layers, T, width]."""
        x = self.t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        eps = self.cfg["norm"]["eps"]
        out = []
        for i, layer in enumerate(self.cfg["layers"]):
            x = layer_forward(x, layer, self.t, i, eps, angle_dtype=self.angle_dtype)
            out.append(x)
        return torch.stack(out)

    def logits(self, tokens):
        key = tuple(tokens)
        if key not in self._memo:
            x = self.residuals(tokens)[-1]
            x = rms_norm(x, self.t["final.norm"], self.cfg["norm"]["eps"])
            self._memo[key] = linear(x, self.t["head"]) * self.cfg["logit_scale"]
        return self._memo[key]
