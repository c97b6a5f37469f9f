"""Gated linear attention with a decaying state per head ("lightning" attention).

``q, k = silu(W_q x), silu(W_k x)`` (heads x dim), ``v = silu(W_v x)`` (heads x vdim); per head
``S_t = decay_h S_(t-1) + k_t v_t^T`` and ``o_t = S_t^T q_t`` with no other scale; the heads of a
token, concatenated, are RMS-normed together with a weight, multiplied by ``sigmoid(W_g x)`` and
projected by ``W_o`` onto the residual stream.  The state ``[heads, dim, vdim]`` is fp32, starts at
zero and lives in the request's state slot between steps.  Every size, the decay factors and the
norm's eps are parameters.
"""
from __future__ import annotations

import torch

from ..registry import MIXERS
from .base import FixedState, Mixer, WeightSpec


@MIXERS.register("linear_attention")
class DecayLinearAttention(Mixer):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.decay_values = [float(d) for d in params["decay"]]
        if len(self.decay_values) != self.heads:
            raise ValueError(f"{len(self.decay_values)} decay factors for {self.heads} heads")
        self.eps = float(params["eps"])
        self.names = {k: params.get(f"{k}_name", k) for k in ("q", "k", "v", "g", "o", "norm")}
        # prompt portions longer than this are cut into chunks that run side by side
        self.chunk = int(params.get("chunk", 64))
        self.qk = self.heads * self.dim
        self.hv = self.heads * self.vdim
        self.cols = 2 * self.qk + 2 * self.hv
        self.w_in = self.w_o = self.norm_w = self.decay = None

    def weight_specs(self):
        n = self.names
        return [WeightSpec(n["q"], (self.qk, self.hidden)), WeightSpec(n["k"], (self.qk, self.hidden)),
                WeightSpec(n["v"], (self.hv, self.hidden)), WeightSpec(n["g"], (self.hv, self.hidden)),
                WeightSpec(n["o"], (self.hidden, self.hv)), WeightSpec(n["norm"], (self.hv,), role="norm", std=0.1)]

    def load(self, tensors):
        n = self.names
        stacked = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]]], dim=0).contiguous()
        self.w_in = self.rt.ops.prepare_matrix(stacked)
        self.w_o = self.rt.ops.prepare_matrix(tensors[n["o"]])
        self.norm_w = tensors[n["norm"]]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(self.rt.device)

    def weight_bytes(self):
        return (self.cols * self.hidden + self.hidden * self.hv) * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        chunks = max_tokens // max(self.chunk, 1) + 1
        return max_tokens * (self.cols * self.rt.dtype.itemsize + self.hv * (4 + self.rt.dtype.itemsize)) \
            + chunks * self.heads * self.dim * self.vdim * 4

    def load_transient_bytes(self):
        return self.cols * self.hidden * self.rt.dtype.itemsize

    def cache_request(self):
        return FixedState((self.heads, self.dim, self.vdim))

    def forward(self, ctx, cache, x, hidden):
        rt = self.rt
        n = hidden.shape[0]
        proj = rt.buffer("linattn_proj", n, self.cols, rt.dtype)
        rt.ops.linear(x, self.w_in, proj)
        o = rt.buffer("linattn_o", n, self.hv, torch.float32)
        # a captured step has one token per sequence; otherwise long portions run chunk-parallel
        chunk = 0
        if not ctx.decode_only and self.chunk > 0 and ctx.max_q_len > 2 * self.chunk:
            chunk = self.chunk
        rt.ops.linear_attention(ctx, proj, o, cache.state, self.decay, self.heads, self.dim, self.vdim,
                                q_off=0, k_off=self.qk, v_off=2 * self.qk, chunk=chunk)
        gated = rt.buffer("linattn_gated", n, self.hv, rt.dtype)
        rt.ops.gate_norm(o, self.norm_w, proj[:, 2 * self.qk + self.hv:], gated, self.eps)
        rt.ops.linear(gated, self.w_o, hidden, residual=hidden)
