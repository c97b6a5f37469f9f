"""Dense two-matrix feed-forward: ``hidden += W_down act(W_up x)``.

``activation``: ``"relu_squared"`` (``max(z, 0)^2``).  The gated three-matrix layer is the
``swiglu`` part.
"""
from __future__ import annotations

from ..registry import FEED_FORWARDS
from .base import FeedForward, WeightSpec

ACTIVATIONS = ("relu_squared",)


@FEED_FORWARDS.register("mlp")
class Mlp(FeedForward):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params.get("activation", "relu_squared")
        if self.activation not in ACTIVATIONS:
            raise ValueError(f"mlp activation '{self.activation}' is not one of {ACTIVATIONS}")
        self.up_name = params.get("up_name", "up")
        self.down_name = params.get("down_name", "down")
        self.w_up = self.w_down = None

    def weight_specs(self):
        return [WeightSpec(self.up_name, (self.inter, self.hidden)), WeightSpec(self.down_name, (self.hidden, self.inter))]

    def load(self, tensors):
        self.w_up = self.rt.ops.prepare_matrix(tensors[self.up_name])
        self.w_down = self.rt.ops.prepare_matrix(tensors[self.down_name])

    def weight_bytes(self):
        return 2 * self.inter * self.hidden * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        return max_tokens * self.inter * self.rt.dtype.itemsize

    def forward(self, ctx, x, hidden):
        ops = self.rt.ops
        act = self.rt.buffer("mlp_act", hidden.shape[0], self.inter, self.rt.dtype)
        ops.linear(x, self.w_up, act)
        ops.relu_squared(act)
        ops.linear(act, self.w_down, hidden, residual=hidden)
