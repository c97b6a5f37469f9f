"""The Malapel decoder as a :class:`ModelSpec`.

The token rows are RMS-normed right after the table (the embedding part's own norm).  Every layer
is the ``pre_norm`` arrangement with norm weights stored as their distance from one
(``weight_offset = 1``).  A span of layers may run several times in a row with the same weights:
the run order names those layers once per pass (each run owns its cache), and before the first
layer of every pass the ``concat_linear`` injection replaces the stream by ``W [x; x0]``, ``x0``
being what the embedding left.  All three mixer types are the ``attention`` part with other
parameters: what a query sees (chunks, everything before it, a sliding window), how scores become
weights (softmax with one more silent member of score 0, softmax, an unnormalised sigmoid with a
bias per head), a norm over the whole q and k projections, key and value widths of their own and a
partial half-split rotation whose angles the kernel forms in fp32.  The feed-forward is the gated
layer with a steeper sigmoid, clamped inputs and a shifted up branch, or ``routed_experts`` with
ungated squared-ReLU experts chosen from the best groups of a softmax router.  Tensor names:
``embed``, ``embed.norm``, ``loop.in``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.malapel import DenseMlp, MalapelConfig, MoeMlp
from ..parts.spec import LayerSpec, ModelSpec, PartSpec
from ..registry import ARCHITECTURES

# constants the design fixes
GATE_SLOPE = 1.702        # the gate is g * sigmoid(GATE_SLOPE * g)
UP_SHIFT = 1.0            # ... times (u + UP_SHIFT)
NORM_OFFSET = 1.0         # a norm's gain is NORM_OFFSET + the stored weight

_MIXER_RULES = {
    "attention": dict(mask="chunk", weights="softmax_plus_one", qk_norm="whole"),
    "attention_2": dict(mask="causal", weights="softmax", qk_norm=False),
    "attention_3": dict(mask="window", weights="sigmoid", qk_norm=False),
}


def build_spec(cfg: MalapelConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms_norm", {"size": width, "eps": eps, "weight_offset": NORM_OFFSET})
    encodings = {}

    def encoding_for(m) -> str:
        params = {"rotary_dim": m.rot_dims, "base": m.rot_base, "pairing": "half_split", "scaling": None}
        for name, ps in encodings.items():
            if ps.params == params:
                return name
        name = f"rot{len(encodings)}"
        encodings[name] = PartSpec("rotary_computed", params)
        return name

    layers = []
    for i, layer in enumerate(cfg.layers):
        m, rules = layer.mixer, _MIXER_RULES[layer.type]
        params = {"hidden_size": width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                  "value_head_dim": m.vdim, "scale": m.scale, "position_encoding": encoding_for(m),
                  "qk_norm": rules["qk_norm"], "qk_norm_eps": eps, "mask": rules["mask"], "weights": rules["weights"],
                  "q_name": "mix.q", "k_name": "mix.k", "v_name": "mix.v", "o_name": "mix.o",
                  "q_norm_name": "mix.q.norm", "k_norm_name": "mix.k.norm", "bias_name": "mix.pb"}
        if rules["mask"] == "chunk":
            params["chunk"] = m.mask_size
        elif rules["mask"] == "window":
            params["window"] = m.mask_size
        mixer = PartSpec("attention", params)
        f = layer.mlp
        if f is None:
            ffn = None
        elif isinstance(f, DenseMlp):
            ffn = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": f.ff, "gate_slope": GATE_SLOPE,
                                      "limit": f.limit, "up_shift": UP_SHIFT, "gate_name": "mlp.gate",
                                      "up_name": "mlp.up", "down_name": "mlp.down"})
        elif isinstance(f, MoeMlp):
            ffn = PartSpec("routed_experts", {
                "hidden_size": width, "expert_size": f.expert_ff, "num_experts": f.experts, "top": f.top,
                "score": "softmax", "renormalize": False, "scale": "output", "weight_scale": f.scale,
                "groups": f.group_count, "groups_kept": f.group_keep, "expert_form": "relu_squared",
                "router_name": "mlp.router", "expert_pattern": "mlp.e{}.{}"})
        else:
            raise TypeError(f"layer {i}: unknown feed-forward {f!r}")
        layers.append(LayerSpec(
            prefix=f"l{i}", block="pre_norm", mixer=mixer, feed_forward=ffn,
            mixer_norm=PartSpec(norm.kind, {**norm.params, "name": "norm1"}),
            ffn_norm=None if ffn is None else PartSpec(norm.kind, {**norm.params, "name": "norm2"})))
    inject = PartSpec("concat_linear", {"hidden_size": width, "name": "loop.in"})
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding_name="embed", layers=tuple(layers), run_order=cfg.run_order(), final_norm=norm,
        final_norm_name="final.norm", lm_head_name="head", position_encodings=encodings,
        embedding=PartSpec("token_embedding", {"name": "embed", "norm": {"name": "embed.norm", "eps": eps,
                                                                          "weight_offset": NORM_OFFSET}}),
        head=PartSpec("linear_head", {"name": "head"}),
        injections=tuple((pos, inject) for pos in cfg.pass_starts()))
    spec.validate()
    return spec


ARCHITECTURES.add(MalapelConfig.ARCHITECTURE, MalapelConfig, build_spec)
