"""The Sarizen decoder as a :class:`ModelSpec`.

Every layer is the ``parallel`` arrangement, ``x <- x + mixer(norm1(x)) + ff(norm2(x))``, and is
described on its own in the configuration, so the spec is built layer by layer: a ``lightning``
layer takes the ``linear_attention`` mixer; a ``latent_attention`` layer the mixer of that name with
a sliding window, per-head sinks, a per-head output gate and an adjacent-pair rotary encoding with
YaRN scaling whose angles the kernel forms in fp32 (one named encoding per distinct set of rotary
constants); the feed-forward is ``mlp`` with a squared ReLU, ``routed_experts`` (sigmoid scores that
scale the chosen experts' inputs, no renormalisation, a shared expert) or absent.  The final norm
is followed by the ``linear_head`` with the configuration's logit scale.  Tensor names:
``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.sarizen import DenseMlp, LatentAttentionMixer, LightningMixer, MoeMlp, SarizenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec
from ..registry import ARCHITECTURES


def build_spec(cfg: SarizenConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms_norm", {"size": width, "eps": eps})
    encodings = {}

    def encoding_for(m: LatentAttentionMixer) -> str:
        s = m.rot_scaling
        params = {"rotary_dim": m.rot_dims, "base": m.rot_base, "pairing": "adjacent",
                  "scaling": None if s is None else {"factor": s.factor, "original": s.original,
                                                     "fast": s.fast, "slow": s.slow}}
        for name, ps in encodings.items():
            if ps.params == params:
                return name
        name = f"rot{len(encodings)}"
        encodings[name] = PartSpec("rotary_computed", params)
        return name

    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, LightningMixer):
            mixer = PartSpec("linear_attention", {
                "hidden_size": width, "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": tuple(m.decay),
                "eps": eps, "q_name": "mix.q", "k_name": "mix.k", "v_name": "mix.v", "g_name": "mix.g",
                "o_name": "mix.o", "norm_name": "mix.norm"})
        elif isinstance(m, LatentAttentionMixer):
            mixer = PartSpec("latent_attention", {
                "hidden_size": width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "window": m.window, "eps": eps, "sink": True, "gate": True,
                "position_encoding": encoding_for(m), "q_name": "mix.q", "dkv_name": "mix.dkv",
                "dkv_norm_name": "mix.dkv.norm", "uk_name": "mix.uk", "uv_name": "mix.uv", "sink_name": "mix.sink",
                "g_name": "mix.g", "o_name": "mix.o"})
        else:
            raise TypeError(f"layer {i}: unknown mixer {m!r}")
        f = layer.mlp
        if f is None:
            ffn = None
        elif isinstance(f, DenseMlp):
            ffn = PartSpec("mlp", {"hidden_size": width, "intermediate_size": f.ff, "activation": "relu_squared",
                                   "up_name": "mlp.up", "down_name": "mlp.down"})
        elif isinstance(f, MoeMlp):
            ffn = PartSpec("routed_experts", {
                "hidden_size": width, "expert_size": f.expert_ff, "num_experts": f.experts, "top": f.top,
                "score": "sigmoid", "renormalize": False, "scale": "input", "shared_size": f.shared_ff,
                "router_name": "mlp.router", "expert_pattern": "mlp.e{}.{}", "shared_pattern": "mlp.shared.{}"})
        else:
            raise TypeError(f"layer {i}: unknown feed-forward {f!r}")
        layers.append(LayerSpec(
            prefix=f"l{i}", block="parallel", mixer=mixer, feed_forward=ffn,
            mixer_norm=PartSpec(norm.kind, {**norm.params, "name": "norm1"}),
            ffn_norm=None if ffn is None else PartSpec(norm.kind, {**norm.params, "name": "norm2"})))
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding_name="embed", layers=tuple(layers), run_order=tuple(range(len(layers))), final_norm=norm,
        final_norm_name="final.norm", lm_head_name="head", position_encodings=encodings,
        head=PartSpec("linear_head", {"name": "head", "logit_scale": cfg.logit_scale}))
    spec.validate()
    return spec


ARCHITECTURES.add(SarizenConfig.ARCHITECTURE, SarizenConfig, build_spec)
