"""The Malapel decoder through the engine against the plain implementation (tests/plain/malapel.py).

Without a GPU the engine runs on the stand-in kernels (tests/emulated_ops.py), which checks the
configuration, the model description, the loop's run order and injections, the parts' use of the
cache, and the step function's cutting and batching; on a B200 the same traces run on the CUDA
kernels in 32-bit and in bfloat16, together with tests that aim at single mechanisms."""
import copy
import os

import numpy as np
import pytest
import torch

from leone_b200.engine.engine import Engine
from leone_b200.registry import config_from_dict, spec_from_config
from tests import replay
from tests.malapel_tiny import PAGE_TOKENS, TINY, as_bf16, dense, layer, mixer, moe, tiny_config, tiny_tensors
from tests.plain import malapel as plain

FP32 = dict(rtol=3e-5, atol_scale=3e-5)
# bfloat16: the gained weights make scores and routers sharp, which also amplifies rounding; the 32-bit
# runs are the sharp tests, these catch a wrong path or operand
BF16 = dict(rtol=1e-1, atol_scale=1e-1)
LENGTHS = [40, 7, 75, 33, 1, 64, 50]


def _plain(which, tensors, bf16=False, raw=None):
    return plain.PlainMalapel(raw or TINY[which], as_bf16(tensors) if bf16 else tensors)


def _engine(which, tensors, dtype, device, ops=None, max_tokens=512, page=None, raw=None, **kw):
    spec = spec_from_config(config_from_dict(raw) if raw is not None else tiny_config(which))
    return Engine(spec, dict(tensors), dtype=dtype, device=device, ops=ops, page_tokens=page or PAGE_TOKENS[which],
                  max_tokens=max_tokens, max_requests=kw.pop("max_requests", 4),
                  max_batch_tokens=kw.pop("max_batch_tokens", 128), **kw)


def _requests(vocab, lengths=LENGTHS, seed=100):
    return {f"r{i}": replay.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


def _traces(reqs):
    return {"whole": replay.trace_whole(reqs), "tail": replay.trace_decode_tail(reqs, tail=20),
            "portions": replay.trace_portions(reqs), "mixed": replay.trace_mixed(reqs, seed=3)}


def _one_layer(kind, m, mlp=None, vocab=64, width=32, loop=None):
    raw = {"architecture": "Malapel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
           "layers": [layer(kind, m, mlp)]}
    if loop:
        raw["loop"] = loop
    return raw


def _random(raw, seed, gain=5.0):
    from leone_b200.engine.model import weight_specs_for_config
    from leone_b200.weights.random_init import random_tensors
    tensors = random_tensors(weight_specs_for_config(config_from_dict(raw)), seed)
    return {k: (v * gain if v.dim() == 2 and k != "loop.in" else (v * 25.0 if k == "loop.in" else v))
            for k, v in tensors.items()}


# -- configuration and description (CPU) ---------------------------------------------------------
def test_config_round_trip_and_spec():
    for which, raw in TINY.items():
        cfg = config_from_dict(raw)
        assert cfg.to_json_dict() == raw
        spec = spec_from_config(cfg)
        assert all(ls.mixer.kind == "attention" and ls.block == "pre_norm" for ls in spec.layers)
        assert [ls.feed_forward is None for ls in spec.layers] == [e["mlp"] is None for e in raw["layers"]]
        assert [(i, pos in dict(spec.injections)) for pos, i in enumerate(spec.run_order)] == plain.run_order(raw)


def test_run_order_of_loops():
    cfg = tiny_config("A")
    assert cfg.run_order() == (0, 1, 0, 1, 0, 1, 2, 3) and cfg.pass_starts() == (0, 2, 4)
    cfg = tiny_config("B")
    assert cfg.run_order() == (0, 1, 1, 2, 3) and cfg.pass_starts() == (1, 2)
    assert tiny_config("C").run_order() == (0, 1, 2, 3) and tiny_config("C").pass_starts() == ()
    assert tiny_config("D").run_order() == (0, 1, 2) and tiny_config("D").pass_starts() == (0,)


def test_config_rejections():
    from leone_b200.config.base import ConfigError
    for patch in (lambda c: c["layers"][0]["mixer"].update(kv_heads=4),
                  lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3),
                  lambda c: c["layers"][0]["mixer"].pop("mask"),
                  lambda c: c["layers"][0].update(type="conv"),
                  lambda c: c["layers"][1]["mlp"]["router"].update(top=5),
                  lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4),
                  lambda c: c["layers"][0]["mlp"].pop("limit"),
                  lambda c: c["loop"].update(stop=9), lambda c: c["loop"].update(start=2),
                  lambda c: c.pop("width"), lambda c: c.update(layers=[])):
        raw = copy.deepcopy(TINY["A"])
        patch(raw)
        with pytest.raises(ConfigError):
            config_from_dict(raw)


# -- the plain implementation's own mechanisms, against their definitions (CPU) -----------------------
def test_plain_masks_and_weight_rules():
    pos = list(range(10))
    assert plain.seen_window(pos, 3)[5].tolist() == [False] * 3 + [True] * 3 + [False] * 4
    assert plain.seen_chunked(pos, 4)[5].tolist() == [False] * 4 + [True] * 2 + [False] * 4
    assert plain.seen_chunked(pos, 4)[4].tolist() == [False] * 4 + [True] + [False] * 5
    s = torch.tensor([[0.3, -1.0, 2.0]], dtype=torch.float64)
    seen = torch.tensor([[True, True, False]])
    w = plain.weights_softmax_with_silent_zero(s, seen)
    e = torch.exp(s[0, :2])
    assert torch.allclose(w[0, :2], e / (1 + e.sum())) and w[0, 2] == 0
    # the weights sum to less than one, by the silent member's share; large scores of either sign are safe
    w = plain.weights_softmax_with_silent_zero(torch.tensor([[5.0, 4.0]], dtype=torch.float64), torch.tensor([[True, True]]))
    assert abs(float(w.sum()) - (1.0 - 1.0 / (1.0 + np.exp(5.0) + np.exp(4.0)))) < 1e-12
    for big in (800.0, -800.0):
        w = plain.weights_softmax_with_silent_zero(torch.tensor([[big]], dtype=torch.float64), torch.tensor([[True]]))
        assert float(w) == (1.0 if big > 0 else 0.0)
    w = plain.weights_sigmoid(s[None], seen[None], torch.tensor([0.5], dtype=torch.float64))
    assert torch.allclose(w[0, 0, :2], torch.sigmoid(s[0, :2] + 0.5)) and w[0, 0, 2] == 0


def test_plain_router_groups():
    # 6 experts in 3 groups worth 0.30, 0.25 and 0.20; two are kept: expert 4 (0.20) cannot be chosen
    # although it scores above expert 0 (0.05), which can
    z = torch.log(torch.tensor([[0.05, 0.30, 0.25, 0.02, 0.20, 0.18]], dtype=torch.float64))
    W = {"router": torch.eye(6, dtype=torch.float64)}
    idx, wt = plain.router_choice(z, W, {"experts": 6, "top": 3, "scale": 2.0, "groups": {"count": 3, "keep": 2}})
    assert idx.tolist() == [[1, 2, 0]] and torch.allclose(wt, torch.tensor([[0.6, 0.5, 0.1]], dtype=torch.float64))
    idx, wt = plain.router_choice(z, W, {"experts": 6, "top": 3, "scale": 1.0})
    assert idx.tolist() == [[1, 2, 4]] and torch.allclose(wt, torch.tensor([[0.3, 0.25, 0.2]], dtype=torch.float64))


# -- the step function on stand-in kernels (CPU) ------------------------------------------------
@pytest.mark.parametrize("which", ["A", "B", "D"])
@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_replay_on_stand_in_kernels(which, mode):
    from tests.emulated_ops import EmulatedOps
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"], [23, 7, 30, 1, 12])
    steps = _traces(reqs)[mode]
    eng = _engine(which, tensors, "float32", "cpu", EmulatedOps(), max_tokens=replay.max_live_tokens(steps))
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain(which, tensors), reqs, what=f"{which} {mode} stand-in", rtol=2e-5, atol_scale=2e-5)
    assert all(f == eng.num_pages for f in eng.cache.free_pages())
