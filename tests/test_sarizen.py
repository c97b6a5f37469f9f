"""The Sarizen decoder through the engine against the plain implementation (tests/plain/sarizen.py).

Without a GPU the engine runs on the stand-in kernels (tests/emulated_ops.py), which checks the
configuration, the model description, the parts' use of the cache and the state slots, and the
step function's cutting and batching; on a B200 the same traces run on the CUDA kernels in 32-bit
and in bfloat16, together with tests that aim at single mechanisms."""
import copy
import math

import numpy as np
import pytest
import torch

from leone_b200.engine.engine import Engine
from leone_b200.registry import config_from_dict, spec_from_config
from tests import replay
from tests.plain import sarizen as plain
from tests.sarizen_tiny import PAGE_TOKENS, TINY, as_bf16, tiny_config, tiny_tensors

FP32 = dict(rtol=3e-5, atol_scale=3e-5)
# bfloat16: the gained weights make scores and routers sharp, which also amplifies rounding; the 32-bit
# runs are the sharp tests, these catch a wrong path or operand
BF16 = dict(rtol=1e-1, atol_scale=1e-1)
LENGTHS = [40, 7, 75, 33, 1, 64, 50]


def _plain(which, tensors, bf16=False):
    return plain.PlainSarizen(TINY[which], as_bf16(tensors) if bf16 else tensors)


def _engine(which, tensors, dtype, device, ops=None, max_tokens=512, page=None, **kw):
    spec = spec_from_config(tiny_config(which))
    return Engine(spec, dict(tensors), dtype=dtype, device=device, ops=ops, page_tokens=page or PAGE_TOKENS[which],
                  max_tokens=max_tokens, max_requests=kw.pop("max_requests", 4),
                  max_batch_tokens=kw.pop("max_batch_tokens", 128), **kw)


def _requests(vocab, lengths=LENGTHS, seed=100):
    return {f"r{i}": replay.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


def _traces(reqs):
    return {"whole": replay.trace_whole(reqs), "tail": replay.trace_decode_tail(reqs, tail=20),
            "portions": replay.trace_portions(reqs), "mixed": replay.trace_mixed(reqs, seed=3)}


# -- configuration and description (CPU) ---------------------------------------------------------
def test_config_round_trip_and_spec():
    for which, raw in TINY.items():
        cfg = config_from_dict(raw)
        assert cfg.to_json_dict() == raw
        spec = spec_from_config(cfg)
        assert [layer.mixer.kind for layer in spec.layers] == \
            ["linear_attention" if e["type"] == "lightning" else "latent_attention" for e in raw["layers"]]
        assert all(layer.block == "parallel" for layer in spec.layers)
        assert [layer.feed_forward is None for layer in spec.layers] == [e["mlp"] is None for e in raw["layers"]]


def test_config_rejections():
    from leone_b200.config.base import ConfigError
    for patch in (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]),
                  lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3),
                  lambda c: c["layers"][0].update(type="conv"),
                  lambda c: c["layers"][1]["mlp"]["router"].update(top=9),
                  lambda c: c.pop("width"), lambda c: c.update(layers=[])):
        raw = copy.deepcopy(TINY["P"])
        patch(raw)
        with pytest.raises(ConfigError):
            config_from_dict(raw)


def test_yarn_frequencies_agree_with_the_plain_formula():
    from leone_b200.parts.rotary import scaled_frequencies
    for dims, base, scaling in ((24, 30000.0, {"factor": 6.0, "original": 1024, "fast": 16.0, "slow": 2.0}),
                                (4, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}),
                                (12, 100.0, None), (64, 1e6, {"factor": 40.0, "original": 4096, "fast": 32, "slow": 1})):
        f, mag = scaled_frequencies(dims, base, scaling)
        pf, pmag = plain.yarn_frequencies(dims, base, scaling)
        assert np.allclose(f, pf.numpy(), rtol=1e-14) and abs(mag - pmag) < 1e-15
        if scaling:
            assert f[0] == 1.0 and abs(f[-1] - base ** (-(dims - 2) / dims) / scaling["factor"]) < 1e-15


# -- the step function on stand-in kernels (CPU) ------------------------------------------------
@pytest.mark.parametrize("which", ["P", "Q"])
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


def test_cache_requests_of_the_mixers():
    from tests.emulated_ops import EmulatedOps
    eng = _engine("P", tiny_tensors("P"), "float32", "cpu", EmulatedOps())
    kinds = sorted((g.spec.kind, g.spec.head_dim, g.spec.window) for g in eng.cache.groups)
    assert kinds == [("full", 48, None), ("window", 48, 9)]        # rank + rot_dim per token, no values
    assert all(v is None for _, v in eng.pools)
    assert sorted(tuple(s.shape[1:]) for s in eng._run_state.values()) == [(2, 16, 32), (3, 24, 16)]


# -- on the GPU ----------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("which", ["P", "Q", "R", "S"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_on_the_gpu(which, dtype, mode):
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"])
    steps = _traces(reqs)[mode]
    pool = replay.max_live_tokens(steps)
    eng = _engine(which, tensors, dtype, "cuda:0", max_tokens=pool)
    out = replay.run_trace_engine(eng, steps)
    tol = FP32 if dtype == "float32" else BF16
    replay.compare(steps, out, _plain(which, tensors, dtype == "bfloat16"), reqs, what=f"{which}/{dtype}/{mode}", **tol)
    if mode == "mixed":
        blocks = sum(-(-len(t) // eng.page_tokens) for t in reqs.values())
        assert blocks > eng.num_pages and len(reqs) > eng.max_requests, "pages and slots must be used again"
    assert all(f == eng.num_pages for f in eng.cache.free_pages())


@pytest.mark.gpu
@pytest.mark.parametrize("switch", ["LEONE_NO_LATENT_MMA", "LEONE_NO_EXPERT_MMA", "LEONE_NO_SHARED_KEY_TILES",
                                    "LEONE_MIXERS_PDL", "LEONE_NO_TENSOR_CORES"])
@pytest.mark.parametrize("which", ["R", "S"])
def test_bfloat16_kernel_switches(which, switch, monkeypatch):
    """Every bfloat16 kernel has an any-size form behind a switch; with the switch thrown the same
    traces still agree with the plain implementation (prompt portions of 100 tokens and decode)."""
    monkeypatch.setenv(switch, "1")
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"], [130, 40, 75])
    steps = replay.trace_portions(reqs, sizes=(100, 2, 1, 1, 30)) + []
    eng = _engine(which, tensors, "bfloat16", "cuda:0", max_tokens=replay.max_live_tokens(steps), max_batch_tokens=128)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain(which, tensors, True), reqs, what=f"{which} with {switch}", **BF16)


@pytest.mark.gpu
@pytest.mark.parametrize("which,layer", [("P", 0), ("P", 1), ("P", 2), ("P", 3), ("Q", 0), ("Q", 1), ("Q", 2)])
def test_each_layer_alone(which, layer):
    """A model of one layer: its mixer and feed-forward with nothing else to hide behind."""
    raw = copy.deepcopy(TINY[which])
    raw["layers"] = [raw["layers"][layer]]
    tensors = {k.replace(f"l{layer}.", "l0."): v for k, v in tiny_tensors(which).items()
               if not k.startswith("l") or k.startswith(f"l{layer}.")}
    reqs = _requests(raw["vocab"], [45, 2, 19])
    steps = replay.trace_portions(reqs, sizes=(2, 7, 1, 2, 13))
    eng = Engine(spec_from_config(config_from_dict(raw)), dict(tensors), dtype="float32", device="cuda:0",
                 page_tokens=PAGE_TOKENS[which], max_tokens=192, max_requests=2, max_batch_tokens=64)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, plain.PlainSarizen(raw, tensors), reqs, what=f"{which} layer {layer}", **FP32)


@pytest.mark.gpu
def test_long_prompt_in_chunks_and_long_decode():
    """A prompt long enough for the chunk-parallel recurrence (several chunks, a ragged last one),
    then 150 single-token steps across many pages and windows; position 0 alone first."""
    for dtype, tol in (("float32", FP32), ("bfloat16", BF16)):
        tensors = tiny_tensors("R")
        reqs = {"one": replay.random_tokens(256, 1, 5), "long": replay.random_tokens(256, 460, 77)}
        steps = replay.trace_decode_tail(reqs, tail=150)
        eng = _engine("R", tensors, dtype, "cuda:0", max_tokens=512, max_batch_tokens=512)
        out = replay.run_trace_engine(eng, steps)
        replay.compare(steps, out, _plain("R", tensors, dtype == "bfloat16"), reqs, what=f"long {dtype}", **tol)


@pytest.mark.gpu
def test_page_size_and_batching_do_not_change_fp32_logits_beyond_rounding():
    tensors = tiny_tensors("P")
    reqs = _requests(97, [50, 21, 64])
    steps = replay.trace_mixed(reqs, seed=5)
    outs = []
    for pt in (4, 16, 64):
        eng = _engine("P", tensors, "float32", "cuda:0", max_tokens=replay.max_live_tokens(steps), page=pt)
        outs.append(replay.run_trace_engine(eng, steps))
    for k in outs[0]:
        assert np.array_equal(outs[0][k], outs[1][k]) and np.array_equal(outs[0][k], outs[2][k])


def _one_layer(mixer_type, mixer, vocab=64, width=32, mlp=None):
    return {"architecture": "Sarizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "layers": [{"type": mixer_type, "mixer": mixer, "mlp": mlp}]}


@pytest.mark.gpu
@pytest.mark.parametrize("window,far", [(None, 299), (40, 39), (40, 40), (17, 16), (17, 17)])
def test_one_key_that_stands_out(window, far):
    """A latent-attention layer whose token 7 (and no other) makes a key that the last query scores
    far above all others: the last position's logits change by a lot when that key is ``far``
    tokens back and just inside the window, and not at all when it is just outside."""
    from tests.sarizen_tiny import latent
    raw = _one_layer("latent_attention", latent(2, 8, 4, 8, 16, 0.5, window=window, dims=4))
    specs_cfg = config_from_dict(raw)
    from leone_b200.engine.model import weight_specs_for_config
    from leone_b200.weights.random_init import random_tensors
    tensors = random_tensors(weight_specs_for_config(specs_cfg), 3)
    for k, v in tensors.items():
        if v.dim() == 2:
            tensors[k] = v * 5
    # token 7 is all coordinate 0 and token 9 all coordinate 1 (the norm keeps directions); the latent's
    # element 0 reads coordinate 0, head 0's first query dimension reads coordinate 1 and its first key
    # dimension reads the latent's element 0: the score of (query 9, key 7) towers over all others
    tensors["embed"][7] = 0.0
    tensors["embed"][7, 0] = 1.0
    tensors["embed"][9] = 0.0
    tensors["embed"][9, 1] = 1.0
    tensors["l0.mix.dkv"][0, 0] += 10.0
    tensors["l0.mix.q"][0, 1] += 40.0
    tensors["l0.mix.uk"][0, 0] += 10.0
    length = far + 1 + 5
    base = [t if t not in (7, 9) else 8 for t in replay.random_tokens(64, length, 9)]
    base[-1] = 9
    marked = list(base)
    marked[length - 1 - far] = 7
    model = plain.PlainSarizen(raw, tensors)
    inside = window is None or far < window
    delta = float((model.logits(marked)[-1] - model.logits(base)[-1]).abs().max())
    assert (delta > 3e-3) == inside, "the test's own premise"
    eng = Engine(spec_from_config(specs_cfg), dict(tensors), dtype="float32", device="cuda:0", page_tokens=16,
                 max_tokens=640, max_requests=2, max_batch_tokens=320)
    for name, toks in (("marked", marked), ("base", base)):
        whole = eng.step([(name, toks, [len(toks) - 1])])[0].cpu()
        eng.close(name)
        want = model.logits(toks)[-1]
        assert float((whole.double() - want).abs().max()) <= 3e-5 * float(want.abs().max()), (name, "prompt")
        eng.step([(name, toks[:-3], [])])
        for t in toks[-3:]:
            last = eng.step([(name, [t], [0])])[0].cpu()
        eng.close(name)
        assert float((last.double() - want).abs().max()) <= 3e-5 * float(want.abs().max()), (name, "decoded")


@pytest.mark.gpu
def test_the_state_keeps_a_far_token_and_the_sink_counts():
    """Linear attention with decay 1 on one head: token 0's contribution must still be in the
    output 300 tokens on.  And a latent layer's logits depend on its sinks."""
    from leone_b200.engine.model import weight_specs_for_config
    from leone_b200.weights.random_init import random_tensors
    from tests.sarizen_tiny import latent, lightning
    raw = _one_layer("lightning", lightning(2, 8, 16, [1.0, 0.5]))
    cfg = config_from_dict(raw)
    tensors = {k: (v * 5 if v.dim() == 2 else v) for k, v in random_tensors(weight_specs_for_config(cfg), 4).items()}
    toks = replay.random_tokens(64, 300, 2)
    other = [(toks[0] + 1) % 64] + toks[1:]
    model = plain.PlainSarizen(raw, tensors)
    assert float((model.logits(toks)[-1] - model.logits(other)[-1]).abs().max()) > 1e-3
    eng = Engine(spec_from_config(cfg), dict(tensors), dtype="float32", device="cuda:0", page_tokens=16, max_tokens=64,
                 max_requests=2, max_batch_tokens=512)
    for name, t in (("a", toks), ("b", other)):
        eng.step([(name, t[:200], [])])
        for x in t[200:]:
            got = eng.step([(name, [x], [0])])[0].cpu()
        want = model.logits(t)[-1]
        assert float((got.double() - want).abs().max()) <= 3e-5 * float(want.abs().max())
    raw = _one_layer("latent_attention", latent(3, 8, 4, 8, 16, 0.4, dims=4))
    cfg = config_from_dict(raw)
    tensors = {k: (v * 5 if v.dim() == 2 else v) for k, v in random_tensors(weight_specs_for_config(cfg), 6).items()}
    tensors["l0.mix.sink"] = torch.tensor([3.0, -2.0, 0.5])
    without = dict(tensors)
    without["l0.mix.sink"] = torch.full((3,), -60.0)
    toks = replay.random_tokens(64, 12, 8)
    model = plain.PlainSarizen(raw, tensors)
    assert float((model.logits(toks) - plain.PlainSarizen(raw, without).logits(toks)).abs().max()) > 1e-2
    eng = Engine(spec_from_config(cfg), dict(tensors), dtype="float32", device="cuda:0", page_tokens=4, max_tokens=64,
                 max_requests=2, max_batch_tokens=64)
    got = eng.step([("s", toks, list(range(12)))]).cpu().double()
    assert float((got - model.logits(toks)).abs().max()) <= 3e-5 * float(model.logits(toks).abs().max())


@pytest.mark.gpu
def test_router_choices_and_weights():
    """The router kernel against the plain choice: sigmoid scores, the largest first, not renormalised."""
    from leone_b200.ops.cuda import CudaOps
    ops = CudaOps("cuda:0", torch.float32)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(50, 72, generator=g)
    w = torch.randn(11, 72, generator=g) * 0.3
    for top in (1, 3, 11):
        chosen = torch.zeros(50 * top, dtype=torch.int32, device="cuda:0")
        weight = torch.zeros(50 * top, dtype=torch.float32, device="cuda:0")
        ops.experts_route(x.cuda(), w.cuda(), chosen, weight, top)
        want_e, want_s = plain.router_choice(x.double(), {"router": w.double()}, top)
        assert torch.equal(chosen.cpu().view(50, top).long(), want_e)
        assert torch.allclose(weight.cpu().view(50, top).double(), want_s, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype, tmp_path):
    """generate(): admission, prompt portions mixed with decode, captured decode steps, finish."""
    from leone_b200 import generate
    from leone_b200.weights.safetensors import write_safetensors
    import os
    folder = str(tmp_path / "model")
    cfg = tiny_config("R")
    cfg.write(folder)
    tensors = tiny_tensors("R")
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    model = _plain("R", tensors, dtype == "bfloat16")
    prompts = [replay.random_tokens(256, n, 60 + n) for n in (1, 9, 40, 23, 5)]
    for kw in (dict(), dict(prefill_chunk=7, max_batch_tokens=16, use_graphs=False, prefill_first=False)):
        got = generate(folder, prompts, 10, dtype=dtype, eos_token_id=-1, max_running=3, **kw)
        for p, toks in zip(prompts, got):
            assert len(toks) == 10
            seq = list(p)
            for t in toks:
                logits = model.logits(seq)[-1]
                gap = float(logits.max() - logits[t])
                assert gap <= (1e-4 if dtype == "float32" else 0.04) * float(logits.abs().max()), (kw, seq, t, gap)
                seq.append(t)
