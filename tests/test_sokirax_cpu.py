"""Sokirax without a GPU: the configuration and its spec, tensor names, the caches a model asks for, the plain
implementation's own consistency."""
import copy

import pytest
import torch

import plain_sokirax as plain
from sokirax_cases import CASES, draw_case


def _cfg(d):
    from gogguf_b200.config import config_from_dict
    return config_from_dict(copy.deepcopy(d))


@pytest.mark.parametrize("name", sorted(CASES))
def test_config_round_trip_and_spec(name):
    from gogguf_b200.engine.model import expected_tensors
    d = CASES[name][0]
    cfg = _cfg(d)
    assert cfg.to_dict() == d
    spec = cfg.to_spec()
    assert len(spec.schedule) == len(d["layers"])
    own = [i for i, l in enumerate(d["layers"]) if "weights_of" not in l]
    assert len(spec.blocks) == len(own)
    for i, (l, e) in enumerate(zip(d["layers"], spec.schedule)):
        assert e.cache_of is None                                  # every run has a cache and state of its own
        assert e.block == own.index(l.get("weights_of", i))
    names = set(expected_tensors(spec))
    assert {"embed", "final.norm", "head"} <= names
    assert not any(n.startswith(f"l{i}.") for n in names for i, l in enumerate(d["layers"]) if "weights_of" in l)
    for i in own:
        l = d["layers"][i]
        assert {f"l{i}.norm1", f"l{i}.norm1b"} <= names
        assert (f"l{i}.norm2b" in names) == (l["mlp"] is not None)
        if l["type"] == "parallel":
            assert {f"l{i}.mix.left.sink", f"l{i}.mix.left.q.norm", f"l{i}.mix.right.g"} <= names
        else:
            assert f"l{i}.mix.q.norm" in names and f"l{i}.mix.sink" not in names
    assert cfg.parameter_count() == sum(int(torch.tensor(t.shape).prod()) for t in expected_tensors(spec).values())


def test_shapes_follow_the_configuration():
    from gogguf_b200.engine.model import expected_tensors
    t = expected_tensors(_cfg(CASES["S"][0]).to_spec())
    assert t["l0.mix.left.q.norm"].shape == (6 * 16,) and t["l0.mix.left.k.norm"].shape == (3 * 16,)
    assert t["l1.mix.q.norm"].shape == (24,) and t["l1.mix.v"].shape == (2 * 40, 96) and t["l1.mix.o"].shape == (96, 4 * 40)
    assert t["l0.mix.right.g"].shape == (3 * 20, 96) and t["l0.mix.left.sink"].shape == (6,)
    assert t["l0.mlp.shared.down"].shape == (96, 56) and t["l0.mlp.e4.gate"].shape == (40, 96)


@pytest.mark.parametrize("bad", [
    lambda d: d["layers"][0].update(type="other"),
    lambda d: d["layers"][1]["mixer"].update(heads=3),                         # not a multiple of kv_heads
    lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.5]),            # one decay per head
    lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7),
    lambda d: d["layers"][2].update(weights_of=2),                             # itself
    lambda d: d["layers"][2].update(weights_of=9),                             # no such layer
    lambda d: d["layers"][4].update(weights_of=2),                             # a layer without tensors
    lambda d: d["layers"][4].update(weights_of=3),                             # other sizes than its source
    lambda d: d["layers"][0]["mlp"]["router"].update(top=9),
    lambda d: d.pop("norm"),
])
def test_bad_configurations_are_refused(bad):
    from gogguf_b200.config import ConfigError
    d = copy.deepcopy(CASES["S"][0])
    bad(d)
    with pytest.raises(ConfigError):
        _cfg(d)


def test_cache_requests_of_every_run():
    """A parallel layer asks for keys and values and for a state; a layer run twice gets both twice; equal requests
    share a group."""
    from gogguf_b200.cache.sequence_cache import KVRequest, SequenceCache, StateRequest
    from gogguf_b200.parts import registry as R
    spec = _cfg(CASES["S"][0]).to_spec()
    reqs = []
    for e in spec.schedule:
        ps = spec.blocks[e.block].mixer
        reqs.append(R.lookup(R.MIXERS, ps.kind, "mixer").cache_request(ps))
    assert isinstance(reqs[0], tuple) and isinstance(reqs[0][0], KVRequest) and isinstance(reqs[0][1], StateRequest)
    assert reqs[0][0] == KVRequest(3, 16, 9, 24) and reqs[0][1].shape == (3, 12, 20)
    assert reqs[1] == KVRequest(2, 24, 70, 40) and reqs[3] == KVRequest(3, 10, None, 6)
    cache = SequenceCache(reqs, [None] * len(reqs), max_tokens=256, dtype=torch.float32)
    assert len(cache.groups) == 3                        # left attention (2 runs), windowed attention (2 runs), full
    v0, v2 = cache.view(0), cache.view(2)
    assert v0[0].group == v2[0].group and v0[0].k.data_ptr() != v2[0].k.data_ptr()
    assert v0[0].v.shape[-1] == 24 and v0[0].k.shape[-1] == 16
    assert v0[1].state.data_ptr() != v2[1].state.data_ptr() and v0[1].state.shape[1:] == (3, 12, 20)
    s = cache.open()
    v0[1].state[s].fill_(3.0)
    cache.plan([s], [70]); cache.commit([s], [70])
    assert not cache.truncate(s, 10)                     # a state holds every token: no way back without a new run
    saved = cache.save_states([s])
    v0[1].state[s].fill_(5.0)
    cache.load_states(saved)
    assert float(v0[1].state[s].max()) == 3.0
    cache.close(s)
    s2 = cache.open()
    assert s2 == s and float(v0[1].state[s2].abs().max()) == 0.0     # the slot comes back with a zeroed state
    cache.check()


def test_stretched_frequencies_by_hand():
    f, mag = plain.rotary_frequencies(dict(base=10000.0, dims=8, scaling=dict(factor=4.0, original=64, fast=8.0, slow=1.0)))
    import math
    d = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(10000.0))
    lo, hi = max(math.floor(d(8.0)), 0), min(math.ceil(d(1.0)), 7)
    assert (lo, hi) == (0, 2)
    base = [10000.0 ** (-2 * i / 8) for i in range(4)]
    assert f[0] == base[0] and abs(f[1] - (base[1] / 4 * 0.5 + base[1] * 0.5)) < 1e-15
    assert f[2] == base[2] / 4 and f[3] == base[3] / 4
    assert abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-15
    assert plain.rotary_frequencies(dict(base=10000.0, dims=8)) == (base, 1.0)


def test_plain_pieces_agree_with_themselves():
    """The recurrence against the sum it unrolls to; a prefix stands alone; a sink of minus infinity is no sink."""
    g = torch.Generator().manual_seed(5)
    n, H, d, dv = 9, 2, 4, 3
    q, k, v = (torch.randn(n, H, s, generator=g, dtype=torch.float64) for s in (d, d, dv))
    decay = [0.8, 1.0]
    o = plain.retention_recurrence(q, k, v, decay)
    for h in range(H):
        for i in range(n):
            ref = sum(decay[h] ** (i - j) * (q[i, h] @ k[j, h]) * v[j, h] for j in range(i + 1))
            assert torch.allclose(o[i, h], ref, atol=1e-12)
    assert torch.equal(plain.retention_recurrence(q[:5], k[:5], v[:5], decay), o[:5])
    a = plain.windowed_softmax_attention(q, k[:, :1], v[:, :1], 0.5, 4, None)
    b = plain.windowed_softmax_attention(q, k[:, :1], v[:, :1], 0.5, 4, torch.full((H,), -1e30, dtype=torch.float64))
    assert torch.allclose(a, b, atol=1e-12)
    c = plain.windowed_softmax_attention(q, k[:, :1], v[:, :1], 0.5, 1, torch.zeros(H, dtype=torch.float64))
    # a window of one and a sink of zero: the token's own value times e^s / (e^s + 1)
    s0 = 0.5 * (q[3, 1] @ k[3, 0])
    assert torch.allclose(c[3, 1], v[3, 0] * torch.exp(s0) / (torch.exp(s0) + 1), atol=1e-12)


@pytest.mark.parametrize("seed", range(6))
def test_drawn_configurations_parse_and_declare_their_tensors(seed):
    from gogguf_b200.engine.model import expected_tensors
    d = draw_case(seed)
    cfg = _cfg(d)
    assert cfg.to_dict() == d
    assert expected_tensors(cfg.to_spec())


def test_a_layer_may_run_the_tensors_of_a_later_one():
    from gogguf_b200.engine.model import expected_tensors
    d = copy.deepcopy(CASES["S"][0])
    first, third = d["layers"][0], d["layers"][2]
    first["weights_of"] = 2
    del third["weights_of"]
    spec = _cfg(d).to_spec()
    assert [e.block for e in spec.schedule] == [1, 0, 1, 2, 0]
    names = set(expected_tensors(spec))
    assert "l2.mix.left.sink" in names and not any(n.startswith("l0.") for n in names)
