"""The Gigopel design without a GPU: configuration, tensor names, the latent cache's bookkeeping, and the plain
implementation against itself (a prefix stands alone; the absorbed form of latent attention equals the expanded one)."""
import copy
import json
import os

import pytest
import torch

import plain_gigopel as plain
from gigopel_cases import CASE_ODD, CASE_ONE, CASE_T, CASES
from gogguf_b200.cache import LatentRequest, SequenceCache
from gogguf_b200.config import ConfigError, GigopelConfig, config_from_dict, load_config
from gogguf_b200.engine.model import expected_tensors, write_random_model
from helpers import read_folder


def test_the_architecture_key_selects_the_class_and_every_size_comes_from_the_keys():
    c = config_from_dict(CASE_T)
    assert isinstance(c, GigopelConfig)
    assert (c.vocab, c.width, c.residual_mult, c.norm_eps, len(c.layers)) == (211, 96, 0.45, 2e-6, 4)
    a = c.layers[2].mixer
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.scale, a.rot_base, a.rot_dims, a.window) == \
        (2, 8, 32, 16, 80, 0.3, 900.0, 16, None)
    assert c.layers[2].mlp is None and c.layers[0].mlp.kind == "dense" and c.layers[0].mlp.ff == 136
    m = c.layers[1].mlp
    assert (m.kind, m.ff, m.experts, m.top, m.limit) == ("moe", 72, 5, 2, 1.5)
    assert config_from_dict(c.to_dict()) == c
    assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv", "type"),
    (("layers", 0, "mixer", "heads"), 0, "heads"),
    (("layers", 0, "mixer", "rot", "dims"), 18, "rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 3, "rot.dims"),
    (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 1, "mlp", "kind"), "glu", "kind"),
    (("layers", 1, "mlp", "router", "top"), 6, "top"),
    (("layers", 1, "mlp", "expert", "limit"), -1.0, "limit"),
    (("norm", "eps"), 0.0, "eps"),
    (("width",), "wide", "width"),
    (("layers",), [], "layers"),
])
def test_bad_values_are_refused(path, value, word):
    d = copy.deepcopy(CASE_T)
    at = d
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_spec_names_the_designs_tensors_and_parts():
    spec = config_from_dict(CASE_T).to_spec()
    names = expected_tensors(spec)
    assert names["embed"].shape == (211, 96) and names["final.norm"].shape == (96,)
    assert names["l0.mix.q"].shape == (3 * 40, 96) and names["l0.mix.dkv"].shape == (64, 96)
    assert names["l0.mix.dkv.norm"].shape == (48,) and names["l0.mix.uk"].shape == (72, 48)
    assert names["l0.mix.uv"].shape == (120, 48) and names["l0.mix.o"].shape == (96, 120)
    assert names["l0.mlp.up"].shape == (136, 96) and names["l0.mlp.act"].shape == (2,)
    assert names["l1.mlp.router"].shape == (5, 96) and names["l1.mlp.e4.down"].shape == (96, 72)
    assert not any(n.startswith("l2.mlp") for n in names)
    assert names["head.weight"].optional                      # the head is the embedding table
    for b in spec.blocks:
        assert b.arrangement == "parallel" and b.params["residual_mult"] == 0.45
        assert b.parts["norm"].get("weight_offset") == 1.0
    assert "feed_forward" not in spec.blocks[2].parts


def test_random_weights_mode_writes_a_folder_that_loads(tmp_path):
    cfg = config_from_dict(CASE_ODD)
    folder = str(tmp_path / "m")
    write_random_model(cfg, 3, folder, dtype="bfloat16", std=0.1, norm_std=0.05)
    assert load_config(folder) == cfg
    c, w = read_folder(folder)
    assert c["architecture"] == "Gigopel" and set(w) == {n for n, d in expected_tensors(cfg.to_spec()).items() if not d.optional}
    assert float(w["l0.norm1"].float().abs().max()) < 0.5            # stored as the distance from one
    assert abs(float(w["l0.mix.dkv.norm"].float().mean()) - 1.0) < 0.2


def test_latent_cache_groups_windows_and_reuse():
    """Layers with equal requests share a store; a windowed store gives pages back; freed pages are taken again."""
    a, b = LatentRequest(width=64, window=70), LatentRequest(width=64, window=7)
    cache = SequenceCache([a, b, LatentRequest(width=112), a], [None] * 4, max_tokens=512, dtype=torch.float32)
    assert len(cache.groups) == 3 and cache.view(0).group == cache.view(3).group != cache.view(1).group
    assert cache.view(0).pool.shape == (8, 64, 64) and cache.view(2).pool.shape == (8, 64, 112)
    assert LatentRequest(width=70).width == 70
    odd = SequenceCache([LatentRequest(width=70)], [None], max_tokens=64, dtype=torch.float32)
    assert odd.view(0).pool.shape[-1] == 72                        # rows start on 16-byte boundaries in bfloat16
    s = cache.open()
    cache.plan([s], [200])
    cache.commit([s], [200])
    held = lambda g: sum(p >= 0 for p in cache.groups[g].seq_pages[s])
    assert held(cache.view(2).group) == 4                           # no window: every page kept
    assert held(cache.view(1).group) == 1                           # window 7: positions 194.. only
    assert held(cache.view(0).group) == 2                           # window 70: positions 131.. -> pages 2 and 3
    before = cache.groups[cache.view(1).group].pages.free_count
    cache.close(s)
    cache.check()
    assert cache.groups[cache.view(1).group].pages.free_count == before + 1
    s2 = cache.open()
    assert s2 == s                                                  # the slot is reused first
    cache.plan([s2], [65])
    assert cache.groups[0].seq_pages[s2][0] in range(8)
    cache.close(s2)
    cache.check()


def _random_model(case, seed=0):
    cfg = config_from_dict(case)
    g = torch.Generator().manual_seed(seed)
    t = {}
    for n, d in expected_tensors(cfg.to_spec()).items():
        if not d.optional:
            t[n] = torch.randn(d.shape, generator=g, dtype=torch.float64) * (0.3 if len(d.shape) > 1 else 0.2)
    return t


@pytest.mark.parametrize("name", sorted(CASES))
def test_plain_prefix_stands_alone(name):
    case = CASES[name][0]
    t = _random_model(case)
    tokens = [int(x) for x in torch.randint(0, case["vocab"], (90,), generator=torch.Generator().manual_seed(1))]
    whole = plain.forward(tokens, t, case)
    for n in (1, 2, 33, 89):
        assert torch.allclose(plain.forward(tokens[:n], t, case), whole[:n], rtol=1e-9, atol=1e-9)


def test_plain_absorbed_form_equals_the_expanded_form():
    """score = (Wuk^T q_plain) . c + q_rot . k_rot and out = Wuv (sum_j p_j c_j): the algebra the kernels rest on,
    checked on the plain implementation's own tensors."""
    mx = CASE_T["layers"][0]["mixer"]
    t = _random_model(CASE_T, seed=4)
    n, W = 50, CASE_T["width"]
    h = torch.randn(n, W, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    want = plain.latent_attention(h, t, "l0.mix.", mx, 2e-6)
    H, d, r, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = (h @ t["l0.mix.q"].T).view(n, H, d + r)
    dkv = h @ t["l0.mix.dkv"].T
    c = plain.wnorm(dkv[:, :R], t["l0.mix.dkv.norm"], 2e-6)
    pos = torch.arange(n)
    kr = plain.rotate_adjacent(dkv[:, R:], pos, mx["rot"]["base"], mx["rot"]["dims"])
    qr = plain.rotate_adjacent(q[..., d:], pos, mx["rot"]["base"], mx["rot"]["dims"])
    uk, uv = t["l0.mix.uk"].view(H, d, R), t["l0.mix.uv"].view(H, dv, R)
    see = plain.visible(n, mx["mask"]["size"])
    out = torch.zeros(n, H, dv, dtype=torch.float64)
    for hd in range(H):
        q_lat = q[:, hd, :d] @ uk[hd]                              # [n, R]
        s = (q_lat @ c.T + qr[:, hd] @ kr.T) * mx["scale"]
        p = torch.softmax(s.masked_fill(~see, float("-inf")), -1)
        out[:, hd] = (p @ c) @ uv[hd].T
    got = out.reshape(n, H * dv) @ t["l0.mix.o"].T
    assert torch.allclose(got, want, rtol=1e-9, atol=1e-10)


def test_plain_mechanisms_on_known_values():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain.rms_unit(x, 0.0), x / (12.5 ** 0.5))
    assert torch.allclose(plain.znorm(x, torch.tensor([1.0, -1.0]), 0.0), torch.tensor([[2 * 3 / 12.5 ** 0.5, 0.0]], dtype=torch.float64))
    v = torch.tensor([[1.0, 0.0, 5.0, 7.0]], dtype=torch.float64)
    assert torch.allclose(plain.rotate_adjacent(v, torch.tensor([0]), 10.0, 2), v)           # position 0: identity
    quarter = plain.rotate_adjacent(torch.tensor([[1.0, 0.0, 5.0, 7.0]] * 2, dtype=torch.float64),
                                    torch.tensor([0, 1]), 10.0, 2)[1]
    assert torch.allclose(quarter, torch.tensor([torch.cos(torch.tensor(1.0)), torch.sin(torch.tensor(1.0)), 5.0, 7.0],
                                                dtype=torch.float64))                       # the rest passes unchanged
    assert plain.visible(5, 2).tolist()[3] == [False, False, True, True, False]
    z = torch.tensor([-2.0, 0.0, 3.0], dtype=torch.float64)
    p, q = torch.tensor(0.0), torch.tensor(0.0)
    ln2 = torch.log(torch.tensor(2.0, dtype=torch.float64))
    want = torch.stack([(0.5 + ln2) * (torch.exp(z[0]) - 1 - z[0]) + z[0] / 2, torch.tensor(0.0, dtype=torch.float64),
                        ln2 * 9 + 1.5])
    assert torch.allclose(plain.xielu(z, p, q), want)
