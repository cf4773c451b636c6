"""The Sokirax decoder through the framework against the plain implementation (tests/plain_sokirax.py):
each mechanism alone, whole prompts layer by layer, portions, decoding, unequal batches, reuse of slots and pages,
windows, page borders and far keys made to stand out, other sizes, the entry point, the replay program."""
import math
import os

import pytest
import torch

import plain_sokirax as plain
from helpers import random_tokens, read_folder, rel_err
from sokirax_cases import (CASES, attn, draw_case, every_expert, layer, make_folder, par, plain_logits, ret, rot,
                           steady)

pytestmark = pytest.mark.gpu

TOL_F32 = 3e-5
TOL_BF16 = 4e-2      # as for the other architectures (tests/helpers.py): rounding alone reaches 3e-2 on single rows
DEV = "cuda:0"


def tol(dtype):
    return TOL_F32 if dtype == "float32" else TOL_BF16


def close(got, want, dtype, routed=True, own32=None) -> bool:
    """float32: every row within TOL_F32, or within three times the distance `own32` of the plain implementation
    run in float32 from the same implementation in float64 where that is larger (a single token's retention output
    is (q . k) v over its root mean square beside eps: where q . k nearly cancels, rounding alone moves it).  bfloat16: every row within TOL_BF16, except that in a model with routed
    experts a few rows may differ: where two experts' logits lie closer than the rounding of the activations, the
    bfloat16 run may take the other one, which changes that token's row by much more than rounding (and the rows
    that read it a little); and a sequence's first token is a sore spot of the design in any precision (its retention
    output is +-v over its length, with the sign of q . k), so among many rows of drawn models a few may stand out.
    Each kernel alone, the float32 runs and the made-up keys hold every row."""
    got, want = got.double().cpu(), want.double().cpu()
    scale = want.abs().max().clamp_min(1e-30)
    rows = (got - want).abs().reshape(got.shape[0], -1).max(dim=1).values / scale
    if dtype == "float32" or not routed:
        bound = tol(dtype)
        if own32 is not None and dtype == "float32":
            bound = max(bound, 3.0 * rel_err(own32, want))
        if not bool(rows.max() < bound):
            worst = rows.argsort(descending=True)[:8].tolist()
            print(f"close: bound {bound:.2e}, median {float(rows.median()):.2e}, worst rows "
                  f"{[(i, round(float(rows[i]), 5)) for i in worst]} of {got.shape[0]}")
        return bool(rows.max() < bound)
    bad = int((rows >= TOL_BF16).sum())
    ok = bad <= max(1, got.shape[0] // 25) and float(rows.median()) < TOL_BF16 / 2
    if not ok:
        worst = rows.argsort(descending=True)[:8].tolist()
        print(f"close: {bad} of {got.shape[0]} rows over {TOL_BF16}, median {float(rows.median()):.2e}, worst rows "
              f"{[(i, round(float(rows[i]), 3)) for i in worst]}")
    return ok


def load(folder, dtype, fast=True, max_tokens=2048, graphs=False):
    from gogguf_b200.engine import Model, Stepper
    from gogguf_b200.engine.graphs import GraphStepper
    model = Model.load(folder, dtype=dtype, fast=fast)
    cache = model.new_cache(max_tokens=max_tokens)
    return model, cache, (GraphStepper if graphs else Stepper)(model, cache)


def run_cut(st, cache, tokens, cuts):
    """One request in portions of the given sizes (the rest one token at a time); logits at every position."""
    from gogguf_b200.engine import StepEntry
    slot = cache.open()
    rows, at = [], 0
    for n in list(cuts) + [1] * (len(tokens) - sum(cuts)):
        rows.append(st.step([StepEntry(slot, tokens[at:at + n], want=list(range(n)))]).clone())
        at += n
    cache.close(slot)
    cache.check()
    return torch.cat(rows, dim=0)


# ----------------------------------------------------------------------------------------------- mechanisms alone
def _K():
    from gogguf_b200.csrc import kernels
    return kernels


def _tables(rt_dict, positions):
    """cos / sin tables of the step's positions by the package's kernel, frequencies by the plain implementation."""
    f, mag = plain.rotary_frequencies(rt_dict)
    inv = torch.tensor(f, dtype=torch.float64, device=DEV)
    cos = torch.empty(len(positions), len(f), device=DEV)
    sin = torch.empty_like(cos)
    _K().rope_tables(positions, inv, cos, sin, mag)
    return cos, sin


def test_stretched_rotation_part_against_the_formula():
    from gogguf_b200.parts.base import Runtime
    from gogguf_b200.parts.position import RotaryYarn
    rt = Runtime(dtype=torch.float32, device=torch.device(DEV))
    for sc in ((4.0, 512, 16.0, 2.0), (8.0, 64, 32.0, 1.0), (1.0, 100, 3.0, 0.5), (40.0, 4096, 1.5, 1.0)):
        for base, dims in ((70000.0, 16), (900.0, 6), (1e6, 64)):
            r = rot(base, dims, sc)
            f, mag = plain.rotary_frequencies(r)
            p = RotaryYarn(dict(theta=base, rotary_dim=dims, factor=sc[0], original=sc[1], fast=sc[2], slow=sc[3]), rt)
            assert torch.allclose(p.inv_freq.cpu(), torch.tensor(f, dtype=torch.float64), rtol=1e-14, atol=0)
            assert abs(p.magnitude - mag) < 1e-15
    pos = torch.tensor([0, 1, 77, 4000], dtype=torch.int32, device=DEV)
    r = rot(900.0, 6, (4.0, 64, 16.0, 2.0))
    cos, sin = _tables(r, pos)
    f, mag = plain.rotary_frequencies(r)
    a = pos.cpu().double()[:, None] * torch.tensor(f, dtype=torch.float64)[None, :]
    assert torch.allclose(cos.cpu().double(), torch.cos(a) * mag, atol=2e-7)
    assert torch.allclose(sin.cpu().double(), torch.sin(a) * mag, atol=2e-7)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,dv,rdims,mode,sink,window", [
    (4, 2, 24, 40, 16, 1, False, 70), (6, 3, 16, 24, 8, 2, True, 9), (2, 2, 16, 16, 16, 2, True, 1),
    (3, 1, 10, 6, 10, 0, True, 0), (8, 2, 64, 64, 32, 2, True, 65), (4, 1, 128, 32, 2, 1, False, 64)])
def test_attention_mechanism_alone(dt, nq, nkv, d, dv, rdims, mode, sink, window):
    """Made-up projections of two requests (one goes on from cached positions) through the preparation kernel and
    attention, against the plain norms, rotation and windowed softmax; then the same request token by token."""
    K = _K()
    g = torch.Generator().manual_seed(nq * 100 + d)
    r = rot(5000.0, rdims, (4.0, 32, 8.0, 1.0))
    eps, scale = 1e-5, 0.3
    lens = [131, 70]
    width = (nq + nkv) * d + nkv * dv
    qw = (1 + 0.2 * torch.randn(d if mode == 1 else nq * d, generator=g)).float()
    kw = (1 + 0.2 * torch.randn(d if mode == 1 else nkv * d, generator=g)).float()
    sk = (1.5 * torch.randn(nq, generator=g)).float() if sink else None
    rows = [torch.randn(n, width, generator=g).to(dt) for n in lens]
    want = []
    for x in rows:
        x = x.double()
        n = x.shape[0]
        q, k, v = x[:, :nq * d], x[:, nq * d:(nq + nkv) * d], x[:, (nq + nkv) * d:]
        if mode == 2:
            q, k = plain.wnorm(q, qw, eps), plain.wnorm(k, kw, eps)
        q, k = q.view(n, nq, d), k.view(n, nkv, d)
        if mode == 1:
            q, k = plain.wnorm(q, qw, eps), plain.wnorm(k, kw, eps)
        q, k = plain.rotate_halves(q, r), plain.rotate_halves(k, r)
        want.append(plain.windowed_softmax_attention(q, k, v.view(n, nkv, dv), scale, window or None,
                                                     sk.double() if sink else None).reshape(n, nq * dv))
    n_pages = 8
    kp = torch.zeros(n_pages, nkv, 64, d, dtype=dt, device=DEV)
    vp = torch.zeros(n_pages, nkv, 64, dv, dtype=dt, device=DEV)
    table = torch.tensor([[5, 2, 7, 0], [1, 6, 0, 0]], dtype=torch.int32, device=DEV)
    wq, wk = (qw.to(DEV), kw.to(DEV)) if mode else (None, None)

    def step(parts):
        """parts: per request (first row, count); returns the attention output rows in the same order."""
        x = torch.cat([rows[b][a:a + c] for b, (a, c) in enumerate(parts) if c]).to(DEV).contiguous()
        pos = torch.cat([torch.arange(a, a + c) for a, c in parts if c]).to(torch.int32).to(DEV)
        sot = torch.cat([torch.full((c,), b) for b, (a, c) in enumerate(parts) if c]).to(torch.int32).to(DEV)
        T = x.shape[0]
        cos, sin = _tables(r, pos)
        q = torch.empty(T, nq * d, dtype=dt, device=DEV)
        o = torch.empty(T, nq * dv, dtype=dt, device=DEV)
        K.qkv_prep(x, q, wq, wk, eps, mode, cos, sin, pos, sot, table, 64, kp, vp, T, nq, nkv, d, dv, rdims)
        K.attention_plain(q, kp, vp, o, pos, sot, table, 64, T, nq, nkv, d, scale, window, dv=dv,
                          sink=sk.to(DEV) if sink else None, out_scale=1.0)
        return o.float().cpu()

    limit = 2e-5 if dt == torch.float32 else 2.5e-2
    got = step([(0, 100), (0, 70)])                       # prompts
    assert rel_err(got[:100], want[0][:100]) < limit and rel_err(got[100:], want[1]) < limit
    got = step([(100, 29), (0, 0)])                       # a portion that goes on from the cache, over a page border
    assert rel_err(got, want[0][100:129]) < limit
    for i in (129, 130):                                  # decoding
        assert rel_err(step([(i, 1), (0, 0)]), want[0][i:i + 1]) < limit
    # a sink that is left out, or scaled, would show: with it the result differs from the plain softmax
    if sink:
        plain_sm = plain.windowed_softmax_attention(
            plain.rotate_halves(torch.zeros(1, nq, d, dtype=torch.float64), r), torch.zeros(1, nkv, d, dtype=torch.float64),
            torch.ones(1, nkv, dv, dtype=torch.float64), scale, None, sk.double())
        assert torch.allclose(plain_sm[0, :, 0], 1 / (1 + torch.exp(sk.double())), atol=1e-12)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dv,rdims,decay", [
    (3, 12, 20, 12, (0.9, 0.97, 0.995)), (2, 64, 128, 32, (0.99, 0.9995)), (1, 128, 64, 2, (1.0,)),
    (2, 16, 16, 16, (0.0, 1.0)), (1, 512, 100, 16, (0.98,)), (2, 40, 200, 8, (0.5, 0.999))])
def test_retention_mechanism_alone(dt, H, d, dv, rdims, decay):
    """Made-up projections of three requests (and a padding row) through retention: token by token, in chunks, and
    a prompt in portions that go on from the state of a slot that was used before."""
    K = _K()
    g = torch.Generator().manual_seed(H * 1000 + d)
    r = rot(3000.0, rdims)
    eps = 1e-5
    lens = [150, 33, 1]
    width = 2 * H * d + 2 * H * dv
    rows = [(torch.randn(n, width, generator=g) * 0.7).to(dt) for n in lens]
    want = []
    for x in rows:
        x = x.double()
        n = x.shape[0]
        q = plain.rotate_halves(x[:, :H * d].reshape(n, H, d), r)
        k = plain.rotate_halves(x[:, H * d:2 * H * d].reshape(n, H, d), r) * d ** -0.5
        v = x[:, 2 * H * d:2 * H * d + H * dv].reshape(n, H, dv)
        gate = x[:, 2 * H * d + H * dv:]
        o = plain.rms_unit(plain.retention_recurrence(q, k, v, list(decay)), eps).reshape(n, H * dv)
        want.append(o * gate * torch.sigmoid(gate) * 1.7)
    state = torch.full((6, H, d, dv), 9.0, device=DEV)              # what an earlier user of the slots left behind
    slots_of = [4, 1, 3]
    dec = torch.tensor(decay, dtype=torch.float32, device=DEV)
    chunk_ok = K.retention_chunk_takes(d, dv)

    def step(parts, form, pad=False):
        reqs = [(b, a, c) for b, (a, c) in enumerate(parts) if c]
        xs = [rows[b][a:a + c] for b, a, c in reqs]
        pos = [torch.arange(a, a + c) for b, a, c in reqs]
        sot = [torch.full((c,), i) for i, (b, a, c) in enumerate(reqs)]
        sl = [slots_of[b] for b, a, c in reqs]
        if pad:                                                       # a padding row, as a replayed batch has them
            xs.append(torch.zeros(1, width, dtype=dt)); pos.append(torch.zeros(1, dtype=torch.long))
            sot.append(torch.full((1,), -1)); sl.append(0)
        x = torch.cat(xs).to(DEV).contiguous()
        T = x.shape[0]
        cu = torch.tensor([0] + list(torch.tensor([len(p) for p in pos]).cumsum(0)), dtype=torch.int32, device=DEV)
        pos_t = torch.cat(pos).to(torch.int32).to(DEV)
        sot_t = torch.cat(sot).to(torch.int32).to(DEV)
        cos, sin = _tables(r, pos_t)
        out = torch.empty(T, H * dv, dtype=dt, device=DEV)
        raw = torch.empty(T, H * dv, dtype=torch.float32, device=DEV)
        K.retention(x, out, raw, state, cos, sin, cu, torch.tensor(sl, dtype=torch.int32, device=DEV), sot_t, dec,
                    T, len(sl), H, d, dv, rdims, d ** -0.5, eps, 1.7, form)
        return out.float().cpu()

    def step_many(parts):
        """The many-CTA chunked form on the same rows (no padding row: the step's own kernel zeroes those)."""
        reqs = [(b, a, c) for b, (a, c) in enumerate(parts) if c]
        x = torch.cat([rows[b][a:a + c] for b, a, c in reqs]).to(DEV).contiguous()
        pos_t = torch.cat([torch.arange(a, a + c) for b, a, c in reqs]).to(torch.int32).to(DEV)
        sot_t = torch.cat([torch.full((c,), i) for i, (b, a, c) in enumerate(reqs)]).to(torch.int32).to(DEV)
        sl = torch.tensor([slots_of[b] for b, a, c in reqs], dtype=torch.int32, device=DEV)
        cu = torch.tensor([0] + list(torch.tensor([c for b, a, c in reqs]).cumsum(0)), dtype=torch.int32, device=DEV)
        T = x.shape[0]
        cos, sin = _tables(r, pos_t)
        out = torch.empty(T, H * dv, dtype=dt, device=DEV)
        scratch = torch.empty(K.retention_chunks_scratch(T, len(reqs), H, d, dv), device=DEV)
        K.retention_chunks(x, out, scratch, state, cos, sin, cu, sl, sot_t, dec, T, len(reqs), H, d, dv, rdims,
                           d ** -0.5, eps, 1.7)
        return out.float().cpu()

    limit = 3e-5 if dt == torch.float32 else 2e-2
    if max(d, dv) <= K.RETENTION_CHUNKS_MAX_HEAD:
        for s in slots_of:
            state[s].zero_()
        got = step_many([(0, 97), (0, 33), (0, 1)])
        assert rel_err(got[:97], want[0][:97]) < limit and rel_err(got[97:130], want[1]) < limit
        assert rel_err(got[130:131], want[2]) < limit
        got = step_many([(97, 53), (0, 0), (0, 0)])                  # goes on from the state, to the prompt's end
        assert rel_err(got, want[0][97:150]) < limit
        assert float(state[5].min()) == 9.0
    for form in (0, 1) if chunk_ok else (0,):
        for s in slots_of:
            state[s].zero_()                                          # what opening a slot does
        before = state[0].clone()
        got = step([(0, 97), (0, 33), (0, 1)], form, pad=True)
        assert rel_err(got[:97], want[0][:97]) < limit and rel_err(got[97:130], want[1]) < limit
        assert rel_err(got[130:131], want[2]) < limit
        assert float(got[131].abs().max()) == 0.0 and torch.equal(state[0], before)     # the padding row
        got = step([(97, 2), (0, 0), (0, 0)], 0)                      # two more tokens
        assert rel_err(got, want[0][97:99]) < limit
        got = step([(99, 50), (0, 0), (0, 0)], form)                  # a portion that goes on from the state
        assert rel_err(got, want[0][99:149]) < limit
        got = step([(149, 1), (0, 0), (0, 0)], 0)                     # decoding
        assert rel_err(got, want[0][149:150]) < limit
        assert float(state[5].min()) == 9.0                           # a slot nobody named is untouched


@pytest.mark.parametrize("d,nq,nkv,window", [(64, 8, 2, 90), (128, 4, 1, 150), (64, 4, 4, 0), (128, 16, 2, 65)])
def test_tensor_core_attention_with_a_sink_and_a_factor(d, nq, nkv, window):
    """The three tensor-core forms (long portions, short portions, decode steps) against the plain kernel on the same
    bfloat16 cache, with a sink per head and a factor on the output; and a sink that matters: leaving it out moves
    the result by far more than the tolerance."""
    from gogguf_b200.csrc import fast_attention
    from gogguf_b200.parts.base import Runtime, StepContext, Workspace
    K = _K()
    g = torch.Generator().manual_seed(d + nq)
    run = fast_attention.try_make(nq, nkv, d, 0.11, window)
    assert run is not None
    rt = Runtime(dtype=torch.bfloat16, device=torch.device(DEV))
    n_pages, lens = 24, [300, 75, 200]
    kp = (torch.randn(n_pages, nkv, 64, d, generator=g)).to(torch.bfloat16).to(DEV)
    vp = (torch.randn(n_pages, nkv, 64, d, generator=g)).to(torch.bfloat16).to(DEV)
    table = torch.tensor([[3, 9, 1, 20, 7], [4, 11, 0, 0, 0], [5, 6, 8, 2, 0]], dtype=torch.int32, device=DEV)
    sink = (4.0 + 2.0 * torch.randn(nq, generator=g)).float().to(DEV)      # about as heavy as fifty keys

    def check(news):
        """news[b]: how many of request b's last positions are this step's tokens."""
        pos = torch.cat([torch.arange(L - c, L) for L, c in zip(lens, news)]).to(torch.int32).to(DEV)
        sot = torch.cat([torch.full((c,), b) for b, c in enumerate(news)]).to(torch.int32).to(DEV)
        T = int(pos.numel())
        cu = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), dtype=torch.int32, device=DEV)
        ctx = StepContext(runtime=rt, ws=Workspace(rt.device), n_tokens=T, n_seqs=len(lens), tokens=None, positions=pos,
                          seq_of_token=sot, cu_seqlens=cu, slots=None,
                          ctx_lens=torch.tensor(lens, dtype=torch.int32, device=DEV), page_tables={}, max_new=max(news),
                          max_ctx=max(lens), decode=all(c == 1 for c in news))
        q = torch.randn(T, nq * d, generator=g).to(torch.bfloat16).to(DEV)
        got = torch.empty(T, nq * d, dtype=torch.bfloat16, device=DEV)
        want = torch.empty_like(got)
        bare = torch.empty_like(got)
        run(q, kp, vp, got, ctx, table, 64, sink=sink, out_scale=1.3)
        K.attention_plain(q, kp, vp, want, pos, sot, table, 64, T, nq, nkv, d, 0.11, window, sink=sink, out_scale=1.3)
        K.attention_plain(q, kp, vp, bare, pos, sot, table, 64, T, nq, nkv, d, 0.11, window, out_scale=1.3)
        assert rel_err(got, want) < 1.2e-2, (news, rel_err(got, want))
        assert rel_err(bare, want) > 0.1

    check([300, 75, 200])      # whole prompts: 128-query tiles on tcgen05
    check([140, 33, 64])       # portions that go on from the cache
    check([20, 3, 31])         # short portions: 64-query tiles
    check([1, 1, 1])           # decode steps


def test_norm_of_a_parts_output_added_to_the_stream():
    K = _K()
    g = torch.Generator().manual_seed(2)
    for rows, H in ((5, 96), (3, 1000), (1, 7), (2, 4096), (600, 2048), (4, 200), (2, 8200)):
        x, y, w = torch.randn(rows, H, generator=g), torch.randn(rows, H, generator=g) * 3, torch.randn(H, generator=g)
        want = x.double() + plain.wnorm(y.double(), w.double(), 1e-5)
        xd = x.to(DEV)
        K.rmsnorm_add(xd, y.to(DEV), w.to(DEV), 1e-5)
        assert rel_err(xd, want) < 2e-6
        # the same with what a product with a folded norm reads of the updated rows
        xd2 = x.to(DEV)
        parts = (H + 127) // 128
        xhat = torch.zeros(rows, H, dtype=torch.bfloat16, device=DEV)
        ssq = torch.full((rows, parts), -1.0, device=DEV)
        K.rmsnorm_add(xd2, y.to(DEV), w.to(DEV), 1e-5, xhat=xhat, ssq=ssq)
        assert torch.equal(xd2, xd) and torch.equal(xhat, xd.to(torch.bfloat16))
        sq = torch.nn.functional.pad(want ** 2, (0, parts * 128 - H)).view(rows, parts, 128).sum(-1)
        assert rel_err(ssq, sq) < 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_with_a_shared_unit_alone(tmp_path, dtype):
    """The feed-forward part by itself, built through the registry from a spec: softmax over the chosen logits, plain
    gated units, one shared unit; sizes that take the tensor-core forms and sizes that do not; one of one expert."""
    from gogguf_b200.config.spec import PartSpec
    from gogguf_b200.parts import registry as R
    from gogguf_b200.parts.base import Runtime, StepContext, Workspace
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    rt = Runtime(dtype=dt, device=torch.device(DEV))
    for W, F, E, top, shared, T in ((96, 40, 5, 2, 56, 37), (64, 48, 1, 1, 0, 9), (256, 128, 6, 3, 192, 300)):
        g = torch.Generator().manual_seed(W + E)
        names = dict(gate="gate", up="up", down="down")
        params = dict(hidden_size=W, intermediate_size=F, num_experts=E, top_k=top, score="softmax", renormalize=True,
                      weight_on="output", activation=dict(kind="silu_glu"),
                      names=dict(router="router", expert="e{}.", **names))
        mlp = dict(kind="moe", expert=dict(ff=F), router=dict(experts=E, top=top))
        if shared:
            params["shared"] = dict(intermediate_size=shared, prefix="shared.", names=names)
            mlp["shared"] = dict(ff=shared)
        ps = PartSpec(kind="routed_experts", prefix="", params=params)
        cls = R.lookup(R.FEED_FORWARDS, "routed_experts", "feed-forward")
        w = {n: (torch.randn(d.shape, generator=g) * (1.0 if n == "router" else 0.15)).to(dt) for n, d in cls.tensors(ps).items()}
        part = cls(ps, {n: t.to(DEV) for n, t in w.items()}, rt)
        h = torch.randn(T, W, generator=g).to(dt)
        want = plain.routed_experts(h.double(), {n: t.double() for n, t in w.items()}, "", mlp)
        ctx = StepContext(runtime=rt, ws=Workspace(rt.device), n_tokens=T, n_seqs=1, tokens=None, positions=None,
                          seq_of_token=torch.zeros(T, dtype=torch.int32, device=DEV), cu_seqlens=None, slots=None,
                          ctx_lens=None, page_tables={}, max_new=T, max_ctx=T, decode=False)
        out = torch.zeros(T, W, device=DEV)
        part.forward(h.to(DEV), out, ctx)
        assert close(out, want, dtype), (W, E, rel_err(out, want))


# ----------------------------------------------------------------------------------------------- whole models
def _case(name, dtype):
    """bfloat16 runs of whole models take the configurations in which every expert is chosen (see `every_expert`)."""
    return name + "B" if dtype == "bfloat16" and name + "B" in CASES else name


@pytest.mark.parametrize("name", ["S", "ONE", "W", "F"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_every_layer(tmp_path_factory, name, dtype):
    from gogguf_b200.engine import LayerTaps, StepEntry
    name = _case(name, dtype)
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    model, cache, st = load(folder, dtype)
    for n in (1, 2, 150) + ((600,) if name == "W" else ()):
        tokens = steady(cfg, w, random_tokens(cfg["vocab"], n, seed=n), dtype)
        want_layers = []
        want = plain_logits(cfg, w, tokens, want_layers)
        logits32, layers32 = plain.forward(cfg, w, tokens, torch.float32, keep_layers=True)
        got_layers = []
        slot = cache.open()
        got = st.step([StepEntry(slot, tokens, want=list(range(n)))],
                      LayerTaps(on_layer=lambda i, rows: got_layers.append(rows.clone()))).clone()
        cache.close(slot)
        assert len(got_layers) == len(cfg["layers"])            # a layer run twice counts twice
        for i, (a, b) in enumerate(zip(got_layers, want_layers)):
            err = rel_err(a, b)
            assert close(a, b, dtype, routed=False, own32=layers32[i]), (err, name, n, "layer", i)
        err = rel_err(got, want)
        assert close(got, want, dtype, routed=False, own32=logits32), (err, name, n)
    if dtype == "bfloat16":
        # the plain kernels on the same weights are the twins of the tensor-core kernels
        _, cache2, st2 = load(folder, dtype, fast=False)
        twin = run_cut(st2, cache2, tokens, [len(tokens)])
        assert close(twin, want, dtype, routed=False)


@pytest.mark.parametrize("name,dtype", [("S", "float32"), ("S", "bfloat16"), ("ONE", "float32"), ("W", "float32"),
                                        ("W", "bfloat16"), ("F", "bfloat16"), ("F", "float32")])
def test_portions_and_decoding_equal_the_whole_prompt(tmp_path_factory, name, dtype):
    name = _case(name, dtype)
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    tokens = steady(cfg, w, random_tokens(cfg["vocab"], 171, seed=12), dtype)
    want = plain_logits(cfg, w, tokens)
    model, cache, st = load(folder, dtype)
    for cuts in ([171], [64, 64, 43], [2, 2, 61, 3, 100], [63, 2, 70], [130], [1, 65, 2, 2]):
        got = run_cut(st, cache, tokens, cuts)
        err = rel_err(got, want)
        assert close(got, want, dtype, routed=False), (err, name, cuts)
    # token by token from the first one, through captured graphs
    _, cache_g, st_g = load(folder, dtype, graphs=True)
    short = tokens[:90]
    got = run_cut(st_g, cache_g, short, [])
    err = rel_err(got, want[:90])
    assert close(got, want[:90], dtype, routed=False), err


@pytest.mark.parametrize("name,dtype", [("S", "float32"), ("S", "bfloat16"), ("W", "bfloat16"), ("ONE", "float32"),
                                        ("F", "bfloat16")])
def test_unequal_batches_reused_slots_and_pages(tmp_path_factory, name, dtype):
    """Requests of different lengths in one batch, decoded together while the short ones leave; the slots, pages and
    states they give back are taken by the next batch (the cache is sized so that it has to reuse them)."""
    from gogguf_b200.engine import StepEntry
    name = _case(name, dtype)
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    model, cache, st = load(folder, dtype, max_tokens=448, graphs=True)
    got_rows, want_rows, own_rows = [], [], []
    for wave in range(3):
        reqs = [steady(cfg, w, random_tokens(cfg["vocab"], n, seed=100 * wave + n), dtype) for n in (1, 65, 130, 7)]
        tails = [3, 20, 9, 40]
        full = [r + random_tokens(cfg["vocab"], t, seed=7 + t + wave) for r, t in zip(reqs, tails)]
        oracle = [plain_logits(cfg, w, f) for f in full]
        own = [plain.forward(cfg, w, f, torch.float32) for f in full]
        slots = [cache.open() for _ in reqs]
        out = st.step([StepEntry(s, r, want=[len(r) - 1]) for s, r in zip(slots, reqs)]).clone()
        for i, r in enumerate(reqs):
            got_rows.append(out[i]); want_rows.append(oracle[i][len(r) - 1]); own_rows.append(own[i][len(r) - 1])
        live = list(range(len(reqs)))
        for k in range(max(tails)):
            live = [i for i in live if k < tails[i]]
            ent = [StepEntry(slots[i], [full[i][len(reqs[i]) + k]], want=[0]) for i in live]
            out = st.step(ent).clone()
            for j, i in enumerate(live):
                got_rows.append(out[j]); want_rows.append(oracle[i][len(reqs[i]) + k])
                own_rows.append(own[i][len(reqs[i]) + k])
            for i in live:
                if k == tails[i] - 1:
                    cache.close(slots[i])
        cache.check()
        assert cache.live_slots == 0
    got, want = torch.stack(got_rows), torch.stack(want_rows)
    err = rel_err(got, want)
    assert close(got, want, dtype, routed=False, own32=torch.stack(own_rows)), err


def test_long_decoding_past_every_window_and_page(tmp_path_factory):
    """A short prompt and 300 decoded tokens in float32: windows of 9 and 70 pass over decoded tokens, windowed
    groups give pages back, the sequence crosses four page borders and the states take every token once."""
    folder = make_folder(tmp_path_factory.getbasetemp(), "S", "float32")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 305, seed=77)
    want = plain_logits(cfg, w, tokens)
    model, cache, st = load(folder, "float32", max_tokens=512, graphs=True)
    got = run_cut(st, cache, tokens, [5])
    err = [(rel_err(got[i], want[i]), i) for i in range(len(tokens))]
    assert max(err)[0] < TOL_F32, max(err)


MARKED, ASKING, PLAIN = 1, 5, 7      # token ids: the one that is asked for, the one whose query asks, a bystander


def _standout_model(tmp, window, decay, left_scale, right_scale, wide=False):
    """A one-layer model (attention beside retention, no feed-forward) whose weights make one key stand out.  The
    marked token's input has a large component along a direction that every other token's input is orthogonal
    to; one element of every key (beyond the rotated ones) copies it, and the asking token's queries are large at
    that element.  So the asking token gives the marked one a score far above all others: whether the marked token
    is visible (attention) or still remembered (retention) decides the output."""
    from gogguf_b200.weights.loader import write_model_folder
    W, V = 64, 64
    H, G, d, dv = (4, 2, 64, 64) if wide else (2, 1, 16, 16)
    Hr, dr, dvr = (2, 64, 64) if wide else (1, 16, 16)
    e = 12                                   # the element that stands out; beyond the rotated ones
    left = attn(H, G, d, dv, 19.0 / math.sqrt(d), window, rot(10000.0, 8))
    right = ret(Hr, dr, dvr, [decay] * Hr, rot(10000.0, 8))
    cfg = dict(architecture="Sokirax", vocab=V, width=W, norm=dict(eps=1e-6),
               layers=[layer("parallel", par(left, right, left_scale, right_scale), None)])
    g = torch.Generator().manual_seed(31)
    embed = torch.randn(V, W, generator=g)
    a = embed[MARKED] / embed[MARKED].norm()
    for j in range(V):
        if j != MARKED:
            embed[j] -= (embed[j] @ a) * a
    m = embed[ASKING] / embed[ASKING].norm()
    small = lambda *s: torch.randn(*s, generator=g) * 0.01
    # the other elements of the keys are of ordinary size: the norm over the projection must not blow rounding up
    lq, lk, rq, rk = small(H * d, W), torch.randn(G * d, W, generator=g) * 0.3, small(Hr * dr, W), small(Hr * dr, W)
    for h in range(H):
        lq[h * d + e] = 0.5 * m
    for h in range(G):
        lk[h * d + e] = 0.5 * a
    for h in range(Hr):
        rq[h * dr + e] = 0.5 * m
        rk[h * dr + e] = 0.5 * a
    w = {"embed": embed, "head": torch.randn(V, W, generator=g) * 0.2, "final.norm": torch.ones(W),
         "l0.norm1": torch.ones(W), "l0.norm1b": torch.ones(W),
         "l0.mix.left.q": lq, "l0.mix.left.k": lk, "l0.mix.left.v": torch.randn(G * dv, W, generator=g) * 0.3,
         "l0.mix.left.q.norm": torch.ones(H * d), "l0.mix.left.k.norm": torch.ones(G * d),
         "l0.mix.left.sink": torch.zeros(H), "l0.mix.left.o": torch.randn(W, H * dv, generator=g) * 0.3,
         "l0.mix.right.q": rq, "l0.mix.right.k": rk, "l0.mix.right.v": torch.randn(Hr * dvr, W, generator=g) * 0.3,
         "l0.mix.right.g": torch.randn(Hr * dvr, W, generator=g) * 0.1,
         "l0.mix.right.o": torch.randn(W, Hr * dvr, generator=g) * 0.3}
    w = {k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}       # values both compute dtypes hold exactly
    folder = os.path.join(str(tmp), f"standout_{window}_{decay}_{left_scale}_{right_scale}_{wide}")
    if not os.path.isdir(folder):
        write_model_folder(folder, cfg, w)
    return folder, cfg, {k: v.float() for k, v in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("window,n", [(40, 100), (64, 130), (65, 200), (1, 70), (None, 700)])
def test_keys_at_the_window_edge_at_page_borders_and_far_away(tmp_path, dtype, wide, window, n):
    """Attention with a sink: the marked token sits just inside the window, just outside it, at the first position,
    on either side of a page border and (without a window) hundreds of positions back; in a prompt, in a portion
    that goes on from the cache, and in decoding.  `wide`: head sizes the tensor-core kernels take."""
    folder, cfg, w = _standout_model(tmp_path, window, 0.9, 1.3, 0.0, wide)
    model, cache, st = load(folder, dtype)
    spots = {0, 63, 64, n - 2} | ({n - window - 1, n - window, n - window + 1} if window else {n - 600, 65})
    for marked in sorted(s for s in spots if 0 <= s < n - 1):
        tokens = [8 + (i * 7) % 50 for i in range(n)]
        tokens[marked], tokens[-1] = MARKED, ASKING
        want = plain_logits(cfg, w, tokens)
        unseen = list(tokens)
        unseen[marked] = PLAIN
        base = plain_logits(cfg, w, unseen)
        inside = window is None or (n - 1) - marked < window
        # the test can tell: seeing the marked token or not moves the last logits by far more than the tolerance
        moved = rel_err(want[-1], base[-1])
        assert (moved > 0.2) == inside, (marked, moved)
        for cuts in ([n], [n - 1], [marked + 1, n - marked - 2]):
            if min(cuts) < 1:
                continue
            got = run_cut(st, cache, tokens, cuts)
            err = rel_err(got[[marked, n - 1]], want[[marked, n - 1]])
            assert close(got[[marked, n - 1]], want[[marked, n - 1]], dtype, routed=False), (err, window, marked, cuts)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("wide", [False, True])
def test_a_token_far_back_in_the_state(tmp_path, dtype, wide):
    """Retention: the marked token lies hundreds of positions back, in another chunk, another portion and another page
    than the asking one; a state that was lost, cut or taken twice on the way would change the asking token's row."""
    n = 700
    folder, cfg, w = _standout_model(tmp_path, 8, 0.999, 0.0, 1.0, wide)
    model, cache, st = load(folder, dtype)
    _, cache_g, st_g = load(folder, dtype, graphs=True)
    for marked in (0, 31, 32, 95, n - 600, n - 2):
        tokens = [8 + (i * 7) % 50 for i in range(n)]
        tokens[marked], tokens[-1] = MARKED, ASKING
        want = plain_logits(cfg, w, tokens)
        unseen = list(tokens)
        unseen[marked] = PLAIN
        assert rel_err(want[-1], plain_logits(cfg, w, unseen)[-1]) > 0.2, marked
        for cuts in ([n], [n - 1], [marked + 1, n - marked - 2], [64, 2, 300, 65]):
            if min(cuts) < 1:
                continue
            got = run_cut(st, cache, tokens, cuts)
            # (not the first row: a single token's output is (q . k) v over its length, whose sign is rounding's
            # where q . k is made of nothing but small numbers, as the marked token's own is here)
            err = rel_err(got[[n // 2, n - 1]], want[[n // 2, n - 1]])
            assert close(got[[n // 2, n - 1]], want[[n // 2, n - 1]], dtype, routed=False), (err, marked, cuts)
        if marked in (0, n - 600):
            got = run_cut(st_g, cache_g, tokens, [n - 40])        # the tail through captured graphs
            assert close(got[[n // 2, n - 1]], want[[n // 2, n - 1]], dtype, routed=False), marked


def test_the_sorted_form_of_the_experts(tmp_path_factory, monkeypatch):
    """Long prompts whose experts' products are large run one tensor-core product per expert on sorted rows; here
    the threshold is lowered so that the small test model takes that form."""
    from gogguf_b200.parts import experts
    folder = make_folder(tmp_path_factory.getbasetemp(), "WB", "bfloat16")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 700, seed=3)
    want = plain_logits(cfg, w, tokens)
    monkeypatch.setattr(experts, "SORTED_FORM_MIN_WORK", 0.0)
    model, cache, st = load(folder, "bfloat16")
    got = run_cut(st, cache, tokens, [700])
    assert any(getattr(p, "_grouped", None) is not None for p in model.parts())
    err = rel_err(got, want)
    assert close(got, want, "bfloat16", routed=False), err


def test_greedy_generation_through_the_entry_point(tmp_path_factory):
    import gogguf_b200 as gg
    for name, dtype in (("S", "float32"), ("WB", "bfloat16")):
        folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype, std=0.3 if dtype == "float32" else 0.12)
        cfg, w = read_folder(folder)
        prompts = [steady(cfg, w, random_tokens(cfg["vocab"], n, 30 + n), dtype) for n in (5, 1, 80)]
        engine = gg.load(folder, gg.LoadOptions(dtype=dtype, max_tokens=1024))
        ctx = engine.new_context()
        out = ctx.generate(prompts, gg.GenerateParams(max_tokens=12, stop_token_ids=[], keep_logits=True))
        rows, refs = [], []
        for p, r in zip(prompts, out):
            assert len(r.tokens) == 12 and r.prompt_tokens == len(p) and len(r.logits) == 12
            whole = plain_logits(cfg, w, list(p) + r.tokens[:-1])
            for k, row in enumerate(r.logits):
                assert int(row.argmax()) == r.tokens[k]            # greedy: the token is the best of its own row
                rows.append(row)
                refs.append(whole[len(p) - 1 + k])
        assert close(torch.stack(rows), torch.stack(refs), dtype), rel_err(torch.stack(rows), torch.stack(refs))
        if dtype == "float32":
            seq = list(prompts[0])
            for tok in out[0].tokens[:6]:
                assert tok == int(plain_logits(cfg, w, seq)[-1].argmax())
                seq.append(tok)
        # a second round in the same context reuses the slots, pages and states the first gave back; without kept
        # logits the loop runs a step ahead of the host and drops the step a finished sequence ran too far
        again = ctx.generate(prompts, gg.GenerateParams(max_tokens=12, stop_token_ids=[]))
        assert [r.tokens for r in again] == [r.tokens for r in out]
        stop = out[2].tokens[4]
        third = ctx.generate(prompts, gg.GenerateParams(max_tokens=12, stop_token_ids=[stop]))
        assert third[2].tokens == out[2].tokens[:out[2].tokens.index(stop)]
        ctx.cache.check()
        assert ctx.cache.live_slots == 0


@pytest.mark.parametrize("seed", list(range(12)))
def test_a_configuration_nobody_chose(tmp_path, seed):
    """Whole, then a prompt and its tail one by one through captured graphs beside a second, shorter request."""
    import json
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine import StepEntry
    from gogguf_b200.engine.model import write_random_model
    drawn = draw_case(seed)
    n = 150
    tokens = random_tokens(drawn["vocab"], n, seed)
    for dtype in ("float32", "bfloat16"):
        cfg = drawn if dtype == "float32" else every_expert(drawn)
        folder = os.path.join(str(tmp_path), dtype)
        write_random_model(config_from_dict(cfg), seed, folder, dtype=dtype, std=0.12, norm_std=0.1)
        c, w = read_folder(folder)
        tokens = steady(c, w, tokens, dtype)
        want = plain_logits(c, w, tokens)
        own = plain.forward(c, w, tokens, torch.float32)
        model, cache, st = load(folder, dtype, max_tokens=1024)
        got = run_cut(st, cache, tokens, [n])
        err = rel_err(got, want)
        assert close(got, want, dtype, own32=own), (err, dtype, json.dumps(cfg))
        _, cache_g, gs = load(folder, dtype, max_tokens=1024, graphs=True)
        a, b = cache_g.open(), cache_g.open()
        cut = n - 40
        rows, refs = [], []
        out = gs.step([StepEntry(a, tokens[:cut], want=[cut - 1]), StepEntry(b, tokens[:9], want=[8])]).clone()
        rows += [out[0], out[1]]
        refs += [want[cut - 1], want[8]]
        owns = [own[cut - 1], own[8]]
        for k in range(cut, n):
            ents = [StepEntry(a, [tokens[k]], want=[0])]
            if 9 + k - cut < 30:
                ents.append(StepEntry(b, [tokens[9 + k - cut]], want=[0]))
            out = gs.step(ents).clone()
            rows.append(out[0])
            refs.append(want[k])
            owns.append(own[k])
            if len(ents) == 2:
                rows.append(out[1])
                refs.append(want[9 + k - cut])
                owns.append(own[9 + k - cut])
        cache_g.close(a)
        cache_g.close(b)
        cache_g.check()
        err = rel_err(torch.stack(rows), torch.stack(refs))
        assert close(torch.stack(rows), torch.stack(refs), dtype, own32=torch.stack(owns)), (err, dtype, json.dumps(cfg))


@pytest.mark.parametrize("name,dtype", [("S", "float32"), ("S", "bfloat16"), ("W", "bfloat16"), ("ONE", "float32")])
def test_trace_replay_through_the_program(tmp_path_factory, tmp_path, name, dtype):
    """bin/trace_run, the program a user runs: requests whole, with their last tokens one by one, and a batch of
    unequal lengths decoded together while the shorter ones end; places where nothing is wanted."""
    name = _case(name, dtype)
    from test_gpu_replay import Trace
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    lens = [150, 33, 97, 1]
    reqs = {f"r{i}": steady(cfg, w, random_tokens(cfg["vocab"], n, seed=40 + i), dtype) for i, n in enumerate(lens)}
    oracle = {k: plain_logits(cfg, w, t) for k, t in reqs.items()}
    got_rows, want_rows = [], []
    tr = Trace(folder, dtype, tmp_path / "out", max_tokens=192 + 64 + 128 + 64)
    try:
        for k, t in reqs.items():                                        # whole, a few places wanted
            want = sorted({0, len(t) // 2, len(t) - 1})
            got = tr.step([{"id": k + "w", "tokens": t, "want": want}], end=[k + "w"])
            got_rows.append(torch.from_numpy(got)); want_rows.append(oracle[k][want])
        t = reqs["r0"]                                                   # the tail one by one
        cut = len(t) - 40
        assert tr.step([{"id": "d", "tokens": t[:cut], "want": []}]) is None
        for i in range(cut, len(t)):
            got = tr.step([{"id": "d", "tokens": [t[i]], "want": [0] if i % 3 else []}], end=["d"] if i == len(t) - 1 else [])
            if i % 3:
                got_rows.append(torch.from_numpy(got)); want_rows.append(oracle["r0"][i:i + 1])
        batch = ["r3", "r1", "r2", "r0"]                                 # together; the shorter ones end earlier
        pre = {k: max(1, len(reqs[k]) - 12) for k in batch}
        got = tr.step([{"id": k + "b", "tokens": reqs[k][:pre[k]], "want": [pre[k] - 1]} for k in batch],
                      end=[k + "b" for k in batch if pre[k] == len(reqs[k])])
        for j, k in enumerate(batch):
            got_rows.append(torch.from_numpy(got[j:j + 1])); want_rows.append(oracle[k][pre[k] - 1:pre[k]])
        pos = dict(pre)
        live = [k for k in batch if pre[k] < len(reqs[k])]
        while live:
            ending = [k for k in live if pos[k] + 1 == len(reqs[k])]
            got = tr.step([{"id": k + "b", "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live],
                          end=[k + "b" for k in ending])
            for j, k in enumerate(live):
                got_rows.append(torch.from_numpy(got[j:j + 1])); want_rows.append(oracle[k][pos[k]:pos[k] + 1])
                pos[k] += 1
            live = [k for k in live if k not in ending]
    finally:
        tr.close()
    err = rel_err(torch.cat(got_rows), torch.cat(want_rows))
    assert close(torch.cat(got_rows), torch.cat(want_rows), dtype), err


def test_a_layer_that_runs_the_tensors_of_a_later_one(tmp_path):
    """The first layer names the third one's tensors: one set of parts, two runs, each with its cache and state."""
    import copy
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine.model import write_random_model
    d = copy.deepcopy(CASES["S"][0])
    d["layers"][0]["weights_of"] = 2
    del d["layers"][2]["weights_of"]
    folder = os.path.join(str(tmp_path), "later")
    write_random_model(config_from_dict(d), 5, folder, dtype="float32", std=0.12, norm_std=0.1)
    cfg, w = read_folder(folder)
    assert "l2.mix.left.q" in w and not any(k.startswith("l0.") for k in w)
    tokens = random_tokens(cfg["vocab"], 140, seed=4)
    want = plain_logits(cfg, w, tokens)
    model, cache, st = load(folder, "float32")
    for cuts in ([140], [70, 3]):
        got = run_cut(st, cache, tokens, cuts)
        assert close(got, want, "float32", own32=plain.forward(cfg, w, tokens, torch.float32)), (cuts, rel_err(got, want))
