"""The Gigopel decoder through the framework against the plain implementation (tests/plain_gigopel.py):
whole prompts, layer by layer, decoding, portions, unequal batches, reuse of slots and pages, windows and page
borders, other sizes, the entry point."""
import pytest
import torch

import plain_gigopel as plain
from gigopel_cases import CASES, dense, layer, make_folder, mixer, moe, plain_logits
from helpers import random_tokens, read_folder, rel_err

pytestmark = pytest.mark.gpu

TOL_F32 = 3e-5
TOL_BF16 = 3e-2


def tol(dtype):
    return TOL_F32 if dtype == "float32" else TOL_BF16


def close(got, want, dtype, routed=True) -> bool:
    """float32: every row within TOL_F32.  bfloat16: every row within TOL_BF16, except that in a model with routed
    experts a few rows may differ: where two experts' scores lie closer than the rounding of the activations, the
    bfloat16 run may take the other one, which changes that token's row by much more than rounding (and the rows
    that read it a little).  Each kernel alone, the float32 runs and the made-up keys hold every row."""
    got, want = got.double().cpu(), want.double().cpu()
    scale = want.abs().max().clamp_min(1e-30)
    rows = (got - want).abs().reshape(got.shape[0], -1).max(dim=1).values / scale
    if dtype == "float32" or not routed:
        return bool(rows.max() < tol(dtype))
    bad = int((rows >= TOL_BF16).sum())
    return bad <= max(1, got.shape[0] // 25) and float(rows.median()) < TOL_BF16 / 3


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


@pytest.mark.parametrize("name", ["T", "ONE", "ODD", "W"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_every_layer(tmp_path_factory, name, dtype):
    from gogguf_b200.engine import LayerTaps, StepEntry
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    model, cache, st = load(folder, dtype)
    for n in (1, 2, 150) + ((600,) if name == "W" else ()):     # 600 tokens: more pairs per expert than one tile holds
        tokens = random_tokens(cfg["vocab"], n, seed=n)
        want_layers = []
        want = plain_logits(cfg, w, tokens, want_layers)
        got_layers = []
        slot = cache.open()
        got = st.step([StepEntry(slot, tokens, want=list(range(n)))],
                      LayerTaps(on_layer=lambda i, rows: got_layers.append(rows.clone()))).clone()
        cache.close(slot)
        for i, (a, b) in enumerate(zip(got_layers, want_layers)):
            assert close(a, b, dtype), (name, n, "layer", i, rel_err(a, b))
        assert len(got_layers) == len(cfg["layers"])
        assert close(got, want, dtype), (name, n, rel_err(got, want))
    if dtype == "bfloat16":
        # the plain kernels on the same weights are the twins of the tensor-core kernels
        _, cache2, st2 = load(folder, dtype, fast=False)
        twin = run_cut(st2, cache2, tokens, [len(tokens)])
        assert close(twin, want, dtype)
        med = lambda x: float(((x.double().cpu() - want).abs().amax(1) / want.abs().max()).median())
        assert med(got) < 1.5 * med(twin) + 2e-3


@pytest.mark.parametrize("name,dtype", [("T", "float32"), ("T", "bfloat16"), ("ONE", "float32"), ("ODD", "bfloat16"),
                                        ("W", "bfloat16")])
def test_portions_and_decoding_equal_the_whole_prompt(tmp_path_factory, name, dtype):
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 171, seed=12)
    want = plain_logits(cfg, w, tokens)
    model, cache, st = load(folder, dtype)
    for cuts in ([171], [64, 64, 43], [2, 2, 61, 3, 100], [63, 2, 70], [130]):
        got = run_cut(st, cache, tokens, cuts)
        assert close(got, want, dtype), (name, cuts, rel_err(got, want))
    # token by token from the first one, through captured graphs where the model is decoded that way
    _, cache_g, st_g = load(folder, dtype, graphs=True)
    short = tokens[:90]
    got = run_cut(st_g, cache_g, short, [])
    assert close(got, want[:90], dtype), rel_err(got, want[:90])


@pytest.mark.parametrize("name,dtype", [("T", "float32"), ("T", "bfloat16"), ("W", "bfloat16"), ("ODD", "float32")])
def test_unequal_batches_reused_slots_and_pages(tmp_path_factory, name, dtype):
    """Requests of different lengths in one batch, decoded together while the short ones leave; the slots and
    pages they give back are taken by the next batch (the cache is sized so that it has to reuse them)."""
    from gogguf_b200.engine import StepEntry
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    model, cache, st = load(folder, dtype, max_tokens=448, graphs=True)
    got_rows, want_rows = [], []
    for wave in range(3):
        reqs = [random_tokens(cfg["vocab"], n, seed=100 * wave + n) for n in (1, 65, 130, 7)]
        tails = [3, 20, 9, 40]
        full = [r + random_tokens(cfg["vocab"], t, seed=7 + t + wave) for r, t in zip(reqs, tails)]
        oracle = [plain_logits(cfg, w, f) for f in full]
        slots = [cache.open() for _ in reqs]
        out = st.step([StepEntry(s, r, want=[len(r) - 1]) for s, r in zip(slots, reqs)]).clone()
        for i, r in enumerate(reqs):
            got_rows.append(out[i]); want_rows.append(oracle[i][len(r) - 1])
        live = list(range(len(reqs)))
        for k in range(max(tails)):
            live = [i for i in live if k < tails[i]]
            ent = [StepEntry(slots[i], [full[i][len(reqs[i]) + k]], want=[0]) for i in live]
            out = st.step(ent).clone()
            for j, i in enumerate(live):
                got_rows.append(out[j]); want_rows.append(oracle[i][len(reqs[i]) + k])
            for i in live:
                if k == tails[i] - 1:
                    cache.close(slots[i])
        cache.check()
        assert cache.live_slots == 0
    got, want = torch.stack(got_rows), torch.stack(want_rows)
    assert close(got, want, dtype), rel_err(got, want)


def test_long_decoding_past_every_window_and_page(tmp_path_factory):
    """A short prompt and 300 decoded tokens in float32: windows of 7 and 70 pass over decoded tokens, windowed
    groups give pages back and the sequence crosses four page borders."""
    folder = make_folder(tmp_path_factory.getbasetemp(), "T", "float32")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 305, seed=77)
    want = plain_logits(cfg, w, tokens)
    model, cache, st = load(folder, "float32", max_tokens=512, graphs=True)
    got = run_cut(st, cache, tokens, [5])
    err = [(rel_err(got[i], want[i]), i) for i in range(len(tokens))]
    assert max(err)[0] < TOL_F32, max(err)


MARKED, ASKING = 1, 5      # token ids: the one that is asked for, and the one whose query asks for it


def _standout_model(tmp, window):
    """A one-layer model without feed-forward whose weights make one key stand out.  The marked token's latent is
    large along its first element and every other token's is zero there (their embeddings are made orthogonal to
    the direction that feeds it); the first plain key element of each head copies that latent element, and the
    asking token's query is large there.  So the asking token gives the marked one a score of about 30 and every
    other key a score of 0: whether the marked token is visible decides the output."""
    import os
    from gogguf_b200.weights.loader import write_model_folder
    W, R, d, r, dv, H, V = 64, 32, 16, 16, 16, 2, 64
    mx = dict(heads=H, dim=d, rot_dim=r, vdim=dv, kv_rank=R, scale=1.0, rot=dict(base=10000.0, dims=r))
    if window:
        mx["mask"] = dict(size=window)
    cfg = dict(architecture="Gigopel", vocab=V, width=W, residual_mult=1.0, norm=dict(eps=1e-6),
               layers=[dict(type="latent_attention", mixer=mx, mlp=None)])
    g = torch.Generator().manual_seed(31)
    embed = torch.randn(V, W, generator=g)
    a = embed[MARKED] / embed[MARKED].norm()
    for j in range(V):
        if j != MARKED:
            embed[j] -= (embed[j] @ a) * a
    m = embed[ASKING] / embed[ASKING].norm()
    dkv = torch.randn(R + r, W, generator=g) * 0.04
    dkv[0] = 4.0 * a
    q = torch.zeros(H * (d + r), W)
    uk = torch.zeros(H * d, R)
    for h in range(H):
        q[h * (d + r)] = (6.0 / 8.0) * m
        uk[h * d, 0] = 1.0
    w = {"embed": embed, "final.norm": torch.zeros(W), "l0.norm1": torch.zeros(W), "l0.mix.q": q, "l0.mix.dkv": dkv,
         "l0.mix.dkv.norm": torch.ones(R), "l0.mix.uk": uk, "l0.mix.uv": torch.randn(H * dv, R, generator=g) * 0.3,
         "l0.mix.o": torch.randn(W, H * dv, generator=g) * 0.3}
    w = {k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}       # values both compute dtypes hold exactly
    folder = os.path.join(str(tmp), f"standout_{window}")
    if not os.path.isdir(folder):
        write_model_folder(folder, cfg, w)
    return folder, cfg, {k: v.float() for k, v in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,n", [(40, 100), (64, 130), (65, 200), (None, 700)])
def test_keys_at_the_window_edge_at_page_borders_and_far_away(tmp_path, dtype, window, n):
    """The marked token sits just inside the window, just outside it, at the first position, on either side of a page
    border and (without a window) hundreds of positions back; in a prompt and in decoding."""
    folder, cfg, w = _standout_model(tmp_path, window)
    model, cache, st = load(folder, dtype)
    spots = {0, 63, 64, n - 2} | ({n - window - 1, n - window, n - window + 1} if window else {n - 600, 65})
    for marked in sorted(s for s in spots if 0 <= s < n - 1):
        tokens = [6 + (i * 7) % 50 for i in range(n)]
        tokens[marked], tokens[-1] = MARKED, ASKING
        want = plain_logits(cfg, w, tokens)
        unseen = list(tokens)
        unseen[marked] = 7
        base = plain_logits(cfg, w, unseen)
        inside = window is None or (n - 1) - marked < window
        # the test can tell: seeing the marked token or not moves the last logits by far more than the tolerance
        moved = rel_err(want[-1], base[-1])
        assert (moved > 0.2) == inside, (marked, moved)
        for cuts in ([n], [n - 1], [marked + 1, n - marked - 2]):
            if min(cuts) < 1:
                continue
            got = run_cut(st, cache, tokens, cuts)
            assert close(got[[marked, n - 1]], want[[marked, n - 1]], dtype, routed=False), (window, marked, cuts)


def test_latent_attention_kernels_agree_on_made_up_queries():
    """The tensor-core kernel against the plain kernel and against a loop in torch, on queries that are a large
    multiple of one cached row: the row just inside the window, just outside it, the first one, a far one."""
    from gogguf_b200.csrc import fast_latent, kernels as K
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(5)
    for H, R, r, window, page_rows in ((3, 48, 16, 37, 64), (16, 128, 32, 130, 64), (5, 272, 16, 0, 64), (1, 16, 16, 64, 64)):
        D = R + r
        n = 333
        row = (D + 7) // 8 * 8
        n_pages = 8
        pool = torch.zeros(n_pages, page_rows, row)
        pages = [5, 2, 7, 0, 3, 6]                      # the sequence's pages are not in order
        keys = torch.randn(n, D, generator=g)
        for j in range(n):
            pool[pages[j // page_rows], j % page_rows, :D] = keys[j]
        # new tokens: the last 70 positions; each head of each token asks for one row
        T = 70
        pos = torch.arange(n - T, n)
        asks = torch.zeros(T, H, dtype=torch.long)
        q = torch.zeros(T, H, D)
        for t in range(T):
            for h in range(H):
                p = int(pos[t])
                choice = [p, max(0, p - window + 1) if window else 0, max(0, p - window) if window else 1,
                          p // 2, (p // 64) * 64, max(0, (p // 64) * 64 - 1)][(t + h) % 6]
                asks[t, h] = choice
                q[t, h] = keys[choice] * (12.0 / keys[choice].norm() ** 2) * 2.0
        scale = 0.5
        pool_b = pool.to(torch.bfloat16)
        q_b = q.to(torch.bfloat16)
        # the loop
        want = torch.zeros(T, H, R, dtype=torch.float64)
        kd = torch.stack([pool_b[pages[j // page_rows], j % page_rows, :D] for j in range(n)]).double()
        for t in range(T):
            p = int(pos[t])
            lo = max(0, p - window + 1) if window else 0
            for h in range(H):
                s = (kd[lo:p + 1] @ q_b[t, h].double()) * scale
                want[t, h] = torch.softmax(s, 0) @ kd[lo:p + 1, :R]
        ints = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        table = ints([pages + [0] * 2])
        positions, sot, cu = ints(pos.tolist()), ints([0] * T), ints([0, T])
        out_plain = torch.empty(T, H, R, dtype=torch.bfloat16, device=dev)
        K.latent_attention_plain(q_b.to(dev), pool_b.to(dev), out_plain, positions, sot, table, page_rows, T, H, R, r,
                                 scale, window)
        assert rel_err(out_plain, want) < 8e-3
        assert fast_latent.mma_takes(R, r)
        out_fast = torch.full((T, H, R), float("nan"), dtype=torch.bfloat16, device=dev)
        fast_latent.latent_attention_mma(q_b.to(dev), pool_b.to(dev), out_fast, cu, positions, sot, table, page_rows,
                                         1, T, H, R, r, scale, window)
        assert rel_err(out_fast, want) < 8e-3, (H, R, r, window)
        # the same tokens as 70 sequences of one token each (a decode step), with padding sequences between them
        B = 2 * T
        cu2 = ints(list(range(B + 1)))
        sot2 = ints([i // 2 if i % 2 == 0 else -1 for i in range(B)])
        pos2 = ints([int(pos[i // 2]) if i % 2 == 0 else 0 for i in range(B)])
        table2 = ints([pages + [0] * 2] * B)             # one row per sequence of the step, padding ones included
        q2 = torch.zeros(B, H, D, dtype=torch.bfloat16)
        q2[0::2] = q_b
        out2 = torch.full((B, H, R), float("nan"), dtype=torch.bfloat16, device=dev)
        fast_latent.latent_attention_mma(q2.to(dev), pool_b.to(dev), out2, cu2, pos2, sot2, table2, page_rows,
                                         B, B, H, R, r, scale, window, max_new=1)
        assert rel_err(out2[0::2], want) < 8e-3
        assert torch.equal(out2[1::2].float().cpu(), torch.zeros(T, H, R))
        # the cached positions cut into shares whose partial results a second kernel merges (steps of few CTAs);
        # more shares than tiles leaves some of them empty
        for splits in (2, 5, 32):
            for (qq, cuq, posq, sotq, tabq, nseq, ntok, pick) in ((q_b, cu, positions, sot, table, 1, T, slice(None)),
                                                                  (q2, cu2, pos2, sot2, table2, B, B, slice(0, None, 2))):
                outs = torch.full((ntok, H, R), float("nan"), dtype=torch.bfloat16, device=dev)
                part_o = torch.full((ntok * H, splits, R), float("nan"), device=dev)
                part_ml = torch.full((ntok * H, splits, 2), float("nan"), device=dev)
                fast_latent.latent_attention_mma(qq.to(dev), pool_b.to(dev), outs, cuq, posq, sotq, tabq, page_rows,
                                                 nseq, ntok, H, R, r, scale, window, splits, part_o, part_ml,
                                                 max_new=ntok if nseq == 1 else 1)
                assert rel_err(outs[pick], want) < 8e-3, (H, R, r, window, splits)
    assert fast_latent.mma_splits(8, 8, 16, 128, 32, 1024, 4096) > 1 and fast_latent.mma_splits(1, 4096, 16, 128, 32, 1024, 4096) == 1
    assert fast_latent.mma_splits(64, 64, 32, 512, 64, 2048, 4096) > 1


def test_per_head_products_on_the_tensor_cores_equal_the_plain_ones():
    from gogguf_b200.csrc import fast_latent, kernels as K
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(6)
    for H, N, Kd, M in ((3, 48, 24, 77), (16, 128, 32, 1), (4, 40, 272, 130), (1, 16, 16, 64)):
        ldx, hx = H * (Kd + 8) + 16, Kd + 8
        x = torch.randn(M, ldx, generator=g).to(torch.bfloat16)
        w = (torch.randn(H, N, Kd, generator=g) * 0.2).to(torch.bfloat16)
        xh = torch.stack([x[:, h * hx:h * hx + Kd] for h in range(H)], 1).double()        # [M, H, K]
        want = 0.7 * torch.einsum("mhk,hnk->mhn", xh, w.double())
        for fn in (K.headwise_gemm, fast_latent.headwise_gemm_mma):
            for odt in (torch.bfloat16, torch.float32):
                out = torch.zeros(M, H, N + 8, dtype=odt, device=dev)
                fn(x.to(dev), ldx, hx, w.to(dev), out, H * (N + 8), N + 8, M, alpha=0.7)
                assert rel_err(out[:, :, :N], want) < (8e-3 if odt == torch.bfloat16 else 1e-5), (fn.__name__, H, N, Kd, M)
                assert float(out[:, :, N:].abs().max()) == 0.0


def test_xielu_router_and_experts_alone():
    """The activation on both sides of zero and far from it; the router with ties and several choices; the
    experts through the index against the plain expert, weight on the input and clamps in play."""
    from gogguf_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    z = torch.tensor([-30.0, -4.0, -1.0, -1e-4, 0.0, 1e-4, 0.5, 3.0, 20.0], device=dev)
    p, q = torch.tensor(0.3), torch.tensor(-0.8)
    out = torch.empty_like(z)
    K.xielu(z, out, float(plain.softplus(p.double())), float(0.5 + plain.softplus(q.double())), 0.6)
    assert rel_err(out, 0.6 * plain.xielu(z.double().cpu(), p, q)) < 1e-6
    zb = (torch.randn(5, 64, generator=torch.Generator().manual_seed(1)) * 3).to(torch.bfloat16)
    for n in (64, 63):            # eight elements per thread, and the element-wise form
        ob = torch.empty(5, n, dtype=torch.bfloat16, device=dev)
        K.xielu(zb[:, :n].contiguous().to(dev), ob, 0.9, 0.7, 0.6)
        wantb = 0.6 * plain.xielu(zb[:, :n].double(), torch.log(torch.expm1(torch.tensor(0.9))), torch.log(torch.expm1(torch.tensor(0.2))))
        assert rel_err(ob, wantb) < 5e-3
    # router logits: float32 sums of a bfloat16 or float32 row against every expert's row
    gr = torch.Generator().manual_seed(8)
    for dt in (torch.float32, torch.bfloat16):
        hr, wrr = torch.randn(5, 72, generator=gr).to(dt), torch.randn(11, 72, generator=gr).to(dt)
        zr = torch.empty(5, 11, device=dev)
        K.moe_router_logits(hr.to(dev), wrr.to(dev), zr, 5)
        assert rel_err(zr, hr.double() @ wrr.double().T) < 1e-6
    # router: rows with ties (the lower index wins), top 3 of 7
    logits = torch.tensor([[0.1, 2.0, 2.0, -1.0, 2.0, 0.3, 0.2], [5.0, -5.0, 0.0, 0.0, 1.0, 1.0, 1.0]], device=dev)
    idx = torch.empty(2, 3, dtype=torch.int32, device=dev)
    wts = torch.empty(2, 3, dtype=torch.float32, device=dev)
    K.moe_route(logits, 3, idx, wts, None)
    assert idx.tolist() == [[1, 2, 4], [0, 4, 5]]
    assert rel_err(wts, torch.sigmoid(torch.gather(logits, 1, idx.long()))) < 1e-6
    K.moe_route(logits, 3, idx, wts, None, softmax=True, renormalize=True)
    sm = torch.softmax(logits, 1).gather(1, idx.long())
    assert rel_err(wts, sm / sm.sum(1, keepdim=True)) < 1e-6
    # experts through the index
    g = torch.Generator(device="cpu").manual_seed(2)
    T, W, F, E, top, limit = 9, 40, 24, 5, 2, 0.5
    t = {f"e{e}.{n}": torch.randn(*s, generator=g) * 0.4 for e in range(E)
         for n, s in (("gate", (F, W)), ("up", (F, W)), ("down", (W, F)))}
    h = torch.randn(T, W, generator=g)
    ch = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wt = torch.rand(T, top, generator=g) + 0.2
    want = torch.zeros(T, W, dtype=torch.float64)
    for i in range(T):
        for k in range(top):
            e = int(ch[i, k])
            want[i] += 0.3 * plain.expert((wt[i, k] * h[i]).double()[None], t, f"e{e}.", limit)[0]
    w_gu = torch.stack([torch.stack([t[f"e{e}.gate"], t[f"e{e}.up"]]) for e in range(E)]).to(dev)
    w_d = torch.stack([t[f"e{e}.down"] for e in range(E)]).to(dev)
    y = torch.empty(T * top, F, device=dev)
    res = torch.zeros(T, W, device=dev)
    K.moe_gate_up(h.to(dev), w_gu, ch.to(dev), wt.to(dev), y, T, top, True, limit, 1.702, 0.3)
    K.moe_down(y, w_d, ch.to(dev), res, T, top, None)
    assert rel_err(res, want) < 1e-5
    # the same on mma.sync in bfloat16: pairs collected per expert, weight on the input and on the output
    for T2, top2 in ((9, 2), (1, 1), (200, 3)):
        h2 = torch.randn(T2, W, generator=g)
        ch2 = torch.stack([torch.randperm(E, generator=g)[:top2] for _ in range(T2)]).to(torch.int32)
        wt2 = torch.rand(T2, top2, generator=g) + 0.2
        P2 = T2 * top2
        for on_input in (True, False):
            want2 = torch.zeros(T2, W, dtype=torch.float64)
            hb = h2.to(torch.bfloat16)
            tb = {k: v.to(torch.bfloat16).double() for k, v in t.items()}
            for i in range(T2):
                for k in range(top2):
                    e = int(ch2[i, k])
                    xin = (wt2[i, k] * hb[i].float()).to(torch.bfloat16).double() if on_input else hb[i].double()
                    o = plain.expert(xin[None], tb, f"e{e}.", limit)[0]
                    want2[i] += 0.3 * o * (1.0 if on_input else float(wt2[i, k]))
            xs = torch.empty(P2, W, dtype=torch.bfloat16, device=dev)
            K.moe_gather(hb.to(dev), wt2.to(dev), None, xs, P2, top2, on_input)
            yb = torch.full((P2, F), float("nan"), dtype=torch.bfloat16, device=dev)
            K.moe_expert_mma(xs, w_gu.to(torch.bfloat16), ch2.to(dev), P2, yb, True, limit, 1.702, 0.3,
                             None if on_input else wt2.to(dev))
            rows2 = torch.full((P2, W), float("nan"), device=dev)
            K.moe_expert_mma(yb, w_d.to(torch.bfloat16), ch2.to(dev), P2, rows2, False)
            res2 = torch.zeros(T2, W, device=dev)
            K.moe_combine(rows2, None, res2, T2, top2, None)
            assert rel_err(res2, want2) < 1e-2, (T2, top2, on_input)
    assert float((torch.einsum("tw,efw->tef", h, torch.stack([t[f"e{e}.gate"] for e in range(E)])).abs() > limit)
                 .float().mean()) > 0.05          # the clamp is in play


def test_the_three_forms_of_the_experts_agree(tmp_path_factory, monkeypatch):
    """Sorted by expert with one tcgen05 product per expert; through the index on mma.sync; through the index on
    the CUDA cores: the same prompt through each."""
    from gogguf_b200.parts import experts, experts_grouped
    folder = make_folder(tmp_path_factory.getbasetemp(), "W", "bfloat16")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 700, seed=4)
    model, cache, st = load(folder, "bfloat16")
    routed = [b.feed_forward for b in model.blocks if hasattr(b.feed_forward, "_grouped")]
    assert routed and all(p._grouped is not None and p._mma for p in routed)
    on_mma = run_cut(st, cache, tokens, [700])
    monkeypatch.setattr(experts, "SORTED_FORM_MIN_WORK", 0.0)          # this small model would not take it by itself
    sorted_form = run_cut(st, cache, tokens, [700])
    monkeypatch.setattr(experts_grouped, "MIN_PAIRS", 1 << 30)
    for p in routed:
        p._mma = False
    on_cuda_cores = run_cut(st, cache, tokens, [700])
    assert not torch.equal(sorted_form, on_mma) and not torch.equal(on_mma, on_cuda_cores)      # three routes
    want = plain_logits(cfg, w, tokens)
    for got in (on_mma, sorted_form, on_cuda_cores):
        assert close(got, want, "bfloat16")
    assert close(sorted_form, on_mma, "bfloat16") and close(on_cuda_cores, on_mma, "bfloat16")


def test_greedy_generation_through_the_entry_point(tmp_path_factory):
    import gogguf_b200 as gg
    for name, dtype in (("T", "float32"), ("W", "bfloat16")):
        folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype, std=0.3 if dtype == "float32" else 0.12)
        cfg, w = read_folder(folder)
        prompts = [random_tokens(cfg["vocab"], n, 30 + n) for n in (5, 1, 80)]
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
        assert close(torch.stack(rows), torch.stack(refs), dtype)
        if dtype == "float32":
            seq = list(prompts[0])
            for tok in out[0].tokens[:6]:
                assert tok == int(plain_logits(cfg, w, seq)[-1].argmax())
                seq.append(tok)
        # a second round in the same context reuses the slots and pages the first gave back
        again = ctx.generate(prompts, gg.GenerateParams(max_tokens=12, stop_token_ids=[]))
        assert [r.tokens for r in again] == [r.tokens for r in out]
        ctx.cache.check()
        assert ctx.cache.live_slots == 0


def draw_case(seed: int) -> dict:
    """A configuration nobody chose: every size, the order of the layers, windows and constants from a seeded generator."""
    import random
    r = random.Random(seed)
    width = r.choice([8, 16, 24]) * r.choice([3, 5, 7, 9])
    layers = []
    shapes = []
    for _ in range(r.choice([1, 2, 3])):                       # a few mixer shapes that layers share or not
        rot_dim = r.choice([2, 8, 16, 32, 48])
        shapes.append(mixer(r.choice([1, 2, 3, 5, 8]), r.choice([4, 8, 16, 24, 40, 64]), rot_dim,
                            r.choice([4, 8, 16, 24, 56]), r.choice([8, 16, 32, 48, 80, 100, 144]),
                            r.choice([0.05, 0.11, 0.3]), r.choice([100.0, 1e4, 300000.0]),
                            dims=r.choice([d for d in (2, 4, 8, 16, 32, 48) if d <= rot_dim]),
                            window=r.choice([None, 1, 2, 17, 63, 64, 65, 128, 200])))
    for _ in range(r.choice([1, 2, 3, 4, 5])):
        kind = r.choice(["none", "dense", "moe", "moe"])
        experts = r.choice([1, 2, 4, 7, 13])
        mlp = None if kind == "none" else dense(r.choice([8, 24, 40, 72, 200])) if kind == "dense" else \
            moe(r.choice([8, 16, 40, 96]), r.choice([0.5, 1.0, 4.0]), experts, r.randint(1, min(experts, 4)))
        layers.append(layer(r.choice(shapes), mlp))
    return dict(architecture="Gigopel", vocab=r.choice([53, 211, 641, 1031]), width=width,
                residual_mult=r.choice([0.2, 0.5, 1.0, 1.3]), norm=dict(eps=r.choice([1e-6, 1e-5, 3e-4])), layers=layers)


@pytest.mark.parametrize("seed", list(range(12)))
def test_a_configuration_nobody_chose(tmp_path, seed):
    """Whole, then a prompt and its tail one by one through captured graphs beside a second, shorter request."""
    import json
    import os
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine import StepEntry
    from gogguf_b200.engine.model import write_random_model
    cfg = draw_case(seed)
    n = 150
    tokens = random_tokens(cfg["vocab"], n, seed)
    for dtype in ("float32", "bfloat16"):
        folder = os.path.join(str(tmp_path), dtype)
        write_random_model(config_from_dict(cfg), seed, folder, dtype=dtype, std=0.12, norm_std=0.1)
        c, w = read_folder(folder)
        want = plain_logits(c, w, tokens)
        model, cache, st = load(folder, dtype, max_tokens=1024)
        got = run_cut(st, cache, tokens, [n])
        assert close(got, want, dtype), (json.dumps(cfg), dtype, rel_err(got, want))
        _, cache_g, gs = load(folder, dtype, max_tokens=1024, graphs=True)
        a, b = cache_g.open(), cache_g.open()
        cut = n - 40
        rows, refs = [], []
        out = gs.step([StepEntry(a, tokens[:cut], want=[cut - 1]), StepEntry(b, tokens[:9], want=[8])]).clone()
        rows += [out[0], out[1]]
        refs += [want[cut - 1], want[8]]
        for k in range(cut, n):
            ents = [StepEntry(a, [tokens[k]], want=[0])]
            if 9 + k - cut < 30:
                ents.append(StepEntry(b, [tokens[9 + k - cut]], want=[0]))
            out = gs.step(ents).clone()
            rows.append(out[0])
            refs.append(want[k])
            if len(ents) == 2:
                rows.append(out[1])
                refs.append(want[9 + k - cut])
        cache_g.close(a)
        cache_g.close(b)
        cache_g.check()
        assert close(torch.stack(rows), torch.stack(refs), dtype), (json.dumps(cfg), dtype)


def test_prompt_attention_in_the_expanded_form_against_a_loop():
    """Several sequences that start at position 0 (one of a single token, one padding sequence between them), queries
    made to ask for one key each: the window's first and last position, the tile borders, the token itself."""
    from gogguf_b200.csrc import fast_latent
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(11)
    for H, d, r, dv, R, window in ((3, 24, 8, 16, 40, 37), (2, 64, 32, 64, 64, 130), (4, 128, 64, 128, 96, 0), (1, 8, 8, 32, 16, 64)):
        assert fast_latent.prompt_takes(d, r, dv)
        lens = [200, 1, 0, 77]                               # 0: a padding sequence of one row
        rows = [n if n else 1 for n in lens]
        T = sum(rows)
        cu = [0]
        for n in rows:
            cu.append(cu[-1] + n)
        sot = []
        for b, n in enumerate(lens):
            sot += [b if n else -1] * (n if n else 1)
        ldq = H * (d + r) + R + r
        qd = torch.zeros(T, ldq)
        qcat = torch.zeros(T, H, R + r)
        kv = torch.randn(T, H * d + H * dv, generator=g)
        ckr = torch.randn(T, R + r, generator=g)
        want = torch.zeros(T, H, dv, dtype=torch.float64)
        scale = 0.5
        kvb, ckrb = kv.to(torch.bfloat16), ckr.to(torch.bfloat16)
        for b, n in enumerate(lens):
            t0 = cu[b]
            for p in range(n):
                for h in range(H):
                    keys = torch.cat([kvb[t0:t0 + n, h * d:(h + 1) * d], ckrb[t0:t0 + n, R:]], dim=1).double()
                    choice = [p, max(0, p - window + 1) if window else 0, max(0, p - window) if window else p // 3,
                              (p // 64) * 64, max(0, (p // 64) * 64 - 1)][(p + h) % 5]
                    q = (keys[choice] * (24.0 / float(keys[choice].norm() ** 2))).float()
                    qd[t0 + p, h * (d + r):h * (d + r) + d] = q[:d]
                    qcat[t0 + p, h, R:] = q[d:]
                    qb = torch.cat([qd[t0 + p, h * (d + r):h * (d + r) + d], qcat[t0 + p, h, R:]]).to(torch.bfloat16).double()
                    lo = max(0, p - window + 1) if window else 0
                    s = (keys[lo:p + 1] @ qb) * scale
                    vals = kvb[t0 + lo:t0 + p + 1, H * d + h * dv:H * d + (h + 1) * dv].double()
                    want[t0 + p, h] = 0.7 * (torch.softmax(s, 0) @ vals)
        ints = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        av = torch.full((T, H, dv), float("nan"), dtype=torch.bfloat16, device=dev)
        fast_latent.latent_prompt_mma(qd.to(torch.bfloat16).to(dev), qcat.to(torch.bfloat16).to(dev), kvb.to(dev), ckrb.to(dev),
                                      av, ints(cu), ints(sot), len(lens), T, H, d, r, dv, R, scale, window, 0.7)
        live = torch.tensor([s >= 0 for s in sot])
        assert rel_err(av[live], want[live]) < 8e-3, (H, d, r, dv, R, window)
        assert float(av[~live].float().abs().max()) == 0.0


def test_prep_norm_rotation_and_cache_write_alone():
    """latent_prep against the plain norm and rotation: a partial rotation, pages out of order, a padding token, the
    dense copy, and no other row of the pool touched."""
    from gogguf_b200.csrc import kernels as K
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(13)
    H, d, r, R, dims, base, eps = 3, 10, 12, 20, 8, 777.0, 1e-5
    T = 7
    pos = torch.tensor([62, 63, 64, 65, 0, 130, 5])
    sot = [0, 0, 0, 0, -1, 1, 1]
    q = torch.randn(T, H * (d + r), generator=g)
    dkv = torch.randn(T, R + r, generator=g)
    nw = torch.rand(R, generator=g) + 0.5
    half = dims // 2
    ang = pos.double()[:, None] * (base ** (-2.0 * torch.arange(half).double() / dims))[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    row = 40                                                  # pool rows wider than R + r
    pool = torch.full((6, 64, row), 9.0)
    table = torch.tensor([[4, 1, 0], [2, 5, 3]], dtype=torch.int32)
    qcat = torch.full((T, H, R + r), 7.0)
    dense = torch.full((T, R + r), 7.0)
    pool_d, qcat_d, dense_d = pool.to(dev), qcat.to(dev), dense.to(dev)
    K.latent_prep(q.to(dev), dkv.to(dev), nw.to(dev), eps, cos.to(dev), sin.to(dev), dims,
                  pos.to(torch.int32).to(dev), torch.tensor(sot, dtype=torch.int32, device=dev), table.to(dev), 64, pool_d,
                  qcat_d, T, H, d, r, R, dense=dense_d)
    c = plain.wnorm(dkv[:, :R].double(), nw, eps)
    kr = plain.rotate_adjacent(dkv[:, R:].double(), pos, base, dims)
    qr = plain.rotate_adjacent(q.view(T, H, d + r)[..., d:].double(), pos, base, dims)
    want_pool = pool.clone().double()
    for t in range(T):
        if sot[t] < 0:
            continue
        page = int(table[sot[t], int(pos[t]) // 64])
        want_pool[page, int(pos[t]) % 64, :R] = c[t]
        want_pool[page, int(pos[t]) % 64, R:R + r] = kr[t]
        assert rel_err(qcat_d[t, :, R:], qr[t]) < 1e-6
        assert rel_err(dense_d[t], torch.cat([c[t], kr[t]])) < 1e-6
        assert float((qcat_d[t, :, :R].cpu() - 7.0).abs().max()) == 0.0       # the absorbed part is another kernel's
    assert float(qcat_d[4, :, R:].abs().max()) == 0.0                          # the padding token: zeros, no cache row
    assert rel_err(pool_d, want_pool) < 1e-6
    assert int((pool_d.cpu() != 9.0).sum()) == 6 * (R + r)                      # six rows written, nothing else


def test_a_part_without_a_factor_of_its_own_gets_it_from_the_block(tmp_path_factory, monkeypatch):
    """The parallel block hands a part that cannot take the residual factor a zeroed buffer and adds factor times
    the buffer itself; the result is the one of parts that take the factor into their last product."""
    from gogguf_b200.parts.experts import RoutedExperts, XieluMLP
    from gogguf_b200.parts.latent_attention import LatentAttentionMixer
    folder = make_folder(tmp_path_factory.getbasetemp(), "T", "float32")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 90, seed=3)
    want = plain_logits(cfg, w, tokens)
    model, cache, st = load(folder, "float32")
    assert all(all(b._direct.values()) for b in model.blocks)
    direct = run_cut(st, cache, tokens, [90])
    for cls in (LatentAttentionMixer, XieluMLP, RoutedExperts):
        monkeypatch.setattr(cls, "scale_output", lambda self, mult: False)
    model2, cache2, st2 = load(folder, "float32")
    assert not any(any(b._direct.values()) for b in model2.blocks)
    through_buffer = run_cut(st2, cache2, tokens, [60, 30])
    assert rel_err(direct, want) < TOL_F32 and rel_err(through_buffer, want) < TOL_F32
    assert not torch.equal(direct, through_buffer)


@pytest.mark.parametrize("name,dtype", [("T", "float32"), ("T", "bfloat16"), ("W", "bfloat16"), ("ODD", "float32")])
def test_trace_replay_through_the_program(tmp_path_factory, tmp_path, name, dtype):
    """bin/trace_run, the program a user runs: requests whole, with their last tokens one by one, and a batch of
    unequal lengths decoded together while the shorter ones end; places where nothing is wanted; a cache that two
    batches do not fit into at once."""
    from test_gpu_replay import Trace
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    lens = [150, 33, 97, 1]
    reqs = {f"r{i}": random_tokens(cfg["vocab"], n, seed=40 + i) for i, n in enumerate(lens)}
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
    assert close(torch.cat(got_rows), torch.cat(want_rows), dtype)
