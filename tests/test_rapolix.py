"""Rapolix through the framework's own step function, cache manager, scheduler and kernels, against the
plain model of ``plain_rapolix.py``.  Model-level cases run twice: on the host with plain Python standing in
for the kernels (what is under test there is the cache manager with a mixer that owns two caches, the packer,
the plan and the parts' wiring), and on a GPU with the kernels themselves.  Kernel-level cases compare each new
kernel with its restatement in ``plain_ops.py`` at sizes of their own."""
import math

import numpy as np
import pytest
import torch

import plain_ops
import plain_rapolix as plain
import rapolix_util as ru
import vukavik_util as vu           # the schedule runner and the error measures are not tied to a model


@pytest.fixture()
def kernels(request, monkeypatch):
    """On the host the plain restatements stand in for the kernels; on a GPU nothing is replaced."""
    def use(device):
        if device == "cpu":
            from vapi_b200 import ops
            for name in plain_ops.ALL:
                monkeypatch.setattr(ops, name, getattr(plain_ops, name))
    return use


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg, seed in (("mixed", ru.MIXED, 1), ("tiny", ru.TINY, 2), ("one_stream", ru.ONE_STREAM, 3),
                            ("single_learned", ru.SINGLE_LEARNED, 4), ("serving_heads", ru.SERVING_HEADS, 6), ("odd", ru.ODD, 7)):
        out[name] = ru.write_model(str(tmp_path_factory.mktemp(name)), cfg, seed)
        out[name + "/bf16"] = ru.write_model(str(tmp_path_factory.mktemp(name + "bf16")), cfg, seed, torch.bfloat16, std=0.05)
    return out


def _check(runner, oracle, requests, schedule, dtype):
    got = vu.run_schedule(runner, requests, schedule)
    for rid, toks in requests.items():
        want = oracle.logits(toks)
        err, pos = vu.worst(got[rid], want)
        if dtype == "bfloat16":
            e = np.abs(got[rid] - want.numpy()).max(-1) / float(want.max() - want.min())
            assert e.mean() <= 0.02 and np.percentile(e, 95) <= vu.limit(dtype) and err <= 0.15, \
                f"request {rid}: mean {e.mean():.3e}, 95th percentile {np.percentile(e, 95):.3e}, worst {err:.3e} at {pos}"
        else:
            assert err <= vu.limit(dtype), f"request {rid}: {err:.3e} of the logit range at position {pos} of {len(toks)}"


# ---- configuration and registry --------------------------------------------------------------------------
def test_the_architecture_is_found_by_its_name_and_every_size_comes_from_the_configuration():
    from vapi_b200.config.model import ConfigError, resolve_architecture
    arch = resolve_architecture(ru.MIXED)
    assert arch.name == "Rapolix"
    plan = arch.plan(arch.parse(ru.MIXED))
    shapes = {s.name: tuple(s.shape) for s in plan.tensor_specs()}
    assert shapes["embed"] == (200, 64) and shapes["head"] == (200, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.left.q"] == (64, 64) and shapes["l0.mix.left.v"] == (48, 64) and shapes["l0.mix.left.g"] == (96, 64)
    assert shapes["l0.mix.left.o"] == (64, 96) and shapes["l0.mix.left.out"] == (64,) and shapes["l0.mix.right.out"] == (64,)
    assert shapes["l0.mix.right.conv"] == (48, 4) and shapes["l0.mix.right.ra"] == (3, 16, 16) and shapes["l0.mix.right.ri.b"] == (3, 16)
    assert shapes["l0.mlp.gate.b"] == (96,) and shapes["l0.mlp.down.b"] == (64,)
    assert shapes["l0.hc1.mix"] == (3, 3) and shapes["l0.hc2.in"] == (3,) and shapes["l2.hc1.out"] == (3,)
    assert shapes["l1.mlp.router"] == (8, 64) and shapes["l1.mlp.correction"] == (8,) and shapes["l1.mlp.e5.up"] == (40, 64)
    assert "l1.mlp.e6.up" not in shapes, "identity experts have no tensors"
    assert shapes["l1.mlp.shared.down"] == (64, 56) and "l3.mlp.shared.up" not in shapes
    assert "l2.norm2" not in shapes and "l2.hc2.in" not in shapes, "a layer without a feed-forward has no second sublayer"
    # each layer's mixer owns a paged cache and a state; unlike shapes get groups of their own
    kinds = [type(s).__name__ for _, s in plan.cache_sites()]
    assert kinds.count("PagedSpec") == 4 and kinds.count("StateSpec") == 4
    assert all(isinstance(site, tuple) for site, _ in plan.cache_sites())
    one = arch.plan(arch.parse(ru.ONE_STREAM))
    assert not any(".hc" in s.name for s in one.tensor_specs()), "one ordinary stream has no stream tensors"
    for bad in ({**ru.MIXED, "layers": [{"type": "attention", "mixer": {}, "mlp": None}]},
                {**ru.MIXED, "layers": [ru.layer(ru.left(), ru.right(), {"kind": "sparse", "ff": 8})]},
                {**ru.MIXED, "layers": [ru.layer(ru.left(), ru.right(width=50, blocks=4), None)]},
                {**ru.MIXED, "layers": [ru.layer(ru.left(), ru.right(), ru.moe(experts=6, identity=1, count=2))]},
                {k: v for k, v in ru.MIXED.items() if k != "norm"}):
        with pytest.raises(ConfigError):
            arch.parse(bad)


# ---- the plain model itself -----------------------------------------------------------------------------
def test_the_plain_model_is_causal_and_its_mechanisms_run_by_hand():
    cfg = ru.TINY
    from vapi_b200.config.model import resolve_architecture
    arch = resolve_architecture(cfg)
    g = torch.Generator().manual_seed(0)
    w = {s.name: torch.randn(s.shape, generator=g, dtype=torch.float64) * 0.3 for s in arch.plan(arch.parse(cfg)).tensor_specs()}
    toks = vu.prompt(cfg, 25, 0)
    a, b = plain.forward(cfg, w, toks), plain.forward(cfg, w, toks[:13])
    assert torch.allclose(a[:13], b, atol=1e-12)
    # the mask: a window of 3 that keeps the first 2
    assert [j for j in range(8) if plain.visible(7, j, 3, 2)] == [0, 1, 5, 6, 7]
    assert [j for j in range(8) if plain.visible(3, j, 3, 2)] == [0, 1, 2, 3]
    assert [j for j in range(8) if plain.visible(5, j, None, 0)] == [0, 1, 2, 3, 4, 5]
    # the position vector
    pe = plain.sinusoid(3, 4, torch.float64)
    assert pe.tolist() == pytest.approx([math.sin(3.0), math.cos(3.0), math.sin(0.03), math.cos(0.03)])
    # the convolution: the last column weighs the current token
    x = torch.tensor([[1.0, 2.0], [0.5, -1.0]], dtype=torch.float64)
    assert torch.allclose(plain.causal_conv(x, torch.tensor([[2.0, 1.0], [0.0, 3.0]], dtype=torch.float64)),
                          torch.tensor([[1.0, 6.0], [2.5, -3.0]], dtype=torch.float64))
    # the router: scores .1 .2 .3 .4 in two groups; the correction lifts output 0 over output 1 and group 0 over
    # nothing; the best group is {2, 3}; weights are the plain scores, normalised
    z = torch.log(torch.tensor([0.1, 0.2, 0.3, 0.4], dtype=torch.float64))
    chosen, weights = plain.route(z, torch.tensor([0.15, 0.0, 0.0, 0.0], dtype=torch.float64), 2, 2, 1)
    assert chosen == [3, 2] and [float(x) for x in weights] == pytest.approx([4 / 7, 3 / 7])
    chosen, weights = plain.route(z, torch.tensor([0.15, 0.0, 0.0, -0.25], dtype=torch.float64), 2, 1, 1)
    assert chosen == [2, 0] and [float(x) for x in weights] == pytest.approx([0.75, 0.25])
    # one channel of the recurrence by hand, two tokens
    m = {"width": 1, "blocks": 1}
    ww = {"y": torch.ones(1, 1), "y.b": torch.zeros(1), "x": torch.ones(1, 1), "x.b": torch.zeros(1), "conv": torch.ones(1, 1),
          "conv.b": torch.zeros(1), "ra": torch.zeros(1, 1, 1), "ra.b": torch.zeros(1, 1), "ri": torch.zeros(1, 1, 1),
          "ri.b": torch.zeros(1, 1), "lam": torch.zeros(1), "o": torch.ones(1, 1)}
    ww = {"p." + k: v.double() for k, v in ww.items()}
    h = torch.tensor([[1.0], [2.0]], dtype=torch.float64)
    a1 = math.exp(-8 * 0.5 * math.log(2.0))
    s1 = math.sqrt(1 - a1 * a1) * 0.5 * 1.0
    s2 = a1 * s1 + math.sqrt(1 - a1 * a1) * 0.5 * 2.0
    gelu = lambda v: 0.5 * v * (1 + math.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))
    got = plain.gated_recurrence(h, ww, "p.", m)
    assert got[:, 0].tolist() == pytest.approx([s1 * gelu(1.0), s2 * gelu(2.0)])


# ---- the new kernels, each against its restatement ------------------------------------------------------------
def _close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    assert torch.isfinite(a).all()
    assert float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max())), f"{float((a - b).abs().max()):.3e}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_streams_read_norm_and_embedding_kernels(dtype):
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(3)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for S, H, n in ((1, 40, 5), (2, 72, 9), (3, 330, 4), (8, 1100, 3)):
        x = torch.randn((n, S, H), generator=g) * 3 + 0.5
        y = torch.randn((n, H), generator=g).to(dtype)
        mix, write, read = torch.eye(S) + 0.3 * torch.randn((S, S), generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
        w = 1 + 0.2 * torch.randn(H, generator=g)
        rows = torch.tensor([n - 1, 0], dtype=torch.int32)
        for kind in ("layer", "rms"):
            for pending in (True, False):
                for rr in (None, rows):
                    for rd in (read, None):
                        xa, xb = x.clone(), x.clone().cuda()
                        want = plain_ops.hyper_read_norm(xa, y if pending else None, mix, write, rd, w, 1e-5, dtype, rr, kind)
                        got = ops.hyper_read_norm(xb, y.cuda() if pending else None, mix.cuda().contiguous(), write.cuda(),
                                                  rd.cuda() if rd is not None else None, w.cuda(), 1e-5, dtype,
                                                  rr.cuda() if rr is not None else None, kind)
                        _close(got, want, tol)
                        _close(xb, xa, 1e-6)            # the streams themselves are float32 either way
        # two mixers' outputs whose own norms and mean ride on the read
        y2, wy, wy2 = (torch.randn((n, H), generator=g) * 7).to(dtype), 1 + 0.2 * torch.randn(H, generator=g), 1 + 0.2 * torch.randn(H, generator=g)
        for second in (True, False):
            for rr in (None, rows):
                xa, xb = x.clone(), x.clone().cuda()
                want = plain_ops.hyper_read_norm(xa, y, mix, write, read, w, 1e-5, dtype, rr, "layer",
                                                 (y2 if second else None, wy, wy2 if second else None, 1e-6, 0.5))
                got = ops.hyper_read_norm(xb, y.cuda(), mix.cuda().contiguous(), write.cuda(), read.cuda(), w.cuda(), 1e-5, dtype,
                                          rr.cuda() if rr is not None else None, "layer",
                                          (y2.cuda() if second else None, wy.cuda(), wy2.cuda() if second else None, 1e-6, 0.5))
                _close(got, want, tol)
                _close(xb, xa, 1e-6 if dtype == torch.float32 else 2e-2)
        xa, xb = x.clone(), x.clone().cuda()
        assert ops.hyper_read_norm(xb, y.cuda(), mix.cuda().contiguous(), write.cuda(), None, None, 1e-5, dtype) is None
        plain_ops.hyper_read_norm(xa, y, mix, write, None, None, 1e-5, dtype)
        _close(xb, xa, 1e-6)
    # the position vector: angles in float32 from frequencies rounded once; positions in the thousands
    V, H = 50, 36
    table = torch.randn((V, H), generator=g).to(dtype)
    toks = torch.randint(0, V, (7,), generator=g, dtype=torch.int32)
    pos = torch.tensor([0, 1, 2, 777, 5000, 5001, 123456], dtype=torch.int32)
    freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(H // 2, dtype=torch.float64) / H)
    got = ops.embed_sinusoid(table.cuda(), toks.cuda(), pos.cuda(), freq.float().cuda(), 3).cpu()
    ang = pos.double()[:, None] * freq.float().double()[None, :]
    want = table[toks.long()].double() + torch.stack([torch.sin(ang), torch.cos(ang)], -1).reshape(7, H)
    assert got.shape == (7, 3, H) and torch.equal(got[:, 0], got[:, 1]) and torch.equal(got[:, 0], got[:, 2])
    assert float((got[:, 0].double() - want).abs().max()) < 2e-2          # one float32 rounding of an angle of 123456
    assert float((got[:4, 0].double() - want[:4]).abs().max()) < 1e-4
    # branches side by side, the wide gate, the cap
    a, b, c = (torch.randn((6, 200), generator=g).to(dtype) * s for s in (1.0, 30.0, 0.01))
    ws = [1 + 0.3 * torch.randn(200, generator=g) for _ in range(3)]
    for k in (1, 2, 3):
        _close(ops.branch_rmsnorm_mean([t.cuda() for t in (a, b, c)[:k]], [t.cuda() for t in ws[:k]], 1e-6, 1.0 / k),
               plain_ops.branch_rmsnorm_mean([a, b, c][:k], ws[:k], 1e-6, 1.0 / k), tol)
    wide = torch.randn((6, 500), generator=g).to(dtype)
    _close(ops.sigmoid_gate(a.cuda(), wide.cuda()[:, 100:300]), plain_ops.sigmoid_gate(a, wide[:, 100:300]), tol)
    z = torch.randn((4, 33), generator=g) * 40
    _close(ops.softcap(z.clone().cuda(), 15.0), 15.0 * torch.tanh(z / 15.0), 1e-5)


def _step_meta(lens, starts, slots, device):
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    pos = torch.cat([torch.arange(s, s + q, dtype=torch.int32) for s, q in zip(starts, lens)])
    seq = torch.cat([torch.full((q,), i, dtype=torch.int32) for i, q in enumerate(lens)])
    return cu.to(device), pos.to(device), seq.to(device), torch.tensor(slots, dtype=torch.int32).to(device)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_recurrence_continues_from_its_state_and_starts_fresh_at_position_zero(dtype):
    """Several sequences in one step: a long portion (many warps cut it into segments), portions of 1, 2 and 17
    tokens, one that continues from a state an earlier step left, one that starts at position 0 in a slot that
    holds another request's state.  Channel counts that are no multiples of 32, parts that are no multiples of 4."""
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(5)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for C, B, L in ((40, 2, 3), (66, 3, 1), (256, 4, 4), (192, 1, 2)):
        bs = C // B
        lens, starts, slots = [300, 1, 2, 17, 1], [0, 40, 7, 0, 0], [2, 0, 4, 1, 3]
        n = sum(lens)
        off = (L - 1) * C
        wide = (torch.randn((n, 2 * C), generator=g) * 1.5).to(dtype)
        w_a, w_i = ((torch.randn((B, bs, bs), generator=g) * 0.4).to(dtype) for _ in range(2))
        b_a, b_i = torch.randn(C, generator=g) * 0.5, torch.randn(C, generator=g) * 0.5
        lam = -1.0 - 5.0 * torch.rand(C, generator=g)
        taps, cb = torch.randn((L, C), generator=g) * 0.5, torch.randn(C, generator=g) * 0.3
        state = torch.randn((6, off + C + 5), generator=g)               # dirty slots, wider than needed
        for dev_ops, dev in ((plain_ops, "cpu"), (ops, "cuda")):
            st = state.clone().to(dev)
            cu, pos, seq, sl = _step_meta(lens, starts, slots, dev)
            wd = wide.to(dev)
            u = dev_ops.causal_conv(wd[:, C:], taps.to(dev), cb.to(dev), st if L > 1 else None, sl, seq, cu, pos, max(lens), None,
                                    act="none")
            out = dev_ops.rglru(u.contiguous(), wd[:, :C], w_a.to(dev), b_a.to(dev), w_i.to(dev), b_i.to(dev), lam.to(dev), 8.0, st,
                                off, sl, cu, pos, None, max_q=max(lens))
            if dev == "cpu":
                want, want_state, want_u = out, st, u
            else:
                _close(u, want_u, tol)
                _close(out, want, tol)
                used = sorted(set(slots))
                _close(st[used, :off + C], want_state[used, :off + C], 3e-5 if dtype == torch.float32 else 3e-2)
                assert torch.equal(st[5].cpu(), state[5]) and torch.equal(st[:, off + C:].cpu(), state[:, off + C:])
        # the request in slot 1 goes on, token by token, from what the portion of 17 left
        cu, pos, seq, sl = _step_meta([1], [17], [1], "cuda")
        st_g, st_c = st, want_state
        for t in range(3):
            row = (torch.randn((1, 2 * C), generator=g)).to(dtype)
            posg = pos + t
            outs = []
            for dev_ops, dev, stt in ((plain_ops, "cpu", st_c), (ops, "cuda", st_g)):
                r = row.to(dev)
                u = dev_ops.causal_conv(r[:, C:], taps.to(dev), cb.to(dev), stt if L > 1 else None, sl.to(dev), seq.to(dev), cu.to(dev),
                                        posg.to(dev), 1, None, act="none")
                outs.append(dev_ops.rglru(u.contiguous(), r[:, :C], w_a.to(dev), b_a.to(dev), w_i.to(dev), b_i.to(dev), lam.to(dev),
                                          8.0, stt, off, sl.to(dev), cu.to(dev), posg.to(dev), None, max_q=1))
            _close(outs[1], outs[0], tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_router_and_the_experts(dtype):
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(9)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for W, ff, E, I, top, groups, keep, n in ((48, 20, 6, 2, 2, 4, 2, 150), (64, 36, 5, 0, 1, 1, 1, 70), (40, 8, 9, 3, 4, 3, 2, 1),
                                              (32, 16, 0, 2, 1, 1, 1, 5), (72, 100, 70, 2, 6, 9, 4, 300),
                                              (64, 200, 4, 0, 2, 1, 1, 700), (136, 72, 3, 1, 2, 2, 1, 900)):
        h = torch.randn((n, W), generator=g).to(dtype)
        router = torch.randn((E + I, W), generator=g) * 0.6
        corr = torch.randn(E + I, generator=g) * 0.05
        ids_c, wts_c, _ = plain_ops.moe_route(h, router, corr, E, top, groups, keep)
        ids_g, wts_g, plan = ops.moe_route(h.cuda(), router.cuda(), corr.cuda(), E, top, groups, keep)
        # a choice may differ only where two corrected scores are as good as tied
        s = torch.softmax(router @ h.float().t(), 0).t()
        for t in range(n):
            if ids_g[t].tolist() != ids_c[t].tolist():
                c = (s[t] + corr)
                a, b = sorted(set(ids_g[t].tolist()) ^ set(ids_c[t].tolist()))[:2]
                assert abs(float(c[a] - c[b])) < 1e-5, f"token {t}: {ids_g[t].tolist()} against {ids_c[t].tolist()}"
        same = [t for t in range(n) if ids_g[t].tolist() == ids_c[t].tolist()]
        assert len(same) >= n - 2
        _close(wts_g[same], wts_c[same], 1e-5)
        assert float((wts_g.sum(1) - 1).abs().max()) < 1e-5
        w_up = (torch.randn((E, ff, W), generator=g) * 0.3).to(dtype) if E else None
        w_down = (torch.randn((E, W, ff), generator=g) * 0.3).to(dtype) if E else None
        shared = torch.randn((n, W), generator=g).to(dtype)
        for sh in (shared, None):
            got = ops.moe_experts(h.cuda(), ids_g, wts_g, plan, w_up.cuda() if E else None, w_down.cuda() if E else None,
                                  sh.cuda() if sh is not None else None)
            want = plain_ops.moe_experts(h, ids_g.cpu(), wts_g.cpu(), None, w_up, w_down, sh)
            _close(got, want, tol)
    _close(ops.relu_squared(h.cuda()), plain_ops.relu_squared(h), tol)


def _planted(klen, qlen, j_star, dk=16, dv=8, page=16, nh=2, nkv=1, device="cuda", dtype=torch.float32):
    """A cache in which key j_star matches the queries far better than any other and carries the value 1 where
    all others carry 0; pages are taken in a scrambled order."""
    g = torch.Generator().manual_seed(klen * 131 + j_star)
    pages = -(-klen // page)
    order = torch.randperm(pages + 3, generator=g)[:pages].to(torch.int32)
    cache = torch.randn((pages + 3, page * nkv * (dk + dv)), generator=g) * 0.01
    direction = torch.randn(dk, generator=g)
    direction /= direction.norm()
    for j in range(klen):
        pg, off = int(order[j // page]), j % page
        cache[pg, off * dk:(off + 1) * dk] = direction * (30.0 if j == j_star else 0.0) + 0.01 * torch.randn(dk, generator=g)
        v0 = page * nkv * dk + off * dv
        cache[pg, v0:v0 + dv] = 1.0 if j == j_star else 0.0
    q = (direction[None, :] + 0.01 * torch.randn((qlen * nh, dk), generator=g)).reshape(qlen, nh * dk)
    return (q.to(device, dtype).contiguous(), cache.to(device, dtype).contiguous(), order[None, :].to(device).contiguous())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,dv,page", [(16, 8, 16), (64, 64, 64), (128, 128, 64)])
@pytest.mark.parametrize("qlen", [1, 5, 40, 100, 300])
def test_a_planted_key_is_seen_inside_the_window_and_among_the_kept_first_tokens(qlen, dk, dv, page, dtype):
    """One key decides every query's output, so a window or a count of kept tokens that is one off shows.  Keys
    just inside and just outside the window, the last kept token and the first one that is not kept, at page
    borders and inside pages, far back among hundreds; in prompts' portions and for single decoded tokens; with
    and without split keys.  In bfloat16 the equal widths run on the tensor-core kernels (one warp for few rows,
    four warps, tcgen05 from 64 tokens on), everything else on the general kernel."""
    from vapi_b200 import ops
    klen = 420
    for window, keep in ((75, 21), (64, 64), (100, 1), (33, 130), (50, 0)):
        edge = klen - window                              # the last query's window starts right behind this key
        for j_star in sorted({0, keep - 1, keep, 63, 64, 127, 128, edge - qlen, edge, edge + 1, klen - qlen, klen - 1} & set(range(klen))):
            q, cache, table = _planted(klen, qlen, j_star, dk=dk, dv=dv, page=page, dtype=dtype)
            cu = torch.tensor([0, qlen], dtype=torch.int32, device="cuda")
            kl = torch.tensor([klen], dtype=torch.int32, device="cuda")
            for splits in (1, 3):
                out = ops.masked_attention(q, q.stride(0), cache, page, table, cu, kl, qlen, 1, qlen, klen, 2, 1, dk, dv, 1.0,
                                           window=window, keep=keep, splits=splits).float().cpu()
                for i in range(qlen):
                    p = klen - qlen + i
                    seen = j_star <= p and (p - j_star < window or j_star < keep)
                    assert abs(float(out[i].mean()) - (1.0 if seen else 0.0)) < 0.02, \
                        f"key {j_star}, query at {p}, window {window}, keep {keep}, {splits} slices: {out[i].mean():.3f}, seen={seen}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,dk,dv,page", [(torch.float32, 24, 40, 16), (torch.bfloat16, 64, 64, 64), (torch.bfloat16, 128, 128, 64)])
def test_windowed_attention_with_kept_tokens_against_its_restatement_in_a_mixed_batch(dtype, dk, dv, page):
    """Random keys and values: a portion of 90 beside a portion of 3 beside single tokens, sequences shorter than
    the window and shorter than the kept count, three query heads a key head."""
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(11)
    nh, nkv = 6, 2
    lens, klens = [90, 3, 1, 1, 64], [400, 10, 2, 333, 64]
    n, S = sum(lens), len(lens)
    pages = sum(-(-k // page) for k in klens)
    table = torch.zeros((S, max(-(-k // page) for k in klens)), dtype=torch.int32)
    perm, at = torch.randperm(pages + 2, generator=g), 0
    for s, k in enumerate(klens):
        for j in range(-(-k // page)):
            table[s, j] = int(perm[at])
            at += 1
    cache = torch.randn((pages + 2, page * nkv * (dk + dv)), generator=g).to(dtype)
    q = (torch.randn((n, nh * dk), generator=g) * 0.7).to(dtype)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    kl = torch.tensor(klens, dtype=torch.int32)
    for window, keep in ((90, 17), (5, 7), (1000, 3), (64, 0)):
        want = plain_ops.masked_attention(q, q.stride(0), cache, page, table, cu, kl, n, S, max(lens), max(klens), nh, nkv, dk, dv,
                                          0.2, window=window, keep=keep)
        got = ops.masked_attention(q.cuda(), q.stride(0), cache.cuda(), page, table.cuda(), cu.cuda(), kl.cuda(), n, S, max(lens),
                                   max(klens), nh, nkv, dk, dv, 0.2, window=window, keep=keep)
        _close(got, want, 3e-5 if dtype == torch.float32 else 3e-2)


# ---- prompts, decoding, portions ------------------------------------------------------------------------------
@pytest.mark.parametrize("device,name,length", [pytest.param("cpu", "tiny", 24, id="host"),
                                                pytest.param("cuda", "mixed", 140, marks=pytest.mark.gpu, id="gpu"),
                                                pytest.param("cuda", "one_stream", 90, marks=pytest.mark.gpu, id="gpu-one-stream"),
                                                pytest.param("cuda", "single_learned", 60, marks=pytest.mark.gpu, id="gpu-single-learned"),
                                                pytest.param("cuda", "odd", 70, marks=pytest.mark.gpu, id="gpu-odd-sizes")])
def test_whole_prompt_token_by_token_and_portions_agree_with_the_plain_model(device, name, length, folders, kernels):
    kernels(device)
    oracle = ru.Oracle(folders[name])
    runner = vu.make_runner(folders[name], "float32", device, num_pages=12)
    toks = vu.prompt(oracle.cfg, length, 21)
    _check(runner, oracle, {"w": toks}, [[("w", length)]], "float32")
    _check(runner, oracle, {"d": toks}, [[("d", 1)]] * length, "float32")          # the first tokens, long decoding
    for sizes in ([2], [5, 3, 2, 1, 17], [16, 1, 15, 33], [64, 7]):
        _check(runner, oracle, {"p": toks}, [[("p", q)] for q in vu.cuts(length, sizes)], "float32")


@pytest.mark.parametrize("device,name,lengths", [pytest.param("cpu", "tiny", [20, 3, 11], id="host"),
                                                 pytest.param("cuda", "mixed", [130, 9, 71, 40, 1, 100], marks=pytest.mark.gpu, id="gpu")])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(device, name, lengths, folders, kernels):
    """Portions of some requests beside single tokens of others; more requests than slots, a pool smaller than all
    of them together, so that pages and slots that were written are handed out again (nothing clears them)."""
    kernels(device)
    oracle = ru.Oracle(folders[name])
    page = 16
    runner = vu.make_runner(folders[name], "float32", device, page_size=page, max_requests=3,
                            num_pages=sum(sorted(-(-n // page) for n in lengths)[-3:]))
    reqs = {f"r{i}": vu.prompt(oracle.cfg, n, 30 + i) for i, n in enumerate(lengths)}
    rng = np.random.RandomState(5)
    waiting, live, at, schedule = list(reqs), [], {k: 0 for k in reqs}, []
    while waiting or live:
        while waiting and len(live) < 3:
            live.append(waiting.pop(0))
        step = []
        for rid in list(live):
            rest = len(reqs[rid]) - at[rid]
            if len(live) > 1 and rng.rand() < 0.25:
                continue
            q = 1 if rest <= 6 else int(min(rest - 6, rng.choice([2, 3, 16, 17, 40])))
            step.append((rid, q))
            at[rid] += q
            if at[rid] == len(reqs[rid]):
                live.remove(rid)
        if step:
            schedule.append(step)
    assert any(len(s) > 1 and {q for _, q in s} != {1} and 1 in {q for _, q in s} for s in schedule)
    _check(runner, oracle, reqs, schedule, "float32")
    # and once more on the same runner: every page and slot has been used before
    _check(runner, oracle, reqs, schedule, "float32")


@pytest.mark.gpu
@pytest.mark.parametrize("name,page", [("mixed", 16), ("serving_heads", 64), ("odd", 16)])
def test_bfloat16_serving_path(name, page, folders, kernels):
    """(`serving_heads`: keys and values of 64 and of 128 on pages of 64 tokens, the shapes that the tensor-core
    attention kernels take; its windows end inside pages, and one layer keeps more first tokens than a page.)"""
    kernels("cuda")
    oracle = ru.Oracle(folders[name + "/bf16"])
    runner = vu.make_runner(folders[name + "/bf16"], "bfloat16", "cuda", num_pages=24, max_tokens=512, page_size=page)
    reqs = {"a": vu.prompt(oracle.cfg, 300, 41), "b": vu.prompt(oracle.cfg, 45, 42)}
    _check(runner, oracle, reqs, [[("a", 300)], [("b", 45)]], "bfloat16")
    _check(runner, oracle, reqs, [[("a", 270), ("b", 2)], [("a", 1), ("b", 20)]] + [[("a", 1), ("b", 1)]] * 23 + [[("a", 1)]] * 6,
           "bfloat16")


@pytest.mark.gpu
def test_float32_on_the_serving_head_sizes(folders, kernels):
    kernels("cuda")
    oracle = ru.Oracle(folders["serving_heads"])
    runner = vu.make_runner(folders["serving_heads"], "float32", "cuda", num_pages=8, max_tokens=512, page_size=64)
    reqs = {"a": vu.prompt(oracle.cfg, 260, 43), "b": vu.prompt(oracle.cfg, 75, 44)}
    _check(runner, oracle, reqs, [[("a", 200), ("b", 2)], [("a", 30), ("b", 70)]] + [[("a", 1), ("b", 1)]] * 3 + [[("a", 1)]] * 27, "float32")


# ---- the engine: scheduler, batching, sampling, entry point -----------------------------------------------------
@pytest.mark.parametrize("device,name,lens,new", [pytest.param("cpu", "tiny", [1, 9, 20], 5, id="host"),
                                                  pytest.param("cuda", "mixed", [1, 33, 150, 7, 64, 90], 24, marks=pytest.mark.gpu, id="gpu")])
def test_greedy_generation_through_the_entry_point(device, name, lens, new, folders, kernels):
    """More requests than slots, prompts cut into portions of 16 beside other requests' decoding; on a GPU pure
    decode steps run as captured graphs."""
    kernels(device)
    from vapi_b200 import LLM, SamplingParams
    oracle = ru.Oracle(folders[name])
    llm = LLM(folders[name], dtype="f32", device=device, num_blocks=40, page_size=16, max_concurrent_seqs=4,
              max_batched_tokens=64, prefill_chunk_tokens=16, max_context=256, cuda_graphs=device == "cuda")
    prompts = [vu.prompt(oracle.cfg, n, 50 + i) for i, n in enumerate(lens)]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    for p, c in zip(prompts, out):
        want = oracle.greedy(p, new)
        if c.tokens != want:                 # only a near-tie of the plain model's own logits may part them
            i = next(k for k in range(new) if c.tokens[k] != want[k])
            top = torch.topk(oracle.logits(list(p) + want[:i])[-1], 2).values
            assert float(top[0] - top[1]) < 1e-3, f"prompt of {len(p)}: token {i} differs without a tie"
    llm.runner.cache.check_invariants()


# ---- trace replay: the program a user replays a trace with ----------------------------------------------------------
def _trace(cfg):
    import replay_util as rp
    reqs = {f"r{i}": vu.prompt(cfg, n, 70 + i) for i, n in enumerate([1, 70, 40, 90, 66])}
    tr = rp.Trace()
    rp.whole(tr, "w", reqs["r1"])
    rp.tail_decode(tr, "t", reqs["r2"], tail=5)
    rp.portions(tr, "p", reqs["r3"], sizes=[2, 3, 61, 2, 1])
    mix = {f"m{k}": v for k, v in reqs.items()}
    rp.mixed(tr, mix, seed=5, decode_tail=3)
    return tr, {"w": reqs["r1"], "t": reqs["r2"], "p": reqs["r3"], **mix}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(dtype, folders, tmp_path):
    import replay_util as rp
    name = "mixed" if dtype == "float32" else "mixed/bf16"
    oracle = ru.Oracle(folders[name])
    tr, tokens = _trace(oracle.cfg)
    got = rp.run_trace(folders[name], dtype, tr, str(tmp_path / "out"))
    ref = {k: oracle.logits(v).float() for k, v in tokens.items()}
    span = max(float(r.max() - r.min()) for r in ref.values())
    e = np.array([np.abs(got[step][i] - ref[rid][pos].numpy()).max() / span
                  for step, rows in tr.rows.items() for i, (rid, pos) in enumerate(rows)])
    assert np.isfinite(e).all()
    if dtype == "float32":
        assert e.max() <= vu.limit(dtype), f"worst {e.max():.3e} of the logit range"
    else:
        assert e.mean() <= 0.02 and np.percentile(e, 95) <= vu.limit(dtype) and e.max() <= 0.15
