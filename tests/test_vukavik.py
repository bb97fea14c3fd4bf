"""Vukavik through the framework's own step function, cache manager, scheduler and kernels, against
the plain model of ``plain_vukavik.py``.  The same cases run twice: on the host with plain Python
standing in for the kernels (what is under test there is the cache manager, the packer, the plan
and the parts' wiring), and on a GPU with the kernels themselves."""
import math

import numpy as np
import pytest
import torch

import plain_ops
import plain_vukavik as plain
import vukavik_util as vu

HOST = pytest.param("cpu", id="host")
GPU = pytest.param("cuda", marks=pytest.mark.gpu, id="gpu")


@pytest.fixture()
def kernels(request, monkeypatch):
    """On the host the plain restatements stand in for the kernels; on a GPU nothing is replaced."""
    def use(device):
        if device == "cpu":
            from vapi_b200 import ops
            for name in plain_ops.ALL:
                monkeypatch.setattr(ops, name, getattr(plain_ops, name))
    return use


def _folder(tmp_path_factory, name, cfg, seed, dtype=torch.float32):
    return vu.write_model(str(tmp_path_factory.mktemp(name)), cfg, seed, dtype)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg, seed in (("mixed", vu.MIXED, 1), ("tiny", vu.TINY, 2), ("no_attention", vu.NO_ATTENTION, 3),
                            ("plain_attention", vu.PLAIN_ATTENTION, 4), ("serving_heads", vu.SERVING_HEADS, 6)):
        out[name] = _folder(tmp_path_factory, name, cfg, seed)
        out[name + "/bf16"] = vu.write_model(str(tmp_path_factory.mktemp(name + "bf16")), cfg, seed, torch.bfloat16, std=0.05)
    for kind, layer in (("attention", vu.attention(ff=None)), ("delta", vu.delta()), ("mamba2", vu.mamba2()),
                        ("delta_shared_keys", vu.delta(heads=6, kv_heads=2, dim=40, vdim=20, conv=4)),
                        ("delta_wide", vu.delta(heads=1, kv_heads=1, dim=136, vdim=72, conv=1)),
                        ("mamba2_wide", vu.mamba2(heads=3, vdim=40, state=72, groups=3, conv=8, norm_groups=3)),
                        ("attention_wide", vu.attention(heads=2, kv_heads=1, dim=136, vdim=72, chunk=33, rot_dims=64, ff=None))):
        out[kind] = _folder(tmp_path_factory, kind, vu.config([layer]), 5)
    return out


def _check(runner, oracle, requests, schedule, dtype):
    got = vu.run_schedule(runner, requests, schedule)
    for rid, toks in requests.items():
        err, pos = vu.worst(got[rid], oracle.logits(toks))
        if dtype == "bfloat16":
            # The norm behind every sublayer enlarges the rounding of a sublayer whose output happens to be
            # small, so single positions stand out, the same ones whichever kernels run: measured on these
            # models over 300 positions, mean 1.0 to 1.1 %, 95th percentile 1.9 to 2.8 %, worst 3.4 to 11 % of
            # the logit range (the general attention kernel and the tensor-core ones within 1 % of each
            # other at every position).  Edges are what the float32 cases and the planted keys pin down.
            want = oracle.logits(toks).numpy()
            e = np.abs(got[rid] - want).max(-1) / float(want.max() - want.min())
            assert e.mean() <= 0.02 and np.percentile(e, 95) <= vu.limit(dtype) and err <= 0.15, \
                f"request {rid}: mean {e.mean():.3e}, 95th percentile {np.percentile(e, 95):.3e}, worst {err:.3e} of the logit range at {pos}"
        else:
            assert err <= vu.limit(dtype), f"request {rid}: {err:.3e} of the logit range at position {pos} of {len(toks)}"


# ---- configuration and registry --------------------------------------------------------------------
def test_the_architecture_is_found_by_its_name_and_every_size_comes_from_the_configuration():
    from vapi_b200.config.model import ConfigError, resolve_architecture
    arch = resolve_architecture(vu.MIXED)
    assert arch.name == "Vukavik"
    plan = arch.plan(arch.parse(vu.MIXED))
    shapes = {s.name: tuple(s.shape) for s in plan.tensor_specs()}
    assert shapes["embed"] == (200, 64) and shapes["head"] == (200, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.q"] == (32, 64) and shapes["l0.mix.v.conv"] == (96, 3) and shapes["l0.mlp.down"] == (64, 96)
    assert shapes["l1.mix.q"] == (64, 64) and shapes["l1.mix.v"] == (48, 64) and shapes["l1.mix.o"] == (64, 96)
    assert shapes["l1.mix.sink"] == (4,) and shapes["l1.mix.g"] == (4, 64) and shapes["l1.mix.q.norm"] == (16,)
    assert shapes["l2.mix.in"] == (2 * 64 + 2 * 2 * 24 + 4, 64) and shapes["l2.mix.conv"] == (64 + 96, 4)
    assert "l2.norm2" not in shapes and "l0.norm2b" in shapes and "l2.norm1b" in shapes
    assert len(plan.position_encodings) == 2, "layers with unlike rotations get tables of their own"
    kinds = {type(s).__name__ for _, s in plan.cache_sites()}
    assert kinds == {"PagedSpec", "StateSpec"}
    for bad in ({**vu.MIXED, "layers": [{"type": "conv", "mixer": {}, "mlp": None}]},
                {**vu.MIXED, "layers": [dict(vu.delta(), mlp={"kind": "sparse", "ff": 8})]},
                {k: v for k, v in vu.MIXED.items() if k != "residual_mult"}):
        with pytest.raises(ConfigError):
            arch.parse(bad)


def test_scaled_frequencies_by_hand():
    from vapi_b200.parts import ScaledRotaryEncoding
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    f, mult = ScaledRotaryEncoding.frequencies(8, 100.0, sc)
    # pair index at which a wave makes t turns in 64 positions: 8 ln(64 / (2 pi t)) / (2 ln 100)
    lo = max(math.floor(8 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(100.0))), 0)
    hi = min(math.ceil(8 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(100.0))), 7)
    assert (lo, hi) == (0, 3)
    base = [100.0 ** (-2 * i / 8) for i in range(4)]
    want = [b / 4.0 * r + b * (1 - r) for b, r in zip(base, [0.0, 1 / 3, 2 / 3, 1.0])]
    assert f == pytest.approx(want) and mult == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert ScaledRotaryEncoding.frequencies(8, 100.0, None) == (base, 1.0)
    assert plain.rotary_frequencies({"dims": 8, "base": 100.0, "scaling": sc})[0] == pytest.approx(want)


# ---- the plain model itself ----------------------------------------------------------------------------
def test_the_plain_model_is_causal_and_its_recurrences_run_by_hand():
    cfg = vu.TINY
    w = {}
    from vapi_b200.config.model import resolve_architecture
    arch = resolve_architecture(cfg)
    g = torch.Generator().manual_seed(0)
    for s in arch.plan(arch.parse(cfg)).tensor_specs():
        w[s.name] = torch.randn(s.shape, generator=g, dtype=torch.float64) * 0.3
    toks = vu.prompt(cfg, 25, 0)
    a, b = plain.forward(cfg, w, toks), plain.forward(cfg, w, toks[:13])
    assert torch.allclose(a[:13], b, atol=1e-12)
    # one head of the delta rule, two tokens, by hand: S1 = k1 (b1 v1)^T; o1 = S1^T q1
    x = torch.tensor([[1.0, 2.0], [0.5, -1.0]], dtype=torch.float64)
    assert torch.allclose(plain.causal_conv(x, torch.tensor([[2.0, 1.0], [0.0, 3.0]], dtype=torch.float64)),
                          torch.tensor([[1.0, 6.0], [2.5, -3.0]], dtype=torch.float64))
    assert float(plain.softplus(torch.tensor(0.0, dtype=torch.float64))) == pytest.approx(math.log(2.0))


# ---- each mechanism alone: one layer of it ---------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["attention", "delta", "mamba2", "delta_shared_keys", "delta_wide", "mamba2_wide",
                                  "attention_wide"])
def test_one_layer_of_each_mixer(kind, folders, kernels):
    kernels("cuda")
    oracle = vu.Oracle(folders[kind])
    runner = vu.make_runner(folders[kind], "float32", "cuda", num_pages=12)
    toks = vu.prompt(oracle.cfg, 150, 11)
    _check(runner, oracle, {"a": toks}, [[("a", 150)]], "float32")
    _check(runner, oracle, {"b": toks}, [[("b", q)] for q in vu.cuts(150, [37, 2, 1, 64, 3])], "float32")


# ---- prompts, decoding, portions ---------------------------------------------------------------------------
@pytest.mark.parametrize("device,name,length", [pytest.param("cpu", "tiny", 24, id="host"),
                                                pytest.param("cuda", "mixed", 140, marks=pytest.mark.gpu, id="gpu"),
                                                pytest.param("cuda", "no_attention", 90, marks=pytest.mark.gpu, id="gpu-no-attention"),
                                                pytest.param("cuda", "plain_attention", 140, marks=pytest.mark.gpu, id="gpu-plain-attention")])
def test_whole_prompt_token_by_token_and_portions_agree_with_the_plain_model(device, name, length, folders, kernels):
    kernels(device)
    oracle = vu.Oracle(folders[name])
    runner = vu.make_runner(folders[name], "float32", device, num_pages=12)
    toks = vu.prompt(oracle.cfg, length, 21)
    _check(runner, oracle, {"w": toks}, [[("w", length)]], "float32")
    _check(runner, oracle, {"d": toks}, [[("d", 1)]] * length, "float32")          # the first tokens, long decoding
    for sizes in ([2], [5, 3, 2, 1, 17], [16, 1, 15, 33], [64, 7]):
        _check(runner, oracle, {"p": toks}, [[("p", q)] for q in vu.cuts(length, sizes)], "float32")


@pytest.mark.parametrize("device,name,lengths", [pytest.param("cpu", "tiny", [20, 3, 11], id="host"),
                                                 pytest.param("cuda", "mixed", [130, 9, 71, 40, 1, 100], marks=pytest.mark.gpu, id="gpu")])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(device, name, lengths, folders, kernels):
    """Portions of some requests beside single tokens of others; more requests than slots, a pool
    smaller than all of them together, so that pages and slots that were written are handed out
    again (nothing clears them)."""
    kernels(device)
    oracle = vu.Oracle(folders[name])
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
            left = len(reqs[rid]) - at[rid]
            if len(live) > 1 and rng.rand() < 0.25:
                continue
            q = 1 if left <= 6 else int(min(left - 6, rng.choice([2, 3, 16, 17, 40])))
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
@pytest.mark.parametrize("name,page", [("mixed", 16), ("plain_attention", 16), ("serving_heads", 64)])
def test_bfloat16_serving_path(name, page, folders, kernels):
    """(`serving_heads`: keys and values of 64 and of 128 on pages of 64 tokens, the shapes that the
    tensor-core attention kernels take.)"""
    kernels("cuda")
    oracle = vu.Oracle(folders[name + "/bf16"])
    runner = vu.make_runner(folders[name + "/bf16"], "bfloat16", "cuda", num_pages=24, max_tokens=512, page_size=page)
    reqs = {"a": vu.prompt(oracle.cfg, 300, 41), "b": vu.prompt(oracle.cfg, 45, 42)}
    _check(runner, oracle, reqs, [[("a", 300)], [("b", 45)]], "bfloat16")
    _check(runner, oracle, reqs, [[("a", 270), ("b", 2)], [("a", 1), ("b", 20)]] + [[("a", 1), ("b", 1)]] * 23 + [[("a", 1)]] * 6,
           "bfloat16")


# ---- chunk edges, far keys, the sink: inputs made so that one key decides -----------------------------------
def _planted(klen, qlen, j_star, dk=16, dv=8, page=16, nh=2, nkv=1, device="cuda", dtype=torch.float32):
    """A cache in which key j_star matches the queries a thousand times better than any other and
    carries the value 1 where all others carry 0; pages are taken in a scrambled order."""
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
@pytest.mark.parametrize("qlen", [1, 5, 40, 100])
def test_a_planted_key_is_seen_exactly_where_the_mask_allows(qlen, dk, dv, page, dtype):
    """In bfloat16 the equal widths run on the tensor-core kernels (one warp for few rows, four warps,
    tcgen05 from 64 tokens on), everything else on the general kernel."""
    from vapi_b200 import ops
    chunk, klen = 48, 150                                     # chunks end inside pages
    for j_star in (3, 47, 48, 95, 96, 143, 144, 149):
        q, cache, table = _planted(klen, qlen, j_star, dk=dk, dv=dv, page=page, dtype=dtype)
        cu = torch.tensor([0, qlen], dtype=torch.int32, device="cuda")
        kl = torch.tensor([klen], dtype=torch.int32, device="cuda")
        sinks = torch.tensor([-30.0, -30.0], device="cuda")
        for ch, splits in ((chunk, 1), (chunk, 3), (0, 1), (0, 4)):
            out = ops.masked_attention(q, q.stride(0), cache, page, table, cu, kl, qlen, 1, qlen, klen, 2, 1, dk, dv, 1.0,
                                       chunk=ch, sinks=sinks, splits=splits).float().cpu()
            for i in range(qlen):
                p = klen - qlen + i
                seen = j_star <= p and (ch == 0 or j_star // ch == p // ch)
                assert abs(float(out[i].mean()) - (1.0 if seen else 0.0)) < 0.02, \
                    f"key {j_star}, query at {p}, chunk {ch}, {splits} slices: {out[i].mean():.3f}, seen={seen}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,dk,dv,page,qlen", [(torch.float32, 16, 8, 16, 1), (torch.bfloat16, 64, 64, 64, 1),
                                                   (torch.bfloat16, 64, 64, 64, 70), (torch.bfloat16, 128, 128, 64, 20)])
def test_a_far_key_among_hundreds_and_the_sink_and_the_gate(dtype, dk, dv, page, qlen):
    from vapi_b200 import ops
    klen = 900
    q, cache, table = _planted(klen, qlen, 2, dk=dk, dv=dv, page=page, dtype=dtype)
    cu = torch.tensor([0, qlen], dtype=torch.int32, device="cuda")
    kl = torch.tensor([klen], dtype=torch.int32, device="cuda")
    args = (q, q.stride(0), cache, page, table, cu, kl, qlen, 1, qlen, klen, 2, 1, dk, dv, 1.0)
    tol = 0.01 if dtype == torch.float32 else 0.03
    for splits in (1, 5):
        out = ops.masked_attention(*args, splits=splits)
        assert abs(float(out.float().mean()) - 1.0) < tol
        # a sink as strong as the planted key's score halves the weights; a zero gate halves them again
        score = float((q[-1, :dk].float() * cache[int(table[0, 0]), 2 * dk:3 * dk].float()).sum())
        sinks = torch.tensor([score, -1e4], device="cuda")
        gate = torch.tensor([[0.0, 30.0]] * qlen, device="cuda", dtype=dtype)
        out = ops.masked_attention(*args, sinks=sinks, gate=gate, splits=splits).float().cpu()
        assert abs(float(out[-1, :dv].mean()) - 0.25) < tol and abs(float(out[-1, dv:].mean()) - 1.0) < tol
    want = plain_ops.masked_attention(*[a.cpu() if torch.is_tensor(a) else a for a in args], sinks=sinks.cpu(), gate=gate.cpu())
    assert torch.allclose(out, want.float(), atol=1e-4 if dtype == torch.float32 else 3e-2)


# ---- the recurrent kernels against their restatements, at sizes that are not powers of two ----------------------
def _step_meta(qlens, starts, slots, device):
    cu = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    pos = np.concatenate([np.arange(s, s + q) for q, s in zip(qlens, starts)]).astype(np.int32)
    seq = np.concatenate([np.full(q, i) for i, q in enumerate(qlens)]).astype(np.int32)
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=device)
    return t(cu), t(pos), t(seq), t(np.array(slots, dtype=np.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_recurrent_kernels_continue_from_their_state_and_start_fresh_at_position_zero(dtype):
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(7)
    qlens, starts, slots = [1, 9, 2, 33], [0, 5, 0, 1], [3, 0, 2, 1]
    cu, pos, seq, sl = _step_meta(qlens, starts, slots, "cuda")
    n = sum(qlens)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    # convolution: channels 52, four taps, state in front of a longer row
    C, L = 52, 4
    x = torch.randn((n, C + 7), generator=g).to(dtype)
    taps, bias = torch.randn((L, C), generator=g), torch.randn(C, generator=g)
    state = torch.randn((5, (L - 1) * C + 11), generator=g)
    want_state = state.clone()
    want = plain_ops.causal_conv_silu(x[:, 3:3 + C], taps, bias, want_state, sl.cpu(), seq.cpu(), cu.cpu(), pos.cpu(), 33)
    dstate = state.cuda()
    got = ops.causal_conv_silu(x.cuda()[:, 3:3 + C], taps.cuda(), bias.cuda(), dstate, sl, seq, cu, pos, 33)
    assert torch.allclose(got.float().cpu(), want.float(), atol=tol, rtol=tol)
    assert torch.allclose(dstate.cpu(), want_state, atol=1e-6)
    # delta rule: 6 heads over 2 key heads, keys of 20, values of 12; state space: 4 heads in 2 groups
    for nh, nkv, dk, dv in ((6, 2, 20, 12), (2, 2, 72, 40), (1, 1, 136, 8)):
        qkv = torch.randn((n, 2 * nkv * dk + nh * dv), generator=g).to(dtype)
        ab = torch.randn((n, 2 * nh + 3), generator=g).to(dtype)
        A, dtb = torch.rand(nh, generator=g) * 2 - 1, torch.randn(nh, generator=g)
        state = torch.randn((5, 9 + nh * dk * dv), generator=g)
        want_state = state.clone()
        want = plain_ops.gated_delta(qkv, ab[:, :2 * nh], A, dtb, want_state, 9, sl.cpu(), cu.cpu(), pos.cpu(), nh, nkv, dk, dv)
        dstate = state.cuda()
        got = ops.gated_delta(qkv.cuda(), ab.cuda()[:, :2 * nh], A.cuda(), dtb.cuda(), dstate, 9, sl, cu, pos, nh, nkv, dk, dv)
        assert torch.allclose(got.cpu(), want, atol=1e-4, rtol=1e-4), (nh, nkv, dk, dv)
        assert torch.allclose(dstate.cpu(), want_state, atol=1e-4, rtol=1e-4)
    for nh, groups, N, P in ((4, 2, 24, 12), (3, 1, 72, 40), (2, 2, 136, 8)):
        xbc = torch.randn((n, nh * P + 2 * groups * N), generator=g).to(dtype)
        dt = torch.randn((n, nh + 5), generator=g).to(dtype)
        A, dtb, D = torch.rand(nh, generator=g) * 2 - 1, torch.randn(nh, generator=g), torch.randn(nh, generator=g)
        state = torch.randn((5, 4 + nh * N * P), generator=g)
        want_state = state.clone()
        want = plain_ops.state_space(xbc, dt[:, 2:2 + nh], A, dtb, D, want_state, 4, sl.cpu(), cu.cpu(), pos.cpu(), nh, groups, N, P)
        dstate = state.cuda()
        got = ops.state_space(xbc.cuda(), dt.cuda()[:, 2:2 + nh], A.cuda(), dtb.cuda(), D.cuda(), dstate, 4, sl, cu, pos, nh, groups, N, P)
        assert torch.allclose(got.cpu(), want, atol=1e-4, rtol=1e-4), (nh, groups, N, P)
        assert torch.allclose(dstate.cpu(), want_state, atol=1e-4, rtol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_kernels_of_the_blocks_and_the_gated_group_norm(dtype):
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(9)
    n, H = 7, 200
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    x, y = torch.randn((n, H), generator=g) * 3, (torch.randn((n, H), generator=g) * 5).to(dtype)
    wp, w = torch.randn(H, generator=g), torch.randn(H, generator=g)
    rows = torch.tensor([5, 0, 6], dtype=torch.int32)
    for r in (None, rows):
        xr, xd = x.clone(), x.cuda()
        want = plain_ops.postnorm_add_rmsnorm(xr, y, wp, 1e-5, 0.3, w, 1e-6, dtype, r)
        got = ops.postnorm_add_rmsnorm(xd, y.cuda(), wp.cuda(), 1e-5, 0.3, w.cuda(), 1e-6, dtype, None if r is None else r.cuda())
        assert torch.allclose(got.float().cpu(), want.float(), atol=tol, rtol=tol)
        assert torch.allclose(xd.cpu(), xr, atol=1e-5), "the stream is float32 and changes only without `rows`"
    xd = x.cuda()
    assert ops.postnorm_add_rmsnorm(xd, y.cuda(), wp.cuda(), 1e-5, 0.3, None, 0.0, dtype) is None
    xr = x.clone()
    plain_ops.postnorm_add_rmsnorm(xr, y, wp, 1e-5, 0.3, None, 0.0, dtype)
    assert torch.allclose(xd.cpu(), xr, atol=1e-5)
    for width, cases in ((120, ((40, 40, False), (60, 120, True), (120, 120, True), (24, 24, False))),
                         (2400, ((1200, 2400, True), (600, 600, False), (2400, 2400, True)))):      # wide groups: a block each
        yy, z = torch.randn((n, width), generator=g) * 2, torch.randn((n, width + 11), generator=g).to(dtype)
        for group, wlen, first in cases:
            wv = torch.randn(wlen, generator=g)
            want = plain_ops.gated_group_rmsnorm(yy, z[:, 4:4 + width], wv, 1e-5, group, first, dtype)
            got = ops.gated_group_rmsnorm(yy.cuda(), z.cuda()[:, 4:4 + width], wv.cuda(), 1e-5, group, first, dtype)
            assert torch.allclose(got.float().cpu(), want.float(), atol=tol, rtol=tol), (group, wlen, first)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_rotation_and_cache_write_for_unlike_widths(dtype):
    from vapi_b200 import ops
    g = torch.Generator().manual_seed(13)
    n, nh, nkv, dk, dv, page = 9, 3, 1, 24, 40, 16
    width = (nh + nkv) * dk + nkv * dv + nh + 5
    qkv = torch.randn((n, width), generator=g).to(dtype)
    qw, kw = torch.randn(dk, generator=g), torch.randn(dk, generator=g)
    pos = torch.arange(100, 100 + n, dtype=torch.int32)
    slots = torch.tensor([70, 71, 3, 4, 5, 130, 131, 0, 15], dtype=torch.int32)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for rot, inter in ((24, True), (10, True), (12, False)):
        freq = torch.rand(rot // 2, generator=g)
        cos, sin = plain_ops.rope_cos_sin_scaled(pos, freq, 1.2)
        dcos, dsin = ops.rope_cos_sin_scaled(pos.cuda(), freq.cuda(), 1.2)
        assert torch.allclose(dcos.cpu(), cos, atol=1e-5) and torch.allclose(dsin.cpu(), sin, atol=1e-5)
        cache = torch.zeros((9, page * nkv * (dk + dv)), dtype=dtype)
        a, b = qkv.clone(), qkv.cuda()
        dcache = cache.cuda()
        plain_ops.qk_norm_rope_write_split(a, nh, nkv, dk, dv, qw, kw, 1e-5, cos, sin, rot, inter, cache, page, slots)
        ops.qk_norm_rope_write_split(b, nh, nkv, dk, dv, qw.cuda(), kw.cuda(), 1e-5, dcos, dsin, rot, inter, dcache, page, slots.cuda())
        assert torch.allclose(b.float().cpu(), a.float(), atol=tol, rtol=tol)
        assert torch.allclose(dcache.float().cpu(), cache.float(), atol=tol, rtol=tol)
        assert torch.equal(b[:, -nh - 5:].cpu(), qkv[:, -nh - 5:]), "columns beyond the heads are left alone"


# ---- the engine: scheduler, batching, sampling, entry point -----------------------------------------------------
@pytest.mark.parametrize("device,name,lens,new", [pytest.param("cpu", "tiny", [1, 9, 20], 5, id="host"),
                                                  pytest.param("cuda", "mixed", [1, 33, 150, 7, 64, 90], 24, marks=pytest.mark.gpu, id="gpu")])
def test_greedy_generation_through_the_entry_point(device, name, lens, new, folders, kernels):
    """More requests than slots, prompts cut into portions of 16 beside other requests' decoding;
    on a GPU pure decode steps run as captured graphs."""
    kernels(device)
    from vapi_b200 import LLM, SamplingParams
    oracle = vu.Oracle(folders[name])
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


# ---- trace replay: the program a user replays a trace with --------------------------------------------------------
def _compare_trace(tr, got, ref, dtype):
    """Differences of every wanted row as fractions of the logit range, judged as `_check` judges them."""
    span = max(float(r.max() - r.min()) for r in ref.values())
    e = np.array([np.abs(got[step][i] - ref[rid][pos].numpy()).max() / span
                  for step, rows in tr.rows.items() for i, (rid, pos) in enumerate(rows)])
    assert np.isfinite(e).all()
    if dtype == "float32":
        assert e.max() <= vu.limit(dtype), f"worst {e.max():.3e} of the logit range"
    else:
        assert e.mean() <= 0.02 and np.percentile(e, 95) <= vu.limit(dtype) and e.max() <= 0.15, \
            f"mean {e.mean():.3e}, 95th percentile {np.percentile(e, 95):.3e}, worst {e.max():.3e} of the logit range"


def _trace(cfg):
    import replay_util as ru
    reqs = {f"r{i}": vu.prompt(cfg, n, 70 + i) for i, n in enumerate([1, 70, 40, 90, 66])}
    tr = ru.Trace()
    ru.whole(tr, "w", reqs["r1"])
    ru.tail_decode(tr, "t", reqs["r2"], tail=5)
    ru.portions(tr, "p", reqs["r3"], sizes=[2, 3, 61, 2, 1])
    mix = {f"m{k}": v for k, v in reqs.items()}
    ru.mixed(tr, mix, seed=5, decode_tail=3)
    tokens = {"w": reqs["r1"], "t": reqs["r2"], "p": reqs["r3"], **mix}
    return tr, tokens


def test_trace_replay_bookkeeping_on_the_host(folders, monkeypatch, capsys, tmp_path):
    import importlib.machinery
    import importlib.util
    import io
    import json
    import os
    import sys
    import replay_util as ru
    from vapi_b200 import ops
    for name in plain_ops.ALL:
        monkeypatch.setattr(ops, name, getattr(plain_ops, name))
    oracle = vu.Oracle(folders["tiny"])
    tr, tokens = _trace(oracle.cfg)
    loader = importlib.machinery.SourceFileLoader("trace_run_script", ru.TRACE_RUN)
    mod = importlib.util.module_from_spec(importlib.util.spec_from_loader("trace_run_script", loader))
    loader.exec_module(mod)
    monkeypatch.setattr(sys, "stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in tr.steps)))
    out_dir = str(tmp_path / "out")
    rc = mod.main(["--model", folders["tiny"], "--dtype", "float32", "--out", out_dir, "--max-tokens", str(tr.peak_tokens),
                   "--device", "cpu"])
    done = [int(l.split()[1]) for l in capsys.readouterr().out.splitlines() if l.startswith("done ")]
    assert rc == 0 and done == list(range(len(tr.steps)))
    got = {step: np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(len(rows), oracle.cfg["vocab"])
           for step, rows in tr.rows.items()}
    _compare_trace(tr, got, {k: oracle.logits(v).float() for k, v in tokens.items()}, "float32")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(dtype, folders, tmp_path):
    import replay_util as ru
    name = "mixed" if dtype == "float32" else "mixed/bf16"
    oracle = vu.Oracle(folders[name])
    tr, tokens = _trace(oracle.cfg)
    got = ru.run_trace(folders[name], dtype, tr, str(tmp_path / "out"))
    _compare_trace(tr, got, {k: oracle.logits(v).float() for k, v in tokens.items()}, dtype)
