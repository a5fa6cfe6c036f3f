"""Nezavik on the step engine against the plain float64 oracle (tests/nezavik_oracle.py): small random models of several
shapes, written to disk as a checkpoint, loaded through the model registry and run through ``HybridSampler.step`` /
``generate`` under different schedules (whole prompts, token by token, portions, mixed batches, reused pages and slots)."""
import json
import math
import os

import pytest
import torch

import nezavik_oracle as O

pytestmark = pytest.mark.gpu


# ---- helpers -----------------------------------------------------------------------------------------------------
def _save(tmp_path, cfg, W, name="m"):
    from safetensors.torch import save_file
    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in W.items()}, os.path.join(d, "model.safetensors"))
    return d


def _engine(tmp_path, cfg, W, dtype="fp32", pool_tokens=1024, slots=4, name="m", **kw):
    from nanorlhf_b200.models.registry import load_model
    from nanorlhf_b200.sampler.hybrid_sampler import HybridSampler
    path = _save(tmp_path, cfg, W, name)
    model = load_model(path, torch_dtype=torch.float32 if dtype == "fp32" else torch.bfloat16, device="cuda")
    eng = HybridSampler(model, dtype=dtype, max_num_seqs=slots, **kw)
    eng.reset_pool(pool_tokens, slots)
    return eng


def _tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def _run_alone(eng, toks, cuts):
    """Feed one sequence in portions ``cuts``; logits of every position."""
    sid = eng.open()
    out, lo = [], 0
    for n in cuts:
        out.append(eng.step([(sid, toks[lo:lo + n], list(range(n)))]).double().cpu())
        lo += n
    eng.close(sid)
    assert lo == len(toks)
    return torch.cat(out)


def _rel(got, want):
    """Worst row error relative to the RMS of the oracle's logits."""
    return ((got - want).pow(2).mean(-1).sqrt().max() / want.pow(2).mean().sqrt()).item()


def _cuts(total, sizes):
    out, i, k = [], 0, 0
    while i < total:
        n = min(sizes[k % len(sizes)], total - i)
        out.append(n)
        i += n
        k += 1
    return out


F32_TOL = 2e-4
BF16_TOL = 6e-2

SHAPES = {
    # every size differs from its neighbours: dim != vdim, state != vdim, kv_heads < heads, groups < heads, parts of the
    # gated norm != heads, window not a multiple of the page, taps differ between the mixers
    "mixed": dict(layers=("parallel", "channel_delta", "delta", "parallel"), sizes={}),
    "single_heads": dict(layers=("delta", "parallel", "channel_delta"),
                         sizes=dict(heads=2, kv_heads=1, dim=8, vdim=40, window=16, s_heads=3, s_groups=1, s_norm_groups=1,
                                    s_state=8, s_vdim=24, s_conv=2, d_heads=3, d_kv=1, d_dim=24, d_vdim=8, d_conv=2, ff=0)),
    "roomy_heads": dict(layers=("channel_delta", "parallel", "parallel", "delta"),
                        sizes=dict(heads=4, kv_heads=1, dim=64, vdim=32, window=50, s_heads=2, s_groups=1, s_norm_groups=1,
                                   s_state=64, s_vdim=32, s_conv=4, d_heads=2, d_kv=2, d_dim=32, d_vdim=64, d_conv=3, ff=72)),
    "wide_window": dict(layers=("parallel",), sizes=dict(heads=4, kv_heads=4, dim=16, vdim=16, window=300, s_heads=2, s_groups=2,
                                                        s_norm_groups=2, s_state=16, s_vdim=16, s_conv=5)),
}


def _model(name, seed=0, width=40, vocab=97):
    s = SHAPES[name]
    cfg = O.make_config(vocab=vocab, width=width, max_positions=512, layers=s["layers"], seed_sizes=s["sizes"])
    return cfg, O.make_weights(cfg, seed=seed, rank=6)


# ---- each layer type alone, whole prompt -------------------------------------------------------------------------
@pytest.mark.parametrize("layer", ["parallel", "delta", "channel_delta"])
@pytest.mark.parametrize("side", ["both", "left", "right"])
def test_single_layer_types(tmp_path, layer, side):
    if layer != "parallel" and side != "both":
        pytest.skip("only the parallel layer has two sides")
    sizes = {"left": dict(right_scale=0.0), "right": dict(left_scale=0.0), "both": {}}[side]
    cfg = O.make_config(layers=(layer,), seed_sizes=sizes, max_positions=128)
    W = O.make_weights(cfg, seed=3)
    toks = _tokens(cfg, 45, 1)
    want = O.forward(cfg, W, toks)
    eng = _engine(tmp_path, cfg, W)
    assert _rel(_run_alone(eng, toks, [len(toks)]), want) < F32_TOL


def test_layer_stream_matches_after_every_layer(tmp_path):
    """The depth-weighted stream after each layer, not only the logits."""
    cfg, W = _model("mixed")
    toks = _tokens(cfg, 20, 2)
    # the engine's stream buffer is internal: compare through truncated models, whose logits read the stream at that depth
    for depth in range(1, len(cfg["layers"]) + 1):
        sub = dict(cfg, layers=cfg["layers"][:depth])
        Wsub = {k: v for k, v in W.items() if not k.startswith("l") or int(k[1:k.index(".")]) < depth}
        want = O.forward(sub, Wsub, toks)
        e2 = _engine(tmp_path, sub, Wsub, name=f"d{depth}")
        assert _rel(_run_alone(e2, toks, [len(toks)]), want) < F32_TOL


# ---- schedules ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])             # bf16: tensor-core attention, bf16 pages and GEMM operands
@pytest.mark.parametrize("shape", list(SHAPES))
def test_prefill_decode_and_portions_agree_with_oracle(tmp_path, shape, dtype):
    cfg, W = _model(shape)
    n = 330 if shape == "wide_window" else 90
    toks = _tokens(cfg, n, 5)
    want = O.forward(cfg, W, toks)
    eng = _engine(tmp_path, cfg, W, dtype=dtype)
    whole = _run_alone(eng, toks, [n])
    if dtype == "bf16":
        assert _rel(whole, want) < BF16_TOL
        for name, cuts in {"prefill_then_decode": [n - 40] + [1] * 40, "ragged": _cuts(n, [3, 37, 2, 16, 1, 17, 5])}.items():
            got = _run_alone(eng, toks, cuts)
            assert _rel(got, want) < BF16_TOL, name
            assert _rel(got, whole) < BF16_TOL / 2, name      # different kernels for portions and single tokens: bf16 rounding
        return
    assert _rel(whole, want) < F32_TOL
    schedules = {
        "by_token": [1] * n,
        "prefill_then_decode": [n - 40] + [1] * 40,
        "pairs": _cuts(n, [2]),
        "ragged": _cuts(n, [3, 37, 2, 16, 1, 17, 5]),
        "page_edges": _cuts(n, [15, 1, 16, 17, 31]),
    }
    for name, cuts in schedules.items():
        got = _run_alone(eng, toks, cuts)
        assert _rel(got, want) < F32_TOL, name
        assert _rel(got, whole) < 5e-5, name              # the cut must not matter beyond rounding


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_width_that_is_no_multiple_of_four(tmp_path, dtype):
    cfg, W = _model("mixed", seed=3, width=42, vocab=53)
    toks = _tokens(cfg, 60, 8)
    want = O.forward(cfg, W, toks)
    eng = _engine(tmp_path, cfg, W, dtype=dtype)
    tol = F32_TOL if dtype == "fp32" else BF16_TOL
    assert _rel(_run_alone(eng, toks, [60]), want) < tol
    assert _rel(_run_alone(eng, toks, [25, 3] + [1] * 32), want) < tol


def test_long_decode(tmp_path):
    cfg, W = _model("mixed")
    toks = _tokens(cfg, 260, 6)
    want = O.forward(cfg, W, toks)
    eng = _engine(tmp_path, cfg, W)
    assert _rel(_run_alone(eng, toks, [10] + [1] * 250), want) < F32_TOL


def test_single_token_sequence_and_first_tokens(tmp_path):
    cfg, W = _model("mixed")
    eng = _engine(tmp_path, cfg, W)
    for n in (1, 2, 3, 5):
        toks = _tokens(cfg, n, 10 + n)
        want = O.forward(cfg, W, toks)
        assert _rel(_run_alone(eng, toks, [n]), want) < F32_TOL
        assert _rel(_run_alone(eng, toks, [1] * n), want) < F32_TOL


def test_mixed_batches_and_reuse_of_pages_and_slots(tmp_path):
    """Unequal requests run together (portions beside single tokens), more requests than slots over time, a pool that only
    fits the live ones: every request must come out as it does alone."""
    cfg, W = _model("mixed")
    lens = [70, 33, 1, 48, 95, 17, 64]
    reqs = [_tokens(cfg, n, 20 + i) for i, n in enumerate(lens)]
    want = [O.forward(cfg, W, t) for t in reqs]
    slots = 3
    eng = _engine(tmp_path, cfg, W, pool_tokens=16 * (5 + 3 + 6 + 1), slots=slots)      # three live requests at most
    portion = [[5, 1, 1, 30, 2, 1], [33], [1], [16, 16, 1, 1, 14], [40, 1, 1, 1, 50, 2], [2, 2, 2, 11], [63, 1]]
    portion = [_cuts(n, p) for n, p in zip(lens, portion)]
    got = [[] for _ in reqs]
    at = [0] * len(reqs)
    part = [0] * len(reqs)
    live, waiting, sid = [], list(range(len(reqs))), {}
    seen_slots, seen_pages = set(), []
    steps = 0
    while live or waiting:
        while waiting and len(live) < slots:
            r = waiting.pop(0)
            sid[r] = eng.open()
            seen_slots.add((r, eng.sched.slot_of(sid[r])))
            live.append(r)
        batch = [r for k, r in enumerate(live) if (steps + k) % 4 != 3] or live[:1]        # some requests sit a step out
        entries = []
        for r in batch:
            n = portion[r][part[r]]
            entries.append((sid[r], reqs[r][at[r]:at[r] + n], list(range(n))))
        logits = eng.step(entries).double().cpu()
        o = 0
        for r in batch:
            n = portion[r][part[r]]
            got[r].append(logits[o:o + n])
            o += n
            at[r] += n
            part[r] += 1
            if at[r] == lens[r]:
                seen_pages.append(set(eng.sched.block_table(sid[r])))
                eng.close(sid[r])
                live.remove(r)
        steps += 1
    for r in range(len(reqs)):
        assert _rel(torch.cat(got[r]), want[r]) < F32_TOL, r
    used = [s for _, s in seen_slots]
    assert len(set(used)) <= slots < len(used)                       # slots were handed out again
    assert any(a & b for i, a in enumerate(seen_pages) for b in seen_pages[i + 1:])       # and so were pages
    assert eng.sched.num_free_blocks() == eng.num_blocks and eng.sched.num_free_slots() == slots


def test_batch_equals_alone_bitwise_close(tmp_path):
    cfg, W = _model("single_heads")
    a, b = _tokens(cfg, 50, 31), _tokens(cfg, 21, 32)
    eng = _engine(tmp_path, cfg, W)
    alone_a, alone_b = _run_alone(eng, a, [50]), _run_alone(eng, b, [20, 1])
    sa, sb = eng.open(), eng.open()
    l1 = eng.step([(sb, b[:20], list(range(20))), (sa, a[:49], list(range(49)))]).double().cpu()
    l2 = eng.step([(sa, a[49:], [0]), (sb, b[20:], [0])]).double().cpu()
    eng.close(sa), eng.close(sb)
    got_a = torch.cat([l1[20:], l2[:1]])
    got_b = torch.cat([l1[:20], l2[1:]])
    assert _rel(got_a, alone_a) < 5e-5 and _rel(got_b, alone_b) < 5e-5


# ---- windows: one key made to stand out ---------------------------------------------------------------------------
def _attention_only_model(window, heads=2, kv_heads=1, dim=16, vdim=8, width=32, vocab=64, max_positions=1024):
    """One parallel layer whose state-space side is switched off, no feed-forward, and weights built so that token 1 is a
    'needle': its key matches the query of token 2 strongly and its value is unlike all others."""
    cfg = O.make_config(vocab=vocab, width=width, max_positions=max_positions, layers=("parallel",),
                        seed_sizes=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=window, scale=1.0,
                                        right_scale=0.0, left_scale=1.0, ff=0, s_heads=1, s_groups=1, s_norm_groups=1, s_state=4,
                                        s_vdim=4))
    W = O.make_weights(cfg, seed=11)
    W["pos"] = torch.zeros_like(W["pos"])                       # content only: a key looks the same wherever it sits
    emb = torch.randn(vocab, width, generator=torch.Generator().manual_seed(12)) * 0.05
    emb[:, 2] = 1.0                                             # a constant coordinate: the ordinary direction of q and k
    emb[1, 0], emb[2, 1] = 4.0, 4.0                             # needle / probe tokens live on their own coordinates
    W["embed"] = emb.to(torch.bfloat16)
    q = torch.zeros(heads * dim, width)
    k = torch.zeros(kv_heads * dim, width)
    v = torch.randn(kv_heads * vdim, width, generator=torch.Generator().manual_seed(13)) * 0.1
    q[::dim, 1] = 8.0                                            # probe token -> query along channel 0 of every head
    k[::dim, 0] = 8.0                                            # needle token -> key along channel 0
    q[1::dim, 2] = 8.0                                           # everyone else: channel 1
    k[1::dim, 2] = 8.0
    v[:, 0] = 3.0                                                # needle token -> a large value
    W["l0.mix.left.q"], W["l0.mix.left.k"], W["l0.mix.left.v"] = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    W["l0.mix.left.q.norm"] = torch.full((dim,), 3.0).to(torch.bfloat16)
    W["l0.mix.left.k.norm"] = torch.full((dim,), 3.0).to(torch.bfloat16)
    return cfg, W


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])             # bf16 pages: prompt portions run on the tensor-core kernel
@pytest.mark.parametrize("window", [16, 23, 70, 300])
def test_needle_just_inside_and_outside_the_window(tmp_path, window, dtype):
    cfg, W = _attention_only_model(window)
    eng = _engine(tmp_path, cfg, W, dtype=dtype, pool_tokens=2048)
    tol = F32_TOL if dtype == "fp32" else BF16_TOL
    fill = _tokens(cfg, 700, 40)
    fill = [t if t > 2 else 3 for t in fill]
    for needle_at in (0, 15, 16):                                # page starts and ends among them
        for dist, seen in ((window - 1, True), (window, False), (1, True)):
            probe_at = needle_at + dist
            toks = list(fill[:probe_at + 3])
            toks[needle_at], toks[probe_at] = 1, 2
            want = O.forward(cfg, W, toks)
            blind = list(toks)
            blind[needle_at] = 3
            effect = _rel(O.forward(cfg, W, blind)[probe_at:probe_at + 1], want[probe_at:probe_at + 1])
            assert (effect > 1e-2) == seen                       # the oracle itself tells inside from outside
            for cuts in ([len(toks)], [probe_at] + [1] * 3, _cuts(len(toks), [7, 2, 16])):
                got = _run_alone(eng, toks, cuts)
                err = _rel(got[probe_at:probe_at + 1], want[probe_at:probe_at + 1])
                assert err < tol and (not seen or err < 0.25 * effect), (needle_at, dist, cuts[:3])
                if dtype == "fp32":                              # (these scores are huge: in bf16 only the probe is telling)
                    assert _rel(got, want) < tol


@pytest.mark.parametrize("D,Dv,Hq,Hkv,window", [(128, 128, 8, 2, 100), (24, 16, 6, 3, 11), (64, 32, 4, 4, 40), (40, 72, 3, 1, 33),
                                                (16, 16, 5, 1, 17), (32, 128, 2, 1, 64), (16, 16, 34, 2, 20), (12, 10, 4, 2, 9)])
@pytest.mark.parametrize("step", ["portions", "single_tokens"])
def test_window_attention_kernels_against_plain_softmax(D, Dv, Hq, Hkv, window, step):
    """Every window-attention kernel on random bf16 pages, entries of unequal length with and without earlier context, against
    a masked softmax written out per query.  Scores are made peaky so that one wrongly seen or missed key shows."""
    from nanorlhf_b200 import _C
    from nanorlhf_b200.ops import hybrid as hy, native
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    native.load()
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(D * 1000 + window)
    old, new = [0, 37, 130, 5, 64, 200], [70, 1, 33, 2, 1, 17]
    if step == "single_tokens":                                  # a decode step: the key walk is cut into parts and merged
        old, new = [1, 37, 130, 15, 64, 200], [1] * 6
    sched = _C.StepScheduler(64, 16, len(old))
    sids = [sched.open() for _ in old]
    sched.plan([s for s, n in zip(sids, old) if n], [n for n in old if n])
    data, E, T, MB = sched.plan(sids, new)
    plan = StepPlan(torch.from_numpy(data).to(dev), E, T, MB)
    kc = (torch.randn(64, Hkv, 16, D, generator=g) * 1.5).to(torch.bfloat16).to(dev)
    vc = torch.randn(64, Hkv, 16, Dv, generator=g).to(torch.bfloat16).to(dev)
    q = (torch.randn(T, Hq * D, generator=g) * 1.5).to(torch.bfloat16).float().to(dev)      # bf16 values: no kernel rounds them
    scale, out_scale = 0.9 / math.sqrt(D) * 2.0, 0.7
    bt, te, pos = plan.block_table.cpu(), plan.tok_entry.cpu(), plan.pos.cpu()
    want = torch.zeros(T, Hq * Dv, dtype=torch.float64)
    kcd, vcd, qd = kc.double().cpu(), vc.double().cpu(), q.double().cpu()
    for t in range(T):
        e, p = int(te[t]), int(pos[t])
        js = list(range(max(0, p - window + 1), p + 1))
        pages = [int(bt[e, j // 16]) for j in js]
        for h in range(Hq):
            kv = h // (Hq // Hkv)
            K = torch.stack([kcd[pg, kv, j % 16] for pg, j in zip(pages, js)])
            V = torch.stack([vcd[pg, kv, j % 16] for pg, j in zip(pages, js)])
            w = torch.softmax((K @ qd[t, h * D:(h + 1) * D]) * scale, 0)
            want[t, h * Dv:(h + 1) * Dv] = out_scale * (w @ V)
    impls = ["simple", "tile"] if Dv % 4 == 0 else ["simple"]
    if D % 8 == 0 and Dv % 8 == 0 and D <= 128 and Dv <= 128:
        impls.append("mma")
    for impl in impls + ["auto"]:
        out = torch.zeros(T, Hq * Dv, dtype=torch.bfloat16, device=dev)
        hy.window_attention(q, kc, vc, plan, window, scale, out_scale, out, impl=impl)
        err = (out.double().cpu() - want).abs().max().item()
        assert err < 2e-2, (impl, err)


@pytest.mark.parametrize("part,nparts", [(12, 5), (10, 3), (64, 2), (256, 3), (300, 1), (1024, 2), (257, 2)])
@pytest.mark.parametrize("gate_act,gate_first", [("silu", True), ("sigmoid", False)])
def test_gated_part_rmsnorm_narrow_and_wide_parts(part, nparts, gate_act, gate_first):
    from nanorlhf_b200.ops import hybrid as hy, native
    native.load()
    g = torch.Generator().manual_seed(part)
    T, n = 9, part * nparts
    y, gate, w = torch.randn(T, n, generator=g), torch.randn(T, n, generator=g), torch.rand(n, generator=g) + 0.5
    act = (lambda z: z * torch.sigmoid(z)) if gate_act == "silu" else torch.sigmoid
    yd, gd = y.double().view(T, nparts, part), act(gate.double()).view(T, nparts, part)
    v = yd * gd if gate_first else yd
    v = v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5) * w.double().view(nparts, part)
    want = 0.6 * (v if gate_first else v * gd).view(T, n)
    out = torch.empty(T, n, device="cuda")
    hy.gated_part_rmsnorm(y.cuda(), gate.cuda(), w.cuda(), part, gate_act, gate_first, 1e-5, 0.6, out)
    assert (out.double().cpu() - want).abs().max() < 1e-4


def _scan_plan(old, new, dev):
    from nanorlhf_b200 import _C
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    sched = _C.StepScheduler(64, 16, len(old))
    sids = [sched.open() for _ in old]
    if any(old):
        sched.plan([s for s, n in zip(sids, old) if n], [n for n in old if n])
    data, E, T, MB = sched.plan(sids, new)
    return StepPlan(torch.from_numpy(data).to(dev), E, T, MB)


@pytest.mark.parametrize("heads,groups,N,P", [(4, 2, 20, 12), (2, 1, 128, 64), (3, 3, 64, 40), (2, 2, 130, 8), (1, 1, 16, 200)])
def test_state_space_scan_kernels_against_a_plain_loop(heads, groups, N, P):
    """Every implementation of the scan, entries of unequal length, some starting from a carried state."""
    from nanorlhf_b200.ops import hybrid as hy, native
    native.load()
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(N * 7 + P)
    old, new = [0, 5, 9, 0], [23, 1, 7, 2]
    plan = _scan_plan(old, new, dev)
    T, E = plan.T, plan.E
    ch = heads * P + 2 * groups * N
    xbc = torch.randn(T, ch + 3, generator=g)
    dt_raw, dt_bias = torch.randn(T, heads, generator=g), torch.randn(heads, generator=g)
    A_log, Dk = torch.rand(heads, generator=g) - 1.0, torch.randn(heads, generator=g)
    st0 = torch.randn(E, heads, N, P, generator=g)
    slots, cu, start = plan.state_slot.cpu().tolist(), plan.cu.cpu().tolist(), plan.start.cpu().tolist()
    want_y = torch.zeros(T, heads * P, dtype=torch.float64)
    want_s = st0.double().clone()
    for e in range(E):
        for h in range(heads):
            S = want_s[slots[e], h] if start[e] > 0 else torch.zeros(N, P, dtype=torch.float64)
            gi = h // (heads // groups)
            for t in range(cu[e], cu[e + 1]):
                r = xbc[t].double()
                x, B, C = r[h * P:(h + 1) * P], r[heads * P + gi * N:heads * P + (gi + 1) * N], r[heads * P + groups * N + gi * N:heads * P + groups * N + (gi + 1) * N]
                dt = torch.nn.functional.softplus(dt_raw[t, h].double() + dt_bias[h].double())
                S = torch.exp(-torch.exp(A_log[h].double()) * dt) * S + dt * torch.outer(B, x)
                want_y[t, h * P:(h + 1) * P] = S.T @ C + Dk[h].double() * x
            want_s[slots[e], h] = S
    ran = 0
    for impl in ("column", "rows", "shared", "auto"):
        st, y = st0.clone().to(dev), torch.zeros(T, heads * P, device=dev)
        try:
            hy.ssd_scan(xbc.to(dev), heads * P, heads * P + groups * N, dt_raw.to(dev), dt_bias.to(dev), A_log.to(dev), Dk.to(dev), st, y,
                        plan, groups, impl=impl)
        except RuntimeError:
            assert impl != "auto"                                # a kernel may not fit these sizes; "auto" always runs
            continue
        ran += 1
        assert (y.double().cpu() - want_y).abs().max() < 1e-3 * want_y.abs().max(), impl
        assert (st.double().cpu() - want_s).abs().max() < 1e-3 * want_s.abs().max(), impl
    assert ran >= 2


@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("heads,kv_heads,D,Dv", [(4, 2, 16, 24), (2, 2, 128, 128), (3, 1, 64, 40), (2, 1, 136, 8), (1, 1, 24, 260)])
def test_delta_rule_scan_kernels_against_a_plain_loop(heads, kv_heads, D, Dv, per_channel):
    from nanorlhf_b200.ops import hybrid as hy, native
    native.load()
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(D * 5 + Dv)
    old, new = [0, 5, 9, 0], [23, 1, 7, 2]
    plan = _scan_plan(old, new, dev)
    T, E = plan.T, plan.E
    nk, nv = kv_heads * D, heads * Dv
    qkv = torch.randn(T, 2 * nk + nv, generator=g)
    qkv[:, :2 * nk] = torch.nn.functional.normalize(qkv[:, :2 * nk].view(T, 2 * kv_heads, D), dim=-1).view(T, 2 * nk)
    beta = torch.rand(T, heads, generator=g)
    decay = torch.rand(T, heads * D if per_channel else heads, generator=g) * 0.5 + 0.5
    st0 = torch.randn(E, heads, D, Dv, generator=g)
    slots, cu, start = plan.state_slot.cpu().tolist(), plan.cu.cpu().tolist(), plan.start.cpu().tolist()
    want_o = torch.zeros(T, nv, dtype=torch.float64)
    want_s = st0.double().clone()
    for e in range(E):
        for h in range(heads):
            S = want_s[slots[e], h] if start[e] > 0 else torch.zeros(D, Dv, dtype=torch.float64)
            gi = h // (heads // kv_heads)
            for t in range(cu[e], cu[e + 1]):
                r = qkv[t].double()
                q, k, v = r[gi * D:(gi + 1) * D], r[nk + gi * D:nk + (gi + 1) * D], r[2 * nk + h * Dv:2 * nk + (h + 1) * Dv]
                gd = decay[t, h * D:(h + 1) * D].double()[:, None] if per_channel else decay[t, h].double()
                S = gd * S
                u = beta[t, h].double() * (v - S.T @ k)
                S = S + torch.outer(k, u)
                want_o[t, h * Dv:(h + 1) * Dv] = S.T @ q
            want_s[slots[e], h] = S
    ran = 0
    for impl in ("column", "rows", "shared", "auto"):
        st, o = st0.clone().to(dev), torch.zeros(T, nv, device=dev)
        try:
            hy.delta_scan(qkv.to(dev), nk, 2 * nk, beta.to(dev), decay.to(dev), st, o, plan, kv_heads, per_channel, impl=impl)
        except RuntimeError:
            assert impl != "auto"
            continue
        ran += 1
        assert (o.double().cpu() - want_o).abs().max() < 1e-3 * want_o.abs().max(), impl
        assert (st.double().cpu() - want_s).abs().max() < 1e-3 * want_s.abs().max(), impl
    assert ran >= 2


def test_far_memory_of_recurrent_layers(tmp_path):
    """A token far back still changes what the recurrent layers put out; the engine must carry it across portions and
    decoded tokens exactly as the whole-sequence evaluation does, and reproduce the change it causes."""
    n = 400
    for layer in ("delta", "channel_delta", "parallel"):
        cfg = O.make_config(layers=(layer,), max_positions=512, seed_sizes=dict(window=8, left_scale=0.0))
        W = O.make_weights(cfg, seed=21)
        for k in W:                                              # slow decay: memory reaches far
            if k.endswith("A_log"):
                W[k] = torch.full_like(W[k], -6.0)
        toks = _tokens(cfg, n, 50)
        want = O.forward(cfg, W, toks)
        far = None
        for dist in (390, 250, 120, 60):                         # the farthest change that still shows clearly
            other = list(toks)
            other[n - 1 - dist] = (toks[n - 1 - dist] + 1) % cfg["vocab"]
            want_other = O.forward(cfg, W, other)
            if _rel(want_other[-1:], want[-1:]) > 20 * F32_TOL:
                far = dist
                break
        assert far is not None, layer
        eng = _engine(tmp_path, cfg, W, name=layer)
        for cuts in ([n], [n - 40] + [1] * 40, _cuts(n, [64, 3, 2, 100])):
            got, got_other = _run_alone(eng, toks, cuts), _run_alone(eng, other, cuts)
            assert _rel(got, want) < F32_TOL and _rel(got_other, want_other) < F32_TOL
            d_got, d_want = got_other[-1:] - got[-1:], want_other[-1:] - want[-1:]
            assert (d_got - d_want).norm() < 0.1 * d_want.norm(), (layer, far)


# ---- serving precision, checkpoint round trip, generation ---------------------------------------------------------
def test_bf16_serving_mode_and_gemm_backends(tmp_path):
    cfg, W = _model("mixed", width=64)
    toks = _tokens(cfg, 80, 60)
    want = O.forward(cfg, W, toks)
    outs = {}
    for backend in ("tc", "vendor"):
        eng = _engine(tmp_path, cfg, W, dtype="bf16", gemm=backend)
        outs[backend] = _run_alone(eng, toks, [50] + [1] * 30)
        assert _rel(outs[backend], want) < BF16_TOL, backend
    assert _rel(outs["tc"], outs["vendor"]) < 1e-2


def test_greedy_generation_through_the_entry_point(tmp_path):
    from nanorlhf_b200.models.registry import load_model
    from nanorlhf_b200.sampler.engine import generate, release_native_engine
    from nanorlhf_b200.utils.tokenizer import ByteTokenizer
    cfg, W = _model("mixed", seed=4)
    path = _save(tmp_path, cfg, W)
    model = load_model(path, torch_dtype=torch.float32, device="cuda")
    tok = ByteTokenizer(vocab_size=cfg["vocab"])
    prompts = [_tokens(cfg, n, 70 + n) for n in (5, 19, 2, 33, 7)]
    new = 12
    # few slots and a small token budget: requests wait, prompts are cut into portions, slots are reused
    out = generate(1, model, tok, prompts, 0.0, new, top_p=1.0, seed=1, backend="native", eos_token_id=-1,
                   rollout_dtype="fp32", max_num_seqs=2, prefill_token_budget=8).cpu()
    release_native_engine(model)
    assert out.shape == (len(prompts), new)
    for p, row in zip(prompts, out.tolist()):
        seq = list(p)
        for t in row:
            lg = O.forward(cfg, W, seq)[-1]
            top2 = lg.topk(2).values
            if (top2[0] - top2[1]) / lg.std() < 1e-3:
                break                                            # a tie within rounding: either choice is greedy
            assert t == int(lg.argmax()), (len(p), len(seq))
            seq.append(t)


def test_sampled_generation_shapes_and_eos(tmp_path):
    from nanorlhf_b200.models.registry import load_model
    from nanorlhf_b200.sampler.engine import generate
    from nanorlhf_b200.utils.tokenizer import ByteTokenizer
    cfg, W = _model("single_heads", seed=5)
    model = load_model(_save(tmp_path, cfg, W), torch_dtype=torch.bfloat16, device="cuda")
    tok = ByteTokenizer(vocab_size=cfg["vocab"])
    prompts = [_tokens(cfg, n, 80 + n) for n in (4, 9)]
    a = generate(3, model, tok, prompts, 0.9, 10, top_p=0.95, seed=7, backend="native", eos_token_id=5)
    b = generate(3, model, tok, prompts, 0.9, 10, top_p=0.95, seed=7, backend="native", eos_token_id=5)
    assert a.shape == (6, 10) and torch.equal(a, b)              # seeded: reproducible
    for row in a.tolist():
        if 5 in row:
            assert all(t == tok.pad_token_id for t in row[row.index(5) + 1:])


# ---- the trace runner as a program ----------------------------------------------------------------------------------
def test_trace_runner_replays_a_mixed_trace(tmp_path):
    """bin/trace_run as a subprocess: five requests over four slots and a pool of 256 tokens, portions beside single tokens,
    requests that pause, end and hand their pages and slots to later ones; the dumped logits against the oracle."""
    import subprocess
    import sys
    import numpy as np
    cfg, W = _model("roomy_heads", seed=9, width=48, vocab=131)
    path = _save(tmp_path, cfg, W)
    reqs = {name: _tokens(cfg, n, 90 + i) for i, (name, n) in enumerate([("a", 70), ("b", 9), ("c", 120), ("d", 33), ("e", 50)])}
    steps = [
        [("a", 0, 40, [39]), ("b", 0, 9, [0, 8])],
        [("a", 40, 1, [0]), ("c", 0, 64, [])],
        [("c", 64, 50, [49]), ("a", 41, 2, [0, 1]), ("d", 0, 17, [16])],
        [("a", 43, 27, [26]), ("d", 17, 1, [0])],                       # b paused since step 0 and ends here
        [("c", 114, 6, [0, 5]), ("d", 18, 15, [14])],
        [("e", 0, 50, [0, 49])],                                        # takes a freed slot and freed pages
    ]
    ends = {3: ["b", "a"], 4: ["c", "d"], 5: ["e"]}
    lines, wanted = [], {}
    for i, st in enumerate(steps):
        ent = [{"id": r, "tokens": reqs[r][lo:lo + n], "want": w} for r, lo, n, w in st]
        lines.append(json.dumps({"step": i, "entries": ent, "end": ends.get(i, [])}))
        wanted[i] = [(r, lo + j) for r, lo, n, w in st for j in w]
    lines.insert(2, json.dumps({"step": "idle", "entries": [], "end": []}))
    out = os.path.join(str(tmp_path), "out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", out,
                            "--max-tokens", "256"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        done = [l.split()[1] for l in r.stdout.splitlines() if l.startswith("done ")]
        assert done == ["0", "1", "idle", "2", "3", "4", "5"]
        full = {name: O.forward(cfg, W, toks) for name, toks in reqs.items()}
        for i, rows in wanted.items():
            got = torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(len(rows), cfg["vocab"]).copy()).double()
            want = torch.stack([full[r][p] for r, p in rows])
            assert _rel(got, want) < tol, (dtype, i)
