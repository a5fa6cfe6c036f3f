"""Vilosun on the step engine against the plain float64 oracle (tests/vilosun_oracle.py): small random models of several
shapes, written to disk as a checkpoint, loaded through the model registry and run through ``HybridSampler.step`` /
``generate`` under different schedules (whole prompts, token by token, portions, mixed batches, reused pages and slots),
and every new kernel alone against the oracle's function for its mechanism."""
import json
import os
import subprocess
import sys

import pytest
import torch

import vilosun_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 2e-4
BF16_TOL = 6e-2


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


def _close(got, want, dtype):
    """Every row within the rounding of the serving mode (bf16 on these tiny widths has a tail: nearly all rows within the
    tolerance, none far outside)."""
    rows = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    if dtype == "fp32":
        return bool(rows.max() < F32_TOL)
    return bool((rows > BF16_TOL).double().mean() <= 0.06 and rows.max() < 3 * BF16_TOL)


def _cuts(total, sizes):
    out, i, k = [], 0, 0
    while i < total:
        n = min(sizes[k % len(sizes)], total - i)
        out.append(n)
        i += n
        k += 1
    return out


SHAPES = {
    # sizes differ from their neighbours: dim != vdim, kv_heads < heads, chunk not a multiple of the page
    "mixed": dict(layers=("attention", "delta", "attention", "delta")),
    # one key/value head, one norm group, one tap, top 1, no pair table, scales of 1, the blend starts at the second attention layer
    "ones": dict(layers=("delta", "attention", "attention", "attention"), groups=1, embed_scale=1.0, logit_scale=1.0, bigram=None,
                 attn=dict(heads=3, kv_heads=1, dim=16, vdim=16, conv=1, size=16, scale=1.0), v_mix=[False, True, True],
                 delta=dict(heads=2, kv_heads=1, dim=8, vdim=24, conv=1), moe=dict(ff=24, experts=3, top=1)),
    # heads == kv_heads everywhere, every expert chosen, wide taps, layers without a feed-forward, three norm groups
    "full": dict(layers=("attention-", "delta", "delta-", "attention"), groups=3,
                 attn=dict(heads=2, kv_heads=2, dim=24, vdim=8, conv=4, size=5), delta=dict(heads=3, kv_heads=3, dim=8, vdim=16, conv=4),
                 moe=dict(ff=8, experts=4, top=4), chunk=[5, 37], v_mix=[True, True]),
    # long chunks (several pages), many experts, a width that is no multiple of 64
    "long_chunk": dict(layers=("attention", "attention"), width=40, attn=dict(heads=4, kv_heads=4, dim=16, vdim=16, size=200),
                       moe=dict(ff=8, experts=17, top=3), chunk=[200, 48], v_mix=[False, False]),
    # sizes of a small real model: grouped key/value heads, three norm groups, four taps, a layer that does not blend
    "medium": dict(vocab=1000, width=384, layers=("delta", "attention", "attention", "delta", "attention"), groups=3, embed_scale=12.0,
                   logit_scale=0.3, bigram=(997, 131, 71), attn=dict(heads=6, kv_heads=2, dim=32, vdim=48, conv=4, size=96, scale=0.2),
                   v_mix=[True, False, True], delta=dict(heads=6, kv_heads=3, dim=32, vdim=48, conv=4), moe=dict(ff=96, experts=8, top=2)),
    # a width that is no multiple of 64, five heads, head sizes off the tensor-core tile, many experts, five norm groups
    "odd": dict(vocab=333, width=200, layers=("attention", "delta", "attention-"), groups=5, embed_scale=2.0, logit_scale=1.5,
                bigram=(50, 3, 1), attn=dict(heads=5, kv_heads=5, dim=24, vdim=40, conv=2, size=33, scale=0.25), v_mix=[True, True],
                delta=dict(heads=4, kv_heads=1, dim=40, vdim=24, conv=3), moe=dict(ff=40, experts=20, top=5)),
}


def _model(name, seed=0, dtype="fp32"):
    cfg = O.make_config(**SHAPES[name])
    W = O.random_weights(cfg, seed=seed)
    return cfg, (_decisive_routers(W) if dtype == "bf16" else W)


def _decisive_routers(W):
    """For bf16 runs: router logits whose order is settled by well-separated biases.  With random routers some token always has
    two experts nearly tied, bf16 rounding of the router's input picks the other one, and that token's logits (and, through the
    recurrent state, later ones) move by far more than rounding -- noise that would hide real faults.  Token-dependent routing
    is checked in float32."""
    out = dict(W)
    g = torch.Generator().manual_seed(11)
    for k in W:
        if k.endswith("mlp.router"):
            out[k] = (W[k].float() * 0.05).to(W[k].dtype)
            out[k + ".b"] = torch.randperm(W[k].shape[0], generator=g).to(W[k].dtype)
    return out


# ---- mechanisms alone: kernels against the oracle's functions -----------------------------------------------------
def _plan(entries, slots, page=16, start=None, pages=None):
    """A hand-made step plan: entries = token counts, sequences start at ``start`` tokens, pages are given or consecutive."""
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    E, T = len(entries), sum(entries)
    start = start or [0] * E
    MB = max((s + n + page - 1) // page for s, n in zip(start, entries))
    cu, te, pos, kv, bt = [0], [], [], [], []
    nxt = 0
    for e, (s, n) in enumerate(zip(start, entries)):
        need = (s + n + page - 1) // page
        pg = pages[e] if pages else list(range(nxt, nxt + need))
        nxt += need
        bt.append(pg + [0] * (MB - len(pg)))
        for j in range(n):
            te.append(e)
            pos.append(s + j)
            kv.append(pg[(s + j) // page] * page + (s + j) % page)
        cu.append(cu[-1] + n)
    flat = [0] * T + cu + te + pos + kv + start + slots + [x for r in bt for x in r]
    return StepPlan(torch.tensor(flat, dtype=torch.int32, device="cuda"), E, T, MB)


def test_hashed_pair_embedding_and_carried_token():
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(0)
    V, W, B = 50, 24, 11
    emb, pair = torch.randn(V, W, generator=g).cuda(), torch.randn(B + 1, W, generator=g).cuda()
    cfg = {"embedding": {"scale": 2.5, "bigram": {"buckets": B, "mul_prev": 40009, "mul_cur": 30011}}}
    toks = torch.randint(0, V, (9,), generator=g).tolist()
    want = O.embed(toks, {"embed": emb.cpu(), "bigram": pair.cpu()}, cfg)
    prev = torch.full((3,), 7, dtype=torch.int32, device="cuda")          # stale tokens of earlier users of the slots
    got = []
    for lo, n in ((0, 1), (1, 2), (3, 5), (8, 1)):                         # the sequence lives in slot 2
        plan = _plan([n], [2], start=[lo])
        plan.tokens.copy_(torch.tensor(toks[lo:lo + n], dtype=torch.int32))
        out = torch.empty(n, W, device="cuda")
        hy.embed_hashed(emb, pair, plan, prev, 2.5, 40009, 30011, B, out)
        got.append(out.double().cpu())
    assert (torch.cat(got) - want).abs().max() < 1e-5
    assert prev.tolist() == [7, 7, toks[-1]]


@pytest.mark.parametrize("groups,W", [(1, 40), (2, 40), (5, 40), (3, 42), (2, 4096), (1, 9216)])
def test_group_norm_residual(groups, W):
    """Parts that fit the vector kernel (a multiple of four columns, up to 8192) and parts that do not."""
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(groups)
    T, eps = 7, 1e-3
    x, o, gate = (torch.randn(T, W, generator=g) for _ in range(3))
    gb, wpost, wpre = (torch.randn(W, generator=g) for _ in range(3))
    y = o.double() * torch.sigmoid(gate.double() + gb.double())
    x2 = x.double() + O.group_rmsnorm(y, wpost, groups, eps)
    h2 = O.group_rmsnorm(x2, wpre, groups, eps)
    xc, h = x.clone().cuda(), torch.empty(T, W, device="cuda")
    wide = torch.zeros(T, W + 8, device="cuda")                           # the gate is a column range of a wider matrix
    wide[:, 8:] = gate.cuda()
    hy.group_norm_residual(xc, o.cuda(), wide[:, 8:], gb.cuda(), wpost.cuda(), wpre.cuda(), groups, eps, h)
    assert (xc.double().cpu() - x2).abs().max() < 1e-5 and (h.double().cpu() - h2).abs().max() < 1e-5
    xc = x.clone().cuda()                                                  # no sublayer result: only the norm
    hy.group_norm_residual(xc, None, None, None, None, wpre.cuda(), groups, eps, h)
    assert (h.double().cpu() - O.group_rmsnorm(x.double(), wpre, groups, eps)).abs().max() < 1e-5


@pytest.mark.parametrize("taps", [1, 2, 5])
def test_biased_convolution_in_portions(taps):
    """The projection's bias is part of the convolved signal and of the carried taps; before the start there are zeros."""
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(taps)
    T, C = 23, 20
    u, b, w = torch.randn(T, C, generator=g), torch.randn(C, generator=g), torch.randn(C, taps, generator=g)
    want = O.causal_conv(u.double() + b.double(), w)
    state = torch.full((2, taps - 1, C), 9.0, device="cuda")              # garbage of an earlier sequence
    got, lo = [], 0
    for n in (1, 1, 2, 9, 3, 7):
        plan = _plan([n], [1], start=[lo])
        out = torch.empty(n, C, device="cuda")
        hy.causal_conv(u[lo:lo + n].cuda(), w.cuda(), None, state, out, plan, in_bias=b.cuda(), act="none")
        got.append(out.double().cpu())
        lo += n
    assert (torch.cat(got) - want).abs().max() < 1e-5


@pytest.mark.parametrize("E,top", [(1, 1), (7, 1), (7, 3), (7, 7), (40, 6)])
def test_router_top_k_and_dense_expert_activations(E, top):
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(E * 10 + top)
    T, ff = 9, 12
    z, zb, gu = torch.randn(T, E, generator=g), torch.randn(E, generator=g), torch.randn(T, E * 2 * ff, generator=g)
    ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, top, device="cuda")
    act = torch.full((T, E * ff), 7.0, device="cuda")
    hy.moe_route(z.cuda(), zb.cuda(), top, gu=gu.cuda(), ff=ff, act=act, ids=ids, wts=wts)
    zz = z.double() + zb.double()
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(zz[t, e]), e))[:top]
        assert ids[t].tolist() == order
        w = torch.softmax(zz[t, order], 0)
        assert (wts[t].double().cpu() - w).abs().max() < 1e-6
        want = torch.zeros(E, ff, dtype=torch.float64)
        for wt, e in zip(w, order):
            gt, up = gu[t, e * 2 * ff:e * 2 * ff + ff].double(), gu[t, e * 2 * ff + ff:(e + 1) * 2 * ff].double()
            want[e] = wt * O.silu(gt) * up
        assert (act[t].double().cpu().view(E, ff) - want).abs().max() < 1e-5


def _attention_case(T, H, G, D, Dv, size, seed, needles=()):
    """Random q / k / v; ``needles``: (query position, key position) pairs whose score is made to stand out, so that seeing or
    not seeing that one key decides the output."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = torch.randn(T, H, D, generator=g), torch.randn(T, G, D, generator=g), torch.randn(T, G, Dv, generator=g)
    for i, j in needles:
        for hh in range(H):
            k[j, hh // (H // G)] = q[i, hh] * 6.0 / q[i, hh].norm()       # one query head per key head wins; the others stay random
        v[j] = v[j] * 8.0
    return q, k, v


def _run_attention(q, k, v, size, scale, temp, slopes, gate, cuts, dtype, impl, pages=None):
    """Keys and values into pages (shuffled page ids), then the kernel over the sequence cut into ``cuts``."""
    from nanorlhf_b200.ops import hybrid as hy
    T, H, D = q.shape
    G, Dv = v.shape[1], v.shape[2]
    td = torch.float32 if dtype == "fp32" else torch.bfloat16
    npages = (T + 15) // 16
    order = pages or [((5 * i + 3) % (npages + 2)) for i in range(npages + 2)][:npages]
    assert len(set(order)) == npages
    kc = torch.zeros(npages + 2, G, 16, D, dtype=td, device="cuda")
    vc = torch.zeros(npages + 2, G, 16, Dv, dtype=td, device="cuda")
    outs, lo = [], 0
    for n in cuts:
        plan = _plan([n], [0], start=[lo], pages=[order[:(lo + n + 15) // 16]])
        vv = v[lo:lo + n].reshape(n, G * Dv).cuda().contiguous()
        hy.kv_write_blend(k[lo:lo + n].reshape(n, G * D).cuda().contiguous(), vv, None, None, kc, vc, plan)
        out = torch.empty(n, H * Dv, dtype=td, device="cuda")
        hy.window_attention(q[lo:lo + n].reshape(n, H * D).cuda().contiguous(), kc, vc, plan, size, scale, 1.0, out, impl=impl,
                            chunked=True, head_scale=None if temp is None else temp.cuda(),
                            head_slope=None if slopes is None else torch.tensor(slopes, device="cuda"),
                            gate=None if gate is None else gate[lo:lo + n].cuda().contiguous())
        outs.append(out.double().cpu())
        lo += n
    return torch.cat(outs).view(T, H, Dv)


ATTN_IMPLS = [("fp32", "tile"), ("fp32", "simple"), ("bf16", "auto"), ("bf16", "mma"), ("bf16", "tile")]


@pytest.mark.parametrize("dtype,impl", ATTN_IMPLS)
@pytest.mark.parametrize("size", [5, 16, 24, 150])
def test_chunk_attention_edges_in_prompts_and_decoding(dtype, impl, size):
    """A loud key just inside the query's chunk (its first position) and one just outside (the last position of the chunk
    before), far keys at the start of a long chunk, chunk edges on and off page borders; prompts, portions and single tokens."""
    T, H, G, D, Dv = 330, 4, 2, 16, 24
    needles = []
    for c in range(size, T - 1, size):
        if len(needles) < 12:
            needles += [(min(c + size - 1, T - 1), c), (c, c - 1), (c + min(2, size - 1), c - 1)]
    q, k, v = _attention_case(T, H, G, D, Dv, size, seed=size, needles=needles)
    temp = torch.rand(H, generator=torch.Generator().manual_seed(1)) + 0.5
    slopes = O.distance_slopes(H)
    gate = torch.randn(T, H, generator=torch.Generator().manual_seed(2))
    want = O.chunk_softmax_attention(q.double(), k.double(), v.double(), size, 0.3, temp.double(), slopes)
    want = want * torch.sigmoid(gate.double()).unsqueeze(-1)
    blind = O.chunk_softmax_attention(q.double(), k.double(), v.double(), size + 1, 0.3, temp.double(), slopes)
    tol = 2e-4 if dtype == "fp32" else 5e-2
    for cuts in ([T], [T - 70] + [1] * 70, _cuts(T, [2, 31, 1, 16, 5, 64, 3])):
        got = _run_attention(q, k, v, size, 0.3, temp, slopes, gate, cuts, dtype, impl)
        err = (got - want).abs().max().item() / want.abs().max().item()
        assert err < tol, (cuts[:3], err)
    # the test is sharp: a mask that is one position off changes the result by far more than the tolerance
    off = blind * torch.sigmoid(gate.double()).unsqueeze(-1)
    assert (off - want).abs().max().item() / want.abs().max().item() > 20 * tol


@pytest.mark.parametrize("dtype,impl", ATTN_IMPLS)
def test_chunk_attention_head_layouts(dtype, impl):
    """Many query heads per key/value head, one each, sizes off the vector widths; without the optional terms too."""
    for (H, G, D, Dv, size) in ((6, 1, 8, 8, 7), (3, 3, 40, 12, 33), (8, 2, 64, 64, 64)):
        T = 100
        if impl == "mma" and (D % 8 or Dv % 8):
            continue                                        # the tensor-core kernel takes head sizes that are multiples of 8
        q, k, v = _attention_case(T, H, G, D, Dv, size, seed=H)
        for temp, slopes in ((None, None), (torch.rand(H) + 0.5, O.distance_slopes(H))):
            want = O.chunk_softmax_attention(q.double(), k.double(), v.double(), size, 0.2, None if temp is None else temp.double(), slopes)
            for cuts in ([T], [60] + [1] * 40):
                got = _run_attention(q, k, v, size, 0.2, temp, slopes, None, cuts, dtype, impl)
                assert (got - want).abs().max().item() / want.abs().max().item() < (2e-4 if dtype == "fp32" else 5e-2)


# ---- each layer type alone, whole prompt --------------------------------------------------------------------------
@pytest.mark.parametrize("layers", [("attention-",), ("delta-",), ("attention",), ("delta",)])
def test_single_layer_types(tmp_path, layers):
    cfg = O.make_config(layers=layers)
    W = O.random_weights(cfg, seed=3)
    toks = _tokens(cfg, 45, 1)
    eng = _engine(tmp_path, cfg, W)
    assert _rel(_run_alone(eng, toks, [len(toks)]), O.forward(cfg, W, toks)) < F32_TOL


def test_layer_stream_matches_after_every_layer(tmp_path):
    """The residual stream after each layer, not only the logits."""
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    import numpy as np
    cfg, W = _model("mixed")
    toks = _tokens(cfg, 20, 2)
    _, want = O.forward(cfg, W, toks, return_layers=True)
    eng = _engine(tmp_path, cfg, W)
    sid = eng.open()
    data, E, T, MB = eng.sched.plan([sid], [len(toks)], 0)
    data[:T] = np.asarray(toks, dtype=np.int32)
    keep = []
    eng._forward_sandwich(StepPlan(torch.from_numpy(data).cuda(), E, T, MB), [], keep)
    assert len(keep) == len(want)
    for got, ref in zip(keep, want):
        assert (got.double().cpu() - ref).abs().max().item() < 1e-4 * ref.abs().max().item()


# ---- schedules -----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", list(SHAPES))
def test_prefill_decode_and_portions_agree_with_oracle(tmp_path, shape, dtype):
    cfg, W = _model(shape, dtype=dtype)
    n = 230 if shape == "long_chunk" else 90
    toks = _tokens(cfg, n, 5)
    want = O.forward(cfg, W, toks)
    eng = _engine(tmp_path, cfg, W, dtype=dtype)
    whole = _run_alone(eng, toks, [n])
    assert _close(whole, want, dtype)
    schedules = {"prefill_then_decode": [n - 40] + [1] * 40, "ragged": _cuts(n, [3, 37, 2, 16, 1, 17, 5]), "pairs": [2] * (n // 2)}
    if dtype == "fp32":
        schedules["by_token"] = [1] * n
    for name, cuts in schedules.items():
        got = _run_alone(eng, toks, cuts)
        assert _close(got, want, dtype), name
        assert _close(got, whole, dtype), name


def test_first_tokens_of_a_sequence(tmp_path):
    """One- and two-token sequences: the spare pair row, zeros before the convolutions' start, an empty recurrent state."""
    cfg, W = _model("mixed")
    eng = _engine(tmp_path, cfg, W)
    for toks in ([5], [5, 5], [0, 96, 3]):
        want = O.forward(cfg, W, toks)
        assert _rel(_run_alone(eng, toks, [len(toks)]), want) < F32_TOL
        assert _rel(_run_alone(eng, toks, [1] * len(toks)), want) < F32_TOL


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_mixed_batches_match_each_request_alone(tmp_path, dtype):
    """Unequal requests share steps (portions beside single tokens, requests that pause); pages and slots are freed and reused."""
    cfg, W = _model("mixed", dtype=dtype)
    eng = _engine(tmp_path, cfg, W, dtype=dtype, pool_tokens=16 * 12, slots=3)
    reqs = {name: _tokens(cfg, n, 10 + i) for i, (name, n) in enumerate([("a", 70), ("b", 23), ("c", 1), ("d", 41), ("e", 64), ("f", 9)])}
    want = {k: O.forward(cfg, W, v) for k, v in reqs.items()}
    got = {k: [] for k in reqs}
    fed = {k: 0 for k in reqs}
    live = {}
    waiting = list(reqs)
    portion = {"a": [16, 3, 1, 1, 30, 2, 1, 16], "b": [2, 1, 20], "c": [1], "d": [40, 1], "e": [5, 1, 1, 57], "f": [3, 3, 3]}
    step = 0
    while waiting or live:
        while waiting and len(live) < 3 and eng.sched.num_free_blocks() * 16 >= len(reqs[waiting[0]]) + 16 * len(live):
            live[waiting.pop(0)] = eng.open()
        entries, names = [], []
        for name in list(live):
            if name == "a" and step % 3 == 2:
                continue                                   # a request may sit out a step
            k = portion[name]
            n = min(k[len(got[name]) % len(k)], len(reqs[name]) - fed[name])
            entries.append((live[name], reqs[name][fed[name]:fed[name] + n], list(range(n))))
            names.append((name, n))
        out = eng.step(entries).double().cpu()
        o = 0
        for name, n in names:
            got[name].append(out[o:o + n])
            o += n
            fed[name] += n
            if fed[name] == len(reqs[name]):
                eng.close(live.pop(name))
        step += 1
    assert eng.sched.num_open() == 0
    for k in reqs:
        assert _close(torch.cat(got[k]), want[k], dtype), k


def test_long_decoding(tmp_path):
    """Hundreds of single-token steps: the recurrent state, the taps and the previous token are carried without drift, and
    chunks keep turning over."""
    cfg, W = _model("full")
    toks = _tokens(cfg, 260, 8)
    eng = _engine(tmp_path, cfg, W)
    assert _rel(_run_alone(eng, toks, [4] + [1] * 256), O.forward(cfg, W, toks)) < F32_TOL


def test_distant_tokens_reach_through_the_recurrent_state(tmp_path):
    """With short chunks only the delta layers carry information further than a chunk: changing an early token must change
    late logits, in the engine as in the oracle, in portions and in decoding."""
    cfg = O.make_config(layers=("attention", "delta"), attn=dict(heads=2, kv_heads=2, dim=8, vdim=8, size=4))
    W = O.random_weights(cfg, seed=4)
    W["l1.mix.dt_bias"] = torch.full_like(W["l1.mix.dt_bias"], -6.0)       # slow decay: a long memory
    a = _tokens(cfg, 120, 3)
    b = list(a)
    b[1] = (b[1] + 1) % cfg["vocab"]
    wa, wb = O.forward(cfg, W, a), O.forward(cfg, W, b)
    assert _rel(wa[-8:], wb[-8:]) > 50 * F32_TOL
    eng = _engine(tmp_path, cfg, W)
    for toks, want in ((a, wa), (b, wb)):
        assert _rel(_run_alone(eng, toks, [100] + [1] * 20)[-8:], want[-8:]) < F32_TOL


def test_blend_uses_the_first_blending_layer_only(tmp_path):
    """Layers without the flag neither provide nor receive values."""
    cfg = O.make_config(layers=("attention", "attention", "delta", "attention", "attention"), v_mix=[False, True, False, True])
    W = O.random_weights(cfg, seed=6)
    specs = [s.mixers[0].v_blend for s in __import__("nanorlhf_b200.models.vilosun", fromlist=["x"]).VilosunConfig.from_dict(cfg).layer_specs()]
    assert specs == [-1, 1, -1, -1, 1]
    toks = _tokens(cfg, 50, 7)
    eng = _engine(tmp_path, cfg, W)
    assert _rel(_run_alone(eng, toks, [30, 2, 17, 1]), O.forward(cfg, W, toks)) < F32_TOL


# ---- generation through the framework's entry point ------------------------------------------------------------------
class _Tok:
    pad_token_id = 0
    eos_token_id = None


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_greedy_generation_through_the_engine_entry_point(tmp_path, dtype):
    from nanorlhf_b200.models.registry import load_model
    from nanorlhf_b200.sampler.engine import generate, release_native_engine
    cfg, W = _model("mixed", dtype=dtype)
    path = _save(tmp_path, cfg, W)
    model = load_model(path, torch_dtype=torch.float32 if dtype == "fp32" else torch.bfloat16, device="cuda")
    prompts = [_tokens(cfg, n, 20 + n) for n in (3, 17, 1, 40, 9)]
    new = 24
    out = generate(1, model, _Tok(), prompts, 0.0, new, top_p=1.0, seed=1, rollout_dtype=dtype, max_num_seqs=3,
                   prefill_token_budget=32).cpu()
    far = 0
    for p, row in zip(prompts, out.tolist()):
        seq = list(p)
        for t in row:
            logits = O.forward(cfg, W, seq)[-1]
            best = int(logits.argmax())
            if dtype == "fp32":
                assert t == best
            elif t != best and float(logits[best] - logits[t]) > 0.05 * float(logits.std()):
                far += 1                                   # bf16: a near tie of two logits may go the other way
            seq.append(t)
    assert far <= 0.05 * len(prompts) * new
    release_native_engine(model)


def test_sampled_generation_is_seeded_and_replays_graphs(tmp_path):
    """Temperature / top-p sampling through the same entry point: rows are reproducible per seed, differ across seeds and
    samples, stay inside the vocabulary; decode steps of a fixed batch replay a CUDA graph."""
    from nanorlhf_b200.models.registry import load_model
    from nanorlhf_b200.sampler.engine import generate, get_native_engine, release_native_engine
    cfg, W = _model("mixed", dtype="bf16")
    model = load_model(_save(tmp_path, cfg, W), torch_dtype=torch.bfloat16, device="cuda")
    prompts = [_tokens(cfg, n, 40 + n) for n in (5, 12)]
    a = generate(2, model, _Tok(), prompts, 1.0, 20, top_p=0.9, seed=7, rollout_dtype="bf16").cpu()
    b = generate(2, model, _Tok(), prompts, 1.0, 20, top_p=0.9, seed=7, rollout_dtype="bf16").cpu()
    c = generate(2, model, _Tok(), prompts, 1.0, 20, top_p=0.9, seed=8, rollout_dtype="bf16").cpu()
    assert a.shape == (4, 20) and torch.equal(a, b) and not torch.equal(a, c)
    assert not torch.equal(a[0], a[1]) and int(a.min()) >= 0 and int(a.max()) < cfg["vocab"]
    assert get_native_engine(model, rollout_dtype="bf16").stats["graph_replays"] > 0
    release_native_engine(model)


def test_trace_runner_replays_a_mixed_trace(tmp_path):
    """bin/trace_run as a subprocess: portions beside single tokens, a pool that forces pages and slots to be reused."""
    import numpy as np
    cfg, W = _model("mixed")
    path = _save(tmp_path, cfg, W)
    reqs = {k: _tokens(cfg, n, 30 + n) for k, n in (("x", 50), ("y", 33), ("z", 2), ("w", 40))}
    steps = [
        {"step": 0, "entries": [{"id": "x", "tokens": reqs["x"][:30], "want": [0, 29]}, {"id": "z", "tokens": reqs["z"], "want": [1]}], "end": ["z"]},
        {"step": 1, "entries": [{"id": "x", "tokens": reqs["x"][30:31], "want": [0]}, {"id": "y", "tokens": reqs["y"][:31], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "y", "tokens": reqs["y"][31:], "want": [0, 1]}, {"id": "x", "tokens": reqs["x"][31:], "want": [18]}], "end": ["x", "y"]},
        {"step": 3, "entries": [{"id": "w", "tokens": reqs["w"], "want": [39]}], "end": ["w"]},
    ]
    outdir = os.path.join(str(tmp_path), "out")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", outdir,
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    full = {k: O.forward(cfg, W, v) for k, v in reqs.items()}
    want = {0: [full["x"][0], full["x"][29], full["z"][1]], 1: [full["x"][30]], 2: [full["y"][31], full["y"][32], full["x"][49]], 3: [full["w"][39]]}
    for i, rows in want.items():
        got = torch.from_numpy(np.fromfile(os.path.join(outdir, f"{i}.f32"), dtype="<f4").reshape(len(rows), cfg["vocab"])).double()
        assert _rel(got, torch.stack(rows)) < F32_TOL


# ---- mixture of experts on the grouped GEMM ---------------------------------------------------------------------------
@pytest.mark.parametrize("T,E,top,W,ff", [(1, 4, 2, 64, 64), (37, 5, 2, 128, 72), (300, 7, 3, 64, 136), (513, 3, 1, 192, 64),
                                          (260, 2, 2, 64, 8), (700, 40, 4, 64, 64), (400, 5, 2, 64, 96), (300, 3, 2, 128, 160)])
def test_grouped_expert_feed_forward(T, E, top, W, ff):
    """Rows sorted by expert through the grouped tensor-core GEMM against a loop over tokens; experts without tokens, experts
    whose rows end inside a tile, more tiles than experts."""
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(T + E)
    h = torch.randn(T, W, generator=g).bfloat16()
    z = torch.randn(T, E, generator=g)
    if E > 3:
        z[:, 1] = -50.0                                     # an expert that nobody chooses
    wgu = (torch.randn(E * 2 * ff, W, generator=g) * W ** -0.5).bfloat16()
    wdn = (torch.randn(E * W, ff, generator=g) * ff ** -0.5).bfloat16()
    ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, top, device="cuda")
    hy.moe_route(z.cuda(), None, top, ids=ids, wts=wts)
    out = torch.empty(T, W, device="cuda")
    hy.moe_grouped_ffn(h.cuda(), ids, wts, wgu.cuda(), wdn.cuda(), E, ff, out)
    if ff % 32 == 0:                                        # the SwiGLU formed in the first GEMM's epilogue gives the same result
        inter = torch.cat([hy.interleave_gate_up(wgu[e * 2 * ff:e * 2 * ff + ff], wgu[e * 2 * ff + ff:(e + 1) * 2 * ff]) for e in range(E)], 0)
        fused = torch.empty(T, W, device="cuda")
        hy.moe_grouped_ffn(h.cuda(), ids, wts, inter.cuda().contiguous(), wdn.cuda(), E, ff, fused, fused_act=True)
        assert (fused - out).abs().max().item() < 2e-3 * max(1.0, out.abs().max().item())
    want = torch.zeros(T, W, dtype=torch.float64)
    hd = h.double()
    for e in range(E):
        rows = (ids.cpu() == e).any(1).nonzero().flatten()
        if not len(rows):
            continue
        gu = hd[rows] @ wgu[e * 2 * ff:(e + 1) * 2 * ff].double().T
        a = (O.silu(gu[:, :ff]) * gu[:, ff:]).bfloat16().double()          # the kernel rounds the activations to bf16 operands
        y = a @ wdn[e * W:(e + 1) * W].double().T
        wt = (wts.cpu().double() * (ids.cpu() == e)).sum(1)[rows]
        want[rows] += wt[:, None] * y
    assert (out.double().cpu() - want).abs().max().item() < 2e-3 * max(1.0, want.abs().max().item())


def test_grouped_and_dense_expert_forms_agree(tmp_path):
    cfg = O.make_config(layers=("delta", "attention"), width=64, moe=dict(ff=24, experts=6, top=2))
    W = _decisive_routers(O.random_weights(cfg, seed=9))
    toks = _tokens(cfg, 150, 4)
    want = O.forward(cfg, W, toks)
    for form in ("grouped", "dense"):
        eng = _engine(tmp_path, cfg, W, dtype="bf16", name=form, moe=form)
        assert any(L.w_gate_up is not None for L in eng.layers) == (form == "grouped")
        assert _close(_run_alone(eng, toks, [100, 2, 47, 1]), want, "bf16"), form
