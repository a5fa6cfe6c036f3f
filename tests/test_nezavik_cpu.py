"""CPU-side pieces of the Nezavik integration: model registry, configuration and checkpoint I/O, the C++ step scheduler
(sequences, KV pages, state slots, step plans, generation policy), and the oracle's own consistency."""
import json
import os

import numpy as np
import pytest
import torch

import nezavik_oracle as O


def _save(tmp_path, cfg, W):
    from safetensors.torch import save_file
    d = str(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in W.items()}, os.path.join(d, "model.safetensors"))
    return d


def test_registry_picks_class_and_engine_by_config(tmp_path):
    from nanorlhf_b200.models.registry import load_model, resolve, sampler_kind
    cls, kind = resolve({"architectures": ["Qwen2ForCausalLM"]})
    assert cls.__name__ == "Qwen2ForCausalLM" and kind == "native"
    cls, kind = resolve({"architecture": "Nezavik"})
    assert cls.__name__ == "NezavikForCausalLM" and kind == "hybrid"
    with pytest.raises(ValueError):
        resolve({"architecture": "Unknown"})
    cfg = O.make_config(layers=("parallel", "channel_delta", "delta"))
    W = O.make_weights(cfg, rank=5)
    model = load_model(_save(tmp_path, cfg, W), torch_dtype=torch.bfloat16, device="cpu")
    assert sampler_kind(model) == "hybrid"
    assert model.tensor("l1.mix.a1").shape == (5, cfg["width"])             # the low-rank width comes from the tensor
    out = os.path.join(str(tmp_path), "again")
    model.save_pretrained(out)
    again = load_model(out, torch_dtype=torch.bfloat16, device="cpu")
    for n in model.names:
        assert torch.equal(model.tensor(n), again.tensor(n)), n


def test_config_reads_every_size_and_rejects_misfits(tmp_path):
    from nanorlhf_b200.models.nezavik import NezavikConfig, NezavikForCausalLM
    cfg = O.make_config(layers=("delta", "parallel"), seed_sizes=dict(ff=0))
    c = NezavikConfig.from_dict(cfg)
    specs = c.layer_specs()
    assert [m.kind for s in specs for m in s.mixers] == ["gated_delta", "window_attention", "ssd"]
    assert specs[0].ff == 0 and specs[1].mixers[0].window == cfg["layers"][1]["mixer"]["left"]["mask"]["size"]
    assert specs[1].mixers[1].out_scale == cfg["layers"][1]["mixer"]["right_scale"]
    W = O.make_weights(cfg)
    assert set(c.tensor_shapes()) == set(W)
    assert all(tuple(W[k].shape) == tuple(v) for k, v in c.tensor_shapes().items())
    W["l0.mix.q"] = W["l0.mix.q"][:-1]
    with pytest.raises(ValueError):
        NezavikForCausalLM.from_pretrained(_save(tmp_path, cfg, W))
    with pytest.raises(ValueError):
        NezavikConfig.from_dict(dict(cfg, layers=[dict(cfg["layers"][0], type="other")]))


def test_random_init_model_has_every_tensor():
    from nanorlhf_b200.models.nezavik import NezavikConfig, NezavikForCausalLM
    cfg = NezavikConfig.from_dict(O.make_config(layers=("channel_delta", "parallel")))
    m = NezavikForCausalLM.from_config(cfg, torch.float32, "cpu", seed=1, rank=4)
    assert set(m.names) == set(cfg.tensor_shapes(4))
    assert all(torch.isfinite(m.tensor(n)).all() for n in m.names)
    assert abs(float(m.tensor("l1.dwa").sum()) - 1.0) < 1e-5


# ---- step scheduler ------------------------------------------------------------------------------------------------
def _plan(s, sids, counts):
    data, E, T, MB = s.plan(sids, counts)
    o = T
    cu = data[o:o + E + 1]; o += E + 1
    tok_entry = data[o:o + T]; o += T
    pos = data[o:o + T]; o += T
    kv = data[o:o + T]; o += T
    start = data[o:o + E]; o += E
    slot = data[o:o + E]; o += E
    bt = data[o:o + E * MB].reshape(E, MB)
    assert o + E * MB == len(data)
    return dict(cu=cu, tok_entry=tok_entry, pos=pos, kv=kv, start=start, slot=slot, bt=bt, T=T)


def test_step_scheduler_plans_pages_and_slots():
    from nanorlhf_b200 import _C
    s = _C.StepScheduler(6, 16, 2)
    a, b = s.open(), s.open()
    assert s.num_free_slots() == 0 and {s.slot_of(a), s.slot_of(b)} == {0, 1}
    with pytest.raises(RuntimeError):
        s.open()
    p = _plan(s, [a, b], [20, 3])
    assert p["T"] == 23 and list(p["cu"]) == [0, 20, 23] and list(p["start"]) == [0, 0]
    assert list(p["pos"][:20]) == list(range(20)) and list(p["pos"][20:]) == [0, 1, 2]
    assert list(p["tok_entry"]) == [0] * 20 + [1] * 3
    ta, tb = s.block_table(a), s.block_table(b)
    assert len(ta) == 2 and len(tb) == 1 and len(set(ta + tb)) == 3
    assert [int(x) for x in p["kv"][:20]] == [ta[i // 16] * 16 + i % 16 for i in range(20)]
    assert list(p["bt"][0]) == ta and p["bt"][1][0] == tb[0]
    p = _plan(s, [b], [14])                                    # crosses into a second page in the middle of a portion
    assert list(p["start"]) == [3] and list(p["pos"]) == list(range(3, 17)) and len(s.block_table(b)) == 2
    assert s.seq_len(b) == 17 and s.num_free_blocks() == 2
    with pytest.raises(RuntimeError):
        s.plan([a], [16 * 3])                                  # more pages than are free: nothing is taken
    assert s.num_free_blocks() == 2 and s.seq_len(a) == 20
    with pytest.raises(ValueError):
        s.plan([a, a], [1, 1])
    slot_b, pages_b = s.slot_of(b), set(s.block_table(b))
    s.close(b)
    assert s.num_free_blocks() == 4 and s.num_free_slots() == 1
    c = s.open()
    assert s.slot_of(c) == slot_b                              # the slot is handed out again
    _plan(s, [c], [40])
    assert set(s.block_table(c)) & pages_b                     # and so are the pages
    s.close(a), s.close(c)
    assert s.num_free_blocks() == 6 and s.num_free_slots() == 2 and s.num_open() == 0
    with pytest.raises(ValueError):
        s.seq_len(a)                                           # a closed sequence is gone


def test_step_scheduler_generation_policy():
    from nanorlhf_b200 import _C
    s = _C.StepScheduler(8, 16, 2)
    r = [s.submit(40, 8), s.submit(5, 8), s.submit(20, 8)]      # 3 + 1 + 2 pages are set aside on admission
    ids, offs, cnts = s.schedule(32)
    assert ids == [r[0]] and offs == [0] and cnts == [32] and s.num_waiting() == 1      # two slots: the third waits
    s.plan([s.seq_of(r[0])], [32]); s.fed(r[0], 32)
    ids, offs, cnts = s.schedule(32)
    assert ids == [r[0], r[1]] and offs == [32, 0] and cnts == [8, 5]
    s.plan([s.seq_of(i) for i in ids], cnts)
    for i, c in zip(ids, cnts):
        s.fed(i, c)
    assert s.schedule(32) == ([], [], [])                       # nothing pending until tokens are pushed
    s.push_token(r[0]); s.push_token(r[1])
    ids, offs, cnts = s.schedule(32)
    assert sorted(ids) == [r[0], r[1]] and cnts == [1, 1]
    s.finish(r[1])
    ids, offs, cnts = s.schedule(4)                             # decode token first, then a portion of the admitted prompt
    assert s.num_waiting() == 0 and ids[0] == r[0] and ids[-1] == r[2] and cnts == [1, 3]
    s.finish(r[0]); s.finish(r[2])
    assert s.num_running() == 0 and s.num_free_blocks() == 8 and s.num_free_slots() == 2


def test_reserved_pages_are_not_taken_by_others():
    from nanorlhf_b200 import _C
    s = _C.StepScheduler(4, 16, 3)
    a = s.open(48)                                              # three pages set aside
    b = s.open()
    s.plan([b], [16])
    with pytest.raises(RuntimeError):
        s.plan([b], [1])                                        # would eat a page that belongs to a's reservation
    s.plan([a], [48])
    assert s.num_free_blocks() == 0
    with pytest.raises(RuntimeError):
        s.open(1)


# ---- the oracle agrees with itself --------------------------------------------------------------------------------
def test_oracle_is_causal_and_windowed():
    cfg = O.make_config(layers=("parallel", "delta", "channel_delta"), seed_sizes=dict(window=4))
    W = O.make_weights(cfg, seed=2)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg["vocab"], (24,), generator=g).tolist()
    full = O.forward(cfg, W, toks)
    assert torch.allclose(O.forward(cfg, W, toks[:10]), full[:10], atol=1e-9)       # no look-ahead
    h = torch.randn(12, cfg["width"], dtype=torch.float64, generator=g)
    m = cfg["layers"][0]["mixer"]["left"]
    a = O.window_attention(h, W, "l0.mix.left.", m, 1e-5)
    h2 = h.clone()
    h2[2] += 1.0                                                                  # position 2 is seen by 2..5 only
    b = O.window_attention(h2, W, "l0.mix.left.", m, 1e-5)
    changed = ((a - b).abs().max(-1).values > 1e-9).nonzero().flatten().tolist()
    assert changed == [2, 3, 4, 5]
