"""CPU-side checks of the Vilosun family: registry, configuration, tensor inventory, checkpoint round trip, and the oracle's own
invariants (the GPU tests compare the engine with this oracle)."""
import json
import os

import pytest
import torch

import vilosun_oracle as O


def _cfg(**kw):
    return O.make_config(**kw)


def test_registry_resolves_by_architecture():
    from nanorlhf_b200.models.registry import resolve
    from nanorlhf_b200.models.vilosun import VilosunForCausalLM
    cls, kind = resolve({"architecture": "Vilosun"})
    assert cls is VilosunForCausalLM and kind == "hybrid"
    assert resolve({"model_type": "vilosun"})[0] is VilosunForCausalLM


def test_config_reads_every_size_and_constant():
    from nanorlhf_b200.models.vilosun import VilosunConfig
    d = _cfg(layers=("delta", "attention-", "attention"), groups=3, eps=3e-4, embed_scale=1.75, logit_scale=0.125,
             bigram=(101, 3, 5), attn=dict(heads=6, kv_heads=3, dim=10, vdim=14, conv=4, scale=0.77), chunk=[9, 31],
             delta=dict(heads=5, kv_heads=5, dim=6, vdim=4, conv=2), moe=dict(ff=20, experts=9, top=4), v_mix=[False, True])
    c = VilosunConfig.from_dict(d)
    st, specs = c.stream_spec(), c.layer_specs()
    assert (st.kind, st.norm_groups, st.gated_residual, st.embed_scale, st.logit_scale) == ("sandwich", 3, True, 1.75, 0.125)
    assert (st.pair_buckets, st.pair_mul_prev, st.pair_mul_cur, st.positions) == (101, 3, 5, False)
    assert c.norm_eps == 3e-4
    a1, a2, dl = specs[1].mixers[0], specs[2].mixers[0], specs[0].mixers[0]
    assert (a1.kind, a1.heads, a1.kv_heads, a1.dim, a1.vdim, a1.conv, a1.scale, a1.window, a1.mask) == ("conv_attention", 6, 3, 10, 14, 4, 0.77, 9, "chunk")
    assert a2.window == 31 and a1.v_blend == -1 and a2.v_blend == 2
    assert (dl.kind, dl.heads, dl.kv_heads, dl.dim, dl.vdim, dl.conv) == ("gated_delta", 5, 5, 6, 4, 2)
    assert specs[1].ff == 0 and (specs[2].ff, specs[2].ff_kind, specs[2].experts, specs[2].top, specs[2].ff_act) == (20, "moe", 9, 4, "swiglu")
    assert VilosunConfig.from_dict(c.to_dict()).to_dict() == c.to_dict()
    no_pair = VilosunConfig.from_dict(_cfg(bigram=None))
    assert no_pair.stream_spec().pair_buckets == 0 and "bigram" not in no_pair.tensor_shapes()


def test_unknown_layer_or_feed_forward_is_refused():
    from nanorlhf_b200.models.vilosun import VilosunConfig
    d = _cfg()
    d["layers"][0]["type"] = "ssm"
    with pytest.raises(ValueError):
        VilosunConfig.from_dict(d)
    d = _cfg()
    d["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(ValueError):
        VilosunConfig.from_dict(d)


def test_tensor_inventory_matches_the_oracle_weights_and_round_trips(tmp_path):
    from safetensors.torch import save_file
    from nanorlhf_b200.models.registry import load_model
    from nanorlhf_b200.models.vilosun import VilosunConfig
    d = _cfg(layers=("attention", "delta-", "attention", "delta"))
    W = O.random_weights(d, seed=1)
    shapes = VilosunConfig.from_dict(d).tensor_shapes()
    unused = {n for n in W if n not in shapes}
    assert unused == {"l0.mix.vmix"}                         # the providing layer's blend weight is never read
    assert all(tuple(W[n].shape) == tuple(s) for n, s in shapes.items())
    path = os.path.join(str(tmp_path), "m")
    os.makedirs(path)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(d, f)
    save_file({k: v.contiguous() for k, v in W.items()}, os.path.join(path, "model.safetensors"))
    m = load_model(path, torch_dtype=torch.bfloat16)
    assert torch.equal(m.tensor("l2.mix.temp"), W["l2.mix.temp"])
    m.save_pretrained(os.path.join(str(tmp_path), "again"))
    m2 = load_model(os.path.join(str(tmp_path), "again"))
    assert all(torch.equal(m.tensor(n), m2.tensor(n)) for n in m.names)
    bad = dict(W)
    bad["l0.mix.q"] = bad["l0.mix.q"][:-1]
    save_file({k: v.contiguous() for k, v in bad.items()}, os.path.join(path, "model.safetensors"))
    with pytest.raises(ValueError):
        load_model(path)


def test_random_init_from_config():
    from nanorlhf_b200.models.vilosun import VilosunConfig, VilosunForCausalLM
    m = VilosunForCausalLM.from_config(VilosunConfig.from_dict(_cfg()), seed=3)
    assert all(torch.isfinite(m.tensor(n).float()).all() for n in m.names)
    assert m.config.vocab_size == 97 and m.config.hidden_size == 48 and m.config.num_hidden_layers == 2


# ---- the oracle's own invariants -------------------------------------------------------------------------------------
def test_oracle_chunks_do_not_leak():
    """Without a pair table and with one-tap convolutions nothing but attention moves information between positions, and
    attention stays inside a chunk: tokens of an earlier chunk cannot change a later chunk's logits."""
    a = [3, 9, 27, 81, 50, 60, 70, 80, 5]
    b = [4, 8, 16, 32] + a[4:]
    d = _cfg(layers=("attention-", "attention"), attn=dict(size=4, conv=1), bigram=None)
    W = O.random_weights(d, seed=2)
    la, lb = O.forward(d, W, a), O.forward(d, W, b)
    assert (la[4:] - lb[4:]).abs().max() < 1e-9
    d = _cfg(layers=("attention-", "attention"), attn=dict(size=5, conv=1), bigram=None)      # position 4 now shares a chunk with 0..3
    la, lb = O.forward(d, W, a), O.forward(d, W, b)
    assert (la[4] - lb[4]).abs().max() > 1e-6 and (la[5:] - lb[5:]).abs().max() < 1e-9


def test_oracle_prefix_property_and_first_token_row():
    d = _cfg()
    W = O.random_weights(d, seed=5)
    toks = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]
    full = O.forward(d, W, toks)
    assert (O.forward(d, W, toks[:6]) - full[:6]).abs().max() < 1e-9
    x = O.embed(toks, W, d)
    assert torch.allclose(x[0], W["embed"].double()[1] * 3.0 + W["bigram"].double()[61])
    assert torch.allclose(x[1], W["embed"].double()[2] * 3.0 + W["bigram"].double()[(1 * 7 + 2 * 13) % 61])


def test_oracle_router_weights():
    d = _cfg(moe=dict(experts=4, top=4, ff=8))
    W = O.random_weights(d, seed=6)
    h = torch.randn(3, d["width"], dtype=torch.float64)
    full = O.moe(h, W, "l0.mlp.", d["layers"][0]["mlp"])
    z = O.lin(W["l0.mlp.router"], h, W["l0.mlp.router.b"])
    p = torch.softmax(z, -1)                                  # every expert chosen: plain softmax weights
    want = torch.zeros_like(full)
    for e in range(4):
        a = O.silu(O.lin(W[f"l0.mlp.e{e}.gate"], h)) * O.lin(W[f"l0.mlp.e{e}.up"], h)
        want += p[:, e:e + 1] * O.lin(W[f"l0.mlp.e{e}.down"], a)
    assert (full - want).abs().max() < 1e-9


def test_gate_up_rows_interleave_per_32_features():
    """The layout the grouped GEMM's SwiGLU epilogue reads: [32 gate rows | 32 up rows] per block of 32 features."""
    from nanorlhf_b200.ops.hybrid import interleave_gate_up
    gate = torch.arange(64 * 3, dtype=torch.float32).view(64, 3)
    w = interleave_gate_up(gate, -gate)
    assert w.shape == (128, 3)
    assert torch.equal(w[:32], gate[:32]) and torch.equal(w[32:64], -gate[:32])
    assert torch.equal(w[64:96], gate[32:]) and torch.equal(w[96:], -gate[32:])
