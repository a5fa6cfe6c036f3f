"""Vilosun: a decoder whose layers alternate chunked softmax attention and gated delta rules, each followed by a
mixture-of-experts feed-forward, on a sandwich-normed stream with gated residuals.

* Embedding: ``x = embed[token] * scale + bigram[(prev * mul_prev + token * mul_cur) mod buckets]``; the first token of a
  sequence takes the table's last row.  The previous token is part of a sequence's state.
* Layer: ``x += norm1b(sigmoid(rg1 h + b) * mixer(h))`` with ``h = norm1(x)``, then the same with norm2 / rg2 / norm2b around
  the feed-forward.  Norms are RMS norms over ``norm.groups`` equal consecutive parts of the vector, with a weight per column.
* ``attention`` mixer: biased q / k / v projections, a short causal convolution (no activation) on each, no rotation; the
  score ``q.k * scale * temp[h] - 2^(-8 (h + 1) / H) * (i - j)`` over the keys of the query's own chunk of ``mask.size``
  positions (chunks counted from position 0); values of every ``v_mix`` layer but the first are blended with the first such
  layer's values of the same token (``(1 - vmix) v + vmix v_first``, this is what the cache holds); a sigmoid gate per head on
  the mixer's input; output projection.
* ``delta`` mixer: gated delta rule with one decay per head (convolution + silu on q / k / v, unit q / k, beta, decay
  ``exp(-exp(A_log) softplus(a + dt_bias))``), per-head RMS norm with a shared weight, silu output gate.
* Feed-forward: ``experts`` SwiGLU experts, the ``top`` largest router logits chosen, weights = softmax over the chosen logits.
* Output: the model's norm (``final.norm``), ``logits = head x * logit_scale``.

This module holds the configuration (every size and constant is read from ``config.json`` or a tensor's shape) and the
checkpoint tensors under their own names; it describes the layers as generic specs (models/hybrid_spec.py) that the step
engine (sampler/hybrid_sampler.py) executes.  There is no forward loop here.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .hybrid_spec import LayerSpec, MixerSpec, StreamSpec, TensorModel
from .registry import register_model

DISTANCE_SLOPE_EXP = 8.0         # head h of H loses 2^(-8 (h + 1) / H) of score per position of distance


@dataclass
class VilosunConfig:
    vocab: int = 256
    width: int = 128
    norm_eps: float = 1e-6
    norm_groups: int = 1
    embed_scale: float = 1.0
    bigram: Optional[dict] = None                            # {"buckets", "mul_prev", "mul_cur"} or None
    logit_scale: float = 1.0
    layers: List[dict] = field(default_factory=list)         # the checkpoint's own layer descriptions
    model_type: str = "vilosun"
    architecture: str = "Vilosun"
    pad_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    max_positions: int = 1 << 30                             # no learned positions: nothing bounds a sequence's length

    @classmethod
    def from_dict(cls, d: dict) -> "VilosunConfig":
        for i, layer in enumerate(d["layers"]):
            if layer["type"] not in ("attention", "delta"):
                raise ValueError(f"layer {i}: unknown layer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        emb = d.get("embedding", {})
        if int(d["width"]) % int(d["norm"].get("groups", 1)):
            raise ValueError("width is not a multiple of norm.groups")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                   norm_groups=int(d["norm"].get("groups", 1)), embed_scale=float(emb.get("scale", 1.0)),
                   bigram=dict(emb["bigram"]) if emb.get("bigram") else None, logit_scale=float(d.get("logit_scale", 1.0)),
                   layers=list(d["layers"]), pad_token_id=d.get("pad_token_id"), eos_token_id=d.get("eos_token_id"))

    def to_dict(self) -> dict:
        emb = {"scale": self.embed_scale}
        if self.bigram:
            emb["bigram"] = self.bigram
        out = {"architecture": self.architecture, "embedding": emb, "layers": self.layers, "logit_scale": self.logit_scale,
               "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "vocab": self.vocab, "width": self.width}
        for k in ("pad_token_id", "eos_token_id"):
            if getattr(self, k) is not None:
                out[k] = getattr(self, k)
        return out

    @classmethod
    def from_pretrained(cls, path: str) -> "VilosunConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_dict(json.load(f))

    # ---- names the engines share with the other model families ----
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def stream_spec(self) -> StreamSpec:
        b = self.bigram or {}
        return StreamSpec(kind="sandwich", norm_groups=self.norm_groups, gated_residual=True, embed_scale=self.embed_scale,
                          positions=False, pair_buckets=int(b.get("buckets", 0)), pair_mul_prev=int(b.get("mul_prev", 0)),
                          pair_mul_cur=int(b.get("mul_cur", 0)), logit_scale=self.logit_scale)

    def layer_specs(self) -> List[LayerSpec]:
        specs = []
        first_blend = -1
        for i, layer in enumerate(self.layers):
            m, p = layer["mixer"], f"l{i}.mix."
            if layer["type"] == "attention":
                blend = -1
                if m.get("v_mix"):
                    if first_blend < 0:
                        first_blend = i
                    blend = first_blend
                mixer = MixerSpec("conv_attention", p, 1.0, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]),
                                  vdim=int(m["vdim"]), window=int(m["mask"]["size"]), mask="chunk", scale=float(m["scale"]),
                                  conv=int(m["conv"]), slope_exp=DISTANCE_SLOPE_EXP, head_temp=True, head_gate=True, v_blend=blend)
            else:
                mixer = MixerSpec("gated_delta", p, 1.0, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]),
                                  vdim=int(m["vdim"]), conv=int(m["conv"]))
            mlp = layer.get("mlp")
            if mlp is None:
                specs.append(LayerSpec(i, [mixer]))
            else:
                specs.append(LayerSpec(i, [mixer], ff=int(mlp["expert"]["ff"]), ff_act="swiglu", ff_kind="moe",
                                       experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"])))
        return specs

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Name -> shape of every checkpoint tensor."""
        W = self.width
        out: Dict[str, tuple] = {"embed": (self.vocab, W)}
        if self.bigram:
            out["bigram"] = (int(self.bigram["buckets"]) + 1, W)
        for spec in self.layer_specs():
            p = f"l{spec.index}."
            for n in ("norm1", "norm1b"):
                out[p + n] = (W,)
            out[p + "rg1"], out[p + "rg1.b"] = (W, W), (W,)
            m = spec.mixers[0]
            q = m.prefix
            if m.kind == "conv_attention":
                for n, rows in (("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim)):
                    out.update({q + n: (rows, W), q + n + ".b": (rows,), q + n + ".conv": (rows, m.conv)})
                if m.v_blend >= 0 and m.v_blend != spec.index:        # the blend weight exists only where values are blended
                    out[q + "vmix"] = ()
                out.update({q + "temp": (m.heads,), q + "g": (m.heads, W), q + "o": (W, m.heads * m.vdim)})
            else:
                nk, nv = m.kv_heads * m.dim, m.heads * m.vdim
                out.update({q + "q": (nk, W), q + "q.conv": (nk, m.conv), q + "k": (nk, W), q + "k.conv": (nk, m.conv),
                            q + "v": (nv, W), q + "v.conv": (nv, m.conv), q + "b": (m.heads, W), q + "A_log": (m.heads,),
                            q + "norm": (m.vdim,), q + "a": (m.heads, W), q + "dt_bias": (m.heads,), q + "g": (nv, W), q + "o": (W, nv)})
            if spec.ff:
                for n in ("norm2", "norm2b"):
                    out[p + n] = (W,)
                out[p + "rg2"], out[p + "rg2.b"] = (W, W), (W,)
                for e in range(spec.experts):
                    out.update({f"{p}mlp.e{e}.gate": (spec.ff, W), f"{p}mlp.e{e}.up": (spec.ff, W), f"{p}mlp.e{e}.down": (W, spec.ff)})
                out[p + "mlp.router"], out[p + "mlp.router.b"] = (spec.experts, W), (spec.experts,)
        out["final.norm"] = (W,)
        out["head"] = (self.vocab, W)
        return out


@register_model("Vilosun", "vilosun", sampler="hybrid")
class VilosunForCausalLM(TensorModel):
    """Vilosun checkpoint tensors under their own names; executed by ``sampler.hybrid_sampler.HybridSampler``."""
    config_class = VilosunConfig

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype=torch.bfloat16, device="cpu", **kw):
        cfg = VilosunConfig.from_pretrained(path)
        # a checkpoint may carry norm / gate tensors of a feed-forward that a layer does not have: they are not used
        from .hf_io import load_state_dict
        sd = load_state_dict(os.path.join(path, "model.safetensors"))
        want = cfg.tensor_shapes()
        missing = [n for n in want if n not in sd]
        if missing:
            raise ValueError(f"checkpoint does not fit its config: missing {missing[:4]}")
        for n, shp in want.items():
            if tuple(sd[n].shape) != tuple(shp):
                raise ValueError(f"tensor {n}: shape {tuple(sd[n].shape)} does not fit the config ({tuple(shp)})")
        model = cls(cfg, want, dtype=torch_dtype, device=device)
        with torch.no_grad():
            for n in model.names:
                model.tensor(n).copy_(sd[n].to(torch_dtype))
        return model

    @staticmethod
    def init_value(n: str, t: torch.Tensor, g: torch.Generator) -> torch.Tensor:
        """Random weights (benchmarks, smoke tests): projections ~ N(0, 1/fan_in), decays and gains in a stable range."""
        leaf = n.rsplit(".", 1)[-1]
        if leaf == "conv":
            return torch.randn(t.shape, generator=g) / (t.shape[1] ** 0.5)
        if t.dim() == 2:
            if leaf in ("embed", "bigram"):
                return torch.randn(t.shape, generator=g) * 0.5
            return torch.randn(t.shape, generator=g) / (t.shape[1] ** 0.5)
        if leaf == "A_log":
            return torch.rand(t.shape, generator=g) * 2.0 - 1.5
        if leaf == "dt_bias":
            return torch.rand(t.shape, generator=g) * 2.5 - 3.0
        if leaf == "b":                                   # biases of projections, gates and routers
            return torch.rand(t.shape, generator=g) * 0.4 - 0.2
        if leaf == "vmix":
            return torch.rand(t.shape, generator=g) * 0.6 + 0.2
        if leaf == "temp":
            return torch.rand(t.shape, generator=g) + 0.5
        return torch.rand(t.shape, generator=g) * 0.5 + 0.75     # gains: norm1, norm1b, norm2, norm2b, norm, final.norm
