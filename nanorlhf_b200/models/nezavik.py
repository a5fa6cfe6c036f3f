"""Nezavik: a decoder whose layers mix sliding-window attention, a state-space scan and gated delta rules.

Every layer reads ONE single-gain RMS norm of the stream and adds ``mixer(h) + ff(h)`` to it (parallel residual); what the
next layer sees is a learned weighted average of the embedding output and of all layer results so far (depth-weighted
average).  Three layer types exist:

``parallel``       sliding-window softmax attention (per-head RMS-normed q / k, no rotary) side by side with a state-space
                   scan (short causal convolution, scalar decay per head, gated part-wise RMS norm); the two results are
                   summed with fixed scales;
``delta``          gated delta rule with one decay per head and a silu output gate;
``channel_delta``  gated delta rule with one decay per head and key channel (low-rank projected) and a low-rank sigmoid gate.

The feed-forward is ``W_down relu(W_up h)^2``; positions are learned vectors added to the token embedding.

This module holds the configuration (read from ``config.json``: every size and constant comes from there or from a
tensor's shape) and the checkpoint tensors under their own names (``l<i>.mix.left.q`` ...).  It describes each layer as a
list of generic mixer specs (``LayerSpec``) that the step engine (sampler/hybrid_sampler.py) executes with the kernels of
``ops/hybrid.py``; there is no per-model forward loop here.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .hybrid_spec import LayerSpec, MixerSpec, StreamSpec, TensorModel
from .registry import register_model


@dataclass
class NezavikConfig:
    vocab: int = 256
    width: int = 128
    max_positions: int = 1024
    norm_eps: float = 1e-6
    layers: List[dict] = field(default_factory=list)        # the checkpoint's own layer descriptions
    model_type: str = "nezavik"
    architecture: str = "Nezavik"
    pad_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "NezavikConfig":
        for i, layer in enumerate(d["layers"]):
            if layer["type"] not in ("parallel", "delta", "channel_delta"):
                raise ValueError(f"layer {i}: unknown layer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), max_positions=int(d["max_positions"]),
                   norm_eps=float(d["norm"]["eps"]), layers=list(d["layers"]),
                   pad_token_id=d.get("pad_token_id"), eos_token_id=d.get("eos_token_id"))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "layers": self.layers, "max_positions": self.max_positions,
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        for k in ("pad_token_id", "eos_token_id"):
            if getattr(self, k) is not None:
                out[k] = getattr(self, k)
        return out

    @classmethod
    def from_pretrained(cls, path: str) -> "NezavikConfig":
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

    def layer_specs(self) -> List[LayerSpec]:
        specs = []
        for i, layer in enumerate(self.layers):
            m, p = layer["mixer"], f"l{i}.mix."
            if layer["type"] == "parallel":
                a, r = m["left"], m["right"]
                mixers = [
                    MixerSpec("window_attention", p + "left.", float(m["left_scale"]), heads=a["heads"], kv_heads=a["kv_heads"],
                              dim=a["dim"], vdim=a["vdim"], window=int(a["mask"]["size"]), scale=float(a["scale"])),
                    MixerSpec("ssd", p + "right.", float(m["right_scale"]), heads=r["heads"], kv_heads=r["groups"], dim=r["state"],
                              vdim=r["vdim"], conv=r["conv"], norm_groups=r["norm_groups"]),
                ]
            else:
                mixers = [MixerSpec("gated_delta", p, 1.0, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
                                    conv=m["conv"], per_channel=layer["type"] == "channel_delta")]
            mlp = layer.get("mlp")
            specs.append(LayerSpec(i, mixers, ff=int(mlp["ff"]) if mlp is not None else 0))
        return specs

    def stream_spec(self) -> StreamSpec:
        return StreamSpec(kind="depth_weighted", positions=True)

    def tensor_shapes(self, rank: int = 16) -> Dict[str, tuple]:
        """Name -> shape of every checkpoint tensor (``rank``: width of the low-rank decay / gate projections, which a
        checkpoint fixes by the shape of ``a1``)."""
        W, out = self.width, {"embed": (self.vocab, self.width), "pos": (self.max_positions, self.width)}
        for spec in self.layer_specs():
            p = f"l{spec.index}."
            out[p + "norm1"] = ()
            for m in spec.mixers:
                q = m.prefix
                if m.kind == "window_attention":
                    out.update({q + "q": (m.heads * m.dim, W), q + "k": (m.kv_heads * m.dim, W), q + "v": (m.kv_heads * m.vdim, W),
                                q + "q.norm": (m.dim,), q + "k.norm": (m.dim,), q + "o": (W, m.heads * m.vdim)})
                elif m.kind == "ssd":
                    inner, ch = m.heads * m.vdim, m.heads * m.vdim + 2 * m.kv_heads * m.dim
                    out.update({q + "in": (inner + ch + m.heads, W), q + "conv": (ch, m.conv), q + "conv.b": (ch,),
                                q + "dt_bias": (m.heads,), q + "A_log": (m.heads,), q + "D": (m.heads,), q + "norm": (inner,),
                                q + "o": (W, inner)})
                else:
                    nk, nv = m.kv_heads * m.dim, m.heads * m.vdim
                    out.update({q + "q": (nk, W), q + "q.conv": (nk, m.conv), q + "k": (nk, W), q + "k.conv": (nk, m.conv),
                                q + "v": (nv, W), q + "v.conv": (nv, m.conv), q + "b": (m.heads, W), q + "A_log": (m.heads,),
                                q + "norm": (m.vdim,), q + "o": (W, nv)})
                    if m.per_channel:
                        out.update({q + "a1": (rank, W), q + "a2": (m.heads * m.dim, rank), q + "dt_bias": (m.heads * m.dim,),
                                    q + "g1": (rank, W), q + "g2": (nv, rank)})
                    else:
                        out.update({q + "a": (m.heads, W), q + "dt_bias": (m.heads,), q + "g": (nv, W)})
            if spec.ff:
                out.update({p + "mlp.up": (spec.ff, W), p + "mlp.down": (W, spec.ff)})
            out[p + "dwa"] = (spec.index + 2,)
        out["final.norm"] = ()
        out["head"] = (self.vocab, W)
        return out


@register_model("Nezavik", sampler="hybrid")
class NezavikForCausalLM(TensorModel):
    """Nezavik checkpoint tensors under their own names; executed by ``sampler.hybrid_sampler.HybridSampler``."""
    config_class = NezavikConfig

    @staticmethod
    def free_shape(name: str) -> bool:                   # only the low-rank width is free
        return name.endswith((".a1", ".g1", ".a2", ".g2"))

    @classmethod
    def from_config(cls, cfg: NezavikConfig, torch_dtype=torch.bfloat16, device="cpu", seed: Optional[int] = None, rank: int = 16):
        """Random weights (benchmarks, smoke tests): projections ~ N(0, 1/fan_in), decays and gains in a stable range."""
        return super().from_config(cfg, torch_dtype=torch_dtype, device=device, seed=seed, rank=rank)

    @staticmethod
    def init_value(n: str, t: torch.Tensor, g: torch.Generator) -> torch.Tensor:
        leaf = n.rsplit(".", 1)[-1]
        if t.dim() == 2 and leaf != "conv":
            v = torch.randn(t.shape, generator=g) / (t.shape[1] ** 0.5)
            if leaf in ("embed", "pos"):
                v = torch.randn(t.shape, generator=g) * (1.0 if leaf == "embed" else 0.3)
        elif leaf == "conv":
            v = torch.randn(t.shape, generator=g) / (t.shape[1] ** 0.5)
        elif leaf == "dwa":
            v = torch.rand(t.shape, generator=g) + 0.2
            v = v / v.sum()
        elif leaf == "A_log":
            v = torch.rand(t.shape, generator=g) * 2.0 - 1.5
        elif leaf == "dt_bias":
            v = torch.rand(t.shape, generator=g) * 2.5 - 3.0
        elif leaf == "b" and t.dim() == 1:
            v = torch.rand(t.shape, generator=g) * 0.2 - 0.1
        else:                                     # gains: norm1, q.norm, k.norm, norm, D, final.norm
            v = torch.rand(t.shape, generator=g) * 0.5 + 0.75
        return v
