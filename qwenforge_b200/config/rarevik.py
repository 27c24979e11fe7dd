"""Typed configuration of the Rarevik decoder: layers listed one by one, each ONE Dynamic-Tanh norm whose output both
sublayers read (a parallel layer), a token shift in front of the mixer, a mixer that is one of two kinds of windowed
attention, and a dense or routed feed-forward (or none); a run of layers may repeat with the same weights, and the
embedding's output is mixed into the stream again at the start of every pass. The logits come from the embedding table.

config.json (every size and every constant that differs between models of the design is read from it):
  architecture      "Rarevik"
  vocab, width
  norm.eps          eps of the RMS norms of q and k (the Dynamic Tanh has none)
  loop              optional {start, stop, times}: layers start .. stop-1 run `times` times in a row, each pass with a cache
                    and state of its own; before the first layer of every pass x <- loop.in [x ; embedding output]
  layers[i].type    "attention":   heads, kv_heads, dim, vdim, scale, conv (taps of the short convolution on q, k, v),
                                   rot.{dims, base}, mask.{size, pool}; RMS norm of q and k before the rotation (halves
                                   paired), pooled blocks before the window, a learned sink per head
                    "attention_2": heads, kv_heads, dim, vdim, scale, rot.{dims, base, scaling{factor, low, high, original}},
                                   mask.size; neighbours paired in the rotation, frequencies rescaled by wavelength, a plain
                                   softmax over the window, a sigmoid gate per head on the output
  layers[i].mlp     null | {kind: "dense", ff} | {kind: "moe", router{experts, top}, expert{ff, limit}, shared{ff, limit} (optional)}
What the design fixes stands here as constants: the exact GELU of the dense feed-forward, the slope 1.702 of the experts'
gate, the softmax over the chosen logits, the sigmoid gate of the shared expert, the tied output table.
A sequence has no longest length: nothing in the design depends on one.

Tensor names: embed, loop.in, final.norm(.b, .alpha); per layer l<i>.norm1(.b, .alpha), l<i>.shift,
l<i>.mix.{q, k, v, o}, attention: l<i>.mix.{q.conv, k.conv, v.conv, q.norm, k.norm, sink}, attention_2: l<i>.mix.g;
dense: l<i>.mlp.{up, down}; moe: l<i>.mlp.router(.b), l<i>.mlp.e<j>.{gate, up, down}, l<i>.mlp.shared.{gate, up, down, sg}.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .registry import ModelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

DENSE_ACTIVATION = "gelu"       # the exact form, through erf
EXPERT_GATE_SLOPE = 1.702       # g * sigmoid(1.702 g) * (u + 1)
NO_LENGTH_LIMIT = 1 << 30       # what the runtime is told where it asks for a longest sequence


def _need(data: Mapping[str, Any], key: str, where: str = "config.json"):
    if not isinstance(data, Mapping) or key not in data or data[key] is None:
        raise ValueError(f"{where}: required key {key!r} is missing")
    return data[key]


def _positive(data, keys, where):
    for key in keys:
        if not float(_need(data, key, where)) > 0:
            raise ValueError(f"{where}: {key} must be positive")


@dataclass(frozen=True)
class RarevikConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    layers: tuple                      # the config's own layer entries (plain dicts), validated
    loop: Optional[tuple] = None       # (start, stop, times)
    torch_dtype: str = "bfloat16"

    architecture = "Rarevik"
    model_type = "rarevik"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RarevikConfig":
        layers = _need(data, "layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        loop = data.get("loop")
        if loop is not None:
            loop = tuple(int(_need(loop, key, "config.json loop")) for key in ("start", "stop", "times"))
        config = cls(vocab=int(_need(data, "vocab")), width=int(_need(data, "width")),
                     eps=float(_need(_need(data, "norm"), "eps", "config.json norm")),
                     layers=tuple(copy.deepcopy(dict(layer)) for layer in layers), loop=loop,
                     torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))))
        config.validate()
        return config

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.eps <= 0:
            raise ValueError("config.json: vocab, width and norm.eps must be positive")
        if self.loop is not None:
            start, stop, times = self.loop
            if not 0 <= start < stop <= len(self.layers) or times < 0:
                raise ValueError(f"config.json loop: 0 <= start < stop <= {len(self.layers)} layers and times >= 0 are required")
        for i, layer in enumerate(self.layers):
            where = f"config.json layers[{i}]"
            kind, mixer = _need(layer, "type", where), _need(layer, "mixer", where)
            where += ".mixer"
            if kind not in ("attention", "attention_2"):
                raise ValueError(f"config.json layers[{i}]: mixer type {kind!r} is not supported ('attention', 'attention_2')")
            _positive(mixer, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
            if int(mixer["heads"]) % int(mixer["kv_heads"]):
                raise ValueError(f"{where}: kv_heads must divide heads")
            rot = _need(mixer, "rot", where)
            if int(_need(rot, "dims", where + ".rot")) % 2 or not 0 <= int(rot["dims"]) <= int(mixer["dim"]):
                raise ValueError(f"{where}.rot: dims must be even and at most dim")
            if int(rot["dims"]):
                _positive(rot, ("base",), where + ".rot")
            _positive(_need(mixer, "mask", where), ("size",), where + ".mask")
            if kind == "attention":
                _positive(mixer, ("conv",), where)
                _positive(mixer["mask"], ("pool",), where + ".mask")
            elif rot.get("scaling"):
                _positive(rot["scaling"], ("factor", "low", "high", "original"), where + ".rot.scaling")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            where = f"config.json layers[{i}].mlp"
            if _need(mlp, "kind", where) == "dense":
                _positive(mlp, ("ff",), where)
            elif mlp["kind"] == "moe":
                router = _need(mlp, "router", where)
                experts, top = int(_need(router, "experts", where + ".router")), int(_need(router, "top", where + ".router"))
                _positive(_need(mlp, "expert", where), ("ff", "limit"), where + ".expert")
                if not 1 <= top <= experts:
                    raise ValueError(f"{where}: 1 <= router.top <= router.experts is required")
                if mlp.get("shared"):
                    _positive(mlp["shared"], ("ff", "limit"), where + ".shared")
            else:
                raise ValueError(f"{where}: kind {mlp['kind']!r} is not supported ('dense', 'moe' or null)")

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [copy.deepcopy(layer) for layer in self.layers], "torch_dtype": self.torch_dtype}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return out

    def _dyt(self, name: str) -> PartSpec:
        return PartSpec("dynamic_tanh", {"width": self.width}, {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})

    def _mixer_spec(self, kind: str, m: Mapping[str, Any], p: str) -> PartSpec:
        dims, pooled = int(m["rot"]["dims"]), kind == "attention"
        position = None
        if dims:
            position = PartSpec("rotary_half" if pooled else "rotary_interleaved",
                                {"head_dim": int(m["dim"]), "rotary_dim": dims, "theta": float(m["rot"]["base"]), "precise": True,
                                 "scaling": None if pooled else (dict(m["rot"]["scaling"]) if m["rot"].get("scaling") else None)})
        params = {"hidden_size": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                  "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "qkv_bias": False, "out_bias": False,
                  "scale": float(m["scale"]), "window": int(m["mask"]["size"]), "position": position}
        tensors = {"q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "o_weight": p + "o"}
        if pooled:
            params.update({"conv_taps": int(m["conv"]), "qk_norm_eps": self.eps, "sink": "learned", "pool": int(m["mask"]["pool"])})
            tensors.update({"q_conv": p + "q.conv", "k_conv": p + "k.conv", "v_conv": p + "v.conv", "q_norm": p + "q.norm",
                            "k_norm": p + "k.norm", "sink": p + "sink"})
        else:
            params["head_gate"] = True
            tensors["g_weight"] = p + "g"
        return PartSpec("gqa_attention", params, tensors)

    def _feed_forward_spec(self, mlp: Mapping[str, Any], p: str) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("activated_mlp", {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]),
                                              "activation": DENSE_ACTIVATION, "bias": False},
                            {"up_weight": p + "up", "down_weight": p + "down"})
        experts = int(mlp["router"]["experts"])
        tensors = {"router": p + "router", "router_bias": p + "router.b"}
        for e in range(experts):
            for which in ("gate", "up", "down"):
                tensors[f"{which}.{e}"] = f"{p}e{e}.{which}"
        shared = None
        if mlp.get("shared"):
            shared = {"size": int(mlp["shared"]["ff"]), "limit": float(mlp["shared"]["limit"]), "gated": True}
            tensors.update({"shared_gate": p + "shared.gate", "shared_up": p + "shared.up", "shared_down": p + "shared.down",
                            "shared_logit": p + "shared.sg"})
        return PartSpec("routed_experts",
                        {"hidden_size": self.width, "expert_size": int(mlp["expert"]["ff"]), "experts": experts,
                         "top": int(mlp["router"]["top"]), "score": "softmax", "renormalize": True, "weight_on": "output",
                         "router_bias": True, "gate": "clamped", "limit": float(mlp["expert"]["limit"]), "alpha": EXPERT_GATE_SLOPE,
                         "shared": shared},
                        tensors)

    def model_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            parts = {"norm": self._dyt(p + "norm1"), "mixer": self._mixer_spec(layer["type"], layer["mixer"], p + "mix."),
                     "mixer_input": PartSpec("token_shift", {"width": self.width}, {"weight": p + "shift"})}
            if layer.get("mlp") is not None:
                parts["feed_forward"] = self._feed_forward_spec(layer["mlp"], p + "mlp.")
            layers.append(LayerSpec("parallel", parts))
        n = len(self.layers)
        if self.loop is None:
            schedule, stream_parts = [ScheduleEntry(i) for i in range(n)], ()
        else:
            start, stop, times = self.loop
            stream_parts = (PartSpec("embedding_mix", {"width": self.width}, {"weight": "loop.in"}),)
            schedule = [ScheduleEntry(i) for i in range(start)]
            for _ in range(times):   # each pass has caches and states of its own: every run is an entry of its own
                schedule += [ScheduleEntry(i, enter=0 if i == start else None) for i in range(start, stop)]
            schedule += [ScheduleEntry(i) for i in range(stop, n)]
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_positions=NO_LENGTH_LIMIT,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "width": self.width}, {"weight": "embed"}),
            layers=tuple(layers), schedule=tuple(schedule), final_norm=self._dyt("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "width": self.width, "tied": True}, {"weight": "embed"}),
            stream_parts=stream_parts)
        spec.validate()
        return spec


register_architecture(RarevikConfig.architecture, RarevikConfig, RarevikConfig.model_type)
