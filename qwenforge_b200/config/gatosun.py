"""Typed configuration of the Gatosun decoder: layers listed one by one, each a pre-norm layer whose sublayers enter the
stream under one multiplier, `x += m * mixer(rms(x)); x += m * ff(rms(x))`, with a mixer that is one of three kinds (a
causal attention whose q and k are normed over their whole rows and whose values may be drawn towards an earlier layer's; a
windowed attention and an RWKV-style time mixing side by side; a gated linear attention) and a feed-forward that is dense
and gated, a mixture of small experts chosen among groups, or absent.

config.json (every size and every constant that differs between models of the design is read from it):
  architecture      "Gatosun"
  vocab, width
  norm.eps          eps of every RMS norm and unit norm
  residual_mult     m above
  layers[i].type    "attention": mixer {heads, kv_heads, dim, vdim, scale, rot.{dims, base}, v_mix (optional)}
                    "parallel":  mixer {left {heads, kv_heads, dim, vdim, scale, rot.{dims, base}, mask.size}, left_scale,
                                        right {heads, dim}, right_scale}
                    "gla":       mixer {heads, dim, vdim, tau}
  layers[i].mlp     null | {kind: "dense", ff}
                         | {kind: "moe", router{experts, top, groups{count, keep} (optional)}, expert{ff}, shared{ff} (optional)}
The rank of the low-rank pairs that set the decays (`w1`/`w2`, `a1`/`a2`) is read from the tensors; a mixer may name it
(`rank`), which the random-weights mode needs.
What the design fixes stands here as constants: the tanh form of GELU in the dense feed-forward and its biases, the square
of relu in the experts, sigmoid scores that are not renormalised, the biases of the causal attention.
A sequence has no longest length: nothing in the design depends on one.

Tensor names: embed, final.norm, head; per layer l<i>.norm1, l<i>.norm2;
attention l<i>.mix.{q, k, v, o}(.b), l<i>.mix.{q.norm, k.norm}, l<i>.mix.vmix (layers with v_mix; the first one's is not read);
parallel l<i>.mix.left.{q, k, v, o}, l<i>.mix.right.{mu.r, mu.k, mu.v, mu.g, mu.w, r, k, v, g, w1, w2, w0, u, norm, o};
gla l<i>.mix.{q, k, v, g, o, norm, a1, a2, a2.b};
dense l<i>.mlp.{gate, up, down}(.b); moe l<i>.mlp.{router, correction}, l<i>.mlp.e<j>.{up, down}, l<i>.mlp.shared.{up, down}.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .registry import ModelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

DENSE_ACTIVATION = "gelu_tanh"   # 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))
EXPERT_ACTIVATION = "relu2"      # the square of relu
NO_LENGTH_LIMIT = 1 << 30        # what the runtime is told where it asks for a longest sequence
VALUE_CHAIN = "v_mix"            # the one chain of layers that share values through a step


def _need(data: Mapping[str, Any], key: str, where: str = "config.json"):
    if not isinstance(data, Mapping) or key not in data or data[key] is None:
        raise ValueError(f"{where}: required key {key!r} is missing")
    return data[key]


def _positive(data, keys, where):
    for key in keys:
        if not float(_need(data, key, where)) > 0:
            raise ValueError(f"{where}: {key} must be positive")


def _check_attention(mixer, where, windowed):
    _positive(mixer, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
    if int(mixer["heads"]) % int(mixer["kv_heads"]):
        raise ValueError(f"{where}: kv_heads must divide heads")
    rot = _need(mixer, "rot", where)
    if int(_need(rot, "dims", where + ".rot")) % 2 or not 0 <= int(rot["dims"]) <= int(mixer["dim"]):
        raise ValueError(f"{where}.rot: dims must be even and at most dim")
    if int(rot["dims"]):
        _positive(rot, ("base",), where + ".rot")
    if windowed:
        _positive(_need(mixer, "mask", where), ("size",), where + ".mask")


@dataclass(frozen=True)
class GatosunConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: tuple          # the config's own layer entries (plain dicts), validated
    torch_dtype: str = "bfloat16"

    architecture = "Gatosun"
    model_type = "gatosun"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "GatosunConfig":
        layers = _need(data, "layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        config = cls(vocab=int(_need(data, "vocab")), width=int(_need(data, "width")),
                     eps=float(_need(_need(data, "norm"), "eps", "config.json norm")),
                     residual_mult=float(_need(data, "residual_mult")),
                     layers=tuple(copy.deepcopy(dict(layer)) for layer in layers),
                     torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))))
        config.validate()
        return config

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.eps <= 0:
            raise ValueError("config.json: vocab, width and norm.eps must be positive")
        shared_values = None
        for i, layer in enumerate(self.layers):
            where = f"config.json layers[{i}]"
            kind, mixer = _need(layer, "type", where), _need(layer, "mixer", where)
            where += ".mixer"
            if kind == "attention":
                _check_attention(mixer, where, False)
                if mixer.get("v_mix"):
                    shape = (int(mixer["kv_heads"]), int(mixer["vdim"]))
                    if shared_values is not None and shape != shared_values:
                        raise ValueError(f"{where}: layers with v_mix must have as many key/value heads of the same value size")
                    shared_values = shape
            elif kind == "parallel":
                _check_attention(_need(mixer, "left", where), where + ".left", True)
                _positive(_need(mixer, "right", where), ("heads", "dim"), where + ".right")
                for key in ("left_scale", "right_scale"):
                    float(_need(mixer, key, where))
            elif kind == "gla":
                _positive(mixer, ("heads", "dim", "vdim", "tau"), where)
            else:
                raise ValueError(f"config.json layers[{i}]: mixer type {kind!r} is not supported ('attention', 'parallel', 'gla')")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            where = f"config.json layers[{i}].mlp"
            if _need(mlp, "kind", where) == "dense":
                _positive(mlp, ("ff",), where)
            elif mlp["kind"] == "moe":
                router = _need(mlp, "router", where)
                experts, top = int(_need(router, "experts", where + ".router")), int(_need(router, "top", where + ".router"))
                _positive(_need(mlp, "expert", where), ("ff",), where + ".expert")
                if not 1 <= top <= experts:
                    raise ValueError(f"{where}: 1 <= router.top <= router.experts is required")
                groups = router.get("groups")
                if groups:
                    count, keep = int(_need(groups, "count", where + ".router.groups")), int(_need(groups, "keep", where + ".router.groups"))
                    if not 1 <= keep <= count or experts % count or keep * (experts // count) < top:
                        raise ValueError(f"{where}.router.groups: count must divide the experts, and the kept groups must hold `top` experts")
                if mlp.get("shared"):
                    _positive(mlp["shared"], ("ff",), where + ".shared")
            else:
                raise ValueError(f"{where}: kind {mlp['kind']!r} is not supported ('dense', 'moe' or null)")

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "residual_mult": self.residual_mult, "layers": [copy.deepcopy(layer) for layer in self.layers],
                "torch_dtype": self.torch_dtype}

    def _rotary(self, m) -> PartSpec | None:
        dims = int(m["rot"]["dims"])
        if not dims:
            return None
        return PartSpec("rotary_half", {"head_dim": int(m["dim"]), "rotary_dim": dims, "theta": float(m["rot"]["base"]), "precise": True})

    def _attention(self, m, p, windowed: bool, value_role) -> PartSpec:
        params = {"hidden_size": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
                  "value_dim": int(m["vdim"]), "scale": float(m["scale"]), "position": self._rotary(m)}
        tensors = {"q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "o_weight": p + "o"}
        if windowed:   # no biases; the unit norm per head follows the rotation
            params.update({"qkv_bias": False, "out_bias": False, "window": int(m["mask"]["size"]), "unit_norm_eps": self.eps})
        else:          # biases everywhere; q and k normed over their whole rows before the rotation
            params.update({"qkv_bias": True, "out_bias": True, "window": 0, "row_norm_eps": self.eps})
            tensors.update({"q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b", "o_bias": p + "o.b",
                            "q_row_norm": p + "q.norm", "k_row_norm": p + "k.norm"})
            if value_role is not None:
                params["value_mix"] = {"role": value_role, "key": VALUE_CHAIN}
                if value_role == "mix":
                    tensors["value_mix"] = p + "vmix"
        return PartSpec("gqa_attention", params, tensors)

    def _mixer_spec(self, kind: str, m: Mapping[str, Any], p: str, value_role) -> PartSpec:
        if kind == "attention":
            return self._attention(m, p, False, value_role)
        if kind == "gla":
            return PartSpec(
                "gated_linear_attention",
                {"hidden_size": self.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]),
                 "tau": float(m["tau"]), "eps": self.eps, "rank": m.get("rank")},
                {"q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "g_weight": p + "g", "o_weight": p + "o",
                 "norm": p + "norm", "a1": p + "a1", "a2": p + "a2", "a2_bias": p + "a2.b"})
        right, q = m["right"], p + "right."
        tensors = {"mu_" + s: q + "mu." + s for s in "rkvgw"}
        tensors.update({s + "_weight": q + s for s in "rkvg"})
        tensors.update({"w1": q + "w1", "w2": q + "w2", "w0": q + "w0", "bonus": q + "u", "norm": q + "norm", "o_weight": q + "o"})
        time_mix = PartSpec("time_mix", {"hidden_size": self.width, "num_heads": int(right["heads"]), "head_dim": int(right["dim"]),
                                         "eps": self.eps, "rank": right.get("rank")}, tensors)
        return PartSpec("side_by_side", {"left": self._attention(m["left"], p + "left.", True, None), "right": time_mix,
                                         "left_scale": float(m["left_scale"]), "right_scale": float(m["right_scale"])})

    def _feed_forward_spec(self, mlp: Mapping[str, Any], p: str) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]),
                                          "activation": DENSE_ACTIVATION, "bias": True},
                            {"gate_weight": p + "gate", "gate_bias": p + "gate.b", "up_weight": p + "up", "up_bias": p + "up.b",
                             "down_weight": p + "down", "down_bias": p + "down.b"})
        router = mlp["router"]
        experts = int(router["experts"])
        tensors = {"router": p + "router", "correction": p + "correction"}
        for e in range(experts):
            tensors[f"up.{e}"], tensors[f"down.{e}"] = f"{p}e{e}.up", f"{p}e{e}.down"
        shared = None
        if mlp.get("shared"):
            shared = {"size": int(mlp["shared"]["ff"]), "gated": False}
            tensors.update({"shared_up": p + "shared.up", "shared_down": p + "shared.down"})
        groups = router.get("groups")
        return PartSpec("routed_experts",
                        {"hidden_size": self.width, "expert_size": int(mlp["expert"]["ff"]), "experts": experts,
                         "top": int(router["top"]), "score": "sigmoid", "renormalize": False, "weight_on": "output",
                         "gate": "none", "activation": EXPERT_ACTIVATION, "correction": True,
                         "groups": (int(groups["count"]), int(groups["keep"])) if groups else None, "shared": shared},
                        tensors)

    def model_spec(self) -> ModelSpec:
        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"width": self.width, "eps": self.eps}, {"weight": name})

        layers, ignored, source_seen = [], [], False
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            value_role = None
            if layer["type"] == "attention" and layer["mixer"].get("v_mix"):
                value_role = "mix" if source_seen else "source"
                if not source_seen:
                    ignored.append(p + "mix.vmix")   # the first such layer's number is not read
                source_seen = True
            parts = {"mixer_norm": norm(p + "norm1"), "mixer": self._mixer_spec(layer["type"], layer["mixer"], p + "mix.", value_role)}
            if layer.get("mlp") is None:
                ignored.append(p + "norm2")   # a file may still carry it
            else:
                parts["feed_forward_norm"] = norm(p + "norm2")
                parts["feed_forward"] = self._feed_forward_spec(layer["mlp"], p + "mlp.")
            layers.append(LayerSpec("pre_norm", parts, {"residual_mult": self.residual_mult}))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_positions=NO_LENGTH_LIMIT,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "width": self.width}, {"weight": "embed"}),
            layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))), final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "width": self.width, "tied": False}, {"weight": "head"}),
            ignored_tensors=tuple(ignored))
        spec.validate()
        return spec


register_architecture(GatosunConfig.architecture, GatosunConfig, GatosunConfig.model_type)
