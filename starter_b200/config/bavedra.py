"""Configuration of the Bavedra decoder, read from the keys of its own ``config.json``.

The design: an embedding times a constant; pre-norm layers (RMS norms with plain gains) around a residual
stream that is a 32-bit sum; per layer one of three mixers (``rglru``: a gated branch times a real-gated
linear recurrence per channel behind a short convolution; ``parallel``: grouped-query attention with a
rotated part, a sliding window, a sink of score zero and the unrotated keys as values, side by side with a
selective state-space recurrence, the two outputs normed over the width and averaged; ``delta``: the gated
delta rule) and one of two feed-forwards (``dense``: squared relu without biases; ``moe``: gated experts
chosen by corrected scores inside the best groups, identity experts, a gated shared expert) or none.  A
layer with ``weights_of: j`` runs layer ``j``'s tensors on a cache and state of its own.  A final norm and an
output head of its own.

``config.json`` gives ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and a list
``layers``; a layer has ``type``, ``mixer``, ``mlp`` and possibly ``weights_of``:

* ``rglru``: ``mixer = {width, blocks, conv}``.
* ``parallel``: ``mixer = {left{heads, kv_heads, dim, vdim, scale, mask{size}?, rot{base, dims}?},
  right{heads, vdim, state, groups, conv, norm_groups}}``.
* ``delta``: ``mixer = {heads, kv_heads, dim, vdim, conv}``.
* ``mlp``: null, ``{kind: "dense", ff}`` or ``{kind: "moe", expert{ff}, router{experts, top, identity?,
  groups{count, keep}?}, shared{ff}?}``.

Every size and constant is read from there; a key this design does not know is an error.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from .kesedra import _lacking, _number, _positive, _unknown
from .qwen3 import ConfigError
from .spec import (
    BiasedFeedForwardSpec,
    GatedDeltaSpec,
    GatedLinearRecurrenceSpec,
    InterleavedRopeSpec,
    ModelSpec,
    NormSpec,
    ParallelMixerSpec,
    RoutedExpertsSpec,
    ScheduleEntry,
    SinkAttentionSpec,
    StateSpaceSpec,
    prenorm32_layer,
)

_TOP = {"architecture", "architectures", "embedding", "layers", "norm", "vocab", "width", "torch_dtype", "dtype"}
#: the multiplier inside the recurrent unit's decay, ``a = exp(-8 r softplus(lam))``: the design fixes it
RGLRU_DECAY_SCALE = 8.0


def _sizes(where: str, raw, keys) -> None:
    _lacking(where, raw, keys)
    _unknown(where, raw, set(keys))
    for key in keys:
        _positive(f"{where}.{key}", raw[key])


def _check_left(where: str, m) -> None:
    _lacking(where, m, ("heads", "kv_heads", "dim", "vdim", "scale"))
    _unknown(where, m, {"heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"})
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _positive(f"{where}.{key}", m[key])
    _number(where + ".scale", m["scale"])
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: {m['heads']} query heads cannot share {m['kv_heads']} key/value heads")
    if m["vdim"] != m["dim"]:
        raise ConfigError(f"{where}: the values are the keys, so vdim={m['vdim']} must equal dim={m['dim']}")
    if m.get("mask") is not None:
        _sizes(where + ".mask", m["mask"], ("size",))
    if m.get("rot") is not None:
        _lacking(where + ".rot", m["rot"], ("base", "dims"))
        _unknown(where + ".rot", m["rot"], {"base", "dims"})
        dims = _positive(where + ".rot.dims", m["rot"]["dims"])
        if not _number(where + ".rot.base", m["rot"]["base"]) > 0.0:
            raise ConfigError(f"{where}.rot.base must be positive")
        if dims % 2 or dims > m["dim"]:
            raise ConfigError(f"{where}.rot.dims={dims} must be even and at most dim={m['dim']}")


def _check_right(where: str, m) -> None:
    _sizes(where, m, ("heads", "vdim", "state", "groups", "conv", "norm_groups"))
    if m["heads"] % m["groups"]:
        raise ConfigError(f"{where}: {m['heads']} heads cannot share {m['groups']} groups")
    if (m["heads"] * m["vdim"]) % m["norm_groups"]:
        raise ConfigError(f"{where}: {m['heads'] * m['vdim']} entries do not split into {m['norm_groups']} norm groups")


def _check_mixer(where: str, kind: str, m) -> None:
    if kind == "rglru":
        _sizes(where, m, ("width", "blocks", "conv"))
        if m["width"] % m["blocks"]:
            raise ConfigError(f"{where}: width={m['width']} does not split into blocks={m['blocks']} equal parts")
    elif kind == "parallel":
        _lacking(where, m, ("left", "right"))
        _unknown(where, m, {"left", "right"})
        _check_left(where + ".left", m["left"])
        _check_right(where + ".right", m["right"])
    elif kind == "delta":
        _sizes(where, m, ("heads", "kv_heads", "dim", "vdim", "conv"))
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{where}: {m['heads']} heads cannot share {m['kv_heads']} query/key heads")
    else:
        raise ConfigError(f"{where[:-6]}.type={kind!r}: this design's mixers are 'rglru', 'parallel' and 'delta'")


def _check_mlp(where: str, mlp) -> None:
    if mlp is None:
        return
    _lacking(where, mlp, ("kind",))
    if mlp["kind"] == "dense":
        _sizes(where, {k: v for k, v in mlp.items() if k != "kind"}, ("ff",))
        return
    if mlp["kind"] != "moe":
        raise ConfigError(f"{where}.kind={mlp['kind']!r}: this design's feed-forwards are 'dense' and 'moe'")
    _lacking(where, mlp, ("expert", "router"))
    _unknown(where, mlp, {"kind", "expert", "router", "shared"})
    _sizes(where + ".expert", mlp["expert"], ("ff",))
    router = mlp["router"]
    _lacking(where + ".router", router, ("experts", "top"))
    _unknown(where + ".router", router, {"experts", "top", "identity", "groups"})
    experts = _positive(where + ".router.experts", router["experts"])
    top = _positive(where + ".router.top", router["top"])
    identity = router.get("identity") or 0
    if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
        raise ConfigError(f"{where}.router.identity={identity!r}: a count is needed")
    outputs = experts + identity
    allowed = outputs
    if router.get("groups") is not None:
        _sizes(where + ".router.groups", router["groups"], ("count", "keep"))
        count, keep = router["groups"]["count"], router["groups"]["keep"]
        if outputs % count or keep > count:
            raise ConfigError(f"{where}.router.groups: {outputs} router outputs in {count} groups of which {keep} are kept")
        allowed = outputs // count * keep
    if top > allowed:
        raise ConfigError(f"{where}.router: top={top} of {allowed} experts that can be chosen")
    if mlp.get("shared") is not None:
        _sizes(where + ".shared", mlp["shared"], ("ff",))


@dataclass(frozen=True)
class BavedraConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple          # the layer dicts as config.json gives them (validated)
    torch_dtype: str = "bfloat16"

    architecture = "Bavedra"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, raw: dict) -> "BavedraConfig":
        _lacking("config.json", raw, ("embedding", "layers", "norm", "vocab", "width"))
        _unknown("the model", raw, _TOP)
        _lacking("norm", raw["norm"], ("eps",))
        _unknown("norm", raw["norm"], {"eps"})
        _lacking("embedding", raw["embedding"], ("scale",))
        _unknown("embedding", raw["embedding"], {"scale"})
        eps = _number("norm.eps", raw["norm"]["eps"])
        if not eps >= 0.0:
            raise ConfigError(f"norm.eps={eps} must not be negative")
        layers = raw["layers"]
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json has no layers")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            _lacking(where, layer, ("type", "mixer"))
            _unknown(where, layer, {"type", "mixer", "mlp", "weights_of"})
            _check_mixer(where + ".mixer", layer["type"], layer["mixer"])
            _check_mlp(where + ".mlp", layer.get("mlp"))
            source = layer.get("weights_of")
            if source is not None and (isinstance(source, bool) or not isinstance(source, int)
                                       or not 0 <= source < len(layers) or source == i):
                raise ConfigError(f"{where}.weights_of={source!r} must name another layer of the model")
            checked.append(copy.deepcopy(dict(layer)))
        for i, layer in enumerate(checked):
            if layer.get("weights_of") is None:
                continue
            owner = cls._owner(checked, i)
            for key in ("type", "mixer", "mlp"):
                if checked[owner].get(key) != layer.get(key):
                    raise ConfigError(f"layers[{i}].weights_of={layer['weights_of']}: its {key} differs from that layer's")
        return cls(
            vocab=_positive("vocab", raw["vocab"]),
            width=_positive("width", raw["width"]),
            embedding_scale=_number("embedding.scale", raw["embedding"]["scale"]),
            norm_eps=eps,
            layers=tuple(checked),
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
        )

    @staticmethod
    def _owner(layers, i: int) -> int:
        """The layer whose tensors layer ``i`` runs: itself, or what its ``weights_of`` leads to (a layer may name
        one that comes later, or one that itself names another)."""
        seen = set()
        while layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError(f"layers[{i}].weights_of leads back to itself: no layer of that circle has tensors")
            seen.add(i)
            i = int(layers[i]["weights_of"])
        return i

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        return {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": copy.deepcopy(list(self.layers)),
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
            "torch_dtype": self.torch_dtype,
        }

    # ------------------------------------------------------------------ meaning

    def _left(self, m: dict, prefix: str):
        rot = m.get("rot")
        spec = SinkAttentionSpec(
            hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
            value_dim=int(m["vdim"]), scale=float(m["scale"]), distance_penalty=False, sink=False, head_gate=False,
            window=int(m["mask"]["size"]) if m.get("mask") is not None else None,
            position=InterleavedRopeSpec(dims=int(rot["dims"]), base=float(rot["base"])) if rot is not None else None,
            fixed_sink=0.0, values_from_keys=True)
        return spec, {n: prefix + n for n in ("q", "k", "o")}

    def _right(self, m: dict, prefix: str):
        spec = StateSpaceSpec(hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["vdim"]),
                              state=int(m["state"]), groups=int(m["groups"]), conv=int(m["conv"]),
                              norm_groups=int(m["norm_groups"]), norm_eps=self.norm_eps)
        names = {"in": prefix + "in", "conv": prefix + "conv", "conv_bias": prefix + "conv.b", "dt_bias": prefix + "dt_bias",
                 "A_log": prefix + "A_log", "D": prefix + "D", "norm": prefix + "norm", "o": prefix + "o"}
        return spec, names

    def _mixer(self, m: dict, kind: str, prefix: str):
        if kind == "rglru":
            spec = GatedLinearRecurrenceSpec(hidden_size=self.width, width=int(m["width"]), blocks=int(m["blocks"]),
                                             conv=int(m["conv"]), decay_scale=RGLRU_DECAY_SCALE)
            names = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b",
                     "ra": "ra", "ra_bias": "ra.b", "ri": "ri", "ri_bias": "ri.b", "lam": "lam", "o": "o"}
            return spec, {f"mixer.{k}": prefix + v for k, v in names.items()}
        if kind == "delta":
            spec = GatedDeltaSpec(hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                                  head_dim=int(m["dim"]), value_dim=int(m["vdim"]), conv=int(m["conv"]),
                                  norm_eps=self.norm_eps)
            names = {"q": "q", "q_conv": "q.conv", "k": "k", "k_conv": "k.conv", "v": "v", "v_conv": "v.conv", "b": "b",
                     "a": "a", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm", "g": "g", "o": "o"}
            return spec, {f"mixer.{k}": prefix + v for k, v in names.items()}
        left, left_names = self._left(m["left"], prefix + "left.")
        right, right_names = self._right(m["right"], prefix + "right.")
        spec = ParallelMixerSpec(hidden_size=self.width, left=left, right=right, norm_eps=self.norm_eps)
        names = {f"mixer.left.{k}": v for k, v in left_names.items()}
        names.update({f"mixer.right.{k}": v for k, v in right_names.items()})
        names.update({"mixer.left_out": prefix + "left.out", "mixer.right_out": prefix + "right.out"})
        return spec, names

    def _feed_forward(self, mlp: dict, prefix: str):
        if mlp["kind"] == "dense":
            spec = BiasedFeedForwardSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), activation="relu2",
                                         bias=False)
            return spec, {"feed_forward.up": prefix + "up", "feed_forward.down": prefix + "down"}
        router = mlp["router"]
        experts = int(router["experts"])
        groups = router.get("groups") or {"count": 1, "keep": 1}
        shared = mlp.get("shared")
        spec = RoutedExpertsSpec(
            hidden_size=self.width, intermediate_size=int(mlp["expert"]["ff"]), experts=experts, top=int(router["top"]),
            expert="gated_silu", scoring="softmax_all", router_bias=False, correction=True,
            group_count=int(groups["count"]), group_keep=int(groups["keep"]),
            identity_experts=int(router.get("identity") or 0), shared_size=int(shared["ff"]) if shared is not None else 0)
        names = {"feed_forward.router": prefix + "router", "feed_forward.correction": prefix + "correction"}
        for e in range(experts):
            for part in ("gate", "up", "down"):
                names[f"feed_forward.e{e}_{part}"] = f"{prefix}e{e}.{part}"
        if shared is not None:
            for part in ("gate", "up", "down"):
                names[f"feed_forward.shared_{part}"] = f"{prefix}shared.{part}"
            names["feed_forward.shared_sg"] = prefix + "shared.sg"
        return spec, names

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec(size=self.width, eps=self.norm_eps, gain_32bit=True)
        layers, place = [], {}
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is not None:
                continue
            prefix = f"l{i}."
            mixer, names = self._mixer(layer["mixer"], layer["type"], prefix + "mix.")
            names["norm1.weight"] = prefix + "norm1"
            mlp = layer.get("mlp")
            if mlp is not None:
                ff, ff_names = self._feed_forward(mlp, prefix + "mlp.")
                names["norm2.weight"] = prefix + "norm2"
                names.update(ff_names)
                spec = prenorm32_layer(mixer, ff, norm, norm, names)
            else:
                spec = prenorm32_layer(mixer, None, norm, None, names)
            place[i] = len(layers)
            layers.append(spec)
        # every layer of config.json is one run, on a cache entry and state of its own; a layer with
        # ``weights_of`` is the same parts once more
        schedule = [ScheduleEntry(layer=place[self._owner(self.layers, i)], cache=i) for i in range(len(self.layers))]
        ignored = tuple(f"l{i}.norm2" for i, layer in enumerate(self.layers)
                        if layer.get("mlp") is None and layer.get("weights_of") is None)
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=self.width,
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=norm,
            tie_embeddings=False,
            embed_name="embed",
            final_norm_name="final.norm",
            lm_head_name="head",
            ignored_tensors=ignored,
            embedding_scale=self.embedding_scale,
        )
