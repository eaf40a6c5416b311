"""Configuration of the Korurax decoder, read from the keys of its own ``config.json``.

The design: pre-norm layers (layer norm with a gain and no bias) around a residual stream that is a
32-bit sum; a sublayer's output enters the stream times ``residual_mult``; behind layer ``i`` the stream
becomes ``sum_j dwa_i[j] X_j`` over the embedding output ``X_0`` and the layer results ``X_1 .. X_(i+1)``.
Per layer one of two mixers (``attention``: grouped-query attention without rotation, inside chunks of
the sequence, with a logarithmic distance penalty, a sink in the softmax and a sigmoid gate per head;
``latent_attention``: causal attention over a cached low-rank latent with a half-split rotated key part
that all heads share) and one of two feed-forwards (``dense``: clamped and gated; ``moe``: routed
squared-relu experts weighted by normalised sigmoid scores) or none; a final layer norm, the embedding
table as output head, and ``cap * tanh(logits / cap)``.

``config.json`` gives ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``residual_mult``,
``logit_softcap`` and a list ``layers``; a layer has ``type``, ``mixer`` and ``mlp``:

* ``attention``: ``mixer = {heads, kv_heads, dim, vdim, scale, mask{size}}``.
* ``latent_attention``: ``mixer = {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot{base, dims}}``.
* ``mlp``: null, ``{kind: "dense", ff, limit}`` or ``{kind: "moe", expert{ff}, router{experts, top, scale}}``.

Every size and constant is read from there; a key this design does not know is an error.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from .kesedra import _lacking, _number, _positive, _unknown
from .qwen3 import ConfigError
from .spec import (
    ClampedGatedFeedForwardSpec,
    DepthAverageSpec,
    LatentAttentionSpec,
    LayerNormSpec,
    ModelSpec,
    PartialRopeSpec,
    RoutedExpertsSpec,
    SinkAttentionSpec,
    default_schedule,
    depth_layer,
)

_TOP = {"architecture", "architectures", "layers", "norm", "vocab", "width", "residual_mult", "logit_softcap",
        "torch_dtype", "dtype"}
_ATTENTION = ("heads", "kv_heads", "dim", "vdim", "scale", "mask")
_LATENT = ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot")


def _check_mlp(where: str, mlp) -> None:
    if mlp is None:
        return
    _lacking(where, mlp, ("kind",))
    if mlp["kind"] == "dense":
        _lacking(where, mlp, ("ff", "limit"))
        _unknown(where, mlp, {"kind", "ff", "limit"})
        _positive(where + ".ff", mlp["ff"])
        if not _number(where + ".limit", mlp["limit"]) > 0.0:
            raise ConfigError(f"{where}.limit must be positive")
    elif mlp["kind"] == "moe":
        _unknown(where, mlp, {"kind", "expert", "router"})
        _lacking(where + ".expert", mlp.get("expert"), ("ff",))
        _unknown(where + ".expert", mlp["expert"], {"ff"})
        _lacking(where + ".router", mlp.get("router"), ("experts", "top", "scale"))
        _unknown(where + ".router", mlp["router"], {"experts", "top", "scale"})
        _positive(where + ".expert.ff", mlp["expert"]["ff"])
        _number(where + ".router.scale", mlp["router"]["scale"])
        experts = _positive(where + ".router.experts", mlp["router"]["experts"])
        top = _positive(where + ".router.top", mlp["router"]["top"])
        if top > experts:
            raise ConfigError(f"{where}.router: top={top} of experts={experts}")
    else:
        raise ConfigError(f"{where}.kind={mlp['kind']!r}: this design's feed-forwards are 'dense' and 'moe'")


@dataclass(frozen=True)
class KoruraxConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_softcap: float
    layers: tuple          # the layer dicts as config.json gives them (validated)
    torch_dtype: str = "bfloat16"

    architecture = "Korurax"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, raw: dict) -> "KoruraxConfig":
        _lacking("config.json", raw, ("layers", "norm", "vocab", "width", "residual_mult", "logit_softcap"))
        _unknown("the model", raw, _TOP)
        _lacking("norm", raw["norm"], ("eps",))
        _unknown("norm", raw["norm"], {"eps"})
        eps = _number("norm.eps", raw["norm"]["eps"])
        if not eps >= 0.0:
            raise ConfigError(f"norm.eps={eps} must not be negative")
        cap = _number("logit_softcap", raw["logit_softcap"])
        if not cap > 0.0:
            raise ConfigError(f"logit_softcap={cap} must be positive")
        layers = raw["layers"]
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json has no layers")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            _lacking(where, layer, ("type", "mixer"))
            _unknown(where, layer, {"type", "mixer", "mlp"})
            mixer = layer["mixer"]
            if layer["type"] == "attention":
                _lacking(where + ".mixer", mixer, _ATTENTION)
                _unknown(where + ".mixer", mixer, set(_ATTENTION))
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive(f"{where}.mixer.{key}", mixer[key])
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"{where}.mixer: {mixer['heads']} query heads cannot share "
                                      f"{mixer['kv_heads']} key/value heads")
                _number(where + ".mixer.scale", mixer["scale"])
                _lacking(where + ".mixer.mask", mixer["mask"], ("size",))
                _unknown(where + ".mixer.mask", mixer["mask"], {"size"})
                _positive(where + ".mixer.mask.size", mixer["mask"]["size"])
            elif layer["type"] == "latent_attention":
                _lacking(where + ".mixer", mixer, _LATENT)
                _unknown(where + ".mixer", mixer, set(_LATENT))
                for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
                    _positive(f"{where}.mixer.{key}", mixer[key])
                _number(where + ".mixer.scale", mixer["scale"])
                _lacking(where + ".mixer.rot", mixer["rot"], ("base", "dims"))
                _unknown(where + ".mixer.rot", mixer["rot"], {"base", "dims"})
                dims = _positive(where + ".mixer.rot.dims", mixer["rot"]["dims"])
                if not _number(where + ".mixer.rot.base", mixer["rot"]["base"]) > 0.0:
                    raise ConfigError(f"{where}.mixer.rot.base must be positive")
                if dims % 2 or dims > mixer["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims={dims} must be even and at most rot_dim="
                                      f"{mixer['rot_dim']}")
            else:
                raise ConfigError(f"{where}.type={layer['type']!r}: this design's mixers are 'attention' and "
                                  "'latent_attention'")
            _check_mlp(where + ".mlp", layer.get("mlp"))
            checked.append(copy.deepcopy(dict(layer)))
        return cls(
            vocab=_positive("vocab", raw["vocab"]),
            width=_positive("width", raw["width"]),
            norm_eps=eps,
            residual_mult=_number("residual_mult", raw["residual_mult"]),
            logit_softcap=cap,
            layers=tuple(checked),
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
        )

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        return {
            "architecture": self.architecture,
            "layers": copy.deepcopy(list(self.layers)),
            "logit_softcap": self.logit_softcap,
            "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "vocab": self.vocab,
            "width": self.width,
            "torch_dtype": self.torch_dtype,
        }

    # ------------------------------------------------------------------ meaning

    def _mixer(self, m: dict, kind: str, prefix: str):
        if kind == "attention":
            spec = SinkAttentionSpec(
                hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                head_dim=int(m["dim"]), value_dim=int(m["vdim"]), scale=float(m["scale"]), distance_penalty=True,
                sink=True, head_gate=True, chunk=int(m["mask"]["size"]))
            names = {f"mixer.{n}": prefix + n for n in ("q", "k", "v", "o", "r1", "r2", "sink", "g")}
            return spec, names
        spec = LatentAttentionSpec(
            hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
            value_dim=int(m["vdim"]), q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
            norm_eps=self.norm_eps,
            position=PartialRopeSpec(dims=int(m["rot"]["dims"]), base=float(m["rot"]["base"])),
            window=None, own_kv=True)
        names = {"mixer.dq": prefix + "dq", "mixer.dq_norm": prefix + "dq.norm", "mixer.uq": prefix + "uq",
                 "mixer.uk": prefix + "uk", "mixer.uv": prefix + "uv", "mixer.o": prefix + "o",
                 "mixer.dkv": prefix + "dkv", "mixer.dkv_norm": prefix + "dkv.norm"}
        return spec, names

    def _feed_forward(self, mlp: dict, prefix: str):
        if mlp["kind"] == "dense":
            spec = ClampedGatedFeedForwardSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]),
                                               limit=float(mlp["limit"]))
            return spec, {"feed_forward.gate": prefix + "gate", "feed_forward.up": prefix + "up",
                          "feed_forward.down": prefix + "down"}
        experts = int(mlp["router"]["experts"])
        spec = RoutedExpertsSpec(hidden_size=self.width, intermediate_size=int(mlp["expert"]["ff"]), experts=experts,
                                 top=int(mlp["router"]["top"]), expert="relu2", scoring="sigmoid_normalised",
                                 weight_scale=float(mlp["router"]["scale"]), router_bias=False)
        names = {"feed_forward.router": prefix + "router"}
        for e in range(experts):
            for part in ("up", "down"):
                names[f"feed_forward.e{e}_{part}"] = f"{prefix}e{e}.{part}"
        return spec, names

    def to_model_spec(self) -> ModelSpec:
        norm = LayerNormSpec(size=self.width, eps=self.norm_eps)
        layers, ignored = [], []
        for i, layer in enumerate(self.layers):
            prefix = f"l{i}."
            mixer, names = self._mixer(layer["mixer"], layer["type"], prefix + "mix.")
            names.update({"norm1.weight": prefix + "norm1", "connection.weights": prefix + "dwa"})
            connection = DepthAverageSpec(levels=i + 2, multiplier=self.residual_mult)
            mlp = layer.get("mlp")
            if mlp is not None:
                ff, ff_names = self._feed_forward(mlp, prefix + "mlp.")
                names["norm2.weight"] = prefix + "norm2"
                names.update(ff_names)
                layers.append(depth_layer(mixer, ff, norm, norm, connection, names))
            else:
                # nothing reads the second norm of a layer without a feed-forward, should a checkpoint carry it
                ignored.append(prefix + "norm2")
                layers.append(depth_layer(mixer, None, norm, None, connection, names))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=self.width,
            layers=tuple(layers),
            schedule=default_schedule(len(layers)),
            final_norm=norm,
            tie_embeddings=True,
            embed_name="embed",
            final_norm_name="final.norm",
            lm_head_name="head",
            ignored_tensors=tuple(ignored),
            logit_softcap=self.logit_softcap,
        )
