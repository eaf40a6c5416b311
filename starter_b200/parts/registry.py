"""From a spec's ``kind`` to the class that implements it.

To add a part: write a spec dataclass with a new ``kind``, a class with the
interface of its family (see the existing ones), and register it here or from
your own module with ``register``.  Nothing else in the library changes.

Families and their interfaces
  mixer         ``__init__(spec, dtype, position)``; ``param_specs()``, ``set_params(params)``,
                ``kv_need()`` -> ``KVNeed`` or None, ``state_need()`` -> ``StateNeed`` or None,
                ``prepare(max_position)``, ``__call__(x, ctx, entry, writes_cache)`` -> ``[T, H]``
  feed_forward  ``__init__(spec, dtype)``; ``param_specs()``, ``set_params``, ``__call__(x, ctx)``
  norm          ``__init__(spec, dtype)``; ``param_specs()``, ``set_params``, ``__call__(x)``,
                ``add(residual, delta)``, ``add_rows(residual, delta, rows)``
  position      ``__init__(spec, dtype, device)``; ``ensure(length)`` -> True if device tables moved;
                ``rotation()`` -> ``Rotation`` (tables, how many dimensions of a head they turn and
                in which layout) for mixers that rotate queries and keys
  connection    ``__init__(spec, dtype)``; ``param_specs()``, ``set_params``; ``open(streams, pending, norm,
                dtype)`` -> a sublayer's normed input (for arrangements over several residual streams)
  arrangement   class attribute ``FAMILIES`` (part name -> family); ``__init__(parts: dict)``;
                ``parts()``; attribute ``mixer`` (the part that owns the layer's cache entry);
                ``__call__(residual, pending, ctx, entry, writes_cache)`` -> ``(residual, pending)``
"""

from __future__ import annotations

from .attention import GroupedQueryAttention
from .attention_diff import DifferentialAttention
from .attention_latent import LatentAttention
from .attention_sink import SinkAttention
from .block import PreNorm32Block, PreNorm32MixerOnlyBlock, PreNormBlock
from .depth import DepthAverage, DepthMixerOnlyBlock, DepthPreNormBlock
from .feedforward import BiasedFeedForward, ClampedGatedFeedForward, GatedFeedForward, RoutedExperts
from .hyper import HyperConnection, HyperMixerOnlyBlock, HyperPreNormBlock
from .norm import RMSNorm
from .parallel import ParallelMixer
from .recurrent import GatedDeltaMixer, GatedLinearRecurrence, StateSpaceMixer
from .norm_dyt import DynamicTanh
from .norm_layer import LayerNorm
from .rotary import InterleavedRotaryTable, PartialRotaryTable, RotaryTable
from .sandwich import SandwichBlock, SandwichMixerOnlyBlock
from .wkv import WkvMixer

FAMILIES = ("mixer", "feed_forward", "norm", "position", "connection", "arrangement")
_REGISTRY = {family: {} for family in FAMILIES}


def register(family: str, kind: str, cls) -> None:
    if family not in _REGISTRY:
        raise ValueError(f"unknown part family {family!r}; families: {', '.join(FAMILIES)}")
    _REGISTRY[family][kind] = cls


def lookup(family: str, kind: str):
    try:
        return _REGISTRY[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(family, {}))) or "none"
        raise ValueError(f"no {family} of kind {kind!r} is registered (known: {known})") from None


register("mixer", "attention", GroupedQueryAttention)
register("feed_forward", "gated_dense", GatedFeedForward)
register("norm", "rmsnorm", RMSNorm)
register("position", "rope", RotaryTable)
register("arrangement", "prenorm", PreNormBlock)
register("mixer", "differential_attention", DifferentialAttention)
register("norm", "dynamic_tanh", DynamicTanh)
register("connection", "hyper", HyperConnection)
register("arrangement", "hyper_prenorm", HyperPreNormBlock)
register("arrangement", "hyper_mixer_only", HyperMixerOnlyBlock)
register("mixer", "latent_attention", LatentAttention)
register("mixer", "wkv", WkvMixer)
register("feed_forward", "dense_biased", BiasedFeedForward)
register("feed_forward", "routed_experts", RoutedExperts)
register("position", "rope_interleaved", InterleavedRotaryTable)
register("arrangement", "sandwich", SandwichBlock)
register("arrangement", "sandwich_mixer_only", SandwichMixerOnlyBlock)
register("mixer", "sink_attention", SinkAttention)
register("feed_forward", "gated_clamped", ClampedGatedFeedForward)
register("norm", "layernorm", LayerNorm)
register("position", "rope_partial", PartialRotaryTable)
register("connection", "depth_average", DepthAverage)
register("arrangement", "depth_prenorm", DepthPreNormBlock)
register("arrangement", "depth_mixer_only", DepthMixerOnlyBlock)
register("arrangement", "prenorm32", PreNorm32Block)
register("arrangement", "prenorm32_mixer_only", PreNorm32MixerOnlyBlock)
register("mixer", "gated_linear_recurrence", GatedLinearRecurrence)
register("mixer", "state_space", StateSpaceMixer)
register("mixer", "gated_delta", GatedDeltaMixer)
register("mixer", "parallel", ParallelMixer)
