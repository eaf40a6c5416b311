from .attention import GroupedQueryAttention
from .attention_diff import DifferentialAttention
from .attention_latent import LatentAttention
from .attention_sink import SinkAttention
from .base import ROLES, ParamSpec, Part, Role, register_role, role_of
from .block import PreNorm32Block, PreNorm32MixerOnlyBlock, PreNormBlock, Summand
from .depth import DepthAverage, DepthMixerOnlyBlock, DepthPreNormBlock, DepthStream, Open
from .feedforward import BiasedFeedForward, ClampedGatedFeedForward, GatedFeedForward, RoutedExperts
from .hyper import HyperConnection, HyperMixerOnlyBlock, HyperPreNormBlock, Pending
from .norm import RMSNorm
from .parallel import ParallelMixer
from .recurrent import GatedDeltaMixer, GatedLinearRecurrence, StateSpaceMixer
from .norm_dyt import DynamicTanh
from .norm_layer import LayerNorm
from .registry import FAMILIES, lookup, register
from .rotary import InterleavedRotaryTable, PartialRotaryTable, Rotation, RotaryTable
from .sandwich import SandwichBlock, SandwichMixerOnlyBlock, Unsummed
from .wkv import WkvMixer

__all__ = ["GatedDeltaMixer", "GatedLinearRecurrence", "ParallelMixer", "PreNorm32Block", "PreNorm32MixerOnlyBlock",
           "StateSpaceMixer", "Summand", "FAMILIES", "ROLES", "Role", "register_role", "role_of", "GatedFeedForward", "GroupedQueryAttention", "DifferentialAttention", "DynamicTanh", "HyperConnection",
           "HyperMixerOnlyBlock", "HyperPreNormBlock", "Pending", "ParamSpec", "Part",
           "PreNormBlock", "RMSNorm", "RotaryTable", "Rotation", "lookup", "register", "BiasedFeedForward", "InterleavedRotaryTable", "LatentAttention", "RoutedExperts",
           "ClampedGatedFeedForward", "DepthAverage", "DepthMixerOnlyBlock", "DepthPreNormBlock", "DepthStream", "Open",
           "LayerNorm", "PartialRotaryTable", "SinkAttention", "SandwichBlock", "SandwichMixerOnlyBlock", "Unsummed", "WkvMixer"]
