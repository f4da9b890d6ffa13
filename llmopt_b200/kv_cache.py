"""Grouped-Q8 cache layout math, mirroring ``Kv_cache.Format`` / ``Kv_cache.Layout``
(lib/kv_cache.ml:1-200): the token pool stores, per token, the int8 K and V
segments of every attention layer back to back followed by one fp16 scale per
group; the checkpoint pool stores the recurrent state of every recurrent layer
the same way.  ``group_size`` is 64 in the reference (lib/kv_cache.ml:4);
32 is accepted here for inputs quantised per 32 elements."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

Q8_GROUP_SIZE = 64


def groups_for_elements(elements: int, group_size: int = Q8_GROUP_SIZE) -> int:
    """Format.groups_for_elements, lib/kv_cache.ml:10-14."""
    if elements < 0:
        raise ValueError("KV element count cannot be negative")
    return elements // group_size + (0 if elements % group_size == 0 else 1)


def bytes_for_elements(elements: int, group_size: int = Q8_GROUP_SIZE) -> int:
    """Format.bytes_for_elements, lib/kv_cache.ml:16-22: one byte per element + 2 per group."""
    return elements + 2 * groups_for_elements(elements, group_size)


@dataclass(frozen=True)
class AttentionLayer:
    kv_heads: int
    head_dim: int

    def __post_init__(self):
        if self.kv_heads <= 0:
            raise ValueError("attention KV layer requires positive kv_heads")
        if self.head_dim <= 0:
            raise ValueError("attention KV layer requires positive head_dim")


@dataclass(frozen=True)
class AttentionRegion:
    geometry: AttentionLayer
    key_offset: int
    value_offset: int
    segment_elements: int


class Layout:
    """Layout.create_heterogeneous, lib/kv_cache.ml:84-180."""

    def __init__(self, attentions: Sequence[AttentionLayer], recurrent_layers: int = 0, recurrent_width: int = 0,
                 recurrent_window: int = 0, group_size: int = Q8_GROUP_SIZE):
        for name, value in (("recurrent_layers", recurrent_layers), ("recurrent_width", recurrent_width),
                            ("recurrent_window", recurrent_window)):
            if value < 0:
                raise ValueError(f"{name} cannot be negative")
        if recurrent_layers > 0 and (recurrent_width == 0 or recurrent_window == 0):
            raise ValueError("recurrent checkpoint layout requires positive width and window")
        self.group_size = group_size
        self.recurrent_layers = recurrent_layers
        self.recurrent_layer_elements = recurrent_width * recurrent_window
        if any(layer.head_dim % group_size for layer in attentions):
            raise ValueError("Q8 KV group_size must divide each attention head dimension")
        if recurrent_layers > 0 and self.recurrent_layer_elements % group_size:
            raise ValueError("Q8 KV group_size must divide each recurrent layer checkpoint")
        regions, offset = [], 0
        for layer in attentions:
            segment = layer.kv_heads * layer.head_dim
            regions.append(AttentionRegion(layer, offset, offset + segment, segment))
            offset += 2 * segment
        self.attentions = tuple(regions)
        self.token_elements = offset
        self.bytes_per_token = bytes_for_elements(offset, group_size)
        self.token_groups = groups_for_elements(offset, group_size)
        self.checkpoint_elements = recurrent_layers * self.recurrent_layer_elements
        self.checkpoint_groups = groups_for_elements(self.checkpoint_elements, group_size)
        self.bytes_per_checkpoint = bytes_for_elements(self.checkpoint_elements, group_size)

    def attention_key_offset(self, layer: int) -> int:
        return self.attentions[layer].key_offset

    def attention_value_offset(self, layer: int) -> int:
        return self.attentions[layer].value_offset
