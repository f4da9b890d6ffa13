"""Tensor-parallel decode over the GPUs of one node (one process per GPU).

The reference is single-device; this module adds the sharding its kernels admit without
changing their arithmetic:

* column split (rows of W): Q/K/V by head, gate/up by intermediate column, LM head by
  vocabulary row -- quantisation groups run along K, so no group is cut;
* row split (K of W): o_proj and down -- each rank multiplies its K slice and writes an
  unrounded fp32 partial sum (``llmopt_w4a16_linear_partial_f32_g64``); the partial sums of
  all ranks are added in rank order, the residual is added and the result rounded to half
  once (``llmopt_tp_exchange_sum_f16``), so every rank holds the same bits;
* attention by KV head: each rank owns a Q8 token pool with its own KV heads only;
* LM head: stage-1 candidates of every rank's vocabulary shard, one argmax over all of them
  (``llmopt_tp_exchange_argmax``).

The exchange kernels read the peers' contributions straight from their memory (CUDA IPC over
NVLink / NVSwitch); there is no collective library on the data path.  Each rank's "region"
holds a small header (epoch, arrival counter, flags) and data slots; ``plan_slots`` assigns a
slot to every exchange of a decode step so that two uses of one slot are at least two
exchanges apart, which is what makes rewriting a slot safe without a second handshake.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Callable, List, Optional, Sequence

import numpy as np

REGION_HEADER_BYTES = 256
CANDIDATE_PARTS = 256  # stage-1 candidates per row (lib/metal_dispatch_linear.ml:640-678)


def shards(config, world: int) -> bool:
    """Whether the model splits evenly over ``world`` ranks (heads, columns and K groups)."""
    if world < 1 or world > 8:
        return False
    if config.conv_layers:
        return world == 1  # the short-conv blocks are not sharded here
    return (config.kv_heads % world == 0 and config.query_heads % world == 0
            and config.intermediate % (64 * world) == 0 and (config.query_heads * config.head_dim) % (64 * world) == 0
            and config.vocabulary % world == 0)


def local_config(config, world: int):
    """The per-rank shapes: heads, intermediate columns and vocabulary rows divided by ``world``."""
    if not shards(config, world):
        raise ValueError(f"{config.name} does not split over {world} ranks")
    return replace(config, name=f"{config.name}/tp{world}", query_heads=config.query_heads // world,
                   kv_heads=config.kv_heads // world, intermediate=config.intermediate // world,
                   vocabulary=config.vocabulary // world)


def _rows(pair, start: int, stop: int):
    packed, scale = pair
    return np.ascontiguousarray(packed[start:stop]), np.ascontiguousarray(scale[start:stop])


def _k_slice(pair, start: int, stop: int):
    """Columns [start, stop) of K: packed bytes hold two k each, scales one per 64."""
    packed, scale = pair
    return (np.ascontiguousarray(packed[:, start // 2:stop // 2]),
            np.ascontiguousarray(scale[:, start // 64:stop // 64]))


def shard_weights(config, weights: dict, rank: int, world: int) -> dict:
    """Rank ``rank``'s share of ``weights`` (the dict of ``model.random_weights``)."""
    local = local_config(config, world)
    dim = config.head_dim
    out = {"embedding": weights["embedding"], "final_norm": weights["final_norm"]}
    vocabulary = local.vocabulary
    out["lm_head"] = _rows(weights["lm_head"], rank * vocabulary, (rank + 1) * vocabulary)
    q_rows, kv_rows, columns = local.query_heads * dim, local.kv_heads * dim, local.intermediate
    for index in range(len(config.layers)):
        source = weights[f"layer{index}"]
        layer = {"input_norm": source["input_norm"], "ffn_norm": source["ffn_norm"]}
        layer["q"] = _rows(source["q"], rank * q_rows, (rank + 1) * q_rows)
        layer["k"] = _rows(source["k"], rank * kv_rows, (rank + 1) * kv_rows)
        layer["v"] = _rows(source["v"], rank * kv_rows, (rank + 1) * kv_rows)
        layer["o"] = _k_slice(source["o"], rank * q_rows, (rank + 1) * q_rows)
        layer["gate"] = _rows(source["gate"], rank * columns, (rank + 1) * columns)
        layer["up"] = _rows(source["up"], rank * columns, (rank + 1) * columns)
        layer["down"] = _k_slice(source["down"], rank * columns, (rank + 1) * columns)
        out[f"layer{index}"] = layer
    return out


def plan_slots(exchanges: int) -> tuple:
    """(slot count, slot of each exchange of one step).  Slots are taken round-robin; the count is
    the smallest of 3, 4, 5, 7 for which the step's last use of a slot and the next step's first use
    of it are also at least two exchanges apart (``exchanges % count != 1``).  A step with a single
    exchange cannot alternate slots by itself and is refused."""
    if exchanges <= 0:
        return 0, []
    if exchanges == 1:
        raise ValueError("a step with a single exchange would reuse its slot in adjacent exchanges")
    for count in (3, 4, 5, 7):
        if exchanges % count != 1:
            return count, [index % count for index in range(exchanges)]
    raise ValueError("no slot count up to 7 fits this number of exchanges")  # first at 421 exchanges


def plan_prompt_slots(slot_count: int, exchanges: int, decode_slots: Sequence[int]) -> list:
    """Slot of each exchange of a prompt pass that runs between decode steps whose exchanges use
    ``decode_slots``: round-robin from a start chosen so that the first is not the decode step's last
    slot and the last is not its first (adjacent exchanges then never share a slot, across the
    border either).  Needs at least three slots."""
    if slot_count < 3:
        raise ValueError("a tensor-parallel prompt needs at least three exchange slots")
    decode = list(decode_slots) or [0]
    for start in range(slot_count):
        candidate = [(start + index) % slot_count for index in range(exchanges)]
        if not candidate or (candidate[0] != decode[-1] and candidate[-1] != decode[0]):
            return candidate
    raise ValueError("no slot order fits between the decode steps' exchanges")


def prompt_row_share(rows: int, world: int, rank: int) -> tuple:
    """[first, last) of the prompt rows rank ``rank`` sums in the reduce-scatter exchange and hands
    out in the all-gather exchange: ceil(rows / world) consecutive rows per rank, the last ranks
    fewer or none (the partition ``llmopt_tp_exchange_reduce_rows_f16`` uses)."""
    share = (rows + world - 1) // world
    first = min(rank * share, rows)
    return first, min(first + share, rows)


def check_slot_plan(slots: Sequence[int]) -> bool:
    """True when, replaying the step forever, two uses of a slot are never adjacent exchanges."""
    doubled = list(slots) + list(slots)
    return all(doubled[i] != doubled[i + 1] for i in range(len(doubled) - 1))


@dataclass
class ExchangeGroup:
    """This rank's view of the group: its own region and the peers' mapped regions."""

    rank: int
    world: int
    slot_bytes: int
    slot_count: int
    regions: list  # Buffer per rank; regions[rank] is this rank's own allocation

    @classmethod
    def create(cls, runtime, rank: int, world: int, slot_bytes: int, slot_count: int,
               all_gather: Optional[Callable[[object], List[object]]] = None) -> "ExchangeGroup":
        """Allocates this rank's region and maps the peers'.  ``all_gather(obj)`` returns the list
        of every rank's ``obj`` in rank order (e.g. ``torch.distributed.all_gather_object``); it
        may be omitted for a group of one."""
        from .cuda_native import Buffer

        slot_bytes = (slot_bytes + 255) // 256 * 256
        region = Buffer.create(runtime, REGION_HEADER_BYTES + slot_bytes * slot_count)  # zero filled: epoch 0
        if world == 1:
            return cls(rank, world, slot_bytes, slot_count, [region])
        if all_gather is None:
            raise ValueError("a group of more than one rank needs an all_gather function")
        exported = all_gather(region.export_handle())
        regions = [region if peer == rank else Buffer.import_handle(runtime, exported[peer]) for peer in range(world)]
        all_gather(("mapped", rank))  # nobody proceeds (and possibly exits) before every peer has mapped
        return cls(rank, world, slot_bytes, slot_count, regions)

    def slot_offset(self, slot: int) -> int:
        if not 0 <= slot < self.slot_count:
            raise ValueError("slot out of range")
        return REGION_HEADER_BYTES + slot * self.slot_bytes

    def slot_view(self, slot: int, nbytes: int):
        """This rank's own slot, as the output buffer of the kernel that produces its contribution."""
        if nbytes > self.slot_bytes:
            raise ValueError("contribution larger than a slot")
        return self.regions[self.rank].view(self.slot_offset(slot), nbytes)

    def sum_record(self, dispatch_item, *, slot: int, rows: int, width: int, residual, output):
        """``llmopt_tp_exchange_sum_f16``: output = half(residual + sum over ranks of the fp32 slot)."""
        from . import parameters

        params = parameters.u32s([self.world, self.rank, rows, width, self.slot_offset(slot), 1 if residual else 0])
        buffers = list(self.regions) + [residual if residual is not None else output, output]
        return dispatch_item(name="llmopt_tp_exchange_sum_f16", buffers=buffers, parameters=params,
                             grid=(256, 1, 1), group=(256, 1, 1))

    def sum_norm_record(self, dispatch_item, *, slot: int, rows: int, width: int, residual, output, norm_weight,
                        normalized, epsilon: float, weight_first: bool):
        """``llmopt_tp_exchange_sum_rms_f16``: the exchange sum and the RMS normalisation of its result
        in one kernel (``normalized`` = what the following rms kernel would have written)."""
        import struct

        params = struct.pack("<6IfI", self.world, self.rank, rows, width, self.slot_offset(slot),
                             1 if residual else 0, epsilon, 1 if weight_first else 0)
        buffers = list(self.regions) + [residual if residual is not None else output, output, norm_weight, normalized]
        return dispatch_item(name="llmopt_tp_exchange_sum_rms_f16", buffers=buffers, parameters=params,
                             grid=(256 * rows, 1, 1), group=(256, 1, 1))

    def sum_rows_records(self, dispatch_item, *, slot: int, slice_slot: int, rows: int, width: int, residual, output):
        """Prompt rows: the exchange sum as a reduce-scatter and an all-gather, two exchanges on two slots
        (``llmopt_tp_exchange_reduce_rows_f16``: this rank's share of the rows from every rank's fp32 partial in
        ``slot``, written to ``output`` and, as fp16, to its own ``slice_slot``; ``llmopt_tp_exchange_gather_rows_f16``:
        the other ranks' shares).  A rank reads each partial once for its own rows only."""
        from . import parameters

        if slot == slice_slot:
            raise ValueError("the fp32 partials and the fp16 shares need different slots")
        if rows * width * 4 > self.slot_bytes:
            raise ValueError("contribution larger than a slot")
        params = parameters.u32s([self.world, self.rank, rows, width, self.slot_offset(slot), 1 if residual else 0,
                                  self.slot_offset(slice_slot)])
        buffers = list(self.regions) + [residual if residual is not None else output, output]
        first = dispatch_item(name="llmopt_tp_exchange_reduce_rows_f16", buffers=buffers, parameters=params,
                              grid=(256, 1, 1), group=(256, 1, 1))
        second = dispatch_item(name="llmopt_tp_exchange_gather_rows_f16", buffers=list(self.regions) + [output],
                               parameters=params, grid=(256, 1, 1), group=(256, 1, 1))
        return [first, second]

    def argmax_record(self, dispatch_item, *, slot: int, rows: int, shard_columns: int, output):
        """``llmopt_tp_exchange_argmax``: best of every rank's stage-1 candidates, global indices."""
        from . import parameters

        params = parameters.u32s([self.world, self.rank, rows, CANDIDATE_PARTS, self.slot_offset(slot), shard_columns])
        return dispatch_item(name="llmopt_tp_exchange_argmax", buffers=list(self.regions) + [output],
                             parameters=params, grid=(256, rows, 1), group=(256, 1, 1))


def torch_all_gather(group=None) -> Callable[[object], List[object]]:
    """``all_gather`` for ``ExchangeGroup.create`` over an initialised torch.distributed group
    (any backend; only Python objects travel)."""
    import torch.distributed as dist

    def gather(obj):
        out = [None] * dist.get_world_size(group)
        dist.all_gather_object(out, obj, group=group)
        return out

    return gather
