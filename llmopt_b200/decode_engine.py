"""Whole-token decode over the hot-path kernels: builds, for one model and batch
size, the per-token dispatch list the reference's schedule executor would
record (embedding, per block: RMSNorm, fused W4A16 QKV, rotary, paged Q8
attention, Q8 cache pack, W4A16 o-proj + residual, W4A16 SwiGLU FFN; or the gated
short-conv block; then the W4A16 LM-head argmax) and hands it to a prebaked plan
— the role of ``Metal_runtime.bind_decode_plan`` + ``Prebaked``
(lib/metal_schedule_executor.ml:495-547, lib/serving_engine.ml:699-790).

The per-token host work of the reference engine (RoPE row, cache slot of the new
token) is done on the device by the plan's row bindings.  Batch > 1 (one token
per sequence per step, per-sequence slot tables) is an extension: the reference
decodes sequences one at a time (lib/serving_engine.ml:1542-1548).

With an ``ExchangeGroup`` the engine builds one rank's share of a tensor-parallel
decode (``tensor_parallel.py``): local heads and columns, fp32 partial sums of the
row-split products exchanged and reduced over peer memory, one argmax over all
ranks' vocabulary shards.  Every rank computes the same hidden state and token.
"""

from __future__ import annotations

import math
import time
from typing import Optional, Sequence

import numpy as np

from . import dispatch, kernel_abi, parameters
from .cuda_native import Batch, Buffer, Prebaked, Runtime, pack_records
from .kv_cache import AttentionLayer, Layout
from .model import ModelConfig
from .quantize import rope_tables


class DecodeEngine:
    def __init__(self, runtime: Runtime, config: ModelConfig, weights: Optional[dict], *, batch: int = 1,
                 capacity: int = 1024, group=None, share_weights_of: Optional["DecodeEngine"] = None):
        """``config`` and ``weights`` are the whole model's, or, with ``group`` (an
        ``ExchangeGroup`` of more than one rank), this rank's ``tensor_parallel.local_config`` /
        ``shard_weights`` share; the embedding table is always whole.  ``share_weights_of``:
        another engine of the same model and capacity on the same runtime whose uploaded weights
        and RoPE tables this one binds instead of uploading its own (``weights`` is then unused)."""
        self.runtime, self.config, self.batch, self.capacity = runtime, config, batch, capacity
        self.group = group  # a group of one rank still takes the exchange kernels (single-GPU check of the plan)
        self.full_vocabulary = config.vocabulary * (self.group.world if self.group else 1)
        self.layout = Layout([AttentionLayer(config.kv_heads, config.head_dim)] * config.attention_layers,
                             group_size=config.kv_group_size)
        self.cache = dispatch.Cache(runtime, self.layout, token_capacity=batch * capacity)
        self._keep = []
        if share_weights_of is not None:
            if share_weights_of.runtime is not runtime or share_weights_of.capacity < capacity:
                raise ValueError("weights can only be shared between engines of one runtime and capacity")
            other = share_weights_of
            self.embedding, self.lm_head, self.final_norm, self.layers = (
                other.embedding, other.lm_head, other.final_norm, other.layers)
            self.cos_table, self.sin_table = other.cos_table, other.sin_table
        else:
            self._upload(weights)
        self._workspace()
        self.plan = None
        self.records = None

    # ---- device state ---------------------------------------------------------------------
    def _tensor(self, array, dtype=None) -> dispatch.Tensor:
        array = np.ascontiguousarray(array)
        names = {np.dtype(np.float16): "float16", np.dtype(np.uint8): "uint8", np.dtype(np.uint32): "uint32"}
        return dispatch.Tensor(Buffer.of_array(self.runtime, array), tuple(array.shape), dtype or names[array.dtype])

    def _empty(self, shape, dtype="float16", itemsize=2) -> dispatch.Tensor:
        return dispatch.Tensor(Buffer.create(self.runtime, math.prod(shape) * itemsize), tuple(shape), dtype)

    def _upload(self, weights: dict) -> None:
        config = self.config
        self.embedding = self._tensor(weights["embedding"])
        self.lm_head = tuple(self._tensor(a) for a in weights["lm_head"])
        self.final_norm = self._tensor(weights["final_norm"])
        self.layers = []
        for index in range(len(config.layers)):
            source = weights[f"layer{index}"]
            layer = {}
            for key, value in source.items():
                layer[key] = tuple(self._tensor(a) for a in value) if isinstance(value, tuple) else self._tensor(value)
            self.layers.append(layer)
        cosine, sine = rope_tables(self.capacity + 1, config.head_dim, config.rope_theta)
        self.cos_table, self.sin_table = self._tensor(cosine), self._tensor(sine)

    def _workspace(self) -> None:
        config, batch = self.config, self.batch
        hidden, dim = config.hidden, config.head_dim
        self.token_ids = self._empty((batch,), "int64", 8)
        self.out_tokens = self._empty((batch,), "int32", 4)
        self.hidden_a = self._empty((batch, hidden))
        self.hidden_b = self._empty((batch, hidden))
        self.normed = self._empty((batch, hidden))
        self.q = self._empty((batch, config.query_heads * dim))
        self.k = self._empty((batch, config.kv_heads * dim))
        self.v = self._empty((batch, config.kv_heads * dim))
        self.q_rot = self._empty((batch, config.query_heads, 1, dim))
        self.k_rot = self._empty((batch, config.kv_heads, 1, dim))
        self.attended = self._empty((batch, config.query_heads * dim))
        self.product = self._empty((batch, config.intermediate))
        self.cos_row = self._empty((1, 1, dim))
        self.sin_row = self._empty((1, 1, dim))
        self.new_slots = self._empty((batch,), "uint32", 4)
        if config.conv_layers:
            self.in_proj = self._empty((batch, 3 * hidden))
            self.conv_out = self._empty((batch, hidden))
            self.conv_states = [self._empty((batch, hidden, 3)) for _ in range(config.conv_layers)]
        # slot(b, position) = b * capacity + position: [batch, capacity] for reads,
        # its transpose [capacity, batch] so one row holds the new slot of every sequence
        table = (np.arange(batch, dtype=np.uint32)[:, None] * self.capacity
                 + np.arange(self.capacity, dtype=np.uint32)[None, :])
        self.slot_table = self._tensor(table, "uint32")
        self.slot_table_by_position = self._tensor(np.ascontiguousarray(table.T), "uint32")

    # ---- the per-token record list ----------------------------------------------------------
    def build(self, past_tokens: int = 0) -> None:
        config, batch, runtime = self.config, self.batch, self.runtime
        hidden, dim = config.hidden, config.head_dim
        commands = Batch(runtime)
        context = dispatch.Context(runtime, batch=commands, decode_uniforms_past_tokens=past_tokens)
        run = lambda name, buffers, params, grid=(256, 1, 1): commands.dispatch(
            name=name, buffers=buffers, parameters=params, grid=grid, group=(256, 1, 1))
        run("llmopt_embedding_f16", [self.token_ids.buffer, self.embedding.buffer, self.hidden_a.buffer],
            parameters.embedding(tokens=batch, vocabulary=self.full_vocabulary, width=hidden), (batch * hidden, 1, 1))
        group = self.group
        exchange = 0  # index of the next exchange of this step (slots are assigned round-robin)
        if group is not None:
            from .tensor_parallel import CANDIDATE_PARTS, plan_slots

            exchanges = 2 * len(config.layers) + (batch + 31) // 32
            slot_count, slot_of = plan_slots(exchanges)
            self._decode_slots = list(slot_of)
            if slot_count > group.slot_count or max(batch * hidden * 4, min(batch, 32) * CANDIDATE_PARTS * 8) > group.slot_bytes:
                raise ValueError("the exchange group's slots are too few or too small for this plan")

        def row_split_linear(source, weight, scale, k_local, residual, output, norm=None):
            """x[:, K slice] . W[:, K slice]^T as an fp32 partial into this rank's slot, then the
            exchange that adds all ranks' partial sums and the residual.  ``norm`` = (weight,
            weight_first): the exchange also writes the RMS-normalised result into ``self.normed``,
            replacing the norm kernel that would follow."""
            nonlocal exchange
            slot = slot_of[exchange]
            exchange += 1
            run("llmopt_w4a16_linear_partial_f32_g64",
                [source.buffer, weight.buffer, scale.buffer, group.slot_view(slot, batch * hidden * 4)],
                parameters.u32s([batch, hidden, k_local]))
            if norm is None or hidden > 8192:
                group.sum_record(commands.dispatch, slot=slot, rows=batch, width=hidden, residual=residual.buffer,
                                 output=output.buffer)
                return False
            group.sum_norm_record(commands.dispatch, slot=slot, rows=batch, width=hidden, residual=residual.buffer,
                                  output=output.buffer, norm_weight=norm[0].buffer, normalized=self.normed.buffer,
                                  epsilon=config.epsilon, weight_first=norm[1])
            return True

        normed_ready = False  # self.normed already holds this layer's normalised input
        current, other = self.hidden_a, self.hidden_b
        attention_index = conv_index = 0
        for layer_index, (kind, layer) in enumerate(zip(config.layers, self.layers)):
            if not normed_ready:
                run("llmopt_rms_norm_f16_simd", [current.buffer, layer["input_norm"].buffer, self.normed.buffer],
                    parameters.rms_norm(rows=batch, width=hidden, epsilon=config.epsilon),
                    (dispatch.simd_rows_grid(batch), 1, 1))
            normed_ready = False
            if kind == "attention":
                dispatch.dispatch_w4a16_qkv_linear_command(
                    context, input=self.normed, q_weight=layer["q"][0], q_scale=layer["q"][1], k_weight=layer["k"][0],
                    k_scale=layer["k"][1], v_weight=layer["v"][0], v_scale=layer["v"][1], q_output=self.q,
                    k_output=self.k, v_output=self.v)
                run("llmopt_rotary_qk_f16_simd_h64",
                    [self.q.buffer, self.k.buffer, self.cos_row.buffer, self.sin_row.buffer, self.q_rot.buffer,
                     self.k_rot.buffer],
                    parameters.rotary_qk(batches=batch, tokens=1, q_heads=config.query_heads, k_heads=config.kv_heads,
                                         width=dim, half_dimension=dim // 2, trig_batches=1),
                    (dispatch.simd_rows_grid(batch * (config.query_heads + config.kv_heads)), 1, 1))
                region = self.layout.attentions[attention_index]
                paged = dispatch.PagedAttentionConfig(
                    token_elements=self.layout.token_elements, key_offset=region.key_offset,
                    value_offset=region.value_offset, group_size=self.layout.group_size,
                    token_stride=self.layout.bytes_per_token, scale=float(np.float32(1.0 / math.sqrt(dim))))
                # Q8 pack of the new token: one item per sequence; a sequence's K (or V)
                # row is kv_heads * D contiguous halves, packed as one "head" of that width
                # (recorded before the attention, which reads only the slots of the past tokens and takes the
                # new token from k_rot / v: a plan runs the rotary and this pack as one kernel)
                pack = parameters.cache_attention_pair(
                    items=batch, key_segment_offset=region.key_offset, value_segment_offset=region.value_offset,
                    heads=1, head_dim=config.kv_heads * dim, group_size=self.layout.group_size,
                    token_elements=self.layout.token_elements, token_groups=self.layout.token_groups,
                    token_stride=self.layout.bytes_per_token, source_items=batch, source_offset=0)
                groups = batch * config.kv_heads * dim // self.layout.group_size
                run("llmopt_cache_pack_attention_q8_pair_simd",
                    [self.k_rot.buffer, self.v.buffer, self.new_slots.buffer, self.cache.token_pool], pack,
                    (dispatch.round_up(groups, 8) * 32, 1, 1))
                value_now = dispatch.Tensor(self.v.buffer, (batch, config.kv_heads, 1, dim))
                attended = dispatch.Tensor(self.attended.buffer, (batch, 1, config.query_heads, dim))
                if batch == 1:
                    slots = dispatch.Tensor(self.slot_table.buffer, (self.capacity,), "uint32")
                    dispatch.dispatch_paged_attention_q8(
                        context, config=paged, query=self.q_rot, current_key=self.k_rot, current_value=value_now,
                        pool=dispatch.Tensor(self.cache.token_pool, (0,), "uint8"), slots=slots, output=attended)
                else:
                    dispatch.dispatch_paged_attention_q8(
                        context, config=paged, query=self.q_rot, current_key=self.k_rot, current_value=value_now,
                        pool=dispatch.Tensor(self.cache.token_pool, (0,), "uint8"), slots=self.slot_table,
                        output=attended, slot_batch_stride=self.capacity)
                if group is None:
                    dispatch.dispatch_w4a16_linear(context, input=self.attended, weight=layer["o"][0],
                                                   scale=layer["o"][1], output=other, bias=current,
                                                   bias_row_stride=hidden)
                else:
                    ffn_normed = row_split_linear(self.attended, layer["o"][0], layer["o"][1],
                                                  config.query_heads * dim, current, other,
                                                  norm=(layer["ffn_norm"], True))
                attention_index += 1
            else:
                dispatch.dispatch_w4a16_linear(context, input=self.normed, weight=layer["in_proj"][0],
                                               scale=layer["in_proj"][1], output=self.in_proj)
                state = self.conv_states[conv_index]
                for b in range(batch):  # the step kernel carries one sequence (lib/metal_recurrent_source.ml:151)
                    dispatch.dispatch_short_conv_step(
                        context,
                        in_proj=dispatch.Tensor(self.in_proj.buffer.view(b * 6 * hidden, 6 * hidden), (1, 1, 3 * hidden)),
                        conv_state=dispatch.Tensor(state.buffer.view(b * 6 * hidden, 6 * hidden), (1, hidden, 3)),
                        conv_weight=layer["conv"],
                        output=dispatch.Tensor(self.conv_out.buffer.view(b * 2 * hidden, 2 * hidden), (1, 1, hidden)))
                dispatch.dispatch_w4a16_linear(context, input=self.conv_out, weight=layer["out_proj"][0],
                                               scale=layer["out_proj"][1], output=other, bias=current,
                                               bias_row_stride=hidden)
                conv_index += 1
            current, other = other, current
            if group is None:
                dispatch.dispatch_w4a16_swiglu_ffn_command(
                    context, m=batch, n=config.intermediate, k=hidden, epsilon=config.epsilon, activation=current,
                    residual=current, gate_weight=layer["gate"][0], gate_scale=layer["gate"][1],
                    up_weight=layer["up"][0], up_scale=layer["up"][1], down_weight=layer["down"][0],
                    down_scale=layer["down"][1], norm_weight=layer["ffn_norm"], output=other, reference_guards=False)
            else:
                # the same three kernels on this rank's intermediate columns; the down projection is
                # the row-split product
                ffn = parameters.w4a16_swiglu_ffn(m=batch, n=config.intermediate, k=hidden, epsilon=config.epsilon)
                if not (kind == "attention" and ffn_normed):
                    run("llmopt_w4a16_swiglu_rms_f16_g64",
                        [current.buffer, layer["ffn_norm"].buffer, self.normed.buffer], ffn, (batch * 256, 1, 1))
                run("llmopt_w4a16_dual_swiglu_f16_g64" + ("" if batch == 1 else "_m4"),
                    [self.normed.buffer, layer["gate"][0].buffer, layer["gate"][1].buffer, layer["up"][0].buffer,
                     layer["up"][1].buffer, self.product.buffer], ffn)
                following = self.layers[layer_index + 1] if layer_index + 1 < len(self.layers) else None
                normed_ready = row_split_linear(
                    self.product, layer["down"][0], layer["down"][1], config.intermediate, current, other,
                    norm=None if following is None else (following["input_norm"], False))
            current, other = other, current
        for row0 in range(0, batch, 32):  # the LM head takes at most 32 rows per dispatch
            rows = min(32, batch - row0)
            if group is not None:
                slot = slot_of[exchange]
                exchange += 1
                run("llmopt_w4a16_lm_head_argmax_stage1_f16",
                    [current.buffer.view(row0 * hidden * 2, rows * hidden * 2), self.final_norm.buffer,
                     self.lm_head[0].buffer, self.lm_head[1].buffer, group.slot_view(slot, rows * CANDIDATE_PARTS * 8)],
                    parameters.w4a16_lm_head_argmax(m=rows, n=config.vocabulary, k=hidden, epsilon=config.epsilon),
                    (256 * 256, rows, 1))
                group.argmax_record(commands.dispatch, slot=slot, rows=rows, shard_columns=config.vocabulary,
                                    output=self.out_tokens.buffer.view(row0 * 4, rows * 4))
                continue
            dispatch.dispatch_w4a16_lm_head_argmax_command(
                context, m=rows, n=config.vocabulary, k=hidden, epsilon=config.epsilon,
                input=dispatch.Tensor(current.buffer.view(row0 * hidden * 2, rows * hidden * 2), (rows, hidden)),
                norm_weight=self.final_norm, weight=self.lm_head[0], scale=self.lm_head[1],
                output=dispatch.Tensor(self.out_tokens.buffer.view(row0 * 4, rows * 4), (rows,), "int32"),
                reference_guards=False, two_stage=False)
        if batch == 1:
            run("llmopt_chain_token_id", [self.out_tokens.buffer, self.token_ids.buffer], b"", (32, 1, 1))
        else:
            run("llmopt_chain_token_ids", [self.out_tokens.buffer, self.token_ids.buffer], parameters.u32s([batch]),
                (batch, 1, 1))
        self.records = list(commands.pending)
        self.final_hidden = current  # [batch, hidden] f16: the last block's output, input of the LM head
        self._context = context
        commands.abort()
        row = self.config.head_dim * 2
        self.plan = Prebaked(runtime, self.records, self.token_ids.buffer, self.out_tokens.buffer, row_bindings=[
            (self.cos_row.buffer, self.cos_table.buffer, row), (self.sin_row.buffer, self.sin_table.buffer, row),
            (self.new_slots.buffer, self.slot_table_by_position.buffer, 4 * self.batch)])

    # ---- prefill ---------------------------------------------------------------------------------
    def prefill(self, tokens: Sequence[int], sequence: int = 0) -> int:
        """The whole prompt of one sequence in one pass — the reference's prefill path
        (``Serving_engine.prefill``, lib/serving_engine.ml:435-570): every linear runs with one row
        per prompt token (the tcgen05 kernels from 17 rows on), attention is the dense causal
        fp16 attention over the prompt's own keys and values, every token's K / V row is packed
        into the Q8 cache (``Cache.with_batch_async``, lib/metal_cache.ml:93-116) and the
        short-conv blocks leave their state behind.  Returns the first generated token; decode
        continues with ``step(..., past_tokens=len(tokens))``.  A sequence is prefilled from an
        empty cache (position 0)."""
        config, runtime = self.config, self.runtime
        group = self.group
        started = time.perf_counter()
        count, hidden, dim = len(tokens), config.hidden, config.head_dim
        if count == 0 or count > self.capacity:
            raise ValueError("the prompt must hold 1 .. capacity tokens")
        if not 0 <= sequence < self.batch:
            raise ValueError("no such sequence")
        if group is not None:
            # Tensor-parallel shard: the same pass over this rank's heads and columns; o_proj and down are
            # row splits whose fp32 partial sums (one slot of rows x hidden floats each) are added in rank order by a
            # reduce-scatter exchange and an all-gather exchange (a second slot carries the fp16 shares).
            # Slots alternate like a decode step's: never the same in adjacent exchanges, the first not
            # the decode step's last, the last not its first.  No exchange of an earlier step may still be in
            # flight on any rank when the prompt starts (true once every rank has read that step's token).
            if count * hidden * 4 > group.slot_bytes:
                raise ValueError("the exchange slots are smaller than rows x hidden fp32 partial sums of this prompt")
            from .tensor_parallel import plan_prompt_slots

            exchanges = 4 * len(config.layers) + 1  # a reduce and a gather exchange per row split, the argmax
            slot_sequence = plan_prompt_slots(group.slot_count, exchanges, getattr(self, "_decode_slots", None) or [0])
        # A prompt of a length (and sequence) seen before replays the list recorded then: only the ids change
        plans = self.__dict__.setdefault("_prefill_plans", {})
        plan = plans.get((count, sequence))
        if plan is not None:
            plan["ids"].buffer.write(0, np.asarray(tokens, np.int64))
            commands = Batch(runtime)
            commands.dispatch_recorded(plan["records"])
            self.prefill_kernels, self.prefill_hidden = plan["kernels"], plan["hidden"]
            recorded = time.perf_counter()
            commands.commit()
            token = int(plan["picked"].buffer.to_numpy(np.int32)[0])
            self.prefill_seconds = (recorded - started, time.perf_counter() - recorded)
            return token
        exchange = 0
        commands = Batch(runtime)
        context = dispatch.Context(runtime, batch=commands)
        run = lambda name, buffers, params, grid=(256, 1, 1): commands.dispatch(
            name=name, buffers=buffers, parameters=params, grid=grid, group=(256, 1, 1))
        ids = self._tensor(np.asarray(tokens, np.int64), "int64")
        current, other = self._empty((count, hidden)), self._empty((count, hidden))
        normed = self._empty((count, hidden))
        q = self._empty((count, config.query_heads * dim))
        k = self._empty((count, config.kv_heads * dim))
        v = self._empty((count, config.kv_heads * dim))
        q_rot = self._empty((1, config.query_heads, count, dim))
        k_rot = self._empty((1, config.kv_heads, count, dim))
        attended = self._empty((1, count, config.query_heads * dim))
        row = dim * 2
        cosine = dispatch.Tensor(self.cos_table.buffer.view(0, count * row), (1, count, dim))
        sine = dispatch.Tensor(self.sin_table.buffer.view(0, count * row), (1, count, dim))
        slots = self.slot_table.buffer.view(sequence * self.capacity * 4, count * 4)
        run("llmopt_embedding_f16", [ids.buffer, self.embedding.buffer, current.buffer],
            parameters.embedding(tokens=count, vocabulary=self.full_vocabulary, width=hidden), (count * hidden, 1, 1))
        attention_index = conv_index = 0
        for kind, layer in zip(config.layers, self.layers):
            run("llmopt_rms_norm_f16_simd", [current.buffer, layer["input_norm"].buffer, normed.buffer],
                parameters.rms_norm(rows=count, width=hidden, epsilon=config.epsilon),
                (dispatch.simd_rows_grid(count), 1, 1))
            if kind == "attention":
                dispatch.dispatch_w4a16_qkv_linear_command(
                    context, input=normed, q_weight=layer["q"][0], q_scale=layer["q"][1], k_weight=layer["k"][0],
                    k_scale=layer["k"][1], v_weight=layer["v"][0], v_scale=layer["v"][1], q_output=q, k_output=k,
                    v_output=v)
                run("llmopt_rotary_qk_f16_simd_h64",
                    [q.buffer, k.buffer, cosine.buffer, sine.buffer, q_rot.buffer, k_rot.buffer],
                    parameters.rotary_qk(batches=1, tokens=count, q_heads=config.query_heads, k_heads=config.kv_heads,
                                         width=dim, half_dimension=dim // 2, trig_batches=1),
                    (dispatch.simd_rows_grid(count * (config.query_heads + config.kv_heads)), 1, 1))
                dispatch.dispatch_attention(
                    context, causal=True, scale=float(np.float32(1.0 / math.sqrt(dim))), query=q_rot, key=k_rot,
                    value=dispatch.Tensor(v.buffer, (1, count, config.kv_heads, dim)), output=attended)
                region = self.layout.attentions[attention_index]
                common = dict(items=count, group_size=self.layout.group_size, token_elements=self.layout.token_elements,
                              token_groups=self.layout.token_groups, token_stride=self.layout.bytes_per_token,
                              source_items=count, source_offset=0)
                # K rows are head-major [kv_heads, T, D]; a V row is kv_heads * D contiguous halves per token
                for source, segment, heads, width in ((k_rot, region.key_offset, config.kv_heads, dim),
                                                      (v, region.value_offset, 1, config.kv_heads * dim)):
                    groups = count * heads * width // self.layout.group_size
                    run("llmopt_cache_pack_attention_q8_simd", [source.buffer, slots, self.cache.token_pool],
                        parameters.cache_attention(segment_offset=segment, heads=heads, head_dim=width, **common),
                        (dispatch.round_up(groups, 8) * 32, 1, 1))
                if group is None:
                    dispatch.dispatch_w4a16_linear(
                        context, input=dispatch.Tensor(attended.buffer, (count, config.query_heads * dim)),
                        weight=layer["o"][0], scale=layer["o"][1], output=other, bias=current, bias_row_stride=hidden)
                else:
                    slot, slice_slot = slot_sequence[exchange], slot_sequence[exchange + 1]
                    exchange += 2
                    run("llmopt_w4a16_linear_partial_f32_g64",
                        [attended.buffer, layer["o"][0].buffer, layer["o"][1].buffer, group.slot_view(slot, count * hidden * 4)],
                        parameters.u32s([count, hidden, config.query_heads * dim]))
                    group.sum_rows_records(commands.dispatch, slot=slot, slice_slot=slice_slot, rows=count, width=hidden,
                                           residual=current.buffer, output=other.buffer)
                attention_index += 1
            else:
                in_proj = self._empty((1, count, 3 * hidden))
                conv_out = self._empty((1, count, hidden))
                dispatch.dispatch_w4a16_linear(context, input=normed, weight=layer["in_proj"][0],
                                               scale=layer["in_proj"][1],
                                               output=dispatch.Tensor(in_proj.buffer, (count, 3 * hidden)))
                state = self.conv_states[conv_index]
                dispatch.dispatch_short_conv_prefill(
                    context, in_proj=in_proj, conv_weight=layer["conv"], output=conv_out,
                    conv_state_out=dispatch.Tensor(state.buffer.view(sequence * 6 * hidden, 6 * hidden), (1, hidden, 3)))
                dispatch.dispatch_w4a16_linear(
                    context, input=dispatch.Tensor(conv_out.buffer, (count, hidden)), weight=layer["out_proj"][0],
                    scale=layer["out_proj"][1], output=other, bias=current, bias_row_stride=hidden)
                conv_index += 1
            current, other = other, current
            if group is None:
                dispatch.dispatch_w4a16_swiglu_ffn_command(
                    context, m=count, n=config.intermediate, k=hidden, epsilon=config.epsilon, activation=current,
                    residual=current, gate_weight=layer["gate"][0], gate_scale=layer["gate"][1], up_weight=layer["up"][0],
                    up_scale=layer["up"][1], down_weight=layer["down"][0], down_scale=layer["down"][1],
                    norm_weight=layer["ffn_norm"], output=other, reference_guards=False)
            else:
                # the same three kernels on this rank's intermediate columns; the down projection is the row split
                ffn = parameters.w4a16_swiglu_ffn(m=count, n=config.intermediate, k=hidden, epsilon=config.epsilon)
                product = self._empty((count, config.intermediate))
                run("llmopt_w4a16_swiglu_rms_f16_g64", [current.buffer, layer["ffn_norm"].buffer, normed.buffer], ffn,
                    (count * 256, 1, 1))
                run("llmopt_w4a16_dual_swiglu_f16_g64_m4",
                    [normed.buffer, layer["gate"][0].buffer, layer["gate"][1].buffer, layer["up"][0].buffer,
                     layer["up"][1].buffer, product.buffer], ffn)
                slot, slice_slot = slot_sequence[exchange], slot_sequence[exchange + 1]
                exchange += 2
                run("llmopt_w4a16_linear_partial_f32_g64",
                    [product.buffer, layer["down"][0].buffer, layer["down"][1].buffer, group.slot_view(slot, count * hidden * 4)],
                    parameters.u32s([count, hidden, config.intermediate]))
                group.sum_rows_records(commands.dispatch, slot=slot, slice_slot=slice_slot, rows=count, width=hidden,
                                       residual=current.buffer, output=other.buffer)
            current, other = other, current
        picked = self._empty((1,), "int32", 4)
        last = current.buffer.view((count - 1) * hidden * 2, hidden * 2)
        if group is None:
            dispatch.dispatch_w4a16_lm_head_argmax_command(
                context, m=1, n=config.vocabulary, k=hidden, epsilon=config.epsilon, input=dispatch.Tensor(last, (1, hidden)),
                norm_weight=self.final_norm, weight=self.lm_head[0], scale=self.lm_head[1], output=picked,
                reference_guards=False, two_stage=False)
        else:
            from .tensor_parallel import CANDIDATE_PARTS

            slot = slot_sequence[exchange]
            exchange += 1
            run("llmopt_w4a16_lm_head_argmax_stage1_f16",
                [last, self.final_norm.buffer, self.lm_head[0].buffer, self.lm_head[1].buffer,
                 group.slot_view(slot, CANDIDATE_PARTS * 8)],
                parameters.w4a16_lm_head_argmax(m=1, n=config.vocabulary, k=hidden, epsilon=config.epsilon), (256 * 256, 1, 1))
            group.argmax_record(commands.dispatch, slot=slot, rows=1, shard_columns=config.vocabulary, output=picked.buffer)
        self.prefill_kernels = len(commands.pending)
        self.prefill_hidden = current  # rows of the last block's output, one per prompt token
        records = pack_records(commands.pending)  # keeps every buffer of the pass alive with the plan
        commands.pending = []
        commands.dispatch_recorded(records)
        while len(plans) >= 2:  # two lengths at most: a plan holds the pass's activations
            plans.pop(next(iter(plans)))
        plans[(count, sequence)] = {"records": records, "ids": ids, "picked": picked, "hidden": current,
                                    "kernels": self.prefill_kernels}
        recorded = time.perf_counter()
        commands.commit()
        token = int(picked.buffer.to_numpy(np.int32)[0])
        # host seconds spent recording the dispatches / executing them (commit until the token is back)
        self.prefill_seconds = (recorded - started, time.perf_counter() - recorded)
        return token

    # ---- stepping ------------------------------------------------------------------------------
    def step(self, tokens: Sequence[int], past_tokens: int) -> list:
        """One host-driven decode step: token ids in, next token ids out (the
        ``Prebaked.execute`` round trip, one per token)."""
        if self.plan is None:
            self.build(past_tokens)
        if len(tokens) != self.batch:
            raise ValueError("one token per sequence is required")
        if past_tokens >= self.capacity:
            raise ValueError("the cache capacity is exhausted")
        if self.batch > 1:
            self.token_ids.buffer.write(0, np.asarray(tokens, np.int64))
        first = self.plan.execute(token=int(tokens[0]), past_tokens=past_tokens)
        if self.batch == 1:
            return [first]
        return self.out_tokens.buffer.to_numpy(np.int32).tolist()

    def generate_chained(self, tokens: Sequence[int], past_tokens: int, steps: int):
        """``steps`` device-chained greedy steps; returns (ids of sequence 0, device ms)."""
        if self.plan is None:
            self.build(past_tokens)
        if past_tokens + steps > self.capacity:
            raise ValueError("the cache capacity is exhausted")
        if self.batch > 1:
            self.token_ids.buffer.write(0, np.asarray(tokens, np.int64))
        return self.plan.execute_chained(token=int(tokens[0]), past_tokens=past_tokens, steps=steps)

    def fill_cache_random(self, past_tokens: int, seed: int = 0) -> None:
        """Pre-fills every sequence's first ``past_tokens`` slots with random int8
        payload and valid fp16 scales (a context that was never computed)."""
        rng = np.random.default_rng(seed)
        stride, elements = self.layout.bytes_per_token, self.layout.token_elements
        block = np.zeros((past_tokens, stride), np.uint8)
        block[:, :elements] = rng.integers(-127, 128, size=(past_tokens, elements), dtype=np.int8).view(np.uint8)
        scales = rng.uniform(0.004, 0.02, size=(past_tokens, (stride - elements) // 2)).astype(np.float16)
        block[:, elements:] = scales.view(np.uint8).reshape(past_tokens, -1)
        first = self.cache.token_pool.view(0, past_tokens * stride)
        first.write(0, block)
        for b in range(1, self.batch):
            first.copy_to(self.cache.token_pool.view(b * self.capacity * stride, past_tokens * stride))
        self.runtime.synchronize()
