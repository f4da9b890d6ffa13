"""CPU restatement of the decode path over the oracle's per-op functions: the same
op sequence and rounding points as the GPU plan (test infrastructure).

``OracleDecoder.forward`` takes any set of (sequence, token) rows.  Every per-row
operation (norm, W4A16 products, rotary, short conv) is independent per row, and
the attention of a row reads the Q8 cache slots of the tokens before it in its own
sequence plus its own fp16 key / value, exactly as one decode step does.  Running a
layer for all rows before the next layer only reorders independent work, so feeding
a prompt in one call, token by token, or several sequences side by side gives the
same state and the same picks bit for bit; the weights of a layer are decoded once
per call instead of once per token."""

import math

import numpy as np

from llmopt_b200.kv_cache import AttentionLayer, Layout
from llmopt_b200.quantize import rope_tables
from oracle import oracle as orc


class OracleDecoder:
    def __init__(self, config, weights, capacity, sequences=1):
        self.config, self.weights, self.capacity = config, weights, capacity
        self.layout = Layout([AttentionLayer(config.kv_heads, config.head_dim)] * config.attention_layers,
                             group_size=config.kv_group_size)
        self.pools = [np.zeros(capacity * self.layout.bytes_per_token, np.uint8) for _ in range(sequences)]
        self.cos, self.sin = rope_tables(capacity + 1, config.head_dim, config.rope_theta)
        self.conv_states = [[np.zeros((config.hidden, 3), np.float16) for _ in range(config.conv_layers)]
                            for _ in range(sequences)]
        self.pasts = [0] * sequences

    # single-sequence views, kept for callers that hold one sequence
    @property
    def pool(self):
        return self.pools[0]

    @property
    def past(self):
        return self.pasts[0]

    def forward(self, rows, emit, want_logits=False):
        """``rows``: list of (sequence, token), consumed in order (a sequence's rows take
        consecutive positions).  ``emit``: row indices whose next-token pick is wanted.
        Returns (picks, logits [len(emit), vocabulary] or None)."""
        config, weights, layout = self.config, self.weights, self.layout
        hidden, dim = config.hidden, config.head_dim
        count = len(rows)
        positions, cursor = [], list(self.pasts)
        for sequence, _ in rows:
            positions.append(cursor[sequence])
            cursor[sequence] += 1
        h = orc.embedding_f16([int(token) for _, token in rows], weights["embedding"])
        attention_index = conv_index = 0
        for index, kind in enumerate(config.layers):
            layer = weights[f"layer{index}"]
            xn = orc.rms_norm(h, layer["input_norm"], config.epsilon)
            if kind == "attention":
                q, k, v = orc.w4a16_qkv_linear(xn, *layer["q"], *layer["k"], *layer["v"])
                q_rot, k_rot = orc.rotary_qk(q.reshape(1, count, config.query_heads, dim),
                                             k.reshape(1, count, config.kv_heads, dim),
                                             self.cos[positions][None], self.sin[positions][None],
                                             half_dimension=dim // 2)
                region = layout.attentions[attention_index]
                v_heads = np.ascontiguousarray(v.reshape(count, config.kv_heads, dim).transpose(1, 0, 2))
                for row, (sequence, _) in enumerate(rows):  # the new tokens' cache rows first ...
                    for segment, source in ((region.key_offset, k_rot[0][:, row:row + 1]),
                                            (region.value_offset, v_heads[:, row:row + 1])):
                        orc.cache_pack_attention_q8(np.ascontiguousarray(source), [positions[row]], self.pools[sequence],
                                                    segment_offset=segment, heads=config.kv_heads, head_dim=dim,
                                                    group_size=layout.group_size, token_elements=layout.token_elements,
                                                    token_stride=layout.bytes_per_token, source_items=1)
                attended = np.empty((count, config.query_heads * dim), np.float16)
                for row, (sequence, _) in enumerate(rows):  # ... then every row over the slots before its own
                    past = positions[row]
                    params = orc.paged_params_bytes(
                        batches=1, query_heads=config.query_heads, kv_heads=config.kv_heads, past_length=past,
                        head_dim=dim, token_elements=layout.token_elements, key_offset=region.key_offset,
                        value_offset=region.value_offset, group_size=layout.group_size,
                        token_stride=layout.bytes_per_token, scale=float(np.float32(1.0 / math.sqrt(dim))))
                    out = orc.attention_q8_paged(
                        np.ascontiguousarray(q_rot[:, :, row:row + 1]), np.ascontiguousarray(k_rot[:, :, row:row + 1]),
                        np.ascontiguousarray(v_heads[None, :, row:row + 1]), self.pools[sequence],
                        np.arange(max(past, 1), dtype=np.uint32), None, params)
                    attended[row] = out.reshape(-1)
                h = orc.w4a16_linear(attended, *layer["o"], bias=h, bias_row_stride=hidden)
                attention_index += 1
            else:
                in_proj = orc.w4a16_linear(xn, *layer["in_proj"])
                out = np.empty((count, hidden), np.float16)
                for row, (sequence, _) in enumerate(rows):  # the step kernel's rounding points, token after token
                    out[row], self.conv_states[sequence][conv_index] = orc.short_conv_step(
                        in_proj[row], self.conv_states[sequence][conv_index], layer["conv"].reshape(hidden, 3))
                h = orc.w4a16_linear(out, *layer["out_proj"], bias=h, bias_row_stride=hidden)
                conv_index += 1
            h, _, _ = orc.w4a16_swiglu_ffn(h, h, *layer["gate"], *layer["up"], *layer["down"], layer["ffn_norm"],
                                           config.epsilon)
        self.pasts = cursor
        self.last_hidden = h  # [rows, hidden] f16: the last block's output of this call
        if not emit:
            return [], None
        picks, logits, _ = orc.w4a16_lm_head_argmax(np.ascontiguousarray(h[list(emit)]), weights["final_norm"],
                                                    *weights["lm_head"], config.epsilon, want_logits=want_logits)
        return [int(pick) for pick in picks], logits

    def prefill_dense(self, tokens, want_logits=False, sequence=0):
        """The reference's prefill path for one sequence starting at position 0: dense causal fp16
        attention over the prompt's own rotated keys and values (nothing is read back from the Q8
        cache), the K / V of every token packed into the cache afterwards, the short-conv blocks
        through the prefill kernel's arithmetic.  Returns (pick after the last token, logits)."""
        config, weights, layout = self.config, self.weights, self.layout
        hidden, dim = config.hidden, config.head_dim
        if self.pasts[sequence] != 0:
            raise ValueError("dense prefill starts from an empty cache")
        count = len(tokens)
        h = orc.embedding_f16([int(t) for t in tokens], weights["embedding"])
        attention_index = conv_index = 0
        for index, kind in enumerate(config.layers):
            layer = weights[f"layer{index}"]
            xn = orc.rms_norm(h, layer["input_norm"], config.epsilon)
            if kind == "attention":
                q, k, v = orc.w4a16_qkv_linear(xn, *layer["q"], *layer["k"], *layer["v"])
                q_rot, k_rot = orc.rotary_qk(q.reshape(1, count, config.query_heads, dim),
                                             k.reshape(1, count, config.kv_heads, dim),
                                             self.cos[:count][None], self.sin[:count][None], half_dimension=dim // 2)
                v_heads = np.ascontiguousarray(v.reshape(1, count, config.kv_heads, dim).transpose(0, 2, 1, 3))
                attended = orc.attention_dense(q_rot, k_rot, v_heads, None, causal=1,
                                               scale=float(np.float32(1.0 / math.sqrt(dim))), kv_heads=config.kv_heads,
                                               token_first_output=1)
                region = layout.attentions[attention_index]
                new_slots = np.arange(count, dtype=np.uint32)
                for segment, source in ((region.key_offset, k_rot[0]), (region.value_offset, v_heads[0])):
                    orc.cache_pack_attention_q8(np.ascontiguousarray(source), new_slots, self.pools[sequence],
                                                segment_offset=segment, heads=config.kv_heads, head_dim=dim,
                                                group_size=layout.group_size, token_elements=layout.token_elements,
                                                token_stride=layout.bytes_per_token, source_items=count)
                h = orc.w4a16_linear(attended.reshape(count, -1), *layer["o"], bias=h, bias_row_stride=hidden)
                attention_index += 1
            else:
                in_proj = orc.w4a16_linear(xn, *layer["in_proj"])
                out, self.conv_states[sequence][conv_index] = orc.short_conv_prefill(
                    in_proj, layer["conv"].reshape(hidden, 3), None)
                h = orc.w4a16_linear(out, *layer["out_proj"], bias=h, bias_row_stride=hidden)
                conv_index += 1
            h, _, _ = orc.w4a16_swiglu_ffn(h, h, *layer["gate"], *layer["up"], *layer["down"], layer["ffn_norm"],
                                           config.epsilon)
        self.pasts[sequence] = count
        self.last_hidden = h
        picks, logits, _ = orc.w4a16_lm_head_argmax(np.ascontiguousarray(h[-1:]), weights["final_norm"],
                                                    *weights["lm_head"], config.epsilon, want_logits=want_logits)
        return int(picks[0]), logits

    def prefill(self, tokens, want_logits=False, sequence=0):
        """A whole prompt of one sequence in one call; returns (pick after its last token, logits)."""
        picks, logits = self.forward([(sequence, token) for token in tokens], [len(tokens) - 1], want_logits)
        return picks[0], logits

    def step(self, token, want_logits=False):
        picks, logits = self.forward([(0, token)], [0], want_logits)
        return picks[0], logits

    def step_all(self, tokens, want_logits=False):
        """One token for every sequence; returns (picks, logits)."""
        return self.forward(list(enumerate(tokens)), list(range(len(tokens))), want_logits)
