"""CPU restatement of one decode step over the oracle's per-op functions: the
same op sequence and rounding points as the GPU plan (test infrastructure)."""

import math

import numpy as np

from llmopt_b200.kv_cache import AttentionLayer, Layout
from llmopt_b200.quantize import rope_tables
from oracle import oracle as orc


class OracleDecoder:
    def __init__(self, config, weights, capacity):
        self.config, self.weights, self.capacity = config, weights, capacity
        self.layout = Layout([AttentionLayer(config.kv_heads, config.head_dim)] * config.attention_layers,
                             group_size=config.kv_group_size)
        self.pool = np.zeros(capacity * self.layout.bytes_per_token, np.uint8)
        self.cos, self.sin = rope_tables(capacity + 1, config.head_dim, config.rope_theta)
        self.conv_states = [np.zeros((config.hidden, 3), np.float16) for _ in range(config.conv_layers)]
        self.past = 0

    def step(self, token, want_logits=False):
        config, weights, layout = self.config, self.weights, self.layout
        hidden, dim = config.hidden, config.head_dim
        h = orc.embedding_f16([token], weights["embedding"])
        slots = np.arange(max(self.past, 1), dtype=np.uint32)
        attention_index = conv_index = 0
        for index, kind in enumerate(config.layers):
            layer = weights[f"layer{index}"]
            xn = orc.rms_norm(h, layer["input_norm"], config.epsilon)
            if kind == "attention":
                q, k, v = orc.w4a16_qkv_linear(xn, *layer["q"], *layer["k"], *layer["v"])
                q_rot, k_rot = orc.rotary_qk(q.reshape(1, 1, config.query_heads, dim), k.reshape(1, 1, config.kv_heads, dim),
                                             self.cos[self.past][None, None, :], self.sin[self.past][None, None, :],
                                             half_dimension=dim // 2)
                region = layout.attentions[attention_index]
                params = orc.paged_params_bytes(
                    batches=1, query_heads=config.query_heads, kv_heads=config.kv_heads, past_length=self.past,
                    head_dim=dim, token_elements=layout.token_elements, key_offset=region.key_offset,
                    value_offset=region.value_offset, group_size=layout.group_size,
                    token_stride=layout.bytes_per_token, scale=float(np.float32(1.0 / math.sqrt(dim))))
                attended = orc.attention_q8_paged(q_rot, k_rot, v.reshape(1, config.kv_heads, 1, dim), self.pool, slots,
                                                  None, params)
                for segment, source in ((region.key_offset, k_rot), (region.value_offset, v)):
                    orc.cache_pack_attention_q8(source.reshape(config.kv_heads, 1, dim), [self.past], self.pool,
                                                segment_offset=segment, heads=config.kv_heads, head_dim=dim,
                                                group_size=layout.group_size, token_elements=layout.token_elements,
                                                token_stride=layout.bytes_per_token, source_items=1)
                h = orc.w4a16_linear(attended.reshape(1, -1), *layer["o"], bias=h, bias_row_stride=hidden)
                attention_index += 1
            else:
                in_proj = orc.w4a16_linear(xn, *layer["in_proj"])
                out, self.conv_states[conv_index] = orc.short_conv_step(in_proj, self.conv_states[conv_index],
                                                                       layer["conv"].reshape(hidden, 3))
                h = orc.w4a16_linear(out.reshape(1, -1), *layer["out_proj"], bias=h, bias_row_stride=hidden)
                conv_index += 1
            h, _, _ = orc.w4a16_swiglu_ffn(h, h, *layer["gate"], *layer["up"], *layer["down"], layer["ffn_norm"],
                                           config.epsilon)
        tokens, logits, best = orc.w4a16_lm_head_argmax(h, weights["final_norm"], *weights["lm_head"], config.epsilon,
                                                        want_logits=want_logits)
        self.past += 1
        return int(tokens[0]), logits
