"""GPU parity of dense fp16 attention (prefill) against the float64 oracle, through the named dispatch."""

import numpy as np
import pytest

from conftest import assert_close_f16
from test_gpu_w4a16 import _ctx, _tensor

pytestmark = pytest.mark.gpu


def _attention(runtime, q, k, v, *, causal, scale, mask=None, token_first_output=False, mask_kind=None):
    from llmopt_b200 import dispatch

    b, h, ql, d = q.shape
    shape = (b, ql, h, d) if token_first_output else (b, h, ql, d)
    out = _tensor(runtime, np.full(shape, np.nan, np.float16))
    mask_tensor = None
    if mask is not None:
        mask_tensor = _tensor(runtime, mask, "bool" if mask_kind == "bool" else None)
    dispatch.dispatch_attention(_ctx(runtime), causal=causal, scale=scale, query=_tensor(runtime, q),
                                key=_tensor(runtime, k), value=_tensor(runtime, v), output=out, mask=mask_tensor)
    return out.buffer.to_numpy(np.float16, shape)


@pytest.mark.parametrize("b,h,kvh,ql,kl,d,causal,tfo,tfv", [
    (1, 3, 3, 8, 8, 64, True, True, False),        # the reference smoke's shape class (head-major in, token-first out)
    (2, 9, 3, 70, 70, 64, True, True, False),      # SmolLM2 head geometry, ragged query tile
    (1, 16, 8, 130, 130, 64, True, False, False),  # LFM attention geometry
    (1, 8, 2, 33, 97, 128, True, True, True),      # cached prefix (past = 64), token-first value
    (2, 4, 4, 40, 56, 128, False, False, False),   # no causal mask
    (1, 2, 1, 5, 5, 80, True, True, False),        # head size without a tensor-core specialisation
    (1, 2, 2, 3, 9, 40, False, False, True),
])
def test_dense_attention_matches_oracle(runtime, oracle, b, h, kvh, ql, kl, d, causal, tfo, tfv):
    rng = np.random.default_rng(20)
    q = rng.standard_normal((b, h, ql, d)).astype(np.float16)
    k = rng.standard_normal((b, kvh, kl, d)).astype(np.float16)
    v = rng.standard_normal((b, kl, kvh, d) if tfv else (b, kvh, kl, d)).astype(np.float16)
    scale = float(np.float32(1.0 / np.sqrt(d)))
    got = _attention(runtime, q, k, v, causal=causal, scale=scale, token_first_output=tfo)
    want = oracle.attention_dense(q, k, v, None, causal=int(causal), scale=scale, kv_heads=kvh,
                                  token_first_output=int(tfo), past_length=max(0, kl - ql), token_first_value=int(tfv))
    assert_close_f16(got, want, label=f"dense attention d={d} q={ql} k={kl}")


@pytest.mark.parametrize("kind", ["bool", "float16"])
def test_dense_attention_masks(runtime, oracle, kind):
    rng = np.random.default_rng(21)
    b, h, ql, kl, d = 2, 4, 37, 37, 64
    q = rng.standard_normal((b, h, ql, d)).astype(np.float16)
    k = rng.standard_normal((b, h, kl, d)).astype(np.float16)
    v = rng.standard_normal((b, h, kl, d)).astype(np.float16)
    keep = rng.random((b, 1, ql, kl)) > 0.3
    keep[0, 0, 5, :] = False  # a query that sees nothing writes zeros
    if kind == "bool":
        mask, dtype = keep.astype(np.uint8), 1
    else:
        mask, dtype = np.where(keep, 0.0, -np.inf).astype(np.float16), 2
    scale = 0.125
    got = _attention(runtime, q, k, v, causal=False, scale=scale, mask=mask, mask_kind=kind)
    want = oracle.attention_dense(q, k, v, mask, causal=0, scale=scale, kv_heads=h, mask_dtype=dtype, mask_batches=b,
                                  mask_heads=1)
    assert np.all(got[0, :, 5, :] == 0)
    assert_close_f16(got, want, label=f"dense attention mask {kind}")
