"""CPU tests of the host side: the C ABI library loads and exports every symbol
the header declares, parameter blocks are byte exact, the cache layout matches the
reference's numbers, and the dispatchers emit the reference's kernel names,
buffer order and grids (checked with a recording runtime; no GPU call is made)."""

import os
import re
import struct

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from llmopt_b200 import _build, cuda_native

    _build.build()
    header = open(os.path.join(ROOT, "include", "llmopt_cuda.h")).read()
    declared = set(re.findall(r"\b(llmopt_cuda_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 45
    lib = cuda_native.load_library()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(cuda_native.SIGNATURES), declared ^ set(cuda_native.SIGNATURES)
    assert lib.llmopt_cuda_last_error() == b""
    # pure host helper: first maximum wins (native/ocaml_metal_stubs.m:2565-2579)
    values = np.array([1.0, 3.0, 3.0, -2.0], np.float16)
    assert cuda_native.f16_argmax(values.tobytes(), 4) == 1
    assert cuda_native.f16_argmax(b"", 0) == 0


def test_parameter_blocks_are_byte_exact():
    from llmopt_b200 import parameters as p

    assert p.u32s([1, 2, 3]) == struct.pack("<3I", 1, 2, 3)
    with pytest.raises(ValueError, match="does not fit uint32"):
        p.u32s([-1])
    with pytest.raises(ValueError, match="does not fit uint32"):
        p.u32s([1 << 32])
    assert p.w4a16_linear(m=2, n=3, k=64, has_bias=True, bias_row_stride=3) == struct.pack("<5I", 2, 3, 64, 1, 3)
    assert p.rms_norm(rows=1, width=576, epsilon=1e-5) == struct.pack("<IIf", 1, 576, 1e-5)
    assert len(p.w4a16_swiglu_ffn(m=1, n=1536, k=576, epsilon=1e-5)) == 16
    block = p.paged_attention_q8(batches=1, query_heads=9, kv_heads=3, past_length=77, head_dimension=64,
                                 mask_batches=0, mask_heads=0, token_elements=128, key_offset=0, value_offset=64,
                                 group_size=64, token_stride=132, scale=0.125, mask_dtype=0)
    assert len(block) == 64 and struct.unpack_from("<I", block, 12)[0] == 77  # patched per token at byte 12
    assert struct.unpack_from("<f", block, 48)[0] == 0.125 and struct.unpack_from("<3I", block, 52) == (1, 0, 0)
    attention = p.attention(batches=1, heads=2, query_length=3, key_length=4, head_dimension=64, mask_batches=0,
                            mask_heads=0, causal=True, scale=0.5)
    assert len(attention) == 56 and struct.unpack_from("<I", attention, 36)[0] == 2  # kv_heads defaults to heads
    assert len(p.cache_attention(items=1, segment_offset=0, heads=1, head_dim=64, group_size=64, token_elements=128,
                                 token_groups=2, token_stride=132, source_items=1, source_offset=0)) == 40
    assert len(p.cache_attention_pair(items=1, key_segment_offset=0, value_segment_offset=64, heads=1, head_dim=64,
                                      group_size=64, token_elements=128, token_groups=2, token_stride=132,
                                      source_items=1, source_offset=0)) == 44
    checkpoint = p.cache_checkpoint(checkpoint=5, layer=1, layer_elements=3072, group_size=64,
                                    checkpoint_elements=30720, checkpoint_groups=480, checkpoint_stride=31680)
    assert len(checkpoint) == 28 and struct.unpack_from("<I", checkpoint, 0)[0] == 5
    assert p.embedding(tokens=1, vocabulary=10, width=4) == struct.pack("<3I", 1, 10, 4)


def test_cache_layout_matches_reference_numbers():
    from llmopt_b200.kv_cache import AttentionLayer, Layout, bytes_for_elements, groups_for_elements

    assert groups_for_elements(65) == 2 and bytes_for_elements(128) == 132
    smol = Layout([AttentionLayer(3, 64)] * 30)
    assert (smol.token_elements, smol.bytes_per_token) == (11520, 11880)
    lfm = Layout([AttentionLayer(8, 64)] * 6, recurrent_layers=10, recurrent_width=1024, recurrent_window=3)
    assert (lfm.bytes_per_token, lfm.bytes_per_checkpoint) == (6336, 31680)
    llama = Layout([AttentionLayer(8, 128)] * 32)
    assert llama.bytes_per_token == 67584
    assert llama.attention_key_offset(3) == 3 * 2048 and llama.attention_value_offset(3) == 3 * 2048 + 1024
    with pytest.raises(ValueError, match="group_size must divide"):
        Layout([AttentionLayer(1, 96)])
    with pytest.raises(ValueError, match="positive width"):
        Layout([], recurrent_layers=1)
    with pytest.raises(ValueError, match="positive kv_heads"):
        AttentionLayer(0, 64)


def test_kernel_abi_surface():
    from llmopt_b200 import kernel_abi

    assert kernel_abi.W4A16_LINEAR == "w4a16-linear-g64" and kernel_abi.W4A16_LM_HEAD_ARGMAX == "w4a16-lm-head-argmax"
    entry = kernel_abi.find_entry(name="llmopt_w4a16_linear_f16_g64_m4", operation=kernel_abi.W4A16_LINEAR,
                                  input_dtype="float16", output_dtype="float16")
    assert entry.threadgroup == (256, 1, 1)
    with pytest.raises(LookupError, match="multiple kernels"):
        kernel_abi.find_entry(operation=kernel_abi.W4A16_LINEAR, input_dtype="float16", output_dtype="float16")
    with pytest.raises(LookupError, match="declares no kernel"):
        kernel_abi.find_entry(name="nope", operation=kernel_abi.ATTENTION, input_dtype="float16", output_dtype="float16")
    with pytest.raises(ValueError, match="unsupported kernel operation"):
        kernel_abi.find_entry(operation="matmul-x", input_dtype="float16", output_dtype="float16")
    with pytest.raises(ValueError):
        kernel_abi.Entry("", kernel_abi.CACHE, "float16", "uint8")
    # every entry name is registered in the native library's table (checked textually: no GPU here)
    source = open(os.path.join(ROOT, "llmopt_b200", "csrc", "runtime.cu")).read()
    family = open(os.path.join(ROOT, "llmopt_b200", "csrc", "norm_family.cu")).read()  # its own name table
    registered = set(re.findall(r'"(llmopt_[a-z0-9_]+)"', source + family))
    assert {e.name for e in kernel_abi.ENTRIES} <= registered


class RecordingRuntime:
    """Stands in for cuda_native.Runtime: records dispatches instead of launching."""

    def __init__(self):
        self.items = []

    def kernel_entry(self, *, operation, input_dtype, output_dtype, name=None):
        from llmopt_b200 import kernel_abi

        return kernel_abi.find_entry(operation=operation, input_dtype=input_dtype, output_dtype=output_dtype, name=name)

    def dispatch(self, entry, *, buffers, parameters, grid, batch=None):
        self.items.append((entry.name, list(buffers), bytes(parameters), tuple(grid)))
        return entry.name


class FakeBuffer:
    def __init__(self, label, nbytes=1 << 30):
        self.label, self.nbytes = label, nbytes

    def byte_length(self):
        return self.nbytes

    def __repr__(self):
        return self.label


def _t(label, shape, dtype="float16"):
    from llmopt_b200 import dispatch

    return dispatch.Tensor(FakeBuffer(label), tuple(shape), dtype)


def test_dispatchers_emit_reference_names_order_and_grids(monkeypatch):
    from llmopt_b200 import dispatch

    runtime = RecordingRuntime()
    context = dispatch.Context(runtime)
    monkeypatch.setattr(dispatch.Buffer, "create", staticmethod(lambda rt, nbytes: FakeBuffer(f"scratch{nbytes}", nbytes)))
    # lib/metal_dispatch_linear.ml:968-982: m = 1 -> _g64, grid round_up(m n, 8) * 32; else _m4 over ceil(m/4) n
    dispatch.dispatch_w4a16_linear(context, input=_t("x", (1, 576)), weight=_t("w", (1536, 288), "uint8"),
                                   scale=_t("s", (1536, 9)), output=_t("y", (1, 1536)))
    name, buffers, params, grid = runtime.items[-1]
    assert name == "llmopt_w4a16_linear_f16_g64" and [b.label for b in buffers] == ["x", "w", "s", "s", "y"]
    assert params == struct.pack("<5I", 1, 1536, 576, 0, 0) and grid == (1536 * 32, 1, 1)
    dispatch.dispatch_w4a16_linear(context, input=_t("x", (5, 576)), weight=_t("w", (29, 288), "uint8"),
                                   scale=_t("s", (29, 9)), output=_t("y", (5, 29)), bias=_t("b", (29,)))
    name, buffers, params, grid = runtime.items[-1]
    assert name == "llmopt_w4a16_linear_f16_g64_m4" and buffers[3].label == "b" and grid == (64 * 32, 1, 1)
    with pytest.raises(dispatch.DispatchError, match="metadata is inconsistent"):
        dispatch.dispatch_w4a16_linear(context, input=_t("x", (1, 100)), weight=_t("w", (8, 50), "uint8"),
                                       scale=_t("s", (8, 1)), output=_t("y", (1, 8)))
    # SwiGLU FFN: three launches, reference guard k <= 2048 (lib/metal_dispatch_linear.ml:284-287)
    ffn = dict(m=1, n=1536, k=576, epsilon=1e-5, activation=_t("a", (1, 576)), residual=_t("r", (1, 576)),
               gate_weight=_t("gw", (1536, 288), "uint8"), gate_scale=_t("gs", (1536, 9)),
               up_weight=_t("uw", (1536, 288), "uint8"), up_scale=_t("us", (1536, 9)),
               down_weight=_t("dw", (576, 768), "uint8"), down_scale=_t("ds", (576, 24)),
               norm_weight=_t("nw", (576,)), output=_t("o", (1, 576)))
    names = dispatch.dispatch_w4a16_swiglu_ffn_command(context, **ffn)
    assert names == ["llmopt_w4a16_swiglu_rms_f16_g64", "llmopt_w4a16_dual_swiglu_f16_g64", "llmopt_w4a16_down_add_f16_g64"]
    assert [b.label for b in runtime.items[-1][1]][1:] == ["dw", "ds", "r", "o"] and runtime.items[-3][3] == (256, 1, 1)
    big = dict(ffn, k=4096, n=14336, activation=_t("a", (1, 4096)), residual=_t("r", (1, 4096)),
               gate_weight=_t("gw", (14336, 2048), "uint8"), gate_scale=_t("gs", (14336, 64)),
               up_weight=_t("uw", (14336, 2048), "uint8"), up_scale=_t("us", (14336, 64)),
               down_weight=_t("dw", (4096, 7168), "uint8"), down_scale=_t("ds", (4096, 224)),
               norm_weight=_t("nw", (4096,)), output=_t("o", (1, 4096)))
    with pytest.raises(dispatch.DispatchError, match="SwiGLU input metadata"):
        dispatch.dispatch_w4a16_swiglu_ffn_command(context, **big)
    assert len(dispatch.dispatch_w4a16_swiglu_ffn_command(context, reference_guards=False, **big)) == 3
    # LM head: two-stage with a 256-candidate buffer per row (lib/metal_dispatch_linear.ml:640-678)
    names = dispatch.dispatch_w4a16_lm_head_argmax_command(
        context, m=1, n=49152, k=576, epsilon=1e-5, input=_t("h", (1, 576)), norm_weight=_t("nw", (576,)),
        weight=_t("w", (49152, 288), "uint8"), scale=_t("s", (49152, 9)), output=_t("tok", (1,), "int32"))
    assert names == ["llmopt_w4a16_lm_head_argmax_stage1_f16", "llmopt_w4a16_lm_head_reduce"]
    assert runtime.items[-2][1][4].nbytes == 256 * 8 and runtime.items[-1][2] == struct.pack("<I", 1)
    # paged attention: kernel choice (lib/metal_dispatch_common.ml:41-57), maskless binds slots twice
    config = dispatch.PagedAttentionConfig(token_elements=128, key_offset=0, value_offset=64, group_size=64,
                                           token_stride=132, scale=1.0)
    names = dispatch.dispatch_paged_attention_q8(
        context, config=config, query=_t("q", (1, 9, 1, 64)), current_key=_t("k", (1, 3, 1, 64)),
        current_value=_t("v", (1, 3, 1, 64)), pool=_t("pool", (0,), "uint8"), slots=_t("slots", (77,), "uint32"),
        output=_t("o", (1, 1, 9, 64)))
    assert names == ["llmopt_attention_q8_paged_simd_h64_gqa3"]
    _, buffers, params, grid = runtime.items[-1]
    assert [b.label for b in buffers] == ["q", "k", "v", "pool", "slots", "slots", "o"]
    assert struct.unpack_from("<I", params, 12)[0] == 77 and grid == (8 * 32, 1, 1)  # rows by kv head: 3 -> 8
    assert dispatch.paged_attention_kernel_name(split8=False, experimental_gqa3_split8=False, query_heads=32,
                                                kv_heads=8, head_dimension=128) == "llmopt_attention_q8_paged_simd_generic"
    with pytest.raises(dispatch.DispatchError, match="requires one query token"):
        dispatch.dispatch_paged_attention_q8(
            context, config=config, query=_t("q", (1, 9, 2, 64)), current_key=_t("k", (1, 3, 2, 64)),
            current_value=_t("v", (1, 3, 2, 64)), pool=_t("pool", (0,), "uint8"), slots=_t("slots", (7,), "uint32"),
            output=_t("o", (1, 2, 9, 64)))
    # short conv prefill picks the _init kernel when an initial state is bound (lib/metal_dispatch_recurrent.ml:115-154)
    dispatch.dispatch_short_conv_prefill(context, in_proj=_t("i", (1, 4, 6)), conv_weight=_t("w", (2, 1, 3)),
                                         output=_t("o", (1, 4, 2)), conv_state_out=_t("so", (1, 2, 3)),
                                         conv_state_in=_t("si", (1, 2, 3)))
    name, buffers, params, _ = runtime.items[-1]
    assert name == "llmopt_short_conv_prefill_init_f16" and buffers[4].label == "si" and params == struct.pack("<3I", 4, 2, 1)


def test_numpy_quantiser_round_trip():
    from llmopt_b200.quantize import pack_int4_weight, rope_tables, unpack_int4_weight

    rng = np.random.default_rng(0)
    weight = rng.standard_normal((7, 128)).astype(np.float32)
    packed, scale = pack_int4_weight(weight)
    assert packed.shape == (7, 64) and scale.shape == (7, 2) and scale.dtype == np.float16
    error = np.abs(unpack_int4_weight(packed, scale) - weight)
    assert np.all(error <= 0.5 * np.repeat(scale.astype(np.float32), 64, axis=1) + 1e-3)  # python/tests/test_quantization.py:33-41
    with pytest.raises(ValueError, match="multiple of 64"):
        pack_int4_weight(np.zeros((2, 100), np.float32))  # python/tests/test_quantization.py:72-74
    cosine, sine = rope_tables(4, 64, 1e5)
    assert cosine.shape == (4, 64) and np.array_equal(cosine[:, :32], cosine[:, 32:]) and cosine[0, 0] == 1.0 and sine[0, 5] == 0


def test_model_byte_accounting():
    from llmopt_b200.model import LLAMA3_8B, SMOLLM2_135M, decode_bytes_per_token

    llama = decode_bytes_per_token(LLAMA3_8B, 1, 8192)
    assert abs(llama["weights"] - 3.99e9) < 0.02e9 and abs(llama["attention"] - 0.5547e9) < 0.001e9
    assert SMOLLM2_135M.attention_layers == 30


def test_host_sampler_matches_the_reference_restatement(oracle):
    """llmopt_cuda_sample_f16 is host code (it samples logits the caller read back): the same seed
    must give the same token as the reference's sampler, restated in the oracle — across
    temperatures, top-k sizes, min-p / top-p cuts and rows full of ties."""
    from llmopt_b200 import cuda_native

    rng = np.random.default_rng(11)
    cases = 0
    for vocabulary in (1, 2, 50, 300, 5000):
        for kind in ("normal", "ties", "peaked"):
            if kind == "normal":
                logits = rng.standard_normal(vocabulary).astype(np.float16)
            elif kind == "ties":
                logits = rng.integers(-2, 3, size=vocabulary).astype(np.float16)
            else:
                logits = (rng.standard_normal(vocabulary) * 8).astype(np.float16)
            for temperature, top_k, top_p, min_p in ((0.0, 0, 0.0, 0.0), (1.0, 1, 0.9, 0.0), (0.7, 40, 0.95, 0.05),
                                                     (1.3, 0, 0.0, 0.0), (1.0, 300, 0.5, 0.0), (0.3, 5, 1.0, 0.2),
                                                     (2.0, 256, 0.99, 0.01)):
                for seed in (1, 7, 123456789, 2 ** 62 + 3):
                    got = cuda_native.sample_f16(logits.tobytes(), vocabulary, temperature=temperature, top_k=top_k,
                                                 top_p=top_p, min_p=min_p, seed=seed)
                    want = oracle.sample_f16(logits, temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p,
                                             seed=seed)
                    assert got == want, (vocabulary, kind, temperature, top_k, top_p, min_p, seed, got, want)
                    cases += 1
    assert cases == 5 * 3 * 7 * 4
    # greedy: first maximum wins; an empty row gives token 0
    row = np.array([1, 5, 5, -2], np.float16)
    assert cuda_native.sample_f16(row.tobytes(), 4, temperature=0.0, top_k=0, top_p=0.0, min_p=0.0, seed=1) == 1
    assert cuda_native.sample_f16(b"", 0, temperature=1.0, top_k=0, top_p=0.0, min_p=0.0, seed=1) == 0
    # the distribution is the softmax of the kept candidates: seeds spread over 64 bits split two equal
    # logits about evenly (the first draw of small seeds is dominated by the seeding constant)
    row = np.array([3.0, 3.0, -20.0], np.float16)
    picks = [cuda_native.sample_f16(row.tobytes(), 3, temperature=1.0, top_k=0, top_p=0.0, min_p=0.0, seed=int(seed))
             for seed in rng.integers(1, 2 ** 63, size=400)]
    assert set(picks) == {0, 1} and 140 <= picks.count(0) <= 260


def test_epilogue_digest_names_and_programs():
    """Kernel names of algebraic epilogues are base + '_' + the first 8 hex digits of
    MD5(dtypes | canonical writeback text) (lib/epilogue.ml:217-229, text of
    lib/applicative_expr.ml:205-283); the texts below are what that emitter prints."""
    import hashlib

    from llmopt_b200 import epilogue as ep

    base = "llmopt_w4a16_linear_f16_g64"
    digest = lambda text: base + "_" + hashlib.md5(text.encode()).hexdigest()[:8]
    bias, up, residual = ep.Value(41), ep.Value(7), ep.Value(99)
    silu = "(acc * (1.0f / (1.0f + metal::exp(-acc))))"
    assert ep.algebraic_kernel_name(base, ep.tagged("none")) == digest("|acc")
    assert ep.algebraic_kernel_name(base, ep.tagged("silu")) == digest("|" + silu)
    assert ep.algebraic_kernel_name(base, ep.tagged("bias", bias)) == digest("f16|(acc + ((float)buf_0[col]))")
    assert ep.algebraic_kernel_name(base, ep.tagged("silu_mul_residual_add", up, residual)) == digest(
        "f16,f16|((" + silu + " * ((float)buf_0[col])) + ((float)buf_1[col]))")
    # value ids do not matter (canonical ordinals), operand dtypes and order do
    assert ep.algebraic_kernel_name(base, ep.tagged("bias", ep.Value(5))) == ep.algebraic_kernel_name(base, ep.tagged("bias", bias))
    assert ep.algebraic_kernel_name(base, ep.tagged("bias", ep.Value(5, "f32"))) != ep.algebraic_kernel_name(base, ep.tagged("bias", bias))
    # a free-form tree: clamp(silu(acc) * b0 + 0.5, -1, b1) with an fp32 second operand
    tree = ep.Triop("clamp", ep.Binop("add", ep.Binop("mul", ep.Unop("silu", ep.ACC), ep.Read(up)), ep.Const(0.5)),
                    ep.Const(-1.0), ep.Read(ep.Value(3, "f32")))
    free = ep.of_expr(tree)
    assert ep.algebraic_kernel_name(base, free) == digest(
        "f16,f32|metal::clamp(((" + silu + " * ((float)buf_0[col])) + 0.5000000f), -1.0000000f, ((float)buf_1[col]))")
    assert ep.matching_tag(free) is None
    assert ep.matching_tag(ep.of_expr(ep.Binop("mul", ep.Unop("gelu", ep.ACC), ep.Read(up)))) == "gelu_mul"
    assert ep.matching_tag(ep.of_expr(ep.Binop("add", ep.ACC, ep.Read(bias)))) == "bias"  # same expression as residual_add
    program, dtypes = ep.compile_program(free)
    assert dtypes == ["f16", "f32"]
    assert program == (bytes([1, 12, 3, 0, 0, 22, 2]) + struct.pack("<f", 0.5) + bytes([20, 2]) + struct.pack("<f", -1.0)
                       + bytes([3, 1, 1, 30]))
    with pytest.raises(ValueError):
        ep.tagged("bias")


def test_serving_package_envelope_round_trip_and_errors():
    """package.llmopt (lib/serving_package.ml:303-373): magic, version 27, stage, target, model,
    kernel library, declared kernels with operation / dtype tags, tensor store, page size, two
    length-prefixed blobs; the reader refuses what the reference's refuses, with its messages."""
    from llmopt_b200 import kernel_abi, serving_package as sp

    kernels = [kernel_abi.find_entry(name=name, operation=operation, input_dtype=i, output_dtype=o)
               for name, operation, i, o in (
                   ("llmopt_w4a16_qkv_linear_f16_g64", kernel_abi.W4A16_QKV_LINEAR, "float16", "float16"),
                   ("llmopt_w4a16_lm_head_argmax_f16", kernel_abi.W4A16_LM_HEAD_ARGMAX, "float16", "int32"),
                   ("llmopt_attention_q8_paged_simd_h64_gqa3", kernel_abi.ATTENTION, "float16", "float16"),
                   ("llmopt_cache_pack_attention_q8_pair_simd", kernel_abi.CACHE, "float16", "uint8"),
                   ("llmopt_rms_rope_qk_f16_simd_h64", kernel_abi.RMS_ROPE_QK, "float16", "float16"))]
    package = sp.Package("serving", "kernels/model.metallib", kernels, schedule=b"\x01\x02\x03", memory_plan=b"\x09",
                         model="smollm2-135m", tensor_store="weights/model.llmoptwt", page_size=16)
    data = package.to_bytes()
    # byte-level layout of the head: magic, u16 version, u8 stage (1 = serving), u8 target, option tag, u32 length
    assert data[:8] == b"LLMOPTPK" and data[8:12] == bytes([27, 0, 1, 0]) and data[12] == 1
    assert data[13:17] == (12).to_bytes(4, "little") and data[17:29] == b"smollm2-135m"
    back = sp.of_bytes(data)
    assert back == package and back.kernels[2].threadgroup == (256, 1, 1)
    assert back.kernels[1].operation == "w4a16-lm-head-argmax" and back.kernels[1].output_dtype == "int32"
    for mutate, message in (
            (lambda b: b"XLMOPTPK" + b[8:], "invalid serving-package magic"),
            (lambda b: b[:8] + bytes([26, 0]) + b[10:], "unsupported serving-package version: 26"),
            (lambda b: b[:10] + bytes([2]) + b[11:], "unknown serving-package stage tag: 2"),
            (lambda b: b[:11] + bytes([1]) + b[12:], "unsupported serving-package target tag: 1"),
            (lambda b: b[:-1], "truncated binary input"),
            (lambda b: b + b"\0", "trailing binary input")):
        with pytest.raises(sp.PackageError, match=message):
            sp.of_bytes(mutate(data))
    with pytest.raises(sp.PackageError, match="must declare a tensor store"):
        sp.of_bytes(sp.Package("serving", "a.metallib", kernels).to_bytes())
    with pytest.raises(sp.PackageError, match="names must be unique"):
        sp.of_bytes(sp.Package("compiled-graph", "a.metallib", kernels + kernels[:1]).to_bytes())
    with pytest.raises(sp.PackageError, match="not canonical"):
        sp.of_bytes(sp.Package("compiled-graph", "../a.metallib", kernels).to_bytes())

    class FakeRuntime:  # has_function / preload_pipeline against a name set
        def __init__(self, names):
            self.names, self.preloaded = set(names), []

        def has_function(self, name):
            return name in self.names

        def preload_pipeline(self, name):
            self.preloaded.append(name)

    runtime = FakeRuntime(entry.name for entry in kernels)
    back.validate_declared_functions(runtime)
    assert runtime.preloaded == [entry.name for entry in kernels]
    runtime.names.discard("llmopt_rms_rope_qk_f16_simd_h64")
    with pytest.raises(sp.PackageError, match="does not define declared kernel: llmopt_rms_rope_qk_f16_simd_h64"):
        back.validate_declared_functions(runtime)
