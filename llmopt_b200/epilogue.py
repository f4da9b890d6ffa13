"""The reference's epilogue algebra for quantised linears (lib/epilogue.ml, lib/applicative_expr.ml)
on the host: the ten tagged forms, free-form expression trees over the accumulator, the canonical
MSL writeback text and the digest-derived kernel names a compiled package uses
(``base_<first 8 hex of MD5(dtypes | writeback)>``, lib/epilogue.ml:217-229), plus what this
library needs to serve such a name: the tag of one of its ten built-in epilogue kernels, or a
postfix program for the expression interpreter kernel.

An expression is a tree of ``Slot`` (the fp32 accumulator), ``Const``, ``Read`` (an operand tensor
read at the output column), ``Unop``, ``Binop`` and ``Triop`` nodes.  Only identity-coordinate
reads are modelled (the parametric W4A16 kernel reads its operands at ``col``,
lib/metal_parametric_codegen.ml:4-39)."""

from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass
from typing import Optional, Sequence, Union

# ---- expression trees (lib/applicative_expr.ml:1-29) ---------------------------------------------

UNOPS = ("neg", "abs", "silu", "gelu", "exp", "log", "rsqrt", "cast_f16", "cast_f32")
BINOPS = ("add", "sub", "mul", "div", "min", "max")
TRIOPS = ("clamp", "where")


@dataclass(frozen=True)
class Value:
    """An operand tensor: ``Ir.Value`` reduced to what the algebra reads (id and dtype)."""

    id: int
    dtype: str = "f16"  # Ir.Dtype.to_string: "f16" or "f32"


@dataclass(frozen=True)
class Slot:
    pass


@dataclass(frozen=True)
class Const:
    value: float


@dataclass(frozen=True)
class Read:
    value: Value


@dataclass(frozen=True)
class Unop:
    op: str
    operand: "Expr"


@dataclass(frozen=True)
class Binop:
    op: str
    left: "Expr"
    right: "Expr"


@dataclass(frozen=True)
class Triop:
    op: str
    first: "Expr"
    second: "Expr"
    third: "Expr"


Expr = Union[Slot, Const, Read, Unop, Binop, Triop]
ACC = Slot()


# ---- the tagged forms (lib/epilogue.ml:5-16, 36-58) -------------------------------------------------

@dataclass(frozen=True)
class Epilogue:
    """One of the ten tagged epilogues, or a free-form expression (``tag`` = "expr")."""

    tag: str
    operands: tuple = ()          # Values in Epilogue.inputs order
    expression: Optional[Expr] = None

    def to_expr(self) -> Expr:
        if self.tag == "expr":
            return self.expression
        read = [Read(value) for value in self.operands]
        silu, gelu = Unop("silu", ACC), Unop("gelu", ACC)
        return {
            "none": lambda: ACC,
            "bias": lambda: Binop("add", ACC, read[0]),
            "silu": lambda: silu,
            "gelu": lambda: gelu,
            "silu_mul": lambda: Binop("mul", silu, read[0]),
            "gelu_mul": lambda: Binop("mul", gelu, read[0]),
            "residual_add": lambda: Binop("add", ACC, read[0]),
            "bias_residual_add": lambda: Binop("add", Binop("add", ACC, read[0]), read[1]),
            "silu_mul_residual_add": lambda: Binop("add", Binop("mul", silu, read[0]), read[1]),
            "gelu_mul_residual_add": lambda: Binop("add", Binop("mul", gelu, read[0]), read[1]),
        }[self.tag]()


TAGS = ("none", "bias", "silu", "gelu", "silu_mul", "gelu_mul", "residual_add", "bias_residual_add",
        "silu_mul_residual_add", "gelu_mul_residual_add")
_OPERAND_COUNT = {"none": 0, "silu": 0, "gelu": 0, "bias": 1, "silu_mul": 1, "gelu_mul": 1, "residual_add": 1,
                  "bias_residual_add": 2, "silu_mul_residual_add": 2, "gelu_mul_residual_add": 2}


def tagged(tag: str, *operands: Value) -> Epilogue:
    if tag not in _OPERAND_COUNT or len(operands) != _OPERAND_COUNT[tag]:
        raise ValueError(f"epilogue {tag} takes {_OPERAND_COUNT.get(tag)} operands")
    return Epilogue(tag, tuple(operands))


def of_expr(expression: Expr) -> Epilogue:
    return Epilogue("expr", tuple(required_values(expression)), expression)


# ---- analysis (lib/applicative_expr.ml:118-137, 184-203) ----------------------------------------------

def required_values(expression: Expr) -> list:
    """Unique operand tensors in first-occurrence order (left to right, pre-order)."""
    seen, ordered = set(), []

    def walk(node):
        if isinstance(node, Read):
            if node.value.id not in seen:
                seen.add(node.value.id)
                ordered.append(node.value)
        elif isinstance(node, Unop):
            walk(node.operand)
        elif isinstance(node, Binop):
            walk(node.left), walk(node.right)
        elif isinstance(node, Triop):
            walk(node.first), walk(node.second), walk(node.third)

    walk(expression)
    return ordered


def canonicalize(expression: Expr) -> Expr:
    """Renames the operand tensors to their ordinal among ``required_values`` (0, 1, ...)."""
    ordinal = {value.id: index for index, value in enumerate(required_values(expression))}

    def rename(node):
        if isinstance(node, Read):
            return Read(Value(ordinal[node.value.id], node.value.dtype))
        if isinstance(node, Unop):
            return Unop(node.op, rename(node.operand))
        if isinstance(node, Binop):
            return Binop(node.op, rename(node.left), rename(node.right))
        if isinstance(node, Triop):
            return Triop(node.op, rename(node.first), rename(node.second), rename(node.third))
        return node

    return rename(expression)


def emit_msl(expression: Expr, *, acc: str = "acc", index: str = "col") -> str:
    """``Applicative_expr.emit_msl_expr`` (lib/applicative_expr.ml:205-283): the exact text the
    reference would compile, hence the text its kernel names are hashed from."""
    def emit(node) -> str:
        if isinstance(node, Slot):
            return acc
        if isinstance(node, Const):
            return "%.7ff" % node.value
        if isinstance(node, Read):
            return f"((float)buf_{node.value.id}[{index}])"
        if isinstance(node, Unop):
            inner = emit(node.operand)
            if node.op == "neg":
                return f"(-{inner})"
            if node.op == "abs":
                return f"metal::abs({inner})"
            if node.op == "silu":
                return f"({inner} * (1.0f / (1.0f + metal::exp(-{inner}))))"
            if node.op == "gelu":
                return (f"(0.5f * {inner} * (1.0f + metal::tanh(metal::clamp(0.7978845608f * ({inner} + 0.044715f * "
                        f"{inner} * {inner} * {inner}), -10.0f, 10.0f))))")
            if node.op in ("exp", "log", "rsqrt"):
                return f"metal::{node.op}({inner})"
            if node.op == "cast_f16":
                return f"((half)({inner}))"
            if node.op == "cast_f32":
                return inner
            raise ValueError(f"unknown unary operation {node.op}")
        if isinstance(node, Binop):
            left, right = emit(node.left), emit(node.right)
            symbol = {"add": "+", "sub": "-", "mul": "*", "div": "/"}.get(node.op)
            if symbol:
                return f"({left} {symbol} {right})"
            if node.op in ("min", "max"):
                return f"metal::{node.op}({left}, {right})"
            raise ValueError(f"unknown binary operation {node.op}")
        if isinstance(node, Triop):
            a, b, c = emit(node.first), emit(node.second), emit(node.third)
            if node.op == "clamp":
                return f"metal::clamp({a}, {b}, {c})"
            if node.op == "where":
                return f"({a} ? {b} : {c})"
        raise ValueError("unknown expression node")

    return emit(expression)


def algebraic_kernel_name(base: str, epilogue: Epilogue) -> str:
    """``Epilogue.algebraic_kernel_name`` (lib/epilogue.ml:217-229)."""
    canonical = canonicalize(epilogue.to_expr())
    writeback = emit_msl(canonical)
    dtypes = ",".join(value.dtype for value in required_values(canonical))
    return base + "_" + hashlib.md5((dtypes + "|" + writeback).encode()).hexdigest()[:8]


def matching_tag(epilogue: Epilogue) -> Optional[str]:
    """The tagged form whose canonical expression equals this epilogue's, if any: such an epilogue is
    served by the built-in ``llmopt_w4a16_linear_f16_g64_epi_<tag>`` kernel."""
    if epilogue.tag != "expr":
        return epilogue.tag
    wanted = canonicalize(epilogue.expression)
    operands = required_values(wanted)
    if any(value.dtype != "f16" for value in operands):
        return None
    for tag in TAGS:  # "bias" and "residual_add" share an expression; the first match is returned
        if _OPERAND_COUNT[tag] == len(operands) and canonicalize(tagged(tag, *operands).to_expr()) == wanted:
            return tag
    return None


# ---- postfix program for the expression interpreter kernel ----------------------------------------------

OPCODES = {"acc": 1, "const": 2, "read": 3, "neg": 10, "abs": 11, "silu": 12, "gelu": 13, "exp": 14, "log": 15,
           "rsqrt": 16, "cast_f16": 17, "add": 20, "sub": 21, "mul": 22, "div": 23, "min": 24, "max": 25, "clamp": 30,
           "where": 31}
MAX_PROGRAM_BYTES = 192
MAX_OPERANDS = 8
MAX_STACK = 12


def compile_program(epilogue: Epilogue) -> tuple:
    """(program bytes, operand dtypes) of the canonical expression: operands are pushed by ordinal,
    so the caller binds them after the five linear buffers in ``required_values`` order."""
    canonical = canonicalize(epilogue.to_expr())
    operands = required_values(canonical)
    if len(operands) > MAX_OPERANDS:
        raise ValueError(f"an expression epilogue reads at most {MAX_OPERANDS} operand tensors")
    code = bytearray()
    depth = peak = 0

    def emit(node):
        nonlocal depth, peak
        if isinstance(node, Slot):
            code.append(OPCODES["acc"])
            depth += 1
        elif isinstance(node, Const):
            code.append(OPCODES["const"])
            code.extend(struct.pack("<f", node.value))
            depth += 1
        elif isinstance(node, Read):
            code.extend((OPCODES["read"], node.value.id, 1 if node.value.dtype == "f32" else 0))
            depth += 1
        elif isinstance(node, Unop):
            emit(node.operand)
            if node.op != "cast_f32":  # all arithmetic is fp32 already
                code.append(OPCODES[node.op])
        elif isinstance(node, Binop):
            emit(node.left), emit(node.right)
            code.append(OPCODES[node.op])
            depth -= 1
        elif isinstance(node, Triop):
            emit(node.first), emit(node.second), emit(node.third)
            code.append(OPCODES[node.op])
            depth -= 2
        else:
            raise ValueError("unknown expression node")
        peak = max(peak, depth)

    emit(canonical)
    if len(code) > MAX_PROGRAM_BYTES or peak > MAX_STACK:
        raise ValueError("expression epilogue is too large for the interpreter kernel")
    return bytes(code), [value.dtype for value in operands]


def bind(runtime, base: str, epilogue: Epilogue) -> str:
    """Makes the digest name of ``epilogue`` over the W4A16 (or Q4_0-block) linear ``base`` resolvable in
    ``runtime``'s library and returns it: an alias of the matching built-in tagged kernel, or a
    registered expression program."""
    name = algebraic_kernel_name(base, epilogue)
    if runtime.has_function(name):
        return name
    # Q4_0-block bases (lib/metal_q4_0_epilogue_codegen.ml) have no built-in tagged kernels: always a program
    tag = None if base.startswith("llmopt_q4_0_linear_f16") else matching_tag(epilogue)
    if tag is not None:
        runtime.register_alias(name, f"llmopt_w4a16_linear_f16_g64_epi_{tag}")
    else:
        program, dtypes = compile_program(epilogue)
        runtime.register_expr_epilogue(name, program, len(dtypes))
    return name
