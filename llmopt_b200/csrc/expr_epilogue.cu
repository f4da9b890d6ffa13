// W4A16 linear with a free-form epilogue expression over the accumulator
// (Epilogue.Expr, lib/epilogue.ml:16; the parametric kernel of
// lib/metal_parametric_codegen.ml:4-39 compiles the expression into its writeback).
//
// The reference generates one Metal kernel per expression and names it by a digest of the
// expression text.  Here the host registers that digest name together with a small postfix
// program; a dispatch of the name runs the plain group-64 product into fp32 scratch (the
// unrounded accumulator) and then one elementwise kernel that evaluates the program per output
// element in fp32, reading operand tensors at the output column, and rounds to half once — the
// arithmetic of the generated writeback `half(<expression>)`.
//
// Buffers: [input, weight, scale, bias_or_scale, output, operand 0, operand 1, ...]
// (operands in first-occurrence order of the expression); params: the 20-byte linear block.
#include "w4a16_gemv.cuh"

namespace llmopt {

struct ExprProgram {
  uint8_t code[192];
  uint32_t length;
  uint32_t operands;
};
const ExprProgram* context_expr_program(Context* ctx, const char* name);

namespace {

enum : uint8_t {
  kAcc = 1, kConst = 2, kRead = 3, kNeg = 10, kAbs = 11, kSilu = 12, kGelu = 13, kExp = 14, kLog = 15, kRsqrt = 16,
  kCastF16 = 17, kAdd = 20, kSub = 21, kMul = 22, kDiv = 23, kMin = 24, kMax = 25, kClamp = 30, kWhere = 31
};
constexpr int kMaxStack = 12;
constexpr int kMaxOperands = 8;

struct ExprOperands {
  const void* pointer[kMaxOperands];
};

__global__ void expr_epilogue_kernel(const float* __restrict__ accumulators, __half* __restrict__ output, uint32_t m,
                                     uint32_t n, ExprProgram program, ExprOperands operands) {
  grid_chain_prologue();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= m * n) return;
  const uint32_t col = gid % n;
  const float acc = accumulators[gid];
  float stack[kMaxStack];
  int top = 0;  // number of values on the stack
  for (uint32_t pc = 0; pc < program.length;) {
    const uint8_t op = program.code[pc++];
    switch (op) {
      case kAcc: stack[top++] = acc; break;
      case kConst: {
        uint32_t bits = program.code[pc] | (program.code[pc + 1] << 8) | (program.code[pc + 2] << 16) |
                        ((uint32_t)program.code[pc + 3] << 24);
        pc += 4;
        stack[top++] = __uint_as_float(bits);
        break;
      }
      case kRead: {
        const uint8_t index = program.code[pc], is_f32 = program.code[pc + 1];
        pc += 2;
        stack[top++] = is_f32 ? static_cast<const float*>(operands.pointer[index])[col]
                              : __half2float(static_cast<const __half*>(operands.pointer[index])[col]);
        break;
      }
      case kNeg: stack[top - 1] = -stack[top - 1]; break;
      case kAbs: stack[top - 1] = fabsf(stack[top - 1]); break;
      case kSilu: stack[top - 1] = stack[top - 1] * (1.0f / (1.0f + expf(-stack[top - 1]))); break;
      case kGelu: {
        const float e = stack[top - 1];
        const float inner = fminf(fmaxf(0.7978845608f * (e + 0.044715f * e * e * e), -10.0f), 10.0f);
        stack[top - 1] = 0.5f * e * (1.0f + tanhf(inner));
        break;
      }
      case kExp: stack[top - 1] = expf(stack[top - 1]); break;
      case kLog: stack[top - 1] = logf(stack[top - 1]); break;
      case kRsqrt: stack[top - 1] = rsqrtf(stack[top - 1]); break;
      case kCastF16: stack[top - 1] = __half2float(__float2half_rn(stack[top - 1])); break;
      case kAdd: stack[top - 2] = __fadd_rn(stack[top - 2], stack[top - 1]); --top; break;
      case kSub: stack[top - 2] = __fsub_rn(stack[top - 2], stack[top - 1]); --top; break;
      case kMul: stack[top - 2] = __fmul_rn(stack[top - 2], stack[top - 1]); --top; break;
      case kDiv: stack[top - 2] = stack[top - 2] / stack[top - 1]; --top; break;
      case kMin: stack[top - 2] = fminf(stack[top - 2], stack[top - 1]); --top; break;
      case kMax: stack[top - 2] = fmaxf(stack[top - 2], stack[top - 1]); --top; break;
      case kClamp: stack[top - 3] = fminf(fmaxf(stack[top - 3], stack[top - 2]), stack[top - 1]); top -= 2; break;
      default: stack[top - 3] = stack[top - 3] != 0.0f ? stack[top - 2] : stack[top - 1]; top -= 2; break;  // kWhere
    }
  }
  output[gid] = __float2half_rn(stack[0]);
}

}  // namespace

// Checks stack discipline and operand indices of a program; returns an error text or nullptr.
const char* validate_expr_program(const uint8_t* code, size_t length, int operand_count) {
  if (length == 0 || length > sizeof(ExprProgram::code)) return "expression program must hold 1..192 bytes";
  if (operand_count < 0 || operand_count > kMaxOperands) return "expression program reads at most 8 operands";
  int depth = 0;
  for (size_t pc = 0; pc < length;) {
    const uint8_t op = code[pc++];
    int pops = 0, pushes = 0;
    switch (op) {
      case kAcc: pushes = 1; break;
      case kConst:
        if (pc + 4 > length) return "expression program ends inside a constant";
        pc += 4, pushes = 1;
        break;
      case kRead:
        if (pc + 2 > length) return "expression program ends inside an operand read";
        if (code[pc] >= operand_count || code[pc + 1] > 1) return "expression program reads an operand it does not bind";
        pc += 2, pushes = 1;
        break;
      case kNeg: case kAbs: case kSilu: case kGelu: case kExp: case kLog: case kRsqrt: case kCastF16:
        pops = 1, pushes = 1;
        break;
      case kAdd: case kSub: case kMul: case kDiv: case kMin: case kMax: pops = 2, pushes = 1; break;
      case kClamp: case kWhere: pops = 3, pushes = 1; break;
      default: return "expression program holds an unknown operation";
    }
    if (depth < pops) return "expression program pops an empty stack";
    depth += pushes - pops;
    if (depth > kMaxStack) return "expression program needs more than 12 stack slots";
  }
  return depth == 1 ? nullptr : "expression program must leave exactly one value";
}

int launch_w4a16_linear_expr(const KernelArgs& args) {
  const ExprProgram* program = args.ctx ? context_expr_program(args.ctx, args.name) : nullptr;
  LLMOPT_REQUIRE(program != nullptr, "no expression program is registered under this name");
  LLMOPT_REQUIRE(args.buffer_count == 5 + (int)program->operands, "unexpected buffer count for this expression epilogue");
  LLMOPT_REQUIRE(args.param_bytes == 20, "expects 20 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 64 == 0, "needs m, n > 0 and k a positive multiple of 64");
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 2, "input buffer is too short");
  LLMOPT_REQUIRE(args.lengths[1] >= (size_t)n * (k / 2) && args.lengths[2] >= (size_t)n * (k / 64) * 2,
                 "weight or scale buffer is too short");
  LLMOPT_REQUIRE(args.lengths[4] >= (size_t)m * n * 2, "output buffer is too short");
  ExprOperands operands = {};
  for (uint32_t i = 0; i < program->operands; ++i) {
    LLMOPT_REQUIRE(args.lengths[5 + i] >= (size_t)n * 2, "epilogue operand is shorter than n");
    operands.pointer[i] = args.buffers[5 + i];
  }
  // the operand dtype is part of the program: an fp32 operand must hold n floats
  for (uint32_t pc = 0; pc < program->length;) {
    const uint8_t op = program->code[pc++];
    if (op == kConst) pc += 4;
    if (op == kRead) {
      if (program->code[pc + 1]) LLMOPT_REQUIRE(args.lengths[5 + program->code[pc]] >= (size_t)n * 4, "fp32 epilogue operand is shorter than n");
      pc += 2;
    }
  }
  float* scratch = (float*)context_scratch(args.ctx, (size_t)m * n * sizeof(float), args.error);
  if (scratch == nullptr) return 1;
  // the unrounded accumulators, at most 32 rows per pass of the fp32-output product
  for (uint32_t row0 = 0; row0 < m; row0 += 32) {
    const uint32_t rows = m - row0 < 32 ? m - row0 : 32;
    GemvProblem problem = {};
    problem.x = (const __half*)args.buffers[0] + (size_t)row0 * k;
    problem.x_rows = rows;
    problem.m = rows;
    problem.k = k;
    problem.matrices = 1;
    problem.mat[0] = {(const uint8_t*)args.buffers[1], (const __half*)args.buffers[2], nullptr, n};
    problem.out_f32 = scratch + (size_t)row0 * n;
    if (int status = launch_w4a16_gemv(args, problem, kEpiLinear, false)) return status;
  }
  const uint32_t total = m * n;
  launch_kernel(args, expr_epilogue_kernel, dim3((total + 255) / 256), dim3(256), 0, (const float*)scratch,
                (__half*)args.buffers[4], m, n, *program, operands);
  return check_launch(args);
}

// The same over a Q4_0-block weight, with the buffer order of the reference's Q4_0 epilogue kernels
// (Writeback.Epilogue, lib/metal_q4_0_epilogue_codegen.ml:7-31): [input, weight, operand 0 .., output] and the
// 16-byte quant-linear parameter block {m, n, k, has_bias}; the flat bias does not exist in this form.
int launch_q4_0_product_f32(const KernelArgs& args, const __half* x, const uint8_t* weight, float* out, uint32_t m, uint32_t n,
                            uint32_t k);
int launch_q4_0_linear_expr(const KernelArgs& args) {
  const ExprProgram* program = args.ctx ? context_expr_program(args.ctx, args.name) : nullptr;
  LLMOPT_REQUIRE(program != nullptr, "no expression program is registered under this name");
  LLMOPT_REQUIRE(args.buffer_count == 3 + (int)program->operands, "unexpected buffer count for this expression epilogue");
  LLMOPT_REQUIRE(args.param_bytes == 16, "expects 16 parameter bytes");
  const uint32_t m = param_u32(args, 0), n = param_u32(args, 1), k = param_u32(args, 2);
  LLMOPT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 32 == 0 && ((uintptr_t)args.buffers[0] & 15u) == 0,
                 "needs m, n > 0, k a positive multiple of 32 and a 16-byte aligned input");
  const int output = 2 + (int)program->operands;
  LLMOPT_REQUIRE(args.lengths[0] >= (size_t)m * k * 2 && args.lengths[1] >= (size_t)n * (k / 32) * 18 &&
                     args.lengths[output] >= (size_t)m * n * 2,
                 "input, weight or output buffer is too short");
  ExprOperands operands = {};
  for (uint32_t i = 0; i < program->operands; ++i) {
    LLMOPT_REQUIRE(args.lengths[2 + i] >= (size_t)n * 2, "epilogue operand is shorter than n");
    operands.pointer[i] = args.buffers[2 + i];
  }
  for (uint32_t pc = 0; pc < program->length;) {  // an fp32 operand must hold n floats
    const uint8_t op = program->code[pc++];
    if (op == kConst) pc += 4;
    if (op == kRead) {
      if (program->code[pc + 1]) LLMOPT_REQUIRE(args.lengths[2 + program->code[pc]] >= (size_t)n * 4, "fp32 epilogue operand is shorter than n");
      pc += 2;
    }
  }
  float* scratch = (float*)context_scratch(args.ctx, (size_t)m * n * sizeof(float), args.error);
  if (scratch == nullptr) return 1;
  if (int status = launch_q4_0_product_f32(args, (const __half*)args.buffers[0], (const uint8_t*)args.buffers[1], scratch, m, n, k))
    return status;
  const uint32_t total = m * n;
  launch_kernel(args, expr_epilogue_kernel, dim3((total + 255) / 256), dim3(256), 0, (const float*)scratch,
                (__half*)args.buffers[output], m, n, *program, operands);
  return check_launch(args);
}

}  // namespace llmopt
