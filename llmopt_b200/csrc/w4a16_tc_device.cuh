// Device helpers shared by the tcgen05 W4A16 kernels: mbarriers with bounded waits, TMA tile loads,
// shared-memory operand descriptors, tcgen05.mma / commit / ld wrappers and the int4 -> fp16 pair
// conversion.
#pragma once
#include <cuda.h>

#include "w4a16_gemv.cuh"
#include "w4a16_gemv_device.cuh"

namespace llmopt {
namespace tc {
using namespace gemv;

constexpr uint32_t kWaitLimit = 1u << 20;

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void barrier_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void barrier_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void barrier_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase of parity `parity`; false when the limit ran out.
__device__ __forceinline__ bool barrier_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t destination, const CUtensorMap* map, int32_t x, int32_t y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(destination), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row
// groups 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t shared_address) {
  uint64_t descriptor = 0;
  descriptor |= (uint64_t)((shared_address & 0x3ffffu) >> 4);  // start address, bits [0, 14)
  descriptor |= (uint64_t)1 << 16;                             // leading byte offset (unused with swizzle)
  descriptor |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset, bits [32, 46)
  descriptor |= (uint64_t)1 << 46;                             // version
  descriptor |= (uint64_t)2 << 61;                             // SWIZZLE_128B
  return descriptor;
}

// Instruction descriptor for kind::f16: fp16 A and B, fp32 accumulator, both K-major, M x N.
__host__ __device__ constexpr uint32_t instruction_descriptor(uint32_t m, uint32_t n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
constexpr uint32_t kInstruction = instruction_descriptor(128, 256);

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate,
                                        uint32_t instruction = kInstruction) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(instruction), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t address, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(address)
      : "memory");
}

// Two packed bytes' worth of one row: byte b of `word` holds k = 2b (low nibble) and 2b + 1.
// Returns half2(w[2b] , w[2b+1]) = (q * scale) for the symmetric form, ((u - zero) * scale) for
// the affine one.  `scales` = (scale, scale / 16): the high nibble is read in place, 16 times
// too large, and the factor is folded into its multiplier (exact: a power of two).
template <bool AFFINE, int BYTE>
__device__ __forceinline__ uint32_t dequant_pair(uint32_t word, uint32_t scales, uint32_t zeros) {
  constexpr uint32_t selector = BYTE | (BYTE << 4) | (BYTE << 8) | (BYTE << 12);
  const uint32_t spread = prmt(word, word, selector);  // the byte in both half-words
  if (AFFINE) {
    // (1024 + u, 1024 + 16 u) -> (u, 16 u) -> minus (zero, 16 zero) -> times (scale, scale / 16)
    const uint32_t biased = lop3_and_xor(spread, 0x00f0000fu, 0x64006400u);
    const uint32_t integers = hsub2_u32(biased, 0x64006400u);
    return hmul2_u32(hsub2_u32(integers, zeros), scales);
  }
  // two's complement nibble q: (q ^ 8) is q + 8 as unsigned; 1024 + 8 + q and 1024 + 128 + 16 q
  const uint32_t biased = lop3_and_xor(spread, 0x00f0000fu, 0x64806408u);
  return hmul2_u32(hsub2_u32(biased, 0x64806408u), scales);
}


// The group scales (or zero points) of four consecutive k-blocks of one weight row, starting at
// k-block `first` (a multiple of 4): one 8-byte load when the row of scales allows it, so that the
// conversion never waits on a load issued only one k-block earlier.  Absent k-blocks read zero.
struct FourHalves {
  __half value[4];
};
__device__ __forceinline__ FourHalves load_four(const __half* row, uint32_t first, uint32_t count, bool vector_ok,
                                                bool present) {
  FourHalves out;
#pragma unroll
  for (int i = 0; i < 4; ++i) out.value[i] = __float2half(0.0f);
  if (!present) return out;
  if (vector_ok && first + 4u <= count) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(row + first));
    *reinterpret_cast<uint2*>(out.value) = raw;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (first + i < count) out.value[i] = __ldg(row + first + i);
  }
  return out;
}

// 16 consecutive accumulator columns of this thread's lane.
__device__ __forceinline__ void tmem_load_16(uint32_t address, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(address)
      : "memory");
}

// 8 consecutive accumulator columns of this thread's lane.
__device__ __forceinline__ void tmem_load_8(uint32_t address, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(address)
               : "memory");
}

// 4 consecutive accumulator columns of this thread's lane.
__device__ __forceinline__ void tmem_load_4(uint32_t address, uint32_t (&v)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "r"(address)
               : "memory");
}

}  // namespace tc
}  // namespace llmopt
