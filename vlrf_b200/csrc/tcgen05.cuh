// Device helpers shared by the tcgen05 kernels: mbarriers with bounded waits, shared-memory matrix
// descriptors and the instruction descriptor of the bfloat16 MMA, its issue and commit, and loads from
// tensor memory.
#pragma once
#include "common.cuh"
#include <cstdint>

namespace {

constexpr uint32_t TC_WAIT_LIMIT = 1u << 21;   // polls of a barrier before a wait gives up

__device__ __forceinline__ uint32_t tsm(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tsm(bar)), "r"(count));
}
__device__ __forceinline__ void tbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tsm(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(tsm(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) written by TMA with
// the 128-byte swizzle: 8-row groups are 1024 bytes apart; version 1 (Blackwell); layout type 2 (128B swizzle).
__device__ __forceinline__ uint64_t umma_desc_k128(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((tsm(tile) >> 4) & 0x3FFF);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: 8 rows × 128 bytes
    d |= (uint64_t)1 << 46;                               // descriptor version
    d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D float32, A and B bfloat16, both K-major, shape M × N
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tsm(bar)) : "memory");
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

// a wait that also gives up when another role of the CTA has already given up
__device__ __forceinline__ bool tbar_wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
        if (tbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void tbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tsm(bar)) : "memory");
}

}  // namespace
