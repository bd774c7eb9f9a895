// tc_tcgen05.cuh -- sm_100a 5th-generation tensor-core helpers: TMEM allocation,
// UMMA shared-memory / instruction descriptors, tcgen05.mma / commit / ld / st.
//
// Descriptor bit layouts follow the PTX ISA "tcgen05 matrix descriptor" and
// "instruction descriptor" tables (the same fields CUTLASS names
// UMMA::SmemDescriptor / UMMA::InstrDescriptor).
#pragma once

#include "tc_common.cuh"

namespace tc {

#ifdef __CUDACC__

// ---- TMEM allocation (one warp, .sync.aligned) --------------------------------------
__device__ __forceinline__ void tmemAlloc(uint32_t *smemDst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(smemDst)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmemRelinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemDealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcFenceBefore() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ------------------------------------------------------------------------
// Shared-memory matrix descriptor: start address >> 4 in [0,14), leading-dimension
// byte offset >> 4 in [16,30), stride-dimension byte offset >> 4 in [32,46),
// version 1 in [46,48), swizzle mode in [61,64) (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t umaSmemDesc(uint32_t smemByteAddr, uint32_t lboBytes, uint32_t sboBytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smemByteAddr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>((lboBytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sboBytes >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
// Instruction descriptor for kind::f16 with f32 accumulation: c_format = F32 (bit 4),
// a/b format F16 (0), a_major bit 15, b_major bit 16 (0 = K-major, 1 = MN-major),
// N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t umaInstrDescF16(uint32_t M, uint32_t N, uint32_t aMajorMN,
                                                       uint32_t bMajorMN) {
    return (1u << 4) | (aMajorMN << 15) | (bMajorMN << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// ---- MMA issue (one thread) ---------------------------------------------------------------
// D(tmem) (+)= A(smem) * B(smem)
__device__ __forceinline__ void umaMmaSS(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
            : "memory");
}
// D(tmem) (+)= A(tmem) * B(smem)
__device__ __forceinline__ void umaMmaTS(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
            ::"r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate)
            : "memory");
}
// The same two with an issue predicate: every lane of the issuing warp runs the surrounding
// (warp-uniform) code so that descriptors and addresses stay uniform values, and only the lane
// with `issue` != 0 executes the instruction itself.
__device__ __forceinline__ void umaMmaSSIf(uint32_t issue, uint32_t dTmem, uint64_t aDesc, uint64_t bDesc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "setp.ne.b32 q, %5, 0;\n\t"
            "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate), "r"(issue)
            : "memory");
}
__device__ __forceinline__ void umaMmaTSIf(uint32_t issue, uint32_t dTmem, uint32_t aTmem, uint64_t bDesc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "setp.ne.b32 q, %5, 0;\n\t"
            "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
            ::"r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate), "r"(issue)
            : "memory");
}
__device__ __forceinline__ void umaCommitIf(uint32_t issue, uint64_t *bar) {
    asm volatile(
            "{\n\t.reg .pred q;\n\t"
            "setp.ne.b32 q, %1, 0;\n\t"
            "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
            ::"r"(smemAddr(bar)), "r"(issue)
            : "memory");
}
// mbarrier arrive once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umaCommit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar))
                 : "memory");
}

// ---- TMEM <-> registers (warp-collective; lane i of warp w touches TMEM lane 32*(w%4)+i) ------
__device__ __forceinline__ void tmemLd32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
              "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
              "=r"(r[30]), "=r"(r[31])
            : "r"(taddr)
            : "memory");
}
__device__ __forceinline__ void tmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemSt32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
            "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
            "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
            ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
            "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
            "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
            "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
            : "memory");
}
__device__ __forceinline__ void tmemSt16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
            "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
            ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
            "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
            : "memory");
}
__device__ __forceinline__ void tmemStWait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

#endif  // __CUDACC__

}  // namespace tc
