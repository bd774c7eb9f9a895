// tc_common.cuh -- sm_100a device helpers shared by the attention kernels:
// mbarrier, TMA (cp.async.bulk.tensor), cp.async, ldmatrix, movmatrix, mma.sync,
// int8 -> fp16 conversion, plus the host-side error plumbing of the C ABI.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tc_attn.h"

namespace tc {

constexpr float kLog2e = 1.4426950408889634f;  // same constant as the reference (GpuCommon.hpp:77)
constexpr float kNegBig = -1e30f;              // initial running max of the GPU kernels

// Device-side error word: a kernel that gives up on a bounded wait ORs a code in
// and returns; tc_device_status() reads and clears it.
enum : uint32_t {
    kDevErrFullWait = 1u,   // consumer waited too long for a TMA stage
    kDevErrEmptyWait = 2u,  // producer waited too long for a free stage
    kDevErrMmaWait = 4u,    // waited too long for a tcgen05 commit
    kDevErrTmemAlloc = 8u,
    kDevErrMergeWait = 16u,  // a block waited too long for the partials of another rank
    kDevErrRowBound = 32u,   // a KV writer was handed a device-side position outside its pool: store skipped
};
// The word lives in one translation unit; kernels receive its device address as
// an argument (devErrorWord(), resolved once per device).
unsigned int *devErrorWord();

// ---- host-side error reporting ---------------------------------------------
void setError(const char *fmt, ...);
int cudaFail(cudaError_t e, const char *what);
#define TC_CUDA_OK(expr)                                    \
    do {                                                    \
        cudaError_t _e = (expr);                            \
        if (_e != cudaSuccess) return tc::cudaFail(_e, #expr); \
    } while (0)
#define TC_REQUIRE(cond, code, ...)      \
    do {                                 \
        if (!(cond)) {                   \
            tc::setError(__VA_ARGS__);   \
            return (code);               \
        }                                \
    } while (0)

int numSMs();

// Tensor-map factory (driver entry point resolved through the runtime, cached
// per (pointer, shape)).  All maps are uint8 / 2-byte / 4-byte element tiles.
struct TensorMapKey {
    const void *base;
    uint64_t dims[4];
    uint64_t strides[3];  // bytes, dims 1..3
    uint32_t box[4];
    uint32_t rank, elemBytes, swizzle;  // swizzle: 0 none, 1 32B, 2 64B, 3 128B
    uint32_t pad_;                      // keeps the struct free of implicit padding (it is memcmp'd)
};
int getTensorMap(const TensorMapKey &key, CUtensorMap *out);

#ifdef __CUDACC__

// ---- mbarrier ----------------------------------------------------------------
constexpr uint32_t kMbarSuspendNs = 20000u;  // upper bound of one hardware-parked poll
__device__ __forceinline__ uint32_t smemAddr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarInit(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarExpectTx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbarArrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}
// One poll of a phase.  The suspend-time hint lets the hardware park the thread until the phase
// completes (or the hint runs out) instead of returning at once: a block here has a dozen warps
// waiting for one another most of the time, and warps that spin through an unhinted try_wait
// take the issue slots of the few warps that have work (measured on the int8 decode kernel).
__device__ __forceinline__ bool mbarTryWait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smemAddr(bar)), "r"(parity), "r"(kMbarSuspendNs)
            : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and records `errBit`) after ~2^26 failed polls
// (each poll may itself suspend for a hardware-chosen time), so a lost arrival
// never turns into an endless spin on a shared GPU.
__device__ __forceinline__ bool mbarWait(uint64_t *bar, uint32_t parity, unsigned int *err,
                                         uint32_t errBit) {
    for (uint32_t i = 0; i < (1u << 26); ++i) {
        if (mbarTryWait(bar, parity)) return true;
    }
    atomicOr(err, errBit);
    return false;
}
__device__ __forceinline__ void fenceBarrierInit() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fenceProxyAsync() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA -----------------------------------------------------------------------
__device__ __forceinline__ void tmaPrefetchDesc(const CUtensorMap *m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tile load global -> shared, completion counted in bytes on `bar`.  The
// innermost coordinate c0 must be a multiple of 16 bytes of elements.
__device__ __forceinline__ void tmaLoad3D(void *dst, const CUtensorMap *m, uint64_t *bar, int c0, int c1,
                                          int c2) {
    asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smemAddr(dst)),
            "l"(reinterpret_cast<uint64_t>(m)), "r"(smemAddr(bar)), "r"(c0), "r"(c1), "r"(c2)
            : "memory");
}
// L2 eviction policies for streaming data: evict_first for rows that are read once, evict_last for
// rows fetched ahead of their use.
__device__ __forceinline__ uint64_t l2PolicyEvictFirst() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2PolicyEvictLast() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tmaLoad3DHint(void *dst, const CUtensorMap *m, uint64_t *bar, int c0, int c1, int c2,
                                              uint64_t policy) {
    asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%3, %4, %5}], [%2], %6;" ::"r"(smemAddr(dst)),
            "l"(reinterpret_cast<uint64_t>(m)), "r"(smemAddr(bar)), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
            : "memory");
}
__device__ __forceinline__ void tmaPrefetchL2_3DHint(const CUtensorMap *m, int c0, int c1, int c2, uint64_t policy) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile.L2::cache_hint [%0, {%1, %2, %3}], %4;" ::"l"(
                         reinterpret_cast<uint64_t>(m)),
                 "r"(c0), "r"(c1), "r"(c2), "l"(policy)
                 : "memory");
}
// The same tile pulled into L2 only (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tmaPrefetchL2_3D(const CUtensorMap *m, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(
                         reinterpret_cast<uint64_t>(m)),
                 "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tmaLoad2D(void *dst, const CUtensorMap *m, uint64_t *bar, int c0, int c1) {
    asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4}], [%2];" ::"r"(smemAddr(dst)),
            "l"(reinterpret_cast<uint64_t>(m)), "r"(smemAddr(bar)), "r"(c0), "r"(c1)
            : "memory");
}
__device__ __forceinline__ void tmaLoad4D(void *dst, const CUtensorMap *m, uint64_t *bar, int c0, int c1,
                                          int c2, int c3) {
    asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smemAddr(dst)),
            "l"(reinterpret_cast<uint64_t>(m)), "r"(smemAddr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
            : "memory");
}

// ---- cp.async (4-byte, for the scale columns riding in the same stage) -------------
__device__ __forceinline__ void cpAsync4(void *dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smemAddr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cpAsyncMbarArriveNoinc(uint64_t *bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smemAddr(bar)) : "memory");
}

// ---- warp-level matrix helpers -----------------------------------------------------
__device__ __forceinline__ void ldmatrixX4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3,
                                           uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrixX4Trans(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3,
                                                uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrixTrans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mmaF16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8,f32) += A(16x8,tf32,row) * B(8x8,tf32,col)
__device__ __forceinline__ void mmaTf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
            "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t toTf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

// ---- exact int8 -> fp16 ----------------------------------------------------------
// w holds four int8 already xor-ed with 0x80 (i.e. x + 128 as unsigned bytes).
// Bytes (b0, b1) become the fp16 pair (x0, x1): 0x6400 | u is 1024 + u exactly,
// minus 1152 gives x.  Two instructions per pair, no rounding anywhere.
__device__ __forceinline__ uint32_t biasedPairLo(uint32_t w) {
    uint32_t h = __byte_perm(w, 0x64646464u, 0x4140);
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&h), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t biasedPairHi(uint32_t w) {
    uint32_t h = __byte_perm(w, 0x64646464u, 0x4342);
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&h), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<uint32_t *>(&r);
}

// Cheaper exact form used by the decode kernel: a byte u placed in the low mantissa
// bits of an fp16 with zero exponent IS the subnormal u * 2^-24, exactly.  With
// u = x + 128 (w already xor-ed with 0x80) the operand carries a +128 offset that
// the caller removes after the MMA with a per-column sum; one prmt per pair.
template <uint32_t SEL>
__device__ __forceinline__ uint32_t subnormalPair(uint32_t w) {
    return __byte_perm(w, 0u, SEL);
}

// Programmatic dependent launch: wait for the grids this one depends on (and for
// their memory to be visible) / let the dependent grid start its prologue.
__device__ __forceinline__ void gridDepWait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void gridDepLaunch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t packHalf2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
// x = hi + lo with both parts fp16: the pair carries ~22 mantissa bits.
__device__ __forceinline__ void splitHalf(float x, float &hi, float &lo) {
    hi = __half2float(__float2half_rn(x));
    lo = x - hi;
}

__device__ __forceinline__ float fastExp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void namedBarSync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

#endif  // __CUDACC__

}  // namespace tc
