// tc_runtime.cu -- host-side plumbing shared by every entry point of the C ABI:
// thread-local error text, the per-device error word that kernels with bounded
// waits report into, SM count, and a cached factory for TMA tensor maps.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "tc_common.cuh"

namespace tc {

static thread_local char t_err[512] = "";

void setError(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
}

int cudaFail(cudaError_t e, const char *what) {
    setError("%s failed: %s", what, cudaGetErrorString(e));
    return TC_ECUDA;
}

__device__ unsigned int g_devErrorStorage = 0;

unsigned int *devErrorWord() {
    // One address per device; resolved lazily with that device current.
    static std::mutex mu;
    static unsigned int *addr[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (addr[dev] == nullptr) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_devErrorStorage) != cudaSuccess) return nullptr;
        addr[dev] = static_cast<unsigned int *>(p);
    }
    return addr[dev];
}

int numSMs() {
    static std::mutex mu;
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lk(mu);
    if (sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    return sms[dev];
}

// ---- tensor maps ---------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encodeFn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    });
    return fn;
}

struct CacheEntry {
    int dev;
    TensorMapKey key;
    CUtensorMap map;
};

// The cache is a fixed ring (no heap growth): entry points that promise not to
// allocate go through here too.
int getTensorMap(const TensorMapKey &key, CUtensorMap *out) {
    static std::mutex mu;
    constexpr int kSlots = 256;
    static CacheEntry cache[kSlots];
    static int used = 0, next = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lk(mu);
        for (int i = 0; i < used; ++i) {
            if (cache[i].dev == dev && std::memcmp(&cache[i].key, &key, sizeof(key)) == 0) {
                *out = cache[i].map;
                return TC_OK;
            }
        }
    }
    EncodeTiledFn fn = encodeFn();
    TC_REQUIRE(fn != nullptr, TC_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMapDataType dt = key.elemBytes == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                             : key.elemBytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    cuuint64_t dims[4];
    cuuint64_t strides[3];
    cuuint32_t box[4], estr[4];
    for (uint32_t i = 0; i < key.rank; ++i) {
        dims[i] = key.dims[i];
        box[i] = key.box[i];
        estr[i] = 1;
    }
    for (uint32_t i = 0; i + 1 < key.rank; ++i) strides[i] = key.strides[i];
    CUtensorMapSwizzle sw = key.swizzle == 3   ? CU_TENSOR_MAP_SWIZZLE_128B
                            : key.swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : key.swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                               : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUtensorMap m;
    CUresult r = fn(&m, dt, key.rank, const_cast<void *>(key.base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TC_REQUIRE(r == CUDA_SUCCESS, TC_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int) r);
    {
        std::lock_guard<std::mutex> lk(mu);
        CacheEntry &e = cache[next];
        e.dev = dev;
        e.key = key;
        e.map = m;
        next = (next + 1) % kSlots;
        if (used < kSlots) ++used;
    }
    *out = m;
    return TC_OK;
}

}  // namespace tc

extern "C" {

const char *tc_strerror(int code) {
    switch (code) {
        case TC_OK: return "ok";
        case TC_EINVAL: return "invalid argument";
        case TC_ECONTEXT_FULL: return "context window full";
        case TC_ECUDA: return "CUDA call failed";
        case TC_EUNSUPPORTED: return "unsupported shape";
        case TC_EWORKSPACE: return "workspace too small";
        case TC_EDEVICE: return "device-side wait ran out";
        default: return "unknown";
    }
}

const char *tc_last_error(void) { return tc::t_err; }

int tc_device_status(tc_stream stream, uint32_t *flags) {
    unsigned int *w = tc::devErrorWord();
    TC_REQUIRE(w != nullptr, TC_ECUDA, "no CUDA device");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned int v = 0;
    TC_CUDA_OK(cudaMemcpyAsync(&v, w, sizeof(v), cudaMemcpyDeviceToHost, st));
    TC_CUDA_OK(cudaStreamSynchronize(st));
    if (v != 0) TC_CUDA_OK(cudaMemsetAsync(w, 0, sizeof(v), st));
    if (flags) *flags = v;
    if (v != 0) {
        tc::setError("a kernel gave up on a bounded wait (flags 0x%x)", v);
        return TC_EDEVICE;
    }
    return TC_OK;
}

}  // extern "C"
