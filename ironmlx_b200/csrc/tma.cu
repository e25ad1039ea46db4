// Host-side helpers shared by the kernels' launchers: the per-device record
// (SM count, which kernel families have had their attributes set on which
// device) and the tiled tensor-map encoder with a small cache.
#include <cuda.h>

#include <atomic>
#include <cstring>
#include <mutex>

#include "internal.h"

namespace imx {

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_dev_mu;
int g_sms[kMaxDevices] = {};
unsigned g_setup[kMaxDevices] = {};       // bit per kernel family (kSetup*)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// What a tensor map is made from: a map is a pure function of these.
struct MapKey {
    const void* base;
    size_t rows, cols, ld_bytes;
    int dt, esize, box_cols, box_rows, swizzle, promote;
};
struct MapEntry {
    MapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int kMapCache = 64;             // per thread: a forward call encodes at most 20 maps

}  // namespace

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

int current_device(DeviceInfo* out) {
    int dev = 0;
    IMX_CHECK_CUDA(cudaGetDevice(&dev));
    IMX_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d is not supported (maximum %d)", dev, kMaxDevices - 1);
    std::lock_guard<std::mutex> lock(g_dev_mu);
    if (g_sms[dev] == 0) {
        int v = 0;
        IMX_CHECK_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
        g_sms[dev] = v;
    }
    out->ordinal = dev;
    out->sms = g_sms[dev];
    return IMX_OK;
}

bool device_needs_setup(int ordinal, int family) {
    std::lock_guard<std::mutex> lock(g_dev_mu);
    return (g_setup[ordinal] & (1u << family)) == 0;
}

void device_mark_setup(int ordinal, int family) {
    std::lock_guard<std::mutex> lock(g_dev_mu);
    g_setup[ordinal] |= 1u << family;
}

int make_tensor_map_2d(const void* base, CUtensorMapDataType dt, size_t esize, size_t rows, size_t cols,
                       size_t ld_bytes, int box_cols, int box_rows, bool swizzle128, CUtensorMap* out,
                       bool promote256, int swizzle_bytes) {
    static EncodeTiledFn fn = nullptr;
    static std::mutex fn_mu;
    {
        std::lock_guard<std::mutex> lock(fn_mu);
        if (fn == nullptr) {
            void* p = nullptr;
            cudaDriverEntryPointQueryResult q;
            IMX_CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
            IMX_REQUIRE(p != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available");
            fn = (EncodeTiledFn)p;
        }
    }
    IMX_REQUIRE(((uintptr_t)base % 16) == 0 && ld_bytes % 16 == 0 && (box_cols * esize) % 16 == 0,
                "tensor map: a matrix is not 16-byte aligned (base %p, row pitch %zu)", base, ld_bytes);
    const int swz = swizzle128 ? 128 : swizzle_bytes;
    // A map depends on nothing but its arguments (it holds the address, not the contents): calls with the same
    // weights and workspace reuse the encoding instead of paying the driver call again.
    MapKey key;
    std::memset(&key, 0, sizeof(key));
    key.base = base; key.rows = rows; key.cols = cols; key.ld_bytes = ld_bytes;
    key.dt = (int)dt; key.esize = (int)esize; key.box_cols = box_cols; key.box_rows = box_rows;
    key.swizzle = swz; key.promote = promote256 ? 1 : 0;
    static thread_local MapEntry cache[kMapCache];
    static thread_local int next = 0;
    for (int i = 0; i < kMapCache; ++i)
        if (cache[i].used && std::memcmp(&cache[i].key, &key, sizeof(key)) == 0) {
            *out = cache[i].map;
            return IMX_OK;
        }
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle mode = swz == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                    : (swz == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                 : (swz == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE));
    const CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, mode,
                          promote256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    IMX_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with %d", (int)r);
    MapEntry& e = cache[next];
    next = (next + 1) % kMapCache;
    e.key = key;
    e.map = *out;
    e.used = true;
    return IMX_OK;
}

}  // namespace imx
