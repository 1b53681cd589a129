// Host-side runtime pieces shared by all kernels: the device status word that bounded
// waits and argument checks write to, and the TMA tensor-map factory.
//
// The driver entry point cuTensorMapEncodeTiled is resolved at run time through the CUDA
// runtime so the library links against nothing but the (static) runtime and still loads on
// a machine without a GPU driver.
#include "common.cuh"
#include <cudaTypedefs.h>
#include <mutex>
#include <unordered_map>
#include <string>
#include <string.h>

#ifdef LLMC_DEBUG_CHECKS
__device__ unsigned int* g_llmc_dbg_status = nullptr;      // where the checks of the debug build report (this device's status word)
extern "C" int llmc_debug_checks_enabled() { return 1; }
#else
extern "C" int llmc_debug_checks_enabled() { return 0; }
#endif

static unsigned int* g_status_dev[64] = {nullptr};
static std::mutex g_mu;

// Device pointer to this device's status word (allocated on first use).
extern "C" unsigned int* llmc_status_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_status_dev[dev]) {
        unsigned int* p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, 256);
#ifdef LLMC_DEBUG_CHECKS
        if (cudaMemcpyToSymbol(g_llmc_dbg_status, &p, sizeof(p)) != cudaSuccess) return nullptr;
#endif
        g_status_dev[dev] = p;
    }
    return g_status_dev[dev];
}

// Read (and optionally clear) the status word. Synchronises the device.
extern "C" int llmc_status_read(int clear, unsigned int* out) {
    unsigned int* p = llmc_status_ptr();
    if (!p) return -1;
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpy(out, p, sizeof(unsigned int), cudaMemcpyDeviceToHost));
    if (clear) CUDA_CHECK(cudaMemset(p, 0, sizeof(unsigned int)));
    return 0;
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
        }
    }
    return fn;
}

struct MapKey {
    uint64_t v[16];
    bool operator==(const MapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = 1469598103934665603ull;
        for (int i = 0; i < 16; i++) { h ^= k.v[i]; h *= 1099511628211ull; }
        return (size_t)h;
    }
};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

int llmc_get_tensormap(CUtensorMap* out, const void* base, int elem_bytes, int rank,
                       const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
    if (rank < 2 || rank > 4) return -2;
    MapKey key; memset(&key, 0, sizeof(key));
    key.v[0] = (uint64_t)base; key.v[1] = ((uint64_t)elem_bytes << 32) | ((uint64_t)rank << 8) | (uint64_t)swizzle;
    for (int i = 0; i < rank; i++) { key.v[2 + i] = dims[i]; key.v[6 + i] = (i > 0) ? strides_bytes[i] : 0; key.v[10 + i] = box[i]; }
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_maps.find(key);
        if (it != g_maps.end()) { *out = it->second; return 0; }
    }
    auto fn = get_encode_fn();
    if (!fn) { fprintf(stderr, "[llmc_b200] cuTensorMapEncodeTiled unavailable\n"); return -3; }
    if (((uint64_t)base & 15) != 0) { fprintf(stderr, "[llmc_b200] tensor map base %p not 16-byte aligned\n", base); return -4; }
    cuuint64_t gdims[4]; cuuint64_t gstr[3]; cuuint32_t gbox[4]; cuuint32_t estr[4];
    for (int i = 0; i < rank; i++) { gdims[i] = dims[i]; gbox[i] = box[i]; estr[i] = 1; }
    for (int i = 1; i < rank; i++) {
        gstr[i - 1] = strides_bytes[i];
        if (strides_bytes[i] % 16 != 0) { fprintf(stderr, "[llmc_b200] tensor map stride %llu not a multiple of 16\n", (unsigned long long)strides_bytes[i]); return -5; }
    }
    CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 :
                             elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CUtensorMapSwizzle sw = swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B :
                            swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstr, gbox, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "[llmc_b200] cuTensorMapEncodeTiled failed (%d): rank %d dims %llu %llu box %u %u\n", (int)r, rank,
                (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
        return -6;
    }
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_maps.size() > 65536) g_maps.clear();
    g_maps[key] = *out;
    return 0;
}

// Drop all cached tensor maps (call after freeing buffers whose addresses may be reused with other shapes).
extern "C" void llmc_tensormap_cache_clear() {
    std::lock_guard<std::mutex> lk(g_mu);
    g_maps.clear();
}

extern "C" int llmc_device_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return n;
}

// ----------------------------------------------------------------------------
// Device memory when it fits, managed memory otherwise.
//
// Optimizer state is touched once per step, so when the device is full it can live in managed memory whose preferred home is
// the host: the update kernel then reads and writes it across the host link instead of the run ending with an allocation
// error (capability parity with cudaMallocConditionallyManaged, llmc/cuda_utils.cuh:213-229 of the reference).
// *managed is set to 1 if the fallback was taken.  force_managed skips the device attempt (used by the tests).
extern "C" int llmc_alloc_device_or_managed(void** out, size_t bytes, int force_managed, int* managed) {
    if (!out || !managed || bytes == 0) return -1;
    *out = nullptr;
    *managed = 0;
    if (!force_managed) {
        cudaError_t e = cudaMalloc(out, bytes);
        if (e == cudaSuccess) return 0;
        (void)cudaGetLastError();                       // clear the sticky-free allocation error before trying again
        if (e != cudaErrorMemoryAllocation) {
            fprintf(stderr, "[llmc_b200] cudaMalloc(%zu): %s\n", bytes, cudaGetErrorString(e));
            return -1;
        }
    }
    int dev = 0;
    CUDA_CHECK(cudaGetDevice(&dev));
    CUDA_CHECK(cudaMallocManaged(out, bytes, cudaMemAttachGlobal));
    // advice is best effort: a platform that rejects it still has working managed memory
    if (cudaMemAdvise(*out, bytes, cudaMemAdviseSetPreferredLocation, cudaCpuDeviceId) != cudaSuccess) (void)cudaGetLastError();
    if (cudaMemAdvise(*out, bytes, cudaMemAdviseSetAccessedBy, dev) != cudaSuccess) (void)cudaGetLastError();
    *managed = 1;
    return 0;
}

extern "C" int llmc_free_device_or_managed(void* p) {
    if (p) CUDA_CHECK(cudaFree(p));
    return 0;
}
