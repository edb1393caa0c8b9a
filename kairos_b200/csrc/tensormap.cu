// Host-side TMA descriptor construction shared by the kernels.  cuTensorMapEncodeTiled is resolved
// through the runtime (no link-time dependency on libcuda).
#include <cuda.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace kairos {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// A descriptor is a pure function of its arguments (base address, extents, strides, box, swizzle), and a
// layer is called again and again with the same ones, so encoded descriptors are kept in a small
// direct-mapped, per-thread table: a repeated call copies 128 bytes instead of going through the driver.
namespace {
struct TmapKey {
    const void* base;
    uint64_t dims[5], strides[4];
    uint32_t box[5];
    int dt, rank, swizzle;
};
struct TmapSlot {
    TmapKey key;
    CUtensorMap map;
    bool valid = false;
};
constexpr int kTmapSlots = 512;
thread_local TmapSlot g_tmap_cache[kTmapSlots];

inline uint64_t tmap_hash(const TmapKey& k) {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(&k);
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(TmapKey); ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
}
}  // namespace

int make_tmap(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
    TmapKey key;
    std::memset(&key, 0, sizeof(key));
    key.base = base;
    key.dt = (int)dt;
    key.rank = rank;
    key.swizzle = (int)swizzle;
    for (int i = 0; i < rank && i < 5; ++i) {
        key.dims[i] = dims[i];
        key.box[i] = box[i];
        if (i + 1 < rank) key.strides[i] = strides_bytes[i];
    }
    TmapSlot& slot = g_tmap_cache[tmap_hash(key) % kTmapSlots];
    if (slot.valid && std::memcmp(&slot.key, &key, sizeof(key)) == 0) {
        *map = slot.map;
        return KAIROS_OK;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return note_cuda_error(cudaErrorNotSupported);
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        e[i] = 1;
        if (i + 1 < rank) s[i] = strides_bytes[i];
    }
    const CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled rejected the tensor map (alignment or extent)");
        return KAIROS_ERR_CUDA;
    }
    std::memcpy(&slot.key, &key, sizeof(key));
    slot.map = *map;
    slot.valid = true;
    return KAIROS_OK;
}

}  // namespace kairos
