// Host-side support of the tensor-core kernels: the per-device status word and TMA tensor maps.
#include "tc_common.cuh"
#include "internal.cuh"

namespace cxxattn {
namespace tc {

namespace {
__device__ int g_status_word = 0;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library has no link-time
// dependency on libcuda (it must load on machines without a driver).
EncodeTiledFn encode_fn() {
    // looked up once, thread-safely (function-local static initialisation)
    static const EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(p);
        return static_cast<EncodeTiledFn>(nullptr);
    }();
    return fn;
}
}  // namespace

int* status_word() {
    static std::atomic<int*> cache[kMaxDevices];
    const int dev = current_device();
    if (dev < 0) return nullptr;
    int* w = cache[dev].load(std::memory_order_relaxed);
    if (w == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        w = static_cast<int*>(p);
        cache[dev].store(w, std::memory_order_relaxed);
    }
    return w;
}

bool make_tmap_bhsd(CUtensorMap* out, const void* base, int B, int S, int H, int Dh, int64_t sb, int64_t ss,
                    int64_t sh, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)Dh, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};  // bytes, dims 1..3
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc
}  // namespace cxxattn
