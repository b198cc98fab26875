// Host-side helpers shared by the TMA-fed kernel files: the tensor-map builder, the test of
// whether TMA can address an array set, the SM count of the current device, and the
// process-wide options of the test / profiling hook prb_debug_set.
#include "kernels.h"
#include "tma.cuh"

namespace prb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

bool make_tile_map(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint32_t mid,
                   uint64_t inner, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || !base) return false;
    if (reinterpret_cast<uintptr_t>(base) & 15u) return false;
    if ((inner * elem_bytes) & 15u) return false;
    if (box_rows > 256 || mid > 256) return false;
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                   : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    cuuint64_t dims[3] = {inner, mid, rows};
    cuuint64_t strides[2] = {inner * elem_bytes, inner * elem_bytes * mid};
    cuuint32_t box[3] = {32, mid, box_rows};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tma_addressable(int dtype, int B, int T, int d) {
    const int elem = dtype == kF32 ? 4 : 2;
    if ((d * elem) & 15) return false;                  // stride rule for wx / states rows
    if ((long long)B * T > 0x7fffff00LL) return false;  // the row coordinate is a 32-bit int
    return encode_fn() != nullptr;
}

int sm_count() {
    constexpr int kMaxDev = 64;
    static int cached[kMaxDev] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

Options& options() {
    static Options o;
    return o;
}

}  // namespace prb
