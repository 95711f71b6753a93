// Host-side plumbing of the C ABI: error strings, device check, tensor-map construction,
// layout helpers.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace quartet {

static thread_local char t_err[512] = "no error";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return QUARTET_OK;
    return fail(QUARTET_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// The calling thread may have no CUDA context bound yet (PyTorch's autograd worker threads bind one
// lazily, and this library carries its own statically linked runtime): bind the primary context of
// the device that owns `ptr` before anything that needs a current context (tensor-map encoding,
// launches).  Cheap when a context is already current.
int bind_context_of(const void* ptr) {
    typedef CUresult (*GetCurFn)(CUcontext*);
    typedef CUresult (*PtrAttrFn)(void*, CUpointer_attribute, CUdeviceptr);
    static GetCurFn get_cur = nullptr;
    static PtrAttrFn ptr_attr = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            get_cur = reinterpret_cast<GetCurFn>(p);
        if (cudaGetDriverEntryPoint("cuPointerGetAttribute", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            ptr_attr = reinterpret_cast<PtrAttrFn>(p);
    });
    if (!get_cur || !ptr_attr) return fail(QUARTET_E_CUDA, "driver entry points unavailable");
    CUcontext ctx = nullptr;
    if (get_cur(&ctx) == CUDA_SUCCESS && ctx != nullptr) return QUARTET_OK;
    int ordinal = -1;
    if (ptr_attr(&ordinal, CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS || ordinal < 0)
        return fail(QUARTET_E_CUDA, "pointer %p is not device memory", ptr);
    return check_cuda(cudaSetDevice(ordinal), "cudaSetDevice");
}

int check_device() {
    static thread_local int cached_dev = -1;
    static thread_local int cached_ok = 0;
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev == cached_dev) return cached_ok ? QUARTET_OK : fail(QUARTET_E_DEVICE, "device %d is not sm_100", dev);
    int major = 0, minor = 0;
    rc = check_cuda(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev), "cudaDeviceGetAttribute");
    if (rc) return rc;
    rc = check_cuda(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev), "cudaDeviceGetAttribute");
    if (rc) return rc;
    cached_dev = dev;
    cached_ok = (major == 10 && minor == 0);
    return cached_ok ? QUARTET_OK : fail(QUARTET_E_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev, major, minor);
}

int device_sm_count(int* sms) {
    static thread_local int cached_dev = -1, cached_sms = 0;
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev != cached_dev) {
        if ((rc = check_cuda(cudaDeviceGetAttribute(&cached_sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute"))) return rc;
        cached_dev = dev;
    }
    *sms = cached_sms;
    return QUARTET_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(QUARTET_E_CUDA, "cuTensorMapEncodeTiled not available from the driver");
    (void)elem_bytes;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    static const CUtensorMapSwizzle sw[4] = {CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                                             CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_SWIZZLE_128B};
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    sw[swizzle & 3], CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(QUARTET_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for %llu x %llu, stride %llu, box %u x %u", (int)r,
                    (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_stride_bytes, box_inner,
                    box_outer);
    return QUARTET_OK;
}

}  // namespace quartet

using namespace quartet;

extern "C" __attribute__((visibility("default"))) int64_t quartet_sf_offset(int64_t row, int64_t kblock, int64_t padded_kblocks) {
    const int64_t block = (row / 128) * (padded_kblocks / 4) + kblock / 4;
    const int64_t r = row % 128;
    return block * 512 + (r % 32) * 16 + (r / 32) * 4 + kblock % 4;
}

extern "C" __attribute__((visibility("default"))) int64_t quartet_sf_bytes(int64_t rows, int64_t cols) {
    const int64_t pr = (rows + 127) / 128 * 128;
    const int64_t pk = (cols / 32 + 3) / 4 * 4;
    return pr * pk;
}

extern "C" __attribute__((visibility("default"))) int quartet_device_status(int32_t* status) {
    if (!status) return fail(QUARTET_E_NULL, "status must be non-NULL");
    *status = 0;
    int rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    if (rc) return rc;
    if ((rc = status_rows(status))) return rc;
    if ((rc = status_tile_t(status))) return rc;
    if ((rc = status_gemm(status))) return rc;
    if ((rc = status_aux(status))) return rc;
    if ((rc = status_probe(status))) return rc;
    if ((rc = status_producer(status))) return rc;
    return QUARTET_OK;
}

extern "C" __attribute__((visibility("default"))) const char* quartet_last_error_string(void) { return t_err; }
extern "C" __attribute__((visibility("default"))) int quartet_version(void) { return 100; }
