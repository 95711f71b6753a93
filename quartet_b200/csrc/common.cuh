// Shared device/host helpers for the sm_100a kernels: error reporting, mbarrier /
// TMA / bulk-copy PTX wrappers with bounded waits, tensor-map construction.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/quartet_b200.h"

namespace quartet {

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
int fail(int code, const char* fmt, ...);  // records the thread-local error string, returns `code`
int check_cuda(cudaError_t e, const char* what);
int check_device();                          // QUARTET_OK iff the current device is sm_100
int bind_context_of(const void* ptr);        // make the context of ptr's device current if the thread has none
int device_sm_count(int* sms);               // SMs of the current device (cached per thread)

// 2-D row-major tensor map over bytes/elements.  `swizzle`: 0 none, 1 = 32B, 2 = 64B, 3 = 128B.
int make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle);

// Each translation unit with kernels has its own fault word and exports a reader that ORs it
// into *out and clears it.
int status_rows(int32_t* out);
int status_tile_t(int32_t* out);
int status_gemm(int32_t* out);
int status_aux(int32_t* out);
int status_probe(int32_t* out);
int status_producer(int32_t* out);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel instantiation, thread and device instead of
// before every launch.  `state` is a thread_local int of the calling (template) function, initialised to -1.
template <typename K>
static inline int set_max_smem_once(K kernel, int bytes, int& state) {
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc || state == dev) return rc;
    if ((rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), "cudaFuncSetAttribute"))) return rc;
    state = dev;
    return QUARTET_OK;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------
// device side
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

static __device__ int32_t g_status;  // fault word of this translation unit

#define QUARTET_DEFINE_STATUS_READER(NAME)                                                          \
    int NAME(int32_t* out) {                                                                        \
        int32_t v = 0, z = 0;                                                                       \
        int rc = check_cuda(cudaMemcpyFromSymbol(&v, g_status, sizeof(v)), "read fault word");      \
        if (rc) return rc;                                                                          \
        if (v) rc = check_cuda(cudaMemcpyToSymbol(g_status, &z, sizeof(z)), "clear fault word");    \
        *out |= v;                                                                                  \
        return rc;                                                                                  \
    }

// Which bounded wait gave up (low byte of the fault word).
enum : int32_t {
    WAIT_QUANT_LOAD = 1,
    WAIT_GEMM_FULL = 2,
    WAIT_GEMM_EMPTY = 3,
    WAIT_GEMM_ACC_FULL = 4,
    WAIT_GEMM_ACC_EMPTY = 5,
    WAIT_GEMM_SF = 6,
    WAIT_GEMM_ALIGN = 7,  // not a wait: dynamic shared memory was not 1024-byte aligned
};

// Programmatic dependent launch.  A kernel launched with launch_pdl() may become resident while the
// kernel before it in the stream is still draining; pdl_wait() returns once that kernel has completed
// and its writes are visible, so everything before it (barrier init, tensor-map prefetch, TMEM
// allocation) overlaps the predecessor's tail and the launch latency.  No global memory is touched
// before pdl_wait().  pdl_launch_dependents() lets the NEXT kernel do the same with this one.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~`limit` polls, records `who` in the fault word and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int32_t who, uint32_t limit = (1u << 24)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    atomicOr(&g_status, who | 0x100);
    return false;
}

// --- TMA (tensor) copies; no cluster multicast anywhere in this library ---
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(src)), "r"(x), "r"(y)
                 : "memory");
}
// --- the same copies with an L2 eviction-priority hint ---
// Operand tiles of a GEMM are re-read by many CTAs and should stay in L2 (evict_last).  (A hint on the
// result's stores bought nothing locally and made stores into another GPU's memory several times slower.)
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void bulk_load_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
// --- untiled bulk copies (16-byte aligned, size % 16 == 0) ---
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

#endif  // __CUDACC__

}  // namespace quartet
