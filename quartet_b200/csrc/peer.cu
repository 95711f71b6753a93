// Weight-gradient shards across GPUs without a library collective on the data path.
//
// Each rank owns a row range of every weight gradient.  The wgrad GEMM of rank r stores the rows that
// rank o owns straight into slot r of o's receive buffer (TMA stores over NVLink, see the scattered
// GEMM entry point); after a stream-ordered barrier among the ranks, the owner sums its slots with the
// kernel below.  This file holds the receive-buffer plumbing (CUDA IPC) and that sum.
//
// The reference leaves this exchange to torch DDP's bucketed all-reduce of full gradients
// (src/main.py:79-85, src/optim/base.py:190-200 of the reference tree).
#include <string.h>

#include "common.cuh"

namespace quartet {

// out[i] = scale * (slot_0[i] + slot_1[i] + ... ), slots summed in index order (deterministic).
// HBM-bound: (n_slots + 1) * 4 bytes per output element.
__global__ void __launch_bounds__(256) shard_reduce_kernel(const float4* __restrict__ slots, int n_slots, int64_t slot_vec4,
                                                           float scale, float4* __restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < slot_vec4; i += stride) {
        float4 acc = __ldcs(slots + i);
        for (int s = 1; s < n_slots; ++s) {
            const float4 v = __ldcs(slots + (int64_t)s * slot_vec4 + i);
            acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
        }
        out[i] = make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
    }
}

}  // namespace quartet

using namespace quartet;

extern "C" __attribute__((visibility("default"))) int quartet_shard_reduce(const float* slots, int32_t n_slots, int64_t slot_elems,
                                                                           float scale, float* out, quartet_stream_t stream) {
    if (!slots || !out) return fail(QUARTET_E_NULL, "slots and out must be non-NULL");
    if (n_slots < 1 || n_slots > 64) return fail(QUARTET_E_ARG, "n_slots must be 1..64 (got %d)", n_slots);
    if (slot_elems < 4 || slot_elems % 4) return fail(QUARTET_E_SHAPE, "slot_elems must be a positive multiple of 4");
    if (!aligned16(slots) || !aligned16(out)) return fail(QUARTET_E_ALIGN, "slots and out must be 16-byte aligned");
    int rc = bind_context_of(out);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    int sms = 0;
    if ((rc = device_sm_count(&sms))) return rc;
    const int64_t vec4 = slot_elems / 4;
    int64_t blocks = (vec4 + 255) / 256;
    const int64_t cap = (int64_t)sms * 8;  // a whole number of waves of 8 CTAs per SM
    if (blocks > cap) blocks = cap;
    shard_reduce_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(slots), n_slots, vec4, scale, reinterpret_cast<float4*>(out));
    return check_cuda(cudaGetLastError(), "shard_reduce launch");
}

// --- receive buffers that peers can map -------------------------------------------------------
// Allocated with cudaMalloc directly (not from a caching allocator) so that the IPC handle names
// exactly this buffer at offset 0.
extern "C" __attribute__((visibility("default"))) int quartet_peer_alloc(uint64_t bytes, void** ptr, void* handle64) {
    if (!ptr || !handle64) return fail(QUARTET_E_NULL, "ptr and handle64 must be non-NULL");
    if (bytes == 0) return fail(QUARTET_E_ARG, "bytes must be positive");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 opaque bytes");
    int rc = check_cuda(cudaMalloc(ptr, bytes), "cudaMalloc (peer buffer)");
    if (rc) return rc;
    cudaIpcMemHandle_t h;
    if ((rc = check_cuda(cudaIpcGetMemHandle(&h, *ptr), "cudaIpcGetMemHandle"))) {
        cudaFree(*ptr);
        *ptr = nullptr;
        return rc;
    }
    memcpy(handle64, &h, 64);
    return QUARTET_OK;
}
extern "C" __attribute__((visibility("default"))) int quartet_peer_free(void* ptr) {
    if (!ptr) return QUARTET_OK;
    return check_cuda(cudaFree(ptr), "cudaFree (peer buffer)");
}
extern "C" __attribute__((visibility("default"))) int quartet_peer_open(const void* handle64, void** ptr) {
    if (!handle64 || !ptr) return fail(QUARTET_E_NULL, "handle64 and ptr must be non-NULL");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    return check_cuda(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}
extern "C" __attribute__((visibility("default"))) int quartet_peer_close(void* ptr) {
    if (!ptr) return QUARTET_OK;
    return check_cuda(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle");
}
// Device-to-device copy on the DMA engines (no SM is used): local rows -> a slot in a peer's buffer.
extern "C" __attribute__((visibility("default"))) int quartet_peer_copy(void* dst, const void* src, uint64_t bytes, quartet_stream_t stream) {
    if (!dst || !src) return fail(QUARTET_E_NULL, "dst and src must be non-NULL");
    if (bytes == 0) return QUARTET_OK;
    return check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)), "cudaMemcpyAsync (peer copy)");
}
