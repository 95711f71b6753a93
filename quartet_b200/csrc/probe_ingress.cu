// Measurement aid: how many bytes per clock ONE SM can take in through bulk asynchronous copies
// (the mechanism that feeds the GEMM's operand ring), as a function of how many threads issue the
// copies, how large a copy is and how many are in flight.  One CTA per SM; `producers` threads in
// different warps each run their own ring of `stages` buffers over an L2-resident source region;
// a partner thread per producer releases a buffer as soon as it has landed.  Nothing is computed.
//
// Findings on B200 that shaped the GEMM: one issuing thread moves ~62 B/clk with 16 KB copies (it can
// start a copy about every 265 cycles); two or more issuing warps saturate the SM's ingress at
// ~70 B/clk, whatever the copy size above 8 KB; the unloaded issue -> landed -> released round trip of
// a 16 KB copy from L2 is ~645 cycles.  Full-rate MXFP4 MMAs on 256 x 256 tiles need 67 B/clk.
#include "common.cuh"

namespace quartet {

constexpr int PROBE_THREADS = 256;
constexpr int PROBE_MAX_PRODUCERS = 4;
constexpr int PROBE_MAX_SMS = 1024;  // size of the host read-back buffer (a local array of the call)

__global__ void __launch_bounds__(PROBE_THREADS, 1)
    probe_ingress_kernel(const uint8_t* __restrict__ src, uint64_t region, int iters, int stages, uint32_t chunk, int producers,
                         long long* __restrict__ cycles) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)producers * stages * chunk);
    unsigned long long* s_elapsed = reinterpret_cast<unsigned long long*>(bars + 2 * producers * stages);
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2 * producers * stages; ++i) mbar_init(&bars[i], 1);
        *s_elapsed = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const long long t0 = clock64();
    if (lane == 0 && w < producers) {
        uint64_t* full = bars + w * 2 * stages;
        uint64_t* empty = full + stages;
        uint8_t* buf = smem + (size_t)w * stages * chunk;
        // Source offsets walk over `slots` chunk-sized, chunk-aligned positions (chunk is a multiple of 128
        // bytes), always reduced modulo `slots`: every copy lies inside [src, src + region) and starts on a
        // 128-byte boundary whatever the region size.
        const uint64_t slots = region / chunk;
        uint64_t slot = ((uint64_t)blockIdx.x * 7919u + (uint64_t)w * 104729u) % slots;
        int s = 0;
        uint32_t ph = 0;
        for (int k = 0; k < iters; ++k) {
            if (!mbar_wait(&empty[s], ph ^ 1, WAIT_QUANT_LOAD)) break;
            mbar_arrive_expect_tx(&full[s], chunk);
            bulk_load(buf + (size_t)s * chunk, src + slot * chunk, chunk, &full[s]);
            slot = (slot + 149u) % slots;
            if (++s == stages) s = 0, ph ^= 1;
        }
    } else if (lane == 0 && w >= PROBE_MAX_PRODUCERS && w < PROBE_MAX_PRODUCERS + producers) {
        uint64_t* full = bars + (w - PROBE_MAX_PRODUCERS) * 2 * stages;
        uint64_t* empty = full + stages;
        int s = 0;
        uint32_t ph = 0;
        for (int k = 0; k < iters; ++k) {
            if (!mbar_wait(&full[s], ph, WAIT_QUANT_LOAD)) break;
            mbar_arrive(&empty[s]);
            if (++s == stages) s = 0, ph ^= 1;
        }
        // the CTA's time is that of its slowest ring
        atomicMax(s_elapsed, (unsigned long long)(clock64() - t0));
    }
    __syncthreads();
    if (threadIdx.x == 0) cycles[blockIdx.x] = (long long)*s_elapsed;
}

// Self-test of the give-up path every kernel of the library shares: one CTA waits, with a short poll limit, on a
// barrier that nothing will ever complete.  The wait runs out, records itself in the fault word and the kernel
// returns normally -- no copy is in flight, no tensor memory is held, the context stays usable.
__global__ void wait_timeout_selftest_kernel(uint32_t poll_limit, int* __restrict__ gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait(&bar, 0, WAIT_QUANT_LOAD, poll_limit);  // phase 0 never completes
        if (gave_up) *gave_up = ok ? 0 : 1;
    }
}

QUARTET_DEFINE_STATUS_READER(status_probe)

}  // namespace quartet

using namespace quartet;

// Scratch of the allocation-free entry point: one cycle count per SM, at most PROBE_STATIC_SMS of them.
// The array is part of the library image, so every GPU that loads the library holds these 2 KB until
// the process exits.  All calls on a device share it.
constexpr int PROBE_STATIC_SMS = 256;
static __device__ __align__(256) long long g_probe_cycles[PROBE_STATIC_SMS];

static int run_probe(const void* src, uint64_t region, int32_t iters, int32_t stages, int32_t chunk, int32_t producers,
                     long long* cycles, int sms, double* bytes_per_clk_per_sm, cudaStream_t s) {
    const size_t smem = (size_t)producers * stages * chunk + 2 * (size_t)producers * stages * 8 + 64;
    int rc = check_cuda(cudaFuncSetAttribute(probe_ingress_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "cudaFuncSetAttribute");
    if (rc) return rc;
    probe_ingress_kernel<<<sms, PROBE_THREADS, smem, s>>>(static_cast<const uint8_t*>(src), region, iters, stages, (uint32_t)chunk, producers, cycles);
    if ((rc = check_cuda(cudaGetLastError(), "probe launch"))) return rc;
    if ((rc = check_cuda(cudaStreamSynchronize(s), "probe run"))) return rc;
    long long host[PROBE_MAX_SMS];
    if ((rc = check_cuda(cudaMemcpy(host, cycles, sizeof(long long) * sms, cudaMemcpyDeviceToHost), "probe read-back"))) return rc;
    long long worst = 1;
    for (int i = 0; i < sms; ++i) worst = host[i] > worst ? host[i] : worst;
    *bytes_per_clk_per_sm = (double)iters * chunk * producers / (double)worst;
    return QUARTET_OK;
}

static int validate_probe(const void* src, uint64_t region, int32_t iters, int32_t stages, int32_t chunk, int32_t producers,
                          const void* result, int* sms) {
    if (!src || !result) return fail(QUARTET_E_NULL, "src and the result pointer must be non-NULL");
    if (producers < 1 || producers > PROBE_MAX_PRODUCERS || stages < 1 || stages > 32 || iters < 1)
        return fail(QUARTET_E_ARG, "need 1..%d producers, 1..32 stages, iters >= 1", PROBE_MAX_PRODUCERS);
    if (chunk < 128 || chunk % 128 || region < 4ull * chunk || (reinterpret_cast<uintptr_t>(src) & 127u))
        return fail(QUARTET_E_ARG, "chunk must be a positive multiple of 128 bytes, region >= 4 chunks, src 128-byte aligned");
    if ((size_t)producers * stages * chunk + 2 * (size_t)producers * stages * 8 + 64 > 220 * 1024)
        return fail(QUARTET_E_ARG, "producers * stages * chunk exceeds the shared memory of an SM");
    int rc = bind_context_of(src);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    if ((rc = device_sm_count(sms))) return rc;
    if (*sms > PROBE_MAX_SMS) return fail(QUARTET_E_ARG, "more SMs than the probe's host buffer holds");
    return QUARTET_OK;
}

// bytes_per_clk_per_sm = iters * chunk * producers / (slowest CTA's cycles).  `src` is a device buffer of
// `region` bytes (keep it below the L2 size to measure the L2 -> SM path), `cycles` a device array of
// one int64 per SM used as scratch for the result.
extern "C" __attribute__((visibility("default"))) int quartet_probe_copy_ingress(const void* src, uint64_t region, int32_t iters, int32_t stages,
                                                                                 int32_t chunk, int32_t producers, int64_t* cycles,
                                                                                 double* bytes_per_clk_per_sm, quartet_stream_t stream) {
    if (!cycles) return fail(QUARTET_E_NULL, "cycles must be non-NULL");
    int sms = 0;
    int rc = validate_probe(src, region, iters, stages, chunk, producers, bytes_per_clk_per_sm, &sms);
    if (rc) return rc;
    return run_probe(src, region, iters, stages, chunk, producers, reinterpret_cast<long long*>(cycles), sms, bytes_per_clk_per_sm,
                     static_cast<cudaStream_t>(stream));
}

// The same measurement for callers that must not allocate device memory while they run: code inside a
// region where the framework's caching allocator is frozen (a memory-pool snapshot, a stream capture in
// progress elsewhere in the process), a plugin that was handed fixed buffers by its host application, or
// a monitoring hook that runs when the device is nearly full and a cudaMalloc would fail or synchronise.
// The kernel's scratch (one cycle count per SM) is the file-scope device array above instead of a caller
// workspace; this call and everything below it call no cudaMalloc / cudaFree and no allocating library.
//   * Limit: devices with more than 256 SMs are rejected with QUARTET_E_ARG.
//   * Set-up: the FIRST call of a thread on a device looks up the array's device address
//     (cudaGetSymbolAddress, checked) with that device current and keeps it; make that first call
//     before any stream capture begins.
//   * Sharing: every call on a device writes the same array (the kernel overwrites all entries it reads
//     back, so nothing needs clearing), and the array keeps the last call's counts.  Calls that overlap
//     on the GPU -- two streams, two host threads -- race on it; the caller serialises them.
extern "C" __attribute__((visibility("default"))) int quartet_probe_copy_ingress_noalloc(const void* src, uint64_t region, int32_t iters,
                                                                                         int32_t stages, int32_t chunk, int32_t producers,
                                                                                         double* bytes_per_clk_per_sm, quartet_stream_t stream) {
    int sms = 0;
    int rc = validate_probe(src, region, iters, stages, chunk, producers, bytes_per_clk_per_sm, &sms);
    if (rc) return rc;
    if (sms > PROBE_STATIC_SMS)
        return fail(QUARTET_E_ARG, "the device has %d SMs, the built-in scratch array holds %d", sms, PROBE_STATIC_SMS);
    static thread_local int cached_dev = -1;
    static thread_local long long* scratch = nullptr;
    int dev = 0;
    if ((rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice"))) return rc;
    if (dev != cached_dev) {  // set-up: the symbol's address on this device
        void* addr = nullptr;
        if ((rc = check_cuda(cudaGetSymbolAddress(&addr, g_probe_cycles), "cudaGetSymbolAddress"))) return rc;
        scratch = static_cast<long long*>(addr), cached_dev = dev;
    }
    return run_probe(src, region, iters, stages, chunk, producers, scratch, sms, bytes_per_clk_per_sm, static_cast<cudaStream_t>(stream));
}

// Launches the self-test above (poll limit 4096: well under a millisecond).  Afterwards quartet_device_status()
// reports a non-zero fault word whose low byte names a load wait, and every other entry point keeps working.
extern "C" __attribute__((visibility("default"))) int quartet_selftest_wait_timeout(int32_t* gave_up_dev, quartet_stream_t stream) {
    if (gave_up_dev) {
        int rc = bind_context_of(gave_up_dev);
        if (rc) return rc;
    }
    int rc = check_device();
    if (rc) return rc;
    wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(4096u, gave_up_dev);
    return check_cuda(cudaGetLastError(), "self-test launch");
}
