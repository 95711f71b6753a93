// Forward quantizer fused into the elementwise step that produces its input, so that the activation of a
// quantized linear layer is never written to memory in bf16 / fp32:
//
//   RMSNorm -> Q   x~ = (x * rstd(row)).type_as(x) * weight          (src/models/llama.py:64-75 of the reference)
//   SwiGLU  -> Q   a  = silu(h[:, :H]) * h[:, H:]                    (src/models/llama.py:112-114)
//
// followed by exactly the arithmetic of the forward quantizer (quest_quantize_group).  Both kernels keep the
// tiling of quant_rows_kernel: one CTA per 128 x 128 tile of the quantized tensor, TMA in, TMA / bulk stores out.
//
// RMSNorm needs a statistic of the whole row before any group can be quantized, so it takes two launches:
// rms_stats_kernel reads the rows once and writes rstd (which the backward pass of the norm needs anyway), the
// quantizer reads them again, last rows first, so that what the first pass left in L2 is found there.  Bytes
// per element with fp32 rows: 4 + 4 read, 0.66 written, against 4 + 4 (the norm's own read and write) + 4 + 0.66
// for the norm followed by the plain quantizer.
// Measured and dropped: (1) walking the tensor in chunks of 20-80 MB, statistics then quantization per chunk
// (slower: the second read of a chunk still came from DRAM); (2) two single-read forms, in which the CTAs that
// share a band of rows exchange their tiles' sums of squares while the tiles wait in shared memory -- through
// global memory in a cooperative launch, and through distributed shared memory in a cluster of up to 8.  Neither
// was faster than the two launches: the exchange sits between a tile's load and its arithmetic, and with three
// or four CTAs per SM too few loads stay in flight.
#include "common.cuh"
#include "quant_math.cuh"

#include <cuda_bf16.h>

namespace quartet {

enum { PRO_RMSNORM = 1, PRO_SWIGLU = 2 };

struct ProducerParams {
    int64_t rows, cols;              // extents of the quantized tensor
    uint8_t* sf;
    int64_t sf_blocks_per_rowblock;  // pad4(cols/32) / 4
    float had_scale, gaussian_scale;
    int has_mask;
    uint32_t box_rows;
    const float* rstd;               // RMSNorm: one per row
    const float* gamma;              // RMSNorm: one per column
    int reverse_rows;                // visit the row tiles from the last to the first
};

constexpr int P_TILE_R = 128, P_TILE_C = 128, P_THREADS = 256;
constexpr int P_CODES_BYTES = P_TILE_R * P_TILE_C / 2;
constexpr int P_MASK_BYTES = P_TILE_R * P_TILE_C / 8;
constexpr int P_SF_BYTES = 512;

template <int PRO, bool F32>
constexpr int producer_smem_bytes() {
    return P_TILE_R * P_TILE_C * (F32 ? 4 : 2) * (PRO == PRO_SWIGLU ? 2 : 1) + P_CODES_BYTES + P_MASK_BYTES + P_SF_BYTES + 64;
}
template <int PRO, bool F32>
constexpr int producer_min_ctas() {
    return PRO == PRO_SWIGLU ? (F32 ? 1 : 3) : (F32 ? 3 : 4);
}

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// silu as torch's CUDA kernel evaluates it: x / (1 + exp(-x)) in fp32 with the accurate exp and an IEEE division.
// (A hand-written division without the IEEE range check and integer bf16 rounding were each measured at 5 % or
// less; the exact forms stay.)
__device__ __forceinline__ float silu_f32(float x) { return __fdiv_rn(x, 1.0f + expf(-x)); }

// silu(up) * gate as torch evaluates it on tensors of this dtype: for bf16, silu's result and the product are each
// rounded to bf16 (two kernels), for fp32 neither is
template <bool F32>
__device__ __forceinline__ float swiglu_value(float up, float gate) {
    const float s = silu_f32(up);
    const float a = (F32 ? s : round_bf16(s)) * gate;
    return F32 ? a : round_bf16(a);
}

template <int PRO, bool F32>
__global__ void __launch_bounds__(P_THREADS, producer_min_ctas<PRO, F32>())
    quant_producer_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_g,
                          const __grid_constant__ CUtensorMap tm_codes, const __grid_constant__ CUtensorMap tm_mask,
                          const ProducerParams p) {
    // Dynamic shared memory is the kernel's only shared memory and starts 1024-byte aligned (checked below): no slack
    // for re-aligning it, which is what lets three CTAs of the bf16 SwiGLU kernel (two 32 KB input tiles) share an SM.
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicOr(&g_status, WAIT_GEMM_ALIGN | 0x100);
        return;
    }
    constexpr int IN_BYTES = P_TILE_R * P_TILE_C * (F32 ? 4 : 2);
    constexpr int NBOX = F32 ? 4 : 2;            // 128-byte-wide boxes per tile row
    constexpr int BOX_BYTES = P_TILE_R * 128;
    constexpr int NIN = PRO == PRO_SWIGLU ? 2 : 1;
    uint8_t* s_in = smem;
    uint8_t* s_codes = smem + NIN * IN_BYTES;
    uint8_t* s_mask = s_codes + P_CODES_BYTES;
    uint8_t* s_sf = s_mask + P_MASK_BYTES;
    uint64_t* bar = reinterpret_cast<uint64_t*>(s_sf + P_SF_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col0 = blockIdx.x * P_TILE_C;
    const int tile_y = p.reverse_rows ? (int)(gridDim.y - 1 - blockIdx.y) : (int)blockIdx.y;
    const int64_t row0 = (int64_t)tile_y * P_TILE_R;

    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();
    if (tid == 0) {
        mbar_arrive_expect_tx(bar, NIN * NBOX * 128u * p.box_rows);
#pragma unroll
        for (int b = 0; b < NBOX; ++b) {
            tma_load_2d(s_in + b * BOX_BYTES, &tm_x, col0 + b * (F32 ? 32 : 64), (int)row0, bar);
            if (PRO == PRO_SWIGLU) tma_load_2d(s_in + IN_BYTES + b * BOX_BYTES, &tm_g, col0 + b * (F32 ? 32 : 64), (int)row0, bar);
        }
    }

    const int row = (warp & 3) * 32 + lane;
    const int64_t grow = row0 + row;
    const float h = p.had_scale;
    float rstd = 0.f;
    if (PRO == PRO_RMSNORM && grow < p.rows) rstd = __ldg(p.rstd + grow);

    mbar_wait(bar, 0, WAIT_QUANT_LOAD);

#pragma unroll 1
    for (int it = 0; it < 2; ++it) {
        const int gk = (warp >> 2) * 2 + it;  // group within the tile row, 0..3
        float w[32];
        load_row_group<F32>(s_in, row, gk, w);
        if (PRO == PRO_RMSNORM) {
            const float4* g4 = reinterpret_cast<const float4*>(p.gamma + col0 + gk * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 g = __ldg(g4 + j);
                const float n0 = w[4 * j] * rstd, n1 = w[4 * j + 1] * rstd, n2 = w[4 * j + 2] * rstd, n3 = w[4 * j + 3] * rstd;
                // `.type_as(x)`: rows held in bf16 round the normalised value before the fp32 weight multiplies it
                w[4 * j] = (F32 ? n0 : round_bf16(n0)) * g.x;
                w[4 * j + 1] = (F32 ? n1 : round_bf16(n1)) * g.y;
                w[4 * j + 2] = (F32 ? n2 : round_bf16(n2)) * g.z;
                w[4 * j + 3] = (F32 ? n3 : round_bf16(n3)) * g.w;
            }
        } else {
            // gate values of the same group, eight at a time
            const uint8_t* s_gate = s_in + IN_BYTES;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float g[8];
                if (F32) {
                    const uint8_t* base = s_gate + gk * BOX_BYTES + row * 128;
                    const float4 q0 = *reinterpret_cast<const float4*>(base + (((2 * j) ^ (row & 7)) << 4));
                    const float4 q1 = *reinterpret_cast<const float4*>(base + (((2 * j + 1) ^ (row & 7)) << 4));
                    g[0] = q0.x, g[1] = q0.y, g[2] = q0.z, g[3] = q0.w, g[4] = q1.x, g[5] = q1.y, g[6] = q1.z, g[7] = q1.w;
                } else {
                    const uint8_t* base = s_gate + (gk >> 1) * BOX_BYTES + row * 128;
                    const int chunk = (gk & 1) * 4 + j;
                    unpack_bf16x8(*reinterpret_cast<const uint4*>(base + ((chunk ^ (row & 7)) << 4)), g);
                }
#pragma unroll
                for (int t = 0; t < 8; ++t) w[8 * j + t] = swiglu_value<F32>(w[8 * j + t], g[t]);
            }
        }
        uint32_t words[4];
        uint32_t mbits;
        int e8m0;
        quest_quantize_group<true>(w, h, p.gaussian_scale, words, mbits, e8m0);
        *reinterpret_cast<uint4*>(s_codes + row * 64 + ((gk ^ ((row >> 1) & 3)) << 4)) = make_uint4(words[0], words[1], words[2], words[3]);
        *reinterpret_cast<uint32_t*>(s_mask + row * 16 + gk * 4) = mbits;
        // rows past the tensor's last one (padding of the 128-row scale block) get scale byte 0, whatever the tile held there
        s_sf[(row & 31) * 16 + (row >> 5) * 4 + gk] = grow < p.rows ? (uint8_t)e8m0 : (uint8_t)0;
    }

    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
        tma_store_2d(&tm_codes, col0 / 2, (int)row0, s_codes);
        if (p.has_mask) tma_store_2d(&tm_mask, col0 / 8, (int)row0, s_mask);
        uint8_t* sf_dst = p.sf + ((int64_t)tile_y * p.sf_blocks_per_rowblock + blockIdx.x) * 512;
        bulk_store(sf_dst, s_sf, 512);
        bulk_commit();
        bulk_wait_read0();
    }
}

// rstd[r] = rsqrt(mean_c x[r, c]^2 + eps): one warp per row, 16-byte loads, fixed summation order (each lane
// sums its chunks in order, then a butterfly over the lanes)
constexpr int STATS_THREADS = 256;
template <bool F32>
__global__ void __launch_bounds__(STATS_THREADS) rms_stats_kernel(const uint8_t* __restrict__ x, int64_t rows, int64_t cols, float eps,
                                                                  float* __restrict__ rstd) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (STATS_THREADS / 32) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int64_t row_bytes = cols * (F32 ? 4 : 2);
    const uint4* src = reinterpret_cast<const uint4*>(x + row * row_bytes);
    const int n16 = (int)(row_bytes >> 4);
    // batches of eight independent 16-byte loads per lane keep enough bytes in flight; the sum is still taken in
    // chunk order, so the result does not depend on the batching
    float acc = 0.f;
    for (int c0 = lane; c0 < n16; c0 += 32 * 8) {
        uint4 q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = c0 + 32 * u;
            q[u] = c < n16 ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (F32) {
                const float a = __uint_as_float(q[u].x), b = __uint_as_float(q[u].y), cc = __uint_as_float(q[u].z), d = __uint_as_float(q[u].w);
                acc = fmaf(a, a, acc), acc = fmaf(b, b, acc), acc = fmaf(cc, cc, acc), acc = fmaf(d, d, acc);
            } else {
                float v[8];
                unpack_bf16x8(q[u], v);
#pragma unroll
                for (int t = 0; t < 8; ++t) acc = fmaf(v[t], v[t], acc);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) rstd[row] = rsqrtf(acc * (1.0f / (float)cols) + eps);
}

// The SwiGLU product written out, with the arithmetic of the fused quantizer above: 16 bytes of `up`, 16 of `gate`
// in, 16 out per thread and trip.
template <bool F32>
__global__ void __launch_bounds__(256) swiglu_kernel(const uint8_t* __restrict__ h, uint8_t* __restrict__ out, int64_t rows, int64_t hidden) {
    constexpr int EB = F32 ? 4 : 2, PER = 16 / EB;
    const int64_t chunks_per_row = hidden / PER, total = rows * chunks_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / chunks_per_row, c = (i - r * chunks_per_row) * PER;
        const uint4 qu = __ldg(reinterpret_cast<const uint4*>(h + (r * 2 * hidden + c) * EB));
        const uint4 qg = __ldg(reinterpret_cast<const uint4*>(h + (r * 2 * hidden + hidden + c) * EB));
        uint4 o;
        if (F32) {
            o.x = __float_as_uint(swiglu_value<true>(__uint_as_float(qu.x), __uint_as_float(qg.x)));
            o.y = __float_as_uint(swiglu_value<true>(__uint_as_float(qu.y), __uint_as_float(qg.y)));
            o.z = __float_as_uint(swiglu_value<true>(__uint_as_float(qu.z), __uint_as_float(qg.z)));
            o.w = __float_as_uint(swiglu_value<true>(__uint_as_float(qu.w), __uint_as_float(qg.w)));
        } else {
            float u[8], g[8];
            unpack_bf16x8(qu, u);
            unpack_bf16x8(qg, g);
            uint32_t w[4];
#pragma unroll
            for (int t = 0; t < 4; ++t)
                w[t] = (__float_as_uint(swiglu_value<false>(u[2 * t], g[2 * t])) >> 16) |
                       (__float_as_uint(swiglu_value<false>(u[2 * t + 1], g[2 * t + 1])) & 0xFFFF0000u);
            o = make_uint4(w[0], w[1], w[2], w[3]);
        }
        *reinterpret_cast<uint4*>(out + (r * hidden + c) * EB) = o;
    }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
template <int PRO, bool F32>
static int launch_producer(const void* x, const void* gate, int64_t pitch_elems, const ProducerParams& p, uint8_t* codes, uint8_t* mask,
                           cudaStream_t stream) {
    CUtensorMap tm_x, tm_g, tm_codes, tm_mask;
    int rc;
    const uint32_t box_rows = p.box_rows;
    const CUtensorMapDataType dt = F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const int eb = F32 ? 4 : 2;
    if ((rc = make_tmap_2d(&tm_x, x, dt, eb, p.cols, p.rows, pitch_elems * eb, F32 ? 32 : 64, box_rows, 3))) return rc;
    if (PRO == PRO_SWIGLU) {
        if ((rc = make_tmap_2d(&tm_g, gate, dt, eb, p.cols, p.rows, pitch_elems * eb, F32 ? 32 : 64, box_rows, 3))) return rc;
    } else {
        tm_g = tm_x;  // never used
    }
    if ((rc = make_tmap_2d(&tm_codes, codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.cols / 2, p.rows, p.cols / 2, 64, box_rows, 2))) return rc;
    if (mask) {
        if ((rc = make_tmap_2d(&tm_mask, mask, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.cols / 8, p.rows, p.cols / 8, 16, box_rows, 0))) return rc;
    } else {
        tm_mask = tm_codes;  // never used: the kernel stores no mask
    }
    auto kern = quant_producer_kernel<PRO, F32>;
    constexpr int smem = producer_smem_bytes<PRO, F32>();
    static thread_local int smem_set = -1;
    if ((rc = set_max_smem_once(kern, smem, smem_set))) return rc;
    dim3 grid((unsigned)(p.cols / P_TILE_C), (unsigned)((p.rows + P_TILE_R - 1) / P_TILE_R));
    return check_cuda(launch_pdl(kern, grid, dim3(P_THREADS), smem, stream, tm_x, tm_g, tm_codes, tm_mask, p), "quant_producer launch");
}

static int validate_producer(const void* x, int x_dtype, int64_t rows, int64_t cols, const void* codes, const void* sf, const void* mask) {
    if (!x || !codes || !sf) return fail(QUARTET_E_NULL, "input, codes and sf must be non-NULL");
    if (x_dtype != QUARTET_BF16 && x_dtype != QUARTET_F32) return fail(QUARTET_E_ARG, "dtype must be 0 (bf16) or 1 (f32)");
    if (rows < 1 || cols < 128 || cols % 128 != 0)
        return fail(QUARTET_E_SHAPE, "need rows >= 1 and a width that is a multiple of 128 (got %lld x %lld)", (long long)rows, (long long)cols);
    if (rows > 0x7FFFFFFF || cols > 0x3FFFFFFF || (rows + 127) / 128 > 65535) return fail(QUARTET_E_SHAPE, "extent too large (rows <= 8388480)");
    if (!aligned16(x) || !aligned16(codes) || !aligned16(sf) || (mask && !aligned16(mask)))
        return fail(QUARTET_E_ALIGN, "pointers must be 16-byte aligned");
    int rc = bind_context_of(x);
    if (rc) return rc;
    return check_device();
}

static int launch_stats(const void* x, int x_dtype, int64_t rows, int64_t cols, float eps, float* rstd, cudaStream_t s) {
    const unsigned grid = (unsigned)((rows + STATS_THREADS / 32 - 1) / (STATS_THREADS / 32));
    const uint8_t* xb = static_cast<const uint8_t*>(x);
    if (x_dtype == QUARTET_F32)
        return check_cuda(launch_pdl(rms_stats_kernel<true>, dim3(grid), dim3(STATS_THREADS), 0, s, xb, rows, cols, eps, rstd), "rms_stats launch");
    return check_cuda(launch_pdl(rms_stats_kernel<false>, dim3(grid), dim3(STATS_THREADS), 0, s, xb, rows, cols, eps, rstd), "rms_stats launch");
}

QUARTET_DEFINE_STATUS_READER(status_producer)

}  // namespace quartet

using namespace quartet;

extern "C" __attribute__((visibility("default"))) int quartet_rms_stats(const void* x, int x_dtype, int64_t rows, int64_t cols, float eps, float* rstd,
                                                                        quartet_stream_t stream) {
    if (!x || !rstd) return fail(QUARTET_E_NULL, "x and rstd must be non-NULL");
    if (x_dtype != QUARTET_BF16 && x_dtype != QUARTET_F32) return fail(QUARTET_E_ARG, "x_dtype must be 0 (bf16) or 1 (f32)");
    if (rows < 1 || cols < 8 || cols % 8 != 0 || rows > 0x7FFFFFFF || cols > 0x3FFFFFFF)
        return fail(QUARTET_E_SHAPE, "need rows >= 1 and cols a multiple of 8 (got %lld x %lld)", (long long)rows, (long long)cols);
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(rstd) & 3)) return fail(QUARTET_E_ALIGN, "x must be 16-byte aligned, rstd 4-byte");
    if (!(eps >= 0.f)) return fail(QUARTET_E_ARG, "eps must be >= 0");
    int rc = bind_context_of(x);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    return launch_stats(x, x_dtype, rows, cols, eps, rstd, static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int quartet_quant_fwd_rmsnorm(const void* x, int x_dtype, int64_t rows, int64_t cols, const float* weight,
                                                                                float eps, float* rstd, float had_scale, float gaussian_scale,
                                                                                uint8_t* codes, uint8_t* sf, uint8_t* mask, quartet_stream_t stream) {
    if (!weight || !rstd) return fail(QUARTET_E_NULL, "weight and rstd must be non-NULL");
    if (!aligned16(weight) || (reinterpret_cast<uintptr_t>(rstd) & 3)) return fail(QUARTET_E_ALIGN, "weight must be 16-byte aligned, rstd 4-byte");
    if (!(eps >= 0.f)) return fail(QUARTET_E_ARG, "eps must be >= 0");
    int rc = validate_producer(x, x_dtype, rows, cols, codes, sf, mask);
    if (rc) return rc;
    const bool f32 = x_dtype == QUARTET_F32;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ProducerParams p{};
    p.rows = rows, p.cols = cols, p.sf = sf;
    p.sf_blocks_per_rowblock = (cols / 32 + 3) / 4;
    p.had_scale = had_scale, p.gaussian_scale = gaussian_scale;
    p.has_mask = mask != nullptr;
    p.box_rows = (uint32_t)(rows < P_TILE_R ? rows : P_TILE_R);
    p.rstd = rstd, p.gamma = weight;
    // two passes: the row statistics, then the quantizer
    if ((rc = launch_stats(x, x_dtype, rows, cols, eps, rstd, s))) return rc;
    p.reverse_rows = 1;  // the rows the statistics pass read last are the likeliest to be in L2 still
    return f32 ? launch_producer<PRO_RMSNORM, true>(x, nullptr, cols, p, codes, mask, s)
               : launch_producer<PRO_RMSNORM, false>(x, nullptr, cols, p, codes, mask, s);
}

extern "C" __attribute__((visibility("default"))) int quartet_quant_fwd_swiglu(const void* h, int h_dtype, int64_t rows, int64_t hidden, float had_scale,
                                                                               float gaussian_scale, uint8_t* codes, uint8_t* sf, uint8_t* mask,
                                                                               quartet_stream_t stream) {
    int rc = validate_producer(h, h_dtype, rows, hidden, codes, sf, mask);
    if (rc) return rc;
    const bool f32 = h_dtype == QUARTET_F32;
    ProducerParams p{};
    p.rows = rows, p.cols = hidden, p.sf = sf;
    p.sf_blocks_per_rowblock = (hidden / 32 + 3) / 4;
    p.had_scale = had_scale, p.gaussian_scale = gaussian_scale;
    p.has_mask = mask != nullptr;
    p.box_rows = (uint32_t)(rows < P_TILE_R ? rows : P_TILE_R);
    const uint8_t* up = static_cast<const uint8_t*>(h);
    const uint8_t* gate = up + hidden * (f32 ? 4 : 2);  // second half of every row; 16-byte aligned since hidden % 128 == 0
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return f32 ? launch_producer<PRO_SWIGLU, true>(up, gate, 2 * hidden, p, codes, mask, s)
               : launch_producer<PRO_SWIGLU, false>(up, gate, 2 * hidden, p, codes, mask, s);
}

// silu(h[:, :hidden]) * h[:, hidden:] written out as [rows, hidden] in h's dtype, bit for bit the values the fused
// quantizer above quantizes.
extern "C" __attribute__((visibility("default"))) int quartet_swiglu(const void* h, int h_dtype, int64_t rows, int64_t hidden, void* out,
                                                                     quartet_stream_t stream) {
    if (!h || !out) return fail(QUARTET_E_NULL, "h and out must be non-NULL");
    if (h_dtype != QUARTET_BF16 && h_dtype != QUARTET_F32) return fail(QUARTET_E_ARG, "h_dtype must be 0 (bf16) or 1 (f32)");
    if (rows < 1 || hidden < 8 || hidden % 8 != 0 || rows > 0x7FFFFFFF || hidden > 0x3FFFFFFF)
        return fail(QUARTET_E_SHAPE, "need rows >= 1 and hidden a multiple of 8 (got %lld x %lld)", (long long)rows, (long long)hidden);
    if (!aligned16(h) || !aligned16(out)) return fail(QUARTET_E_ALIGN, "pointers must be 16-byte aligned");
    int rc = bind_context_of(h);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    const bool f32 = h_dtype == QUARTET_F32;
    const int64_t total = rows * hidden / (f32 ? 4 : 8);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t* hb = static_cast<const uint8_t*>(h);
    uint8_t* ob = static_cast<uint8_t*>(out);
    if (f32)
        swiglu_kernel<true><<<(unsigned)blocks, 256, 0, s>>>(hb, ob, rows, hidden);
    else
        swiglu_kernel<false><<<(unsigned)blocks, 256, 0, s>>>(hb, ob, rows, hidden);
    return check_cuda(cudaGetLastError(), "swiglu launch");
}
