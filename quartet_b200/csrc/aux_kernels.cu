// Small element-wise companions of the quantizers: de-quantization (codes + scales -> values) and
// the stand-alone straight-through backward of the forward quantizer (mask, then rotate back).
// One thread owns one group of 32 values; plain vectorised global accesses.
#include "common.cuh"
#include "quant_math.cuh"

namespace quartet {

__device__ __forceinline__ int64_t sf_off(int64_t row, int64_t kb, int64_t blocks_per_rowblock) {
    const int64_t r = row & 127;
    return ((row >> 7) * blocks_per_rowblock + (kb >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3);
}

template <bool F32OUT>
__device__ __forceinline__ void store_group(void* out, int64_t elem0, const float (&v)[32]) {
    if (F32OUT) {
        float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + elem0);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
        uint4* o = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out) + elem0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                __nv_bfloat162 t = __floats2bfloat162_rn(v[8 * j + 2 * k], v[8 * j + 2 * k + 1]);
                w[k] = *reinterpret_cast<uint32_t*>(&t);
            }
            o[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

template <bool F32OUT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf,
                                                      int64_t rows, int64_t cols, float scale, void* __restrict__ out) {
    const int64_t kbs = cols >> 5;
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= rows * kbs) return;
    const int64_t row = g / kbs, kb = g % kbs;
    const uint32_t sfb = sf[sf_off(row, kb, (kbs + 3) >> 2)];
    const float sc = __uint_as_float(sfb << 23) * scale;
    const uint4 q = *reinterpret_cast<const uint4*>(codes + g * 16);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    float v[32];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float2 f = e2m1x2_to_float2((w[i >> 2] >> (8 * (i & 3))) & 0xFFu);
        v[2 * i] = f.x * sc;
        v[2 * i + 1] = f.y * sc;
    }
    store_group<F32OUT>(out, g * 32, v);
}

template <bool F32IN, bool F32OUT>
__global__ void __launch_bounds__(256) unrotate_mask_kernel(const void* __restrict__ gin, const uint8_t* __restrict__ mask,
                                                            int64_t n_groups, float had_scale, void* __restrict__ out) {
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= n_groups) return;
    float v[32];
    if (F32IN) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(gin) + g * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 q = p[j];
            v[4 * j] = q.x, v[4 * j + 1] = q.y, v[4 * j + 2] = q.z, v[4 * j + 3] = q.w;
        }
    } else {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(gin) + g * 32);
#pragma unroll
        for (int j = 0; j < 4; ++j) unpack_bf16x8(p[j], &v[8 * j]);
    }
    if (mask) {
        const uint32_t m = *reinterpret_cast<const uint32_t*>(mask + g * 4);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = ((m >> i) & 1u) ? v[i] : 0.f;
    }
    wht32(v);  // the Sylvester matrix is symmetric: (.) @ H^T is the same transform
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= had_scale;
    store_group<F32OUT>(out, g * 32, v);
}

// One warp: lane j reads draw[j] (0 or 1; the reference turns it into the sign 2 * draw - 1), and the word of
// negated columns (bit j set <=> sign -1 <=> draw 0) is XOR-ed into *word: H <- H @ diag(s) on the sign word.
template <bool F32>
__global__ void fold_signs_kernel(const void* __restrict__ draw, uint32_t* __restrict__ word) {
    const int lane = threadIdx.x;
    const float v = F32 ? static_cast<const float*>(draw)[lane] : __bfloat162float(static_cast<const __nv_bfloat16*>(draw)[lane]);
    const uint32_t neg = __ballot_sync(0xFFFFFFFFu, v == 0.f);
    if (lane == 0) *word ^= neg;
}

QUARTET_DEFINE_STATUS_READER(status_aux)

}  // namespace quartet

using namespace quartet;

extern "C" __attribute__((visibility("default"))) int quartet_dequant(const uint8_t* codes, const uint8_t* sf, int64_t rows, int64_t cols, float scale,
                               void* out, int out_dtype, quartet_stream_t stream) {
    if (!codes || !sf || !out) return fail(QUARTET_E_NULL, "codes, sf and out must be non-NULL");
    if (rows < 1 || cols < 32 || cols % 32 != 0) return fail(QUARTET_E_SHAPE, "need rows >= 1 and cols a multiple of 32");
    if (!aligned16(codes) || !aligned16(out)) return fail(QUARTET_E_ALIGN, "pointers must be 16-byte aligned");
    if (out_dtype != QUARTET_BF16 && out_dtype != QUARTET_F32) return fail(QUARTET_E_ARG, "out_dtype must be 0 or 1");
    int rc = bind_context_of(codes);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    const int64_t groups = rows * (cols / 32);
    const unsigned blocks = (unsigned)((groups + 255) / 256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (out_dtype == QUARTET_F32)
        dequant_kernel<true><<<blocks, 256, 0, s>>>(codes, sf, rows, cols, scale, out);
    else
        dequant_kernel<false><<<blocks, 256, 0, s>>>(codes, sf, rows, cols, scale, out);
    return check_cuda(cudaGetLastError(), "dequant launch");
}

extern "C" __attribute__((visibility("default"))) int quartet_unrotate_mask(const void* g, int g_dtype, const uint8_t* mask, int64_t rows, int64_t cols,
                                     float had_scale, void* out, int out_dtype, quartet_stream_t stream) {
    if (!g || !out) return fail(QUARTET_E_NULL, "g and out must be non-NULL");
    if (rows < 1 || cols < 32 || cols % 32 != 0) return fail(QUARTET_E_SHAPE, "need rows >= 1 and cols a multiple of 32");
    if (!aligned16(g) || !aligned16(out) || (mask && (reinterpret_cast<uintptr_t>(mask) & 3)))
        return fail(QUARTET_E_ALIGN, "g/out must be 16-byte aligned, mask 4-byte aligned");
    if ((g_dtype | out_dtype) & ~1) return fail(QUARTET_E_ARG, "dtypes must be 0 (bf16) or 1 (f32)");
    int rc = bind_context_of(g);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    const int64_t groups = rows * (cols / 32);
    const unsigned blocks = (unsigned)((groups + 255) / 256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (g_dtype == QUARTET_F32 && out_dtype == QUARTET_F32)
        unrotate_mask_kernel<true, true><<<blocks, 256, 0, s>>>(g, mask, groups, had_scale, out);
    else if (g_dtype == QUARTET_F32)
        unrotate_mask_kernel<true, false><<<blocks, 256, 0, s>>>(g, mask, groups, had_scale, out);
    else if (out_dtype == QUARTET_F32)
        unrotate_mask_kernel<false, true><<<blocks, 256, 0, s>>>(g, mask, groups, had_scale, out);
    else
        unrotate_mask_kernel<false, false><<<blocks, 256, 0, s>>>(g, mask, groups, had_scale, out);
    return check_cuda(cudaGetLastError(), "unrotate_mask launch");
}

extern "C" __attribute__((visibility("default"))) int quartet_fold_signs(const void* draw, int draw_dtype, uint32_t* word, quartet_stream_t stream) {
    if (!draw || !word) return fail(QUARTET_E_NULL, "draw and word must be non-NULL");
    if (draw_dtype != QUARTET_BF16 && draw_dtype != QUARTET_F32) return fail(QUARTET_E_ARG, "draw_dtype must be 0 (bf16) or 1 (f32)");
    if (reinterpret_cast<uintptr_t>(word) & 3) return fail(QUARTET_E_ALIGN, "word must be 4-byte aligned");
    int rc = bind_context_of(word);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (draw_dtype == QUARTET_F32)
        fold_signs_kernel<true><<<1, 32, 0, s>>>(draw, word);
    else
        fold_signs_kernel<false><<<1, 32, 0, s>>>(draw, word);
    return check_cuda(cudaGetLastError(), "fold_signs launch");
}
