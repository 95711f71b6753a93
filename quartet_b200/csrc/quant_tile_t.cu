// Transposing backward quantizers: groups of 32 run along the ROWS of the source, the result is
// the quantized TRANSPOSE (codes_t [cols, rows/2], scales logical [cols, rows/32]).
//
//   SRC_BF16 / SRC_F32  source is a dense tensor        -> `g_quantizer(e.T.contiguous())`
//                                                           (backward.py:81 of the reference)
//   SRC_MXFP4           source is codes + blocked scales -> `g_quantizer(w.T.contiguous())`,
//                                                           `g_quantizer(x.T.contiguous())`
//                                                           (backward.py:73,82)
//
// One CTA handles a 128 x 128 source tile.  TMA loads it into shared memory; a thread owns two
// adjacent source columns over 32 consecutive source rows (= two output groups), reads them
// column-wise from shared memory (conflict-free: a warp reads 32 neighbouring words of one row),
// rotates/rounds/packs in registers and stages 2 x 16 B of codes; the transposed 128 x 64 B code
// tile and the tile's single 512-byte scale block leave through TMA / bulk stores.
#include "common.cuh"
#include "quant_math.cuh"

namespace quartet {

enum { SRC_BF16 = 0, SRC_F32 = 1, SRC_MXFP4 = 2 };

struct TileTParams {
    int64_t rows, cols;       // source extents
    const uint8_t* sf_in;     // SRC_MXFP4: blocked scales of the source
    int64_t sf_in_blocks_per_rowblock;
    float in_scale;
    uint8_t* sf_t;            // blocked scales of the transposed result
    int64_t sf_t_blocks_per_rowblock;  // pad4(rows/32) / 4
    float had_scale;
    uint32_t signs;
    const uint32_t* signs_dev;
    uint64_t seed, offset;
    const float* noise;
    // dual mode: the row-wise quantization of the same source, from the same tile in shared memory
    uint8_t* sf_rows;
    int64_t sf_rows_blocks_per_rowblock;  // pad4(cols/32) / 4
    uint64_t seed_rows;
};

constexpr int TT = 128, TT_THREADS = 256;

template <int SRC>
__host__ __device__ constexpr int tile_in_bytes() {
    return SRC == SRC_BF16 ? TT * TT * 2 : (SRC == SRC_F32 ? TT * TT * 4 : TT * TT / 2 + 512);
}
template <int SRC, bool DUAL>
constexpr int tile_smem_bytes() {
    return tile_in_bytes<SRC>() + (DUAL ? 2 : 1) * (TT * 64 + 512) + 64 + 1024;
}

// DUAL: besides the quantized transpose, the kernel also emits the row-wise quantization of the same
// tile (what quartet_quant_bwd computes, bit for bit, with its own seed), so that the backward pass
// reads the output-gradient once for Q(E) and Q(E^T).
template <int SRC, int ROUND, bool DUAL>
__global__ void __launch_bounds__(TT_THREADS, (SRC == SRC_F32 && DUAL) ? 2 : 4)
    quant_tile_t_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_out,
                        const __grid_constant__ CUtensorMap tm_rows, const TileTParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int IN_BYTES = tile_in_bytes<SRC>();
    constexpr int BOX_BYTES = TT * 128;
    uint8_t* s_in = smem;
    uint8_t* s_codes = smem + IN_BYTES;   // [128 out rows][64 B]
    uint8_t* s_sf = s_codes + TT * 64;    // 512 B
    uint8_t* s_codes_r = s_sf + 512;      // dual mode: [128 rows][64 B] + 512 B of scales
    uint8_t* s_sf_r = s_codes_r + TT * 64;
    uint64_t* bar = reinterpret_cast<uint64_t*>(DUAL ? s_sf_r + 512 : s_sf + 512);

    const int tid = threadIdx.x;
    const int col0 = blockIdx.x * TT;              // source column of the tile = output row
    const int row0 = blockIdx.y * TT;              // source row of the tile    = output column

    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();  // no global access before this point
    if (tid == 0) {
        if (SRC == SRC_MXFP4) {
            mbar_arrive_expect_tx(bar, TT * 64 + 512);
            tma_load_2d(s_in, &tm_in, col0 / 2, row0, bar);
            const uint8_t* sf_src = p.sf_in + ((int64_t)blockIdx.y * p.sf_in_blocks_per_rowblock + blockIdx.x) * 512;
            bulk_load(s_in + TT * 64, sf_src, 512, bar);
        } else {
            constexpr int NBOX = SRC == SRC_F32 ? 4 : 2;
            mbar_arrive_expect_tx(bar, NBOX * BOX_BYTES);
#pragma unroll
            for (int b = 0; b < NBOX; ++b)
                tma_load_2d(s_in + b * BOX_BYTES, &tm_in, col0 + b * (SRC == SRC_F32 ? 32 : 64), row0, bar);
        }
    }

    const uint32_t signs = p.signs_dev ? __ldg(p.signs_dev) : p.signs;
    uint32_t flip[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) flip[q] = spread_sign_bits((signs >> (8 * q)) & 0xFFu);

    mbar_wait(bar, 0, WAIT_QUANT_LOAD);

    const int cp = tid & 63;   // source column pair within the tile
    const int rg = tid >> 6;   // group of 32 source rows within the tile
    const int64_t out_kb = (int64_t)(row0 >> 5) + rg;           // scale block along the output row
    const int64_t groups_per_out_row = p.rows >> 5;

    // The two columns of the pair are processed one after the other (the second pass re-reads shared
    // memory): 32 live values instead of 64 keeps the kernel at 64 registers, i.e. twice the warps per SM.
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
        float a[32];  // column 2cp + c over rows rg*32 .. rg*32+31
        if (SRC == SRC_BF16) {
            const uint8_t* base = s_in + (cp >> 5) * BOX_BYTES + c * 2;
            const int chunk = (cp & 31) >> 2, word = cp & 3;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int r = rg * 32 + i;
                const uint32_t v = *reinterpret_cast<const uint16_t*>(base + r * 128 + ((chunk ^ (r & 7)) << 4) + word * 4);
                a[i] = __uint_as_float(v << 16);
            }
        } else if (SRC == SRC_F32) {
            const uint8_t* base = s_in + (cp >> 4) * BOX_BYTES + c * 4;
            const int chunk = (cp & 15) >> 1, half = cp & 1;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int r = rg * 32 + i;
                a[i] = *reinterpret_cast<const float*>(base + r * 128 + ((chunk ^ (r & 7)) << 4) + half * 8);
            }
        } else {
            const uint8_t* s_sfin = s_in + TT * 64;
            const int kb = cp >> 4;  // source scale block (32 source columns) of this column pair
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int r = rg * 32 + i;
                const uint32_t byte = s_in[r * 64 + cp];
                const uint32_t sfb = s_sfin[i * 16 + rg * 4 + kb];  // (r % 32) * 16 + (r / 32) * 4 + kb
                const float sc = __uint_as_float(sfb << 23) * p.in_scale;
                const float2 f = e2m1x2_to_float2(byte);
                a[i] = (c ? f.y : f.x) * sc;
            }
        }
        wht32(a);
        const int oc = 2 * cp + c;                               // output row within the tile
        const int64_t orow = (int64_t)col0 + oc;
        const uint64_t g = (uint64_t)orow * (uint64_t)groups_per_out_row + (uint64_t)out_kb;
        const int64_t flat = orow * p.rows + out_kb * 32;
        uint32_t words[4];
        int e8m0;
        absmax_quantize_group<ROUND>(a, p.had_scale, g, flat, true, p.seed, p.offset, p.noise, flip, words, e8m0);
        // 64B-swizzled staging (16-byte chunk c of row r at chunk c ^ ((r >> 1) & 3)), matching the store's tensor map
        *reinterpret_cast<uint4*>(s_codes + oc * 64 + ((rg ^ ((oc >> 1) & 3)) << 4)) = make_uint4(words[0], words[1], words[2], words[3]);
        s_sf[(oc & 31) * 16 + (oc >> 5) * 4 + rg] = (uint8_t)e8m0;
    }

    if (DUAL && SRC != SRC_MXFP4) {
        // row-wise pass over the same tile: thread -> (row, two of the row's four groups), as in quant_rows
        const int warp = tid >> 5, lane = tid & 31;
        const int row = (warp & 3) * 32 + lane;
        const int64_t grow = (int64_t)row0 + row;
#pragma unroll 1
        for (int it = 0; it < 2; ++it) {
            const int gk = (warp >> 2) * 2 + it;
            float w[32];
            load_row_group<SRC == SRC_F32>(s_in, row, gk, w);
            wht32(w);
            const uint64_t g = (uint64_t)grow * (uint64_t)(p.cols >> 5) + (uint64_t)((col0 >> 5) + gk);
            const int64_t flat = grow * p.cols + col0 + gk * 32;
            uint32_t words[4];
            int e8m0;
            absmax_quantize_group<ROUND>(w, p.had_scale, g, flat, true, p.seed_rows, p.offset, p.noise, flip, words, e8m0);
            *reinterpret_cast<uint4*>(s_codes_r + row * 64 + ((gk ^ ((row >> 1) & 3)) << 4)) = make_uint4(words[0], words[1], words[2], words[3]);
            s_sf_r[(row & 31) * 16 + (row >> 5) * 4 + gk] = (uint8_t)e8m0;
        }
    }

    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
        tma_store_2d(&tm_out, row0 / 2, col0, s_codes);
        uint8_t* sf_dst = p.sf_t + ((int64_t)blockIdx.x * p.sf_t_blocks_per_rowblock + blockIdx.y) * 512;
        bulk_store(sf_dst, s_sf, 512);
        if (DUAL) {
            tma_store_2d(&tm_rows, col0 / 2, row0, s_codes_r);
            bulk_store(p.sf_rows + ((int64_t)blockIdx.y * p.sf_rows_blocks_per_rowblock + blockIdx.x) * 512, s_sf_r, 512);
        }
        bulk_commit();
        bulk_wait_read0();
    }
}

// ---------------------------------------------------------------------------
// MXFP4 source (quartet_requant_t): its own kernel.  The source tile is 128 rows x 64 code bytes plus one
// 512-byte scale block.  The scales are first expanded to floats (times in_scale) in shared memory, grouped
// as [32-row group][32-column block][row], so that a thread fetches the 32 scales of its rows with eight
// 128-bit loads instead of 32 byte loads, shifts and multiplies.  A thread owns one source byte column (two
// adjacent source columns) over 32 rows: every byte is loaded and decoded ONCE (cvt.rn.f16x2.e2m1x2 yields
// both values); the second column's values wait, already scaled, as packed halves of one register per row
// pair while the first column is rotated, rounded and packed.  Launched for in_scale == 1 only (what the
// backward pass uses); any other in_scale takes the generic tile kernel above, with identical results.
// ---------------------------------------------------------------------------
constexpr int RQ_IN_BYTES = TT * 64 + 512;       // codes + scale block, as the copies deliver them
constexpr int RQ_SCALE_FLOATS = 4 * 4 * 32;      // [row group][column block][row]
constexpr int RQ_SMEM = RQ_IN_BYTES + RQ_SCALE_FLOATS * 4 + TT * 64 + 512 + 64 + 1024;

__device__ __forceinline__ uint32_t e2m1x2_to_half2_bits(uint32_t byte) {
    uint32_t h2;
    asm("{\n\t.reg .b8 lo, hi;\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tmov.b16 {lo, hi}, t;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, lo;\n\t}"
        : "=r"(h2)
        : "r"(byte));
    return h2;
}

#ifndef RQ_MIN_CTAS
#define RQ_MIN_CTAS 4
#endif
template <int ROUND>
__global__ void __launch_bounds__(TT_THREADS, RQ_MIN_CTAS)
    requant_t_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_out, const TileTParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_in = smem;                                                  // [128 rows][64 B] codes, then 512 B of scales
    float* s_scale = reinterpret_cast<float*>(smem + RQ_IN_BYTES);         // 2 KB
    uint8_t* s_codes = smem + RQ_IN_BYTES + RQ_SCALE_FLOATS * 4;           // [128 out rows][64 B], 64B-swizzled
    uint8_t* s_sf = s_codes + TT * 64;                                     // 512 B
    uint64_t* bar = reinterpret_cast<uint64_t*>(s_sf + 512);

    const int tid = threadIdx.x;
    const int col0 = blockIdx.x * TT, row0 = blockIdx.y * TT;
    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();  // no global access before this point
    if (tid == 0) {
        mbar_arrive_expect_tx(bar, TT * 64 + 512);
        tma_load_2d(s_in, &tm_in, col0 / 2, row0, bar);
        bulk_load(s_in + TT * 64, p.sf_in + ((int64_t)blockIdx.y * p.sf_in_blocks_per_rowblock + blockIdx.x) * 512, 512, bar);
    }
    const uint32_t signs = p.signs_dev ? __ldg(p.signs_dev) : p.signs;
    uint32_t flip[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) flip[q] = spread_sign_bits((signs >> (8 * q)) & 0xFFu);

    mbar_wait(bar, 0, WAIT_QUANT_LOAD);
    {   // scale bytes -> floats: source byte (r % 32) * 16 + (r / 32) * 4 + kb  ->  s_scale[((r / 32) * 4 + kb) * 32 + r % 32]
        const uint8_t* s_sfin = s_in + TT * 64;
        const uint32_t two = *reinterpret_cast<const uint16_t*>(s_sfin + 2 * tid);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int b = 2 * tid + j;
            const int i = b >> 4, rgq = (b >> 2) & 3, kb = b & 3;
            s_scale[(rgq * 4 + kb) * 32 + i] = __uint_as_float(((two >> (8 * j)) & 0xFFu) << 23) * p.in_scale;
        }
    }
    __syncthreads();

    const int cp = tid & 63;   // source byte column = source column pair
    const int rg = tid >> 6;   // group of 32 source rows
    const int64_t out_kb = (int64_t)(row0 >> 5) + rg;
    const int64_t groups_per_out_row = p.rows >> 5;
    const float4* sc4 = reinterpret_cast<const float4*>(s_scale + (rg * 4 + (cp >> 4)) * 32);

    float a[32];        // the column being quantized
    uint32_t held[16];  // the second column, rows 2j and 2j+1 as the upper halves of their fp32 patterns
    {
        // in_scale == 1 (the only case this kernel is launched for): a value is grid * 2^k, at most two mantissa
        // bits, so the upper 16 bits of its fp32 pattern hold it exactly and the second column waits in 16
        // registers instead of 32
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 sc = sc4[q];
            const float scv[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
            for (int t = 0; t < 4; t += 2) {
                const int i = 4 * q + t;
                const uint32_t h0 = e2m1x2_to_half2_bits(s_in[(rg * 32 + i) * 64 + cp]);
                const uint32_t h1 = e2m1x2_to_half2_bits(s_in[(rg * 32 + i + 1) * 64 + cp]);
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&h0));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&h1));
                a[i] = f0.x * scv[t];
                a[i + 1] = f1.x * scv[t + 1];
                held[i >> 1] = __byte_perm(__float_as_uint(f0.y * scv[t]), __float_as_uint(f1.y * scv[t + 1]), 0x7632);
            }
        }
    }
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
        if (c == 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                a[2 * j] = __uint_as_float(held[j] << 16);
                a[2 * j + 1] = __uint_as_float(held[j] & 0xFFFF0000u);
            }
        }
        wht32(a);
        const int oc = 2 * cp + c;
        const int64_t orow = (int64_t)col0 + oc;
        const uint64_t g = (uint64_t)orow * (uint64_t)groups_per_out_row + (uint64_t)out_kb;
        const int64_t flat = orow * p.rows + out_kb * 32;
        uint32_t words[4];
        int e8m0;
        absmax_quantize_group<ROUND>(a, p.had_scale, g, flat, true, p.seed, p.offset, p.noise, flip, words, e8m0);
        // 64-byte rows, 16-byte chunk c of row r stored at chunk c ^ ((r >> 1) & 3): the layout the 64B-swizzled
        // tensor map of the store expects, and conflict-free for these 16-byte stores
        *reinterpret_cast<uint4*>(s_codes + oc * 64 + ((rg ^ ((oc >> 1) & 3)) << 4)) = make_uint4(words[0], words[1], words[2], words[3]);
        s_sf[(oc & 31) * 16 + (oc >> 5) * 4 + rg] = (uint8_t)e8m0;
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
        tma_store_2d(&tm_out, row0 / 2, col0, s_codes);
        bulk_store(p.sf_t + ((int64_t)blockIdx.x * p.sf_t_blocks_per_rowblock + blockIdx.y) * 512, s_sf, 512);
        bulk_commit();
        bulk_wait_read0();
    }
}

template <int ROUND>
static int launch_requant_t(const void* src, const TileTParams& p, uint8_t* codes_t, cudaStream_t stream) {
    CUtensorMap tm_in, tm_out;
    int rc = make_tmap_2d(&tm_in, src, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.cols / 2, p.rows, p.cols / 2, 64, TT, 0);
    if (rc) return rc;
    if ((rc = make_tmap_2d(&tm_out, codes_t, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.rows / 2, p.cols, p.rows / 2, 64, TT, 2))) return rc;
    auto kern = requant_t_kernel<ROUND>;
    static thread_local int smem_set = -1;
    if ((rc = set_max_smem_once(kern, RQ_SMEM, smem_set))) return rc;
    dim3 grid((unsigned)(p.cols / TT), (unsigned)(p.rows / TT));
    return check_cuda(launch_pdl(kern, grid, dim3(TT_THREADS), RQ_SMEM, stream, tm_in, tm_out, p), "requant_t launch");
}

template <int SRC, int ROUND, bool DUAL = false>
static int launch_tile_t(const void* src, const TileTParams& p, uint8_t* codes_t, cudaStream_t stream, uint8_t* codes_rows = nullptr) {
    CUtensorMap tm_in, tm_out, tm_rows;
    int rc;
    if (SRC == SRC_F32)
        rc = make_tmap_2d(&tm_in, src, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.cols, p.rows, p.cols * 4, 32, TT, 3);
    else if (SRC == SRC_BF16)
        rc = make_tmap_2d(&tm_in, src, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.cols, p.rows, p.cols * 2, 64, TT, 3);
    else
        rc = make_tmap_2d(&tm_in, src, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.cols / 2, p.rows, p.cols / 2, 64, TT, 0);
    if (rc) return rc;
    rc = make_tmap_2d(&tm_out, codes_t, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.rows / 2, p.cols, p.rows / 2, 64, TT, 2);
    if (rc) return rc;
    tm_rows = tm_out;
    if (DUAL && (rc = make_tmap_2d(&tm_rows, codes_rows, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.cols / 2, p.rows, p.cols / 2, 64, TT, 2))) return rc;
    auto kern = quant_tile_t_kernel<SRC, ROUND, DUAL>;
    constexpr int smem = tile_smem_bytes<SRC, DUAL>();
    static thread_local int smem_set = -1;
    rc = set_max_smem_once(kern, smem, smem_set);
    if (rc) return rc;
    dim3 grid((unsigned)(p.cols / TT), (unsigned)(p.rows / TT));
    return check_cuda(launch_pdl(kern, grid, dim3(TT_THREADS), smem, stream, tm_in, tm_out, tm_rows, p), "quant_tile_t launch");
}

static int validate_tile_t(const void* src, int64_t rows, int64_t cols, const void* codes_t, const void* sf_t, int rounding,
                           const float* noise) {
    if (!src || !codes_t || !sf_t) return fail(QUARTET_E_NULL, "source, codes_t and sf_t must be non-NULL");
    if (rows < 128 || cols < 128 || rows % 128 != 0 || cols % 128 != 0)
        return fail(QUARTET_E_SHAPE, "need rows and cols to be multiples of 128 (got %lld x %lld)", (long long)rows, (long long)cols);
    if (rows > 0x7FFFFFFF || cols > 0x7FFFFFFF || rows / 128 > 65535)
        return fail(QUARTET_E_SHAPE, "extent too large (rows <= 8388480)");
    if (!aligned16(src) || !aligned16(codes_t) || !aligned16(sf_t)) return fail(QUARTET_E_ALIGN, "pointers must be 16-byte aligned");
    if (rounding < 0 || rounding > 3) return fail(QUARTET_E_ARG, "rounding must be 0..3");
    if (rounding == QUARTET_ROUND_SR_NOISE && !noise) return fail(QUARTET_E_NULL, "noise tensor required for rounding mode 2");
    if (rounding == QUARTET_ROUND_SR_TLRAND && rows * cols > 0x7FFFFFFFLL)
        return fail(QUARTET_E_SHAPE, "rounding mode 3 indexes elements with 31 bits");
    int rc = bind_context_of(src);
    if (rc) return rc;
    return check_device();
}

template <int SRC>
static int dispatch_round(const void* src, const TileTParams& p, uint8_t* codes_t, int rounding, cudaStream_t s) {
    switch (rounding) {
        case 0: return launch_tile_t<SRC, 0>(src, p, codes_t, s);
        case 1: return launch_tile_t<SRC, 1>(src, p, codes_t, s);
        case 2: return launch_tile_t<SRC, 2>(src, p, codes_t, s);
        default: return launch_tile_t<SRC, 3>(src, p, codes_t, s);
    }
}

QUARTET_DEFINE_STATUS_READER(status_tile_t)

}  // namespace quartet

using namespace quartet;

extern "C" __attribute__((visibility("default"))) int quartet_quant_bwd_t(const void* x, int x_dtype, int64_t rows, int64_t cols, float had_scale,
                                   uint32_t signs, const uint32_t* signs_dev, int rounding, uint64_t seed,
                                   uint64_t offset, const float* noise, uint8_t* codes_t, uint8_t* sf_t,
                                   quartet_stream_t stream) {
    int rc = validate_tile_t(x, rows, cols, codes_t, sf_t, rounding, noise);
    if (rc) return rc;
    if (x_dtype != QUARTET_BF16 && x_dtype != QUARTET_F32) return fail(QUARTET_E_ARG, "x_dtype must be 0 (bf16) or 1 (f32)");
    TileTParams p{};
    p.rows = rows, p.cols = cols;
    p.sf_t = sf_t, p.sf_t_blocks_per_rowblock = ((rows / 32 + 3) / 4);
    p.had_scale = had_scale, p.signs = signs, p.signs_dev = signs_dev;
    p.seed = seed, p.offset = offset, p.noise = noise;
    p.in_scale = 1.f;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return x_dtype == QUARTET_F32 ? dispatch_round<SRC_F32>(x, p, codes_t, rounding, s)
                                  : dispatch_round<SRC_BF16>(x, p, codes_t, rounding, s);
}

extern "C" __attribute__((visibility("default"))) int quartet_requant_t(const uint8_t* codes, const uint8_t* sf, int64_t rows, int64_t cols, float in_scale,
                                 float had_scale, uint32_t signs, const uint32_t* signs_dev, int rounding,
                                 uint64_t seed, uint64_t offset, const float* noise, uint8_t* codes_t, uint8_t* sf_t,
                                 quartet_stream_t stream) {
    int rc = validate_tile_t(codes, rows, cols, codes_t, sf_t, rounding, noise);
    if (rc) return rc;
    if (!sf) return fail(QUARTET_E_NULL, "sf must be non-NULL");
    if (!aligned16(sf)) return fail(QUARTET_E_ALIGN, "sf must be 16-byte aligned");
    TileTParams p{};
    p.rows = rows, p.cols = cols;
    p.sf_in = sf, p.sf_in_blocks_per_rowblock = ((cols / 32 + 3) / 4);
    p.in_scale = in_scale;
    p.sf_t = sf_t, p.sf_t_blocks_per_rowblock = ((rows / 32 + 3) / 4);
    p.had_scale = had_scale, p.signs = signs, p.signs_dev = signs_dev;
    p.seed = seed, p.offset = offset, p.noise = noise;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in_scale != 1.0f) return dispatch_round<SRC_MXFP4>(codes, p, codes_t, rounding, s);  // general scale: the generic tile kernel
    switch (rounding) {
        case 0: return launch_requant_t<0>(codes, p, codes_t, s);
        case 1: return launch_requant_t<1>(codes, p, codes_t, s);
        case 2: return launch_requant_t<2>(codes, p, codes_t, s);
        default: return launch_requant_t<3>(codes, p, codes_t, s);
    }
}

// Q(E) and Q(E^T) from one read of E: codes/sf are what quartet_quant_bwd(x, ..., seed_rows) writes,
// codes_t/sf_t what quartet_quant_bwd_t(x, ..., seed_t) writes.
extern "C" __attribute__((visibility("default"))) int quartet_quant_bwd_dual(const void* x, int x_dtype, int64_t rows, int64_t cols, float had_scale,
                                      uint32_t signs, const uint32_t* signs_dev, int rounding, uint64_t seed_rows,
                                      uint64_t seed_t, uint64_t offset, uint8_t* codes, uint8_t* sf, uint8_t* codes_t,
                                      uint8_t* sf_t, quartet_stream_t stream) {
    int rc = validate_tile_t(x, rows, cols, codes_t, sf_t, rounding, nullptr);
    if (rc) return rc;
    if (!codes || !sf) return fail(QUARTET_E_NULL, "codes and sf must be non-NULL");
    if (!aligned16(codes) || !aligned16(sf)) return fail(QUARTET_E_ALIGN, "pointers must be 16-byte aligned");
    if (x_dtype != QUARTET_BF16 && x_dtype != QUARTET_F32) return fail(QUARTET_E_ARG, "x_dtype must be 0 (bf16) or 1 (f32)");
    if (rounding != QUARTET_ROUND_NEAREST && rounding != QUARTET_ROUND_SR_PHILOX)
        return fail(QUARTET_E_ARG, "the dual quantizer supports rounding modes 0 and 1 (got %d)", rounding);
    TileTParams p{};
    p.rows = rows, p.cols = cols;
    p.sf_t = sf_t, p.sf_t_blocks_per_rowblock = ((rows / 32 + 3) / 4);
    p.sf_rows = sf, p.sf_rows_blocks_per_rowblock = ((cols / 32 + 3) / 4);
    p.had_scale = had_scale, p.signs = signs, p.signs_dev = signs_dev;
    p.seed = seed_t, p.seed_rows = seed_rows, p.offset = offset, p.noise = nullptr;
    p.in_scale = 1.f;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (x_dtype == QUARTET_F32)
        return rounding ? launch_tile_t<SRC_F32, 1, true>(x, p, codes_t, s, codes) : launch_tile_t<SRC_F32, 0, true>(x, p, codes_t, s, codes);
    return rounding ? launch_tile_t<SRC_BF16, 1, true>(x, p, codes_t, s, codes) : launch_tile_t<SRC_BF16, 0, true>(x, p, codes_t, s, codes);
}
