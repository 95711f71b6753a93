// Row-wise MXFP4 quantizers: groups of 32 run along the contiguous (column) axis.
//
//   KIND_QUEST   forward quantizer   (mxfp4_triton.py:33-57,130-174 of the reference)
//   KIND_ABSMAX  backward quantizer  (mxfp4_triton.py:58-61,70-129)
//
// One CTA handles a 128-row x 128-column tile: TMA brings the tile into 128B-swizzled shared
// memory, each thread owns whole groups (rotation, statistics, rounding and packing stay in its
// registers), results are staged in shared memory and leave through TMA / bulk stores, so every
// global access is a full-width asynchronous copy.  HBM-bound: 2 B read, 0.53-0.66 B written per
// element.
#include "common.cuh"
#include "quant_math.cuh"

namespace quartet {

enum { KIND_QUEST = 0, KIND_ABSMAX = 1 };

struct RowsParams {
    int64_t rows, cols;
    uint8_t* sf;
    int64_t sf_blocks_per_rowblock;  // pad4(cols/32) / 4
    float had_scale, gaussian_scale;
    uint32_t signs;
    const uint32_t* signs_dev;
    uint64_t seed, offset;
    const float* noise;
    int has_mask;
    uint32_t box_rows;
};

constexpr int TILE_R = 128, TILE_C = 128, ROWS_THREADS = 256;
constexpr int OUT_CODES_BYTES = TILE_R * TILE_C / 2;  // 8192
constexpr int OUT_MASK_BYTES = TILE_R * TILE_C / 8;   // 2048
constexpr int OUT_SF_BYTES = 512;

template <bool F32>
constexpr int rows_smem_bytes() {
    return TILE_R * TILE_C * (F32 ? 4 : 2) + OUT_CODES_BYTES + OUT_MASK_BYTES + OUT_SF_BYTES + 64 + 1024;
}

// ROT = false: the 32-point rotation is skipped (the values are quantized as they are, h = 1): for tensors
// that were rotated elsewhere with a general matrix, and for the reference's rotation-free quantizer.
template <int KIND, int ROUND, bool F32, bool ROT>
__global__ void __launch_bounds__(ROWS_THREADS, F32 ? 3 : 4) quant_rows_kernel(const __grid_constant__ CUtensorMap tm_x,
                                                                  const __grid_constant__ CUtensorMap tm_codes,
                                                                  const __grid_constant__ CUtensorMap tm_mask,
                                                                  const RowsParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int IN_BYTES = TILE_R * TILE_C * (F32 ? 4 : 2);
    constexpr int NBOX = F32 ? 4 : 2;          // 128-byte-wide boxes per tile row
    constexpr int BOX_BYTES = TILE_R * 128;    // one box: 128 rows x 128 B
    uint8_t* s_in = smem;
    uint8_t* s_codes = smem + IN_BYTES;
    uint8_t* s_mask = s_codes + OUT_CODES_BYTES;
    uint8_t* s_sf = s_mask + OUT_MASK_BYTES;
    uint64_t* bar = reinterpret_cast<uint64_t*>(s_sf + OUT_SF_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col0 = blockIdx.x * TILE_C;
    const int64_t row0 = (int64_t)blockIdx.y * TILE_R;

    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();  // the tensor this kernel reads (and the buffers it overwrites) belong to the previous kernel until here
    if (tid == 0) {
        mbar_arrive_expect_tx(bar, NBOX * 128u * p.box_rows);
#pragma unroll
        for (int b = 0; b < NBOX; ++b) tma_load_2d(s_in + b * BOX_BYTES, &tm_x, col0 + b * (F32 ? 32 : 64), (int)row0, bar);
    }

    uint32_t signs = 0;
    if (KIND == KIND_ABSMAX) signs = p.signs_dev ? __ldg(p.signs_dev) : p.signs;
    uint32_t flip[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) flip[q] = spread_sign_bits((signs >> (8 * q)) & 0xFFu);

    mbar_wait(bar, 0, WAIT_QUANT_LOAD);

    const int row = (warp & 3) * 32 + lane;
    const int64_t grow = row0 + row;
    const float h = p.had_scale;

#pragma unroll 1
    for (int it = 0; it < 2; ++it) {
        const int gk = (warp >> 2) * 2 + it;  // group within the tile row, 0..3
        float w[32];
        load_row_group<F32>(s_in, row, gk, w);
        uint32_t words[4];
        uint32_t mbits = 0;
        int e8m0;
        if (KIND == KIND_QUEST) {
            quest_quantize_group<ROT>(w, h, p.gaussian_scale, words, mbits, e8m0);
        } else {
            if (ROT) wht32(w);
            const uint64_t g = (uint64_t)grow * (uint64_t)(p.cols >> 5) + (uint64_t)((col0 >> 5) + gk);
            const int64_t flat = grow * p.cols + col0 + gk * 32;
            absmax_quantize_group<ROUND>(w, h, g, flat, grow < p.rows, p.seed, p.offset, p.noise, flip, words, e8m0);
        }
        // 64-byte rows, 16-byte chunk c of row r at chunk c ^ ((r >> 1) & 3): what the 64B-swizzled tensor map of
        // the store expects; a quarter-warp's eight 16-byte stores then fall into eight different bank groups
        *reinterpret_cast<uint4*>(s_codes + row * 64 + ((gk ^ ((row >> 1) & 3)) << 4)) = make_uint4(words[0], words[1], words[2], words[3]);
        if (KIND == KIND_QUEST) *reinterpret_cast<uint32_t*>(s_mask + row * 16 + gk * 4) = mbits;
        // rows past the tensor's last one (padding of the 128-row scale block) get scale byte 0, whatever the tile held there
        s_sf[(row & 31) * 16 + (row >> 5) * 4 + gk] = grow < p.rows ? (uint8_t)e8m0 : (uint8_t)0;
    }

    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
        tma_store_2d(&tm_codes, col0 / 2, (int)row0, s_codes);
        if (KIND == KIND_QUEST && p.has_mask) tma_store_2d(&tm_mask, col0 / 8, (int)row0, s_mask);
        uint8_t* sf_dst = p.sf + ((int64_t)blockIdx.y * p.sf_blocks_per_rowblock + blockIdx.x) * 512;
        bulk_store(sf_dst, s_sf, 512);
        bulk_commit();
        bulk_wait_read0();
    }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
template <int KIND, int ROUND, bool F32, bool ROT = true>
static int launch_rows(const void* x, const RowsParams& p, uint8_t* codes, uint8_t* mask, cudaStream_t stream) {
    CUtensorMap tm_x, tm_codes, tm_mask;
    int rc;
    const uint32_t box_rows = p.box_rows;
    if (F32)
        rc = make_tmap_2d(&tm_x, x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.cols, p.rows, p.cols * 4, 32, box_rows, 3);
    else
        rc = make_tmap_2d(&tm_x, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.cols, p.rows, p.cols * 2, 64, box_rows, 3);
    if (rc) return rc;
    rc = make_tmap_2d(&tm_codes, codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.cols / 2, p.rows, p.cols / 2, 64, box_rows, 2);
    if (rc) return rc;
    if (mask) {
        rc = make_tmap_2d(&tm_mask, mask, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.cols / 8, p.rows, p.cols / 8, 16, box_rows, 0);
        if (rc) return rc;
    } else {
        tm_mask = tm_codes;  // never used: the kernel stores no mask
    }
    auto kern = quant_rows_kernel<KIND, ROUND, F32, ROT>;
    constexpr int smem = rows_smem_bytes<F32>();
    static thread_local int smem_set = -1;
    rc = set_max_smem_once(kern, smem, smem_set);
    if (rc) return rc;
    dim3 grid((unsigned)(p.cols / TILE_C), (unsigned)((p.rows + TILE_R - 1) / TILE_R));
    return check_cuda(launch_pdl(kern, grid, dim3(ROWS_THREADS), smem, stream, tm_x, tm_codes, tm_mask, p), "quant_rows launch");
}

static int validate_rows(const void* x, int x_dtype, int64_t rows, int64_t cols, const void* codes, const void* sf) {
    if (!x || !codes || !sf) return fail(QUARTET_E_NULL, "x, codes and sf must be non-NULL");
    if (x_dtype != QUARTET_BF16 && x_dtype != QUARTET_F32) return fail(QUARTET_E_ARG, "x_dtype must be 0 (bf16) or 1 (f32)");
    if (rows < 1 || cols < 128 || cols % 128 != 0)
        return fail(QUARTET_E_SHAPE, "need rows >= 1 and cols a multiple of 128 (got %lld x %lld)", (long long)rows, (long long)cols);
    if (rows > 0x7FFFFFFF || cols > 0x7FFFFFFF || (rows + 127) / 128 > 65535)
        return fail(QUARTET_E_SHAPE, "extent too large (rows <= 8388480)");
    if (!aligned16(x) || !aligned16(codes) || !aligned16(sf)) return fail(QUARTET_E_ALIGN, "pointers must be 16-byte aligned");
    int rc = bind_context_of(x);
    if (rc) return rc;
    return check_device();
}

QUARTET_DEFINE_STATUS_READER(status_rows)

}  // namespace quartet

using namespace quartet;

extern "C" __attribute__((visibility("default"))) int quartet_quant_fwd(const void* x, int x_dtype, int64_t rows, int64_t cols, float had_scale,
                                 float gaussian_scale, uint8_t* codes, uint8_t* sf, uint8_t* mask,
                                 quartet_stream_t stream) {
    int rc = validate_rows(x, x_dtype, rows, cols, codes, sf);
    if (rc) return rc;
    if (mask && !aligned16(mask)) return fail(QUARTET_E_ALIGN, "mask must be 16-byte aligned");
    RowsParams p{};
    p.rows = rows, p.cols = cols, p.sf = sf;
    p.sf_blocks_per_rowblock = ((cols / 32 + 3) / 4);
    p.had_scale = had_scale, p.gaussian_scale = gaussian_scale;
    p.has_mask = mask != nullptr;
    p.box_rows = (uint32_t)(rows < TILE_R ? rows : TILE_R);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (x_dtype == QUARTET_F32) return launch_rows<KIND_QUEST, 0, true>(x, p, codes, mask, s);
    return launch_rows<KIND_QUEST, 0, false>(x, p, codes, mask, s);
}

extern "C" __attribute__((visibility("default"))) int quartet_quant_bwd(const void* x, int x_dtype, int64_t rows, int64_t cols, float had_scale,
                                 uint32_t signs, const uint32_t* signs_dev, int rounding, uint64_t seed,
                                 uint64_t offset, const float* noise, uint8_t* codes, uint8_t* sf,
                                 quartet_stream_t stream) {
    int rc = validate_rows(x, x_dtype, rows, cols, codes, sf);
    if (rc) return rc;
    if (rounding < 0 || rounding > 3) return fail(QUARTET_E_ARG, "rounding must be 0..3");
    if (rounding == QUARTET_ROUND_SR_NOISE && !noise) return fail(QUARTET_E_NULL, "noise tensor required for rounding mode 2");
    if (rounding == QUARTET_ROUND_SR_TLRAND && rows * cols > 0x7FFFFFFFLL)
        return fail(QUARTET_E_SHAPE, "rounding mode 3 indexes elements with 31 bits");
    RowsParams p{};
    p.rows = rows, p.cols = cols, p.sf = sf;
    p.sf_blocks_per_rowblock = ((cols / 32 + 3) / 4);
    p.had_scale = had_scale;
    p.signs = signs, p.signs_dev = signs_dev;
    p.seed = seed, p.offset = offset, p.noise = noise;
    p.box_rows = (uint32_t)(rows < TILE_R ? rows : TILE_R);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f32 = x_dtype == QUARTET_F32;
#define QB(R)                                                                     \
    case R:                                                                       \
        return f32 ? launch_rows<KIND_ABSMAX, R, true>(x, p, codes, nullptr, s)   \
                   : launch_rows<KIND_ABSMAX, R, false>(x, p, codes, nullptr, s);
    switch (rounding) {
        QB(0) QB(1) QB(2) QB(3)
    }
#undef QB
    return fail(QUARTET_E_ARG, "unreachable");
}

// Group-of-32 scaling, rounding and packing WITHOUT the rotation: x is quantized as it is.
extern "C" __attribute__((visibility("default"))) int quartet_quant_group32(const void* x, int x_dtype, int64_t rows, int64_t cols, int kind,
                                     float gaussian_scale, int rounding, uint64_t seed, uint64_t offset, const float* noise,
                                     uint8_t* codes, uint8_t* sf, uint8_t* mask, quartet_stream_t stream) {
    if (kind != 0 && kind != 1) return fail(QUARTET_E_ARG, "kind must be 0 (std-scaled, round to nearest, clip mask) or 1 (absmax-scaled)");
    if (kind == 1) {
        if (rounding < 0 || rounding > 3) return fail(QUARTET_E_ARG, "rounding must be 0..3");
        if (rounding == QUARTET_ROUND_SR_NOISE && !noise) return fail(QUARTET_E_NULL, "noise tensor required for rounding mode 2");
        if (rounding == QUARTET_ROUND_SR_TLRAND && rows * cols > 0x7FFFFFFFLL) return fail(QUARTET_E_SHAPE, "rounding mode 3 indexes elements with 31 bits");
    }
    if (mask && !aligned16(mask)) return fail(QUARTET_E_ALIGN, "mask must be 16-byte aligned");
    int rc = validate_rows(x, x_dtype, rows, cols, codes, sf);
    if (rc) return rc;
    RowsParams p{};
    p.rows = rows, p.cols = cols, p.sf = sf;
    p.sf_blocks_per_rowblock = ((cols / 32 + 3) / 4);
    p.had_scale = 1.0f, p.gaussian_scale = gaussian_scale;
    p.seed = seed, p.offset = offset, p.noise = noise;
    p.box_rows = (uint32_t)(rows < TILE_R ? rows : TILE_R);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f32 = x_dtype == QUARTET_F32;
    if (kind == 0) {
        p.has_mask = mask != nullptr;
        return f32 ? launch_rows<KIND_QUEST, 0, true, false>(x, p, codes, mask, s) : launch_rows<KIND_QUEST, 0, false, false>(x, p, codes, mask, s);
    }
#define QG(R)                                                                              \
    case R:                                                                                \
        return f32 ? launch_rows<KIND_ABSMAX, R, true, false>(x, p, codes, nullptr, s)     \
                   : launch_rows<KIND_ABSMAX, R, false, false>(x, p, codes, nullptr, s);
    switch (rounding) {
        QG(0) QG(1) QG(2) QG(3)
    }
#undef QG
    return fail(QUARTET_E_ARG, "unreachable");
}
