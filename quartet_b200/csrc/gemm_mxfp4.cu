// Block-scaled MXFP4 GEMM for sm_100a:  D[M,N] = alpha * A[M,K] . B[N,K]^T
//
//   A, B    packed e2m1 (two per byte), K-major, row pitch K/2 bytes
//   SFA/SFB E8M0 scales, one per 32 K-elements, in 512-byte blocks of 128 rows x 4 scales
//   D       bf16 or fp32, row-major; optional fused "mask, then rotate back by the 32-point
//           Hadamard" epilogue (the straight-through backward of the forward quantizer).
//
// Structure of the one-CTA kernel (one CTA per SM, persistent over 128 x BN output tiles, 320 threads);
// the two-CTA kernel further down keeps the roles and spreads them over a CTA pair and 512 threads:
//   warp 0      TMA producer: per K-stage (256 elements) two tensor copies (A, B; 128B swizzle)
//               and the stage's scale blocks as plain bulk copies, all signalling one mbarrier
//   warp 1      allocates TMEM and issues tcgen05.mma.kind::mxf4.block_scale back to back (K = 64
//               per instruction, fp32 accumulators in TMEM); tcgen05.commit releases the stage /
//               publishes the accumulator
//   warps 6-9   scale feeders: move the stage's E8M0 bytes shared -> registers -> tensor memory
//               (tcgen05.st), one warp per TMEM lane quadrant, so that the tensor pipe only ever
//               sees MMAs (scale copies issued in the MMA stream serialise with them)
//   warps 2-5   epilogue: tcgen05.ld one accumulator row x 32 columns per thread (= exactly one
//               Hadamard group), scale, optional mask + un-rotation, convert, stage the 32 x 32
//               block in swizzled shared memory, TMA store
// Two-CTA kernel (cta_group::2, 256 x 256 tile per pair): each CTA stages its own rows of A and half
// of B; three warps issue the copies (A, B, scales); the scale copies and their tensor-memory feed run
// ahead of the operands on their own barriers; consecutive tiles use overlapping accumulator column
// ranges so that the next tile's MMAs start while the previous epilogue is still draining; tiles are
// visited in compact bands; the fp32 result can be scattered by row range to per-owner destinations.
// Every wait is bounded; a wait that gives up records itself in the fault word and the CTA
// winds down (frees its TMEM) instead of hanging.
#include "common.cuh"
#include "quant_math.cuh"
#include "tcgen05.cuh"

namespace quartet {

constexpr int BM = 128;
constexpr int BK_BYTES = 128;   // 256 e2m1 elements per stage along K
constexpr int GEMM_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warps 6-9 scale feeders
constexpr int GEMM2_THREADS = 512; // two-CTA kernel: warps 0, 10, 15 issue copies (A, B, scales), 11-14 are four more epilogue warps

template <int BN>
struct GemmCfg {
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int ACC_STAGES = BN == 256 ? 1 : 2;
    static constexpr int A_BYTES = BM * BK_BYTES;           // 16 KB
    static constexpr int B_BYTES = BN * BK_BYTES;           // 16 / 32 KB
    static constexpr int SFA_BYTES = 1024;                  // 2 K-chunks x 512 B
    static constexpr int SFB_BLOCKS = BN / 128;             // 128-row scale blocks a tile can touch
    static constexpr int SFB_BYTES = SFB_BLOCKS * 1024;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
    static constexpr int NSEG = BN / 32;                    // 32-row segments of B = scale columns per K-chunk
    static constexpr int SFB_ST = NSEG <= 4 ? 4 : 8;        // columns written per tcgen05.st
    static constexpr int SF_COLS = 8 + 2 * SFB_ST;          // SFA 2 x 4, SFB 2 x SFB_ST columns per stage
    static constexpr int ACC_COL0 = 0;
    static constexpr int SF_COL0 = ACC_STAGES * BN;         // ring of STAGES scale slots follows
    static constexpr int TMEM_COLS = 512;
    static constexpr int STG_BYTES = 4 * 4096;              // epilogue staging, 4 KB per epilogue warp
    static constexpr int SMEM = STAGES * STAGE_BYTES + STG_BYTES + 512 + 1024;
    static_assert(SF_COL0 + STAGES * SF_COLS <= TMEM_COLS, "tensor memory capacity");
    static_assert(SMEM <= 232448, "shared memory capacity");
};

struct GemmParams {
    const uint8_t* a_sf;
    const uint8_t* b_sf;
    int M, N, K;
    int k_chunks;            // K / 128
    int m_tiles, n_tiles;
    float alpha;
    const uint8_t* mask;     // [M, N/8] or NULL
    float had_scale;
    int d_f32;
    int rows_per_owner;      // > 0: output rows are scattered to per-owner destinations (two-CTA kernel only)
};

// Destinations of a scattered output: rows [o * rows_per_owner, (o + 1) * rows_per_owner) of D are
// stored through map o, as a dense [rows_per_owner, N] fp32 matrix that may live in another GPU's
// memory (plain TMA stores over NVLink; nothing here reads peer memory).
constexpr int MAX_OWNERS = 8;
struct ScatterMaps {
    CUtensorMap m[MAX_OWNERS];
};

// ---------------------------------------------------------------------------
// tcgen05 wrappers specific to the block-scaled kind (the shared ones are in tcgen05.cuh)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tc_mma_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        :
        : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// Instruction descriptor, kind::mxf4, E2M1 x E2M1, UE8M0 scales, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t make_idesc(int n, uint32_t sf_id) {
    uint32_t d = 0;
    d |= sf_id << 4;                    // B scale id (byte pair within the 32-bit scale column)
    d |= 1u << 7;                       // A format E2M1
    d |= 1u << 10;                      // B format E2M1
    d |= (uint32_t)(n >> 3) << 17;      // N
    d |= 1u << 23;                      // scale format UE8M0
    d |= (uint32_t)(BM >> 4) << 24;     // M
    d |= sf_id << 29;                   // A scale id
    return d;
}

// Bounded wait on wall-clock time (2 s), for the pipeline barriers.
__device__ __forceinline__ bool gemm_wait(uint64_t* bar, uint32_t parity, int32_t who, volatile int* dead) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*dead) return false;
    uint64_t t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u) {
            uint64_t now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            if (now - t0 > 2000000000ull || *dead) break;
        }
    }
    atomicOr(&g_status, who | 0x100);
    *dead = 1;
    return false;
}

// Epilogue of one 32-row x 32-column block held as one accumulator row per thread: scale, optional
// mask + un-rotation (the 32 columns are exactly one Hadamard group), convert, stage 32 rows x 64
// bytes in swizzled shared memory and hand them to TMA -- one store of 32 rows x 64 bytes for bf16, two
// of 16 rows x 128 bytes for fp32.  Two 2 KB staging buffers per warp alternate.
template <int NBUF>
__device__ __forceinline__ void epilogue_block(const uint32_t (&r)[32], const GemmParams& p, const CUtensorMap* tm_d,
                                               int64_t row, int row0, int col, uint8_t* stg, uint32_t& n_stores, int lane) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
    if (p.mask) {
        const uint32_t m = *reinterpret_cast<const uint32_t*>(p.mask + row * (p.N >> 3) + (col >> 3));
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = ((m >> i) & 1u) ? v[i] : 0.f;
        wht32(v);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= p.had_scale;
    }
    if (p.d_f32) {
        // two stores of 16 rows x 128 bytes (128B-swizzled staging): full 128-byte row segments, which is
        // what keeps stores to another GPU's memory efficient on NVLink
#pragma unroll
        for (int hf = 0; hf < 2; ++hf, ++n_stores) {
            uint8_t* buf = stg + (NBUF == 2 ? (n_stores & 1) * 2048 : 0);
            if (lane == 0) { if (NBUF == 2) bulk_wait_read1(); else bulk_wait_read0(); }
            __syncwarp();
            if ((lane >> 4) == hf) {
                uint8_t* dst = buf + (lane & 15) * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<float4*>(dst + ((j ^ (lane & 7)) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(tm_d, col, row0 + 16 * hf, buf);
                bulk_commit();
            }
        }
    } else {
        uint8_t* buf = stg + (NBUF == 2 ? (n_stores & 1) * 2048 : 0);
        ++n_stores;
        if (lane == 0) { if (NBUF == 2) bulk_wait_read1(); else bulk_wait_read0(); }
        __syncwarp();
        uint8_t* dst = buf + lane * 64;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                __nv_bfloat162 t = __floats2bfloat162_rn(v[8 * j + 2 * k], v[8 * j + 2 * k + 1]);
                w[k] = *reinterpret_cast<uint32_t*>(&t);
            }
            *reinterpret_cast<uint4*>(dst + ((j ^ ((lane >> 1) & 3)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(tm_d, col, row0, buf);
            bulk_commit();
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_mxfp4_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                                    const __grid_constant__ CUtensorMap tm_b,
                                                                    const __grid_constant__ CUtensorMap tm_d,
                                                                    const GemmParams p) {
    using C = GemmCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_a = smem;
    uint8_t* s_b = s_a + C::STAGES * C::A_BYTES;
    uint8_t* s_stg = s_b + C::STAGES * C::B_BYTES;           // 1024-aligned
    uint8_t* s_sfa = s_stg + C::STG_BYTES;
    uint8_t* s_sfb = s_sfa + C::STAGES * C::SFA_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_sfb + C::STAGES * C::SFB_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = full + C::STAGES;
    uint64_t* sf_full = empty + C::STAGES;
    uint64_t* acc_full = sf_full + C::STAGES;
    uint64_t* acc_empty = acc_full + C::ACC_STAGES;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(acc_empty + C::ACC_STAGES);
    volatile int* dead = reinterpret_cast<volatile int*>(s_tmem + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
            mbar_init(&sf_full[i], 4);
        }
        for (int i = 0; i < C::ACC_STAGES; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 4);
        }
        *dead = 0;
        fence_mbar_init();
        prefetch_tmap(&tm_a);
        prefetch_tmap(&tm_b);
        prefetch_tmap(&tm_d);
    }
    if (warp == 1) {
        tmem_alloc(s_tmem, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    const int n_tiles_total = p.m_tiles * p.n_tiles;
    const int k_stages = (p.k_chunks + 1) >> 1;
    const int64_t sf_blocks_per_rowblock = p.k_chunks;  // K/128 scale blocks per 128 rows

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < n_tiles_total && !*dead; tile += gridDim.x) {
                const int m_blk = tile % p.m_tiles, n_blk = tile / p.m_tiles;
                const int m0 = m_blk * BM, n0 = n_blk * BN;
                const int blk0 = n0 / 128;
                const int n_blocks = (min(n0 + BN, p.N) - 1) / 128 - blk0 + 1;
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1;
                    if (!gemm_wait(&empty[s], ph ^ 1, WAIT_GEMM_EMPTY, dead)) break;
                    const int nch = min(2, p.k_chunks - 2 * ks);
                    mbar_arrive_expect_tx(&full[s], C::A_BYTES + C::B_BYTES + nch * 512 * (1 + n_blocks));
                    tma_load_2d(s_a + s * C::A_BYTES, &tm_a, ks * BK_BYTES, m0, &full[s]);
                    tma_load_2d(s_b + s * C::B_BYTES, &tm_b, ks * BK_BYTES, n0, &full[s]);
                    bulk_load(s_sfa + s * C::SFA_BYTES, p.a_sf + ((int64_t)m_blk * sf_blocks_per_rowblock + 2 * ks) * 512,
                              nch * 512, &full[s]);
                    for (int rb = 0; rb < n_blocks; ++rb)
                        bulk_load(s_sfb + s * C::SFB_BYTES + rb * 1024,
                                  p.b_sf + ((int64_t)(blk0 + rb) * sf_blocks_per_rowblock + 2 * ks) * 512, nch * 512,
                                  &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            uint32_t it = 0, acc_it = 0;
            for (int tile = blockIdx.x; tile < n_tiles_total && !*dead; tile += gridDim.x, ++acc_it) {
                const int as = acc_it % C::ACC_STAGES;
                const uint32_t aph = (acc_it / C::ACC_STAGES) & 1;
                if (!gemm_wait(&acc_empty[as], aph ^ 1, WAIT_GEMM_ACC_EMPTY, dead)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + C::ACC_COL0 + as * BN;
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1;
                    if (!gemm_wait(&full[s], ph, WAIT_GEMM_FULL, dead)) break;
                    if (!gemm_wait(&sf_full[s], ph, WAIT_GEMM_SF, dead)) break;
                    tc_fence_after();
                    const int nch = min(2, p.k_chunks - 2 * ks);
                    const uint32_t sf_tmem = tmem_base + C::SF_COL0 + s * C::SF_COLS;
                    const uint64_t adesc = make_desc_sw128(smem_u32(s_a + s * C::A_BYTES));
                    const uint64_t bdesc = make_desc_sw128(smem_u32(s_b + s * C::B_BYTES));
                    for (int c = 0; c < nch; ++c) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const uint32_t koff = (uint32_t)((c * 2 + j) * 32) >> 4;  // 64 elements = 32 bytes
                            const uint32_t sfid = (uint32_t)j * 2u;
                            tc_mma_mxf4(d_tmem, adesc + koff, bdesc + koff, make_idesc(BN, sfid),
                                        (sf_tmem + c * 4) | (sfid << 30), (sf_tmem + 8 + c * C::SFB_ST) | (sfid << 30),
                                        (ks | c | j) != 0);
                        }
                    }
                    tc_commit(&empty[s]);  // frees the stage once the MMAs above have read it
                }
                tc_commit(&acc_full[as]);  // accumulator complete
            }
        }
    } else if (warp >= 6) {
        // ------------------------------ scale feeders ------------------------------
        // Each of the four warps copies the stage's scale bytes from shared memory into its own
        // 32-lane quadrant of tensor memory: row r of a 128-row block lives in lane r % 32, 32-bit
        // column r / 32 (one byte per 32-element K-block), replicated in all four quadrants.
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < n_tiles_total && !*dead; tile += gridDim.x) {
            const int n0 = (tile / p.m_tiles) * BN;
            const int seg0 = (n0 % 128) / 32;  // first 32-row segment of the tile inside its first scale block
            for (int ks = 0; ks < k_stages; ++ks, ++it) {
                const int s = it % C::STAGES;
                const uint32_t ph = (it / C::STAGES) & 1;
                if (!gemm_wait(&full[s], ph, WAIT_GEMM_FULL, dead)) break;
                const int nch = min(2, p.k_chunks - 2 * ks);
                const uint32_t sf_tmem = tmem_base + lane_base + C::SF_COL0 + s * C::SF_COLS;
                const uint8_t* sfa = s_sfa + s * C::SFA_BYTES + lane * 16;
                const uint8_t* sfb = s_sfb + s * C::SFB_BYTES + lane * 16;
                for (int c = 0; c < nch; ++c) {
                    uint32_t r[8];
                    const uint4 va = *reinterpret_cast<const uint4*>(sfa + c * 512);
                    r[0] = va.x, r[1] = va.y, r[2] = va.z, r[3] = va.w;
                    tc_st4(sf_tmem + c * 4, r);
#pragma unroll
                    for (int j = 0; j < C::SFB_ST; ++j) {
                        const int seg = seg0 + j;
                        r[j] = j < C::NSEG ? *reinterpret_cast<const uint32_t*>(sfb + (seg >> 2) * 1024 + c * 512 + (seg & 3) * 4) : 0u;
                    }
                    if (C::SFB_ST == 4)
                        tc_st4(sf_tmem + 8 + c * C::SFB_ST, r);
                    else
                        tc_st8(sf_tmem + 8 + c * C::SFB_ST, r);
                }
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sf_full[s]);
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int q = warp & 3;  // TMEM lane quadrant this warp may read
        uint8_t* stg = s_stg + (warp - 2) * 4096;
        uint32_t acc_it = 0, n_stores = 0;
        for (int tile = blockIdx.x; tile < n_tiles_total && !*dead; tile += gridDim.x, ++acc_it) {
            const int m_blk = tile % p.m_tiles, n_blk = tile / p.m_tiles;
            const int n0 = n_blk * BN;
            const int as = acc_it % C::ACC_STAGES;
            const uint32_t aph = (acc_it / C::ACC_STAGES) & 1;
            if (!gemm_wait(&acc_full[as], aph, WAIT_GEMM_ACC_FULL, dead)) break;
            tc_fence_after();
            const int row0 = m_blk * BM + q * 32;
            const int64_t row = (int64_t)row0 + lane;
            const int n_chunks = min(BN, p.N - n0) / 32;
            for (int ch = 0; ch < n_chunks; ++ch) {
                uint32_t r[32];
                tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + C::ACC_COL0 + as * BN + ch * 32, r);
                tc_wait_ld();
                epilogue_block<2>(r, p, &tm_d, row, row0, n0 + ch * 32, stg, n_stores, lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
        }
        if (lane == 0) bulk_wait0();
    }

    // ------------------------------ wind-down ------------------------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*dead) {
        // a wait gave up: give copies still in flight time to land before shared memory is released
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ===========================================================================================
// Two-CTA variant (cta_group::2): a cluster of two CTAs on one TPC computes a 256 x BN tile.
// Each CTA stages its own 128 rows of A and HALF of the B tile (BN/2 rows); one thread of the
// leader CTA issues MMAs that read both CTAs' shared memory and accumulate into both CTAs' tensor
// memory (rows 0-127 of the tile in the leader, 128-255 in its peer).  Per output element this
// halves the B traffic through shared memory and cuts the L2 -> SM operand traffic by a third,
// which is what bounds the one-CTA kernel.  Scales: each CTA feeds SFA of its own rows and SFB of
// the whole tile into its own tensor memory.  Cross-CTA signalling uses remote mbarrier arrives
// and tcgen05.commit onto the peer's barriers; no multicast copy is involved.
// ===========================================================================================
template <int BN, int NSTG = 1>
struct Gemm2Cfg {
    static constexpr int NSEG = BN / 32;                     // 32-row segments of B = scale columns per K-chunk
    static constexpr int SFB_ST = NSEG <= 4 ? 4 : 8;         // columns written per tcgen05.st
    static constexpr int SF_COLS = 8 + 2 * SFB_ST;           // SFA 2 x 4, SFB 2 x SFB_ST columns per stage
    static constexpr int ACC_STAGES = (2 * BN + 2 * SF_COLS <= 512) ? 2 : 1;
    // A 256-column accumulator leaves no room for a second one beside the scales.  Consecutive tiles
    // then alternate between columns [0, 256) and [128, 384): the two share only columns [128, 256),
    // which the epilogue pulls into registers first, so the next tile's MMAs start after a quarter of
    // a drain instead of a whole epilogue.
    static constexpr bool OVERLAP = ACC_STAGES == 1;
    static constexpr int ACC_SHIFT = 128;
    static constexpr int SF_COL0 = OVERLAP ? BN + ACC_SHIFT : ACC_STAGES * BN;
    static constexpr int SF_SLOTS = (512 - SF_COL0) / SF_COLS >= 4 ? 4 : 2;
    static constexpr int TMEM_COLS = 512;
    static constexpr int A_BYTES = BM * BK_BYTES;            // 16 KB
    static constexpr int B_BYTES = (BN / 2) * BK_BYTES;      // this CTA's half of the B tile
    static constexpr int SFA_BYTES = 1024;
    static constexpr int SFB_BLOCKS = (BN % 128 == 0) ? BN / 128 : BN / 128 + 2;  // 128-row scale blocks a tile can touch
    static constexpr int SFB_BYTES = SFB_BLOCKS * 1024;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
    static constexpr int STG_BYTES = 8 * NSTG * 2048;        // epilogue staging: NSTG buffers of 2 KB per epilogue warp (8 warps)
    static constexpr int STAGES = (232448 - STG_BYTES - 512) / STAGE_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + STG_BYTES + 512;
    static_assert(SF_COL0 + SF_SLOTS * SF_COLS <= TMEM_COLS, "tensor memory capacity");
    static_assert(SF_SLOTS < STAGES, "scale slots are recycled through the stage barriers");
    static_assert(B_BYTES % 1024 == 0, "operand stages stay 1024-byte aligned");
};

// One lane of a fully converged warp (elect.sync): the issuing warp runs its loop on all 32 lanes so
// that ring indices, descriptors and addresses stay warp-uniform, and only the tcgen05 instructions
// themselves are predicated on the elected lane.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
        "elect.sync rx|px, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, px;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    // default semantics (as the pipelines of CUTLASS use for consumer -> producer signalling across
    // CTAs); an explicit .release.cluster here costs ~1500 cycles per arrive
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on a barrier (given by its shared::cluster address) once all MMAs issued so far are done
__device__ __forceinline__ void tc_commit2(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
                 : "memory");
}
// the same, arriving on the barrier at this shared-memory offset in BOTH CTAs of the pair (one
// instruction instead of two commits; only the completion signal is multicast, no data copy)
__device__ __forceinline__ void tc_commit2_pair(uint32_t own_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     own_addr),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void tc_mma2_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        :
        : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
__device__ __forceinline__ uint32_t make_idesc2(int n, uint32_t sf_id) {
    uint32_t d = 0;
    d |= sf_id << 4;
    d |= 1u << 7;
    d |= 1u << 10;
    d |= (uint32_t)(n >> 3) << 17;
    d |= 1u << 23;
    d |= (uint32_t)(256 >> 4) << 24;    // M = 256 across the CTA pair
    d |= sf_id << 29;
    return d;
}

// Tile order of the persistent two-CTA kernel.  Tiles that run at the same time (consecutive
// indices) form a compact block of RASTER_BAND row pairs by as many column tiles, so that the rows of A
// and B a wave reads are few and each is shared by many CTAs while it is hot in the L2 of their die.
constexpr int RASTER_BAND = 8;
__device__ __forceinline__ void tile_coords(int tile, int m_pairs, int n_tiles, int& m_pair, int& n_blk) {
    const int per_band = RASTER_BAND * n_tiles;
    const int band = tile / per_band, within = tile - band * per_band;
    const int rows = min(RASTER_BAND, m_pairs - band * RASTER_BAND);
    n_blk = within / rows;
    m_pair = band * RASTER_BAND + (within - n_blk * rows);
}

template <int BN, int NSTG>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM2_THREADS, 1)
    gemm_mxfp4_2cta_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                           const __grid_constant__ CUtensorMap tm_d, const __grid_constant__ CUtensorMap tm_sfb,
                           const __grid_constant__ ScatterMaps sc, const GemmParams p) {
    using C = Gemm2Cfg<BN, NSTG>;
    // Dynamic shared memory is the kernel's only shared memory and starts 1024-byte aligned (checked
    // below); no slack is reserved for re-aligning it, which is what makes room for a sixth stage.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicOr(&g_status, WAIT_GEMM_ALIGN | 0x100);
        return;
    }
    uint8_t* s_a = smem;
    uint8_t* s_b = s_a + C::STAGES * C::A_BYTES;
    uint8_t* s_stg = s_b + C::STAGES * C::B_BYTES;
    uint8_t* s_sfa = s_stg + C::STG_BYTES;
    uint8_t* s_sfb = s_sfa + C::STAGES * C::SFA_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_sfb + C::STAGES * C::SFB_BYTES);
    uint64_t* full = bars;                            // local: this CTA's copies of a stage have landed
    uint64_t* empty = full + C::STAGES;               // local: the pair's MMAs are done with the stage
    uint64_t* sf_full = empty + C::STAGES;            // leader only: 8 feeder warps (both CTAs) have fed the stage
    uint64_t* sf_land = sf_full + C::STAGES;          // local: the stage's scale blocks have landed
    uint64_t* sf_free = sf_land + C::STAGES;          // local: the 4 feeder warps hold the stage's scales in registers
    uint64_t* acc_full = sf_free + C::STAGES;         // local: accumulator complete
    uint64_t* acc_empty = acc_full + C::ACC_STAGES;   // leader only: 8 epilogue warps (both CTAs) have drained it
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(acc_empty + C::ACC_STAGES);
    volatile int* dead = reinterpret_cast<volatile int*>(s_tmem + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::STAGES; ++i) {
            mbar_init(&full[i], 2);  // the A and B producers
            mbar_init(&empty[i], 1);
            mbar_init(&sf_full[i], 8);
            mbar_init(&sf_land[i], 1);
            mbar_init(&sf_free[i], 4);
        }
        for (int i = 0; i < C::ACC_STAGES; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 16);  // 8 epilogue warps in each CTA
        }
        *dead = 0;
        fence_mbar_init();
        prefetch_tmap(&tm_a);
        prefetch_tmap(&tm_b);
        prefetch_tmap(&tm_d);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc2(s_tmem, C::TMEM_COLS);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrive / commit
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    pdl_launch_dependents();
    pdl_wait();  // barriers, tensor memory and the cluster are set up; global memory is touched only from here on

    const int m_pairs = p.m_tiles >> 1;
    const int n_tiles_total = m_pairs * p.n_tiles;
    const int n_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;
    const int k_stages = (p.k_chunks + 1) >> 1;
    const int64_t sf_blocks_per_rowblock = p.k_chunks;

    if (warp == 0 || warp == 10 || warp == 15) {
        // ------------------------------ TMA producers (both CTAs) ------------------------------
        // Three threads in three warps, each counting on the stage's one `full` barrier: warp 0 copies this
        // CTA's rows of A, warp 10 its half of B, warp 15 the scales (one bulk copy for A's, one tensor copy
        // for all row blocks of B's).  A thread can start a copy only every few hundred cycles, and a
        // stage's MMAs take 520: with one or two issuing threads the copies of a stage started too late.
        if (lane == 0) {
            const int role = warp == 0 ? 0 : (warp == 10 ? 1 : 2);
            const uint64_t keep = l2_policy_evict_last();  // operands and scales are re-read by other CTAs
            uint32_t s = 0, ph = 0;
            for (int tile = cluster_id; tile < n_tiles_total && !*dead; tile += n_clusters) {
                int m_pair, n_blk;
                tile_coords(tile, m_pairs, p.n_tiles, m_pair, n_blk);
                const int m_blk = m_pair * 2 + (int)rank;
                const int m0 = m_blk * BM, n0 = n_blk * BN;
                const uint8_t* sfa_src = p.a_sf + (int64_t)m_blk * sf_blocks_per_rowblock * 512;
                for (int ks = 0; ks < k_stages; ++ks) {
                    // operand buffers are free once the stage's MMAs are done; the scale buffers as soon as the
                    // feeders have them in registers, so the scale copies run several stages ahead
                    if (!gemm_wait(role == 2 ? &sf_free[s] : &empty[s], ph ^ 1, WAIT_GEMM_EMPTY, dead)) break;
                    if (role == 0) {
                        mbar_arrive_expect_tx(&full[s], C::A_BYTES);
                        tma_load_2d_hint(s_a + s * C::A_BYTES, &tm_a, ks * BK_BYTES, m0, &full[s], keep);
                    } else if (role == 1) {
                        mbar_arrive_expect_tx(&full[s], C::B_BYTES);
                        tma_load_2d_hint(s_b + s * C::B_BYTES, &tm_b, ks * BK_BYTES, n0 + (int)rank * (BN / 2), &full[s], keep);
                    } else {
                        // the tensor copy always delivers its full box (out-of-range parts are zero-filled)
                        const int nch = min(2, p.k_chunks - 2 * ks);
                        mbar_arrive_expect_tx(&sf_land[s], nch * 512 + C::SFB_BYTES);
                        bulk_load_hint(s_sfa + s * C::SFA_BYTES, sfa_src + (int64_t)ks * 1024, nch * 512, &sf_land[s], keep);
                        tma_load_2d_hint(s_sfb + s * C::SFB_BYTES, &tm_sfb, ks * 256, n0 / 128, &sf_land[s], keep);
                    }
                    if (++s == C::STAGES) s = 0, ph ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        if (leader) {
            // ring positions are kept as (index, phase) pairs: no division in the issue loop
            uint32_t s = 0, ph = 0, slot = 0, as = 0, aph = 0, acc_it = 0;
            const uint32_t idesc0 = make_idesc2(BN, 0), idesc1 = make_idesc2(BN, 2);
            const uint32_t a_base = smem_u32(s_a), b_base = smem_u32(s_b);
            const uint32_t empty_own = smem_u32(&empty[0]), accf_own = smem_u32(&acc_full[0]);
            for (int tile = cluster_id; tile < n_tiles_total && !*dead; tile += n_clusters) {
                if (!gemm_wait(&acc_empty[as], aph ^ 1, WAIT_GEMM_ACC_EMPTY, dead)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (C::OVERLAP ? (acc_it & 1) * C::ACC_SHIFT : as * BN);
                ++acc_it;
                // Two stages per trip when the second is ready as well: the fixed cost of a trip (barrier
                // polls, fence, warp re-convergence) is then paid once per eight MMAs.
                for (int ks = 0; ks < k_stages;) {
                    int n2 = (ks + 1 < k_stages) ? 2 : 1;
                    const uint32_t s1 = (s + 1 == C::STAGES) ? 0 : s + 1, ph1 = (s + 1 == C::STAGES) ? ph ^ 1 : ph;
                    const uint32_t slot1 = (slot + 1 == C::SF_SLOTS) ? 0 : slot + 1;
                    // the feeders arrive only after the stage's copies have landed in BOTH CTAs, so this
                    // one barrier per stage covers operands and scales
                    if (!gemm_wait(&sf_full[s], ph, WAIT_GEMM_SF, dead)) break;
                    if (n2 == 2 && !mbar_try_wait(&sf_full[s1], ph1)) n2 = 1;  // pair up only if the next stage is ready too
                    tc_fence_after();
                    if (elect_one()) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (h < n2) {
                                const uint32_t sh = h ? s1 : s, sloth = h ? slot1 : slot;
                                const int nch = min(2, p.k_chunks - 2 * (ks + h));
                                const uint32_t sf_tmem = tmem_base + C::SF_COL0 + sloth * C::SF_COLS;
                                const uint64_t adesc = make_desc_sw128(a_base + sh * C::A_BYTES);
                                const uint64_t bdesc = make_desc_sw128(b_base + sh * C::B_BYTES);
                                tc_mma2_mxf4(d_tmem, adesc, bdesc, idesc0, sf_tmem, sf_tmem + 8, (ks + h) != 0);
                                tc_mma2_mxf4(d_tmem, adesc + 2, bdesc + 2, idesc1, sf_tmem | (2u << 30), (sf_tmem + 8) | (2u << 30), 1);
                                if (nch == 2) {
                                    tc_mma2_mxf4(d_tmem, adesc + 4, bdesc + 4, idesc0, sf_tmem + 4, sf_tmem + 8 + C::SFB_ST, 1);
                                    tc_mma2_mxf4(d_tmem, adesc + 6, bdesc + 6, idesc1, (sf_tmem + 4) | (2u << 30),
                                                 (sf_tmem + 8 + C::SFB_ST) | (2u << 30), 1);
                                }
                                // one completion event, signalled to both CTAs: frees the operand stage and the scale slot
                                tc_commit2_pair(empty_own + sh * 8);
                            }
                        }
                    }
                    __syncwarp();
                    for (int h = 0; h < n2; ++h) {
                        if (++s == C::STAGES) s = 0, ph ^= 1;
                        if (++slot == C::SF_SLOTS) slot = 0;
                    }
                    ks += n2;
                }
                if (elect_one()) tc_commit2_pair(accf_own + as * 8);
                __syncwarp();
                if (++as == C::ACC_STAGES) as = 0, aph ^= 1;
            }
        }
    } else if (warp >= 6 && warp <= 9) {
        // ------------------------------ scale feeders (both CTAs) ------------------------------
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        uint32_t it = 0;
        for (int tile = cluster_id; tile < n_tiles_total && !*dead; tile += n_clusters) {
            int m_pair, n_blk;
            tile_coords(tile, m_pairs, p.n_tiles, m_pair, n_blk);
            const int n0 = n_blk * BN;
            const int seg0 = (n0 % 128) / 32;
            for (int ks = 0; ks < k_stages; ++ks, ++it) {
                const int s = it % C::STAGES;
                const uint32_t ph = (it / C::STAGES) & 1;
                if (!gemm_wait(&sf_land[s], ph, WAIT_GEMM_FULL, dead)) break;
                const int nch = min(2, p.k_chunks - 2 * ks);
                const uint32_t sf_tmem = tmem_base + lane_base + C::SF_COL0 + (it % C::SF_SLOTS) * C::SF_COLS;
                const uint8_t* sfa = s_sfa + s * C::SFA_BYTES + lane * 16;
                const uint8_t* sfb = s_sfb + s * C::SFB_BYTES + lane * 16;
                // shared -> registers first, so that only the tensor-memory stores remain once the slot is free
                uint32_t ra[2][8], rb[2][8];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const uint4 va = c < nch ? *reinterpret_cast<const uint4*>(sfa + c * 512) : make_uint4(0, 0, 0, 0);
                    ra[c][0] = va.x, ra[c][1] = va.y, ra[c][2] = va.z, ra[c][3] = va.w;
#pragma unroll
                    for (int j = 0; j < C::SFB_ST; ++j) {
                        const int seg = seg0 + j;
                        rb[c][j] = (j < C::NSEG && c < nch)
                                       ? *reinterpret_cast<const uint32_t*>(sfb + (seg >> 2) * 1024 + c * 512 + (seg & 3) * 4)
                                       : 0u;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sf_free[s]);  // the scale copies of a later stage may reuse the buffers
                // the scale slot was last read by the MMAs of iteration it - SF_SLOTS; their completion is
                // what the `empty` barrier of that iteration's operand stage reports
                if (it >= (uint32_t)C::SF_SLOTS) {
                    const uint32_t pit = it - C::SF_SLOTS;
                    if (!gemm_wait(&empty[pit % C::STAGES], (pit / C::STAGES) & 1, WAIT_GEMM_EMPTY, dead)) break;
                    tc_fence_after();
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    if (c < nch) {
                        tc_st4(sf_tmem + c * 4, ra[c]);
                        if (C::SFB_ST == 4)
                            tc_st4(sf_tmem + 8 + c * C::SFB_ST, rb[c]);
                        else
                            tc_st8(sf_tmem + 8 + c * C::SFB_ST, rb[c]);
                    }
                }
                tc_wait_st();
                tc_fence_before();
                // the scales usually sit in tensor memory before the operands arrive; the arrive below tells
                // the MMA issuer that BOTH are there for this CTA
                if (!gemm_wait(&full[s], ph, WAIT_GEMM_FULL, dead)) break;
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&sf_full[s]), 0));
            }
        }
    } else if ((warp >= 2 && warp <= 5) || warp >= 11) {
        // ------------------------------ epilogue (both CTAs) ------------------------------
        // Two warps per TMEM lane quadrant: warps 2-5 drain the even 32-column blocks of the tile,
        // warps 11-14 the odd ones; the next block's tcgen05.ld is in flight while one is processed.
        const int q = warp & 3;
        const int par = warp >= 11 ? 1 : 0;
        uint8_t* stg = s_stg + (par * 4 + q) * (NSTG * 2048);
        uint32_t acc_it = 0, n_stores = 0;
        for (int tile = cluster_id; tile < n_tiles_total && !*dead; tile += n_clusters, ++acc_it) {
            int m_pair, n_blk;
            tile_coords(tile, m_pairs, p.n_tiles, m_pair, n_blk);
            const int m_blk = m_pair * 2 + (int)rank;
            const int n0 = n_blk * BN;
            const int as = acc_it % C::ACC_STAGES;
            if (!gemm_wait(&acc_full[as], (acc_it / C::ACC_STAGES) & 1, WAIT_GEMM_ACC_FULL, dead)) break;
            tc_fence_after();
            const int64_t row = (int64_t)(m_blk * BM + q * 32) + lane;
            // where this warp's 32 rows are stored: the one output, or their owner's slice of it
            int row0 = m_blk * BM + q * 32;
            const CUtensorMap* tmd = &tm_d;
            if (p.rows_per_owner > 0) {
                const int owner = row0 / p.rows_per_owner;
                tmd = &sc.m[owner];
                row0 -= owner * p.rows_per_owner;
            }
            const int n_chunks = min(BN, p.N - n0) / 32;
            uint32_t ra[32], rb[32];
            if constexpr (C::OVERLAP) {
                // this warp's four blocks, those in the shared columns first
                const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (acc_it & 1) * C::ACC_SHIFT;
                const int shared0 = (acc_it & 1) ? 0 : C::ACC_SHIFT / 32;
                const int c0 = shared0 + par, c1 = c0 + 2, c2 = (shared0 ^ (C::ACC_SHIFT / 32)) + par, c3 = c2 + 2;
                if (c0 < n_chunks) tc_ld32(t0 + c0 * 32, ra);
                if (c1 < n_chunks) tc_ld32(t0 + c1 * 32, rb);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[0]), 0));
                if (c0 < n_chunks) epilogue_block<NSTG>(ra, p, tmd, row, row0, n0 + c0 * 32, stg, n_stores, lane);
                if (c2 < n_chunks) tc_ld32(t0 + c2 * 32, ra);
                if (c1 < n_chunks) epilogue_block<NSTG>(rb, p, tmd, row, row0, n0 + c1 * 32, stg, n_stores, lane);
                if (c3 < n_chunks) tc_ld32(t0 + c3 * 32, rb);
                tc_wait_ld();
                if (c2 < n_chunks) epilogue_block<NSTG>(ra, p, tmd, row, row0, n0 + c2 * 32, stg, n_stores, lane);
                if (c3 < n_chunks) epilogue_block<NSTG>(rb, p, tmd, row, row0, n0 + c3 * 32, stg, n_stores, lane);
                // all of this tile's tensor-memory reads are complete before the warp's next arrive
                tc_fence_before();
            } else {
                const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN;
                if (par < n_chunks) tc_ld32(t0 + par * 32, ra);
                for (int ch = par; ch < n_chunks; ch += 4) {
                    tc_wait_ld();
                    if (ch + 2 < n_chunks) tc_ld32(t0 + (ch + 2) * 32, rb);
                    epilogue_block<NSTG>(ra, p, tmd, row, row0, n0 + ch * 32, stg, n_stores, lane);
                    if (ch + 2 < n_chunks) {
                        tc_wait_ld();
                        if (ch + 4 < n_chunks) tc_ld32(t0 + (ch + 4) * 32, ra);
                        epilogue_block<NSTG>(rb, p, tmd, row, row0, n0 + (ch + 2) * 32, stg, n_stores, lane);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[as]), 0));
            }
        }
        if (lane == 0) bulk_wait0();
    }

    // ------------------------------ wind-down ------------------------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*dead) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    cluster_sync_all();  // neither CTA leaves while its peer may still touch its barriers or memory
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, C::TMEM_COLS);
    }
}

template <int BN, int NSTG = 1>
static int launch_gemm_2cta(const uint8_t* a, const uint8_t* b, void* d, const GemmParams& p0, cudaStream_t stream,
                            void* const* owners = nullptr, int n_owners = 0) {
    using C = Gemm2Cfg<BN, NSTG>;
    GemmParams p = p0;
    p.n_tiles = (p.N + BN - 1) / BN;
    CUtensorMap tm_a, tm_b, tm_d;
    int rc = make_tmap_2d(&tm_a, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.K / 2, p.M, p.K / 2, BK_BYTES, BM, 3);
    if (rc) return rc;
    rc = make_tmap_2d(&tm_b, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.K / 2, p.N, p.K / 2, BK_BYTES, BN / 2, 3);
    if (rc) return rc;
    static ScatterMaps sc;  // stays zero unless the output is scattered (then rebuilt below, per call)
    ScatterMaps sc_call;
    const ScatterMaps* scp = &sc;
    if (n_owners > 0) {
        for (int o = 0; o < n_owners; ++o)
            if ((rc = make_tmap_2d(&sc_call.m[o], owners[o], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.N, p.rows_per_owner,
                                   (uint64_t)p.N * 4, 32, 16, 3)))
                return rc;
        for (int o = n_owners; o < MAX_OWNERS; ++o) sc_call.m[o] = sc_call.m[0];
        tm_d = sc_call.m[0];
        scp = &sc_call;
    } else if (p.d_f32)
        rc = make_tmap_2d(&tm_d, d, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.N, p.M, (uint64_t)p.N * 4, 32, 16, 3);
    else
        rc = make_tmap_2d(&tm_d, d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.M, (uint64_t)p.N * 2, 32, 32, 2);
    if (rc) return rc;
    // B's scales as a 2-D tensor of 32-bit words: one row per 128-row block, k_chunks * 128 words each;
    // a stage takes two chunks (256 words) of every row block of the tile in one copy
    CUtensorMap tm_sfb;
    static_assert(BN % 128 == 0, "the scale copy of the two-CTA kernel assumes tiles that start on a 128-row scale block");
    if ((rc = make_tmap_2d(&tm_sfb, p.b_sf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (uint64_t)p.k_chunks * 128, (uint64_t)((p.N + 127) / 128),
                           (uint64_t)p.k_chunks * 512, 256, BN / 128, 0)))
        return rc;
    auto kern = gemm_mxfp4_2cta_kernel<BN, NSTG>;
    static thread_local int smem_set = -1;
    rc = set_max_smem_once(kern, C::SMEM, smem_set);
    if (rc) return rc;
    int dev = 0, sms = 0;
    if ((rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice"))) return rc;
    if ((rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute"))) return rc;
    // A persistent kernel must not launch more clusters than can be resident at once: on parts
    // where some TPCs have a single SM enabled that is fewer than SMs / 2.
    static thread_local int cached_dev = -1, cached_clusters = 0;
    if (cached_dev != dev) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)sms, 1, 1);
        cfg.blockDim = dim3(GEMM2_THREADS, 1, 1);
        cfg.dynamicSmemBytes = C::SMEM;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
        cfg.attrs = &attr, cfg.numAttrs = 1;
        int n = 0;
        if ((rc = check_cuda(cudaOccupancyMaxActiveClusters(&n, kern, &cfg), "cudaOccupancyMaxActiveClusters"))) return rc;
        if (n < 1) return fail(QUARTET_E_CUDA, "no CTA pair can be resident");
        cached_dev = dev, cached_clusters = n;
    }
    const int pair_tiles = (p.m_tiles / 2) * p.n_tiles;
    const int clusters = pair_tiles < cached_clusters ? pair_tiles : cached_clusters;
    rc = check_cuda(launch_pdl(kern, dim3(clusters * 2), dim3(GEMM2_THREADS), C::SMEM, stream, tm_a, tm_b, tm_d, tm_sfb, *scp, p), "gemm (2-CTA) launch");
    if (rc) return rc;
    return check_cuda(cudaGetLastError(), "gemm (2-CTA) launch");
}

template <int BN>
static int launch_gemm(const uint8_t* a, const uint8_t* b, void* d, const GemmParams& p0, cudaStream_t stream) {
    using C = GemmCfg<BN>;
    GemmParams p = p0;
    p.n_tiles = (p.N + BN - 1) / BN;
    CUtensorMap tm_a, tm_b, tm_d;
    int rc = make_tmap_2d(&tm_a, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.K / 2, p.M, p.K / 2, BK_BYTES, BM, 3);
    if (rc) return rc;
    rc = make_tmap_2d(&tm_b, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.K / 2, p.N, p.K / 2, BK_BYTES, p.N < BN ? p.N : BN, 3);
    if (rc) return rc;
    if (p.d_f32)
        rc = make_tmap_2d(&tm_d, d, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.N, p.M, (uint64_t)p.N * 4, 32, 16, 3);
    else
        rc = make_tmap_2d(&tm_d, d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.M, (uint64_t)p.N * 2, 32, 32, 2);
    if (rc) return rc;
    auto kern = gemm_mxfp4_kernel<BN>;
    static thread_local int smem_set = -1;
    rc = set_max_smem_once(kern, C::SMEM, smem_set);
    if (rc) return rc;
    int dev = 0, sms = 0;
    if ((rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice"))) return rc;
    if ((rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute"))) return rc;
    const int tiles = p.m_tiles * p.n_tiles;
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, GEMM_THREADS, C::SMEM, stream>>>(tm_a, tm_b, tm_d, p);
    return check_cuda(cudaGetLastError(), "gemm launch");
}

QUARTET_DEFINE_STATUS_READER(status_gemm)

}  // namespace quartet

using namespace quartet;

extern "C" __attribute__((visibility("default"))) int quartet_gemm_mxfp4_tn(const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                                     int64_t M, int64_t N, int64_t K, float alpha, const uint8_t* mask,
                                     float had_scale, void* d, int d_dtype, quartet_stream_t stream) {
    if (!a || !a_sf || !b || !b_sf || !d) return fail(QUARTET_E_NULL, "a, a_sf, b, b_sf and d must be non-NULL");
    if (M < 128 || N < 128 || K < 128 || M % 128 || N % 128 || K % 128)
        return fail(QUARTET_E_SHAPE, "M, N, K must be multiples of 128 (got %lld, %lld, %lld)", (long long)M, (long long)N,
                    (long long)K);
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return fail(QUARTET_E_SHAPE, "extent too large");
    if (!aligned16(a) || !aligned16(b) || !aligned16(a_sf) || !aligned16(b_sf) || !aligned16(d) ||
        (mask && (reinterpret_cast<uintptr_t>(mask) & 3)))
        return fail(QUARTET_E_ALIGN, "operands must be 16-byte aligned (mask: 4-byte)");
    if (d_dtype != QUARTET_BF16 && d_dtype != QUARTET_F32) return fail(QUARTET_E_ARG, "d_dtype must be 0 or 1");
    int rc = bind_context_of(a);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    GemmParams p{};
    p.a_sf = a_sf, p.b_sf = b_sf;
    p.M = (int)M, p.N = (int)N, p.K = (int)K;
    p.k_chunks = (int)(K / 128);
    p.m_tiles = (int)(M / BM);
    p.alpha = alpha, p.mask = mask, p.had_scale = had_scale;
    p.d_f32 = d_dtype == QUARTET_F32;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Tile width: 256 unless the output is narrow and not a multiple of 256; CTA pairs need an even number
    // of 128-row tiles.
    const bool wide = N % 256 == 0 || N > 1024;
    if (wide && M % 256 == 0) {
        return launch_gemm_2cta<256>(a, b, d, p, s);
    }
    if (wide) return launch_gemm<256>(a, b, d, p, s);
    return launch_gemm<128>(a, b, d, p, s);
}

// Same contraction with the fp32 result scattered by row range: rows [o * rows_per_owner, (o + 1) *
// rows_per_owner) go to owners[o], a dense [rows_per_owner, N] fp32 matrix (typically the slot this
// rank owns in GPU o's receive buffer).
extern "C" __attribute__((visibility("default"))) int quartet_gemm_mxfp4_tn_scatter(
    const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf, int64_t M, int64_t N, int64_t K, float alpha,
    const uint8_t* mask, float had_scale, void* const* owners, int32_t n_owners, int64_t rows_per_owner, quartet_stream_t stream) {
    if (!a || !a_sf || !b || !b_sf || !owners) return fail(QUARTET_E_NULL, "a, a_sf, b, b_sf and owners must be non-NULL");
    if (n_owners < 1 || n_owners > MAX_OWNERS) return fail(QUARTET_E_ARG, "n_owners must be 1..%d (got %d)", MAX_OWNERS, n_owners);
    if (M < 256 || N < 256 || K < 128 || M % 256 || N % 256 || K % 128)
        return fail(QUARTET_E_SHAPE, "scatter needs M, N multiples of 256 and K a multiple of 128 (got %lld, %lld, %lld)",
                    (long long)M, (long long)N, (long long)K);
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return fail(QUARTET_E_SHAPE, "extent too large");
    if (rows_per_owner < 32 || rows_per_owner % 32 || rows_per_owner * n_owners != M)
        return fail(QUARTET_E_SHAPE, "rows_per_owner must be a multiple of 32 with rows_per_owner * n_owners == M");
    if (!aligned16(a) || !aligned16(b) || !aligned16(a_sf) || !aligned16(b_sf) || (mask && (reinterpret_cast<uintptr_t>(mask) & 3)))
        return fail(QUARTET_E_ALIGN, "operands must be 16-byte aligned (mask: 4-byte)");
    for (int o = 0; o < n_owners; ++o)
        if (!owners[o] || !aligned16(owners[o])) return fail(QUARTET_E_ALIGN, "owners[%d] must be a 16-byte aligned device pointer", o);
    int rc = bind_context_of(a);
    if (rc) return rc;
    if ((rc = check_device())) return rc;
    GemmParams p{};
    p.a_sf = a_sf, p.b_sf = b_sf;
    p.M = (int)M, p.N = (int)N, p.K = (int)K;
    p.k_chunks = (int)(K / 128);
    p.m_tiles = (int)(M / BM);
    p.alpha = alpha, p.mask = mask, p.had_scale = had_scale;
    p.d_f32 = 1;
    p.rows_per_owner = (int)rows_per_owner;
    // two staging buffers per epilogue warp (and five operand stages instead of six): a store to a peer
    // holds its staging buffer longer than a local one
    return launch_gemm_2cta<256, 2>(a, b, nullptr, p, static_cast<cudaStream_t>(stream), owners, n_owners);
}
