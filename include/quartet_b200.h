/*
 * quartet_b200 -- C ABI of the B200 (sm_100a) MXFP4 quantized-linear path.
 *
 * Every entry point takes raw DEVICE pointers, extents and a CUDA stream
 * (a cudaStream_t passed as void*; NULL = the legacy default stream).  The
 * caller owns every buffer; no call allocates device memory.  Calls return 0
 * on success and a negative QUARTET_E_* code on rejection (nothing was
 * launched); quartet_last_error_string() describes the last rejection on the
 * calling thread.  Nothing throws, aborts or traps.
 *
 * Data formats (pinned by the reference's real-quantized op contracts,
 * notebooks/benchmark_mxfp4.ipynb:881-979):
 *   codes  uint8 [rows, cols/2]   two e2m1 codes per byte, even element in the
 *                                 low nibble; code = sign<<3 | index into
 *                                 {0, .5, 1, 1.5, 2, 3, 4, 6}
 *   sf     uint8, E8M0 (value 2^(b-127)), one per 32 elements of a row, stored
 *          in 512-byte blocks of 128 rows x 4 scales; logical shape
 *          [pad128(rows), pad4(cols/32)]; byte offset = quartet_sf_offset().
 *          The row-wise quantizers write 0 for the padding rows of the last
 *          128-row block.
 *   mask   uint8 [rows, cols/8]   1 bit per element, LSB first; 1 = |v| < 6
 *
 * Reference paths are given relative to the reference project root.
 */
#ifndef QUARTET_B200_H
#define QUARTET_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* quartet_stream_t;

enum {
    QUARTET_OK = 0,
    QUARTET_E_NULL = -1,      /* a required pointer is NULL */
    QUARTET_E_SHAPE = -2,     /* extent not supported (see each call) */
    QUARTET_E_ALIGN = -3,     /* pointer not 16-byte aligned */
    QUARTET_E_ARG = -4,       /* bad enum / flag value */
    QUARTET_E_CUDA = -5,      /* a CUDA runtime/driver call failed */
    QUARTET_E_DEVICE = -6     /* not an sm_100 device */
};

enum { QUARTET_BF16 = 0, QUARTET_F32 = 1 };

/* rounding modes of the backward (absmax-scaled) quantizers */
enum {
    QUARTET_ROUND_NEAREST = 0,    /* AlbertTsengQuantizer(stochastic=False) */
    QUARTET_ROUND_SR_PHILOX = 1,  /* stochastic, library's own Philox4x32-7 dither stream (seed, offset) */
    QUARTET_ROUND_SR_NOISE = 2,   /* stochastic, caller-supplied fp32 uniform noise tensor, reference `u < p` rule */
    QUARTET_ROUND_SR_TLRAND = 3   /* stochastic, reference-compatible stream: tl.rand(seed, flat_offset) */
};

/*
 * Forward quantizer: 32-point Hadamard rotation along `cols`, std-based scale,
 * round to nearest, clip mask.
 * Replaces mxfp4_forward_kernel with quest=True, stochastic_round=False
 * (src/models/quantization/quantizers/mxfp4_triton.py:33-57,130-174) as called by
 * QuestMXFP4QuantizerFn.forward (src/models/quantization/quantizers/mxfp4.py:129-140);
 * output contract = fusedQuantizeMx (notebooks/benchmark_mxfp4.ipynb:897-921).
 * x: [rows, cols] row-major, dtype QUARTET_BF16 / QUARTET_F32; cols % 128 == 0, rows >= 1.
 * had_scale: magnitude of the rotation matrix entries (bf16(32^-1/2) = 0.1767578125 when the
 * reference has cast H to bf16, 32^-1/2 in fp32 otherwise).  mask may be NULL.
 */
int quartet_quant_fwd(const void* x, int x_dtype, int64_t rows, int64_t cols, float had_scale, float gaussian_scale,
                      uint8_t* codes, uint8_t* sf, uint8_t* mask, quartet_stream_t stream);

/*
 * Forward quantizer fused into the elementwise step that produces its input: the activation of a
 * quantized linear layer is quantized straight from the tensor the step reads, and is never
 * written in bf16 / fp32.  Same outputs and output contract as quartet_quant_fwd.
 *
 * quartet_quant_fwd_rmsnorm: the input is RMSNorm(x) as src/models/llama.py:64-75 computes it,
 *   (x * rsqrt(mean(x^2) + eps)).type_as(x) * weight      (weight: fp32 [cols]; result fp32),
 * feeding c_attn (llama.py:124) and mlp.w12 (llama.py:113).  x: [rows, cols] bf16 / fp32,
 * cols % 128 == 0.  rstd ([rows] fp32, required) receives rsqrt(mean(x^2) + eps) per row: the
 * norm's backward needs it.  Two launches: the statistics, then the quantization (each reads the rows).
 * quartet_rms_stats: the statistics alone (cols % 8 == 0).
 *
 * quartet_quant_fwd_swiglu: the input is silu(h[:, :hidden]) * h[:, hidden:] (llama.py:112-114,
 * feeding mlp.c_proj); h: [rows, 2 * hidden] bf16 / fp32 row-major, hidden % 128 == 0.  For bf16
 * the value of silu and the product are each rounded to bf16, as the two torch kernels round them;
 * silu is x / (1 + exp(-x)) in fp32.
 */
int quartet_rms_stats(const void* x, int x_dtype, int64_t rows, int64_t cols, float eps, float* rstd, quartet_stream_t stream);
int quartet_quant_fwd_rmsnorm(const void* x, int x_dtype, int64_t rows, int64_t cols, const float* weight, float eps, float* rstd,
                              float had_scale, float gaussian_scale, uint8_t* codes, uint8_t* sf, uint8_t* mask,
                              quartet_stream_t stream);
int quartet_quant_fwd_swiglu(const void* h, int h_dtype, int64_t rows, int64_t hidden, float had_scale, float gaussian_scale,
                             uint8_t* codes, uint8_t* sf, uint8_t* mask, quartet_stream_t stream);
/* The same product written out as [rows, hidden] in h's dtype (hidden % 8 == 0): the values the fused quantizer
 * quantizes, for callers that need the activation itself, and the handle by which the tests pin its arithmetic to
 * torch's (all 65536 bf16 inputs of silu). */
int quartet_swiglu(const void* h, int h_dtype, int64_t rows, int64_t hidden, void* out, quartet_stream_t stream);

/*
 * Backward quantizer, row-wise: rotation (H @ diag(signs)), absmax scale
 * E8M0 = floor(log2 amax) - 2, rounding per `rounding`.  The 4/3 of the reference's
 * shared exponent (2^e / 0.75) is NOT in the scale bytes; fold it into the GEMM alpha.
 * Replaces mxfp4_forward_kernel with quest=False (mxfp4_triton.py:58-61,70-129) as called by
 * AlbertTsengQuantizerFn.forward (mxfp4.py:17-28) on `e` (src/models/quantization/backward.py:72).
 * signs: bit j set = coefficient j of every group negated; if signs_dev != NULL the kernel
 * reads the word from device memory instead (no host sync after re_randomize, mxfp4.py:52-60).
 * noise: fp32 [rows, cols], only for QUARTET_ROUND_SR_NOISE.
 */
int quartet_quant_bwd(const void* x, int x_dtype, int64_t rows, int64_t cols, float had_scale, uint32_t signs,
                      const uint32_t* signs_dev, int rounding, uint64_t seed, uint64_t offset, const float* noise,
                      uint8_t* codes, uint8_t* sf, quartet_stream_t stream);

/*
 * The quantizers' scaling, rounding and packing WITHOUT the built-in rotation: x [rows, cols] is taken as
 * already rotated (or as not to be rotated) and quantized in groups of 32 along `cols`.
 * kind 0: std-based scale, round to nearest (ties toward zero), clip mask -- the quest=True branch of
 *         mxfp4_forward_kernel after its `tl.dot` (mxfp4_triton.py:48-57,130-174), and the rotation-free
 *         mxfp4_quant_kernel of the post-training tools (src/quarot_utils/mxfp4_quant_utils.py:24-113);
 * kind 1: absmax scale with the rounding modes of quartet_quant_bwd (mxfp4_triton.py:58-61,70-129).
 * Serves rotations this library has no kernel for -- a dense random orthogonal matrix (rerotate="O32",
 * mxfp4.py:61-64) or hadamard_dim 64 / 128 (sweep_tokens_backward.sh:52-53): the caller multiplies by the
 * matrix, this call does the rest.  Noise and the tl.rand offsets index x row-major.
 */
int quartet_quant_group32(const void* x, int x_dtype, int64_t rows, int64_t cols, int kind, float gaussian_scale,
                          int rounding, uint64_t seed, uint64_t offset, const float* noise, uint8_t* codes, uint8_t* sf,
                          uint8_t* mask, quartet_stream_t stream);

/*
 * Backward quantizer of the TRANSPOSE: groups of 32 run along `rows` of x; writes
 * codes_t [cols, rows/2] and sf_t (logical [cols, rows/32]).
 * Replaces `g_quantizer(e.reshape(M,-1).T.contiguous())` (backward.py:81); contract =
 * backward_t_bf16 (benchmark_mxfp4.ipynb:924-937).  rows % 128 == 0, cols % 128 == 0.
 * noise (QUARTET_ROUND_SR_NOISE) and the QUARTET_ROUND_SR_TLRAND offsets index the
 * transposed tensor [cols, rows] row-major, as the reference kernel would see it.
 */
int quartet_quant_bwd_t(const void* x, int x_dtype, int64_t rows, int64_t cols, float had_scale, uint32_t signs,
                        const uint32_t* signs_dev, int rounding, uint64_t seed, uint64_t offset, const float* noise,
                        uint8_t* codes_t, uint8_t* sf_t, quartet_stream_t stream);

/*
 * Q(E) and Q(E^T) from one read of E (both are needed by every backward pass, backward.py:72 and :81
 * of the reference): codes/sf are exactly what quartet_quant_bwd(x, ..., seed_rows) writes and
 * codes_t/sf_t exactly what quartet_quant_bwd_t(x, ..., seed_t) writes.  rows and cols multiples of 128;
 * rounding 0 (nearest) or 1 (own Philox stream).
 */
int quartet_quant_bwd_dual(const void* x, int x_dtype, int64_t rows, int64_t cols, float had_scale, uint32_t signs,
                           const uint32_t* signs_dev, int rounding, uint64_t seed_rows, uint64_t seed_t, uint64_t offset,
                           uint8_t* codes, uint8_t* sf, uint8_t* codes_t, uint8_t* sf_t, quartet_stream_t stream);

/*
 * De-quantize + transpose + backward-quantize of an MXFP4 tensor.
 * Replaces `g_quantizer(w.T.contiguous())` / `g_quantizer(x.reshape(M,-1).T.contiguous())`
 * (backward.py:73,82) on the saved forward-quantized operands; contract = backward_qt_bf16
 * (benchmark_mxfp4.ipynb:940-957).  Input value = grid[code] * 2^(sf-127) * in_scale.
 * rows % 128 == 0, cols % 128 == 0.
 */
int quartet_requant_t(const uint8_t* codes, const uint8_t* sf, int64_t rows, int64_t cols, float in_scale,
                      float had_scale, uint32_t signs, const uint32_t* signs_dev, int rounding, uint64_t seed,
                      uint64_t offset, const float* noise, uint8_t* codes_t, uint8_t* sf_t, quartet_stream_t stream);

/*
 * Block-scaled MXFP4 GEMM, D[M,N] = alpha * A[M,K] . B[N,K]^T, both operands K-major.
 * Replaces F.linear(xq, wq) (backward.py:62), F.linear(Q(e), Q(w^T)) (backward.py:71-75) and
 * einsum("ib,jb->ij", Q(e^T), Q(x^T)) (backward.py:79-83); contract = matmul_mxf4_bf16_tn
 * (benchmark_mxfp4.ipynb:882-895).  M, N, K % 128 == 0.
 * If mask != NULL ([M, N/8] bits), the epilogue also applies the forward quantizer's
 * straight-through backward, ((alpha*acc) * mask).view(-1,32) @ H^T (mxfp4.py:142-146),
 * with H = had_scale * Sylvester-32.  d_dtype: QUARTET_BF16 or QUARTET_F32.
 */
int quartet_gemm_mxfp4_tn(const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf, int64_t M,
                          int64_t N, int64_t K, float alpha, const uint8_t* mask, float had_scale, void* d,
                          int d_dtype, quartet_stream_t stream);

/*
 * The whole layer in one host call per direction: exactly the kernel sequences the entry points above launch one
 * by one, for callers whose per-call cost matters (a Python caller pays tens of microseconds per entry point).
 *
 * quartet_linear_fwd = QuantizedLinear.forward with the forward quantizer on both operands
 * (src/models/quantization/__init__.py:36-42): (xc, xs, xm) = quant_fwd(x [M, K]), (wc, ws, wm) = quant_fwd(w [N, K]),
 * y [M, N] = gemm(xc, wc).  The six packed outputs are what the backward needs.  M, N, K multiples of 128.
 *
 * quartet_linear_bwd = QEQWtt_QEtQXttFn.backward (backward.py:64-85) followed by the straight-through backward of both
 * forward quantizers (mxfp4.py:142-146): dx [M, K] and dw [N, K] from e [M, N] and the packed outputs of the forward.
 * dx or dw may be NULL (not computed).  seeds4 is a HOST array of four seeds, used in the reference's call order
 * E, Wq^T, E^T, Xq^T; rounding 0, 1 or 3.  alpha = (4/3 * out_scale)^2.  workspace: device memory, 256-byte aligned, of
 * quartet_linear_bwd_workspace_bytes(M, N, K) bytes (the packed operands of the two backward GEMMs).
 */
int quartet_linear_fwd(const void* x, int x_dtype, const void* w, int w_dtype, int64_t M, int64_t N, int64_t K,
                       float had_scale_x, float had_scale_w, float gaussian_scale, uint8_t* xc, uint8_t* xs, uint8_t* xm,
                       uint8_t* wc, uint8_t* ws, uint8_t* wm, void* y, int y_dtype, quartet_stream_t stream);
int64_t quartet_linear_bwd_workspace_bytes(int64_t M, int64_t N, int64_t K);
int quartet_linear_bwd(const void* e, int e_dtype, int64_t M, int64_t N, int64_t K, const uint8_t* xc, const uint8_t* xs,
                       const uint8_t* xm, const uint8_t* wc, const uint8_t* ws, const uint8_t* wm, float had_scale_b,
                       uint32_t signs, const uint32_t* signs_dev, int rounding, const uint64_t* seeds4, uint64_t offset,
                       float alpha, float had_scale_x, float had_scale_w, uint8_t* workspace, void* dx, int dx_dtype, void* dw,
                       int dw_dtype, quartet_stream_t stream);

/*
 * Stand-alone straight-through backward of the forward quantizer:
 * out = ((g * mask).view(-1,32) @ H^T).view(rows, cols)  (mxfp4.py:142-146); mask NULL = all ones
 * (AlbertTsengQuantizerFn.backward, mxfp4.py:30-34).  cols % 32 == 0.
 */
int quartet_unrotate_mask(const void* g, int g_dtype, const uint8_t* mask, int64_t rows, int64_t cols, float had_scale,
                          void* out, int out_dtype, quartet_stream_t stream);

/*
 * Sign re-randomisation of the backward rotation, H <- H @ diag(2 * draw - 1) (AlbertTsengQuantizer.re_randomize
 * with rerotate="signs", mxfp4.py:52-60), on the device-resident sign word the quantizers read through
 * `signs_dev`: draw is the device tensor of 32 zeros / ones the reference's torch.randint call produces (bf16 or
 * fp32), bit j of *word is flipped where draw[j] == 0.  One launch, no host synchronisation.
 */
int quartet_fold_signs(const void* draw, int draw_dtype, uint32_t* word, quartet_stream_t stream);

/*
 * codes + scales -> values (still in the rotated basis), out = grid[code] * 2^(sf-127) * scale.
 * Gives the tensor the reference kernel stores (mxfp4_triton.py:168-174); used by the
 * pseudo-quantizing wrapper mxfp4_forward_kernel_wrapper (mxfp4_triton.py:177-220).
 */
int quartet_dequant(const uint8_t* codes, const uint8_t* sf, int64_t rows, int64_t cols, float scale, void* out,
                    int out_dtype, quartet_stream_t stream);

/*
 * The same contraction with the fp32 result scattered by row range: rows [o * rows_per_owner,
 * (o + 1) * rows_per_owner) of D are stored to owners[o] as a dense [rows_per_owner, N] matrix.
 * owners is a HOST array of n_owners (<= 8) device pointers, which may be mappings of other GPUs'
 * memory (quartet_peer_open): the weight-gradient GEMM then delivers every rank's partial rows to the
 * rank that owns them while it computes, in place of the all-reduce torch DDP runs on full gradients
 * in the reference (src/main.py:79-85).  M, N multiples of 256; rows_per_owner a multiple of 32.
 */
int quartet_gemm_mxfp4_tn_scatter(const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf, int64_t M,
                                  int64_t N, int64_t K, float alpha, const uint8_t* mask, float had_scale,
                                  void* const* owners, int32_t n_owners, int64_t rows_per_owner, quartet_stream_t stream);

/* out[i] = scale * sum_s slots[s * slot_elems + i], slots added in index order. */
int quartet_shard_reduce(const float* slots, int32_t n_slots, int64_t slot_elems, float scale, float* out,
                         quartet_stream_t stream);

/*
 * Receive buffers other GPUs of the node can map: quartet_peer_alloc allocates `bytes` on the current
 * device and fills 64 opaque bytes that another PROCESS passes to quartet_peer_open to obtain a
 * pointer valid on its own device (CUDA IPC; peer access is enabled on first use).
 */
int quartet_peer_alloc(uint64_t bytes, void** ptr, void* handle64);
int quartet_peer_free(void* ptr);
int quartet_peer_open(const void* handle64, void** ptr);
int quartet_peer_close(void* ptr);
/* Asynchronous device-to-device copy (DMA engines, no SM): e.g. local partial rows -> a slot of a peer's buffer. */
int quartet_peer_copy(void* dst, const void* src, uint64_t bytes, quartet_stream_t stream);

/*
 * Measurement aid (no reference counterpart): bytes per clock one SM takes in through bulk asynchronous
 * copies from `src` (`region` bytes, keep it L2-resident), with `producers` (1..4) issuing threads per SM,
 * each running a ring of `stages` buffers of `chunk` bytes for `iters` copies.  `src` must be 128-byte
 * aligned, `chunk` a multiple of 128 and `region` at least 4 chunks; every copy stays inside the region.
 * `cycles` is a device array of one int64 per SM; the call synchronises the stream and writes the result
 * to the host.
 */
int quartet_probe_copy_ingress(const void* src, uint64_t region, int32_t iters, int32_t stages, int32_t chunk,
                               int32_t producers, int64_t* cycles, double* bytes_per_clk_per_sm, quartet_stream_t stream);

/*
 * quartet_probe_copy_ingress for callers that cannot allocate device memory (no counterpart in the
 * reference): code running while the framework's allocator is frozen, plugins that work inside buffers
 * their host application handed them, hooks that run when the device is almost full.  No workspace
 * argument and no allocation of any kind: the per-SM cycle counts live in a 256-entry device array
 * inside the library (2 KB held by every GPU that loads it, until exit).  A device with more than 256 SMs
 * is rejected with QUARTET_E_ARG.  The first call of a thread on a device looks up the array's address;
 * make it before any stream capture.  All calls on a device share the one array: calls that overlap on
 * the GPU (two streams, two host threads) race on it and must be serialised by the caller.
 */
int quartet_probe_copy_ingress_noalloc(const void* src, uint64_t region, int32_t iters, int32_t stages, int32_t chunk,
                                       int32_t producers, double* bytes_per_clk_per_sm, quartet_stream_t stream);

/*
 * Self-test of the bounded waits (no reference counterpart): one CTA waits, with a poll limit of 4096, on a barrier
 * that nothing completes; the wait gives up, records itself in the fault word and the kernel returns normally.
 * gave_up_dev (device int32, may be NULL) receives 1.  quartet_device_status() then reports a non-zero word.
 */
int quartet_selftest_wait_timeout(int32_t* gave_up_dev, quartet_stream_t stream);

/* Host helpers for the blocked scale layout (`to_blocked`, benchmark_mxfp4.ipynb:1015-1016). */
int64_t quartet_sf_offset(int64_t row, int64_t kblock, int64_t padded_kblocks);
int64_t quartet_sf_bytes(int64_t rows, int64_t cols);

/*
 * Reads and clears the device-side fault word of the current device (synchronises the
 * device).  Non-zero means a kernel gave up on a bounded wait (bits 0-7: which wait).
 */
int quartet_device_status(int32_t* status);

const char* quartet_last_error_string(void);
int quartet_version(void);

#ifdef __cplusplus
}
#endif
#endif /* QUARTET_B200_H */
