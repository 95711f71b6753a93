// The whole QuantizedLinear forward / backward as ONE host call each: the same kernels the single entry points
// launch, in the same order, without returning to the caller's language between them.  For small layers the
// time between launches is the host's, and a Python caller pays tens of microseconds per entry point.
//
//   forward   Xq = Q_f(X), Wq = Q_f(W), Y = Xq Wq^T                        (quantization/__init__.py:36-42 of the reference)
//   backward  Q_b(E), Q_b(Wq^T), dX = unrotate(mask_x * 16/9 * ...);        (backward.py:64-85, mxfp4.py:142-146)
//             Q_b(E^T), Q_b(Xq^T), dW = unrotate(mask_w * 16/9 * ...)
#include "common.cuh"

using namespace quartet;

static inline int64_t pad256(int64_t v) { return (v + 255) / 256 * 256; }

namespace {
struct BwdWorkspace {
    int64_t ec, es, etc, ets, wtc, wts, xtc, xts, total;
};
BwdWorkspace layout_bwd(int64_t M, int64_t N, int64_t K) {
    BwdWorkspace w{};
    int64_t off = 0;
    auto take = [&](int64_t bytes) {
        const int64_t at = off;
        off += pad256(bytes);
        return at;
    };
    w.ec = take(M * N / 2), w.es = take(quartet_sf_bytes(M, N));
    w.etc = take(N * M / 2), w.ets = take(quartet_sf_bytes(N, M));
    w.wtc = take(K * N / 2), w.wts = take(quartet_sf_bytes(K, N));
    w.xtc = take(K * M / 2), w.xts = take(quartet_sf_bytes(K, M));
    w.total = off;
    return w;
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int quartet_linear_fwd(
    const void* x, int x_dtype, const void* w, int w_dtype, int64_t M, int64_t N, int64_t K, float had_scale_x, float had_scale_w,
    float gaussian_scale, uint8_t* xc, uint8_t* xs, uint8_t* xm, uint8_t* wc, uint8_t* ws, uint8_t* wm, void* y, int y_dtype,
    quartet_stream_t stream) {
    if (M < 128 || N < 128 || K < 128 || M % 128 || N % 128 || K % 128)
        return fail(QUARTET_E_SHAPE, "M, N, K must be multiples of 128 (got %lld, %lld, %lld)", (long long)M, (long long)N, (long long)K);
    int rc = quartet_quant_fwd(x, x_dtype, M, K, had_scale_x, gaussian_scale, xc, xs, xm, stream);
    if (rc) return rc;
    if ((rc = quartet_quant_fwd(w, w_dtype, N, K, had_scale_w, gaussian_scale, wc, ws, wm, stream))) return rc;
    return quartet_gemm_mxfp4_tn(xc, xs, wc, ws, M, N, K, 1.0f, nullptr, had_scale_x, y, y_dtype, stream);
}

extern "C" __attribute__((visibility("default"))) int64_t quartet_linear_bwd_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    return layout_bwd(M, N, K).total;
}

extern "C" __attribute__((visibility("default"))) int quartet_linear_bwd(
    const void* e, int e_dtype, int64_t M, int64_t N, int64_t K, const uint8_t* xc, const uint8_t* xs, const uint8_t* xm,
    const uint8_t* wc, const uint8_t* ws, const uint8_t* wm, float had_scale_b, uint32_t signs, const uint32_t* signs_dev, int rounding,
    const uint64_t* seeds4, uint64_t offset, float alpha, float had_scale_x, float had_scale_w, uint8_t* workspace, void* dx, int dx_dtype,
    void* dw, int dw_dtype, quartet_stream_t stream) {
    if (!e || !workspace || !seeds4) return fail(QUARTET_E_NULL, "e, workspace and seeds4 must be non-NULL");
    if (!dx && !dw) return QUARTET_OK;
    if (M < 128 || N < 128 || K < 128 || M % 128 || N % 128 || K % 128)
        return fail(QUARTET_E_SHAPE, "M, N, K must be multiples of 128 (got %lld, %lld, %lld)", (long long)M, (long long)N, (long long)K);
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(QUARTET_E_ALIGN, "workspace must be 256-byte aligned");
    if (rounding != QUARTET_ROUND_NEAREST && rounding != QUARTET_ROUND_SR_PHILOX && rounding != QUARTET_ROUND_SR_TLRAND)
        return fail(QUARTET_E_ARG, "rounding must be 0 (nearest), 1 (own stream) or 3 (reference-compatible stream)");
    const BwdWorkspace L = layout_bwd(M, N, K);
    uint8_t *ec = workspace + L.ec, *es = workspace + L.es, *etc = workspace + L.etc, *ets = workspace + L.ets;
    uint8_t *wtc = workspace + L.wtc, *wts = workspace + L.wts, *xtc = workspace + L.xtc, *xts = workspace + L.xts;
    int rc;
    // the four quantizations take their seeds in the reference's call order: E, Wq^T, E^T, Xq^T (backward.py:69-83)
    const bool dual = dx && dw && rounding != QUARTET_ROUND_SR_TLRAND;
    if (dual && (rc = quartet_quant_bwd_dual(e, e_dtype, M, N, had_scale_b, signs, signs_dev, rounding, seeds4[0], seeds4[2], offset, ec, es, etc,
                                             ets, stream)))
        return rc;
    if (dx) {
        if (!dual && (rc = quartet_quant_bwd(e, e_dtype, M, N, had_scale_b, signs, signs_dev, rounding, seeds4[0], offset, nullptr, ec, es, stream)))
            return rc;
        if ((rc = quartet_requant_t(wc, ws, N, K, 1.0f, had_scale_b, signs, signs_dev, rounding, seeds4[1], offset, nullptr, wtc, wts, stream))) return rc;
        if ((rc = quartet_gemm_mxfp4_tn(ec, es, wtc, wts, M, K, N, alpha, xm, had_scale_x, dx, dx_dtype, stream))) return rc;
    }
    if (dw) {
        if (!dual && (rc = quartet_quant_bwd_t(e, e_dtype, M, N, had_scale_b, signs, signs_dev, rounding, seeds4[2], offset, nullptr, etc, ets, stream)))
            return rc;
        if ((rc = quartet_requant_t(xc, xs, M, K, 1.0f, had_scale_b, signs, signs_dev, rounding, seeds4[3], offset, nullptr, xtc, xts, stream))) return rc;
        if ((rc = quartet_gemm_mxfp4_tn(etc, ets, xtc, xts, N, K, M, alpha, wm, had_scale_w, dw, dw_dtype, stream))) return rc;
    }
    return QUARTET_OK;
}
