// Per-group arithmetic shared by the quantizer kernels: 32-point Walsh-Hadamard in
// registers, Philox4x32, the three rounding rules and e2m1 packing.
// One thread owns one group of 32 values throughout.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace quartet {

// Packed single-precision pairs (add/sub/mul/fma.f32x2): one issue slot for two IEEE fp32 operations,
// each lane rounded exactly like its scalar counterpart.  The quantizers are bound by instruction
// issue, not by memory, so halving the issue count of the butterflies is what matters.
typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t pack2(float lo, float hi) {
    f32x2_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2_t add2(f32x2_t a, f32x2_t b) {
    f32x2_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2_t sub2(f32x2_t a, f32x2_t b) {
    f32x2_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2_t mul2(f32x2_t a, f32x2_t b) {
    f32x2_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2_t fma2(f32x2_t a, f32x2_t b, f32x2_t c) {
    f32x2_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ float max3_abs(float m, float a, float b) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(m), "f"(fabsf(a)), "f"(fabsf(b)));
    return r;
}

// Unnormalised Sylvester-ordered WHT: w_j = sum_i x_i (-1)^popc(i & j).  The stride-1 butterflies run
// as scalar operations while the pairs (2i, 2i+1) are formed; the four wider strides are packed.
// Butterfly stages commute and every lane operation is the scalar one, so the result is bit-identical
// to the plain five-stage network.
__device__ __forceinline__ void wht32(float (&v)[32]) {
    f32x2_t p[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float a = v[2 * i], b = v[2 * i + 1];
        p[i] = pack2(a + b, a - b);
    }
#pragma unroll
    for (int s = 1; s < 16; s <<= 1) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if ((i & s) == 0) {
                const f32x2_t a = p[i], b = p[i + s];
                p[i] = add2(a, b);
                p[i + s] = sub2(a, b);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) unpack2(p[i], v[2 * i], v[2 * i + 1]);
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& q, float* out) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}

// One group of 32 consecutive row elements out of a 128-row tile that TMA laid down as 128-byte-wide
// boxes (128 rows x 128 B each, 128B swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7)).
// `gk` = group index within the tile row (0..3).
// BOX = bytes of one box (its rows x 128): 128-row boxes for the 128 x 128 tiles, fewer rows for wider tiles.
template <bool F32, int BOX>
__device__ __forceinline__ void load_row_group_box(const uint8_t* s_in, int row, int gk, float (&w)[32]) {
    if (F32) {
        const uint8_t* base = s_in + gk * BOX + row * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 q = *reinterpret_cast<const float4*>(base + ((j ^ (row & 7)) << 4));
            w[4 * j] = q.x, w[4 * j + 1] = q.y, w[4 * j + 2] = q.z, w[4 * j + 3] = q.w;
        }
    } else {
        const uint8_t* base = s_in + (gk >> 1) * BOX + row * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int chunk = (gk & 1) * 4 + j;
            const uint4 q = *reinterpret_cast<const uint4*>(base + ((chunk ^ (row & 7)) << 4));
            unpack_bf16x8(q, &w[8 * j]);
        }
    }
}
template <bool F32>
__device__ __forceinline__ void load_row_group(const uint8_t* s_in, int row, int gk, float (&w)[32]) {
    load_row_group_box<F32, 128 * 128>(s_in, row, gk, w);
}

// ---------------------------------------------------------------------------
// Philox4x32 (Salmon et al. 2011), word order as in triton/language/random.py:13-41.
// ---------------------------------------------------------------------------
// Rounds of the library's OWN dither stream.  Seven is the fewest rounds at which Philox4x32 passes BigCrush
// (Salmon et al. 2011, table 2; ten is their default, with margin); the dither of a 4-bit rounding needs far
// less.  The Philox calls are 40 % of the instructions of the stochastic-rounding quantizers, which are bound
// by instruction issue: seven rounds instead of ten make them 5-8 % faster.  (The reference-compatible stream,
// tl_rand below, keeps Triton's ten.)
constexpr int OWN_PHILOX_ROUNDS = 7;
struct Philox4 {
    uint32_t w[4];
};
template <int ROUNDS = 10>
__device__ __forceinline__ Philox4 philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
    constexpr uint32_t KA = 0x9E3779B9u, KB = 0xBB67AE85u, RA = 0xD2511F53u, RB = 0xCD9E8D57u;
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        const uint32_t hb = __umulhi(RB, c2), lb = RB * c2;
        const uint32_t ha = __umulhi(RA, c0), la = RA * c0;
        c0 = hb ^ c1 ^ k0;
        c2 = ha ^ c3 ^ k1;
        c1 = lb;
        c3 = la;
        k0 += KA;
        k1 += KB;
    }
    return Philox4{{c0, c1, c2, c3}};
}
// tl.rand(seed, offset): first Philox word -> [0, 1)  (triton/language/random.py:127-157)
__device__ __forceinline__ float tl_rand(uint64_t seed, uint32_t offset) {
    const Philox4 p = philox4x32<10>(offset, 0u, 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32));
    int32_t x = (int32_t)p.w[0];
    x = x < 0 ? -x - 1 : x;
    return __int2float_rn(x) * 4.6566127342e-10f;
}

// ---------------------------------------------------------------------------
// scales
// ---------------------------------------------------------------------------
// floor(log2(s)) + 127 for a positive normal float = its exponent field.
__device__ __forceinline__ int exp_field(float s) { return (int)((__float_as_uint(s) >> 23) & 0xFFu); }
__device__ __forceinline__ float pow2_biased(int b) { return __uint_as_float((uint32_t)b << 23); }  // 2^(b-127), 1<=b<=254

// ---------------------------------------------------------------------------
// rounding
// ---------------------------------------------------------------------------
// Eight values -> eight e2m1 codes in one word (element 0 in the lowest nibble) with the hardware
// round-to-nearest-even conversion.  Differs from the reference's strict-`>` ladder
// (mxfp4_triton.py:131-159) only when |v| is EXACTLY 0.75, 1.75 or 3.5; cvt_e2m1x8_ties_down repairs those.
__device__ __forceinline__ uint32_t cvt_e2m1x8_rn(const float* v) {
    uint32_t r;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t.reg .b16 h0, h1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b16 h0, {b0, b1};\n\tmov.b16 h1, {b2, b3};\n\tmov.b32 %0, {h0, h1};\n\t}"
        : "=r"(r)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return r;
}

// One byte (two codes) -> two floats, exact.
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
    uint32_t h2;
    asm("{\n\t.reg .b8 lo, hi;\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tmov.b16 {lo, hi}, t;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, lo;\n\t}"
        : "=r"(h2)
        : "r"(byte));
    return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

// Reference ladder index for |v| with strict `>` (ties toward the smaller magnitude).
__device__ __forceinline__ int rtn_index_exact(float a) {
    return (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
}

// Reference stochastic rounding: bracket by strict `>`, p = (a - lo) / (hi - lo), up iff u < p.
__device__ __forceinline__ int sr_index_exact(float a, float u) {
    const int lo = (a > 0.5f) + (a > 1.0f) + (a > 1.5f) + (a > 2.0f) + (a > 3.0f) + (a > 4.0f);
    const float glo = lo < 4 ? 0.5f * lo : (lo == 4 ? 2.0f : (lo == 5 ? 3.0f : 4.0f));
    const float inv_step = lo < 4 ? 2.0f : (lo < 6 ? 1.0f : 0.5f);
    const float p = (a - glo) * inv_step;  // exact: the step is a power of two
    return lo + ((u < p) ? 1 : 0);
}

// Hardware stochastic rounding of four values to e2m1 (nibble k of the result = value k).
// Measured behaviour of cvt.rs on sm_100a: each value gets a 16-bit dither D assembled from two
// bytes b0..b3 of `rbits` and rounds away from zero iff D + floor(65536 * frac) >= 65536, where
// frac is the position of |v| between its two neighbouring grid points (|v| >= 6 saturates to 6):
//   value 0: D = b2:b0      value 1: D = rev(b0):rev(b2)      (rev = the byte bit-reversed)
//   value 2: D = b3:b1      value 3: D = rev(b1):rev(b3)
// so P(up) = frac to within 2^-16: unbiased for every practical purpose.
__device__ __forceinline__ uint32_t cvt_rs_e2m1x4(float x0, float x1, float x2, float x3, uint32_t rbits) {
    uint16_t r;
    asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;" : "=h"(r) : "f"(x3), "f"(x2), "f"(x1), "f"(x0), "r"(rbits));
    return r;
}

// Eight values -> eight e2m1 codes rounded exactly like the reference ladder (round to nearest, ties toward
// the SMALLER magnitude: mxfp4_triton.py:131-159).  The hardware round-to-nearest-even conversion agrees
// with the ladder everywhere except at |v| == 0.75, 1.75, 3.5, which it rounds up.  Those are found without
// a compare per value: the stochastic-rounding conversion with the constant dither 0x7FFE in all four
// positions (rbits 0x7F7FFEFE, see cvt_rs_e2m1x4) rounds up iff the value lies at least 2^-15 of a grid
// step above the midpoint, so it rounds every exact tie DOWN and differs from round-to-nearest-even only
// for values in the sliver [midpoint, midpoint + 2^-15 step) -- about one group in a thousand.  Words
// on which the two conversions disagree are redone with the ladder itself.
__device__ __forceinline__ uint32_t cvt_e2m1x8_ties_down(const float* v) {
    const uint32_t rn = cvt_e2m1x8_rn(v);
    constexpr uint32_t DITHER = 0x7F7FFEFEu;
    const uint32_t rs = cvt_rs_e2m1x4(v[0], v[1], v[2], v[3], DITHER) | (cvt_rs_e2m1x4(v[4], v[5], v[6], v[7], DITHER) << 16);
    if (rs == rn) return rn;
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        r |= ((uint32_t)rtn_index_exact(fabsf(v[i])) | ((__float_as_uint(v[i]) >> 28) & 8u)) << (4 * i);
    return r;
}

__device__ __forceinline__ uint32_t spread_sign_bits(uint32_t s8) {
    // bit i of s8 -> bit 4i+3 (the sign bit of nibble i)
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) r |= ((s8 >> i) & 1u) << (4 * i + 3);
    return r;
}

// ---------------------------------------------------------------------------
// Forward ("Quest") quantization of one group of 32 (mxfp4_triton.py:33-57,130-174 of the reference): rotate,
// scale by the power of two at or below gaussian_scale * std + 1e-8, round to nearest with ties toward zero, and
// report which values lie strictly inside the grid (|v| < 6) as 32 mask bits.  w holds the group on entry and
// the rotated values on return.  ROT = false skips the rotation (h must then be 1).
// ---------------------------------------------------------------------------
// The part after the moments: w holds the rotated values WITHOUT the factor h; mean and mean_sq are the moments of
// the rotated group with it.
__device__ __forceinline__ void quest_finish_group(const float (&w)[32], float h, float mean, float mean_sq, float gaussian_scale,
                                                   uint32_t (&words)[4], uint32_t& mbits, int& e8m0) {
    const float var = fmaxf(mean_sq - mean * mean, 0.f);
    const float scales = gaussian_scale * sqrtf(var) + 1e-8f;
    e8m0 = exp_field(scales);
    const float c = h * pow2_biased(254 - e8m0);  // h * 2^-e
    float v[32];
    const f32x2_t c2 = pack2(c, c), m36 = pack2(-36.f, -36.f);
    // mask bit = |v| < 6  <=>  v * v - 36 < 0; the fused multiply-add rounds the exact difference, so its
    // sign is exact (and |v| == 6 gives +0: clipped, as in the reference's strict `<`)
    mbits = 0;
#pragma unroll
    for (int i = 15; i >= 0; --i) {
        const f32x2_t vp = mul2(pack2(w[2 * i], w[2 * i + 1]), c2);
        unpack2(vp, v[2 * i], v[2 * i + 1]);
        float t0, t1;
        unpack2(fma2(vp, vp, m36), t0, t1);
        mbits = __funnelshift_l(__float_as_uint(t1), mbits, 1);
        mbits = __funnelshift_l(__float_as_uint(t0), mbits, 1);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) words[q] = cvt_e2m1x8_ties_down(&v[8 * q]);
    // (the reference gives exact zeros a minus sign, `v > 0 ? + : -`; here +0 stays +0)
}

template <bool ROT>
__device__ __forceinline__ void quest_quantize_group(float (&w)[32], float h, float gaussian_scale, uint32_t (&words)[4],
                                                     uint32_t& mbits, int& e8m0) {
    // statistics that do not need the rotated values: sum_j xh_j = 32 h x_0 (only row 0 of the
    // Sylvester matrix has a non-zero column sum) and sum_j xh_j^2 = 32 h^2 sum_i x_i^2 (Parseval).
    float x0 = w[0];
    if (!ROT) {
        // no rotation: the group's own sum takes the place of 32 h x_0 (h = 1 here, see below)
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) s += w[i];
        x0 = s * (1.0f / 32.0f);
    }
    // two interleaved partial sums (even / odd elements) in one packed accumulator
    f32x2_t acc = pack2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const f32x2_t pr = pack2(w[2 * i], w[2 * i + 1]);
        acc = fma2(pr, pr, acc);
    }
    float s_even, s_odd;
    unpack2(acc, s_even, s_odd);
    const float sumsq = s_even + s_odd;
    if (ROT) wht32(w);
    // rotated: sum_j xh_j = 32 h x_0 and sum_j xh_j^2 = 32 h^2 sum_i x_i^2; un-rotated (h = 1): the plain moments
    const float mean = ROT ? h * x0 : x0;
    const float mean_sq = ROT ? (h * h) * sumsq : sumsq * (1.0f / 32.0f);
    quest_finish_group(w, h, mean, mean_sq, gaussian_scale, words, mbits, e8m0);
}


// ---------------------------------------------------------------------------
// Backward (absmax-scaled) quantization of one rotated group.
//   w      unnormalised WHT output; the rotated values are h * w
//   g      index of the group in the OUTPUT tensor (row-major over [out_rows, out_cols/32]);
//          counter of the own Philox stream
//   flat   index of the group's first element in the output tensor, for the caller-supplied noise
//          tensor and the tl.rand-compatible stream
//   flip   sign-vector of the rotation (H @ diag(s)) spread onto nibble sign bits
// Scale byte: E8M0 = floor(log2 amax) - 2 + 127 (the reference's extra 1/0.75 goes into the GEMM
// alpha, mxfp4_triton.py:60).
// ---------------------------------------------------------------------------
template <int ROUND>
__device__ __forceinline__ void absmax_quantize_group(const float (&w)[32], float h, uint64_t g, int64_t flat,
                                                      bool noise_valid, uint64_t seed, uint64_t offset,
                                                      const float* noise, const uint32_t (&flip)[4],
                                                      uint32_t (&words)[4], int& e8m0) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = max3_abs(amax, w[2 * i], w[2 * i + 1]);
    amax *= h;  // max |h w| = h max|w|  (h > 0, rounding is monotone)
    const int eb = exp_field(amax);
    e8m0 = max(eb - 2, 0);
    if (ROUND == 1 /* QUARTET_ROUND_SR_PHILOX */) {
        const bool zero = eb < 3;
        const float c = zero ? 0.f : (0.75f * h) * pow2_biased(254 - e8m0);
        const f32x2_t c2 = pack2(c, c);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint64_t ctr = 2 * g + j;
            const Philox4 r = philox4x32<OWN_PHILOX_ROUNDS>((uint32_t)ctr, (uint32_t)(ctr >> 32), (uint32_t)offset,
                                            (uint32_t)(offset >> 32), (uint32_t)seed, (uint32_t)(seed >> 32));
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
                const int i = 16 * j + 4 * wd;
                float x0, x1, x2, x3;
                unpack2(mul2(pack2(w[i], w[i + 1]), c2), x0, x1);
                unpack2(mul2(pack2(w[i + 2], w[i + 3]), c2), x2, x3);
                const uint32_t r16 = cvt_rs_e2m1x4(x0, x1, x2, x3, r.w[wd]);
                if (wd & 1)
                    words[2 * j + (wd >> 1)] = (words[2 * j + (wd >> 1)] | (r16 << 16)) ^ flip[2 * j + (wd >> 1)];
                else
                    words[2 * j + (wd >> 1)] = r16;
            }
        }
    } else {
        // reference-exact arithmetic: shared = fl(2^e / 0.75), v = xh / shared (IEEE division)
        float shared;
        if (eb >= 3)
            shared = pow2_biased(eb - 2) * 1.33333337306976318359375f;
        else if (eb == 0)
            shared = 0.f;
        else
            shared = ldexpf(1.33333337306976318359375f, eb - 129);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t acc = 0;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const int i = 8 * q + t;
                const float v = __fdiv_rn(w[i] * h, shared);
                const float a = fabsf(v);
                int idx;
                if (ROUND == 0 /* QUARTET_ROUND_NEAREST */) {
                    idx = rtn_index_exact(a);
                } else {
                    float u;
                    if (ROUND == 2 /* QUARTET_ROUND_SR_NOISE */)
                        u = noise_valid ? __ldg(noise + flat + i) : 0.f;
                    else
                        u = tl_rand(seed, (uint32_t)(flat + i));
                    idx = sr_index_exact(a, u);
                }
                acc |= ((uint32_t)idx | ((v > 0.f) ? 0u : 8u)) << (4 * t);
            }
            words[q] = acc ^ flip[q];
        }
    }
}

}  // namespace quartet
