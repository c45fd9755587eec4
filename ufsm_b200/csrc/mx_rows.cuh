/* Four lanes a row: the access pattern of the elementwise kernels on MX tensors with 32-wide rows (reference layout: code rows of 32 or
   16 bytes, then one scale byte a row).  Lane q of a quad (q = lane & 3) owns channels [8 q, 8 q + 8) of a row, i.e. 8 code bytes
   (MX-fp8) or 4 (MX-fp4); the eight quads of a warp take eight consecutive rows, so one load or store instruction of a warp covers 256
   (128) contiguous bytes, and a thread keeps several such trips in flight.  The row's amax crosses the quad with two shuffles. */
#pragma once
#include "mx_common.cuh"

/* this lane's codes of row `row`: fp8 in (x, y), fp4 in x */
template <int BITS> __device__ __forceinline__ uint2 qrow_ld(const uint8_t *__restrict__ codes, size_t row, int q) {
    if (BITS == 8) return __ldg((const uint2 *)(codes + row * 32) + q);
    return make_uint2(__ldg((const unsigned *)(codes + row * 16) + q), 0u);
}
/* codes -> the eight decoded values times the row's scale factor, as four pairs (the fp32 arithmetic of these kernels runs on
   packed pairs, fma.rn.f32x2 and its siblings: half the issue slots of the scalar forms, each half an IEEE operation of its own) */
template <int BITS> __device__ __forceinline__ void qrow_dec(uint2 raw, float fx, float2 *r) {
    float t[8];
    if (BITS == 8) { dec_e4m3x4(raw.x, t); dec_e4m3x4(raw.y, t + 4); } else dec_e2m1x8(raw.x, t);
    const float2 f2 = make_float2(fx, fx);
#pragma unroll
    for (int j = 0; j < 4; j++) r[j] = __fmul2_rn(make_float2(t[2 * j], t[2 * j + 1]), f2);
}
/* magnitude of the larger of |a|, |b|, a NaN if either is one; the sign of the result carries no meaning */
__device__ __forceinline__ float absmax_nan(float a, float b) { float d; asm("max.NaN.xorsign.abs.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d; }
/* this lane's eight values of a row -> its codes; returns the row's scale byte (the same in the four lanes).  All 32 lanes of the warp
   call it together.  Same results as mx_encode_row32: NaN-propagating amax, v * 2^-e, hardware conversion. */
template <int BITS> __device__ __forceinline__ unsigned qrow_enc(const float2 *r, uint2 &w) {
    const float a01 = absmax_nan(absmax_nan(r[0].x, r[0].y), absmax_nan(r[1].x, r[1].y)), a23 = absmax_nan(absmax_nan(r[2].x, r[2].y), absmax_nan(r[3].x, r[3].y));
    unsigned am = __float_as_uint(absmax_nan(a01, a23)) & 0x7fffffffu;
    am = max(am, __shfl_xor_sync(0xffffffffu, am, 1));
    am = max(am, __shfl_xor_sync(0xffffffffu, am, 2));
    const int e = mx_exp(__uint_as_float(am), BITS == 4 ? 1.f / 6.f : 1.f / 448.f);
    const float m = exp2i(-e);
    const float2 m2 = make_float2(m, m);
    float2 s[4];
#pragma unroll
    for (int j = 0; j < 4; j++) s[j] = __fmul2_rn(r[j], m2);
    if (BITS == 8) { w.x = cvt_e4m3x4(s[0].x, s[0].y, s[1].x, s[1].y); w.y = cvt_e4m3x4(s[2].x, s[2].y, s[3].x, s[3].y); }
    else { w.x = cvt_e2m1x2(s[0].x, s[0].y) | (cvt_e2m1x2(s[1].x, s[1].y) << 8) | (cvt_e2m1x2(s[2].x, s[2].y) << 16) | (cvt_e2m1x2(s[3].x, s[3].y) << 24); w.y = 0u; }
    return (unsigned)(e + 127) & 0xffu;
}
template <int BITS> __device__ __forceinline__ void qrow_st(uint8_t *__restrict__ codes, size_t row, int q, uint2 w) {
    if (BITS == 8) ((uint2 *)(codes + row * 32))[q] = w; else ((unsigned *)(codes + row * 16))[q] = w.x;
}
/* u / (1 + exp(-u)) through the two hardware approximations, ex2 and rcp (about 2^-22 relative each; the argument of ex2 adds
   |u| 2^-24): within about 1e-6 relative of the definition for the arguments a normalised tensor produces, which is the accuracy class
   of the reference's own __expf form.  Beyond u = -87, where 1 + exp(-u) reaches 2^126, the result is a zero for a true value below 1e-36. */
__device__ __forceinline__ float silu_hw(float u) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(u * -1.44269504088896341f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
    return u * r;
}
__device__ __forceinline__ float2 silu_ab2(float2 x, float2 a, float2 b) { const float2 u = __ffma2_rn(x, a, b); return make_float2(silu_hw(u.x), silu_hw(u.y)); }
