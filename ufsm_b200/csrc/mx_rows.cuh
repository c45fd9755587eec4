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
/* codes -> the eight decoded values times the row's scale factor */
template <int BITS> __device__ __forceinline__ void qrow_dec(uint2 raw, float fx, float *r) {
    if (BITS == 8) { dec_e4m3x4(raw.x, r); dec_e4m3x4(raw.y, r + 4); } else dec_e2m1x8(raw.x, r);
#pragma unroll
    for (int k = 0; k < 8; k++) r[k] *= fx;
}
/* this lane's eight values of a row -> its codes; returns the row's scale byte (the same in the four lanes).  All 32 lanes of the warp
   call it together.  Same arithmetic as mx_encode_row32: NaN-propagating amax on the magnitude bits, v * 2^-e, hardware conversion. */
template <int BITS> __device__ __forceinline__ unsigned qrow_enc(const float *r, uint2 &w) {
    unsigned am = 0u;
#pragma unroll
    for (int k = 0; k < 8; k++) am = amax_u(am, r[k]);
    am = max(am, __shfl_xor_sync(0xffffffffu, am, 1));
    am = max(am, __shfl_xor_sync(0xffffffffu, am, 2));
    const int e = mx_exp(__uint_as_float(am), BITS == 4 ? 1.f / 6.f : 1.f / 448.f);
    const float m = exp2i(-e);
    if (BITS == 8) { w.x = cvt_e4m3x4(r[0] * m, r[1] * m, r[2] * m, r[3] * m); w.y = cvt_e4m3x4(r[4] * m, r[5] * m, r[6] * m, r[7] * m); }
    else { w.x = cvt_e2m1x8(r, m); w.y = 0u; }
    return (unsigned)(e + 127) & 0xffu;
}
template <int BITS> __device__ __forceinline__ void qrow_st(uint8_t *__restrict__ codes, size_t row, int q, uint2 w) {
    if (BITS == 8) ((uint2 *)(codes + row * 32))[q] = w; else ((unsigned *)(codes + row * 16))[q] = w.x;
}
/* silu(fma(x, a, b)) with the accurate expf and an IEEE division */
__device__ __forceinline__ float silu_ab(float x, float a, float b) { const float u = __fmaf_rn(x, a, b); return __fdiv_rn(u, __fadd_rn(1.f, expf(-u))); }
