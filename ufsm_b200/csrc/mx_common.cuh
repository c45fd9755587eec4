/* Device helpers shared by the MX kernels: block exponent, element encoders / decoders, error latch. */
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/ufsm_mx.h"

/* ---- error latch (host side; the convention of the reference's LPCK / lp_check, src/lp_common.cuh:35-38) ---- */
void umx_latch(const char *where, cudaError_t e);
void umx_latch_msg(const char *msg);
int umx_ready(const char *where);   /* 1 when a usable sm_100 device is current; otherwise latches and returns 0 */
#define UMX_CK(where) do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) umx_latch(where, e_); } while (0)
void *umx_ws(int slot, size_t bytes);   /* per-device scratch that only grows (the role of the reference's nn_ws registry, src/nn.h:732-739) */
int *umx_errflag(void);                 /* device int the kernels report bounded-wait failures into */
int umx_errflag_read(void);             /* synchronises, reads and clears it */
extern long g_umx_launches;
int umx_prof_open(double flops);   /* conv launch timing (runtime.cu): returns a slot or -1 when profiling is off */
void umx_prof_close(int id);

/* ---- programmatic dependent launch: a kernel launched through umx_launch may be scheduled while its predecessor in the stream is still
   running; it calls pdl_wait() before its first access to memory the predecessor may write or read, and pdl_trigger() as early as it
   likes to let its own successor be scheduled.  What is gained is the launch latency (and, in the conv kernels, the prologue: barrier
   set-up, TMEM allocation, weight loads) of some 80 dependent launches per forward.  UMX_PDL=0 in the environment turns it off. ---- */
int umx_pdl(void);
#ifdef __CUDACC__
#include <string.h>
template <typename... KA, typename... A>
static inline void umx_launch(void (*kern)(KA...), dim3 grid, dim3 block, size_t smem, A... args) {
    cudaLaunchConfig_t cfg; memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = 0;
    cudaLaunchAttribute at[1]; memset(at, 0, sizeof at);
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
    if (umx_pdl()) { cfg.attrs = at; cfg.numAttrs = 1; }
    cudaLaunchKernelEx(&cfg, kern, static_cast<KA>(args)...);
}
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

/* ---- MX arithmetic ---- */
/* exponent e of the block scale 2^e = exponent of amax / qmax rounded up, clamped to [-126, 126]; NaN / inf amax -> 128 (scale
   byte 0xFF).  Same rule as src/lp_common.cuh:492-500. */
__device__ __forceinline__ int mx_exp(float amax, float inv_qmax) {
    const unsigned u = __float_as_uint(__fmul_rn(amax, inv_qmax)) & 0x7fffffffu;
    if (u >= 0x7f800000u) return 128;
    const int eb = (int)((u + 0x7fffffu) >> 23);            /* the biased exponent, one more when the mantissa is not zero */
    return max(1, min(253, eb)) - 127;
}
__device__ __forceinline__ float exp2i(int e) { return __uint_as_float((unsigned)(127 + e) << 23); }
/* NaN-propagating amax on the magnitude bits (src/lp_common.cuh:486) */
__device__ __forceinline__ unsigned amax_u(unsigned a, float v) { return max(a, __float_as_uint(v) & 0x7fffffffu); }
/* scale byte -> factor; 0xFF -> +inf, 0 -> 2^-127 */
__device__ __forceinline__ float mx_scale(unsigned b) { b &= 0xffu; return b == 0xffu ? __uint_as_float(0x7f800000u) : b == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(b << 23); }

/* four floats -> four e4m3 bytes (a lowest): cvt.rn.satfinite, the hardware conversion the reference's integer code mirrors */
__device__ __forceinline__ unsigned cvt_e4m3x4(float a, float b, float c, float d) {
    unsigned short lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return (unsigned)lo | ((unsigned)hi << 16);
}
/* two floats -> one byte of two e2m1 nibbles (lo in the low nibble) */
__device__ __forceinline__ unsigned cvt_e2m1x2(float lo, float hi) {
    unsigned short r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(r) : "f"(hi), "f"(lo));
    return (unsigned)r & 0xffu;
}
__device__ __forceinline__ unsigned cvt_e2m1x8(const float *v, float m) {
    return cvt_e2m1x2(v[0] * m, v[1] * m) | (cvt_e2m1x2(v[2] * m, v[3] * m) << 8) | (cvt_e2m1x2(v[4] * m, v[5] * m) << 16) | (cvt_e2m1x2(v[6] * m, v[7] * m) << 24);
}
__device__ __forceinline__ float dec_e4m3(unsigned b) {
    const unsigned e = (b >> 3) & 15u, m = b & 7u;
    if ((b & 0x7fu) == 0x7fu) return __uint_as_float(0x7fc00000u | ((b & 0x80u) << 24));
    const float v = e ? (float)(8u + m) * __uint_as_float((117u + e) << 23) : (float)m * 0.001953125f;
    return (b & 0x80u) ? -v : v;
}
__device__ __forceinline__ float dec_e2m1(unsigned n) {
    const unsigned k = n & 7u;
    const float v = (float)(k < 4u ? k : k == 4u ? 4u : k == 5u ? 6u : k == 6u ? 8u : 12u) * 0.5f;
    return (n & 8u) ? -v : v;
}
/* four e4m3 bytes / eight e2m1 nibbles of a word -> floats, through the hardware conversions to packed halves (every code is exact in fp16;
   the e4m3 NaN code becomes a NaN) */
__device__ __forceinline__ void dec_e4m3x4(unsigned w, float *o) {
    unsigned lo, hi;
    asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}" : "=r"(lo), "=r"(hi) : "r"(w));
    const float2 f0 = __half22float2(*(const __half2 *)&lo), f1 = __half22float2(*(const __half2 *)&hi);
    o[0] = f0.x; o[1] = f0.y; o[2] = f1.x; o[3] = f1.y;
}
__device__ __forceinline__ void dec_e2m1x8(unsigned w, float *o) {
    unsigned h0, h1, h2, h3;
    asm("{\n\t.reg .b8 a, b, c, d;\n\tmov.b32 {a, b, c, d}, %4;\n\tcvt.rn.f16x2.e2m1x2 %0, a;\n\tcvt.rn.f16x2.e2m1x2 %1, b;\n\tcvt.rn.f16x2.e2m1x2 %2, c;\n\tcvt.rn.f16x2.e2m1x2 %3, d;\n\t}"
        : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(w));
    const float2 f0 = __half22float2(*(const __half2 *)&h0), f1 = __half22float2(*(const __half2 *)&h1), f2 = __half22float2(*(const __half2 *)&h2), f3 = __half22float2(*(const __half2 *)&h3);
    o[0] = f0.x; o[1] = f0.y; o[2] = f1.x; o[3] = f1.y; o[4] = f2.x; o[5] = f2.y; o[6] = f3.x; o[7] = f3.y;
}
/* a row of 32 fp16 values (16 packed pairs) -> MX-fp8 codes w[0..8) and the scale byte; the same bytes as mx_encode_row32<8> of the
   values converted to fp32.  amax, scaling and conversion stay on packed halves when the block scale 2^-e is a normal fp16 (the product
   is then exact, or below 2^-14 where E4M3 rounds to zero either way); other rows take the fp32 path. */
__device__ __forceinline__ unsigned mx_encode_row32_h8(const __half2 *h, unsigned *w) {
    __half2 a2 = __habs2(h[0]);
#pragma unroll
    for (int k = 1; k < 16; k++) a2 = __hmax2_nan(a2, __habs2(h[k]));
    const float am = __half2float(__hmax_nan(__low2half(a2), __high2half(a2)));
    const int e = mx_exp(__uint_as_float(__float_as_uint(am) & 0x7fffffffu), 1.f / 448.f);
    if (e >= -15 && e <= 14) {
        const unsigned mh = (unsigned)(15 - e) << 10, m2 = mh | (mh << 16);
        const __half2 mm = *(const __half2 *)&m2;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const __half2 s0 = __hmul2(h[2 * j], mm), s1 = __hmul2(h[2 * j + 1], mm);
            unsigned short c0, c1;
            asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(c0) : "r"(*(const unsigned *)&s0));
            asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(c1) : "r"(*(const unsigned *)&s1));
            w[j] = (unsigned)c0 | ((unsigned)c1 << 16);
        }
    } else {
        const float m = exp2i(-e);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float2 p0 = __half22float2(h[2 * j]), p1 = __half22float2(h[2 * j + 1]);
            w[j] = cvt_e4m3x4(p0.x * m, p0.y * m, p1.x * m, p1.y * m);
        }
    }
    return (unsigned)(e + 127) & 0xffu;
}
/* a row of 32 floats -> MX codes: q8 receives 32 bytes (BITS 8: w[0..8)) or 16 bytes (BITS 4: w[0..4)); returns the scale byte */
template <int BITS> __device__ __forceinline__ unsigned mx_encode_row32(const float *v, unsigned *w) {
    unsigned am = 0u;
#pragma unroll
    for (int k = 0; k < 32; k++) am = amax_u(am, v[k]);
    const int e = mx_exp(__uint_as_float(am), BITS == 4 ? 1.f / 6.f : 1.f / 448.f);
    const float m = exp2i(-e);
    if (BITS == 4) {
#pragma unroll
        for (int j = 0; j < 4; j++) w[j] = cvt_e2m1x8(v + 8 * j, m);
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) w[j] = cvt_e4m3x4(v[4 * j] * m, v[4 * j + 1] * m, v[4 * j + 2] * m, v[4 * j + 3] * m);
    }
    return (unsigned)(e + 127) & 0xffu;
}
