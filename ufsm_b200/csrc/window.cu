/* Device-side pieces of the sliding-window path: the CT input conversion and the Gaussian-weighted blend of a patch's logits into
   the rank's accumulators (the role of k_i3_blend, src/nn_ink3dext.cu:58-73, in the reference).  HBM-bound elementwise passes. */
#include "mx_common.cuh"

__global__ void __launch_bounds__(256) u8_to_h16_k(const uint8_t *__restrict__ x, __half *__restrict__ y, size_t n) {
    pdl_trigger(); pdl_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] = __float2half_rn(__fdiv_rn((float)x[i], 255.f));
}
/* x: uint8 CT values on the device -> fp16 intensity x / 255 (one rounding of the exact quotient) */
extern "C" void umx_u8_to_h16(const uint8_t *x, size_t n, void *y) {
    if (!umx_ready("umx_u8_to_h16")) return;
    size_t g = (n + 255) / 256; if (g > 148u * 16u) g = 148u * 16u; if (!g) g = 1;
    umx_launch(u8_to_h16_k, dim3((unsigned)g), dim3(256), 0, x, (__half *)y, n);
    g_umx_launches++;
    UMX_CK("umx_u8_to_h16");
}
/* acc[c][z - zlo][y][x] += w(z) w(y) w(x) logits[c][patch voxel], wsum likewise, for the patch at (z0, y0, x0); one thread per patch
   voxel, channels looped (patches are added one launch at a time, so no two threads touch the same accumulator) */
template <typename T>
__global__ void __launch_bounds__(256) blend_add_k(const T *__restrict__ logits, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0,
                                                    const float *__restrict__ w1d, float *__restrict__ acc, float *__restrict__ wsum) {
    pdl_trigger(); pdl_wait();
    const size_t PS = (size_t)P * P * P, plane = (size_t)V * V, AS = plane * zext;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < PS; i += (size_t)gridDim.x * blockDim.x) {
        const int x = (int)(i % P), y = (int)((i / P) % P), z = (int)(i / ((size_t)P * P));
        const int gz = z0 + z - zlo, gy = y0 + y, gx = x0 + x;
        if (gz < 0 || gz >= zext || gy >= V || gx >= V) continue;
        const float w = __fmul_rn(__fmul_rn(w1d[z], w1d[y]), w1d[x]);
        const size_t gv = (size_t)gz * plane + (size_t)gy * V + gx;
        for (int c = 0; c < nh; c++) acc[(size_t)c * AS + gv] = __fmaf_rn(w, (float)logits[(size_t)c * PS + i], acc[(size_t)c * AS + gv]);
        wsum[gv] += w;
    }
}
extern "C" void umx_blend_add(const void *logits, int fmt, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0, const float *w1d, float *acc, float *wsum) {
    if (!umx_ready("umx_blend_add")) return;
    const size_t PS = (size_t)P * P * P; size_t g = (PS + 255) / 256; if (g > 148u * 16u) g = 148u * 16u;
    if (fmt == UMX_F16) umx_launch(blend_add_k<__half>, dim3((unsigned)g), dim3(256), 0, (const __half *)logits, nh, P, V, zlo, zext, z0, y0, x0, w1d, acc, wsum);
    else umx_launch(blend_add_k<float>, dim3((unsigned)g), dim3(256), 0, (const float *)logits, nh, P, V, zlo, zext, z0, y0, x0, w1d, acc, wsum);
    g_umx_launches++;
    UMX_CK("umx_blend_add");
}
extern "C" long umx_launch_count(void) { return g_umx_launches; }
extern "C" int umx_peek_device_error(void) { return umx_errflag_read(); }
