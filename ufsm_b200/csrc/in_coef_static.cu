/* InstanceNorm coefficients of a stored blocked-fp16 tensor without any allocation.

   Who needs this: code that runs where the CUDA allocator must not be called, e.g. a worker that has handed all device memory to
   its own pool at start-up, a caller inside a latency-critical loop where cudaMalloc's implicit device synchronisation would stall
   every other stream, or a host that forbids allocation after initialisation.  umx_in_coef needs a caller-allocated buffer of partial
   sums that the conv epilogue filled; this entry point computes the same coefficients from the stored tensor alone and keeps the
   partial sums in a fixed array that is part of the library's device image.

   The array: UMX_STATIC_DOUBLES doubles (4 MiB), file scope, present on every GPU that loads the library until the process exits.
   In host code its name is only a stand-in for the symbol, not a device address, so the address is taken once per device with
   cudaGetSymbolAddress while that device is current (the first call on a device does this) and handed to the kernels as an ordinary
   pointer.

   Sharing: every call on a device uses the same array and leaves its partial sums behind.  Nothing has to start at zero: a call
   writes every slot it later reads, so stale contents from an earlier (larger or smaller) call are never seen.  Two calls that overlap
   on the GPU (different streams or host threads on one device) would race on the array; issue them one after the other, as the
   library's single-stream convention already does. */
#include "mx_common.cuh"

#define UMX_STATIC_DOUBLES (1 << 19)
#define UMX_STATIC_CHUNKS 64            /* voxel chunks per (sample, channel) */

static __device__ __align__(256) double g_in_scratch[UMX_STATIC_DOUBLES];
static double *g_in_scratch_ptr[16];    /* per device: the array's device address, taken at set-up */

/* partial sums of chunk t of block blk of sample n: part[((n * T + t) * Cop + c) * 2 + {0, 1}]; a thread owns one channel and every
   eighth voxel of the chunk, the eight phases are added in a fixed order */
__global__ void __launch_bounds__(256) in_part_static_k(const __half *__restrict__ y, int C, size_t S, int T, double *__restrict__ part) {
    const int t = blockIdx.x, blk = blockIdx.y, n = blockIdx.z, nb = gridDim.y, Cop = nb * 32;
    const int c = threadIdx.x & 31, ph = threadIdx.x >> 5;
    const size_t v0 = S * t / T, v1 = S * (t + 1) / T;
    const __half *p = y + ((size_t)n * nb + blk) * S * 32 + c;
    double s = 0.0, q = 0.0;
    for (size_t v = v0 + ph; v < v1; v += 8) { const double x = (double)__half2float(p[v * 32]); s += x; q += x * x; }
    __shared__ double ss[8][32], sq[8][32];
    ss[ph][c] = s; sq[ph][c] = q;
    __syncthreads();
    if (ph == 0) {
        for (int k = 1; k < 8; k++) { s += ss[k][c]; q += sq[k][c]; }
        double *d = part + (((size_t)n * T + t) * Cop + blk * 32 + c) * 2;
        d[0] = s; d[1] = q;
    }
}
/* one block per (channel, sample): the T chunk sums in a fixed order, then a = gamma rstd, b = beta - mean a */
__global__ void __launch_bounds__(64) in_coef_static_k(const double *__restrict__ part, int C, int Cop, int T, double S, const float *gamma, const float *beta, float eps, float *coef) {
    const int c = blockIdx.x, n = blockIdx.y;
    __shared__ double ss[64], sq[64];
    double s = 0.0, q = 0.0;
    for (int t = threadIdx.x; t < T; t += 64) { const double *p = part + (((size_t)n * T + t) * Cop + c) * 2; s += p[0]; q += p[1]; }
    ss[threadIdx.x] = s; sq[threadIdx.x] = q;
    __syncthreads();
    for (int o = 32; o > 0; o >>= 1) { if ((int)threadIdx.x < o) { ss[threadIdx.x] += ss[threadIdx.x + o]; sq[threadIdx.x] += sq[threadIdx.x + o]; } __syncthreads(); }
    if (threadIdx.x == 0) {
        const double m = ss[0] / S, v = fmax(sq[0] / S - m * m, 0.0);
        const float rs = (float)(1.0 / sqrt(v + (double)eps)), a = __fmul_rn(rs, gamma ? gamma[c] : 1.f);
        coef[2 * ((size_t)n * C + c)] = a;
        coef[2 * ((size_t)n * C + c) + 1] = __fmaf_rn(-(float)m, a, beta ? beta[c] : 0.f);
    }
}

/* y: device, blocked fp16 [n][blk][voxel][32] of C channels on an N x D x H x W grid (what a conv stores with UMX_OUT_H16B);
   gamma / beta: device [C] or NULL; coef: device floats [N][C][2], the output.  Returns 0; -1 after latching an error when
   N * 64 * (C rounded up to 32) * 2 exceeds UMX_STATIC_DOUBLES (e.g. N = 1: up to 4096 channels; N = 8: up to 512), when a
   dimension is below 1, when a launch failed, or when no usable device is current.  Calls no allocator of any kind. */
extern "C" int umx_in_coef_static(const void *y, int N, int C, int D, int H, int W, const float *gamma, const float *beta, float eps, float *coef) {
    if (!umx_ready("umx_in_coef_static")) return -1;
    const int nb = (C + 31) / 32, Cop = nb * 32, T = UMX_STATIC_CHUNKS;
    const size_t need = (size_t)N * T * Cop * 2;
    if (D < 1 || H < 1 || W < 1) { umx_latch_msg("umx_in_coef_static: D, H and W must be at least 1"); return -1; }
    if (N < 1 || C < 1 || need > (size_t)UMX_STATIC_DOUBLES) {
        char b[256]; snprintf(b, sizeof b, "umx_in_coef_static: N = %d, C = %d needs %zu doubles of scratch; the built-in array holds %d (N x 64 x roundup32(C) x 2 must fit)", N, C, need, UMX_STATIC_DOUBLES);
        umx_latch_msg(b);
        return -1;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) { umx_latch_msg("umx_in_coef_static: no current device"); return -1; }
    if (!g_in_scratch_ptr[dev]) {   /* set-up, once per device, with that device current */
        double *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void **)&p, g_in_scratch);
        if (e != cudaSuccess || !p) { umx_latch("umx_in_coef_static: cudaGetSymbolAddress", e); return -1; }
        g_in_scratch_ptr[dev] = p;
    }
    double *part = g_in_scratch_ptr[dev];
    const size_t S = (size_t)D * H * W;
    in_part_static_k<<<dim3(T, nb, N), 256>>>((const __half *)y, C, S, T, part);
    in_coef_static_k<<<dim3(C, N), 64>>>(part, C, Cop, T, (double)S, gamma, beta, eps, coef);
    g_umx_launches += 2;
    const cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) { umx_latch("umx_in_coef_static", le); return -1; }
    return 0;
}
