/* The back end of the reference's predict on the device (src/nn.h:871-885, src/nn_elem.cu:1096-1178): one head's logits of a
   D x W x W window become probability bytes, the window's halo is cropped, and what is left of the interior inside the output shard
   is written at its place in a device shard buffer.  byte = trunc(255 / (1 + exp(-logit)) + 0.5) where the CT voxel is material
   (CT >= iso, or its bit in a mask built from the CT beforehand), 0 elsewhere.

   Geometry (place_isect of the reference): window voxel (z, y, x) sits at shard coordinate (oz + z, oy + y, ox + x); it is written when
   it is interior (z in [hz, D - hz), y and x in [halo, W - halo)) and inside the shard's extent ([0, ez) x [0, ey) x [0, ex)).  The box of
   such voxels is worked out on the host and a thread takes four consecutive x of one box row, so a warp reads and writes runs of 128
   voxels of a row. */
#include "mx_common.cuh"

namespace {

struct PlaceBox { int z0, y0, x0, nz, ny, nx; };
PlaceBox place_box_of(int D, int W, int hz, int halo, int oz, int oy, int ox, int ez, int ey, int ex) {
    PlaceBox b;
    b.z0 = hz > -oz ? hz : -oz; b.y0 = halo > -oy ? halo : -oy; b.x0 = halo > -ox ? halo : -ox;
    const int z1 = D - hz < ez - oz ? D - hz : ez - oz, y1 = W - halo < ey - oy ? W - halo : ey - oy, x1 = W - halo < ex - ox ? W - halo : ex - ox;
    b.nz = z1 > b.z0 ? z1 - b.z0 : 0; b.ny = y1 > b.y0 ? y1 - b.y0 : 0; b.nx = x1 > b.x0 ? x1 - b.x0 : 0;
    return b;
}
__device__ __forceinline__ unsigned prob255(float l) { return (unsigned)(__fdividef(255.f, 1.f + __expf(-l)) + 0.5f) & 0xffu; }
template <typename LT> __device__ __forceinline__ float logit_at(const LT *lg, size_t k);
template <> __device__ __forceinline__ float logit_at<float>(const float *lg, size_t k) { return __ldg(lg + k); }
template <> __device__ __forceinline__ float logit_at<__half>(const __half *lg, size_t k) { return __half2float(__ldg(lg + k)); }

/* MASK 0: material where ct[k] >= iso; 1: where bit k of `bits` is set.  zoff: the window is held from its plane zoff on (a half of a split window) */
template <typename LT, int MASK>
__global__ void __launch_bounds__(256) pred_place_k(const LT *__restrict__ lg, const uint8_t *__restrict__ ct, const uint32_t *__restrict__ bits, PlaceBox B, int W, int zoff,
                                                    int oz, int oy, int ox, int shard, uint8_t *__restrict__ dsh, int iso) {
    const int nq = (B.nx + 3) >> 2;                         /* groups of four x a row */
    const size_t total = (size_t)B.nz * B.ny * nq;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int q = (int)(i % nq), y = B.y0 + (int)((i / nq) % B.ny), z = B.z0 + (int)(i / ((size_t)nq * B.ny));
        const int xa = B.x0 + 4 * q, n = min(4, B.x0 + B.nx - xa);
        const size_t k = ((size_t)(z - zoff) * W + y) * W + xa;
        uint8_t *o = dsh + ((size_t)(oz + z) * shard + (oy + y)) * shard + (ox + xa);
        unsigned v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            v[j] = 0u;
            if (j < n) {
                const bool on = MASK ? (__ldg(bits + ((k + j) >> 5)) >> ((k + j) & 31)) & 1u : (int)__ldg(ct + k + j) >= iso;
                if (on) v[j] = prob255(logit_at<LT>(lg, k + j));
            }
        }
        if (n == 4 && !((size_t)o & 3)) *(uint32_t *)o = v[0] | (v[1] << 8) | (v[2] << 16) | (v[3] << 24);
        else for (int j = 0; j < n; j++) o[j] = (uint8_t)v[j];
    }
}
__global__ void __launch_bounds__(256) pred_out_k(const void *lg, int h16, const uint8_t *__restrict__ ct, size_t n, uint8_t *__restrict__ out) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __ldg(ct + i) ? (uint8_t)prob255(h16 ? logit_at<__half>((const __half *)lg, i) : logit_at<float>((const float *)lg, i)) : (uint8_t)0;
}
/* one 32-voxel word a thread: two 16-byte loads where the bytes are there and aligned, byte compares four at a time */
__global__ void __launch_bounds__(256) ctmask_k(const uint8_t *__restrict__ ct, size_t n, uint32_t *__restrict__ bits, int t) {
    const size_t w = blockIdx.x * (size_t)blockDim.x + threadIdx.x, i0 = w * 32;
    if (i0 >= n) return;
    uint32_t m = 0;
    if (t > 255) { bits[w] = 0u; return; }
    if (i0 + 32 <= n && !((size_t)(ct + i0) & 15)) {
        const uint4 u0 = __ldg((const uint4 *)(ct + i0)), u1 = __ldg((const uint4 *)(ct + i0) + 1);
        const uint32_t v[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w}, tt = (uint32_t)t * 0x01010101u;
#pragma unroll
        for (int j = 0; j < 8; j++) m |= ((((__vcmpgeu4(v[j], tt) & 0x01010101u) * 0x01020408u) >> 24) & 15u) << (4 * j);
    } else {
        const int cnt = (int)min((size_t)32, n - i0);
        for (int j = 0; j < cnt; j++) m |= (uint32_t)((int)__ldg(ct + i0 + j) >= t) << j;
    }
    bits[w] = m;
}

/* ---- seam feather (the blend of src/predict.c:282-333, which the reference runs on host threads over downloaded windows) ----
   Windows lie on a grid with interior S per axis; each window's prediction E covers its interior and B voxels of its upper halo per axis
   (E = S + B).  The output over the interior is E itself except in the lower shell (a coordinate below B), where the upper spills of the
   windows before it are blended in: the window shifted back by delta in {0, 1}^3 (bit 0 x, 1 y, 2 z) has the weight
   prod_axis (delta ? 1 - u(v) : u(v)), u(j) = sin^2(pi / 2 (j + 0.5) / B) for v < B (1 / 0 above), normalised over the windows present.
   A neighbour's spill is its z slab [B][E][E] when it lies a window back in z, else its y slab [S][B][E] when back in y, else its x slab
   [S][S][B] (fe_val).  fp32 products and sums in the reference's order, without contraction. */
struct FeatherArgs { int S, B, E, osh; int oo[3], on[3]; const uint8_t *e; const uint8_t *nb[8]; const float *u; uint8_t *out; };
__device__ __forceinline__ float fe_val(const FeatherArgs &f, int d, int z, int y, int x) {
    if (!d) return (float)__ldg(f.e + ((size_t)z * f.E + y) * f.E + x);
    const uint8_t *p = f.nb[d];
    const int uz = z + ((d & 4) ? f.S : 0), uy = y + ((d & 2) ? f.S : 0), ux = x + ((d & 1) ? f.S : 0);
    if (uz >= f.S) return (float)__ldg(p + ((size_t)(uz - f.S) * f.E + uy) * f.E + ux);
    if (uy >= f.S) return (float)__ldg(p + ((size_t)uz * f.B + (uy - f.S)) * f.E + ux);
    return (float)__ldg(p + ((size_t)uz * f.S + uy) * f.B + (ux - f.S));
}
__global__ void __launch_bounds__(256) feather_k(const FeatherArgs f) {
    const size_t total = (size_t)f.on[0] * f.on[1] * f.on[2];
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int lx = (int)(i % f.on[2]), ly = (int)((i / f.on[2]) % f.on[1]), lz = (int)(i / ((size_t)f.on[2] * f.on[1]));
        const int z = f.oo[0] + lz, y = f.oo[1] + ly, x = f.oo[2] + lx, B = f.B;
        unsigned v;
        if (z >= B && y >= B && x >= B) v = __ldg(f.e + ((size_t)z * f.E + y) * f.E + x);
        else {
            float s = 0.f, w = 0.f;
            for (int d = 0; d < 8; d++) {
                if (d && !f.nb[d]) continue;
                const int dz = d >> 2 & 1, dy = d >> 1 & 1, dx = d & 1;
                if ((dz && z >= B) || (dy && y >= B) || (dx && x >= B)) continue;
                const float wi = __fmul_rn(__fmul_rn(z < B ? __ldg(f.u + dz * B + z) : 1.f, y < B ? __ldg(f.u + dy * B + y) : 1.f), x < B ? __ldg(f.u + dx * B + x) : 1.f);
                s = __fadd_rn(s, __fmul_rn(wi, fe_val(f, d, z, y, x)));
                w = __fadd_rn(w, wi);
            }
            v = w > 0.f ? (unsigned)fminf(255.f, __fadd_rn(__fdiv_rn(s, w), 0.5f)) : 0u;
        }
        f.out[((size_t)lz * f.osh + ly) * f.osh + lx] = (uint8_t)v;
    }
}
/* a window's upper slabs, kept for the windows after it (feather_keep, src/predict.c:362-376) */
__global__ void __launch_bounds__(256) feather_keep_k(const uint8_t *__restrict__ e, int S, int B, uint8_t *__restrict__ zs, uint8_t *__restrict__ ys, uint8_t *__restrict__ xs) {
    const int E = S + B;
    const size_t nz = (size_t)B * E * E, ny = (size_t)S * B * E, nx = (size_t)S * S * B;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nz + ny + nx; i += (size_t)gridDim.x * blockDim.x) {
        if (i < nz) zs[i] = e[(size_t)S * E * E + i];
        else if (i < nz + ny) { const size_t k = i - nz; const int x = (int)(k % E), y = (int)((k / E) % B), z = (int)(k / ((size_t)E * B)); ys[k] = e[((size_t)z * E + S + y) * E + x]; }
        else { const size_t k = i - nz - ny; const int x = (int)(k % B), y = (int)((k / B) % S), z = (int)(k / ((size_t)B * S)); xs[k] = e[((size_t)z * E + y) * E + S + x]; }
    }
}

int g_logits_h16[16], g_iso[16];
int cur_dev() { int d = 0; cudaGetDevice(&d); return d & 15; }
unsigned grid_of(size_t n) { const size_t g = (n + 255) / 256; return (unsigned)(g < 1 ? 1 : g > 148 * 32 ? 148 * 32 : g); }

template <int MASK>
void place(const char *fn, const void *lg, const uint8_t *ct, const uint32_t *bits, PlaceBox B, int W, int zoff, int oz, int oy, int ox, int shard, uint8_t *dsh) {
    if (!umx_ready(fn)) return;
    const size_t n = (size_t)B.nz * B.ny * ((B.nx + 3) >> 2);
    if (!n) return;
    const int d = cur_dev(), iso = g_iso[d] < 1 ? 1 : g_iso[d];
    if (g_logits_h16[d]) umx_launch(pred_place_k<__half, MASK>, dim3(grid_of(n)), dim3(256), 0, (const __half *)lg, ct, bits, B, W, zoff, oz, oy, ox, shard, dsh, iso);
    else umx_launch(pred_place_k<float, MASK>, dim3(grid_of(n)), dim3(256), 0, (const float *)lg, ct, bits, B, W, zoff, oz, oy, ox, shard, dsh, iso);
    g_umx_launches++;
    UMX_CK(fn);
}

}   // namespace

/* src/nn.h:385: the prediction readers take fp16 logits (per device, as the reference's flag is per process with one device a thread) */
extern "C" void nn_set_logits_h16(int on) { g_logits_h16[cur_dev()] = on != 0; }
/* src/nn_elem.cu:1104-1106: outputs only where CT >= t (1: CT > 0) */
extern "C" void nn_set_pred_iso(int t) { g_iso[cur_dev()] = t < 1 ? 1 : t; }
extern "C" int nn_get_pred_iso(void) { const int v = g_iso[cur_dev()]; return v < 1 ? 1 : v; }
/* src/nn_elem.cu:1098-1103: every voxel of a window, no crop; material where CT != 0 */
extern "C" void nn_pred_output(const float *lg, const uint8_t *ct, size_t n, uint8_t *out) {
    if (!umx_ready("nn_pred_output") || !n) return;
    umx_launch(pred_out_k, dim3(grid_of(n)), dim3(256), 0, (const void *)lg, g_logits_h16[cur_dev()], ct, n, out);
    g_umx_launches++;
    UMX_CK("nn_pred_output");
}
/* src/nn_elem.cu:1125-1132 */
extern "C" void nn_pred_place_d(const float *lg, const uint8_t *ct, int D, int W, int hz, int halo, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh) {
    place<0>("nn_pred_place_d", lg, ct, nullptr, place_box_of(D, W, hz, halo, oz, oy, ox, ez, ey, ex), W, 0, oz, oy, ox, shard, dsh);
}
extern "C" void nn_pred_place(const float *lg, const uint8_t *ct, int W, int halo, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh) {
    nn_pred_place_d(lg, ct, W, W, halo, halo, oz, oy, ox, ez, ey, ex, shard, dsh);
}
/* src/nn_elem.cu:1133-1144: the CT window's material voxels as bits (word k >> 5, bit k & 31) */
extern "C" void nn_pred_ctmask_t(const uint8_t *ct, size_t n, uint32_t *bits, int t) {
    if (!umx_ready("nn_pred_ctmask") || !n) return;
    const size_t words = (n + 31) / 32;
    ctmask_k<<<(unsigned)((words + 255) / 256), 256>>>(ct, n, bits, t < 1 ? 1 : t > 255 ? 256 : t);
    g_umx_launches++;
    UMX_CK("nn_pred_ctmask");
}
extern "C" void nn_pred_ctmask(const uint8_t *ct, size_t n, uint32_t *bits) { nn_pred_ctmask_t(ct, n, bits, 1); }
/* src/nn_elem.cu:1145-1160: the same place with the mask bits */
extern "C" void nn_pred_place_m_d(const float *lg, const uint32_t *bits, int D, int W, int hz, int halo, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh) {
    place<1>("nn_pred_place_m_d", lg, nullptr, bits, place_box_of(D, W, hz, halo, oz, oy, ox, ez, ey, ex), W, 0, oz, oy, ox, shard, dsh);
}
extern "C" void nn_pred_place_m(const float *lg, const uint32_t *bits, int W, int halo, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh) {
    nn_pred_place_m_d(lg, bits, W, W, halo, halo, oz, oy, ox, ez, ey, ex, shard, dsh);
}
/* src/nn_elem.cu:1161-1178: a window held as planes [zoff, zoff + D) (one half of a split window): its planes [zlo, zhi) that lie in the interior */
extern "C" void nn_pred_place_mz(const float *lg, const uint32_t *bits, int W, int halo, int zlo, int zhi, int zoff, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh) {
    if (zlo < halo) zlo = halo;
    if (zhi > W - halo) zhi = W - halo;
    if (zhi <= zlo) return;
    PlaceBox B = place_box_of(W, W, halo, halo, oz, oy, ox, ez, ey, ex);
    const int z0 = B.z0 > zlo ? B.z0 : zlo, z1 = B.z0 + B.nz < zhi ? B.z0 + B.nz : zhi;
    B.z0 = z0; B.nz = z1 > z0 ? z1 - z0 : 0;
    place<1>("nn_pred_place_mz", lg, nullptr, bits, B, W, zoff, oz, oy, ox, shard, dsh);
}

/* The seam feather's blend on the device (the arithmetic of fe_blend / fe_rows, src/predict.c:305-333): f->e, f->nb[1..7] (NULL: no such
   window), f->out are device pointers; the interior voxels [oo, oo + on) per axis of this window go to out[(lz osh + ly) osh + lx].
   The weight table of a band width is built on the host (double sin, as feather_init) and kept on the device. */
extern "C" int umx_feather_blend(const umx_feather_t *h) {
    if (!umx_ready("umx_feather_blend")) return -1;
    if (!h || h->S < 1 || h->B < 1 || h->B > 1024 || h->B > h->S || !h->e || !h->out) { umx_latch_msg("umx_feather_blend: bad arguments"); return -1; }
    for (int d = 0; d < 3; d++) if (h->oo[d] < 0 || h->on[d] < 0 || h->oo[d] + h->on[d] > h->S || h->on[d] > h->osh) { umx_latch_msg("umx_feather_blend: output box outside the interior or the shard"); return -1; }
    static float *utab[16]; static int ub[16];
    const int dv = cur_dev();
    if (!utab[dv] || ub[dv] != h->B) {
        float hu[2048];
        for (int j = 0; j < h->B; j++) { const double s = sin(3.14159265358979323846 / 2 * (j + 0.5) / h->B); hu[j] = (float)(s * s); hu[h->B + j] = (float)(1 - s * s); }
        cudaDeviceSynchronize();
        if (!utab[dv]) utab[dv] = (float *)nn_malloc(2048 * sizeof(float));
        if (!utab[dv]) return -1;
        nn_h2d(utab[dv], hu, (size_t)2 * h->B * sizeof(float));
        ub[dv] = h->B;
    }
    FeatherArgs f; memset(&f, 0, sizeof f);
    f.S = h->S; f.B = h->B; f.E = h->S + h->B; f.osh = h->osh; f.e = h->e; f.u = utab[dv]; f.out = h->out;
    for (int d = 0; d < 3; d++) { f.oo[d] = h->oo[d]; f.on[d] = h->on[d]; }
    for (int d = 1; d < 8; d++) f.nb[d] = h->nb[d];
    const size_t n = (size_t)f.on[0] * f.on[1] * f.on[2];
    if (!n) return 0;
    feather_k<<<grid_of(n), 256>>>(f);
    g_umx_launches++;
    UMX_CK("umx_feather_blend");
    return 0;
}
extern "C" void umx_feather_keep(const uint8_t *e, int S, int B, uint8_t *zslab, uint8_t *yslab, uint8_t *xslab) {
    if (!umx_ready("umx_feather_keep") || S < 1 || B < 1) return;
    const int E = S + B;
    feather_keep_k<<<grid_of((size_t)B * E * E + (size_t)S * B * E + (size_t)S * S * B), 256>>>(e, S, B, zslab, yslab, xslab);
    g_umx_launches++;
    UMX_CK("umx_feather_keep");
}
