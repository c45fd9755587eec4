/* MX block-scaled implicit-GEMM 3-D convolution forward on the sm_100a tensor cores (tcgen05, TMEM accumulators, TMA staging).

   GEMM view.  M = 128 output voxels of one tile (8 along x by 16 along y of one z plane), N = up to 128 output channels,
   K = taps x input channels in steps of one MX block pair: 32 E4M3 bytes (kind::mxf8f6f4, one UE8M0 scale per row) or 64 E2M1
   nibbles (kind::mxf4, two scales per row) per tcgen05.mma.  The activation tensor is the reference's channel-blocked MX
   storage (src/lp_common.cuh:100-106), so one voxel's K step is 32 contiguous bytes (fp8) or two 16-byte rows of adjacent
   blocks (fp4).

   Operand staging.  A 3^3 conv loads, per (input block, dz), one halo plane of 18 x 10 voxels with TMA (out-of-range voxels are
   zero-filled: that is the padding) as two 16-byte-wide planes [k half][y][x][16 B].  In that layout the canonical K-major
   no-swizzle UMMA operand (8 rows x 16 B core matrices; stride 160 B between the 16 y groups, 2880 B between the K halves) of
   every (dy, dx) tap is the same tile at a start address shifted by (dy * 10 + dx) * 16 bytes (the fp8 planes sit 2944 B apart so
   that each TMA destination is 128-byte aligned), so nine MMAs reuse one load.
   Weights are prepared once into the exact shared-memory image of a stage ([tap][k half][row][16 B] + scale bytes in the
   TMEM scale layout) and arrive with one bulk copy.  1^3 convs (head, the 2^3 stride-2 down conv on a space-to-depth copy, the
   transposed conv as a GEMM to 8 Cout columns) run the same pipeline with one tap and four K items a stage.

   Scale factors.  tcgen05 block-scaled MMAs read scales from TMEM: row r of a 128-row operand at lane r % 32, column r / 32,
   byte = scale id.  The scale of an A row depends on the tap (it is the shifted voxel's), so four epilogue warps gather, per
   stage, the nine shifted scale sets from the scale plane into that layout in shared memory, and the MMA thread copies them to
   TMEM with tcgen05.cp before issuing the stage's MMAs.  Out-of-range voxels get scale 1 (their codes are zero).

   Roles (192 threads): warp 0 lane 0 = TMA producer; warp 1 = TMEM allocation, lane 0 = MMA issue; warps 2-5 = scale gather,
   then the epilogue (tcgen05.ld of 32 channels per voxel = one MX block per thread: bias, fp16 store or MX requantisation;
   InstanceNorm partial sums are taken by a separate pass over the stored output).  Every wait is bounded; a wait that gives up records (code, block, stage) in a device
   flag, raises a block-wide abort flag and the block tears down normally. */
#include "conv_epi.cuh"
#include "tc_ptx.cuh"
#include <stdlib.h>
#include <string.h>

namespace {

constexpr int kThreads = 192;
constexpr int kTmemCols = 256;
constexpr int kSfBase = 128;        /* TMEM columns: [0, 128) accumulators, then two scale buffers of 40 (A 20 | B 20) */
constexpr long long kWaitLimit = 4000000000ll;   /* clock cycles (about two seconds) */

struct ConvArgs {
    int N, D, H, W;                 /* the grid of GEMM rows */
    int nkb;                        /* 32-channel blocks of the activation tensor */
    int nki;                        /* K items per tap: nkb (fp8) or ceil(nkb / 2) (fp4) */
    int taps, bits;
    int cop, nt, ntiles_n;          /* GEMM columns (padded to 32), column tile, column tiles */
    int tiles_x, tiles_y;
    int ring;                       /* pipeline depth */
    int stage_bytes, offW, offSFB, offA, offSFA;
    int w_stage_bytes, nst;         /* packed weight bytes per stage, stages per column tile */
    int items_max, ipq, nquad;      /* K items per stage, items per scale quad (4 fp8 / 2 fp4), quads per stage */
    const uint8_t *x_sc;
    const uint8_t *wpk;
    /* K split: ksplit blocks share one output tile, each takes a contiguous range of the stages and leaves its fp32 accumulators in
       ks_part [tile][split][32-column chunk][column quad][row][4] (a warp's 32 rows of one quad are 512 contiguous bytes); the block that draws the tile's last ticket adds the parts in split order and
       runs the epilogue (no block waits for another; the order of the additions is fixed) */
    int ksplit; float *ks_part; unsigned *ks_tickets;
    /* 3^3 stride-2 pad-1 conv: K item = (tap, input block), each item's A tile is its own strided TMA load from the input grid Di x Hi x Wi */
    int s2, nbi, nit, Di, Hi, Wi;       /* stride-2 conv: blocks of the input tensor, K items per tap, input grid */
    EpiArgs e;
    int *err;
};

__device__ unsigned g_ks_tickets[8192];      /* one per output tile of a split launch; the last block of a tile resets it */


__device__ __forceinline__ void raise(const ConvArgs &a, volatile int *abort_flag, int code, int stage) {
    if (atomicCAS(a.err, 0, code) == 0) { a.err[1] = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)); a.err[2] = stage; a.err[3] = (int)threadIdx.x; }
    *abort_flag = 1;
    __threadfence_block();
}

template <int BITS>
__global__ void __launch_bounds__(kThreads) conv_mx_k(const __grid_constant__ CUtensorMap map0, const ConvArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    /* control block, then the stage ring at the next 1024-byte boundary */
    uint64_t *bars = (uint64_t *)smem_raw;                       /* [0, ring) tma full, [ring, 2 ring) scale full, [2 ring, 3 ring) empty, 3 ring: accumulator full */
    uint32_t *tmem_slot = (uint32_t *)(smem_raw + 256);
    volatile int *abort_flag = (volatile int *)(smem_raw + 260);
    uint8_t *stages = smem_raw + 1024;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = a.ring;
    const uint32_t bar_tma = smem_u32(bars), bar_sf = bar_tma + 8 * R, bar_empty = bar_tma + 16 * R, bar_acc = bar_tma + 24 * R, bar_red = bar_acc + 8;

    const int txy = blockIdx.x, tx = txy % a.tiles_x, ty = txy / a.tiles_x;
    const int z = blockIdx.y;
    const int sp = (int)blockIdx.z % a.ksplit, bz = (int)blockIdx.z / a.ksplit;
    const int n = bz / a.ntiles_n, ntile = bz % a.ntiles_n;
    const int x0 = tx * 8, y0 = ty * 16;
    const int n0 = ntile * a.nt, n_cur = min(a.nt, a.cop - n0);
    /* this block's stages: all of them, or its share (whole input items of a 3^3 conv, so that every share has a live stage) */
    int st_lo = 0, st_hi = a.nst;
    if (a.ksplit > 1) {
        if (a.taps == 27) { st_lo = 3 * (a.nki * sp / a.ksplit); st_hi = 3 * (a.nki * (sp + 1) / a.ksplit); }
        else { st_lo = a.nst * sp / a.ksplit; st_hi = a.nst * (sp + 1) / a.ksplit; }
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < R; i++) { mbar_init(bar_tma + 8 * i, 1); mbar_init(bar_sf + 8 * i, 128); mbar_init(bar_empty + 8 * i, 1); }
        mbar_init(bar_acc, 1); mbar_init(bar_red, 128); mbar_init(bar_red + 8, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    pdl_trigger();
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();                                  /* from here on the block touches activations */
    const uint32_t tmem = *tmem_slot;

    /* a stage is live unless it is a 3^3 stage whose input plane lies outside the volume (it would add zeros) */
    auto stage_live = [&](int st) -> bool { if (a.taps != 27) return true; const int zi = z + st % 3 - 1; return zi >= 0 && zi < a.D; };
    auto stage_items = [&](int st) -> int { return a.taps == 27 ? 9 : min(4, a.nki - 4 * st); };

    if (warp == 0) {
        /* ---------------- TMA producer ---------------- */
        if (lane == 0) {
            tma_prefetch_desc(&map0);
            int it = 0;
            const uint8_t *wbase = a.wpk + (size_t)ntile * a.nst * a.w_stage_bytes;
            for (int st = st_lo; st < st_hi; st++) {
                if (!stage_live(st)) continue;
                const int s = it % R, ph = (it / R) & 1;
                if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, kWaitLimit)) { raise(a, abort_flag, 1, st); break; }
                uint8_t *sb = stages + (size_t)s * a.stage_bytes;
                const uint32_t bar = bar_tma + 8 * s;
                const int items = stage_items(st);
                const int abytes = a.taps == 27 ? 5760 : items * 4096;
                mbar_expect_tx(bar, (uint32_t)(abytes + a.w_stage_bytes));
                bulk_g2s(smem_u32(sb + a.offW), wbase + (size_t)st * a.w_stage_bytes, (uint32_t)a.w_stage_bytes, bar);
                /* two 16-byte-wide planes per K item (fp8: the halves of block ki; fp4: blocks 2 ki and 2 ki + 1) */
                if (a.taps == 27) {
                    const int ki = st / 3, zi = z + st % 3 - 1;
                    tma_load_4d(smem_u32(sb + a.offA), &map0, bar, (x0 - 1) * 16, y0 - 1, zi, BITS == 8 ? (n * a.nkb + ki) * 2 : n * a.nkb + 2 * ki);
                } else {
                    for (int j = 0; j < items; j++) {
                        const int ki = 4 * st + j;
                        if (a.s2) {   /* every second voxel of the input, starting at 2 v + tap - 1 (voxels outside the grid arrive as zeros: the padding) */
                            /* K item ki = tap * a.nit + i: fp8: block i (its two half planes); fp4: blocks 2 i and 2 i + 1 (the second may lie past the
                               sample's last block: its weights are zero and its scale is read as 1) */
                            const int tap = ki / a.nit, blk = ki - tap * a.nit;
                            tma_load_5d(smem_u32(sb + a.offA + j * 4096), &map0, bar, 0, 2 * x0 + tap % 3 - 1, 2 * y0 + (tap / 3) % 3 - 1, 2 * z + tap / 9 - 1, BITS == 8 ? (n * a.nbi + blk) * 2 : n * a.nbi + 2 * blk);
                        } else
                        tma_load_4d(smem_u32(sb + a.offA + j * 4096), &map0, bar, x0 * 16, y0, z, BITS == 8 ? (n * a.nkb + ki) * 2 : n * a.nkb + 2 * ki);
                    }
                }
                it++;
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issue: one thread; everything that does not change with the stage is worked out before the loop ---------------- */
        if (lane == 0) {
            int it = 0, s = 0, ph = 0; bool ok = true;
            const uint32_t sb0 = smem_u32(stages), sstep = (uint32_t)a.stage_bytes >> 4;
            const uint32_t sf_hi = desc_hi(128), b_hi = desc_hi(128), a_hi = a.taps == 27 ? desc_hi(160) : desc_hi(128);
            const uint32_t sfa_lo0 = desc_lo(sb0 + a.offSFA, 0), sfb_lo0 = desc_lo(sb0 + a.offSFB, 0);
            const uint32_t a_lo0 = desc_lo(sb0 + a.offA, a.taps == 27 ? 2880 : 2048), b_lo0 = desc_lo(sb0 + a.offW, (uint32_t)a.nt * 16);
            const uint32_t idesc0 = BITS == 8 ? idesc_mxf8(n_cur, 0, 0) : idesc_mxf4(n_cur, 0, 0);
            const uint32_t bstep = (uint32_t)a.nt * 2;
            for (int st = st_lo; st < st_hi && ok; st++) {
                if (!stage_live(st)) continue;
                if (!mbar_wait(bar_sf + 8 * s, ph, abort_flag, kWaitLimit)) { raise(a, abort_flag, 3, st); ok = false; break; }
                if (!mbar_wait(bar_tma + 8 * s, ph, abort_flag, kWaitLimit)) { raise(a, abort_flag, 2, st); ok = false; break; }
                tc_fence_after();
                const uint32_t so = (uint32_t)s * sstep;
                const uint32_t sfa_t = tmem + kSfBase + (it & 1) * 40, sfb_t = sfa_t + 20;
                if (a.taps == 27) {
                    constexpr int NQ = BITS == 8 ? 3 : 5;
#pragma unroll
                    for (int q = 0; q < NQ; q++) {
                        utccp_32x128b(sfa_t + 4 * q, desc_make(sfa_lo0 + so + 32u * q, sf_hi));
                        utccp_32x128b(sfb_t + 4 * q, desc_make(sfb_lo0 + so + 32u * q, sf_hi));
                    }
                    issue_items<BITS, 9, true>(tmem, a_lo0 + so, a_hi, b_lo0 + so, b_hi, bstep, 0, idesc0, sfa_t, sfb_t, it == 0, 9);
                } else {
                    const int items = stage_items(st), nq = (items + a.ipq - 1) / a.ipq;
                    for (int q = 0; q < nq; q++) {
                        utccp_32x128b(sfa_t + 4 * q, desc_make(sfa_lo0 + so + 32u * q, sf_hi));
                        utccp_32x128b(sfb_t + 4 * q, desc_make(sfb_lo0 + so + 32u * q, sf_hi));
                    }
                    issue_items<BITS, 4, false>(tmem, a_lo0 + so, a_hi, b_lo0 + so, b_hi, bstep, 256, idesc0, sfa_t, sfb_t, it == 0, items);
                }
                umma_commit(bar_empty + 8 * s);
                it++; if (++s == R) { s = 0; ph ^= 1; }
            }
            umma_commit(bar_acc);   /* also after a give-up: the epilogue must not wait for its full limit */
        }
    } else {
        /* ---------------- scale gather, then epilogue ---------------- */
        const int q4 = warp & 3, r = q4 * 32 + lane;             /* TMEM lane quarter of this warp; GEMM row of this thread */
        const int ry = r >> 3, rx = r & 7;
        const int oy = y0 + ry, ox = x0 + rx;
        const bool row_ok = oy < a.H && ox < a.W;
        const size_t S = (size_t)a.D * a.H * a.W;
        int it = 0; bool ok = true;
        for (int st = st_lo; st < st_hi && ok; st++) {
            if (!stage_live(st)) continue;
            const int s = it % R, ph = (it / R) & 1;
            if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, kWaitLimit)) { raise(a, abort_flag, 4, st); ok = false; break; }
            uint32_t *sfa = (uint32_t *)(stages + (size_t)s * a.stage_bytes + a.offSFA);
            const int items = stage_items(st);
            uint32_t wq[5] = {0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu};
            if (a.taps == 27) {
                const int ki = st / 3, zi = z + st % 3 - 1;
#pragma unroll
                for (int j = 0; j < 9; j++) {
                    const int iy = oy + j / 3 - 1, ix = ox + j % 3 - 1;
                    const bool in = iy >= 0 && iy < a.H && ix >= 0 && ix < a.W;
                    const size_t vox = ((size_t)zi * a.H + iy) * a.W + ix;
                    if (BITS == 8) {
                        const unsigned b = in ? a.x_sc[((size_t)n * a.nkb + ki) * S + vox] : 127u;
                        wq[j >> 2] = (wq[j >> 2] & ~(0xffu << (8 * (j & 3)))) | (b << (8 * (j & 3)));
                    } else {
                        const unsigned b0 = in ? a.x_sc[((size_t)n * a.nkb + 2 * ki) * S + vox] : 127u;
                        const unsigned b1 = (in && 2 * ki + 1 < a.nkb) ? a.x_sc[((size_t)n * a.nkb + 2 * ki + 1) * S + vox] : 127u;
                        const unsigned h = b0 | (b1 << 8);
                        wq[j >> 1] = (wq[j >> 1] & ~(0xffffu << (16 * (j & 1)))) | (h << (16 * (j & 1)));
                    }
                }
            } else {
                const size_t vox = ((size_t)z * a.H + oy) * a.W + ox;
                for (int j = 0; j < items; j++) {
                    const int ki = 4 * st + j;
                    if (a.s2) {
                        const int tap = ki / a.nit, blk = ki - tap * a.nit;
                        const int iz = 2 * z + tap / 9 - 1, iy = 2 * oy + (tap / 3) % 3 - 1, ix = 2 * ox + tap % 3 - 1;
                        const bool in = row_ok && iz >= 0 && iz < a.Di && iy >= 0 && iy < a.Hi && ix >= 0 && ix < a.Wi;
                        const size_t Si = (size_t)a.Di * a.Hi * a.Wi, vi = ((size_t)iz * a.Hi + iy) * a.Wi + ix;
                        if (BITS == 8) {
                            const unsigned b = in ? a.x_sc[((size_t)n * a.nbi + blk) * Si + vi] : 127u;
                            wq[j >> 2] = (wq[j >> 2] & ~(0xffu << (8 * (j & 3)))) | (b << (8 * (j & 3)));
                        } else {
                            const unsigned b0 = in ? a.x_sc[((size_t)n * a.nbi + 2 * blk) * Si + vi] : 127u;
                            const unsigned b1 = (in && 2 * blk + 1 < a.nbi) ? a.x_sc[((size_t)n * a.nbi + 2 * blk + 1) * Si + vi] : 127u;
                            const unsigned h = b0 | (b1 << 8);
                            wq[j >> 1] = (wq[j >> 1] & ~(0xffffu << (16 * (j & 1)))) | (h << (16 * (j & 1)));
                        }
                    } else if (BITS == 8) {
                        const unsigned b = row_ok ? a.x_sc[((size_t)n * a.nkb + ki) * S + vox] : 127u;
                        wq[j >> 2] = (wq[j >> 2] & ~(0xffu << (8 * (j & 3)))) | (b << (8 * (j & 3)));
                    } else {
                        const unsigned b0 = row_ok ? a.x_sc[((size_t)n * a.nkb + 2 * ki) * S + vox] : 127u;
                        const unsigned b1 = (row_ok && 2 * ki + 1 < a.nkb) ? a.x_sc[((size_t)n * a.nkb + 2 * ki + 1) * S + vox] : 127u;
                        const unsigned h = b0 | (b1 << 8);
                        wq[j >> 1] = (wq[j >> 1] & ~(0xffffu << (16 * (j & 1)))) | (h << (16 * (j & 1)));
                    }
                }
            }
            /* quad q: word (lane, column) = row 32 * column + lane -> this thread's word is at lane * 4 + quarter */
#pragma unroll
            for (int q = 0; q < 5; q++) if (q < a.nquad) sfa[q * 128 + lane * 4 + q4] = wq[q];
            fence_proxy_async();
            mbar_arrive(bar_sf + 8 * s);
            it++;
        }
        /* ---- epilogue ---- */
        if (!mbar_wait(bar_acc, 0, abort_flag, kWaitLimit)) raise(a, abort_flag, 5, 0);
        tc_fence_after();
        const int nchunk = n_cur >> 5;
        if (!*abort_flag && a.ksplit > 1) {
            const size_t tile_id = ((size_t)bz * a.D + z) * gridDim.x + txy;
            const size_t tile_f = (size_t)(a.nt >> 5) * 4096;                    /* floats of one part */
            float *mine = a.ks_part + (tile_id * a.ksplit + sp) * tile_f + (size_t)r * 4;
            for (int jc = 0; jc < nchunk; jc++) {
                uint32_t rr[32];
                tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(jc * 32), rr);
                tmem_ld_wait();
#pragma unroll
                for (int k = 0; k < 8; k++) __stcg((uint4 *)(mine + (size_t)jc * 4096 + k * 512), make_uint4(rr[4 * k], rr[4 * k + 1], rr[4 * k + 2], rr[4 * k + 3]));
            }
            __threadfence();
            volatile unsigned *last_s = (volatile unsigned *)(smem_raw + 264);
            bool dead = false; uint32_t red_ph = 0;
            /* the 128 epilogue threads meet on an mbarrier (a bounded wait) */
            auto esync = [&]() { mbar_arrive(bar_red); if (!mbar_wait(bar_red, red_ph, abort_flag, kWaitLimit)) { raise(a, abort_flag, 6, 0); dead = true; } red_ph ^= 1u; };
            esync();
            if (r == 0) { const unsigned tk = atomicAdd(&a.ks_tickets[tile_id], 1u); const unsigned l = tk == (unsigned)a.ksplit - 1u; if (l) a.ks_tickets[tile_id] = 0u; *last_s = l; }
            esync();
            if (!dead && *last_s) {
                /* the parts of one 32-column chunk (16 KB per split) come into the now idle stage ring with bulk copies, the next chunk's
                   while this one goes through the epilogue: summing straight from global memory is a chain of L2 round trips */
                __threadfence();
                asm volatile("fence.proxy.async;" ::: "memory");
                const uint32_t bar_ld = bar_red + 8;
                const float *tile0 = a.ks_part + tile_id * a.ksplit * tile_f;
                auto fetch = [&](int jc) {
                    if (r == 0) {
                        mbar_expect_tx(bar_ld, (uint32_t)a.ksplit * 16384u);
                        for (int s2 = 0; s2 < a.ksplit; s2++) bulk_g2s(smem_u32(stages + (size_t)s2 * 16384), tile0 + (size_t)s2 * tile_f + (size_t)jc * 4096, 16384u, bar_ld);
                    }
                };
                fetch(0);
                for (int jc = 0; jc < nchunk && !dead; jc++) {
                    if (!mbar_wait(bar_ld, (uint32_t)(jc & 1), abort_flag, kWaitLimit)) { raise(a, abort_flag, 7, jc); break; }
                    float v[32];
                    const float *p0 = (const float *)stages + (size_t)r * 4;
#pragma unroll
                    for (int k = 0; k < 8; k++) { const float4 t = *(const float4 *)(p0 + k * 512); v[4 * k] = t.x; v[4 * k + 1] = t.y; v[4 * k + 2] = t.z; v[4 * k + 3] = t.w; }
                    for (int s2 = 1; s2 < a.ksplit; s2++) {
                        const float *ps = p0 + (size_t)s2 * 4096;
#pragma unroll
                        for (int k = 0; k < 8; k++) { const float4 t = *(const float4 *)(ps + k * 512); v[4 * k] += t.x; v[4 * k + 1] += t.y; v[4 * k + 2] += t.z; v[4 * k + 3] += t.w; }
                    }
                    esync();                                   /* every thread has read the chunk: the ring may take the next one */
                    if (dead) break;
                    if (jc + 1 < nchunk) fetch(jc + 1);
                    epi_chunk(a.e, n, z, oy, ox, row_ok, (n0 >> 5) + jc, v);
                }
            }
        } else if (!*abort_flag) {
            for (int jc = 0; jc < nchunk; jc++) {
                uint32_t rr[32];
                tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(jc * 32), rr);
                tmem_ld_wait();
                float v[32];
#pragma unroll
                for (int k = 0; k < 32; k++) v[k] = __uint_as_float(rr[k]);
                epi_chunk(a.e, n, z, oy, ox, row_ok, (n0 >> 5) + jc, v);
            }
        }
    }
    /* ---------------- teardown ---------------- */
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && warp == 0 && lane == 0) {
        /* after a give-up: let this thread's own copies in flight land (bounded) before the block's shared memory is released */
        for (int s = 0; s < R; s++) { const long long t0 = clock64(); while (!mbar_try(bar_tma + 8 * s, 0) && !mbar_try(bar_tma + 8 * s, 1) && clock64() - t0 < 20000000ll) { } }
    }
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, kTmemCols); }
}

/* ---- weight preparation: fp32 weights -> the shared-memory image of every (column tile, stage): items x [k half][row][16 B]
   codes, then the scale bytes in the TMEM scale layout (quad, lane, column, byte).  One thread per (column tile, stage, item, row).
   Quantisation per (row, tap, 32 input channels) as the reference's prep_w8_k / prep_w4_k (src/lp_f8fwd.cu:54-71,
   src/lp_f4fwd.cu:53-66). ---- */
__global__ void __launch_bounds__(128) prep_w_k(const PrepArgs p) {
    const size_t total = (size_t)p.ntiles_n * p.nst * p.items_max * p.nt;
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i == 0 && p.bias_p) for (int c = 0; c < p.cop; c++) {
        float b = 0.f;
        if (p.bias) { if (p.kind == UMX_TCONV2) { const int o = c % (32 * p.cob_t); b = o < p.co ? p.bias[o] : 0.f; } else b = c < p.co ? p.bias[c] : 0.f; }
        p.bias_p[c] = b;
    }
    if (i >= total) return;
    const int rl = (int)(i % p.nt), j = (int)((i / p.nt) % p.items_max), st = (int)((i / ((size_t)p.nt * p.items_max)) % p.nst), ntile = (int)(i / ((size_t)p.nt * p.items_max * p.nst));
    const int row = ntile * p.nt + rl;
    int tap, ki;
    if (p.taps == 27) { ki = st / 3; tap = (st % 3) * 9 + j; } else { ki = 4 * st + j; tap = 0; }
    uint8_t *stg = p.wpk + ((size_t)ntile * p.nst + st) * p.w_stage_bytes;
    const bool live = row < p.cop && ki < p.nki;
    unsigned w[8]; unsigned sb[2] = {127u, 127u};
    float v[32];
    if (p.bits == 8) {
#pragma unroll
        for (int k = 0; k < 32; k++) v[k] = live ? prep_src(p, row, tap, ki, k) : 0.f;
        sb[0] = mx_encode_row32<8>(v, w);
    } else {
        unsigned w4[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
#pragma unroll
            for (int k = 0; k < 32; k++) v[k] = live ? prep_src(p, row, tap, 2 * ki + h, k) : 0.f;
            sb[h] = mx_encode_row32<4>(v, w4);
#pragma unroll
            for (int t = 0; t < 4; t++) w[4 * h + t] = w4[t];
        }
    }
    if (!live) { sb[0] = 127u; sb[1] = 127u; }
    uint4 *d0 = (uint4 *)(stg + ((size_t)(j * 2 + 0) * p.nt + rl) * 16), *d1 = (uint4 *)(stg + ((size_t)(j * 2 + 1) * p.nt + rl) * 16);
    *d0 = make_uint4(w[0], w[1], w[2], w[3]); *d1 = make_uint4(w[4], w[5], w[6], w[7]);
    uint8_t *sf = stg + (size_t)p.items_max * p.nt * 32;
    const int q = j / p.ipq, l = rl & 31, c = rl >> 5;
    if (p.bits == 8) sf[q * 512 + l * 16 + c * 4 + (j & 3)] = (uint8_t)sb[0];
    else { sf[q * 512 + l * 16 + c * 4 + (j & 1) * 2] = (uint8_t)sb[0]; sf[q * 512 + l * 16 + c * 4 + (j & 1) * 2 + 1] = (uint8_t)sb[1]; }
}

typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_fn get_encode() {
    static encode_fn fn = nullptr;
    if (!fn) {
        void *p = nullptr; cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) { umx_latch_msg("cuTensorMapEncodeTiled is not available from the driver"); return nullptr; }
        fn = (encode_fn)p;
    }
    return fn;
}
int ceil_div(int a, int b) { return (a + b - 1) / b; }

}   // namespace

void umx_conv_ks_tickets_reset(void) { void *p = nullptr; if (cudaGetSymbolAddress(&p, g_ks_tickets) == cudaSuccess && p) cudaMemset(p, 0, sizeof(unsigned) * 8192); }
int umx_conv_r_fits(const umx_conv *c);
uint8_t *umx_conv_r_prepare(const umx_conv *c, const float *w_dev);
int umx_conv_fwd_r(const umx_conv *c, const void *x, const CUtensorMap *m0, void *enc, int N, int D, int H, int W, const EpiArgs &e,
                   double *part, const float *gamma, const float *beta, float eps, float *coef);
extern "C" void umx_in_stats_coef(const void *y, int N, int C, int D, int H, int W, const float *gamma, const float *beta, float eps, double *part, float *coef);
void umx_in_part(const void *y, int N, int C, int D, int H, int W, double *part);
uint8_t *umx_conv_p_prepare(const umx_conv *c, const float *w_dev);
uint8_t *umx_conv_stem_prepare(const umx_conv *c, const float *w_dev);
int umx_conv_fwd_stem(const umx_conv *c, const void *x, int src8, int N, int D, int H, int W, void *y);
int umx_conv_fwd_p(const umx_conv *c, const void *x, void *enc, int N, int D, int H, int W, const EpiArgs &e);
const uint8_t *umx_prob_table(void);


static umx_conv *conv_build(int kind, const float *w_dev, const float *bias_dev, int co, int ci, int bits) {
    if (!umx_ready("umx_conv_create")) return nullptr;
    if ((bits != 8 && bits != 4) || kind < 0 || kind > 4 || co < 1 || ci < 1 ) { fprintf(stderr, "umx_conv_create: bad arguments (kind %d, co %d, ci %d, bits %d)\n", kind, co, ci, bits); abort(); }
    umx_conv *c = (umx_conv *)calloc(1, sizeof *c);
    c->kind = kind; c->co = co; c->ci = ci; c->bits = bits;
    c->taps = kind == UMX_CONV3 ? 27 : 1;
    const int nbi = ceil_div(ci, 32);
    /* K blocks of the GEMM: (sub-voxel or tap) x input blocks; the MX-fp4 stride-2 conv pads the blocks of a tap to an even count, so that a
       K item of two blocks never spans two taps (two different shifts of the input) */
    c->nkb = kind == UMX_DOWN2 ? 8 * nbi : kind == UMX_CONV3S2 ? 27 * (bits == 4 ? 2 * ceil_div(nbi, 2) : nbi) : nbi;
    c->nki = bits == 8 ? c->nkb : ceil_div(c->nkb, 2);
    c->cob_t = ceil_div(co, 32);
    c->cop = (kind == UMX_TCONV2 ? 8 : 1) * c->cob_t * 32;
    c->nt = c->cop >= 128 ? 128 : c->cop;               /* 32, 64, 96 or 128 */
    c->ntiles_n = ceil_div(c->cop, c->nt);
    c->items_max = c->taps == 27 ? 9 : 4;
    c->ipq = bits == 8 ? 4 : 2;
    c->nquad = ceil_div(c->items_max, c->ipq);
    c->nst = c->taps == 27 ? 3 * c->nki : ceil_div(c->nki, 4);
    c->w_stage_bytes = c->items_max * c->nt * 32 + c->nquad * 512;
    const size_t wb = (size_t)c->ntiles_n * c->nst * c->w_stage_bytes;
    c->wpk = (uint8_t *)nn_malloc(wb); c->bias_p = (float *)nn_malloc((size_t)c->cop * 4);
    if (!c->wpk || !c->bias_p) { umx_conv_free(c); return nullptr; }
    cudaMemset(c->wpk, 127, wb);   /* unused scale slots read as 1 */
    PrepArgs p; memset(&p, 0, sizeof p);
    p.w = w_dev; p.wpk = c->wpk; p.bias = bias_dev; p.bias_p = c->bias_p; p.kind = kind; p.co = co; p.ci = ci; p.bits = bits; p.cop = c->cop; p.cob_t = c->cob_t;
    p.nkb = c->nkb; p.nki = c->nki; p.taps = c->taps; p.nt = c->nt; p.ntiles_n = c->ntiles_n; p.nst = c->nst; p.items_max = c->items_max; p.ipq = c->ipq; p.nquad = c->nquad; p.w_stage_bytes = c->w_stage_bytes;
    const size_t total = (size_t)c->ntiles_n * c->nst * c->items_max * c->nt;
    prep_w_k<<<(unsigned)((total + 127) / 128), 128>>>(p);
    g_umx_launches++;
    c->wr = umx_conv_r_prepare(c, w_dev);
    c->wp = umx_conv_p_prepare(c, w_dev);
    c->wstem = umx_conv_stem_prepare(c, w_dev);
    UMX_CK("umx_conv_create");
    /* the conv kernels read the prepared weights and the bias before their griddepcontrol.wait (they are layer constants that may load while
       the previous kernel still runs), so the preparation kernels must have finished before a conv can be launched behind them */
    cudaStreamSynchronize(0);
    return c;
}
extern "C" umx_conv *umx_conv_create_dev(int kind, const float *w_dev, const float *bias_dev, int co, int ci, int bits) { return conv_build(kind, w_dev, bias_dev, co, ci, bits); }
extern "C" umx_conv *umx_conv_create(int kind, const float *w, const float *bias, int co, int ci, int bits) {
    if (!umx_ready("umx_conv_create")) return nullptr;
    const size_t nw = (size_t)co * ci * ((kind == UMX_CONV3 || kind == UMX_CONV3S2) ? 27 : kind == UMX_CONV1 ? 1 : 8);
    float *wd = (float *)nn_malloc(nw * 4), *bd = bias ? (float *)nn_malloc((size_t)co * 4) : nullptr;
    if (!wd || (bias && !bd)) { nn_free(wd); nn_free(bd); return nullptr; }
    nn_h2d(wd, w, nw * 4); if (bias) nn_h2d(bd, bias, (size_t)co * 4);
    umx_conv *c = conv_build(kind, wd, bd, co, ci, bits);
    cudaDeviceSynchronize();
    nn_free(wd); nn_free(bd);
    return c;
}
extern "C" void umx_conv_free(umx_conv *c) { if (!c) return; nn_free(c->wpk); nn_free(c->bias_p); nn_free(c->wr); nn_free(c->wp); nn_free(c->wstem); free(c); }
int umx_stats_chunks(int D, int H, int W);
/* room for 512 partial sums of two doubles per (sample, channel): the statistics pass uses up to that many voxel chunks, the conv epilogue
   one entry per block */
extern "C" size_t umx_stats_doubles(int N, int co, int D, int H, int W) { (void)D; (void)H; (void)W; return (size_t)N * 512 * (size_t)(ceil_div(co, 32) * 32) * 2; }

static int g_last_kernel = -1;
extern "C" int umx_conv_last_kernel(void) { return g_last_kernel; }
struct NormArgs { const float *gamma, *beta; float eps; float *coef; };
static int conv_fwd_impl(const umx_conv *c, const void *x, int N, int D, int H, int W, void *y, int out_mode, int out_bits, int nb_dst, int b0, double *part, int flags, const NormArgs *nrm) {
    if (!umx_ready("umx_conv_fwd")) return -1;
    if (!c) { umx_latch_msg("umx_conv_fwd: no conv"); return -1; }
    if (part && (out_mode != UMX_OUT_H16B || c->kind == UMX_TCONV2)) { fprintf(stderr, "umx_conv_fwd: partial sums only with a blocked fp16 output of a plain conv\n"); abort(); }
    if (out_mode == UMX_OUT_PROB8 && (!c || c->kind != UMX_CONV1 || part || nb_dst)) { fprintf(stderr, "umx_conv_fwd: probability bytes only from a 1^3 conv into a tensor of its own\n"); abort(); }
    if ((out_mode == UMX_OUT_MX || out_mode == UMX_OUT_MXRAW) && out_bits != 8 && out_bits != 4) { fprintf(stderr, "umx_conv_fwd: MX output needs out_bits 8 or 4\n"); abort(); }
    if (flags & (UMX_X_H16 | UMX_X_U8)) {
        /* x is the fp16 tensor [N][ci][D][H][W] itself.  The tap-packed kernel takes the one-channel 3^3 case as it is; everything else is
           quantised into scratch first and goes the usual way. */
        if (c->kind != UMX_CONV3 && c->kind != UMX_CONV1) { fprintf(stderr, "umx_conv_fwd: an fp16 input only for the 3^3 and 1^3 convs\n"); abort(); }
        /* UMX_STEM=0 in the environment (read at every such call): always quantise first.  That path adds the taps of a one-channel conv one
           by one in ascending order, as a sequential fp32 loop does; the tap-packed tile adds them inside one MMA. */
        const char *env = getenv("UMX_STEM");
        const bool stem_on = !(env && *env == '0');
        if (stem_on && c->wstem && out_mode == UMX_OUT_H16B && !nb_dst) {
            const int r = umx_conv_fwd_stem(c, x, (flags & UMX_X_U8) != 0, N, D, H, W, y);
            if (r < 0) return -1;
            if (r == 0) {
                g_last_kernel = 3;
                if (nrm) umx_in_stats_coef(y, N, c->co, D, H, W, nrm->gamma, nrm->beta, nrm->eps, part, nrm->coef);
                else if (part) umx_in_part(y, N, c->co, D, H, W, part);
                return 0;
            }
        }
        if (flags & UMX_X_U8) {                             /* bytes -> fp16 in scratch */
            const size_t nx = (size_t)N * c->ci * D * H * W;
            void *h = umx_ws(12, nx * 2);
            if (!h) return -1;
            umx_u8_to_h16((const uint8_t *)x, nx, h);
            x = h;
        }
        void *ws = umx_ws(1, umx_mx_bytes32(c->bits, N, c->ci, (size_t)D * H * W));
        if (!ws) return -1;
        umx_pm_to_mx32(x, UMX_F16, N, c->ci, (size_t)D * H * W, ws, c->bits, UMX_LAYOUT_SPLIT);
        x = ws; flags = (flags & ~(UMX_X_H16 | UMX_X_U8)) | UMX_X_SPLIT;
    }
    encode_fn enc = get_encode(); if (!enc) return -1;
    ConvArgs a; memset(&a, 0, sizeof a);
    /* the stride-2 3^3 conv is given its input grid; its GEMM rows are the output grid ceil(D / 2) x ceil(H / 2) x ceil(W / 2) */
    const bool s2 = c->kind == UMX_CONV3S2;
    const int Dx = D, Hx = H, Wx = W, nbx = s2 ? ceil_div(c->ci, 32) : c->nkb;  /* grid and 32-channel blocks of the tensor x */
    const size_t Sx = (size_t)Dx * Hx * Wx;
    if (s2) { D = (D + 1) / 2; H = (H + 1) / 2; W = (W + 1) / 2; a.s2 = 1; a.nbi = nbx; a.nit = c->nki / 27; a.Di = Dx; a.Hi = Hx; a.Wi = Wx; }
    a.N = N; a.D = D; a.H = H; a.W = W; a.nkb = c->nkb; a.nki = c->nki; a.taps = c->taps; a.bits = c->bits;
    a.cop = c->cop; a.nt = c->nt; a.ntiles_n = c->ntiles_n; a.tiles_x = ceil_div(W, 8); a.tiles_y = ceil_div(H, 16);
    a.w_stage_bytes = c->w_stage_bytes; a.nst = c->nst; a.items_max = c->items_max; a.ipq = c->ipq; a.nquad = c->nquad;
    const int abytes = c->taps == 27 ? 5760 : 4 * 4096;
    auto up128 = [](int v) { return (v + 127) & ~127; };
    a.offW = 0; a.offSFB = c->items_max * c->nt * 32; a.offA = up128(c->w_stage_bytes); a.offSFA = a.offA + up128(abytes);
    a.stage_bytes = (a.offSFA + c->nquad * 512 + 1023) & ~1023;
    /* per device, looked up once: the multiprocessor count and the address of the ticket array */
    static int sms_of[16]; static unsigned *tickets_of[16];
    int d0 = 0; cudaGetDevice(&d0); d0 &= 15;
    if (!sms_of[d0]) {
        int v = 148; cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d0);
        unsigned *t = nullptr;
        if (cudaGetSymbolAddress((void **)&t, g_ks_tickets) != cudaSuccess) { umx_latch_msg("umx_conv_fwd: ticket array"); return -1; }
        tickets_of[d0] = t; sms_of[d0] = v;
    }
    const int sms = sms_of[d0];
    /* two blocks a multiprocessor (two issuing threads keep the tensor pipe busier than one) for the narrow tiles, and for the wide ones when
       there are more blocks than multiprocessors; a deep ring for one block otherwise */
    const long long blocks_all = (long long)a.tiles_x * a.tiles_y * D * N * a.ntiles_n;
    const int budget = (c->nt > 64 && blocks_all <= sms) ? 200 * 1024 : 100 * 1024;
    a.ring = budget / a.stage_bytes; if (a.ring > 8) a.ring = 8; if (a.ring < 2) a.ring = 2;
    const size_t S = (size_t)D * H * W;
    const int rb = c->bits == 8 ? 32 : 16;
    a.x_sc = (const uint8_t *)x + (size_t)N * nbx * Sx * rb;
    a.wpk = c->wpk;
    a.e.N = N; a.e.D = D; a.e.H = H; a.e.W = W; a.e.cop = c->cop; a.e.bias = c->bias_p;
    a.e.out_mode = out_mode; a.e.out_bits = out_bits; a.e.tconv = c->kind == UMX_TCONV2; a.e.co_real = c->co; a.e.cob_t = c->cob_t;
    a.e.nb_dst = nb_dst ? nb_dst : c->cob_t; a.e.b0 = nb_dst ? b0 : 0;
    a.e.y = y; a.e.y_split = (flags & UMX_Y_SPLIT) != 0; a.err = umx_errflag();
    if (out_mode == UMX_OUT_PROB8) { a.e.ptab = umx_prob_table(); if (!a.e.ptab) return -1; }
    if (!a.err) return -1;
    /* tensor map over the activation codes seen as 16-byte-wide planes [plane][z][y][x * 16 B]: fp8 in the split layout has two planes a
       block, fp4 one.  A box is (10 or 8 voxels) x (18 or 16 rows) x 1 plane of z x 2 planes; voxels outside the volume read as zero. */
    if (c->bits == 8 && !(flags & UMX_X_SPLIT)) {   /* reference layout: re-lay the codes into scratch first */
        void *ws = umx_ws(1, umx_mx_bytes32(8, N, nbx * 32, Sx));
        if (!ws) return -1;
        umx_mx_relayout(x, 8, N, nbx * 32, Sx, ws, UMX_LAYOUT_SPLIT);
        x = ws; a.x_sc = (const uint8_t *)x + (size_t)N * nbx * Sx * 32;
    }
    CUtensorMap m0; memset(&m0, 0, sizeof m0);
    if (s2) {
        /* [plane][z][y][x][16 B] with a traversal stride of two voxels along x and y: a box of 16 x 32 voxel positions delivers 8 x 16 voxels */
        const cuuint64_t gd[5] = {16, (cuuint64_t)Wx, (cuuint64_t)Hx, (cuuint64_t)Dx, (cuuint64_t)N * nbx * (c->bits == 8 ? 2 : 1)};
        const cuuint64_t gs[4] = {16, (cuuint64_t)Wx * 16, (cuuint64_t)Wx * Hx * 16, (cuuint64_t)Sx * 16};
        const cuuint32_t box[5] = {16, 16, 32, 1, 2}, es[5] = {1, 2, 2, 1, 1};
        const CUresult r0 = enc(&m0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, (void *)x, gd, gs, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r0 != CUDA_SUCCESS) { char b[160]; snprintf(b, sizeof b, "umx_conv_fwd: cuTensorMapEncodeTiled failed (%d) for the stride-2 map of %d x %d x %d x %d, %d blocks", (int)r0, N, Dx, Hx, Wx, nbx); umx_latch_msg(b); return -1; }
    } else {
        const cuuint32_t bx = c->taps == 27 ? 10 : 8, by = c->taps == 27 ? 18 : 16;
        const cuuint64_t gd[4] = {(cuuint64_t)W * 16, (cuuint64_t)H, (cuuint64_t)D, (cuuint64_t)N * c->nkb * (c->bits == 8 ? 2 : 1)};
        const cuuint64_t gs[3] = {(cuuint64_t)W * 16, (cuuint64_t)W * H * 16, (cuuint64_t)S * 16};
        const cuuint32_t box[4] = {bx * 16, by, 1, 2}, es[4] = {1, 1, 1, 1};
        const CUresult r0 = enc(&m0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void *)x, gd, gs, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r0 != CUDA_SUCCESS) { char b[160]; snprintf(b, sizeof b, "umx_conv_fwd: cuTensorMapEncodeTiled failed (%d) for %d x %d x %d x %d, %d blocks", (int)r0, N, D, H, W, c->nkb); umx_latch_msg(b); return -1; }
    }
    /* algorithmic work: 2 x output voxels x real input channels x real output channels x taps (no credit for padding) */
    const double flops = 2.0 * (double)N * S * (c->kind == UMX_DOWN2 ? 8.0 : 1.0) * c->ci * (double)c->co * (c->kind == UMX_TCONV2 ? 8.0 : 1.0) * ((c->taps == 27 || s2) ? 27.0 : 1.0);
    static int force_v1 = -1;
    if (force_v1 < 0) { const char *ev = getenv("UMX_CONV_V1"); force_v1 = ev && *ev && *ev != '0'; }
    /* InstanceNorm statistics are a separate pass over the stored output (umx_in_part below) */
    if (!force_v1 && c->wr) {   /* resident weights: the persistent z-marching kernel, when the geometry allows */
        const int pid = umx_prof_open(flops);
        int rc = (nrm && (flags & UMX_STATS_EPILOGUE)) ? umx_conv_fwd_r(c, x, &m0, (void *)enc, N, D, H, W, a.e, part, nrm->gamma, nrm->beta, nrm->eps, nrm->coef) : 1;
        const bool fused = rc == 0;
        if (rc > 0) rc = umx_conv_fwd_r(c, x, &m0, (void *)enc, N, D, H, W, a.e, nullptr, nullptr, nullptr, 0.f, nullptr);
        if (rc <= 0) {
            umx_prof_close(pid);
            g_umx_launches++; g_last_kernel = 1;
            UMX_CK("umx_conv_fwd");
            if (rc == 0 && nrm && !fused) umx_in_stats_coef(y, N, c->co, D, H, W, nrm->gamma, nrm->beta, nrm->eps, part, nrm->coef);
            else if (rc == 0 && part && !nrm) umx_in_part(y, N, c->co, D, H, W, part);
            return rc;
        }
    }
    if (!force_v1 && c->wp) {   /* one tap, resident weights: the streaming kernel */
        const int pid = umx_prof_open(flops);
        const int rc = umx_conv_fwd_p(c, x, (void *)enc, N, D, H, W, a.e);
        if (rc <= 0) {
            umx_prof_close(pid);
            g_umx_launches++; g_last_kernel = 2;
            UMX_CK("umx_conv_fwd");
            if (rc == 0 && nrm) umx_in_stats_coef(y, N, c->co, D, H, W, nrm->gamma, nrm->beta, nrm->eps, part, nrm->coef);
            else if (rc == 0 && part) umx_in_part(y, N, c->co, D, H, W, part);
            return rc;
        }
    }
    if (out_mode == UMX_OUT_PROB8) {
        /* not the head's shape: fp16 plane-major logits into scratch, then the probability pass (the same bytes) */
        const size_t ny = (size_t)N * c->co * S;
        void *t = umx_ws(12, ny * 2);
        if (!t) return -1;
        const int rc = conv_fwd_impl(c, x, N, D, H, W, t, UMX_OUT_PM16, 0, 0, 0, nullptr, flags | (c->bits == 8 ? UMX_X_SPLIT : 0), nullptr);
        if (rc == 0) umx_h16_to_prob_u8(t, ny, (uint8_t *)y);
        return rc;
    }
    const size_t smem = 1024 + (size_t)a.ring * a.stage_bytes;
    static size_t smem_set[16];
    int dev = 0; cudaGetDevice(&dev); dev &= 15;
    if (smem_set[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(conv_mx_k<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(conv_mx_k<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024));
        if (e != cudaSuccess) { umx_latch("umx_conv_fwd: shared memory attribute", e); return -1; }
        smem_set[dev] = 227 * 1024;
    }
    /* K split for the layers with fewer tiles than multiprocessors (the deep levels); chosen from one sample's geometry so that a sample's
       result does not depend on the batch it is in */
    a.ksplit = 1;
    {
        static int no_split = -1;
        if (no_split < 0) { const char *ev = getenv("UMX_KSPLIT"); no_split = ev && *ev == '0'; }
        const long long blocks1 = (long long)a.tiles_x * a.tiles_y * D * a.ntiles_n, tiles_all = blocks1 * N;
        const int units = c->taps == 27 ? c->nki : c->nst;
        long long ks = blocks1 > 0 ? sms / blocks1 : 1;
        if (ks > units) ks = units;
        if (ks > c->nst / 6) ks = c->nst / 6;              /* at least six stages a share: shorter shares cost more in the reduction than they save */
        if (ks > 16) ks = 16;
        /* the parts of a chunk are summed from the stage ring; the bound is that of the shallow ring, whatever ring this launch has, so that
           the split does not change with the batch */
        { int rs = 100 * 1024 / a.stage_bytes; if (rs > 8) rs = 8; if (rs < 2) rs = 2; const long long cap = (long long)rs * a.stage_bytes / 16384; if (ks > cap) ks = cap; }
        if (!no_split && ks >= 2 && tiles_all <= 8192) {
            const size_t bytes = (size_t)tiles_all * (size_t)ks * (size_t)(c->nt >> 5) * 4096 * 4;
            void *ws = umx_ws(5, bytes);
            if (!ws) return -1;
            a.ks_tickets = tickets_of[d0];
            a.ksplit = (int)ks; a.ks_part = (float *)ws;
        }
    }
    const dim3 grid(a.tiles_x * a.tiles_y, D, N * a.ntiles_n * a.ksplit);
    const int pid = umx_prof_open(flops);
    if (c->bits == 8) umx_launch(conv_mx_k<8>, grid, dim3(kThreads), smem, m0, a); else umx_launch(conv_mx_k<4>, grid, dim3(kThreads), smem, m0, a);
    umx_prof_close(pid);
    g_umx_launches++; g_last_kernel = 0;
    UMX_CK("umx_conv_fwd");
    if (nrm) umx_in_stats_coef(y, N, c->co, D, H, W, nrm->gamma, nrm->beta, nrm->eps, part, nrm->coef);
    else if (part) umx_in_part(y, N, c->co, D, H, W, part);
    return 0;
}
extern "C" int umx_conv_fwd(const umx_conv *c, const void *x, int N, int D, int H, int W, void *y, int out_mode, int out_bits, int nb_dst, int b0, double *part, int flags) {
    return conv_fwd_impl(c, x, N, D, H, W, y, out_mode, out_bits, nb_dst, b0, part, flags, nullptr);
}
/* conv -> blocked fp16 y, and the InstanceNorm coefficients (a, b) per (sample, channel) of that stored tensor; part: scratch of
   umx_stats_doubles doubles.  The resident-weight kernel takes the sums in its epilogue (fp32 inside 32-voxel units, exact above them);
   only under UMX_STATS_EPILOGUE; otherwise, and for the other kernels, the conv is followed by the statistics pass.  gamma / beta: device arrays or NULL (1 / 0). */
extern "C" int umx_conv_fwd_norm(const umx_conv *c, const void *x, int N, int D, int H, int W, void *y, double *part, const float *gamma, const float *beta, float eps, float *coef, int flags) {
    if (!part || !coef) { fprintf(stderr, "umx_conv_fwd_norm: part and coef are required\n"); abort(); }
    if (c && c->kind == UMX_TCONV2) { fprintf(stderr, "umx_conv_fwd_norm: not for the transposed conv\n"); abort(); }
    const NormArgs nrm = {gamma, beta, eps, coef};
    return conv_fwd_impl(c, x, N, D, H, W, y, UMX_OUT_H16B, 0, 0, 0, part, flags, &nrm);
}
