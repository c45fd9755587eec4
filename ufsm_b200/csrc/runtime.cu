/* Device runtime of the library: device selection, memory, the error latch, growing scratch buffers. */
#include "mx_common.cuh"
#include <stdlib.h>
#include <string.h>

long g_umx_launches = 0;
static thread_local char g_err[512];
static thread_local int g_has_err = 0;
static int g_ready[16];   /* per device: 0 unknown, 1 usable sm_100, -1 not usable */

void umx_latch_msg(const char *msg) {
    if (g_has_err) return;
    snprintf(g_err, sizeof g_err, "%s", msg);
    g_has_err = 1;
}
void umx_latch(const char *where, cudaError_t e) {
    char b[512]; snprintf(b, sizeof b, "%s: %s", where, cudaGetErrorString(e));
    umx_latch_msg(b);
}
int umx_ready(const char *where) {
    int d = -1;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess || d < 0 || d >= 16) { char b[256]; snprintf(b, sizeof b, "%s: no CUDA device (%s); this library has no CPU path", where, cudaGetErrorString(e)); umx_latch_msg(b); cudaGetLastError(); return 0; }
    if (!g_ready[d]) {
        cudaDeviceProp p; e = cudaGetDeviceProperties(&p, d);
        g_ready[d] = (e == cudaSuccess && p.major == 10) ? 1 : -1;
    }
    if (g_ready[d] < 0) { char b[256]; snprintf(b, sizeof b, "%s: device %d is not sm_100 (B200); this library has no other path", where, d); umx_latch_msg(b); return 0; }
    return 1;
}
static int *g_flag[16];
void umx_conv_r_tickets_reset(void);
void umx_conv_ks_tickets_reset(void);
void umx_stat_tickets_reset(void);
extern "C" const char *lp_check(void) {
    int d = -1;
    if (!g_has_err && cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < 16 && g_flag[d]) umx_errflag_read();   /* a kernel's bounded wait that gave up */
    if (!g_has_err) return nullptr;
    g_has_err = 0;
    return g_err;
}
extern "C" const char *nn_check(void) { return lp_check(); }
/* 1 when this thread has latched an error; unlike lp_check it neither reads the device's flag (a synchronising copy) nor clears the latch */
extern "C" int umx_has_error(void) { return g_has_err; }
extern "C" int nn_init(int device) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) { umx_latch("nn_init", e); return -1; }
    return umx_ready("nn_init") ? 0 : -1;
}
extern "C" void *nn_malloc(size_t bytes) {
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
    if (e != cudaSuccess) { umx_latch("nn_malloc", e); return nullptr; }
    return p;
}
extern "C" void nn_free(void *p) { if (p) cudaFree(p); }
extern "C" void nn_zero(void *p, size_t bytes) { cudaError_t e = cudaMemset(p, 0, bytes); if (e != cudaSuccess) umx_latch("nn_zero", e); }
extern "C" void nn_h2d(void *dst, const void *src, size_t bytes) { cudaError_t e = cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice); if (e != cudaSuccess) umx_latch("nn_h2d", e); }
extern "C" void nn_d2h(void *dst, const void *src, size_t bytes) { cudaError_t e = cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost); if (e != cudaSuccess) umx_latch("nn_d2h", e); }
extern "C" void nn_sync(void) {
    cudaError_t e = cudaDeviceSynchronize(); if (e != cudaSuccess) { umx_latch("nn_sync", e); return; }
    int d = -1; if (cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < 16 && g_flag[d]) umx_errflag_read();
}
extern "C" void *nn_malloc_host(size_t bytes) {
    void *p = nullptr;
    cudaError_t e = cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault);
    if (e != cudaSuccess) { umx_latch("nn_malloc_host", e); return nullptr; }
    return p;
}
extern "C" void nn_free_host(void *p) { if (p) cudaFreeHost(p); }

/* ---- copy streams and events for the host entry that overlaps the copies of one patch with the forward of the next.  Streams are
   non-blocking (they do not synchronise with the legacy default stream the kernels run on); the order is made with events. ---- */
int umx_pdl(void) { static int v = -1; if (v < 0) { const char *e = getenv("UMX_PDL"); v = !(e && *e == '0'); } return v; }
extern "C" void *umx_stream_new(void) { cudaStream_t s = nullptr; cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking); if (e != cudaSuccess) { umx_latch("umx_stream_new", e); return nullptr; } return (void *)s; }
extern "C" void umx_stream_free(void *s) { if (s) cudaStreamDestroy((cudaStream_t)s); }
extern "C" void *umx_event_new(void) { cudaEvent_t ev = nullptr; cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming); if (e != cudaSuccess) { umx_latch("umx_event_new", e); return nullptr; } return (void *)ev; }
extern "C" void umx_event_free(void *ev) { if (ev) cudaEventDestroy((cudaEvent_t)ev); }
/* stream NULL = the legacy default stream */
extern "C" void umx_event_record(void *ev, void *stream) { cudaError_t e = cudaEventRecord((cudaEvent_t)ev, (cudaStream_t)stream); if (e != cudaSuccess) umx_latch("umx_event_record", e); }
extern "C" void umx_stream_wait(void *stream, void *ev) { cudaError_t e = cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)ev, 0); if (e != cudaSuccess) umx_latch("umx_stream_wait", e); }
extern "C" void umx_event_sync(void *ev) { cudaError_t e = cudaEventSynchronize((cudaEvent_t)ev); if (e != cudaSuccess) umx_latch("umx_event_sync", e); }
extern "C" void umx_stream_sync(void *stream) { cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream); if (e != cudaSuccess) umx_latch("umx_stream_sync", e); }
extern "C" void umx_copy_async(void *dst, const void *src, size_t bytes, int to_device, void *stream) {
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e != cudaSuccess) umx_latch("umx_copy_async", e);
}

/* height rows of width bytes, the rows dpitch / spitch bytes apart */
extern "C" void umx_copy2d_async(void *dst, size_t dpitch, const void *src, size_t spitch, size_t width, size_t height, int to_device, void *stream) {
    cudaError_t e = cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, height, to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e != cudaSuccess) umx_latch("umx_copy2d_async", e);
}

/* scratch: per device, per slot, grows on demand, never shrinks */
enum { WS_SLOTS = 13 };
static void *g_ws[16][WS_SLOTS];
static size_t g_ws_bytes[16][WS_SLOTS];
void *umx_ws(int slot, size_t bytes) {
    int d = 0; cudaGetDevice(&d); d &= 15;
    if (g_ws_bytes[d][slot] < bytes) {
        if (g_ws[d][slot]) { cudaDeviceSynchronize(); cudaFree(g_ws[d][slot]); }
        const size_t nb = bytes + bytes / 4 + 256;
        cudaError_t e = cudaMalloc(&g_ws[d][slot], nb);
        if (e != cudaSuccess) { umx_latch("umx_ws", e); g_ws[d][slot] = nullptr; g_ws_bytes[d][slot] = 0; return nullptr; }
        g_ws_bytes[d][slot] = nb;
    }
    return g_ws[d][slot];
}
int *umx_errflag(void) {
    int d = 0; cudaGetDevice(&d); d &= 15;
    if (!g_flag[d]) {
        if (cudaMalloc(&g_flag[d], 256) != cudaSuccess) { umx_latch_msg("umx_errflag: cudaMalloc failed"); return nullptr; }
        cudaMemset(g_flag[d], 0, 256);
    }
    return g_flag[d];
}
int umx_errflag_read(void) {
    int *f = umx_errflag(); if (!f) return -1;
    int h[64] = {0};
    cudaError_t e = cudaMemcpy(h, f, sizeof h, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { umx_latch("umx_errflag_read", e); return -1; }
    if (h[0]) {
        /* h[0..3]: the first wait that gave up (role code, block, stage, thread).  h[16 + 4 r ..]: where each role r of that block stood when
           it left its loop: stage, barrier (byte offset in the block's barrier array), parity; a stage counter far from the others' points
           at the role that broke the protocol. */
        static const char *role[8] = {"?", "producer", "mma-tma", "mma-scales", "gather", "epilogue", "weights", "mma-slot"};
        char b[500]; int n = snprintf(b, sizeof b, "conv kernel: bounded wait gave up (code %d, block %d, stage %d, thread %d;", h[0], h[1], h[2], h[3]);
        for (int r = 1; r < 8 && n < (int)sizeof b - 60; r++) if (h[16 + 4 * r + 3]) n += snprintf(b + n, sizeof b - n, " %s at stage %d on barrier +%d parity %d;", role[r], h[16 + 4 * r], h[16 + 4 * r + 1], h[16 + 4 * r + 2]);
        snprintf(b + n, sizeof b - n, ")");
        umx_latch_msg(b);
        /* blocks that gave up left without drawing their tickets: zero the ticket counters of the kernels that finalise from the last block,
           so that later launches count from zero again, then clear the flag */
        umx_conv_r_tickets_reset(); umx_conv_ks_tickets_reset(); umx_stat_tickets_reset();
        cudaMemset(f, 0, 256);
    }
    return h[0];
}

/* ---- timing on the launching (legacy default) stream ---- */
struct umx_timer { cudaEvent_t a, b; };
extern "C" void *umx_timer_new(void) {
    umx_timer *t = (umx_timer *)calloc(1, sizeof *t);
    if (cudaEventCreate(&t->a) != cudaSuccess || cudaEventCreate(&t->b) != cudaSuccess) { umx_latch_msg("umx_timer_new: cudaEventCreate failed"); free(t); return nullptr; }
    return t;
}
extern "C" void umx_timer_start(void *tv) { umx_timer *t = (umx_timer *)tv; cudaDeviceSynchronize(); cudaEventRecord(t->a, 0); }
extern "C" float umx_timer_stop_ms(void *tv) {
    umx_timer *t = (umx_timer *)tv; float ms = 0.f;
    cudaEventRecord(t->b, 0);
    cudaError_t e = cudaEventSynchronize(t->b);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t->a, t->b);
    if (e != cudaSuccess) { umx_latch("umx_timer_stop_ms", e); return -1.f; }
    return ms;
}
/* the two halves of umx_timer_stop_ms: record the stop event now; wait for it and read the time later (a caller that wants to do
   host work, such as sampling clocks, while the timed launches are still running) */
extern "C" void umx_timer_mark(void *tv) { cudaEventRecord(((umx_timer *)tv)->b, 0); }
extern "C" float umx_timer_read_ms(void *tv) {
    umx_timer *t = (umx_timer *)tv; float ms = 0.f;
    cudaError_t e = cudaEventSynchronize(t->b);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t->a, t->b);
    if (e != cudaSuccess) { umx_latch("umx_timer_read_ms", e); return -1.f; }
    return ms;
}
extern "C" void umx_timer_free(void *tv) { umx_timer *t = (umx_timer *)tv; if (!t) return; cudaEventDestroy(t->a); cudaEventDestroy(t->b); free(t); }

/* per-launch timing of the conv kernel: between umx_prof_begin and umx_prof_end every conv launch is bracketed by two events */
enum { PROF_MAX = 8192 };
static cudaEvent_t g_pev[2 * PROF_MAX];
static double g_pflops[PROF_MAX];
static int g_pn = 0, g_pon = 0, g_pmade = 0;
extern "C" void umx_prof_begin(void) {
    if (!g_pmade) { for (int i = 0; i < 2 * PROF_MAX; i++) cudaEventCreate(&g_pev[i]); g_pmade = 1; }
    g_pn = 0; g_pon = 1;
}
int umx_prof_open(double flops) { if (!g_pon || g_pn >= PROF_MAX) return -1; g_pflops[g_pn] = flops; cudaEventRecord(g_pev[2 * g_pn], 0); return g_pn; }
void umx_prof_close(int id) { if (id < 0) return; cudaEventRecord(g_pev[2 * id + 1], 0); g_pn = id + 1; }
/* returns the number of conv launches seen; ms: their summed device time, flops: their summed algorithmic FLOPs */
extern "C" int umx_prof_end(double *ms, double *flops) {
    g_pon = 0; *ms = 0; *flops = 0;
    cudaDeviceSynchronize();
    for (int i = 0; i < g_pn; i++) { float t = 0.f; if (cudaEventElapsedTime(&t, g_pev[2 * i], g_pev[2 * i + 1]) == cudaSuccess) *ms += t; *flops += g_pflops[i]; }
    return g_pn;
}
/* after umx_prof_end: device time (ms) and algorithmic FLOPs of the i-th conv launch seen; returns 0, or -1 past the end */
extern "C" int umx_prof_get(int i, double *ms, double *flops) {
    if (i < 0 || i >= g_pn) return -1;
    float t = 0.f; cudaEventElapsedTime(&t, g_pev[2 * i], g_pev[2 * i + 1]);
    *ms = t; *flops = g_pflops[i];
    return 0;
}
