/* Reference pin (test infrastructure only): the reference's own software MX conversions, src/mx_sw.cuh of the ufsm source tree,
   compiled for the host from where that file lies (never copied) and exported with a C ABI so the oracle's independent
   formulations can be compared with them value by value.  Built by oracle/Makefile into oracle/_ref/libmxsw_ref.so when the
   reference tree is present. */
#include "mx_sw.cuh"
#include <stddef.h>
#include <stdint.h>
extern "C" {
unsigned ref_enc_e4m3(float x) { return mxsw_enc_e4m3(x); }
unsigned ref_enc_e2m1(float x) { return mxsw_enc_e2m1(x); }
float ref_dec_e4m3(unsigned b) { return mxsw_dec_val_e4m3(b); }
float ref_dec_e2m1(unsigned n) { return mxsw_dec_val_e2m1(n); }
unsigned ref_e4m3_h16(unsigned b) { return mxsw_e4m3_h16(b); }
unsigned ref_e2m1_h16(unsigned n) { return mxsw_e2m1_h16(n); }
void ref_enc_e4m3_n(const float *x, size_t n, uint8_t *y) { for (size_t i = 0; i < n; i++) y[i] = (uint8_t)mxsw_enc_e4m3(x[i]); }
void ref_enc_e2m1_n(const float *x, size_t n, uint8_t *y) { for (size_t i = 0; i < n; i++) y[i] = (uint8_t)mxsw_enc_e2m1(x[i]); }
/* encoders over the fp32 bit patterns first, first + step, ... (count values): the number of inputs where the oracle's encoder
   (passed in) differs from the reference's */
typedef unsigned (*enc_fn)(float);
size_t ref_sweep_diff(int fmt, enc_fn orc, uint32_t first, uint32_t step, size_t count, uint32_t *first_bad) {
    size_t bad = 0;
    #pragma omp parallel for reduction(+ : bad)
    for (size_t i = 0; i < count; i++) {
        const uint32_t u = first + (uint32_t)i * step; float f; __builtin_memcpy(&f, &u, 4);
        const unsigned a = fmt == 4 ? mxsw_enc_e2m1(f) : mxsw_enc_e4m3(f), b = orc(f);
        if (a != b) { bad++; if (first_bad) *first_bad = u; }
    }
    return bad;
}
}
