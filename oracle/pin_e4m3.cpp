// Checks the oracle's E4M3 encoder/decoder against NVIDIA's host-side
// implementation in cuda_fp8.h (the code the reference's quantiser calls on
// the device, q36_engine.cu:2425).  Exhaustive over every float whose
// magnitude lies in [2^-14, 2^11) plus a strided sweep of all other bit
// patterns.  Prints the number of mismatches; exit status 0 iff none.
// TEST INFRASTRUCTURE ONLY.
#include <cuda_fp8.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cmath>
extern "C" uint8_t orc_e4m3_encode(float x);
extern "C" float orc_e4m3_decode(uint8_t b);
static inline uint8_t nv_enc(float x) { return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3); }
int main() {
    long bad = 0, n = 0;
    for (uint32_t e = 127 - 14; e < 127 + 11; ++e)
        for (uint32_t m = 0; m < (1u << 23); ++m)
            for (uint32_t s = 0; s < 2; ++s) {
                uint32_t u = (s << 31) | (e << 23) | m; float x; memcpy(&x, &u, 4);
                if (nv_enc(x) != orc_e4m3_encode(x)) { if (bad < 5) printf("mismatch %a nv=%02x orc=%02x\n", x, nv_enc(x), orc_e4m3_encode(x)); ++bad; }
                ++n;
            }
    for (uint64_t u64 = 0; u64 < (1ull << 32); u64 += 4099) {
        uint32_t u = (uint32_t)u64; float x; memcpy(&x, &u, 4);
        if (nv_enc(x) != orc_e4m3_encode(x)) { if (bad < 5) printf("mismatch %a nv=%02x orc=%02x\n", x, nv_enc(x), orc_e4m3_encode(x)); ++bad; }
        ++n;
    }
    for (int b = 0; b < 256; ++b) {
        __nv_fp8_e4m3 q; memcpy(&q, &b, 1); float want = (float)q, got = orc_e4m3_decode((uint8_t)b);
        if (!(want == got || (std::isnan(want) && std::isnan(got)))) { printf("decode mismatch %02x %g %g\n", b, want, got); ++bad; }
        ++n;
    }
    printf("checked %ld values, %ld mismatches\n", n, bad);
    return bad ? 1 : 0;
}
