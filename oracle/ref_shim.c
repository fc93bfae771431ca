/* Thin C entry points over the reference's own dequantiser header, compiled
 * from where it lies in the reference tree (never copied into this
 * repository).  The build recipe is oracle/Makefile; the output goes to
 * oracle/_ref/.  TEST INFRASTRUCTURE ONLY: used to validate the restated
 * dequantiser in q36_oracle.c and as the timed CPU baseline. */
#include <stdbool.h>
#include <stdint.h>
#include "q36.h"
#include "q36_dequant.cuh"

float ref_e8m0_half(uint8_t e) { return q36_e8m0_half(e); }
float ref_fp16(uint16_t h) { return q36_fp16(h); }
int ref_sizeof_block_mxfp4(void) { return (int)sizeof(block_mxfp4); }
void ref_deq_mxfp4_block(const uint8_t *blk, float *out) { q36_deq_mxfp4((const block_mxfp4 *)blk, out); }
/* q36_deq_row(Q36_GGML_MXFP4, ...) exactly as test_dequant.c drives it */
void ref_deq_mxfp4_row(const uint8_t *blocks, int64_t n, float *out) {
    q36_deq_row(Q36_GGML_MXFP4, blocks, (int)n, out);
}
