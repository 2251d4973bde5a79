/* TEST INFRASTRUCTURE.  Host shim around the reference's own q8_0 quantiser.
 *
 * The reference's quantiser exists only as device code (f32_to_q8_k, src/q4_rocm.cu:7221-7238; no
 * compiler for it is present here).  Its body is plain C, so oracle/Makefile cuts the function out of
 * the reference tree at build time into _ref/f32_to_q8_k.inc (generated, never committed) and this file
 * supplies the handful of device names it uses: the launch qualifier, the index variables, and
 * __half / __float2half through the F16C hardware conversion (round to nearest even).  Compiled with
 * -O2 -ffp-contract=off and no fast-math, so the divisions and the multiply are the IEEE ones.
 * tests/test_oracle.py pins the oracle's restatement (q4o_quant_q8_0) to this function bit for bit. */
#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

typedef uint16_t __half;
static inline __half __float2half(float f) { return (__half)_cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }
#define __global__
static struct { uint32_t x; } blockIdx, blockDim, threadIdx;

#include "_ref/f32_to_q8_k.inc"

__attribute__((visibility("default"))) void q4ref_f32_to_q8(const float *src, uint8_t *dst, uint64_t nblocks) {
    blockDim.x = 1u << 20;
    for (uint64_t b = 0; b < nblocks; b++) {
        blockIdx.x = (uint32_t)(b >> 20);
        threadIdx.x = (uint32_t)(b & ((1u << 20) - 1u));
        f32_to_q8_k(src, dst, nblocks);
    }
}
