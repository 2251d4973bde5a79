/*
 * A C host of libq4gpu: plain C99, includes include/q4_gpu.h and links the shared library the way the
 * reference links its device code into its C programs (reference Makefile:21-25).  It replays the
 * reference's own fixture for this path (src/q4_test.c:134-238: 2 query heads, 1 kv head, hd 32, 2
 * tokens over 4 positions, inputs by formula, expected values from a dense softmax on the unquantised
 * rows) through q4_hip_f32_to_f16 / q4_hip_f32_to_q8 / q4_hip_qsa_decode_n with the tolerances the
 * reference asserts (f32 1e-3, f16 2e-2, q8_0 8e-2), then drives the library-owned store through the
 * additive entry points from C as well.  Exit status 0 = every check passed.
 *
 * Built and run by tests/test_c_abi.py:  gcc -std=c99 -Wall -Wextra -Werror -pedantic fixture.c -lq4gpu -lm
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "q4_gpu.h"

enum { N_HEAD = 2, N_KVH = 1, HD = 32, N_TOK = 2, N_POS = 4, KV_BASE = 0 };
enum { NQ = N_TOK * N_HEAD * HD, NKV = N_POS * N_KVH * HD };

static int failures = 0;

static void check(int ok, const char *what) {
    printf("%s %s\n", ok ? "ok  " : "FAIL", what);
    if (!ok) failures++;
}

/* the fixture's inputs (src/q4_test.c:146-153) */
static void fill_inputs(float *q, float *k, float *v, float *gate) {
    int i;
    for (i = 0; i < NKV; i++) {
        k[i] = (float)((i * 17) % 11) * 0.05f - 0.2f;
        v[i] = (float)((i * 13) % 9) * 0.07f;
    }
    for (i = 0; i < NQ; i++) {
        q[i] = (float)((i * 3) % 7) * 0.1f;
        gate[i] = (float)((i % 5) - 2) * 0.3f;
    }
}

/* causal attention of token t over rows [0, KV_BASE + t], times sigmoid(gate), in double precision */
static void expected(const float *q, const float *k, const float *v, const float *gate, float scale, float *ref) {
    int t, h, p, d;
    for (t = 0; t < N_TOK; t++)
        for (h = 0; h < N_HEAD; h++) {
            const int rows = KV_BASE + t + 1, kh = h / (N_HEAD / N_KVH);
            const float *qh = q + (t * N_HEAD + h) * HD;
            double s[N_POS], top = -1e300, sum = 0.0;
            for (p = 0; p < rows; p++) {
                double dot = 0.0;
                for (d = 0; d < HD; d++) dot += (double)qh[d] * k[(p * N_KVH + kh) * HD + d];
                s[p] = dot * scale;
                if (s[p] > top) top = s[p];
            }
            for (p = 0; p < rows; p++) {
                s[p] = exp(s[p] - top);
                sum += s[p];
            }
            for (d = 0; d < HD; d++) {
                double a = 0.0;
                for (p = 0; p < rows; p++) a += s[p] * v[(p * N_KVH + kh) * HD + d];
                ref[(t * N_HEAD + h) * HD + d] =
                    (float)(a / sum / (1.0 + exp(-(double)gate[(t * N_HEAD + h) * HD + d])));
            }
        }
}

static float max_abs_diff(const float *a, const float *b, int n) {
    float m = 0.f;
    int i;
    for (i = 0; i < n; i++) {
        float e = fabsf(a[i] - b[i]);
        if (!(e <= m)) m = e; /* also catches NaN */
    }
    return m;
}

int main(void) {
    float q[NQ], gate[NQ], out[NQ], ref[NQ], k[NKV], v[NKV];
    const float scale = 1.f / sqrtf((float)HD);
    float *dq, *dk, *dv, *dg, *dout;
    void *kc[3], *vc[3];
    static const float tol[3] = {1e-3f, 2e-2f, 8e-2f};
    static const char *name[3] = {"reference fixture, f32 KV within 1e-3", "reference fixture, f16 KV within 2e-2",
                                  "reference fixture, q8_0 KV within 8e-2"};
    int kind;

    if (!q4_hip_init()) {
        fprintf(stderr, "q4_hip_init failed: no usable CUDA device\n");
        return 2;
    }
    check(q4_hip_ok(), "q4_hip_ok after init");
    fill_inputs(q, k, v, gate);
    expected(q, k, v, gate, scale, ref);

    dq = (float *)q4_hip_malloc(sizeof q);
    dg = (float *)q4_hip_malloc(sizeof gate);
    dout = (float *)q4_hip_malloc(sizeof out);
    dk = (float *)q4_hip_malloc(sizeof k);
    dv = (float *)q4_hip_malloc(sizeof v);
    kc[0] = dk;
    vc[0] = dv;
    kc[1] = q4_hip_malloc(NKV * 2);
    vc[1] = q4_hip_malloc(NKV * 2);
    kc[2] = q4_hip_malloc(NKV / 32 * 34);
    vc[2] = q4_hip_malloc(NKV / 32 * 34);
    if (!dq || !dg || !dout || !dk || !dv || !kc[1] || !vc[1] || !kc[2] || !vc[2]) {
        fprintf(stderr, "q4_hip_malloc failed\n");
        return 2;
    }
    check(q4_hip_h2d(dq, q, sizeof q) && q4_hip_h2d(dg, gate, sizeof gate) && q4_hip_h2d(dk, k, sizeof k) &&
              q4_hip_h2d(dv, v, sizeof v),
          "uploads");
    check(q4_hip_f32_to_f16(kc[1], dk, NKV) && q4_hip_f32_to_f16(vc[1], dv, NKV), "q4_hip_f32_to_f16");
    check(q4_hip_f32_to_q8(kc[2], dk, NKV) && q4_hip_f32_to_q8(vc[2], dv, NKV), "q4_hip_f32_to_q8");
    for (kind = 0; kind < 3; kind++) {
        memset(out, 0, sizeof out);
        if (!q4_hip_qsa_decode_n(dq, kc[kind], vc[kind], dg, dout, N_HEAD, N_KVH, HD, N_TOK, KV_BASE, N_POS, scale, kind) ||
            !q4_hip_d2h(out, dout, sizeof out)) {
            check(0, name[kind]);
            continue;
        }
        check(max_abs_diff(out, ref, NQ) <= tol[kind], name[kind]);
    }
    /* the reference's conventions: NULL gate and zero sizes are rejected, never crash */
    check(!q4_hip_qsa_decode_n(dq, dk, dv, NULL, dout, N_HEAD, N_KVH, HD, N_TOK, KV_BASE, N_POS, scale, 0),
          "NULL gate rejected by the reference entry point");
    check(!q4_hip_f32_to_q8(kc[2], dk, 0) && !q4_hip_f32_to_q8(kc[2], dk, 33), "zero / ragged q8 sizes rejected");

    /* the additive entry points from C: a library-owned q8_0 store, fused K+V append, decode of the last
     * token (same rows, same expectation as token N_TOK-1 of the fixture when it sees all N_POS rows) */
    {
        q4_gpu_kv *kv = q4_gpu_kv_create(1, N_KVH, HD, N_POS, 2);
        float ref_last[N_HEAD * HD];
        int h, p, d;
        check(kv != NULL, "q4_gpu_kv_create");
        if (kv) {
            check(q4_gpu_kv_append(kv, 0, dk, dv, 0, N_POS), "q4_gpu_kv_append");
            check(q4_gpu_kv_decode(kv, 0, dq + (N_TOK - 1) * N_HEAD * HD, 0, dg + (N_TOK - 1) * N_HEAD * HD, dout, N_HEAD,
                                   NULL, 0, 0, N_POS, scale),
                  "q4_gpu_kv_decode");
            check(q4_hip_d2h(out, dout, sizeof ref_last), "download");
            for (h = 0; h < N_HEAD; h++) {
                const float *qh = q + ((N_TOK - 1) * N_HEAD + h) * HD;
                double s[N_POS], top = -1e300, sum = 0.0;
                for (p = 0; p < N_POS; p++) {
                    double dot = 0.0;
                    for (d = 0; d < HD; d++) dot += (double)qh[d] * k[p * HD + d];
                    s[p] = dot * scale;
                    if (s[p] > top) top = s[p];
                }
                for (p = 0; p < N_POS; p++) {
                    s[p] = exp(s[p] - top);
                    sum += s[p];
                }
                for (d = 0; d < HD; d++) {
                    double a = 0.0;
                    for (p = 0; p < N_POS; p++) a += s[p] * v[p * HD + d];
                    ref_last[h * HD + d] = (float)(a / sum / (1.0 + exp(-(double)gate[((N_TOK - 1) * N_HEAD + h) * HD + d])));
                }
            }
            check(max_abs_diff(out, ref_last, N_HEAD * HD) <= 8e-2f, "store decode over all rows, q8_0, within 8e-2");
            q4_gpu_kv_destroy(kv);
        }
    }
    check(q4_gpu_last_error() == 0, "status word clean");

    q4_hip_free(dq); q4_hip_free(dg); q4_hip_free(dout); q4_hip_free(dk); q4_hip_free(dv);
    q4_hip_free(kc[1]); q4_hip_free(vc[1]); q4_hip_free(kc[2]); q4_hip_free(vc[2]);
    q4_hip_shutdown();
    check(!q4_hip_ok(), "q4_hip_ok false after shutdown");
    printf("%d failure(s)\n", failures);
    return failures ? 1 : 0;
}
