/*
 * q4_oracle.c -- CPU restatement of the reference's KV-cache + attention arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing that ships may include, link or call this file; it is
 * the checker for the CUDA path (tests, the smoke check, and the CPU-baseline leg of the
 * benchmark).  Every function cites the reference code it restates (paths are relative to
 * the reference project).  Build: `make -C oracle` (gcc -O2 -ffp-contract=off, no fast-math:
 * the bit-exact quantiser contract is the IEEE evaluation of the reference's source).
 *
 * Parity pins:
 *  - q4o_f16_to_f32 / q4o_dequant_q8_0 are checked bit-for-bit against the reference's own
 *    q4_f16_to_f32 / q4_dequant_row compiled in place (oracle/_ref).
 *  - q4o_attn is checked against the reference's only hot-path fixture (src/q4_test.c:134-238).
 *  - q4o_quant_q8_0 has no golden vector in the reference (the quantiser exists only as GPU
 *    code, src/q4_rocm.cu:7221-7238); it is pinned by the source and by a round trip through
 *    the reference's dequantiser.
 *
 * KV layout used here is the reference's (src/q4_fwd.c:644-655): a cache is
 * [token][kv_head][row], row = hd/32 blocks of {fp16 scale, 32 x int8} for q8_0 (kind 2),
 * hd x fp16 (kind 1) or hd x fp32 (kind 0).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define Q4O_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ generator ---------- */
/* Counter-based generator shared by every test and bench input: splitmix64 finaliser over
 * (key(seed, stream) + index).  Not from the reference (its inputs are model activations). */
static inline uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
static inline uint64_t key64(uint64_t seed, uint64_t stream) {
    return mix64(mix64(seed) ^ (0xD1B54A32D192ED03ull * (stream + 1)));
}
Q4O_API uint64_t q4o_u64(uint64_t seed, uint64_t stream, uint64_t i) {
    return mix64(key64(seed, stream) + i);
}
/* Box-Muller in fp64, rounded once to fp32. */
Q4O_API void q4o_normal_f32(uint64_t seed, uint64_t stream, uint64_t offset, uint64_t n,
                            float *out) {
    const uint64_t k = key64(seed, stream);
    for (uint64_t j = 0; j < n; j++) {
        uint64_t i = offset + j;
        double u1 = ((double)(mix64(k + 2 * i) >> 11) + 0.5) * (1.0 / 9007199254740992.0);
        double u2 = ((double)(mix64(k + 2 * i + 1) >> 11) + 0.5) * (1.0 / 9007199254740992.0);
        out[j] = (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2));
    }
}
static int cmp_i32(const void *a, const void *b) {
    int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
    return x < y ? -1 : x > y;
}
/* Selection recipe of the benchmark configs: 4 sink tokens, the `recent` most recent tokens and
 * `nrand` positions drawn without replacement (partial Fisher-Yates) from what lies between;
 * sorted, unique, padded with -1 to `width`.  When ctx <= width every position is selected
 * (the reference's expansion does the same, src/q4_rocm.cu:7675-7678).  Returns the count. */
Q4O_API uint32_t q4o_select(uint64_t seed, uint64_t stream, uint32_t ctx, uint32_t sink,
                            uint32_t recent, uint32_t nrand, int32_t *out, uint32_t width) {
    uint32_t n = 0;
    if (ctx <= sink + recent + nrand || ctx <= width) {
        uint32_t m = ctx < width ? ctx : width;
        for (uint32_t i = 0; i < m; i++) out[n++] = (int32_t)(ctx - m + i);
    } else {
        for (uint32_t i = 0; i < sink; i++) out[n++] = (int32_t)i;
        uint32_t lo = sink, hi = ctx - recent, span = hi - lo;
        /* sparse Fisher-Yates: only touched slots are materialised */
        uint32_t cap = 1;
        while (cap < 4 * nrand + 16) cap <<= 1;
        uint32_t *hk = malloc(sizeof(uint32_t) * cap), *hv = malloc(sizeof(uint32_t) * cap);
        memset(hk, 0xff, sizeof(uint32_t) * cap);
        const uint64_t k = key64(seed, stream);
        for (uint32_t i = 0; i < nrand; i++) {
            uint32_t j = i + (uint32_t)(mix64(k + i) % (uint64_t)(span - i));
            /* value at slot j (default j), value at slot i (default i) */
            uint32_t vj = j, vi = i, pj, pi;
            for (pj = (j * 2654435761u) & (cap - 1); hk[pj] != 0xffffffffu; pj = (pj + 1) & (cap - 1))
                if (hk[pj] == j) { vj = hv[pj]; break; }
            for (pi = (i * 2654435761u) & (cap - 1); hk[pi] != 0xffffffffu; pi = (pi + 1) & (cap - 1))
                if (hk[pi] == i) { vi = hv[pi]; break; }
            out[n++] = (int32_t)(lo + vj);
            /* slot j now holds what slot i held */
            for (pj = (j * 2654435761u) & (cap - 1); hk[pj] != 0xffffffffu && hk[pj] != j;
                 pj = (pj + 1) & (cap - 1)) {}
            hk[pj] = j;
            hv[pj] = vi;
        }
        free(hk);
        free(hv);
        for (uint32_t i = 0; i < recent; i++) out[n++] = (int32_t)(hi + i);
        qsort(out, n, sizeof(int32_t), cmp_i32);
    }
    for (uint32_t i = n; i < width; i++) out[i] = -1;
    return n;
}

/* ------------------------------------------------------------------ fp16 --------------- */
/* fp16 -> fp32: restates q4_f16_to_f32, src/q4_quant.c:21-46 (sub-normals normalised by hand). */
Q4O_API float q4o_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16, ex = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
    if (ex == 0) {
        if (man == 0) u = sign;
        else {
            uint32_t e = 113;
            while (!(man & 0x400u)) { man <<= 1; e--; }
            u = sign | (e << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (ex == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((ex + 112) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}
/* fp32 -> fp16, round-to-nearest-even: the device `__float2half` the reference's quantiser and
 * f16 append use (src/q4_rocm.cu:7210,7230,7978). */
Q4O_API uint16_t q4o_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u, ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (ax > 0x7f800000u ? 0x200u : 0));
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to >= 65520 -> inf */
    if (ax < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25 -> 0 (ties to even) */
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u, shift, half_bits;
    if (e < -14) { shift = (uint32_t)(13 + (-14 - e)); half_bits = 0; }
    else { shift = 13; half_bits = (uint32_t)(e + 15) << 10; man &= 0x7fffffu; }
    uint32_t q = man >> shift, rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1))) q++;
    return (uint16_t)(sign | (half_bits + q)); /* carry into the exponent is the right answer */
}
Q4O_API void q4o_f32_to_f16_n(const float *src, uint16_t *dst, uint64_t n) {
    for (uint64_t i = 0; i < n; i++) dst[i] = q4o_f32_to_f16(src[i]);
}
Q4O_API float q4o_bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
Q4O_API uint16_t q4o_f32_to_bf16(float f) { /* RNE */
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40);
    return (uint16_t)((x + 0x7fffu + ((x >> 16) & 1)) >> 16);
}

/* ------------------------------------------------------------------ q8_0 --------------- */
/* Quantiser: restates f32_to_q8_k (src/q4_rocm.cu:7221-7238) and the q8 branch of kv_append_k
 * (:7967-7985): amax over 32 values, d = amax/127 (fp32 divide), id = 1/d, code =
 * clamp(rintf(x*id), +-127), scale stored as RNE fp16 of the fp32 d. */
Q4O_API void q4o_quant_q8_0(const float *src, uint8_t *dst, uint64_t n) {
    const uint64_t nb = n / 32;
    for (uint64_t b = 0; b < nb; b++) {
        const float *x = src + b * 32;
        float amax = 0.f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
        volatile float d = amax / 127.f;
        volatile float id = d > 0.f ? 1.f / d : 0.f;
        uint8_t *o = dst + b * 34;
        uint16_t h = q4o_f32_to_f16(d);
        memcpy(o, &h, 2);
        for (int i = 0; i < 32; i++) {
            int q = (int)rintf(x[i] * id);
            if (q > 127) q = 127;
            if (q < -127) q = -127;
            o[2 + i] = (uint8_t)(int8_t)q;
        }
    }
}
/* Dequantiser: restates dequant_q8_0 (src/q4_quant.c:123-132): (float)code * f16->f32(scale). */
Q4O_API void q4o_dequant_q8_0(const uint8_t *src, uint64_t n, float *dst) {
    const uint64_t nb = n / 32;
    for (uint64_t b = 0; b < nb; b++) {
        uint16_t h;
        memcpy(&h, src + b * 34, 2);
        const float d = q4o_f16_to_f32(h);
        const int8_t *qs = (const int8_t *)(src + b * 34 + 2);
        for (int j = 0; j < 32; j++) dst[b * 32 + j] = (float)qs[j] * d;
    }
}
/* Bytes of one (token, kv head) row: kv_token_bytes / n_kvh, src/q4_fwd.c:644-650. */
static size_t row_bytes(uint32_t hd, int kind) {
    return kind == 2 ? (size_t)(hd / 32u) * 34u : (size_t)hd * (kind == 1 ? 2u : 4u);
}
Q4O_API uint64_t q4o_kv_token_bytes(uint32_t n_kvh, uint32_t hd, int kind) {
    return (uint64_t)n_kvh * row_bytes(hd, kind);
}
/* kv_write for `rows` tokens (src/q4_fwd.c:657-661): quantise / convert / copy n = rows*kvw floats. */
Q4O_API void q4o_kv_write(void *dst, const float *src, uint64_t n, int kind) {
    if (kind == 2) q4o_quant_q8_0(src, (uint8_t *)dst, n);
    else if (kind == 1) q4o_f32_to_f16_n(src, (uint16_t *)dst, n);
    else memcpy(dst, src, n * sizeof(float));
}
static void load_row(const uint8_t *cache, uint32_t n_kvh, uint32_t hd, int kind, uint32_t p,
                     uint32_t kh, float *dst) {
    const uint8_t *r = cache + ((size_t)p * n_kvh + kh) * row_bytes(hd, kind);
    if (kind == 2) q4o_dequant_q8_0(r, hd, dst);
    else if (kind == 1) {
        for (uint32_t i = 0; i < hd; i++) {
            uint16_t h;
            memcpy(&h, r + 2 * i, 2);
            dst[i] = q4o_f16_to_f32(h);
        }
    } else memcpy(dst, r, (size_t)hd * 4);
}

/* ------------------------------------------------------------------ RoPE / prep -------- */
/* Interleaved-pair rotary embedding on the first n_rot dims: the GPU formula
 * (src/q4_rocm.cu:6253-6261; CPU twin rope_head, src/q4_fwd.c:231-247, equal when the
 * fourth rope section is empty). */
Q4O_API void q4o_rope(float *x, uint32_t n_rot, int32_t pos, float base) {
    uint32_t np = n_rot / 2;
    for (uint32_t p = 0; p < np; p++) {
        float freq = powf(base, -(float)p / (float)np);
        float ang = (float)pos * freq;
        float c = cosf(ang), si = sinf(ang);
        float x0 = x[2 * p], x1 = x[2 * p + 1];
        x[2 * p] = x0 * c - x1 * si;
        x[2 * p + 1] = x0 * si + x1 * c;
    }
}
/* cos/sin table [n_pos][n_rot/2][2] so a device kernel can be checked bit-for-bit without
 * depending on its libm. */
Q4O_API void q4o_rope_table(uint32_t n_rot, int32_t pos0, uint32_t n_pos, float base, float *cs) {
    uint32_t np = n_rot / 2;
    for (uint32_t t = 0; t < n_pos; t++)
        for (uint32_t p = 0; p < np; p++) {
            float freq = powf(base, -(float)p / (float)np);
            float ang = (float)(pos0 + (int32_t)t) * freq;
            cs[((size_t)t * np + p) * 2] = cosf(ang);
            cs[((size_t)t * np + p) * 2 + 1] = sinf(ang);
        }
}
static void rms_scale(const float *x, const float *w, float *y, uint32_t n, float eps) {
    /* src/q4_rocm.cu:6240-6251: fp32 sum of squares, rsqrt(ss/hd + eps), times weight */
    float ss = 0.f;
    for (uint32_t i = 0; i < n; i++) ss += x[i] * x[i];
    float sc = 1.0f / sqrtf(ss / (float)n + eps);
    for (uint32_t i = 0; i < n; i++) y[i] = x[i] * sc * (w ? w[i] : 1.f);
}
/* qsa_q_prep_k (src/q4_rocm.cu:6229-6262): split [q|gate], RMSNorm q, RoPE at pos0+t. */
Q4O_API void q4o_q_prep(const float *qg, const float *wn, float *q, float *g, uint32_t n_head,
                        uint32_t hd, uint32_t n_rot, int32_t pos0, float base, float eps,
                        uint32_t n_tok) {
    for (uint32_t t = 0; t < n_tok; t++)
        for (uint32_t h = 0; h < n_head; h++) {
            const float *src = qg + ((size_t)t * n_head + h) * hd * 2;
            float *qd = q + ((size_t)t * n_head + h) * hd, *gd = g + ((size_t)t * n_head + h) * hd;
            memcpy(gd, src + hd, (size_t)hd * 4);
            rms_scale(src, wn, qd, hd, eps);
            q4o_rope(qd, n_rot, pos0 + (int32_t)t, base);
        }
}
/* qsa_k_prep_k (src/q4_rocm.cu:6264-6294): RMSNorm + RoPE in place. */
Q4O_API void q4o_k_prep(float *k, const float *wn, uint32_t n_kvh, uint32_t hd, uint32_t n_rot,
                        int32_t pos0, float base, float eps, uint32_t n_tok) {
    for (uint32_t t = 0; t < n_tok; t++)
        for (uint32_t h = 0; h < n_kvh; h++) {
            float *kh = k + ((size_t)t * n_kvh + h) * hd;
            rms_scale(kh, wn, kh, hd, eps);
            q4o_rope(kh, n_rot, pos0 + (int32_t)t, base);
        }
}

/* ------------------------------------------------------------------ attention ---------- */
/* One (token, head): scalar two-pass softmax attention, the loops of qsa_one
 * (src/q4_fwd.c:365-397; the same arithmetic is inlined in src/q4_test.c:155-182), run over
 * rows dequantised from the cache.  `pos` lists the positions (entries < 0 are padding and are
 * skipped, src/q4_rocm.cu:6852-6865); all masked -> output 0 (:7001).  acc64 accumulates in
 * fp64 to separate oracle noise from kernel error. */
static void attn_one(const float *q, const uint8_t *kc, const uint8_t *vc, const float *gate,
                     float *out, uint32_t n_kvh, uint32_t hd, int kind, uint32_t kh, float scale,
                     const int32_t *pos, uint32_t n_pos, uint32_t dense_n, int acc64, float *sc,
                     float *row) {
    uint32_t n = pos ? n_pos : dense_n;
    if (!acc64) {
        float m = -INFINITY;
        for (uint32_t j = 0; j < n; j++) {
            int32_t p = pos ? pos[j] : (int32_t)j;
            if (p < 0) { sc[j] = -INFINITY; continue; }
            load_row(kc, n_kvh, hd, kind, (uint32_t)p, kh, row);
            float dot = 0;
            for (uint32_t i = 0; i < hd; i++) dot += q[i] * row[i];
            sc[j] = dot * scale;
            if (sc[j] > m) m = sc[j];
        }
        float sum = 0;
        for (uint32_t j = 0; j < n; j++) {
            sc[j] = (sc[j] == -INFINITY) ? 0.f : expf(sc[j] - m);
            sum += sc[j];
        }
        float inv = sum > 0 ? 1.f / sum : 0;
        for (uint32_t i = 0; i < hd; i++) out[i] = 0.f;
        for (uint32_t j = 0; j < n; j++) {
            int32_t p = pos ? pos[j] : (int32_t)j;
            if (p < 0) continue;
            float w = sc[j] * inv;
            load_row(vc, n_kvh, hd, kind, (uint32_t)p, kh, row);
            for (uint32_t i = 0; i < hd; i++) out[i] += w * row[i];
        }
        if (gate)
            for (uint32_t i = 0; i < hd; i++) out[i] *= 1.0f / (1.0f + expf(-gate[i]));
    } else {
        double m = -INFINITY;
        double *s64 = (double *)malloc(sizeof(double) * (n ? n : 1));
        double *o64 = (double *)calloc(hd, sizeof(double));
        for (uint32_t j = 0; j < n; j++) {
            int32_t p = pos ? pos[j] : (int32_t)j;
            if (p < 0) { s64[j] = -INFINITY; continue; }
            load_row(kc, n_kvh, hd, kind, (uint32_t)p, kh, row);
            double dot = 0;
            for (uint32_t i = 0; i < hd; i++) dot += (double)q[i] * (double)row[i];
            s64[j] = dot * (double)scale;
            if (s64[j] > m) m = s64[j];
        }
        double sum = 0;
        for (uint32_t j = 0; j < n; j++) {
            s64[j] = (s64[j] == -INFINITY) ? 0.0 : exp(s64[j] - m);
            sum += s64[j];
        }
        double inv = sum > 0 ? 1.0 / sum : 0;
        for (uint32_t j = 0; j < n; j++) {
            int32_t p = pos ? pos[j] : (int32_t)j;
            if (p < 0) continue;
            load_row(vc, n_kvh, hd, kind, (uint32_t)p, kh, row);
            for (uint32_t i = 0; i < hd; i++) o64[i] += s64[j] * inv * (double)row[i];
        }
        for (uint32_t i = 0; i < hd; i++)
            out[i] = (float)(gate ? o64[i] / (1.0 + exp(-(double)gate[i])) : o64[i]);
        free(s64);
        free(o64);
    }
}

/* Decode / causal-batch attention over the cache, reference semantics of q4_hip_qsa_decode_n and
 * q4_hip_qsa_decode_idx (src/q4_rocm.cu:7249-7364):
 *  dense  (idx == NULL): token t attends [0, min(kv_base+t+1, max_kv)) (:6773-6774,7032-7033);
 *  indexed: token t attends idx[t*width*(1 or n_kvh) ...]; idx_kvh_stride = 0 means one list per
 *  token shared by all kv heads (the reference), otherwise the list of kv head kh starts
 *  idx_kvh_stride entries after that of kh-1 (the benchmark configs: one list per kv head) and
 *  token t's lists start at t*n_kvh*idx_kvh_stride.
 * q,out,gate: [n_tok][n_head][hd] fp32; gate may be NULL (no gate).  threads > 1 uses OpenMP
 * over (token, head).  Returns 0 on success. */
Q4O_API int q4o_attn(const float *q, const void *kcache, const void *vcache, const float *gate,
                     float *out, uint32_t n_head, uint32_t n_kvh, uint32_t hd, uint32_t n_tok,
                     uint32_t kv_base, uint32_t max_kv, float scale, int kind, const int32_t *idx,
                     uint32_t width, uint32_t idx_kvh_stride, int acc64, int threads) {
    if (!q || !kcache || !vcache || !out || !n_head || !n_kvh || !hd || !n_tok) return 1;
    if (n_head % n_kvh || (kind == 2 && hd % 32)) return 1;
    const uint32_t gqa = n_head / n_kvh;
    const long total = (long)n_tok * n_head;
    uint32_t maxn = idx ? width : (kv_base + n_tok < max_kv ? kv_base + n_tok : max_kv);
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
#endif
    {
        float *sc = (float *)malloc(sizeof(float) * (maxn ? maxn : 1));
        float *row = (float *)malloc(sizeof(float) * hd);
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 1)
#endif
        for (long w = 0; w < total; w++) {
            uint32_t t = (uint32_t)(w / n_head), h = (uint32_t)(w % n_head), kh = h / gqa;
            uint32_t n_kv = kv_base + t + 1;
            if (n_kv > max_kv) n_kv = max_kv;
            const int32_t *pos = NULL;
            if (idx)
                pos = idx_kvh_stride ? idx + ((size_t)t * n_kvh + kh) * idx_kvh_stride
                                     : idx + (size_t)t * width;
            attn_one(q + ((size_t)t * n_head + h) * hd, (const uint8_t *)kcache,
                     (const uint8_t *)vcache, gate ? gate + ((size_t)t * n_head + h) * hd : NULL,
                     out + ((size_t)t * n_head + h) * hd, n_kvh, hd, kind, kh, scale, pos, width,
                     n_kv, acc64, sc, row);
        }
        free(sc);
        free(row);
    }
    (void)threads;
    return 0;
}

/* Online-softmax partial over positions [p0, p1) of the list (or of [0,n_kv) when idx is NULL) for
 * one decode token: part[h] = {m, l, acc[hd]}, the record gqa_dec_split_k writes
 * (src/q4_rocm.cu:6780,6957-6963): acc = sum exp(s-m) v, l = sum exp(s-m), l = 0 when the slice
 * holds no live position. */
Q4O_API int q4o_attn_partial(const float *q, const void *kcache, const void *vcache, float *part,
                             uint32_t n_head, uint32_t n_kvh, uint32_t hd, float scale, int kind,
                             const int32_t *idx, uint32_t idx_kvh_stride, uint32_t p0, uint32_t p1) {
    if (!q || !kcache || !vcache || !part || !n_head || !n_kvh || !hd) return 1;
    const uint32_t gqa = n_head / n_kvh;
    float *row = (float *)malloc(sizeof(float) * hd);
    uint32_t n = p1 > p0 ? p1 - p0 : 0;
    float *sc = (float *)malloc(sizeof(float) * (n ? n : 1));
    for (uint32_t h = 0; h < n_head; h++) {
        uint32_t kh = h / gqa;
        const int32_t *pos = idx ? idx + (size_t)kh * idx_kvh_stride : NULL;
        float *pv = part + (size_t)h * (hd + 2);
        float m = -INFINITY;
        for (uint32_t j = 0; j < n; j++) {
            int32_t p = pos ? pos[p0 + j] : (int32_t)(p0 + j);
            if (p < 0) { sc[j] = -INFINITY; continue; }
            load_row((const uint8_t *)kcache, n_kvh, hd, kind, (uint32_t)p, kh, row);
            float dot = 0;
            for (uint32_t i = 0; i < hd; i++) dot += q[(size_t)h * hd + i] * row[i];
            sc[j] = dot * scale;
            if (sc[j] > m) m = sc[j];
        }
        float l = 0;
        for (uint32_t i = 0; i < hd; i++) pv[2 + i] = 0.f;
        for (uint32_t j = 0; j < n; j++) {
            int32_t p = pos ? pos[p0 + j] : (int32_t)(p0 + j);
            if (p < 0 || sc[j] == -INFINITY) continue;
            float w = expf(sc[j] - m);
            l += w;
            load_row((const uint8_t *)vcache, n_kvh, hd, kind, (uint32_t)p, kh, row);
            for (uint32_t i = 0; i < hd; i++) pv[2 + i] += w * row[i];
        }
        pv[0] = l > 0 ? m : 0.f;
        pv[1] = l;
    }
    free(row);
    free(sc);
    return 0;
}

/* Merge of n_parts partial records per head (gqa_dec_comb_k, src/q4_rocm.cu:6990-7010):
 * M = max m_s; w_s = l_s > 0 ? exp(m_s - M) : 0; out = sum w_s acc_s / sum w_s l_s, times
 * sigmoid(gate) when a gate is given.  parts: [n_parts][n_head][hd+2]. */
Q4O_API void q4o_lse_merge(const float *parts, uint32_t n_parts, uint32_t n_head, uint32_t hd,
                           const float *gate, float *out) {
    for (uint32_t h = 0; h < n_head; h++) {
        float M = -1.0e30f;
        for (uint32_t s = 0; s < n_parts; s++) {
            const float *pv = parts + ((size_t)s * n_head + h) * (hd + 2);
            if (pv[1] > 0.f) M = fmaxf(M, pv[0]);
        }
        float wsum = 0.f;
        for (uint32_t i = 0; i < hd; i++) out[(size_t)h * hd + i] = 0.f;
        for (uint32_t s = 0; s < n_parts; s++) {
            const float *pv = parts + ((size_t)s * n_head + h) * (hd + 2);
            float ws = pv[1] > 0.f ? expf(pv[0] - M) : 0.f;
            wsum += ws * pv[1];
            for (uint32_t i = 0; i < hd; i++) out[(size_t)h * hd + i] += ws * pv[2 + i];
        }
        float inv = wsum > 0.f ? 1.f / wsum : 0.f;
        for (uint32_t i = 0; i < hd; i++) {
            float gv = gate ? 1.f / (1.f + expf(-gate[(size_t)h * hd + i])) : 1.f;
            out[(size_t)h * hd + i] = out[(size_t)h * hd + i] * inv * gv;
        }
    }
}

/* Many independent decode-attention problems in one call, OpenMP over (item, head): the CPU
 * baseline of the batched multi-session decode.  Each item is one q4o_attn call with n_tok = 1. */
typedef struct {
    const float *q;
    const void *kcache, *vcache;
    const float *gate;
    float *out;
    const int32_t *idx;
    uint32_t width, idx_kvh_stride, kv_base, max_kv;
} q4o_item;
Q4O_API int q4o_attn_items(const q4o_item *items, uint32_t n_items, uint32_t n_head, uint32_t n_kvh,
                           uint32_t hd, float scale, int kind, int threads) {
    if (!items || !n_items || !n_head || !n_kvh || !hd || n_head % n_kvh) return 1;
    const uint32_t gqa = n_head / n_kvh;
    const long total = (long)n_items * n_head;
    uint32_t maxn = 1;
    for (uint32_t i = 0; i < n_items; i++) {
        uint32_t n = items[i].idx ? items[i].width : items[i].kv_base + 1;
        if (n > maxn) maxn = n;
    }
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
#endif
    {
        float *sc = (float *)malloc(sizeof(float) * maxn);
        float *row = (float *)malloc(sizeof(float) * hd);
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 1)
#endif
        for (long w = 0; w < total; w++) {
            const q4o_item *it = items + w / n_head;
            uint32_t h = (uint32_t)(w % n_head), kh = h / gqa;
            uint32_t n_kv = it->kv_base + 1 > it->max_kv ? it->max_kv : it->kv_base + 1;
            const int32_t *pos = NULL;
            if (it->idx) pos = it->idx_kvh_stride ? it->idx + (size_t)kh * it->idx_kvh_stride : it->idx;
            attn_one(it->q + (size_t)h * hd, (const uint8_t *)it->kcache, (const uint8_t *)it->vcache,
                     it->gate ? it->gate + (size_t)h * hd : NULL, it->out + (size_t)h * hd, n_kvh, hd, kind,
                     kh, scale, pos, it->width, n_kv, 0, sc, row);
        }
        free(sc);
        free(row);
    }
    (void)threads;
    return 0;
}

/* ------------------------------------------------------------------ QSA indexer -------- */
/* qsa_pool_k (src/q4_rocm.cu:7366-7402): block b = mean of `ratio` raw fp16 keys (summed in token
 * order, divided once), RMSNorm whose sum of squares is the kernel's shared-memory tree
 * (red[d] += red[d + st], st = 64, 32, .. 1), weight, RoPE at the block's first position. */
Q4O_API void q4o_ix_pool(const uint16_t *raw, float *pool, const float *wn, uint32_t hd, uint32_t ratio,
                         uint32_t b0, uint32_t b1, uint32_t n_rot, float base, float eps) {
    if (hd != 128) return;
    for (uint32_t b = b0; b < b1; b++) {
        float v[128], red[128];
        const uint16_t *src = raw + (size_t)b * ratio * hd;
        for (uint32_t d = 0; d < hd; d++) {
            float s = 0.f;
            for (uint32_t j = 0; j < ratio; j++) s += q4o_f16_to_f32(src[(size_t)j * hd + d]);
            v[d] = s / (float)ratio;
            red[d] = v[d] * v[d];
        }
        for (uint32_t st = 64; st > 0; st >>= 1)
            for (uint32_t d = 0; d < st; d++) red[d] += red[d + st];
        float inv = 1.f / sqrtf(red[0] / (float)hd + eps);
        for (uint32_t d = 0; d < hd; d++) v[d] = v[d] * inv * (wn ? wn[d] : 1.f);
        for (uint32_t d = 0; d + 1 < hd && d < n_rot; d += 2) {
            uint32_t p = d >> 1;
            float freq = powf(base, -(float)p / (float)(n_rot / 2u));
            float ang = (float)(b * ratio) * freq;
            float c = cosf(ang), si = sinf(ang);
            float x0 = v[d], x1 = v[d + 1];
            v[d] = x0 * c - x1 * si;
            v[d + 1] = x0 * si + x1 * c;
        }
        memcpy(pool + (size_t)b * hd, v, sizeof(float) * hd);
    }
}

/* qsa_score_k (src/q4_rocm.cu:7405-7436): score[t][b] = sum_h relu(q[t][h] . pool[b]) for the blocks
 * token t can see (b < (pos + 1) / ratio), else -1e30.  `dot += q[i] * k[i]` in dim order is one
 * fused multiply-add per term on the GPU (hipcc contracts a * b + c by default), restated as fmaf. */
Q4O_API void q4o_ix_score(const float *q, const float *pool, float *score, uint32_t n_tok, uint32_t n_blocks,
                          uint32_t stride, uint32_t n_head, uint32_t hd, uint32_t pos0, uint32_t ratio) {
    for (uint32_t t = 0; t < n_tok; t++) {
        uint32_t pos = pos0 + t, n_vis = ratio ? (pos + 1) / ratio : 0;
        for (uint32_t b = 0; b < n_blocks; b++) {
            float s = -1.0e30f;
            if (b < n_vis) {
                s = 0.f;
                const float *kb = pool + (size_t)b * hd;
                for (uint32_t h = 0; h < n_head; h++) {
                    const float *qq = q + ((size_t)t * n_head + h) * hd;
                    float dot = 0.f;
                    for (uint32_t i = 0; i < hd; i++) dot = fmaf(qq[i], kb[i], dot);
                    s += fmaxf(dot, 0.f);
                }
            }
            score[(size_t)t * stride + b] = s;
        }
    }
}

static uint32_t ix_key(float f) {   /* qsa_tk_xkey (:7464-7467): order-preserving uint of a float */
    uint32_t u;
    memcpy(&u, &f, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
static int ix_cmp_desc(const void *a, const void *b) {
    uint32_t x = *(const uint32_t *)a, y = *(const uint32_t *)b;
    return x < y ? 1 : x > y ? -1 : 0;
}
/* qsa_topk_k + qsa_write_sel (src/q4_rocm.cu:7722-7846): the need = min(n_vis, k_blk) best blocks by
 * (score descending, index ascending), emitted as: every block above the threshold key in ascending
 * index order, then threshold ties in ascending index order; each expands to its `ratio` positions;
 * then the positions of the newest partial block up to pos; then -1.  All blocks fit (need == n_vis):
 * the dense prefix 0..pos, -1 beyond. */
Q4O_API void q4o_ix_topk(const float *score, int32_t *sel, uint32_t n_tok, uint32_t stride, uint32_t k_blk,
                         uint32_t ratio, uint32_t pos0, uint32_t width) {
    for (uint32_t t = 0; t < n_tok; t++) {
        uint32_t pos = pos0 + t, n_vis = ratio ? (pos + 1) / ratio : 0;
        uint32_t need = n_vis < k_blk ? n_vis : k_blk;
        const float *row = score + (size_t)t * stride;
        int32_t *out = sel + (size_t)t * width;
        if (need == n_vis) {
            for (uint32_t w = 0; w < width; w++) out[w] = w <= pos ? (int32_t)w : -1;
            continue;
        }
        uint32_t *keys = (uint32_t *)malloc(sizeof(uint32_t) * n_vis);
        for (uint32_t b = 0; b < n_vis; b++) keys[b] = ix_key(row[b]);
        qsort(keys, n_vis, sizeof(uint32_t), ix_cmp_desc);
        uint32_t thr = keys[need - 1];
        free(keys);
        int32_t *chosen = (int32_t *)malloc(sizeof(int32_t) * need);
        uint32_t n = 0;
        for (uint32_t b = 0; b < n_vis && n < need; b++)
            if (ix_key(row[b]) > thr) chosen[n++] = (int32_t)b;
        for (uint32_t b = 0; b < n_vis && n < need; b++)
            if (ix_key(row[b]) == thr) chosen[n++] = (int32_t)b;
        uint32_t w = 0;
        for (uint32_t i = 0; i < n && w < width; i++)
            for (uint32_t j = 0; j < ratio && w < width; j++) out[w++] = (int32_t)((uint32_t)chosen[i] * ratio + j);
        uint32_t tail = n_vis * ratio;
        while (tail <= pos && w < width) out[w++] = (int32_t)tail++;
        while (w < width) out[w++] = -1;
        free(chosen);
    }
}

Q4O_API int q4o_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Processors this process may run on, whatever OMP_NUM_THREADS says (launchers of multi-process jobs
 * set it to 1); 1 without OpenMP.  The timed baseline passes this as its explicit thread count. */
Q4O_API int q4o_host_procs(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}
