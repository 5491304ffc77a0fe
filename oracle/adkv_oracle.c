/* CPU restatement of the ADKV hot path in plain C (TEST INFRASTRUCTURE, not product code).
 *
 * Used only as the checker in tests and as the timed CPU baseline of bench.py.  The
 * product library never links or calls it.
 *
 * Follows the reference project at:
 *   - recurrence: src/adkv/train/train_model.py:6-22 and :70-81 (same operation order as
 *     the Triton evaluation kernel, src/adkv/hf/llama_adkv_eval.py:87-97);
 *   - packed layout: src/adkv/kernel/gemv.cu:266-305, :502-510 (4-bit); the 2-bit layout
 *     (16 tokens per word, code stored as q + 2) is defined by this project;
 *   - decode step: src/adkv/kernel/gemv.cu:744-814, :1105-1159 and the caller's glue
 *     src/adkv/hf/llama_adkv.py:263-276.
 *
 * Parity pin: checked bit for bit against oracle/adkv_oracle.py, which is itself checked
 * against fixtures produced by executing the reference's torch code (tests/golden/).
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (no FMA contraction, so every
 * float operation below is one IEEE operation, as in the reference's eager torch code).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_EPS 1e-8f /* train_model.py:9 */

static float h2f(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

/* One token of one channel: quantise x against (zp, s) -- train_model.py:72, :8-17. */
static inline float quant1(float x, float zp, float s, float lo, float hi, float *rh)
{
    float ss = fmaxf(s, ORACLE_EPS);
    float q = clampf(rintf((x - zp) / ss), lo, hi);
    *rh = q * ss;
    return q;
}

/* State update from the code alone -- train_model.py:77-81. */
static inline void advance1(float q, float rh, float *zp, float *s, float alpha, float beta, float target,
                            float smin, float smax)
{
    *zp = *zp + alpha * rh;
    float err = fabsf(q) - target;
    *s = clampf(*s + *s * beta * err, smin, smax);
}

/* torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the timed baseline sets the count itself. */
void oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Prefill quantise: x [B,H,T,D] fp16 -> words [B,H,n_super_cap,D]; params [5][H*D] float
 * (zp_init, scale_init, alpha, beta, target); tail (nullable) [B,H,2,D] float. */
int oracle_encode(uint32_t *words, const uint16_t *x, const float *params, int B, int H, int T, int D,
                  int n_super_cap, int bits, float smin, float smax, float *tail)
{
    const int tpw = 32 / bits, bias = 1 << (bits - 1);
    const float lo = (float)-bias, hi = (float)(bias - 1);
    const int need = (T + tpw - 1) / tpw;
    if (need > n_super_cap) return -1;
    const size_t HD = (size_t)H * D;
#pragma omp parallel for schedule(dynamic, 1)
    for (int bh = 0; bh < B * H; ++bh) {
        const int h = bh % H;
        const float *zp0 = params + 0 * HD + (size_t)h * D, *s0 = params + 1 * HD + (size_t)h * D;
        const float *al = params + 2 * HD + (size_t)h * D, *be = params + 3 * HD + (size_t)h * D;
        const float *tg = params + 4 * HD + (size_t)h * D;
        float *zp = (float *)malloc(sizeof(float) * D), *s = (float *)malloc(sizeof(float) * D);
        memcpy(zp, zp0, sizeof(float) * D);
        memcpy(s, s0, sizeof(float) * D);
        uint32_t *w = words + (size_t)bh * n_super_cap * D;
        memset(w, 0, sizeof(uint32_t) * (size_t)need * D);
        const uint16_t *xb = x + (size_t)bh * T * D;
        for (int t = 0; t < T; ++t) {
            uint32_t *wr = w + (size_t)(t / tpw) * D;
            const int sh = bits * (t % tpw);
            for (int c = 0; c < D; ++c) {
                float rh, q = quant1(h2f(xb[(size_t)t * D + c]), zp[c], s[c], lo, hi, &rh);
                wr[c] |= (uint32_t)((int)q + bias) << sh;
                advance1(q, rh, &zp[c], &s[c], al[c], be[c], tg[c], smin, smax);
            }
        }
        if (tail) {
            memcpy(tail + (size_t)bh * 2 * D, zp, sizeof(float) * D);
            memcpy(tail + (size_t)bh * 2 * D + D, s, sizeof(float) * D);
        }
        free(zp);
        free(s);
    }
    return 0;
}

/* Replay tokens [0,T) of one stream; calls back per token with x_hat[D]. Leaves (zp,s) = state after T-1. */
static void replay_stream(const uint32_t *w, int T, int D, int bits, const float *al, const float *be,
                          const float *tg, float smin, float smax, float *zp, float *s, float *xhat_all)
{
    const int tpw = 32 / bits, bias = 1 << (bits - 1);
    const uint32_t field = (1u << bits) - 1u;
    for (int t = 0; t < T; ++t) {
        const uint32_t *wr = w + (size_t)(t / tpw) * D;
        const int sh = bits * (t % tpw);
        float *xh = xhat_all + (size_t)t * D;
        for (int c = 0; c < D; ++c) {
            float q = (float)((int)((wr[c] >> sh) & field) - bias);
            float ss = fmaxf(s[c], ORACLE_EPS);
            float rh = q * ss;
            xh[c] = rh + zp[c];
            advance1(q, rh, &zp[c], &s[c], al[c], be[c], tg[c], smin, smax);
        }
    }
}

/* Quantise x_new with the current state, write it as token T, return x_hat (gemv.cu:744-764). */
static void append_stream(uint32_t *w, int T, int D, int bits, const uint16_t *x_new, const float *zp,
                          const float *s, float *xhat)
{
    const int tpw = 32 / bits, bias = 1 << (bits - 1);
    const float lo = (float)-bias, hi = (float)(bias - 1);
    const uint32_t field = (1u << bits) - 1u;
    uint32_t *wr = w + (size_t)(T / tpw) * D;
    const int sh = bits * (T % tpw);
    for (int c = 0; c < D; ++c) {
        float rh, q = quant1(h2f(x_new[c]), zp[c], s[c], lo, hi, &rh);
        wr[c] = (wr[c] & ~(field << sh)) | ((uint32_t)((int)q + bias) << sh);
        xhat[c] = rh + zp[c];
    }
}

/* One fused decode step (llama_adkv.py:263-276 composed with gemv.cu semantics).
 * q [B,Hq,D] fp16; caches [B,Hkv,n_super_cap,D] words; k_new/v_new [B,Hkv,D] fp16;
 * kparams/vparams [5][Hkv*D] float; mask (nullable) [B, T+1] float, shared by all heads;
 * out [B,Hq,D] float.  Appends token T to both caches.  first_stream/n_streams select a
 * contiguous range of (b, kv-head) streams so a bounded sample can be timed. */
int oracle_decode_attn(const uint16_t *q, uint32_t *kw, uint32_t *vw, const uint16_t *k_new,
                       const uint16_t *v_new, const float *kparams, const float *vparams, const float *mask,
                       float *out, int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits,
                       float scaling, float smin, float smax, int first_stream, int n_streams)
{
    const int tpw = 32 / bits, G = Hq / Hkv;
    if (T / tpw >= n_super_cap) return -1;
    const size_t HD = (size_t)Hkv * D;
    if (n_streams < 0) n_streams = B * Hkv - first_stream;
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < n_streams; ++i) {
        const int bh = first_stream + i, b = bh / Hkv, h = bh % Hkv;
        float *xh = (float *)malloc(sizeof(float) * (size_t)(T + 1) * D);
        float *zp = (float *)malloc(sizeof(float) * D), *s = (float *)malloc(sizeof(float) * D);
        double *logit = (double *)malloc(sizeof(double) * (size_t)(T + 1) * G);
        /* K */
        memcpy(zp, kparams + 0 * HD + (size_t)h * D, sizeof(float) * D);
        memcpy(s, kparams + 1 * HD + (size_t)h * D, sizeof(float) * D);
        uint32_t *kws = kw + (size_t)bh * n_super_cap * D;
        replay_stream(kws, T, D, bits, kparams + 2 * HD + (size_t)h * D, kparams + 3 * HD + (size_t)h * D,
                      kparams + 4 * HD + (size_t)h * D, smin, smax, zp, s, xh);
        append_stream(kws, T, D, bits, k_new + (size_t)bh * D, zp, s, xh + (size_t)T * D);
        for (int g = 0; g < G; ++g) {
            const uint16_t *qv = q + ((size_t)b * Hq + (size_t)h * G + g) * D;
            double m = -INFINITY;
            for (int t = 0; t <= T; ++t) {
                double acc = 0.0;
                for (int c = 0; c < D; ++c) acc += (double)h2f(qv[c]) * (double)xh[(size_t)t * D + c];
                acc = acc * (double)scaling + (mask ? (double)mask[(size_t)b * (T + 1) + t] : 0.0);
                logit[(size_t)g * (T + 1) + t] = acc;
                if (acc > m) m = acc;
            }
            if (!isfinite(m)) m = 0.0;
            double l = 0.0;
            for (int t = 0; t <= T; ++t) {
                double e = exp(logit[(size_t)g * (T + 1) + t] - m);
                logit[(size_t)g * (T + 1) + t] = e;
                l += e;
            }
            for (int t = 0; t <= T; ++t) logit[(size_t)g * (T + 1) + t] /= l;
        }
        /* V */
        memcpy(zp, vparams + 0 * HD + (size_t)h * D, sizeof(float) * D);
        memcpy(s, vparams + 1 * HD + (size_t)h * D, sizeof(float) * D);
        uint32_t *vws = vw + (size_t)bh * n_super_cap * D;
        replay_stream(vws, T, D, bits, vparams + 2 * HD + (size_t)h * D, vparams + 3 * HD + (size_t)h * D,
                      vparams + 4 * HD + (size_t)h * D, smin, smax, zp, s, xh);
        append_stream(vws, T, D, bits, v_new + (size_t)bh * D, zp, s, xh + (size_t)T * D);
        for (int g = 0; g < G; ++g) {
            float *o = out + ((size_t)b * Hq + (size_t)h * G + g) * D;
            for (int c = 0; c < D; ++c) {
                double acc = 0.0;
                for (int t = 0; t <= T; ++t) acc += logit[(size_t)g * (T + 1) + t] * (double)xh[(size_t)t * D + c];
                o[c] = (float)acc;
            }
        }
        free(xh); free(zp); free(s); free(logit);
    }
    return 0;
}
