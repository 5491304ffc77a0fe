// Part of libadkv_b200.so (sm_100a).  See include/adkv_b200.h for the contract of every entry point
// and the reference interface each one replaces.
#include "adkv_host.h"

#include <algorithm>
using std::min;

namespace adkv {

// =========================================================================================
// Prefill quantise + pack (canonical arithmetic).  One 64-thread CTA per (batch, head); a thread
// owns two adjacent channels: per token the warp reads 128 contiguous bytes of the fp16 row
// (half2 per lane) and per supergroup it writes 256 contiguous bytes (uint2 per lane).  The next
// word's tokens are fetched while the current word is quantised.
constexpr int kEncThreads = kD / 2;
constexpr int kEncStages = 2;   // 32-token (8 KB) tiles of fp16 input in flight per CTA.  16 KB per CTA lets 14 CTAs share an SM,
                                // which is what a launch over several layers needs (8 layers: 0.645 ms per layer with 2
                                // stages, 0.688 ms with 3); K and V of one layer are 6.9 CTAs per SM either way (0.86 ms)

// Eight tokens for the two channels of a thread,
// speculative quantiser (see quantize_spec) on the channel pair with packed fp32 arithmetic: half the
// issue slots for the adds and multiplies, every element rounded exactly as by the scalar instruction.
// Min/max, the reciprocal and the compare have no packed form and stay scalar.  Returns true when some
// code is in doubt and the group must be redone with the exactly rounded division.
// A word is assembled by shifting: every new code enters at the top (one funnel shift takes the low BITS bits of
// its source) and pushes the earlier tokens down, so after TPW tokens token 0 sits in the lowest field.
template <int BITS, bool GUARDED>
__device__ __forceinline__ bool encode_group(const __half2 *xin /* 8 rows of kD/2 */, Chan (&ch)[2],
                                             uint32_t (&word)[2], float smin, float smax, f32x2 one)
{
    using C = Codec<BITS>;
    constexpr float M = 12582912.f + float(C::BIAS);   // 1.5 * 2^23 + BIAS: the low bits of (v + M) are code + BIAS
    bool doubt = !(ch[0].s < 1e29f) || !(ch[1].s < 1e29f);   // reciprocal would flush to zero
    f32x2 zp = pk2(ch[0].zp, ch[1].zp), s = pk2(ch[0].s, ch[1].s);
    const f32x2 alpha = pk2(ch[0].alpha, ch[1].alpha), beta = pk2(ch[0].beta, ch[1].beta);
    const f32x2 neg_t = pk2(-ch[0].tc, -ch[1].tc), m2 = pk2(M, M);
    static_for<8>([&](auto jc) {
        constexpr int j = decltype(jc)::value;
        const float2 xf = __half22float2(xin[j * (kD / 2)]);
        float s0, s1;
        upk2(s, s0, s1);
        if (GUARDED) {
            s0 = fmaxf(s0, kEps);
            s1 = fmaxf(s1, kEps);
        }
        const f32x2 ss = GUARDED ? pk2(s0, s1) : s;
        float i0, i1;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(i0) : "f"(s0));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(i1) : "f"(s1));
        const f32x2 v = mul2(sub2(pk2(xf.x, xf.y), zp), pk2(i0, i1));
        float v0, v1;
        upk2(v, v0, v1);
        const f32x2 vc = pk2(fminf(fmaxf(v0, C::qlo()), C::qhi()), fminf(fmaxf(v1, C::qlo()), C::qhi()));
        const f32x2 t = add2(vc, m2);
        const f32x2 q = sub2(t, m2);
        float d0, d1;
        upk2(sub2(vc, q), d0, d1);
        // clamped quotient within 4e-6 of a rounding boundary: cannot tell which way the exact one rounds
        doubt |= !(fabsf(d0) < 0.5f - 4e-6f) || !(fabsf(d1) < 0.5f - 4e-6f);
        const f32x2 rh = mul2(q, ss);
        uint32_t t0, t1;
        asm("mov.b64 {%0, %1}, %2;" : "=r"(t0), "=r"(t1) : "l"(t));
        word[0] = __funnelshift_r(word[0], t0, BITS);
        word[1] = __funnelshift_r(word[1], t1, BITS);
        // state update, canonical order (products are added as fma(x, 1, y): see add_product2)
        zp = add_product2(mul2(alpha, rh), one, zp);
        const f32x2 s_new = add_product2(mul2(mul2(s, beta), add2(abs2(q), neg_t)), one, s);
        if (GUARDED) {
            float n0, n1;
            upk2(s_new, n0, n1);
            s = pk2(fminf(fmaxf(n0, smin), smax), fminf(fmaxf(n1, smin), smax));
        } else {
            s = s_new;
        }
    });
    upk2(zp, ch[0].zp, ch[1].zp);
    upk2(s, ch[0].s, ch[1].s);
    return doubt;
}

// One tensor (K or V) of a launch; blockIdx.y selects it, so K and V of a layer are quantised side by side.
struct EncTensor {
    uint32_t *cache;
    const __half *x;
    ParamPtrs p;
    float *tail;
    float *ckpt;   // state checkpoints [B*H][n_ckpt_cap][2][D] or nullptr; entry k = state before token (k+1)*interval
};
struct CkptSpec {
    int interval;     // tokens between checkpoints (multiple of 32), 0 = none
    int n_ckpt_cap;
    int D;            // head dim (128, 256 or 512); a CTA handles one 128-channel slice of one stream
};
constexpr int kEncMaxTensors = 16;   // tensors per launch: K and V of up to 8 layers (the struct is a kernel parameter)
struct EncBatch {
    EncTensor t[kEncMaxTensors];
};

// WIDE = false: head dim 128, all strides are compile-time constants.
template <int BITS, bool WIDE>
__global__ void __launch_bounds__(kEncThreads) encode_kernel(EncBatch batch, CkptSpec cs, int H, int T,
                                                             int n_super_cap, int t_start, float smin, float smax)
{
    using C = Codec<BITS>;
    const EncTensor &et = batch.t[blockIdx.y];
    uint32_t *__restrict__ cache = et.cache;
    const __half *__restrict__ x = et.x;
    const ParamPtrs p = et.p;
    float *__restrict__ tail = et.tail;
    const int D = WIDE ? cs.D : kD, S = WIDE ? D / kD : 1;
    const int bh = blockIdx.x / S, h = bh % H, c0 = kD * (blockIdx.x % S) + 2 * threadIdx.x;   // c0: channel in the head
    const size_t po = size_t(h) * D + c0;
    Chan ch[2];
    float beta[2], target[2];
    {
        const float2 al = __half22float2(*reinterpret_cast<const __half2 *>(p.alpha + po));
        const float2 be = __half22float2(*reinterpret_cast<const __half2 *>(p.beta + po));
        const float2 tg = __half22float2(*reinterpret_cast<const __half2 *>(p.target + po));
        float2 zp, sc;
        if (t_start > 0) {
            zp = *reinterpret_cast<const float2 *>(tail + size_t(bh) * 2 * D + c0);
            sc = *reinterpret_cast<const float2 *>(tail + size_t(bh) * 2 * D + D + c0);
        } else {
            zp = __half22float2(*reinterpret_cast<const __half2 *>(p.zp_init + po));
            sc = __half22float2(*reinterpret_cast<const __half2 *>(p.scale_init + po));
        }
        ch[0] = Chan{zp.x, sc.x, al.x, be.x, tg.x};
        ch[1] = Chan{zp.y, sc.y, al.y, be.y, tg.y};
        beta[0] = be.x; beta[1] = be.y; target[0] = tg.x; target[1] = tg.y;
    }
    SafeRange safe;
    safe.template init<BITS, 2>(beta, target, smin, smax);
    const f32x2 one = opaque_ones2();

    __shared__ alignas(128) __half buf[kEncStages][32 * kD];
    __shared__ uint64_t bar[kEncStages];
    if (threadIdx.x == 0) {
        for (int i = 0; i < kEncStages; ++i) mbar_init(&bar[i], 1);
        mbar_init_fence();
    }
    __syncthreads();

    uint2 *w = reinterpret_cast<uint2 *>(cache + size_t(bh) * n_super_cap * D + c0);       // stride D/2 per word row
    const __half2 *xs = reinterpret_cast<const __half2 *>(x + size_t(bh) * T * D + c0);    // stride D/2 per token
    const int RS = D / 2;          // row stride in global memory (uint2 words / half2 inputs)
    constexpr int SRS = kD / 2;    // row stride of the staged slice in shared memory

    // one token with a run-time field position, exactly rounded division (partial words, redone groups)
    // (the word is shifted, not indexed: see encode_group)
    auto exact_token = [&](int t, uint32_t(&word)[2]) {
        const float2 xv = __half22float2(xs[size_t(t - t_start) * RS]);
        const float xa[2] = {xv.x, xv.y};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float rh;
            const float q = quantize<BITS>(xa[c], ch[c], rh);
            word[c] = __funnelshift_r(word[c], uint32_t(int(q) + C::BIAS), BITS);
            advance_canonical(q, rh, ch[c], smin, smax);
        }
    };

    // checkpoint k is written when the state before token (k+1)*interval is reached
    float *ckpt = (et.ckpt && cs.interval > 0) ? et.ckpt + size_t(bh) * cs.n_ckpt_cap * 2 * D + c0 : nullptr;
    int next_ckpt = ckpt ? (t_start / cs.interval + 1) * cs.interval : 0x7fffffff;
    auto checkpoint = [&](int t_reached) {
        if (t_reached == next_ckpt) {
            const int k = next_ckpt / cs.interval - 1;
            if (k < cs.n_ckpt_cap) {
                *reinterpret_cast<float2 *>(ckpt + size_t(k) * 2 * D) = make_float2(ch[0].zp, ch[1].zp);
                *reinterpret_cast<float2 *>(ckpt + size_t(k) * 2 * D + D) = make_float2(ch[0].s, ch[1].s);
            }
            next_ckpt += cs.interval;
        }
    };

    const int t_end = t_start + T;
    int t = t_start;
    uint32_t word[2] = {0u, 0u};
    // a chunk that starts inside a word keeps the fields already there (moved to the top, where the shifting
    // assembly expects the tokens seen so far)
    if (t % C::TPW != 0 && t < t_end) {
        const uint2 old = w[size_t(t / C::TPW) * RS];
        const int up = BITS * (C::TPW - t % C::TPW);
        word[0] = old.x << up;
        word[1] = old.y << up;
    }
    // tokens up to the next multiple of 8
    for (; t < t_end && t % 8 != 0; ++t) {
        exact_token(t, word);
        checkpoint(t + 1);
        if ((t + 1) % C::TPW == 0) {
            w[size_t(t / C::TPW) * RS] = make_uint2(word[0], word[1]);
            word[0] = word[1] = 0u;
        }
    }
    // Groups of 8 tokens.  The fp16 rows of the stream are contiguous, so they are staged through a
    // ring of 32-token tiles filled by bulk copies (1-D TMA, issued by thread 0) that run ahead of
    // the quantiser by kEncStages - 1 tiles.
    const int n_groups = (t_end - t) / 8;
    const int n_tiles = (n_groups + 3) / 4;
    const __half *src = x + (size_t(bh) * T + (t - t_start)) * D + kD * (blockIdx.x % S);
    auto issue = [&](int i) {
        const int rows = min(4, n_groups - 4 * i) * 8;
        const uint32_t bytes = uint32_t(rows) * kD * 2;
        mbar_expect_tx(&bar[i % kEncStages], bytes);
        if (S == 1) {
            bulk_load(&buf[i % kEncStages][0], src + size_t(i) * 32 * kD, bytes, &bar[i % kEncStages]);
        } else {   // the slice's 256-byte rows are strided in global memory: one copy per token row
            for (int r = 0; r < rows; ++r)
                bulk_load(&buf[i % kEncStages][r * kD], src + (size_t(i) * 32 + r) * D, kD * 2, &bar[i % kEncStages]);
        }
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < min(kEncStages, n_tiles); ++i) issue(i);
#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
        const bool landed = mbar_wait_bounded(&bar[i % kEncStages], (i / kEncStages) & 1, kStatKWait);
        if (!__syncthreads_and(landed)) {
            // give up as one CTA; let copies already in flight land (bounded) before the memory is released
            for (int k = i; k < min(n_tiles, i + kEncStages); ++k)
                if (!mbar_wait_bounded(&bar[k % kEncStages], (k / kEncStages) & 1, kStatDrain)) break;
            return;
        }
        const int ng = min(4, n_groups - 4 * i);
#pragma unroll 1
        for (int g = 0; g < ng; ++g, t += 8) {
            const __half2 *rows = reinterpret_cast<const __half2 *>(&buf[i % kEncStages][0]) + g * 8 * SRS + threadIdx.x;
            const Chan saved[2] = {ch[0], ch[1]};
            const uint32_t word_in[2] = {word[0], word[1]};
            const bool doubt = safe.holds(ch) ? encode_group<BITS, false>(rows, ch, word, smin, smax, one)
                                              : encode_group<BITS, true>(rows, ch, word, smin, smax, one);
            if (doubt) {   // rare, per thread: redo the group from the saved state with the exact quantiser
                ch[0] = saved[0];
                ch[1] = saved[1];
                word[0] = word_in[0];
                word[1] = word_in[1];
                for (int j = 0; j < 8; ++j) exact_token(t + j, word);
            }
            checkpoint(t + 8);
            if ((t + 8) % C::TPW == 0) {
                w[size_t(t / C::TPW) * RS] = make_uint2(word[0], word[1]);
                word[0] = word[1] = 0u;
            }
        }
        __syncthreads();   // every thread is done with this stage
        if (threadIdx.x == 0 && i + kEncStages < n_tiles) issue(i + kEncStages);
    }
    // trailing tokens; unused fields of the last word stay zero
    for (; t < t_end; ++t) {
        exact_token(t, word);
        checkpoint(t + 1);
    }
    if (t % C::TPW != 0) {   // bring the tokens of the last, partial word down; its unused fields are zero
        const int down = BITS * (C::TPW - t % C::TPW);
        w[size_t(t / C::TPW) * RS] = make_uint2(word[0] >> down, word[1] >> down);
    }
    if (tail) {
        *reinterpret_cast<float2 *>(tail + size_t(bh) * 2 * D + c0) = make_float2(ch[0].zp, ch[1].zp);
        *reinterpret_cast<float2 *>(tail + size_t(bh) * 2 * D + D + c0) = make_float2(ch[0].s, ch[1].s);
    }
}

// Single-token append from the persisted tail state.
template <int BITS>
__global__ void __launch_bounds__(kD) append_kernel(EncBatch batch, CkptSpec cs, int H, int T, int n_super_cap,
                                                    float smin, float smax)
{
    using C = Codec<BITS>;
    const EncTensor &et = batch.t[blockIdx.y];
    uint32_t *__restrict__ cache = et.cache;
    const __half *__restrict__ x_new = et.x;
    const ParamPtrs p = et.p;
    float *__restrict__ tail = et.tail;
    const int D = cs.D, S = D / kD;
    const int bh = blockIdx.x / S, h = bh % H, c = kD * (blockIdx.x % S) + threadIdx.x;
    const size_t po = size_t(h) * D + c;
    Chan ch;
    ch.alpha = __half2float(p.alpha[po]);
    ch.beta = __half2float(p.beta[po]);
    ch.tc = __half2float(p.target[po]);
    ch.zp = tail[size_t(bh) * 2 * D + c];
    ch.s = tail[size_t(bh) * 2 * D + D + c];
    float rh;
    const float q = quantize<BITS>(__half2float(x_new[size_t(bh) * D + c]), ch, rh);
    uint32_t *slot = cache + (size_t(bh) * n_super_cap + T / C::TPW) * D + c;
    const int sh = BITS * (T % C::TPW);
    *slot = (*slot & ~(C::FIELD << sh)) | (uint32_t(int(q) + C::BIAS) << sh);
    advance_canonical(q, rh, ch, smin, smax);
    tail[size_t(bh) * 2 * D + c] = ch.zp;
    tail[size_t(bh) * 2 * D + D + c] = ch.s;
    if (et.ckpt && cs.interval > 0 && (T + 1) % cs.interval == 0) {
        const int k = (T + 1) / cs.interval - 1;
        if (k < cs.n_ckpt_cap) {
            float *dst = et.ckpt + (size_t(bh) * cs.n_ckpt_cap + k) * 2 * D;
            dst[c] = ch.zp;
            dst[D + c] = ch.s;
        }
    }
}

}  // namespace adkv

using namespace adkv;

ADKV_DEFINE_TU_STATUS(adkv_tu_status_encode)

static int encode_check(const void *cache, const void *x, const adkv_params *p, const void *tail, int T, int t_start)
{
    if (!cache || (!x && T > 0) || !params_ok(p)) return ADKV_E_NULL;
    if (t_start > 0 && !tail) return ADKV_E_START;
    if ((reinterpret_cast<uintptr_t>(cache) & 7u) || (reinterpret_cast<uintptr_t>(x) & 15u) ||
        (reinterpret_cast<uintptr_t>(tail) & 7u) || (reinterpret_cast<uintptr_t>(p->zp_init) & 3u) ||
        (reinterpret_cast<uintptr_t>(p->scale_init) & 3u) || (reinterpret_cast<uintptr_t>(p->alpha) & 3u) ||
        (reinterpret_cast<uintptr_t>(p->beta) & 3u) || (reinterpret_cast<uintptr_t>(p->target) & 3u))
        return ADKV_E_ALIGN;
    return 0;
}

static EncTensor enc_tensor(void *cache, const void *x, const adkv_params *p, void *tail, void *ckpt = nullptr)
{
    return EncTensor{static_cast<uint32_t *>(cache), static_cast<const __half *>(x), to_ptrs(p),
                     static_cast<float *>(tail), static_cast<float *>(ckpt)};
}

static int ckpt_check(const void *k_ckpt, const void *v_ckpt, int interval, int n_ckpt_cap, int t_last_plus_1)
{
    if (interval <= 0 || interval % 32 != 0 || n_ckpt_cap < 0) return ADKV_E_SHAPE;
    if (!k_ckpt || !v_ckpt) return ADKV_E_NULL;
    if ((reinterpret_cast<uintptr_t>(k_ckpt) & 15u) || (reinterpret_cast<uintptr_t>(v_ckpt) & 15u)) return ADKV_E_ALIGN;
    if (t_last_plus_1 / interval > n_ckpt_cap) return ADKV_E_CAPACITY;
    return 0;
}

static int launch_encode(const EncBatch &b, int n, int B, int H, int T, int D, int n_super_cap, int bits,
                         int t_start, float smin, float smax, void *stream, CkptSpec cs = CkptSpec{0, 0, 0})
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cs.D = D;
    const dim3 grid(B * H * (D / kD), n);
    if (D == kD) {
        if (bits == 4) encode_kernel<4, false><<<grid, kEncThreads, 0, s>>>(b, cs, H, T, n_super_cap, t_start, smin, smax);
        else encode_kernel<2, false><<<grid, kEncThreads, 0, s>>>(b, cs, H, T, n_super_cap, t_start, smin, smax);
    } else {
        if (bits == 4) encode_kernel<4, true><<<grid, kEncThreads, 0, s>>>(b, cs, H, T, n_super_cap, t_start, smin, smax);
        else encode_kernel<2, true><<<grid, kEncThreads, 0, s>>>(b, cs, H, T, n_super_cap, t_start, smin, smax);
    }
    return launch_status();
}

static int launch_append(const EncBatch &b, int n, int B, int H, int T, int D, int n_super_cap, int bits,
                         float smin, float smax, void *stream, CkptSpec cs = CkptSpec{0, 0, 0})
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cs.D = D;
    const dim3 grid(B * H * (D / kD), n);
    if (bits == 4) append_kernel<4><<<grid, kD, 0, s>>>(b, cs, H, T, n_super_cap, smin, smax);
    else append_kernel<2><<<grid, kD, 0, s>>>(b, cs, H, T, n_super_cap, smin, smax);
    return launch_status();
}

ADKV_HIDDEN int adkv_half_encode(void *k_cache, const void *k, const adkv_params *kp, void *k_tail, void *k_ckpt,
                                 void *v_cache, const void *v, const adkv_params *vp, void *v_tail, void *v_ckpt,
                                 int interval, int n_ckpt_cap, int n, int B, int H, int T, int D, int n_super_cap,
                                 int bits, int t_start, cudaStream_t s);
ADKV_HIDDEN int adkv_half_append(void *k_cache, const void *k_new, const adkv_params *kp, void *k_tail, void *k_ckpt,
                                 void *v_cache, const void *v_new, const adkv_params *vp, void *v_tail, void *v_ckpt,
                                 int interval, int n_ckpt_cap, int n, int B, int H, int T, int D, int n_super_cap,
                                 int bits, cudaStream_t s);

extern "C" {

int adkv_encode_kv_flags(void *k_cache, const void *k, const adkv_params *kp, void *k_tail, void *k_ckpt,
                         void *v_cache, const void *v, const adkv_params *vp, void *v_tail, void *v_ckpt,
                         int interval, int n_ckpt_cap, int B, int H, int T, int D, int n_super_cap, int bits,
                         int t_start, float scale_min, float scale_max, unsigned flags, void *stream)
{
    const bool pair = v_cache != nullptr;
    if (interval < 0 || (interval > 0 && !pair)) return ADKV_E_SHAPE;   // checkpoints are kept for K and V together
    if (!(flags & ADKV_FLAG_HALF_STATE)) {
        if (interval > 0)
            return adkv_encode_kv_ckpt(k_cache, k, kp, k_tail, k_ckpt, v_cache, v, vp, v_tail, v_ckpt, interval, n_ckpt_cap,
                                       B, H, T, D, n_super_cap, bits, t_start, scale_min, scale_max, stream);
        return pair ? adkv_encode_kv(k_cache, k, kp, k_tail, v_cache, v, vp, v_tail, B, H, T, D, n_super_cap, bits,
                                     t_start, scale_min, scale_max, stream)
                    : adkv_encode(k_cache, k, kp, k_tail, B, H, T, D, n_super_cap, bits, t_start, scale_min, scale_max,
                                  stream);
    }
    if (t_start < 0) return ADKV_E_SHAPE;
    if (int rc = encode_check(k_cache, k, kp, k_tail, T, t_start)) return rc;
    if (pair)
        if (int rc = encode_check(v_cache, v, vp, v_tail, T, t_start)) return rc;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, t_start + T)) return rc;
    if (interval > 0)
        if (int rc = ckpt_check(k_ckpt, v_ckpt, interval, n_ckpt_cap, t_start + T)) return rc;
    if (B * H == 0 || (T == 0 && !((k_tail || v_tail) && t_start == 0))) return 0;
    return adkv_half_encode(k_cache, k, kp, k_tail, k_ckpt, v_cache, v, vp, v_tail, v_ckpt, interval, n_ckpt_cap,
                            pair ? 2 : 1, B, H, T, D, n_super_cap, bits, t_start, static_cast<cudaStream_t>(stream));
}

int adkv_append_kv_flags(void *k_cache, const void *k_new, const adkv_params *kp, void *k_tail, void *k_ckpt,
                         void *v_cache, const void *v_new, const adkv_params *vp, void *v_tail, void *v_ckpt,
                         int interval, int n_ckpt_cap, int B, int H, int T, int D, int n_super_cap, int bits,
                         float scale_min, float scale_max, unsigned flags, void *stream)
{
    const bool pair = v_cache != nullptr;
    if (interval < 0 || (interval > 0 && !pair)) return ADKV_E_SHAPE;
    if (!(flags & ADKV_FLAG_HALF_STATE)) {
        if (interval > 0)
            return adkv_append_kv_ckpt(k_cache, k_new, kp, k_tail, k_ckpt, v_cache, v_new, vp, v_tail, v_ckpt, interval,
                                       n_ckpt_cap, B, H, T, D, n_super_cap, bits, scale_min, scale_max, stream);
        return pair ? adkv_append_kv(k_cache, k_new, kp, k_tail, v_cache, v_new, vp, v_tail, B, H, T, D, n_super_cap,
                                     bits, scale_min, scale_max, stream)
                    : adkv_append(k_cache, k_new, kp, k_tail, B, H, T, D, n_super_cap, bits, scale_min, scale_max, stream);
    }
    if (!k_cache || !k_new || !k_tail || !params_ok(kp)) return ADKV_E_NULL;
    if (pair && (!v_new || !v_tail || !params_ok(vp))) return ADKV_E_NULL;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, T + 1)) return rc;
    if (interval > 0)
        if (int rc = ckpt_check(k_ckpt, v_ckpt, interval, n_ckpt_cap, T + 1)) return rc;
    if (B * H == 0) return 0;
    return adkv_half_append(k_cache, k_new, kp, k_tail, k_ckpt, v_cache, v_new, vp, v_tail, v_ckpt, interval, n_ckpt_cap,
                            pair ? 2 : 1, B, H, T, D, n_super_cap, bits, static_cast<cudaStream_t>(stream));
}

int adkv_encode(void *cache, const void *x, const adkv_params *p, void *tail, int B, int H, int T, int D,
                int n_super_cap, int bits, int t_start, float scale_min, float scale_max, void *stream)
{
    if (t_start < 0) return ADKV_E_SHAPE;
    if (int rc = encode_check(cache, x, p, tail, T, t_start)) return rc;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, t_start + T)) return rc;
    if (B * H == 0 || (T == 0 && !(tail && t_start == 0))) return 0;
    EncBatch b{};
    b.t[0] = enc_tensor(cache, x, p, tail);
    return launch_encode(b, 1, B, H, T, D, n_super_cap, bits, t_start, scale_min, scale_max, stream);
}

int adkv_encode_kv(void *k_cache, const void *k, const adkv_params *kp, void *k_tail, void *v_cache, const void *v,
                   const adkv_params *vp, void *v_tail, int B, int H, int T, int D, int n_super_cap, int bits,
                   int t_start, float scale_min, float scale_max, void *stream)
{
    if (t_start < 0) return ADKV_E_SHAPE;
    if (int rc = encode_check(k_cache, k, kp, k_tail, T, t_start)) return rc;
    if (int rc = encode_check(v_cache, v, vp, v_tail, T, t_start)) return rc;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, t_start + T)) return rc;
    if (B * H == 0 || (T == 0 && !((k_tail || v_tail) && t_start == 0))) return 0;
    EncBatch b{};
    b.t[0] = enc_tensor(k_cache, k, kp, k_tail);
    b.t[1] = enc_tensor(v_cache, v, vp, v_tail);
    return launch_encode(b, 2, B, H, T, D, n_super_cap, bits, t_start, scale_min, scale_max, stream);
}

int adkv_append(void *cache, const void *x_new, const adkv_params *p, void *tail, int B, int H, int T, int D,
                int n_super_cap, int bits, float scale_min, float scale_max, void *stream)
{
    if (!cache || !x_new || !tail || !params_ok(p)) return ADKV_E_NULL;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, T + 1)) return rc;
    if (B * H == 0) return 0;
    EncBatch b{};
    b.t[0] = enc_tensor(cache, x_new, p, tail);
    return launch_append(b, 1, B, H, T, D, n_super_cap, bits, scale_min, scale_max, stream);
}

int adkv_append_kv(void *k_cache, const void *k_new, const adkv_params *kp, void *k_tail, void *v_cache,
                   const void *v_new, const adkv_params *vp, void *v_tail, int B, int H, int T, int D,
                   int n_super_cap, int bits, float scale_min, float scale_max, void *stream)
{
    if (!k_cache || !k_new || !k_tail || !params_ok(kp) || !v_cache || !v_new || !v_tail || !params_ok(vp))
        return ADKV_E_NULL;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, T + 1)) return rc;
    if (B * H == 0) return 0;
    EncBatch b{};
    b.t[0] = enc_tensor(k_cache, k_new, kp, k_tail);
    b.t[1] = enc_tensor(v_cache, v_new, vp, v_tail);
    return launch_append(b, 2, B, H, T, D, n_super_cap, bits, scale_min, scale_max, stream);
}

int adkv_encode_kv_layers(const adkv_layer_kv *layers, int n_layers, int B, int H, int T, int D, int n_super_cap,
                          int bits, int t_start, float scale_min, float scale_max, void *stream)
{
    if (!layers) return ADKV_E_NULL;
    if (n_layers < 0 || t_start < 0) return ADKV_E_SHAPE;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, t_start + T)) return rc;
    for (int l = 0; l < n_layers; ++l) {
        if (int rc = encode_check(layers[l].k_cache, layers[l].k, &layers[l].kp, layers[l].k_tail, T, t_start)) return rc;
        if (int rc = encode_check(layers[l].v_cache, layers[l].v, &layers[l].vp, layers[l].v_tail, T, t_start)) return rc;
    }
    if (B * H == 0 || T == 0) return 0;
    for (int l0 = 0; l0 < n_layers; l0 += kEncMaxTensors / 2) {
        const int n = min(kEncMaxTensors / 2, n_layers - l0);
        EncBatch b{};
        for (int l = 0; l < n; ++l) {
            const adkv_layer_kv &L = layers[l0 + l];
            b.t[2 * l] = enc_tensor(L.k_cache, L.k, &L.kp, L.k_tail);
            b.t[2 * l + 1] = enc_tensor(L.v_cache, L.v, &L.vp, L.v_tail);
        }
        if (int rc = launch_encode(b, 2 * n, B, H, T, D, n_super_cap, bits, t_start, scale_min, scale_max, stream)) return rc;
    }
    return 0;
}

int adkv_append_kv_layers(const adkv_layer_kv *layers, int n_layers, int B, int H, int T, int D, int n_super_cap,
                          int bits, float scale_min, float scale_max, void *stream)
{
    if (!layers) return ADKV_E_NULL;
    if (n_layers < 0) return ADKV_E_SHAPE;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, T + 1)) return rc;
    for (int l = 0; l < n_layers; ++l) {
        const adkv_layer_kv &L = layers[l];
        if (!L.k_cache || !L.k || !L.k_tail || !params_ok(&L.kp) || !L.v_cache || !L.v || !L.v_tail || !params_ok(&L.vp))
            return ADKV_E_NULL;
    }
    if (B * H == 0) return 0;
    for (int l0 = 0; l0 < n_layers; l0 += kEncMaxTensors / 2) {
        const int n = min(kEncMaxTensors / 2, n_layers - l0);
        EncBatch b{};
        for (int l = 0; l < n; ++l) {
            const adkv_layer_kv &L = layers[l0 + l];
            b.t[2 * l] = enc_tensor(L.k_cache, L.k, &L.kp, L.k_tail);
            b.t[2 * l + 1] = enc_tensor(L.v_cache, L.v, &L.vp, L.v_tail);
        }
        if (int rc = launch_append(b, 2 * n, B, H, T, D, n_super_cap, bits, scale_min, scale_max, stream)) return rc;
    }
    return 0;
}

int adkv_encode_kv_ckpt(void *k_cache, const void *k, const adkv_params *kp, void *k_tail, void *k_ckpt,
                        void *v_cache, const void *v, const adkv_params *vp, void *v_tail, void *v_ckpt,
                        int interval, int n_ckpt_cap, int B, int H, int T, int D, int n_super_cap, int bits,
                        int t_start, float scale_min, float scale_max, void *stream)
{
    if (t_start < 0) return ADKV_E_SHAPE;
    if (int rc = encode_check(k_cache, k, kp, k_tail, T, t_start)) return rc;
    if (int rc = encode_check(v_cache, v, vp, v_tail, T, t_start)) return rc;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, t_start + T)) return rc;
    if (int rc = ckpt_check(k_ckpt, v_ckpt, interval, n_ckpt_cap, t_start + T)) return rc;
    if (B * H == 0 || (T == 0 && !((k_tail || v_tail) && t_start == 0))) return 0;
    EncBatch b{};
    b.t[0] = enc_tensor(k_cache, k, kp, k_tail, k_ckpt);
    b.t[1] = enc_tensor(v_cache, v, vp, v_tail, v_ckpt);
    return launch_encode(b, 2, B, H, T, D, n_super_cap, bits, t_start, scale_min, scale_max, stream,
                         CkptSpec{interval, n_ckpt_cap, D});
}

int adkv_append_kv_ckpt(void *k_cache, const void *k_new, const adkv_params *kp, void *k_tail, void *k_ckpt,
                        void *v_cache, const void *v_new, const adkv_params *vp, void *v_tail, void *v_ckpt,
                        int interval, int n_ckpt_cap, int B, int H, int T, int D, int n_super_cap, int bits,
                        float scale_min, float scale_max, void *stream)
{
    if (!k_cache || !k_new || !k_tail || !params_ok(kp) || !v_cache || !v_new || !v_tail || !params_ok(vp))
        return ADKV_E_NULL;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, T + 1)) return rc;
    if (int rc = ckpt_check(k_ckpt, v_ckpt, interval, n_ckpt_cap, T + 1)) return rc;
    if (B * H == 0) return 0;
    EncBatch b{};
    b.t[0] = enc_tensor(k_cache, k_new, kp, k_tail, k_ckpt);
    b.t[1] = enc_tensor(v_cache, v_new, vp, v_tail, v_ckpt);
    return launch_append(b, 2, B, H, T, D, n_super_cap, bits, scale_min, scale_max, stream,
                         CkptSpec{interval, n_ckpt_cap, D});
}

}  // extern "C"
