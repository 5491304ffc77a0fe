// Part of libadkv_b200.so (sm_100a).  Kernels of ADKV_FLAG_HALF_STATE: the arithmetic of the reference's own CUDA
// kernels (fp16 state, src/adkv/kernel/gemv.cu:150-164), so that caches are interchangeable with theirs.  See
// include/adkv_b200.h for the contract of the entry points that dispatch here.
#include "adkv_host.h"

#include "adkv_half.cuh"
#include "adkv_io.cuh"
#include "adkv_softmax.cuh"

namespace adkv {

// =========================================================================================
// Fused decode step, as decode_attn_kernel: one CTA per (batch, kv head); warp 0 scans K, warp 1 scans V.
template <int BITS, int G>
__global__ void __launch_bounds__(64) decode_attn_half_kernel(KArgs ka, VArgs va, const float *__restrict__ mask,
                                                              long long mask_stride_b, float scaling,
                                                              const int *__restrict__ seq_lens)
{
    __shared__ alignas(128) uint8_t kbuf[kStages * Tile<BITS>::BYTES];
    __shared__ alignas(128) uint8_t vbuf[kStages * Tile<BITS>::BYTES];
    __shared__ alignas(16) float red[G * 8 * 36];
    __shared__ alignas(16) float2 wts[G * kTileTok];
    __shared__ FusedShared<G> fs;
    __shared__ uint64_t kbar[kStages], vbar[kStages];

    const int bh = blockIdx.x, b = bh / ka.Hkv, h = bh % ka.Hkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (seq_lens) {
        const int T = seq_lens[b];
        if (T < 0 || T / Codec<BITS>::TPW >= ka.n_super_cap) {
            if (threadIdx.x == 0) atomicExch(&g_status, kStatCapacity);
            return;
        }
        ka.T = T;
        va.T = T;
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(&kbar[i], 1); mbar_init(&vbar[i], 1); }
        fs.init_barriers(1);
        mbar_init_fence();
    }
    __syncthreads();
    const Seg seg{0, ka.T, true, nullptr, nullptr, 0};
    if (warp == 0) {
        RingSink<G> sink{&fs, 0, 0};
        k_warp_h<BITS, G>(ka, seg, b, h, lane, kbuf, kbar, red, sink);
    } else {
        SoftmaxSrc<G, 1, true> src;
        src.sh = &fs;
        src.wts = wts;
        src.mask = mask ? mask + size_t(b) * mask_stride_b : nullptr;
        src.scale2 = scaling * 1.4426950408889634f;
        src.n_tiles = (va.T + kTileTok - 1) / kTileTok;
        src.t_begin = 0;
        src.init();
        v_warp_h<BITS, G>(va, seg, b, h, lane, vbuf, vbar, wts, src);
    }
}

// =========================================================================================
// The reference's two-kernel decode in its own arithmetic: 2 streams per CTA, one warp each.
template <int BITS, int G>
__global__ void __launch_bounds__(32 * kStreamsPerCta) forward_qk_half_kernel(KArgs ka, __half *__restrict__ logits,
                                                                              int n_streams)
{
    __shared__ alignas(128) uint8_t kbuf[kStreamsPerCta][kStages * Tile<BITS>::BYTES];
    __shared__ alignas(16) float red[kStreamsPerCta][G * 8 * 36];
    __shared__ uint64_t kbar[kStreamsPerCta][kStages];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        for (int i = 0; i < kStages; ++i) mbar_init(&kbar[warp][i], 1);
        mbar_init_fence();
    }
    __syncthreads();
    const int bh = blockIdx.x * kStreamsPerCta + warp;
    if (bh >= n_streams) return;
    const int b = bh / ka.Hkv, h = bh % ka.Hkv;
    GlobalLogitSink<G> sink;
#pragma unroll
    for (int g = 0; g < G; ++g) sink.row[g] = logits + (size_t(b) * ka.Hq + size_t(h) * G + g) * (ka.T + 1);
    sink.T = ka.T;
    const Seg seg{0, ka.T, true, nullptr, nullptr, 0};
    k_warp_h<BITS, G>(ka, seg, b, h, lane, kbuf[warp], kbar[warp], red[warp], sink);
}

template <int BITS, int G>
__global__ void __launch_bounds__(32 * kStreamsPerCta) forward_ov_half_kernel(VArgs va, const __half *__restrict__ attn,
                                                                              int n_streams)
{
    __shared__ alignas(128) uint8_t vbuf[kStreamsPerCta][kStages * Tile<BITS>::BYTES];
    __shared__ alignas(16) float2 wts[kStreamsPerCta][G * kTileTok];
    __shared__ uint64_t vbar[kStreamsPerCta][kStages];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        for (int i = 0; i < kStages; ++i) mbar_init(&vbar[warp][i], 1);
        mbar_init_fence();
    }
    __syncthreads();
    const int bh = blockIdx.x * kStreamsPerCta + warp;
    if (bh >= n_streams) return;
    const int b = bh / va.Hkv, h = bh % va.Hkv;
    GlobalWeightSrc<G, true> src;
#pragma unroll
    for (int g = 0; g < G; ++g) src.row[g] = attn + (size_t(b) * va.Hq + size_t(h) * G + g) * (va.T + 1);
    src.wts = wts[warp];
    const Seg seg{0, va.T, true, nullptr, nullptr, 0};
    v_warp_h<BITS, G>(va, seg, b, h, lane, vbuf[warp], vbar[warp], wts[warp], src);
}

// =========================================================================================
// Prefill quantise + pack (gemv.cu:168-308 in its arithmetic).  One 64-thread CTA per (batch, head, 128-channel
// slice); a thread owns one channel pair.  The fp16 rows are staged through a ring of 32-token tiles (bulk
// copies); groups of 8 tokens are quantised speculatively with the approximate reciprocal and redone with the
// correctly rounded division where a quotient lies too close to a rounding boundary to be sure.
constexpr int kEncThreadsH = kD / 2;
constexpr int kEncStagesH = 3;

struct EncTensorH {
    uint32_t *cache;
    const __half *x;
    ParamPtrs p;
    float *tail;   // [B, H, 2, D] float holding fp16-representable values, or nullptr
    float *ckpt;   // state checkpoints [B*H][n_ckpt_cap][2][D] (same convention as the fp32 kernels) or nullptr
};
struct CkptSpecH {
    int interval;     // tokens between checkpoints (multiple of 32), 0 = none
    int n_ckpt_cap;
};
struct EncBatchH {
    EncTensorH t[2];
};

struct PairState {
    h2 zp, sc;
};

__device__ __forceinline__ void update_h(h2 q, PairState &s, h2 alpha, h2 beta, h2 omt)
{
    s.zp = h2_fma(alpha, h2_mul(q, s.sc), s.zp);
    s.sc = h2_mul(s.sc, h2_fma(beta, h2_abs(q), omt));
}

// (words are assembled by shifting the codes in at the top, as in encode_group of adkv_encode.cu)
template <int BITS>
__device__ __forceinline__ bool encode_group_h(const __half2 *xin /* 8 rows of kD/2 */, PairState &st, h2 alpha, h2 beta,
                                               h2 omt, uint32_t (&word)[2])
{
    using C = Codec<BITS>;
    constexpr float M = 12582912.f + float(C::BIAS);   // 1.5 * 2^23 + BIAS: the low bits of (v + M) are code + BIAS
    bool doubt = false;
    static_for<8>([&](auto jc) {
        constexpr int j = decltype(jc)::value;
        const float2 xf = __half22float2(xin[j * (kD / 2)]);
        const float z0 = h2_lo(st.zp), z1 = h2_hi(st.zp), s0 = h2_lo(st.sc), s1 = h2_hi(st.sc);
        float i0, i1;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(i0) : "f"(s0));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(i1) : "f"(s1));
        const float v0 = __fmul_rn(__fsub_rn(xf.x, z0), i0), v1 = __fmul_rn(__fsub_rn(xf.y, z1), i1);
        const float c0 = fminf(fmaxf(v0, C::qlo()), C::qhi()), c1 = fminf(fmaxf(v1, C::qlo()), C::qhi());
        const float t0 = __fadd_rn(c0, M), t1 = __fadd_rn(c1, M);
        const float q0 = __fsub_rn(t0, M), q1 = __fsub_rn(t1, M);
        // not finite (zero or infinite scale, NaN) or within 4e-6 of a rounding boundary: redo exactly
        doubt |= !(fabsf(v0) < 1e30f) || !(fabsf(v1) < 1e30f) || !(fabsf(c0 - q0) < 0.5f - 4e-6f) ||
                 !(fabsf(c1 - q1) < 0.5f - 4e-6f);
        word[0] = __funnelshift_r(word[0], __float_as_uint(t0), BITS);
        word[1] = __funnelshift_r(word[1], __float_as_uint(t1), BITS);
        update_h(h2_pack(q0, q1), st, alpha, beta, omt);
    });
    return doubt;
}

template <int BITS, bool WIDE>
__global__ void __launch_bounds__(kEncThreadsH) encode_half_kernel(EncBatchH batch, CkptSpecH cs, int H, int T, int D_arg,
                                                                   int n_super_cap, int t_start)
{
    const int D = WIDE ? D_arg : kD;
    using C = Codec<BITS>;
    const EncTensorH &et = batch.t[blockIdx.y];
    uint32_t *__restrict__ cache = et.cache;
    const __half *__restrict__ x = et.x;
    const ParamPtrs p = et.p;
    float *__restrict__ tail = et.tail;
    const int S = WIDE ? D / kD : 1;
    const int bh = blockIdx.x / S, h = bh % H, c0 = kD * (blockIdx.x % S) + 2 * threadIdx.x;
    const size_t po = size_t(h) * D + c0;
    const h2 alpha = *reinterpret_cast<const h2 *>(p.alpha + po), beta = *reinterpret_cast<const h2 *>(p.beta + po);
    const h2 omt = h2_fma(h2_neg(beta), *reinterpret_cast<const h2 *>(p.target + po), kOne2);
    PairState st;
    if (t_start > 0) {
        const float2 zp = *reinterpret_cast<const float2 *>(tail + size_t(bh) * 2 * D + c0);
        const float2 sc = *reinterpret_cast<const float2 *>(tail + size_t(bh) * 2 * D + D + c0);
        st.zp = h2_pack(zp.x, zp.y);
        st.sc = h2_pack(sc.x, sc.y);
    } else {
        st.zp = *reinterpret_cast<const h2 *>(p.zp_init + po);
        st.sc = *reinterpret_cast<const h2 *>(p.scale_init + po);
    }

    __shared__ alignas(128) __half buf[kEncStagesH][32 * kD];
    __shared__ uint64_t bar[kEncStagesH];
    if (threadIdx.x == 0) {
        for (int i = 0; i < kEncStagesH; ++i) mbar_init(&bar[i], 1);
        mbar_init_fence();
    }
    __syncthreads();

    uint2 *w = reinterpret_cast<uint2 *>(cache + size_t(bh) * n_super_cap * D + c0);
    const __half2 *xs = reinterpret_cast<const __half2 *>(x + size_t(bh) * T * D + c0);
    const int RS = D / 2;
    constexpr int SRS = kD / 2;

    auto exact_token = [&](int t, uint32_t(&word)[2]) {
        const float2 xv = __half22float2(xs[size_t(t - t_start) * RS]);
        const int q0 = quantize_h<BITS>(xv.x, h2_lo(st.zp), h2_lo(st.sc));
        const int q1 = quantize_h<BITS>(xv.y, h2_hi(st.zp), h2_hi(st.sc));
        word[0] = __funnelshift_r(word[0], uint32_t(q0 + C::BIAS), BITS);
        word[1] = __funnelshift_r(word[1], uint32_t(q1 + C::BIAS), BITS);
        update_h(h2_pack(float(q0), float(q1)), st, alpha, beta, omt);
    };

    // checkpoint k is written when the state before token (k+1)*interval is reached
    float *ckpt = (et.ckpt && cs.interval > 0) ? et.ckpt + size_t(bh) * cs.n_ckpt_cap * 2 * D + c0 : nullptr;
    int next_ckpt = ckpt ? (t_start / cs.interval + 1) * cs.interval : 0x7fffffff;
    auto checkpoint = [&](int t_reached) {
        if (t_reached == next_ckpt) {
            const int k = next_ckpt / cs.interval - 1;
            if (k < cs.n_ckpt_cap) {
                *reinterpret_cast<float2 *>(ckpt + size_t(k) * 2 * D) = make_float2(h2_lo(st.zp), h2_hi(st.zp));
                *reinterpret_cast<float2 *>(ckpt + size_t(k) * 2 * D + D) = make_float2(h2_lo(st.sc), h2_hi(st.sc));
            }
            next_ckpt += cs.interval;
        }
    };

    const int t_end = t_start + T;
    int t = t_start;
    uint32_t word[2] = {0u, 0u};
    if (t % C::TPW != 0 && t < t_end) {   // a chunk that starts inside a word keeps the fields already there
        const uint2 old = w[size_t(t / C::TPW) * RS];
        const int up = BITS * (C::TPW - t % C::TPW);
        word[0] = old.x << up;
        word[1] = old.y << up;
    }
    for (; t < t_end && t % 8 != 0; ++t) {
        exact_token(t, word);
        checkpoint(t + 1);
        if ((t + 1) % C::TPW == 0) {
            w[size_t(t / C::TPW) * RS] = make_uint2(word[0], word[1]);
            word[0] = word[1] = 0u;
        }
    }
    const int n_groups = (t_end - t) / 8;
    const int n_tiles = (n_groups + 3) / 4;
    const __half *src = x + (size_t(bh) * T + (t - t_start)) * D + kD * (blockIdx.x % S);
    auto issue = [&](int i) {
        const int rows = min(4, n_groups - 4 * i) * 8;
        const uint32_t bytes = uint32_t(rows) * kD * 2;
        mbar_expect_tx(&bar[i % kEncStagesH], bytes);
        if (S == 1) {
            bulk_load(&buf[i % kEncStagesH][0], src + size_t(i) * 32 * kD, bytes, &bar[i % kEncStagesH]);
        } else {
            for (int r = 0; r < rows; ++r)
                bulk_load(&buf[i % kEncStagesH][r * kD], src + (size_t(i) * 32 + r) * D, kD * 2, &bar[i % kEncStagesH]);
        }
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < min(kEncStagesH, n_tiles); ++i) issue(i);
#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
        const bool landed = mbar_wait_bounded(&bar[i % kEncStagesH], (i / kEncStagesH) & 1, kStatKWait);
        if (!__syncthreads_and(landed)) {
            for (int k = i; k < min(n_tiles, i + kEncStagesH); ++k)
                if (!mbar_wait_bounded(&bar[k % kEncStagesH], (k / kEncStagesH) & 1, kStatDrain)) break;
            return;
        }
        const int ng = min(4, n_groups - 4 * i);
#pragma unroll 1
        for (int g = 0; g < ng; ++g, t += 8) {
            const __half2 *rows = reinterpret_cast<const __half2 *>(&buf[i % kEncStagesH][0]) + g * 8 * SRS + threadIdx.x;
            const PairState saved = st;
            const uint32_t word_in[2] = {word[0], word[1]};
            const bool doubt = encode_group_h<BITS>(rows, st, alpha, beta, omt, word);
            if (doubt) {
                st = saved;
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
        __syncthreads();
        if (threadIdx.x == 0 && i + kEncStagesH < n_tiles) issue(i + kEncStagesH);
    }
    for (; t < t_end; ++t) {
        exact_token(t, word);
        checkpoint(t + 1);
    }
    if (t % C::TPW != 0) {
        const int down = BITS * (C::TPW - t % C::TPW);
        w[size_t(t / C::TPW) * RS] = make_uint2(word[0] >> down, word[1] >> down);
    }
    if (tail) {
        *reinterpret_cast<float2 *>(tail + size_t(bh) * 2 * D + c0) = make_float2(h2_lo(st.zp), h2_hi(st.zp));
        *reinterpret_cast<float2 *>(tail + size_t(bh) * 2 * D + D + c0) = make_float2(h2_lo(st.sc), h2_hi(st.sc));
    }
}

// Single-token append from the persisted tail state (gemv.cu:91-146 without the replay that precedes it there).
template <int BITS>
__global__ void __launch_bounds__(kEncThreadsH) append_half_kernel(EncBatchH batch, CkptSpecH cs, int H, int T, int D,
                                                                   int n_super_cap)
{
    using C = Codec<BITS>;
    const EncTensorH &et = batch.t[blockIdx.y];
    float *__restrict__ tail = et.tail;
    const int S = D / kD;
    const int bh = blockIdx.x / S, h = bh % H, c0 = kD * (blockIdx.x % S) + 2 * threadIdx.x;
    const size_t po = size_t(h) * D + c0;
    const h2 alpha = *reinterpret_cast<const h2 *>(et.p.alpha + po), beta = *reinterpret_cast<const h2 *>(et.p.beta + po);
    const h2 omt = h2_fma(h2_neg(beta), *reinterpret_cast<const h2 *>(et.p.target + po), kOne2);
    float2 *tz = reinterpret_cast<float2 *>(tail + size_t(bh) * 2 * D + c0);
    float2 *ts = reinterpret_cast<float2 *>(tail + size_t(bh) * 2 * D + D + c0);
    const float2 zp = *tz, sc = *ts;
    PairState st{h2_pack(zp.x, zp.y), h2_pack(sc.x, sc.y)};
    const float2 xv = __half22float2(*reinterpret_cast<const __half2 *>(et.x + size_t(bh) * D + c0));
    const int q0 = quantize_h<BITS>(xv.x, zp.x, sc.x), q1 = quantize_h<BITS>(xv.y, zp.y, sc.y);
    uint2 *slot = reinterpret_cast<uint2 *>(et.cache + (size_t(bh) * n_super_cap + T / C::TPW) * D + c0);
    const int sh = BITS * (T % C::TPW);
    uint2 wv = *slot;
    wv.x = (wv.x & ~(C::FIELD << sh)) | (uint32_t(q0 + C::BIAS) << sh);
    wv.y = (wv.y & ~(C::FIELD << sh)) | (uint32_t(q1 + C::BIAS) << sh);
    *slot = wv;
    update_h(h2_pack(float(q0), float(q1)), st, alpha, beta, omt);
    *tz = make_float2(h2_lo(st.zp), h2_hi(st.zp));
    *ts = make_float2(h2_lo(st.sc), h2_hi(st.sc));
    if (et.ckpt && cs.interval > 0 && (T + 1) % cs.interval == 0) {
        const int k = (T + 1) / cs.interval - 1;
        if (k < cs.n_ckpt_cap) {
            float *dst = et.ckpt + (size_t(bh) * cs.n_ckpt_cap + k) * 2 * D + c0;
            *reinterpret_cast<float2 *>(dst) = *tz;
            *reinterpret_cast<float2 *>(dst + D) = *ts;
        }
    }
}

}  // namespace adkv

using namespace adkv;

ADKV_DEFINE_TU_STATUS(adkv_tu_status_half)

ADKV_HIDDEN int adkv_half_decode_attn(const KArgs &ka, const VArgs &va, const float *mask, long long mask_stride_b,
                                      float scaling, int B, int bits, const int *seq_lens, cudaStream_t s)
{
    if (ka.D != kD) return ADKV_E_FLAGS;
    ADKV_DISPATCH_H(bits, ka.Hq / ka.Hkv,
                    (decode_attn_half_kernel<BITS, G><<<B * ka.Hkv, 64, 0, s>>>(ka, va, mask, mask_stride_b, scaling,
                                                                               seq_lens)))
    return launch_status();
}

ADKV_HIDDEN int adkv_half_forward_qk(const KArgs &ka, __half *logits, int B, int bits, cudaStream_t s)
{
    if (ka.D != kD) return ADKV_E_FLAGS;
    const int n_streams = B * ka.Hkv, grid = (n_streams + kStreamsPerCta - 1) / kStreamsPerCta;
    ADKV_DISPATCH_H(bits, ka.Hq / ka.Hkv,
                    (forward_qk_half_kernel<BITS, G><<<grid, 32 * kStreamsPerCta, 0, s>>>(ka, logits, n_streams)))
    return launch_status();
}

ADKV_HIDDEN int adkv_half_forward_ov(const VArgs &va, const __half *attn, int B, int bits, cudaStream_t s)
{
    if (va.D != kD) return ADKV_E_FLAGS;
    const int n_streams = B * va.Hkv, grid = (n_streams + kStreamsPerCta - 1) / kStreamsPerCta;
    ADKV_DISPATCH_H(bits, va.Hq / va.Hkv,
                    (forward_ov_half_kernel<BITS, G><<<grid, 32 * kStreamsPerCta, 0, s>>>(va, attn, n_streams)))
    return launch_status();
}

static EncTensorH enc_tensor_h(void *cache, const void *x, const adkv_params *p, void *tail, void *ckpt)
{
    return EncTensorH{static_cast<uint32_t *>(cache), static_cast<const __half *>(x), to_ptrs(p),
                      static_cast<float *>(tail), static_cast<float *>(ckpt)};
}

// n tensors (1 or 2) of one layer; arguments already validated by the caller.
ADKV_HIDDEN int adkv_half_encode(void *k_cache, const void *k, const adkv_params *kp, void *k_tail, void *k_ckpt,
                                 void *v_cache, const void *v, const adkv_params *vp, void *v_tail, void *v_ckpt,
                                 int interval, int n_ckpt_cap, int n, int B, int H, int T, int D, int n_super_cap,
                                 int bits, int t_start, cudaStream_t s)
{
    EncBatchH b{};
    b.t[0] = enc_tensor_h(k_cache, k, kp, k_tail, k_ckpt);
    if (n == 2) b.t[1] = enc_tensor_h(v_cache, v, vp, v_tail, v_ckpt);
    const CkptSpecH cs{interval, n_ckpt_cap};
    const dim3 grid(B * H * (D / kD), n);
    if (D == kD) {
        if (bits == 4) encode_half_kernel<4, false><<<grid, kEncThreadsH, 0, s>>>(b, cs, H, T, D, n_super_cap, t_start);
        else encode_half_kernel<2, false><<<grid, kEncThreadsH, 0, s>>>(b, cs, H, T, D, n_super_cap, t_start);
    } else {
        if (bits == 4) encode_half_kernel<4, true><<<grid, kEncThreadsH, 0, s>>>(b, cs, H, T, D, n_super_cap, t_start);
        else encode_half_kernel<2, true><<<grid, kEncThreadsH, 0, s>>>(b, cs, H, T, D, n_super_cap, t_start);
    }
    return launch_status();
}

ADKV_HIDDEN int adkv_half_append(void *k_cache, const void *k_new, const adkv_params *kp, void *k_tail, void *k_ckpt,
                                 void *v_cache, const void *v_new, const adkv_params *vp, void *v_tail, void *v_ckpt,
                                 int interval, int n_ckpt_cap, int n, int B, int H, int T, int D, int n_super_cap,
                                 int bits, cudaStream_t s)
{
    EncBatchH b{};
    b.t[0] = enc_tensor_h(k_cache, k_new, kp, k_tail, k_ckpt);
    if (n == 2) b.t[1] = enc_tensor_h(v_cache, v_new, vp, v_tail, v_ckpt);
    const CkptSpecH cs{interval, n_ckpt_cap};
    const dim3 grid(B * H * (D / kD), n);
    if (bits == 4) append_half_kernel<4><<<grid, kEncThreadsH, 0, s>>>(b, cs, H, T, D, n_super_cap);
    else append_half_kernel<2><<<grid, kEncThreadsH, 0, s>>>(b, cs, H, T, D, n_super_cap);
    return launch_status();
}
