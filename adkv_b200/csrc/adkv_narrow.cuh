// Decode-side scans with a 128-wide head split over two warps per tensor ("narrow" scans).
//
// The whole-head scans of adkv_decode.cuh give one K warp and one V warp to a (batch, kv head) stream, and a
// stream is serial in its tokens.  A decode step over few streams -- a small batch, or one GPU's share of a batch
// that was split over several -- then leaves most of an SM's warp slots empty while every warp is bound by the
// latency of its own dependent instruction chain.  Here lane l of slice j owns the channel pair 64j + 2l, 64j + 2l + 1:
// twice the warps per stream, half the arithmetic per warp and token.  Logits are sums over all channels, so the
// two K warps post partial logits to a shared-memory ring slot and the consumers add them in a fixed order
// (FusedShared<G, 2>, as the 256/512-wide kernels do with their 128-channel slices).  The reference splits the
// channels of a head over warps for head dims 256 and 512 only (src/adkv/kernel/gemv.cu:336-353, 857-874,
// 1208-1225).  The arithmetic per channel is that of adkv_decode.cuh, value for value; only the order in which
// the per-lane partial logits are summed differs.
#pragma once
#include "adkv_softmax.cuh"

namespace adkv {

constexpr int kNarrowCh = 64;                 // channels per slice
constexpr int kNarrowSlices = kD / kNarrowCh;

template <int BITS>
struct NarrowTile {
    static constexpr int WORDS = kTileTok / Codec<BITS>::TPW;   // word rows per tile
    static constexpr int ROW_BYTES = kNarrowCh * 4;             // this slice's part of a 512-byte word row
    static constexpr int BYTES = WORDS * ROW_BYTES;             // 4-bit: 1024, 2-bit: 512
};

// Per-warp bulk-copy ring over one slice of a stream: every word row contributes ROW_BYTES at a stride of 512.
template <int BITS, int STAGES = kStages>
struct NarrowRing {
    uint8_t *buf;           // STAGES * NarrowTile::BYTES, 128-byte aligned
    uint64_t *bar;          // STAGES barriers
    const uint8_t *src;     // first word row of this slice
    int n_tiles, T;
    int wait_code;

    __device__ __forceinline__ int tile_rows(int i) const
    {
        const int ntok = min(kTileTok, T - i * kTileTok);
        return (ntok + Codec<BITS>::TPW - 1) / Codec<BITS>::TPW;
    }
    // lane 0 only
    __device__ __forceinline__ void issue(int i) const
    {
        const int st = i % STAGES, rows = tile_rows(i);
        mbar_expect_tx(&bar[st], uint32_t(rows) * NarrowTile<BITS>::ROW_BYTES);
        const uint8_t *row = src + size_t(i) * NarrowTile<BITS>::WORDS * (kD * 4);
        uint8_t *dst = buf + st * NarrowTile<BITS>::BYTES;
        for (int r = 0; r < rows; ++r, row += kD * 4, dst += NarrowTile<BITS>::ROW_BYTES)
            bulk_load(dst, row, NarrowTile<BITS>::ROW_BYTES, &bar[st]);
    }
    __device__ __forceinline__ void prologue(int lane) const
    {
        if (lane == 0)
            for (int i = 0; i < min(STAGES, n_tiles); ++i) issue(i);
    }
    __device__ __forceinline__ bool wait(int i) const
    {
        return mbar_wait_bounded(&bar[i % STAGES], (i / STAGES) & 1, wait_code);
    }
    __device__ __forceinline__ const uint2 *tile(int i, int lane) const
    {
        return reinterpret_cast<const uint2 *>(buf + (i % STAGES) * NarrowTile<BITS>::BYTES) + lane;
    }
    __device__ __forceinline__ void release_and_refill(int i, int lane) const
    {
        __syncwarp();
        if (lane == 0 && i + STAGES < n_tiles) issue(i + STAGES);
    }
    __device__ __forceinline__ void drain(int from) const
    {
        const int issued = min(n_tiles, from + STAGES);
        for (int i = from; i < issued; ++i)
            if (!mbar_wait_bounded(&bar[i % STAGES], (i / STAGES) & 1, kStatDrain)) break;
    }
};

// Parameters of the lane's channel pair (element `off` of the [Hkv, 128] tensors, off even).
template <int BITS, bool EXACT>
__device__ __forceinline__ void load_chan2(Chan (&ch)[2], SafeRange &safe, const ParamPtrs &p, size_t off, float smin,
                                           float smax)
{
    const float2 za = __half22float2(*reinterpret_cast<const __half2 *>(p.zp_init + off));
    const float2 sb = __half22float2(*reinterpret_cast<const __half2 *>(p.scale_init + off));
    const float2 al = __half22float2(*reinterpret_cast<const __half2 *>(p.alpha + off));
    const float2 be = __half22float2(*reinterpret_cast<const __half2 *>(p.beta + off));
    const float2 tg = __half22float2(*reinterpret_cast<const __half2 *>(p.target + off));
    ch[0] = Chan{za.x, sb.x, al.x, be.x, EXACT ? tg.x : fmaf(-be.x, tg.x, 1.0f)};
    ch[1] = Chan{za.y, sb.y, al.y, be.y, EXACT ? tg.y : fmaf(-be.y, tg.y, 1.0f)};
    const float beta[2] = {be.x, be.y}, target[2] = {tg.x, tg.y};
    safe.template init<BITS, 2>(beta, target, smin, smax);
}

__device__ __forceinline__ void load_init_state2(Chan (&ch)[2], const float *init, int c0)
{
    if (init) {
        const float2 zp = *reinterpret_cast<const float2 *>(init + c0);
        const float2 sc = *reinterpret_cast<const float2 *>(init + kD + c0);
        ch[0].zp = zp.x; ch[1].zp = zp.y;
        ch[0].s = sc.x; ch[1].s = sc.y;
    }
}

__device__ __forceinline__ void store_state2(float *dst, const Chan (&ch)[2], int c0)
{
    *reinterpret_cast<float2 *>(dst + c0) = make_float2(ch[0].zp, ch[1].zp);
    *reinterpret_cast<float2 *>(dst + kD + c0) = make_float2(ch[0].s, ch[1].s);
}

__device__ __forceinline__ float2 load_half2f(const __half *p)
{
    return __half22float2(*reinterpret_cast<const __half2 *>(p));
}

// append_new_token (adkv_decode.cuh) for a channel pair.
template <int BITS, int ARITH>
__device__ __forceinline__ void append_new_token2(Chan (&ch)[2], const ParamPtrs &p, size_t poff, float *tail,
                                                  bool tail_keep, const __half *x_new, uint2 *slot, int T, float smin,
                                                  float smax, float *ckpt_out, int c0, float (&xh)[2])
{
    using C = Codec<BITS>;
    const float2 xn2 = load_half2f(x_new);
    const float xn[2] = {xn2.x, xn2.y};
    const uint2 wv = *slot;
    uint32_t ww[2] = {wv.x, wv.y};
    const int sh = BITS * (T % C::TPW);
    if (tail) {
        const float2 tg = load_half2f(p.target + poff);
        load_init_state2(ch, tail, c0);
        ch[0].tc = tg.x;
        ch[1].tc = tg.y;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float rh;
            const float q = quantize<BITS>(xn[c], ch[c], rh);
            xh[c] = __fadd_rn(rh, ch[c].zp);
            ww[c] = (ww[c] & ~(C::FIELD << sh)) | (uint32_t(int(q) + C::BIAS) << sh);
            advance_canonical(q, rh, ch[c], smin, smax);
        }
        if (!tail_keep) store_state2(tail, ch, c0);
    } else {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float rh;
            const float q = quantize<BITS>(xn[c], ch[c], rh);
            xh[c] = __fadd_rn(rh, ch[c].zp);
            ww[c] = (ww[c] & ~(C::FIELD << sh)) | (uint32_t(int(q) + C::BIAS) << sh);
            if (ckpt_out) advance_like_replay<ARITH == kArithCanon>(q, rh, ch[c], smin, smax);
        }
    }
    *slot = make_uint2(ww[0], ww[1]);
    if (ckpt_out) store_state2(ckpt_out, ch, c0);
}

// ---------------------------------------------------------------------------------- K side

// Unguarded full 8-token group of a channel pair (packed fp32).
template <int BITS, int G, bool EXACT>
__device__ __forceinline__ void k_chunk_n2(const uint2 &w, const FieldConsts<BITS> &fc, Chan (&ch)[2], const PairConst &pc,
                                           f32x2 one, const f32x2 (&qv2)[G], float *red, int lane)
{
    uint32_t ga = w.x, gb = w.y;
    f32x2 zp = pk2(ch[0].zp, ch[1].zp), s = pk2(ch[0].s, ch[1].s);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        static_for<4>([&](auto kc) {
            constexpr int k = decltype(kc)::value;
            const f32x2 q2 = fc.template code2<k>(ga, gb);
            const f32x2 xh = replay_step2<EXACT>(q2, zp, s, pc, one);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float a, b;
                upk2(mul2(qv2[g], xh), a, b);
                red[(g * 8 + 4 * half + k) * 36 + lane] = a + b;
            }
        });
        ga >>= 4 * BITS;
        gb >>= 4 * BITS;
    }
    upk2(zp, ch[0].zp, ch[1].zp);
    upk2(s, ch[0].s, ch[1].s);
}

// Guarded and / or partial 8-token group, one channel at a time.
template <int BITS, int G, bool EXACT>
__device__ __forceinline__ void k_chunk_n(const uint2 &w, Chan (&ch)[2], const float (&qv)[G][2], float *red, int lane,
                                          int count, float smin, float smax)
{
    const uint32_t grp[2] = {w.x, w.y};
#pragma unroll 1
    for (int j = 0; j < 8; ++j) {
        float part[G];
#pragma unroll
        for (int g = 0; g < G; ++g) part[g] = 0.f;
        if (j < count) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float xh = replay_step<EXACT, true>(code_f_rt<BITS>(grp[c], j), ch[c], smin, smax);
#pragma unroll
                for (int g = 0; g < G; ++g) part[g] = fmaf(qv[g][c], xh, part[g]);
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) red[(g * 8 + j) * 36 + lane] = part[g];
    }
}

template <int BITS, int G, int ARITH, class Sink, int STAGES = kStages>
__device__ __forceinline__ void k_warp_n(const KArgs &a, const Seg &seg, int b, int h, int lane, uint8_t *ring_buf,
                                         uint64_t *ring_bar, float *red, Sink &sink)
{
    using C = Codec<BITS>;
    constexpr bool EXACT = ARITH == kArithCanon;
    const int bh = b * a.Hkv + h;
    const int c0 = kNarrowCh * seg.slice + 2 * lane;      // first of this lane's two channels
    Chan ch[2];
    SafeRange safe;
    FieldConsts<BITS> fc;
    fc.init();
    load_chan2<BITS, EXACT>(ch, safe, a.p, size_t(h) * kD + c0, a.smin, a.smax);
    load_init_state2(ch, seg.init, c0);
    float qv[G][2];
    f32x2 qv2[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float2 v = load_half2f(a.q + (size_t(b) * a.Hq + size_t(h) * G + g) * kD + c0);
        qv[g][0] = v.x; qv[g][1] = v.y;
        qv2[g] = pk2(v.x, v.y);
    }
    PairConst pc;
    pc.alpha = pk2(ch[0].alpha, ch[1].alpha);
    pc.beta = pk2(ch[0].beta, ch[1].beta);
    pc.tc = EXACT ? pk2(-ch[0].tc, -ch[1].tc) : pk2(ch[0].tc, ch[1].tc);
    const f32x2 one = opaque_ones2();

    uint8_t *stream = a.cache + (size_t(bh) * a.n_super_cap * kD + size_t(kNarrowCh) * seg.slice) * 4;
    const int n_tok = seg.t_end - seg.t_begin;
    NarrowRing<BITS, STAGES> ring{ring_buf, ring_bar, stream + size_t(seg.t_begin / C::TPW) * (kD * 4),
                                  (n_tok + kTileTok - 1) / kTileTok, n_tok, kStatKWait};
    ring.prologue(lane);

    bool ok = true;
    int i = 0;
    for (; i < ring.n_tiles; ++i) {
        if (!(ok = ring.wait(i))) break;
        if (!(ok = sink.begin_tile(i))) break;
        const uint2 *tile = ring.tile(i, lane);
        const int ntok = min(kTileTok, n_tok - i * kTileTok);
        float sum[G];
#pragma unroll 1
        for (int wd = 0; wd * C::TPW < ntok; ++wd) {
            uint2 w = tile[wd * (kNarrowCh / 2)];
            const int count = ntok - wd * C::TPW;   // valid fields in this word (may exceed TPW)
#pragma unroll 1
            for (int c8 = 0; c8 < C::TPW / 8 && c8 * 8 < count; ++c8) {
                if (count - c8 * 8 >= 8 && safe.holds(ch)) k_chunk_n2<BITS, G, EXACT>(w, fc, ch, pc, one, qv2, red, lane);
                else k_chunk_n<BITS, G, EXACT>(w, ch, qv, red, lane, count - c8 * 8, a.smin, a.smax);
                reduce8<G>(red, lane, sum);
#pragma unroll
                for (int g = 0; g < G; ++g) sink.put8(i, g, wd * C::TPW + c8 * 8, sum[g], lane);
                if (C::TPW == 16) { w.x >>= 16; w.y >>= 16; }
            }
        }
        sink.end_tile(i, lane);
        ring.release_and_refill(i, lane);
    }
    if (!ok) {
        ring.drain(i);
        return;
    }
    if (!seg.append) return;
    float xh[2];
    append_new_token2<BITS, ARITH>(ch, a.p, size_t(h) * kD + c0, a.tail ? a.tail + size_t(bh) * 2 * kD : nullptr,
                                   a.tail_keep, a.x_new + size_t(bh) * kD + c0,
                                   reinterpret_cast<uint2 *>(stream + size_t(a.T / C::TPW) * (kD * 4)) + lane, a.T, a.smin,
                                   a.smax, seg.ckpt_out, c0, xh);
    if (!sink.begin_tile(ring.n_tiles)) return;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float s = warp_sum(fmaf(qv[g][1], xh[1], qv[g][0] * xh[0]));
        if (lane == 0) sink.put_self(g, s);
    }
    sink.finish(lane);
}

// ---------------------------------------------------------------------------------- V side

template <int BITS, int G, bool EXACT>
__device__ __forceinline__ void v_chunk_n2(const uint2 &w, const FieldConsts<BITS> &fc, Chan (&ch)[2], const PairConst &pc,
                                           f32x2 one, const float2 *wts2, int tok0, float (&acc)[G][2])
{
    uint32_t ga = w.x, gb = w.y;
    f32x2 zp = pk2(ch[0].zp, ch[1].zp), s = pk2(ch[0].s, ch[1].s);
    f32x2 acc2[G];
#pragma unroll
    for (int g = 0; g < G; ++g) acc2[g] = pk2(acc[g][0], acc[g][1]);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        f32x2 wt[G][4];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const ulonglong2 x = *reinterpret_cast<const ulonglong2 *>(wts2 + g * kTileTok + tok0 + 4 * half);
            const ulonglong2 y = *reinterpret_cast<const ulonglong2 *>(wts2 + g * kTileTok + tok0 + 4 * half + 2);
            wt[g][0] = x.x; wt[g][1] = x.y; wt[g][2] = y.x; wt[g][3] = y.y;
        }
        static_for<4>([&](auto kc) {
            constexpr int k = decltype(kc)::value;
            const f32x2 q2 = fc.template code2<k>(ga, gb);
            const f32x2 xh = replay_step2<EXACT>(q2, zp, s, pc, one);
#pragma unroll
            for (int g = 0; g < G; ++g) acc2[g] = fma2(wt[g][k], xh, acc2[g]);
        });
        ga >>= 4 * BITS;
        gb >>= 4 * BITS;
    }
    upk2(zp, ch[0].zp, ch[1].zp);
    upk2(s, ch[0].s, ch[1].s);
#pragma unroll
    for (int g = 0; g < G; ++g) upk2(acc2[g], acc[g][0], acc[g][1]);
}

template <int BITS, int G, bool EXACT>
__device__ __forceinline__ void v_chunk_n(const uint2 &w, Chan (&ch)[2], const float2 *wts2, int tok0, float (&acc)[G][2],
                                          int count, float smin, float smax)
{
    const uint32_t grp[2] = {w.x, w.y};
#pragma unroll 1
    for (int j = 0; j < 8 && j < count; ++j) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const float xh = replay_step<EXACT, true>(code_f_rt<BITS>(grp[c], j), ch[c], smin, smax);
#pragma unroll
            for (int g = 0; g < G; ++g) acc[g][c] = fmaf(wts2[g * kTileTok + tok0 + j].x, xh, acc[g][c]);
        }
    }
}

// Adapter: the softmax sources of adkv_softmax.cuh rescale and normalise four accumulators per head; a narrow lane
// has two, carried in the first half of a four-wide array.
template <int G>
__device__ __forceinline__ void widen(const float (&a2)[G][2], float (&a4)[G][4])
{
#pragma unroll
    for (int g = 0; g < G; ++g) { a4[g][0] = a2[g][0]; a4[g][1] = a2[g][1]; a4[g][2] = 0.f; a4[g][3] = 0.f; }
}
template <int G>
__device__ __forceinline__ void narrow(const float (&a4)[G][4], float (&a2)[G][2])
{
#pragma unroll
    for (int g = 0; g < G; ++g) { a2[g][0] = a4[g][0]; a2[g][1] = a4[g][1]; }
}

// Src: SoftmaxSrc<G, 2> (tile_weights, self_weight, norm).  The result is written here: two channels per lane.
template <int BITS, int G, int ARITH, class Src, int STAGES = kStages>
__device__ __forceinline__ void v_warp_n(const VArgs &a, const Seg &seg, int b, int h, int lane, uint8_t *ring_buf,
                                         uint64_t *ring_bar, const float2 *wts, Src &src)
{
    using C = Codec<BITS>;
    constexpr bool EXACT = ARITH == kArithCanon;
    const int bh = b * a.Hkv + h;
    const int c0 = kNarrowCh * seg.slice + 2 * lane;
    Chan ch[2];
    SafeRange safe;
    FieldConsts<BITS> fc;
    fc.init();
    load_chan2<BITS, EXACT>(ch, safe, a.p, size_t(h) * kD + c0, a.smin, a.smax);
    load_init_state2(ch, seg.init, c0);
    PairConst pc;
    pc.alpha = pk2(ch[0].alpha, ch[1].alpha);
    pc.beta = pk2(ch[0].beta, ch[1].beta);
    pc.tc = EXACT ? pk2(-ch[0].tc, -ch[1].tc) : pk2(ch[0].tc, ch[1].tc);
    const f32x2 one = opaque_ones2();
    float acc4[G][4];      // [g][0..1] are this lane's accumulators (see widen / narrow)
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc4[g][c] = 0.f;

    uint8_t *stream = a.cache + (size_t(bh) * a.n_super_cap * kD + size_t(kNarrowCh) * seg.slice) * 4;
    const int n_tok = seg.t_end - seg.t_begin;
    NarrowRing<BITS, STAGES> ring{ring_buf, ring_bar, stream + size_t(seg.t_begin / C::TPW) * (kD * 4),
                                  (n_tok + kTileTok - 1) / kTileTok, n_tok, kStatVWait};
    ring.prologue(lane);

    bool ok = true;
    int i = 0;
    for (; i < ring.n_tiles; ++i) {
        const int ntok = min(kTileTok, n_tok - i * kTileTok);
        if (!(ok = src.tile_weights(i, ntok, lane, acc4))) break;
        if (!(ok = ring.wait(i))) break;
        const uint2 *tile = ring.tile(i, lane);
        float acc[G][2];
        narrow<G>(acc4, acc);
#pragma unroll 1
        for (int wd = 0; wd * C::TPW < ntok; ++wd) {
            uint2 w = tile[wd * (kNarrowCh / 2)];
            const int count = ntok - wd * C::TPW;
#pragma unroll 1
            for (int c8 = 0; c8 < C::TPW / 8 && c8 * 8 < count; ++c8) {
                const int tok0 = wd * C::TPW + c8 * 8;
                if (count - c8 * 8 >= 8 && safe.holds(ch)) v_chunk_n2<BITS, G, EXACT>(w, fc, ch, pc, one, wts, tok0, acc);
                else v_chunk_n<BITS, G, EXACT>(w, ch, wts, tok0, acc, count - c8 * 8, a.smin, a.smax);
                if (C::TPW == 16) { w.x >>= 16; w.y >>= 16; }
            }
        }
        widen<G>(acc, acc4);
        ring.release_and_refill(i, lane);   // also orders this tile's reads of wts before the next fill
    }
    if (!ok) {
        ring.drain(i);
        src_give_up(src, c0, 0);
        return;
    }
    if (seg.append) {
        float w_self[G];
        if (!src.self_weight(lane, acc4, w_self, a.T)) {
            src_give_up(src, c0, 0);
            return;
        }
        float xh[2];
        append_new_token2<BITS, ARITH>(ch, a.p, size_t(h) * kD + c0, a.tail ? a.tail + size_t(bh) * 2 * kD : nullptr,
                                       a.tail_keep, a.x_new + size_t(bh) * kD + c0,
                                       reinterpret_cast<uint2 *>(stream + size_t(a.T / C::TPW) * (kD * 4)) + lane, a.T,
                                       a.smin, a.smax, seg.ckpt_out, c0, xh);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            acc4[g][0] = fmaf(w_self[g], xh[0], acc4[g][0]);
            acc4[g][1] = fmaf(w_self[g], xh[1], acc4[g][1]);
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float inv = 1.0f / src.norm(g);
        const __half2 o = __floats2half2_rn(acc4[g][0] * inv, acc4[g][1] * inv);
        *reinterpret_cast<__half2 *>(a.out + (size_t(b) * a.Hq + size_t(h) * G + g) * kD + c0) = o;
    }
}

}  // namespace adkv
