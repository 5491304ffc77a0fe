// The recurrence in the arithmetic of the reference's CUDA kernels (src/adkv/kernel/gemv.cu:150-164): state and
// constants are fp16 pairs, one step is
//     zp <- fma(alpha, q * sc, zp)        sc <- sc * fma(beta, |q|, omt)        omt = 1 - beta * target
// with every operation rounded to fp16 once (omt with ONE rounding: that is what the reference's build produces,
// its multiply and subtract being contracted), no eps guard and no scale clamp; the quantiser is
// clamp(round_half_even((x - zp) / sc)) in fp32 with a correctly rounded division.  Caches written with this
// arithmetic are interchangeable with the ones the reference's kernels write and read.
//
// Decode-side scans mirror k_warp / v_warp of adkv_decode.cuh (same ring, same sink / source interfaces); a lane
// owns two channel pairs, which is exactly one fp16x2 register per state variable and pair.
#pragma once
#include "adkv_decode.cuh"

namespace adkv {

typedef uint32_t h2;   // two fp16 values: low half = even channel of the pair (the layout of a __half2 load)

__device__ __forceinline__ h2 h2_mul(h2 a, h2 b)
{
    h2 r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ h2 h2_add(h2 a, h2 b)
{
    h2 r;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ h2 h2_sub(h2 a, h2 b)
{
    h2 r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ h2 h2_fma(h2 a, h2 b, h2 c)
{
    h2 r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ h2 h2_abs(h2 a)
{
    h2 r;
    asm("abs.f16x2 %0, %1;" : "=r"(r) : "r"(a));
    return r;
}
__device__ __forceinline__ h2 h2_neg(h2 a) { return a ^ 0x80008000u; }
__device__ __forceinline__ float h2_lo(h2 a) { return __half2float(__ushort_as_half((unsigned short)(a & 0xffffu))); }
__device__ __forceinline__ float h2_hi(h2 a) { return __half2float(__ushort_as_half((unsigned short)(a >> 16))); }
__device__ __forceinline__ h2 h2_pack(float lo, float hi)
{
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const h2 *>(&v);
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// fp16 bit pattern of a positive, exactly representable normal number (compile time).
__host__ __device__ constexpr uint32_t h_bits(double v)
{
    int e = 0;
    while (v >= 2.0) { v *= 0.5; ++e; }
    while (v < 1.0) { v *= 2.0; --e; }
    return (uint32_t(e + 15) << 10) | uint32_t((v - 1.0) * 1024.0);
}
__host__ __device__ constexpr uint32_t h_bits2(double v) { return h_bits(v) * 0x10001u; }

constexpr h2 kOne2 = 0x3C003C00u;

struct HPair {
    h2 zp, sc, alpha, beta, omt;
};

// The five fp16 parameters of channels off .. off+3 as two pairs.
__device__ __forceinline__ void load_pairs(HPair (&hp)[2], const ParamPtrs &p, size_t off)
{
    const uint2 a = *reinterpret_cast<const uint2 *>(p.zp_init + off);
    const uint2 b = *reinterpret_cast<const uint2 *>(p.scale_init + off);
    const uint2 c = *reinterpret_cast<const uint2 *>(p.alpha + off);
    const uint2 d = *reinterpret_cast<const uint2 *>(p.beta + off);
    const uint2 e = *reinterpret_cast<const uint2 *>(p.target + off);
    hp[0] = HPair{a.x, b.x, c.x, d.x, h2_fma(h2_neg(d.x), e.x, kOne2)};
    hp[1] = HPair{a.y, b.y, c.y, d.y, h2_fma(h2_neg(d.y), e.y, kOne2)};
}

// State update alone (after an appended token).
__device__ __forceinline__ void advance_h(h2 q, HPair &c)
{
    c.zp = h2_fma(c.alpha, h2_mul(q, c.sc), c.zp);
    c.sc = h2_mul(c.sc, h2_fma(c.beta, h2_abs(q), c.omt));
}

// Checkpointed states are stored as float [2][head_dim] (zp, scale) in both arithmetics; fp16 values pass
// through float exactly in either direction.
__device__ __forceinline__ void load_init_state_h(HPair (&hp)[2], const float *init, int c0, int D)
{
    if (init) {
        const float4 zp = *reinterpret_cast<const float4 *>(init + c0);
        const float4 sc = *reinterpret_cast<const float4 *>(init + D + c0);
        hp[0].zp = h2_pack(zp.x, zp.y); hp[1].zp = h2_pack(zp.z, zp.w);
        hp[0].sc = h2_pack(sc.x, sc.y); hp[1].sc = h2_pack(sc.z, sc.w);
    }
}

__device__ __forceinline__ void store_state_h(float *dst, const HPair (&hp)[2], int c0, int D)
{
    *reinterpret_cast<float4 *>(dst + c0) = make_float4(h2_lo(hp[0].zp), h2_hi(hp[0].zp), h2_lo(hp[1].zp), h2_hi(hp[1].zp));
    *reinterpret_cast<float4 *>(dst + D + c0) =
        make_float4(h2_lo(hp[0].sc), h2_hi(hp[0].sc), h2_lo(hp[1].sc), h2_hi(hp[1].sc));
}

// One token of a channel pair: dequantised values (q * sc + zp with the state BEFORE the token), then the update.
__device__ __forceinline__ h2 step_h(h2 q, HPair &c)
{
    const h2 qs = h2_mul(q, c.sc);
    const h2 xh = h2_add(qs, c.zp);
    c.zp = h2_fma(c.alpha, qs, c.zp);
    c.sc = h2_mul(c.sc, h2_fma(c.beta, h2_abs(q), c.omt));
    return xh;
}

// Codes of one byte row of a channel pair.  A byte of the word of channel 2p and the same byte of channel 2p+1
// are brought to byte 0 and byte 2 of one register (one byte permute); field k of both is then masked into the
// mantissas of (1024, 1024) with one logic operation: the result is (1024 + f * 2^(BITS*k)) in both halves, and
// one fp16x2 multiply-add maps it to f - BIAS exactly.
template <int BITS>
struct ByteFields {
    static constexpr int FPB = 8 / BITS;       // fields (tokens) per byte
    template <int BYTE>
    static __device__ __forceinline__ uint32_t gather(uint32_t wa, uint32_t wb)
    {
        return prmt(wa, wb, uint32_t(BYTE | (BYTE << 4) | ((4 + BYTE) << 8) | ((4 + BYTE) << 12)));
    }
    template <int K>
    static __device__ __forceinline__ h2 code(uint32_t bytes)
    {
        constexpr int P = BITS * K;
        constexpr uint32_t mask = (Codec<BITS>::FIELD << P) * 0x10001u;
        uint32_t v;
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(bytes), "n"(mask), "r"(0x64006400u));
        if (P == 0) return h2_sub(v, h_bits2(1024.0 + Codec<BITS>::BIAS));
        return h2_fma(v, h_bits2(1.0 / double(1 << P)), h2_neg(h_bits2(1024.0 / double(1 << P) + Codec<BITS>::BIAS)));
    }
};

// code (-BIAS .. BIAS-1) of token j of a word as an fp16 pair, run-time position (partial words, appends)
template <int BITS>
__device__ __forceinline__ h2 code_h_rt(uint32_t wa, uint32_t wb, int j)
{
    using C = Codec<BITS>;
    const int qa = int((wa >> (BITS * j)) & C::FIELD) - C::BIAS, qb = int((wb >> (BITS * j)) & C::FIELD) - C::BIAS;
    return h2_pack(float(qa), float(qb));
}

// The reference's quantiser (gemv.cu:150-154): fp32 difference and correctly rounded division of the fp16
// operands, round to nearest even, clamp as integers (a NaN quotient gives 0, an infinite one saturates).
template <int BITS>
__device__ __forceinline__ int quantize_h(float x, float zp, float sc)
{
    const int q = __float2int_rn(__fdiv_rn(__fsub_rn(x, zp), sc));
    return max(-Codec<BITS>::BIAS, min(Codec<BITS>::BIAS - 1, q));
}

// ---------------------------------------------------------------------------------- K side

// 8 tokens (BITS bytes of each word, starting at byte 0 of the words given) for the lane's two channel pairs.
// Per token the lane's partial dot products over its even and its odd channels are formed in fp16 (as the
// reference does) and stored as one register to red[(g*8 + token)*36 + lane].
// PARTIAL: only the first `count` tokens exist; the others neither advance the state nor contribute.
template <int BITS, int G, bool PARTIAL>
__device__ __forceinline__ void k_chunk_h(const uint4 &w, HPair (&hp)[2], const h2 (&qv)[G][2], uint32_t *red, int lane,
                                          int count)
{
    using F = ByteFields<BITS>;
    static_for<BITS>([&](auto bc) {
        constexpr int b = decltype(bc)::value;
        const uint32_t by0 = F::template gather<b>(w.x, w.y), by1 = F::template gather<b>(w.z, w.w);
        static_for<F::FPB>([&](auto kc) {
            constexpr int k = decltype(kc)::value;
            constexpr int j = b * F::FPB + k;
            if (!PARTIAL || j < count) {
                const h2 x0 = step_h(F::template code<k>(by0), hp[0]);
                const h2 x1 = step_h(F::template code<k>(by1), hp[1]);
#pragma unroll
                for (int g = 0; g < G; ++g) red[(g * 8 + j) * 36 + lane] = h2_fma(qv[g][1], x1, h2_mul(qv[g][0], x0));
            } else {
#pragma unroll
                for (int g = 0; g < G; ++g) red[(g * 8 + j) * 36 + lane] = 0u;
            }
        });
    });
}

// Sum the partials left by k_chunk_h over the 32 lanes and the two halves (fp16, as the reference's butterfly
// does).  Afterwards lane l (every lane, replicated over l>>3) holds the sum for token (l & 7) of head g as a
// float: the contract of reduce8.
template <int G>
__device__ __forceinline__ void reduce8_h(const uint32_t *red, int lane, float (&sum)[G])
{
    __syncwarp();
    const int row = lane & 7, cb = (lane >> 3) * 8;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint4 a = *reinterpret_cast<const uint4 *>(&red[(g * 8 + row) * 36 + cb]);
        const uint4 b = *reinterpret_cast<const uint4 *>(&red[(g * 8 + row) * 36 + cb + 4]);
        h2 s = h2_add(h2_add(h2_add(a.x, a.y), h2_add(a.z, a.w)), h2_add(h2_add(b.x, b.y), h2_add(b.z, b.w)));
        s = h2_add(s, __shfl_xor_sync(kFull, s, 8));
        s = h2_add(s, __shfl_xor_sync(kFull, s, 16));
        sum[g] = h2_lo(s) + h2_hi(s);
    }
    __syncwarp();
}

template <int BITS, int G, class Sink, int STAGES = kStages, bool WIDE = false>
__device__ __forceinline__ void k_warp_h(const KArgs &a, const Seg &seg, int b, int h, int lane, uint8_t *ring_buf,
                                         uint64_t *ring_bar, float *red_f, Sink &sink)
{
    using C = Codec<BITS>;
    uint32_t *red = reinterpret_cast<uint32_t *>(red_f);
    const int bh = b * a.Hkv + h;
    const int D = WIDE ? a.D : kD, slice = WIDE ? seg.slice : 0;
    const int c0 = kD * slice + 4 * lane;
    HPair hp[2];
    load_pairs(hp, a.p, size_t(h) * D + c0);
    load_init_state_h(hp, seg.init, c0, D);
    h2 qv[G][2];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint2 v = *reinterpret_cast<const uint2 *>(a.q + (size_t(b) * a.Hq + size_t(h) * G + g) * D + c0);
        qv[g][0] = v.x;
        qv[g][1] = v.y;
    }
    const uint32_t row_stride = uint32_t(D) * 4;
    uint8_t *stream = a.cache + (size_t(bh) * a.n_super_cap * D + size_t(kD) * slice) * 4;
    const int n_tok = seg.t_end - seg.t_begin;
    StreamRing<BITS, STAGES, WIDE> ring{ring_buf, ring_bar, stream + size_t(seg.t_begin / C::TPW) * row_stride,
                                  (n_tok + kTileTok - 1) / kTileTok, n_tok, kStatKWait, row_stride};
    ring.prologue(lane);

    bool ok = true;
    int i = 0;
    for (; i < ring.n_tiles; ++i) {
        if (!(ok = ring.wait(i))) break;
        if (!(ok = sink.begin_tile(i))) break;
        const uint4 *tile = ring.tile(i, lane);
        const int ntok = min(kTileTok, n_tok - i * kTileTok);
        float sum[G];
        if (ntok == kTileTok) {
            uint4 w = tile[0];
#pragma unroll 1
            for (int wd = 0; wd < Tile<BITS>::WORDS; ++wd) {
                const uint4 w_next = tile[min(wd + 1, Tile<BITS>::WORDS - 1) * (kD / 4)];
#pragma unroll 1
                for (int c8 = 0; c8 < C::TPW / 8; ++c8) {
                    k_chunk_h<BITS, G, false>(w, hp, qv, red, lane, 8);
                    reduce8_h<G>(red, lane, sum);
#pragma unroll
                    for (int g = 0; g < G; ++g) sink.put8(i, g, wd * C::TPW + c8 * 8, sum[g], lane);
                    if (C::TPW == 16) { w.x >>= 16; w.y >>= 16; w.z >>= 16; w.w >>= 16; }
                }
                w = w_next;
            }
        } else {
#pragma unroll 1
            for (int wd = 0; wd * C::TPW < ntok; ++wd) {
                uint4 w = tile[wd * (kD / 4)];
                const int count = ntok - wd * C::TPW;
#pragma unroll 1
                for (int c8 = 0; c8 < C::TPW / 8 && c8 * 8 < count; ++c8) {
                    k_chunk_h<BITS, G, true>(w, hp, qv, red, lane, count - c8 * 8);
                    reduce8_h<G>(red, lane, sum);
#pragma unroll
                    for (int g = 0; g < G; ++g) sink.put8(i, g, wd * C::TPW + c8 * 8, sum[g], lane);
                    if (C::TPW == 16) { w.x >>= 16; w.y >>= 16; w.z >>= 16; w.w >>= 16; }
                }
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

    // Append k_new as token T with the state left by token T-1 (gemv.cu:744-764), then its own logit from the
    // dequantised value (gemv.cu:766-814), accumulated in fp32 here.
    const uint2 xn = *reinterpret_cast<const uint2 *>(a.x_new + size_t(bh) * D + c0);
    const h2 xnp[2] = {xn.x, xn.y};
    uint4 *slot = reinterpret_cast<uint4 *>(stream + size_t(a.T / C::TPW) * row_stride) + lane;
    uint4 wv = *slot;
    uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    const int sh = BITS * (a.T % C::TPW);
    float xh[4];
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        const int q0 = quantize_h<BITS>(h2_lo(xnp[p]), h2_lo(hp[p].zp), h2_lo(hp[p].sc));
        const int q1 = quantize_h<BITS>(h2_hi(xnp[p]), h2_hi(hp[p].zp), h2_hi(hp[p].sc));
        ww[2 * p] = (ww[2 * p] & ~(C::FIELD << sh)) | (uint32_t(q0 + C::BIAS) << sh);
        ww[2 * p + 1] = (ww[2 * p + 1] & ~(C::FIELD << sh)) | (uint32_t(q1 + C::BIAS) << sh);
        const h2 qf = h2_pack(float(q0), float(q1));
        const h2 deq = h2_fma(qf, hp[p].sc, hp[p].zp);
        xh[2 * p] = h2_lo(deq);
        xh[2 * p + 1] = h2_hi(deq);
        if (seg.ckpt_out) advance_h(qf, hp[p]);
    }
    *slot = make_uint4(ww[0], ww[1], ww[2], ww[3]);
    if (seg.ckpt_out) store_state_h(seg.ckpt_out, hp, c0, D);
    if (!sink.begin_tile(ring.n_tiles)) return;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float s = h2_lo(qv[g][0]) * xh[0];
        s = fmaf(h2_hi(qv[g][0]), xh[1], s);
        s = fmaf(h2_lo(qv[g][1]), xh[2], s);
        s = fmaf(h2_hi(qv[g][1]), xh[3], s);
        s = warp_sum(s);
        if (lane == 0) sink.put_self(g, s);
    }
    sink.finish(lane);
}

// ---------------------------------------------------------------------------------- V side

// 8 tokens for the lane's two channel pairs: weight * value accumulated in fp16 over the 8 tokens, then added
// to the fp32 accumulators (the reference accumulates all tokens in fp16, gemv.cu:1087).  wts: [G][32] fp16
// pairs (w, w), written by a source with HALF_W set.
template <int BITS, int G, bool PARTIAL>
__device__ __forceinline__ void v_chunk_h(const uint4 &w, HPair (&hp)[2], const uint32_t *wts, int tok0,
                                          float (&acc)[G][4], int count)
{
    using F = ByteFields<BITS>;
    h2 part[G][2];
    h2 wt[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint4 a = *reinterpret_cast<const uint4 *>(wts + g * kTileTok + tok0);
        const uint4 b = *reinterpret_cast<const uint4 *>(wts + g * kTileTok + tok0 + 4);
        wt[g][0] = a.x; wt[g][1] = a.y; wt[g][2] = a.z; wt[g][3] = a.w;
        wt[g][4] = b.x; wt[g][5] = b.y; wt[g][6] = b.z; wt[g][7] = b.w;
    }
    static_for<BITS>([&](auto bc) {
        constexpr int b = decltype(bc)::value;
        const uint32_t by0 = F::template gather<b>(w.x, w.y), by1 = F::template gather<b>(w.z, w.w);
        static_for<F::FPB>([&](auto kc) {
            constexpr int k = decltype(kc)::value;
            constexpr int j = b * F::FPB + k;
            if (!PARTIAL || j < count) {
                const h2 x0 = step_h(F::template code<k>(by0), hp[0]);
                const h2 x1 = step_h(F::template code<k>(by1), hp[1]);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    part[g][0] = j == 0 ? h2_mul(wt[g][j], x0) : h2_fma(wt[g][j], x0, part[g][0]);
                    part[g][1] = j == 0 ? h2_mul(wt[g][j], x1) : h2_fma(wt[g][j], x1, part[g][1]);
                }
            }
        });
    });
#pragma unroll
    for (int g = 0; g < G; ++g) {
        acc[g][0] += h2_lo(part[g][0]);
        acc[g][1] += h2_hi(part[g][0]);
        acc[g][2] += h2_lo(part[g][1]);
        acc[g][3] += h2_hi(part[g][1]);
    }
}

template <int BITS, int G, class Src, int STAGES = kStages, bool WIDE = false>
__device__ __forceinline__ void v_warp_h(const VArgs &a, const Seg &seg, int b, int h, int lane, uint8_t *ring_buf,
                                         uint64_t *ring_bar, const float2 *wts_f2, Src &src)
{
    using C = Codec<BITS>;
    const uint32_t *wts = reinterpret_cast<const uint32_t *>(wts_f2);   // the source stores fp16 pairs there
    const int bh = b * a.Hkv + h;
    const int D = WIDE ? a.D : kD, slice = WIDE ? seg.slice : 0;
    const int c0 = kD * slice + 4 * lane;
    HPair hp[2];
    load_pairs(hp, a.p, size_t(h) * D + c0);
    load_init_state_h(hp, seg.init, c0, D);
    float acc[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[g][c] = 0.f;

    const uint32_t row_stride = uint32_t(D) * 4;
    uint8_t *stream = a.cache + (size_t(bh) * a.n_super_cap * D + size_t(kD) * slice) * 4;
    const int n_tok = seg.t_end - seg.t_begin;
    StreamRing<BITS, STAGES, WIDE> ring{ring_buf, ring_bar, stream + size_t(seg.t_begin / C::TPW) * row_stride,
                                  (n_tok + kTileTok - 1) / kTileTok, n_tok, kStatVWait, row_stride};
    ring.prologue(lane);

    bool ok = true;
    int i = 0;
    for (; i < ring.n_tiles; ++i) {
        const int ntok = min(kTileTok, n_tok - i * kTileTok);
        if (!(ok = src.tile_weights(i, ntok, lane, acc))) break;
        if (!(ok = ring.wait(i))) break;
        const uint4 *tile = ring.tile(i, lane);
        if (ntok == kTileTok) {
            uint4 w = tile[0];
#pragma unroll 1
            for (int wd = 0; wd < Tile<BITS>::WORDS; ++wd) {
                const uint4 w_next = tile[min(wd + 1, Tile<BITS>::WORDS - 1) * (kD / 4)];
#pragma unroll 1
                for (int c8 = 0; c8 < C::TPW / 8; ++c8) {
                    v_chunk_h<BITS, G, false>(w, hp, wts, wd * C::TPW + c8 * 8, acc, 8);
                    if (C::TPW == 16) { w.x >>= 16; w.y >>= 16; w.z >>= 16; w.w >>= 16; }
                }
                w = w_next;
            }
        } else {
#pragma unroll 1
            for (int wd = 0; wd * C::TPW < ntok; ++wd) {
                uint4 w = tile[wd * (kD / 4)];
                const int count = ntok - wd * C::TPW;
#pragma unroll 1
                for (int c8 = 0; c8 < C::TPW / 8 && c8 * 8 < count; ++c8) {
                    v_chunk_h<BITS, G, true>(w, hp, wts, wd * C::TPW + c8 * 8, acc, count - c8 * 8);
                    if (C::TPW == 16) { w.x >>= 16; w.y >>= 16; w.z >>= 16; w.w >>= 16; }
                }
            }
        }
        ring.release_and_refill(i, lane);
    }
    if (!ok) {
        ring.drain(i);
        src_give_up(src, c0, 0);
        return;
    }

    if (seg.append) {   // gemv.cu:1105-1159
        float w_self[G];
        if (!src.self_weight(lane, acc, w_self, a.T)) {
            src_give_up(src, c0, 0);
            return;
        }
        const uint2 xn = *reinterpret_cast<const uint2 *>(a.x_new + size_t(bh) * D + c0);
        const h2 xnp[2] = {xn.x, xn.y};
        uint4 *slot = reinterpret_cast<uint4 *>(stream + size_t(a.T / C::TPW) * row_stride) + lane;
        uint4 wv = *slot;
        uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        const int sh = BITS * (a.T % C::TPW);
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const int q0 = quantize_h<BITS>(h2_lo(xnp[p]), h2_lo(hp[p].zp), h2_lo(hp[p].sc));
            const int q1 = quantize_h<BITS>(h2_hi(xnp[p]), h2_hi(hp[p].zp), h2_hi(hp[p].sc));
            ww[2 * p] = (ww[2 * p] & ~(C::FIELD << sh)) | (uint32_t(q0 + C::BIAS) << sh);
            ww[2 * p + 1] = (ww[2 * p + 1] & ~(C::FIELD << sh)) | (uint32_t(q1 + C::BIAS) << sh);
            const h2 qf = h2_pack(float(q0), float(q1));
            const h2 deq = h2_fma(qf, hp[p].sc, hp[p].zp);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                acc[g][2 * p] = fmaf(w_self[g], h2_lo(deq), acc[g][2 * p]);
                acc[g][2 * p + 1] = fmaf(w_self[g], h2_hi(deq), acc[g][2 * p + 1]);
            }
            if (seg.ckpt_out) advance_h(qf, hp[p]);
        }
        *slot = make_uint4(ww[0], ww[1], ww[2], ww[3]);
        if (seg.ckpt_out) store_state_h(seg.ckpt_out, hp, c0, D);
    }
    src.store(a, b, h, c0, acc);
}

// Scan of one tensor of a stream in the arithmetic MODE selects: kArithFma (0) and kArithCanon (1) are the fp32
// recurrence (adkv_decode.cuh); 2 = the fp16-state arithmetic above.
constexpr int kModeHalf = 2;

template <int BITS, int G, int MODE, class Sink, int ST = kStages, bool WIDE = false, bool OUTLINE = false>
__device__ __forceinline__ void k_scan(const KArgs &a, const Seg &seg, int b, int h, int lane, uint8_t *buf, uint64_t *bar,
                                       float *red, Sink &sink)
{
    if constexpr (MODE == kModeHalf) k_warp_h<BITS, G, Sink, ST, WIDE>(a, seg, b, h, lane, buf, bar, red, sink);
    else k_warp<BITS, G, MODE, Sink, ST, WIDE, OUTLINE>(a, seg, b, h, lane, buf, bar, red, sink);
}

template <int BITS, int G, int MODE, class Src, int ST = kStages, bool WIDE = false, bool OUTLINE = false>
__device__ __forceinline__ void v_scan(const VArgs &a, const Seg &seg, int b, int h, int lane, uint8_t *buf, uint64_t *bar,
                                       const float2 *wts, Src &src)
{
    if constexpr (MODE == kModeHalf) v_warp_h<BITS, G, Src, ST, WIDE>(a, seg, b, h, lane, buf, bar, wts, src);
    else v_warp<BITS, G, MODE, Src, ST, WIDE, OUTLINE>(a, seg, b, h, lane, buf, bar, wts, src);
}

}  // namespace adkv
