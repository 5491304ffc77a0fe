// Decode-side scans over one (batch, kv head) stream of the packed cache.
//
// One warp owns a tensor (K or V) of a stream; lane l owns channels 4l..4l+3, i.e. one 16-byte
// vector of every supergroup.  The stream is brought into shared memory in tiles of 32 tokens
// by non-multicast bulk copies (1-D TMA) that complete on mbarriers; each warp runs its own
// ring, issued by its lane 0, so no other warp can stall it.
//
// K warp: replays the recurrence, forms per-lane partial dot products with the query for 8
// tokens at a time, reduces them across lanes through a shared-memory transpose, and hands the
// logits to a sink (shared-memory ring in the fused kernel, fp16 global in forward_qk).
// V warp: takes softmax weights for a tile (from the ring, with online softmax, or from fp16
// global in forward_ov), replays the recurrence and accumulates weight * value.
// Both then quantise the new token with the state the replay left (token T-1), write it into
// slot T and add its own contribution (src/adkv/kernel/gemv.cu:744-814, 1105-1159).
#pragma once
#include <type_traits>
#include "adkv_device.cuh"

namespace adkv {

constexpr int kTileTok = 32;   // tokens per tile
constexpr int kStages = 3;     // bulk-copy ring depth per warp
constexpr int kLogitSlots = 4; // logits ring depth (fused kernel)

// Replay arithmetic of the fp32 recurrence (template parameter ARITH of the scans below):
//   kArithFma   contracted: zp = fma(alpha, q*s, zp), s = s * fma(beta, |q|, 1 - beta*target)
//   kArithCanon the reference's order, one rounding per operation (src/adkv/train/train_model.py:70-81)
// (2 is taken by the fp16-state arithmetic, adkv_half.cuh.)  Only kArithCanon reproduces the encoder's state bit
// for bit.  kArithFma is meant for decoding next to a persisted tail state (KArgs::tail), which then supplies
// the canonical state the appended token is quantised with.
constexpr int kArithFma = 0, kArithCanon = 1;

template <int BITS>
struct Tile {
    static constexpr int WORDS = kTileTok / Codec<BITS>::TPW;   // words per channel per tile
    static constexpr int BYTES = WORDS * kD * 4;                // 4-bit: 2048, 2-bit: 1024
};

// Per-warp bulk-copy ring over the words of one stream.
// WIDE = false: head dim 128, the stream is contiguous and its geometry is known at compile time (keeps the
// 128-wide kernels free of the registers and branches the strided case needs).
template <int BITS, int STAGES = kStages, bool WIDE = false>
struct StreamRing {
    uint8_t *buf;           // STAGES * Tile::BYTES, 128-byte aligned
    uint64_t *bar;          // STAGES barriers
    const uint8_t *src;     // first word row of this warp's 128-channel slice of the stream
    int n_tiles, T;
    int wait_code;
    uint32_t row_stride;    // bytes between word rows in global memory: 4 * head_dim (512 = contiguous slice)

    __device__ __forceinline__ uint32_t tile_bytes(int i) const
    {
        const int ntok = min(kTileTok, T - i * kTileTok);
        const int words = (ntok + Codec<BITS>::TPW - 1) / Codec<BITS>::TPW;
        return uint32_t(words) * kD * 4;
    }
    // lane 0 only
    __device__ __forceinline__ void issue(int i) const
    {
        const int st = i % STAGES;
        const uint32_t bytes = tile_bytes(i);
        mbar_expect_tx(&bar[st], bytes);
        if (!WIDE || row_stride == kD * 4) {
            bulk_load(buf + st * Tile<BITS>::BYTES, src + size_t(i) * Tile<BITS>::BYTES, bytes, &bar[st]);
        } else {   // head_dim > 128: the slice's 512-byte rows are strided, one copy per row
            const uint8_t *row = src + size_t(i) * Tile<BITS>::WORDS * row_stride;
            for (uint32_t off = 0; off < bytes; off += kD * 4, row += row_stride)
                bulk_load(buf + st * Tile<BITS>::BYTES + off, row, kD * 4, &bar[st]);
        }
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
    __device__ __forceinline__ const uint4 *tile(int i, int lane) const
    {
        return reinterpret_cast<const uint4 *>(buf + (i % STAGES) * Tile<BITS>::BYTES) + lane;
    }
    // all lanes, after the tile has been consumed
    __device__ __forceinline__ void release_and_refill(int i, int lane) const
    {
        __syncwarp();
        if (lane == 0 && i + STAGES < n_tiles) issue(i + STAGES);
    }
    // After a failed wait: give copies already issued a bounded chance to land before the
    // shared memory is handed back.
    __device__ __forceinline__ void drain(int from) const
    {
        const int issued = min(n_tiles, from + STAGES);
        for (int i = from; i < issued; ++i)
            if (!mbar_wait_bounded(&bar[i % STAGES], (i / STAGES) & 1, kStatDrain)) break;
    }
};

// ---------------------------------------------------------------------------------- K side

// Replay 8 tokens (fields 0..7 of the 4 words in `w`; the caller shifts the second half of a 16-token
// word down) and leave the per-lane partial dot products of head g, token j in red[(g*8 + j)*36 + lane].
// The two halves of 4 tokens run through ONE body in a two-trip loop, which halves the straight-line
// code (with several query heads per KV head the unrolled body no longer fitted the instruction
// cache).  `count`: valid fields when PARTIAL (the others are stored as zero).
template <int BITS, int G, bool EXACT, bool PARTIAL, bool GUARDED>
__device__ __forceinline__ void k_chunk(const uint4 &w, const FieldConsts<BITS> &fc, Chan (&ch)[4],
                                        const float (&qv)[G][4], float *red, int lane, int count, float smin,
                                        float smax)
{
    uint32_t grp[4] = {w.x, w.y, w.z, w.w};
    // one query head: both halves unrolled (measured faster); several heads: one body, two trips
#pragma unroll(G == 1 ? 2 : 1)
    for (int half = 0; half < 2; ++half) {
        static_for<4>([&](auto kc) {
            constexpr int k = decltype(kc)::value;
            float part[G];
            if (!PARTIAL || 4 * half + k < count) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float q = fc.template code<k>(grp[c]);
                    const float xh = replay_step<EXACT, GUARDED>(q, ch[c], smin, smax);
#pragma unroll
                    for (int g = 0; g < G; ++g) part[g] = c == 0 ? qv[g][0] * xh : fmaf(qv[g][c], xh, part[g]);
                }
            } else {
#pragma unroll
                for (int g = 0; g < G; ++g) part[g] = 0.f;
            }
#pragma unroll
            for (int g = 0; g < G; ++g) red[(g * 8 + 4 * half + k) * 36 + lane] = part[g];
        });
#pragma unroll
        for (int c = 0; c < 4; ++c) grp[c] >>= 4 * BITS;
    }
}

// The unguarded, full 8-token case of k_chunk on channel pairs (packed fp32): identical results for the
// state; the per-lane partial dot product is summed in a different order (pairs first).
template <int BITS, int G, bool EXACT>
__device__ __forceinline__ void k_chunk2(const uint4 &w, const FieldConsts<BITS> &fc, Chan (&ch)[4],
                                         const PairConst (&pc)[2], f32x2 one, const f32x2 (&qv2)[G][2], float *red,
                                         int lane)
{
    uint32_t grp[4] = {w.x, w.y, w.z, w.w};
    f32x2 zp[2] = {pk2(ch[0].zp, ch[1].zp), pk2(ch[2].zp, ch[3].zp)};
    f32x2 s[2] = {pk2(ch[0].s, ch[1].s), pk2(ch[2].s, ch[3].s)};
#pragma unroll(G == 1 ? 2 : 1)
    for (int half = 0; half < 2; ++half) {
        static_for<4>([&](auto kc) {
            constexpr int k = decltype(kc)::value;
            f32x2 part[G];
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const f32x2 q2 = fc.template code2<k>(grp[2 * p], grp[2 * p + 1]);
                const f32x2 xh = replay_step2<EXACT>(q2, zp[p], s[p], pc[p], one);
#pragma unroll
                for (int g = 0; g < G; ++g) part[g] = p == 0 ? mul2(qv2[g][0], xh) : fma2(qv2[g][1], xh, part[g]);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float a, b;
                upk2(part[g], a, b);
                red[(g * 8 + 4 * half + k) * 36 + lane] = a + b;
            }
        });
#pragma unroll
        for (int c = 0; c < 4; ++c) grp[c] >>= 4 * BITS;
    }
    upk2(zp[0], ch[0].zp, ch[1].zp);
    upk2(zp[1], ch[2].zp, ch[3].zp);
    upk2(s[0], ch[0].s, ch[1].s);
    upk2(s[1], ch[2].s, ch[3].s);
}

// Sum the partials left by k_chunk over the 32 lanes: each lane reads 8 lanes' values of one token
// (two 16-byte loads from the padded transpose) and two shuffles finish the job; afterwards lane l
// (every lane, replicated over l>>3) holds the full sum for token (l & 7) of head g.
// red: float [G][8][36] of this warp.
template <int G>
__device__ __forceinline__ void reduce8(const float *red, int lane, float (&sum)[G])
{
    __syncwarp();
    const int row = lane & 7, cb = (lane >> 3) * 8;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float4 a = *reinterpret_cast<const float4 *>(&red[(g * 8 + row) * 36 + cb]);
        const float4 b = *reinterpret_cast<const float4 *>(&red[(g * 8 + row) * 36 + cb + 4]);
        float s = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
        s += __shfl_xor_sync(kFull, s, 8);
        s += __shfl_xor_sync(kFull, s, 16);
        sum[g] = s;
    }
    __syncwarp();
}

// The part of a stream one warp pair works on.  The whole-stream kernels use {0, T, true, nullptr, nullptr, 0};
// the checkpointed kernel gives every segment its own pair of warps.
struct Seg {
    int t_begin;          // first token replayed (a multiple of kTileTok)
    int t_end;            // one past the last token replayed
    bool append;          // quantise x_new as token t_end (== T), write it, add its own term
    const float *init;    // state before token t_begin of this stream, [2][head_dim] (zp, scale); nullptr = parameters
    float *ckpt_out;      // where to store the state after the appended token, [2][head_dim]; nullptr = nowhere
    int slice;            // which 128-channel slice of the head this warp owns (0 for head_dim 128)
};

__device__ __forceinline__ void load_init_state(Chan (&ch)[4], const float *init, int c0, int D)
{
    if (init) {
        const float4 zp = *reinterpret_cast<const float4 *>(init + c0);
        const float4 sc = *reinterpret_cast<const float4 *>(init + D + c0);
        ch[0].zp = zp.x; ch[1].zp = zp.y; ch[2].zp = zp.z; ch[3].zp = zp.w;
        ch[0].s = sc.x; ch[1].s = sc.y; ch[2].s = sc.z; ch[3].s = sc.w;
    }
}

__device__ __forceinline__ void store_state(float *dst, const Chan (&ch)[4], int c0, int D)
{
    *reinterpret_cast<float4 *>(dst + c0) = make_float4(ch[0].zp, ch[1].zp, ch[2].zp, ch[3].zp);
    *reinterpret_cast<float4 *>(dst + D + c0) = make_float4(ch[0].s, ch[1].s, ch[2].s, ch[3].s);
}

struct KArgs {
    const __half *q;        // [B, Hq, D]
    uint8_t *cache;         // [B, Hkv, n_super_cap, D] words
    const __half *x_new;    // [B, Hkv, D]
    ParamPtrs p;
    int Hq, Hkv, T, n_super_cap;
    float smin, smax;
    int D;                  // head dim (128, 256 or 512)
    float *tail = nullptr;  // [B, Hkv, 2, D] canonical state after token T-1 (zp then scale), or nullptr
    bool tail_keep = false; // leave `tail` as it is instead of advancing it over the appended token
};

// Append the new token of this lane's 4 channels as token T: quantise, merge the code into word `slot`, return the
// dequantised values in xh.  Without a tail the state the replay left in `ch` is used (it is the encoder's state
// only when the replay was canonical).  With a tail the token is quantised with that state -- the canonical one
// after token T-1, as encode / append / an earlier decode step left it -- whatever arithmetic replayed the cache,
// and the tail then advances canonically; `ch` is not read.  ckpt_out, if set, receives the state after token T.
template <int BITS, int ARITH>
__device__ __forceinline__ void append_new_token(Chan (&ch)[4], const ParamPtrs &p, size_t poff, float *tail,
                                                 bool tail_keep, const __half *x_new, uint4 *slot, int T, float smin,
                                                 float smax, float *ckpt_out, int c0, int D, float (&xh)[4])
{
    using C = Codec<BITS>;
    float xn[4];
    load_half4(xn, x_new);
    uint4 wv = *slot;
    uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    const int sh = BITS * (T % C::TPW);
    if (tail) {
        float tg[4];
        load_half4(tg, p.target + poff);
        load_init_state(ch, tail, c0, D);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            ch[c].tc = tg[c];   // canonical form of the constant, whatever the replay used
            float rh;
            const float q = quantize<BITS>(xn[c], ch[c], rh);
            xh[c] = __fadd_rn(rh, ch[c].zp);
            ww[c] = (ww[c] & ~(C::FIELD << sh)) | (uint32_t(int(q) + C::BIAS) << sh);
            advance_canonical(q, rh, ch[c], smin, smax);
        }
        if (!tail_keep) store_state(tail, ch, c0, D);
    } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float rh;
            const float q = quantize<BITS>(xn[c], ch[c], rh);
            xh[c] = __fadd_rn(rh, ch[c].zp);
            ww[c] = (ww[c] & ~(C::FIELD << sh)) | (uint32_t(int(q) + C::BIAS) << sh);
            if (ckpt_out) advance_like_replay<ARITH == kArithCanon>(q, rh, ch[c], smin, smax);
        }
    }
    *slot = make_uint4(ww[0], ww[1], ww[2], ww[3]);
    if (ckpt_out) store_state(ckpt_out, ch, c0, D);
}

struct Chan4 {
    Chan c[4];
};

// The guarded, possibly partial chunk as a real function call.  It runs where a scale sits near a clamp bound (or
// under the eps guard) and for the ragged last tile of a stream: rarely.  Inlined next to the packed fast path it
// made the scan loops large enough to miss the instruction cache on every tile; as a call the loops hold only the
// fast path.  State and operands travel by value in registers.  Opt-in per kernel (template parameter OUTLINE of
// k_warp / v_warp): a call changes the register allocation of the whole kernel, and with more than two query heads per
// KV head the operands no longer fit the registers of the calling convention, which would move the accumulators to
// local memory for the whole scan.  The fused whole-head kernel uses it for 4-bit codes with one query head per KV head (measured:
// 15 % faster at 128-token contexts, no change at 4096).
template <int G>
struct QueryRegs {
    float v[G][4];
};
template <int BITS, int G, bool EXACT>
__device__ __noinline__ Chan4 k_chunk_guarded(uint4 w, Chan4 st, QueryRegs<G> q, float *red, int lane, int count,
                                              float smin, float smax)
{
    FieldConsts<BITS> fc;
    fc.init();
    k_chunk<BITS, G, EXACT, true, true>(w, fc, st.c, q.v, red, lane, count, smin, smax);
    return st;
}

// Sink interface (duck-typed):
//   bool begin_tile(int i)            wait for room; false = bounded wait gave up
//   void put8(int i, int g, int tok_in_tile, float v, int lane)   called by lanes 0..7 with tok = base + lane
//   void end_tile(int i, int lane)
//   void put_self(int g, float v)     lane 0
//   void finish(int lane)
template <int BITS, int G, int ARITH, class Sink, int STAGES = kStages, bool WIDE = false, bool OUTLINE = false>
__device__ __forceinline__ void k_warp(const KArgs &a, const Seg &seg, int b, int h, int lane, uint8_t *ring_buf,
                                       uint64_t *ring_bar, float *red, Sink &sink)
{
    using C = Codec<BITS>;
    constexpr bool EXACT = ARITH == kArithCanon;
    const int bh = b * a.Hkv + h;
    const int D = WIDE ? a.D : kD, slice = WIDE ? seg.slice : 0;
    const int c0 = kD * slice + 4 * lane;      // first of this lane's 4 channels within the head
    const uint32_t row_stride = uint32_t(D) * 4;
    uint8_t *stream = a.cache + (size_t(bh) * a.n_super_cap * D + size_t(kD) * slice) * 4;
    const int n_tok = seg.t_end - seg.t_begin;
    StreamRing<BITS, STAGES, WIDE> ring{ring_buf, ring_bar, stream + size_t(seg.t_begin / C::TPW) * row_stride,
                          (n_tok + kTileTok - 1) / kTileTok, n_tok, kStatKWait, row_stride};
    ring.prologue(lane);   // first: the copies of the first tiles fly while the parameters below are loaded
    Chan ch[4];
    SafeRange safe;
    FieldConsts<BITS> fc;
    fc.init();
    load_chan4<BITS, EXACT>(ch, safe, a.p, size_t(h) * D + c0, a.smin, a.smax);
    load_init_state(ch, seg.init, c0, D);
    float qv[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) load_half4(qv[g], a.q + (size_t(b) * a.Hq + size_t(h) * G + g) * D + c0);
    PairConst pc[2];
    make_pair_consts<EXACT>(ch, pc);
    const f32x2 one = opaque_ones2();   // read once: a constant-memory load per chunk would stall the chain
    f32x2 qv2[G][2];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        qv2[g][0] = pk2(qv[g][0], qv[g][1]);
        qv2[g][1] = pk2(qv[g][2], qv[g][3]);
    }


    auto guarded = [&](const uint4 &w, int count, auto partial_tag) {
        if constexpr (!OUTLINE) {
            k_chunk<BITS, G, EXACT, decltype(partial_tag)::value, true>(w, fc, ch, qv, red, lane, count, a.smin, a.smax);
        } else {
            Chan4 st;
            QueryRegs<G> qr;
#pragma unroll
            for (int c = 0; c < 4; ++c) st.c[c] = ch[c];
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int c = 0; c < 4; ++c) qr.v[g][c] = qv[g][c];
            st = k_chunk_guarded<BITS, G, EXACT>(w, st, qr, red, lane, count, a.smin, a.smax);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                ch[c].zp = st.c[c].zp;
                ch[c].s = st.c[c].s;
            }
        }
    };

    bool ok = true;
    int i = 0;
    for (; i < ring.n_tiles; ++i) {
        if (!(ok = ring.wait(i))) break;
        if (!(ok = sink.begin_tile(i))) break;
        const uint4 *tile = ring.tile(i, lane);
        const int ntok = min(kTileTok, n_tok - i * kTileTok);
        float sum[G];
        if (ntok == kTileTok) {
            // not unrolled over the words of the tile: the loop body must stay resident in the
            // instruction cache while K and V warps of many streams interleave
            uint4 w = tile[0];
#pragma unroll 1
            for (int wd = 0; wd < Tile<BITS>::WORDS; ++wd) {
                const uint4 w_next = tile[min(wd + 1, Tile<BITS>::WORDS - 1) * (kD / 4)];
#pragma unroll 1
                for (int c8 = 0; c8 < C::TPW / 8; ++c8) {
                    if (safe.holds(ch)) k_chunk2<BITS, G, EXACT>(w, fc, ch, pc, one, qv2, red, lane);
                    else guarded(w, 8, std::false_type{});
                    reduce8<G>(red, lane, sum);
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
                const int count = ntok - wd * C::TPW;   // valid fields in this word (may exceed TPW)
#pragma unroll 1
                for (int c8 = 0; c8 < C::TPW / 8 && c8 * 8 < count; ++c8) {
                    guarded(w, count - c8 * 8, std::true_type{});
                    reduce8<G>(red, lane, sum);
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
    // Append k_new as token T with the state after token T-1, then its own logit from the
    // dequantised value.
    float xh[4];
    append_new_token<BITS, ARITH>(ch, a.p, size_t(h) * D + c0, a.tail ? a.tail + size_t(bh) * 2 * D : nullptr,
                                  a.tail_keep, a.x_new + size_t(bh) * D + c0,
                                  reinterpret_cast<uint4 *>(stream + size_t(a.T / C::TPW) * row_stride) + lane, a.T,
                                  a.smin, a.smax, seg.ckpt_out, c0, D, xh);
    if (!sink.begin_tile(ring.n_tiles)) return;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) s = fmaf(qv[g][c], xh[c], s);
        s = warp_sum(s);
        if (lane == 0) sink.put_self(g, s);
    }
    sink.finish(lane);
}

// ---------------------------------------------------------------------------------- V side

template <int BITS, int G, bool EXACT, bool PARTIAL, bool GUARDED>
__device__ __forceinline__ void v_chunk(const uint4 &w, const FieldConsts<BITS> &fc, Chan (&ch)[4],
                                        const float2 *wts /* [G][32] smem, each weight twice */, int tok0,
                                        float (&acc)[G][4], int count, float smin, float smax)
{
    uint32_t grp[4] = {w.x, w.y, w.z, w.w};
    // one query head: both halves unrolled (measured faster); several heads: one body, two trips
#pragma unroll(G == 1 ? 2 : 1)
    for (int half = 0; half < 2; ++half) {
        float wt[G][4];
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int k = 0; k < 4; ++k) wt[g][k] = wts[g * kTileTok + tok0 + 4 * half + k].x;
        }
        static_for<4>([&](auto kc) {
            constexpr int k = decltype(kc)::value;
            if (!PARTIAL || 4 * half + k < count) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float q = fc.template code<k>(grp[c]);
                    const float xh = replay_step<EXACT, GUARDED>(q, ch[c], smin, smax);
#pragma unroll
                    for (int g = 0; g < G; ++g) acc[g][c] = fmaf(wt[g][k], xh, acc[g][c]);
                }
            }
        });
#pragma unroll
        for (int c = 0; c < 4; ++c) grp[c] >>= 4 * BITS;
    }
}

// The unguarded, full 8-token case of v_chunk on channel pairs (packed fp32).  `wts2` holds every weight
// twice ([G][32] float2) so that one 8-byte load yields the packed multiplier.
template <int BITS, int G, bool EXACT>
__device__ __forceinline__ void v_chunk2(const uint4 &w, const FieldConsts<BITS> &fc, Chan (&ch)[4],
                                         const PairConst (&pc)[2], f32x2 one, const float2 *wts2, int tok0,
                                         float (&acc)[G][4])
{
    uint32_t grp[4] = {w.x, w.y, w.z, w.w};
    f32x2 zp[2] = {pk2(ch[0].zp, ch[1].zp), pk2(ch[2].zp, ch[3].zp)};
    f32x2 s[2] = {pk2(ch[0].s, ch[1].s), pk2(ch[2].s, ch[3].s)};
    f32x2 acc2[G][2];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        acc2[g][0] = pk2(acc[g][0], acc[g][1]);
        acc2[g][1] = pk2(acc[g][2], acc[g][3]);
    }
#pragma unroll(G == 1 ? 2 : 1)
    for (int half = 0; half < 2; ++half) {
        f32x2 wt[G][4];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const ulonglong2 a = *reinterpret_cast<const ulonglong2 *>(wts2 + g * kTileTok + tok0 + 4 * half);
            const ulonglong2 b = *reinterpret_cast<const ulonglong2 *>(wts2 + g * kTileTok + tok0 + 4 * half + 2);
            wt[g][0] = a.x; wt[g][1] = a.y; wt[g][2] = b.x; wt[g][3] = b.y;
        }
        static_for<4>([&](auto kc) {
            constexpr int k = decltype(kc)::value;
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const f32x2 q2 = fc.template code2<k>(grp[2 * p], grp[2 * p + 1]);
                const f32x2 xh = replay_step2<EXACT>(q2, zp[p], s[p], pc[p], one);
#pragma unroll
                for (int g = 0; g < G; ++g) acc2[g][p] = fma2(wt[g][k], xh, acc2[g][p]);
            }
        });
#pragma unroll
        for (int c = 0; c < 4; ++c) grp[c] >>= 4 * BITS;
    }
    upk2(zp[0], ch[0].zp, ch[1].zp);
    upk2(zp[1], ch[2].zp, ch[3].zp);
    upk2(s[0], ch[0].s, ch[1].s);
    upk2(s[1], ch[2].s, ch[3].s);
#pragma unroll
    for (int g = 0; g < G; ++g) {
        upk2(acc2[g][0], acc[g][0], acc[g][1]);
        upk2(acc2[g][1], acc[g][2], acc[g][3]);
    }
}

struct VArgs {
    uint8_t *cache;         // [B, Hkv, n_super_cap, D] words
    const __half *x_new;    // [B, Hkv, D]
    __half *out;            // [B, Hq, D]
    ParamPtrs p;
    int Hq, Hkv, T, n_super_cap;
    float smin, smax;
    int D;                  // head dim (128, 256 or 512)
    float *tail = nullptr;  // as KArgs::tail, for the V cache
    bool tail_keep = false;
};

// A V scan that gives up on a bounded wait tells its source, if the source cares (give_up is optional): the
// checkpointed kernel's source then marks its partial result as unusable instead of leaving stale memory behind.
template <class S>
__device__ __forceinline__ auto src_give_up(S &s, int c0, int) -> decltype(s.give_up(c0), void()) { s.give_up(c0); }
template <class S>
__device__ __forceinline__ void src_give_up(S &, int, long) {}

// Source interface (duck-typed):
//   bool tile_weights(int i, int ntok, int lane, float (&acc)[G][4])
//        fill wts[g][0..31] for tile i (0 for tokens >= ntok); may rescale acc (online softmax);
//        false = bounded wait gave up
//   bool self_weight(int lane, float (&acc)[G][4], float (&w_self)[G], int T)
//   void store(const VArgs&, int b, int h, int c0, const float (&acc)[G][4])   write the result (c0: first channel)
//   void give_up(int c0)              optional: called instead of store() when a bounded wait gave up

// v_chunk's guarded, possibly partial form as a real function call (see k_chunk_guarded).
template <int G>
struct VState {
    Chan c[4];
    float acc[G][4];
};
template <int BITS, int G, bool EXACT>
__device__ __noinline__ VState<G> v_chunk_guarded(uint4 w, VState<G> st, const float2 *wts, int tok0, int count,
                                                  float smin, float smax)
{
    FieldConsts<BITS> fc;
    fc.init();
    v_chunk<BITS, G, EXACT, true, true>(w, fc, st.c, wts, tok0, st.acc, count, smin, smax);
    return st;
}

template <int BITS, int G, int ARITH, class Src, int STAGES = kStages, bool WIDE = false, bool OUTLINE = false>
__device__ __forceinline__ void v_warp(const VArgs &a, const Seg &seg, int b, int h, int lane, uint8_t *ring_buf,
                                       uint64_t *ring_bar, const float2 *wts, Src &src)
{
    using C = Codec<BITS>;
    constexpr bool EXACT = ARITH == kArithCanon;
    const int bh = b * a.Hkv + h;
    const int D = WIDE ? a.D : kD, slice = WIDE ? seg.slice : 0;
    const int c0 = kD * slice + 4 * lane;
    const uint32_t row_stride = uint32_t(D) * 4;
    uint8_t *stream = a.cache + (size_t(bh) * a.n_super_cap * D + size_t(kD) * slice) * 4;
    const int n_tok = seg.t_end - seg.t_begin;
    StreamRing<BITS, STAGES, WIDE> ring{ring_buf, ring_bar, stream + size_t(seg.t_begin / C::TPW) * row_stride,
                          (n_tok + kTileTok - 1) / kTileTok, n_tok, kStatVWait, row_stride};
    ring.prologue(lane);   // first: the copies of the first tiles fly while the parameters below are loaded
    Chan ch[4];
    SafeRange safe;
    FieldConsts<BITS> fc;
    fc.init();
    load_chan4<BITS, EXACT>(ch, safe, a.p, size_t(h) * D + c0, a.smin, a.smax);
    load_init_state(ch, seg.init, c0, D);
    PairConst pc[2];
    make_pair_consts<EXACT>(ch, pc);
    const f32x2 one = opaque_ones2();   // read once: a constant-memory load per chunk would stall the chain
    float acc[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[g][c] = 0.f;


    auto guarded = [&](const uint4 &w, int tok0, int count, auto partial_tag) {
        if constexpr (!OUTLINE) {
            v_chunk<BITS, G, EXACT, decltype(partial_tag)::value, true>(w, fc, ch, wts, tok0, acc, count, a.smin, a.smax);
        } else {
            VState<G> st;
#pragma unroll
            for (int c = 0; c < 4; ++c) st.c[c] = ch[c];
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int c = 0; c < 4; ++c) st.acc[g][c] = acc[g][c];
            st = v_chunk_guarded<BITS, G, EXACT>(w, st, wts, tok0, count, a.smin, a.smax);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                ch[c].zp = st.c[c].zp;
                ch[c].s = st.c[c].s;
            }
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[g][c] = st.acc[g][c];
        }
    };

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
                    const int tok0 = wd * C::TPW + c8 * 8;
                    if (safe.holds(ch)) v_chunk2<BITS, G, EXACT>(w, fc, ch, pc, one, wts, tok0, acc);
                    else guarded(w, tok0, 8, std::false_type{});
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
                    guarded(w, wd * C::TPW + c8 * 8, count - c8 * 8, std::true_type{});
                    if (C::TPW == 16) { w.x >>= 16; w.y >>= 16; w.z >>= 16; w.w >>= 16; }
                }
            }
        }
        ring.release_and_refill(i, lane);   // also orders this tile's reads of wts before the next fill
    }
    if (!ok) {
        ring.drain(i);
        src_give_up(src, c0, 0);
        return;
    }

    if (seg.append) {
        float xh[4];
        float w_self[G];
        if (!src.self_weight(lane, acc, w_self, a.T)) {
            src_give_up(src, c0, 0);
            return;
        }
        append_new_token<BITS, ARITH>(ch, a.p, size_t(h) * D + c0, a.tail ? a.tail + size_t(bh) * 2 * D : nullptr,
                                      a.tail_keep, a.x_new + size_t(bh) * D + c0,
                                      reinterpret_cast<uint4 *>(stream + size_t(a.T / C::TPW) * row_stride) + lane, a.T,
                                      a.smin, a.smax, seg.ckpt_out, c0, D, xh);
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[g][c] = fmaf(w_self[g], xh[c], acc[g][c]);
    }
    src.store(a, b, h, c0, acc);
}

// Final division by the softmax denominator and fp16 store of the 4 channels of every head.
template <int G, class Src>
__device__ __forceinline__ void store_normalised(const Src &src, const VArgs &a, int b, int h, int c0,
                                                 const float (&acc)[G][4])
{
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float inv = 1.0f / src.norm(g);
        float o[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) o[c] = acc[g][c] * inv;
        store_half4(a.out + (size_t(b) * a.Hq + size_t(h) * G + g) * a.D + c0, o);
    }
}

}  // namespace adkv
