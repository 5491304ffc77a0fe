// Pieces shared by the fused decode kernels: the logits ring between the K and V warp of a stream, the
// K-side sink that fills it and the V-side source that turns logits into online-softmax weights.
#pragma once
#include "adkv_decode.cuh"

namespace adkv {

// S = number of 128-channel slices of the head (head_dim / 128): each slice has its own K warp, which
// contributes a partial logit, and its own V warp, which sums the S partials.  The full barrier of a slot
// therefore collects S arrivals (one per K warp) and the empty barrier S arrivals (one per V warp).
template <int G, int S = 1>
struct FusedShared {
    float lring[kLogitSlots][S][G][kTileTok];
    uint64_t lfull[kLogitSlots], lempty[kLogitSlots];
    __device__ __forceinline__ void init_barriers(int n_consumers)
    {
        for (int i = 0; i < kLogitSlots; ++i) {
            mbar_init(&lfull[i], S);
            mbar_init(&lempty[i], n_consumers);
        }
    }
};

template <int G, int S = 1>
struct RingSink {
    FusedShared<G, S> *sh;
    int slot;
    int sl;      // this K warp's slice
    __device__ __forceinline__ bool begin_tile(int i)
    {
        slot = i % kLogitSlots;
        return mbar_wait_bounded(&sh->lempty[slot], ((i / kLogitSlots) & 1) ^ 1, kStatLEmptyWait);
    }
    __device__ __forceinline__ void put8(int, int g, int tok, float v, int lane)
    {
        if (lane < 8) sh->lring[slot][sl][g][tok + lane] = v;
    }
    __device__ __forceinline__ void end_tile(int, int lane)
    {
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->lfull[slot]);
    }
    __device__ __forceinline__ void put_self(int g, float v) { sh->lring[slot][sl][g][0] = v; }
    __device__ __forceinline__ void finish(int lane) { end_tile(0, lane); }
};

// Weights of a tile for the V warp: [G][32] float2 (w, w), or with HALF_W [G][32] fp16 pairs (w, w) in the first
// half of the same array (the fp16-state kernels multiply in fp16x2).
template <bool HALF_W>
__device__ __forceinline__ void put_weight(float2 *wts, int idx, float w)
{
    if (HALF_W) {
        const __half2 h = __floats2half2_rn(w, w);
        reinterpret_cast<uint32_t *>(wts)[idx] = *reinterpret_cast<const uint32_t *>(&h);
    } else {
        wts[idx] = make_float2(w, w);
    }
}

template <int G, int S = 1, bool HALF_W = false>
struct SoftmaxSrc {
    FusedShared<G, S> *sh;
    float2 *wts;           // [G][32], every weight stored twice (packed multiplier for a channel pair)
    const float *mask;     // row of this batch or nullptr
    float scale2;          // scaling * log2(e)
    int n_tiles;           // tiles of this segment
    int t_begin;           // first token of this segment (mask index of local token 0)
    float m[G], l[G];

    __device__ __forceinline__ void init()
    {
#pragma unroll
        for (int g = 0; g < G; ++g) { m[g] = -INFINITY; l[g] = 0.f; }
    }
    // online-softmax update of head g with this lane's logit v (already in log2 units, -inf if invalid)
    __device__ __forceinline__ float update(int g, float v, float (&acc)[G][4])
    {
        const float m_new = fmaxf(m[g], warp_max(v));
        const bool dead = (m_new == -INFINITY);
        const float corr = dead ? 1.f : exp2f(m[g] - m_new);
        const float pw = dead ? 0.f : exp2f(v - m_new);
        l[g] = fmaf(l[g], corr, warp_sum(pw));
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[g][c] *= corr;
        m[g] = m_new;
        return pw;
    }
    __device__ __forceinline__ bool tile_weights(int i, int ntok, int lane, float (&acc)[G][4])
    {
        const int slot = i % kLogitSlots;
        const float mk = (mask && lane < ntok) ? mask[t_begin + i * kTileTok + lane] * 1.4426950408889634f : 0.f;
        if (!mbar_wait_bounded(&sh->lfull[slot], (i / kLogitSlots) & 1, kStatLFullWait)) return false;
        float x[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            x[g] = sh->lring[slot][0][g][lane];
#pragma unroll
            for (int k = 1; k < S; ++k) x[g] += sh->lring[slot][k][g][lane];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->lempty[slot]);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float v = lane < ntok ? fmaf(x[g], scale2, mk) : -INFINITY;
            const float pw = update(g, v, acc);
            put_weight<HALF_W>(wts, g * kTileTok + lane, pw);
        }
        __syncwarp();
        return true;
    }
    __device__ __forceinline__ bool self_weight(int lane, float (&acc)[G][4], float (&w_self)[G], int T)
    {
        const int slot = n_tiles % kLogitSlots;
        if (!mbar_wait_bounded(&sh->lfull[slot], (n_tiles / kLogitSlots) & 1, kStatLFullWait)) return false;
        const float mk = mask ? mask[T] * 1.4426950408889634f : 0.f;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float xs = sh->lring[slot][0][g][0];
#pragma unroll
            for (int k = 1; k < S; ++k) xs += sh->lring[slot][k][g][0];
            const float v = fmaf(xs, scale2, mk);
            // all lanes hold the same v: update() would count it 32 times, so do it by hand
            const float m_new = fmaxf(m[g], v);
            const bool dead = (m_new == -INFINITY);
            const float corr = dead ? 1.f : exp2f(m[g] - m_new);
            const float pw = dead ? 0.f : exp2f(v - m_new);
            l[g] = fmaf(l[g], corr, pw);
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[g][c] *= corr;
            m[g] = m_new;
            w_self[g] = pw;
        }
        return true;
    }
    __device__ __forceinline__ float norm(int g) const { return l[g]; }
    __device__ __forceinline__ void store(const VArgs &a, int b, int h, int c0, const float (&acc)[G][4]) const
    {
        store_normalised<G>(*this, a, b, h, c0, acc);
    }
};

}  // namespace adkv
