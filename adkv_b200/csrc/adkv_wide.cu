// Part of libadkv_b200.so (sm_100a).  See include/adkv_b200.h for the contract of every entry point.
//
// Head dims 256 and 512 (the reference's "channel split" configurations, src/adkv/kernel/gemv.cu:336-353,
// 857-874, 1208-1225).  A head is S = D/128 slices of 128 channels; every slice keeps the lane ownership of
// the 128-wide kernels (lane l owns 4 channels of its slice) and gets its own K warp and V warp inside the
// stream's CTA.  Logits are sums over all channels, so the S K warps post partial logits to a shared-memory
// ring slot and every consumer adds the S partials (no atomics, fixed summation order).
#include "adkv_host.h"

#include "adkv_half.cuh"
#include "adkv_softmax.cuh"

namespace adkv {

template <int S>
struct WideCfg {
    static constexpr int STAGES = S >= 4 ? 2 : 3;   // keeps the static shared memory of 2*S rings under 48 KB
};

// ------------------------------------------------------------------------------------------ fused
template <int BITS, int G, int MODE, int S>
__global__ void __launch_bounds__(64 * S) decode_attn_wide_kernel(KArgs ka, VArgs va, const float *__restrict__ mask,
                                                                  long long mask_stride_b, float scaling)
{
    constexpr int ST = WideCfg<S>::STAGES;
    __shared__ alignas(128) uint8_t kbuf[S][ST * Tile<BITS>::BYTES];
    __shared__ alignas(128) uint8_t vbuf[S][ST * Tile<BITS>::BYTES];
    __shared__ alignas(16) float red[S][G * 8 * 36];
    __shared__ alignas(16) float2 wts[S][G * kTileTok];
    __shared__ FusedShared<G, S> fs;
    __shared__ uint64_t kbar[S][ST], vbar[S][ST];

    const int bh = blockIdx.x, b = bh / ka.Hkv, h = bh % ka.Hkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int role = warp / S, sl = warp % S;
    if (threadIdx.x == 0) {
        for (int k = 0; k < S; ++k)
            for (int i = 0; i < ST; ++i) { mbar_init(&kbar[k][i], 1); mbar_init(&vbar[k][i], 1); }
        fs.init_barriers(S);
        mbar_init_fence();
    }
    __syncthreads();
    const Seg seg{0, ka.T, true, nullptr, nullptr, sl};
    if (role == 0) {
        RingSink<G, S> sink{&fs, 0, sl};
        k_scan<BITS, G, MODE, RingSink<G, S>, ST, true>(ka, seg, b, h, lane, kbuf[sl], kbar[sl], red[sl], sink);
    } else {
        SoftmaxSrc<G, S, MODE == kModeHalf> src;
        src.sh = &fs;
        src.wts = wts[sl];
        src.mask = mask ? mask + size_t(b) * mask_stride_b : nullptr;
        src.scale2 = scaling * 1.4426950408889634f;
        src.n_tiles = (va.T + kTileTok - 1) / kTileTok;
        src.t_begin = 0;
        src.init();
        v_scan<BITS, G, MODE, SoftmaxSrc<G, S, MODE == kModeHalf>, ST, true>(va, seg, b, h, lane, vbuf[sl], vbar[sl], wts[sl],
                                                                       src);
    }
}

// ------------------------------------------------------------------------------------------ q.K^T
// K warps only.  Warp 0 doubles as the consumer of the ring: once all S partials of a tile are in, it adds
// them and writes the fp16 logits.
template <int G, int S>
struct WriterSink : RingSink<G, S> {
    __half *row[G];   // logits row of each q head of this stream: [T+1]
    int T;
    __device__ __forceinline__ void flush(int i, int lane, int n)   // n logits of tile i, or the self logit
    {
        auto *sh = this->sh;
        const int slot = this->slot;
        if (!mbar_wait_bounded(&sh->lfull[slot], (i / kLogitSlots) & 1, kStatLFullWait)) return;
        if (lane < n) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float x = sh->lring[slot][0][g][lane];
#pragma unroll
                for (int k = 1; k < S; ++k) x += sh->lring[slot][k][g][lane];
                row[g][min(i * kTileTok, T) + lane] = __float2half_rn(x);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->lempty[slot]);
    }
    __device__ __forceinline__ void end_tile(int i, int lane)
    {
        RingSink<G, S>::end_tile(i, lane);
        flush(i, lane, min(kTileTok, T - i * kTileTok));
    }
    __device__ __forceinline__ void finish(int lane)
    {
        RingSink<G, S>::end_tile(0, lane);
        flush((T + kTileTok - 1) / kTileTok, lane, 1);   // the self logit goes to position T
    }
};

template <int BITS, int G, int MODE, int S>
__global__ void __launch_bounds__(32 * S) forward_qk_wide_kernel(KArgs ka, __half *__restrict__ logits)
{
    constexpr int ST = WideCfg<S>::STAGES;
    __shared__ alignas(128) uint8_t kbuf[S][ST * Tile<BITS>::BYTES];
    __shared__ alignas(16) float red[S][G * 8 * 36];
    __shared__ FusedShared<G, S> fs;
    __shared__ uint64_t kbar[S][ST];
    const int bh = blockIdx.x, b = bh / ka.Hkv, h = bh % ka.Hkv;
    const int sl = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int k = 0; k < S; ++k)
            for (int i = 0; i < ST; ++i) mbar_init(&kbar[k][i], 1);
        fs.init_barriers(1);
        mbar_init_fence();
    }
    __syncthreads();
    const Seg seg{0, ka.T, true, nullptr, nullptr, sl};
    if (sl == 0) {
        WriterSink<G, S> sink;
        sink.sh = &fs;
        sink.slot = 0;
        sink.sl = 0;
        sink.T = ka.T;
#pragma unroll
        for (int g = 0; g < G; ++g) sink.row[g] = logits + (size_t(b) * ka.Hq + size_t(h) * G + g) * (ka.T + 1);
        k_scan<BITS, G, MODE, WriterSink<G, S>, ST, true>(ka, seg, b, h, lane, kbuf[0], kbar[0], red[0], sink);
    } else {
        RingSink<G, S> sink{&fs, 0, sl};
        k_scan<BITS, G, MODE, RingSink<G, S>, ST, true>(ka, seg, b, h, lane, kbuf[sl], kbar[sl], red[sl], sink);
    }
}

// ------------------------------------------------------------------------------------------ P.V
template <int G, bool HALF_W>
struct WideWeightSrc {
    const __half *row[G];
    float2 *wts;
    __device__ __forceinline__ bool tile_weights(int i, int ntok, int lane, float (&)[G][4])
    {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float wv = lane < ntok ? __half2float(row[g][i * kTileTok + lane]) : 0.f;
            put_weight<HALF_W>(wts, g * kTileTok + lane, wv);
        }
        __syncwarp();
        return true;
    }
    __device__ __forceinline__ bool self_weight(int, float (&)[G][4], float (&w_self)[G], int T)
    {
#pragma unroll
        for (int g = 0; g < G; ++g) w_self[g] = __half2float(row[g][T]);
        return true;
    }
    __device__ __forceinline__ float norm(int) const { return 1.f; }
    __device__ __forceinline__ void store(const VArgs &a, int b, int h, int c0, const float (&acc)[G][4]) const
    {
        store_normalised<G>(*this, a, b, h, c0, acc);
    }
};

template <int BITS, int G, int MODE, int S>
__global__ void __launch_bounds__(32 * S) forward_ov_wide_kernel(VArgs va, const __half *__restrict__ attn)
{
    constexpr int ST = WideCfg<S>::STAGES;
    __shared__ alignas(128) uint8_t vbuf[S][ST * Tile<BITS>::BYTES];
    __shared__ alignas(16) float2 wts[S][G * kTileTok];
    __shared__ uint64_t vbar[S][ST];
    const int bh = blockIdx.x, b = bh / va.Hkv, h = bh % va.Hkv;
    const int sl = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        for (int i = 0; i < ST; ++i) mbar_init(&vbar[sl][i], 1);
        mbar_init_fence();
    }
    __syncthreads();
    WideWeightSrc<G, MODE == kModeHalf> src;
#pragma unroll
    for (int g = 0; g < G; ++g) src.row[g] = attn + (size_t(b) * va.Hq + size_t(h) * G + g) * (va.T + 1);
    src.wts = wts[sl];
    const Seg seg{0, va.T, true, nullptr, nullptr, sl};
    v_scan<BITS, G, MODE, WideWeightSrc<G, MODE == kModeHalf>, ST, true>(va, seg, b, h, lane, vbuf[sl], vbar[sl], wts[sl], src);
}

// Dispatch over (bits, arithmetic, slices, group size); group sizes are limited by the 48 KB of static shared memory.
#define ADKV_WIDE_G(BITS_, MODE_, S_, G_, CALL)                                                               \
    { constexpr int BITS = BITS_; constexpr int MODE = MODE_; constexpr int S = S_; constexpr int G = G_; CALL; }
#define ADKV_WIDE_S(BITS_, MODE_, S_, g_, CALL)                                   \
    if (g_ == 1) ADKV_WIDE_G(BITS_, MODE_, S_, 1, CALL)                           \
    else if (g_ == 2) ADKV_WIDE_G(BITS_, MODE_, S_, 2, CALL)                      \
    else return ADKV_E_SHAPE;
#define ADKV_WIDE_E(BITS_, MODE_, s_, g_, CALL)                                   \
    if (s_ == 2) { ADKV_WIDE_S(BITS_, MODE_, 2, g_, CALL) } else { ADKV_WIDE_S(BITS_, MODE_, 4, g_, CALL) }
#define ADKV_WIDE_M(BITS_, mode_, s_, g_, CALL)                                   \
    if (mode_ == 2) { ADKV_WIDE_E(BITS_, 2, s_, g_, CALL) }                       \
    else if (mode_ == 1) { ADKV_WIDE_E(BITS_, 1, s_, g_, CALL) }                  \
    else { ADKV_WIDE_E(BITS_, 0, s_, g_, CALL) }
#define ADKV_WIDE_DISPATCH(bits_, mode_, s_, g_, CALL)                            \
    if (bits_ == 4) { ADKV_WIDE_M(4, mode_, s_, g_, CALL) } else { ADKV_WIDE_M(2, mode_, s_, g_, CALL) }

}  // namespace adkv

using namespace adkv;

ADKV_DEFINE_TU_STATUS(adkv_tu_status_wide)

// Called by the public entry points for D = 256 / 512 after argument validation.
ADKV_HIDDEN int adkv_wide_decode_attn(const KArgs &ka, const VArgs &va, const float *mask, long long mask_stride_b,
                                      float scaling, int B, int bits, int mode, cudaStream_t s)
{
    const int S = ka.D / kD, g = ka.Hq / ka.Hkv;
    ADKV_WIDE_DISPATCH(bits, mode, S, g,
                       (decode_attn_wide_kernel<BITS, G, MODE, S><<<B * ka.Hkv, 64 * S, 0, s>>>(ka, va, mask,
                                                                                                  mask_stride_b,
                                                                                                  scaling)))
    return launch_status();
}

ADKV_HIDDEN int adkv_wide_forward_qk(const KArgs &ka, __half *logits, int B, int bits, int mode, cudaStream_t s)
{
    const int S = ka.D / kD, g = ka.Hq / ka.Hkv;
    ADKV_WIDE_DISPATCH(bits, mode, S, g,
                       (forward_qk_wide_kernel<BITS, G, MODE, S><<<B * ka.Hkv, 32 * S, 0, s>>>(ka, logits)))
    return launch_status();
}

ADKV_HIDDEN int adkv_wide_forward_ov(const VArgs &va, const __half *attn, int B, int bits, int mode, cudaStream_t s)
{
    const int S = va.D / kD, g = va.Hq / va.Hkv;
    ADKV_WIDE_DISPATCH(bits, mode, S, g,
                       (forward_ov_wide_kernel<BITS, G, MODE, S><<<B * va.Hkv, 32 * S, 0, s>>>(va, attn)))
    return launch_status();
}
