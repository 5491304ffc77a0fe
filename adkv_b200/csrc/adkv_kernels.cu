// Kernels and C ABI of the ADKV hot path for B200 (sm_100a).  See include/adkv_b200.h for the
// contract of every entry point and the reference interface each one replaces.
#include "../../include/adkv_b200.h"

#include "adkv_decode.cuh"

namespace adkv {

// =========================================================================================
// Prefill quantise + pack (canonical arithmetic).  One CTA per (batch, head), one thread per
// channel: the warp reads 64 contiguous bytes of a token row and writes 128 contiguous bytes
// of a supergroup.  The next word's tokens are fetched while the current word is quantised.
template <int BITS>
__global__ void __launch_bounds__(kD) encode_kernel(uint32_t *__restrict__ cache, const __half *__restrict__ x,
                                                    ParamPtrs p, float *__restrict__ tail, int H, int T,
                                                    int n_super_cap, int t_start, float smin, float smax)
{
    using C = Codec<BITS>;
    const int bh = blockIdx.x, h = bh % H, c = threadIdx.x;
    const size_t po = size_t(h) * kD + c;
    Chan ch;
    ch.alpha = __half2float(p.alpha[po]);
    ch.beta = __half2float(p.beta[po]);
    ch.tc = __half2float(p.target[po]);
    if (t_start > 0) {
        ch.zp = tail[size_t(bh) * 2 * kD + c];
        ch.s = tail[size_t(bh) * 2 * kD + kD + c];
    } else {
        ch.zp = __half2float(p.zp_init[po]);
        ch.s = __half2float(p.scale_init[po]);
    }
    uint32_t *w = cache + size_t(bh) * n_super_cap * kD + c;
    const __half *xs = x + size_t(bh) * T * kD + c;   // token t_start + i is row i

    const int t_end = t_start + T;
    int t = t_start;
    // leading partial word (chunked prefill that starts inside a word)
    if (t % C::TPW != 0 && t < t_end) {
        const int sg = t / C::TPW;
        uint32_t word = w[size_t(sg) * kD] & ((1u << (BITS * (t % C::TPW))) - 1u);
        for (; t < t_end && t / C::TPW == sg; ++t) {
            float rh;
            const float q = quantize<BITS>(__half2float(xs[size_t(t - t_start) * kD]), ch, rh);
            word |= uint32_t(int(q) + C::BIAS) << (BITS * (t % C::TPW));
            advance_canonical(q, rh, ch, smin, smax);
        }
        w[size_t(sg) * kD] = word;
    }
    // full words, software-pipelined loads
    __half cur[C::TPW], nxt[C::TPW];
    const int n_full = (t_end - t) / C::TPW;
    if (n_full > 0) {
#pragma unroll
        for (int j = 0; j < C::TPW; ++j) cur[j] = xs[size_t(t - t_start + j) * kD];
    }
    for (int i = 0; i < n_full; ++i, t += C::TPW) {
        if (i + 1 < n_full) {
#pragma unroll
            for (int j = 0; j < C::TPW; ++j) nxt[j] = xs[size_t(t - t_start + C::TPW + j) * kD];
        }
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < C::TPW; ++j) {
            float rh;
            const float q = quantize<BITS>(__half2float(cur[j]), ch, rh);
            word |= uint32_t(int(q) + C::BIAS) << (BITS * j);
            advance_canonical(q, rh, ch, smin, smax);
        }
        w[size_t(t / C::TPW) * kD] = word;
#pragma unroll
        for (int j = 0; j < C::TPW; ++j) cur[j] = nxt[j];
    }
    // trailing partial word: unused fields stay zero
    if (t < t_end) {
        const int sg = t / C::TPW;
        uint32_t word = 0;
        for (; t < t_end; ++t) {
            float rh;
            const float q = quantize<BITS>(__half2float(xs[size_t(t - t_start) * kD]), ch, rh);
            word |= uint32_t(int(q) + C::BIAS) << (BITS * (t % C::TPW));
            advance_canonical(q, rh, ch, smin, smax);
        }
        w[size_t(sg) * kD] = word;
    }
    if (tail) {
        tail[size_t(bh) * 2 * kD + c] = ch.zp;
        tail[size_t(bh) * 2 * kD + kD + c] = ch.s;
    }
}

// Single-token append from the persisted tail state.
template <int BITS>
__global__ void __launch_bounds__(kD) append_kernel(uint32_t *__restrict__ cache, const __half *__restrict__ x_new,
                                                    ParamPtrs p, float *__restrict__ tail, int H, int T,
                                                    int n_super_cap, float smin, float smax)
{
    using C = Codec<BITS>;
    const int bh = blockIdx.x, h = bh % H, c = threadIdx.x;
    const size_t po = size_t(h) * kD + c;
    Chan ch;
    ch.alpha = __half2float(p.alpha[po]);
    ch.beta = __half2float(p.beta[po]);
    ch.tc = __half2float(p.target[po]);
    ch.zp = tail[size_t(bh) * 2 * kD + c];
    ch.s = tail[size_t(bh) * 2 * kD + kD + c];
    float rh;
    const float q = quantize<BITS>(__half2float(x_new[size_t(bh) * kD + c]), ch, rh);
    uint32_t *slot = cache + (size_t(bh) * n_super_cap + T / C::TPW) * kD + c;
    const int sh = BITS * (T % C::TPW);
    *slot = (*slot & ~(C::FIELD << sh)) | (uint32_t(int(q) + C::BIAS) << sh);
    advance_canonical(q, rh, ch, smin, smax);
    tail[size_t(bh) * 2 * kD + c] = ch.zp;
    tail[size_t(bh) * 2 * kD + kD + c] = ch.s;
}

// =========================================================================================
// Fused decode step: one CTA per (batch, kv head); warp 0 scans K, warp 1 scans V.

template <int G>
struct FusedShared {
    float lring[kLogitSlots][G][kTileTok];
    uint64_t lfull[kLogitSlots], lempty[kLogitSlots];
};

template <int G>
struct RingSink {
    FusedShared<G> *sh;
    int slot;
    __device__ __forceinline__ bool begin_tile(int i)
    {
        slot = i % kLogitSlots;
        return mbar_wait_bounded(&sh->lempty[slot], ((i / kLogitSlots) & 1) ^ 1, kStatLEmptyWait);
    }
    __device__ __forceinline__ void put8(int, int g, int tok, float v, int lane)
    {
        if (lane < 8) sh->lring[slot][g][tok + lane] = v;
    }
    __device__ __forceinline__ void end_tile(int, int lane)
    {
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->lfull[slot]);
    }
    __device__ __forceinline__ void put_self(int g, float v) { sh->lring[slot][g][0] = v; }
    __device__ __forceinline__ void finish(int lane) { end_tile(0, lane); }
};

template <int G>
struct SoftmaxSrc {
    FusedShared<G> *sh;
    float *wts;            // [G][32]
    const float *mask;     // row of this batch or nullptr
    float scale2;          // scaling * log2(e)
    int n_tiles;
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
        const float mk = (mask && lane < ntok) ? mask[i * kTileTok + lane] * 1.4426950408889634f : 0.f;
        if (!mbar_wait_bounded(&sh->lfull[slot], (i / kLogitSlots) & 1, kStatLFullWait)) return false;
        float x[G];
#pragma unroll
        for (int g = 0; g < G; ++g) x[g] = sh->lring[slot][g][lane];
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->lempty[slot]);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float v = lane < ntok ? fmaf(x[g], scale2, mk) : -INFINITY;
            wts[g * kTileTok + lane] = update(g, v, acc);
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
            const float v = fmaf(sh->lring[slot][g][0], scale2, mk);
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
};

template <int BITS, int G, bool EXACT>
__global__ void __launch_bounds__(64) decode_attn_kernel(KArgs ka, VArgs va, const float *__restrict__ mask,
                                                         long long mask_stride_b, float scaling)
{
    __shared__ alignas(128) uint8_t kbuf[kStages * Tile<BITS>::BYTES];
    __shared__ alignas(128) uint8_t vbuf[kStages * Tile<BITS>::BYTES];
    __shared__ alignas(16) float red[8 * 36];
    __shared__ alignas(16) float wts[G * kTileTok];
    __shared__ FusedShared<G> fs;
    __shared__ uint64_t kbar[kStages], vbar[kStages];

    const int bh = blockIdx.x, b = bh / ka.Hkv, h = bh % ka.Hkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(&kbar[i], 1); mbar_init(&vbar[i], 1); }
        for (int i = 0; i < kLogitSlots; ++i) { mbar_init(&fs.lfull[i], 1); mbar_init(&fs.lempty[i], 1); }
        mbar_init_fence();
    }
    __syncthreads();
    if (warp == 0) {
        RingSink<G> sink{&fs, 0};
        k_warp<BITS, G, EXACT>(ka, b, h, lane, kbuf, kbar, red, sink);
    } else {
        SoftmaxSrc<G> src;
        src.sh = &fs;
        src.wts = wts;
        src.mask = mask ? mask + size_t(b) * mask_stride_b : nullptr;
        src.scale2 = scaling * 1.4426950408889634f;
        src.n_tiles = (va.T + kTileTok - 1) / kTileTok;
        src.init();
        v_warp<BITS, G, EXACT>(va, b, h, lane, vbuf, vbar, wts, src);
    }
}

// =========================================================================================
// Unfused entry points (the reference's two-kernel decode): 4 streams per CTA, one warp each.

constexpr int kStreamsPerCta = 4;

template <int G>
struct GlobalLogitSink {
    __half *row[G];   // logits row of each q head of this stream: [T+1]
    int T;
    __device__ __forceinline__ bool begin_tile(int) { return true; }
    __device__ __forceinline__ void put8(int i, int g, int tok, float v, int lane)
    {
        const int t = i * kTileTok + tok + lane;
        if (lane < 8 && t < T) row[g][t] = __float2half_rn(v);
    }
    __device__ __forceinline__ void end_tile(int, int) {}
    __device__ __forceinline__ void put_self(int g, float v) { row[g][T] = __float2half_rn(v); }
    __device__ __forceinline__ void finish(int) {}
};

template <int BITS, int G, bool EXACT>
__global__ void __launch_bounds__(32 * kStreamsPerCta) forward_qk_kernel(KArgs ka, __half *__restrict__ logits,
                                                                         int n_streams)
{
    __shared__ alignas(128) uint8_t kbuf[kStreamsPerCta][kStages * Tile<BITS>::BYTES];
    __shared__ alignas(16) float red[kStreamsPerCta][8 * 36];
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
    k_warp<BITS, G, EXACT>(ka, b, h, lane, kbuf[warp], kbar[warp], red[warp], sink);
}

template <int G>
struct GlobalWeightSrc {
    const __half *row[G];   // attention weights of each q head of this stream: [T+1]
    float *wts;
    __device__ __forceinline__ bool tile_weights(int i, int ntok, int lane, float (&)[G][4])
    {
#pragma unroll
        for (int g = 0; g < G; ++g)
            wts[g * kTileTok + lane] = lane < ntok ? __half2float(row[g][i * kTileTok + lane]) : 0.f;
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
};

template <int BITS, int G, bool EXACT>
__global__ void __launch_bounds__(32 * kStreamsPerCta) forward_ov_kernel(VArgs va, const __half *__restrict__ attn,
                                                                         int n_streams)
{
    __shared__ alignas(128) uint8_t vbuf[kStreamsPerCta][kStages * Tile<BITS>::BYTES];
    __shared__ alignas(16) float wts[kStreamsPerCta][G * kTileTok];
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
    GlobalWeightSrc<G> src;
#pragma unroll
    for (int g = 0; g < G; ++g) src.row[g] = attn + (size_t(b) * va.Hq + size_t(h) * G + g) * (va.T + 1);
    src.wts = wts[warp];
    v_warp<BITS, G, EXACT>(va, b, h, lane, vbuf[warp], vbar[warp], wts[warp], src);
}

// =========================================================================================
// Host side.

static ParamPtrs to_ptrs(const adkv_params *p)
{
    return ParamPtrs{static_cast<const __half *>(p->zp_init), static_cast<const __half *>(p->scale_init),
                     static_cast<const __half *>(p->alpha), static_cast<const __half *>(p->beta),
                     static_cast<const __half *>(p->target)};
}

static bool params_ok(const adkv_params *p)
{
    return p && p->zp_init && p->scale_init && p->alpha && p->beta && p->target;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static bool aligned8(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }

static bool params_aligned(const adkv_params *p)
{
    return aligned8(p->zp_init) && aligned8(p->scale_init) && aligned8(p->alpha) && aligned8(p->beta) &&
           aligned8(p->target);
}

static int launch_status()
{
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : int(e);
}

static int check_common(int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits, int n_written_end)
{
    if (D != kD) return ADKV_E_HEAD_DIM;
    if (bits != 2 && bits != 4) return ADKV_E_BITS;
    if (B < 0 || Hq <= 0 || Hkv <= 0 || T < 0 || n_super_cap < 0 || Hq % Hkv != 0) return ADKV_E_SHAPE;
    const int tpw = 32 / bits;
    if ((long long)(n_written_end + tpw - 1) / tpw > (long long)n_super_cap) return ADKV_E_CAPACITY;
    return 0;
}

// Dispatch over (bits, group size, arithmetic).
#define ADKV_DISPATCH_G(BITS_, EXACT_, G_, CALL) \
    switch (G_) {                                \
    case 1: { constexpr int BITS = BITS_; constexpr bool EXACT = EXACT_; constexpr int G = 1; CALL; } break; \
    case 2: { constexpr int BITS = BITS_; constexpr bool EXACT = EXACT_; constexpr int G = 2; CALL; } break; \
    case 4: { constexpr int BITS = BITS_; constexpr bool EXACT = EXACT_; constexpr int G = 4; CALL; } break; \
    case 8: { constexpr int BITS = BITS_; constexpr bool EXACT = EXACT_; constexpr int G = 8; CALL; } break; \
    default: return ADKV_E_SHAPE;                \
    }
#define ADKV_DISPATCH(bits_, exact_, G_, CALL)                            \
    if (bits_ == 4) {                                                     \
        if (exact_) { ADKV_DISPATCH_G(4, true, G_, CALL) } else { ADKV_DISPATCH_G(4, false, G_, CALL) } \
    } else {                                                              \
        if (exact_) { ADKV_DISPATCH_G(2, true, G_, CALL) } else { ADKV_DISPATCH_G(2, false, G_, CALL) } \
    }

}  // namespace adkv

using namespace adkv;

extern "C" {

int adkv_abi_version(void) { return ADKV_ABI_VERSION; }

const char *adkv_strerror(int code)
{
    switch (code) {
    case 0: return "success";
    case ADKV_E_NULL: return "adkv: a required pointer is NULL";
    case ADKV_E_HEAD_DIM: return "adkv: head dim not supported by this build (D must be 128)";
    case ADKV_E_BITS: return "adkv: bits must be 2 or 4";
    case ADKV_E_SHAPE: return "adkv: invalid sizes (negative, Hq not a multiple of Hkv, or group size not in {1,2,4,8})";
    case ADKV_E_CAPACITY: return "adkv: cache capacity too small for the tokens to be written";
    case ADKV_E_ALIGN: return "adkv: pointer not sufficiently aligned (cache 16 bytes, fp16 rows 8 bytes)";
    case ADKV_E_START: return "adkv: t_start > 0 needs a tail state";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "adkv: unknown error";
    }
}

int adkv_encode(void *cache, const void *x, const adkv_params *p, void *tail, int B, int H, int T, int D,
                int n_super_cap, int bits, int t_start, float scale_min, float scale_max, void *stream)
{
    if (!cache || (!x && T > 0) || !params_ok(p)) return ADKV_E_NULL;
    if (t_start < 0) return ADKV_E_SHAPE;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, t_start + T)) return rc;
    if (t_start > 0 && !tail) return ADKV_E_START;
    if (B * H == 0 || (T == 0 && !(tail && t_start == 0))) return 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (bits == 4)
        encode_kernel<4><<<B * H, kD, 0, s>>>(static_cast<uint32_t *>(cache), static_cast<const __half *>(x),
                                              to_ptrs(p), static_cast<float *>(tail), H, T, n_super_cap, t_start,
                                              scale_min, scale_max);
    else
        encode_kernel<2><<<B * H, kD, 0, s>>>(static_cast<uint32_t *>(cache), static_cast<const __half *>(x),
                                              to_ptrs(p), static_cast<float *>(tail), H, T, n_super_cap, t_start,
                                              scale_min, scale_max);
    return launch_status();
}

int adkv_append(void *cache, const void *x_new, const adkv_params *p, void *tail, int B, int H, int T, int D,
                int n_super_cap, int bits, float scale_min, float scale_max, void *stream)
{
    if (!cache || !x_new || !tail || !params_ok(p)) return ADKV_E_NULL;
    if (int rc = check_common(B, H, H, T, D, n_super_cap, bits, T + 1)) return rc;
    if (B * H == 0) return 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (bits == 4)
        append_kernel<4><<<B * H, kD, 0, s>>>(static_cast<uint32_t *>(cache), static_cast<const __half *>(x_new),
                                              to_ptrs(p), static_cast<float *>(tail), H, T, n_super_cap, scale_min,
                                              scale_max);
    else
        append_kernel<2><<<B * H, kD, 0, s>>>(static_cast<uint32_t *>(cache), static_cast<const __half *>(x_new),
                                              to_ptrs(p), static_cast<float *>(tail), H, T, n_super_cap, scale_min,
                                              scale_max);
    return launch_status();
}

int adkv_forward_qk(const void *q, void *k_cache, const void *k_new, const adkv_params *p, void *logits, int B,
                    int Hq, int Hkv, int T, int D, int n_super_cap, int bits, float scale_min, float scale_max,
                    unsigned flags, void *stream)
{
    if (!q || !k_cache || !k_new || !logits || !params_ok(p)) return ADKV_E_NULL;
    if (int rc = check_common(B, Hq, Hkv, T, D, n_super_cap, bits, T + 1)) return rc;
    if (!aligned16(k_cache) || !aligned8(q) || !aligned8(k_new) || !params_aligned(p)) return ADKV_E_ALIGN;
    if (B == 0) return 0;
    const KArgs ka{static_cast<const __half *>(q), static_cast<uint8_t *>(k_cache),
                   static_cast<const __half *>(k_new), to_ptrs(p), Hq, Hkv, T, n_super_cap, scale_min, scale_max};
    const int n_streams = B * Hkv, grid = (n_streams + kStreamsPerCta - 1) / kStreamsPerCta;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool exact = !(flags & ADKV_FLAG_FAST_REPLAY);
    ADKV_DISPATCH(bits, exact, Hq / Hkv,
                  (forward_qk_kernel<BITS, G, EXACT><<<grid, 32 * kStreamsPerCta, 0, s>>>(
                      ka, static_cast<__half *>(logits), n_streams)))
    return launch_status();
}

int adkv_forward_ov(const void *attn, void *v_cache, const void *v_new, const adkv_params *p, void *out, int B,
                    int Hq, int Hkv, int T, int D, int n_super_cap, int bits, float scale_min, float scale_max,
                    unsigned flags, void *stream)
{
    if (!attn || !v_cache || !v_new || !out || !params_ok(p)) return ADKV_E_NULL;
    if (int rc = check_common(B, Hq, Hkv, T, D, n_super_cap, bits, T + 1)) return rc;
    if (!aligned16(v_cache) || !aligned8(out) || !aligned8(v_new) || !params_aligned(p)) return ADKV_E_ALIGN;
    if (B == 0) return 0;
    const VArgs va{static_cast<uint8_t *>(v_cache), static_cast<const __half *>(v_new), static_cast<__half *>(out),
                   to_ptrs(p), Hq, Hkv, T, n_super_cap, scale_min, scale_max};
    const int n_streams = B * Hkv, grid = (n_streams + kStreamsPerCta - 1) / kStreamsPerCta;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool exact = !(flags & ADKV_FLAG_FAST_REPLAY);
    ADKV_DISPATCH(bits, exact, Hq / Hkv,
                  (forward_ov_kernel<BITS, G, EXACT><<<grid, 32 * kStreamsPerCta, 0, s>>>(
                      va, static_cast<const __half *>(attn), n_streams)))
    return launch_status();
}

int adkv_decode_attn(const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new,
                     const adkv_params *kp, const adkv_params *vp, const void *mask, long long mask_stride_b,
                     void *out, int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits, float scaling,
                     float scale_min, float scale_max, unsigned flags, void *stream)
{
    if (!q || !k_cache || !v_cache || !k_new || !v_new || !out || !params_ok(kp) || !params_ok(vp))
        return ADKV_E_NULL;
    if (int rc = check_common(B, Hq, Hkv, T, D, n_super_cap, bits, T + 1)) return rc;
    if (!aligned16(k_cache) || !aligned16(v_cache) || !aligned8(q) || !aligned8(out) || !aligned8(k_new) ||
        !aligned8(v_new) || !params_aligned(kp) || !params_aligned(vp))
        return ADKV_E_ALIGN;
    if (B == 0) return 0;
    const KArgs ka{static_cast<const __half *>(q), static_cast<uint8_t *>(k_cache),
                   static_cast<const __half *>(k_new), to_ptrs(kp), Hq, Hkv, T, n_super_cap, scale_min, scale_max};
    const VArgs va{static_cast<uint8_t *>(v_cache), static_cast<const __half *>(v_new), static_cast<__half *>(out),
                   to_ptrs(vp), Hq, Hkv, T, n_super_cap, scale_min, scale_max};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool exact = !(flags & ADKV_FLAG_FAST_REPLAY);
    ADKV_DISPATCH(bits, exact, Hq / Hkv,
                  (decode_attn_kernel<BITS, G, EXACT><<<B * Hkv, 64, 0, s>>>(
                      ka, va, static_cast<const float *>(mask), mask_stride_b, scaling)))
    return launch_status();
}

int adkv_device_status(int *status, void *stream)
{
    if (!status) return ADKV_E_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return int(e);
    e = cudaMemcpyFromSymbol(status, g_status, sizeof(int));
    if (e != cudaSuccess) return int(e);
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return e == cudaSuccess ? 0 : int(e);
}

}  // extern "C"
