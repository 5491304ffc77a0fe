// Part of libadkv_b200.so (sm_100a).  See include/adkv_b200.h for the contract of every entry point
// and the reference interface each one replaces.
#include "adkv_host.h"

#include "adkv_softmax.cuh"

namespace adkv {

// =========================================================================================
// Fused decode step: one CTA per (batch, kv head); warp 0 scans K, warp 1 scans V.

// Whether the guarded chunk bodies of this instantiation are function calls (see k_chunk_guarded).  Measured on a
// B200 against the inline form, streams of 32 heads x 128: 4-bit codes with one query head per KV head gain 13 % at
// 128-token contexts and lose nothing elsewhere; 2-bit codes gain 17 % there but lose 7 % in the canonical replay and
// 14 % with 512 streams per launch, so they keep the inline form, as do the instantiations with several query heads.
template <int BITS, int G>
constexpr bool kOutOfLineGuarded = BITS == 4 && G == 1;

template <int BITS, int G, int ARITH>
__global__ void __launch_bounds__(64) decode_attn_kernel(KArgs ka, VArgs va, const float *__restrict__ mask,
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
        // per-sequence token counts held on the device (ragged batches; also lets a captured launch be
        // replayed while the sequences grow).  The host could not check the capacity, so it is checked here.
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
        k_warp<BITS, G, ARITH, RingSink<G>, kStages, false, kOutOfLineGuarded<BITS, G>>(ka, seg, b, h, lane, kbuf, kbar, red, sink);
    } else {
        SoftmaxSrc<G> src;
        src.sh = &fs;
        src.wts = wts;
        src.mask = mask ? mask + size_t(b) * mask_stride_b : nullptr;
        src.scale2 = scaling * 1.4426950408889634f;
        src.n_tiles = (va.T + kTileTok - 1) / kTileTok;
        src.t_begin = 0;
        src.init();
        v_warp<BITS, G, ARITH, SoftmaxSrc<G>, kStages, false, kOutOfLineGuarded<BITS, G>>(va, seg, b, h, lane, vbuf, vbar, wts, src);
    }
}

}  // namespace adkv

using namespace adkv;

// adkv_decode_attn splits the channels of a head over two warp pairs up to this many (batch, kv head) streams per
// launch: measured on a B200 (4096 tokens, 4-bit) the split is no slower only while there is at most about one
// stream per SM (128 streams: 200 us either way); from 256 streams on the whole-head kernel is faster (512 streams:
// 274 us against 324 us), because the split costs a quarter more instructions and both are then bound by issue.
constexpr long long kSplitChannelsMaxStreams = 160;

ADKV_HIDDEN int adkv_half_decode_attn(const KArgs &ka, const VArgs &va, const float *mask, long long mask_stride_b,
                                      float scaling, int B, int bits, const int *seq_lens, cudaStream_t s);
ADKV_HIDDEN int adkv_narrow_decode_attn(const KArgs &ka, const VArgs &va, const float *mask, long long mask_stride_b,
                                        float scaling, int B, int bits, bool exact, cudaStream_t s);
ADKV_HIDDEN int adkv_wide_decode_attn(const KArgs &ka, const VArgs &va, const float *mask, long long mask_stride_b,
                                      float scaling, int B, int bits, int mode, cudaStream_t s);

ADKV_DEFINE_TU_STATUS(adkv_tu_status_fused)

extern "C" {

int adkv_decode_attn(const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new,
                     const adkv_params *kp, const adkv_params *vp, void *k_tail, void *v_tail, const void *mask,
                     long long mask_stride_b,
                     void *out, int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits, float scaling,
                     float scale_min, float scale_max, unsigned flags, void *stream)
{
    if (!q || !k_cache || !v_cache || !k_new || !v_new || !out || !params_ok(kp) || !params_ok(vp))
        return ADKV_E_NULL;
    if (int rc = check_common(B, Hq, Hkv, T, D, n_super_cap, bits, T + 1)) return rc;
    if (int rc = check_tails(k_tail, v_tail, flags)) return rc;
    if (!aligned16(k_cache) || !aligned16(v_cache) || !aligned8(q) || !aligned8(out) || !aligned8(k_new) ||
        !aligned8(v_new) || !params_aligned(kp) || !params_aligned(vp))
        return ADKV_E_ALIGN;
    if (B == 0) return 0;
    const bool keep = flags & ADKV_FLAG_TAIL_KEEP;
    const KArgs ka{static_cast<const __half *>(q), static_cast<uint8_t *>(k_cache),
                   static_cast<const __half *>(k_new), to_ptrs(kp), Hq, Hkv, T, n_super_cap, scale_min, scale_max, D,
                   static_cast<float *>(k_tail), keep};
    const VArgs va{static_cast<uint8_t *>(v_cache), static_cast<const __half *>(v_new), static_cast<__half *>(out),
                   to_ptrs(vp), Hq, Hkv, T, n_super_cap, scale_min, scale_max, D, static_cast<float *>(v_tail), keep};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool half = flags & ADKV_FLAG_HALF_STATE, exact = !(flags & ADKV_FLAG_FAST_REPLAY);
    if (D != kD)
        return adkv_wide_decode_attn(ka, va, static_cast<const float *>(mask), mask_stride_b, scaling, B, bits,
                                     half ? 2 : int(exact), s);
    if (half)
        return adkv_half_decode_attn(ka, va, static_cast<const float *>(mask), mask_stride_b, scaling, B, bits, nullptr, s);
    // Very few streams: split every head over two warp pairs (adkv_narrow.cu).
    const bool split = (flags & ADKV_FLAG_SPLIT_CHANNELS) ||
                       (!(flags & ADKV_FLAG_NO_SPLIT_CHANNELS) && (long long)B * Hkv <= kSplitChannelsMaxStreams);
    if (split)
        return adkv_narrow_decode_attn(ka, va, static_cast<const float *>(mask), mask_stride_b, scaling, B, bits, exact, s);
    ADKV_DISPATCH(bits, exact, Hq / Hkv,
                  (decode_attn_kernel<BITS, G, ARITH><<<B * Hkv, 64, 0, s>>>(
                      ka, va, static_cast<const float *>(mask), mask_stride_b, scaling, nullptr)))
    return launch_status();
}

int adkv_decode_attn_varlen(const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new,
                            const adkv_params *kp, const adkv_params *vp, void *k_tail, void *v_tail,
                            const void *seq_lens, void *out, int B, int Hq, int Hkv, int D, int n_super_cap, int bits,
                            float scaling, float scale_min, float scale_max, unsigned flags, void *stream)
{
    if (!q || !k_cache || !v_cache || !k_new || !v_new || !out || !seq_lens || !params_ok(kp) || !params_ok(vp))
        return ADKV_E_NULL;
    if (D != kD) return ADKV_E_HEAD_DIM;   // device-side lengths: 128-wide heads only
    if (int rc = check_common(B, Hq, Hkv, 0, D, n_super_cap, bits, 1)) return rc;
    if (int rc = check_tails(k_tail, v_tail, flags)) return rc;
    if (!aligned16(k_cache) || !aligned16(v_cache) || !aligned8(q) || !aligned8(out) || !aligned8(k_new) ||
        !aligned8(v_new) || !params_aligned(kp) || !params_aligned(vp) || (reinterpret_cast<uintptr_t>(seq_lens) & 3u))
        return ADKV_E_ALIGN;
    if (B == 0) return 0;
    const bool keep = flags & ADKV_FLAG_TAIL_KEEP;
    const KArgs ka{static_cast<const __half *>(q), static_cast<uint8_t *>(k_cache),
                   static_cast<const __half *>(k_new), to_ptrs(kp), Hq, Hkv, 0, n_super_cap, scale_min, scale_max, D,
                   static_cast<float *>(k_tail), keep};
    const VArgs va{static_cast<uint8_t *>(v_cache), static_cast<const __half *>(v_new), static_cast<__half *>(out),
                   to_ptrs(vp), Hq, Hkv, 0, n_super_cap, scale_min, scale_max, D, static_cast<float *>(v_tail), keep};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (flags & ADKV_FLAG_HALF_STATE)
        return adkv_half_decode_attn(ka, va, nullptr, 0, scaling, B, bits, static_cast<const int *>(seq_lens), s);
    const bool exact = !(flags & ADKV_FLAG_FAST_REPLAY);
    ADKV_DISPATCH(bits, exact, Hq / Hkv,
                  (decode_attn_kernel<BITS, G, ARITH><<<B * Hkv, 64, 0, s>>>(ka, va, nullptr, 0, scaling,
                                                                            static_cast<const int *>(seq_lens))))
    return launch_status();
}

}  // extern "C"
