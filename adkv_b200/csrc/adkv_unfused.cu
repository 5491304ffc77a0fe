// Part of libadkv_b200.so (sm_100a).  See include/adkv_b200.h for the contract of every entry point
// and the reference interface each one replaces.
#include "adkv_host.h"

#include "adkv_io.cuh"

namespace adkv {

// =========================================================================================
// Unfused entry points (the reference's two-kernel decode): 2 streams per CTA, one warp each.

template <int BITS, int G, bool EXACT>
__global__ void __launch_bounds__(32 * kStreamsPerCta) forward_qk_kernel(KArgs ka, __half *__restrict__ logits,
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
    k_warp<BITS, G, EXACT>(ka, seg, b, h, lane, kbuf[warp], kbar[warp], red[warp], sink);
}

template <int BITS, int G, bool EXACT>
__global__ void __launch_bounds__(32 * kStreamsPerCta) forward_ov_kernel(VArgs va, const __half *__restrict__ attn,
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
    GlobalWeightSrc<G> src;
#pragma unroll
    for (int g = 0; g < G; ++g) src.row[g] = attn + (size_t(b) * va.Hq + size_t(h) * G + g) * (va.T + 1);
    src.wts = wts[warp];
    const Seg seg{0, va.T, true, nullptr, nullptr, 0};
    v_warp<BITS, G, EXACT>(va, seg, b, h, lane, vbuf[warp], vbar[warp], wts[warp], src);
}

}  // namespace adkv

using namespace adkv;

ADKV_HIDDEN int adkv_half_forward_qk(const KArgs &ka, __half *logits, int B, int bits, cudaStream_t s);
ADKV_HIDDEN int adkv_half_forward_ov(const VArgs &va, const __half *attn, int B, int bits, cudaStream_t s);
ADKV_HIDDEN int adkv_wide_forward_qk(const KArgs &ka, __half *logits, int B, int bits, int mode, cudaStream_t s);
ADKV_HIDDEN int adkv_wide_forward_ov(const VArgs &va, const __half *attn, int B, int bits, int mode, cudaStream_t s);

ADKV_DEFINE_TU_STATUS(adkv_tu_status_unfused)

extern "C" {

int adkv_forward_qk(const void *q, void *k_cache, const void *k_new, const adkv_params *p, void *logits, int B,
                    int Hq, int Hkv, int T, int D, int n_super_cap, int bits, float scale_min, float scale_max,
                    unsigned flags, void *stream)
{
    if (!q || !k_cache || !k_new || !logits || !params_ok(p)) return ADKV_E_NULL;
    if (int rc = check_common(B, Hq, Hkv, T, D, n_super_cap, bits, T + 1)) return rc;
    if (!aligned16(k_cache) || !aligned8(q) || !aligned8(k_new) || !params_aligned(p)) return ADKV_E_ALIGN;
    if (B == 0) return 0;
    const KArgs ka{static_cast<const __half *>(q), static_cast<uint8_t *>(k_cache),
                   static_cast<const __half *>(k_new), to_ptrs(p), Hq, Hkv, T, n_super_cap, scale_min, scale_max, D};
    const int n_streams = B * Hkv, grid = (n_streams + kStreamsPerCta - 1) / kStreamsPerCta;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool half = flags & ADKV_FLAG_HALF_STATE, exact = !(flags & ADKV_FLAG_FAST_REPLAY);
    if (D != kD) return adkv_wide_forward_qk(ka, static_cast<__half *>(logits), B, bits, half ? 2 : int(exact), s);
    if (half) return adkv_half_forward_qk(ka, static_cast<__half *>(logits), B, bits, s);
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
                   to_ptrs(p), Hq, Hkv, T, n_super_cap, scale_min, scale_max, D};
    const int n_streams = B * Hkv, grid = (n_streams + kStreamsPerCta - 1) / kStreamsPerCta;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool half = flags & ADKV_FLAG_HALF_STATE, exact = !(flags & ADKV_FLAG_FAST_REPLAY);
    if (D != kD) return adkv_wide_forward_ov(va, static_cast<const __half *>(attn), B, bits, half ? 2 : int(exact), s);
    if (half) return adkv_half_forward_ov(va, static_cast<const __half *>(attn), B, bits, s);
    ADKV_DISPATCH(bits, exact, Hq / Hkv,
                  (forward_ov_kernel<BITS, G, EXACT><<<grid, 32 * kStreamsPerCta, 0, s>>>(
                      va, static_cast<const __half *>(attn), n_streams)))
    return launch_status();
}

}  // extern "C"
