// Part of libadkv_b200.so (sm_100a).  See include/adkv_b200.h for the contract of every entry point.
//
// Fused decode step for launches with few (batch, kv head) streams: the 128-wide head is split over two K warps
// and two V warps per stream (adkv_narrow.cuh).  Reached through adkv_decode_attn.
#include "adkv_host.h"

#include "adkv_narrow.cuh"

namespace adkv {

template <int BITS, int G, int ARITH>
__global__ void __launch_bounds__(64 * kNarrowSlices) decode_attn_narrow_kernel(KArgs ka, VArgs va,
                                                                                const float *__restrict__ mask,
                                                                                long long mask_stride_b, float scaling)
{
    constexpr int S = kNarrowSlices;
    __shared__ alignas(128) uint8_t kbuf[S][kStages * NarrowTile<BITS>::BYTES];
    __shared__ alignas(128) uint8_t vbuf[S][kStages * NarrowTile<BITS>::BYTES];
    __shared__ alignas(16) float red[S][G * 8 * 36];
    __shared__ alignas(16) float2 wts[S][G * kTileTok];
    __shared__ FusedShared<G, S> fs;
    __shared__ uint64_t kbar[S][kStages], vbar[S][kStages];

    const int bh = blockIdx.x, b = bh / ka.Hkv, h = bh % ka.Hkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int role = warp / S, sl = warp % S;
    if (threadIdx.x == 0) {
        for (int k = 0; k < S; ++k)
            for (int i = 0; i < kStages; ++i) { mbar_init(&kbar[k][i], 1); mbar_init(&vbar[k][i], 1); }
        fs.init_barriers(S);
        mbar_init_fence();
    }
    __syncthreads();
    const Seg seg{0, ka.T, true, nullptr, nullptr, sl};
    if (role == 0) {
        RingSink<G, S> sink{&fs, 0, sl};
        k_warp_n<BITS, G, ARITH>(ka, seg, b, h, lane, kbuf[sl], kbar[sl], red[sl], sink);
    } else {
        SoftmaxSrc<G, S> src;
        src.sh = &fs;
        src.wts = wts[sl];
        src.mask = mask ? mask + size_t(b) * mask_stride_b : nullptr;
        src.scale2 = scaling * 1.4426950408889634f;
        src.n_tiles = (va.T + kTileTok - 1) / kTileTok;
        src.t_begin = 0;
        src.init();
        v_warp_n<BITS, G, ARITH>(va, seg, b, h, lane, vbuf[sl], vbar[sl], wts[sl], src);
    }
}

}  // namespace adkv

using namespace adkv;

ADKV_DEFINE_TU_STATUS(adkv_tu_status_narrow)

// Arguments checked by adkv_decode_attn (head dim 128, fp32 arithmetic).
ADKV_HIDDEN int adkv_narrow_decode_attn(const KArgs &ka, const VArgs &va, const float *mask, long long mask_stride_b,
                                        float scaling, int B, int bits, bool exact, cudaStream_t s)
{
    ADKV_DISPATCH(bits, exact, ka.Hq / ka.Hkv,
                  (decode_attn_narrow_kernel<BITS, G, ARITH><<<B * ka.Hkv, 64 * kNarrowSlices, 0, s>>>(
                      ka, va, mask, mask_stride_b, scaling)))
    return launch_status();
}
