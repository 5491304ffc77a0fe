// Part of libadkv_b200.so (sm_100a).  See include/adkv_b200.h for the contract of every entry point
// and the reference interface each one replaces.
#include "adkv_host.h"

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

}  // namespace adkv

using namespace adkv;

extern "C" {

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

}  // extern "C"
