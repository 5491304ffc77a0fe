// Part of libadkv_b200.so (sm_100a).  See include/adkv_b200.h for the contract of every entry point.
//
// Decode over a checkpointed cache: with the recurrence state stored every `interval` tokens, the
// segments between checkpoints are independent, so every (stream, segment) gets its own K/V warp
// pair instead of one pair walking the whole sequence.  Segments leave un-normalised partial results
// (running maximum, denominator, weighted sums) in caller-provided scratch memory; a second small
// kernel merges them.  The idea of boundary state checkpoints is the reference paper's (appendix on
// long contexts); the reference code has no implementation of it.
#include "adkv_host.h"

#include <mutex>

#include "adkv_half.cuh"
#include "adkv_softmax.cuh"

namespace adkv {

constexpr int kPartStride = 4 + kD;   // floats per (stream, segment, head): max (log2 units), denominator, 2 pad, kD sums

template <int G, bool HALF_W>
struct PartialSrc : SoftmaxSrc<G, 1, HALF_W> {
    float *part;   // [G][kPartStride] of this (stream, segment)
    __device__ __forceinline__ void store(const VArgs &, int, int, int c0, const float (&acc)[G][4]) const
    {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (c0 == 0) {
                part[g * kPartStride] = this->m[g];
                part[g * kPartStride + 1] = this->l[g];
            }
            *reinterpret_cast<float4 *>(part + g * kPartStride + 4 + c0) =
                make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        }
    }
    // The segment could not be finished (a bounded wait gave up; the status word says which): leave a partial
    // that turns the merged output of these heads into NaN, so that neither the scratch contents of an earlier
    // call nor an output that silently lacks a segment can pass for a result.
    __device__ __forceinline__ void give_up(int c0) const
    {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (c0 == 0) {
                part[g * kPartStride] = -INFINITY;
                part[g * kPartStride + 1] = __int_as_float(0x7fc00000);
            }
            *reinterpret_cast<float4 *>(part + g * kPartStride + 4 + c0) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
};

struct CkptArgs {
    float *k_ckpt, *v_ckpt;   // [B*Hkv][n_ckpt_cap][2][kD]; entry k = state before token (k+1)*interval
    int interval, n_ckpt_cap;
    bool mute_k;              // self-test (ADKV_FLAG_SELFTEST_MUTE_K): the K warps do nothing, so every V warp's wait runs out
};

// Guarded chunk bodies as function calls (see k_chunk_guarded): measured 2-3 % faster for 4-bit codes with one query
// head per KV head at every batch and checkpoint interval tried; not measured for the other instantiations.
template <int BITS, int G>
constexpr bool kOutOfLineGuardedSegments = BITS == 4 && G == 1;

template <int BITS, int G, int MODE>
__global__ void __launch_bounds__(64) decode_attn_split_kernel(KArgs ka, VArgs va, const float *__restrict__ mask,
                                                               long long mask_stride_b, float scaling, CkptArgs ck,
                                                               float *__restrict__ scratch)
{
    __shared__ alignas(128) uint8_t kbuf[kStages * Tile<BITS>::BYTES];
    __shared__ alignas(128) uint8_t vbuf[kStages * Tile<BITS>::BYTES];
    __shared__ alignas(16) float red[G * 8 * 36];
    __shared__ alignas(16) float2 wts[G * kTileTok];
    __shared__ FusedShared<G> fs;
    __shared__ uint64_t kbar[kStages], vbar[kStages];

    const int bh = blockIdx.x, b = bh / ka.Hkv, h = bh % ka.Hkv;
    const int j = blockIdx.y, n_seg = gridDim.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(&kbar[i], 1); mbar_init(&vbar[i], 1); }
        fs.init_barriers(1);
        mbar_init_fence();
    }
    __syncthreads();

    const int T = ka.T;
    Seg seg;
    seg.t_begin = j * ck.interval;
    seg.t_end = min(T, (j + 1) * ck.interval);
    seg.append = (j == n_seg - 1);
    seg.slice = 0;
    const size_t stream_ckpt = size_t(bh) * ck.n_ckpt_cap;
    const bool write_ckpt = seg.append && (T + 1) % ck.interval == 0;
    const size_t out_idx = write_ckpt ? stream_ckpt + (T + 1) / ck.interval - 1 : 0;
    if (warp == 0) {
        if (ck.mute_k) return;
        seg.init = j ? ck.k_ckpt + (stream_ckpt + j - 1) * 2 * kD : nullptr;
        seg.ckpt_out = write_ckpt ? ck.k_ckpt + out_idx * 2 * kD : nullptr;
        RingSink<G> sink{&fs, 0, 0};
        k_scan<BITS, G, MODE, RingSink<G>, kStages, false, kOutOfLineGuardedSegments<BITS, G>>(ka, seg, b, h, lane, kbuf, kbar, red, sink);
    } else {
        seg.init = j ? ck.v_ckpt + (stream_ckpt + j - 1) * 2 * kD : nullptr;
        seg.ckpt_out = write_ckpt ? ck.v_ckpt + out_idx * 2 * kD : nullptr;
        PartialSrc<G, MODE == kModeHalf> src;
        src.sh = &fs;
        src.wts = wts;
        src.mask = mask ? mask + size_t(b) * mask_stride_b : nullptr;
        src.scale2 = scaling * 1.4426950408889634f;
        src.n_tiles = (seg.t_end - seg.t_begin + kTileTok - 1) / kTileTok;
        src.t_begin = seg.t_begin;
        src.part = scratch + (size_t(bh) * n_seg + j) * G * kPartStride;
        src.init();
        v_scan<BITS, G, MODE, PartialSrc<G, MODE == kModeHalf>, kStages, false, kOutOfLineGuardedSegments<BITS, G>>(va, seg, b, h, lane, vbuf, vbar, wts, src);
    }
}

// out[b, hq, c] = sum_j acc_j[c] * 2^(m_j - M) / sum_j l_j * 2^(m_j - M),  M = max_j m_j.
__global__ void __launch_bounds__(kD) merge_partials_kernel(const float *__restrict__ scratch, __half *__restrict__ out,
                                                            int Hq, int Hkv, int n_seg)
{
    const int bhq = blockIdx.x, b = bhq / Hq, hq = bhq % Hq, G = Hq / Hkv, h = hq / G, g = hq % G;
    const int c = threadIdx.x;
    // Launched as a programmatic dependent of the segment kernel (its launch latency is paid while that kernel
    // still runs): wait here until the segment kernel has completed and its partials are visible.  Without
    // that launch attribute the instruction does nothing.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float *base = scratch + (size_t(b * Hkv + h) * n_seg * G + g) * kPartStride;
    const size_t seg_stride = size_t(G) * kPartStride;
    float M = -INFINITY;
    for (int j = 0; j < n_seg; ++j) M = fmaxf(M, base[j * seg_stride]);
    float L = 0.f, A = 0.f;
    for (int j = 0; j < n_seg; ++j) {
        const float m = base[j * seg_stride];
        const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
        L = fmaf(base[j * seg_stride + 1], w, L);
        A = fmaf(base[j * seg_stride + 4 + c], w, A);
    }
    out[size_t(bhq) * kD + c] = __float2half_rn(A / L);
}

}  // namespace adkv

using namespace adkv;

ADKV_DEFINE_TU_STATUS(adkv_tu_status_split)

// The merge follows the segment kernel on the same stream as its programmatic dependent: set up early, started
// when the segment kernel is done (griddepcontrol.wait in the kernel orders the memory).
static int launch_merge(const float *scratch, __half *out, int B, int Hq, int Hkv, int n_seg, cudaStream_t s)
{
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(B * Hq);
    cfg.blockDim = dim3(kD);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, merge_partials_kernel, scratch, out, Hq, Hkv, n_seg);
    return e == cudaSuccess ? launch_status() : int(e);
}

extern "C" {

long long adkv_decode_attn_ckpt_scratch_bytes(int B, int Hq, int Hkv, int T, int interval)
{
    if (B < 0 || Hq <= 0 || Hkv <= 0 || T < 0 || interval <= 0 || Hq % Hkv != 0) return ADKV_E_SHAPE;
    return (long long)B * Hq * (T / interval + 1) * kPartStride * (long long)sizeof(float);
}

int adkv_decode_attn_ckpt(const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new,
                          const adkv_params *kp, const adkv_params *vp, void *k_tail, void *v_tail, void *k_ckpt,
                          void *v_ckpt, int interval, int n_ckpt_cap, const void *mask, long long mask_stride_b, void *out, void *scratch,
                          long long scratch_bytes, int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits,
                          float scaling, float scale_min, float scale_max, unsigned flags, void *stream)
{
    if (!q || !k_cache || !v_cache || !k_new || !v_new || !out || !params_ok(kp) || !params_ok(vp) || !scratch ||
        !k_ckpt || !v_ckpt)
        return ADKV_E_NULL;
    if (D != kD) return ADKV_E_HEAD_DIM;   // checkpointed decode: 128-wide heads only
    if (int rc = check_common(B, Hq, Hkv, T, D, n_super_cap, bits, T + 1)) return rc;
    if (int rc = check_tails(k_tail, v_tail, flags)) return rc;
    if (interval <= 0 || interval % kTileTok != 0 || n_ckpt_cap < 0) return ADKV_E_SHAPE;
    if ((T + 1) / interval > n_ckpt_cap) return ADKV_E_CAPACITY;
    if (!aligned16(k_cache) || !aligned16(v_cache) || !aligned8(q) || !aligned8(out) || !aligned8(k_new) ||
        !aligned8(v_new) || !params_aligned(kp) || !params_aligned(vp) || !aligned16(k_ckpt) || !aligned16(v_ckpt) ||
        !aligned16(scratch))
        return ADKV_E_ALIGN;
    if (scratch_bytes < adkv_decode_attn_ckpt_scratch_bytes(B, Hq, Hkv, T, interval)) return ADKV_E_SCRATCH;
    if (B == 0) return 0;
    const bool keep = flags & ADKV_FLAG_TAIL_KEEP;
    const KArgs ka{static_cast<const __half *>(q), static_cast<uint8_t *>(k_cache),
                   static_cast<const __half *>(k_new), to_ptrs(kp), Hq, Hkv, T, n_super_cap, scale_min, scale_max, D,
                   static_cast<float *>(k_tail), keep};
    const VArgs va{static_cast<uint8_t *>(v_cache), static_cast<const __half *>(v_new), static_cast<__half *>(out),
                   to_ptrs(vp), Hq, Hkv, T, n_super_cap, scale_min, scale_max, D, static_cast<float *>(v_tail), keep};
    const CkptArgs ck{static_cast<float *>(k_ckpt), static_cast<float *>(v_ckpt), interval, n_ckpt_cap,
                      (flags & ADKV_FLAG_SELFTEST_MUTE_K) != 0};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool exact = !(flags & ADKV_FLAG_FAST_REPLAY);
    const int n_seg = T / interval + 1;
    if (n_seg > 65535) return ADKV_E_SHAPE;
    const dim3 grid(B * Hkv, n_seg);
    if (flags & ADKV_FLAG_HALF_STATE) {
        ADKV_DISPATCH_H(bits, Hq / Hkv,
                        (decode_attn_split_kernel<BITS, G, kModeHalf><<<grid, 64, 0, s>>>(
                          ka, va, static_cast<const float *>(mask), mask_stride_b, scaling, ck,
                          static_cast<float *>(scratch))))
    } else {
        ADKV_DISPATCH(bits, exact, Hq / Hkv,
                      (decode_attn_split_kernel<BITS, G, ARITH><<<grid, 64, 0, s>>>(
                          ka, va, static_cast<const float *>(mask), mask_stride_b, scaling, ck,
                          static_cast<float *>(scratch))))
    }
    if (int rc = launch_status()) return rc;
    return launch_merge(static_cast<const float *>(scratch), static_cast<__half *>(out), B, Hq, Hkv, n_seg, s);
}

}  // extern "C"

// =========================================================================================
// The same decode step for callers that are not in a position to provide scratch memory.
//
// Some hosts of this library cannot allocate: an inference server that has handed every byte of HBM
// to its own block pool at start-up has nothing left for cudaMalloc to give (and would not want the
// fragmentation), and a plugin that is only ever passed device pointers by its host runtime has no
// allocator to ask.  For them the partial results live in the fixed array below instead of a
// caller-owned buffer.  Every process that loads the library pays for the array on every GPU it
// touches until it exits, which is why it is kept to ADKV_STATIC_SCRATCH_BYTES.
namespace adkv {

static __device__ __align__(256) float g_static_scratch[ADKV_STATIC_SCRATCH_BYTES / sizeof(float)];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: handing it
// to a kernel would fault or, where the GPU can reach host memory, quietly use the wrong memory.
// The device address is asked for once per device, with that device current, and remembered.
constexpr int kMaxDevices = 64;
static float *g_static_scratch_addr[kMaxDevices];
static bool g_static_scratch_known[kMaxDevices];
static std::mutex g_static_scratch_lock;

static int static_scratch_of_current_device(float **addr)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return int(e);
    if (dev < 0 || dev >= kMaxDevices) return ADKV_E_SHAPE;
    std::lock_guard<std::mutex> guard(g_static_scratch_lock);
    if (!g_static_scratch_known[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return int(e);
        g_static_scratch_addr[dev] = static_cast<float *>(p);
        g_static_scratch_known[dev] = true;
    }
    *addr = g_static_scratch_addr[dev];
    return 0;
}

}  // namespace adkv

extern "C" {

int adkv_decode_attn_ckpt_static(const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new,
                                 const adkv_params *kp, const adkv_params *vp, void *k_tail, void *v_tail,
                                 void *k_ckpt, void *v_ckpt, int interval, int n_ckpt_cap, const void *mask, long long mask_stride_b, void *out,
                                 int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits, float scaling,
                                 float scale_min, float scale_max, unsigned flags, void *stream)
{
    const long long need = adkv_decode_attn_ckpt_scratch_bytes(B, Hq, Hkv, T, interval);
    if (need < 0) return int(need);
    if (need > (long long)ADKV_STATIC_SCRATCH_BYTES) return ADKV_E_STATIC_MAX;
    float *scratch = nullptr;
    if (int rc = static_scratch_of_current_device(&scratch)) return rc;
    // Nothing in the array has to start at zero: the segment kernel writes every slot the merge kernel
    // reads -- its result, or a NaN marker where a bounded wait gave up -- so what an earlier call left
    // behind is always overwritten.
    return adkv_decode_attn_ckpt(q, k_cache, v_cache, k_new, v_new, kp, vp, k_tail, v_tail, k_ckpt, v_ckpt, interval,
                                 n_ckpt_cap, mask, mask_stride_b, out, scratch, (long long)ADKV_STATIC_SCRATCH_BYTES, B, Hq, Hkv,
                                 T, D, n_super_cap, bits, scaling, scale_min, scale_max, flags, stream);
}

}  // extern "C"
