// Device-side building blocks of the ADKV kernels (sm_100a): code extraction, the fp32
// recurrence in its canonical and contracted forms, mbarrier / bulk-copy (1-D TMA) wrappers
// with bounded waits.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>
#include <utility>

namespace adkv {

// Compile-time loop: f(std::integral_constant<int, 0>{}) ... f(std::integral_constant<int, N-1>{}).
template <class F, int... I>
__device__ __forceinline__ void static_for_impl(F &&f, std::integer_sequence<int, I...>)
{
    (f(std::integral_constant<int, I>{}), ...);
}
template <int N, class F>
__device__ __forceinline__ void static_for(F &&f)
{
    static_for_impl(f, std::make_integer_sequence<int, N>{});
}

constexpr int kD = 128;              // head dim served by this build
constexpr float kEps = 1e-8f;        // src/adkv/train/train_model.py:9
constexpr unsigned kFull = 0xffffffffu;

// Status codes written to g_status when a bounded wait gives up (1-5) or an argument only the device can
// see is unusable (6).
constexpr int kStatKWait = 1, kStatVWait = 2, kStatLFullWait = 3, kStatLEmptyWait = 4, kStatDrain = 5;
constexpr int kStatSelfTest = 7;   // the wait of adkv_selftest_wait_timeout ran out, as it must
constexpr int kStatCapacity = 6;   // a device-side sequence length did not fit the cache: that stream was skipped

// One status word per translation unit that includes this header (the library is one unit).
static __device__ int g_status = 0;

// ------------------------------------------------------------------------------------------
// Codes.  Word (sg, c) holds TPW tokens of channel c, token j in bits [BITS*j, BITS*j+BITS)
// as code + BIAS (4-bit layout: src/adkv/kernel/gemv.cu:266-305).
template <int BITS>
struct Codec {
    static constexpr int TPW = 32 / BITS;
    static constexpr int BIAS = 1 << (BITS - 1);
    static constexpr uint32_t FIELD = (1u << BITS) - 1u;
    __host__ __device__ static constexpr float qlo() { return -float(BIAS); }
    __host__ __device__ static constexpr float qhi() { return float(BIAS - 1); }
};

// A value the optimiser cannot see through: keeps a constant in a register for the whole kernel
// instead of being re-materialised as an immediate at every use.
__device__ __forceinline__ uint32_t opaque_u32(uint32_t v)
{
    uint32_t r;
    asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

// Codes as floats without integer-to-float conversions.  A group of 4 consecutive fields is taken
// from the word shifted down to bit 0; field k of the group then sits at bit p = BITS*k inside the
// mantissa.  Masking it in place into the bit pattern of 2^(23-p) gives the float 2^(23-p) + field,
// and subtracting 2^(23-p) + BIAS is exact.  The exponent pattern lives in a register and the mask is
// an immediate so that the mask-and-merge is a single three-input logic operation.
template <int BITS>
struct FieldConsts {
    uint32_t e[4];
    uint32_t negc[4];   // bit pattern of -(2^(23-p) + BIAS), kept in a register to build packed operands
    __device__ __forceinline__ void init()
    {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            e[k] = opaque_u32(uint32_t(127 + 23 - BITS * k) << 23);
            negc[k] = opaque_u32(__float_as_uint(-(float(1u << (23 - BITS * k)) + float(Codec<BITS>::BIAS))));
        }
    }
    // codes of field K of two words as a packed pair
    template <int K>
    __device__ __forceinline__ unsigned long long code2(uint32_t ga, uint32_t gb) const
    {
        uint32_t a, b;
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(a) : "r"(ga), "n"(Codec<BITS>::FIELD << (BITS * K)), "r"(e[K]));
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(b) : "r"(gb), "n"(Codec<BITS>::FIELD << (BITS * K)), "r"(e[K]));
        unsigned long long f, c, r;
        asm("mov.b64 %0, {%1, %2};" : "=l"(f) : "r"(a), "r"(b));
        asm("mov.b64 %0, {%1, %1};" : "=l"(c) : "r"(negc[K]));
        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(f), "l"(c));
        return r;
    }
    template <int K>
    __device__ __forceinline__ float code(uint32_t group) const
    {
        constexpr float c = float(1u << (23 - BITS * K)) + float(Codec<BITS>::BIAS);
        uint32_t bits;
        // (group & mask) | exponent as ONE lop3 (the compiler otherwise emits two): LUT 0xEA = (a & b) | c
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(bits) : "r"(group), "n"(Codec<BITS>::FIELD << (BITS * K)), "r"(e[K]));
        return __fsub_rn(__uint_as_float(bits), c);
    }
};

template <int BITS>
__device__ __forceinline__ float code_f_rt(uint32_t w, int j)
{
    using C = Codec<BITS>;
    return float(int((w >> (BITS * j)) & C::FIELD) - C::BIAS);
}

// ------------------------------------------------------------------------------------------
// The recurrence (src/adkv/train/train_model.py:70-81).  tc = target (canonical) or
// 1 - beta*target (contracted form).
struct Chan {
    float zp, s, alpha, beta, tc;
};

// Decoder side of one token: dequantise code q with the current state, then advance.
// GUARDED = false drops the eps guard and the scale clamp; the caller uses it only where
// `SafeRange` proves both to be the identity for the tokens processed, so results are unchanged.
template <bool EXACT, bool GUARDED>
__device__ __forceinline__ float replay_step(float q, Chan &c, float smin, float smax)
{
    const float ss = GUARDED ? fmaxf(c.s, kEps) : c.s;
    const float rh = __fmul_rn(q, ss);
    const float xh = __fadd_rn(rh, c.zp);
    float s_new;
    if (EXACT) {
        c.zp = __fadd_rn(c.zp, __fmul_rn(c.alpha, rh));
        const float err = __fsub_rn(fabsf(q), c.tc);
        s_new = __fadd_rn(c.s, __fmul_rn(__fmul_rn(c.s, c.beta), err));
    } else {
        c.zp = fmaf(c.alpha, rh, c.zp);
        s_new = c.s * fmaf(c.beta, fabsf(q), c.tc);
    }
    c.s = GUARDED ? fminf(fmaxf(s_new, smin), smax) : s_new;
    return xh;
}

// ------------------------------------------------------------------------------------------
// Packed fp32 pairs.  sm_100 executes add/mul/fma.rn.f32x2 at the same FP32 rate as the scalar forms
// but in half the issue slots; the replay is bound by issue slots, so the unguarded body works on
// channel pairs.  Each element is rounded exactly like the scalar instruction (".rn", no flush).
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pk2(float lo, float hi)
{
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c)
{
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// a + b for a packed product `a`, as fma(a, 1, b): bit-identical to add.rn (a * 1 is exact), but not
// something the assembler can merge with the multiply that produced `a`.  ptxas contracts
// mul.rn.f32x2 + add.rn.f32x2 into FFMA2 when the product has no other use -- explicit ".rn", asm
// volatile and -fmad=false do not stop it (seen in the opcode counters and as few-ulp drift of the
// replayed state) -- and that would break the canonical, separately rounded order.  `one` must be
// a value the assembler cannot see through (PairOnes).
__device__ __forceinline__ f32x2 add_product2(f32x2 a, f32x2 one, f32x2 b) { return fma2(a, one, b); }

__device__ __forceinline__ f32x2 abs2(f32x2 v)
{
    float lo, hi;
    upk2(v, lo, hi);
    return pk2(fabsf(lo), fabsf(hi));
}

// Per-pair constants of the recurrence.  tc = -target (canonical) or 1 - beta*target (contracted).
struct PairConst {
    f32x2 alpha, beta, tc;
};

// (1.0f, 1.0f) read from constant memory at run time: the assembler propagates immediates even out of
// volatile asm, but it cannot assume the contents of a __constant__ variable.
static __constant__ float c_one = 1.0f;
__device__ __forceinline__ f32x2 opaque_ones2()
{
    const float v = *const_cast<const volatile float *>(&c_one);
    return pk2(v, v);
}

template <bool EXACT>
__device__ __forceinline__ void make_pair_consts(const Chan (&ch)[4], PairConst (&pc)[2])
{
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        pc[p].alpha = pk2(ch[2 * p].alpha, ch[2 * p + 1].alpha);
        pc[p].beta = pk2(ch[2 * p].beta, ch[2 * p + 1].beta);
        pc[p].tc = EXACT ? pk2(-ch[2 * p].tc, -ch[2 * p + 1].tc) : pk2(ch[2 * p].tc, ch[2 * p + 1].tc);
    }
}

// Unguarded decoder step on a channel pair: same operations, same order, same roundings as
// replay_step<EXACT, false> on each element.
template <bool EXACT>
__device__ __forceinline__ f32x2 replay_step2(f32x2 q2, f32x2 &zp, f32x2 &s, const PairConst &c, f32x2 one)
{
    const f32x2 rh = mul2(q2, s);
    const f32x2 xh = add_product2(rh, one, zp);
    const f32x2 aq = abs2(q2);
    if (EXACT) {
        zp = add_product2(mul2(c.alpha, rh), one, zp);
        s = add_product2(mul2(mul2(s, c.beta), add2(aq, c.tc)), one, s);
    } else {
        zp = fma2(c.alpha, rh, zp);
        s = mul2(s, fma2(c.beta, aq, c.tc));
    }
    return xh;
}

// Interval of scales from which 8 further updates cannot leave [max(smin, eps), smax]: inside it the
// clamp and the eps guard are the identity and the unguarded step gives bit-identical results.
// One conservative interval per lane (intersection over its channels).
struct SafeRange {
    float lo, hi;
    template <int BITS, int N>
    __device__ __forceinline__ void init(const float (&beta)[N], const float (&target)[N], float smin, float smax)
    {
        lo = 0.f;
        hi = INFINITY;
#pragma unroll
        for (int c = 0; c < N; ++c) {
            const float g0 = 1.f - beta[c] * target[c];                      // |q| = 0
            const float g1 = g0 + beta[c] * float(Codec<BITS>::BIAS);        // |q| = largest code magnitude
            const float gmn = fminf(fminf(g0, g1), 1.f), gmx = fmaxf(fmaxf(g0, g1), 1.f);
            float pmn = gmn * gmn, pmx = gmx * gmx;                          // 8th powers
            pmn *= pmn; pmn *= pmn;
            pmx *= pmx; pmx *= pmx;
            // approximate division (2 ulp) is far inside the 2e-5 margin that keeps the interval conservative
            const float l = gmn > 0.f ? __fdividef(fmaxf(smin, kEps), pmn * (1.f - 2e-5f)) : INFINITY;
            const float h = __fdividef(smax, pmx * (1.f + 2e-5f));
            lo = fmaxf(lo, l);
            hi = fminf(hi, h);
        }
        if (!(lo <= hi)) { lo = INFINITY; hi = 0.f; }
    }
    // warp-uniform: every channel of every lane is inside its interval
    __device__ __forceinline__ bool holds(const Chan (&ch)[4]) const
    {
        // chained, not a tree: the chain maps onto the three-input minimum / maximum instruction
        const float mn = fminf(fminf(fminf(ch[0].s, ch[1].s), ch[2].s), ch[3].s);
        const float mx = fmaxf(fmaxf(fmaxf(ch[0].s, ch[1].s), ch[2].s), ch[3].s);
        return __all_sync(kFull, mn >= lo && mx <= hi);
    }
    __device__ __forceinline__ bool holds(const Chan (&ch)[2]) const
    {
        return __all_sync(kFull, fminf(ch[0].s, ch[1].s) >= lo && fmaxf(ch[0].s, ch[1].s) <= hi);
    }
};

// Encoder side of one token, canonical order only (train_model.py:72, :8-17).  Returns the
// code as a float; rh = q * max(s, eps).
template <int BITS>
__device__ __forceinline__ float quantize(float x, const Chan &c, float &rh)
{
    const float ss = fmaxf(c.s, kEps);
    const float v = __fdiv_rn(__fsub_rn(x, c.zp), ss);
    const float q = fminf(fmaxf(rintf(v), Codec<BITS>::qlo()), Codec<BITS>::qhi());
    rh = __fmul_rn(q, ss);
    return q;
}

// State update after an appended token, in the arithmetic the replay uses (always with guard and clamp).
template <bool EXACT>
__device__ __forceinline__ void advance_like_replay(float q, float rh, Chan &c, float smin, float smax)
{
    float s_new;
    if (EXACT) {
        c.zp = __fadd_rn(c.zp, __fmul_rn(c.alpha, rh));
        s_new = __fadd_rn(c.s, __fmul_rn(__fmul_rn(c.s, c.beta), __fsub_rn(fabsf(q), c.tc)));
    } else {
        c.zp = fmaf(c.alpha, rh, c.zp);
        s_new = c.s * fmaf(c.beta, fabsf(q), c.tc);
    }
    c.s = fminf(fmaxf(s_new, smin), smax);
}

// Speculative form of quantize(): the quotient is formed with the approximate reciprocal (error
// below 2.2e-6 for |v| < 16) and rounded with the 1.5*2^23 trick after clamping (clamp and
// round-to-nearest-even commute because the limits are integers).  The result equals the canonical
// one unless the approximate quotient lies within 4e-6 of a rounding boundary k + 0.5; that case
// sets `doubt`, and the caller redoes the tokens with quantize() from a saved state.  No branch
// sits on the token-to-token dependency chain.  `tbits` carries the code in its low bits:
// field = (tbits & FIELD) ^ BIAS.  GUARDED as in replay_step.
template <int BITS, bool GUARDED>
__device__ __forceinline__ float quantize_spec(float x, const Chan &c, float &rh, uint32_t &tbits, bool &doubt)
{
    constexpr float M = 12582912.f;   // 1.5 * 2^23
    const float ss = GUARDED ? fmaxf(c.s, kEps) : c.s;
    const float r = __fsub_rn(x, c.zp);
    float inv;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(ss));
    const float v = __fmul_rn(r, inv);
    const float t = __fadd_rn(fminf(fmaxf(v, Codec<BITS>::qlo()), Codec<BITS>::qhi()), M);
    const float q = __fsub_rn(t, M);
    doubt |= !(fabsf(fabsf(__fsub_rn(v, q)) - 0.5f) > 4e-6f);
    rh = __fmul_rn(q, ss);
    tbits = __float_as_uint(t);
    return q;
}

template <bool GUARDED>
__device__ __forceinline__ void advance_canonical_g(float q, float rh, Chan &c, float smin, float smax)
{
    c.zp = __fadd_rn(c.zp, __fmul_rn(c.alpha, rh));
    const float err = __fsub_rn(fabsf(q), c.tc);
    const float s_new = __fadd_rn(c.s, __fmul_rn(__fmul_rn(c.s, c.beta), err));
    c.s = GUARDED ? fminf(fmaxf(s_new, smin), smax) : s_new;
}

__device__ __forceinline__ void advance_canonical(float q, float rh, Chan &c, float smin, float smax)
{
    c.zp = __fadd_rn(c.zp, __fmul_rn(c.alpha, rh));
    const float err = __fsub_rn(fabsf(q), c.tc);
    c.s = fminf(fmaxf(__fadd_rn(c.s, __fmul_rn(__fmul_rn(c.s, c.beta), err)), smin), smax);
}

// ------------------------------------------------------------------------------------------
// mbarrier + bulk copy (non-multicast 1-D TMA) wrappers.
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Wait for a phase with a wall-clock limit (1 s).  Every lane of the calling warp must call it;
// the result is warp-uniform.  On failure the status word records `code`.  A warp that finds the
// phase incomplete sleeps between polls so that it does not take issue slots from the warps it is
// waiting for.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int code,
                                                  uint64_t limit_ns = 1000000000ull)
{
    bool ok = mbar_try_wait(bar, parity);
    if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        for (uint32_t it = 1;; ++it) {
            __nanosleep(it < 256 ? 32 : 512);   // short naps first: with one stream per SM, 128 ns naps cost 8 % of the step
            ok = mbar_try_wait(bar, parity);
            if (ok) break;
            if ((it & 63u) == 0 && globaltimer_ns() - t0 > limit_ns) break;
        }
    }
    ok = __all_sync(kFull, ok);
    if (!ok && (threadIdx.x & 31) == 0) atomicExch(&g_status, code);
    return ok;
}

// Global -> shared bulk copy completing on an mbarrier.  dst, src 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
    return v;
}

// Load the five fp16 parameters of 4 consecutive channels starting at element `off` of the [Hkv, D] tensors.
struct ParamPtrs {
    const __half *zp_init, *scale_init, *alpha, *beta, *target;
};

template <int BITS, bool EXACT>
__device__ __forceinline__ void load_chan4(Chan (&ch)[4], SafeRange &safe, const ParamPtrs &p, size_t off,
                                           float smin, float smax)
{
    const uint2 a = *reinterpret_cast<const uint2 *>(p.zp_init + off);
    const uint2 b = *reinterpret_cast<const uint2 *>(p.scale_init + off);
    const uint2 c = *reinterpret_cast<const uint2 *>(p.alpha + off);
    const uint2 d = *reinterpret_cast<const uint2 *>(p.beta + off);
    const uint2 e = *reinterpret_cast<const uint2 *>(p.target + off);
    const __half2 *pa = reinterpret_cast<const __half2 *>(&a), *pb = reinterpret_cast<const __half2 *>(&b),
                  *pc = reinterpret_cast<const __half2 *>(&c), *pd = reinterpret_cast<const __half2 *>(&d),
                  *pe = reinterpret_cast<const __half2 *>(&e);
    float beta[4], target[4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float2 za = __half22float2(pa[i]), sb = __half22float2(pb[i]), al = __half22float2(pc[i]),
                     be = __half22float2(pd[i]), tg = __half22float2(pe[i]);
        ch[2 * i] = Chan{za.x, sb.x, al.x, be.x, EXACT ? tg.x : fmaf(-be.x, tg.x, 1.0f)};
        ch[2 * i + 1] = Chan{za.y, sb.y, al.y, be.y, EXACT ? tg.y : fmaf(-be.y, tg.y, 1.0f)};
        beta[2 * i] = be.x; beta[2 * i + 1] = be.y;
        target[2 * i] = tg.x; target[2 * i + 1] = tg.y;
    }
    safe.template init<BITS, 4>(beta, target, smin, smax);
}

__device__ __forceinline__ void load_half4(float (&v)[4], const __half *p)
{
    const uint2 a = *reinterpret_cast<const uint2 *>(p);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&a.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&a.y));
    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
}

__device__ __forceinline__ void store_half4(__half *p, const float (&v)[4])
{
    const __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
    uint2 a;
    a.x = *reinterpret_cast<const uint32_t *>(&lo);
    a.y = *reinterpret_cast<const uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(p) = a;
}

}  // namespace adkv
