// Host-side helpers shared by the translation units of libadkv_b200.so.
#pragma once
#include "../../include/adkv_b200.h"
#include "adkv_device.cuh"

#define ADKV_HIDDEN __attribute__((visibility("hidden")))

namespace adkv {

static inline ParamPtrs to_ptrs(const adkv_params *p)
{
    return ParamPtrs{static_cast<const __half *>(p->zp_init), static_cast<const __half *>(p->scale_init),
                     static_cast<const __half *>(p->alpha), static_cast<const __half *>(p->beta),
                     static_cast<const __half *>(p->target)};
}

static inline bool params_ok(const adkv_params *p)
{
    return p && p->zp_init && p->scale_init && p->alpha && p->beta && p->target;
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline bool aligned8(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }

static inline bool params_aligned(const adkv_params *p)
{
    return aligned8(p->zp_init) && aligned8(p->scale_init) && aligned8(p->alpha) && aligned8(p->beta) &&
           aligned8(p->target);
}

static inline int launch_status()
{
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : int(e);
}

static inline int check_common(int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits, int n_written_end)
{
    if (D != 128 && D != 256 && D != 512) return ADKV_E_HEAD_DIM;
    if (bits != 2 && bits != 4) return ADKV_E_BITS;
    if (B < 0 || Hq <= 0 || Hkv <= 0 || T < 0 || n_super_cap < 0 || Hq % Hkv != 0) return ADKV_E_SHAPE;
    const int tpw = 32 / bits;
    if ((long long)(n_written_end + tpw - 1) / tpw > (long long)n_super_cap) return ADKV_E_CAPACITY;
    return 0;
}

// Tail states of the decode entry points: both or neither, 16-byte aligned, fp32 arithmetic only.
static inline int check_tails(const void *k_tail, const void *v_tail, unsigned flags)
{
    if (!k_tail && !v_tail) return 0;
    if (!k_tail || !v_tail || (flags & ADKV_FLAG_HALF_STATE)) return ADKV_E_FLAGS;
    if (!aligned16(k_tail) || !aligned16(v_tail)) return ADKV_E_ALIGN;
    return 0;
}

// Every translation unit that includes adkv_device.cuh has its own device status word; this defines the hidden
// function through which adkv_device_status reads and clears the one of the unit it is expanded in.
#define ADKV_DEFINE_TU_STATUS(fn_name)                                                \
    ADKV_HIDDEN int fn_name(int *out)                                                 \
    {                                                                                 \
        cudaError_t e = cudaMemcpyFromSymbol(out, adkv::g_status, sizeof(int));       \
        if (e != cudaSuccess) return int(e);                                          \
        const int zero = 0;                                                           \
        e = cudaMemcpyToSymbol(adkv::g_status, &zero, sizeof(int));                   \
        return e == cudaSuccess ? 0 : int(e);                                         \
    }

// Dispatch over (bits, group size, arithmetic).  CALL sees BITS, G, EXACT and ARITH (kArithCanon / kArithFma).
#define ADKV_DISPATCH_G(BITS_, EXACT_, G_, CALL) \
    switch (G_) {                                \
    case 1: { constexpr int BITS = BITS_; constexpr bool EXACT = EXACT_; constexpr int ARITH = EXACT_ ? 1 : 0; constexpr int G = 1; (void)EXACT; (void)ARITH; CALL; } break; \
    case 2: { constexpr int BITS = BITS_; constexpr bool EXACT = EXACT_; constexpr int ARITH = EXACT_ ? 1 : 0; constexpr int G = 2; (void)EXACT; (void)ARITH; CALL; } break; \
    case 4: { constexpr int BITS = BITS_; constexpr bool EXACT = EXACT_; constexpr int ARITH = EXACT_ ? 1 : 0; constexpr int G = 4; (void)EXACT; (void)ARITH; CALL; } break; \
    case 8: { constexpr int BITS = BITS_; constexpr bool EXACT = EXACT_; constexpr int ARITH = EXACT_ ? 1 : 0; constexpr int G = 8; (void)EXACT; (void)ARITH; CALL; } break; \
    default: return ADKV_E_SHAPE;                \
    }
#define ADKV_DISPATCH(bits_, exact_, G_, CALL)                            \
    if (bits_ == 4) {                                                     \
        if (exact_) { ADKV_DISPATCH_G(4, true, G_, CALL) } else { ADKV_DISPATCH_G(4, false, G_, CALL) } \
    } else {                                                              \
        if (exact_) { ADKV_DISPATCH_G(2, true, G_, CALL) } else { ADKV_DISPATCH_G(2, false, G_, CALL) } \
    }


// Dispatch over (bits, group size) for kernels without an EXACT parameter.
#define ADKV_DISPATCH_H(bits_, G_, CALL)                                              \
    switch ((bits_) * 16 + (G_)) {                                                    \
    case 4 * 16 + 1: { constexpr int BITS = 4; constexpr int G = 1; CALL; } break;    \
    case 4 * 16 + 2: { constexpr int BITS = 4; constexpr int G = 2; CALL; } break;    \
    case 4 * 16 + 4: { constexpr int BITS = 4; constexpr int G = 4; CALL; } break;    \
    case 4 * 16 + 8: { constexpr int BITS = 4; constexpr int G = 8; CALL; } break;    \
    case 2 * 16 + 1: { constexpr int BITS = 2; constexpr int G = 1; CALL; } break;    \
    case 2 * 16 + 2: { constexpr int BITS = 2; constexpr int G = 2; CALL; } break;    \
    case 2 * 16 + 4: { constexpr int BITS = 2; constexpr int G = 4; CALL; } break;    \
    case 2 * 16 + 8: { constexpr int BITS = 2; constexpr int G = 8; CALL; } break;    \
    default: return ADKV_E_SHAPE;                                                     \
    }

}  // namespace adkv
