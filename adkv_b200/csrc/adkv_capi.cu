// Part of libadkv_b200.so (sm_100a).  See include/adkv_b200.h for the contract of every entry point
// and the reference interface each one replaces.
#include "adkv_host.h"

ADKV_HIDDEN int adkv_tu_status_fused(int *out);
ADKV_HIDDEN int adkv_tu_status_unfused(int *out);
ADKV_HIDDEN int adkv_tu_status_encode(int *out);
ADKV_HIDDEN int adkv_tu_status_split(int *out);
ADKV_HIDDEN int adkv_tu_status_wide(int *out);
ADKV_HIDDEN int adkv_tu_status_half(int *out);
ADKV_HIDDEN int adkv_tu_status_narrow(int *out);

namespace adkv {

// One warp waits on a barrier that nothing ever completes: the bounded wait must give up after `limit_ns`,
// record its code in the status word and let the kernel end normally.
__global__ void selftest_wait_kernel(unsigned long long limit_ns)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
    }
    __syncwarp();
    mbar_wait_bounded(&bar, 0, kStatSelfTest, limit_ns);
}

}  // namespace adkv

ADKV_DEFINE_TU_STATUS(adkv_tu_status_capi)

extern "C" {

int adkv_abi_version(void) { return ADKV_ABI_VERSION; }

const char *adkv_strerror(int code)
{
    switch (code) {
    case 0: return "success";
    case ADKV_E_NULL: return "adkv: a required pointer is NULL";
    case ADKV_E_HEAD_DIM: return "adkv: head dim not supported (128, 256 or 512; checkpointed and device-length decode: 128)";
    case ADKV_E_BITS: return "adkv: bits must be 2 or 4";
    case ADKV_E_SHAPE: return "adkv: invalid sizes (negative, Hq not a multiple of Hkv, or group size not in {1,2,4,8}; {1,2} for head dims 256/512)";
    case ADKV_E_CAPACITY: return "adkv: cache capacity too small for the tokens to be written";
    case ADKV_E_ALIGN: return "adkv: pointer not sufficiently aligned (cache 16 bytes, fp16 rows 8 bytes)";
    case ADKV_E_START: return "adkv: t_start > 0 needs a tail state";
    case ADKV_E_SCRATCH: return "adkv: scratch memory too small for this problem";
    case ADKV_E_FLAGS:
        return "adkv: flag or optional argument not available in this combination (tail states need both tensors and "
               "the fp32 arithmetic)";
    case ADKV_E_STATIC_MAX:
        return "adkv: problem needs more than the 16 MiB of built-in scratch (ADKV_STATIC_SCRATCH_BYTES); use "
               "adkv_decode_attn_ckpt with caller-owned scratch, or a larger checkpoint interval";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "adkv: unknown error";
    }
}

int adkv_device_status(int *status, void *stream)
{
    if (!status) return ADKV_E_NULL;
    const cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return int(e);
    int a = 0, b = 0, c = 0, d = 0, w = 0, t = 0, hf = 0, nr = 0;
    if (int rc = adkv_tu_status_fused(&a)) return rc;
    if (int rc = adkv_tu_status_unfused(&b)) return rc;
    if (int rc = adkv_tu_status_encode(&c)) return rc;
    if (int rc = adkv_tu_status_split(&d)) return rc;
    if (int rc = adkv_tu_status_wide(&w)) return rc;
    if (int rc = adkv_tu_status_capi(&t)) return rc;
    if (int rc = adkv_tu_status_half(&hf)) return rc;
    if (int rc = adkv_tu_status_narrow(&nr)) return rc;
    *status = a ? a : (b ? b : (c ? c : (d ? d : (w ? w : (hf ? hf : (nr ? nr : t))))));
    return 0;
}

int adkv_selftest_wait_timeout(int limit_ms, void *stream)
{
    if (limit_ms <= 0 || limit_ms > 2000) return ADKV_E_SHAPE;
    adkv::selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(1000000ull * (unsigned long long)limit_ms);
    return adkv::launch_status();
}

}  // extern "C"
