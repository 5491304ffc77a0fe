/* adkv_b200 -- C ABI of the B200 (sm_100a) ADKV hot path.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless stated, every
 * call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 * default stream) and performs no host synchronisation and no allocation.  The library
 * never keeps a pointer across calls: the caller owns and may replace the caches between
 * calls (the reference's cache object reallocates them as they grow,
 * src/adkv/hf/llama_adkv.py:104-123).
 *
 * Return value: 0 on success, < 0 for an argument error (ADKV_E_*), > 0 for a CUDA runtime
 * error code (cudaError_t) raised by the launch.  adkv_strerror() gives text for both.
 *
 * Head dims: D = 128, 256 or 512, as in the reference (src/adkv/hf/llama_adkv.py:97-99).
 *
 * Packed cache layout (src/adkv/kernel/gemv.cu:502-510 for 4 bits): per (batch, kv head) a
 * row-major array uint32[n_super_cap][D]; word (sg, c) holds the codes of channel c for the
 * tokens of supergroup sg, token j of the supergroup in bits [bits*j, bits*j+bits) stored as
 * code - lower_limit (4-bit: q + 8, 8 tokens per word; 2-bit: q + 2, 16 tokens per word --
 * the 2-bit layout has no counterpart in the reference).  As a uint8 tensor this is the
 * reference's [B, H, n_super_cap, D/4, 4, 4] tile.
 *
 * Arithmetic: the fp32 recurrence of src/adkv/train/train_model.py:6-22, 70-81 (the
 * reference's torch/Triton definition), evaluated with one rounding per operation in that
 * order ("canonical").  ADKV_FLAG_FAST_REPLAY lets the decode kernels replay the cached
 * tokens with fused multiply-adds instead (zp = fma(alpha, q*s, zp), s = clamp(s * fma(beta, |q|, 1 - beta*target))): attention
 * outputs stay within tolerance, and an appended code may differ from the canonical one by
 * one step in rare cases.  ADKV_FLAG_HALF_STATE selects the OTHER arithmetic the reference has: the fp16 state of
 * its CUDA kernels (src/adkv/kernel/gemv.cu:150-164), bit-compatible with caches those kernels wrote.
 */
#ifndef ADKV_B200_H
#define ADKV_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#define ADKV_ABI_VERSION 2

/* argument errors */
#define ADKV_E_NULL      (-1)  /* a required pointer is NULL */
#define ADKV_E_HEAD_DIM  (-2)  /* D is not 128, 256 or 512 (the _ckpt, _varlen and _static entry points: 128 only) */
#define ADKV_E_BITS      (-3)  /* bits is not 2 or 4 */
#define ADKV_E_SHAPE     (-4)  /* negative size, Hq not a multiple of Hkv, or Hq/Hkv not in {1,2,4,8} ({1,2} for D > 128) */
#define ADKV_E_CAPACITY  (-5)  /* the cache has no room for the tokens to be written */
#define ADKV_E_ALIGN     (-6)  /* a pointer is not 16-byte aligned */
#define ADKV_E_START     (-7)  /* chunked encode: t_start given without a tail state */
#define ADKV_E_SCRATCH   (-8)  /* the scratch memory given is smaller than the problem needs */
#define ADKV_E_STATIC_MAX (-9) /* problem needs more than ADKV_STATIC_SCRATCH_BYTES of built-in scratch */
#define ADKV_E_FLAGS     (-10) /* a flag or optional argument is not available in this combination (tail states with
                                  ADKV_FLAG_HALF_STATE; only one of the two tail states given) */

/* Size of the library's built-in scratch array (see adkv_decode_attn_ckpt_static). */
#define ADKV_STATIC_SCRATCH_BYTES (16u << 20)

/* flags */
#define ADKV_FLAG_FAST_REPLAY 1u  /* decode kernels: contracted (FMA) replay of cached tokens */
/* The arithmetic of the reference's own CUDA kernels instead of the fp32 definition: recurrence state and
 * constants in fp16, zp <- fma(alpha, q*sc, zp), sc <- sc * fma(beta, |q|, 1 - beta*target), no eps guard, no
 * scale clamp (scale_min / scale_max are ignored, as they are there), quantiser in fp32
 * (src/adkv/kernel/gemv.cu:150-164).  Codes, appended codes and tail states are bit-identical to what the
 * reference's encode_kv / forward_qk / forward_ov produce, so caches can be exchanged with them; logits and
 * outputs are accumulated more accurately than there (fp32 across tokens) and agree within fp16 accumulation
 * error.  Takes precedence over ADKV_FLAG_FAST_REPLAY.  Available in every entry point that takes flags, for the
 * head dims that entry point serves. */
#define ADKV_FLAG_HALF_STATE 2u
/* Decode entry points with tail states: quantise the new token with the tail, but leave the tail as it is instead
 * of advancing it over that token.  The call can then be repeated with the same T (the appended code overwrites
 * itself): benchmarks that time one step over and over, and callers that may still reject the token. */
#define ADKV_FLAG_TAIL_KEEP 4u
/* adkv_decode_attn, head dim 128, fp32 arithmetic: how the channels of a head are laid over warps.  By default the
 * library decides from the number of (batch, kv head) streams of the call: a launch with very few streams (about
 * one per SM or fewer) splits every head over two K warps and two V warps so that the GPU has more warps to
 * interleave; larger launches keep one warp per tensor and stream, which needs fewer instructions in all.  Results agree up to the summation order of the logits.  These two flags force one
 * or the other (tests, tuning); with both set, SPLIT wins. */
#define ADKV_FLAG_SPLIT_CHANNELS 8u
#define ADKV_FLAG_NO_SPLIT_CHANNELS 16u
/* Self-test of the failure path of adkv_decode_attn_ckpt (no counterpart in the reference): the K warps return at
 * once, so every V warp waits for logits that never come.  Each wait gives up after its 1 s limit, the kernels end
 * normally, adkv_device_status reports 3, nothing is appended, and every element of `out` is NaN -- a segment that
 * could not be finished marks its partial result instead of leaving whatever the scratch memory held. */
#define ADKV_FLAG_SELFTEST_MUTE_K 0x80000000u

/* The five per-(kv head, channel) parameter tensors, fp16 [Hkv, D] each
 * (src/adkv/hf/llama_adkv.py:27: zp_init, scale_init, alpha, beta, quant_target). */
typedef struct adkv_params {
    const void *zp_init;
    const void *scale_init;
    const void *alpha;
    const void *beta;
    const void *target;
} adkv_params;

int adkv_abi_version(void);
const char *adkv_strerror(int code);

/* Prefill quantise + pack.  Replaces encode_kv (src/adkv/kernel/gemv.cu:368-414, called from
 * src/adkv/hf/llama_adkv.py:144-153).
 *   cache  uint32 [B, H, n_super_cap, D]   written for tokens [t_start, t_start+T)
 *   x      fp16   [B, H, T, D]
 *   tail   float  [B, H, 2, D] (zp then scale) or NULL.  When given it receives the state after
 *          the last token; with t_start > 0 it must hold the state after token t_start-1 on
 *          entry (chunked prefill, which the reference cannot do: llama_adkv.py:195-197).
 * With t_start == 0 the recurrence starts from (zp_init, scale_init) and the unused fields of
 * the last written word are zeroed (gemv.cu:243, 300-305). */
int adkv_encode(void *cache, const void *x, const adkv_params *p, void *tail,
                int B, int H, int T, int D, int n_super_cap, int bits, int t_start,
                float scale_min, float scale_max, void *stream);

/* The same for K and V of one layer in ONE launch (twice the streams in flight: the quantiser is bound by
 * its token-sequential chain, not by bandwidth).  Replaces the pair of encode_kv calls of
 * src/adkv/hf/llama_adkv.py:144-153.  Both tensors share shapes, bits, t_start and clamp bounds. */
int adkv_encode_kv(void *k_cache, const void *k, const adkv_params *kp, void *k_tail,
                   void *v_cache, const void *v, const adkv_params *vp, void *v_tail,
                   int B, int H, int T, int D, int n_super_cap, int bits, int t_start,
                   float scale_min, float scale_max, void *stream);

/* Single-token append from a persisted tail state (no replay).  No direct counterpart in the
 * reference, whose append happens inside forward_qk/forward_ov after a full replay
 * (src/adkv/kernel/gemv.cu:91-146, 744-764); same arithmetic, same slot.
 *   x_new fp16 [B, H, D]; tail float [B, H, 2, D] in/out; T = index of the token written. */
int adkv_append(void *cache, const void *x_new, const adkv_params *p, void *tail,
                int B, int H, int T, int D, int n_super_cap, int bits,
                float scale_min, float scale_max, void *stream);

/* adkv_append for K and V of one layer in one launch. */
int adkv_append_kv(void *k_cache, const void *k_new, const adkv_params *kp, void *k_tail,
                   void *v_cache, const void *v_new, const adkv_params *vp, void *v_tail,
                   int B, int H, int T, int D, int n_super_cap, int bits,
                   float scale_min, float scale_max, void *stream);

/* K and V of one layer for the layered calls below.  `k` / `v`: the fp16 tokens to quantise ([B, H, T, D] for prefill,
 * [B, H, D] for an append); tails as in adkv_encode / adkv_append (required for an append). */
typedef struct adkv_layer_kv {
    void *k_cache; const void *k; adkv_params kp; void *k_tail;
    void *v_cache; const void *v; adkv_params vp; void *v_tail;
} adkv_layer_kv;

/* adkv_encode_kv / adkv_append_kv for several layers at once: `layers` is a HOST array of n_layers descriptors, all
 * layers share shapes, bits and clamp bounds, and K and V of up to 8 layers go into one launch.  No counterpart in the
 * reference, which quantises one tensor per call (src/adkv/hf/llama_adkv.py:144-153).  For callers that hold the
 * fp16 K/V of many layers at once -- converting an existing fp16 cache, or appending the token of a step to every
 * layer's cache after the layers have run: the quantiser is bound by its token-sequential chain and by launch
 * overhead, not by bandwidth, so more independent streams per launch and fewer launches are what it needs. */
int adkv_encode_kv_layers(const adkv_layer_kv *layers, int n_layers, int B, int H, int T, int D, int n_super_cap,
                          int bits, int t_start, float scale_min, float scale_max, void *stream);
int adkv_append_kv_layers(const adkv_layer_kv *layers, int n_layers, int B, int H, int T, int D, int n_super_cap,
                          int bits, float scale_min, float scale_max, void *stream);

/* The general forms of prefill and append: adkv_encode_kv(_ckpt) / adkv_append_kv(_ckpt) with a `flags` argument
 * (ADKV_FLAG_HALF_STATE selects the arithmetic of the reference's CUDA kernels; with 0 they are the calls above and
 * below).  v_cache == NULL: one tensor only (the K arguments; no checkpoints then).  interval == 0: no state
 * checkpoints (k_ckpt / v_ckpt ignored); otherwise as adkv_encode_kv_ckpt / adkv_append_kv_ckpt.  Tail and
 * checkpoints keep their float formats in both arithmetics (fp16 state values are stored exactly). */
int adkv_encode_kv_flags(void *k_cache, const void *k, const adkv_params *kp, void *k_tail, void *k_ckpt,
                         void *v_cache, const void *v, const adkv_params *vp, void *v_tail, void *v_ckpt,
                         int interval, int n_ckpt_cap, int B, int H, int T, int D, int n_super_cap, int bits,
                         int t_start, float scale_min, float scale_max, unsigned flags, void *stream);
int adkv_append_kv_flags(void *k_cache, const void *k_new, const adkv_params *kp, void *k_tail, void *k_ckpt,
                         void *v_cache, const void *v_new, const adkv_params *vp, void *v_tail, void *v_ckpt,
                         int interval, int n_ckpt_cap, int B, int H, int T, int D, int n_super_cap, int bits,
                         float scale_min, float scale_max, unsigned flags, void *stream);

/* q.K^T over the packed cache + append of k_new as token T + self logit.  Replaces forward_qk
 * (src/adkv/kernel/gemv.cu:883-939, called from src/adkv/hf/llama_adkv.py:264).
 *   q fp16 [B, Hq, D]; k_cache [B, Hkv, n_super_cap, D] words; k_new fp16 [B, Hkv, D];
 *   logits fp16 [B, Hq, T+1] (unscaled, unmasked; entry T is the dequantised new token's). */
int adkv_forward_qk(const void *q, void *k_cache, const void *k_new, const adkv_params *p, void *logits,
                    int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits,
                    float scale_min, float scale_max, unsigned flags, void *stream);

/* P.V over the packed cache + append of v_new as token T + self term.  Replaces forward_ov
 * (src/adkv/kernel/gemv.cu:1233-1288, called from src/adkv/hf/llama_adkv.py:273).
 *   attn fp16 [B, Hq, T+1]; v_cache words; v_new fp16 [B, Hkv, D]; out fp16 [B, Hq, D]. */
int adkv_forward_ov(const void *attn, void *v_cache, const void *v_new, const adkv_params *p, void *out,
                    int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits,
                    float scale_min, float scale_max, unsigned flags, void *stream);

/* Fused decode step: q.K^T, * scaling, + mask, softmax, P.V, both appends, one launch.  Replaces the
 * sequence forward_qk -> torch softmax -> forward_ov of src/adkv/hf/llama_adkv.py:263-276.
 *   mask float [B, T+1] additive, shared by all heads (row stride mask_stride_b elements), or NULL.
 *   out  fp16 [B, Hq, D].
 *   k_tail, v_tail  float [B, Hkv, 2, D] (zp then scale), both or neither; in/out.  The reference keeps no
 *          state between steps: its kernels replay the cache and quantise the new token with whatever state
 *          the replay ends in (src/adkv/kernel/gemv.cu:744-764), which ties the replay to the encoder's exact
 *          arithmetic.  With tail states -- the state after token T-1 as adkv_encode* / adkv_append* / the
 *          previous decode step left it -- the new token is quantised from the tail (bit-identical to the
 *          encoder, in O(1)), the tail advances to the state after token T, and the replay of tokens [0, T)
 *          only feeds the attention sums, so ADKV_FLAG_FAST_REPLAY then costs no exactness of the stored codes.
 *          Not available with ADKV_FLAG_HALF_STATE (ADKV_E_FLAGS): that arithmetic is the encoder's own. */
int adkv_decode_attn(const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new,
                     const adkv_params *kp, const adkv_params *vp, void *k_tail, void *v_tail,
                     const void *mask, long long mask_stride_b,
                     void *out, int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits,
                     float scaling, float scale_min, float scale_max, unsigned flags, void *stream);

/* adkv_decode_attn (tail states as there) with per-sequence token counts held on the device: seq_lens int32 [B];
 * sequence b attends over its tokens [0, seq_lens[b]) and appends its new token at seq_lens[b].  No counterpart in the reference
 * (one host integer T for the whole batch, src/adkv/kernel/gemv.py:25).  Serves ragged batches without padding
 * masks, and -- because no argument changes from step to step when the caller increments seq_lens on the
 * device -- a launch that is replayed unchanged.  A length that does not fit the cache cannot be rejected on
 * the host: that stream is skipped and adkv_device_status reports 6. */
int adkv_decode_attn_varlen(const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new,
                            const adkv_params *kp, const adkv_params *vp, void *k_tail, void *v_tail,
                            const void *seq_lens, void *out,
                            int B, int Hq, int Hkv, int D, int n_super_cap, int bits, float scaling,
                            float scale_min, float scale_max, unsigned flags, void *stream);

/* ---- State checkpoints (opt-in; no counterpart in the reference's code, proposed in its paper for long
 * contexts).  A checkpoint tensor float [B, H, n_ckpt_cap, 2, D] per cache holds, in entry k, the recurrence
 * state (zp then scale) before token (k+1)*interval; `interval` is a multiple of 32.  With them the token
 * axis splits into independent segments: 8 bytes per channel per `interval` tokens buy `T/interval + 1`
 * times the parallelism, which is what small-batch long-context decode lacks. */

/* adkv_encode_kv that also writes every checkpoint reached in [t_start, t_start+T]. */
int adkv_encode_kv_ckpt(void *k_cache, const void *k, const adkv_params *kp, void *k_tail, void *k_ckpt,
                        void *v_cache, const void *v, const adkv_params *vp, void *v_tail, void *v_ckpt,
                        int interval, int n_ckpt_cap, int B, int H, int T, int D, int n_super_cap, int bits,
                        int t_start, float scale_min, float scale_max, void *stream);

/* adkv_append_kv that also writes the checkpoint when token T completes an interval. */
int adkv_append_kv_ckpt(void *k_cache, const void *k_new, const adkv_params *kp, void *k_tail, void *k_ckpt,
                        void *v_cache, const void *v_new, const adkv_params *vp, void *v_tail, void *v_ckpt,
                        int interval, int n_ckpt_cap, int B, int H, int T, int D, int n_super_cap, int bits,
                        float scale_min, float scale_max, void *stream);

/* Bytes of scratch adkv_decode_attn_ckpt needs (negative: ADKV_E_*). */
long long adkv_decode_attn_ckpt_scratch_bytes(int B, int Hq, int Hkv, int T, int interval);

/* adkv_decode_attn over a checkpointed cache: one K/V warp pair per (stream, segment), partial results in
 * `scratch` (caller-owned device memory of at least adkv_decode_attn_ckpt_scratch_bytes, 16-byte aligned,
 * contents irrelevant on entry), then a merge kernel.  Appends token T to both caches and writes the
 * checkpoint when T completes an interval.  Same result as adkv_decode_attn up to fp32 summation order.
 * k_tail / v_tail as in adkv_decode_attn; with them the checkpoint written is the advanced tail. */
int adkv_decode_attn_ckpt(const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new,
                          const adkv_params *kp, const adkv_params *vp, void *k_tail, void *v_tail,
                          void *k_ckpt, void *v_ckpt, int interval,
                          int n_ckpt_cap, const void *mask, long long mask_stride_b, void *out, void *scratch,
                          long long scratch_bytes, int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits,
                          float scaling, float scale_min, float scale_max, unsigned flags, void *stream);

/* adkv_decode_attn_ckpt for callers that cannot allocate device memory.  (No counterpart in the reference:
 * its wrappers allocate with torch inside every call.)  Meant for hosts whose HBM is entirely owned by their
 * own pool, or that only ever receive device pointers and have no allocator to call: inputs and outputs are
 * still the caller's, but the partial results go to a fixed array inside the library instead of a `scratch`
 * argument, and the call itself allocates nothing (no cudaMalloc/cudaFree, no allocating library routine).
 *   - Limit: adkv_decode_attn_ckpt_scratch_bytes(B, Hq, Hkv, T, interval) must not exceed
 *     ADKV_STATIC_SCRATCH_BYTES (16 MiB, i.e. B*Hq*(T/interval+1) <= 31775); larger problems return
 *     ADKV_E_STATIC_MAX and launch nothing.  The array is resident on every GPU the process uses, from
 *     library load to exit, whether or not this entry point is ever called.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current); make that first call outside any stream capture.  Later calls only launch.
 *   - All calls on a device share the one array, and it keeps whatever the previous call wrote.  Nothing in it
 *     needs clearing (every slot read is written first within the call), but two calls that overlap on the
 *     GPU -- different streams, or different host threads -- race on it: serialise them. */
int adkv_decode_attn_ckpt_static(const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new,
                                 const adkv_params *kp, const adkv_params *vp, void *k_tail, void *v_tail,
                                 void *k_ckpt, void *v_ckpt,
                                 int interval, int n_ckpt_cap, const void *mask, long long mask_stride_b, void *out,
                                 int B, int Hq, int Hkv, int T, int D, int n_super_cap, int bits, float scaling,
                                 float scale_min, float scale_max, unsigned flags, void *stream);

/* Reads and clears the device-side status word of the current device (HOST pointer `status`;
* synchronises `stream`).  Non-zero means a kernel gave up on a bounded wait (1-5: which wait) or skipped a
 * stream whose device-side length did not fit the cache (6).  Intended for tests and diagnostics, not for the hot path. */
int adkv_device_status(int *status, void *stream);

/* Self-test of the bounded waits (no counterpart in the reference): launches one warp that waits on a barrier
 * nothing will ever complete.  The wait gives up after limit_ms (1..2000), the kernel ends normally, and
 * adkv_device_status then reports 7.  Every wait in the library's kernels uses the same routine with a 1 s
 * limit, so a lost copy or a missing partner ends as a status code, not as a hang. */
int adkv_selftest_wait_timeout(int limit_ms, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ADKV_B200_H */
