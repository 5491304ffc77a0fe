// Sink and source of the unfused entry points: logits go to / weights come from fp16 rows in global memory
// (the reference's forward_qk / forward_ov contract, src/adkv/kernel/gemv.py:16-97).
#pragma once
#include "adkv_softmax.cuh"

namespace adkv {

constexpr int kStreamsPerCta = 2;   // unfused kernels: 2 streams per CTA, one warp each

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

template <int G, bool HALF_W = false>
struct GlobalWeightSrc {
    const __half *row[G];   // attention weights of each q head of this stream: [T+1]
    float2 *wts;   // every weight stored twice
    __device__ __forceinline__ bool tile_weights(int i, int ntok, int lane, float (&)[G][4])
    {
#pragma unroll
        for (int g = 0; g < G; ++g)
        {
            const float wv = lane < ntok ? __half2float(row[g][i * kTileTok + lane]) : 0.f;
            put_weight<HALF_W>(wts, g * kTileTok + lane, wv);
        }
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
    __device__ __forceinline__ void store(const VArgs &a, int b, int h, int c0, const float (&acc)[G][4]) const
    {
        store_normalised<G>(*this, a, b, h, c0, acc);
    }
};

}  // namespace adkv
