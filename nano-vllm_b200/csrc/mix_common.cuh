// Shared pieces of libb200mix.so: the sequence-mixing and feed-forward kernels of hybrid decoders (latent attention with
// a softmax sink, selective-scan recurrences, routed experts, weight-only layer norm), for sm_100a.
//
// Every kernel is a template over the activation type T (float or __nv_bfloat16): the bf16 instance is the serving
// path, the float instance keeps every tensor in 32 bits.  What the kernels accumulate (norm statistics, softmax, the
// residual stream, recurrent state, router scores) is fp32 in both.
#pragma once
#include "common.cuh"
#include "b200_mixers.h"

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__device__ __forceinline__ void stf(T* p, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// round-trip through T (what a tensor of type T would hold)
template <typename T>
__device__ __forceinline__ float rnd(float v);
template <>
__device__ __forceinline__ float rnd<float>(float v) { return v; }
template <>
__device__ __forceinline__ float rnd<__nv_bfloat16>(float v) { return round_bf16(v); }

// Per-sequence extent of a step.  Varlen steps (prompt portions, mixed batches) carry cumulative query / key lengths;
// decode steps carry one token per row and the row's total length (0 marks a CUDA-graph padding row).
struct SeqSpan {
    int q0;      // first row of this sequence in the step's token arrays
    int qlen;    // tokens of this step
    int klen;    // tokens after this step (cached + new)
};
__device__ __forceinline__ SeqSpan seq_span(const int32_t* cu_q, const int32_t* cu_k, const int32_t* ctx_lens, int s) {
    SeqSpan r;
    if (cu_q != nullptr) {
        r.q0 = cu_q[s];
        r.qlen = cu_q[s + 1] - r.q0;
        r.klen = cu_k[s + 1] - cu_k[s];
    } else {
        r.q0 = s;
        r.klen = ctx_lens[s];
        r.qlen = r.klen > 0 ? 1 : 0;
    }
    return r;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; ++i) t += red[i];
    return t;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.0f + expf(-x)); }

#define B200M_DISPATCH(is32, ...)              \
    do {                                       \
        if (is32) {                            \
            using T = float;                   \
            __VA_ARGS__;                       \
        } else {                               \
            using T = __nv_bfloat16;           \
            __VA_ARGS__;                       \
        }                                      \
    } while (0)
