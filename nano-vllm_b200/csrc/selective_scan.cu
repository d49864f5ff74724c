// Selective-scan (Mamba-1) recurrence with per-sequence state slots.
//
// Per channel c and state n, with u the convolved + SiLU'd input, dt = softplus(dt_raw + bias), A = -exp(A_log) (given):
//     S[c, n] <- exp(dt_c * A[c, n]) * S[c, n] + dt_c * u_c * B_n ;   y_c = sum_n S[c, n] * C_n + D_c * u_c ;   out = y * silu(z)
// A sequence owns one slot: its fp32 state S [channels, state] and the last (taps - 1) inputs of the causal convolution.
// A step whose sequence has no tokens behind it starts from zeros whatever the slot holds, so a slot needs no clearing
// when it changes hands.
//
//   causal_conv_kernel      : depthwise causal convolution + bias + SiLU over a varlen batch, history taken from the slot
//   conv_state_update_kernel: the slot's history after the step (run after the convolution: it overwrites what that reads)
//   selective_scan_kernel   : the recurrence, serial over a sequence's tokens, 4 lanes per channel holding the state in
//                             registers; one token per sequence is the decode case of the same kernel
#include "mix_common.cuh"

namespace {

// conv_state: [slots, taps - 1, channels] fp32, row taps-2 is the newest input.
template <typename T>
__global__ void __launch_bounds__(256) causal_conv_kernel(const T* __restrict__ x, int64_t x_stride, const T* __restrict__ w,
                                                          const T* __restrict__ bias, const float* __restrict__ conv_state,
                                                          const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q,
                                                          const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens,
                                                          T* __restrict__ out, int channels, int taps, int tok_tile) {
    B200_PDL_SYNC();
    const int s = blockIdx.z;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    const int i0 = blockIdx.y * tok_tile;
    if (i0 >= sp.qlen) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const bool has_hist = sp.klen - sp.qlen > 0;
    const float* hist = conv_state + (int64_t)state_slots[s] * (taps - 1) * channels;
    const float b = bias ? ldf(bias + c) : 0.f;
    const int i1 = min(sp.qlen, i0 + tok_tile);
    for (int i = i0; i < i1; ++i) {
        float a = b;
        for (int k = 0; k < taps; ++k) {
            const int m = i - (taps - 1 - k);              // local index of the input under tap k (the last tap is token i)
            float v = 0.f;
            if (m >= 0) v = ldf(x + (int64_t)(sp.q0 + m) * x_stride + c);
            else if (has_hist) v = hist[(int64_t)(taps - 1 + m) * channels + c];
            a = fmaf(ldf(w + (int64_t)c * taps + k), v, a);
        }
        stf(out + (int64_t)(sp.q0 + i) * channels + c, siluf_(a));
    }
}

template <typename T>
__global__ void __launch_bounds__(256) conv_state_update_kernel(const T* __restrict__ x, int64_t x_stride, float* __restrict__ conv_state,
                                                                const int32_t* __restrict__ state_slots,
                                                                const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k,
                                                                const int32_t* __restrict__ ctx_lens, int channels, int taps) {
    B200_PDL_SYNC();
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen <= 0) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const bool has_hist = sp.klen - sp.qlen > 0;
    float* hist = conv_state + (int64_t)state_slots[s] * (taps - 1) * channels;
    for (int j = 0; j < taps - 1; ++j) {                   // ascending: row j reads row j + qlen > j of the old history
        const int m = sp.qlen - (taps - 1) + j;
        float v = 0.f;
        if (m >= 0) v = ldf(x + (int64_t)(sp.q0 + m) * x_stride + c);
        else if (has_hist) v = hist[(int64_t)(taps - 1 + m) * channels + c];
        hist[(int64_t)j * channels + c] = v;
    }
}

__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

constexpr int SCAN_LANES = 4;          // lanes that share one channel's state
constexpr int SCAN_CH = 32;            // channels per CTA (128 threads)

// NPL states per lane: state n = k * SCAN_LANES + sub, k < NPL.
template <typename T, int NPL>
__global__ void __launch_bounds__(SCAN_LANES * SCAN_CH) selective_scan_kernel(
    const T* __restrict__ u,            // [n, channels]
    const T* __restrict__ dt_raw,       // [n, channels]
    const T* __restrict__ dt_bias,      // [channels]
    const float* __restrict__ A,        // [channels, nstate]  (negative)
    const T* __restrict__ Bm, const T* __restrict__ Cm, int64_t bc_stride,   // [n, nstate] with a row stride
    const T* __restrict__ Dv,           // [channels]
    const T* __restrict__ z, int64_t z_stride,                               // [n, channels] with a row stride
    float* __restrict__ state,          // [slots, channels, nstate]
    const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k,
    const int32_t* __restrict__ ctx_lens, T* __restrict__ y, int channels, int nstate) {
    B200_PDL_SYNC();
    const int s = blockIdx.y;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    if (sp.qlen <= 0) return;
    const int sub = threadIdx.x % SCAN_LANES;
    const int c = blockIdx.x * SCAN_CH + threadIdx.x / SCAN_LANES;
    const bool live = c < channels;
    const int cc = live ? c : channels - 1;
    float* st = state + ((int64_t)state_slots[s] * channels + cc) * nstate;
    const bool has_hist = sp.klen - sp.qlen > 0;
    float S[NPL], a[NPL];
#pragma unroll
    for (int k = 0; k < NPL; ++k) {
        const int n = k * SCAN_LANES + sub;
        S[k] = (has_hist && n < nstate) ? st[n] : 0.f;
        a[k] = n < nstate ? A[(int64_t)cc * nstate + n] : 0.f;
    }
    const float bias = ldf(dt_bias + cc), dskip = ldf(Dv + cc);
    for (int i = 0; i < sp.qlen; ++i) {
        const int64_t t = sp.q0 + i;
        const float uu = ldf(u + t * channels + cc);
        const float dt = softplusf_(ldf(dt_raw + t * channels + cc) + bias);
        const float du = dt * uu;
        float part = 0.f;
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            const int n = k * SCAN_LANES + sub;
            if (n < nstate) {
                S[k] = fmaf(expf(dt * a[k]), S[k], du * ldf(Bm + t * bc_stride + n));
                part = fmaf(S[k], ldf(Cm + t * bc_stride + n), part);
            }
        }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        if (live && sub == 0) {
            const float zz = ldf(z + t * z_stride + cc);
            stf(y + t * channels + cc, (part + dskip * uu) * siluf_(zz));
        }
    }
    if (live) {
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            const int n = k * SCAN_LANES + sub;
            if (n < nstate) st[n] = S[k];
        }
    }
}

}  // namespace

extern "C" int b200m_causal_conv(const void* x, int64_t x_stride, const void* w, const void* bias, float* conv_state,
                                 const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k, const int32_t* ctx_lens,
                                 void* out, int num_seqs, int max_q, int channels, int taps, int is32, void* stream) {
    if (!x || !w || !conv_state || !state_slots || !out || channels <= 0 || taps <= 0) return B200_EINVAL;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (num_seqs <= 0 || max_q <= 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int tok_tile = 16;
    dim3 grid((channels + 255) / 256, (max_q + tok_tile - 1) / tok_tile, num_seqs);
    B200M_DISPATCH(is32, B200_LAUNCH((causal_conv_kernel<T>), grid, 256, 0, st, static_cast<const T*>(x), x_stride,
                                     static_cast<const T*>(w), static_cast<const T*>(bias), conv_state, state_slots, cu_q, cu_k,
                                     ctx_lens, static_cast<T*>(out), channels, taps, tok_tile));
    int rc = b200_launch_status(nullptr);
    if (rc != B200_OK || taps == 1) return rc;
    dim3 grid2((channels + 255) / 256, num_seqs);
    B200M_DISPATCH(is32, B200_LAUNCH((conv_state_update_kernel<T>), grid2, 256, 0, st, static_cast<const T*>(x), x_stride,
                                     conv_state, state_slots, cu_q, cu_k, ctx_lens, channels, taps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_selective_scan(const void* u, const void* dt_raw, const void* dt_bias, const float* A, const void* Bm,
                                    const void* Cm, int64_t bc_stride, const void* Dv, const void* z, int64_t z_stride,
                                    float* state, const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k,
                                    const int32_t* ctx_lens, void* y, int num_seqs, int channels, int nstate, int is32,
                                    void* stream) {
    if (!u || !dt_raw || !dt_bias || !A || !Bm || !Cm || !Dv || !z || !state || !state_slots || !y) return B200_EINVAL;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (channels <= 0 || nstate <= 0) return B200_EINVAL;
    if (nstate > 32 * SCAN_LANES) return B200_EUNSUPPORTED;
    if (num_seqs <= 0) return B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((channels + SCAN_CH - 1) / SCAN_CH, num_seqs);
#define SCAN_GO(N)                                                                                                             \
    B200M_DISPATCH(is32, B200_LAUNCH((selective_scan_kernel<T, N>), grid, SCAN_LANES * SCAN_CH, 0, st, static_cast<const T*>(u), \
                                     static_cast<const T*>(dt_raw), static_cast<const T*>(dt_bias), A, static_cast<const T*>(Bm), \
                                     static_cast<const T*>(Cm), bc_stride, static_cast<const T*>(Dv), static_cast<const T*>(z),  \
                                     z_stride, state, state_slots, cu_q, cu_k, ctx_lens, static_cast<T*>(y), channels, nstate))
    const int npl = (nstate + SCAN_LANES - 1) / SCAN_LANES;
    if (npl <= 2) SCAN_GO(2);
    else if (npl <= 4) SCAN_GO(4);
    else if (npl <= 8) SCAN_GO(8);
    else if (npl <= 16) SCAN_GO(16);
    else SCAN_GO(32);
#undef SCAN_GO
    return b200_launch_status(nullptr);
}
