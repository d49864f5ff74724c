// Row-wise pieces of a hybrid decoder layer: embedding into an fp32 residual stream, the residual update fused with a
// weight-only layer norm, RMS norm of a projection output, and the feed-forward activations.
#include "mix_common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) embed_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table,
                                                            float* __restrict__ out, T* __restrict__ copy, int width, int64_t vocab) {
    B200_PDL_SYNC();
    const int row = blockIdx.x;
    int64_t id = ids[row];
    if (id < 0 || id >= vocab) id = 0;
    const T* src = table + id * width;
    float* dst = out + (int64_t)row * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const T v = src[c];
        dst[c] = ldf(&v);
        if (copy) copy[(int64_t)row * width + c] = v;
    }
}

// Norm on a sublayer's OUTPUT, then the residual update:  x[row] += mult * y[row] / sqrt(mean(y^2) + eps) * (w_offset + w).
// y is the branch output in the activation type, or (y32) in fp32.  `copy`, when given, receives the updated row in the
// activation type: the operand of the next sublayer's projections, which read the stream itself.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) add_normed_kernel(float* __restrict__ x, const T* __restrict__ y,
                                                                 const float* __restrict__ y32, const T* __restrict__ w, float mult,
                                                                 float w_offset, T* __restrict__ copy, int cols, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[ROW_THREADS / 32];
    const int64_t base = (int64_t)blockIdx.x * cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = y32 ? y32[base + c] : ldf(y + base + c);
        q = fmaf(v, v, q);
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)cols + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = y32 ? y32[base + c] : ldf(y + base + c);
        const float r = fmaf(mult, v * rstd * (w_offset + ldf(w + c)), x[base + c]);
        x[base + c] = r;
        if (copy) stf(copy + base + c, r);
    }
}

// out[i] = x[row] / sqrt(mean(x[row]^2) + eps) * (w_offset + w) for row = rows_idx[i] (or i) of an fp32 stream.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows_idx,
                                                                   const T* __restrict__ w, float w_offset, T* __restrict__ out,
                                                                   int cols, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[ROW_THREADS / 32];
    const int64_t row = rows_idx ? rows_idx[blockIdx.x] : blockIdx.x;
    const float* xr = x + row * cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) q = fmaf(xr[c], xr[c], q);
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)cols + eps);
    T* o = out + (int64_t)blockIdx.x * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) stf(o + c, xr[c] * rstd * (w_offset + ldf(w + c)));
}

// x[row] += (a[row] + b[row] + b32[row])  (each term optional), then out[i] = LN(x[row]) * w, where the statistics are the
// mean and the mean of squared deviations of the updated row.  rows_idx (optional) names the rows to normalise: the
// update is then skipped (it must have happened already) and out has one row per index.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) add_layernorm_kernel(float* __restrict__ x, const T* __restrict__ a,
                                                                    const T* __restrict__ b, const float* __restrict__ b32,
                                                                    const T* __restrict__ w, T* __restrict__ out,
                                                                    const int32_t* __restrict__ rows_idx, int cols, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[ROW_THREADS / 32];
    const int orow = blockIdx.x;
    const int64_t row = rows_idx ? rows_idx[orow] : orow;
    float* xr = x + row * cols;
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float v = xr[c];
        if (!rows_idx && (a || b || b32)) {
            float d = 0.f;
            if (a) d += ldf(a + row * cols + c);
            if (b) d += ldf(b + row * cols + c);
            if (b32) d += b32[row * cols + c];
            v += d;
            xr[c] = v;
        }
        s += v;
    }
    if (out == nullptr) return;
    const float mean = block_sum(s, red) / (float)cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {      // same thread wrote these elements: no fence needed
        const float d = xr[c] - mean;
        q = fmaf(d, d, q);
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)cols + eps);
    T* o = out + (int64_t)orow * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) stf(o + c, (xr[c] - mean) * rstd * ldf(w + c));
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_any_kernel(const T* __restrict__ x, int64_t x_stride, const T* __restrict__ w,
                                                                  T* __restrict__ out, int64_t out_stride, int cols, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[ROW_THREADS / 32];
    const T* xr = x + (int64_t)blockIdx.x * x_stride;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = ldf(xr + c);
        q = fmaf(v, v, q);
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)cols + eps);
    T* o = out + (int64_t)blockIdx.x * out_stride;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) stf(o + c, ldf(xr + c) * rstd * ldf(w + c));
}

__device__ __forceinline__ float gelu_tanh_(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// kind 0: x = [gate | up] per row, out = gelu_tanh(gate) * up;  kind 1: out = relu(x)^2 (no second half);
// kind 2: x = [gate | up], out = silu(gate) * up
template <typename T>
__global__ void ff_act_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int n, int kind) {
    B200_PDL_SYNC();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * n) return;
    const int64_t r = i / n;
    const int c = (int)(i - r * n);
    if (kind == 1) {
        const float v = fmaxf(ldf(x + i), 0.f);
        stf(out + i, v * v);
    } else {
        const float g = ldf(x + r * 2 * n + c), u = ldf(x + r * 2 * n + n + c);
        stf(out + i, (kind == 0 ? gelu_tanh_(g) : siluf_(g)) * u);
    }
}

// bf16 rows whose halves are multiples of 8: 8 columns per thread, 128-bit accesses, one row per blockIdx.y
__global__ void __launch_bounds__(256) ff_act_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int n, int kind) {
    B200_PDL_SYNC();
    const int c = (blockIdx.x * 256 + threadIdx.x) << 3;
    if (c >= n) return;
    const int64_t r = blockIdx.y;
    float o[8];
    if (kind == 1) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(x + r * n + c), v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float t = fmaxf(v[e], 0.f);
            o[e] = t * t;
        }
    } else {
        float gt[8], up[8];
        unpack8(*reinterpret_cast<const uint4*>(x + r * 2 * n + c), gt);
        unpack8(*reinterpret_cast<const uint4*>(x + r * 2 * n + n + c), up);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (kind == 0 ? gelu_tanh_(gt[e]) : siluf_(gt[e])) * up[e];
    }
    *reinterpret_cast<uint4*>(out + r * n + c) = pack8(o);
}

}  // namespace

extern "C" int b200m_abi_version(void) { return 2; }

extern "C" int b200m_embed(const int64_t* ids, const void* table, float* out, void* copy, int n, int width, int64_t vocab, int is32,
                           void* stream) {
    if (!ids || !table || !out || n < 0 || width <= 0 || vocab <= 0) return B200_EINVAL;
    if (n == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((embed_kernel<T>), n, ROW_THREADS, 0, static_cast<cudaStream_t>(stream), ids,
                                     static_cast<const T*>(table), out, static_cast<T*>(copy), width, vocab));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_add_normed(float* x, const void* y, const float* y32, const void* w, float mult, float w_offset, void* copy,
                                int rows, int cols, float eps, int is32, void* stream) {
    if (!x || (!y && !y32) || !w || rows < 0 || cols <= 0) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((add_normed_kernel<T>), rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream), x,
                                     static_cast<const T*>(y), y32, static_cast<const T*>(w), mult, w_offset,
                                     static_cast<T*>(copy), cols, eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_rmsnorm_rows(const float* x, const int32_t* rows_idx, const void* w, float w_offset, void* out, int rows,
                                  int cols, float eps, int is32, void* stream) {
    if (!x || !w || !out || rows < 0 || cols <= 0) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((rmsnorm_rows_kernel<T>), rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream), x, rows_idx,
                                     static_cast<const T*>(w), w_offset, static_cast<T*>(out), cols, eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_add_layernorm(float* x, const void* a, const void* b, const float* b32, const void* w, void* out,
                                   const int32_t* rows_idx, int rows, int cols, float eps, int is32, void* stream) {
    if (!x || rows < 0 || cols <= 0 || (out && !w)) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((add_layernorm_kernel<T>), rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream), x,
                                     static_cast<const T*>(a), static_cast<const T*>(b), b32, static_cast<const T*>(w),
                                     static_cast<T*>(out), rows_idx, cols, eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_rmsnorm(const void* x, int64_t x_stride, const void* w, void* out, int64_t out_stride, int rows, int cols,
                             float eps, int is32, void* stream) {
    if (!x || !w || !out || rows < 0 || cols <= 0) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((rmsnorm_any_kernel<T>), rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream),
                                     static_cast<const T*>(x), x_stride, static_cast<const T*>(w), static_cast<T*>(out),
                                     out_stride, cols, eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_ff_act(const void* x, void* out, int64_t rows, int n, int kind, int is32, void* stream) {
    if (!x || !out || rows < 0 || n <= 0 || kind < 0 || kind > 2) return B200_EINVAL;
    if (rows == 0) return B200_OK;
    if (!is32 && n % 8 == 0 && rows <= 65535 * 32 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        for (int64_t r0 = 0; r0 < rows; r0 += 65535) {             // grid.y limit
            const int64_t nr = rows - r0 < 65535 ? rows - r0 : 65535;
            const int64_t in_row = kind == 1 ? n : 2 * (int64_t)n;
            B200_LAUNCH((ff_act_vec_kernel), dim3((n / 8 + 255) / 256, (unsigned)nr), 256, 0, static_cast<cudaStream_t>(stream),
                        static_cast<const __nv_bfloat16*>(x) + r0 * in_row, static_cast<__nv_bfloat16*>(out) + r0 * n, n, kind);
        }
        return b200_launch_status(nullptr);
    }
    const int64_t total = rows * n;
    B200M_DISPATCH(is32, B200_LAUNCH((ff_act_kernel<T>), (unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream),
                                     static_cast<const T*>(x), static_cast<T*>(out), rows, n, kind));
    return b200_launch_status(nullptr);
}
