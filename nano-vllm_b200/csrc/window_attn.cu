// Grouped-query attention with a sliding window and a linear distance bias over a paged key/value cache.
//
// Per token the cache holds one row [k (G * dim) | v (G * vdim)] per layer that owns a key/value projection; query head h
// reads key/value head h / (H / G).  There is no rotation: position enters through the bias and the window only.
//     s_ij = (q_i . k_j) * scale - slope[h] * (i - j),   visible: 0 <= i - j < window   (window <= 0: every j <= i)
//     p = softmax over the visible j,   out_i = sum_j p_ij v_j
// Softmax statistics and the output accumulate in fp32 in both element types.
//
//   qk_norm_store_kernel : RMS norm of the WHOLE query projection and of the whole key projection (one statistic per token
//                          over all heads, weight per column), queries normalised in place, keys and values scattered to the
//                          token's cache slot
//   window_attn_kernel   : any mix of prompt portions and single tokens on the fp32 FMA pipe (one warp per (token, head),
//                          key/value tiles shared by the warps of a CTA through shared memory)
//   window_attn_mma_kernel (bf16): the same on the tensor cores, 64 (token, head) rows x 64-key tiles, double-buffered
//                          asynchronous copies; single-token steps may split a long window over several CTAs
#include "mix_common.cuh"

namespace {

constexpr int WA_WARPS = 8;
constexpr int WA_TILE = 32;

template <typename T>
__global__ void __launch_bounds__(256) qk_norm_store_kernel(T* __restrict__ qkv, int64_t stride, int q_cols, int k_cols, int v_cols,
                                                            const T* __restrict__ wq, const T* __restrict__ wk,
                                                            const int32_t* __restrict__ slots, T* __restrict__ cache, float eps) {
    B200_PDL_SYNC();
    __shared__ float red[8];
    const int t = blockIdx.x;
    T* x = qkv + (int64_t)t * stride;
    if (wq != nullptr) {
        float q = 0.f;
        for (int c = threadIdx.x; c < q_cols; c += blockDim.x) {
            const float v = ldf(x + c);
            q = fmaf(v, v, q);
        }
        const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)q_cols + eps);
        for (int c = threadIdx.x; c < q_cols; c += blockDim.x) stf(x + c, ldf(x + c) * rstd * ldf(wq + c));
    }
    if (k_cols + v_cols == 0) return;
    const int slot = slots[t];
    if (slot < 0) return;                                  // block-uniform
    T* dst = cache + (int64_t)slot * (k_cols + v_cols);
    const T* k = x + q_cols;
    float rstd = 1.0f;
    if (wk != nullptr) {
        float q = 0.f;
        for (int c = threadIdx.x; c < k_cols; c += blockDim.x) {
            const float v = ldf(k + c);
            q = fmaf(v, v, q);
        }
        rstd = 1.0f / sqrtf(block_sum(q, red) / (float)k_cols + eps);
    }
    for (int c = threadIdx.x; c < k_cols; c += blockDim.x) stf(dst + c, wk ? ldf(k + c) * rstd * ldf(wk + c) : ldf(k + c));
    for (int c = threadIdx.x; c < v_cols; c += blockDim.x) dst[k_cols + c] = k[k_cols + c];
}

// One warp per (token, head-in-group) pair; a CTA covers WA_WARPS consecutive pairs of one sequence and one key/value head.
// OACC = ceil(vdim / 32): output accumulators per lane.
template <typename T, int OACC>
__global__ void __launch_bounds__(WA_WARPS * 32) window_attn_kernel(
    const T* __restrict__ q, int64_t q_stride,        // [total_q, >= H * dim]
    const T* __restrict__ cache, int row_elems, int v_off,
    const int32_t* __restrict__ block_tables, int bt_stride, int block_size,
    const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k, const int32_t* __restrict__ ctx_lens,
    const float* __restrict__ slopes, int window,
    T* __restrict__ out,                              // [total_q, H * vdim]
    int H, int G, int dim, int vdim, float scale) {
    B200_PDL_SYNC();
    extern __shared__ float smem[];
    const int D = dim + vdim;
    const int DS = D | 1;                                  // odd row stride: lanes reading one column of 32 rows hit 32 banks
    float* tile = smem;                                    // [WA_TILE][DS]: k (dim) | v (vdim) of one key/value head
    float* qs = tile + WA_TILE * DS;                       // [WA_WARPS][dim]
    float* pb = qs + WA_WARPS * dim;                       // [WA_WARPS][WA_TILE]
    const int s = blockIdx.y, g = blockIdx.z, rep = H / G;
    const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npairs = sp.qlen * rep;
    const int pair0 = blockIdx.x * WA_WARPS;
    if (pair0 >= npairs) return;
    const int pair = pair0 + warp;
    const bool active = pair < npairs;
    const int i = active ? pair / rep : 0, h = g * rep + (active ? pair % rep : 0);
    const int first = sp.klen - sp.qlen;                   // position of this step's first token
    const int pos = first + i;
    const int i_lo = pair0 / rep, i_hi = min(sp.qlen - 1, (pair0 + WA_WARPS - 1) / rep);
    const int kmax = first + i_hi + 1;                     // keys any warp of this CTA may see: [kmin, kmax)
    const int kmin = window > 0 ? max(0, first + i_lo - window + 1) : 0;
    const int my_lo = window > 0 ? max(0, pos - window + 1) : 0;
    float* myq = qs + warp * dim;
    if (active) {
        const T* qr = q + (int64_t)(sp.q0 + i) * q_stride + (int64_t)h * dim;
        for (int c = lane; c < dim; c += 32) myq[c] = ldf(qr + c) * scale;
    }
    const float slope = (active && slopes) ? slopes[h] : 0.f;
    float m = -INFINITY, l = 0.f;
    float acc[OACC];
#pragma unroll
    for (int k = 0; k < OACC; ++k) acc[k] = 0.f;
    const int32_t* bt = block_tables + (int64_t)s * bt_stride;
    for (int j0 = kmin; j0 < kmax; j0 += WA_TILE) {
        __syncthreads();                                   // previous tile consumed (and the queries written)
        const int rows = min(WA_TILE, kmax - j0);
        for (int e = threadIdx.x; e < rows * D; e += blockDim.x) {
            const int r = e / D, c = e - r * D;
            const int j = j0 + r;
            const int64_t slot = (int64_t)bt[j / block_size] * block_size + (j % block_size);
            const T* src = cache + slot * row_elems;
            tile[r * DS + c] = ldf(c < dim ? src + (int64_t)g * dim + c : src + v_off + (int64_t)g * vdim + (c - dim));
        }
        __syncthreads();
        if (active && j0 <= pos && j0 + rows > my_lo) {    // the tile holds at least one key this row sees
            const int j = j0 + lane;
            const bool valid = lane < rows && j <= pos && j >= my_lo;
            float sc = -INFINITY;
            if (valid) {
                const float* kr = tile + lane * DS;
                float a = 0.f;
                for (int c = 0; c < dim; ++c) a = fmaf(myq[c], kr[c], a);
                sc = a - slope * (float)(pos - j);
            }
            const float m_new = fmaxf(m, warp_max(sc));
            const float alpha = expf(m - m_new);
            const float p = valid ? expf(sc - m_new) : 0.f;
            l = l * alpha + warp_sum(p);
            m = m_new;
            pb[warp * WA_TILE + lane] = p;
            __syncwarp();
            const int r_lo = max(0, my_lo - j0), r_hi = min(rows, pos - j0 + 1);
#pragma unroll
            for (int k = 0; k < OACC; ++k) {
                const int c = lane + 32 * k;
                float a = acc[k] * alpha;
                if (c < vdim)
                    for (int r = r_lo; r < r_hi; ++r) a = fmaf(pb[warp * WA_TILE + r], tile[r * DS + dim + c], a);
                acc[k] = a;
            }
            __syncwarp();
        }
    }
    if (active) {
        const float inv = 1.0f / l;
        T* o = out + ((int64_t)(sp.q0 + i) * H + h) * vdim;
#pragma unroll
        for (int k = 0; k < OACC; ++k) {
            const int c = lane + 32 * k;
            if (c < vdim) stf(o + c, acc[k] * inv);
        }
    }
}

template <typename K>
int wa_ensure_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return B200_OK;
    if (bytes > 227 * 1024) return B200_EUNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) {
        b200_tls_cuda_error() = cudaGetErrorString(e);
        return B200_ECUDA;
    }
    return B200_OK;
}

template <typename T, int OACC>
int launch_window_fma(const void* q, int64_t q_stride, const void* cache, int row_elems, int v_off, const int32_t* block_tables,
                      int bt_stride, int block_size, const int32_t* cu_q, const int32_t* cu_k, const int32_t* ctx_lens,
                      const float* slopes, int window, void* out, int num_seqs, int max_q, int H, int G, int dim, int vdim,
                      float scale, cudaStream_t stream) {
    const int D = dim + vdim;
    const size_t smem = sizeof(float) * ((size_t)WA_TILE * (D | 1) + (size_t)WA_WARPS * dim + WA_WARPS * WA_TILE);
    int rc = wa_ensure_smem(window_attn_kernel<T, OACC>, smem);
    if (rc != B200_OK) return rc;
    dim3 grid((max_q * (H / G) + WA_WARPS - 1) / WA_WARPS, num_seqs, G);
    B200_LAUNCH((window_attn_kernel<T, OACC>), grid, WA_WARPS * 32, smem, stream, static_cast<const T*>(q), q_stride,
                static_cast<const T*>(cache), row_elems, v_off, block_tables, bt_stride, block_size, cu_q, cu_k, ctx_lens, slopes,
                window, static_cast<T*>(out), H, G, dim, vdim, scale);
    return b200_launch_status(nullptr);
}

}  // namespace

extern "C" int b200m_qk_norm_store(void* qkv, int64_t stride, int q_cols, int k_cols, int v_cols, const void* q_norm_w,
                                   const void* k_norm_w, const int32_t* slots, void* cache, int n, float eps, int is32,
                                   void* stream) {
    if (!qkv || n < 0 || q_cols < 0 || k_cols < 0 || v_cols < 0 || stride < q_cols + k_cols + v_cols) return B200_EINVAL;
    if (k_cols + v_cols > 0 && (!slots || !cache)) return B200_EINVAL;
    if (n == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((qk_norm_store_kernel<T>), n, 256, 0, static_cast<cudaStream_t>(stream), static_cast<T*>(qkv),
                                     stride, q_cols, k_cols, v_cols, static_cast<const T*>(q_norm_w),
                                     static_cast<const T*>(k_norm_w), slots, static_cast<T*>(cache), eps));
    return b200_launch_status(nullptr);
}

extern "C" int b200m_window_attention(const void* q, int64_t q_stride, const void* cache, int row_elems, int v_off,
                                      const int32_t* block_tables, int bt_stride, int block_size, const int32_t* cu_q,
                                      const int32_t* cu_k, const int32_t* ctx_lens, const float* slopes, int window, void* out,
                                      int total_q, int num_seqs, int max_q, int num_heads, int num_kv_heads, int dim, int vdim,
                                      float scale, int is32, int flags, int splits, float* part, void* stream) {
    if (!q || !cache || !block_tables || !out || total_q < 0 || num_seqs < 0 || num_heads <= 0 || num_kv_heads <= 0 ||
        num_heads % num_kv_heads || dim <= 0 || vdim <= 0 || block_size <= 0)
        return B200_EINVAL;
    if ((cu_q == nullptr) != (cu_k == nullptr) || (cu_q == nullptr && ctx_lens == nullptr)) return B200_EINVAL;
    if (total_q == 0 || num_seqs == 0 || max_q <= 0) return B200_OK;
    if (vdim > 512) return B200_EUNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    (void)flags;
    (void)splits;
    (void)part;
#define WA_FMA(OACC)                                                                                                             \
    B200M_DISPATCH(is32, return (launch_window_fma<T, OACC>(q, q_stride, cache, row_elems, v_off, block_tables, bt_stride,       \
                                                            block_size, cu_q, cu_k, ctx_lens, slopes, window, out, num_seqs,     \
                                                            max_q, num_heads, num_kv_heads, dim, vdim, scale, st)))
    const int oacc = (vdim + 31) / 32;
    if (oacc <= 1) WA_FMA(1);
    if (oacc <= 2) WA_FMA(2);
    if (oacc <= 4) WA_FMA(4);
    if (oacc <= 8) WA_FMA(8);
    WA_FMA(16);
#undef WA_FMA
    return B200_EUNSUPPORTED;
}
