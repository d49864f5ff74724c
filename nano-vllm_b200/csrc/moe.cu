// Routed experts: sigmoid router with top-k selection, token -> expert grouping on the device (no host round trip, so a
// step stays graph-capturable), grouped expert GEMMs over the grouped rows, and the weighted combine.
//
//   moe_route_kernel  : scores = sigmoid(logits) in fp32; the `top` largest per token with their scores as weights
//   moe_route_grouped_kernel: scores = softmax(logits) (or sigmoid); the choice is made on score + correction, among the experts of
//                       the best groups only; weights are the plain scores of the chosen, renormalised and scaled; experts past
//                       `num_real` are identity experts (no tensors: index -1, handled by the combine)
//   moe_align_kernel  : counting sort of the (token, choice) pairs by expert; every expert's run is padded to a multiple of
//                       the GEMM's row tile so one tile never spans two experts
//   moe_gemm_kernel   : C[i, :] = act(A[src(i), :] * scale(i)) . W[e(i)]^T, one expert per row tile
//   moe_combine_kernel: per token, the sum of its choices' rows (fixed order) plus the gated shared expert
#include "mix_common.cuh"

namespace {

// One warp per token: lane l looks at experts l, l + 32, ...; the chosen ones are struck from a per-lane bit mask (so the kernel
// serves up to 1024 experts), and every round ends in a warp arg-max that prefers the lower index among equal logits.  Lane 0's
// result is broadcast before it is struck, so exactly the reported expert leaves the candidates whatever the logits hold (a NaN
// counts as minus infinity): the indices are always valid and distinct.
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int64_t ld, int n, int E, int top,
                                                        int32_t* __restrict__ idx, float* __restrict__ wgt) {
    B200_PDL_SYNC();
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n) return;
    const float* z = logits + (int64_t)t * ld;
    constexpr int NONE = 0x7fffffff;
    uint32_t taken = 0;
    for (int k = 0; k < top; ++k) {
        int best = NONE;
        float bv = -INFINITY;
        for (int i = 0, e = lane; e < E; ++i, e += 32) {
            float v = z[e];
            if (!(v == v)) v = -INFINITY;
            if (!((taken >> i) & 1u) && (best == NONE || v > bv)) {
                best = e;
                bv = v;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int ob = __shfl_xor_sync(0xffffffffu, best, off);
            if (ob != NONE && (best == NONE || ov > bv || (ov == bv && ob < best))) {
                bv = ov;
                best = ob;
            }
        }
        best = __shfl_sync(0xffffffffu, best, 0);
        bv = __shfl_sync(0xffffffffu, bv, 0);
        if (best == NONE) best = 0;                       // cannot happen while top <= E; keeps the index in range regardless
        if ((best & 31) == lane) taken |= 1u << (best >> 5);
        if (lane == 0) {
            idx[(int64_t)t * top + k] = best;
            wgt[(int64_t)t * top + k] = sigmoidf_(bv);
        }
    }
}

constexpr int RG_MAX = 1024;       // experts (identity ones included) the grouped router serves
constexpr int RG_WARPS = 4;

// One warp per token.  s = softmax(z) over all `E` router outputs (score_kind 0) or sigmoid(z) (1); choice score c = s +
// correction.  The E outputs form `n_groups` equal groups of neighbours; a group's score is its largest c, and only experts of
// the `keep` best groups can be chosen (with n_groups <= 1 or keep >= n_groups: all).  The `top` largest c among those win;
// their weights are s (without the correction), divided by their sum + 1e-20 when `renorm`, times `scale`.  Equal scores go
// to the lower index; a NaN counts as minus infinity.  idx is the expert, or -1 for the identity experts e >= num_real.
__global__ void __launch_bounds__(RG_WARPS * 32) moe_route_grouped_kernel(const float* __restrict__ logits, int64_t ld, int n, int E, int top,
                                                                          const float* __restrict__ correction, int n_groups, int keep,
                                                                          int num_real, int score_kind, int renorm, float scale,
                                                                          int32_t* __restrict__ idx, float* __restrict__ wgt) {
    B200_PDL_SYNC();
    __shared__ float sh_s[RG_WARPS][RG_MAX];          // plain scores
    __shared__ float sh_g[RG_WARPS][RG_MAX];          // group scores; after the group choice: 1 = open, 0 = closed
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * RG_WARPS + warp;
    if (t >= n) return;
    const float* z = logits + (int64_t)t * ld;
    float* sc = sh_s[warp];
    float* gs = sh_g[warp];
    constexpr int NONE = 0x7fffffff;
    if (score_kind == 0) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float p = expf(z[e] - mx);
            sc[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) sc[e] *= inv;
    } else {
        for (int e = lane; e < E; e += 32) sc[e] = sigmoidf_(z[e]);
    }
    __syncwarp();
    const bool grouped = n_groups > 1 && keep < n_groups;
    const int gsize = grouped ? E / n_groups : E;
    if (grouped) {
        for (int gi = lane; gi < n_groups; gi += 32) {
            float best = -INFINITY;
            for (int e = gi * gsize; e < (gi + 1) * gsize; ++e) {
                float c = sc[e] + (correction ? correction[e] : 0.f);
                if (!(c == c)) c = -INFINITY;
                best = fmaxf(best, c);
            }
            gs[gi] = best;
        }
        __syncwarp();
        uint32_t open = 0;                            // bit i: group lane + 32 i is kept
        for (int k = 0; k < keep; ++k) {
            int best = NONE;
            float bv = -INFINITY;
            for (int i = 0, gi = lane; gi < n_groups; ++i, gi += 32) {
                const float v = gs[gi];
                if (!((open >> i) & 1u) && (best == NONE || v > bv)) {
                    best = gi;
                    bv = v;
                }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
                const int ob = __shfl_xor_sync(0xffffffffu, best, off);
                if (ob != NONE && (best == NONE || ov > bv || (ov == bv && ob < best))) {
                    bv = ov;
                    best = ob;
                }
            }
            best = __shfl_sync(0xffffffffu, best, 0);
            if (best != NONE && (best & 31) == lane) open |= 1u << (best >> 5);
        }
        __syncwarp();
        for (int i = 0, gi = lane; gi < n_groups; ++i, gi += 32) gs[gi] = ((open >> i) & 1u) ? 1.f : 0.f;
        __syncwarp();
    }
    uint32_t taken = 0;
    float wsum = 0.f;
    for (int k = 0; k < top; ++k) {
        int best = NONE;
        float bv = -INFINITY;
        for (int i = 0, e = lane; e < E; ++i, e += 32) {
            if ((taken >> i) & 1u) continue;
            if (grouped && gs[e / gsize] == 0.f) continue;
            float c = sc[e] + (correction ? correction[e] : 0.f);
            if (!(c == c)) c = -INFINITY;
            if (best == NONE || c > bv) {
                best = e;
                bv = c;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int ob = __shfl_xor_sync(0xffffffffu, best, off);
            if (ob != NONE && (best == NONE || ov > bv || (ov == bv && ob < best))) {
                bv = ov;
                best = ob;
            }
        }
        best = __shfl_sync(0xffffffffu, best, 0);
        if (best == NONE) best = 0;                   // only if fewer than `top` experts are open; keeps the index in range
        if ((best & 31) == lane) taken |= 1u << (best >> 5);
        const float w = sc[best];
        wsum += w;
        if (lane == 0) {
            idx[(int64_t)t * top + k] = best < num_real ? best : -1;
            wgt[(int64_t)t * top + k] = w;
        }
    }
    __syncwarp();
    const float f = (renorm ? 1.0f / (wsum + 1e-20f) : 1.0f) * scale;
    for (int k = lane; k < top; k += 32) wgt[(int64_t)t * top + k] *= f;
}

// One CTA.  pairs = n * top entries of idx.  Outputs: sorted_rows[cap] (pair index, or -1 for padding), pos_of[pairs]
// (where each pair went), tile_expert[max_tiles], num_tiles[0].  counts: scratch of 2 * E ints.
__global__ void __launch_bounds__(1024) moe_align_kernel(const int32_t* __restrict__ idx, int pairs, int E, int bm,
                                                         int32_t* __restrict__ sorted_rows, int cap, int32_t* __restrict__ pos_of,
                                                         int32_t* __restrict__ tile_expert, int32_t* __restrict__ num_tiles,
                                                         int32_t* __restrict__ counts) {
    B200_PDL_SYNC();
    __shared__ int32_t sh_counts[2048];
    const bool in_shared = E <= 1024;                            // the usual case: counters in shared memory, `counts` unused
    int32_t* cnt = in_shared ? sh_counts : counts;               // [E] pairs per expert
    int32_t* start = in_shared ? sh_counts + 1024 : counts + E;  // [E] first sorted row of the expert
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    for (int i = threadIdx.x; i < cap; i += blockDim.x) sorted_rows[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x)
        if (idx[i] >= 0) atomicAdd(&cnt[min(idx[i], E - 1)], 1);      // a negative index is a pair without an expert GEMM; one too large is counted at the edge, never written through
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            const int tiles = (cnt[e] + bm - 1) / bm;
            for (int k = 0; k < tiles; ++k) tile_expert[at / bm + k] = e;
            at += tiles * bm;
            cnt[e] = 0;
        }
        num_tiles[0] = at / bm;
    }
    __syncthreads();
    // rows of one expert in ascending pair order would need a stable sort; the order inside an expert changes nothing in
    // the results (rows are independent), so an atomic cursor is enough
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        if (idx[i] < 0) {
            pos_of[i] = -1;
            continue;
        }
        const int e = min(idx[i], E - 1);
        const int p = start[e] + atomicAdd(&cnt[e], 1);
        sorted_rows[p] = i;
        pos_of[i] = p;
    }
}

constexpr int MG_BM = 64, MG_BN = 64, MG_BK = 32;
constexpr int MG_TM = MG_BM / 16;          // rows per thread of the FMA kernel (16 x 16 threads)

// A rows: src_rows == nullptr -> row i of A itself (the grouped intermediate); else pair = sorted_rows[i], token = pair / top,
// A row = tokens[token] * wgt[pair] (rounded to T: it is the expert's input tensor; wgt == nullptr: the token's row as is).
// act: 0 none, 1 relu^2, 2 gated: W = [gate rows (N/2) ; up rows (N/2)] and C[i, o] = silu(gate_o) * up_o has N/2 columns; a CTA
// then stages the gate rows and the up rows of its N/2-column slice side by side.
template <typename T, typename TO>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const T* __restrict__ A, int64_t a_stride, const int32_t* __restrict__ sorted_rows,
                                                       const float* __restrict__ wgt, int top, bool gather,
                                                       const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ num_tiles,
                                                       const T* __restrict__ W, int N, int K, TO* __restrict__ C, int act) {
    B200_PDL_SYNC();
    const int tile = blockIdx.y;
    if (tile >= num_tiles[0]) return;
    __shared__ float As[MG_BM][MG_BK + 1];
    __shared__ float Ws[MG_BN][MG_BK + 1];
    __shared__ int src[MG_BM];
    __shared__ float sc[MG_BM];
    const int e = tile_expert[tile];
    const T* We = W + (int64_t)e * N * K;
    const bool gated = act == 2;
    const int half = N >> 1;
    const int row0 = tile * MG_BM, col0 = blockIdx.x * (gated ? MG_BN / 2 : MG_BN);
    if (threadIdx.x < MG_BM) {
        const int p = sorted_rows[row0 + threadIdx.x];
        src[threadIdx.x] = p < 0 ? -1 : (gather ? p / top : row0 + (int)threadIdx.x);
        sc[threadIdx.x] = (p >= 0 && gather && wgt) ? wgt[p] : 1.0f;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 x 16 threads, MG_TM rows x 4 columns each
    float acc[MG_TM][4] = {};
    for (int k0 = 0; k0 < K; k0 += MG_BK) {
        for (int i = threadIdx.x; i < MG_BM * MG_BK; i += 256) {
            const int r = i / MG_BK, k = i % MG_BK;
            float v = 0.f;
            if (src[r] >= 0 && k0 + k < K) {
                v = ldf(A + (int64_t)src[r] * a_stride + k0 + k);
                if (gather && wgt) v = rnd<T>(v * sc[r]);
            }
            As[r][k] = v;
        }
        for (int i = threadIdx.x; i < MG_BN * MG_BK; i += 256) {
            const int c = i / MG_BK, k = i % MG_BK;
            int wr = col0 + c, lim = N;
            if (gated) {
                wr = c < MG_BN / 2 ? col0 + c : half + col0 + c - MG_BN / 2;
                lim = c < MG_BN / 2 ? half : N;
            }
            Ws[c][k] = (wr < lim && k0 + k < K) ? ldf(We + (int64_t)wr * K + k0 + k) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < MG_BK; ++k) {
            float av[MG_TM];
#pragma unroll
            for (int r = 0; r < MG_TM; ++r) av[r] = As[ty * MG_TM + r][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float w = Ws[tx + 16 * j][k];
#pragma unroll
                for (int r = 0; r < MG_TM; ++r) acc[r][j] = fmaf(av[r], w, acc[r][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < MG_TM; ++r) {
        const int row = ty * MG_TM + r;
        if (src[row] < 0) continue;
        if (gated) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int col = col0 + tx + 16 * j;
                if (col < half) stf(C + (int64_t)(row0 + row) * half + col, siluf_(acc[r][j]) * acc[r][j + 2]);
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = col0 + tx + 16 * j;
            if (col >= N) continue;
            float v = acc[r][j];
            if (act == 1) {
                v = fmaxf(v, 0.f);
                v = v * v;
            }
            stf(C + (int64_t)(row0 + row) * N + col, v);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Tensor-core form of the grouped GEMM (bf16): one 64-row tile of one expert x 128 output columns per CTA (8 warps, 32 x 32 each), K in steps of 64
// through a two-stage shared-memory ring (weights by cp.async, the gathered / weighted input rows through registers),
// mma.sync m16n8k16 with fp32 accumulation.  Needs K % 8 == 0 and 16-byte aligned rows; other shapes take the FMA kernel.
// ---------------------------------------------------------------------------------------------------------------------------
constexpr int MM_BN = 128, MM_BK = 64, MM_LD = MM_BK + 8;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename TO>
__global__ void __launch_bounds__(256) moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, int64_t a_stride,
                                                           const int32_t* __restrict__ sorted_rows, const float* __restrict__ wgt, int top,
                                                           bool gather, const int32_t* __restrict__ tile_expert,
                                                           const int32_t* __restrict__ num_tiles, const __nv_bfloat16* __restrict__ W, int N,
                                                           int K, TO* __restrict__ C, int act) {
    B200_PDL_SYNC();
    const int tile = blockIdx.y;
    if (tile >= num_tiles[0]) return;
    extern __shared__ __align__(16) unsigned char mm_smem[];
    typedef __nv_bfloat16 (*ATile)[MG_BM][MM_LD];
    typedef __nv_bfloat16 (*BTile)[MM_BN][MM_LD];
    ATile As = reinterpret_cast<ATile>(mm_smem);                                                  // [2][MG_BM][MM_LD]
    BTile Bs = reinterpret_cast<BTile>(mm_smem + 2 * MG_BM * MM_LD * sizeof(__nv_bfloat16));      // [2][MM_BN][MM_LD]
    __shared__ int src[MG_BM];
    __shared__ float sc[MG_BM];
    const int e = tile_expert[tile];
    const __nv_bfloat16* We = W + (int64_t)e * N * K;
    const bool gated = act == 2;                       // tile row 2 o' = gate row, 2 o' + 1 = up row of output column col0 + o'
    const int half = N >> 1;
    const int row0 = tile * MG_BM, col0 = blockIdx.x * (gated ? MM_BN / 2 : MM_BN);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wr = warp >> 2, wc = warp & 3;                            // this warp's 32 rows and 32 columns of the tile
    if (tid < MG_BM) {
        const int p = sorted_rows[row0 + tid];
        src[tid] = p < 0 ? -1 : (gather ? p / top : row0 + tid);
        sc[tid] = (p >= 0 && gather && wgt) ? wgt[p] : 1.0f;
    }
    __syncthreads();
    auto load_stage = [&](int st, int k0) {
        for (int i = tid; i < MM_BN * (MM_BK / 8); i += 256) {          // weights: 128 rows x 8 chunks of 16 bytes
            const int r = i >> 3, c = (i & 7) << 3;
            int wr = col0 + r;
            bool ok = wr < N && k0 + c < K;
            if (gated) {
                wr = col0 + (r >> 1);
                ok = wr < half && k0 + c < K;
                wr += (r & 1) ? half : 0;
            }
            cp_async16(smem_u32(&Bs[st][r][c]), ok ? (const void*)(We + (int64_t)wr * K + k0 + c) : (const void*)We, ok ? 16 : 0);
        }
        for (int i = tid; i < MG_BM * (MM_BK / 8); i += 256) {          // input rows: gathered, weighted, rounded
            const int r = i >> 3, c = (i & 7) << 3;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (src[r] >= 0 && k0 + c < K) {
                v = *reinterpret_cast<const uint4*>(A + (int64_t)src[r] * a_stride + k0 + c);
                if (gather && wgt) {
                    float f[8];
                    unpack8(v, f);
#pragma unroll
                    for (int q = 0; q < 8; ++q) f[q] *= sc[r];
                    v = pack8(f);
                }
            }
            *reinterpret_cast<uint4*>(&As[st][r][c]) = v;
        }
        cp_async_commit();
    };
    float acc[2][4][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.f;
    const int nk = (K + MM_BK - 1) / MM_BK;
    load_stage(0, 0);
    for (int it = 0; it < nk; ++it) {
        const int st = it & 1;
        if (it + 1 < nk) {
            load_stage(st ^ 1, (it + 1) * MM_BK);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t a_base = smem_u32(&As[st][wr * 32 + (lane & 15)][(lane >> 4) << 3]);
        const uint32_t b_base = smem_u32(&Bs[st][wc * 32 + (lane & 7) + ((lane >> 4) << 3)][((lane >> 3) & 1) << 3]);
#pragma unroll
        for (int kk = 0; kk < MM_BK; kk += 16) {
            uint32_t a[2][4];
            ldsm4(a_base + kk * 2, a[0][0], a[0][1], a[0][2], a[0][3]);
            ldsm4(a_base + (16 * MM_LD + kk) * 2, a[1][0], a[1][1], a[1][2], a[1][3]);
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t b0, b1, b2, b3;
                ldsm4(b_base + (np * 16 * MM_LD + kk) * 2, b0, b1, b2, b3);
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    mma16816(acc[mt][2 * np], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
                    mma16816(acc[mt][2 * np + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
                }
            }
        }
        __syncthreads();
    }
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int row = wr * 32 + mt * 16 + g + 8 * hh;
            if (src[row] < 0) continue;
            if (gated) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int col = col0 + wc * 16 + nt * 4 + t4;
                    if (col < half) stf(C + (int64_t)(row0 + row) * half + col, siluf_(acc[mt][nt][2 * hh]) * acc[mt][nt][2 * hh + 1]);
                }
                continue;
            }
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int col = col0 + wc * 32 + nt * 8 + 2 * t4 + q;
                    if (col >= N) continue;
                    float v = acc[mt][nt][2 * hh + q];
                    if (act == 1) {
                        v = fmaxf(v, 0.f);
                        v = v * v;
                    }
                    stf(C + (int64_t)(row0 + row) * N + col, v);
                }
        }
}

// out[t, :] = sum_k w[t, k] * rows[pos_of[t * top + k], :] + sigmoid(gate_logit[t]) * shared[t, :]   (w = 1 without wgt; gate = 1
// without gate_logit).  A choice without a grouped row (pos_of < 0: an identity expert) contributes w[t, k] * ident[t, :].
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ rows, const int32_t* __restrict__ pos_of, int top,
                                   const T* __restrict__ shared, const float* __restrict__ gate_logit, int64_t gate_ld,
                                   const float* __restrict__ wgt, const float* __restrict__ ident, float* __restrict__ out, int n,
                                   int width) {
    B200_PDL_SYNC();
    const int t = blockIdx.x;
    float g = 0.f;
    if (shared) g = gate_logit ? sigmoidf_(gate_logit[(int64_t)t * gate_ld]) : 1.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float a = 0.f;
        for (int k = 0; k < top; ++k) {
            const int p = pos_of[(int64_t)t * top + k];
            const float w = wgt ? wgt[(int64_t)t * top + k] : 1.0f;
            if (p >= 0)
                a = fmaf(w, rows[(int64_t)p * width + c], a);
            else if (ident)
                a = fmaf(w, ident[(int64_t)t * width + c], a);
        }
        if (shared) a = fmaf(g, ldf(shared + (int64_t)t * width + c), a);
        out[(int64_t)t * width + c] = a;
    }
}

}  // namespace

extern "C" int b200m_moe_tile_rows(void) { return MG_BM; }

extern "C" int b200m_moe_route(const float* logits, int64_t ld, int n, int num_experts, int top, int32_t* idx, float* wgt, void* stream) {
    if (!logits || !idx || !wgt || n < 0 || num_experts <= 0 || top <= 0 || top > num_experts) return B200_EINVAL;
    if (num_experts > 1024) return B200_EUNSUPPORTED;
    if (n == 0) return B200_OK;
    B200_LAUNCH((moe_route_kernel), (n + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream), logits, ld, n, num_experts, top, idx, wgt);
    return b200_launch_status(nullptr);
}

extern "C" int b200m_moe_route_grouped(const float* logits, int64_t ld, int n, int num_outputs, int top, const float* correction,
                                       int n_groups, int keep, int num_real, int score_kind, int renorm, float scale, int32_t* idx,
                                       float* wgt, void* stream) {
    if (!logits || !idx || !wgt || n < 0 || num_outputs <= 0 || top <= 0 || top > num_outputs || num_real < 0 || num_real > num_outputs)
        return B200_EINVAL;
    if (n_groups > 1 && (num_outputs % n_groups || keep <= 0)) return B200_EINVAL;
    if (n_groups > 1 && keep < n_groups && top > keep * (num_outputs / n_groups)) return B200_EINVAL;
    if (score_kind < 0 || score_kind > 1) return B200_EINVAL;
    if (num_outputs > RG_MAX) return B200_EUNSUPPORTED;
    if (n == 0) return B200_OK;
    B200_LAUNCH((moe_route_grouped_kernel), (n + RG_WARPS - 1) / RG_WARPS, RG_WARPS * 32, 0, static_cast<cudaStream_t>(stream), logits, ld,
                n, num_outputs, top, correction, n_groups, keep, num_real, score_kind, renorm, scale, idx, wgt);
    return b200_launch_status(nullptr);
}

extern "C" int b200m_moe_align(const int32_t* idx, int pairs, int num_experts, int32_t* sorted_rows, int cap, int32_t* pos_of,
                               int32_t* tile_expert, int32_t* num_tiles, int32_t* counts, void* stream) {
    if (!idx || !sorted_rows || !pos_of || !tile_expert || !num_tiles || !counts || pairs < 0 || num_experts <= 0) return B200_EINVAL;
    if (cap % MG_BM || cap < ((pairs + num_experts * (MG_BM - 1)) / MG_BM) * MG_BM) return B200_EWORKSPACE;
    B200_LAUNCH((moe_align_kernel), 1, 1024, 0, static_cast<cudaStream_t>(stream), idx, pairs, num_experts, (int)MG_BM, sorted_rows, cap,
                pos_of, tile_expert, num_tiles, counts);
    return b200_launch_status(nullptr);
}

extern "C" int b200m_moe_gemm(const void* A, int64_t a_stride, const int32_t* sorted_rows, const float* wgt, int top, int gather,
                              const int32_t* tile_expert, const int32_t* num_tiles, int max_tiles, const void* W, int N, int K,
                              void* C, int out_f32, int act, int is32, void* stream) {
    if (!A || !sorted_rows || !tile_expert || !num_tiles || !W || !C || N <= 0 || K <= 0 || max_tiles < 0) return B200_EINVAL;
    if (gather && top <= 0) return B200_EINVAL;
    if (act < 0 || act > 2 || (act == 2 && (N & 1))) return B200_EINVAL;
    if (max_tiles == 0) return B200_OK;
    const int n_out = act == 2 ? N / 2 : N;                // output columns
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool tc = !is32 && (K % 8 == 0) && (a_stride % 8 == 0) && ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) % 16 == 0);
    if (tc) {
        dim3 g2(act == 2 ? (n_out + MM_BN / 2 - 1) / (MM_BN / 2) : (N + MM_BN - 1) / MM_BN, max_tiles);
        using bf = __nv_bfloat16;
        const size_t smem = 2 * (size_t)(MG_BM + MM_BN) * MM_LD * sizeof(bf);
        cudaError_t ce = out_f32 ? cudaFuncSetAttribute(moe_gemm_mma_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                 : cudaFuncSetAttribute(moe_gemm_mma_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ce != cudaSuccess) {
            b200_tls_cuda_error() = cudaGetErrorString(ce);
            return B200_ECUDA;
        }
        if (out_f32)
            B200_LAUNCH((moe_gemm_mma_kernel<float>), g2, 256, smem, st, static_cast<const bf*>(A), a_stride, sorted_rows, wgt, top, gather != 0,
                        tile_expert, num_tiles, static_cast<const bf*>(W), N, K, static_cast<float*>(C), act);
        else
            B200_LAUNCH((moe_gemm_mma_kernel<bf>), g2, 256, smem, st, static_cast<const bf*>(A), a_stride, sorted_rows, wgt, top, gather != 0,
                        tile_expert, num_tiles, static_cast<const bf*>(W), N, K, static_cast<bf*>(C), act);
        return b200_launch_status(nullptr);
    }
    dim3 grid(act == 2 ? (n_out + MG_BN / 2 - 1) / (MG_BN / 2) : (N + MG_BN - 1) / MG_BN, max_tiles);
    if (out_f32) {
        B200M_DISPATCH(is32, B200_LAUNCH((moe_gemm_kernel<T, float>), grid, 256, 0, st, static_cast<const T*>(A), a_stride, sorted_rows,
                                         wgt, top, gather != 0, tile_expert, num_tiles, static_cast<const T*>(W), N, K,
                                         static_cast<float*>(C), act));
    } else {
        B200M_DISPATCH(is32, B200_LAUNCH((moe_gemm_kernel<T, T>), grid, 256, 0, st, static_cast<const T*>(A), a_stride, sorted_rows,
                                         wgt, top, gather != 0, tile_expert, num_tiles, static_cast<const T*>(W), N, K,
                                         static_cast<T*>(C), act));
    }
    return b200_launch_status(nullptr);
}

extern "C" int b200m_moe_combine(const float* rows, const int32_t* pos_of, int top, const void* shared, const float* gate_logit,
                                 int64_t gate_ld, const float* wgt, const float* ident, float* out, int n, int width, int is32,
                                 void* stream) {
    if (!rows || !pos_of || !out || n < 0 || width <= 0 || top <= 0) return B200_EINVAL;
    if (n == 0) return B200_OK;
    B200M_DISPATCH(is32, B200_LAUNCH((moe_combine_kernel<T>), n, 256, 0, static_cast<cudaStream_t>(stream), rows, pos_of, top,
                                     static_cast<const T*>(shared), gate_logit, gate_ld, wgt, ident, out, n, width));
    return b200_launch_status(nullptr);
}
