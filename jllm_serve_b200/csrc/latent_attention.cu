// Attention over a cached latent: the two kernels around the paged attention kernels.
//
// A latent-attention mixer keeps ONE row c_t of `rank` values per position (c_t = rmsnorm(Wd h_t) * gain) and makes every
// head's keys and values from it: k = Wuk c, v = Wuv c. With q' = Wuk_h^T q_h the score q_h . k_j equals q' . c_j, and
// sum_j p_j v_j = Wuv_h (sum_j p_j c_j): attention with one key/value head of width `rank` whose keys and values are the
// same cached rows, between two small products per head. The attention itself is the engine's paged attention
// (kv_heads = 1, head_dim = rank). Here:
//
//   latent_norm_store   RMSNorm of the down-projected rows (float32 arithmetic) and their write into the paged cache
//   latent_prepare      the same for a mixer whose queries go through a latent of their own and whose cached row ends in a
//                       rotated key part that all heads share: from one float32 row of the stacked down projections it
//                       makes the normed query latent (compute type) and the cached row [normed latent, rotated part]
//   rope_heads          the rotated part of every query head, turned by the row's position and placed behind the head's
//                       latent-space query (where `gemm_heads` put it), so that one dot product with a cached row gives
//                       both terms of the score
//   gemm_heads          out[r, h, :] = f(r, h) * W[h] a[r, h, :] for every head h at once (W [heads, N, K]); f = alpha, or
//                       alpha * sigmoid(gate[r, h]) (the mixer's output gate). float32: on the CUDA cores with one
//                       accumulator per element in ascending k. bfloat16: 64 x 64 tiles per (head, block) on the tensor
//                       cores (mma.sync m16n8k16, float32 accumulation), operands staged in shared memory 32 k at a
//                       time. Either way a row's result depends on that row alone, not on the batch.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
latent_norm_store_kernel(const T* __restrict__ src, int ld, VecRef gain, const int* __restrict__ slots, T* __restrict__ cache,
                         int rank, float eps, long long cache_rows) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const T* row = src + (size_t)r * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(row[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)rank + eps);
    const int slot = slots[r];
    if (!jllm_in_bounds(slot, cache_rows, BOUNDS_SLOT)) return;
    T* dst = cache + (size_t)slot * rank;
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        dst[i] = from_float<T>(__fmul_rn(__fmul_rn(to_float(row[i]), inv), gain[i]));
}

// Turns neighbouring pairs: (u, v) -> (u cos - v sin, v cos + u sin), the angle of pair i from the position's table row.
__device__ __forceinline__ void turn_pair(float u, float v, float c, float s, float& a, float& b) {
    a = __fsub_rn(__fmul_rn(u, c), __fmul_rn(v, s));
    b = __fadd_rn(__fmul_rn(v, c), __fmul_rn(u, s));
}

// One block per row. src [rows, ld] float32: the query latent's q_rank values at q_off (q_rank = 0: none), the latent's
// rank values at d_off and the rope_dim values of the rotated part behind them. cq [rows, q_rank]; cache rows of
// rank + rope_dim values. cos / sin [positions, rotary_dim / 2]: pairs (2i, 2i + 1), i < rotary_dim / 2, of the rotated
// part are turned, the rest of it is copied.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* __restrict__ src, int ld, int q_off, int q_rank, VecRef q_gain, T* __restrict__ cq, int d_off,
                      int rank, int rope_dim, VecRef gain, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                      int rotary_dim, const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ cache,
                      float eps, long long cache_rows, int write_latent) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const float* row = src + (size_t)r * ld;
    if (q_rank > 0) {
        const float* q = row + q_off;
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(q[i], q[i], ss);
        ss = block_sum(ss, scratch);
        const float inv = 1.f / sqrtf(ss / (float)q_rank + eps);
        T* dst = cq + (size_t)r * q_rank;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) dst[i] = from_float<T>(__fmul_rn(__fmul_rn(q[i], inv), q_gain[i]));
    }
    if (!write_latent) return;
    const float* d = row + d_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(d[i], d[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)rank + eps);
    const int slot = slots[r];
    if (!jllm_in_bounds(slot, cache_rows, BOUNDS_SLOT)) return;
    T* dst = cache + (size_t)slot * (rank + rope_dim);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(__fmul_rn(__fmul_rn(d[i], inv), gain[i]));
    const int half = rotary_dim / 2;
    const float* c = cos_t + (size_t)positions[r] * half;
    const float* s = sin_t + (size_t)positions[r] * half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float a, b;
        turn_pair(d[rank + 2 * i], d[rank + 2 * i + 1], c[i], s[i], a, b);
        dst[rank + 2 * i] = from_float<T>(a);
        dst[rank + 2 * i + 1] = from_float<T>(b);
    }
    for (int i = rotary_dim + threadIdx.x; i < rope_dim; i += blockDim.x) dst[rank + i] = from_float<T>(d[rank + i]);
}

// q [rows, ldq]: head h's rope_dim values at h * q_head + q_off; out [rows, ldo]: they go to h * o_head + o_off.
template <typename T>
__global__ void __launch_bounds__(128)
rope_heads_kernel(const T* __restrict__ q, int ldq, int q_head, int q_off, T* __restrict__ out, int ldo, int o_head, int o_off,
                  int heads, int rope_dim, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rotary_dim,
                  const int* __restrict__ positions) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, half = rotary_dim / 2, pairs = rope_dim / 2;
    const float* c = cos_t + (size_t)positions[r] * half;
    const float* s = sin_t + (size_t)positions[r] * half;
    for (int e = threadIdx.x; e < heads * pairs; e += blockDim.x) {
        const int h = e / pairs, i = e - h * pairs;
        const T* src = q + (size_t)r * ldq + (size_t)h * q_head + q_off + 2 * i;
        T* dst = out + (size_t)r * ldo + (size_t)h * o_head + o_off + 2 * i;
        float a = to_float(src[0]), b = to_float(src[1]);
        if (i < half) turn_pair(a, b, c[i], s[i], a, b);
        dst[0] = from_float<T>(a);
        dst[1] = from_float<T>(b);
    }
    if (rope_dim & 1) {        // an odd width's last value is never part of a pair
        for (int h = threadIdx.x; h < heads; h += blockDim.x)
            out[(size_t)r * ldo + (size_t)h * o_head + o_off + rope_dim - 1] = q[(size_t)r * ldq + (size_t)h * q_head + q_off + rope_dim - 1];
    }
}

// What `gemm_heads` is asked to do beside its product (rope_dim > 0): the rope_dim values that follow a head's K inputs are
// turned by the row's position and placed behind the head's N outputs. One more block per (row tile, head) does it.
struct HeadRope {
    int rope_dim, rotary_dim;
    const float* cos_t;
    const float* sin_t;
    const int* positions;
};

template <typename T>
__device__ __forceinline__ void rope_tile(const T* __restrict__ ah, int lda, T* __restrict__ oh, int ldo, int m0, int M, int K, int N,
                                          const HeadRope& rp) {
    const int half = rp.rotary_dim / 2, pairs = rp.rope_dim / 2;
    for (int e = threadIdx.x; e < 64 * pairs; e += blockDim.x) {
        const int m = m0 + e / pairs, i = e % pairs;
        if (m >= M) break;
        const T* src = ah + (size_t)m * lda + K + 2 * i;
        T* dst = oh + (size_t)m * ldo + N + 2 * i;
        float a = to_float(src[0]), b = to_float(src[1]);
        if (i < half) {
            const size_t at = (size_t)rp.positions[m] * half + i;
            turn_pair(a, b, rp.cos_t[at], rp.sin_t[at], a, b);
        }
        dst[0] = from_float<T>(a);
        dst[1] = from_float<T>(b);
    }
    if (rp.rope_dim & 1)
        for (int e = threadIdx.x; e < 64 && m0 + e < M; e += blockDim.x)
            oh[(size_t)(m0 + e) * ldo + N + rp.rope_dim - 1] = ah[(size_t)(m0 + e) * lda + K + rp.rope_dim - 1];
}

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_heads_kernel(const T* __restrict__ a, int lda, const T* __restrict__ w, T* __restrict__ out, int ldo,
                  const T* __restrict__ gate, int ld_gate, float alpha, int M, int N, int K, int a_head, int o_head, HeadRope rp) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    pdl_wait();
    pdl_trigger();
    if (rp.rope_dim > 0 && blockIdx.x == gridDim.x - 1) {
        rope_tile(a + (size_t)blockIdx.z * a_head, lda, out + (size_t)blockIdx.z * o_head, ldo, blockIdx.y * BM, M, K, N, rp);
        return;
    }
    const int tid = threadIdx.x, h = blockIdx.z;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;
    const T* ah = a + (size_t)h * a_head;
    const T* wh = w + (size_t)h * N * K;
    float acc[TM][TN] = {};
    const int lr = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int m = m0 + lr, n = n0 + lr;
            as[lk + j][lr] = (m < M && k < K) ? to_float(ah[(size_t)m * lda + k]) : 0.f;
            ws[lk + j][lr] = (n < N && k < K) ? to_float(wh[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
        float f = alpha;
        if (gate != nullptr) {
            const float gv = to_float(gate[(size_t)m * ld_gate + h]);
            f = __fmul_rn(alpha, 1.f / (1.f + expf(-gv)));
        }
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) out[(size_t)m * ldo + (size_t)h * o_head + n] = from_float<T>(__fmul_rn(acc[i][j], f));
        }
    }
}

// The bfloat16 product on the tensor cores. Four warps; warp w holds rows [16 w, 16 w + 16) of the block's 64 x 64 tile
// as eight m16n8 accumulators. Shared rows are padded to 40 values, so that the eight rows a fragment load touches fall
// into different banks. VEC: K, the row strides and the base addresses allow 16-byte loads.
constexpr int HK = 32, HPAD = 40;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool VEC>
__global__ void __launch_bounds__(128)
gemm_heads_mma_kernel(const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w,
                      __nv_bfloat16* __restrict__ out, int ldo, const __nv_bfloat16* __restrict__ gate, int ld_gate,
                      float alpha, int M, int N, int K, int a_head, int o_head, HeadRope rp) {
    __shared__ __align__(16) __nv_bfloat16 as[64][HPAD];
    __shared__ __align__(16) __nv_bfloat16 ws[64][HPAD];
    pdl_wait();
    pdl_trigger();
    if (rp.rope_dim > 0 && blockIdx.x == gridDim.x - 1) {
        rope_tile(a + (size_t)blockIdx.z * a_head, lda, out + (size_t)blockIdx.z * o_head, ldo, blockIdx.y * 64, M, K, N, rp);
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3, h = blockIdx.z;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const __nv_bfloat16* ah = a + (size_t)h * a_head;
    const __nv_bfloat16* wh = w + (size_t)h * N * K;
    float acc[8][4] = {};
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
    for (int k0 = 0; k0 < K; k0 += HK) {
        if (VEC) {
            // 64 rows x 4 chunks of 8 values per tile: two chunks a thread and tile
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = tid + 128 * j, row = c >> 2, kc = (c & 3) * 8, k = k0 + kc;
                uint4 va = make_uint4(0, 0, 0, 0), vw = va;
                if (k < K) {        // (K is a multiple of 8 here: a chunk is inside or outside as a whole)
                    if (m0 + row < M) va = *reinterpret_cast<const uint4*>(ah + (size_t)(m0 + row) * lda + k);
                    if (n0 + row < N) vw = *reinterpret_cast<const uint4*>(wh + (size_t)(n0 + row) * K + k);
                }
                *reinterpret_cast<uint4*>(&as[row][kc]) = va;
                *reinterpret_cast<uint4*>(&ws[row][kc]) = vw;
            }
        } else {
            for (int e = tid; e < 64 * HK; e += 128) {
                const int row = e / HK, kc = e - row * HK, k = k0 + kc;
                as[row][kc] = (m0 + row < M && k < K) ? ah[(size_t)(m0 + row) * lda + k] : zero;
                ws[row][kc] = (n0 + row < N && k < K) ? wh[(size_t)(n0 + row) * K + k] : zero;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HK; kk += 16) {
            const int r = warp * 16 + g;
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(&as[r][kk + 2 * t]);
            const uint32_t a1 = *reinterpret_cast<const uint32_t*>(&as[r + 8][kk + 2 * t]);
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(&as[r][kk + 2 * t + 8]);
            const uint32_t a3 = *reinterpret_cast<const uint32_t*>(&as[r + 8][kk + 2 * t + 8]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&ws[8 * j + g][kk + 2 * t]);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&ws[8 * j + g][kk + 2 * t + 8]);
                mma_bf16_16816(acc[j], a0, a1, a2, a3, b0, b1);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int m = m0 + warp * 16 + g + 8 * half;
        if (m >= M) continue;
        float f = alpha;
        if (gate != nullptr) {
            const float gv = to_float(gate[(size_t)m * ld_gate + h]);
            f = __fmul_rn(alpha, 1.f / (1.f + expf(-gv)));
        }
        __nv_bfloat16* dst = out + (size_t)m * ldo + (size_t)h * o_head;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + 8 * j + 2 * t;
            if (n < N) dst[n] = __float2bfloat16_rn(__fmul_rn(acc[j][2 * half], f));
            if (n + 1 < N) dst[n + 1] = __float2bfloat16_rn(__fmul_rn(acc[j][2 * half + 1], f));
        }
    }
}

}  // namespace

JLLM_BOUNDS_READER(latent_attention)

// src [rows, ld] (the down-projected rows), cache [cache_rows, rank] (a page pool seen as rows: slot = page * page_size
// + offset), both of type `dtype`.
JLLM_EXPORT int jllm_latent_norm_store(const void* src, int dtype, int ld, const void* gain, int gain_dtype,
                                       const int* slots, void* cache, long long cache_rows, int rows, int rank, float eps,
                                       cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && rank > 0 && ld >= rank, "latent_norm_store: rows=%d rank=%d ld=%d", rows, rank, ld);
    if (rows == 0) return JLLM_OK;
    const VecRef g{gain, gain_dtype};
    if (dtype == JLLM_F32)
        jllm_launch(latent_norm_store_kernel<float>, dim3(rows), dim3(128), 0, stream, LAUNCH_DEPENDENT, (const float*)src,
                    ld, g, slots, (float*)cache, rank, eps, cache_rows);
    else
        jllm_launch(latent_norm_store_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream, LAUNCH_DEPENDENT,
                    (const __nv_bfloat16*)src, ld, g, slots, (__nv_bfloat16*)cache, rank, eps, cache_rows);
    return jllm_check_launch("latent_norm_store");
}

// a [M, lda] with head h's K values at column h * a_head (0: h * K); w [heads, N, K]; out [M, ldo] with head h's N values at
// h * o_head (0: h * N); gate (or null) [M, ld_gate] with head h's gate at column h.
JLLM_EXPORT int jllm_gemm_heads(const void* a, int dtype, int lda, const void* w, void* out, int ldo, const void* gate,
                                int ld_gate, float alpha, int M, int heads, int N, int K, int a_head, int o_head, int rope_dim,
                                const float* cos_t, const float* sin_t, int rotary_dim, const int* positions,
                                cudaStream_t stream) {
    JLLM_REQUIRE(M >= 0 && heads > 0 && N > 0 && K > 0, "gemm_heads: M=%d heads=%d N=%d K=%d", M, heads, N, K);
    if (a_head == 0) a_head = K;
    if (o_head == 0) o_head = N;
    JLLM_REQUIRE(rope_dim >= 0 && rotary_dim >= 0 && rotary_dim <= rope_dim && rotary_dim % 2 == 0 && a_head >= K + rope_dim &&
                     o_head >= N + rope_dim && (rope_dim == 0 || positions != nullptr),
                 "gemm_heads: rope_dim=%d rotary_dim=%d with heads every %d / %d values", rope_dim, rotary_dim, a_head, o_head);
    const HeadRope rp{rope_dim, rotary_dim, cos_t, sin_t, positions};
    JLLM_REQUIRE(a_head >= K && o_head >= N && lda >= (heads - 1) * a_head + K && ldo >= (heads - 1) * o_head + N &&
                     heads <= 65535 && (M + BM - 1) / BM <= 65535,
                 "gemm_heads: lda=%d ldo=%d for %d heads of K=%d (every %d), N=%d (every %d)", lda, ldo, heads, K, a_head, N, o_head);
    if (M == 0) return JLLM_OK;
    const dim3 grid((N + BN - 1) / BN + (rope_dim > 0 ? 1 : 0), (M + BM - 1) / BM, heads);
    static_assert(BM == 64 && BN == 64, "both kernels take 64 x 64 tiles");
    if (dtype == JLLM_F32) {
        jllm_launch(gemm_heads_kernel<float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (const float*)a, lda,
                    (const float*)w, (float*)out, ldo, (const float*)gate, ld_gate, alpha, M, N, K, a_head, o_head, rp);
        return jllm_check_launch("gemm_heads");
    }
    const bool vec = K % 8 == 0 && lda % 8 == 0 && a_head % 8 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0;
    if (vec)
        jllm_launch(gemm_heads_mma_kernel<true>, grid, dim3(128), 0, stream, LAUNCH_DEPENDENT, (const __nv_bfloat16*)a, lda,
                    (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)gate, ld_gate, alpha, M, N, K, a_head, o_head, rp);
    else
        jllm_launch(gemm_heads_mma_kernel<false>, grid, dim3(128), 0, stream, LAUNCH_DEPENDENT, (const __nv_bfloat16*)a, lda,
                    (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)gate, ld_gate, alpha, M, N, K, a_head, o_head, rp);
    return jllm_check_launch("gemm_heads");
}

// src [rows, ld] float32 (the stacked down projections); cq [rows, q_rank] and the cache [cache_rows, rank + rope_dim] of
// type `dtype`. q_rank = 0: no query latent; write_latent = 0: the run caches nothing of its own.
JLLM_EXPORT int jllm_latent_prepare(const float* src, int ld, int q_off, int q_rank, const void* q_gain, void* cq, int d_off,
                                    int rank, int rope_dim, const void* gain, int gain_dtype, const float* cos_t,
                                    const float* sin_t, int rotary_dim, const int* positions, const int* slots, void* cache,
                                    int dtype, long long cache_rows, int rows, float eps, int write_latent, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && q_rank >= 0 && rank > 0 && rope_dim >= 0 && rotary_dim >= 0 && rotary_dim <= rope_dim &&
                     rotary_dim % 2 == 0,
                 "latent_prepare: rows=%d q_rank=%d rank=%d rope_dim=%d rotary_dim=%d", rows, q_rank, rank, rope_dim, rotary_dim);
    if (rows == 0 || (q_rank == 0 && !write_latent)) return JLLM_OK;
    const VecRef g{gain, gain_dtype}, qg{q_gain, gain_dtype};
    if (dtype == JLLM_F32)
        jllm_launch(latent_prepare_kernel<float>, dim3(rows), dim3(128), 0, stream, LAUNCH_DEPENDENT, src, ld, q_off, q_rank, qg,
                    (float*)cq, d_off, rank, rope_dim, g, cos_t, sin_t, rotary_dim, positions, slots, (float*)cache, eps,
                    cache_rows, write_latent);
    else
        jllm_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream, LAUNCH_DEPENDENT, src, ld, q_off,
                    q_rank, qg, (__nv_bfloat16*)cq, d_off, rank, rope_dim, g, cos_t, sin_t, rotary_dim, positions, slots,
                    (__nv_bfloat16*)cache, eps, cache_rows, write_latent);
    return jllm_check_launch("latent_prepare");
}

JLLM_EXPORT int jllm_rope_heads(const void* q, int dtype, int ldq, int q_head, int q_off, void* out, int ldo, int o_head,
                                int o_off, int rows, int heads, int rope_dim, const float* cos_t, const float* sin_t,
                                int rotary_dim, const int* positions, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && rope_dim > 0 && rotary_dim >= 0 && rotary_dim <= rope_dim && rotary_dim % 2 == 0,
                 "rope_heads: rows=%d heads=%d rope_dim=%d rotary_dim=%d", rows, heads, rope_dim, rotary_dim);
    if (rows == 0) return JLLM_OK;
    if (dtype == JLLM_F32)
        jllm_launch(rope_heads_kernel<float>, dim3(rows), dim3(128), 0, stream, LAUNCH_DEPENDENT, (const float*)q, ldq, q_head,
                    q_off, (float*)out, ldo, o_head, o_off, heads, rope_dim, cos_t, sin_t, rotary_dim, positions);
    else
        jllm_launch(rope_heads_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream, LAUNCH_DEPENDENT, (const __nv_bfloat16*)q,
                    ldq, q_head, q_off, (__nv_bfloat16*)out, ldo, o_head, o_off, heads, rope_dim, cos_t, sin_t, rotary_dim,
                    positions);
    return jllm_check_launch("rope_heads");
}
