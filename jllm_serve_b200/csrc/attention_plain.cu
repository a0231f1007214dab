// Causal grouped-query attention over the paged cache, one thread block per (row, query head).
//
// The kernel of the float32 path, and the one the bfloat16 path falls back to for head sizes its
// tensor-core kernels refuse (a head size they do not take, keys and values of different widths). A row at
// position P of request `seg` sees the keys [first, P] of that request, first = jllm_first_key(P, window): 0,
// max(0, P + 1 - window) under a window, the start of P's own chunk of -window positions under chunks. Two passes over the keys: the
// maximum score first (exact in any order), then exp(score - max), their sum and the weighted sum of
// the values, both in ascending key order. A row's result therefore depends on its own query and
// keys only: not on how the prompt was cut, not on the other rows of the batch, not on the pages.
//
// Two things a mixer may add. `keep_first` > 0 (with a window): the request's first keep_first keys stay visible to every
// later row, so a row sees [0, keep_first) and [first, P]; the keys in between are passed over. `sink` (one number per query
// head, else null): the softmax's denominator also holds exp(sink[h]), a key without a value that is not multiplied by the
// scale; the running maximum starts from it, so nothing overflows whichever is larger.
//
// Layouts: q [rows, q_stride] with head h at h * head_dim; cache K and V
// [pages, kv_heads, page_size, cache_dim], a key in the first head_dim values of its row and a value in the first
// value_dim; out [rows, out_stride] with head h at h * value_dim; block_tables [segments, table_stride]
// (page id of position p of a segment: table[p / page_size]).
#include "common.cuh"

namespace {

constexpr int THREADS = 128;
constexpr int MAX_DIMS_PER_THREAD = 8;  // value_dim <= 1024

template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_plain_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                       const T* __restrict__ v_cache, T* __restrict__ out, int out_stride,
                       const int* __restrict__ row_seg, const int* __restrict__ row_pos,
                       const int* __restrict__ block_tables, int table_stride, int heads, int kv_heads, int head_dim,
                       int value_dim, int cache_dim, int page_size, int num_pages, int window, float scale, int keep_first,
                       VecRef sink, int has_sink) {
    extern __shared__ float smem[];
    float* qs = smem;                  // head_dim
    float* es = qs + head_dim;         // THREADS
    float* scratch = es + THREADS;     // 33
    const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int kvh = h / (heads / kv_heads);
    const int P = row_pos[r];
    const int first = jllm_first_key(P, window);
    const int kept = window > 0 ? min(keep_first, first) : 0;      // keys [0, kept) in front of the window
    const int* table = block_tables + (size_t)row_seg[r] * table_stride;
    const T* qrow = q + (size_t)r * q_stride + (size_t)h * head_dim;
    for (int i = tid; i < head_dim; i += THREADS) qs[i] = to_float(qrow[i]);
    __syncthreads();

    auto key_row = [&](const T* cache, int s) -> const T* {   // nullptr only in the checked build, for a bad table
        const long long page = jllm_page_of(table, s / page_size, table_stride, num_pages);
        if (kCheckBounds && page < 0) return nullptr;
        return cache + (((size_t)page * kv_heads + kvh) * page_size + (s % page_size)) * cache_dim;
    };
    auto score_of = [&](int s) -> float {
        const T* kr = key_row(k_cache, s);
        if (kCheckBounds && kr == nullptr) return -INFINITY;
        float acc = 0.f;
        for (int i = 0; i < head_dim; ++i) acc = fmaf(qs[i], to_float(kr[i]), acc);
        return __fmul_rn(acc, scale);
    };

    // the visible keys in ascending order: index u < kept is key u, index u >= kept is key first + (u - kept)
    const int visible = kept + (P + 1 - first);
    auto key_at = [&](int u) -> int { return u < kept ? u : first + (u - kept); };
    float m = has_sink ? sink[h] : -INFINITY;
    for (int u = tid; u < visible; u += THREADS) m = fmaxf(m, score_of(key_at(u)));
    m = block_max(m, scratch);

    float acc[MAX_DIMS_PER_THREAD] = {};
    float sum = has_sink ? expf(sink[h] - m) : 0.f;
    for (int u0 = 0; u0 < visible; u0 += THREADS) {
        const int u = u0 + tid;
        __syncthreads();
        es[tid] = u < visible ? expf(score_of(key_at(u)) - m) : 0.f;
        __syncthreads();
        const int n = min(THREADS, visible - u0);
        for (int j = 0; j < n; ++j) {
            const float e = es[j];
            sum += e;
            const T* vr = key_row(v_cache, key_at(u0 + j));
            if (kCheckBounds && vr == nullptr) continue;
#pragma unroll
            for (int c = 0; c < MAX_DIMS_PER_THREAD; ++c) {
                const int d = tid + c * THREADS;
                if (d < value_dim) acc[c] = fmaf(e, to_float(vr[d]), acc[c]);
            }
        }
    }
    const float inv = 1.f / sum;
    T* orow = out + (size_t)r * out_stride + (size_t)h * value_dim;
#pragma unroll
    for (int c = 0; c < MAX_DIMS_PER_THREAD; ++c) {
        const int d = tid + c * THREADS;
        if (d < value_dim) orow[d] = from_float<T>(__fmul_rn(acc[c], inv));
    }
}

}  // namespace

JLLM_BOUNDS_READER(attention_plain)

JLLM_EXPORT int jllm_attention_plain(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                     int out_stride, const int* row_seg, const int* row_pos, const int* block_tables,
                                     int table_stride, int rows, int heads, int kv_heads, int head_dim, int value_dim,
                                     int cache_dim, int page_size, int window, float scale, int dtype, int keep_first,
                                     const void* sink, int sink_dtype, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && head_dim > 0 && page_size > 0,
                 "attention: rows=%d heads=%d kv_heads=%d head_dim=%d page_size=%d", rows, heads, kv_heads, head_dim,
                 page_size);
    JLLM_REQUIRE(value_dim > 0 && value_dim <= THREADS * MAX_DIMS_PER_THREAD && head_dim <= 8192,
                 "attention: head_dim=%d is above 8192 or value_dim=%d above %d", head_dim, value_dim, THREADS * MAX_DIMS_PER_THREAD);
    JLLM_REQUIRE(cache_dim >= head_dim && cache_dim >= value_dim, "attention: cache rows of %d values hold no key of %d or value of %d",
                 cache_dim, head_dim, value_dim);
    JLLM_REQUIRE(heads <= 65535, "attention: heads=%d", heads);
    JLLM_REQUIRE(keep_first >= 0 && (keep_first == 0 || window > 0), "attention: keep_first=%d needs a window (window=%d)",
                 keep_first, window);
    const VecRef sk{sink, sink_dtype};
    const int has_sink = sink != nullptr;
    if (rows == 0) return JLLM_OK;
    const dim3 grid(rows, heads);
    const int num_pages = jllm_pool_pages();
    const size_t smem = (head_dim + THREADS + 33) * sizeof(float);
    if (dtype == JLLM_F32)
        attention_plain_kernel<float><<<grid, THREADS, smem, stream>>>(
            (const float*)q, q_stride, (const float*)k_cache, (const float*)v_cache, (float*)out, out_stride, row_seg,
            row_pos, block_tables, table_stride, heads, kv_heads, head_dim, value_dim, cache_dim, page_size, num_pages, window, scale,
            keep_first, sk, has_sink);
    else
        attention_plain_kernel<__nv_bfloat16><<<grid, THREADS, smem, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
            (__nv_bfloat16*)out, out_stride, row_seg, row_pos, block_tables, table_stride, heads, kv_heads, head_dim,
            value_dim, cache_dim, page_size, num_pages, window, scale, keep_first, sk, has_sink);
    return jllm_check_launch("attention_plain");
}
