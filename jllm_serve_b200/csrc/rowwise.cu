// Row-wise kernels: embedding gather, RMSNorm, SwiGLU, and the fused per-head q/k RMSNorm +
// rotary position encoding + write of keys and values into the paged cache.
//
// All arithmetic is 32-bit float whatever the storage type; each row's result depends on that row
// alone (fixed reduction order), so it is the same in any batch.
#include <cstdlib>

#include "head_rotate.cuh"

// ---------------------------------------------------------------------------------------------------
// x[r, :] = table[ids[r], :]  (float residual stream from a float or bfloat16 table)
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ x,
                                  int dim, int vocab) {
    const int r = blockIdx.x;
    int id = ids[r];
    jllm_in_bounds(id, vocab, BOUNDS_TOKEN);           // checked build: recorded
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // ids are validated on the host; never read out of bounds
    const T* src = table + (size_t)id * dim;
    float* dst = x + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = to_float(src[i]);
}

JLLM_BOUNDS_READER(rowwise)

JLLM_EXPORT int jllm_embed_rows(const int* ids, const void* table, int table_dtype, float* x, int rows, int dim,
                                int vocab, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0 && vocab > 0, "embed_rows: rows=%d dim=%d vocab=%d", rows, dim, vocab);
    if (rows == 0) return JLLM_OK;
    if (table_dtype == JLLM_F32)
        embed_rows_kernel<float><<<rows, 256, 0, stream>>>(ids, (const float*)table, x, dim, vocab);
    else
        embed_rows_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>(ids, (const __nv_bfloat16*)table, x, dim, vocab);
    return jllm_check_launch("embed_rows");
}

// ---------------------------------------------------------------------------------------------------
// ids[r] < 0 stands for "row -ids[r] - 1 of the tokens the step before sampled" (still on the device, the host has not
// read them yet): put them in place. One block; a step has at most some hundreds of rows.
// ---------------------------------------------------------------------------------------------------
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ sampled, int rows, int sampled_rows) {
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
        const int t = ids[r];
        if (t < 0) {
            const int j = -t - 1;
            ids[r] = j < sampled_rows ? sampled[j] : 0;
        }
    }
}

JLLM_EXPORT int jllm_feed_tokens(int* ids, const int* sampled, int rows, int sampled_rows, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && sampled_rows >= 0, "feed_tokens: rows=%d sampled=%d", rows, sampled_rows);
    if (rows == 0) return JLLM_OK;
    feed_tokens_kernel<<<1, 256, 0, stream>>>(ids, sampled, rows, sampled_rows);
    return jllm_check_launch("feed_tokens");
}

// ---------------------------------------------------------------------------------------------------
// RMSNorm: out[r] = (x[src(r)] * (1 / sqrt(mean(x^2) + eps))) * gain, src(r) = row_index ? row_index[r] : r
// The scale is taken in double from a float mean, as the reference does.
// ---------------------------------------------------------------------------------------------------
// (rms_scale: head_rotate.cuh)

template <typename Tout>
__global__ void rmsnorm_kernel(const float* __restrict__ x, VecRef gain, Tout* __restrict__ out,
                               const int* __restrict__ row_index, int dim, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(row_index ? row_index[r] : r) * dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = src[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float s = rms_scale(ss, dim, eps);
    Tout* dst = out + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = from_float<Tout>(__fmul_rn(__fmul_rn(src[i], s), gain[i]));
}

// The same for widths that are a multiple of 4 and at most 8192: the row is read once, as float4, and kept in
// registers between the sum of squares and the scaling.
template <typename Tout>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(const float* __restrict__ x, VecRef gain, Tout* __restrict__ out, const int* __restrict__ row_index,
                   int dim, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, n4 = dim >> 2;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(row_index ? row_index[r] : r) * dim);
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + 256 * j;
        v[j] = i < n4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[j].x, v[j].x, ss);
        ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss);
        ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float s = rms_scale(ss, dim, eps);
    Tout* dst = out + (size_t)r * dim;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i >= n4) break;
        const float a = __fmul_rn(__fmul_rn(v[j].x, s), gain[4 * i + 0]), b = __fmul_rn(__fmul_rn(v[j].y, s), gain[4 * i + 1]);
        const float c = __fmul_rn(__fmul_rn(v[j].z, s), gain[4 * i + 2]), d = __fmul_rn(__fmul_rn(v[j].w, s), gain[4 * i + 3]);
        if constexpr (sizeof(Tout) == 4) {
            reinterpret_cast<float4*>(dst)[i] = make_float4(a, b, c, d);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
            uint2 p;
            p.x = *reinterpret_cast<uint32_t*>(&lo);
            p.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(dst)[i] = p;
        }
    }
}

JLLM_EXPORT int jllm_rmsnorm(const float* x, const void* gain, int gain_dtype, void* out, int out_dtype,
                             const int* row_index, int rows, int dim, float eps, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0, "rmsnorm: rows=%d dim=%d", rows, dim);
    if (rows == 0) return JLLM_OK;
    const VecRef g{gain, gain_dtype};
    if (dim % 4 == 0 && dim <= 8192 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        if (out_dtype == JLLM_F32)
            jllm_launch(rmsnorm_vec_kernel<float>, dim3(rows), dim3(256), 0, stream, true, x, g, (float*)out, row_index, dim,
                        eps);
        else
            jllm_launch(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, true, x, g,
                        (__nv_bfloat16*)out, row_index, dim, eps);
        return jllm_check_launch("rmsnorm");
    }
    const int threads = dim >= 2048 ? 512 : 256;
    if (out_dtype == JLLM_F32)
        jllm_launch(rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, stream, true, x, g, (float*)out, row_index, dim, eps);
    else
        jllm_launch(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, true, x, g, (__nv_bfloat16*)out,
                    row_index, dim, eps);
    return jllm_check_launch("rmsnorm");
}

// ---------------------------------------------------------------------------------------------------
// Dynamic Tanh: out[r] = tanh(a * x[src(r)]) * w + b, src(r) = row_index ? row_index[r] : r. A norm without statistics:
// no mean, no variance, no reduction; a is one scalar per norm.
// ---------------------------------------------------------------------------------------------------
template <typename Tout>
__global__ void __launch_bounds__(256)
dynamic_tanh_kernel(const float* __restrict__ x, VecRef w, VecRef b, float a, Tout* __restrict__ out,
                    const int* __restrict__ row_index, int dim) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(row_index ? row_index[r] : r) * dim;
    Tout* dst = out + (size_t)r * dim;
    if ((dim & 3) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15u) == 0) {      // four values a thread at a time
        for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            const float y0 = __fadd_rn(__fmul_rn(tanhf(__fmul_rn(a, v.x)), w[i]), b[i]);
            const float y1 = __fadd_rn(__fmul_rn(tanhf(__fmul_rn(a, v.y)), w[i + 1]), b[i + 1]);
            const float y2 = __fadd_rn(__fmul_rn(tanhf(__fmul_rn(a, v.z)), w[i + 2]), b[i + 2]);
            const float y3 = __fadd_rn(__fmul_rn(tanhf(__fmul_rn(a, v.w)), w[i + 3]), b[i + 3]);
            if constexpr (sizeof(Tout) == 4) {
                *reinterpret_cast<float4*>(dst + i) = make_float4(y0, y1, y2, y3);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
                uint2 p;
                p.x = *reinterpret_cast<uint32_t*>(&lo);
                p.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst + i) = p;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        dst[i] = from_float<Tout>(__fadd_rn(__fmul_rn(tanhf(__fmul_rn(a, src[i])), w[i]), b[i]));
}

JLLM_EXPORT int jllm_dynamic_tanh(const float* x, const void* w, const void* b, int vec_dtype, float a, void* out,
                                  int out_dtype, const int* row_index, int rows, int dim, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0, "dynamic_tanh: rows=%d dim=%d", rows, dim);
    if (rows == 0) return JLLM_OK;
    const VecRef wv{w, vec_dtype}, bv{b, vec_dtype};
    if (out_dtype == JLLM_F32)
        jllm_launch(dynamic_tanh_kernel<float>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, wv, bv, a, (float*)out,
                    row_index, dim);
    else
        jllm_launch(dynamic_tanh_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, wv, bv, a,
                    (__nv_bfloat16*)out, row_index, dim);
    return jllm_check_launch("dynamic_tanh");
}

// ---------------------------------------------------------------------------------------------------
// x += scale * y (float32, elementwise): the residual sum of a part that cannot scale its own result
// ---------------------------------------------------------------------------------------------------
__global__ void add_scaled_kernel(float* __restrict__ x, const float* __restrict__ y, float scale, size_t total) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] = fmaf(scale, y[i], x[i]);
}

JLLM_EXPORT int jllm_add_scaled(float* x, const float* y, float scale, long long total, cudaStream_t stream) {
    JLLM_REQUIRE(total >= 0, "add_scaled: total=%lld", total);
    if (total == 0) return JLLM_OK;
    const int blocks = (int)min((long long)65535, (total + 255) / 256);
    jllm_launch(add_scaled_kernel, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, y, scale, (size_t)total);
    return jllm_check_launch("add_scaled");
}

// ---------------------------------------------------------------------------------------------------
// Gated hidden units: h[r, j] = act(gate_up[r, j]) * gate_up[r, hidden + j], act = silu (kind 1) or the tanh form of GELU (kind 2)
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ h, int hidden, size_t total, int kind) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / hidden, j = i - r * hidden;
        const float g = to_float(gate_up[r * 2 * hidden + j]);
        const float u = to_float(gate_up[r * 2 * hidden + hidden + j]);
        h[i] = from_float<T>(__fmul_rn(glu_act<false>(g, kind), u));
    }
}

JLLM_EXPORT int jllm_swiglu(const void* gate_up, void* h, int dtype, int rows, int hidden, int kind, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && hidden > 0, "swiglu: rows=%d hidden=%d", rows, hidden);
    if (rows == 0) return JLLM_OK;
    const size_t total = (size_t)rows * hidden;
    const size_t most = (size_t)(jllm_device_sm_count() > 0 ? jllm_device_sm_count() : 1) * 16;   // the kernel strides
    const int blocks = (int)((total + 255) / 256 > most ? most : (total + 255) / 256);
    if (dtype == JLLM_F32)
        jllm_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, true, (const float*)gate_up, (float*)h, hidden,
                    total, kind);
    else
        jllm_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, true, (const __nv_bfloat16*)gate_up,
                    (__nv_bfloat16*)h, hidden, total, kind);
    return jllm_check_launch("swiglu");
}

// ---------------------------------------------------------------------------------------------------
// Per (row, head): optional RMSNorm over the head, rotate-half RoPE over the first rotary_dim values,
// then queries go back in place and keys / values go into the paged cache.
//
// qkv is [rows, row_stride] with queries, keys, values side by side ((heads + 2 kv_heads) * head_dim values;
// heads * head_dim when the run reads another run's cache and writes no keys or values). The cache of one layer run is
// K[pages, kv_heads, page_size, head_dim] and V alike; row r is written at slot[r] = page * page_size + offset.
// cos/sin are [positions, rotary_dim / 2] float tables (angles made in double on the host).
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_rope_store_kernel(T* __restrict__ qkv, VecRef q_gain, VecRef k_gain, int use_norm, float eps,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          int rotary_dim, const int* __restrict__ positions,
                                          const int* __restrict__ slots, T* __restrict__ k_cache,
                                          T* __restrict__ v_cache, int heads, int kv_heads, int head_dim,
                                          int page_size, int num_slots, int row_stride) {
    extern __shared__ float vec[];  // head_dim floats + 33 scratch
    float* scratch = vec + head_dim;
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, h = blockIdx.y;
    T* src = qkv + (size_t)r * row_stride + (size_t)h * head_dim;
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) vec[i] = to_float(src[i]);
    __syncthreads();
    if (is_q || is_k) {
        if (use_norm) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < head_dim; i += blockDim.x) ss = fmaf(vec[i], vec[i], ss);
            ss = block_sum(ss, scratch);
            const float s = rms_scale(ss, head_dim, eps);
            const VecRef g = is_q ? q_gain : k_gain;
            for (int i = threadIdx.x; i < head_dim; i += blockDim.x) vec[i] = __fmul_rn(__fmul_rn(vec[i], s), g[i]);
            __syncthreads();
        }
        if (rotary_dim > 0) {
            const int half = rotary_dim >> 1;
            const float* c = cos_t + (size_t)positions[r] * half;
            const float* s = sin_t + (size_t)positions[r] * half;
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const float a = vec[i], b = vec[i + half];
                vec[i] = __fsub_rn(__fmul_rn(a, c[i]), __fmul_rn(b, s[i]));
                vec[i + half] = __fadd_rn(__fmul_rn(b, c[i]), __fmul_rn(a, s[i]));
            }
            __syncthreads();
        }
    }
    if (is_q) {
        for (int i = threadIdx.x; i < head_dim; i += blockDim.x) src[i] = from_float<T>(vec[i]);
    } else {
        const int kvh = is_k ? h - heads : h - heads - kv_heads;
        const int slot = slots[r];
        if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;      // checked build: the write is dropped
        const size_t page = slot / page_size, off = slot % page_size;
        T* dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + kvh) * page_size + off) * head_dim;
        for (int i = threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = from_float<T>(vec[i]);
    }
}

// The same with one warp per (row, head), for head sizes 64, 128 and 256 rotated over their whole width: lane l
// owns V = head_dim / 64 neighbouring values of the first half and their partners in the second half, so the
// rotation needs no exchange and the sum of squares is a warp shuffle; 8 heads per block, no shared memory.
template <typename T, int V>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_warp_kernel(T* __restrict__ qkv, VecRef q_gain, VecRef k_gain, int use_norm, float eps,
                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                               const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ k_cache,
                               T* __restrict__ v_cache, int heads, int kv_heads, int page_size, int num_slots, int row_stride,
                               int heads_total, long long items) {
    constexpr int HD = 64 * V, HALF = 32 * V;
    pdl_wait();
    pdl_trigger();
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= items) return;
    const int r = (int)(item / heads_total), h = (int)(item % heads_total), lane = threadIdx.x & 31;
    T* src = qkv + (size_t)r * row_stride + (size_t)h * HD;
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    float a[V], b[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        a[i] = to_float(src[lane * V + i]);
        b[i] = to_float(src[HALF + lane * V + i]);
    }
    if (is_q || is_k)
        head_norm_rope<V>(a, b, lane, use_norm, eps, is_q ? q_gain : k_gain, cos_t + (size_t)positions[r] * HALF,
                          sin_t + (size_t)positions[r] * HALF);
    T* dst = src;
    if (!is_q) {
        const int kvh = is_k ? h - heads : h - heads - kv_heads;
        const int slot = slots[r];
        if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;      // checked build: the write is dropped
        const size_t page = slot / page_size, off = slot % page_size;
        dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + kvh) * page_size + off) * HD;
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
        dst[lane * V + i] = from_float<T>(a[i]);
        dst[HALF + lane * V + i] = from_float<T>(b[i]);
    }
}

// The same for bfloat16 with 16-byte accesses: 4 V lanes share one (row, head), each owning 8 neighbouring values of
// the first half and their partners in the second half; a warp takes 8 / V heads of a row side by side (they are
// neighbours in memory), so that it has 1 KB of loads in flight instead of 128 bytes. The arithmetic of one value
// is that of the kernels above.
template <int V>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, VecRef q_gain, VecRef k_gain, int use_norm, float eps,
                              const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                              const int* __restrict__ positions, const int* __restrict__ slots,
                              __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int heads,
                              int kv_heads, int page_size, int num_slots, int row_stride, int heads_total, long long items) {
    constexpr int HD = 64 * V, HALF = 32 * V, LANES = 4 * V, PER_WARP = 32 / LANES;
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31, sub = lane % LANES;
    const long long item = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * PER_WARP + lane / LANES;
    const bool live = item < items;
    const int r = live ? (int)(item / heads_total) : 0, h = live ? (int)(item % heads_total) : 0;
    __nv_bfloat16* src = qkv + (size_t)r * row_stride + (size_t)h * HD;
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    float a[8], b[8];
    {
        const uint4 ua = live ? *reinterpret_cast<const uint4*>(src + sub * 8) : make_uint4(0, 0, 0, 0);
        const uint4 ub = live ? *reinterpret_cast<const uint4*>(src + HALF + sub * 8) : make_uint4(0, 0, 0, 0);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ua);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&ub);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
            a[2 * i] = fa.x; a[2 * i + 1] = fa.y;
            b[2 * i] = fb.x; b[2 * i + 1] = fb.y;
        }
    }
    if (is_q || is_k) {
        if (use_norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(a[i], a[i], ss);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(b[i], b[i], ss);
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float s = rms_scale(ss, HD, eps);
            const VecRef g = is_q ? q_gain : k_gain;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                a[i] = __fmul_rn(__fmul_rn(a[i], s), g[sub * 8 + i]);
                b[i] = __fmul_rn(__fmul_rn(b[i], s), g[HALF + sub * 8 + i]);
            }
        }
        const float4* c4 = reinterpret_cast<const float4*>(cos_t + (size_t)positions[r] * HALF + sub * 8);
        const float4* s4 = reinterpret_cast<const float4*>(sin_t + (size_t)positions[r] * HALF + sub * 8);
        const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x0 = a[i], x1 = b[i];
            a[i] = __fsub_rn(__fmul_rn(x0, c[i]), __fmul_rn(x1, sn[i]));
            b[i] = __fadd_rn(__fmul_rn(x1, c[i]), __fmul_rn(x0, sn[i]));
        }
    }
    if (!live) return;
    __nv_bfloat16* dst = src;
    if (!is_q) {
        const int kvh = is_k ? h - heads : h - heads - kv_heads;
        const int slot = slots[r];
        if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;      // checked build: the write is dropped
        const size_t page = slot / page_size, off = slot % page_size;
        dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + kvh) * page_size + off) * HD;
    }
    uint4 oa, ob;
    __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
    __nv_bfloat162* qb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        qa[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
        qb[i] = __floats2bfloat162_rn(b[2 * i], b[2 * i + 1]);
    }
    *reinterpret_cast<uint4*>(dst + sub * 8) = oa;
    *reinterpret_cast<uint4*>(dst + HALF + sub * 8) = ob;
}

JLLM_EXPORT int jllm_qk_norm_rope_store(void* qkv, int dtype, const void* q_gain, const void* k_gain, int gain_dtype,
                                        int use_norm, float eps, const float* cos_t, const float* sin_t,
                                        int rotary_dim, const int* positions, const int* slots, void* k_cache,
                                        void* v_cache, int write_kv, int rows, int row_stride, int heads, int kv_heads,
                                        int head_dim, int page_size, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && kv_heads > 0 && head_dim > 0 && page_size > 0,
                 "qk_norm_rope_store: rows=%d heads=%d kv_heads=%d head_dim=%d page_size=%d", rows, heads, kv_heads,
                 head_dim, page_size);
    JLLM_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim,
                 "qk_norm_rope_store: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, head_dim);
    JLLM_REQUIRE(row_stride >= (write_kv ? heads + 2 * kv_heads : heads) * head_dim,
                 "qk_norm_rope_store: row_stride=%d is too small", row_stride);
    JLLM_REQUIRE(head_dim <= 8192, "qk_norm_rope_store: head_dim=%d is above 8192", head_dim);
    if (rows == 0) return JLLM_OK;
    const int num_slots = (int)min((long long)jllm_pool_pages() * page_size, 2147483647ll);   // 0 = not known
    const dim3 grid(rows, write_kv ? heads + 2 * kv_heads : heads);
    const int threads = head_dim <= 64 ? 32 : (head_dim <= 128 ? 64 : 128);
    const size_t smem = (head_dim + 33) * sizeof(float);
    const VecRef qg{q_gain, gain_dtype}, kg{k_gain, gain_dtype};
    if ((head_dim == 64 || head_dim == 128 || head_dim == 256) && rotary_dim == head_dim) {
        const int heads_total = write_kv ? heads + 2 * kv_heads : heads;
        const long long items = (long long)rows * heads_total;
        const dim3 wgrid((unsigned)((items + 7) / 8));
#define JLLM_WARP_ROPE(T, V)                                                                                          \
    jllm_launch(qk_norm_rope_store_warp_kernel<T, V>, wgrid, dim3(256), 0, stream, true, (T*)qkv, qg, kg, use_norm, eps, \
                cos_t, sin_t, positions, slots, (T*)k_cache, (T*)v_cache, heads, kv_heads, page_size, num_slots, row_stride,      \
                heads_total, items)
        const int v = head_dim / 64;
        // the 16-byte kernel from 32 rows on (fewer rows are too few warps for it; JLLM_B200_ROPE_VEC_MIN_ROWS moves that)
        static const int vec_min_rows = [] {
            const char* e = getenv("JLLM_B200_ROPE_VEC_MIN_ROWS");
            return e ? atoi(e) : 32;
        }();
        if (dtype == JLLM_BF16 && rows >= vec_min_rows && row_stride % 8 == 0 && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)k_cache % 16) == 0 &&
            ((uintptr_t)v_cache % 16) == 0 && ((uintptr_t)cos_t % 16) == 0 && ((uintptr_t)sin_t % 16) == 0) {
            const long long per_block = 8 * (8 / v);
            const dim3 vgrid((unsigned)((items + per_block - 1) / per_block));
#define JLLM_VEC_ROPE(V)                                                                                              \
    jllm_launch(qk_norm_rope_store_vec_kernel<V>, vgrid, dim3(256), 0, stream, true, (__nv_bfloat16*)qkv, qg, kg,     \
                use_norm, eps, cos_t, sin_t, positions, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, heads, \
                kv_heads, page_size, num_slots, row_stride, heads_total, items)
            if (v == 1) JLLM_VEC_ROPE(1); else if (v == 2) JLLM_VEC_ROPE(2); else JLLM_VEC_ROPE(4);
#undef JLLM_VEC_ROPE
            return jllm_check_launch("qk_norm_rope_store");
        }
        if (dtype == JLLM_F32) {
            if (v == 1) JLLM_WARP_ROPE(float, 1); else if (v == 2) JLLM_WARP_ROPE(float, 2); else JLLM_WARP_ROPE(float, 4);
        } else {
            if (v == 1) JLLM_WARP_ROPE(__nv_bfloat16, 1); else if (v == 2) JLLM_WARP_ROPE(__nv_bfloat16, 2);
            else JLLM_WARP_ROPE(__nv_bfloat16, 4);
        }
#undef JLLM_WARP_ROPE
        return jllm_check_launch("qk_norm_rope_store");
    }
    if (dtype == JLLM_F32)
        jllm_launch(qk_norm_rope_store_kernel<float>, grid, dim3(threads), smem, stream, true,
            (float*)qkv, qg, kg, use_norm, eps, cos_t, sin_t, rotary_dim, positions, slots, (float*)k_cache,
            (float*)v_cache, heads, kv_heads, head_dim, page_size, num_slots, row_stride);
    else
        jllm_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, true,
            (__nv_bfloat16*)qkv, qg, kg, use_norm, eps, cos_t, sin_t, rotary_dim, positions, slots,
            (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, heads, kv_heads, head_dim, page_size, num_slots, row_stride);
    return jllm_check_launch("qk_norm_rope_store");
}

// ---------------------------------------------------------------------------------------------------
// The general form of the per-head preparation, for mixers whose heads the kernel above does not take: key and value
// heads of different widths, rotation of interleaved pairs, a unit norm behind the rotation. One warp per (row, head),
// the head's values in the warp's slice of shared memory, in this order:
//   1. (pre_norm) RMSNorm over the head with the gains q_gain / k_gain;
//   2. rotation of the first rotary_dim values by the angles of the row's position, pair i = (i, i + rotary_dim / 2)
//      ("half", pairing 0) or (2i, 2i + 1) ("interleaved", pairing 1);
//   3. (post_norm) the head divided by its root mean square (no gain).
// Queries go back in place; keys and values go into the paged cache, whose rows are cache_dim wide (keys fill the
// first key_dim values of a row, values the first value_dim). qkv [rows, row_stride]: queries at column q_off (heads x
// key_dim), keys at k_off (kv_heads x key_dim), values at v_off (kv_heads x value_dim).
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename T>
__global__ void __launch_bounds__(256)
head_prepare_kernel(T* __restrict__ qkv, int row_stride, int q_off, int k_off, int v_off, VecRef q_gain, VecRef k_gain,
                    int pre_norm, int post_norm, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                    int rotary_dim, int pairing, const int* __restrict__ positions, const int* __restrict__ slots,
                    T* __restrict__ k_cache, T* __restrict__ v_cache, int heads, int kv_heads, int key_dim, int value_dim,
                    int cache_dim, int page_size, int num_slots, int heads_total, long long items, int width) {
    extern __shared__ float head_smem[];
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= items) return;
    float* vec = head_smem + (size_t)(threadIdx.x >> 5) * width;
    const int r = (int)(item / heads_total), h = (int)(item % heads_total);
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    const int n = is_q || is_k ? key_dim : value_dim;
    T* src = qkv + (size_t)r * row_stride +
             (is_q ? q_off + (size_t)h * key_dim
                   : is_k ? k_off + (size_t)(h - heads) * key_dim : v_off + (size_t)(h - heads - kv_heads) * value_dim);
    // (two values a lane and access where the row allows it: half as many loads and stores)
    const bool pairs = (n & 1) == 0 && (((uintptr_t)src) & (2 * sizeof(T) - 1)) == 0;
    if (pairs) {
        for (int i = lane; i < n / 2; i += 32) {
            const float2 v = load_pair(src + 2 * i);
            vec[2 * i] = v.x;
            vec[2 * i + 1] = v.y;
        }
    } else {
        for (int i = lane; i < n; i += 32) vec[i] = to_float(src[i]);
    }
    __syncwarp();
    if (is_q || is_k) {
        if (pre_norm) {
            float ss = 0.f;
            for (int i = lane; i < n; i += 32) ss = fmaf(vec[i], vec[i], ss);
            const float s = rms_scale(warp_sum(ss), n, eps);
            const VecRef g = is_q ? q_gain : k_gain;
            for (int i = lane; i < n; i += 32) vec[i] = __fmul_rn(__fmul_rn(vec[i], s), g[i]);
            __syncwarp();
        }
        if (rotary_dim > 0) {
            const int half = rotary_dim >> 1;
            const float* c = cos_t + (size_t)positions[r] * half;
            const float* s = sin_t + (size_t)positions[r] * half;
            for (int i = lane; i < half; i += 32) {
                const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
                const float a = vec[ia], b = vec[ib];
                vec[ia] = __fsub_rn(__fmul_rn(a, c[i]), __fmul_rn(b, s[i]));
                vec[ib] = __fadd_rn(__fmul_rn(b, c[i]), __fmul_rn(a, s[i]));
            }
            __syncwarp();
        }
        if (post_norm) {
            float ss = 0.f;
            for (int i = lane; i < n; i += 32) ss = fmaf(vec[i], vec[i], ss);
            const float s = rms_scale(warp_sum(ss), n, eps);
            for (int i = lane; i < n; i += 32) vec[i] = __fmul_rn(vec[i], s);
            __syncwarp();
        }
    }
    T* dst = src;
    if (!is_q) {
        const int kvh = is_k ? h - heads : h - heads - kv_heads;
        const int slot = slots[r];
        if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;      // checked build: the write is dropped
        const size_t page = slot / page_size, off = slot % page_size;
        dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + kvh) * page_size + off) * cache_dim;
    }
    if (pairs && (((uintptr_t)dst) & (2 * sizeof(T) - 1)) == 0) {
        for (int i = lane; i < n / 2; i += 32) store_pair(dst + 2 * i, vec[2 * i], vec[2 * i + 1]);
    } else {
        for (int i = lane; i < n; i += 32) dst[i] = from_float<T>(vec[i]);
    }
}

// The same for bfloat16 heads of 64, 128 or 256 values of one width (key_dim = value_dim = cache_dim = 8 * LANES): a head
// in the registers of LANES lanes, 8 neighbouring values and one 16-byte access each, 32 / LANES heads a warp. An
// interleaved pair lies inside a lane; the partner of a half pair lies rotary_dim / 16 lanes away (rotary_dim a multiple
// of 16) and comes by shuffles. Value by value the arithmetic is that of the kernel above; the sums of squares are grouped
// by lane.
template <int LANES>
__global__ void __launch_bounds__(256)
head_prepare_vec_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride, int q_off, int k_off, int v_off, VecRef q_gain,
                        VecRef k_gain, int pre_norm, int post_norm, float eps, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, int rotary_dim, int pairing, const int* __restrict__ positions,
                        const int* __restrict__ slots, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                        int heads, int kv_heads, int page_size, int num_slots, int heads_total, long long items) {
    constexpr int HD = 8 * LANES, PER_WARP = 32 / LANES;
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31, sub = lane % LANES;
    const long long item = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * PER_WARP + lane / LANES;
    const bool live = item < items;
    const int r = live ? (int)(item / heads_total) : 0, h = live ? (int)(item % heads_total) : 0;
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    __nv_bfloat16* src = qkv + (size_t)r * row_stride +
                         (is_q ? q_off + (size_t)h * HD : is_k ? k_off + (size_t)(h - heads) * HD
                                                               : v_off + (size_t)(h - heads - kv_heads) * HD);
    float x[8];
    {
        const uint4 u = live ? *reinterpret_cast<const uint4*>(src + sub * 8) : make_uint4(0, 0, 0, 0);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p[i]);
            x[2 * i] = f.x;
            x[2 * i + 1] = f.y;
        }
    }
    auto group_sum = [&](float v) {
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
    };
    const bool turns = is_q || is_k;      // (values are only copied; all lanes still take part in the shuffles)
    if (pre_norm) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
        const float s = rms_scale(group_sum(ss), HD, eps);
        const VecRef g = is_q ? q_gain : k_gain;
        if (turns) {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(__fmul_rn(x[i], s), g[sub * 8 + i]);
        }
    }
    if (rotary_dim > 0) {
        const int half = rotary_dim >> 1, e0 = sub * 8;
        const float* c = cos_t + (size_t)positions[r] * half;
        const float* sn = sin_t + (size_t)positions[r] * half;
        if (pairing) {       // pairs (2i, 2i + 1): inside the lane
            if (turns && e0 < rotary_dim) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int pr = e0 / 2 + i;
                    const float a = x[2 * i], b = x[2 * i + 1];
                    x[2 * i] = __fsub_rn(__fmul_rn(a, c[pr]), __fmul_rn(b, sn[pr]));
                    x[2 * i + 1] = __fadd_rn(__fmul_rn(b, c[pr]), __fmul_rn(a, sn[pr]));
                }
            }
        } else {             // pairs (i, i + half): the partner's 8 values lie half / 8 lanes up or down
            const int shift = half >> 3;
            const bool low = e0 < half, in = e0 < rotary_dim;
            const int from = (lane / LANES) * LANES + (low ? sub + shift : sub - shift);
            float y[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = __shfl_sync(0xffffffffu, x[i], (in ? from : lane) & 31);
            if (turns && in) {
                const int p0 = low ? e0 : e0 - half;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // low: (a, b) = (mine, partner) -> a cos - b sin; high: (a, b) = (partner, mine) -> b cos + a sin
                    x[i] = low ? __fsub_rn(__fmul_rn(x[i], c[p0 + i]), __fmul_rn(y[i], sn[p0 + i]))
                               : __fadd_rn(__fmul_rn(x[i], c[p0 + i]), __fmul_rn(y[i], sn[p0 + i]));
                }
            }
        }
    }
    if (post_norm) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
        const float s = rms_scale(group_sum(ss), HD, eps);
        if (turns) {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], s);
        }
    }
    if (!live) return;
    __nv_bfloat16* dst = src;
    if (!is_q) {
        const int kvh = is_k ? h - heads : h - heads - kv_heads;
        const int slot = slots[r];
        if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;      // checked build: the write is dropped
        const size_t page = slot / page_size, off = slot % page_size;
        dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + kvh) * page_size + off) * HD;
    }
    uint4 o;
    __nv_bfloat162* q2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) q2[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    *reinterpret_cast<uint4*>(dst + sub * 8) = o;
}

JLLM_EXPORT int jllm_head_prepare(void* qkv, int dtype, int row_stride, int q_off, int k_off, int v_off, const void* q_gain,
                                  const void* k_gain, int gain_dtype, int pre_norm, int post_norm, float eps,
                                  const float* cos_t, const float* sin_t, int rotary_dim, int pairing, const int* positions,
                                  const int* slots, void* k_cache, void* v_cache, int write_kv, int rows, int heads,
                                  int kv_heads, int key_dim, int value_dim, int cache_dim, int page_size,
                                  cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && kv_heads > 0 && key_dim > 0 && value_dim > 0 && page_size > 0,
                 "head_prepare: rows=%d heads=%d kv_heads=%d key_dim=%d value_dim=%d page_size=%d", rows, heads, kv_heads,
                 key_dim, value_dim, page_size);
    JLLM_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= key_dim && (pairing == 0 || pairing == 1),
                 "head_prepare: rotary_dim=%d must be even and at most key_dim=%d; pairing=%d", rotary_dim, key_dim, pairing);
    JLLM_REQUIRE(!write_kv || (cache_dim >= key_dim && cache_dim >= value_dim),
                 "head_prepare: cache rows of %d values do not hold keys of %d and values of %d", cache_dim, key_dim, value_dim);
    JLLM_REQUIRE(!pre_norm || (q_gain && k_gain), "head_prepare: a norm with gains needs both gains");
    const int width = key_dim > value_dim ? key_dim : value_dim;
    JLLM_REQUIRE(width <= 4096, "head_prepare: a head of %d values is above 4096", width);
    if (rows == 0) return JLLM_OK;
    const int num_slots = (int)min((long long)jllm_pool_pages() * page_size, 2147483647ll);   // 0 = not known
    const int heads_total = write_kv ? heads + 2 * kv_heads : heads;
    const long long items = (long long)rows * heads_total;
    const dim3 grid((unsigned)((items + 7) / 8));
    const size_t smem = (size_t)8 * width * sizeof(float);
    const VecRef qg{q_gain, gain_dtype}, kg{k_gain, gain_dtype};
    if (dtype == JLLM_BF16 && key_dim == value_dim && (!write_kv || cache_dim == key_dim) &&
        (key_dim == 64 || key_dim == 128 || key_dim == 256) && (pairing ? rotary_dim % 8 == 0 : rotary_dim % 16 == 0) &&
        row_stride % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 && ((uintptr_t)qkv % 16) == 0 &&
        ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0) {
        const int lanes = key_dim / 8;
        const long long per_block = 8 * (32 / lanes);
        const dim3 vgrid((unsigned)((items + per_block - 1) / per_block));
#define JLLM_HEAD_VEC(L)                                                                                                      \
    jllm_launch(head_prepare_vec_kernel<L>, vgrid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (__nv_bfloat16*)qkv, row_stride, q_off, \
                k_off, v_off, qg, kg, pre_norm, post_norm, eps, cos_t, sin_t, rotary_dim, pairing, positions, slots,              \
                (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, heads, kv_heads, page_size, num_slots, heads_total, items)
        if (lanes == 8) JLLM_HEAD_VEC(8); else if (lanes == 16) JLLM_HEAD_VEC(16); else JLLM_HEAD_VEC(32);
#undef JLLM_HEAD_VEC
        return jllm_check_launch("head_prepare");
    }
    if (dtype == JLLM_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(head_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        jllm_launch(head_prepare_kernel<float>, grid, dim3(256), smem, stream, LAUNCH_DEPENDENT, (float*)qkv, row_stride, q_off,
                    k_off, v_off, qg, kg, pre_norm, post_norm, eps, cos_t, sin_t, rotary_dim, pairing, positions, slots,
                    (float*)k_cache, (float*)v_cache, heads, kv_heads, key_dim, value_dim, cache_dim, page_size, num_slots,
                    heads_total, items, width);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(head_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        jllm_launch(head_prepare_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, LAUNCH_DEPENDENT, (__nv_bfloat16*)qkv,
                    row_stride, q_off, k_off, v_off, qg, kg, pre_norm, post_norm, eps, cos_t, sin_t, rotary_dim, pairing,
                    positions, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, heads, kv_heads, key_dim, value_dim,
                    cache_dim, page_size, num_slots, heads_total, items, width);
    }
    return jllm_check_launch("head_prepare");
}

// ---------------------------------------------------------------------------------------------------
// out[r, h, :] *= sigmoid(gate[r, h]): one gate value per row and head on the attention's result (heads x value_dim
// values a row), the gate a column block of the mixer's stacked input product. In place.
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ att, int ld_att, const T* __restrict__ gate, int ld_gate, int heads,
                                 int value_dim, size_t total) {
    pdl_wait();
    pdl_trigger();
    const size_t per_row = (size_t)heads * value_dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / per_row, c = i - r * per_row;
        const float g = to_float(gate[r * ld_gate + c / value_dim]);
        T* p = att + r * ld_att + c;
        *p = from_float<T>(__fmul_rn(to_float(*p), 1.f / (1.f + expf(-g))));
    }
}

// The same for bfloat16 rows whose heads are whole 16-byte pieces: a thread takes 8 values of one head.
__global__ void __launch_bounds__(256)
head_gate_vec_kernel(__nv_bfloat16* __restrict__ att, int ld_att, const __nv_bfloat16* __restrict__ gate, int ld_gate,
                     int value_dim, int pieces_per_row, unsigned total) {
    pdl_wait();
    pdl_trigger();
    const unsigned i = blockIdx.x * 256u + threadIdx.x;
    if (i >= total) return;
    const unsigned r = i / pieces_per_row, c = (i - r * pieces_per_row) * 8;
    const float g = __bfloat162float(gate[(size_t)r * ld_gate + c / value_dim]);
    const float f = 1.f / (1.f + expf(-g));
    uint4* p = reinterpret_cast<uint4*>(att + (size_t)r * ld_att + c);
    uint4 v = *p;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(__fmul_rn(x.x, f), __fmul_rn(x.y, f));
    }
    *p = v;
}

JLLM_EXPORT int jllm_head_gate(void* att, int dtype, int ld_att, const void* gate, int ld_gate, int rows, int heads,
                               int value_dim, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && value_dim > 0, "head_gate: rows=%d heads=%d value_dim=%d", rows, heads, value_dim);
    if (rows == 0) return JLLM_OK;
    if (dtype == JLLM_BF16 && value_dim % 8 == 0 && ld_att % 8 == 0 && ((uintptr_t)att % 16) == 0 &&
        (long long)rows * heads * value_dim / 8 < 4000000000ll) {
        const int pieces = heads * value_dim / 8;
        const unsigned total_pieces = (unsigned)rows * pieces;
        jllm_launch(head_gate_vec_kernel, dim3((total_pieces + 255) / 256), dim3(256), 0, stream, LAUNCH_DEPENDENT,
                    (__nv_bfloat16*)att, ld_att, (const __nv_bfloat16*)gate, ld_gate, value_dim, pieces, total_pieces);
        return jllm_check_launch("head_gate");
    }
    const size_t total = (size_t)rows * heads * value_dim;
    const size_t most = (size_t)(jllm_device_sm_count() > 0 ? jllm_device_sm_count() : 1) * 16;
    const int blocks = (int)((total + 255) / 256 > most ? most : (total + 255) / 256);
    if (dtype == JLLM_F32)
        jllm_launch(head_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, (float*)att, ld_att,
                    (const float*)gate, ld_gate, heads, value_dim, total);
    else
        jllm_launch(head_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, (__nv_bfloat16*)att,
                    ld_att, (const __nv_bfloat16*)gate, ld_gate, heads, value_dim, total);
    return jllm_check_launch("head_gate");
}

// ---------------------------------------------------------------------------------------------------
// Norms behind a part: x[r] += scale * (rmsnorm(a[r]) * gain_a  [+ rmsnorm(b[r]) * gain_b]), all float32 rows of
// `dim` values. With one input it is the norm between a part's result and the residual sum; with two (and scale 1/2) the
// mean of two normed results. `accumulate` 0 writes x instead of adding to it. A block per row; the row is read twice.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
norm_sum_kernel(float* __restrict__ x, const float* __restrict__ a, VecRef gain_a, const float* __restrict__ b, VecRef gain_b,
                int dim, float eps, float scale, int accumulate) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const size_t row = (size_t)blockIdx.x * dim;
    const float* pa = a + row;
    const float* pb = b ? b + row : nullptr;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        sa = fmaf(pa[i], pa[i], sa);
        if (pb) sb = fmaf(pb[i], pb[i], sb);
    }
    sa = block_sum(sa, scratch);
    const float ra = rms_scale(sa, dim, eps);
    float rb = 0.f;
    if (pb) {
        sb = block_sum(sb, scratch);
        rb = rms_scale(sb, dim, eps);
    }
    float* px = x + row;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = __fmul_rn(__fmul_rn(pa[i], ra), gain_a[i]);
        if (pb) v = __fadd_rn(v, __fmul_rn(__fmul_rn(pb[i], rb), gain_b[i]));
        v = __fmul_rn(v, scale);
        px[i] = accumulate ? __fadd_rn(px[i], v) : v;
    }
}

// The same with the rows in registers between the sums and the results: a thread owns V groups of four neighbouring values
// of each row (dim a multiple of 4, at most 256 x 4 V values), every row is read once and all of a thread's loads are on their
// way together. The same arithmetic in the same order per value; the sums of squares are grouped by thread, as above.
template <int V>
__global__ void __launch_bounds__(256)
norm_sum_vec_kernel(float* __restrict__ x, const float* __restrict__ a, VecRef gain_a, const float* __restrict__ b, VecRef gain_b,
                    int dim, float eps, float scale, int accumulate) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const size_t row = (size_t)blockIdx.x * dim;
    const int groups = dim >> 2;
    float4 va[V], vb[V];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int u = 0; u < V; ++u) {
        const int gi = threadIdx.x + u * 256;
        va[u] = gi < groups ? *reinterpret_cast<const float4*>(a + row + 4 * gi) : make_float4(0.f, 0.f, 0.f, 0.f);
        vb[u] = (b && gi < groups) ? *reinterpret_cast<const float4*>(b + row + 4 * gi) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < V; ++u) {
        sa = fmaf(va[u].x, va[u].x, sa); sa = fmaf(va[u].y, va[u].y, sa); sa = fmaf(va[u].z, va[u].z, sa); sa = fmaf(va[u].w, va[u].w, sa);
        sb = fmaf(vb[u].x, vb[u].x, sb); sb = fmaf(vb[u].y, vb[u].y, sb); sb = fmaf(vb[u].z, vb[u].z, sb); sb = fmaf(vb[u].w, vb[u].w, sb);
    }
    sa = block_sum(sa, scratch);
    const float ra = rms_scale(sa, dim, eps);
    float rb = 0.f;
    if (b) {
        sb = block_sum(sb, scratch);
        rb = rms_scale(sb, dim, eps);
    }
#pragma unroll
    for (int u = 0; u < V; ++u) {
        const int gi = threadIdx.x + u * 256;
        if (gi >= groups) continue;
        const float pa[4] = {va[u].x, va[u].y, va[u].z, va[u].w}, pb[4] = {vb[u].x, vb[u].y, vb[u].z, vb[u].w};
        float4 old = accumulate ? *reinterpret_cast<const float4*>(x + row + 4 * gi) : make_float4(0.f, 0.f, 0.f, 0.f);
        float res[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = 4 * gi + k;
            float v = __fmul_rn(__fmul_rn(pa[k], ra), gain_a[i]);
            if (b) v = __fadd_rn(v, __fmul_rn(__fmul_rn(pb[k], rb), gain_b[i]));
            v = __fmul_rn(v, scale);
            res[k] = accumulate ? __fadd_rn(res[k], v) : v;
        }
        *reinterpret_cast<float4*>(x + row + 4 * gi) = make_float4(res[0], res[1], res[2], res[3]);
    }
}

JLLM_EXPORT int jllm_norm_sum(float* x, const float* a, const void* gain_a, const float* b, const void* gain_b, int gain_dtype,
                              int rows, int dim, float eps, float scale, int accumulate, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0 && a && gain_a && (!b || gain_b), "norm_sum: rows=%d dim=%d", rows, dim);
    if (rows == 0) return JLLM_OK;
    const bool aligned = dim % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)a % 16) == 0 && (!b || ((uintptr_t)b % 16) == 0);
    if (aligned && dim <= 8192) {
        const int v = (dim / 4 + 255) / 256;
#define JLLM_NORM_SUM(V)                                                                                                   \
    jllm_launch(norm_sum_vec_kernel<V>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, a, VecRef{gain_a, gain_dtype}, b, \
                VecRef{gain_b, gain_dtype}, dim, eps, scale, accumulate)
        if (v <= 1) JLLM_NORM_SUM(1); else if (v <= 2) JLLM_NORM_SUM(2); else if (v <= 4) JLLM_NORM_SUM(4); else JLLM_NORM_SUM(8);
#undef JLLM_NORM_SUM
        return jllm_check_launch("norm_sum");
    }
    jllm_launch(norm_sum_kernel, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, a, VecRef{gain_a, gain_dtype}, b,
                VecRef{gain_b, gain_dtype}, dim, eps, scale, accumulate);
    return jllm_check_launch("norm_sum");
}

// ---------------------------------------------------------------------------------------------------
// The norms between a part's result and the next part's input, in one pass over a row (float32, `dim` values):
//   v = a                                            (one result), or
//   v = scale * (rmsnorm(a) * gain_a + rmsnorm(b) * gain_b)     (two results side by side, each normed)
//   x += rmsnorm(v) * gain_post                      (the norm behind the part, then the residual sum)
//   next = rmsnorm(x) * gain_next                    (optional: the norm in front of the part that follows; `next` has
//                                                     the compute type)
// The same arithmetic, in the same order, as norm_sum (twice) and rmsnorm one after the other. A block per row; the row
// lives in shared memory between the steps.
// ---------------------------------------------------------------------------------------------------
template <typename Tnext>
__global__ void __launch_bounds__(256)
norm_chain_kernel(float* __restrict__ x, const float* __restrict__ a, VecRef gain_a, const float* __restrict__ b, VecRef gain_b,
                  float scale, VecRef gain_post, VecRef gain_next, Tnext* __restrict__ next, int dim, float eps) {
    extern __shared__ float row_smem[];     // dim floats
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const size_t row = (size_t)blockIdx.x * dim;
    const float* pa = a + row;
    if (b) {
        const float* pb = b + row;
        float sa = 0.f, sb = 0.f;
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            sa = fmaf(pa[i], pa[i], sa);
            sb = fmaf(pb[i], pb[i], sb);
        }
        sa = block_sum(sa, scratch);
        sb = block_sum(sb, scratch);
        const float ra = rms_scale(sa, dim, eps), rb = rms_scale(sb, dim, eps);
        for (int i = threadIdx.x; i < dim; i += blockDim.x)
            row_smem[i] = __fmul_rn(__fadd_rn(__fmul_rn(__fmul_rn(pa[i], ra), gain_a[i]), __fmul_rn(__fmul_rn(pb[i], rb), gain_b[i])), scale);
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) row_smem[i] = pa[i];
    }
    // (every thread reads back only what it wrote: no barrier is needed between the steps beyond those of the sums)
    float sv = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) sv = fmaf(row_smem[i], row_smem[i], sv);
    sv = block_sum(sv, scratch);
    const float rv = rms_scale(sv, dim, eps);
    float* px = x + row;
    float sx = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = __fadd_rn(px[i], __fmul_rn(__fmul_rn(row_smem[i], rv), gain_post[i]));
        px[i] = v;
        row_smem[i] = v;
        sx = fmaf(v, v, sx);
    }
    if (next == nullptr) return;
    sx = block_sum(sx, scratch);
    const float rx = rms_scale(sx, dim, eps);
    Tnext* pn = next + row;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) pn[i] = from_float<Tnext>(__fmul_rn(__fmul_rn(row_smem[i], rx), gain_next[i]));
}

// The same with the row in registers (widths that are a multiple of 4, at most 1,024 * V values): a, b and x are all
// requested before anything is computed, so the row pays one trip to memory instead of one per step. Value by value the
// arithmetic is that of the kernel above (the partial sums of squares are grouped by thread as there).
template <typename Tnext, int V>
__global__ void __launch_bounds__(256)
norm_chain_vec_kernel(float* __restrict__ x, const float* __restrict__ a, VecRef gain_a, const float* __restrict__ b,
                      VecRef gain_b, float scale, VecRef gain_post, VecRef gain_next, Tnext* __restrict__ next, int dim, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const size_t row = (size_t)blockIdx.x * dim;
    const int n4 = dim >> 2;
    const float4* pa = reinterpret_cast<const float4*>(a + row);
    const float4* pb = b ? reinterpret_cast<const float4*>(b + row) : nullptr;
    float4* px = reinterpret_cast<float4*>(x + row);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 va[V], vb[V], vx[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int i = threadIdx.x + 256 * j;
        va[j] = i < n4 ? pa[i] : zero;
        vb[j] = (pb && i < n4) ? pb[i] : zero;
        vx[j] = i < n4 ? px[i] : zero;
    }
    auto squares = [](const float4& v, float acc) {
        acc = fmaf(v.x, v.x, acc); acc = fmaf(v.y, v.y, acc); acc = fmaf(v.z, v.z, acc); return fmaf(v.w, v.w, acc);
    };
    if (pb) {
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int j = 0; j < V; ++j) { sa = squares(va[j], sa); sb = squares(vb[j], sb); }
        sa = block_sum(sa, scratch);
        sb = block_sum(sb, scratch);
        const float ra = rms_scale(sa, dim, eps), rb = rms_scale(sb, dim, eps);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const int i = 4 * (threadIdx.x + 256 * j);
            if (i >= dim) break;
            float* pva = reinterpret_cast<float*>(&va[j]);
            const float* pvb = reinterpret_cast<const float*>(&vb[j]);
#pragma unroll
            for (int c = 0; c < 4; ++c)
                pva[c] = __fmul_rn(__fadd_rn(__fmul_rn(__fmul_rn(pva[c], ra), gain_a[i + c]), __fmul_rn(__fmul_rn(pvb[c], rb), gain_b[i + c])), scale);
        }
    }
    float sv = 0.f;
#pragma unroll
    for (int j = 0; j < V; ++j) sv = squares(va[j], sv);
    sv = block_sum(sv, scratch);
    const float rv = rms_scale(sv, dim, eps);
    float sx = 0.f;
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int i4 = threadIdx.x + 256 * j;
        if (i4 >= n4) break;
        const float* pva = reinterpret_cast<const float*>(&va[j]);
        float* pvx = reinterpret_cast<float*>(&vx[j]);
#pragma unroll
        for (int c = 0; c < 4; ++c) pvx[c] = __fadd_rn(pvx[c], __fmul_rn(__fmul_rn(pva[c], rv), gain_post[4 * i4 + c]));
        px[i4] = vx[j];
        sx = squares(vx[j], sx);
    }
    if (next == nullptr) return;
    sx = block_sum(sx, scratch);
    const float rx = rms_scale(sx, dim, eps);
    Tnext* pn = next + row;
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int i4 = threadIdx.x + 256 * j;
        if (i4 >= n4) break;
        const float* pvx = reinterpret_cast<const float*>(&vx[j]);
        float o[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) o[c] = __fmul_rn(__fmul_rn(pvx[c], rx), gain_next[4 * i4 + c]);
        if constexpr (sizeof(Tnext) == 4) {
            reinterpret_cast<float4*>(pn)[i4] = make_float4(o[0], o[1], o[2], o[3]);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
            uint2 p;
            p.x = *reinterpret_cast<uint32_t*>(&lo);
            p.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(pn)[i4] = p;
        }
    }
}

JLLM_EXPORT int jllm_norm_chain(float* x, const float* a, const void* gain_a, const float* b, const void* gain_b, float scale,
                                const void* gain_post, const void* gain_next, void* next, int next_dtype, int gain_dtype,
                                int rows, int dim, float eps, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0 && a && gain_post && (!b || (gain_a && gain_b)) && (!next || gain_next),
                 "norm_chain: rows=%d dim=%d", rows, dim);
    JLLM_REQUIRE(dim <= 48 * 256, "norm_chain: a row of %d values is above %d", dim, 48 * 256);
    if (rows == 0) return JLLM_OK;
    const size_t smem = (size_t)dim * sizeof(float);
    const VecRef ga{gain_a, gain_dtype}, gb{gain_b, gain_dtype}, gp{gain_post, gain_dtype}, gn{gain_next, gain_dtype};
    if (dim % 4 == 0 && dim <= 8192 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0 &&
        ((uintptr_t)next % 16) == 0) {
#define JLLM_CHAIN(T, V)                                                                                                      \
    jllm_launch(norm_chain_vec_kernel<T, V>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, a, ga, b, gb, scale, gp, gn, \
                (T*)next, dim, eps)
        const int v = (dim / 4 + 255) / 256;
        if (next_dtype == JLLM_F32) {
            if (v <= 1) JLLM_CHAIN(float, 1); else if (v <= 2) JLLM_CHAIN(float, 2); else if (v <= 4) JLLM_CHAIN(float, 4);
            else JLLM_CHAIN(float, 8);
        } else {
            if (v <= 1) JLLM_CHAIN(__nv_bfloat16, 1); else if (v <= 2) JLLM_CHAIN(__nv_bfloat16, 2);
            else if (v <= 4) JLLM_CHAIN(__nv_bfloat16, 4); else JLLM_CHAIN(__nv_bfloat16, 8);
        }
#undef JLLM_CHAIN
        return jllm_check_launch("norm_chain");
    }
    if (next_dtype == JLLM_F32)
        jllm_launch(norm_chain_kernel<float>, dim3(rows), dim3(256), smem, stream, LAUNCH_DEPENDENT, x, a, ga, b, gb, scale, gp,
                    gn, (float*)next, dim, eps);
    else
        jllm_launch(norm_chain_kernel<__nv_bfloat16>, dim3(rows), dim3(256), smem, stream, LAUNCH_DEPENDENT, x, a, ga, b, gb,
                    scale, gp, gn, (__nv_bfloat16*)next, dim, eps);
    return jllm_check_launch("norm_chain");
}
