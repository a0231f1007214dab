// What happens to the residual stream between the parts of a layer whose norms sit BEHIND the parts, and between layers:
//
//   layernorm        out[r] = ((x[s] - mean) / sqrt(var + eps)) * w * out_scale, s = row_index ? row_index[r] : r, var the mean
//                    of the squared deviations (two passes over the row); the model's last norm
//   norm_add         x[r] += norm(a[r]) * w, norm the layer norm above (center = 1) or x / sqrt(mean(x^2) + eps) (center = 0);
//                    optionally next_out[r] = x[r] in the compute type (the input of the part that follows, which reads the
//                    stream itself and not a normed copy)
//   token_shift      out[r] = x[r] + (p - x[r]) * mu with p the row in front of r in its request: x[r - 1] inside a segment,
//                    the request's saved row (its state slot; zeros for a new request) for a segment's first row. The last
//                    row of every segment is saved for the next step: by the same launch when every segment is one row (each
//                    value is read and then written by one thread), else by `token_shift_save` behind it, because a
//                    segment's first and last rows are then different blocks.
//   depth_mix        out = sum_j a[j] * X_j over n planes of one stack (ascending j), X_j at stack + j * plane
//   norm_add_mix     norm_add, depth_mix and (where every segment is one row) the NEXT layer's token_shift in one launch, a
//                    block per row: x[r] += norm(a[r]) * w is the newest plane of the stack, the mix of all planes goes to the
//                    plane behind it, and its blend with the next layer's saved row leaves in the compute type
//   scale_values     x *= s
//
// All arithmetic is float32; a row's result depends on that row (and the one in front of it) alone.
#include "common.cuh"

namespace {

__device__ __forceinline__ bool rows_vec4(const void* a, const void* b, int dim) {
    return (dim & 3) == 0 && ((((uintptr_t)a) | ((uintptr_t)b)) & 15u) == 0;
}

// mean and 1 / sqrt(var + eps) of a row (center) or 0 and 1 / sqrt(mean(x^2) + eps)
__device__ __forceinline__ void row_statistics(const float* __restrict__ src, int dim, float eps, int center, float* scratch,
                                               float& mean, float& inv) {
    mean = 0.f;
    if (center) {
        float s = 0.f;
        for (int i = threadIdx.x; i < dim; i += blockDim.x) s += src[i];
        mean = block_sum(s, scratch) / (float)dim;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float d = src[i] - mean;
        ss = fmaf(d, d, ss);
    }
    ss = block_sum(ss, scratch);
    inv = 1.f / sqrtf(ss / (float)dim + eps);
}

template <typename Tout>
__global__ void __launch_bounds__(256)
layernorm_kernel(const float* __restrict__ x, VecRef gain, Tout* __restrict__ out, const int* __restrict__ row_index, int dim,
                 float eps, int center, float out_scale) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(row_index ? row_index[r] : r) * dim;
    float mean, inv;
    row_statistics(src, dim, eps, center, scratch, mean, inv);
    Tout* dst = out + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        dst[i] = from_float<Tout>(__fmul_rn(__fmul_rn(__fmul_rn(src[i] - mean, inv), gain[i]), out_scale));
}

template <typename Tnext>
__global__ void __launch_bounds__(256)
norm_add_kernel(float* __restrict__ x, const float* __restrict__ a, VecRef gain, Tnext* __restrict__ next_out, int dim, float eps,
                int center) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const float* src = a + (size_t)r * dim;
    float* xr = x + (size_t)r * dim;
    float mean, inv;
    row_statistics(src, dim, eps, center, scratch, mean, inv);
    Tnext* nxt = next_out ? next_out + (size_t)r * dim : nullptr;
    if (rows_vec4(src, xr, dim) && (nxt == nullptr || (((uintptr_t)nxt) & 15u) == 0)) {
        for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            float4 o = *reinterpret_cast<const float4*>(xr + i);
            o.x = __fadd_rn(o.x, __fmul_rn(__fmul_rn(v.x - mean, inv), gain[i]));
            o.y = __fadd_rn(o.y, __fmul_rn(__fmul_rn(v.y - mean, inv), gain[i + 1]));
            o.z = __fadd_rn(o.z, __fmul_rn(__fmul_rn(v.z - mean, inv), gain[i + 2]));
            o.w = __fadd_rn(o.w, __fmul_rn(__fmul_rn(v.w - mean, inv), gain[i + 3]));
            *reinterpret_cast<float4*>(xr + i) = o;
            if (nxt != nullptr) {
                if constexpr (sizeof(Tnext) == 4) {
                    *reinterpret_cast<float4*>(nxt + i) = o;
                } else {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                    uint2 p;
                    p.x = *reinterpret_cast<uint32_t*>(&lo);
                    p.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(nxt + i) = p;
                }
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float o = __fadd_rn(xr[i], __fmul_rn(__fmul_rn(src[i] - mean, inv), gain[i]));
        xr[i] = o;
        if (nxt != nullptr) nxt[i] = from_float<Tnext>(o);
    }
}

template <typename Tout>
__global__ void __launch_bounds__(256)
token_shift_kernel(const float* __restrict__ x, VecRef mu, float* __restrict__ state, const int* __restrict__ row_seg,
                   const int* __restrict__ seg_start, const int* __restrict__ state_slots, Tout* __restrict__ out, int dim,
                   int slots, int save) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, seg = row_seg[r];
    const int slot = state_slots[seg];
    if (!jllm_in_bounds(slot, slots, BOUNDS_SLOT)) return;
    float* saved = state + (size_t)slot * dim;
    const float* cur = x + (size_t)r * dim;
    const float* before = r == seg_start[seg] ? saved : cur - dim;
    Tout* dst = out + (size_t)r * dim;
    if (rows_vec4(cur, saved, dim) && (((uintptr_t)dst) & 7u) == 0) {
        for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            const float4 c = *reinterpret_cast<const float4*>(cur + i), p = *reinterpret_cast<const float4*>(before + i);
            const float y0 = __fadd_rn(c.x, __fmul_rn(p.x - c.x, mu[i])), y1 = __fadd_rn(c.y, __fmul_rn(p.y - c.y, mu[i + 1]));
            const float y2 = __fadd_rn(c.z, __fmul_rn(p.z - c.z, mu[i + 2])), y3 = __fadd_rn(c.w, __fmul_rn(p.w - c.w, mu[i + 3]));
            if constexpr (sizeof(Tout) == 4) {
                dst[i] = y0; dst[i + 1] = y1; dst[i + 2] = y2; dst[i + 3] = y3;
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
                uint2 q;
                q.x = *reinterpret_cast<uint32_t*>(&lo);
                q.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst + i) = q;
            }
            if (save) *reinterpret_cast<float4*>(saved + i) = c;
        }
        return;
    }
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float c = cur[i], p = before[i];
        dst[i] = from_float<Tout>(__fadd_rn(c, __fmul_rn(p - c, mu[i])));
        if (save) saved[i] = c;
    }
}

__global__ void __launch_bounds__(256)
token_shift_save_kernel(const float* __restrict__ x, float* __restrict__ state, const int* __restrict__ seg_start,
                        const int* __restrict__ seg_len, const int* __restrict__ state_slots, int dim, int slots) {
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x, slot = state_slots[seg];
    if (seg_len[seg] <= 0 || !jllm_in_bounds(slot, slots, BOUNDS_SLOT)) return;
    const float* last = x + (size_t)(seg_start[seg] + seg_len[seg] - 1) * dim;
    float* saved = state + (size_t)slot * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) saved[i] = last[i];
}

constexpr int MIX_MAX = 256;       // planes of a depth mix

template <int V>
__global__ void __launch_bounds__(256)
depth_mix_kernel(const float* __restrict__ stack, size_t plane, VecRef weights, int n, float* __restrict__ out, size_t count) {
    __shared__ float a[MIX_MAX];
    pdl_wait();
    pdl_trigger();
    for (int j = threadIdx.x; j < n; j += blockDim.x) a[j] = weights[j];
    __syncthreads();
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V; i < count; i += (size_t)gridDim.x * blockDim.x * V) {
        if constexpr (V == 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < n; ++j) {
                const float4 v = *reinterpret_cast<const float4*>(stack + (size_t)j * plane + i);
                acc.x = fmaf(a[j], v.x, acc.x);
                acc.y = fmaf(a[j], v.y, acc.y);
                acc.z = fmaf(a[j], v.z, acc.z);
                acc.w = fmaf(a[j], v.w, acc.w);
            }
            *reinterpret_cast<float4*>(out + i) = acc;
        } else {
            float acc = 0.f;
            for (int j = 0; j < n; ++j) acc = fmaf(a[j], stack[(size_t)j * plane + i], acc);
            out[i] = acc;
        }
    }
}

// x: the rows of plane n - 1 of the stack (read and written); mix_out: the rows of the plane that takes the mix. With
// `shift`: h_out[r] = mix + (saved - mix) * mu and saved = mix, for the one-row segment of row r (the next layer's state).
template <typename Tout>
__global__ void __launch_bounds__(256)
norm_add_mix_kernel(float* __restrict__ x, const float* __restrict__ a, VecRef gain, int dim, float eps, int center,
                    const float* __restrict__ stack, size_t plane, VecRef weights, int n, float* __restrict__ mix_out, int shift,
                    VecRef mu, float* __restrict__ state, int slots, const int* __restrict__ row_seg,
                    const int* __restrict__ state_slots, Tout* __restrict__ h_out) {
    __shared__ float scratch[33];
    __shared__ float wj[MIX_MAX];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    for (int j = threadIdx.x; j < n; j += blockDim.x) wj[j] = weights[j];
    const float* src = a + (size_t)r * dim;
    float* xr = x + (size_t)r * dim;
    float* mr = mix_out + (size_t)r * dim;
    float mean, inv;
    row_statistics(src, dim, eps, center, scratch, mean, inv);      // (its barriers also publish wj)
    float* saved = nullptr;
    if (shift) {
        const int slot = state_slots[row_seg[r]];
        if (!jllm_in_bounds(slot, slots, BOUNDS_SLOT)) return;
        saved = state + (size_t)slot * dim;
    }
    Tout* hr = shift ? h_out + (size_t)r * dim : nullptr;
    const float* lower = stack + (size_t)r * dim;
    if (rows_vec4(src, xr, dim) && rows_vec4(mr, lower, dim) && (plane & 3) == 0 && (!shift || rows_vec4(saved, hr, dim))) {
        for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            float4 o = *reinterpret_cast<const float4*>(xr + i);
            o.x = __fadd_rn(o.x, __fmul_rn(__fmul_rn(v.x - mean, inv), gain[i]));
            o.y = __fadd_rn(o.y, __fmul_rn(__fmul_rn(v.y - mean, inv), gain[i + 1]));
            o.z = __fadd_rn(o.z, __fmul_rn(__fmul_rn(v.z - mean, inv), gain[i + 2]));
            o.w = __fadd_rn(o.w, __fmul_rn(__fmul_rn(v.w - mean, inv), gain[i + 3]));
            *reinterpret_cast<float4*>(xr + i) = o;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < n - 1; ++j) {
                const float4 p = *reinterpret_cast<const float4*>(lower + (size_t)j * plane + i);
                acc.x = fmaf(wj[j], p.x, acc.x);
                acc.y = fmaf(wj[j], p.y, acc.y);
                acc.z = fmaf(wj[j], p.z, acc.z);
                acc.w = fmaf(wj[j], p.w, acc.w);
            }
            acc.x = fmaf(wj[n - 1], o.x, acc.x);
            acc.y = fmaf(wj[n - 1], o.y, acc.y);
            acc.z = fmaf(wj[n - 1], o.z, acc.z);
            acc.w = fmaf(wj[n - 1], o.w, acc.w);
            *reinterpret_cast<float4*>(mr + i) = acc;
            if (shift) {
                const float4 p = *reinterpret_cast<const float4*>(saved + i);
                const float y0 = __fadd_rn(acc.x, __fmul_rn(p.x - acc.x, mu[i])), y1 = __fadd_rn(acc.y, __fmul_rn(p.y - acc.y, mu[i + 1]));
                const float y2 = __fadd_rn(acc.z, __fmul_rn(p.z - acc.z, mu[i + 2])), y3 = __fadd_rn(acc.w, __fmul_rn(p.w - acc.w, mu[i + 3]));
                if constexpr (sizeof(Tout) == 4) {
                    *reinterpret_cast<float4*>(hr + i) = make_float4(y0, y1, y2, y3);
                } else {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
                    uint2 q;
                    q.x = *reinterpret_cast<uint32_t*>(&lo);
                    q.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(hr + i) = q;
                }
                *reinterpret_cast<float4*>(saved + i) = acc;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float o = __fadd_rn(xr[i], __fmul_rn(__fmul_rn(src[i] - mean, inv), gain[i]));
        xr[i] = o;
        float acc = 0.f;
        for (int j = 0; j < n - 1; ++j) acc = fmaf(wj[j], lower[(size_t)j * plane + i], acc);
        acc = fmaf(wj[n - 1], o, acc);
        mr[i] = acc;
        if (shift) {
            hr[i] = from_float<Tout>(__fadd_rn(acc, __fmul_rn(saved[i] - acc, mu[i])));
            saved[i] = acc;
        }
    }
}

__global__ void scale_values_kernel(float* __restrict__ x, float s, size_t count) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        x[i] = __fmul_rn(x[i], s);
}

}  // namespace

JLLM_BOUNDS_READER(residual_paths)

JLLM_EXPORT int jllm_layernorm(const float* x, const void* gain, int gain_dtype, void* out, int out_dtype, const int* row_index,
                               int rows, int dim, float eps, int center, float out_scale, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0, "layernorm: rows=%d dim=%d", rows, dim);
    if (rows == 0) return JLLM_OK;
    const VecRef g{gain, gain_dtype};
    if (out_dtype == JLLM_F32)
        jllm_launch(layernorm_kernel<float>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, g, (float*)out, row_index, dim,
                    eps, center, out_scale);
    else
        jllm_launch(layernorm_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, g,
                    (__nv_bfloat16*)out, row_index, dim, eps, center, out_scale);
    return jllm_check_launch("layernorm");
}

// x, a float32 [rows, dim]; next_out (or null) [rows, dim] of type next_dtype.
JLLM_EXPORT int jllm_norm_add(float* x, const float* a, const void* gain, int gain_dtype, void* next_out, int next_dtype, int rows,
                              int dim, float eps, int center, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0, "norm_add: rows=%d dim=%d", rows, dim);
    if (rows == 0) return JLLM_OK;
    const VecRef g{gain, gain_dtype};
    if (next_dtype == JLLM_F32)
        jllm_launch(norm_add_kernel<float>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, a, g, (float*)next_out, dim, eps,
                    center);
    else
        jllm_launch(norm_add_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, a, g,
                    (__nv_bfloat16*)next_out, dim, eps, center);
    return jllm_check_launch("norm_add");
}

// x float32 [rows, dim]; state float32 [slots, dim]; out [rows, dim] of type out_dtype. `single`: every segment is one row.
JLLM_EXPORT int jllm_token_shift(const float* x, const void* mu, int mu_dtype, float* state, int slots, const int* row_seg,
                                 const int* seg_start, const int* seg_len, const int* state_slots, void* out, int out_dtype,
                                 int rows, int segments, int dim, int single, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && segments >= 0 && dim > 0 && slots > 0, "token_shift: rows=%d segments=%d dim=%d slots=%d", rows,
                 segments, dim, slots);
    if (rows == 0) return JLLM_OK;
    const VecRef m{mu, mu_dtype};
    if (out_dtype == JLLM_F32)
        jllm_launch(token_shift_kernel<float>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, m, state, row_seg, seg_start,
                    state_slots, (float*)out, dim, slots, single);
    else
        jllm_launch(token_shift_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, m, state, row_seg,
                    seg_start, state_slots, (__nv_bfloat16*)out, dim, slots, single);
    if (!single)
        jllm_launch(token_shift_save_kernel, dim3(segments), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, state, seg_start, seg_len,
                    state_slots, dim, slots);
    return jllm_check_launch("token_shift");
}

// stack: n planes of float32, plane j at stack + j * plane (floats); out float32 [count].
JLLM_EXPORT int jllm_depth_mix(const float* stack, long long plane, const void* weights, int weights_dtype, int n, float* out,
                               long long count, cudaStream_t stream) {
    JLLM_REQUIRE(n >= 1 && n <= MIX_MAX && count >= 0 && plane >= 0, "depth_mix: n=%d (at most %d) count=%lld", n, MIX_MAX, count);
    if (count == 0) return JLLM_OK;
    const VecRef w{weights, weights_dtype};
    const bool vec = count % 4 == 0 && plane % 4 == 0 && ((((uintptr_t)stack) | ((uintptr_t)out)) & 15u) == 0;
    const size_t items = vec ? (size_t)count / 4 : (size_t)count;
    const int blocks = (int)min((size_t)(8 * 148), (items + 255) / 256);
    if (vec)
        jllm_launch(depth_mix_kernel<4>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, stack, (size_t)plane, w, n, out,
                    (size_t)count);
    else
        jllm_launch(depth_mix_kernel<1>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, stack, (size_t)plane, w, n, out,
                    (size_t)count);
    return jllm_check_launch("depth_mix");
}

// stack: n planes of [rows, dim] float32 (plane j at stack + j * plane), the last of them x; a float32 [rows, dim]; mix_out
// float32 [rows, dim]. mu (or null: no shift): the next layer's shift vector, with its state [slots, dim], the batch's
// row -> segment and segment -> slot tables (every segment one row) and h_out [rows, dim] of type out_dtype.
JLLM_EXPORT int jllm_norm_add_mix(float* x, const float* a, const void* gain, int gain_dtype, int rows, int dim, float eps,
                                  int center, const float* stack, long long plane, const void* weights, int weights_dtype, int n,
                                  float* mix_out, const void* mu, int mu_dtype, float* state, int slots, const int* row_seg,
                                  const int* state_slots, void* h_out, int out_dtype, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0 && n >= 1 && n <= MIX_MAX && plane >= 0, "norm_add_mix: rows=%d dim=%d n=%d", rows, dim, n);
    JLLM_REQUIRE(mu == nullptr || (state != nullptr && slots > 0 && row_seg != nullptr && state_slots != nullptr && h_out != nullptr),
                 "norm_add_mix: a shift needs its state, the batch's tables and an output");
    if (rows == 0) return JLLM_OK;
    const VecRef g{gain, gain_dtype}, w{weights, weights_dtype}, m{mu, mu_dtype};
    const int shift = mu != nullptr;
    if (out_dtype == JLLM_F32)
        jllm_launch(norm_add_mix_kernel<float>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, a, g, dim, eps, center, stack,
                    (size_t)plane, w, n, mix_out, shift, m, state, slots, row_seg, state_slots, (float*)h_out);
    else
        jllm_launch(norm_add_mix_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, a, g, dim, eps, center,
                    stack, (size_t)plane, w, n, mix_out, shift, m, state, slots, row_seg, state_slots, (__nv_bfloat16*)h_out);
    return jllm_check_launch("norm_add_mix");
}

JLLM_EXPORT int jllm_scale_values(float* x, float s, long long count, cudaStream_t stream) {
    JLLM_REQUIRE(count >= 0, "scale_values: count=%lld", count);
    if (count == 0) return JLLM_OK;
    const int blocks = (int)min((size_t)65535, ((size_t)count + 255) / 256);
    jllm_launch(scale_values_kernel, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, x, s, (size_t)count);
    return jllm_check_launch("scale_values");
}
