// Routed experts: the router, and the weighting of the experts' hidden rows.
//
// The router scores every expert for every row in float32: s = sigmoid(Wr h), Wr [experts, dim] float32. The `top`
// experts with the largest s + correction are chosen (the lowest index wins a tie); the row's weights are the chosen s
// divided by their sum + 1e-20 (if `normalize`), times `scale`; the others get 0. The weights leave as a dense
// [rows, experts] float32 table: the feed-forward runs the experts as ONE product over their stacked gate / up rows
// and ONE over their down matrices laid side by side along k, and a row's hidden values of expert e are multiplied by
// its weight in between (`scale_expert_hidden`), so that experts a row does not use add exactly nothing.
//
// What a design may ask of the router beyond that: scores that are a softmax over all entries instead of a logistic function
// of each (`softmax`); entries behind the experts that have no weights and hand the row through as it is (`identity`: the
// router matrix has experts + identity rows, the chosen identity entries' weights leave as ONE number, their sum, in the
// column behind the experts' and the gates'); and rows behind those that are not routed at all but give a logistic gate per
// row (`gates`: a shared expert's), which leave in the columns behind the experts'.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
route_experts_kernel(const T* __restrict__ h, int ld, const float* __restrict__ router, VecRef correction, int has_correction,
                     float* __restrict__ weights, int dim, int real, int top, float scale, int normalize, int identity, int gates,
                     int softmax, int ld_out) {
    // `real` experts have weights; entries [real, real + identity) hand the row through; rows [entries, entries + gates) of the
    // router matrix are gates. `experts` below counts every row of the matrix.
    const int entries = real + identity, experts = entries + gates;
    extern __shared__ float smem[];
    float* s = smem;                   // [experts] scores
    float* c = s + (experts + 1) / 2 * 2;      // [experts] choice scores, -inf once taken
    float* hs = c + (experts + 1) / 2 * 2;     // [dim] the row, read once (on a 16-byte boundary)
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* row = h + (size_t)r * ld;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) hs[i] = to_float(row[i]);
    __syncthreads();
    const bool vec = (dim & 3) == 0 && (((uintptr_t)router) & 15u) == 0;
    for (int e = warp; e < experts; e += warps) {
        const float* wr = router + (size_t)e * dim;
        float acc = 0.f;
        if (vec) {      // a lane takes four neighbouring values at a time, four such loads on their way together; the
                        // order of the sum is fixed all the same
            float part[4] = {0.f, 0.f, 0.f, 0.f};
            for (int i0 = lane * 4; i0 < dim; i0 += 512) {
                float4 b[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    b[u] = i0 + 128 * u < dim ? *reinterpret_cast<const float4*>(wr + i0 + 128 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (i0 + 128 * u < dim) {
                        const float4 a = *reinterpret_cast<const float4*>(hs + i0 + 128 * u);
                        part[u] = fmaf(a.x, b[u].x, part[u]);
                        part[u] = fmaf(a.y, b[u].y, part[u]);
                        part[u] = fmaf(a.z, b[u].z, part[u]);
                        part[u] = fmaf(a.w, b[u].w, part[u]);
                    }
                }
            }
            acc = (part[0] + part[1]) + (part[2] + part[3]);
        } else {
            for (int i = lane; i < dim; i += 32) acc = fmaf(hs[i], wr[i], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            const float sc = (softmax && e < entries) ? acc : 1.f / (1.f + expf(-acc));
            s[e] = sc;
            c[e] = (has_correction && e < entries) ? sc + correction[e] : sc;
        }
    }
    __syncthreads();
    // the row's table is put together in shared memory (one thread's choice is a chain of dependent steps: in global memory
    // every step of it was a round trip) and written out by all threads
    float* out = hs + ((dim + 3) & ~3);
    for (int e = threadIdx.x; e < ld_out; e += blockDim.x) out[e] = 0.f;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (softmax) {                 // the logits become scores: exp(z - max) over their sum, in entry order
            float top_z = -INFINITY, total = 0.f;
            for (int e = 0; e < entries; ++e) top_z = fmaxf(top_z, s[e]);
            for (int e = 0; e < entries; ++e) {
                s[e] = expf(s[e] - top_z);
                total += s[e];
            }
            for (int e = 0; e < entries; ++e) {
                s[e] = s[e] / total;
                c[e] = has_correction ? s[e] + correction[e] : s[e];
            }
        }
        float sum = 0.f, through = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float bv = -INFINITY;
            for (int e = 0; e < entries; ++e)
                if (c[e] > bv) { bv = c[e]; best = e; }
            c[best] = -INFINITY;
            if (best < real) out[best] = s[best];
            else through += s[best];
            sum += s[best];
        }
        const float f = normalize ? scale / (sum + 1e-20f) : scale;
        for (int e = 0; e < real; ++e) out[e] = __fmul_rn(out[e], f);
        for (int g = 0; g < gates; ++g) out[real + g] = __fmul_rn(s[entries + g], scale);
        if (identity) out[real + gates] = __fmul_rn(through, f);
    }
    __syncthreads();
    float* dst = weights + (size_t)r * ld_out;
    for (int e = threadIdx.x; e < ld_out; e += blockDim.x) dst[e] = out[e];
}

template <typename T>
__global__ void scale_expert_hidden_kernel(T* __restrict__ hidden, const float* __restrict__ weights, int experts, int ff,
                                           size_t total, int ld_w, int shared_ff) {
    // behind the experts' values may lie `shared_ff` values of one more unit, whose weight is column `experts` of the table
    pdl_wait();
    pdl_trigger();
    const size_t routed = (size_t)experts * ff, width = routed + shared_ff;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width, col = i - r * width;
        hidden[i] = from_float<T>(__fmul_rn(to_float(hidden[i]), weights[r * ld_w + (col < routed ? col / ff : experts)]));
    }
}

// The same, 16 bytes a thread (ff a multiple of the 16-byte group: a group lies inside one expert).
template <typename T>
__global__ void scale_expert_hidden_vec_kernel(T* __restrict__ hidden, const float* __restrict__ weights, int experts, int ff,
                                               size_t groups, int ld_w, int shared_ff) {
    constexpr int N = 16 / sizeof(T);
    pdl_wait();
    pdl_trigger();
    const size_t routed = (size_t)experts * ff, width = routed + shared_ff;
    for (size_t gi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += (size_t)gridDim.x * blockDim.x) {
        const size_t i = gi * N, r = i / width, col = i - r * width;
        const float wt = weights[r * ld_w + (col < routed ? col / ff : experts)];
        uint4 raw = *reinterpret_cast<const uint4*>(hidden + i);
        T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int k = 0; k < N; ++k) v[k] = from_float<T>(__fmul_rn(to_float(v[k]), wt));
        *reinterpret_cast<uint4*>(hidden + i) = raw;
    }
}

// The gated unit whose two inputs are cut off: g = min(w gate, limit), u = clamp(w up, -limit, limit), y = g sigmoid(alpha g)
// (u + 1); w the row's weight for the expert the unit belongs to (the weight multiplies the expert's INPUT, which by
// linearity of the two products is the same as multiplying their results), 1 without a weight table. gate_up [rows,
// 2 * width]: all gate values, then all up values; width = experts * ff + shared_ff: behind the experts' units may lie
// those of a shared expert that every row uses with weight 1 and a limit of its own. An expert the row does not use
// (w = 0) gives exact zeros.
__device__ __forceinline__ float clamped_unit(float gate, float up, float w, float limit, float alpha) {
    const float g = fminf(__fmul_rn(w, gate), limit);
    const float u = fminf(fmaxf(__fmul_rn(w, up), -limit), limit);
    return __fmul_rn(g / (1.f + expf(-__fmul_rn(alpha, g))), u + 1.f);
}

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gate_up, const float* __restrict__ weights, T* __restrict__ out,
                                   int experts, int ff, float limit, int shared_ff, float shared_limit, float alpha,
                                   size_t total) {
    pdl_wait();
    pdl_trigger();
    const size_t routed = (size_t)experts * ff, width = routed + shared_ff;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width, col = i - r * width;
        const bool own = col < routed;
        const float w = own && weights ? weights[r * experts + col / ff] : 1.f;
        const T* row = gate_up + r * 2 * width;
        out[i] = from_float<T>(clamped_unit(to_float(row[col]), to_float(row[width + col]), w, own ? limit : shared_limit, alpha));
    }
}

// The same, 16 bytes a thread (ff and shared_ff multiples of the 16-byte group: a group lies inside one expert).
template <typename T>
__global__ void __launch_bounds__(256)
glu_clamped_vec_kernel(const T* __restrict__ gate_up, const float* __restrict__ weights, T* __restrict__ out, int experts, int ff,
                       float limit, int shared_ff, float shared_limit, float alpha, int rows) {
    constexpr int N = 16 / sizeof(T);
    pdl_wait();
    pdl_trigger();
    const int routed = experts * ff, width = routed + shared_ff, groups = width / N;
    const int r = blockIdx.y;
    if (r >= rows) return;
    const T* row = gate_up + (size_t)r * 2 * width;
    T* dst = out + (size_t)r * width;
    for (int gi = blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += gridDim.x * blockDim.x) {
        const int col = gi * N;
        const bool own = col < routed;
        const float w = own && weights ? weights[(size_t)r * experts + col / ff] : 1.f;
        uint4 res;
        T* y = reinterpret_cast<T*>(&res);
        if (w == 0.f) {         // the row does not use this expert: its units are not read
#pragma unroll
            for (int k = 0; k < N; ++k) y[k] = from_float<T>(0.f);
        } else {
            const uint4 graw = *reinterpret_cast<const uint4*>(row + col), uraw = *reinterpret_cast<const uint4*>(row + width + col);
            const T* g = reinterpret_cast<const T*>(&graw);
            const T* u = reinterpret_cast<const T*>(&uraw);
            const float lim = own ? limit : shared_limit;
#pragma unroll
            for (int k = 0; k < N; ++k) y[k] = from_float<T>(clamped_unit(to_float(g[k]), to_float(u[k]), w, lim, alpha));
        }
        *reinterpret_cast<uint4*>(dst + col) = res;
    }
}

}  // namespace

// gate_up [rows, 2 * (experts * ff + shared_ff)], out [rows, experts * ff + shared_ff], both contiguous and of type
// `dtype`; weights [rows, experts] float32 or null.
JLLM_EXPORT int jllm_glu_clamped(const void* gate_up, const float* weights, void* out, int dtype, int rows, int experts, int ff,
                                 float limit, int shared_ff, float shared_limit, float alpha, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && experts > 0 && ff > 0 && limit > 0.f && shared_ff >= 0 && (shared_ff == 0 || shared_limit > 0.f),
                 "glu_clamped: rows=%d experts=%d ff=%d limit=%g shared_ff=%d shared_limit=%g", rows, experts, ff, (double)limit,
                 shared_ff, (double)shared_limit);
    if (rows == 0) return JLLM_OK;
    const int width = experts * ff + shared_ff;
    const int per = dtype == JLLM_F32 ? 4 : 8;
    if (ff % per == 0 && shared_ff % per == 0 && ((uintptr_t)gate_up % 16) == 0 && ((uintptr_t)out % 16) == 0 && rows <= 65535) {
        const dim3 grid(max(1, min(64, (width / per + 255) / 256)), rows);
        if (dtype == JLLM_F32)
            jllm_launch(glu_clamped_vec_kernel<float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (const float*)gate_up, weights,
                        (float*)out, experts, ff, limit, shared_ff, shared_limit, alpha, rows);
        else
            jllm_launch(glu_clamped_vec_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT,
                        (const __nv_bfloat16*)gate_up, weights, (__nv_bfloat16*)out, experts, ff, limit, shared_ff, shared_limit,
                        alpha, rows);
        return jllm_check_launch("glu_clamped");
    }
    const size_t total = (size_t)rows * width;
    const int blocks = (int)min((size_t)65535, (total + 255) / 256);
    if (dtype == JLLM_F32)
        jllm_launch(glu_clamped_kernel<float>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, (const float*)gate_up, weights,
                    (float*)out, experts, ff, limit, shared_ff, shared_limit, alpha, total);
    else
        jllm_launch(glu_clamped_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT,
                    (const __nv_bfloat16*)gate_up, weights, (__nv_bfloat16*)out, experts, ff, limit, shared_ff, shared_limit, alpha,
                    total);
    return jllm_check_launch("glu_clamped");
}

// h [rows, ld] of type `dtype` (the normed rows); router [experts + identity + gates, dim] float32; correction
// [experts + identity] or null; weights [rows, ld_out] float32: the experts' weights, then the gates, then (with identity
// entries) the sum of the chosen identity entries' weights.
JLLM_EXPORT int jllm_route_experts(const void* h, int dtype, int ld, const float* router, const void* correction,
                                   int correction_dtype, float* weights, int rows, int dim, int real, int top, float scale,
                                   int normalize, int identity, int gates, int softmax, int ld_out, cudaStream_t stream) {
    const int experts = real + identity + gates;
    JLLM_REQUIRE(rows >= 0 && dim > 0 && real > 0 && identity >= 0 && gates >= 0 && top >= 1 && top <= real + identity &&
                 experts <= 4096 && ld_out >= real + gates + (identity ? 1 : 0),
                 "route_experts: rows=%d dim=%d experts=%d identity=%d gates=%d top=%d ld_out=%d", rows, dim, real, identity, gates,
                 top, ld_out);
    if (rows == 0) return JLLM_OK;
    const VecRef c{correction, correction_dtype};
    const int padded = (experts + 1) / 2 * 2;       // the row's copy behind the two score arrays starts on 16 bytes
    const size_t smem = (2 * (size_t)padded + ((dim + 3) & ~3) + ld_out) * sizeof(float);
    JLLM_REQUIRE(smem <= 200 * 1024, "route_experts: dim=%d and experts=%d need %zu bytes of shared memory", dim, experts, smem);
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(route_experts_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(route_experts_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return jllm_fail(JLLM_CUDA_ERROR, "route_experts: %zu bytes of shared memory refused", smem);
    }
    if (dtype == JLLM_F32)
        jllm_launch(route_experts_kernel<float>, dim3(rows), dim3(256), smem, stream, LAUNCH_DEPENDENT, (const float*)h, ld,
                    router, c, (int)(correction != nullptr), weights, dim, real, top, scale, normalize, identity, gates, softmax, ld_out);
    else
        jllm_launch(route_experts_kernel<__nv_bfloat16>, dim3(rows), dim3(256), smem, stream, LAUNCH_DEPENDENT,
                    (const __nv_bfloat16*)h, ld, router, c, (int)(correction != nullptr), weights, dim, real, top, scale,
                    normalize, identity, gates, softmax, ld_out);
    return jllm_check_launch("route_experts");
}

// hidden [rows, experts * ff + shared_ff] (contiguous): the values of expert e are multiplied by weights[r, e], the last
// shared_ff values by weights[r, experts]; weights [rows, ld_w] float32.
JLLM_EXPORT int jllm_scale_expert_hidden(void* hidden, int dtype, const float* weights, int rows, int experts, int ff,
                                         int ld_w, int shared_ff, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && experts > 0 && ff > 0 && shared_ff >= 0 && ld_w >= experts + (shared_ff ? 1 : 0),
                 "scale_expert_hidden: rows=%d experts=%d ff=%d shared_ff=%d ld_w=%d", rows, experts, ff, shared_ff, ld_w);
    if (rows == 0) return JLLM_OK;
    const size_t total = (size_t)rows * ((size_t)experts * ff + shared_ff);
    const int per = dtype == JLLM_F32 ? 4 : 8;
    if (ff % per == 0 && shared_ff % per == 0 && ((uintptr_t)hidden % 16) == 0) {
        const size_t groups = total / per;
        const int vblocks = (int)min((size_t)65535, (groups + 255) / 256);
        if (dtype == JLLM_F32)
            jllm_launch(scale_expert_hidden_vec_kernel<float>, dim3(vblocks), dim3(256), 0, stream, LAUNCH_DEPENDENT,
                        (float*)hidden, weights, experts, ff, groups, ld_w, shared_ff);
        else
            jllm_launch(scale_expert_hidden_vec_kernel<__nv_bfloat16>, dim3(vblocks), dim3(256), 0, stream, LAUNCH_DEPENDENT,
                        (__nv_bfloat16*)hidden, weights, experts, ff, groups, ld_w, shared_ff);
        return jllm_check_launch("scale_expert_hidden");
    }
    const int blocks = (int)min((size_t)65535, (total + 255) / 256);
    if (dtype == JLLM_F32)
        jllm_launch(scale_expert_hidden_kernel<float>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, (float*)hidden,
                    weights, experts, ff, total, ld_w, shared_ff);
    else
        jllm_launch(scale_expert_hidden_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT,
                    (__nv_bfloat16*)hidden, weights, experts, ff, total, ld_w, shared_ff);
    return jllm_check_launch("scale_expert_hidden");
}
