// Small element-by-element kernels between the products.
//
//   sigmoid_gate     y[r, i] <- y[r, i] * sigmoid(g[r, i]) * scale      a gate of full width in front of an output projection
//   activation       x <- act(x) in place; act: the erf form of GELU, z (1 + erf(z / sqrt 2)) / 2
//   add_rows_scaled  x[r, :] += w[r] * h[r, :]                          a row's input handed through with a weight of its own
//
// Float32 arithmetic; T is the stored type.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ y, int ld_y, const T* __restrict__ g, int ld_g, int width, float scale) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y;
    T* yr = y + (size_t)r * ld_y;
    const T* gr = g + (size_t)r * ld_g;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < width; i += gridDim.x * blockDim.x) {
        const float s = 1.f / (1.f + expf(-to_float(gr[i])));
        yr[i] = from_float<T>(__fmul_rn(__fmul_rn(to_float(yr[i]), s), scale));
    }
}

// The same, 16 bytes a thread (rows and the gate's view on 16-byte boundaries, the width a multiple of the group).
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_vec_kernel(T* __restrict__ y, int ld_y, const T* __restrict__ g, int ld_g, int width, float scale) {
    constexpr int N = 16 / sizeof(T);
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y;
    T* yr = y + (size_t)r * ld_y;
    const T* gr = g + (size_t)r * ld_g;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * N; i < width; i += gridDim.x * blockDim.x * N) {
        uint4 yv = *reinterpret_cast<const uint4*>(yr + i);
        const uint4 gv = *reinterpret_cast<const uint4*>(gr + i);
        T* ye = reinterpret_cast<T*>(&yv);
        const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
        for (int k = 0; k < N; ++k) {
            const float s = 1.f / (1.f + expf(-to_float(ge[k])));
            ye[k] = from_float<T>(__fmul_rn(__fmul_rn(to_float(ye[k]), s), scale));
        }
        *reinterpret_cast<uint4*>(yr + i) = yv;
    }
}

enum : int { ACT_GELU_ERF = 1 };

template <typename T>
__global__ void __launch_bounds__(256)
activation_vec_kernel(T* __restrict__ x, size_t groups, int kind) {
    constexpr int N = 16 / sizeof(T);
    pdl_wait();
    pdl_trigger();
    for (size_t gi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += (size_t)gridDim.x * blockDim.x) {
        uint4 raw = *reinterpret_cast<const uint4*>(x + gi * N);
        T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int k = 0; k < N; ++k) {
            const float z = to_float(v[k]);
            v[k] = from_float<T>(0.5f * z * (1.f + erff(z * 0.70710678118654752f)));
        }
        *reinterpret_cast<uint4*>(x + gi * N) = raw;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
activation_kernel(T* __restrict__ x, size_t total, int kind) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float z = to_float(x[i]);
        x[i] = from_float<T>(0.5f * z * (1.f + erff(z * 0.70710678118654752f)));
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
add_rows_scaled_kernel(float* __restrict__ x, const T* __restrict__ h, int ld_h, const float* __restrict__ w, int ld_w, int dim) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y;
    const float wt = w[(size_t)r * ld_w];
    if (wt == 0.f) return;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += gridDim.x * blockDim.x)
        x[(size_t)r * dim + i] = fmaf(wt, to_float(h[(size_t)r * ld_h + i]), x[(size_t)r * dim + i]);
}

}  // namespace

JLLM_EXPORT int jllm_sigmoid_gate(void* y, int ld_y, const void* g, int ld_g, int dtype, int rows, int width, float scale,
                                  cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && rows <= 65535 && width > 0, "sigmoid_gate: rows=%d width=%d", rows, width);
    if (rows == 0) return JLLM_OK;
    const int per = dtype == JLLM_F32 ? 4 : 8;
    if (width % per == 0 && ld_y % per == 0 && ld_g % per == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)g % 16) == 0) {
        const dim3 vgrid(max(1, min(16, (width / per + 255) / 256)), rows);
        if (dtype == JLLM_F32)
            jllm_launch(sigmoid_gate_vec_kernel<float>, vgrid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (float*)y, ld_y, (const float*)g,
                        ld_g, width, scale);
        else
            jllm_launch(sigmoid_gate_vec_kernel<__nv_bfloat16>, vgrid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (__nv_bfloat16*)y, ld_y,
                        (const __nv_bfloat16*)g, ld_g, width, scale);
        return jllm_check_launch("sigmoid_gate");
    }
    const dim3 grid(max(1, min(32, (width + 255) / 256)), rows);
    if (dtype == JLLM_F32)
        jllm_launch(sigmoid_gate_kernel<float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (float*)y, ld_y, (const float*)g, ld_g,
                    width, scale);
    else
        jllm_launch(sigmoid_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (__nv_bfloat16*)y, ld_y,
                    (const __nv_bfloat16*)g, ld_g, width, scale);
    return jllm_check_launch("sigmoid_gate");
}

JLLM_EXPORT int jllm_activation(void* x, int dtype, long long total, int kind, cudaStream_t stream) {
    JLLM_REQUIRE(total >= 0 && kind == ACT_GELU_ERF, "activation: total=%lld kind=%d (built: 1, the erf form of GELU)", total, kind);
    if (total == 0) return JLLM_OK;
    const int per = dtype == JLLM_F32 ? 4 : 8;
    if (total % per == 0 && ((uintptr_t)x % 16) == 0) {
        const long long groups = total / per;
        const int vblocks = (int)min((long long)65535, (groups + 255) / 256);
        if (dtype == JLLM_F32)
            jllm_launch(activation_vec_kernel<float>, dim3(vblocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, (float*)x, (size_t)groups, kind);
        else
            jllm_launch(activation_vec_kernel<__nv_bfloat16>, dim3(vblocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, (__nv_bfloat16*)x,
                        (size_t)groups, kind);
        return jllm_check_launch("activation");
    }
    const int blocks = (int)min((long long)65535, (total + 255) / 256);
    if (dtype == JLLM_F32)
        jllm_launch(activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, (float*)x, (size_t)total, kind);
    else
        jllm_launch(activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, (__nv_bfloat16*)x,
                    (size_t)total, kind);
    return jllm_check_launch("activation");
}

JLLM_EXPORT int jllm_add_rows_scaled(float* x, const void* h, int dtype, int ld_h, const float* w, int ld_w, int rows, int dim,
                                     cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && rows <= 65535 && dim > 0, "add_rows_scaled: rows=%d dim=%d", rows, dim);
    if (rows == 0) return JLLM_OK;
    const dim3 grid(max(1, min(32, (dim + 255) / 256)), rows);
    if (dtype == JLLM_F32)
        jllm_launch(add_rows_scaled_kernel<float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, x, (const float*)h, ld_h, w, ld_w,
                    dim);
    else
        jllm_launch(add_rows_scaled_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, x, (const __nv_bfloat16*)h,
                    ld_h, w, ld_w, dim);
    return jllm_check_launch("add_rows_scaled");
}
