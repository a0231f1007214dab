// Recurrences whose state decays by ONE number per head and token, and what feeds them.
//
// The recurrence itself, per (request, head), with a state S [dk, dv] in float32 that lives in a state slot:
//
//     S_t = a_t S_(t-1) + (b_t k_t) v_t^T,        o_t = S_t^T (s q_t)  [+ D_head v_t]
//
// a_t = exp(la_t) and b_t are float32 numbers per (row, head) that a gate kernel in front has made; q, k, v are the
// projections as a product (or the convolution below) left them; several heads may share a q and a k (`q_groups`,
// `k_groups`: head h reads group h / (heads / groups)). With a normalizer (`nstate` [slots, heads, dk]) the kernel also
// carries n_t = a_t n_(t-1) + b_t k_t and divides: o_t / (max(|n_t . s q_t|, floor_t) + 1e-6), floor_t per (row, head).
// Two designs run on it: a selective state space (a = exp(-exp(A_log) dt), b = dt, k = B, q = C, v = x, the skip D) and a
// matrix memory with exponential gates (a = exp(f + m' - m), b = exp(i - m), floor = exp(-m), m the running maximum that
// keeps the exponentials in range).
//
// The gate kernels:
//   ssm_gates     dt = softplus(dt_raw + dt_bias); la = -exp(A_log) dt; b = dt                        per (row, head)
//   memory_gates  i = cap tanh((i_raw + bi) / cap), f = logsigmoid(cap tanh((f_raw + bf) / cap)); m_t = max(f + m_(t-1), i);
//                 la = f + m_(t-1) - m_t, b = exp(i - m_t), floor = exp(-m_t); m is a state [slots, heads] that starts at 0.
//                 The maximum is a chain whose steps compose, so a block shares a (segment, head)'s tokens out in runs.
// and the short causal convolution per channel in front of the state space:
//   causal_conv   y[t, c] = silu(bias[c] + sum_r w[c, r] u[t - (taps - 1) + r, c]), u from the rows of the same segment, and
//                 in front of the segment's first row from the request's state [slots, taps - 1, channels] (float32: the raw
//                 inputs of its last taps - 1 tokens, zero for a new request), which a second launch brings up to date
//                 once every row has been read (the same launch in a step of single rows).
// Everything here is float32 arithmetic; T is the type of the projections and of the convolution's result.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// ---- gates ---------------------------------------------------------------------------------------------------------
__global__ void ssm_gates_kernel(const float* __restrict__ dt_raw, int ld, VecRef dt_bias, VecRef a_log, float* __restrict__ la,
                                 float* __restrict__ b, int rows, int heads) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * heads) return;
    const int r = i / heads, h = i - r * heads;
    const float dt = softplus_f(__fadd_rn(dt_raw[(size_t)r * ld + h], dt_bias[h]));
    la[i] = -__fmul_rn(expf(a_log[h]), dt);
    b[i] = dt;
}

// A block per (segment, head). The running maximum m_t = max(f_t + m_(t-1), i_t) is a chain, but one whose steps compose: a
// run of tokens acts on the m in front of it as m -> max(m + F, I) with F the sum of its f and I what the run alone would
// leave; two runs in a row give (F1 + F2, max(I1 + F2, I2)). Every thread takes a run of neighbouring tokens (the gates'
// transcendental functions are the work, and they are all independent), the runs' maps are composed in order by one thread,
// and every thread walks its run again from the m that stands in front of it.
__global__ void __launch_bounds__(256)
memory_gates_kernel(const float* __restrict__ raw, int ld, int i_off, int f_off, VecRef i_bias, VecRef f_bias,
                    float cap, float* __restrict__ mstate, int num_slots, const int* __restrict__ seg_start,
                    const int* __restrict__ seg_len, const int* __restrict__ state_slots, float* __restrict__ la,
                    float* __restrict__ b, float* __restrict__ floor_out, int segments, int heads) {
    __shared__ float sF[256], sI[256];
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x / heads, h = blockIdx.x - seg * heads, tid = threadIdx.x;
    const int first = seg_start[seg], n = seg_len[seg], slot = state_slots[seg];
    if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    const float bi = i_bias[h], bf = f_bias[h], inv_cap = 1.f / cap;
    const int per = (n + 255) / 256, lo = min(n, tid * per), hi = min(n, lo + per);
    auto gates = [&](int t, float& ig, float& fg) {
        const size_t r = (size_t)(first + t);
        ig = cap * tanhf((raw[r * ld + i_off + h] + bi) * inv_cap);
        fg = logsigmoid_f(cap * tanhf((raw[r * ld + f_off + h] + bf) * inv_cap));
    };
    // this thread's run as a map of the m in front of it: (F, I); an empty run is (0, -inf)
    float F = 0.f, I = -INFINITY;
    for (int t = lo; t < hi; ++t) {
        float ig, fg;
        gates(t, ig, fg);
        F += fg;
        I = fmaxf(I + fg, ig);
    }
    sF[tid] = F;
    sI[tid] = I;
    __syncthreads();
    // the m in front of every run: thread 0 walks the 256 maps in order (each step an add and a max)
    if (tid == 0) {
        float m = mstate[(size_t)slot * heads + h];
        for (int k = 0; k < 256; ++k) {
            const float f_run = sF[k], i_run = sI[k];
            sF[k] = m;
            m = fmaxf(m + f_run, i_run);
        }
        mstate[(size_t)slot * heads + h] = m;
    }
    __syncthreads();
    float m = sF[tid];
    for (int t = lo; t < hi; ++t) {
        float ig, fg;
        gates(t, ig, fg);
        const float m_new = fmaxf(fg + m, ig);
        const size_t r = (size_t)(first + t);
        la[r * heads + h] = fg + m - m_new;
        b[r * heads + h] = expf(ig - m_new);
        floor_out[r * heads + h] = expf(-m_new);
        m = m_new;
    }
}

// The normalizer of a matrix memory as one more value column. n_t = a_t n_(t-1) + b_t k_t is the recurrence of S with a value
// that is always 1, and n_t . q is that column's output: so the values get a column of ones behind them (`memory_values`: a
// head's dv values, a 1, zeros up to a width of dvp), the state is [dk, dvp] with n in column dv, the recurrence (token by
// token or in chunks) needs no case of its own, and `memory_divide` takes the column out again:
// o[:, :dv] / (max(|o[:, dv]|, floor) + 1e-6).
template <typename T>
__global__ void __launch_bounds__(256)
memory_values_kernel(const T* __restrict__ v, int ld, int off, T* __restrict__ out, int heads, int dv, int dvp) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y, width = heads * dvp;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < width; i += gridDim.x * blockDim.x) {
        const int h = i / dvp, c = i - h * dvp;
        out[(size_t)r * width + i] = c < dv ? v[(size_t)r * ld + off + (size_t)h * dv + c] : from_float<T>(c == dv ? 1.f : 0.f);
    }
}

__global__ void __launch_bounds__(256)
memory_divide_kernel(const float* __restrict__ o, const float* __restrict__ floor_in, float* __restrict__ out, int heads, int dv,
                     int dvp) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y, width = heads * dv;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < width; i += gridDim.x * blockDim.x) {
        const int h = i / dv, c = i - h * dv;
        const float* src = o + ((size_t)r * heads + h) * dvp;
        const float den = fmaxf(fabsf(src[dv]), floor_in[(size_t)r * heads + h]) + 1e-6f;
        out[(size_t)r * width + i] = src[c] / den;
    }
}

// ---- the short convolution -------------------------------------------------------------------------------------------
constexpr int MAX_TAPS = 16;

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const TI* __restrict__ u, int ld, int off, VecRef w, VecRef bias, float* __restrict__ state, int num_slots,
                   const int* __restrict__ row_seg, const int* __restrict__ seg_start, const int* __restrict__ state_slots,
                   TO* __restrict__ y, int ld_y, int rows, int channels, int taps, int single) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= channels || r >= rows) return;
    const int seg = row_seg[r], t = r - seg_start[seg], slot = state_slots[seg];
    if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    float* st = state + (size_t)slot * (taps - 1) * channels;
    float acc = bias[c];
    for (int j = 0; j < taps; ++j) {            // tap j reads the input of local index t - (taps - 1) + j
        const int at = t - (taps - 1) + j;
        const float in = at >= 0 ? to_float(u[(size_t)(r - (taps - 1) + j) * ld + off + c]) : st[(size_t)(taps - 1 + at) * channels + c];
        acc = fmaf(w[(size_t)c * taps + j], in, acc);
        // a step of single rows (t = 0): this thread alone touches (slot, channel); entry j - 1 has been read one turn ago
        if (single && j > 0) st[(size_t)(j - 1) * channels + c] = in;
    }
    y[(size_t)r * ld_y + c] = from_float<TO>(acc / (1.f + expf(-acc)));
}

// The same for prompt portions with a window of inputs in registers: a thread owns one channel of ROWS neighbouring rows, so
// an input is read once and not `taps` times. Where a row begins a segment (or the thread's run) the window is filled anew, from
// the rows in front of it or, in front of the segment's first row, from the request's state.
template <typename TI, typename TO, int TAPS, int ROWS>
__global__ void __launch_bounds__(256)
causal_conv_rows_kernel(const TI* __restrict__ u, int ld, int off, VecRef w, VecRef bias, const float* __restrict__ state,
                        int num_slots, const int* __restrict__ row_seg, const int* __restrict__ seg_start,
                        const int* __restrict__ state_slots, TO* __restrict__ y, int ld_y, int rows, int channels) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r0 = blockIdx.y * ROWS;
    if (c >= channels) return;
    float wt[TAPS], win[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wt[j] = w[(size_t)c * TAPS + j];
    const float bc = bias[c];
    int seg_now = -1;
    for (int r = r0; r < min(rows, r0 + ROWS); ++r) {
        const int seg = row_seg[r];
        const float in = to_float(u[(size_t)r * ld + off + c]);
        if (seg != seg_now) {           // the window in front of this row: earlier rows of the segment, else the state
            seg_now = seg;
            const int t = r - seg_start[seg], slot = state_slots[seg];
            const bool ok = jllm_in_bounds(slot, num_slots, BOUNDS_SLOT);
            const float* st = state + (size_t)(ok ? slot : 0) * (TAPS - 1) * channels;
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) {
                const int at = t - (TAPS - 1) + j;
                win[j] = at >= 0 ? to_float(u[(size_t)(r - (TAPS - 1) + j) * ld + off + c]) : (ok ? st[(size_t)(TAPS - 1 + at) * channels + c] : 0.f);
            }
        }
        win[TAPS - 1] = in;
        float acc = bc;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) acc = fmaf(wt[j], win[j], acc);
        y[(size_t)r * ld_y + c] = from_float<TO>(acc / (1.f + expf(-acc)));
#pragma unroll
        for (int j = 0; j + 1 < TAPS; ++j) win[j] = win[j + 1];
    }
}

template <typename TI>
__global__ void __launch_bounds__(256)
conv_state_kernel(const TI* __restrict__ u, int ld, int off, float* __restrict__ state, int num_slots,
                  const int* __restrict__ seg_start, const int* __restrict__ seg_len, const int* __restrict__ state_slots,
                  int channels, int taps) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, seg = blockIdx.y;
    if (c >= channels) return;
    const int first = seg_start[seg], n = seg_len[seg], slot = state_slots[seg];
    if (n <= 0 || !jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    float* st = state + (size_t)slot * (taps - 1) * channels;
    float keep[MAX_TAPS];
    for (int j = 0; j + 1 < taps; ++j) {        // the new entry j is the input of local index n - (taps - 1) + j
        const int at = n - (taps - 1) + j;
        keep[j] = at >= 0 ? to_float(u[(size_t)(first + at) * ld + off + c]) : st[(size_t)(taps - 1 + at) * channels + c];
    }
    for (int j = 0; j + 1 < taps; ++j) st[(size_t)j * channels + c] = keep[j];
}

// ---- the recurrence, token by token -----------------------------------------------------------------------------------
// A block owns CB = 32 value columns of one (segment, head). Thread (g, c) keeps R rows (g R .. g R + R - 1) of column c of
// the state in registers from the segment's first token to its last. TOKENS tokens at a time are staged in shared memory
// (b k, s q, v, a); a token's partial sums over the row groups meet in shared memory and are added in group order. Warp 0
// also carries the normalizer, a lane owning every 32nd key channel.
constexpr int TOK = 8;
constexpr int CB = 32;

template <typename T, int R>
__global__ void __launch_bounds__(1024)
scalar_gated_recurrent_kernel(const T* __restrict__ qp, int ld_q, int q_off, int q_groups, const T* __restrict__ kp, int ld_k,
                              int k_off, int k_groups, const T* __restrict__ vp, int ld_v, int v_off,
                              const float* __restrict__ la, const float* __restrict__ bsc, const float* __restrict__ floor_in,
                              VecRef skip, int has_skip, float* __restrict__ state, float* __restrict__ nstate, int num_slots,
                              const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                              const int* __restrict__ state_slots, float* __restrict__ o, int heads, int dk, int dv,
                              float q_scale) {
    extern __shared__ __align__(16) float smem[];
    const int G = blockDim.x / CB;
    float* ks = smem;                    // [TOK][dk]   b k
    float* qs = ks + TOK * dk;           // [TOK][dk]   s q
    float* vs = qs + TOK * dk;           // [TOK][CB]
    float* as = vs + TOK * CB;           // [TOK]       a
    float* nq = as + TOK;                // [TOK]       the divisor (1 without a normalizer)
    float* part = nq + TOK;              // [TOK][G][CB]
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CB;
    const int tid = threadIdx.x, c = tid % CB, g = tid / CB, j = c0 + c;
    const int first = seg_start[seg], n = seg_len[seg], slot = state_slots[seg];
    if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    float* S = state + (((size_t)slot * heads + h) * dk) * dv;
    const int qg = h / (heads / q_groups), kg = h / (heads / k_groups);
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        s[r] = (i < dk && j < dv) ? S[(size_t)i * dv + j] : 0.f;
    }
    // the normalizer: lane l of warp 0 owns channels l, l + 32, ... (up to 16 of them: dk <= 512)
    float nn[16];
    float* N = nstate ? nstate + ((size_t)slot * heads + h) * dk : nullptr;
    if (N && tid < 32) {
#pragma unroll
        for (int u = 0; u < 16; ++u) nn[u] = tid + 32 * u < dk ? N[tid + 32 * u] : 0.f;
    }
    const float d_skip = has_skip ? skip[h] : 0.f;
    for (int t0 = 0; t0 < n; t0 += TOK) {
        const int nt = min(TOK, n - t0);
        for (int e = tid; e < nt * dk; e += blockDim.x) {
            const int t = e / dk, i = e - t * dk;
            const size_t r = (size_t)(first + t0 + t);
            ks[e] = __fmul_rn(bsc[r * heads + h], to_float(kp[r * ld_k + k_off + (size_t)kg * dk + i]));
            qs[e] = __fmul_rn(to_float(qp[r * ld_q + q_off + (size_t)qg * dk + i]), q_scale);
        }
        for (int e = tid; e < nt * CB; e += blockDim.x) {
            const int t = e / CB, cc = e - t * CB;
            vs[e] = c0 + cc < dv ? to_float(vp[(size_t)(first + t0 + t) * ld_v + v_off + (size_t)h * dv + c0 + cc]) : 0.f;
        }
        if (tid < nt) as[tid] = expf(la[(size_t)(first + t0 + tid) * heads + h]);
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float a = as[t], v = vs[t * CB + c];
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int r = 0; r < R; r += 2) {
                const int i = g * R + r;
                if (i < dk) {
                    s[r] = fmaf(a, s[r], __fmul_rn(ks[t * dk + i], v));
                    acc0 = fmaf(s[r], qs[t * dk + i], acc0);
                }
                if (i + 1 < dk) {
                    s[r + 1] = fmaf(a, s[r + 1], __fmul_rn(ks[t * dk + i + 1], v));
                    acc1 = fmaf(s[r + 1], qs[t * dk + i + 1], acc1);
                }
            }
            part[(t * G + g) * CB + c] = acc0 + acc1;
        }
        if (tid < 32) {
            for (int t = 0; t < nt; ++t) {
                float d = 1.f;
                if (N) {
                    float dot = 0.f;
#pragma unroll
                    for (int u = 0; u < 16; ++u) {
                        const int i = tid + 32 * u;
                        if (i < dk) {
                            nn[u] = fmaf(as[t], nn[u], ks[t * dk + i]);
                            dot = fmaf(nn[u], qs[t * dk + i], dot);
                        }
                    }
                    dot = warp_sum(dot);
                    d = fmaxf(fabsf(dot), floor_in[(size_t)(first + t0 + t) * heads + h]) + 1e-6f;
                }
                if (tid == 0) nq[t] = d;
            }
        }
        __syncthreads();
        for (int e = tid; e < nt * CB; e += blockDim.x) {
            const int t = e / CB, cc = e - t * CB;
            if (c0 + cc >= dv) continue;
            float acc = 0.f;
            for (int gg = 0; gg < G; ++gg) acc += part[(t * G + gg) * CB + cc];
            if (N) acc = acc / nq[t];
            if (has_skip) acc = fmaf(d_skip, vs[t * CB + cc], acc);
            o[(size_t)(first + t0 + t) * ((size_t)heads * dv) + (size_t)h * dv + c0 + cc] = acc;
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        if (i < dk && j < dv) S[(size_t)i * dv + j] = s[r];
    }
    if (N && tid < 32 && blockIdx.z == 0) {
#pragma unroll
        for (int u = 0; u < 16; ++u)
            if (tid + 32 * u < dk) N[tid + 32 * u] = nn[u];
    }
}

template <typename T, int R>
int launch_recurrent(const void* q, int ld_q, int q_off, int q_groups, const void* k, int ld_k, int k_off, int k_groups,
                     const void* v, int ld_v, int v_off, const float* la, const float* b, const float* floor_in, VecRef skip,
                     int has_skip, float* state, float* nstate, int num_slots, const int* seg_start, const int* seg_len,
                     const int* state_slots, float* o, int segments, int heads, int dk, int dv, float q_scale,
                     cudaStream_t stream) {
    const int G = (dk + R - 1) / R;
    const size_t smem = (size_t)(2 * TOK * dk + TOK * CB + 2 * TOK + TOK * G * CB) * sizeof(float);
    auto kernel = scalar_gated_recurrent_kernel<T, R>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return jllm_fail(JLLM_CUDA_ERROR, "scalar_gated_recurrent: %zu bytes of shared memory refused", smem);
    jllm_launch(kernel, dim3(segments, heads, (dv + CB - 1) / CB), dim3(G * CB), smem, stream, LAUNCH_DEPENDENT, (const T*)q,
                ld_q, q_off, q_groups, (const T*)k, ld_k, k_off, k_groups, (const T*)v, ld_v, v_off, la, b, floor_in, skip,
                has_skip, state, nstate, num_slots, seg_start, seg_len, state_slots, o, heads, dk, dv, q_scale);
    return jllm_check_launch("scalar_gated_recurrent");
}

template <typename T>
int launch_recurrent_rows(int dk, const void* q, int ld_q, int q_off, int q_groups, const void* k, int ld_k, int k_off,
                          int k_groups, const void* v, int ld_v, int v_off, const float* la, const float* b,
                          const float* floor_in, VecRef skip, int has_skip, float* state, float* nstate, int num_slots,
                          const int* seg_start, const int* seg_len, const int* state_slots, float* o, int segments, int heads,
                          int dv, float q_scale, cudaStream_t stream) {
#define JLLM_SGR(R)                                                                                                          \
    return launch_recurrent<T, R>(q, ld_q, q_off, q_groups, k, ld_k, k_off, k_groups, v, ld_v, v_off, la, b, floor_in, skip,   \
                                  has_skip, state, nstate, num_slots, seg_start, seg_len, state_slots, o, segments, heads, dk, \
                                  dv, q_scale, stream)
    if (dk <= 64) JLLM_SGR(4);
    if (dk <= 128) JLLM_SGR(8);
    if (dk <= 256) JLLM_SGR(16);
    JLLM_SGR(32);
#undef JLLM_SGR
}

}  // namespace

JLLM_BOUNDS_READER(gated_recurrence)

// dt_raw: a float32 view [rows, ld] whose first `heads` columns are the raw step sizes; la, b [rows, heads] float32.
JLLM_EXPORT int jllm_ssm_gates(const float* dt_raw, int ld, const void* dt_bias, const void* a_log, int vec_dtype, float* la,
                               float* b, int rows, int heads, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && ld >= heads, "ssm_gates: rows=%d heads=%d ld=%d", rows, heads, ld);
    if (rows == 0) return JLLM_OK;
    const int total = rows * heads;
    jllm_launch(ssm_gates_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, LAUNCH_DEPENDENT, dt_raw, ld,
                VecRef{dt_bias, vec_dtype}, VecRef{a_log, vec_dtype}, la, b, rows, heads);
    return jllm_check_launch("ssm_gates");
}

// raw: a float32 view [rows, ld] with the input gate's raw values at column i_off and the forget gate's at f_off (heads
// each); mstate [slots, heads] float32; la, b, floor_out [rows, heads] float32.
JLLM_EXPORT int jllm_memory_gates(const float* raw, int ld, int i_off, int f_off, const void* i_bias, const void* f_bias,
                                  int vec_dtype, float cap, float* mstate, int num_slots, const int* seg_start,
                                  const int* seg_len, const int* state_slots, float* la, float* b, float* floor_out,
                                  int segments, int heads, cudaStream_t stream) {
    JLLM_REQUIRE(segments >= 0 && heads > 0 && cap > 0.f, "memory_gates: segments=%d heads=%d cap=%g", segments, heads,
                 (double)cap);
    if (segments == 0) return JLLM_OK;
    const int total = segments * heads;
    jllm_launch(memory_gates_kernel, dim3(total), dim3(256), 0, stream, LAUNCH_DEPENDENT, raw, ld, i_off, f_off,
                VecRef{i_bias, vec_dtype}, VecRef{f_bias, vec_dtype}, cap, mstate, num_slots, seg_start, seg_len, state_slots,
                la, b, floor_out, segments, heads);
    return jllm_check_launch("memory_gates");
}

// v: a view [rows, ld] of type `dtype` with heads x dv values at column `off`; out [rows, heads x dvp] of the same type.
JLLM_EXPORT int jllm_memory_values(const void* v, int dtype, int ld, int off, void* out, int rows, int heads, int dv, int dvp,
                                   cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && rows <= 65535 && heads > 0 && dv > 0 && dvp > dv, "memory_values: rows=%d heads=%d dv=%d dvp=%d", rows,
                 heads, dv, dvp);
    if (rows == 0) return JLLM_OK;
    const dim3 grid(max(1, min(32, (heads * dvp + 255) / 256)), rows);
    if (dtype == JLLM_F32)
        jllm_launch(memory_values_kernel<float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (const float*)v, ld, off, (float*)out,
                    heads, dv, dvp);
    else
        jllm_launch(memory_values_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (const __nv_bfloat16*)v, ld,
                    off, (__nv_bfloat16*)out, heads, dv, dvp);
    return jllm_check_launch("memory_values");
}

// o [rows, heads x dvp] float32 with the normalizer's output in column dv of every head; floor_in [rows, heads]; out
// [rows, heads x dv] float32.
JLLM_EXPORT int jllm_memory_divide(const float* o, const float* floor_in, float* out, int rows, int heads, int dv, int dvp,
                                   cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && rows <= 65535 && heads > 0 && dv > 0 && dvp > dv, "memory_divide: rows=%d heads=%d dv=%d dvp=%d", rows,
                 heads, dv, dvp);
    if (rows == 0) return JLLM_OK;
    const dim3 grid(max(1, min(32, (heads * dv + 255) / 256)), rows);
    jllm_launch(memory_divide_kernel, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, o, floor_in, out, heads, dv, dvp);
    return jllm_check_launch("memory_divide");
}

// u: a view [rows, ld] of type `in_dtype` whose columns [off, off + channels) are the convolution's inputs; w [channels, taps]
// and bias [channels] of type `vec_dtype`; state [slots, taps - 1, channels] float32; y [rows, ld_y] of type `out_dtype`.
JLLM_EXPORT int jllm_causal_conv(const void* u, int in_dtype, int ld, int off, const void* w, const void* bias, int vec_dtype,
                                 float* state, int num_slots, const int* row_seg, const int* seg_start, const int* seg_len,
                                 const int* state_slots, void* y, int out_dtype, int ld_y, int rows, int segments, int channels,
                                 int taps, int single, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && channels > 0 && taps >= 1 && taps <= MAX_TAPS && rows <= 65535 * 64,
                 "causal_conv: rows=%d channels=%d taps=%d (at most %d)", rows, channels, taps, MAX_TAPS);
    if (rows == 0) return JLLM_OK;
    JLLM_REQUIRE(rows <= 65535 && segments <= 65535, "causal_conv: %d rows or %d segments in one launch", rows, segments);
    const VecRef wv{w, vec_dtype}, bv{bias, vec_dtype};
    const dim3 grid((channels + 255) / 256, rows), sgrid((channels + 255) / 256, segments);
    constexpr int RUN = 16;      // rows of a thread's run in the windowed form
    const dim3 rgrid((channels + 255) / 256, (rows + RUN - 1) / RUN);
#define JLLM_CONV_ROWS(TI, TO, TAPS)                                                                                            \
    jllm_launch(causal_conv_rows_kernel<TI, TO, TAPS, RUN>, rgrid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (const TI*)u, ld,    \
                off, wv, bv, (const float*)state, num_slots, row_seg, seg_start, state_slots, (TO*)y, ld_y, rows, channels)
#define JLLM_CONV(TI, TO)                                                                                                       \
    do {                                                                                                                        \
        if (!single && taps == 4) JLLM_CONV_ROWS(TI, TO, 4);                                                                    \
        else if (!single && taps == 3) JLLM_CONV_ROWS(TI, TO, 3);                                                               \
        else if (!single && taps == 2) JLLM_CONV_ROWS(TI, TO, 2);                                                               \
        else                                                                                                                    \
        jllm_launch(causal_conv_kernel<TI, TO>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (const TI*)u, ld, off, wv, bv,    \
                    state, num_slots, row_seg, seg_start, state_slots, (TO*)y, ld_y, rows, channels, taps, single);             \
        if (!single && taps > 1)                                                                                                \
            jllm_launch(conv_state_kernel<TI>, sgrid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (const TI*)u, ld, off, state,     \
                        num_slots, seg_start, seg_len, state_slots, channels, taps);                                            \
    } while (0)
    if (in_dtype == JLLM_F32 && out_dtype == JLLM_F32) JLLM_CONV(float, float);
    else if (in_dtype == JLLM_F32) JLLM_CONV(float, __nv_bfloat16);
    else if (out_dtype == JLLM_F32) JLLM_CONV(__nv_bfloat16, float);
    else JLLM_CONV(__nv_bfloat16, __nv_bfloat16);
#undef JLLM_CONV
#undef JLLM_CONV_ROWS
    return jllm_check_launch("causal_conv");
}

// q, k, v: views of type `dtype` with row strides ld_q, ld_k, ld_v and the given column offsets; la, b (and floor_in with a
// normalizer) [rows, heads] float32; state [slots, heads, dk, dv] and nstate [slots, heads, dk] (or null) float32;
// skip [heads] of type `skip_dtype` or null; o [rows, heads x dv] float32.
JLLM_EXPORT int jllm_scalar_gated_recurrent(const void* q, int ld_q, int q_off, int q_groups, const void* k, int ld_k, int k_off,
                                            int k_groups, const void* v, int ld_v, int v_off, int dtype, const float* la,
                                            const float* b, const float* floor_in, const void* skip, int skip_dtype,
                                            float* state, float* nstate, int num_slots, const int* seg_start,
                                            const int* seg_len, const int* state_slots, float* o, int segments, int heads,
                                            int dk, int dv, float q_scale, cudaStream_t stream) {
    JLLM_REQUIRE(segments >= 0 && heads > 0 && dk > 0 && dk <= 1024 && (nstate == nullptr || dk <= 512) && dv > 0,
                 "scalar_gated_recurrent: segments=%d heads=%d dk=%d (at most 1024; 512 with a normalizer) dv=%d", segments, heads,
                 dk, dv);
    JLLM_REQUIRE(q_groups > 0 && k_groups > 0 && heads % q_groups == 0 && heads % k_groups == 0,
                 "scalar_gated_recurrent: %d heads do not share %d queries or %d keys evenly", heads, q_groups, k_groups);
    JLLM_REQUIRE(nstate == nullptr || floor_in != nullptr, "scalar_gated_recurrent: a normalizer needs its floor");
    JLLM_REQUIRE(heads <= 65535 && (dv + CB - 1) / CB <= 65535, "scalar_gated_recurrent: heads=%d dv=%d", heads, dv);
    if (segments == 0) return JLLM_OK;
    const VecRef sk{skip, skip_dtype};
    if (dtype == JLLM_F32)
        return launch_recurrent_rows<float>(dk, q, ld_q, q_off, q_groups, k, ld_k, k_off, k_groups, v, ld_v, v_off, la, b,
                                            floor_in, sk, skip != nullptr, state, nstate, num_slots, seg_start, seg_len,
                                            state_slots, o, segments, heads, dv, q_scale, stream);
    return launch_recurrent_rows<__nv_bfloat16>(dk, q, ld_q, q_off, q_groups, k, ld_k, k_off, k_groups, v, ld_v, v_off, la, b,
                                                floor_in, sk, skip != nullptr, state, nstate, num_slots, seg_start, seg_len,
                                                state_slots, o, segments, heads, dv, q_scale, stream);
}
