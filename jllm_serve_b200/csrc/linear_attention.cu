// Gated linear attention: the recurrence over a request's tokens, and the per-head norm and gate of its output.
//
// Per head, with dk key channels and dv value channels, a request carries a state S [dk, dv] in 32-bit floats:
//     S_t = diag(d_t) S_(t-1) + k_t v_t^T,    o_t = S_t^T (scale * q_t),    d_t = sigmoid(z_t)^(1 / tau)
// d_t is formed as exp(log_sigmoid(z_t) / tau) in float32 by a kernel in front. The columns of S do not depend on one
// another, so a block owns CB columns (32, or 16 where that gives more SMs a block) of one (segment, head). A thread holds R
// rows of one column in registers (row group g, column c); every token's k, d, q and v are staged through shared
// memory eight tokens at a time, the next eight being fetched into registers while these are worked on, and the G
// partial sums of o_t are added in the order of g. A token's arithmetic is the same sequence of operations wherever its
// portion begins, whatever else the batch holds and however the columns are dealt out, so the result has the same
// bits for every cut.
//
// A segment is a run of consecutive rows of one request (a prompt portion, or one decoded token); its state lies in
// `state[slot]` ([slots, heads, dk, dv]), is read at the segment's first token and written back after its last. The
// same kernel serves a prompt and a decode step; the float32 and the bfloat16 path differ in the type of q, k, v only.
#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int TOKENS = 8;       // tokens staged at a time

// d = sigmoid(z)^(1 / tau), in place over [rows, heads x dk] float32: log(sigmoid(z)) = min(z, 0) - log1p(exp(-|z|)),
// times 1 / tau, exponentiated. Done once per step and element, in front of the recurrence (whose blocks would
// otherwise each redo it for the columns they own).
__global__ void gla_decay_kernel(float* __restrict__ z, float inv_tau, size_t total, int as_log) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float v = z[i];
        const float l = __fmul_rn(fminf(v, 0.f) - log1pf(expf(-fabsf(v))), inv_tau);
        z[i] = as_log ? l : expf(l);        // (the chunked kernels want the logarithm: they add it up over a chunk)
    }
}

// Linear attention with ONE fixed decay per head (no decay projection; "lightning" attention) runs through the same
// kernels: this pass fills the decay table with decay[h] for every key channel of head h (its logarithm for the chunked
// form; a decay of 0 becomes a logarithm of -1e30, whose differences are 0 or below -1e30 and never NaN), and applies
// the activation of such a mixer to its projections in place: q, k, v <- silu (activation 1). A block per row.
__device__ __forceinline__ float2 load_two(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_two(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store_two(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_two(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename T>
__global__ void __launch_bounds__(256)
fixed_decay_prepare_kernel(T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, float* __restrict__ z,
                           const float* __restrict__ decay, int heads, int dk, int dv, int as_log, int activation) {
    pdl_wait();
    pdl_trigger();
    const size_t r = blockIdx.x;
    float* zr = z + r * heads * dk;
    if (z == nullptr) {
        // (the tensor-core form of the chunks takes the decays themselves: no table)
    } else if ((dk & 3) == 0) {        // (the table's rows are whole float4s then: heads * dk is a multiple of 4, z is an allocation's start)
        for (int i = threadIdx.x; i < heads * dk / 4; i += blockDim.x) {
            const float d = decay[(4 * i) / dk], e = as_log ? fmaxf(logf(d), -1e30f) : d;
            reinterpret_cast<float4*>(zr)[i] = make_float4(e, e, e, e);
        }
    } else {
        for (int i = threadIdx.x; i < heads * dk; i += blockDim.x) {
            const float d = decay[i / dk];
            zr[i] = as_log ? fmaxf(logf(d), -1e30f) : d;
        }
    }
    if (!activation) return;
    T* row = proj + r * ld;
    auto silu = [](float x) { return x / (1.f + expf(-x)); };
    auto run = [&](int off, int n) {
        T* p = row + off;
        if ((n & 1) == 0 && (((uintptr_t)p) & (2 * sizeof(T) - 1)) == 0) {
            for (int i = threadIdx.x; i < n / 2; i += blockDim.x) {
                const float2 v = load_two(p + 2 * i);
                store_two(p + 2 * i, silu(v.x), silu(v.y));
            }
        } else {
            for (int i = threadIdx.x; i < n; i += blockDim.x) p[i] = from_float<T>(silu(to_float(p[i])));
        }
    };
    run(q_off, heads * dk);
    run(k_off, heads * dk);
    run(v_off, heads * dv);
}

template <typename T>
int launch_fixed_decay(void* proj, int ld, int q_off, int k_off, int v_off, float* z, const float* decay, int rows, int heads,
                       int dk, int dv, int as_log, int activation, cudaStream_t stream) {
    jllm_launch(fixed_decay_prepare_kernel<T>, dim3(rows), dim3(256), 0, stream, LAUNCH_DEPENDENT, (T*)proj, ld, q_off, k_off,
                v_off, z, decay, heads, dk, dv, as_log, activation);
    return jllm_check_launch("fixed_decay_prepare");
}

template <typename T, int R, int CB, bool V4>
__global__ void __launch_bounds__(1024)
gla_recurrent_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                     float* __restrict__ state, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                     const int* __restrict__ state_slots, float* __restrict__ o, int heads, int dk, int dv, float q_scale,
                     int num_slots, const float* __restrict__ head_decay, int activation) {
    // `head_decay` (else null): one fixed decay per head instead of the table; `activation` 1: q, k and v are taken through
    // silu as they are fetched (and rounded to the projections' type, as a pass that stored them would have left them)
    constexpr int EPT = TOKENS * R / CB;            // staged values of k (and of q, of d) a thread fetches per round
    extern __shared__ __align__(16) float smem[];
    const int threads = blockDim.x, G = threads / CB;
    const int stage = TOKENS * (3 * dk + CB);       // floats of one staging buffer: k, d, q [TOKENS][dk], v [TOKENS][CB]
    float* part = smem + 2 * stage;                 // [TOKENS][G][CB]
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CB;
    const int tid = threadIdx.x, c = tid % CB, g = tid / CB, j = c0 + c;
    const int first = seg_start[seg], n = seg_len[seg], slot = state_slots[seg];
    if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    float* S = state + (((size_t)slot * heads + h) * dk) * dv;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        s[r] = (i < dk && j < dv) ? S[(size_t)i * dv + j] : 0.f;
    }
    // which staged values this thread fetches: the same places of every round, worked out once
    int st[EPT], sp[EPT], sd[EPT];                  // token within the round (TOKENS: none), offsets into proj and decay
#pragma unroll
    for (int u = 0; u < EPT; ++u) {
        const int e = tid + u * threads;
        st[u] = e < TOKENS * dk ? e / dk : TOKENS;
        const int i = e - st[u] * dk;
        sp[u] = st[u] * ld + h * dk + i;
        sd[u] = st[u] * heads * dk + h * dk + i;
    }
    const int vt = tid / CB, vc = tid - vt * CB;    // the one value of v this thread fetches (threads >= TOKENS x CB / 1)
    const int vpt = (TOKENS * CB + threads - 1) / threads;
    float fk[EPT], fq[EPT], fd[EPT], fv[TOKENS];
    const float fixed = head_decay ? head_decay[h] : 1.f;
    auto act = [&](float x) { return activation ? to_float(from_float<T>(x / (1.f + expf(-x)))) : x; };

    auto fetch = [&](int t0) {      // the round that starts at token t0: from global memory into registers
        const int nt = min(TOKENS, n - t0);
        const size_t base = (size_t)(first + t0);
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            fk[u] = fq[u] = 0.f;
            fd[u] = 1.f;
            if (st[u] < nt) {
                const T* p = proj + base * ld + sp[u];
                fk[u] = act(to_float(p[k_off]));
                fq[u] = act(to_float(p[q_off]));
                fd[u] = head_decay ? fixed : decay[base * ((size_t)heads * dk) + sd[u]];
            }
        }
#pragma unroll
        for (int u = 0; u < TOKENS; ++u) {
            fv[u] = 0.f;
            if (u < vpt) {
                const int t = vt + u * (threads / CB);
                if (t < nt && c0 + vc < dv) fv[u] = act(to_float(proj[(base + t) * ld + v_off + (size_t)h * dv + c0 + vc]));
            }
        }
    };
    auto park = [&](int b) {        // ... and from the registers into staging buffer b
        float* ks = smem + b * stage;
        float* ds = ks + TOKENS * dk;
        float* qs = ds + TOKENS * dk;
        float* vs = qs + TOKENS * dk;
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            const int e = tid + u * threads;
            if (e < TOKENS * dk) {
                ks[e] = fk[u];
                ds[e] = fd[u];
                qs[e] = __fmul_rn(fq[u], q_scale);
            }
        }
#pragma unroll
        for (int u = 0; u < TOKENS; ++u) {
            const int t = vt + u * (threads / CB);
            if (u < vpt && t < TOKENS) vs[t * CB + vc] = fv[u];
        }
    };

    if (n > 0) {
        fetch(0);
        park(0);
    }
    __syncthreads();
    const bool rows_in = g * R < dk;
    for (int t0 = 0, b = 0; t0 < n; t0 += TOKENS, b ^= 1) {
        const int nt = min(TOKENS, n - t0);
        const bool more = t0 + TOKENS < n;
        if (more) fetch(t0 + TOKENS);               // on their way while this round's tokens are worked on
        const float* ks = smem + b * stage + g * R;
        const float* ds = ks + TOKENS * dk;
        const float* qs = ds + TOKENS * dk;
        const float* vs = smem + b * stage + 3 * TOKENS * dk;
        for (int t = 0; t < nt; ++t) {
            const float v = vs[t * CB + c];
            float acc0 = 0.f, acc1 = 0.f;
            if constexpr (V4) {     // dk a multiple of 4: four rows' k, d and q in one load each
                if (rows_in) {
#pragma unroll
                    for (int r = 0; r < R; r += 4) {
                        if (g * R + r < dk) {
                            const float4 kk = *reinterpret_cast<const float4*>(ks + t * dk + r);
                            const float4 dd = *reinterpret_cast<const float4*>(ds + t * dk + r);
                            const float4 qq = *reinterpret_cast<const float4*>(qs + t * dk + r);
                            s[r] = fmaf(dd.x, s[r], __fmul_rn(kk.x, v));
                            s[r + 1] = fmaf(dd.y, s[r + 1], __fmul_rn(kk.y, v));
                            s[r + 2] = fmaf(dd.z, s[r + 2], __fmul_rn(kk.z, v));
                            s[r + 3] = fmaf(dd.w, s[r + 3], __fmul_rn(kk.w, v));
                            acc0 = fmaf(s[r], qq.x, acc0);
                            acc1 = fmaf(s[r + 1], qq.y, acc1);
                            acc0 = fmaf(s[r + 2], qq.z, acc0);
                            acc1 = fmaf(s[r + 3], qq.w, acc1);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; r += 2) {
                    if (g * R + r < dk) {
                        s[r] = fmaf(ds[t * dk + r], s[r], __fmul_rn(ks[t * dk + r], v));
                        acc0 = fmaf(s[r], qs[t * dk + r], acc0);
                    }
                    if (g * R + r + 1 < dk) {
                        s[r + 1] = fmaf(ds[t * dk + r + 1], s[r + 1], __fmul_rn(ks[t * dk + r + 1], v));
                        acc1 = fmaf(s[r + 1], qs[t * dk + r + 1], acc1);
                    }
                }
            }
            part[(t * G + g) * CB + c] = acc0 + acc1;
        }
        if (more) park(b ^ 1);                      // (the other buffer: its last readers passed the barrier below)
        __syncthreads();
        for (int e = tid; e < nt * CB; e += threads) {
            const int t = e / CB, cc = e - t * CB;
            if (c0 + cc >= dv) continue;
            float acc = 0.f;
            for (int gg = 0; gg < G; ++gg) acc += part[(t * G + gg) * CB + cc];
            o[(size_t)(first + t0 + t) * ((size_t)heads * dv) + (size_t)h * dv + c0 + cc] = acc;
        }
        __syncthreads();                            // `part` and buffer b may be written again
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        if (i < dk && j < dv) S[(size_t)i * dv + j] = s[r];
    }
}

template <typename T, int R, int CB, bool V4>
int launch_recurrent(const void* proj, int ld, int q_off, int k_off, int v_off, const float* decay, float* state,
                     const int* seg_start, const int* seg_len, const int* state_slots, float* o, int segments, int heads,
                     int dk, int dv, float q_scale, int num_slots, const float* head_decay, int activation,
                     cudaStream_t stream) {
    const int per_warp = 32 / CB;
    const int G = ((dk + R - 1) / R + per_warp - 1) / per_warp * per_warp;       // row groups: whole warps
    const size_t smem = (size_t)(2 * TOKENS * (3 * dk + CB) + TOKENS * G * CB) * sizeof(float);
    auto kernel = gla_recurrent_kernel<T, R, CB, V4>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return jllm_fail(JLLM_CUDA_ERROR, "gla_recurrent: %zu bytes of shared memory refused", smem);
    jllm_launch(kernel, dim3(segments, heads, (dv + CB - 1) / CB), dim3(G * CB), smem, stream, LAUNCH_DEPENDENT,
                (const T*)proj, ld, q_off, k_off, v_off, decay, state, seg_start, seg_len, state_slots, o, heads, dk, dv,
                q_scale, num_slots, head_decay, activation);
    return jllm_check_launch("gla_recurrent");
}

// Columns per block: 32 (a warp is one row group), or 16 where 32 columns per block leave SMs without one. The choice
// changes which thread holds which value, not what is computed.
template <typename T, int R>
int launch_recurrent_cols(const void* proj, int ld, int q_off, int k_off, int v_off, const float* decay, float* state,
                          const int* seg_start, const int* seg_len, const int* state_slots, float* o, int segments,
                          int heads, int dk, int dv, float q_scale, int num_slots, const float* head_decay, int activation,
                          cudaStream_t stream) {
    const long long sms = max(1, jllm_device_sm_count());
    const long long units = (long long)segments * heads;
    const bool wide = units * ((dv + 31) / 32) >= sms || dv <= 16;
#define JLLM_GLA_COLS(CB, V4)                                                                                                  \
    return launch_recurrent<T, R, CB, V4>(proj, ld, q_off, k_off, v_off, decay, state, seg_start, seg_len, state_slots, o, \
                                          segments, heads, dk, dv, q_scale, num_slots, head_decay, activation, stream)
    if (dk % 4 == 0) {
        if (wide) JLLM_GLA_COLS(32, true);
        JLLM_GLA_COLS(16, true);
    }
    if (wide) JLLM_GLA_COLS(32, false);
    JLLM_GLA_COLS(16, false);
#undef JLLM_GLA_COLS
}

// ---- a prompt portion in chunks of 16 tokens ---------------------------------------------------------------------------
// Within a chunk that starts with the state S0, with L_t the sum of the log-decays of the chunk's tokens up to t (per key
// channel, <= 0) and L the sum over the whole chunk:
//     o_t = (q_t * exp(L_t))^T S0  +  sum over s <= t of a_ts v_s,     a_ts = sum_i q_t[i] k_s[i] exp(L_t[i] - L_s[i])
//     S   = diag(exp(L)) S0 + sum_s (k_s * exp(L - L_s)) v_s^T
// Every exponent is a difference that is <= 0: nothing overflows however strong a decay is. The same multiply-adds as
// token by token (plus the a_ts, a sixteenth more), but as small matrix products whose rows do not wait for one another:
// `prepare` makes q * exp(L_t), k * exp(L - L_s), exp(L) and the a_ts for all chunks of all segments at once (nothing
// there depends on the state), and `chunk` walks a segment's chunks in order, a block per (segment, head, 32 columns of
// S) as in the kernel above. All of it float32; against the token-by-token kernel only the grouping of sums differs.
constexpr int CHUNK = 16;

template <typename T>
__global__ void __launch_bounds__(128)
gla_chunk_prepare_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, float* __restrict__ logd,
                         const int* __restrict__ seg_start, const int* __restrict__ seg_len, float* __restrict__ qb,
                         float* __restrict__ ke, float* __restrict__ scores, int heads, int dk, float q_scale) {
    extern __shared__ __align__(16) float smem[];
    const int dkp = dk + 1;                 // rows one float apart in the banks: threads of a warp read one column of many rows
    float* L = smem;                        // [CHUNK][dkp]
    float* Q = L + CHUNK * dkp;
    float* K = Q + CHUNK * dkp;
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x, t0 = blockIdx.y * CHUNK, h = blockIdx.z, n = seg_len[seg];
    if (t0 >= n) return;
    const int nt = min(CHUNK, n - t0);
    const size_t row0 = (size_t)seg_start[seg] + t0, hd = (size_t)heads * dk;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
        float run = 0.f;
        for (int t = 0; t < nt; ++t) {
            run += logd[(row0 + t) * hd + (size_t)h * dk + i];
            L[t * dkp + i] = run;
            const T* p = proj + (row0 + t) * ld + (size_t)h * dk + i;
            Q[t * dkp + i] = __fmul_rn(to_float(p[q_off]), q_scale);
            K[t * dkp + i] = to_float(p[k_off]);
        }
        for (int t = 0; t < nt; ++t) {
            qb[(row0 + t) * hd + (size_t)h * dk + i] = __fmul_rn(Q[t * dkp + i], expf(L[t * dkp + i]));
            ke[(row0 + t) * hd + (size_t)h * dk + i] = __fmul_rn(K[t * dkp + i], expf(run - L[t * dkp + i]));
        }
        logd[row0 * hd + (size_t)h * dk + i] = expf(run);      // the chunk's whole decay, at its first row
    }
    __syncthreads();
    for (int p = threadIdx.x; p < CHUNK * CHUNK; p += blockDim.x) {
        const int t = p / CHUNK, sx = p - t * CHUNK;
        if (t >= nt) continue;
        float acc = 0.f;
        if (sx <= t)
            for (int i = 0; i < dk; ++i)
                acc = fmaf(__fmul_rn(Q[t * dkp + i], K[sx * dkp + i]), expf(L[t * dkp + i] - L[sx * dkp + i]), acc);
        scores[((row0 + t) * heads + h) * CHUNK + sx] = acc;
    }
}

template <typename T, int R, bool V4>
__global__ void __launch_bounds__(512)
gla_chunk_kernel(const T* __restrict__ proj, int ld, int v_off, const float* __restrict__ chunk_decay,
                 const float* __restrict__ qb, const float* __restrict__ ke, const float* __restrict__ scores,
                 float* __restrict__ state, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                 const int* __restrict__ state_slots, float* __restrict__ o, int heads, int dk, int dv, int num_slots) {
    extern __shared__ __align__(16) float smem[];
    const int threads = blockDim.x, G = threads >> 5;
    const int stage = 2 * CHUNK * dk + CHUNK * 32 + CHUNK * CHUNK + dk;     // qb, ke [CHUNK][dk], v [CHUNK][32], a, decay [dk]
    float* part = smem + 2 * stage;                                         // [CHUNK][G][32]
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
    const int tid = threadIdx.x, c = tid & 31, g = tid >> 5, j = c0 + c;
    const int first = seg_start[seg], n = seg_len[seg], slot = state_slots[seg];
    if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    float* S = state + (((size_t)slot * heads + h) * dk) * dv;
    const size_t hd = (size_t)heads * dk;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        s[r] = (i < dk && j < dv) ? S[(size_t)i * dv + j] : 0.f;
    }
    constexpr int EPT = CHUNK * R / 32;         // values of qb (and of ke) a thread fetches per chunk: CHUNK x dk / threads
    float fq[EPT], fk[EPT], fv, fa, fd;
    const int vt = tid >> 5, vpt_ok = tid < CHUNK * 32;      // (threads >= 32 x ... : v has CHUNK x 32 values)
    auto fetch = [&](int t0) {
        const int nt = min(CHUNK, n - t0);
        const size_t base = (size_t)(first + t0);
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            const int e = tid + u * threads, t = e / dk, i = e - t * dk;
            fq[u] = fk[u] = 0.f;
            if (e < CHUNK * dk && t < nt) {
                fq[u] = qb[(base + t) * hd + (size_t)h * dk + i];
                fk[u] = ke[(base + t) * hd + (size_t)h * dk + i];
            }
        }
        fv = fa = 0.f;
        fd = 1.f;
        // v: one value a thread where the block has CHUNK x 32 threads or more, else several rounds (below)
        if (vpt_ok && vt < nt && j < dv && threads >= CHUNK * 32)
            fv = to_float(proj[(base + vt) * ld + v_off + (size_t)h * dv + j]);
        if (tid < CHUNK * CHUNK && threads >= CHUNK * CHUNK) {
            const int t = tid / CHUNK;
            if (t < nt) fa = scores[((base + t) * heads + h) * CHUNK + (tid - t * CHUNK)];
        }
        if (tid < dk) fd = chunk_decay[base * hd + (size_t)h * dk + tid];
    };
    auto park = [&](int b, int t0) {
        float* qs = smem + b * stage;
        float* ks = qs + CHUNK * dk;
        float* vs = ks + CHUNK * dk;
        float* as = vs + CHUNK * 32;
        float* dsm = as + CHUNK * CHUNK;
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            const int e = tid + u * threads;
            if (e < CHUNK * dk) {
                qs[e] = fq[u];
                ks[e] = fk[u];
            }
        }
        if (threads >= CHUNK * 32) {
            if (vpt_ok) vs[tid] = fv;
        } else {        // a small block: it reads its values of v here, late (they are few)
            const int nt = min(CHUNK, n - t0);
            for (int e = tid; e < CHUNK * 32; e += threads) {
                const int t = e >> 5, cc = e & 31;
                vs[e] = (t < nt && c0 + cc < dv) ? to_float(proj[(size_t)(first + t0 + t) * ld + v_off + (size_t)h * dv + c0 + cc]) : 0.f;
            }
        }
        if (threads >= CHUNK * CHUNK) {
            if (tid < CHUNK * CHUNK) as[tid] = fa;
        } else {
            const int nt = min(CHUNK, n - t0);
            for (int e = tid; e < CHUNK * CHUNK; e += threads) {
                const int t = e / CHUNK;
                as[e] = t < nt ? scores[(((size_t)(first + t0 + t)) * heads + h) * CHUNK + (e - t * CHUNK)] : 0.f;
            }
        }
        for (int i = tid; i < dk; i += threads)
            dsm[i] = i == tid ? fd : chunk_decay[(size_t)(first + t0) * hd + (size_t)h * dk + i];
    };
    if (n > 0) {
        fetch(0);
        park(0, 0);
    }
    __syncthreads();
    for (int t0 = 0, b = 0; t0 < n; t0 += CHUNK, b ^= 1) {
        const int nt = min(CHUNK, n - t0);
        const bool more = t0 + CHUNK < n;
        if (more) fetch(t0 + CHUNK);
        const float* qs = smem + b * stage;
        const float* ks = qs + CHUNK * dk;
        const float* vs = ks + CHUNK * dk;
        const float* as = vs + CHUNK * 32;
        const float* dsm = as + CHUNK * CHUNK;
        // what the state at the chunk's start gives every token, and the state at its end
        float acc[CHUNK];
#pragma unroll
        for (int t = 0; t < CHUNK; ++t) acc[t] = 0.f;
        float vreg[CHUNK];
#pragma unroll
        for (int t = 0; t < CHUNK; ++t) vreg[t] = vs[t * 32 + c];
        if constexpr (V4) {     // dk a multiple of 4: four rows' values in one load (shared-memory instructions are what
                                // bounds this loop: an SM issues one a clock)
#pragma unroll
            for (int r = 0; r < R; r += 4) {
                const int i = g * R + r;
                if (i < dk) {
                    const float4 d4 = *reinterpret_cast<const float4*>(dsm + i);
                    const float a0 = s[r], a1 = s[r + 1], a2 = s[r + 2], a3 = s[r + 3];
                    float n0 = __fmul_rn(d4.x, a0), n1 = __fmul_rn(d4.y, a1), n2 = __fmul_rn(d4.z, a2), n3 = __fmul_rn(d4.w, a3);
#pragma unroll
                    for (int t = 0; t < CHUNK; ++t) {
                        const float4 q4 = *reinterpret_cast<const float4*>(qs + t * dk + i);
                        const float4 k4 = *reinterpret_cast<const float4*>(ks + t * dk + i);
                        acc[t] = fmaf(q4.x, a0, acc[t]);
                        acc[t] = fmaf(q4.y, a1, acc[t]);
                        acc[t] = fmaf(q4.z, a2, acc[t]);
                        acc[t] = fmaf(q4.w, a3, acc[t]);
                        n0 = fmaf(k4.x, vreg[t], n0);
                        n1 = fmaf(k4.y, vreg[t], n1);
                        n2 = fmaf(k4.z, vreg[t], n2);
                        n3 = fmaf(k4.w, vreg[t], n3);
                    }
                    s[r] = n0;
                    s[r + 1] = n1;
                    s[r + 2] = n2;
                    s[r + 3] = n3;
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = g * R + r;
                if (i < dk) {
                    const float s0 = s[r];
                    float sn = __fmul_rn(dsm[i], s0);
#pragma unroll
                    for (int t = 0; t < CHUNK; ++t) {
                        acc[t] = fmaf(qs[t * dk + i], s0, acc[t]);
                        sn = fmaf(ks[t * dk + i], vreg[t], sn);
                    }
                    s[r] = sn;
                }
            }
        }
#pragma unroll
        for (int t = 0; t < CHUNK; ++t) part[(t * G + g) * 32 + c] = acc[t];
        if (more) park(b ^ 1, t0 + CHUNK);
        __syncthreads();
        for (int e = tid; e < nt * 32; e += threads) {
            const int t = e >> 5, cc = e & 31;
            if (c0 + cc >= dv) continue;
            // four running sums each way: one chain of dependent additions would be all latency (the order is fixed)
            float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
            int gg = 0;
            for (; gg + 4 <= G; gg += 4) {
                p0 += part[(t * G + gg) * 32 + cc];
                p1 += part[(t * G + gg + 1) * 32 + cc];
                p2 += part[(t * G + gg + 2) * 32 + cc];
                p3 += part[(t * G + gg + 3) * 32 + cc];
            }
            for (; gg < G; ++gg) p0 += part[(t * G + gg) * 32 + cc];
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            int sx = 0;
            for (; sx + 4 <= t + 1; sx += 4) {
                a0 = fmaf(as[t * CHUNK + sx], vs[sx * 32 + cc], a0);
                a1 = fmaf(as[t * CHUNK + sx + 1], vs[(sx + 1) * 32 + cc], a1);
                a2 = fmaf(as[t * CHUNK + sx + 2], vs[(sx + 2) * 32 + cc], a2);
                a3 = fmaf(as[t * CHUNK + sx + 3], vs[(sx + 3) * 32 + cc], a3);
            }
            for (; sx <= t; ++sx) a0 = fmaf(as[t * CHUNK + sx], vs[sx * 32 + cc], a0);
            o[(size_t)(first + t0 + t) * ((size_t)heads * dv) + (size_t)h * dv + c0 + cc] =
                ((p0 + p1) + (p2 + p3)) + ((a0 + a1) + (a2 + a3));
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        if (i < dk && j < dv) S[(size_t)i * dv + j] = s[r];
    }
}

template <typename T, int R, bool V4>
int launch_chunked(const void* proj, int ld, int v_off, const float* chunk_decay, const float* qb, const float* ke,
                   const float* scores, float* state, const int* seg_start, const int* seg_len, const int* state_slots,
                   float* o, int segments, int heads, int dk, int dv, int num_slots, cudaStream_t stream) {
    const int G = (dk + R - 1) / R;
    const size_t smem = (size_t)(2 * (2 * CHUNK * dk + CHUNK * 32 + CHUNK * CHUNK + dk) + CHUNK * G * 32) * sizeof(float);
    auto kernel = gla_chunk_kernel<T, R, V4>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return jllm_fail(JLLM_CUDA_ERROR, "gla_chunk: %zu bytes of shared memory refused", smem);
    jllm_launch(kernel, dim3(segments, heads, (dv + 31) / 32), dim3(G * 32), smem, stream, LAUNCH_DEPENDENT, (const T*)proj, ld,
                v_off, chunk_decay, qb, ke, scores, state, seg_start, seg_len, state_slots, o, heads, dk, dv, num_slots);
    return jllm_check_launch("gla_chunk");
}

// y[r, h, :] = o[r, h, :] / sqrt(mean(o[r, h, :]^2) + eps) * gain * act(gate[r, h, :]) * scale, act = silu or (gate_kind bit 0)
// sigmoid; one warp per (row, head). A norm over all heads together is the case heads = 1. Bit 1 of gate_kind: the gate
// comes first, y = rms(o * act(gate)) * gain * scale (the statistics are those of the gated values). Bit 2: the gain has a
// value per column of the whole row (heads x dv) and not one per column of a head.
template <typename T, typename TG = T>
__global__ void __launch_bounds__(256)
gated_head_norm_kernel(const float* __restrict__ o, const TG* __restrict__ gate, int ld_gate, VecRef gain, T* __restrict__ y,
                       int rows, int heads, int dv, float eps, float scale, int gate_kind) {
    pdl_wait();
    pdl_trigger();
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= rows * heads) return;
    const int r = w / heads, h = w - r * heads;
    const float* src = o + ((size_t)r * heads + h) * dv;
    const TG* gp = gate + (size_t)r * ld_gate + (size_t)h * dv;
    const bool logistic = gate_kind & 1, gate_first = gate_kind & 2;
    const int g0 = (gate_kind & 4) ? h * dv : 0;
    auto gate_of = [&](int i) {
        const float gv = to_float(gp[i]);
        return (logistic ? 1.f : gv) / (1.f + expf(-gv));                          // silu, or (bit 0) the logistic function
    };
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) {
        const float v = gate_first ? __fmul_rn(src[i], gate_of(i)) : src[i];
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dv + eps);
    T* dst = y + ((size_t)r * heads + h) * dv;
    for (int i = lane; i < dv; i += 32) {
        const float gated = gate_of(i);
        if (gate_first)
            dst[i] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(src[i], gated), inv), gain[g0 + i]), scale));
        else
            dst[i] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(src[i], inv), gain[g0 + i]), gated), scale));
    }
}

// The same with a block per (row, head), for norms over many values (all heads of a row together: thousands): a warp
// alone would walk them one after the other.
template <typename T, typename TG = T>
__global__ void __launch_bounds__(256)
gated_row_norm_kernel(const float* __restrict__ o, const TG* __restrict__ gate, int ld_gate, VecRef gain, T* __restrict__ y,
                      int heads, int dv, float eps, float scale, int gate_kind) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x / heads, h = blockIdx.x - r * heads;
    const float* src = o + ((size_t)r * heads + h) * dv;
    const TG* gp = gate + (size_t)r * ld_gate + (size_t)h * dv;
    const bool logistic = gate_kind & 1, gate_first = gate_kind & 2;
    const int g0 = (gate_kind & 4) ? h * dv : 0;
    auto gate_of = [&](int i) {
        const float gv = to_float(gp[i]);
        return (logistic ? 1.f : gv) / (1.f + expf(-gv));
    };
    float ss = 0.f;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        const float v = gate_first ? __fmul_rn(src[i], gate_of(i)) : src[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)dv + eps);
    T* dst = y + ((size_t)r * heads + h) * dv;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        const float gated = gate_of(i);
        if (gate_first)
            dst[i] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(src[i], gated), inv), gain[g0 + i]), scale));
        else
            dst[i] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(src[i], inv), gain[g0 + i]), gated), scale));
    }
}


// ---- prompt portions of the fixed-decay form on the tensor cores (bfloat16 path) ---------------------------------------
// With ONE decay d per head the decay's powers are scalars per token, so a chunk of 64 tokens is four matrix products
// whose operands are the projections themselves (q, k, v: bfloat16 as the stacked product left them) and whose decay
// weights are applied in float32:
//     P[t, s] = (q_t . k_s) d^(t - s)  for s <= t, else 0                  scores from the tensor cores, float32; times the power
//     o_t     = sum_s P[t, s] v_s  +  d^(t + 1) (q_t^T S0)                  S0: the state in front of the chunk
//     S       = d^n S0 + sum_s (d^(n - 1 - s) k_s) v_s^T                    n: the chunk's tokens
// Everything float32 that becomes a tensor-core operand (P, the weighted keys, the state) is split into a bfloat16 value
// and the bfloat16 of what that rounding left over, and multiplied as two operands: 16 bits of mantissa instead of 8, the
// accumulation in float32. The state itself stays in float32 registers from the first chunk to the last (it is the
// accumulator of the last product) and is read from and written to its slot once per portion.
//
// A block owns DVB (64 or 32) value columns of one (segment, head): the state's columns do not depend on one another; the
// narrower blocks are taken when the wider ones would leave SMs without one (every block makes P for itself). Eight
// warps: warp w takes the 16 tokens (w & 3) of the chunk for P and o, with half (w >> 2) of the keys or of the block's
// value columns, and for the state 16 of the block's value columns with a half or a quarter of the key channels. Operands lie in shared
// memory with the contraction index contiguous (rows padded by 16 bytes: the eight 16-byte rows of an 8 x 8 matrix hit 32
// different banks), so every product is the same "row times row" tile loop fed by ldmatrix.
namespace lightning {

constexpr int C = 64;            // tokens of a chunk
constexpr int LDC = C + 8;       // row length of operands whose contraction runs over the chunk's tokens

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four 8 x 8 matrices of bfloat16 from shared memory into the fragments of a warp (lane l names the 16-byte row l & 7
// of matrix l >> 3)
__device__ __forceinline__ void ldmatrix4(uint32_t (&r)[4], const __nv_bfloat16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// the A fragment (16 rows from `row0`, 16 contraction values from `k0`) of a row-major operand
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const __nv_bfloat16* m, int ld, int row0, int k0, int lane) {
    ldmatrix4(a, m + (size_t)(row0 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + k0 + (lane >> 4) * 8);
}

// the B fragments of two neighbouring tiles (8 output columns each, from `n0`; 16 contraction values from `k0`) of an
// operand stored [columns][contraction]: b[0], b[1] for the first tile, b[2], b[3] for the second
__device__ __forceinline__ void load_b2(uint32_t (&b)[4], const __nv_bfloat16* m, int ld, int n0, int k0, int lane) {
    ldmatrix4(b, m + (size_t)(n0 + (lane & 7) + (lane >> 4) * 8) * ld + k0 + ((lane >> 3) & 1) * 8);
}

// v = hi + lo with hi = bfloat16(v), lo = bfloat16(v - hi)
__device__ __forceinline__ void split(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

__device__ __forceinline__ void store_split2(__nv_bfloat16* hi, __nv_bfloat16* lo, float a, float b) {
    __nv_bfloat16 ah, al, bh, bl;
    split(a, ah, al);
    split(b, bh, bl);
    __nv_bfloat162 h2, l2;
    h2.x = ah; h2.y = bh; l2.x = al; l2.y = bl;
    *reinterpret_cast<__nv_bfloat162*>(hi) = h2;
    *reinterpret_cast<__nv_bfloat162*>(lo) = l2;
}

template <int DK, int DVB>
__global__ void __launch_bounds__(256)
chunk_kernel(const __nv_bfloat16* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
             const float* __restrict__ head_decay, float* __restrict__ state, const int* __restrict__ seg_start,
             const int* __restrict__ seg_len, const int* __restrict__ state_slots, float* __restrict__ o, int heads, int dv,
             int num_slots, float q_scale) {
    constexpr int LDQ = DK + 8;          // row length of operands whose contraction runs over the key channels
    constexpr int OT = DVB / 16;         // 8-wide tiles of the value columns a warp takes for o (half of the block's)
    constexpr int ST = DVB / 16;         // 16-wide tiles of the block's value columns (rows of the transposed state)
    constexpr int SPARTS = 8 / ST;       // warps that share such a tile, each with a part of the key channels
    constexpr int NS = DK / SPARTS / 8;  // 8-wide tiles of a warp's part of the key channels
    extern __shared__ __align__(16) unsigned char lightning_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lightning_smem);   // [C][LDQ]     q
    __nv_bfloat16* Ks = Qs + C * LDQ;                                       // [C][LDQ]     k
    __nv_bfloat16* Vt = Ks + C * LDQ;                                       // [DVB][LDC]   v, transposed
    __nv_bfloat16* Kh = Vt + DVB * LDC;                                     // [DK][LDC]    weighted k, transposed: value
    __nv_bfloat16* Kl = Kh + DK * LDC;                                      //              ... and what its rounding left
    __nv_bfloat16* Ph = Kl + DK * LDC;                                      // [C][LDC]     P
    __nv_bfloat16* Pl = Ph + C * LDC;
    __nv_bfloat16* Sh = Pl + C * LDC;                                       // [DVB][LDQ]   the state, transposed
    __nv_bfloat16* Sl = Sh + DVB * LDQ;
    float* pw = reinterpret_cast<float*>(Sl + DVB * LDQ);                   // [C + 1]      d^0 .. d^C
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DVB;
    const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int mt = w & 3, half = w >> 2, smt = w % ST, spart = w / ST;
    const int first = seg_start[seg], n = seg_len[seg], slot = state_slots[seg];
    if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    float* S = state + (((size_t)slot * heads + h) * DK) * dv;
    if (tid <= C) {
        const float d = head_decay[h];
        pw[tid] = expf((float)tid * fmaxf(logf(d), -1e30f));      // (a decay of 0: d^0 = 1, every other power 0)
    }
    // the state, transposed: this thread's values are (value column c0 + smt * 16 + g [+ 8], key channel spart * DK / SPARTS + j * 8 + 2 t [+ 1])
    float sacc[NS][4];
    const int vrow = smt * 16 + g, kcol0 = spart * (DK / SPARTS) + 2 * t;
#pragma unroll
    for (int j = 0; j < NS; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = c0 + vrow + (e >> 1) * 8, ch = kcol0 + j * 8 + (e & 1);
            sacc[j][e] = col < dv ? S[(size_t)ch * dv + col] : 0.f;
        }
    auto park_state = [&]() {
#pragma unroll
        for (int j = 0; j < NS; ++j) {
            const int ch = kcol0 + j * 8;
            store_split2(Sh + (size_t)vrow * LDQ + ch, Sl + (size_t)vrow * LDQ + ch, sacc[j][0], sacc[j][1]);
            store_split2(Sh + (size_t)(vrow + 8) * LDQ + ch, Sl + (size_t)(vrow + 8) * LDQ + ch, sacc[j][2], sacc[j][3]);
        }
    };
    park_state();
    const size_t row_o = (size_t)heads * dv;
    // a chunk's q, k (16-byte pieces; neighbouring lanes take neighbouring tokens, so that the transposed stores fall into
    // different banks) and v in registers: requested a chunk ahead
    constexpr int QI = C * (DK / 8) / 256, VI = C * (DVB / 8) / 256;
    uint4 fq[QI], fk[QI], fv[VI];
    auto fetch = [&](int t0) {
        const int nt = min(C, n - t0);
#pragma unroll
        for (int u = 0; u < QI; ++u) {
            const int e = tid + u * 256, piece = e / C, srow = e - piece * C;
            fq[u] = fk[u] = make_uint4(0, 0, 0, 0);
            if (srow < nt) {
                const __nv_bfloat16* base = proj + (size_t)(first + t0 + srow) * ld + (size_t)h * DK + piece * 8;
                fq[u] = *reinterpret_cast<const uint4*>(base + q_off);
                fk[u] = *reinterpret_cast<const uint4*>(base + k_off);
            }
        }
#pragma unroll
        for (int u = 0; u < VI; ++u) {
            const int e = tid + u * 256, piece = e / C, srow = e - piece * C;
            fv[u] = make_uint4(0, 0, 0, 0);
            if (srow < nt && c0 + piece * 8 < dv)
                fv[u] = *reinterpret_cast<const uint4*>(proj + (size_t)(first + t0 + srow) * ld + v_off + (size_t)h * dv + c0 + piece * 8);
        }
    };
    if (n > 0) fetch(0);
    for (int t0 = 0; t0 < n; t0 += C) {
        const int nt = min(C, n - t0);
        __syncthreads();       // pw and the parked state are written; the tiles of the chunk before are no longer read
        // ---- the chunk's q, k, v, fetched while the chunk before was worked on, go into shared memory (the weighted k
        //      and v transposed on their way); then the next chunk's are requested ----
#pragma unroll
        for (int u = 0; u < QI; ++u) {
            const int e = tid + u * 256, piece = e / C, srow = e - piece * C;
            *reinterpret_cast<uint4*>(Qs + (size_t)srow * LDQ + piece * 8) = fq[u];
            *reinterpret_cast<uint4*>(Ks + (size_t)srow * LDQ + piece * 8) = fk[u];
            const float wgt = srow < nt ? pw[nt - 1 - srow] : 0.f;
            const __nv_bfloat16* kv = reinterpret_cast<const __nv_bfloat16*>(&fk[u]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                __nv_bfloat16 hi, lo;
                split(__bfloat162float(kv[i]) * wgt, hi, lo);
                Kh[(size_t)(piece * 8 + i) * LDC + srow] = hi;
                Kl[(size_t)(piece * 8 + i) * LDC + srow] = lo;
            }
        }
#pragma unroll
        for (int u = 0; u < VI; ++u) {
            const int e = tid + u * 256, piece = e / C, srow = e - piece * C;
            const __nv_bfloat16* vv = reinterpret_cast<const __nv_bfloat16*>(&fv[u]);
#pragma unroll
            for (int i = 0; i < 8; ++i) Vt[(size_t)(piece * 8 + i) * LDC + srow] = vv[i];
        }
        if (t0 + C < n) fetch(t0 + C);
        __syncthreads();
        // ---- P = q k^T for this warp's 16 tokens and 32 keys, times the decay's powers; parked as two operands ----
        float acc[4][4] = {};
        float o2[OT][4] = {};
        for (int k0 = 0; k0 < DK; k0 += 16) {
            uint32_t a[4];
            load_a(a, Qs, LDQ, mt * 16, k0, lane);
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                uint32_t b[4];
                load_b2(b, Ks, LDQ, half * 32 + j * 8, k0, lane);
                mma_bf16(acc[j], a, b[0], b[1]);
                mma_bf16(acc[j + 1], a, b[2], b[3]);
            }
            // ... and q^T S0 for this warp's 16 tokens and its half of the block's value columns (the state as two operands)
#pragma unroll
            for (int j = 0; j < OT; j += 2) {
                uint32_t b[4];
                load_b2(b, Sh, LDQ, half * (DVB / 2) + j * 8, k0, lane);
                mma_bf16(o2[j], a, b[0], b[1]);
                mma_bf16(o2[j + 1], a, b[2], b[3]);
                load_b2(b, Sl, LDQ, half * (DVB / 2) + j * 8, k0, lane);
                mma_bf16(o2[j], a, b[0], b[1]);
                mma_bf16(o2[j + 1], a, b[2], b[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int key = half * 32 + j * 8 + 2 * t;
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int tok = mt * 16 + g + hrow * 8;
                const float p0 = key <= tok ? __fmul_rn(__fmul_rn(acc[j][2 * hrow], q_scale), pw[tok - key]) : 0.f;
                const float p1 = key + 1 <= tok ? __fmul_rn(__fmul_rn(acc[j][2 * hrow + 1], q_scale), pw[tok - key - 1]) : 0.f;
                store_split2(Ph + (size_t)tok * LDC + key, Pl + (size_t)tok * LDC + key, p0, p1);
            }
        }
        __syncthreads();
        // ---- o = P v + d^(t + 1) q^T S0 ----
        float o1[OT][4] = {};
        for (int k0 = 0; k0 < C; k0 += 16) {
            uint32_t ah[4], al[4];
            load_a(ah, Ph, LDC, mt * 16, k0, lane);
            load_a(al, Pl, LDC, mt * 16, k0, lane);
#pragma unroll
            for (int j = 0; j < OT; j += 2) {
                uint32_t b[4];
                load_b2(b, Vt, LDC, half * (DVB / 2) + j * 8, k0, lane);
                mma_bf16(o1[j], ah, b[0], b[1]);
                mma_bf16(o1[j], al, b[0], b[1]);
                mma_bf16(o1[j + 1], ah, b[2], b[3]);
                mma_bf16(o1[j + 1], al, b[2], b[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < OT; ++j) {
            const int col = c0 + half * (DVB / 2) + j * 8 + 2 * t;
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int tok = mt * 16 + g + hrow * 8;
                if (tok < nt && col < dv) {
                    const float f = __fmul_rn(pw[tok + 1], q_scale);
                    float* dst = o + (size_t)(first + t0 + tok) * row_o + (size_t)h * dv + col;
                    dst[0] = __fadd_rn(o1[j][2 * hrow], __fmul_rn(f, o2[j][2 * hrow]));
                    if (col + 1 < dv) dst[1] = __fadd_rn(o1[j][2 * hrow + 1], __fmul_rn(f, o2[j][2 * hrow + 1]));
                }
            }
        }
        // ---- S = d^n S0 + v^T (weighted k): this warp's 16 value columns and its part of the key channels ----
        const float dn = pw[nt];
#pragma unroll
        for (int j = 0; j < NS; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[j][e] = __fmul_rn(sacc[j][e], dn);
        for (int k0 = 0; k0 < C; k0 += 16) {
            uint32_t a[4];
            load_a(a, Vt, LDC, smt * 16, k0, lane);
#pragma unroll
            for (int j = 0; j < NS; j += 2) {
                uint32_t b[4];
                load_b2(b, Kh, LDC, spart * (DK / SPARTS) + j * 8, k0, lane);
                mma_bf16(sacc[j], a, b[0], b[1]);
                mma_bf16(sacc[j + 1], a, b[2], b[3]);
                load_b2(b, Kl, LDC, spart * (DK / SPARTS) + j * 8, k0, lane);
                mma_bf16(sacc[j], a, b[0], b[1]);
                mma_bf16(sacc[j + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();       // everyone has read the parked state of the chunk before
        park_state();
    }
#pragma unroll
    for (int j = 0; j < NS; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = c0 + vrow + (e >> 1) * 8, ch = kcol0 + j * 8 + (e & 1);
            if (col < dv) S[(size_t)ch * dv + col] = sacc[j][e];
        }
}

// ---- the same chunks with a decay and an input scale per TOKEN (and head) ------------------------------------------------
// S_t = a_t S_(t-1) + (b_t k_t) v_t^T, o_t = S_t^T (s q_t) [+ D v_t]: with cl_t the sum of log a over the chunk's tokens up to
// t, a chunk is the same four products:
//     P[t, s] = (q_t . k_s) s exp(cl_t - cl_s) b_s  for s <= t       o_t = sum_s P[t, s] v_s + exp(cl_t) s (q_t^T S0) [+ D v_t]
//     S       = exp(cl_n) S0 + sum_s (b_s exp(cl_n - cl_s) k_s) v_s^T
// Every exponent is a difference that is <= 0. The float32 factors meet float32 values (the scores behind their product, the
// keys in front of theirs, the state in its registers) and become tensor-core operands as two bfloat16 values each, as above.
// q and k may be shared by the heads of a group; the sources may be float32 (rounded to bfloat16 on their way into shared
// memory: they are projections, the operands the products take) or bfloat16.
__device__ __forceinline__ uint4 load8(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 load8(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    __nv_bfloat162 r0 = __floats2bfloat162_rn(a.x, a.y), r1 = __floats2bfloat162_rn(a.z, a.w);
    __nv_bfloat162 r2 = __floats2bfloat162_rn(b.x, b.y), r3 = __floats2bfloat162_rn(b.z, b.w);
    uint4 out;
    out.x = *reinterpret_cast<uint32_t*>(&r0);
    out.y = *reinterpret_cast<uint32_t*>(&r1);
    out.z = *reinterpret_cast<uint32_t*>(&r2);
    out.w = *reinterpret_cast<uint32_t*>(&r3);
    return out;
}

template <typename TS, int DK, int DVB>
__global__ void __launch_bounds__(256)
gated_chunk_kernel(const TS* __restrict__ qp, int ld_q, int q_off, int q_groups, const TS* __restrict__ kp, int ld_k, int k_off,
                   int k_groups, const TS* __restrict__ vp, int ld_v, int v_off, const float* __restrict__ la,
                   const float* __restrict__ bsc, VecRef skip, int has_skip, float* __restrict__ state,
                   const int* __restrict__ seg_start, const int* __restrict__ seg_len, const int* __restrict__ state_slots,
                   float* __restrict__ o, int heads, int dv, int num_slots, float q_scale) {
    constexpr int LDQ = DK + 8;
    constexpr int OT = DVB / 16;
    constexpr int ST = DVB / 16;
    constexpr int SPARTS = 8 / ST;
    constexpr int NS = DK / SPARTS / 8;
    extern __shared__ __align__(16) unsigned char lightning_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lightning_smem);   // [C][LDQ]     q
    __nv_bfloat16* Ks = Qs + C * LDQ;                                       // [C][LDQ]     k
    __nv_bfloat16* Vt = Ks + C * LDQ;                                       // [DVB][LDC]   v, transposed
    __nv_bfloat16* Kh = Vt + DVB * LDC;                                     // [DK][LDC]    weighted k, transposed: value
    __nv_bfloat16* Kl = Kh + DK * LDC;                                      //              ... and what its rounding left
    __nv_bfloat16* Ph = Kl + DK * LDC;                                      // [C][LDC]     P
    __nv_bfloat16* Pl = Ph + C * LDC;
    __nv_bfloat16* Sh = Pl + C * LDC;                                       // [DVB][LDQ]   the state, transposed
    __nv_bfloat16* Sl = Sh + DVB * LDQ;
    float* cl = reinterpret_cast<float*>(Sl + DVB * LDQ);                   // [C]  the chunk's log decays, summed up to each token
    float* bs = cl + C;                                                     // [C]  its input scales (0 past the chunk's end)
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DVB;
    const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int mt = w & 3, half = w >> 2, smt = w % ST, spart = w / ST;
    const int first = seg_start[seg], n = seg_len[seg], slot = state_slots[seg];
    if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    const int qg = h / (heads / q_groups), kg = h / (heads / k_groups);
    float* S = state + (((size_t)slot * heads + h) * DK) * dv;
    const float d_skip = has_skip ? skip[h] : 0.f;
    float sacc[NS][4];
    const int vrow = smt * 16 + g, kcol0 = spart * (DK / SPARTS) + 2 * t;
#pragma unroll
    for (int j = 0; j < NS; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = c0 + vrow + (e >> 1) * 8, ch = kcol0 + j * 8 + (e & 1);
            sacc[j][e] = col < dv ? S[(size_t)ch * dv + col] : 0.f;
        }
    auto park_state = [&]() {
#pragma unroll
        for (int j = 0; j < NS; ++j) {
            const int ch = kcol0 + j * 8;
            store_split2(Sh + (size_t)vrow * LDQ + ch, Sl + (size_t)vrow * LDQ + ch, sacc[j][0], sacc[j][1]);
            store_split2(Sh + (size_t)(vrow + 8) * LDQ + ch, Sl + (size_t)(vrow + 8) * LDQ + ch, sacc[j][2], sacc[j][3]);
        }
    };
    park_state();
    const size_t row_o = (size_t)heads * dv;
    constexpr int QI = C * (DK / 8) / 256, VI = C * (DVB / 8) / 256;
    uint4 fq[QI], fk[QI], fv[VI];
    float fla = 0.f, fb = 0.f;              // this thread's token's gates (threads below C), a chunk ahead like q, k and v
    auto fetch = [&](int t0) {
        const int nt = min(C, n - t0);
#pragma unroll
        for (int u = 0; u < QI; ++u) {
            const int e = tid + u * 256, piece = e / C, srow = e - piece * C;
            fq[u] = fk[u] = make_uint4(0, 0, 0, 0);
            if (srow < nt) {
                const size_t r = (size_t)(first + t0 + srow);
                fq[u] = load8(qp + r * ld_q + q_off + (size_t)qg * DK + piece * 8);
                fk[u] = load8(kp + r * ld_k + k_off + (size_t)kg * DK + piece * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < VI; ++u) {
            const int e = tid + u * 256, piece = e / C, srow = e - piece * C;
            fv[u] = make_uint4(0, 0, 0, 0);
            if (srow < nt && c0 + piece * 8 < dv)
                fv[u] = load8(vp + (size_t)(first + t0 + srow) * ld_v + v_off + (size_t)h * dv + c0 + piece * 8);
        }
        if (tid < C) {
            fla = 0.f;
            fb = 0.f;
            if (tid < nt) {
                fla = la[(size_t)(first + t0 + tid) * heads + h];
                fb = bsc[(size_t)(first + t0 + tid) * heads + h];
            }
        }
    };
    if (n > 0) fetch(0);
    for (int t0 = 0; t0 < n; t0 += C) {
        const int nt = min(C, n - t0);
        __syncthreads();       // the parked state is written; the tiles and gates of the chunk before are no longer read
        // ---- the chunk's gates: log decays summed up to each token (two warps scan 32 tokens each, the second adds the
        //      first's total), input scales ----
        if (tid < C) {
            float v = fla;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, v, d);
                if (lane >= d) v += up;
            }
            cl[tid] = v;
            bs[tid] = fb;
        }
        __syncthreads();
        if (tid >= 32 && tid < C) cl[tid] += cl[31];
        __syncthreads();
        const float cl_end = cl[nt - 1];
#pragma unroll
        for (int u = 0; u < QI; ++u) {
            const int e = tid + u * 256, piece = e / C, srow = e - piece * C;
            *reinterpret_cast<uint4*>(Qs + (size_t)srow * LDQ + piece * 8) = fq[u];
            *reinterpret_cast<uint4*>(Ks + (size_t)srow * LDQ + piece * 8) = fk[u];
            const float wgt = srow < nt ? __fmul_rn(bs[srow], expf(cl_end - cl[srow])) : 0.f;
            const __nv_bfloat16* kv = reinterpret_cast<const __nv_bfloat16*>(&fk[u]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                __nv_bfloat16 hi, lo;
                split(__bfloat162float(kv[i]) * wgt, hi, lo);
                Kh[(size_t)(piece * 8 + i) * LDC + srow] = hi;
                Kl[(size_t)(piece * 8 + i) * LDC + srow] = lo;
            }
        }
#pragma unroll
        for (int u = 0; u < VI; ++u) {
            const int e = tid + u * 256, piece = e / C, srow = e - piece * C;
            const __nv_bfloat16* vv = reinterpret_cast<const __nv_bfloat16*>(&fv[u]);
#pragma unroll
            for (int i = 0; i < 8; ++i) Vt[(size_t)(piece * 8 + i) * LDC + srow] = vv[i];
        }
        if (t0 + C < n) fetch(t0 + C);
        __syncthreads();
        // ---- P = q k^T for this warp's 16 tokens and 32 keys, times the decays between key and token and the key's scale ----
        float acc[4][4] = {};
        float o2[OT][4] = {};
        for (int k0 = 0; k0 < DK; k0 += 16) {
            uint32_t a[4];
            load_a(a, Qs, LDQ, mt * 16, k0, lane);
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                uint32_t b[4];
                load_b2(b, Ks, LDQ, half * 32 + j * 8, k0, lane);
                mma_bf16(acc[j], a, b[0], b[1]);
                mma_bf16(acc[j + 1], a, b[2], b[3]);
            }
#pragma unroll
            for (int j = 0; j < OT; j += 2) {
                uint32_t b[4];
                load_b2(b, Sh, LDQ, half * (DVB / 2) + j * 8, k0, lane);
                mma_bf16(o2[j], a, b[0], b[1]);
                mma_bf16(o2[j + 1], a, b[2], b[3]);
                load_b2(b, Sl, LDQ, half * (DVB / 2) + j * 8, k0, lane);
                mma_bf16(o2[j], a, b[0], b[1]);
                mma_bf16(o2[j + 1], a, b[2], b[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int key = half * 32 + j * 8 + 2 * t;
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int tok = mt * 16 + g + hrow * 8;
                const float ct = cl[tok];
                const float p0 = key <= tok ? __fmul_rn(__fmul_rn(acc[j][2 * hrow], q_scale), __fmul_rn(expf(ct - cl[key]), bs[key])) : 0.f;
                const float p1 = key + 1 <= tok
                                     ? __fmul_rn(__fmul_rn(acc[j][2 * hrow + 1], q_scale), __fmul_rn(expf(ct - cl[key + 1]), bs[key + 1])) : 0.f;
                store_split2(Ph + (size_t)tok * LDC + key, Pl + (size_t)tok * LDC + key, p0, p1);
            }
        }
        __syncthreads();
        // ---- o = P v + exp(cl_t) s q^T S0 [+ D v] ----
        float o1[OT][4] = {};
        for (int k0 = 0; k0 < C; k0 += 16) {
            uint32_t ah[4], al[4];
            load_a(ah, Ph, LDC, mt * 16, k0, lane);
            load_a(al, Pl, LDC, mt * 16, k0, lane);
#pragma unroll
            for (int j = 0; j < OT; j += 2) {
                uint32_t b[4];
                load_b2(b, Vt, LDC, half * (DVB / 2) + j * 8, k0, lane);
                mma_bf16(o1[j], ah, b[0], b[1]);
                mma_bf16(o1[j], al, b[0], b[1]);
                mma_bf16(o1[j + 1], ah, b[2], b[3]);
                mma_bf16(o1[j + 1], al, b[2], b[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < OT; ++j) {
            const int lcol = half * (DVB / 2) + j * 8 + 2 * t, col = c0 + lcol;
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int tok = mt * 16 + g + hrow * 8;
                if (tok < nt && col < dv) {
                    const float f = __fmul_rn(expf(cl[tok]), q_scale);
                    float* dst = o + (size_t)(first + t0 + tok) * row_o + (size_t)h * dv + col;
                    float r0 = __fadd_rn(o1[j][2 * hrow], __fmul_rn(f, o2[j][2 * hrow]));
                    float r1 = __fadd_rn(o1[j][2 * hrow + 1], __fmul_rn(f, o2[j][2 * hrow + 1]));
                    if (has_skip) {
                        r0 = fmaf(d_skip, __bfloat162float(Vt[(size_t)lcol * LDC + tok]), r0);
                        r1 = fmaf(d_skip, __bfloat162float(Vt[(size_t)(lcol + 1) * LDC + tok]), r1);
                    }
                    dst[0] = r0;
                    if (col + 1 < dv) dst[1] = r1;
                }
            }
        }
        // ---- S = exp(cl_n) S0 + v^T (weighted k) ----
        const float dn = expf(cl_end);
#pragma unroll
        for (int j = 0; j < NS; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[j][e] = __fmul_rn(sacc[j][e], dn);
        for (int k0 = 0; k0 < C; k0 += 16) {
            uint32_t a[4];
            load_a(a, Vt, LDC, smt * 16, k0, lane);
#pragma unroll
            for (int j = 0; j < NS; j += 2) {
                uint32_t b[4];
                load_b2(b, Kh, LDC, spart * (DK / SPARTS) + j * 8, k0, lane);
                mma_bf16(sacc[j], a, b[0], b[1]);
                mma_bf16(sacc[j + 1], a, b[2], b[3]);
                load_b2(b, Kl, LDC, spart * (DK / SPARTS) + j * 8, k0, lane);
                mma_bf16(sacc[j], a, b[0], b[1]);
                mma_bf16(sacc[j + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
        park_state();
    }
#pragma unroll
    for (int j = 0; j < NS; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = c0 + vrow + (e >> 1) * 8, ch = kcol0 + j * 8 + (e & 1);
            if (col < dv) S[(size_t)ch * dv + col] = sacc[j][e];
        }
}

template <int DK, int DVB>
constexpr size_t smem_bytes() {
    return (size_t)(2 * C * (DK + 8) + DVB * LDC + 2 * DK * LDC + 2 * C * LDC + 2 * DVB * (DK + 8)) * sizeof(__nv_bfloat16) +
           (C + 1) * sizeof(float);
}

// whether the tensor-core form takes this shape (JLLM_B200_LIGHTNING_TC=0 keeps every shape on the float32 kernels)
inline bool fits(int dtype, int ld, int q_off, int k_off, int v_off, int dk, int dv, const void* proj) {
    static const bool on = [] {
        const char* e = getenv("JLLM_B200_LIGHTNING_TC");
        return !(e && e[0] == '0');
    }();
    return on && dtype == JLLM_BF16 && (dk == 64 || dk == 128) && dv % 8 == 0 && ld % 8 == 0 && q_off % 8 == 0 &&
           k_off % 8 == 0 && v_off % 8 == 0 && ((uintptr_t)proj % 16) == 0;
}

}  // namespace lightning

}  // namespace

JLLM_BOUNDS_READER(linear_attention)

// A test's switch: the value columns a block of the tensor-core chunk kernel owns (32 or 64; 0: chosen from the shape).
static int g_lightning_width = 0;
JLLM_EXPORT int jllm_lightning_block_width(int width) {
    JLLM_REQUIRE(width == 0 || width == 32 || width == 64, "lightning_block_width: %d is not 0, 32 or 64", width);
    g_lightning_width = width;
    return JLLM_OK;
}

// proj [rows, ld]: q at column q_off (heads x dk), k at k_off, v at v_off (heads x dv); z [rows, heads x dk] float32:
// the decay logits, which this call turns into the decays in place; state [num_slots, heads, dk, dv] float32; o [rows,
// heads x dv] float32. Two launches.
JLLM_EXPORT int jllm_gla_recurrent(const void* proj, int dtype, int ld, int q_off, int k_off, int v_off, float* z, int rows,
                                   float* state, int num_slots, const int* seg_start, const int* seg_len,
                                   const int* state_slots, float* o, int segments, int heads, int dk, int dv, float q_scale,
                                   float tau, const float* head_decay, int activation, cudaStream_t stream) {
    JLLM_REQUIRE(segments >= 0 && rows >= 0 && heads > 0 && dk > 0 && dv > 0 && tau > 0.f,
                 "gla_recurrent: segments=%d heads=%d dk=%d dv=%d", segments, heads, dk, dv);
    JLLM_REQUIRE(dk <= 512 && heads <= 65535 && (dv + 7) / 8 <= 65535, "gla_recurrent: dk=%d is above 512", dk);
    if (segments == 0 || rows == 0) return JLLM_OK;
    const float inv_tau = 1.f / tau;
    if (head_decay) {
        // one fixed decay per head: the recurrence takes the decays themselves and activates q, k, v as it fetches them (no
        // table, no pass in front; `proj` is left as it is)
    } else {       // the decay logits become decays, in place
        const size_t total = (size_t)rows * heads * dk;
        const int blocks = (int)min((size_t)65535, (total + 255) / 256);
        jllm_launch(gla_decay_kernel, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, z, inv_tau, total, 0);
        const int code = jllm_check_launch("gla_decay");
        if (code) return code;
    }
#define JLLM_GLA(T, R)                                                                                                       \
    return launch_recurrent_cols<T, R>(proj, ld, q_off, k_off, v_off, z, state, seg_start, seg_len, state_slots, o, segments, \
                                       heads, dk, dv, q_scale, num_slots, head_decay, head_decay ? activation : 0, stream)
    // A step of single tokens is a chain of a few round trips to memory per block, whatever the block's size: many rows a
    // thread make blocks small enough for several to share an SM. A prompt portion waits more than it computes: few rows
    // a thread, so that more threads hide more of the waiting (at most 32 row groups of 32 columns: 1,024 threads).
    // (Only the grouping of the partial sums of o differs between the two.)
    const bool single = rows == segments;
    if (dtype == JLLM_F32) {
        if (single) JLLM_GLA(float, 16);
        if (dk <= 128) JLLM_GLA(float, 4);
        if (dk <= 256) JLLM_GLA(float, 8);
        JLLM_GLA(float, 16);
    }
    if (single) JLLM_GLA(__nv_bfloat16, 16);
    if (dk <= 128) JLLM_GLA(__nv_bfloat16, 4);
    if (dk <= 256) JLLM_GLA(__nv_bfloat16, 8);
    JLLM_GLA(__nv_bfloat16, 16);
#undef JLLM_GLA
}

// The same recurrence for steps with prompt portions, in chunks of 16 tokens (three launches: the log-decays in place
// of z, the chunks' operands, the walk through the chunks). qb, ke [rows, heads x dk] and scores [rows, heads x 16] are
// float32 scratch; `max_len`: the longest segment's rows.
JLLM_EXPORT int jllm_gla_chunked(const void* proj, int dtype, int ld, int q_off, int k_off, int v_off, float* z, int rows,
                                 float* qb, float* ke, float* scores, float* state, int num_slots, const int* seg_start,
                                 const int* seg_len, const int* state_slots, float* o, int segments, int max_len, int heads,
                                 int dk, int dv, float q_scale, float tau, const float* head_decay, int activation,
                                 cudaStream_t stream) {
    JLLM_REQUIRE(segments >= 0 && rows >= 0 && heads > 0 && dk > 0 && dv > 0 && tau > 0.f && max_len >= 0,
                 "gla_chunked: segments=%d heads=%d dk=%d dv=%d", segments, heads, dk, dv);
    JLLM_REQUIRE(dk <= 512 && heads <= 65535 && (dv + 31) / 32 <= 65535 && (max_len + CHUNK - 1) / CHUNK <= 65535,
                 "gla_chunked: dk=%d is above 512, or a segment of %d rows is too long", dk, max_len);
    if (segments == 0 || rows == 0 || max_len == 0) return JLLM_OK;
    if (head_decay && lightning::fits(dtype, ld, q_off, k_off, v_off, dk, dv, proj)) {
        // one decay per head, bfloat16 projections, key heads of 64 or 128: the chunks of 64 tokens on the tensor cores
        if (activation) {
            const int code = launch_fixed_decay<__nv_bfloat16>((void*)proj, ld, q_off, k_off, v_off, nullptr, head_decay, rows,
                                                               heads, dk, dv, 1, activation, stream);
            if (code) return code;
        }
        // blocks of 64 value columns, or of 32 where those would leave SMs without a block
        const int sms = jllm_device_sm_count() > 0 ? jllm_device_sm_count() : 1;
        const bool narrow = g_lightning_width ? g_lightning_width == 32 : (long long)segments * heads * ((dv + 63) / 64) < sms;
#define JLLM_LIGHTNING(DK_, DVB_)                                                                                             \
    do {                                                                                                                      \
        const size_t smem = lightning::smem_bytes<DK_, DVB_>();                                                               \
        cudaFuncSetAttribute(lightning::chunk_kernel<DK_, DVB_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        jllm_launch(lightning::chunk_kernel<DK_, DVB_>, dim3(segments, heads, (dv + DVB_ - 1) / DVB_), dim3(256), smem, stream, \
                    LAUNCH_DEPENDENT, (const __nv_bfloat16*)proj, ld, q_off, k_off, v_off, head_decay, state, seg_start, seg_len, \
                    state_slots, o, heads, dv, num_slots, q_scale);                                                           \
    } while (0)
        if (dk == 64) {
            if (narrow) JLLM_LIGHTNING(64, 32); else JLLM_LIGHTNING(64, 64);
        } else {
            if (narrow) JLLM_LIGHTNING(128, 32); else JLLM_LIGHTNING(128, 64);
        }
#undef JLLM_LIGHTNING
        return jllm_check_launch("lightning_chunk");
    }
    if (head_decay) {
        const int code = dtype == JLLM_F32
            ? launch_fixed_decay<float>((void*)proj, ld, q_off, k_off, v_off, z, head_decay, rows, heads, dk, dv, 1, activation, stream)
            : launch_fixed_decay<__nv_bfloat16>((void*)proj, ld, q_off, k_off, v_off, z, head_decay, rows, heads, dk, dv, 1, activation, stream);
        if (code) return code;
    } else {
        const size_t total = (size_t)rows * heads * dk;
        const int blocks = (int)min((size_t)65535, (total + 255) / 256);
        jllm_launch(gla_decay_kernel, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, z, 1.f / tau, total, 1);
        const int code = jllm_check_launch("gla_decay");
        if (code) return code;
    }
    {
        const size_t smem = (size_t)3 * CHUNK * (dk + 1) * sizeof(float);
        const dim3 grid(segments, (max_len + CHUNK - 1) / CHUNK, heads);
        if (dtype == JLLM_F32) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(gla_chunk_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            jllm_launch(gla_chunk_prepare_kernel<float>, grid, dim3(128), smem, stream, LAUNCH_DEPENDENT, (const float*)proj, ld,
                        q_off, k_off, z, seg_start, seg_len, qb, ke, scores, heads, dk, q_scale);
        } else {
            if (smem > 48 * 1024) cudaFuncSetAttribute(gla_chunk_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            jllm_launch(gla_chunk_prepare_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, LAUNCH_DEPENDENT,
                        (const __nv_bfloat16*)proj, ld, q_off, k_off, z, seg_start, seg_len, qb, ke, scores, heads, dk, q_scale);
        }
        const int code = jllm_check_launch("gla_chunk_prepare");
        if (code) return code;
    }
#define JLLM_GLA_CHUNK(T, R)                                                                                                  \
    return dk % 4 == 0 ? launch_chunked<T, R, true>(proj, ld, v_off, z, qb, ke, scores, state, seg_start, seg_len, state_slots, \
                                                    o, segments, heads, dk, dv, num_slots, stream)                           \
                       : launch_chunked<T, R, false>(proj, ld, v_off, z, qb, ke, scores, state, seg_start, seg_len,            \
                                                     state_slots, o, segments, heads, dk, dv, num_slots, stream)
    if (dtype == JLLM_F32) {
        if (dk <= 32) JLLM_GLA_CHUNK(float, 4);
        if (dk <= 128) JLLM_GLA_CHUNK(float, 8);
        if (dk <= 256) JLLM_GLA_CHUNK(float, 16);
        JLLM_GLA_CHUNK(float, 32);
    }
    if (dk <= 32) JLLM_GLA_CHUNK(__nv_bfloat16, 4);
    if (dk <= 128) JLLM_GLA_CHUNK(__nv_bfloat16, 8);
    if (dk <= 256) JLLM_GLA_CHUNK(__nv_bfloat16, 16);
    JLLM_GLA_CHUNK(__nv_bfloat16, 32);
#undef JLLM_GLA_CHUNK
}

JLLM_EXPORT int jllm_gated_head_norm(const float* o, const void* gate, int dtype, int ld_gate, const void* gain,
                                     int gain_dtype, void* y, int rows, int heads, int dv, float eps, float scale,
                                     int gate_kind, int gate_dtype, cudaStream_t stream) {
    // `dtype`: the type of y; `gate_dtype`: the gate's (the same, or float32 beside a bfloat16 y: a gate that a product left
    // in float32)
    JLLM_REQUIRE(rows >= 0 && heads > 0 && dv > 0, "gated_head_norm: rows=%d heads=%d dv=%d", rows, heads, dv);
    JLLM_REQUIRE(gate_dtype == dtype || gate_dtype == JLLM_F32, "gated_head_norm: a gate of type %d beside a result of type %d",
                 gate_dtype, dtype);
    if (rows == 0) return JLLM_OK;
    const VecRef g{gain, gain_dtype};
    const long long warps = (long long)rows * heads;
    const bool wide_gate = gate_dtype != dtype;
    // long norms: a block each; also norms of 256 values and more where a step has so few of them that a warp each would
    // leave the device idle (a step of single rows)
    if ((dv > 512 || (dv >= 256 && warps <= 2048)) && warps <= 2147483647ll) {
        if (dtype == JLLM_F32)
            jllm_launch(gated_row_norm_kernel<float>, dim3((unsigned)warps), dim3(256), 0, stream, LAUNCH_DEPENDENT, o,
                        (const float*)gate, ld_gate, g, (float*)y, heads, dv, eps, scale, gate_kind);
        else if (wide_gate)
            jllm_launch(gated_row_norm_kernel<__nv_bfloat16, float>, dim3((unsigned)warps), dim3(256), 0, stream, LAUNCH_DEPENDENT, o,
                        (const float*)gate, ld_gate, g, (__nv_bfloat16*)y, heads, dv, eps, scale, gate_kind);
        else
            jllm_launch(gated_row_norm_kernel<__nv_bfloat16>, dim3((unsigned)warps), dim3(256), 0, stream, LAUNCH_DEPENDENT, o,
                        (const __nv_bfloat16*)gate, ld_gate, g, (__nv_bfloat16*)y, heads, dv, eps, scale, gate_kind);
        return jllm_check_launch("gated_head_norm");
    }
    const dim3 grid((unsigned)((warps + 7) / 8));
    if (dtype == JLLM_F32)
        jllm_launch(gated_head_norm_kernel<float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, o, (const float*)gate,
                    ld_gate, g, (float*)y, rows, heads, dv, eps, scale, gate_kind);
    else if (wide_gate)
        jllm_launch(gated_head_norm_kernel<__nv_bfloat16, float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, o,
                    (const float*)gate, ld_gate, g, (__nv_bfloat16*)y, rows, heads, dv, eps, scale, gate_kind);
    else
        jllm_launch(gated_head_norm_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, o,
                    (const __nv_bfloat16*)gate, ld_gate, g, (__nv_bfloat16*)y, rows, heads, dv, eps, scale, gate_kind);
    return jllm_check_launch("gated_head_norm");
}


// The recurrence with a decay and an input scale per token and head (`jllm_scalar_gated_recurrent`, which this stands in for
// where a step holds prompt portions) in chunks of 64 tokens on the tensor cores: key heads of 64 or 128 channels, no
// normalizer. q, k, v: views of type `dtype` (float32 or bfloat16) with 16-byte aligned rows and pieces. Returns
// JLLM_UNSUPPORTED without launching where the shape is not taken (the caller then runs token by token).
JLLM_EXPORT int jllm_scalar_gated_chunked(const void* q, int ld_q, int q_off, int q_groups, const void* k, int ld_k, int k_off,
                                          int k_groups, const void* v, int ld_v, int v_off, int dtype, const float* la,
                                          const float* b, const void* skip, int skip_dtype, float* state, int num_slots,
                                          const int* seg_start, const int* seg_len, const int* state_slots, float* o,
                                          int segments, int heads, int dk, int dv, float q_scale, cudaStream_t stream) {
    const int per = dtype == JLLM_F32 ? 4 : 8;          // values of a 16-byte piece
    const bool aligned = ld_q % per == 0 && ld_k % per == 0 && ld_v % per == 0 && q_off % per == 0 && k_off % per == 0 &&
                         v_off % per == 0 && dv % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k % 16) == 0 &&
                         ((uintptr_t)v % 16) == 0;
    if (!(dk == 64 || dk == 128) || !aligned || heads % q_groups || heads % k_groups || heads > 65535) return JLLM_UNSUPPORTED;
    if (segments == 0) return JLLM_OK;
    const VecRef sk{skip, skip_dtype};
    const int has_skip = skip != nullptr;
    const long long sms = max(1, jllm_device_sm_count());
    const bool wide = g_lightning_width ? g_lightning_width == 64 : (long long)segments * heads * ((dv + 63) / 64) >= sms;
#define JLLM_GATED_CHUNK(TS, DK, DVB)                                                                                          \
    do {                                                                                                                        \
        auto kernel = lightning::gated_chunk_kernel<TS, DK, DVB>;                                                               \
        const size_t smem = lightning::smem_bytes<DK, DVB>() + 2 * lightning::C * sizeof(float);                                \
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)                \
            return jllm_fail(JLLM_CUDA_ERROR, "gated_chunk: %zu bytes of shared memory refused", smem);                         \
        jllm_launch(kernel, dim3(segments, heads, (dv + DVB - 1) / DVB), dim3(256), smem, stream, LAUNCH_DEPENDENT,             \
                    (const TS*)q, ld_q, q_off, q_groups, (const TS*)k, ld_k, k_off, k_groups, (const TS*)v, ld_v, v_off, la, b, \
                    sk, has_skip, state, seg_start, seg_len, state_slots, o, heads, dv, num_slots, q_scale);                    \
        return jllm_check_launch("gated_chunk");                                                                                \
    } while (0)
    if (dtype == JLLM_F32) {
        if (dk == 64) { if (wide) JLLM_GATED_CHUNK(float, 64, 64); JLLM_GATED_CHUNK(float, 64, 32); }
        if (wide) JLLM_GATED_CHUNK(float, 128, 64);
        JLLM_GATED_CHUNK(float, 128, 32);
    }
    if (dk == 64) { if (wide) JLLM_GATED_CHUNK(__nv_bfloat16, 64, 64); JLLM_GATED_CHUNK(__nv_bfloat16, 64, 32); }
    if (wide) JLLM_GATED_CHUNK(__nv_bfloat16, 128, 64);
    JLLM_GATED_CHUNK(__nv_bfloat16, 128, 32);
#undef JLLM_GATED_CHUNK
}
