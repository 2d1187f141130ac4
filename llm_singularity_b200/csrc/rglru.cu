// The recurrent branch of a gated linear recurrent unit with real gates (RG-LRU), for any mix of prompt
// portions and single tokens:
//
//     u_t = conv(x)_t                  a causal convolution per channel over the x branch (taps, bias)
//     r_t = sigmoid(R u_t + b_r)       R, I block-diagonal (their products come from outside, 32-bit)
//     i_t = sigmoid(I u_t + b_i)
//     log a_t = -c * r_t * softplus(lam)        a_t = exp(log a_t)
//     S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t        out_t = S_t * act(y_t + b_y)
//
// All of it is 32-bit (with one split: where the gates' maps are bfloat16, u enters their products on the
// tensor cores as the sum of two bfloat16 numbers, 16 bits of mantissa, see rglru_conv_kernel; the 32-bit
// path multiplies u as it is): the projections arrive in 32-bit, the convolution sums, the gates, decays, the
// state and the product with the other branch are formed in 32-bit, and only out is rounded to the
// compute dtype.  sqrt(1 - a^2) is formed as sqrt(-expm1(2 log a)), which keeps its digits where a is
// close to one.  A request's state is S (one number a channel) and the x branch's last taps - 1 inputs,
// one row per request slot each; both are zero when a request begins, so the zeros before a sequence's
// start and the first token's S_(t-1) = 0 need no special case.
//
// Long portions are walked in segments side by side (see rglru_segment_kernel).
//
// Three kernels: the convolution (a thread per token and channel); the gates (the same, in place:
// the two gate products become a_t and the input sqrt(1 - a_t^2) i_t u_t, the y branch becomes its
// activation); the walk (a thread per request and channel, tokens in order, three loads and one
// multiply-add a step, loads of the steps ahead in flight), which also leaves the new state and the
// convolution's last inputs in the slot.
#include "common.cuh"

LSB_DEFINE_STATUS()

// u[t, c] = cb[c] + sum_k w[c, k] * xin[t - (taps - 1 - k), c], xin = proj x + xb; before the portion's
// first token xin comes from the slot's last inputs (zeros before the sequence's start).
__global__ void rglru_conv_kernel(const float* __restrict__ proj, long long ld, int x_off,
                                  const float* __restrict__ x_bias, const float* __restrict__ w,
                                  const float* __restrict__ conv_bias, int taps, const float* __restrict__ conv_state,
                                  const int* __restrict__ token_req, const int* __restrict__ q_start,
                                  const int* __restrict__ table_rows, int slots, float* __restrict__ u, int width,
                                  int tokens, __nv_bfloat16* __restrict__ split, int bw) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (c >= width) return;
    const int r = token_req[t];
    const int first = q_start[r];
    const int slot = table_rows[r];
    if (slot < 0 || slot >= slots) {
        lsb_set_status(LSB_BAD_ROW);
        u[(size_t)t * width + c] = 0.f;
        return;
    }
    const float xb = x_bias ? x_bias[c] : 0.f;
    float acc = conv_bias ? conv_bias[c] : 0.f;
    for (int k = 0; k < taps; ++k) {
        const int src = t - (taps - 1 - k);
        float x;
        if (src >= first) x = proj[(size_t)src * ld + x_off + c] + xb;
        else x = conv_state[((size_t)slot * (taps - 1) + (taps - 1 - (first - src))) * width + c];
        acc += w[(size_t)c * taps + k] * x;
    }
    u[(size_t)t * width + c] = acc;
    if (split) {
        // u as the sum of two bfloat16 numbers (the rounded value and the rounded rest: 16 bits of mantissa
        // together), side by side per block, [t, b, hi(bw) | lo(bw)]: the operand of a tensor-core product
        // against the gates' maps repeated along k, whose 32-bit sums then hold u's digits
        const int b = c / bw, o = c - b * bw;
        const __nv_bfloat16 hi = __float2bfloat16_rn(acc);
        __nv_bfloat16* dst = split + (size_t)t * 2 * width + (size_t)b * 2 * bw + o;
        dst[0] = hi;
        dst[bw] = __float2bfloat16_rn(acc - __bfloat162float(hi));
    }
}

__device__ __forceinline__ float rglru_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float rglru_softplus(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }
__device__ __forceinline__ float rglru_gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// In place: gates[t, b, 0:bw] (r's product) <- a_t, gates[t, b, bw:2bw] (i's product) <- sqrt(1 - a_t^2) i_t u_t,
// proj y <- act(y + yb); channel c = b * bw + o.
__global__ void rglru_gate_kernel(float* __restrict__ gates, const float* __restrict__ r_bias,
                                  const float* __restrict__ i_bias, const float* __restrict__ lam, float rate,
                                  const float* __restrict__ u, float* __restrict__ proj, long long ld, int y_off,
                                  const float* __restrict__ y_bias, int width, int bw) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (c >= width) return;
    const int b = c / bw, o = c - b * bw;
    float* g = gates + (size_t)t * 2 * width + (size_t)b * 2 * bw + o;
    const float rg = rglru_sigmoid(g[0] + (r_bias ? r_bias[c] : 0.f));
    const float ig = rglru_sigmoid(g[bw] + (i_bias ? i_bias[c] : 0.f));
    const float log_a = -rate * rg * rglru_softplus(lam[c]);
    g[0] = expf(log_a);
    g[bw] = sqrtf(-expm1f(2.f * log_a)) * ig * u[(size_t)t * width + c];
    float* y = proj + (size_t)t * ld + y_off + c;
    y[0] = rglru_gelu_tanh(y[0] + (y_bias ? y_bias[c] : 0.f));
}

constexpr int kWalkAhead = 8;

template <typename T>
__global__ void __launch_bounds__(64)
rglru_walk_kernel(const float* __restrict__ gates, const float* __restrict__ proj, long long ld, int x_off, int y_off,
                  const float* __restrict__ x_bias, int taps, float* __restrict__ state, float* __restrict__ conv_state,
                  const int* __restrict__ q_start, const int* __restrict__ table_rows, int slots, T* __restrict__ out,
                  int width, int bw) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= width) return;
    const int first = q_start[r], end = q_start[r + 1];
    const int slot = table_rows[r];
    if (slot < 0 || slot >= slots) {
        lsb_set_status(LSB_BAD_ROW);
        for (int t = first; t < end; ++t) out[(size_t)t * width + c] = lsb_from_float<T>(0.f);
        return;
    }
    const int b = c / bw, o = c - b * bw;
    const float* g = gates + (size_t)b * 2 * bw + o;
    float S = state[(size_t)slot * width + c];
    for (int t0 = first; t0 < end; t0 += kWalkAhead) {
        float a[kWalkAhead], in[kWalkAhead], y[kWalkAhead];
#pragma unroll
        for (int j = 0; j < kWalkAhead; ++j) {
            const int t = t0 + j;
            const bool live = t < end;
            a[j] = live ? g[(size_t)t * 2 * width] : 1.f;
            in[j] = live ? g[(size_t)t * 2 * width + bw] : 0.f;
            y[j] = live ? proj[(size_t)t * ld + y_off + c] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < kWalkAhead; ++j) {
            S = a[j] * S + in[j];
            if (t0 + j < end) out[(size_t)(t0 + j) * width + c] = lsb_from_float<T>(S * y[j]);
        }
    }
    state[(size_t)slot * width + c] = S;
    // the convolution's last inputs: entry j of the slot is the input taps - 1 - j tokens before the next one
    const int n = end - first, keep = taps - 1;
    const float xb = x_bias ? x_bias[c] : 0.f;
    float* cs = conv_state + (size_t)slot * keep * width + c;
    for (int j = 0; j < keep; ++j) {
        const int back = keep - j;                      // how far before the next token
        // (increasing j reads entries j + n > j of the old state: none has been written yet)
        cs[(size_t)j * width] = back <= n ? proj[(size_t)(end - back) * ld + x_off + c] + xb : cs[(size_t)(j + n) * width];
    }
}

// Long portions in segments walked side by side.  A token's step is S <- a S + in, so a segment walked from
// zero gives E (its own contribution) and the product P of its a's; the chain start(s + 1) = P_s start(s) + E_s
// runs over the segments of a request in order (and leaves the new state and the convolution's last inputs
// in the slot, as the single walk does); then every segment is walked again from its start for the outputs.
// seg_pe: [requests * segs, 2, width] (P, then E; the chain writes a segment's start over its P).
__global__ void __launch_bounds__(64)
rglru_segment_kernel(const float* __restrict__ gates, const int* __restrict__ q_start, int seg_len, int segs,
                     float* __restrict__ seg_pe, int width, int bw) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y / segs, sg = blockIdx.y % segs;
    if (c >= width) return;
    const int first = q_start[r] + sg * seg_len, end = min(q_start[r + 1], first + seg_len);
    if (first >= end) return;
    const int b = c / bw, o = c - b * bw;
    const float* g = gates + (size_t)b * 2 * bw + o;
    float P = 1.f, E = 0.f;
    for (int t0 = first; t0 < end; t0 += kWalkAhead) {
        float a[kWalkAhead], in[kWalkAhead];
#pragma unroll
        for (int j = 0; j < kWalkAhead; ++j) {
            const bool live = t0 + j < end;
            a[j] = live ? g[(size_t)(t0 + j) * 2 * width] : 1.f;
            in[j] = live ? g[(size_t)(t0 + j) * 2 * width + bw] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < kWalkAhead; ++j) {
            E = a[j] * E + in[j];
            P *= a[j];
        }
    }
    float* pe = seg_pe + ((size_t)blockIdx.y * 2) * width + c;
    pe[0] = P;
    pe[width] = E;
}

__global__ void __launch_bounds__(64)
rglru_chain_kernel(float* __restrict__ seg_pe, const float* __restrict__ proj, long long ld, int x_off,
                   const float* __restrict__ x_bias, int taps, float* __restrict__ state, float* __restrict__ conv_state,
                   const int* __restrict__ q_start, const int* __restrict__ table_rows, int slots, int seg_len, int segs,
                   int width) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= width) return;
    const int first = q_start[r], end = q_start[r + 1];
    const int slot = table_rows[r];
    if (slot < 0 || slot >= slots) {
        lsb_set_status(LSB_BAD_ROW);
        return;
    }
    float S = state[(size_t)slot * width + c];
    const int n = end - first, used = (n + seg_len - 1) / seg_len;
    for (int sg = 0; sg < used; ++sg) {
        float* pe = seg_pe + ((size_t)(r * segs + sg) * 2) * width + c;
        const float P = pe[0], E = pe[width];
        pe[0] = S;
        S = P * S + E;
    }
    state[(size_t)slot * width + c] = S;
    const int keep = taps - 1;
    const float xb = x_bias ? x_bias[c] : 0.f;
    float* cs = conv_state + (size_t)slot * keep * width + c;
    for (int j = 0; j < keep; ++j) {
        const int back = keep - j;
        cs[(size_t)j * width] = back <= n ? proj[(size_t)(end - back) * ld + x_off + c] + xb : cs[(size_t)(j + n) * width];
    }
}

template <typename T>
__global__ void __launch_bounds__(64)
rglru_segment_out_kernel(const float* __restrict__ gates, const float* __restrict__ proj, long long ld, int y_off,
                         const float* __restrict__ seg_pe, const int* __restrict__ q_start, int seg_len, int segs,
                         T* __restrict__ out, int width, int bw) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y / segs, sg = blockIdx.y % segs;
    if (c >= width) return;
    const int first = q_start[r] + sg * seg_len, end = min(q_start[r + 1], first + seg_len);
    if (first >= end) return;
    const int b = c / bw, o = c - b * bw;
    const float* g = gates + (size_t)b * 2 * bw + o;
    float S = seg_pe[((size_t)blockIdx.y * 2) * width + c];
    for (int t0 = first; t0 < end; t0 += kWalkAhead) {
        float a[kWalkAhead], in[kWalkAhead], y[kWalkAhead];
#pragma unroll
        for (int j = 0; j < kWalkAhead; ++j) {
            const int t = t0 + j;
            const bool live = t < end;
            a[j] = live ? g[(size_t)t * 2 * width] : 1.f;
            in[j] = live ? g[(size_t)t * 2 * width + bw] : 0.f;
            y[j] = live ? proj[(size_t)t * ld + y_off + c] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < kWalkAhead; ++j) {
            S = a[j] * S + in[j];
            if (t0 + j < end) out[(size_t)(t0 + j) * width + c] = lsb_from_float<T>(S * y[j]);
        }
    }
}

// seg_pe: 32-bit scratch of n_requests * ceil(max_q_len / seg_len) * 2 * width numbers
LSB_API int lsb_rglru_walk_segments(const float* gates, const float* proj, long long ld, int x_off, int y_off,
                                    const float* x_bias, int taps, float* state, float* conv_state, const int* q_start,
                                    const int* table_rows, int slots, void* out, int dtype, int width, int blocks,
                                    int n_requests, int max_q_len, int seg_len, float* seg_pe, cudaStream_t stream) {
    if (n_requests <= 0 || max_q_len <= 0) return 0;
    if (width <= 0 || blocks <= 0 || width % blocks || taps <= 0 || seg_len <= 0 || !seg_pe) return (int)cudaErrorInvalidValue;
    const int segs = (max_q_len + seg_len - 1) / seg_len;
    if ((long long)n_requests * segs > 65535) return (int)cudaErrorInvalidValue;
    const dim3 grid((width + 63) / 64, n_requests * segs);
    int rc = lsb_launch(rglru_segment_kernel, grid, dim3(64), 0, stream, 1, gates, q_start, seg_len, segs, seg_pe, width,
                        width / blocks);
    if (rc) return rc;
    rc = lsb_launch(rglru_chain_kernel, dim3((width + 63) / 64, n_requests), dim3(64), 0, stream, 1, seg_pe, proj, ld, x_off,
                    x_bias, taps, state, conv_state, q_start, table_rows, slots, seg_len, segs, width);
    if (rc) return rc;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(rglru_segment_out_kernel<T>, grid, dim3(64), 0, stream, 1, gates, proj, ld,
                                                y_off, (const float*)seg_pe, q_start, seg_len, segs, (T*)out, width,
                                                width / blocks));
    return 0;
}

LSB_API int lsb_rglru_conv(const float* proj, long long ld, int x_off, const float* x_bias, const float* w,
                           const float* conv_bias, int taps, const float* conv_state, const int* token_req,
                           const int* q_start, const int* table_rows, int slots, float* u, int width, int tokens,
                           void* split, int blocks, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || taps <= 0 || tokens > 65535 * 32) return (int)cudaErrorInvalidValue;
    if (tokens > 65535 || (split && (blocks <= 0 || width % blocks))) return (int)cudaErrorInvalidValue;
    return lsb_launch(rglru_conv_kernel, dim3((width + 127) / 128, tokens), dim3(128), 0, stream, 1, proj, ld, x_off,
                      x_bias, w, conv_bias, taps, conv_state, token_req, q_start, table_rows, slots, u, width, tokens,
                      (__nv_bfloat16*)split, split ? width / blocks : width);
}

LSB_API int lsb_rglru_gates(float* gates, const float* r_bias, const float* i_bias, const float* lam, float rate,
                            const float* u, float* proj, long long ld, int y_off, const float* y_bias, int width,
                            int blocks, int tokens, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || blocks <= 0 || width % blocks || tokens > 65535) return (int)cudaErrorInvalidValue;
    return lsb_launch(rglru_gate_kernel, dim3((width + 127) / 128, tokens), dim3(128), 0, stream, 1, gates, r_bias,
                      i_bias, lam, rate, u, proj, ld, y_off, y_bias, width, width / blocks);
}

LSB_API int lsb_rglru_walk(const float* gates, const float* proj, long long ld, int x_off, int y_off,
                           const float* x_bias, int taps, float* state, float* conv_state, const int* q_start,
                           const int* table_rows, int slots, void* out, int dtype, int width, int blocks,
                           int n_requests, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (width <= 0 || blocks <= 0 || width % blocks || taps <= 0 || n_requests > 65535) return (int)cudaErrorInvalidValue;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(rglru_walk_kernel<T>, dim3((width + 63) / 64, n_requests), dim3(64), 0,
                                                stream, 1, gates, proj, ld, x_off, y_off, x_bias, taps, state,
                                                conv_state, q_start, table_rows, slots, (T*)out, width,
                                                width / blocks));
    return 0;
}
