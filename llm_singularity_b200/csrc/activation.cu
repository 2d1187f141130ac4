// The activation of a gated feed-forward on a fused gate/up product whose columns alternate
// gate_i, up_i: out[t, i] = act(gu[t, 2i]) * gu[t, 2i + 1], evaluated in 32-bit.  act: silu(g) =
// g / (1 + exp(-g)); gelu in its tanh form, 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)));
// or none (gate * up); or the capped form with a limit L: g' = min(g, L), u' = clamp(u, -L, L),
// out = g' sigmoid(1.702 g') (u' + 1).
//
// Replaces silu_mul_kernel of the reference (kernels/src/activations.cu:11-21), which
// reads two separate fp32 buffers and knows silu only.  The bfloat16 tensor-core product applies
// the same formulas in its epilogue; this kernel serves the 32-bit path and shapes that product
// does not take.
#include "common.cuh"

LSB_DEFINE_STATUS()

enum : int { LSB_ACT_SILU = 1, LSB_ACT_GELU_TANH = 2, LSB_ACT_NONE = 3, LSB_ACT_CAPPED_GLU = 5 };

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gate_up, T* __restrict__ out,
                                 int inter, long long total, int act, float limit) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        // out is [tokens, inter] and gate_up [tokens, 2 * inter]: element idx reads 2 idx, 2 idx + 1
        const float g = lsb_to_float(gate_up[2 * idx]);
        float u = lsb_to_float(gate_up[2 * idx + 1]);
        float a;
        if (act == LSB_ACT_CAPPED_GLU) {
            const float gc = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit) + 1.f;
            a = gc / (1.f + expf(-1.702f * gc));
        } else if (act == LSB_ACT_SILU) a = g / (1.f + expf(-g));
        else if (act == LSB_ACT_GELU_TANH)
            a = 0.5f * g * (1.f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
        else a = g;
        out[idx] = lsb_from_float<T>(a * u);
    }
}

LSB_API int lsb_gated_act(const void* gate_up, void* out, int dtype, int tokens, int inter, int act, float limit,
                          cudaStream_t stream) {
    const long long total = (long long)tokens * inter;
    if (total <= 0) return 0;
    if ((act < LSB_ACT_SILU || act > LSB_ACT_NONE) && act != LSB_ACT_CAPPED_GLU) return (int)cudaErrorInvalidValue;
    int dev = 0, sms = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return (int)err;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > (long long)sms * 32) blocks = (long long)sms * 32;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(gated_act_kernel<T>, dim3((int)blocks), dim3(threads), 0, stream, 1,
                                                (const T*)gate_up, (T*)out, inter, total, act, limit));
    return 0;
}

// A plain (ungated) activation on every element, evaluated in 32-bit.  LSB_ACT_BENT_SQUARE is a
// two-branch activation with two learnt numbers handed in already transformed: right of zero a
// parabola, c_pos z^2 + z / 2; left of it a saturating branch, c_neg (e^z - 1 - z) + z / 2
// (c_pos = softplus(p), c_neg = 1/2 + softplus(q) for the stored p and q).
enum : int { LSB_ACT_BENT_SQUARE = 4 };

__device__ __forceinline__ float plain_act_of(float z, int act, float c_pos, float c_neg) {
    if (act == LSB_ACT_SILU) return z / (1.f + expf(-z));
    if (act == LSB_ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608f * (z + 0.044715f * z * z * z)));
    if (act == LSB_ACT_BENT_SQUARE) return z > 0.f ? c_pos * z * z + 0.5f * z : c_neg * (expm1f(z) - z) + 0.5f * z;
    return z;
}

// 16 bytes a thread and turn where the count and both addresses allow (`wide`), one value otherwise.
template <typename T>
__global__ void plain_act_kernel(const T* __restrict__ x, T* __restrict__ out, long long total, int act, float c_pos,
                                 float c_neg, int wide) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    constexpr int N = 16 / (int)sizeof(T);
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (wide) {
        const long long groups = total / N;
        for (; idx < groups; idx += stride) {
            uint4 raw = reinterpret_cast<const uint4*>(x)[idx];
            T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
            for (int i = 0; i < N; ++i) v[i] = lsb_from_float<T>(plain_act_of(lsb_to_float(v[i]), act, c_pos, c_neg));
            reinterpret_cast<uint4*>(out)[idx] = raw;
        }
        return;
    }
    for (; idx < total; idx += stride) out[idx] = lsb_from_float<T>(plain_act_of(lsb_to_float(x[idx]), act, c_pos, c_neg));
}

LSB_API int lsb_plain_act(const void* x, void* out, int dtype, long long total, int act, float c_pos, float c_neg,
                          cudaStream_t stream) {
    if (total <= 0) return 0;
    if (act < LSB_ACT_SILU || act > LSB_ACT_BENT_SQUARE) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    const int per = dtype == LSB_F32 ? 4 : 8;    // values in 16 bytes
    const int wide = total % 8 == 0 && ((reinterpret_cast<size_t>(x) | reinterpret_cast<size_t>(out)) & 15) == 0;
    const long long work = wide ? total / per : total;
    long long blocks = (work + threads - 1) / threads;
    if (blocks < 1) blocks = 1;
    if (blocks > 148LL * 32) blocks = 148LL * 32;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(plain_act_kernel<T>, dim3((int)blocks), dim3(threads), 0, stream, 1,
                                                (const T*)x, (T*)out, total, act, c_pos, c_neg, wide));
    return 0;
}

// x <- cap * tanh(x / cap) in place on 32-bit values (a soft cap on logits).
__global__ void softcap_kernel(float* __restrict__ x, long long total, float cap) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const float inv = 1.f / cap;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

LSB_API int lsb_softcap(float* x, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
    long long blocks = (total + 255) / 256;
    if (blocks > 148LL * 32) blocks = 148LL * 32;
    return lsb_launch(softcap_kernel, dim3((int)blocks), dim3(256), 0, stream, 1, x, total, cap);
}
