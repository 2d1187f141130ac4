// Routed experts: choosing, sorting rows by expert, the two grouped products and the sum.
//
//   moe_route    per token: scores from the 32-bit router logits (sigmoid, or softmax over all
//                experts), the `top` largest (the lower index wins a tie), optionally divided by
//                their sum -> ids [T, top], weights [T, top].
//   moe_align    the (token, choice) pairs sorted by expert into rows; each expert's rows start
//                on a multiple of the row tile, so a tile of rows belongs to one expert.  Writes
//                pos [T * top] (the row of each pair), row_token / row_scale [capacity] (-1 / 0 in
//                the padding) and tile_expert [capacity / tile] (-1 beyond the last used tile).
//   moe_up       rows gathered from x (times the row's weight if the weight goes on the input),
//                times the expert's gate/up matrix (rows alternate gate_i, up_i), act(g) * u.
//   moe_down     times the expert's down matrix -> y [capacity, hidden] 32-bit.
//   moe_combine  out[t] = sum over the token's choices of y[pos] (times the weight if it goes on
//                the output), rounded to T once.
//
// Each output row depends only on its own input row and its expert's weights, and the sum runs
// over a token's choices in their order, so where a row landed does not change any result.
#include "common.cuh"

#include <float.h>

LSB_DEFINE_STATUS()

constexpr int kTile = 32;               // rows per tile; an expert's rows are padded to this

// act(g) * u of a gated expert; act 5 is the capped form with a limit L: min(g, L) sigmoid(1.702 min(g, L))
// (clamp(u, -L, L) + 1)
__device__ __forceinline__ float moe_gate_mul(float z, float up, int act, float limit) {
    if (act == 5) {
        const float g = fminf(z, limit);
        return g / (1.f + expf(-1.702f * g)) * (fminf(fmaxf(up, -limit), limit) + 1.f);
    }
    if (act == 1) return z / (1.f + expf(-z)) * up;
    if (act == 2) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))) * up;
    return z * up;
}

// How scores are made and weighted: `score` 0 sigmoid, 1 softmax over all experts; `bias` (one number an
// expert, may be null) is added to the scores for the choice only; the chosen scores are divided by
// their sum + eps if `renorm`, and multiplied by `scale`.
struct RouteOpts {
    int score, renorm;
    const float* bias;
    float scale, eps;
};

constexpr int kMaxTop = 32;

// One warp chooses for one token (all lanes call it together).
__device__ __forceinline__ void route_token(const float* __restrict__ z, int E, int top, const RouteOpts ro,
                                            int* __restrict__ ids, float* __restrict__ wts, int lane) {
    const int score = ro.score, renorm = ro.renorm;
    float zmax = -FLT_MAX, denom = 1.f;
    if (score == 1) {
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
        zmax = lsb_warp_max(zmax);
        float s = 0.f;
        for (int e = lane; e < E; e += 32) s += expf(z[e] - zmax);
        denom = lsb_warp_sum(s);
    }
    int chosen[kMaxTop];
    float val[kMaxTop];
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -FLT_MAX;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= (chosen[j] == e);
            // (without a bias the logits order the experts as their scores do)
            const float c = ro.bias ? (score == 1 ? expf(z[e] - zmax) / denom : 1.f / (1.f + expf(-z[e]))) + ro.bias[e] : z[e];
            if (!taken && (c > best || (c == best && e < bi))) { best = c; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        chosen[k] = bi;
        if (ro.bias) best = z[bi];
        val[k] = score == 1 ? expf(best - zmax) / denom : 1.f / (1.f + expf(-best));
        total += val[k];
    }
    if (lane == 0) {
        for (int k = 0; k < top; ++k) {
            ids[k] = chosen[k];
            wts[k] = (renorm ? val[k] / (total + ro.eps) : val[k]) * ro.scale;
        }
    }
}

__global__ void moe_route_kernel(const float* __restrict__ logits, int n_tokens, int E, int top,
                                 RouteOpts ro, int* __restrict__ ids, float* __restrict__ wts) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_tokens) return;
    route_token(logits + (size_t)warp * E, E, top, ro, ids + (size_t)warp * top, wts + (size_t)warp * top, lane);
}

__global__ void __launch_bounds__(1024)
moe_align_kernel(int* __restrict__ ids, float* __restrict__ wts, int n, int top, int E,
                 int cap_tiles, int tile, int* __restrict__ pos, int* __restrict__ row_token,
                 float* __restrict__ row_scale, int* __restrict__ tile_expert,
                 const float* __restrict__ logits, RouteOpts ro) {
    extern __shared__ int shi[];
    int* counts = shi;                  // E
    int* starts = shi + E;              // E + 1, in rows
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    if (logits) {                       // a step of few tokens: the choosing is done here too, a warp a token
        for (int t = threadIdx.x >> 5; t < n / top; t += blockDim.x >> 5)
            route_token(logits + (size_t)t * E, E, top, ro, ids + (size_t)t * top, wts + (size_t)t * top,
                        threadIdx.x & 31);
        __syncthreads();
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    for (int i = threadIdx.x; i < cap_tiles * tile; i += blockDim.x) { row_token[i] = -1; row_scale[i] = 0.f; }
    for (int i = threadIdx.x; i < cap_tiles; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = ids[i];
        if (e < 0 || e >= E) { lsb_set_status(LSB_BAD_ROW); pos[i] = -1; continue; }
        pos[i] = atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            starts[e] = at;
            at += (counts[e] + tile - 1) / tile * tile;
        }
        starts[E] = at;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        for (int ti = starts[e] / tile; ti < starts[e + 1] / tile && ti < cap_tiles; ++ti)
            tile_expert[ti] = e;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (pos[i] < 0) continue;
        const int p = starts[ids[i]] + pos[i];
        pos[i] = p;
        if (p < cap_tiles * tile) { row_token[p] = i / top; row_scale[p] = wts[i]; }
    }
}

// MODE 0 (up):   A row = T(scale * x[row_token]) (scale 1 unless on_input), B = w[e] [2F, K], gated
//                epilogue -> out T [capacity, F]
// MODE 1 (down): A = h [capacity, K] T, B = w[e] [N, K] -> out 32-bit [capacity, N]
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ A, const int* __restrict__ row_token,
                const float* __restrict__ row_scale, int on_input, const T* __restrict__ W,
                const int* __restrict__ tile_expert, void* __restrict__ out_, int N, int K, int act, float limit) {
    __shared__ float As[kTile][kTile + 1];
    __shared__ float Bs[kTile][kTile + 1];
    __shared__ int tok_sh[kTile];
    __shared__ float scale_sh[kTile];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int e = tile_expert[blockIdx.y];
    if (e < 0) return;
    const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    if (threadIdx.x < kTile) {
        tok_sh[threadIdx.x] = row_token[m0 + threadIdx.x];
        scale_sh[threadIdx.x] = on_input ? row_scale[m0 + threadIdx.x] : 1.f;
    }
    __syncthreads();
    const T* B = W + (size_t)e * N * K;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += kTile) {
        for (int i = ty; i < kTile; i += 8) {
            const int k = k0 + tx, n = n0 + i;
            float a = 0.f;
            if (k < K && tok_sh[i] >= 0) {
                if (MODE == 0)
                    a = lsb_to_float(lsb_from_float<T>(scale_sh[i] * lsb_to_float(A[(size_t)tok_sh[i] * K + k])));
                else
                    a = lsb_to_float(A[(size_t)(m0 + i) * K + k]);
            }
            As[i][tx] = a;
            Bs[i][tx] = (n < N && k < K) ? lsb_to_float(B[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kTile; ++k) {
            const float bv = Bs[tx][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] += As[ty + 8 * j][k] * bv;
        }
        __syncthreads();
    }
    const int n = n0 + tx;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int m = m0 + ty + 8 * j;
        if (MODE == 0) {
            const float up = __shfl_down_sync(0xffffffffu, acc[j], 1);
            if (!(tx & 1) && n + 1 < N)
                ((T*)out_)[(size_t)m * (N / 2) + n / 2] = lsb_from_float<T>(moe_gate_mul(acc[j], up, act, limit));
        } else if (n < N) {
            ((float*)out_)[(size_t)m * N + n] = acc[j];
        }
    }
}

// One block per (token, choice) pair: only rows that stand for a pair are written.  The padding
// rows of a tile keep whatever the buffer held: a row of a product depends on its own operand row
// alone, and nothing reads the padding rows' results.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ pos,
                                  const float* __restrict__ wts, int on_input, int top, int capacity, int n,
                                  T* __restrict__ rows) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t pair = blockIdx.x;
    const int r = pos[pair];
    if (r < 0 || r >= capacity) return;
    const size_t tok = pair / top;
    const float sc = on_input ? wts[pair] : 1.f;
    const T* src = x + tok * n;
    T* dst = rows + (size_t)r * n;
    if (sizeof(T) == 2 && n % 8 == 0 && (((uintptr_t)x | (uintptr_t)rows) & 15) == 0) {
        for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {      // 16 bytes a thread and pass
            uint4 raw = *reinterpret_cast<const uint4*>(src + i);
            __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(p[k]);
                p[k] = __floats2bfloat162_rn(sc * f.x, sc * f.y);
            }
            *reinterpret_cast<uint4*>(dst + i) = raw;
        }
        return;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        dst[i] = lsb_from_float<T>(sc * lsb_to_float(src[i]));
}

template <typename T, typename TY>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ pos,
                                   const float* __restrict__ wts, int on_output, int top, int n,
                                   int capacity, T* __restrict__ out, const T* __restrict__ add) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const int p = pos[t * top + k];
            if (p < 0 || p >= capacity) continue;
            const float v = lsb_to_float(y[(size_t)p * n + i]);
            s += on_output ? wts[t * top + k] * v : v;
        }
        if (add) s += lsb_to_float(add[t * n + i]);          // (what every token passes besides its chosen experts)
        out[t * n + i] = lsb_from_float<T>(s);
    }
}

LSB_API int lsb_moe_tile() { return kTile; }

LSB_API int lsb_moe_route(const float* logits, int n_tokens, int E, int top, int score, int renorm,
                          const float* bias, float scale, float eps, int* ids, float* wts, cudaStream_t stream) {
    const RouteOpts ro = {score, renorm, bias, scale, eps};
    if (n_tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || top > kMaxTop || score < 0 || score > 1) return (int)cudaErrorInvalidValue;
    const int warps_per_block = 4;
    return lsb_launch(moe_route_kernel, dim3((n_tokens + warps_per_block - 1) / warps_per_block),
                      dim3(32 * warps_per_block), 0, stream, 1, logits, n_tokens, E, top, ro, ids, wts);
}

// logits given (32-bit [tokens, E]): ids and wts are chosen here first (see lsb_moe_route) and written
LSB_API int lsb_moe_align(int* ids, float* wts, int n_tokens, int top, int E, int cap_tiles,
                          int tile, int* pos, int* row_token, float* row_scale, int* tile_expert,
                          const float* logits, int score, int renorm, const float* bias, float scale, float eps,
                          cudaStream_t stream) {
    const RouteOpts ro = {score, renorm, bias, scale, eps};
    if (n_tokens <= 0) return 0;
    const long long n = (long long)n_tokens * top;
    if (E <= 0 || E > 8192 || tile <= 0 || cap_tiles < (n + tile - 1) / tile + E) return (int)cudaErrorInvalidValue;
    if (logits && (top > kMaxTop || top > E || score < 0 || score > 1)) return (int)cudaErrorInvalidValue;
    return lsb_launch(moe_align_kernel, dim3(1), dim3(1024), (size_t)(2 * E + 1) * sizeof(int), stream, 1,
                      ids, wts, (int)n, top, E, cap_tiles, tile, pos, row_token, row_scale, tile_expert, logits, ro);
}

// rows[pos[t, k]] = T(wts[t, k] * x[t]): the operand of the grouped tensor-core product, which wants
// its rows in place
LSB_API int lsb_moe_gather(const void* x, int dtype, const int* pos, const float* wts, int on_input,
                           int n_tokens, int top, int capacity, int n, void* rows, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(moe_gather_kernel<T>, dim3((unsigned)((long long)n_tokens * top)), dim3(128),
                                                0, stream, 1, (const T*)x, pos, wts, on_input, top, capacity, n,
                                                (T*)rows));
    return 0;
}

LSB_API int lsb_moe_up(const void* x, int dtype, const int* row_token, const float* row_scale, int on_input,
                       const void* w, const int* tile_expert, int cap_tiles, void* out, int F, int K,
                       int act, float limit, cudaStream_t stream) {
    if (cap_tiles <= 0) return 0;
    if (F <= 0 || K <= 0 || cap_tiles > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((2 * F + kTile - 1) / kTile, cap_tiles);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(moe_gemm_kernel<T, 0>, grid, dim3(256), 0, stream, 1,
                                                (const T*)x, row_token, row_scale, on_input, (const T*)w,
                                                tile_expert, out, 2 * F, K, act, limit));
    return 0;
}

LSB_API int lsb_moe_down(const void* h, int dtype, const int* row_token, const void* w,
                         const int* tile_expert, int cap_tiles, float* out, int N, int K,
                         cudaStream_t stream) {
    if (cap_tiles <= 0) return 0;
    if (N <= 0 || K <= 0 || cap_tiles > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((N + kTile - 1) / kTile, cap_tiles);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(moe_gemm_kernel<T, 1>, grid, dim3(256), 0, stream, 1,
                                                (const T*)h, row_token, (const float*)nullptr, 0, (const T*)w,
                                                tile_expert, (void*)out, N, K, 0, 0.f));
    return 0;
}

// y_same: the expert rows are stored in the output's type (the tensor-core path), else 32-bit
LSB_API int lsb_moe_combine(const void* y, int y_same, const int* pos, const float* wts, int on_output,
                            int n_tokens, int top, int n, int capacity, void* out, int dtype, const void* add,
                            cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    LSB_DISPATCH_DTYPE(dtype, {
        if (y_same)
            return lsb_launch(moe_combine_kernel<T, T>, dim3(n_tokens), dim3(256), 0, stream, 1, (const T*)y, pos,
                              wts, on_output, top, n, capacity, (T*)out, (const T*)add);
        return lsb_launch(moe_combine_kernel<T, float>, dim3(n_tokens), dim3(256), 0, stream, 1, (const float*)y,
                          pos, wts, on_output, top, n, capacity, (T*)out, (const T*)add);
    });
    return 0;
}
