// Rows of a residual stream whose sublayers are normed on both sides:
//
//     x <- x + mult * unit(y) * w_post  [+ step]        out = unit(x) * w_next
//
// with unit(z) = z / sqrt(mean(z^2) + eps).  One kernel does the norm behind a sublayer, the sum
// into the 32-bit stream, an optional vector added to every row (the step vector of a pass through
// looped layers) and the norm in front of the next sublayer; each of the three is optional.  The
// gathered form does the same for selected rows and leaves the stream alone (the rows whose
// logits are wanted).  All arithmetic is 32-bit; y and out are in the compute dtype.
//
// The second kernel is the meeting point of mixers that run side by side on one input:
// out = (1 / n) * sum_b unit(y_b) * w_b, each branch normed over the row with its own weight.
//
// One thread block per row; the row waits in shared memory between the passes.
#include "common.cuh"

LSB_DEFINE_STATUS()

constexpr int kRowThreads = 256;

// four consecutive elements of a row at once (the row's width a multiple of four, 16-byte aligned)
__device__ __forceinline__ float4 row_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 row_load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void row_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void row_store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

// The same as stream_norm_kernel below with 16-byte accesses.
template <typename T, bool GATHER>
__global__ void __launch_bounds__(kRowThreads)
stream_norm_vec4_kernel(float* __restrict__ residual, const T* __restrict__ y, const float* __restrict__ post_w,
                        float post_eps, float mult, const float* __restrict__ step, const int* __restrict__ rows,
                        const float* __restrict__ next_w, float next_eps, T* __restrict__ out, int hidden,
                        int n_rows_total) {
    extern __shared__ float row_sh[];
    __shared__ float scratch[33];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r_out = blockIdx.x;
    int r_in = r_out;
    if (GATHER) {
        r_in = rows[r_out];
        if (r_in < 0 || r_in >= n_rows_total) {
            if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW);
            if (out)
                for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)r_out * hidden + i] = lsb_from_float<T>(0.f);
            return;
        }
    }
    float* res = residual + (size_t)r_in * hidden;
    const T* yr = y ? y + (size_t)r_in * hidden : nullptr;
    float inv_y = 1.f;
    if (yr && post_w) {
        float ss = 0.f;
        for (int i = 4 * threadIdx.x; i < hidden; i += 4 * kRowThreads) {
            const float4 v = row_load4(yr + i);
            row_store4(row_sh + i, v);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = lsb_block_sum(ss, scratch);
        inv_y = rsqrtf(ss / (float)hidden + post_eps);
    }
    float ss = 0.f;
    for (int i = 4 * threadIdx.x; i < hidden; i += 4 * kRowThreads) {
        float4 x = row_load4(res + i);
        if (yr) {
            if (post_w) {
                const float4 v = row_load4(row_sh + i), w = row_load4(post_w + i);
                x.x += mult * (v.x * inv_y * w.x);
                x.y += mult * (v.y * inv_y * w.y);
                x.z += mult * (v.z * inv_y * w.z);
                x.w += mult * (v.w * inv_y * w.w);
            } else {
                const float4 v = row_load4(yr + i);
                x.x += mult * v.x;
                x.y += mult * v.y;
                x.z += mult * v.z;
                x.w += mult * v.w;
            }
        }
        if (step) {
            const float4 v = row_load4(step + i);
            x.x += v.x;
            x.y += v.y;
            x.z += v.z;
            x.w += v.w;
        }
        if (!GATHER && (yr || step)) row_store4(res + i, x);
        row_store4(row_sh + i, x);
        ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    if (!out) return;
    ss = lsb_block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + next_eps);
    T* o = out + (size_t)r_out * hidden;
    for (int i = 4 * threadIdx.x; i < hidden; i += 4 * kRowThreads) {
        const float4 x = row_load4(row_sh + i), w = row_load4(next_w + i);
        row_store4(o + i, make_float4(x.x * inv * w.x, x.y * inv * w.y, x.z * inv * w.z, x.w * inv * w.w));
    }
}

template <typename T, bool GATHER>
__global__ void __launch_bounds__(kRowThreads)
stream_norm_kernel(float* __restrict__ residual, const T* __restrict__ y, const float* __restrict__ post_w,
                   float post_eps, float mult, const float* __restrict__ step, const int* __restrict__ rows,
                   const float* __restrict__ next_w, float next_eps, T* __restrict__ out, int hidden,
                   int n_rows_total) {
    extern __shared__ float row_sh[];
    __shared__ float scratch[33];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r_out = blockIdx.x;
    int r_in = r_out;
    if (GATHER) {
        r_in = rows[r_out];
        if (r_in < 0 || r_in >= n_rows_total) {
            if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW);
            if (out)
                for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)r_out * hidden + i] = lsb_from_float<T>(0.f);
            return;
        }
    }
    float* res = residual + (size_t)r_in * hidden;
    const T* yr = y ? y + (size_t)r_in * hidden : nullptr;
    float inv_y = 1.f;
    if (yr && post_w) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < hidden; i += kRowThreads) {
            const float v = lsb_to_float(yr[i]);
            row_sh[i] = v;
            ss += v * v;
        }
        ss = lsb_block_sum(ss, scratch);
        inv_y = rsqrtf(ss / (float)hidden + post_eps);
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += kRowThreads) {
        float x = res[i];
        if (yr) x += post_w ? mult * (row_sh[i] * inv_y * post_w[i]) : mult * lsb_to_float(yr[i]);
        if (step) x += step[i];
        if (!GATHER && (yr || step)) res[i] = x;
        row_sh[i] = x;
        ss += x * x;
    }
    if (!out) return;
    ss = lsb_block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + next_eps);
    T* o = out + (size_t)r_out * hidden;
    for (int i = threadIdx.x; i < hidden; i += kRowThreads) o[i] = lsb_from_float<T>(row_sh[i] * inv * next_w[i]);
}

// y, post_w, step, next_w / out may each be null (post_w null with y given: a plain sum of mult * y).
// rows null: every row of the stream, in place; else the rows named, the stream untouched.
LSB_API int lsb_stream_norm(float* residual, const void* y, const float* post_w, float post_eps, float mult,
                            const float* step, const int* rows, int n_rows, const float* next_w, float next_eps,
                            void* out, int dtype, int n_rows_total, int hidden, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (hidden <= 0 || (out && !next_w)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    // 16-byte accesses: rows a multiple of four wide, every operand on a 16-byte boundary
    bool vec = hidden % 4 == 0;
    for (const void* ptr : {(const void*)residual, y, (const void*)post_w, (const void*)step, (const void*)next_w, (const void*)out})
        vec = vec && ((uintptr_t)ptr % 16 == 0);
#define LSB_STREAM_NORM(KERNEL, G)                                                                    \
    do {                                                                                              \
        if (smem > 48 * 1024) {                                                                       \
            int rc = (int)cudaFuncSetAttribute(KERNEL<T, G>,                                          \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (rc) return rc;                                                                        \
        }                                                                                             \
        return lsb_launch(KERNEL<T, G>, dim3(n_rows), dim3(kRowThreads), smem, stream, 1, residual,   \
                          (const T*)y, post_w, post_eps, mult, step, rows, next_w, next_eps, (T*)out, hidden,  \
                          n_rows_total);                                                              \
    } while (0)
    LSB_DISPATCH_DTYPE(dtype, {
        if (vec && rows) LSB_STREAM_NORM(stream_norm_vec4_kernel, true);
        else if (vec) LSB_STREAM_NORM(stream_norm_vec4_kernel, false);
        else if (rows) LSB_STREAM_NORM(stream_norm_kernel, true);
        else LSB_STREAM_NORM(stream_norm_kernel, false);
    });
#undef LSB_STREAM_NORM
    return 0;
}

constexpr int kMaxBranches = 4;
struct Branches {
    const void* y[kMaxBranches];
    const float* w[kMaxBranches];
    int n;
};

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
branch_mean_kernel(Branches br, float eps, T* __restrict__ out, int hidden) {
    __shared__ float scratch[33];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t base = (size_t)blockIdx.x * hidden;
    float inv[kMaxBranches];
#pragma unroll
    for (int b = 0; b < kMaxBranches; ++b) {
        inv[b] = 0.f;
        if (b < br.n) {
            const T* yb = (const T*)br.y[b] + base;
            float ss = 0.f;
            for (int i = threadIdx.x; i < hidden; i += kRowThreads) {
                const float v = lsb_to_float(yb[i]);
                ss += v * v;
            }
            ss = lsb_block_sum(ss, scratch);
            inv[b] = rsqrtf(ss / (float)hidden + eps);
        }
    }
    const float share = 1.f / (float)br.n;
    for (int i = threadIdx.x; i < hidden; i += kRowThreads) {
        float s = 0.f;
#pragma unroll
        for (int b = 0; b < kMaxBranches; ++b)
            if (b < br.n) s += lsb_to_float(((const T*)br.y[b])[base + i]) * inv[b] * br.w[b][i];
        out[base + i] = lsb_from_float<T>(s * share);
    }
}

// The same with 16-byte accesses and every branch's row read once: a thread keeps its share of each
// branch (rows up to kBranchRegs * 4 * 256 wide) between the sums of squares and the mean.
constexpr int kBranchRegs = 2;

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
branch_mean_vec4_kernel(Branches br, float eps, T* __restrict__ out, int hidden) {
    __shared__ float scratch[33];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t base = (size_t)blockIdx.x * hidden;
    float4 keep[kMaxBranches][kBranchRegs];
    float inv[kMaxBranches];
#pragma unroll
    for (int b = 0; b < kMaxBranches; ++b) {
#pragma unroll
        for (int u = 0; u < kBranchRegs; ++u) {
            const int i = 4 * (threadIdx.x + u * kRowThreads);
            keep[b][u] = (b < br.n && i < hidden) ? row_load4((const T*)br.y[b] + base + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
#pragma unroll
    for (int b = 0; b < kMaxBranches; ++b) {
        inv[b] = 0.f;
        if (b < br.n) {
            float ss = 0.f;
#pragma unroll
            for (int u = 0; u < kBranchRegs; ++u)
                ss += keep[b][u].x * keep[b][u].x + keep[b][u].y * keep[b][u].y + keep[b][u].z * keep[b][u].z +
                      keep[b][u].w * keep[b][u].w;
            ss = lsb_block_sum(ss, scratch);
            inv[b] = rsqrtf(ss / (float)hidden + eps);
        }
    }
    const float share = 1.f / (float)br.n;
#pragma unroll
    for (int u = 0; u < kBranchRegs; ++u) {
        const int i = 4 * (threadIdx.x + u * kRowThreads);
        if (i < hidden) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int b = 0; b < kMaxBranches; ++b) {
                if (b < br.n) {
                    const float4 w = row_load4(br.w[b] + i);
                    acc.x += keep[b][u].x * inv[b] * w.x;
                    acc.y += keep[b][u].y * inv[b] * w.y;
                    acc.z += keep[b][u].z * inv[b] * w.z;
                    acc.w += keep[b][u].w * inv[b] * w.w;
                }
            }
            row_store4(out + base + i, make_float4(acc.x * share, acc.y * share, acc.z * share, acc.w * share));
        }
    }
}

LSB_API int lsb_branch_max() { return kMaxBranches; }

// out = sum over the branches of scale_b * y_b, summed in 32-bit (branches side by side whose results
// are added with fixed factors, no norm).
struct BranchScales { float s[kMaxBranches]; };

template <typename T>
__global__ void branch_sum_kernel(Branches br, BranchScales sc, T* __restrict__ out, long long count) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int b = 0; b < kMaxBranches; ++b)
            if (b < br.n) s += sc.s[b] * lsb_to_float(((const T*)br.y[b])[i]);
        out[i] = lsb_from_float<T>(s);
    }
}

LSB_API int lsb_branch_sum(const void* const* ys, const float* scales, int n, void* out, int dtype, int n_rows, int hidden,
                           cudaStream_t stream) {
    const long long count = (long long)n_rows * hidden;
    if (count <= 0) return 0;
    if (n <= 0 || n > kMaxBranches) return (int)cudaErrorInvalidValue;
    Branches br;
    BranchScales sc;
    br.n = n;
    for (int b = 0; b < kMaxBranches; ++b) {
        br.y[b] = b < n ? ys[b] : nullptr;
        br.w[b] = nullptr;
        sc.s[b] = b < n ? scales[b] : 0.f;
    }
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(branch_sum_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, 1, br, sc, (T*)out, count));
    return 0;
}

// ys, ws: n pointers each (rows of the branches in the compute dtype, their 32-bit weights).
LSB_API int lsb_branch_mean(const void* const* ys, const float* const* ws, int n, float eps, void* out, int dtype,
                            int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n <= 0 || n > kMaxBranches || hidden <= 0) return (int)cudaErrorInvalidValue;
    Branches br;
    br.n = n;
    for (int b = 0; b < kMaxBranches; ++b) {
        br.y[b] = b < n ? ys[b] : nullptr;
        br.w[b] = b < n ? ws[b] : nullptr;
    }
    bool vec = hidden % 4 == 0 && hidden <= kBranchRegs * 4 * kRowThreads && (uintptr_t)out % 16 == 0;
    for (int b = 0; b < n; ++b) vec = vec && (uintptr_t)ys[b] % 16 == 0 && (uintptr_t)ws[b] % 16 == 0;
    LSB_DISPATCH_DTYPE(dtype, {
        if (vec) return lsb_launch(branch_mean_vec4_kernel<T>, dim3(n_rows), dim3(kRowThreads), 0, stream, 1, br, eps, (T*)out, hidden);
        return lsb_launch(branch_mean_kernel<T>, dim3(n_rows), dim3(kRowThreads), 0, stream, 1, br, eps, (T*)out, hidden);
    });
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The same stream with centred norms that carry a weight and a bias (layer norm):
//
//     x <- x + mult * (cn(y) * w_post + b_post)        out = cn(x) * w_next + b_next
//
// with cn(z) = (z - mean z) / sqrt(mean((z - mean z)^2) + eps).  The mean is taken first and the
// variance from the deviations (two passes over the row in shared memory), all in 32-bit.
template <int V, typename T> struct RowIo;
template <typename T> struct RowIo<1, T> {
    static __device__ __forceinline__ void load(const T* p, float* v) { v[0] = lsb_to_float(p[0]); }
    static __device__ __forceinline__ void store(T* p, const float* v) { p[0] = lsb_from_float<T>(v[0]); }
};
template <typename T> struct RowIo<4, T> {
    static __device__ __forceinline__ void load(const T* p, float* v) {
        const float4 x = row_load4(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(T* p, const float* v) { row_store4(p, make_float4(v[0], v[1], v[2], v[3])); }
};

// mean and 1 / sqrt(variance + eps) of the row in shared memory
template <int V>
__device__ __forceinline__ void centred_stats(const float* row_sh, int hidden, float sum, float eps, float* scratch,
                                              float& mean, float& inv) {
    mean = lsb_block_sum(sum, scratch) / (float)hidden;
    float ss = 0.f;
    for (int i = V * threadIdx.x; i < hidden; i += V * kRowThreads) {
        float v[V];
        RowIo<V, float>::load(row_sh + i, v);
#pragma unroll
        for (int u = 0; u < V; ++u) ss += (v[u] - mean) * (v[u] - mean);
    }
    inv = rsqrtf(lsb_block_sum(ss, scratch) / (float)hidden + eps);
}

template <typename T, bool GATHER, int V>
__global__ void __launch_bounds__(kRowThreads)
stream_centred_norm_kernel(float* __restrict__ residual, const T* __restrict__ y, const float* __restrict__ post_w,
                           const float* __restrict__ post_b, float post_eps, float mult, const int* __restrict__ rows,
                           const float* __restrict__ next_w, const float* __restrict__ next_b, float next_eps,
                           T* __restrict__ out, int hidden, int n_rows_total) {
    extern __shared__ float row_sh[];
    __shared__ float scratch[33];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r_out = blockIdx.x;
    int r_in = r_out;
    if (GATHER) {
        r_in = rows[r_out];
        if (r_in < 0 || r_in >= n_rows_total) {
            if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW);
            if (out)
                for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)r_out * hidden + i] = lsb_from_float<T>(0.f);
            return;
        }
    }
    float* res = residual + (size_t)r_in * hidden;
    const T* yr = y ? y + (size_t)r_in * hidden : nullptr;
    float mean_y = 0.f, inv_y = 1.f;
    if (yr && post_w) {
        float s = 0.f;
        for (int i = V * threadIdx.x; i < hidden; i += V * kRowThreads) {
            float v[V];
            RowIo<V, T>::load(yr + i, v);
            RowIo<V, float>::store(row_sh + i, v);
#pragma unroll
            for (int u = 0; u < V; ++u) s += v[u];
        }
        centred_stats<V>(row_sh, hidden, s, post_eps, scratch, mean_y, inv_y);
    }
    float sum = 0.f;
    for (int i = V * threadIdx.x; i < hidden; i += V * kRowThreads) {
        float x[V];
        RowIo<V, float>::load(res + i, x);
        if (yr) {
            float v[V];
            if (post_w) {
                float w[V], b[V];
                RowIo<V, float>::load(row_sh + i, v);
                RowIo<V, float>::load(post_w + i, w);
                RowIo<V, float>::load(post_b + i, b);
#pragma unroll
                for (int u = 0; u < V; ++u) x[u] += mult * ((v[u] - mean_y) * inv_y * w[u] + b[u]);
            } else {
                RowIo<V, T>::load(yr + i, v);
#pragma unroll
                for (int u = 0; u < V; ++u) x[u] += mult * v[u];
            }
            if (!GATHER) RowIo<V, float>::store(res + i, x);
        }
        RowIo<V, float>::store(row_sh + i, x);
#pragma unroll
        for (int u = 0; u < V; ++u) sum += x[u];
    }
    if (!out) return;
    float mean, inv;
    centred_stats<V>(row_sh, hidden, sum, next_eps, scratch, mean, inv);
    T* o = out + (size_t)r_out * hidden;
    for (int i = V * threadIdx.x; i < hidden; i += V * kRowThreads) {
        float x[V], w[V], b[V];
        RowIo<V, float>::load(row_sh + i, x);
        RowIo<V, float>::load(next_w + i, w);
        RowIo<V, float>::load(next_b + i, b);
#pragma unroll
        for (int u = 0; u < V; ++u) x[u] = (x[u] - mean) * inv * w[u] + b[u];
        RowIo<V, T>::store(o + i, x);
    }
}

// y, (post_w, post_b) and (next_w, next_b, out) may each be null (post_w null with y given: a plain sum of
// mult * y).  rows null: every row of the stream, in place; else the rows named, the stream untouched.
LSB_API int lsb_stream_centred_norm(float* residual, const void* y, const float* post_w, const float* post_b,
                                    float post_eps, float mult, const int* rows, int n_rows, const float* next_w,
                                    const float* next_b, float next_eps, void* out, int dtype, int n_rows_total,
                                    int hidden, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (hidden <= 0 || (out && !(next_w && next_b)) || (post_w && !post_b)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    bool vec = hidden % 4 == 0;
    for (const void* ptr : {(const void*)residual, y, (const void*)post_w, (const void*)post_b, (const void*)next_w,
                            (const void*)next_b, (const void*)out})
        vec = vec && ((uintptr_t)ptr % 16 == 0);
#define LSB_CENTRED_NORM(G, V)                                                                                     \
    do {                                                                                                           \
        if (smem > 48 * 1024) {                                                                                    \
            int rc = (int)cudaFuncSetAttribute(stream_centred_norm_kernel<T, G, V>,                                \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
            if (rc) return rc;                                                                                     \
        }                                                                                                          \
        return lsb_launch(stream_centred_norm_kernel<T, G, V>, dim3(n_rows), dim3(kRowThreads), smem, stream, 1,   \
                          residual, (const T*)y, post_w, post_b, post_eps, mult, rows, next_w, next_b, next_eps,   \
                          (T*)out, hidden, n_rows_total);                                                          \
    } while (0)
    LSB_DISPATCH_DTYPE(dtype, {
        if (vec && rows) LSB_CENTRED_NORM(true, 4);
        else if (vec) LSB_CENTRED_NORM(false, 4);
        else if (rows) LSB_CENTRED_NORM(true, 1);
        else LSB_CENTRED_NORM(false, 1);
    });
#undef LSB_CENTRED_NORM
    return 0;
}
