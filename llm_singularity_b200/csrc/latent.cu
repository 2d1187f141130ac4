// Attention over a cached latent: every token keeps one row [kv_rank + rot_dim] in a paged
// cache, the normed latent c followed by a rotated key part that all heads share.  A head's
// unrotated key is W_uk c and its value W_uv c; neither is ever formed.  The query's unrotated
// part is carried through W_uk instead (q' = W_uk^T q, kv_rank wide), so that the score is
// (q' . c + q_rot . k_rot) * scale, and the value product follows the weighted sum of latents:
// o = W_uv (sum_j p_j c_j).  All heads therefore read the same rows, one "key head" of width
// kv_rank + rot_dim whose first kv_rank dims are also the values.
//
//   latent_prep       per token: c_q = rmsnorm(down[:q_rank]) * w_q  -> T;  for layers that write
//                     the cache: c = rmsnorm(down[q_rank : q_rank + kv_rank]) * w_kv and the last
//                     rot_dim values rotated by the token's position -> the token's cache row.
//   latent_query_rot  the rotated part of each head's query -> qf[t, h, kv_rank:], 32-bit.
//   batched_nt        C[m, b, :] = A[m, b, :] B[b]^T for every head b (32-bit accumulation): the
//                     query's trip through W_uk, and the value product through W_uv.
//   latent_attention  causal softmax attention of the step's rows over their requests' cache rows.
//
// Rotation: dims (2i, 2i+1) of the rotated part turn by pos * inv_freq[i] for i < rot_dims / 2
// (pairing 1), or dims (i, i + rot_dims/2) (pairing 0); dims from rot_dims on pass unchanged.
// Norms, angles, scores, softmax and the weighted sums are 32-bit.
#include "common.cuh"

#include <float.h>

LSB_DEFINE_STATUS()

constexpr int kPrepThreads = 128;

__device__ __forceinline__ void rotate_write(const float* in, float* out, int n, int rot_dims,
                                             int pairing, float pos, const float* inv_freq, int i) {
    // element i of out (i < n)
    if (i >= rot_dims) { out[i] = in[i]; return; }
    const int half = rot_dims / 2;
    int pair, other;
    bool first;
    if (pairing == 1) { pair = i >> 1; first = !(i & 1); other = first ? i + 1 : i - 1; }
    else { pair = i < half ? i : i - half; first = i < half; other = first ? i + half : i - half; }
    float s, c;
    sincosf(pos * inv_freq[pair], &s, &c);
    out[i] = first ? in[i] * c - in[other] * s : in[i] * c + in[other] * s;
}

template <typename T>
__global__ void __launch_bounds__(kPrepThreads)
latent_prep_kernel(const float* __restrict__ down, long long ld, int q_rank, int kv_rank, int rot_dim,
                   const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                   const float* __restrict__ inv_freq, int rot_dims, int pairing,
                   const int* __restrict__ positions, const int* __restrict__ token_req,
                   const int* __restrict__ table_rows, const int* __restrict__ block_table,
                   int table_stride, T* __restrict__ pages, int page_size, int num_pages,
                   T* __restrict__ cq, int write) {
    extern __shared__ float sh[];
    float* scratch = sh;                 // 33
    float* rot_in = sh + 33;             // rot_dim
    float* rot_out = rot_in + rot_dim;   // rot_dim
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t t = blockIdx.x;
    const float* row = down + t * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss += row[i] * row[i];
    ss = lsb_block_sum(ss, scratch);
    float f = 1.f / sqrtf(ss / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
        cq[t * q_rank + i] = lsb_from_float<T>(row[i] * f * wq[i]);
    if (!write) return;
    const int pos = positions[t];
    const int page = block_table[(size_t)table_rows[token_req[t]] * table_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) lsb_set_status(LSB_BAD_PAGE);
        return;
    }
    T* dst = pages + ((size_t)page * page_size + pos % page_size) * (kv_rank + rot_dim);
    const float* lat = row + q_rank;
    ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) ss += lat[i] * lat[i];
    ss = lsb_block_sum(ss, scratch);
    f = 1.f / sqrtf(ss / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = lsb_from_float<T>(lat[i] * f * wkv[i]);
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) rot_in[i] = lat[kv_rank + i];
    __syncthreads();
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x)
        rotate_write(rot_in, rot_out, rot_dim, rot_dims, pairing, (float)pos, inv_freq, i);
    __syncthreads();
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) dst[kv_rank + i] = lsb_from_float<T>(rot_out[i]);
}

// q: [T, heads * (plain + rot_dim)] 32-bit; qf: [T, heads, kv_rank + rot_dim] 32-bit
__global__ void latent_query_rot_kernel(const float* __restrict__ q, float* __restrict__ qf, int heads,
                                        int plain, int rot_dim, int kv_rank, int rot_dims, int pairing,
                                        const float* __restrict__ inv_freq, const int* __restrict__ positions) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const size_t t = blockIdx.x;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < heads * rot_dim; i += blockDim.x) {
        const int h = i / rot_dim, j = i % rot_dim;
        const float* in = q + (t * heads + h) * (size_t)(plain + rot_dim) + plain;
        float* out = qf + (t * heads + h) * (size_t)(kv_rank + rot_dim) + kv_rank;
        rotate_write(in, out, rot_dim, rot_dims, pairing, pos, inv_freq, j);
    }
}

// ---------------------------------------------------------------------- batched product
// C[m, b, n] = sum_k A[m, b, k] * B[b, n, k]; A rows lda apart, batches a_bs apart (elements), the
// same for C; B is [batch, N, K] dense.  32 x 32 output tile per block, K in slabs of 32.
constexpr int kBt = 32;

template <typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256)
batched_nt_kernel(const TA* __restrict__ A, long long lda, long long a_bs, const TB* __restrict__ B,
                  TC* __restrict__ C, long long ldc, long long c_bs, int M, int N, int K) {
    __shared__ float As[kBt][kBt + 1];
    __shared__ float Bs[kBt][kBt + 1];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int b = blockIdx.z;
    const int m0 = blockIdx.y * kBt, n0 = blockIdx.x * kBt;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;     // ty in [0, 8): rows ty, ty+8, ...
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += kBt) {
        for (int i = ty; i < kBt; i += 8) {
            const int m = m0 + i, n = n0 + i, k = k0 + tx;
            As[i][tx] = (m < M && k < K) ? lsb_to_float(A[(size_t)m * lda + (size_t)b * a_bs + k]) : 0.f;
            Bs[i][tx] = (n < N && k < K) ? lsb_to_float(B[((size_t)b * N + n) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kBt; ++k) {
            const float bv = Bs[tx][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] += As[ty + 8 * j][k] * bv;
        }
        __syncthreads();
    }
    const int n = n0 + tx;
    if (n < N) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty + 8 * j;
            if (m < M) C[(size_t)m * ldc + (size_t)b * c_bs + n] = lsb_from_float<TC>(acc[j]);
        }
    }
}

// ---------------------------------------------------------------------------- attention
// One warp owns a (row, head).  Lanes split the keys of a 32-key chunk for the scores and split
// the latent dims for the weighted sum.  qf rows are [kv_rank + rot_dim]; a cache row has the
// same width and its first kv_rank dims are the values.
constexpr int kLatWarps = 4;
constexpr int kLatAccs = 32;            // kv_rank up to 32 * 32

template <typename T>
__global__ void __launch_bounds__(kLatWarps * 32)
latent_attention_kernel(const float* __restrict__ qf, const T* __restrict__ pages,
                        const int* __restrict__ q_start, const int* __restrict__ kv_len_arr,
                        const int* __restrict__ table_rows, const int* __restrict__ block_table,
                        int table_stride, T* __restrict__ out, int heads, int kv_rank, int rot_dim,
                        int page_size, int num_pages, float scale) {
    extern __shared__ float q_sh[];                          // [kLatWarps][kv_rank + rot_dim]
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.z, h = blockIdx.y;
    const int width = kv_rank + rot_dim;
    const int qs = q_start[r];
    const int q_len = q_start[r + 1] - qs;
    const int i = blockIdx.x * kLatWarps + warp;
    if (i >= q_len) return;
    const int kv_len = kv_len_arr[r];
    const int p = kv_len - q_len + i;
    const int t = qs + i;
    const int* bt = block_table + (size_t)table_rows[r] * table_stride;
    float* qw = q_sh + warp * width;
    const float* q = qf + ((size_t)t * heads + h) * width;
    for (int d = lane; d < width; d += 32) qw[d] = q[d] * scale;
    __syncwarp();

    float acc[kLatAccs];
#pragma unroll
    for (int c = 0; c < kLatAccs; ++c) acc[c] = 0.f;
    float m = -FLT_MAX, l = 0.f;
    for (int base = 0; base <= p; base += 32) {
        const int kj = base + lane;
        float s = -FLT_MAX;
        long long off = -1;
        if (kj <= p) {
            const int page = bt[kj / page_size];
            if (page < 0 || page >= num_pages) {
                lsb_set_status(LSB_BAD_PAGE);
            } else {
                off = ((long long)page * page_size + (kj % page_size)) * width;
                const T* k = pages + off;
                s = 0.f;
                for (int d = 0; d < width; ++d) s += qw[d] * lsb_to_float(k[d]);
            }
        }
        const float m_new = fmaxf(m, lsb_warp_max(s));
        const float corr = expf(m - m_new);
        const float pj = (off >= 0) ? expf(s - m_new) : 0.f;
        l = l * corr + lsb_warp_sum(pj);
#pragma unroll
        for (int c = 0; c < kLatAccs; ++c) acc[c] *= corr;
        const int n_valid = min(32, p - base + 1);
        for (int j = 0; j < n_valid; ++j) {
            const float w = __shfl_sync(0xffffffffu, pj, j);
            const long long voff = __shfl_sync(0xffffffffu, off, j);
            if (voff < 0) continue;
            const T* v = pages + voff;
#pragma unroll
            for (int c = 0; c < kLatAccs; ++c) {
                const int d = lane + 32 * c;
                if (d < kv_rank) acc[c] += w * lsb_to_float(v[d]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* o = out + ((size_t)t * heads + h) * kv_rank;
#pragma unroll
    for (int c = 0; c < kLatAccs; ++c) {
        const int d = lane + 32 * c;
        if (d < kv_rank) o[d] = lsb_from_float<T>(acc[c] * inv);
    }
}

// ------------------------------------------------------------------------------- entries
LSB_API int lsb_latent_prep(const float* down, long long ld, int n_tokens, int q_rank, int kv_rank,
                            int rot_dim, const float* wq, const float* wkv, float eps,
                            const float* inv_freq, int rot_dims, int pairing, const int* positions,
                            const int* token_req, const int* table_rows, const int* block_table,
                            int table_stride, void* pages, int dtype, int page_size, int num_pages,
                            void* cq, int write, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (q_rank <= 0 || (write && (kv_rank <= 0 || rot_dim < 0 || rot_dims > rot_dim || rot_dims % 2)))
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(33 + 2 * (rot_dim > 0 ? rot_dim : 1)) * sizeof(float);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
        latent_prep_kernel<T>, dim3(n_tokens), dim3(kPrepThreads), smem, stream, 1, down, ld, q_rank,
        kv_rank, rot_dim, wq, wkv, eps, inv_freq, rot_dims, pairing, positions, token_req, table_rows,
        block_table, table_stride, (T*)pages, page_size, num_pages, (T*)cq, write));
    return 0;
}

LSB_API int lsb_latent_query_rot(const float* q, float* qf, int n_tokens, int heads, int plain,
                                 int rot_dim, int kv_rank, int rot_dims, int pairing,
                                 const float* inv_freq, const int* positions, cudaStream_t stream) {
    if (n_tokens <= 0 || rot_dim <= 0) return 0;
    if (rot_dims > rot_dim || rot_dims % 2) return (int)cudaErrorInvalidValue;
    return lsb_launch(latent_query_rot_kernel, dim3(n_tokens), dim3(128), 0, stream, 1, q, qf, heads,
                      plain, rot_dim, kv_rank, rot_dims, pairing, inv_freq, positions);
}

// types: 0 = 32-bit, 1 = bfloat16, for A, B and C in turn
LSB_API int lsb_batched_nt(const void* A, int ta, long long lda, long long a_bs, const void* B, int tb,
                           void* C, int tc, long long ldc, long long c_bs, int M, int N, int K,
                           int batch, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (K <= 0 || batch > 65535 || (M + kBt - 1) / kBt > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((N + kBt - 1) / kBt, (M + kBt - 1) / kBt, batch);
#define LSB_BNT(TA, TB, TC)                                                                           \
    return lsb_launch(batched_nt_kernel<TA, TB, TC>, grid, dim3(256), 0, stream, 1, (const TA*)A, lda, \
                      a_bs, (const TB*)B, (TC*)C, ldc, c_bs, M, N, K)
    typedef __nv_bfloat16 bf;
    if (ta == 0 && tb == 0 && tc == 0) LSB_BNT(float, float, float);
    if (ta == 0 && tb == 1 && tc == 0) LSB_BNT(float, bf, float);
    if (ta == 1 && tb == 1 && tc == 0) LSB_BNT(bf, bf, float);
    if (ta == 1 && tb == 1 && tc == 1) LSB_BNT(bf, bf, bf);
    if (ta == 0 && tb == 1 && tc == 1) LSB_BNT(float, bf, bf);
#undef LSB_BNT
    return (int)cudaErrorInvalidValue;
}

LSB_API int lsb_latent_attention(const float* qf, const void* pages, int dtype, const int* q_start,
                                 const int* kv_len, const int* table_rows, const int* block_table,
                                 int table_stride, void* out, int n_requests, int max_q_len, int heads,
                                 int kv_rank, int rot_dim, int page_size, int num_pages, float scale,
                                 cudaStream_t stream) {
    if (n_requests <= 0 || max_q_len <= 0) return 0;
    if (kv_rank <= 0 || kv_rank > 32 * kLatAccs || rot_dim < 0 || heads <= 0 || heads > 65535 ||
        n_requests > 65535)
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)kLatWarps * (kv_rank + rot_dim) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    dim3 grid((max_q_len + kLatWarps - 1) / kLatWarps, heads, n_requests);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
        latent_attention_kernel<T>, grid, dim3(kLatWarps * 32), smem, stream, 1, qf, (const T*)pages,
        q_start, kv_len, table_rows, block_table, table_stride, (T*)out, heads, kv_rank, rot_dim,
        page_size, num_pages, scale));
    return 0;
}

// A gate of one number per head on the heads' outputs, in place: x[t, h, :] *= sigmoid(gate[t, h]), the
// gate numbers 32-bit in rows of `gate_ld` (they come out of the same product as the latents).
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const float* __restrict__ gate, long long gate_ld, int heads,
                                 int dim, long long total) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long th = i / dim;
        const long long t = th / heads;
        const int h = (int)(th - t * heads);
        const float g = 1.f / (1.f + expf(-gate[t * gate_ld + h]));
        x[i] = lsb_from_float<T>(lsb_to_float(x[i]) * g);
    }
}

LSB_API int lsb_head_gate(void* x, int dtype, const float* gate, long long gate_ld, int tokens, int heads, int dim,
                          cudaStream_t stream) {
    const long long total = (long long)tokens * heads * dim;
    if (total <= 0) return 0;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(head_gate_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, 1, (T*)x, gate,
                                                gate_ld, heads, dim, total));
    return 0;
}
