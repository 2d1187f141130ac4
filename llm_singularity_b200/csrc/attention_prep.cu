// What happens to queries, keys and values between their projection and the attention itself,
// for mixers whose key size and value size may differ, as one kernel per step:
//
//   * a bias per channel (q, k, v), added in 32-bit;
//   * a norm per head of q and of k: z / sqrt(mean(z^2) + eps) * w, one weight of head size for
//     all heads of q and one for all heads of k; or (`norm_all`) one norm over all heads of q at
//     once and one over all heads of k, with weights as long as the whole projection;
//   * each value head divided by its root mean square (`v_unit`: no weight, the same eps);
//   * values mixed with those another layer made of the same token in this step (`v_first`, rows of
//     `v_first_ld` elements in the compute dtype): v <- (1 - lambda) v + lambda v_first, lambda one
//     32-bit number on the device; the mixed values are what is cached;
//   * a query temperature: q *= 1 + coef * ln(floor((pos + 1) / every) + 1);
//   * rotation of the first `rotary_dim` dims of every q and k head by pos * inv_freq[i], pairs
//     (2i, 2i + 1) ("adjacent") or (i, i + rotary_dim / 2) ("half"), angle formed in 32-bit;
//   * queries go to q_out [tokens, nh * dk]; keys and values to the token's place in the cache
//     pages, [page][kv head][offset][dk] and [page][kv head][offset][dv].
//
// Each of the first four is optional.  The projections come as rows of one matrix, q at q_off, k
// at k_off, v at v_off, in the compute dtype.  One block per token: all its query and key channels
// are brought into shared memory in one sweep, then a warp works on a head at a time; a token's
// sines and cosines are formed once and serve all its heads.
#include "common.cuh"

LSB_DEFINE_STATUS()

constexpr int kPrepWarps = 8;
constexpr int kPrepMaxDim = 512;

struct PrepArgs {
    const void* proj; long long ld; int q_off, k_off, v_off;
    int nh, nkv, dk, dv;
    const float *q_bias, *k_bias, *v_bias;
    const float *q_norm, *k_norm; float norm_eps;
    int norm_all, v_unit;
    float temp_coef; int temp_every;
    const float* inv_freq; int rotary_dim, adjacent;
    const int *positions, *token_req, *table_rows, *block_table; int table_stride;
    void *q_out, *k_pages, *v_pages; int page_size, num_pages, store;
    const void* v_first; long long v_first_ld; const float* v_lambda;
    int vec;        // 16-byte loads of the projections: every offset, ld, dk and dv a multiple of 16 bytes
};

// 16 bytes of T as floats
template <typename T> struct PrepVec;
template <> struct PrepVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void widen(const uint4& raw, float (&f)[4]) {
        f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
    }
};
template <> struct PrepVec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void widen(const uint4& raw, float (&f)[8]) {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 v = __bfloat1622float2(p[j]);
            f[2 * j] = v.x;
            f[2 * j + 1] = v.y;
        }
    }
};

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32) attention_prep_kernel(PrepArgs a) {
    extern __shared__ float all_sh[];                   // [(nh + nkv) * dk]
    __shared__ float cs_sh[2][kPrepMaxDim / 2];
    __shared__ float sum_sh[33];
    lsb_pdl_launch_dependents();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // positions are metadata of the step (on the device before its first kernel starts): the
    // temperature and the token's sines and cosines, shared by all its heads, are formed while the
    // projection before this kernel is still running
    const int pos = a.positions[t];
    float temp = 1.f;
    if (a.temp_every > 0) temp = 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.f);
    for (int i = threadIdx.x; i < (a.rotary_dim >> 1); i += blockDim.x)
        sincosf((float)pos * a.inv_freq[i], &cs_sh[1][i], &cs_sh[0][i]);
    __syncthreads();
    const int slot_row = a.store ? a.table_rows[a.token_req[t]] : 0;      // (metadata too)
    lsb_pdl_wait();                                 // (the block table is written by a kernel of this step)
    // the first of the token's query and key channels are asked for before the block table is, so that
    // the two latencies pass together
    const T* row = (const T*)a.proj + (size_t)t * a.ld;
    const int nq = a.nh * a.dk, nall = nq + a.nkv * a.dk;
    constexpr int kAhead = 4, VEC = PrepVec<T>::N;
    T ahead[kAhead];
    uint4 ahead_v[2];
    if (a.vec) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = (threadIdx.x + u * kPrepWarps * 32) * VEC;
            if (i < nall) ahead_v[u] = *reinterpret_cast<const uint4*>(row + (i < nq ? a.q_off + i : a.k_off + i - nq));
        }
    } else {
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const int i = threadIdx.x + u * kPrepWarps * 32;
            if (i < nall) ahead[u] = row[i < nq ? a.q_off + i : a.k_off + i - nq];
        }
    }
    long long k_base = -1, v_base = -1;             // element offsets of (page, head 0, offset, 0)
    if (a.store) {
        const int page_idx = pos / a.page_size;
        int page = -1;
        if (page_idx < a.table_stride) page = a.block_table[(size_t)slot_row * a.table_stride + page_idx];
        if (page < 0 || page >= a.num_pages) {
            if (threadIdx.x == 0) lsb_set_status(LSB_BAD_PAGE);
        } else {
            const long long at = (long long)page * a.nkv * a.page_size + (pos % a.page_size);
            k_base = at * a.dk;
            v_base = at * a.dv;
        }
    }
    const int half_rot = a.rotary_dim >> 1;
    // every query and key channel of the token, with its bias, into shared memory in one sweep (all
    // loads in flight together); the heads are then worked on from there, a warp per head
    auto stage_vec = [&](int i, const uint4& raw) {
        const bool is_q = i < nq;
        const int c = is_q ? i : i - nq;
        float f[VEC];
        PrepVec<T>::widen(raw, f);
        const float* bias = is_q ? a.q_bias : a.k_bias;
#pragma unroll
        for (int e = 0; e < VEC; ++e) all_sh[i + e] = bias ? f[e] + bias[c + e] : f[e];
    };
    if (a.vec) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = (threadIdx.x + u * kPrepWarps * 32) * VEC;
            if (i < nall) stage_vec(i, ahead_v[u]);
        }
        for (int i = (threadIdx.x + 2 * kPrepWarps * 32) * VEC; i < nall; i += kPrepWarps * 32 * VEC)
            stage_vec(i, *reinterpret_cast<const uint4*>(row + (i < nq ? a.q_off + i : a.k_off + i - nq)));
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
        const int i = threadIdx.x + u * kPrepWarps * 32;
        if (!a.vec && i < nall) {
            const bool is_q = i < nq;
            const int c = is_q ? i : i - nq;
            float x = lsb_to_float(ahead[u]);
            const float* bias = is_q ? a.q_bias : a.k_bias;
            if (bias) x += bias[c];
            all_sh[i] = x;
        }
    }
    for (int i = a.vec ? nall : threadIdx.x + kAhead * kPrepWarps * 32; i < nall; i += kPrepWarps * 32) {
        const bool is_q = i < nq;
        const int c = is_q ? i : i - nq;
        float x = lsb_to_float(row[(is_q ? a.q_off : a.k_off) + c]);
        const float* bias = is_q ? a.q_bias : a.k_bias;
        if (bias) x += bias[c];
        all_sh[i] = x;
    }
    __syncthreads();
    float inv_all_q = 1.f, inv_all_k = 1.f;
    if (a.norm_all && a.q_norm) {                       // one mean of squares over all of q, one over all of k
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < nall; i += kPrepWarps * 32) {
            const float x = all_sh[i];
            if (i < nq) sq += x * x;
            else sk += x * x;
        }
        inv_all_q = rsqrtf(lsb_block_sum(sq, sum_sh) / (float)nq + a.norm_eps);
        inv_all_k = rsqrtf(lsb_block_sum(sk, sum_sh) / (float)(nall - nq) + a.norm_eps);
    }
    for (int head = warp; head < a.nh + a.nkv; head += kPrepWarps) {
        const bool is_q = head < a.nh;
        const int hh = is_q ? head : head - a.nh;
        const float* hs = all_sh + (size_t)head * a.dk;
        const float* nw = is_q ? a.q_norm : a.k_norm;
        if (nw && a.norm_all) nw += (size_t)hh * a.dk;
        float inv = 1.f;
        if (nw && a.norm_all) {
            inv = is_q ? inv_all_q : inv_all_k;
        } else if (nw) {
            float ss = 0.f;
            for (int d = lane; d < a.dk; d += 32) ss += hs[d] * hs[d];
            inv = rsqrtf(lsb_warp_sum(ss) / (float)a.dk + a.norm_eps);
        }
        const float mul = is_q ? temp : 1.f;
        T* dst = nullptr;
        if (is_q) dst = (T*)a.q_out + ((size_t)t * a.nh + hh) * a.dk;
        else if (k_base >= 0) dst = (T*)a.k_pages + k_base + (long long)hh * a.page_size * a.dk;
        if (dst) {
            // work items: pairs of dims; the rotating pairs first, then the rest two by two
            const int pairs = (a.dk + 1) >> 1;
            for (int i = lane; i < pairs; i += 32) {
                int ia, ib;
                if (i < half_rot) {
                    ia = a.adjacent ? 2 * i : i;
                    ib = a.adjacent ? 2 * i + 1 : i + half_rot;
                } else {
                    ia = a.rotary_dim + 2 * (i - half_rot);
                    ib = ia + 1;
                }
                float x0 = hs[ia] * (nw ? inv * nw[ia] : 1.f) * mul;
                float x1 = ib < a.dk ? hs[ib] * (nw ? inv * nw[ib] : 1.f) * mul : 0.f;
                if (i < half_rot) {
                    const float c = cs_sh[0][i], s = cs_sh[1][i];
                    const float r0 = x0 * c - x1 * s, r1 = x1 * c + x0 * s;
                    x0 = r0;
                    x1 = r1;
                }
                if (ib == ia + 1 && ib < a.dk && (((uintptr_t)(dst + ia)) & (2 * sizeof(T) - 1)) == 0) {
                    if constexpr (sizeof(T) == 2) *reinterpret_cast<__nv_bfloat162*>(dst + ia) = __floats2bfloat162_rn(x0, x1);
                    else *reinterpret_cast<float2*>(dst + ia) = make_float2(x0, x1);
                } else {
                    dst[ia] = lsb_from_float<T>(x0);
                    if (ib < a.dk) dst[ib] = lsb_from_float<T>(x1);
                }
            }
        }
    }
    if (v_base >= 0 && a.v_unit) {
        const T* v = row + a.v_off;
        for (int head = warp; head < a.nkv; head += kPrepWarps) {
            float ss = 0.f;
            for (int d = lane; d < a.dv; d += 32) {
                float x = lsb_to_float(v[head * a.dv + d]);
                if (a.v_bias) x += a.v_bias[head * a.dv + d];
                ss += x * x;
            }
            const float inv = rsqrtf(lsb_warp_sum(ss) / (float)a.dv + a.norm_eps);
            for (int d = lane; d < a.dv; d += 32) {
                float x = lsb_to_float(v[head * a.dv + d]);
                if (a.v_bias) x += a.v_bias[head * a.dv + d];
                ((T*)a.v_pages)[v_base + (long long)head * a.page_size * a.dv + d] = lsb_from_float<T>(x * inv);
            }
        }
    } else if (v_base >= 0 && a.vec && !a.v_bias && !a.v_first) {
        const T* v = row + a.v_off;
        for (int w = threadIdx.x * VEC; w < a.nkv * a.dv; w += blockDim.x * VEC) {
            const int head = w / a.dv, d = w - head * a.dv;
            *reinterpret_cast<uint4*>((T*)a.v_pages + v_base + (long long)head * a.page_size * a.dv + d) =
                *reinterpret_cast<const uint4*>(v + w);
        }
    } else if (v_base >= 0) {
        const T* v = row + a.v_off;
        for (int w = threadIdx.x; w < a.nkv * a.dv; w += blockDim.x) {
            const int head = w / a.dv, d = w - head * a.dv;
            float x = lsb_to_float(v[w]);
            if (a.v_bias) x += a.v_bias[w];
            if (a.v_first) {
                const float lam = a.v_lambda[0];
                x = (1.f - lam) * x + lam * lsb_to_float(((const T*)a.v_first)[(size_t)t * a.v_first_ld + w]);
            }
            ((T*)a.v_pages)[v_base + (long long)head * a.page_size * a.dv + d] = lsb_from_float<T>(x);
        }
    }
}

LSB_API int lsb_attention_prep_max_dim() { return kPrepMaxDim; }

LSB_API int lsb_attention_prep(const void* proj, int dtype, long long ld, int q_off, int k_off, int v_off, int tokens,
                               int nh, int nkv, int dk, int dv, const float* q_bias, const float* k_bias,
                               const float* v_bias, const float* q_norm, const float* k_norm, float norm_eps,
                               int norm_all, int v_unit, float temp_coef, int temp_every, const float* inv_freq, int rotary_dim, int adjacent,
                               const int* positions, const int* token_req, const int* table_rows,
                               const int* block_table, int table_stride, void* q_out, void* k_pages, void* v_pages,
                               int page_size, int num_pages, int store, const void* v_first, long long v_first_ld,
                               const float* v_lambda, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (dk <= 0 || dk > kPrepMaxDim || dv <= 0 || nh <= 0 || nkv <= 0 || rotary_dim % 2 || rotary_dim > dk ||
        rotary_dim < 0 || (rotary_dim > 0 && !inv_freq) || (v_first && (!v_lambda || v_unit)))
        return (int)cudaErrorInvalidValue;
    PrepArgs a;
    a.proj = proj; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.nh = nh; a.nkv = nkv; a.dk = dk; a.dv = dv;
    a.q_bias = q_bias; a.k_bias = k_bias; a.v_bias = v_bias;
    a.q_norm = q_norm; a.k_norm = k_norm; a.norm_eps = norm_eps;
    a.norm_all = norm_all; a.v_unit = v_unit;
    a.temp_coef = temp_coef; a.temp_every = temp_every;
    a.inv_freq = inv_freq; a.rotary_dim = rotary_dim; a.adjacent = adjacent;
    a.positions = positions; a.token_req = token_req; a.table_rows = table_rows; a.block_table = block_table;
    a.table_stride = table_stride;
    a.q_out = q_out; a.k_pages = k_pages; a.v_pages = v_pages; a.page_size = page_size; a.num_pages = num_pages;
    a.store = store;
    a.v_first = v_first; a.v_first_ld = v_first_ld; a.v_lambda = v_lambda;
    const int per16 = dtype == LSB_F32 ? 4 : 8;
    a.vec = ((uintptr_t)proj % 16 == 0 && (uintptr_t)v_pages % 16 == 0 && ld % per16 == 0 && q_off % per16 == 0 &&
             k_off % per16 == 0 && v_off % per16 == 0 && dk % per16 == 0 && dv % per16 == 0) ? 1 : 0;
    const size_t smem = (size_t)(nh + nkv) * dk * sizeof(float);
    if (smem > 160 * 1024) return (int)cudaErrorInvalidValue;
    LSB_DISPATCH_DTYPE(dtype, {
        if (smem > 32 * 1024) {
            int rc = (int)cudaFuncSetAttribute(attention_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (rc) return rc;
        }
        return lsb_launch(attention_prep_kernel<T>, dim3(tokens), dim3(kPrepWarps * 32), smem, stream, 1, a);
    });
    return 0;
}
