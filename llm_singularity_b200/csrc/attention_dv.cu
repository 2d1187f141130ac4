// Softmax attention over the paged cache for mixers whose keys and values have sizes of their own
// (dk for queries and keys, dv for values) and whose mask may be cut into chunks:
//
//   query row i of request r sits at position p = kv_len - q_len + i and sees the keys at
//   positions [lo, p], lo = max(window > 0 ? p - window + 1 : 0, chunk > 0 ? (p / chunk) * chunk : 0)
//
// (chunks are counted from position 0 of the sequence, wherever a prompt was cut).  Query head h
// reads kv head h / (nh / nkv); scores (q . k) * scale; softmax by running maximum and sum; the
// weighted sum of values is divided by the sum at the end and, if a gate is given, multiplied by
// sigmoid(gate[t, h * dv + c]) on the way out.  Keys are [page][kv head][offset][dk], values
// [page][kv head][offset][dv].  Scores, weights and sums are 32-bit.  Two options ride in `flags`:
// kDvLinearBias takes slope_h * (p - j) off the score of key j for the query at p, slope_h = 2^(-8 (h + 1) / nh);
// `softcap` > 0 replaces a scaled score s by softcap * tanh(s / softcap) before that.
// kDvSink adds one to the softmax's denominator (a place with score 0 and no value, so a row's weights
// sum to less than one), kDvGateHeads reads one gate number per head, gate[t, h], instead of one per
// output channel.
//
// Generic form (any sizes, 32-bit or bfloat16 storage): one warp owns a (row, head); lanes split
// the keys of a 32-key stretch for the scores and the value dims for the weighted sum.
//
// Tensor-core form (bfloat16, dk and dv multiples of 16 up to 128): a block owns a request, a kv
// head and 64 "rows", a row being (query position, query head of the kv head's group) with the
// head running fastest, so that all heads of a group share every key and value tile that is
// loaded.  Tiles of 64 keys and their values come from the pages into shared memory through
// cp.async, two buffers deep; a warp holds 16 rows' queries as mma.sync A fragments, forms S = Q K^T
// on the tensor cores (m16n8k16, 32-bit accumulators), does the masked softmax with a running
// maximum in registers, and feeds the weights straight back as the A fragments of O += P V.
// A step whose requests bring at most 16 rows each (single tokens: one row per head of the group) gets
// blocks of 16 rows whose four warps work side by side, each on 16 of a tile's 64 keys, merging
// through shared memory at the end; the ring of tiles is then four deep, and where the blocks are
// few a row tile's keys are shared among up to eight blocks whose partial sums a second kernel
// brings together, since such a step waits on memory alone.
#include "common.cuh"

#include <float.h>

LSB_DEFINE_STATUS()

constexpr int kDvWarps = 4;
constexpr int kDvMaxDim = 256;
constexpr int kDvSink = 1, kDvGateHeads = 2, kDvLinearBias = 4;

template <typename T>
__device__ __forceinline__ float dv_dot(const float* __restrict__ q, const T* __restrict__ k, int n, bool vec) {
    float s = 0.f;
    if (vec) {
        if constexpr (sizeof(T) == 4) {
            for (int d = 0; d < n; d += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(k + d);
                s += q[d] * kv.x + q[d + 1] * kv.y + q[d + 2] * kv.z + q[d + 3] * kv.w;
            }
        } else {
            for (int d = 0; d < n; d += 8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
                const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(p[j]);
                    s += q[d + 2 * j] * f.x + q[d + 2 * j + 1] * f.y;
                }
            }
        }
    } else {
        for (int d = 0; d < n; ++d) s += q[d] * lsb_to_float(k[d]);
    }
    return s;
}

template <typename T>
__global__ void __launch_bounds__(kDvWarps * 32)
attention_dv_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                            const int* __restrict__ q_start, const int* __restrict__ kv_len_arr,
                            const int* __restrict__ table_rows, const int* __restrict__ block_table, int table_stride,
                            const T* __restrict__ gate, long long gate_stride, T* __restrict__ out,
                            int nh, int nkv, int dk, int dv, int page_size, int num_pages, float scale, int window,
                            int chunk, int vec, int flags, float softcap) {
    __shared__ float q_sh[kDvWarps][kDvMaxDim];
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.z, h = blockIdx.y;
    const int qs = q_start[r];
    const int q_len = q_start[r + 1] - qs;
    const int i = blockIdx.x * kDvWarps + warp;             // row within the request
    if (i >= q_len) return;                                  // whole warp leaves together
    const int kv_len = kv_len_arr[r];
    const int p = kv_len - q_len + i;
    int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
    const int g = h / (nh / nkv);
    const int t = qs + i;
    const int* bt = block_table + (size_t)table_rows[r] * table_stride;

    const T* qr = q + ((size_t)t * nh + h) * dk;
    for (int d = lane; d < dk; d += 32) q_sh[warp][d] = lsb_to_float(qr[d]) * scale;
    __syncwarp();
    const float slope = (flags & kDvLinearBias) ? exp2f(-8.f * (float)(h + 1) / (float)nh) : 0.f;

    constexpr int kAccs = kDvMaxDim / 32;
    float acc[kAccs];
#pragma unroll
    for (int c = 0; c < kAccs; ++c) acc[c] = 0.f;
    float m = -FLT_MAX, l = 0.f;

    for (int base = lo; base <= p; base += 32) {
        const int kj = base + lane;
        float s = -FLT_MAX;
        long long at = -1;                                   // (page, kv head, offset) as a row number
        if (kj <= p) {
            const int page = bt[kj / page_size];
            if (page < 0 || page >= num_pages) {
                lsb_set_status(LSB_BAD_PAGE);
            } else {
                at = ((long long)page * nkv + g) * page_size + (kj % page_size);
                s = dv_dot<T>(q_sh[warp], k_pages + at * dk, dk, vec != 0);
                if (softcap > 0.f) s = softcap * tanhf(s / softcap);
                s -= slope * (float)(p - kj);
            }
        }
        const float m_new = fmaxf(m, lsb_warp_max(s));
        const float corr = expf(m - m_new);                  // m == -FLT_MAX first: exp(-huge) = 0
        const float pj = (at >= 0) ? expf(s - m_new) : 0.f;
        l = l * corr + lsb_warp_sum(pj);
#pragma unroll
        for (int c = 0; c < kAccs; ++c) acc[c] *= corr;
        const int n_valid = min(32, p - base + 1);
        for (int j = 0; j < n_valid; ++j) {
            const float w = __shfl_sync(0xffffffffu, pj, j);
            const long long vat = __shfl_sync(0xffffffffu, at, j);
            if (vat < 0) continue;
            const T* v = v_pages + vat * dv;
#pragma unroll
            for (int c = 0; c < kAccs; ++c) {
                const int d = lane + 32 * c;
                if (d < dv) acc[c] += w * lsb_to_float(v[d]);
            }
        }
        m = m_new;
    }
    if (flags & kDvSink) l += expf(-m);                      // the sink's weight relative to the maximum (inf: all weights vanish)
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* o = out + ((size_t)t * nh + h) * dv;
    const bool per_head = (flags & kDvGateHeads) != 0;
    const T* gr = gate ? gate + (size_t)t * gate_stride + (per_head ? (size_t)h : (size_t)h * dv) : nullptr;
#pragma unroll
    for (int c = 0; c < kAccs; ++c) {
        const int d = lane + 32 * c;
        if (d < dv) {
            float y = acc[c] * inv;
            if (gr) y *= 1.f / (1.f + expf(-lsb_to_float(gr[per_head ? 0 : d])));
            o[d] = lsb_from_float<T>(y);
        }
    }
}

// ------------------------------------------------------------------ tensor-core form
constexpr int kMmaRows = 64, kMmaKeys = 64, kMmaThreads = 128;

__device__ __forceinline__ void dv_mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void dv_cp_async16(void* dst, const void* src, bool real) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = real ? 16 : 0;                       // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ uint32_t dv_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int DKP, int DVP, int STAGES, bool NARROW>
__global__ void __launch_bounds__(kMmaThreads)
attention_dv_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ q_start,
                        const int* __restrict__ kv_len_arr, const int* __restrict__ table_rows,
                        const int* __restrict__ block_table, int table_stride,
                        const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                        __nv_bfloat16* __restrict__ out, int nh, int nkv, int dk, int dv, int page_size,
                        int num_pages, float scale_log2, int window, int chunk, int ksplit, float* __restrict__ scratch,
                        int flags, float scale, float softcap) {
    constexpr int KS = DKP + 8, VS = DVP + 8;          // row strides in elements: 4 words past a multiple of 32
    extern __shared__ __align__(16) unsigned char dv_smem[];
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(dv_smem);       // [STAGES][64][KS]
    __nv_bfloat16* Vs = Ks + STAGES * kMmaKeys * KS;                     // [STAGES][64][VS]
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r = blockIdx.z, g = blockIdx.y, group = nh / nkv;
    const bool sink = (flags & kDvSink) != 0, per_head = (flags & kDvGateHeads) != 0;
    const int gate_w = per_head ? 1 : dv;              // gate numbers a head has
    const int qs = q_start[r];
    const int q_len = q_start[r + 1] - qs;
    const int rows_total = q_len * group;
    constexpr bool split = NARROW;                     // 16 rows a block, the warps side by side on the keys
    constexpr int NJ = NARROW ? 2 : 8;                 // blocks of 8 keys a warp takes of a tile
    constexpr int NKK = NARROW ? 1 : 4;                // and the same keys as k-steps of 16
    const int block_rows = split ? 16 : kMmaRows;
    // (16-row blocks may share a row tile's keys among `ksplit` blocks, merged by a second kernel)
    const int row_tile = NARROW ? blockIdx.x / ksplit : blockIdx.x, key_part = NARROW ? blockIdx.x % ksplit : 0;
    const int tile_row0 = row_tile * block_rows;
    if (tile_row0 >= rows_total) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tid4 = lane & 3;
    const int kv_len = kv_len_arr[r];
    const int p_base = kv_len - q_len;
    auto lowest = [&](int p) {
        int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
        if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
        return lo;
    };
    const int last_row = min(tile_row0 + block_rows, rows_total) - 1;
    const int last_pos = p_base + last_row / group;
    const int key_lo = lowest(p_base + tile_row0 / group);            // the first key any row of the block sees
    int kt0 = key_lo / kMmaKeys, kt1 = last_pos / kMmaKeys;
    if (NARROW && ksplit > 1) {                       // this block's share of the key tiles (it may be empty)
        const int per = (kt1 - kt0 + ksplit) / ksplit;
        kt0 += key_part * per;
        kt1 = min(kt1, kt0 + per - 1);
    }
    const int* bt = block_table + (size_t)table_rows[r] * table_stride;

    // this thread's two rows (gid and gid + 8 of the warp's slab)
    const int slab = tile_row0 + (split ? 0 : warp * 16);
    const int row_a = slab + gid, row_b = row_a + 8;
    const bool ok_a = row_a < rows_total, ok_b = row_b < rows_total;
    const int pos_a = p_base + row_a / group, pos_b = p_base + row_b / group;
    const int lo_a = lowest(pos_a), lo_b = lowest(pos_b);
    const int h_a = g * group + row_a % group, h_b = g * group + row_b % group;
    const size_t t_a = (size_t)qs + row_a / group, t_b = (size_t)qs + row_b / group;
    const int dk_steps = dk >> 4, dv_blocks = dv >> 3;
    // scores that are capped or carry a bias growing with the distance leave the base-2 form for a moment
    const bool modified = softcap > 0.f || (flags & kDvLinearBias) != 0;
    const float slope_a = (flags & kDvLinearBias) ? exp2f(-8.f * (float)(h_a + 1) / (float)nh) : 0.f;
    const float slope_b = (flags & kDvLinearBias) ? exp2f(-8.f * (float)(h_b + 1) / (float)nh) : 0.f;

    uint32_t qa[DKP / 16][4];
    {
        const __nv_bfloat16* qa_row = q + (t_a * nh + h_a) * dk;
        const __nv_bfloat16* qb_row = q + (t_b * nh + h_b) * dk;
#pragma unroll
        for (int ks = 0; ks < DKP / 16; ++ks) {
            qa[ks][0] = qa[ks][1] = qa[ks][2] = qa[ks][3] = 0u;
            if (ks < dk_steps) {
                const int c = ks * 16 + 2 * tid4;
                if (ok_a) {
                    qa[ks][0] = *reinterpret_cast<const uint32_t*>(qa_row + c);
                    qa[ks][2] = *reinterpret_cast<const uint32_t*>(qa_row + c + 8);
                }
                if (ok_b) {
                    qa[ks][1] = *reinterpret_cast<const uint32_t*>(qb_row + c);
                    qa[ks][3] = *reinterpret_cast<const uint32_t*>(qb_row + c + 8);
                }
            }
        }
    }
    float o[DVP / 8][4];
#pragma unroll
    for (int nb = 0; nb < DVP / 8; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
    float m_a = -FLT_MAX, m_b = -FLT_MAX, l_a = 0.f, l_b = 0.f;

    // Loading: a thread owns half of one key row of a tile (its key chunks, then its value chunks, 16
    // bytes each).  The row's place in the pages is looked up one tile ahead of the copies that need it,
    // so that the block table's latency passes behind the tile being worked on.
    const int my_row = threadIdx.x >> 1, my_half = threadIdx.x & 1;
    // (what `place` returns is not looked at before the copies of the next turn of the loop use it: a
    // branch on the page id here would make every turn wait for the block table)
    constexpr int kNoRow = -2, kPastEnd = -1;          // a page id a request never holds / nothing to load
    auto place = [&](int kt) -> int {
        const int kj = kt * kMmaKeys + my_row;
        // (keys behind every row's window are never looked up: their pages may have gone back to the pool)
        if (kt > kt1 || kj > last_pos || kj < key_lo) return kPastEnd;
        const int page = bt[kj / page_size];
        return page < 0 ? kNoRow : page;
    };
    auto load_tile = [&](int page, int kt, int buf) {
        long long at = -1;
        if (page >= num_pages || page == kNoRow) lsb_set_status(LSB_BAD_PAGE);
        else if (page >= 0) at = ((long long)page * nkv + g) * page_size + ((kt * kMmaKeys + my_row) % page_size);
        __nv_bfloat16* kd = Ks + (buf * kMmaKeys + my_row) * KS;
        __nv_bfloat16* vd = Vs + (buf * kMmaKeys + my_row) * VS;
        const __nv_bfloat16* ksrc = k_pages + (at < 0 ? 0 : at * dk);
        const __nv_bfloat16* vsrc = v_pages + (at < 0 ? 0 : at * dv);
        const int kper = dk >> 3, vper = dv >> 3;
#pragma unroll 4
        for (int c = my_half; c < kper; c += 2) dv_cp_async16(kd + c * 8, ksrc + (at < 0 ? 0 : c * 8), at >= 0);
#pragma unroll 4
        for (int c = my_half; c < vper; c += 2) dv_cp_async16(vd + c * 8, vsrc + (at < 0 ? 0 : c * 8), at >= 0);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    const bool active = split || slab < rows_total;    // a warp whose slab lies past the rows only helps loading
    // the padding of the key and value rows (columns past dk and dv) is zeroed once; copies never touch it
    for (int idx = threadIdx.x; idx < STAGES * kMmaKeys; idx += kMmaThreads) {
        for (int c = dk; c < DKP; ++c) Ks[idx * KS + c] = __float2bfloat16_rn(0.f);
        for (int c = dv; c < DVP; ++c) Vs[idx * VS + c] = __float2bfloat16_rn(0.f);
    }
    // a group of copies is committed for every tile slot, real or not, so that the count the wait
    // names is the same in every turn of the loop
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (kt0 + st <= kt1) load_tile(place(kt0 + st), kt0 + st, st);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    int at_next = place(kt0 + STAGES - 1);
    // rows of this warp see every key of a tile that lies wholly between these two
    const int slab_lo = lowest(p_base + min(slab + 15, rows_total - 1) / group), slab_hi = p_base + slab / group;
    const bool slab_full = slab + 15 < rows_total;
    for (int kt = kt0; kt <= kt1; ++kt) {
        const int buf = (kt - kt0) % STAGES;
        if (kt + STAGES - 1 <= kt1) load_tile(at_next, kt + STAGES - 1, (kt - kt0 + STAGES - 1) % STAGES);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        at_next = place(kt + STAGES);
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");
        __syncthreads();
        if (active) {
            // (nothing in the blocks of tensor-core work below depends on a run-time size: the padding
            // of K and of the queries is zero, and the columns of O past dv are never written out, so
            // the compiler is free to keep many independent MMAs in flight)
            const int key0 = NARROW ? warp * 16 : 0;           // this warp's first key of the tile
            const __nv_bfloat16* kb = Ks + (buf * kMmaKeys + key0) * KS;
            const __nv_bfloat16* vb = Vs + (buf * kMmaKeys + key0) * VS;
            float s[NJ][4];
#pragma unroll
            for (int j = 0; j < NJ; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DKP / 16; ++ks) {
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const __nv_bfloat16* krow = kb + (j * 8 + gid) * KS + 2 * tid4 + ks * 16;
                    dv_mma_16816(s[j], qa[ks], *reinterpret_cast<const uint32_t*>(krow),
                                 *reinterpret_cast<const uint32_t*>(krow + 8));
                }
            }
            const int tile_key0 = kt * kMmaKeys + key0;
            const bool interior = slab_full && tile_key0 >= slab_lo && tile_key0 + NJ * 8 - 1 <= slab_hi;
            if (modified) {
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = tile_key0 + j * 8 + 2 * tid4 + (e & 1);
                        const bool ok = e < 2 ? (ok_a && key >= lo_a && key <= pos_a) : (ok_b && key >= lo_b && key <= pos_b);
                        float v = s[j][e] * scale;
                        if (softcap > 0.f) v = softcap * tanhf(v / softcap);
                        v -= e < 2 ? slope_a * (float)(pos_a - key) : slope_b * (float)(pos_b - key);
                        s[j][e] = ok ? v * 1.4426950408889634f : -FLT_MAX;
                    }
                }
            } else if (interior) {
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[j][e] *= scale_log2;
                }
            } else {
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = tile_key0 + j * 8 + 2 * tid4 + (e & 1);
                        const bool ok = e < 2 ? (ok_a && key >= lo_a && key <= pos_a) : (ok_b && key >= lo_b && key <= pos_b);
                        s[j][e] = ok ? s[j][e] * scale_log2 : -FLT_MAX;
                    }
                }
            }
            float mx_a = -FLT_MAX, mx_b = -FLT_MAX;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
                mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float corr_a = exp2f(m_a - mn_a), corr_b = exp2f(m_b - mn_b);
            m_a = mn_a;
            m_b = mn_b;
            float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // (a masked score is -FLT_MAX; while a row has seen no key its maximum is that too)
                    const float pv = s[j][e] > -1e37f ? exp2f(s[j][e] - (e < 2 ? mn_a : mn_b)) : 0.f;
                    s[j][e] = pv;
                    if (e < 2) sum_a += pv;
                    else sum_b += pv;
                }
            }
            l_a = l_a * corr_a + sum_a;
            l_b = l_b * corr_b + sum_b;
#pragma unroll
            for (int nb = 0; nb < DVP / 8; ++nb) {
                o[nb][0] *= corr_a;
                o[nb][1] *= corr_a;
                o[nb][2] *= corr_b;
                o[nb][3] *= corr_b;
            }
#pragma unroll
            for (int kk = 0; kk < NKK; ++kk) {
                uint32_t pa[4];
                pa[0] = dv_pack(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = dv_pack(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = dv_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = dv_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
                const uint32_t vaddr = (uint32_t)__cvta_generic_to_shared(vb + (kk * 16 + (lane & 15)) * VS);
#pragma unroll
                for (int nb = 0; nb < DVP / 8; ++nb) {
                    uint32_t b0, b1;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                                 : "=r"(b0), "=r"(b1) : "r"(vaddr + nb * 16));
                    dv_mma_16816(o[nb], pa, b0, b1);
                }
            }
        }
        __syncthreads();
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    if (split) {
        // every warp holds the same 16 rows over its own keys: merge through shared memory
        float* part = reinterpret_cast<float*>(dv_smem);          // [4][16][DVP + 2]: O, then m and l
        constexpr int PS = DVP + 2;
        float* mine = part + (warp * 16) * PS;
#pragma unroll
        for (int nb = 0; nb < DVP / 8; ++nb) {
            if (nb < dv_blocks) {
                mine[gid * PS + nb * 8 + 2 * tid4] = o[nb][0];
                mine[gid * PS + nb * 8 + 2 * tid4 + 1] = o[nb][1];
                mine[(gid + 8) * PS + nb * 8 + 2 * tid4] = o[nb][2];
                mine[(gid + 8) * PS + nb * 8 + 2 * tid4 + 1] = o[nb][3];
            }
        }
        if (tid4 == 0) {
            mine[gid * PS + DVP] = m_a;
            mine[gid * PS + DVP + 1] = l_a;
            mine[(gid + 8) * PS + DVP] = m_b;
            mine[(gid + 8) * PS + DVP + 1] = l_b;
        }
        __syncthreads();
        const int rows_here = last_row - tile_row0 + 1;
        for (int idx = threadIdx.x; idx < rows_here * dv; idx += kMmaThreads) {
            const int row_l = idx / dv, c = idx - row_l * dv, row = tile_row0 + row_l;
            float mm = -FLT_MAX;
#pragma unroll
            for (int w = 0; w < 4; ++w) mm = fmaxf(mm, part[(w * 16 + row_l) * PS + DVP]);
            float num = 0.f, den = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(part[(w * 16 + row_l) * PS + DVP] - mm);
                num += f * part[(w * 16 + row_l) * PS + c];
                den += f * part[(w * 16 + row_l) * PS + DVP + 1];
            }
            if (ksplit > 1) {                          // sums relative to mm, then mm and the weights' sum
                float* dst = scratch + ((((size_t)r * nkv + g) * (gridDim.x / ksplit) + row_tile) * ksplit + key_part) * 16 * (dv + 2) +
                             (size_t)row_l * (dv + 2);
                dst[c] = num;
                if (c == 0) {
                    dst[dv] = mm;
                    dst[dv + 1] = den;
                }
                continue;
            }
            if (sink) den += exp2f(-mm);
            float y = den > 0.f ? num / den : 0.f;
            const size_t t = (size_t)qs + row / group;
            const int h = g * group + row % group;
            if (gate) y *= 1.f / (1.f + __expf(-__bfloat162float(gate[t * gate_stride + (size_t)h * gate_w + (per_head ? 0 : c)])));
            out[(t * nh + h) * dv + c] = __float2bfloat16_rn(y);
        }
        return;
    }
    if (!active) return;
    if (sink) {
        l_a += exp2f(-m_a);
        l_b += exp2f(-m_b);
    }
    const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
    float gh_a = 1.f, gh_b = 1.f;                      // one gate number per head
    if (gate && per_head) {
        if (ok_a) gh_a = 1.f / (1.f + __expf(-__bfloat162float(gate[t_a * gate_stride + h_a])));
        if (ok_b) gh_b = 1.f / (1.f + __expf(-__bfloat162float(gate[t_b * gate_stride + h_b])));
    }
#pragma unroll
    for (int nb = 0; nb < DVP / 8; ++nb) {
        if (nb < dv_blocks) {
            const int c = nb * 8 + 2 * tid4;
            if (ok_a) {
                float y0 = o[nb][0] * inv_a * gh_a, y1 = o[nb][1] * inv_a * gh_a;
                if (gate && !per_head) {
                    const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + t_a * gate_stride + (size_t)h_a * dv + c));
                    y0 *= 1.f / (1.f + __expf(-gv.x));
                    y1 *= 1.f / (1.f + __expf(-gv.y));
                }
                *reinterpret_cast<__nv_bfloat162*>(out + (t_a * nh + h_a) * dv + c) = __floats2bfloat162_rn(y0, y1);
            }
            if (ok_b) {
                float y0 = o[nb][2] * inv_b * gh_b, y1 = o[nb][3] * inv_b * gh_b;
                if (gate && !per_head) {
                    const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + t_b * gate_stride + (size_t)h_b * dv + c));
                    y0 *= 1.f / (1.f + __expf(-gv.x));
                    y1 *= 1.f / (1.f + __expf(-gv.y));
                }
                *reinterpret_cast<__nv_bfloat162*>(out + (t_b * nh + h_b) * dv + c) = __floats2bfloat162_rn(y0, y1);
            }
        }
    }
}

// The partial sums of `ksplit` blocks that shared a row tile's keys, brought together:
// scratch [request, kv head, row tile, part, 16 rows, dv + 2].
constexpr int kMaxParts = 8;
__global__ void __launch_bounds__(kMmaThreads)
attention_dv_merge_kernel(const float* __restrict__ scratch, const int* __restrict__ q_start,
                          const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                          __nv_bfloat16* __restrict__ out, int nh, int nkv, int dv, int ksplit, int flags) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r = blockIdx.z, g = blockIdx.y, group = nh / nkv;
    const int qs = q_start[r];
    const int rows_total = (q_start[r + 1] - qs) * group;
    const int tile_row0 = blockIdx.x * 16;
    if (tile_row0 >= rows_total) return;
    const int rows_here = min(16, rows_total - tile_row0);
    const float* base = scratch + (((size_t)r * nkv + g) * gridDim.x + blockIdx.x) * ksplit * 16 * (dv + 2);
    for (int idx = threadIdx.x; idx < rows_here * dv; idx += kMmaThreads) {
        const int row_l = idx / dv, c = idx - row_l * dv, row = tile_row0 + row_l;
        // (all parts' values are asked for at once: at most kMaxParts of them)
        float pm[kMaxParts], pl[kMaxParts], pv[kMaxParts];
#pragma unroll
        for (int p = 0; p < kMaxParts; ++p) {
            const float* src = base + ((size_t)(p < ksplit ? p : 0) * 16 + row_l) * (dv + 2);
            pm[p] = p < ksplit ? src[dv] : -FLT_MAX;
            pl[p] = p < ksplit ? src[dv + 1] : 0.f;
            pv[p] = p < ksplit ? src[c] : 0.f;
        }
        float mm = -FLT_MAX;
#pragma unroll
        for (int p = 0; p < kMaxParts; ++p) mm = fmaxf(mm, pm[p]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int p = 0; p < kMaxParts; ++p) {
            const float f = exp2f(pm[p] - mm);
            num += f * pv[p];
            den += f * pl[p];
        }
        if (flags & kDvSink) den += exp2f(-mm);
        float y = den > 0.f ? num / den : 0.f;
        const size_t t = (size_t)qs + row / group;
        const int h = g * group + row % group;
        const bool per_head = (flags & kDvGateHeads) != 0;
        if (gate) y *= 1.f / (1.f + __expf(-__bfloat162float(gate[t * gate_stride + (per_head ? (size_t)h : (size_t)h * dv + c)])));
        out[(t * nh + h) * dv + c] = __float2bfloat16_rn(y);
    }
}

// How a step of this shape is launched: bit 0: 16-row blocks; bit 1: four tiles in flight; bits 8..:
// how many blocks share a row tile's keys.  A function of the shape alone (never of the sequences'
// lengths), so that a captured launch stays valid as sequences grow.  shape: 0 chooses; 1: 64-row
// blocks; 2: 16-row blocks, two tiles in flight; 3: 16-row blocks, four; 4: as 3, keys shared by 3 blocks.
LSB_API int lsb_attention_dv_mma_plan(int n_requests, int max_q_len, int nh, int nkv, int chunk, int sms, int shape) {
    if (sms <= 0) sms = 148;
    const long long rows = (long long)max_q_len * (nh / nkv);
    const long long thin = (rows + 15) / 16 * nkv * n_requests;
    // (16-row blocks for prompt portions were measured too: with the grid small they gain nothing over
    // 64-row blocks, 56 against 49 us for one prompt of 2,048 tokens and four heads, and lose at any size
    // that fills the chip, since every block loads whole tiles for a quarter of the arithmetic)
    const int narrow = shape == 1 ? 0 : shape >= 2 ? 1 : rows <= 16 ? 1 : 0;
    const int deep = (shape >= 3 || (shape == 0 && narrow && thin <= 2 * sms)) ? 1 : 0;
    long long ksplit = 1;
    if (shape == 4) ksplit = 3;
    else if (shape == 0 && narrow) {
        ksplit = (2 * sms) / thin;
        if (ksplit > kMaxParts) ksplit = kMaxParts;
        if (chunk > 0 && ksplit > (chunk + kMmaKeys - 1) / kMmaKeys) ksplit = (chunk + kMmaKeys - 1) / kMmaKeys;
        if (ksplit < 1) ksplit = 1;
    }
    return narrow | (deep << 1) | ((int)ksplit << 8);
}

// bfloat16 only; dk and dv multiples of 16, at most 128; sms: the device's multiprocessors (what a small grid is measured against); q, the pages, the gate and out 16-byte aligned
// with gate_stride even.
LSB_API int lsb_attention_dv_mma_supported(int dk, int dv) {
    return dk > 0 && dv > 0 && dk % 16 == 0 && dv % 16 == 0 && dk <= 128 && dv <= 128;
}

LSB_API int lsb_attention_dv_mma(const void* q, const void* k_pages, const void* v_pages, const int* q_start,
                                 const int* kv_len, const int* table_rows, const int* block_table, int table_stride,
                                 const void* gate, long long gate_stride, void* out, int n_requests, int max_q_len,
                                 int nh, int nkv, int dk, int dv, int page_size, int num_pages, float scale, int window,
                                 int chunk, int sms, int shape, float* scratch, int flags, float softcap,
                                 cudaStream_t stream) {
    if (n_requests <= 0 || max_q_len <= 0) return 0;
    if (sms <= 0) sms = 148;
    if (!lsb_attention_dv_mma_supported(dk, dv) || nkv <= 0 || nh % nkv || window < 0 || chunk < 0 || n_requests > 65535 ||
        nkv > 65535 || (gate_stride & 1))
        return (int)cudaErrorInvalidValue;
    const int group = nh / nkv;
    const long long rows = (long long)max_q_len * group;
    const int plan = lsb_attention_dv_mma_plan(n_requests, max_q_len, nh, nkv, chunk, sms, shape);
    const int narrow = plan & 1, ksplit = plan >> 8;
    const bool deep = (plan & 2) != 0;
    if (ksplit > 1 && !scratch) return (int)cudaErrorInvalidValue;
    const unsigned tiles = (unsigned)(narrow ? (rows + 15) / 16 : (rows + kMmaRows - 1) / kMmaRows);
    dim3 grid(tiles * ksplit, nkv, n_requests);
    const float scale_log2 = scale * 1.4426950408889634f;
#define LSB_DV_MMA(DKP, DVP, STAGES, NARROW)                                                                     \
    do {                                                                                                         \
        const size_t smem = (size_t)STAGES * kMmaKeys * ((DKP + 8) + (DVP + 8)) * sizeof(__nv_bfloat16);         \
        if (smem > 48 * 1024) {                                                                                  \
            rc = (int)cudaFuncSetAttribute(attention_dv_mma_kernel<DKP, DVP, STAGES, NARROW>,                    \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
            if (rc) return rc;                                                                                   \
        }                                                                                                        \
        rc = lsb_launch(attention_dv_mma_kernel<DKP, DVP, STAGES, NARROW>, grid, dim3(kMmaThreads), smem,        \
                          stream, 1, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages,                     \
                          (const __nv_bfloat16*)v_pages, q_start, kv_len, table_rows, block_table, table_stride, \
                          (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, nh, nkv, dk, dv,         \
                          page_size, num_pages, scale_log2, window, chunk, ksplit, scratch, flags, scale, softcap);              \
    } while (0)
#define LSB_DV_MMA_SHAPE(DKP, DVP)                                                                               \
    do {                                                                                                         \
        if (deep) LSB_DV_MMA(DKP, DVP, 4, true);                                                                 \
        else if (narrow) LSB_DV_MMA(DKP, DVP, 2, true);                                                          \
        else LSB_DV_MMA(DKP, DVP, 2, false);                                                                     \
    } while (0)
#define LSB_DV_MMA_V(DKP)                                                                                        \
    do {                                                                                                         \
        if (dv <= 32) LSB_DV_MMA_SHAPE(DKP, 32);                                                                 \
        else if (dv <= 64) LSB_DV_MMA_SHAPE(DKP, 64);                                                            \
        else LSB_DV_MMA_SHAPE(DKP, 128);                                                                         \
    } while (0)
    int rc = 0;
    if (dk <= 64) LSB_DV_MMA_V(64);
    else LSB_DV_MMA_V(128);
#undef LSB_DV_MMA_V
#undef LSB_DV_MMA_SHAPE
#undef LSB_DV_MMA
    if (rc || ksplit <= 1) return rc;
    return lsb_launch(attention_dv_merge_kernel, dim3(tiles, nkv, n_requests), dim3(kMmaThreads), 0, stream, 1,
                      (const float*)scratch, q_start, (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, nh, nkv,
                      dv, ksplit, flags);
}

LSB_API int lsb_attention_dv_max_dim() { return kDvMaxDim; }

// q [tokens, nh * dk], out [tokens, nh * dv]; gate (or null) has rows `gate_stride` elements apart
// with the nh * dv gate values first.
LSB_API int lsb_attention_dv_generic(const void* q, const void* k_pages, const void* v_pages, const int* q_start,
                                     const int* kv_len, const int* table_rows, const int* block_table,
                                     int table_stride, const void* gate, long long gate_stride, void* out, int dtype,
                                     int n_requests, int max_q_len, int nh, int nkv, int dk, int dv, int page_size,
                                     int num_pages, float scale, int window, int chunk, int flags, float softcap,
                                     cudaStream_t stream) {
    if (n_requests <= 0 || max_q_len <= 0) return 0;
    if (dk <= 0 || dk > kDvMaxDim || dv <= 0 || dv > kDvMaxDim || nkv <= 0 || nh % nkv || window < 0 || chunk < 0)
        return (int)cudaErrorInvalidValue;
    if (n_requests > 65535 || nh > 65535) return (int)cudaErrorInvalidValue;
    const int al = dtype == LSB_F32 ? 4 : 8;
    const int vec = (dk % al == 0 && (uintptr_t)k_pages % 16 == 0) ? 1 : 0;
    dim3 grid((max_q_len + kDvWarps - 1) / kDvWarps, nh, n_requests);
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(
        attention_dv_generic_kernel<T>, grid, dim3(kDvWarps * 32), 0, stream, 1, (const T*)q, (const T*)k_pages,
        (const T*)v_pages, q_start, kv_len, table_rows, block_table, table_stride, (const T*)gate, gate_stride,
        (T*)out, nh, nkv, dk, dv, page_size, num_pages, scale, window, chunk, vec, flags, softcap));
    return 0;
}
