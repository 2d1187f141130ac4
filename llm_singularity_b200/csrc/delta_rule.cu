// Delta-rule memories: a matrix state S [key channels, value channels] per head and request that a
// token first lets fade, then corrects along a key, then reads.  Two forms share the walk:
//
//   scalar gates (MODE 0):   S <- g S;  e = beta (v - S^T k);  S <- S + k e^T;  o = S^T q
//       g and beta one number per token and head; q and k unit vectors of a key head that several
//       value heads may share (value head h reads key head h / (heads / key_heads))
//   channel gates (MODE 1):  S <- diag(w) S - (a * u) (u^T S) + k v^T;  o = S^T r
//       w and a one number per key channel, u the unit vector along k; both terms read the state the
//       token found
//
// for any mix of prompt portions and single decode tokens, each request continuing from the state
// its slot holds.  S is 32-bit, stored [slot, head, value channel, key channel] (key channels
// contiguous).  Everything that enters the walk is formed in 32-bit by a preparation kernel from the
// projections' outputs:
//
//   gated_delta_prep    a short causal convolution per channel over time (taps [channels, n], the
//                       last one meets the current token; the n - 1 inputs before a portion come from
//                       the slot's convolution state, zeros at a request's start), silu, unit length
//                       per key head (q also times key_dim^-1/2), beta = sigmoid(.), and the fade
//                       g = exp(-exp(A_log) * softplus(. + dt_bias))
//   conv_state_update   the slot's last n - 1 inputs after the step
//   channel_delta_prep  u = k / sqrt(sum k^2 + eps), a = sigmoid(. + bias), w = exp(-rate * sigmoid(. + w0))
//   delta_output        each head's read-out divided by its root mean square, times a weight, times
//                       sigmoid or silu of a gate projection
//   tanh_rows           the hidden activation of a two-step (low-rank) projection
//
// The walk: a block owns (request, head, a tile of value columns) and takes the request's tokens in
// order, so the result does not depend on how a prompt was cut.  A column's key channels are dealt to
// `split` neighbouring lanes, 32 each, kept in registers; dots are finished by shuffles.  The tokens'
// vectors come through shared memory in chunks of 16 tokens, a chunk copied while the one before is walked.
//
// Long portions are cut into segments that are walked side by side, since a walk is a chain of
// dependent steps and one portion alone gives the chip few of them.  A token's step is linear in the
// state, S <- A_t S + k x^T with A_t = g (I - beta k k^T) or diag(w) - (a * u) u^T, so a segment walked
// from nothing gives its own contribution E, and the identity's columns walked through the same steps
// (with nothing written) give the product P of its transitions; a small kernel chains the segments,
// start(s + 1) = P_s start(s) + E_s; every segment is then walked again from its start for the outputs.
// The sums form in another order than in one walk: equal beyond rounding.
#include "common.cuh"
#include <type_traits>

LSB_DEFINE_STATUS()

constexpr int kDeltaThreads = 128;
constexpr int kDeltaChunk = 16;      // tokens staged at a time (8 where two buffers of 16 would leave an SM fewer than four blocks)
constexpr int kDeltaPer = 32;        // key channels of a column that one lane keeps
constexpr int kDeltaPad = 4;         // words between the shares of neighbouring lanes in shared memory
constexpr int kDeltaMaxSplit = 8;

__device__ __forceinline__ float delta_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ void delta_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void delta_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void delta_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void delta_copy_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ float delta_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// ------------------------------------------------------------------ scalar gates: preparation
struct GatedPrepArgs {
    const void* proj; long long ld; int q_off, k_off, v_off;
    int G, H, D, V, taps;
    const float *q_taps, *k_taps, *v_taps;         // [channels, taps]
    float* conv_state; int n_slots;                 // [slots, taps - 1, 2 G D + H V]
    const float* raw; long long raw_ld;             // [T, 2 H]: beta's projection, then the fade's
    const float *a_log, *dt_bias;
    const int *token_req, *q_start, *table_rows;
    float *qk_out, *v_out, *scal_out;               // [T, 2 G D], [T, H V], [T, 2 H]
    float unit_eps;
};

constexpr int kPrepMaxThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kPrepMaxThreads) gated_delta_prep_kernel(GatedPrepArgs a) {
    extern __shared__ float ch_sh[];                // the token's channels after convolution and silu
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = a.token_req[t];
    const int t0 = a.q_start[r], i = t - t0;
    const int slot = a.table_rows[r];
    if (slot < 0 || slot >= a.n_slots) {
        if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW);
        return;
    }
    const int GD = a.G * a.D, C = 2 * GD + a.H * a.V, m = a.taps - 1;
    const T* proj = (const T*)a.proj;
    const float* old = a.conv_state + (size_t)slot * m * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        int lc, off;
        const float* taps;
        if (c < GD) { lc = c; off = a.q_off; taps = a.q_taps; }
        else if (c < 2 * GD) { lc = c - GD; off = a.k_off; taps = a.k_taps; }
        else { lc = c - 2 * GD; off = a.v_off; taps = a.v_taps; }
        float acc = 0.f;
        for (int j = 0; j < a.taps; ++j) {
            const int ii = i - (m - j);             // the portion's token this tap meets
            const float x = ii >= 0 ? lsb_to_float(proj[(size_t)(t0 + ii) * a.ld + off + lc]) : old[(size_t)(m + ii) * C + c];
            acc += taps[(size_t)lc * a.taps + j] * x;
        }
        ch_sh[c] = acc * delta_sigmoid(acc);
    }
    __syncthreads();
    for (int head = warp; head < 2 * a.G; head += blockDim.x >> 5) {
        const float* hs = ch_sh + (size_t)head * a.D;
        float ss = 0.f;
        for (int d = lane; d < a.D; d += 32) ss += hs[d] * hs[d];
        float inv = rsqrtf(lsb_warp_sum(ss) + a.unit_eps);
        if (head < a.G) inv *= rsqrtf((float)a.D);
        for (int d = lane; d < a.D; d += 32) a.qk_out[(size_t)t * 2 * GD + (size_t)head * a.D + d] = hs[d] * inv;
    }
    for (int c = threadIdx.x; c < a.H * a.V; c += blockDim.x) a.v_out[(size_t)t * a.H * a.V + c] = ch_sh[2 * GD + c];
    for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
        const float zb = a.raw[(size_t)t * a.raw_ld + h], za = a.raw[(size_t)t * a.raw_ld + a.H + h];
        a.scal_out[(size_t)t * 2 * a.H + h] = expf(-expf(a.a_log[h]) * delta_softplus(za + a.dt_bias[h]));
        a.scal_out[(size_t)t * 2 * a.H + a.H + h] = delta_sigmoid(zb);
    }
}

// The last taps - 1 inputs of every request of the step, for the next step: from the portion where it
// is long enough, from the old state (moved up) where it is not.
template <typename T>
__global__ void __launch_bounds__(kDeltaThreads)
conv_state_update_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, int GD, int HV,
                         int taps, float* __restrict__ conv_state, int n_slots, const int* __restrict__ q_start,
                         const int* __restrict__ table_rows) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r = blockIdx.y;
    const int t0 = q_start[r], L = q_start[r + 1] - t0, m = taps - 1;
    const int slot = table_rows[r];
    if (slot < 0 || slot >= n_slots || L <= 0) return;
    const int C = 2 * GD + HV;
    float* st = conv_state + (size_t)slot * m * C;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < C; c += gridDim.x * blockDim.x) {
        const int col = c < GD ? q_off + c : c < 2 * GD ? k_off + c - GD : v_off + c - 2 * GD;
        // (ascending j: what entry j takes from the old state lies at j + L, not yet written)
        for (int j = 0; j < m; ++j) {
            const int ii = L - m + j;
            st[(size_t)j * C + c] = ii >= 0 ? lsb_to_float(proj[(size_t)(t0 + ii) * ld + col]) : st[(size_t)(j + L) * C + c];
        }
    }
}

// ------------------------------------------------------------------ channel gates: preparation
struct ChannelPrepArgs {
    const void* proj; long long ld; int r_off, k_off, v_off;
    int H, D, V;
    const float* decay_raw; long long decay_ld; const float* decay_bias;     // [T, H D] + [H D]
    const float* remove_raw; long long remove_ld; const float* remove_bias;
    float decay_rate, unit_eps;
    float *vec_out, *v_out;                         // [T, H, 5, D]: r, k, u, a * u, w;  [T, H V]
};

template <typename T>
__global__ void __launch_bounds__(kDeltaThreads) channel_delta_prep_kernel(ChannelPrepArgs a) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* row = (const T*)a.proj + (size_t)t * a.ld;
    for (int h = warp; h < a.H; h += kDeltaThreads / 32) {
        const T* k = row + a.k_off + (size_t)h * a.D;
        float ss = 0.f;
        for (int d = lane; d < a.D; d += 32) {
            const float x = lsb_to_float(k[d]);
            ss += x * x;
        }
        const float inv = rsqrtf(lsb_warp_sum(ss) + a.unit_eps);
        float* o = a.vec_out + ((size_t)t * a.H + h) * 5 * a.D;
        for (int d = lane; d < a.D; d += 32) {
            const int c = h * a.D + d;
            const float kd = lsb_to_float(k[d]), u = kd * inv;
            const float rem = delta_sigmoid(a.remove_raw[(size_t)t * a.remove_ld + c] + a.remove_bias[c]);
            const float w = expf(-a.decay_rate * delta_sigmoid(a.decay_raw[(size_t)t * a.decay_ld + c] + a.decay_bias[c]));
            o[d] = lsb_to_float(row[a.r_off + c]);
            o[a.D + d] = kd;
            o[2 * a.D + d] = u;
            o[3 * a.D + d] = rem * u;
            o[4 * a.D + d] = w;
        }
        for (int d = lane; d < a.V; d += 32)
            a.v_out[((size_t)t * a.H + h) * a.V + d] = lsb_to_float(row[a.v_off + (size_t)h * a.V + d]);
    }
}

// ------------------------------------------------------------------------------ the walk
// SEG 0: a request's whole portion from its slot's state, outputs, the slot's state left behind.
// SEG 1: one segment of a portion from nothing: the V value columns start at zero and gather what the
//        segment's tokens write (E); D more columns start as the identity and take no writes, which
//        leaves the product P of the segment's transitions (a token's step is linear in the state:
//        S <- A_t S + k x^T, and a column of the identity walks through the same steps with x = 0).
//        No outputs; E and P go to seg_acc [the segment's scratch row, head, V + D, D].
// SEG 2: one segment from its start state (seg_start, laid out like the state), outputs only.
// Between 1 and 2 delta_chain_kernel forms start(s + 1) = P_s start(s) + E_s segment after segment.
// Three times the arithmetic of one walk, a chain a segment long.
template <int MODE, int SEG>
__global__ void __launch_bounds__(kDeltaThreads)
delta_scan_kernel(const float* __restrict__ vecs, const float* __restrict__ scal, const float* __restrict__ vals,
                  float* __restrict__ state, int n_slots, const int* __restrict__ q_start,
                  const int* __restrict__ table_rows, float* __restrict__ out, int H, int G, int D, int V, int split,
                  int seg_len, int max_segs, float* __restrict__ seg_acc, const float* __restrict__ seg_start,
                  int chunk) {
    constexpr int NV = MODE == 0 ? 2 : 5;          // vectors of key size a token brings
    extern __shared__ __align__(16) float sh[];
    const int cols = blockDim.x / split;
    const int Dp = split * (kDeltaPer + kDeltaPad);
    float* vec_sh = sh;                                 // [2][chunk][NV][Dp]
    float* val_sh = vec_sh + 2 * chunk * NV * Dp;       // [2][chunk][cols]
    float* scal_sh = val_sh + 2 * chunk * cols;         // [2][chunk][2]
    const bool wide = (D & 3) == 0 && (reinterpret_cast<size_t>(vecs) & 15) == 0;
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int r = SEG ? blockIdx.z / max_segs : blockIdx.z, sidx = SEG ? blockIdx.z % max_segs : 0;
    const int h = blockIdx.y;
    const int col0 = blockIdx.x * cols;
    const int part = threadIdx.x % split, lc = threadIdx.x / split;
    const int col = col0 + lc;
    const int Vs = SEG == 1 ? V + D : V;            // columns walked
    int t0 = q_start[r], t1 = q_start[r + 1];
    // (a request's segment s keeps its E, P and start in scratch row t0 / seg_len + r + s: rows of
    // different requests never meet, and a step needs tokens / seg_len + requests rows at most)
    const size_t zrow = SEG ? (size_t)(t0 / seg_len + r + sidx) : 0;
    if (SEG) {
        t0 += sidx * seg_len;
        if (t0 >= t1) return;                       // the request has fewer segments
        t1 = min(t1, t0 + seg_len);
    }
    const int slot = table_rows[r];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) lsb_set_status(LSB_BAD_ROW);
        return;
    }
    // (channels past D and value columns past V are never staged: zero once, so that a lane's unused
    // registers stay zero and the identity's columns meet no write)
    for (int idx = threadIdx.x; idx < 2 * chunk * (NV * Dp + cols); idx += blockDim.x) vec_sh[idx] = 0.f;
    const bool live = col < Vs;
    float* srow = SEG == 1 ? seg_acc + ((zrow * H + h) * Vs + (live ? col : 0)) * D
                           : state + (((size_t)slot * H + h) * V + (live ? col : 0)) * D;
    const float* first = SEG == 2 ? seg_start + ((zrow * H + h) * V + (live ? col : 0)) * D : srow;
    // (the state's share lives in pairs: the walk's arithmetic is the two-wide 32-bit FMA of sm_100,
    // one instruction for two channels, each channel rounded as the one-wide form rounds it)
    float2 s[kDeltaPer / 2];
#pragma unroll
    for (int i = 0; i < kDeltaPer; ++i) {
        const int d = part * kDeltaPer + i;
        float x;
        if (SEG == 1) x = (live && col >= V && d == col - V) ? 1.f : 0.f;
        else x = (live && d < D) ? first[d] : 0.f;
        if (i & 1) s[i >> 1].y = x;
        else s[i >> 1].x = x;
    }
    const int g = MODE == 0 ? h / (H / G) : 0;
    // A chunk's operands arrive by asynchronous copies into one of two buffers while the chunk before is
    // walked: 16 bytes a copy where the key size and the addresses allow, 4 bytes otherwise.
    auto stage = [&](int b, int c0) {
        const int n = min(chunk, t1 - c0);
        float* vdst = vec_sh + b * (chunk * NV * Dp);
        if (wide) {
            const int D4 = D >> 2;
            for (int idx = threadIdx.x; idx < n * NV * D4; idx += blockDim.x) {
                const int tok = idx / (NV * D4), rem = idx - tok * NV * D4, v = rem / D4, d = (rem - v * D4) << 2;
                const size_t src = MODE == 0 ? ((size_t)(c0 + tok) * 2 + v) * G * D + (size_t)g * D + d
                                             : (((size_t)(c0 + tok) * H + h) * NV + v) * D + d;
                delta_copy16(vdst + (tok * NV + v) * Dp + (d / kDeltaPer) * (kDeltaPer + kDeltaPad) + d % kDeltaPer, vecs + src);
            }
        } else {
            for (int idx = threadIdx.x; idx < n * NV * D; idx += blockDim.x) {
                const int tok = idx / (NV * D), rem = idx - tok * NV * D, v = rem / D, d = rem - v * D;
                const size_t src = MODE == 0 ? ((size_t)(c0 + tok) * 2 + v) * G * D + (size_t)g * D + d
                                             : (((size_t)(c0 + tok) * H + h) * NV + v) * D + d;
                delta_copy4(vdst + (tok * NV + v) * Dp + (d / kDeltaPer) * (kDeltaPer + kDeltaPad) + d % kDeltaPer, vecs + src);
            }
        }
        float* wdst = val_sh + b * (chunk * cols);
        for (int idx = threadIdx.x; idx < n * cols; idx += blockDim.x) {
            const int tok = idx / cols, c = idx - tok * cols;
            if (col0 + c < V) delta_copy4(wdst + idx, vals + ((size_t)(c0 + tok) * H + h) * V + col0 + c);
        }
        if (MODE == 0) {
            for (int idx = threadIdx.x; idx < n * 2; idx += blockDim.x)
                delta_copy4(scal_sh + b * (chunk * 2) + idx, scal + (size_t)(c0 + idx / 2) * 2 * H + (size_t)(idx & 1) * H + h);
        }
    };
    __syncthreads();                                // the zeros are in place before a copy lands among them
    if (t0 < t1) stage(0, t0);
    delta_copy_commit();
    int buf = 0;
    for (int c0 = t0; c0 < t1; c0 += chunk, buf ^= 1) {
        const int n = min(chunk, t1 - c0);
        if (c0 + chunk < t1) stage(buf ^ 1, c0 + chunk);
        delta_copy_commit();
        delta_copy_wait_but_one();                  // this chunk's copies have landed; the next one's may fly
        __syncthreads();
        const float* vec_b = vec_sh + buf * (chunk * NV * Dp);
        const float* val_b = val_sh + buf * (chunk * cols);
        const float* scal_b = scal_sh + buf * (chunk * 2);
#pragma unroll 2
        for (int tok = 0; tok < n; ++tok) {
            const float* vb = vec_b + tok * NV * Dp + part * (kDeltaPer + kDeltaPad);
            const float v_in = val_b[tok * cols + lc];
            // (dots gather in four partial sums, so that a token's chain of dependent additions is a
            // quarter as long; every walk sums in this same order)
            float2 o01 = make_float2(0.f, 0.f), o23 = make_float2(0.f, 0.f);
            float2 d01 = make_float2(0.f, 0.f), d23 = make_float2(0.f, 0.f);
            if (MODE == 0) {
                const float fade = scal_b[tok * 2], beta = scal_b[tok * 2 + 1];
                const float2 fade2 = make_float2(fade, fade);
                const float4* q4 = reinterpret_cast<const float4*>(vb);
                const float4* k4 = reinterpret_cast<const float4*>(vb + Dp);
#pragma unroll
                for (int i = 0; i < kDeltaPer / 4; ++i) {
                    const float4 k = k4[i];
                    s[2 * i] = __fmul2_rn(s[2 * i], fade2);
                    s[2 * i + 1] = __fmul2_rn(s[2 * i + 1], fade2);
                    d01 = __ffma2_rn(make_float2(k.x, k.y), s[2 * i], d01);
                    d23 = __ffma2_rn(make_float2(k.z, k.w), s[2 * i + 1], d23);
                }
                float dot = (d01.x + d01.y) + (d23.x + d23.y);
                for (int w = split >> 1; w > 0; w >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, w);
                const float e = beta * (v_in - dot);
                const float2 e2 = make_float2(e, e);
#pragma unroll
                for (int i = 0; i < kDeltaPer / 4; ++i) {
                    const float4 k = k4[i];
                    s[2 * i] = __ffma2_rn(make_float2(k.x, k.y), e2, s[2 * i]);
                    s[2 * i + 1] = __ffma2_rn(make_float2(k.z, k.w), e2, s[2 * i + 1]);
                    if (SEG != 1) {
                        const float4 q = q4[i];
                        o01 = __ffma2_rn(make_float2(q.x, q.y), s[2 * i], o01);
                        o23 = __ffma2_rn(make_float2(q.z, q.w), s[2 * i + 1], o23);
                    }
                }
            } else {
                const float4* r4 = reinterpret_cast<const float4*>(vb);
                const float4* k4 = reinterpret_cast<const float4*>(vb + Dp);
                const float4* u4 = reinterpret_cast<const float4*>(vb + 2 * Dp);
                const float4* a4 = reinterpret_cast<const float4*>(vb + 3 * Dp);
                const float4* w4 = reinterpret_cast<const float4*>(vb + 4 * Dp);
#pragma unroll
                for (int i = 0; i < kDeltaPer / 4; ++i) {
                    const float4 u = u4[i];
                    d01 = __ffma2_rn(make_float2(u.x, u.y), s[2 * i], d01);
                    d23 = __ffma2_rn(make_float2(u.z, u.w), s[2 * i + 1], d23);
                }
                float dot = (d01.x + d01.y) + (d23.x + d23.y);
                for (int w = split >> 1; w > 0; w >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, w);
                const float2 nd2 = make_float2(-dot, -dot), v2 = make_float2(v_in, v_in);
#pragma unroll
                for (int i = 0; i < kDeltaPer / 4; ++i) {
                    const float4 k = k4[i], au = a4[i], w = w4[i];
                    // w s - (a u) dot + k v, as a product and two FMAs
                    float2 lo = __fmul2_rn(make_float2(w.x, w.y), s[2 * i]);
                    float2 hi = __fmul2_rn(make_float2(w.z, w.w), s[2 * i + 1]);
                    lo = __ffma2_rn(make_float2(au.x, au.y), nd2, lo);
                    hi = __ffma2_rn(make_float2(au.z, au.w), nd2, hi);
                    s[2 * i] = __ffma2_rn(make_float2(k.x, k.y), v2, lo);
                    s[2 * i + 1] = __ffma2_rn(make_float2(k.z, k.w), v2, hi);
                    if (SEG != 1) {
                        const float4 q = r4[i];
                        o01 = __ffma2_rn(make_float2(q.x, q.y), s[2 * i], o01);
                        o23 = __ffma2_rn(make_float2(q.z, q.w), s[2 * i + 1], o23);
                    }
                }
            }
            if (SEG != 1) {
                float o = (o01.x + o01.y) + (o23.x + o23.y);
                for (int w = split >> 1; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
                if (live && part == 0) out[((size_t)(c0 + tok) * H + h) * V + col] = o;
            }
        }
        __syncthreads();                            // every lane has walked this buffer before it is filled again
    }
    if (live && SEG != 2) {
#pragma unroll
        for (int i = 0; i < kDeltaPer; ++i) {
            const int d = part * kDeltaPer + i;
            if (d < D) srow[d] = (i & 1) ? s[i >> 1].y : s[i >> 1].x;
        }
    }
}

// The chain over a request's segments: start(0) is the slot's state, start(s + 1) = P_s start(s) + E_s,
// and the slot's state becomes the start after the last segment.  A block owns kChainRows value rows of
// a head.  With the rows stored [value, key]:
//     next[v][d] = E[v][d] + sum_c P[c][d] * cur[v][c]      (P's column c lies in row V + c of seg_acc)
// Thread (d, part) sums a share of the c (a quarter; a half for key sizes above 128) for all the block's
// rows at key channel d; the shares meet in shared memory, always in the same order, and the thread then
// keeps its part of the rows.
constexpr int kChainRows = 8;
constexpr int kChainBatch = 16;

template <int kChainSplit>
__global__ void __launch_bounds__(512)
delta_chain_kernel(float* __restrict__ state, int n_slots, const float* __restrict__ seg_acc, float* __restrict__ seg_start,
                   const int* __restrict__ q_start, const int* __restrict__ table_rows, int H, int D, int V, int seg_len,
                   int max_segs) {
    constexpr int kChainOwn = kChainRows / kChainSplit;
    extern __shared__ __align__(16) float chain_sh[];
    const int Dr = blockDim.x;                       // D rounded up to whole warps
    const int cper = ((D + kChainSplit * kChainBatch - 1) / (kChainSplit * kChainBatch)) * kChainBatch;
    float* cur = chain_sh;                           // [kChainSplit * cper][kChainRows], zeros past D
    float* part = cur + kChainSplit * cper * kChainRows;   // [kChainSplit][kChainRows][Dr]
    lsb_pdl_launch_dependents();
    for (int i = threadIdx.y * Dr + threadIdx.x; i < kChainSplit * cper * kChainRows; i += Dr * kChainSplit) cur[i] = 0.f;
    lsb_pdl_wait();
    const int r = blockIdx.z, h = blockIdx.y, v0 = blockIdx.x * kChainRows, d = threadIdx.x, pt = threadIdx.y;
    const int L = q_start[r + 1] - q_start[r];
    const int n_seg = (L + seg_len - 1) / seg_len;
    const int slot = table_rows[r];
    if (n_seg <= 0) return;
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0 && threadIdx.y == 0) lsb_set_status(LSB_BAD_ROW);
        return;
    }
    const int Vs = V + D;
    const bool mine = d < D;
    const int dd = mine ? d : 0;
    const int my0 = v0 + pt * kChainOwn;             // the first of the rows this thread keeps
    float own[kChainOwn];
    float* srow = state + ((size_t)slot * H + h) * V * D;
#pragma unroll
    for (int j = 0; j < kChainOwn; ++j) own[j] = (mine && my0 + j < V) ? srow[(size_t)(my0 + j) * D + d] : 0.f;
    __syncthreads();                                 // the zeros are in place
    for (int sg = 0; sg < n_seg; ++sg) {
        const size_t z = (size_t)(q_start[r] / seg_len + r + sg);
        const float* E = seg_acc + (z * H + h) * Vs * D;
        const float* P = E + (size_t)V * D;
        float e[kChainOwn];
        if (mine) {
            float* st = seg_start + (z * H + h) * V * D;
#pragma unroll
            for (int j = 0; j < kChainOwn; ++j) {
                if (my0 + j < V) st[(size_t)(my0 + j) * D + d] = own[j];
                cur[d * kChainRows + pt * kChainOwn + j] = own[j];
                e[j] = my0 + j < V ? E[(size_t)(my0 + j) * D + d] : 0.f;
            }
        }
        __syncthreads();
        float acc[kChainRows];
#pragma unroll
        for (int v = 0; v < kChainRows; ++v) acc[v] = 0.f;
        // (a batch of P's rows is asked for at once, so that their latencies overlap; rows past D meet
        // the zeros of cur)
        for (int c0 = pt * cper; c0 < (pt + 1) * cper; c0 += kChainBatch) {
            float p[kChainBatch];
#pragma unroll
            for (int j = 0; j < kChainBatch; ++j) p[j] = P[(size_t)min(c0 + j, D - 1) * D + dd];
#pragma unroll
            for (int j = 0; j < kChainBatch; ++j) {
                const float4 a = *reinterpret_cast<const float4*>(cur + (c0 + j) * kChainRows);
                const float4 b = *reinterpret_cast<const float4*>(cur + (c0 + j) * kChainRows + 4);
                acc[0] += p[j] * a.x; acc[1] += p[j] * a.y; acc[2] += p[j] * a.z; acc[3] += p[j] * a.w;
                acc[4] += p[j] * b.x; acc[5] += p[j] * b.y; acc[6] += p[j] * b.z; acc[7] += p[j] * b.w;
            }
        }
#pragma unroll
        for (int v = 0; v < kChainRows; ++v) part[(pt * kChainRows + v) * Dr + d] = acc[v];
        __syncthreads();                             // every lane has read cur; the quarters are in place
        if (mine) {
#pragma unroll
            for (int j = 0; j < kChainOwn; ++j) {
                float sum = e[j];
#pragma unroll
                for (int g = 0; g < kChainSplit; ++g) sum += part[(g * kChainRows + pt * kChainOwn + j) * Dr + d];
                own[j] = sum;
            }
        }
        // (the quarters are written again only after the next segment's first barrier)
    }
    if (mine) {
#pragma unroll
        for (int j = 0; j < kChainOwn; ++j)
            if (my0 + j < V) srow[(size_t)(my0 + j) * D + d] = own[j];
    }
}

// ------------------------------------------------------------------ read-out norm and gate
// out[t, h, c] = x[t, h, c] / sqrt(mean_c x^2 + eps) * w[(h V + c) mod w_len] * act(gate[t, h V + c]);
// gate_act 0: no gate, 1: sigmoid, 2: silu.  A warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(kDeltaThreads)
delta_output_kernel(const float* __restrict__ x, const float* __restrict__ w, int w_len, const T* __restrict__ gate,
                    long long gate_stride, int gate_act, T* __restrict__ out, long long pairs, int H, int V, float eps) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const long long pair = (long long)blockIdx.x * (kDeltaThreads / 32) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const int lane = threadIdx.x & 31;
    const long long t = pair / H;
    const int h = (int)(pair - t * H);
    const float* xr = x + pair * V;
    float ss = 0.f;
    for (int c = lane; c < V; c += 32) ss += xr[c] * xr[c];
    const float inv = rsqrtf(lsb_warp_sum(ss) / (float)V + eps);
    for (int c = lane; c < V; c += 32) {
        float y = xr[c] * inv * w[(h * V + c) % w_len];
        if (gate_act) {
            const float z = lsb_to_float(gate[t * gate_stride + (long long)h * V + c]);
            y *= gate_act == 1 ? delta_sigmoid(z) : z * delta_sigmoid(z);
        }
        out[pair * V + c] = lsb_from_float<T>(y);
    }
}

template <typename T>
__global__ void tanh_rows_kernel(const float* __restrict__ x, long long ld, int off, int n, T* __restrict__ out, long long count) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / n;
        out[i] = lsb_from_float<T>(tanhf(x[t * ld + off + (i - t * n)]));
    }
}

// -------------------------------------------------------------------------- entry points
LSB_API int lsb_delta_max_key_dim() { return kDeltaPer * kDeltaMaxSplit; }

LSB_API int lsb_gated_delta_prep(const void* proj, int dtype, long long ld, int q_off, int k_off, int v_off, int tokens,
                                 int n_requests, int G, int H, int D, int V, int taps, const float* q_taps,
                                 const float* k_taps, const float* v_taps, float* conv_state, int n_slots,
                                 const float* raw, long long raw_ld, const float* a_log, const float* dt_bias,
                                 const int* token_req, const int* q_start, const int* table_rows, float* qk_out,
                                 float* v_out, float* scal_out, float unit_eps, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (G <= 0 || H <= 0 || H % G || D <= 0 || V <= 0 || taps < 1 || n_requests <= 0 || n_requests > 65535)
        return (int)cudaErrorInvalidValue;
    GatedPrepArgs a;
    a.proj = proj; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.G = G; a.H = H; a.D = D; a.V = V; a.taps = taps;
    a.q_taps = q_taps; a.k_taps = k_taps; a.v_taps = v_taps;
    a.conv_state = conv_state; a.n_slots = n_slots;
    a.raw = raw; a.raw_ld = raw_ld; a.a_log = a_log; a.dt_bias = dt_bias;
    a.token_req = token_req; a.q_start = q_start; a.table_rows = table_rows;
    a.qk_out = qk_out; a.v_out = v_out; a.scal_out = scal_out; a.unit_eps = unit_eps;
    const int C = 2 * G * D + H * V;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    LSB_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) {
            int rc = (int)cudaFuncSetAttribute(gated_delta_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (rc) return rc;
        }
        // (a thread for every four channels, within 128 .. 512)
        int threads = ((C / 4 + 31) / 32) * 32;
        threads = threads < kDeltaThreads ? kDeltaThreads : threads > kPrepMaxThreads ? kPrepMaxThreads : threads;
        int rc = lsb_launch(gated_delta_prep_kernel<T>, dim3(tokens), dim3(threads), smem, stream, 1, a);
        if (rc || taps == 1) return rc;
        const int bx = (C + kDeltaThreads - 1) / kDeltaThreads;
        return lsb_launch(conv_state_update_kernel<T>, dim3(bx > 64 ? 64 : bx, n_requests), dim3(kDeltaThreads), 0, stream, 1,
                          (const T*)proj, ld, q_off, k_off, v_off, G * D, H * V, taps, conv_state, n_slots, q_start,
                          table_rows);
    });
    return 0;
}

LSB_API int lsb_channel_delta_prep(const void* proj, int dtype, long long ld, int r_off, int k_off, int v_off, int tokens,
                                   int H, int D, int V, const float* decay_raw, long long decay_ld, const float* decay_bias,
                                   const float* remove_raw, long long remove_ld, const float* remove_bias,
                                   float decay_rate, float unit_eps, float* vec_out, float* v_out, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0) return (int)cudaErrorInvalidValue;
    ChannelPrepArgs a;
    a.proj = proj; a.ld = ld; a.r_off = r_off; a.k_off = k_off; a.v_off = v_off;
    a.H = H; a.D = D; a.V = V;
    a.decay_raw = decay_raw; a.decay_ld = decay_ld; a.decay_bias = decay_bias;
    a.remove_raw = remove_raw; a.remove_ld = remove_ld; a.remove_bias = remove_bias;
    a.decay_rate = decay_rate; a.unit_eps = unit_eps;
    a.vec_out = vec_out; a.v_out = v_out;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(channel_delta_prep_kernel<T>, dim3(tokens), dim3(kDeltaThreads), 0, stream, 1, a));
    return 0;
}

// mode 0: scalar gates (vecs [T, 2, G, D]: q then k; scal [T, 2, H]: fade then beta); mode 1: channel
// gates (vecs [T, H, 5, D]: r, k, u, a * u, w).  vals [T, H, V]; state [slots, H, V, D]; out [T, H, V].
// seg_len > 0 with scratch given and a portion longer than a segment: portions are walked in segments
// side by side; seg_acc [rows, H, V + D, D] and seg_start [rows, H, V, D] with rows = tokens / seg_len +
// requests (segment s of the request that starts at token t0 uses row t0 / seg_len + request + s).
LSB_API int lsb_delta_scan(int mode, const float* vecs, const float* scal, const float* vals, float* state, int n_slots,
                           const int* q_start, const int* table_rows, int n_requests, float* out, int H, int G, int D,
                           int V, int seg_len, int max_q_len, float* seg_acc, float* seg_start, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || D > kDeltaPer * kDeltaMaxSplit || n_requests > 65535 || H > 65535 ||
        (mode == 0 && (G <= 0 || H % G || !scal)) || (mode != 0 && mode != 1))
        return (int)cudaErrorInvalidValue;
    int split = 1;
    while (split * kDeltaPer < D) split *= 2;
    const bool segmented = seg_len > 0 && seg_acc && seg_start && max_q_len > seg_len;
    const int max_segs = segmented ? (max_q_len + seg_len - 1) / seg_len : 1;
    if ((long long)n_requests * max_segs > 65535) return (int)cudaErrorInvalidValue;
    const int NV = mode == 0 ? 2 : 5;
    if (mode != 0) G = H;
    // walked columns -> threads of a block, blocks, shared memory
    auto shape = [&](int columns, int* threads, dim3* grid, size_t* smem, int* chunk) {
        int th = ((columns * split + 31) / 32) * 32;
        if (th > kDeltaThreads) th = kDeltaThreads;
        const int cols = th / split;
        *threads = th;
        *grid = dim3((columns + cols - 1) / cols, H, n_requests * max_segs);
        *chunk = kDeltaChunk;
        *smem = (size_t)2 * kDeltaChunk * (NV * split * (kDeltaPer + kDeltaPad) + cols + 2) * sizeof(float);
        if (*smem > 56 * 1024) { *chunk = kDeltaChunk / 2; *smem /= 2; }
    };
    const int Dr = ((D + 31) / 32) * 32;
    auto chain = [&](auto split_c) -> int {
        constexpr int SPLIT = decltype(split_c)::value;
        const int cper = ((D + SPLIT * kChainBatch - 1) / (SPLIT * kChainBatch)) * kChainBatch;
        const size_t csm = (size_t)SPLIT * kChainRows * (cper + Dr) * sizeof(float);
        return lsb_launch(delta_chain_kernel<SPLIT>, dim3((V + kChainRows - 1) / kChainRows, H, n_requests), dim3(Dr, SPLIT),
                          csm, stream, 1, state, n_slots, (const float*)seg_acc, seg_start, q_start, table_rows, H, D, V,
                          seg_len, max_segs);
    };
#define LSB_DELTA_LAUNCH(MODE, SEG, COLUMNS)                                                                   \
    do {                                                                                                       \
        int threads, chunk; dim3 grid; size_t smem;                                                            \
        shape(COLUMNS, &threads, &grid, &smem, &chunk);                                                              \
        if (smem > 48 * 1024) {                                                                                \
            int rc = (int)cudaFuncSetAttribute(delta_scan_kernel<MODE, SEG>,                                   \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            if (rc) return rc;                                                                                 \
        }                                                                                                      \
        int rc = lsb_launch(delta_scan_kernel<MODE, SEG>, grid, dim3(threads), smem, stream, 1, vecs, scal, vals, state, \
                            n_slots, q_start, table_rows, out, H, G, D, V, split, seg_len, max_segs, seg_acc,  \
                            (const float*)seg_start, chunk);                                                          \
        if (rc) return rc;                                                                                     \
    } while (0)
#define LSB_DELTA_MODE(MODE)                                                                                   \
    do {                                                                                                       \
        if (!segmented) {                                                                                      \
            LSB_DELTA_LAUNCH(MODE, 0, V);                                                                      \
        } else {                                                                                               \
            LSB_DELTA_LAUNCH(MODE, 1, V + D);                                                                  \
            int rc = Dr <= 128 ? chain(std::integral_constant<int, 4>()) : chain(std::integral_constant<int, 2>()); \
            if (rc) return rc;                                                                                 \
            LSB_DELTA_LAUNCH(MODE, 2, V);                                                                      \
        }                                                                                                      \
    } while (0)
    if (mode == 0) LSB_DELTA_MODE(0);
    else LSB_DELTA_MODE(1);
#undef LSB_DELTA_MODE
#undef LSB_DELTA_LAUNCH
    return 0;
}

LSB_API int lsb_delta_output(const float* x, const float* w, int w_len, const void* gate, long long gate_stride,
                             int gate_act, void* out, int dtype, int tokens, int H, int V, float eps, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (H <= 0 || V <= 0 || w_len <= 0 || gate_act < 0 || gate_act > 2 || (gate_act && !gate)) return (int)cudaErrorInvalidValue;
    const long long pairs = (long long)tokens * H;
    const long long blocks = (pairs + kDeltaThreads / 32 - 1) / (kDeltaThreads / 32);
    if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(delta_output_kernel<T>, dim3((unsigned)blocks), dim3(kDeltaThreads), 0, stream, 1,
                                                x, w, w_len, (const T*)gate, gate_stride, gate_act, (T*)out, pairs, H, V, eps));
    return 0;
}

LSB_API int lsb_tanh_rows(const float* x, long long ld, int off, int n, void* out, int dtype, int rows, cudaStream_t stream) {
    const long long count = (long long)rows * n;
    if (count <= 0) return 0;
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(tanh_rows_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, 1, x, ld, off, n,
                                                (T*)out, count));
    return 0;
}
