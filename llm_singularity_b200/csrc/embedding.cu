// Token embedding gather: out[t, :] = float(table[ids[t], :]) * scale (the product in 32-bit).
//
// Replaces the reference's embedding_lookup_kernel (kernels/src/embedding.cu:12-26),
// which copies fp32 rows; here the table is in the compute dtype and the rows are
// widened into the 32-bit residual stream.  One thread block per token.
#include "common.cuh"

LSB_DEFINE_STATUS()

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab, float scale) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) lsb_set_status(LSB_BAD_TOKEN);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = lsb_to_float(row[i]) * scale;
}

// The same with a second table added, whose row is a hash of the token and the one before it in its
// sequence: row (prev * mul_prev + token * mul_cur) mod buckets, and row `buckets` (the table's last)
// for a sequence's first token.  The token before the first of a step's portion is the request's state,
// one int per slot in `last_token`; the block of a request's first token of the step reads it and then
// leaves the portion's last token there.  The sum of the two rows is formed in 32-bit.
template <typename T>
__global__ void embedding_pair_kernel(const T* __restrict__ table, const T* __restrict__ pair_table,
                                      const int* __restrict__ ids, const int* __restrict__ positions,
                                      const int* __restrict__ token_req, const int* __restrict__ q_start,
                                      const int* __restrict__ table_rows, int* __restrict__ last_token,
                                      float* __restrict__ out, int hidden, int vocab, int buckets,
                                      long long mul_prev, long long mul_cur, int slots, float scale) {
    lsb_pdl_launch_dependents();
    lsb_pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const int r = token_req[t];
    const int first = q_start[r], end = q_start[r + 1];
    const int slot = table_rows[r];
    float* o = out + (size_t)t * hidden;
    int prev = 0;
    const bool slot_ok = slot >= 0 && slot < slots;
    if (t > first) prev = ids[t - 1];
    else if (slot_ok) prev = last_token[slot];
    if (t == first) {
        __syncthreads();                        // every thread has read the slot before one writes it
        if (threadIdx.x == 0 && slot_ok) last_token[slot] = ids[end - 1];
    }
    if (id < 0 || id >= vocab || prev < 0 || prev >= vocab || !slot_ok) {
        if (threadIdx.x == 0) lsb_set_status(slot_ok ? LSB_BAD_TOKEN : LSB_BAD_ROW);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const long long pair = positions[t] == 0 ? (long long)buckets
                                             : ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
    const T* row = table + (size_t)id * hidden;
    const T* prow = pair_table + (size_t)pair * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        o[i] = lsb_to_float(row[i]) * scale + lsb_to_float(prow[i]);
}

LSB_API int lsb_embedding_pair(const void* table, const void* pair_table, int dtype, const int* ids,
                               const int* positions, const int* token_req, const int* q_start,
                               const int* table_rows, int* last_token, float* out, int tokens, int hidden,
                               int vocab, int buckets, long long mul_prev, long long mul_cur, int slots, float scale,
                               cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (buckets <= 0 || mul_prev < 0 || mul_cur < 0) return (int)cudaErrorInvalidValue;
    int threads = hidden < 256 ? ((hidden + 31) / 32) * 32 : 256;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(embedding_pair_kernel<T>, dim3(tokens), dim3(threads), 0, stream, 1,
                                                (const T*)table, (const T*)pair_table, ids, positions, token_req,
                                                q_start, table_rows, last_token, out, hidden, vocab, buckets,
                                                mul_prev, mul_cur, slots, scale));
    return 0;
}

LSB_API int lsb_embedding(const void* table, int dtype, const int* ids, float* out,
                          int tokens, int hidden, int vocab, float scale, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    int threads = hidden < 256 ? ((hidden + 31) / 32) * 32 : 256;
    LSB_DISPATCH_DTYPE(dtype, return lsb_launch(embedding_kernel<T>, dim3(tokens), dim3(threads), 0, stream, 1,
                                                (const T*)table, ids, out, hidden, vocab, scale));
    return 0;
}
