// Token embedding with a hashed bigram table added:
//     x[t, :] = table[id_t, :] + bigram[row_t, :]
//     row_t   = (id_{t-1} * mul_prev + id_t * mul_cur) mod buckets,  or `buckets` (the table's last row) for a
//               sequence's first token
// written as the float32 residual stream.  The token before a step's first token of a sequence is per-sequence
// state: an int32 per slot, read here and renewed by last_token_kernel after this kernel (a second launch, because
// in a step of many tokens the reader and the writer of a slot's word are different blocks).  The hash is
// computed in 64 bits.  One block per token; an id outside [0, V) writes zeros and raises the error word.
#include "common.cuh"

template <typename TW>
__global__ void bigram_embedding_kernel(const int* __restrict__ ids, const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                                        const int* __restrict__ cu_q, const int* __restrict__ slots, const int* __restrict__ last_token,
                                        const TW* __restrict__ table, const TW* __restrict__ bigram, float* __restrict__ out, int H, int V,
                                        int buckets, long long mul_prev, long long mul_cur, int* __restrict__ err) {
    pdl_grid_sync();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicExch(err, 1);
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        return;
    }
    long long row = buckets;
    if (token_pos[t] > 0) {
        const int seq = token_seq[t];
        const int prev = t > cu_q[seq] ? ids[t - 1] : last_token[slots[seq]];
        row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const TW* a = table + (size_t)id * H;
    const TW* b = bigram + (size_t)row * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = to_f32(a[c]) + to_f32(b[c]);
}

__global__ void last_token_kernel(const int* __restrict__ ids, const int* __restrict__ cu_q, const int* __restrict__ slots,
                                  int* __restrict__ last_token, int B) {
    pdl_grid_sync();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) last_token[slots[b]] = ids[cu_q[b + 1] - 1];
}

extern "C" int illm_bigram_embedding(const int* ids, const int* token_pos, const int* token_seq, const int* cu_q, const int* slots,
                                     int* last_token, const void* table, const void* bigram, int table_dtype, float* out, int T, int B, int H,
                                     int V, int buckets, long long mul_prev, long long mul_cur, int* err, void* stream) {
    if (T <= 0) return 0;
    if (buckets <= 0 || B <= 0) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 2048 ? 256 : 128;
    if (table_dtype == ILLM_BF16)
        illm_launch(bigram_embedding_kernel<bf16>, dim3(T), dim3(threads), 0, s, ids, token_pos, token_seq, cu_q, slots, (const int*)last_token,
                    (const bf16*)table, (const bf16*)bigram, out, H, V, buckets, mul_prev, mul_cur, err);
    else if (table_dtype == ILLM_F32)
        illm_launch(bigram_embedding_kernel<float>, dim3(T), dim3(threads), 0, s, ids, token_pos, token_seq, cu_q, slots,
                    (const int*)last_token, (const float*)table, (const float*)bigram, out, H, V, buckets, mul_prev, mul_cur, err);
    else
        return ILLM_ERR_BAD_ARG;
    illm_launch(last_token_kernel, dim3((B + 127) / 128), dim3(128), 0, s, ids, cu_q, slots, last_token, B);
    return illm_launch_status();
}
