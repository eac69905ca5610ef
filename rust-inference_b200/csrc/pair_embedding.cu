// Token embedding plus a hashed embedding of the pair (previous token, token).
//
//   x[t] = table[id_t] + pairs[row_t]                       float32 sum of the two rows
//   row_t = (id_(t-1) * mul_prev + id_t * mul_cur) mod buckets,  and row `buckets` (the table's last row) for the
//           first token of a sequence (position 0)
// The previous token of a step's first token is the sequence's last token of the step before: one int32 per cache
// slot (`last_token` [slots]), which this call brings up to date.  The read of the old value and the write of the new
// one must not meet: in a step in which every sequence brings one token the same thread does both (update_state 1);
// otherwise the main kernel only reads and a second small kernel writes afterwards.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(128)
embed_pair_hash_kernel(const int* __restrict__ ids, const T* __restrict__ table, const T* __restrict__ pairs,
                       float* __restrict__ out, int* __restrict__ last_token, const int* __restrict__ tok_seq,
                       const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                       const int* __restrict__ seq_start, int dim, int vocab, int buckets, long long mul_prev,
                       long long mul_cur, int update_state, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(err, 1);
        return;
    }
    const int b = tok_seq[t], pos = tok_pos[t];
    const int slot = seq_slot[b];
    long long row = buckets;
    if (pos > 0) {
        int prev = t > seq_start[b] ? ids[t - 1] : last_token[slot];
        if (prev < 0 || prev >= vocab) {
            if (threadIdx.x == 0) atomicExch(err, 1);
            prev = 0;
        }
        row = ((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets;
        if (row < 0) row += buckets;
    }
    const T* a = table + (size_t)id * dim;
    const T* p = pairs + (size_t)row * dim;
    float* o = out + (size_t)t * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = ld_f(a + i) + ld_f(p + i);
    if (update_state && t == seq_start[b + 1] - 1) {
        __syncthreads();                          // every thread of the block has read last_token
        if (threadIdx.x == 0) last_token[slot] = id;
    }
}

__global__ void pair_state_update_kernel(const int* __restrict__ ids, int* __restrict__ last_token,
                                         const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int seqs) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= seqs) return;
    const int end = seq_start[b + 1];
    if (end > seq_start[b]) last_token[seq_slot[b]] = ids[end - 1];
}

// single: every sequence of the step brings exactly one token
extern "C" int ri_embed_pair_hash(const int* ids, const void* table, const void* pairs, float* out, int* last_token,
                                  const int* tok_seq, const int* tok_pos, const int* seq_slot, const int* seq_start,
                                  int tokens, int seqs, int dim, int vocab, int buckets, long long mul_prev,
                                  long long mul_cur, int single, int dtype, int* err_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && seqs > 0 && dim > 0 && vocab > 0 && buckets > 0, "embed_pair_hash: bad sizes");
    RI_REQUIRE(dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16, "embed_pair_hash: unknown dtype %d", dtype);
    const int upd = single && tokens == seqs ? 1 : 0;
    if (dtype == RI_DTYPE_F32)
        ri_launch_pdl(embed_pair_hash_kernel<float>, dim3(tokens), dim3(128), 0, stream, ids, (const float*)table,
                      (const float*)pairs, out, last_token, tok_seq, tok_pos, seq_slot, seq_start, dim, vocab, buckets,
                      mul_prev, mul_cur, upd, err_flag);
    else
        ri_launch_pdl(embed_pair_hash_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, ids,
                      (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, out, last_token, tok_seq, tok_pos, seq_slot,
                      seq_start, dim, vocab, buckets, mul_prev, mul_cur, upd, err_flag);
    RI_CHECK_LAUNCH("embed_pair_hash");
    if (!upd) {
        ri_launch_pdl(pair_state_update_kernel, dim3((seqs + 127) / 128), dim3(128), 0, stream, ids, last_token, seq_slot,
                      seq_start, seqs);
        RI_CHECK_LAUNCH("pair_state_update");
    }
    return 0;
}
