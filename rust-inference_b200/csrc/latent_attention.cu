// Latent attention, the step between the projections and the attention over the cache.
//
// A token's key and value are not stored per head: the cache holds one row per token,
//     [ c (rank elements), r (rot elements) ]
// where c is the RMS-normed latent (x / sqrt(mean(x^2) + eps) * gain over the rank elements of the down
// projection) and r the rotated key part that all heads share.  With the key up-projection folded into
// the query (qa[h] = Wuk[h]^T q_plain[h], a product done before this kernel), head h's score against a
// cached row is  qa[h] . c + rot(q_turn[h]) . r,  and the weighted sum of the rows' first `rank` elements
// is what the value up-projection is applied to afterwards.  So attention runs as many query heads over ONE
// key/value head of rank + rot elements whose values are the keys themselves.
//
// This kernel, one block per (new token, head) and one more per token for the cache row (a prompt's many tokens:
// one block for all heads of a token):
//   * the row's block norms the latent, rotates the shared key part and appends the row to the token's page;
//   * a head's block writes its query row  qf[t, h] = [ qa[t, h] (rank), rot(q_turn[t, h]) (rot) ].
// Rotation: neighbouring elements (2i, 2i+1) are turned by the angle of position x frequency i; the
// table [positions, rot/2, 2] holds cos and sin (with any factor on both already in it).
// All arithmetic is float32; T (float or bfloat16) is the storage type.
//
//   proj  [tokens, ld]: the stacked projection; q of head h at columns q_col + h (dim + rot) .., its last rot
//                       elements are the part to rotate; the down projection at columns dkv_col .. + rank + rot
//   qa    [tokens, H, rank];  qf [tokens, H, rank + rot];  pool [pages, page_size, rank + rot]
#include "common.cuh"

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, long long ld, int q_col, int dkv_col,
                                   const T* __restrict__ qa, T* __restrict__ qf, T* __restrict__ pool,
                                   const int* __restrict__ page_table, const int* __restrict__ tok_seq,
                                   const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                                   const float* __restrict__ gain, float eps, const float* __restrict__ table,
                                   int table_rows, int H, int dim, int rot, int rank, int mpps, int page_size,
                                   int num_pages, int write, int heads_per_block, int* __restrict__ err) {
    __shared__ float red[33];
    pdl_trigger();
    const int t = blockIdx.x;
    const int h0 = blockIdx.y * heads_per_block;           // h0 >= H: the cache row
    const int h = h0 >= H ? H : h0;
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    pdl_wait();
    if (pos < 0 || pos >= table_rows) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        return;
    }
    const T* row = proj + (size_t)t * ld;
    const float* cs = table + (size_t)pos * rot;              // [rot/2][2]
    const int Dk = rank + rot;
    if (h == H) {
        if (!write) return;
        const int page = (pos / page_size) < mpps ? page_table[(size_t)slot * mpps + pos / page_size] : -1;
        float ss = 0.0f;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) {
            const float v = ld_f(row + dkv_col + i);
            ss += v * v;
        }
        const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)rank + eps);
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(err, 2);
            return;
        }
        T* dst = pool + ((size_t)page * page_size + pos % page_size) * Dk;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) st_f(dst + i, ld_f(row + dkv_col + i) * inv * gain[i]);
        for (int j = threadIdx.x; j < rot / 2; j += blockDim.x) {
            const float u = ld_f(row + dkv_col + rank + 2 * j), v = ld_f(row + dkv_col + rank + 2 * j + 1);
            const float c = cs[2 * j], s = cs[2 * j + 1];
            st_f(dst + rank + 2 * j, u * c - v * s);
            st_f(dst + rank + 2 * j + 1, v * c + u * s);
        }
        return;
    }
    const int h1 = min(H, h0 + heads_per_block), half = rot / 2;
    for (int idx = threadIdx.x; idx < (h1 - h0) * rank; idx += blockDim.x) {
        const int hh = h0 + idx / rank, i = idx % rank;
        qf[((size_t)t * H + hh) * Dk + i] = qa[((size_t)t * H + hh) * rank + i];
    }
    for (int idx = threadIdx.x; idx < (h1 - h0) * half; idx += blockDim.x) {
        const int hh = h0 + idx / half, j = idx % half;
        const T* qr = row + q_col + (size_t)hh * (dim + rot) + dim;
        const float u = ld_f(qr + 2 * j), v = ld_f(qr + 2 * j + 1);
        const float c = cs[2 * j], s = cs[2 * j + 1];
        T* dst = qf + ((size_t)t * H + hh) * Dk + rank;
        st_f(dst + 2 * j, u * c - v * s);
        st_f(dst + 2 * j + 1, v * c + u * s);
    }
}

extern "C" int ri_latent_prep(const void* proj, long long ld, int q_col, int dkv_col, const void* qa, void* qf, void* pool,
                              const int* page_table, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                              const float* gain, float eps, const float* table, int table_rows, int tokens, int H, int dim,
                              int rot, int rank, int mpps, int page_size, int num_pages, int write, int dtype, int* err_flag,
                              cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && H > 0 && dim >= 0 && rank > 0 && rot >= 0 && rot % 2 == 0, "latent_prep: bad sizes");
    RI_REQUIRE(rot == 0 || table, "latent_prep: a rotated part needs the table of angles");
    RI_REQUIRE(H < 65535, "latent_prep: %d heads: too many for one launch", H);
    // few tokens: a block per head, so that the step's handful of rows is spread over the SMs; many: a block per token
    const int hpb = tokens >= 256 ? H : 1;
    const int threads = 128;          // the same in both layouts: the latent norm's sum is taken over the block
#define LP_GO(T)                                                                                                             \
    ri_launch_pdl(latent_prep_kernel<T>, dim3(tokens, (H + hpb - 1) / hpb + 1), dim3(threads), 0, stream, (const T*)proj, ld, \
                  q_col, dkv_col, (const T*)qa, (T*)qf, (T*)pool, page_table, tok_seq, tok_pos, seq_slot, gain, eps, table,  \
                  table_rows, H, dim, rot, rank, mpps, page_size, num_pages, write, hpb, err_flag)
    if (dtype == RI_DTYPE_F32) LP_GO(float);
    else if (dtype == RI_DTYPE_BF16) LP_GO(__nv_bfloat16);
    else RI_FAIL(-1, "latent_prep: unknown dtype %d", dtype);
#undef LP_GO
    RI_CHECK_LAUNCH("latent_prep");
    return 0;
}
