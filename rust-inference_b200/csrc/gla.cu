// Gated linear attention: a matrix-valued state per (sequence, head) that every token decays, feeds and reads.
//
//   a_t[d] = sigmoid(z_t[d] + bias[d])^(1/tau)                     decay of key channel d, in (0, 1)
//   S_t[d, j] = a_t[d] S_(t-1)[d, j] + k_t[d] v_t[j]               state [dim, vdim], float32, zero at a sequence's start
//   o_t[j] = sum over d of S_t[d, j] (q_t[d] qscale)               d ascending, one accumulator
// then per head  y_t = o_t / sqrt(mean_j(o_t[j]^2) + eps) * gain * silu(g_t)   (`gla_head_norm_gate`).
//
// `gla_recurrent`: a block owns one (sequence, head, tile of value columns j) and walks the sequence's new
// tokens in order; a thread owns one column of the state, which lives in shared memory ([dim][tile]), and is
// loaded from / stored to the sequence's slot of the state tensor at the ends.  The decay is computed as
// exp(log_sigmoid(z) / tau) with float32 functions; q, k, v and z come from bfloat16 or float32 projections and
// are widened once.  A token's result depends on the tokens before it only through the state, so prompts,
// pieces of prompts and single tokens give the same bits.
//
//   proj [tokens, ld]: q of head h at columns q_col + h dim .., k at k_col + h dim .., v at v_col + h vdim ..
//   z    [tokens, H dim] (the low-rank decay projection, bias not yet added);  bias [H dim] float32
//   state [slots, H, dim, vdim] float32;  o [tokens, H, vdim] float32
#include "common.cuh"

#define GLA_TILE 64

__device__ __forceinline__ float gla_decay(float z, float inv_tau) {
    // log(sigmoid(z)) = min(z, 0) - log1p(exp(-|z|))
    const float ls = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
    return expf(ls * inv_tau);
}

template <typename T>
__global__ void __launch_bounds__(GLA_TILE)
gla_recurrent_kernel(const T* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, const T* __restrict__ z,
                     const float* __restrict__ bias, float inv_tau, float qscale, float* __restrict__ state,
                     float* __restrict__ o, const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int H,
                     int dim, int vdim) {
    extern __shared__ float gla_smem[];
    float* S = gla_smem;                              // [dim][GLA_TILE]
    float* tok = S + (size_t)dim * GLA_TILE;          // two buffers of [3][dim]: decay, key, query
    pdl_trigger();
    const int b = blockIdx.z, h = blockIdx.y;
    const int j = blockIdx.x * GLA_TILE + threadIdx.x;
    const bool mine = j < vdim;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    const int slot = seq_slot[b];
    pdl_wait();
    float* st = state + ((size_t)slot * H + h) * dim * vdim;
    for (int d = 0; d < dim; d++) S[d * GLA_TILE + threadIdx.x] = mine ? st[(size_t)d * vdim + j] : 0.0f;
    for (int t = t0; t < t1; t++) {
        float* cur = tok + (size_t)((t - t0) & 1) * 3 * dim;
        const T* row = proj + (size_t)t * ld;
        for (int d = threadIdx.x; d < dim; d += GLA_TILE) {
            cur[d] = gla_decay(ld_f(z + ((size_t)t * H + h) * dim + d) + bias[h * dim + d], inv_tau);
            cur[dim + d] = ld_f(row + k_col + h * dim + d);
            cur[2 * dim + d] = ld_f(row + q_col + h * dim + d) * qscale;
        }
        const float v = mine ? ld_f(row + v_col + h * vdim + j) : 0.0f;
        __syncthreads();              // the token's vectors are there (the other buffer is free again after this barrier)
        float acc = 0.0f;
        for (int d = 0; d < dim; d++) {
            const float s = fmaf(cur[d], S[d * GLA_TILE + threadIdx.x], cur[dim + d] * v);
            S[d * GLA_TILE + threadIdx.x] = s;
            acc = fmaf(s, cur[2 * dim + d], acc);
        }
        if (mine) o[((size_t)t * H + h) * vdim + j] = acc;
    }
    if (mine)
        for (int d = 0; d < dim; d++) st[(size_t)d * vdim + j] = S[d * GLA_TILE + threadIdx.x];
}

extern "C" int ri_gla_recurrent(const void* proj, long long ld, int q_col, int k_col, int v_col, const void* z,
                                const float* bias, float tau, float qscale, float* state, float* o, const int* seq_slot,
                                const int* seq_start, int seqs, int H, int dim, int vdim, int dtype, cudaStream_t stream) {
    if (seqs == 0) return 0;
    RI_REQUIRE(seqs > 0 && H > 0 && dim > 0 && vdim > 0 && tau > 0.0f, "gla_recurrent: bad sizes");
    RI_REQUIRE(seqs <= 65535 && H <= 65535, "gla_recurrent: %d sequences, %d heads: too many for one launch", seqs, H);
    const size_t smem = ((size_t)dim * GLA_TILE + 6 * (size_t)dim) * sizeof(float);
    RI_REQUIRE(smem <= 200 * 1024, "gla_recurrent: %d key channels per head do not fit in shared memory", dim);
    const dim3 grid((vdim + GLA_TILE - 1) / GLA_TILE, H, seqs);
    cudaError_t e = cudaSuccess;
#define GLA_GO(T)                                                                                                          \
    do {                                                                                                                   \
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(gla_recurrent_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) RI_FAIL((int)e, "gla_recurrent: %s", cudaGetErrorString(e));                                 \
        ri_launch_pdl(gla_recurrent_kernel<T>, grid, dim3(GLA_TILE), smem, stream, (const T*)proj, ld, q_col, k_col, v_col, \
                      (const T*)z, bias, 1.0f / tau, qscale, state, o, seq_slot, seq_start, H, dim, vdim);                 \
    } while (0)
    if (dtype == RI_DTYPE_F32) GLA_GO(float);
    else if (dtype == RI_DTYPE_BF16) GLA_GO(__nv_bfloat16);
    else RI_FAIL(-1, "gla_recurrent: unknown dtype %d", dtype);
#undef GLA_GO
    RI_CHECK_LAUNCH("gla_recurrent");
    return 0;
}

// y[t, h, j] = T( o[t, h, j] / sqrt(mean_j o[t, h, :]^2 + eps) * gain[j] * f(g[t, h vdim + j]) ),  f: silu (fn 1) or
// sigmoid (fn 0); a warp per (token, head), the sum of squares over the warp's tree.
template <typename T>
__global__ void gla_head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gain, float eps,
                                          const T* __restrict__ g, long long ldg, T* __restrict__ y, int H, int vdim,
                                          int fn, size_t units) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const size_t unit = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const size_t t = unit / H;
    const int h = (int)(unit - t * H);
    const float* op = o + unit * vdim;
    float ss = 0.0f;
    for (int j = lane; j < vdim; j += 32) ss += op[j] * op[j];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    for (int j = lane; j < vdim; j += 32) {
        const float zg = ld_f(g + t * ldg + (size_t)h * vdim + j);
        const float s = 1.0f / (1.0f + expf(-zg));
        st_f(y + unit * vdim + j, op[j] * inv * gain[j] * (fn == 1 ? zg * s : s));
    }
}

extern "C" int ri_gla_head_norm_gate(const float* o, const float* gain, float eps, const void* g, long long ldg, void* y,
                                     int tokens, int H, int vdim, int fn, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && H > 0 && vdim > 0, "gla_head_norm_gate: bad sizes");
    const size_t units = (size_t)tokens * H;
    const unsigned blocks = (unsigned)((units + 7) / 8);
    if (dtype == RI_DTYPE_F32)
        ri_launch_pdl(gla_head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, gain, eps, (const float*)g, ldg, (float*)y, H, vdim, fn, units);
    else if (dtype == RI_DTYPE_BF16)
        ri_launch_pdl(gla_head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, o, gain, eps, (const __nv_bfloat16*)g, ldg, (__nv_bfloat16*)y, H, vdim, fn, units);
    else RI_FAIL(-1, "gla_head_norm_gate: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("gla_head_norm_gate");
    return 0;
}
