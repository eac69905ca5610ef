// The gated delta rule: a recurrent mixer with a matrix-valued state per (sequence, head), and the short causal
// convolution in front of it.
//
// `short_conv`: per channel c a convolution over time with `taps` weights w[c, 0 .. taps-1] (the last one is the
// current token's), zeros before a sequence's start, then silu:
//     y_t[c] = silu( sum_j w[c, j] x_(t - (taps-1-j))[c] )                    float32, j ascending
// The inputs of a sequence's last taps-1 tokens are its state ([slots, taps-1, C] float32, oldest first), so a prompt,
// its pieces and single tokens give the same bits.  x is a block of columns of a projection (compute type T).
//
// `delta_rule_recurrent`: per head h with q/k head h / (H / G), for every new token in order
//     qn = q / sqrt(sum q^2 + 1e-6) * qscale,   kn = k / sqrt(sum k^2 + 1e-6)
//     g[d] = exp(-exp(A_log[h]) * softplus(z[h, d] + dt_bias[h, d]))          decay of key channel d
//     beta = sigmoid(b[h])
//     S[d, j] <- g[d] S[d, j];   u[j] = beta (v[j] - sum_d S[d, j] kn[d]);   S[d, j] <- S[d, j] + kn[d] u[j]
//     o[j] = sum_d S[d, j] qn[d]                                              (reads the current token's write)
// all in float32; S [dim, vdim] lives in the sequence's slot of `state` [slots, H, dim, vdim].
// A block owns 32 value columns of one (sequence, head); a column is shared by four neighbouring lanes, each with a
// quarter of the key channels in registers (channel d = part + 4 i).  The block stages GROUP tokens at a time in
// shared memory (normalised q and k, decay, beta, values); the sums over d are taken over each lane's channels in
// ascending order and then over the four lanes by two shuffles, an order that depends on the head's size only, so the
// result does not depend on how a sequence's tokens were cut into steps.
#include "common.cuh"

__device__ __forceinline__ float dr_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float dr_softplus(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

template <typename T>
__global__ void __launch_bounds__(256)
short_conv_kernel(const T* __restrict__ x, long long ld, int col0, const float* __restrict__ w, float* __restrict__ y,
                  float* __restrict__ state, const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_start, int tokens, int C, int taps, int update) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= C) return;
    const int b = tok_seq[t];
    const int t0 = seq_start[b];
    const int slot = seq_slot[b];
    float* st = state + (size_t)slot * (taps - 1) * C + c;
    float acc = 0.0f;
    for (int j = 0; j < taps; j++) {
        const int r = (t - t0) - (taps - 1 - j);                 // index among the step's tokens of this sequence
        const float v = r >= 0 ? ld_f(x + (size_t)(t0 + r) * ld + col0 + c) : st[(size_t)(taps - 1 + r) * C];
        acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    y[(size_t)t * C + c] = dr_silu(acc);
    if (update) {                                                // one token per sequence: this thread alone owns st
        for (int j = 0; j + 1 < taps - 1; j++) st[(size_t)j * C] = st[(size_t)(j + 1) * C];
        if (taps > 1) st[(size_t)(taps - 2) * C] = ld_f(x + (size_t)t * ld + col0 + c);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const T* __restrict__ x, long long ld, int col0, float* __restrict__ state,
                        const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= C) return;
    const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
    float* st = state + (size_t)seq_slot[b] * (taps - 1) * C + c;
    for (int j = 0; j < taps - 1; j++) {                         // ascending: an old entry is read before it is overwritten
        const int r = n - (taps - 1) + j;
        st[(size_t)j * C] = r >= 0 ? ld_f(x + (size_t)(t0 + r) * ld + col0 + c) : st[(size_t)(j + n) * C];
    }
}

extern "C" int ri_short_conv(const void* x, long long ld, int col0, const float* w, float* y, float* state,
                             const int* tok_seq, const int* seq_slot, const int* seq_start, int tokens, int seqs, int C,
                             int taps, int single, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && seqs > 0 && C > 0 && taps >= 1, "short_conv: bad sizes");
    RI_REQUIRE(seqs <= 65535 && C <= 65535 * 256, "short_conv: too many sequences or channels for one launch");
    RI_REQUIRE(dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16, "short_conv: unknown dtype %d", dtype);
    const int upd = single && tokens == seqs ? 1 : 0;
    const dim3 grid(tokens, (C + 255) / 256);
    if (dtype == RI_DTYPE_F32)
        ri_launch_pdl(short_conv_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, ld, col0, w, y, state, tok_seq,
                      seq_slot, seq_start, tokens, C, taps, upd);
    else
        ri_launch_pdl(short_conv_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)x, ld, col0, w, y,
                      state, tok_seq, seq_slot, seq_start, tokens, C, taps, upd);
    RI_CHECK_LAUNCH("short_conv");
    if (!upd && taps > 1) {
        const dim3 g2((C + 255) / 256, seqs);
        if (dtype == RI_DTYPE_F32)
            ri_launch_pdl(short_conv_state_kernel<float>, g2, dim3(256), 0, stream, (const float*)x, ld, col0, state, seq_slot,
                          seq_start, C, taps);
        else
            ri_launch_pdl(short_conv_state_kernel<__nv_bfloat16>, g2, dim3(256), 0, stream, (const __nv_bfloat16*)x, ld, col0,
                          state, seq_slot, seq_start, C, taps);
        RI_CHECK_LAUNCH("short_conv_state");
    }
    return 0;
}

// ---- the recurrence -------------------------------------------------------------------------------------------------
#define DR_SPLIT 4                  // lanes that share a value column
#define DR_BCOLS 32                 // value columns per block
#define DR_THREADS (DR_SPLIT * DR_BCOLS)

// CH: key channels per lane (dim <= 4 CH); GROUP: tokens staged at a time
template <typename T, int CH, int GROUP>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ qkv, int C, int q_col, int k_col, int v_col, const T* __restrict__ proj,
                  long long ld, int b_col, const T* __restrict__ z, const float* __restrict__ dt_bias,
                  const float* __restrict__ a_log, float qscale, float* __restrict__ state, float* __restrict__ o,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int H, int G, int dim, int vdim) {
    constexpr int DIMC = CH * DR_SPLIT;
    __shared__ float s_g[GROUP][DIMC], s_k[GROUP][DIMC], s_q[GROUP][DIMC], s_v[GROUP][DR_BCOLS], s_beta[GROUP];
    pdl_trigger();
    const int b = blockIdx.z, h = blockIdx.y;
    const int kvh = h / (H / G);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int part = threadIdx.x % DR_SPLIT, col = threadIdx.x / DR_SPLIT;
    const int j = blockIdx.x * DR_BCOLS + col;
    const bool mine = j < vdim;
    const float rate = expf(a_log[h]);
    pdl_wait();
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    float* st = state + ((size_t)seq_slot[b] * H + h) * dim * vdim;
    float S[CH];
#pragma unroll
    for (int i = 0; i < CH; i++) {
        const int d = part + DR_SPLIT * i;
        S[i] = (mine && d < dim) ? st[(size_t)d * vdim + j] : 0.0f;
    }
    for (int base = t0; base < t1; base += GROUP) {
        __syncthreads();                                         // the group before has been used
        // a warp stages a token: unit vectors of q and k, the decays, beta
        for (int g = warp; g < GROUP; g += DR_THREADS / 32) {
            const int t = base + g;
            if (t >= t1) break;
            const float* row = qkv + (size_t)t * C;
            float sq = 0.0f, sk = 0.0f;
            for (int d = lane; d < dim; d += 32) {
                const float qv = row[q_col + kvh * dim + d], kv = row[k_col + kvh * dim + d];
                sq = fmaf(qv, qv, sq);
                sk = fmaf(kv, kv, sk);
            }
            const float iq = qscale / sqrtf(warp_sum(sq) + 1e-6f), ik = 1.0f / sqrtf(warp_sum(sk) + 1e-6f);
            for (int d = lane; d < DIMC; d += 32) {
                const bool in = d < dim;
                s_q[g][d] = in ? row[q_col + kvh * dim + d] * iq : 0.0f;
                s_k[g][d] = in ? row[k_col + kvh * dim + d] * ik : 0.0f;
                s_g[g][d] = in ? expf(-rate * dr_softplus(ld_f(z + ((size_t)t * H + h) * dim + d) + dt_bias[h * dim + d])) : 0.0f;
            }
            if (lane == 0) s_beta[g] = 1.0f / (1.0f + expf(-ld_f(proj + (size_t)t * ld + b_col + h)));
        }
        for (int i = threadIdx.x; i < GROUP * DR_BCOLS; i += DR_THREADS) {
            const int g = i / DR_BCOLS, cc = i % DR_BCOLS, jj = blockIdx.x * DR_BCOLS + cc;
            s_v[g][cc] = (base + g < t1 && jj < vdim) ? qkv[(size_t)(base + g) * C + v_col + h * vdim + jj] : 0.0f;
        }
        __syncthreads();
        const int n = min(GROUP, t1 - base);
        for (int g = 0; g < n; g++) {
            float pred = 0.0f;
#pragma unroll
            for (int i = 0; i < CH; i++) {
                const int d = part + DR_SPLIT * i;
                S[i] *= s_g[g][d];
                pred = fmaf(S[i], s_k[g][d], pred);
            }
            pred += __shfl_xor_sync(0xffffffffu, pred, 1);
            pred += __shfl_xor_sync(0xffffffffu, pred, 2);
            const float u = s_beta[g] * (s_v[g][col] - pred);
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < CH; i++) {
                const int d = part + DR_SPLIT * i;
                S[i] = fmaf(s_k[g][d], u, S[i]);
                acc = fmaf(S[i], s_q[g][d], acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0 && mine) o[((size_t)(base + g) * H + h) * vdim + j] = acc;
        }
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < CH; i++) {
            const int d = part + DR_SPLIT * i;
            if (d < dim) st[(size_t)d * vdim + j] = S[i];
        }
    }
}

// qkv [tokens, C] float32 (the convolution's output): q of q/k head g at columns q_col + g dim .., k at k_col + g dim ..,
// v of head h at v_col + h vdim ..;  proj [tokens, ld] (compute type): beta's logit of head h at column b_col + h;
// z [tokens, H dim] (compute type): the decay's projection, dt_bias [H dim] and a_log [H] float32;
// state [slots, H, dim, vdim] float32, updated in place;  o [tokens, H, vdim] float32.
extern "C" int ri_delta_rule_recurrent(const float* qkv, int C, int q_col, int k_col, int v_col, const void* proj,
                                       long long ld, int b_col, const void* z, const float* dt_bias, const float* a_log,
                                       float qscale, float* state, float* o, const int* seq_slot, const int* seq_start,
                                       int seqs, int H, int G, int dim, int vdim, int single, int dtype,
                                       cudaStream_t stream) {
    if (seqs == 0) return 0;
    RI_REQUIRE(seqs > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0, "delta_rule_recurrent: bad sizes");
    RI_REQUIRE(seqs <= 65535 && H <= 65535, "delta_rule_recurrent: %d sequences, %d heads: too many for one launch", seqs, H);
    RI_REQUIRE(dim <= 256, "delta_rule_recurrent: %d key channels per head (up to 256 are built)", dim);
    RI_REQUIRE(dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16, "delta_rule_recurrent: unknown dtype %d", dtype);
    const dim3 grid((vdim + DR_BCOLS - 1) / DR_BCOLS, H, seqs);
#define DR_GO(T, CH, GROUP)                                                                                              \
    ri_launch_pdl(delta_rule_kernel<T, CH, GROUP>, grid, dim3(DR_THREADS), 0, stream, qkv, C, q_col, k_col, v_col,        \
                  (const T*)proj, ld, b_col, (const T*)z, dt_bias, a_log, qscale, state, o, seq_slot, seq_start, H, G,   \
                  dim, vdim)
#define DR_BY_GROUP(T, CH)                                                                                               \
    do {                                                                                                                 \
        if (single) DR_GO(T, CH, 1);                                                                                     \
        else DR_GO(T, CH, (CH > 32 ? 4 : 8));                                                                            \
    } while (0)
#define DR_BY_DIM(T)                                                                                                     \
    do {                                                                                                                 \
        if (dim <= 32) DR_BY_GROUP(T, 8);                                                                                \
        else if (dim <= 64) DR_BY_GROUP(T, 16);                                                                          \
        else if (dim <= 128) DR_BY_GROUP(T, 32);                                                                         \
        else DR_BY_GROUP(T, 64);                                                                                         \
    } while (0)
    if (dtype == RI_DTYPE_F32) DR_BY_DIM(float);
    else DR_BY_DIM(__nv_bfloat16);
#undef DR_BY_DIM
#undef DR_BY_GROUP
#undef DR_GO
    RI_CHECK_LAUNCH("delta_rule_recurrent");
    return 0;
}
