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
//          = sum_d (g[d] S_old[d, j]) qn[d] + u[j] (kn . qn)                   (the form the kernel computes)
// all in float32; S [dim, vdim] lives in the sequence's slot of `state` [slots, H, dim, vdim].
// What does not depend on the token before (unit vectors, decays, beta) is computed for all tokens at once by a kernel
// of its own; the recurrence kernel only walks the tokens.  There a block owns 32 value columns of one (sequence, head);
// a column is shared by four neighbouring lanes, each with a quarter of the key channels in registers.  Every sum over
// d has one order that depends on the head's size only, so the result does not depend on how a sequence's tokens were
// cut into steps.
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

// bfloat16 inputs, eight neighbouring channels per thread (16-byte loads of the inputs, of the weights in their
// transposed copy wt [taps, C], of the state; two 16-byte stores): an element's arithmetic and its order are the scalar
// kernel's.  For C, ld and col0 multiples of 8 and 16-byte aligned bases.
__global__ void __launch_bounds__(128)
short_conv_x8_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int col0, const float* __restrict__ wt,
                     float* __restrict__ y, float* __restrict__ state, const int* __restrict__ tok_seq,
                     const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int C, int taps, int update) {
    pdl_trigger();
    pdl_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    const int t = blockIdx.x;
    if (c >= C) return;
    const int b = tok_seq[t];
    const int t0 = seq_start[b];
    float* st = state + (size_t)seq_slot[b] * (taps - 1) * C + c;
    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    float cur[8];
    for (int j = 0; j < taps; j++) {
        const int r = (t - t0) - (taps - 1 - j);
        float v[8];
        if (r >= 0) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(t0 + r) * ld + col0 + c);
            const unsigned u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                v[2 * e] = __uint_as_float(u[e] << 16);
                v[2 * e + 1] = __uint_as_float(u[e] & 0xffff0000u);
            }
        } else {
            const float4 a = *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 + r) * C);
            const float4 bq = *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 + r) * C + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = bq.x; v[5] = bq.y; v[6] = bq.z; v[7] = bq.w;
        }
        const float4 w0 = *reinterpret_cast<const float4*>(wt + (size_t)j * C + c);
        const float4 w1 = *reinterpret_cast<const float4*>(wt + (size_t)j * C + c + 4);
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int e = 0; e < 8; e++) {
            acc[e] = fmaf(wv[e], v[e], acc[e]);
            cur[e] = v[e];                                        // after the last tap: the current token's inputs
        }
    }
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; e++) o[e] = dr_silu(acc[e]);
    *reinterpret_cast<float4*>(y + (size_t)t * C + c) = make_float4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<float4*>(y + (size_t)t * C + c + 4) = make_float4(o[4], o[5], o[6], o[7]);
    if (update && taps > 1) {
        for (int j = 0; j + 1 < taps - 1; j++) {
            *reinterpret_cast<float4*>(st + (size_t)j * C) = *reinterpret_cast<const float4*>(st + (size_t)(j + 1) * C);
            *reinterpret_cast<float4*>(st + (size_t)j * C + 4) = *reinterpret_cast<const float4*>(st + (size_t)(j + 1) * C + 4);
        }
        *reinterpret_cast<float4*>(st + (size_t)(taps - 2) * C) = make_float4(cur[0], cur[1], cur[2], cur[3]);
        *reinterpret_cast<float4*>(st + (size_t)(taps - 2) * C + 4) = make_float4(cur[4], cur[5], cur[6], cur[7]);
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

// wt: the weights once more as [taps, C] (may be null: then the scalar kernel runs)
extern "C" int ri_short_conv(const void* x, long long ld, int col0, const float* w, const float* wt, float* y, float* state,
                             const int* tok_seq, const int* seq_slot, const int* seq_start, int tokens, int seqs, int C,
                             int taps, int single, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && seqs > 0 && C > 0 && taps >= 1, "short_conv: bad sizes");
    RI_REQUIRE(seqs <= 65535 && C <= 65535 * 256, "short_conv: too many sequences or channels for one launch");
    RI_REQUIRE(dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16, "short_conv: unknown dtype %d", dtype);
    const int upd = single && tokens == seqs ? 1 : 0;
    const dim3 grid(tokens, (C + 255) / 256);
    const bool x8 = dtype == RI_DTYPE_BF16 && wt && C % 8 == 0 && ld % 8 == 0 && col0 % 8 == 0 &&
                    (((uintptr_t)x | (uintptr_t)wt | (uintptr_t)y | (uintptr_t)state) & 15) == 0;
    if (x8)
        ri_launch_pdl(short_conv_x8_kernel, dim3(tokens, (C / 8 + 127) / 128), dim3(128), 0, stream, (const __nv_bfloat16*)x, ld,
                      col0, wt, y, state, tok_seq, seq_slot, seq_start, C, taps, upd);
    else if (dtype == RI_DTYPE_F32)
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

// ---- what the recurrence reads, made ready for all tokens at once ------------------------------------------------------
// One block per token: q and k of every q/k head become unit vectors in place (q also times qscale), the decays
// g[h, d] = exp(-exp(A_log[h]) softplus(z[h, d] + dt_bias[h, d])), beta[h] = sigmoid(b[h]) and the products k . q of the
// unit vectors are written as float32 (`beta` [tokens, H + G]: the betas, then the products).
template <typename T>
__global__ void __launch_bounds__(128)
delta_prep_kernel(float* __restrict__ qkv, int C, int q_col, int k_col, const T* __restrict__ proj, long long ld, int b_col,
                  const T* __restrict__ z, const float* __restrict__ dt_bias, const float* __restrict__ a_log, float qscale,
                  float* __restrict__ decay, float* __restrict__ beta, int H, int G, int dim) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* row = qkv + (size_t)t * C;
    // (a token's work is spread over gridDim.y blocks when the step has few tokens)
    for (int g = blockIdx.y * 4 + warp; g < G; g += 4 * gridDim.y) {      // a warp per q/k head: both unit vectors and their product
        float* q = row + q_col + g * dim;
        float* k = row + k_col + g * dim;
        float sq = 0.0f, sk = 0.0f, qk = 0.0f;
        for (int d = lane; d < dim; d += 32) {
            sq = fmaf(q[d], q[d], sq);
            sk = fmaf(k[d], k[d], sk);
            qk = fmaf(q[d], k[d], qk);
        }
        const float iq = qscale / sqrtf(warp_sum(sq) + 1e-6f), ik = 1.0f / sqrtf(warp_sum(sk) + 1e-6f);
        qk = warp_sum(qk);
        for (int d = lane; d < dim; d += 32) {
            q[d] *= iq;
            k[d] *= ik;
        }
        if (lane == 0) beta[(size_t)t * (H + G) + H + g] = qk * iq * ik;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H * dim; i += blockDim.x * gridDim.y) {
        const float rate = expf(a_log[i / dim]);
        decay[(size_t)t * H * dim + i] = expf(-rate * dr_softplus(ld_f(z + (size_t)t * H * dim + i) + dt_bias[i]));
    }
    for (int h = blockIdx.y * blockDim.x + threadIdx.x; h < H; h += blockDim.x * gridDim.y)
        beta[(size_t)t * (H + G) + h] = 1.0f / (1.0f + expf(-ld_f(proj + (size_t)t * ld + b_col + h)));
}

// ---- the recurrence -------------------------------------------------------------------------------------------------
#ifndef DR_THREADS
#define DR_THREADS 128
#endif

// SPLIT: neighbouring lanes that share a value column (a block owns DR_THREADS / SPLIT columns); CH: key channels per
// lane (dim <= SPLIT CH; lane `part` of a column has channels 4 SPLIT i + 4 part .. + 3, so that the lanes of a column
// read neighbouring 16-byte pieces of a staged vector); GROUP: tokens staged at a time.  The recurrence is a chain from
// token to token, so a warp's time per token is what counts: many lanes per column keep the chain short (a handful of
// channels per lane, then log2(SPLIT) shuffles), and the many small blocks put warps on every SM even for one sequence.
// The next group's values are loaded into registers before the group at hand is computed and stored into the other of
// two buffers afterwards: one barrier per group, and memory works while the arithmetic runs.  A sum over d is taken in
// four partial sums per lane (channels 4 i + j into sum j), added as (s0 + s1) + (s2 + s3), then over the lanes.
// The read-out after the write, o = (S' + k u^T)^T q with S' the decayed state, is taken as S'^T q + u (k . q): both
// sums over d then run over the same S' side by side (their shuffles travel together), and the write S' + k u^T is
// off the chain to the next token's sums by one multiply-add.
template <int CH, int SPLIT, int GROUP>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ qkv, int C, int q_col, int k_col, int v_col, const float* __restrict__ decay,
                  const float* __restrict__ beta, float* __restrict__ state, float* __restrict__ o,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int H, int G, int dim, int vdim) {
    constexpr int DIMC = CH * SPLIT;
    constexpr int DR_BCOLS = DR_THREADS / SPLIT;
    constexpr int PER = (GROUP * DIMC + DR_THREADS - 1) / DR_THREADS;      // staged elements per thread and array
    constexpr int VPER = (GROUP * DR_BCOLS + DR_THREADS - 1) / DR_THREADS;
    __shared__ __align__(16) float s_g[2][GROUP][DIMC], s_k[2][GROUP][DIMC], s_q[2][GROUP][DIMC];
    __shared__ float s_v[2][GROUP][DR_BCOLS], s_beta[2][GROUP], s_kq[2][GROUP];
    static_assert(2 * GROUP <= DR_THREADS, "a thread per staged beta and per staged product");
    // (the kernel after this one is let in only when the walk is over, see below)
    const int b = blockIdx.z, h = blockIdx.y;
    const int kvh = h / (H / G);
    const int part = threadIdx.x % SPLIT, col = threadIdx.x / SPLIT;
    const int j = blockIdx.x * DR_BCOLS + col;
    const bool mine = j < vdim;
    pdl_wait();
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    float* st = state + ((size_t)seq_slot[b] * H + h) * dim * vdim;
    float S[CH];
#pragma unroll
    for (int i = 0; i < CH; i++) {
        const int d = 4 * SPLIT * (i / 4) + 4 * part + (i & 3);
        S[i] = (mine && d < dim) ? st[(size_t)d * vdim + j] : 0.0f;
    }
    float rg[PER], rk[PER], rq[PER], rv[VPER], rb = 0.0f;
    auto fetch = [&](int base) {
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = threadIdx.x + e * DR_THREADS;
            const int g = idx / DIMC, d = idx % DIMC, t = base + g;
            rg[e] = rk[e] = rq[e] = 0.0f;
            if (g < GROUP && t < t1 && d < dim) {
                rg[e] = decay[((size_t)t * H + h) * dim + d];
                rk[e] = qkv[(size_t)t * C + k_col + kvh * dim + d];
                rq[e] = qkv[(size_t)t * C + q_col + kvh * dim + d];
            }
        }
#pragma unroll
        for (int e = 0; e < VPER; e++) {
            const int idx = threadIdx.x + e * DR_THREADS;
            const int g = idx / DR_BCOLS, jj = blockIdx.x * DR_BCOLS + idx % DR_BCOLS;
            rv[e] = (g < GROUP && base + g < t1 && jj < vdim) ? qkv[(size_t)(base + g) * C + v_col + h * vdim + jj] : 0.0f;
        }
        if (threadIdx.x < 2 * GROUP) {
            const int g = threadIdx.x % GROUP;
            rb = base + g < t1 ? beta[(size_t)(base + g) * (H + G) + (threadIdx.x < GROUP ? h : H + kvh)] : 0.0f;
        }
    };
    auto store = [&](int buf) {
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = threadIdx.x + e * DR_THREADS;
            if (idx < GROUP * DIMC) {
                (&s_g[buf][0][0])[idx] = rg[e];
                (&s_k[buf][0][0])[idx] = rk[e];
                (&s_q[buf][0][0])[idx] = rq[e];
            }
        }
#pragma unroll
        for (int e = 0; e < VPER; e++) {
            const int idx = threadIdx.x + e * DR_THREADS;
            if (idx < GROUP * DR_BCOLS) (&s_v[buf][0][0])[idx] = rv[e];
        }
        if (threadIdx.x < GROUP) s_beta[buf][threadIdx.x] = rb;
        else if (threadIdx.x < 2 * GROUP) s_kq[buf][threadIdx.x - GROUP] = rb;
    };
    fetch(t0);
    int buf = 0;
    for (int base = t0; base < t1; base += GROUP) {
        store(buf);
        __syncthreads();             // this group is staged (the other buffer was last read before the barrier before)
        if (base + GROUP < t1) fetch(base + GROUP);
        const int n = min(GROUP, t1 - base);
        for (int g = 0; g < n; g++) {
            float p[4] = {0.0f, 0.0f, 0.0f, 0.0f}, a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            float4 kr[CH / 4];
#pragma unroll
            for (int i = 0; i < CH; i += 4) {
                const int at = 4 * SPLIT * (i / 4) + 4 * part;
                const float4 gg = *reinterpret_cast<const float4*>(&s_g[buf][g][at]);
                const float4 kk = *reinterpret_cast<const float4*>(&s_k[buf][g][at]);
                const float4 qq = *reinterpret_cast<const float4*>(&s_q[buf][g][at]);
                kr[i / 4] = kk;
                S[i] *= gg.x;     p[0] = fmaf(S[i], kk.x, p[0]);     a[0] = fmaf(S[i], qq.x, a[0]);
                S[i + 1] *= gg.y; p[1] = fmaf(S[i + 1], kk.y, p[1]); a[1] = fmaf(S[i + 1], qq.y, a[1]);
                S[i + 2] *= gg.z; p[2] = fmaf(S[i + 2], kk.z, p[2]); a[2] = fmaf(S[i + 2], qq.z, a[2]);
                S[i + 3] *= gg.w; p[3] = fmaf(S[i + 3], kk.w, p[3]); a[3] = fmaf(S[i + 3], qq.w, a[3]);
            }
            float pred = (p[0] + p[1]) + (p[2] + p[3]);
            float acc = (a[0] + a[1]) + (a[2] + a[3]);
#pragma unroll
            for (int sh = 1; sh < SPLIT; sh <<= 1) {
                pred += __shfl_xor_sync(0xffffffffu, pred, sh);
                acc += __shfl_xor_sync(0xffffffffu, acc, sh);
            }
            const float u = s_beta[buf][g] * (s_v[buf][g][col] - pred);
#pragma unroll
            for (int i = 0; i < CH; i += 4) {
                S[i] = fmaf(kr[i / 4].x, u, S[i]);
                S[i + 1] = fmaf(kr[i / 4].y, u, S[i + 1]);
                S[i + 2] = fmaf(kr[i / 4].z, u, S[i + 2]);
                S[i + 3] = fmaf(kr[i / 4].w, u, S[i + 3]);
            }
            acc = fmaf(u, s_kq[buf][g], acc);
            if (part == 0 && mine) o[((size_t)(base + g) * H + h) * vdim + j] = acc;
        }
        buf ^= 1;
    }
    pdl_trigger();               // the next kernel may come in once the walk is over
    if (mine) {
#pragma unroll
        for (int i = 0; i < CH; i++) {
            const int d = 4 * SPLIT * (i / 4) + 4 * part + (i & 3);
            if (d < dim) st[(size_t)d * vdim + j] = S[i];
        }
    }
}

// qkv [tokens, C] float32 (the convolution's output; its q and k columns are made unit vectors in place): q of q/k head g
// at columns q_col + g dim .., k at k_col + g dim .., v of head h at v_col + h vdim ..;  proj [tokens, ld] (compute type):
// beta's logit of head h at column b_col + h;  z [tokens, H dim] (compute type): the decay's projection, dt_bias [H dim]
// and a_log [H] float32;  decay [tokens, H dim] and beta [tokens, H + G]: float32 scratch that this call fills;
// state [slots, H, dim, vdim] float32, updated in place;  o [tokens, H, vdim] float32.
extern "C" int ri_delta_rule_recurrent(float* qkv, int C, int q_col, int k_col, int v_col, const void* proj, long long ld,
                                       int b_col, const void* z, const float* dt_bias, const float* a_log, float qscale,
                                       float* decay, float* beta, float* state, float* o, const int* seq_slot,
                                       const int* seq_start, int tokens, int seqs, int H, int G, int dim, int vdim,
                                       int single, int dtype, cudaStream_t stream) {
    if (seqs == 0 || tokens == 0) return 0;
    RI_REQUIRE(seqs > 0 && tokens > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0, "delta_rule_recurrent: bad sizes");
    RI_REQUIRE(seqs <= 65535 && H <= 65535, "delta_rule_recurrent: %d sequences, %d heads: too many for one launch", seqs, H);
    RI_REQUIRE(dim <= 512, "delta_rule_recurrent: %d key channels per head (up to 512 are built)", dim);
    const int spread = tokens >= 256 ? 1 : (H * dim + 127) / 128 > 16 ? 16 : (H * dim + 127) / 128;
    const dim3 pgrid(tokens, spread);
    if (dtype == RI_DTYPE_F32)
        ri_launch_pdl(delta_prep_kernel<float>, pgrid, dim3(128), 0, stream, qkv, C, q_col, k_col, (const float*)proj, ld,
                      b_col, (const float*)z, dt_bias, a_log, qscale, decay, beta, H, G, dim);
    else if (dtype == RI_DTYPE_BF16)
        ri_launch_pdl(delta_prep_kernel<__nv_bfloat16>, pgrid, dim3(128), 0, stream, qkv, C, q_col, k_col,
                      (const __nv_bfloat16*)proj, ld, b_col, (const __nv_bfloat16*)z, dt_bias, a_log, qscale, decay, beta, H, G, dim);
    else RI_FAIL(-1, "delta_rule_recurrent: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("delta_prep");
    // The recurrence kernel is launched the ordinary way, not as a dependent launch: its few long-lived blocks (a chain of
    // dependent instructions, one warp per scheduler) must spread one per SM, and blocks that come in while the kernel
    // before still holds most SMs pile up on the first SMs that get free and stay there (2,048 tokens of 8 heads of
    // 128 x 128: 0.97 ms as a dependent launch, 0.59 ms as an ordinary one).
#define DR_GO(CH, SPLIT, GROUP)                                                                                          \
    do {                                                                                                                 \
        const int bcols = DR_THREADS / SPLIT;                                                                            \
        const dim3 grid((vdim + bcols - 1) / bcols, H, seqs);                                                            \
        delta_rule_kernel<CH, SPLIT, GROUP><<<grid, dim3(DR_THREADS), 0, stream>>>(                                       \
            (const float*)qkv, C, q_col, k_col, v_col, (const float*)decay, (const float*)beta, state, o, seq_slot,      \
            seq_start, H, G, dim, vdim);                                                                                 \
    } while (0)
#define DR_BY_GROUP(CH, SPLIT, GROUP)                                                                                    \
    do {                                                                                                                 \
        if (single) DR_GO(CH, SPLIT, 1);                                                                                 \
        else DR_GO(CH, SPLIT, GROUP);                                                                                    \
    } while (0)
    if (dim <= 16) DR_BY_GROUP(4, 4, 16);
    else if (dim <= 32) DR_BY_GROUP(4, 8, 16);
    else if (dim <= 64) DR_BY_GROUP(4, 16, 16);
    else if (dim <= 128) DR_BY_GROUP(8, 16, 8);
    else if (dim <= 256) DR_BY_GROUP(16, 16, 4);
    else DR_BY_GROUP(32, 16, 2);
#undef DR_BY_GROUP
#undef DR_GO
    RI_CHECK_LAUNCH("delta_rule_recurrent");
    return 0;
}
