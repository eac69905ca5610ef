// The norm in front of a sublayer for a model whose residual is kept as several streams
// (hyper-connections), with everything around it in the same pass over the data.
//
// resid [n, S, dim] float32 holds S streams per token.  One block per output row does, element by element:
//   1. the update that the sublayer before left pending (its output y [n, dim], not yet added):
//          x'_t = sum over s of mix[s, t] x_s  +  outw[t] y        for every stream t, all from the old streams
//      (written back to resid, unless only some rows are read: then nothing after this call reads resid);
//   2. the sublayer's input  u = sum over t of read[t] x'_t        (read absent: the plain sum of the streams);
//   3. the norm of the row u:  layer norm without bias  (u - mean) / sqrt(var + eps) * gain,  var = mean((u - mean)^2),
//      or RMS norm  u / sqrt(mean(u^2) + eps) * gain.
// With S = 1, mix = read = outw = [1] this is the ordinary pre-norm residual: x' = x + y, u = x'.
// All of it is float32 whatever the compute type T of y and of the output; every sum has a fixed order
// (streams ascending, then the block's tree over the row), so a row's result does not depend on the batch.
#include "common.cuh"

#define SN_MAX_STREAMS 16
#define SN_KIND_LAYERNORM 0
#define SN_KIND_RMSNORM 1

// NS: the number of streams when it is 1 to 8 (the loops over streams are then unrolled over registers), 0: any
// number up to SN_MAX_STREAMS, read at run time.
template <typename T, int NS>
__global__ void __launch_bounds__(512)
stream_norm_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ mix,
                   const float* __restrict__ outw, const float* __restrict__ read, const int* __restrict__ rows,
                   const float* __restrict__ gain, T* __restrict__ out, int streams, int dim, float eps, int kind,
                   int write_back, const T* __restrict__ delta2, const float* __restrict__ outw2,
                   const T* __restrict__ delta3, const float* __restrict__ outw3, const float* __restrict__ bias) {
    constexpr int SN_CAP = NS ? NS : SN_MAX_STREAMS;
    const int S = NS ? NS : streams;
    extern __shared__ float sn_row[];                 // [dim]
    __shared__ float red[33];
    __shared__ float s_mix[SN_MAX_STREAMS * SN_MAX_STREAMS], s_out[SN_MAX_STREAMS], s_read[SN_MAX_STREAMS];
    __shared__ float s_out2[SN_MAX_STREAMS], s_out3[SN_MAX_STREAMS];
    pdl_trigger();
    // the connection weights are parameters: read before the wait for the kernel in front
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = mix ? mix[i] : (i / S == i % S ? 1.0f : 0.0f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        s_out[i] = outw ? outw[i] : 1.0f;
        s_out2[i] = outw2 ? outw2[i] : 1.0f;
        s_out3[i] = outw3 ? outw3[i] : 1.0f;
        s_read[i] = read ? read[i] : 1.0f;
    }
    pdl_wait();
    __syncthreads();
    const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* rp = resid + r * S * dim;
    const T* dp = delta ? delta + r * dim : nullptr;
    const T* dp2 = (delta && delta2) ? delta2 + r * dim : nullptr;
    const T* dp3 = (delta && delta3) ? delta3 + r * dim : nullptr;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float x[SN_CAP];
#pragma unroll
        for (int s = 0; s < SN_CAP; s++)
            if (s < S) x[s] = rp[(size_t)s * dim + i];
        float u = 0.0f;
        if (dp) {
            const float y = ld_f(dp + i);
            const float y2 = dp2 ? ld_f(dp2 + i) : 0.0f;
            const float y3 = dp3 ? ld_f(dp3 + i) : 0.0f;
#pragma unroll
            for (int t = 0; t < SN_CAP; t++)
                if (t < S) {
                    float a = 0.0f;
#pragma unroll
                    for (int s = 0; s < SN_CAP; s++)
                        if (s < S) a = fmaf(s_mix[s * S + t], x[s], a);
                    a = fmaf(s_out[t], y, a);
                    if (dp2) a = fmaf(s_out2[t], y2, a);
                    if (dp3) a = fmaf(s_out3[t], y3, a);
                    if (write_back) rp[(size_t)t * dim + i] = a;
                    u = fmaf(s_read[t], a, u);
                }
        } else {
#pragma unroll
            for (int t = 0; t < SN_CAP; t++)
                if (t < S) u = fmaf(s_read[t], x[t], u);
        }
        sn_row[i] = u;
        sum += kind == SN_KIND_LAYERNORM ? u : u * u;
    }
    float total = block_sum(sum, red);
    float mean = 0.0f, inv;
    if (kind == SN_KIND_LAYERNORM) {
        mean = total / (float)dim;
        float sq = 0.0f;
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            const float d = sn_row[i] - mean;
            sq += d * d;
        }
        inv = 1.0f / sqrtf(block_sum(sq, red) / (float)dim + eps);
    } else {
        inv = 1.0f / sqrtf(total / (float)dim + eps);
    }
    T* op = out + (size_t)blockIdx.x * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        st_f(op + i, (sn_row[i] - mean) * inv * gain[i] + (bias ? bias[i] : 0.0f));
}

// The same for rows whose length is a multiple of 4 (and 16-byte aligned data): four neighbouring elements per
// thread and trip, 16-byte loads and stores.  An element's own arithmetic is as above; the row's sums are taken
// over other partial sums, so the two kernels may differ in the last bit (which one runs depends on the row
// length and the addresses only, never on the batch).
__device__ __forceinline__ float4 sn_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 sn_ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void sn_st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void sn_st4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const unsigned*>(&a);
    u.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename T, int NS>
__global__ void __launch_bounds__(512)
stream_norm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ mix,
                       const float* __restrict__ outw, const float* __restrict__ read, const int* __restrict__ rows,
                       const float* __restrict__ gain, T* __restrict__ out, int dim, float eps, int kind, int write_back,
                       const T* __restrict__ delta2, const float* __restrict__ outw2, const T* __restrict__ delta3,
                       const float* __restrict__ outw3, const float* __restrict__ bias) {
    extern __shared__ __align__(16) float sn_row[];                 // [dim]
    __shared__ float red[33];
    __shared__ float s_mix[NS * NS], s_out[NS], s_read[NS], s_out2[NS], s_out3[NS];
    pdl_trigger();
    for (int i = threadIdx.x; i < NS * NS; i += blockDim.x) s_mix[i] = mix ? mix[i] : (i / NS == i % NS ? 1.0f : 0.0f);
    for (int i = threadIdx.x; i < NS; i += blockDim.x) {
        s_out[i] = outw ? outw[i] : 1.0f;
        s_out2[i] = outw2 ? outw2[i] : 1.0f;
        s_out3[i] = outw3 ? outw3[i] : 1.0f;
        s_read[i] = read ? read[i] : 1.0f;
    }
    const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    pdl_wait();
    __syncthreads();
    float* rp = resid + r * NS * dim;
    const T* dp = delta ? delta + r * dim : nullptr;
    const T* dp2 = (delta && delta2) ? delta2 + r * dim : nullptr;
    const T* dp3 = (delta && delta3) ? delta3 + r * dim : nullptr;
    const int nvec = dim >> 2;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float x[NS][4];
#pragma unroll
        for (int s = 0; s < NS; s++) {
            const float4 v = sn_ld4(rp + (size_t)s * dim + 4 * i);
            x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
        }
        float u[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (dp) {
            const float4 yv = sn_ld4(dp + 4 * i);
            const float y[4] = {yv.x, yv.y, yv.z, yv.w};
            float4 yv2 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (dp2) yv2 = sn_ld4(dp2 + 4 * i);
            const float y2[4] = {yv2.x, yv2.y, yv2.z, yv2.w};
            float4 yv3 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (dp3) yv3 = sn_ld4(dp3 + 4 * i);
            const float y3[4] = {yv3.x, yv3.y, yv3.z, yv3.w};
#pragma unroll
            for (int t = 0; t < NS; t++) {
                float a[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    a[e] = 0.0f;
#pragma unroll
                    for (int s = 0; s < NS; s++) a[e] = fmaf(s_mix[s * NS + t], x[s][e], a[e]);
                    a[e] = fmaf(s_out[t], y[e], a[e]);
                    if (dp2) a[e] = fmaf(s_out2[t], y2[e], a[e]);
                    if (dp3) a[e] = fmaf(s_out3[t], y3[e], a[e]);
                    u[e] = fmaf(s_read[t], a[e], u[e]);
                }
                if (write_back) sn_st4(rp + (size_t)t * dim + 4 * i, make_float4(a[0], a[1], a[2], a[3]));
            }
        } else {
#pragma unroll
            for (int t = 0; t < NS; t++)
#pragma unroll
                for (int e = 0; e < 4; e++) u[e] = fmaf(s_read[t], x[t][e], u[e]);
        }
        *reinterpret_cast<float4*>(sn_row + 4 * i) = make_float4(u[0], u[1], u[2], u[3]);
        if (kind == SN_KIND_LAYERNORM) sum += (u[0] + u[1]) + (u[2] + u[3]);
        else sum += (u[0] * u[0] + u[1] * u[1]) + (u[2] * u[2] + u[3] * u[3]);
    }
    float total = block_sum(sum, red);
    float mean = 0.0f, inv;
    if (kind == SN_KIND_LAYERNORM) {
        mean = total / (float)dim;
        float sq = 0.0f;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(sn_row + 4 * i);
            const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
            sq += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
        }
        inv = 1.0f / sqrtf(block_sum(sq, red) / (float)dim + eps);
    } else {
        inv = 1.0f / sqrtf(total / (float)dim + eps);
    }
    T* op = out + (size_t)blockIdx.x * dim;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        const float4 v = *reinterpret_cast<const float4*>(sn_row + 4 * i);
        const float4 g = sn_ld4(gain + 4 * i);
        float4 bb = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (bias) bb = sn_ld4(bias + 4 * i);
        sn_st4(op + 4 * i, make_float4((v.x - mean) * inv * g.x + bb.x, (v.y - mean) * inv * g.y + bb.y,
                                       (v.z - mean) * inv * g.z + bb.z, (v.w - mean) * inv * g.w + bb.w));
    }
}

// delta2, outw2 and delta3, outw3: further pending outputs that join in the same pass (x_t += outw2[t] delta2 + outw3[t]
// delta3, in this order after the first); bias: added to the normed row (a layer norm with a bias).  Each may be null.
extern "C" int ri_stream_norm2(float* resid, const void* delta, const float* mix, const float* outw, const float* read,
                               const int* rows, const float* gain, void* out, const void* delta2, const float* outw2,
                               const void* delta3, const float* outw3, const float* bias, int n_rows, int streams, int dim, float eps, int kind, int dtype,
                               cudaStream_t stream) {
    if (n_rows == 0) return 0;
    RI_REQUIRE(n_rows > 0 && dim > 0, "stream_norm: bad sizes rows=%d dim=%d", n_rows, dim);
    RI_REQUIRE(streams >= 1 && streams <= SN_MAX_STREAMS, "stream_norm: %d streams (1 to %d are built)", streams, SN_MAX_STREAMS);
    RI_REQUIRE(kind == SN_KIND_LAYERNORM || kind == SN_KIND_RMSNORM, "stream_norm: unknown norm %d", kind);
    const size_t smem = (size_t)dim * sizeof(float);
    RI_REQUIRE(smem <= 200 * 1024, "stream_norm: a row of %d elements does not fit in shared memory (limit 51200)", dim);
    int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
    const int write_back = rows ? 0 : 1;
    // rows of whole float4s at aligned addresses, up to 8 streams: the vector kernel
    const int unit = dtype == RI_DTYPE_F32 ? 15 : 7;
    RI_REQUIRE((delta || !delta2) && (delta2 || !delta3), "stream_norm: pending outputs are given first, second, third");
    const bool vec = dim % 4 == 0 && streams <= 8 && (((uintptr_t)resid | (uintptr_t)gain | (uintptr_t)bias) & 15) == 0 &&
                     (((uintptr_t)delta | (uintptr_t)delta2 | (uintptr_t)delta3 | (uintptr_t)out) & unit) == 0;
    if (vec) {
        const int nvec = dim / 4;
        // by the row length alone: the order of a row's additions must not depend on how many rows the step has
        threads = nvec >= 256 ? 256 : ((nvec + 31) / 32) * 32;
    }
    RI_REQUIRE(dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16, "stream_norm: unknown dtype %d", dtype);
    cudaError_t e = cudaSuccess;
#define SN_VEC(T, NS)                                                                                                    \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            e = cudaFuncSetAttribute(stream_norm_vec_kernel<T, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) RI_FAIL((int)e, "stream_norm: %s", cudaGetErrorString(e));                                 \
        ri_launch_pdl(stream_norm_vec_kernel<T, NS>, dim3(n_rows), dim3(threads), smem, stream, resid, (const T*)delta,   \
                      mix, outw, read, rows, gain, (T*)out, dim, eps, kind, write_back, (const T*)delta2, outw2,        \
                      (const T*)delta3, outw3, bias);                                                                    \
    } while (0)
#define SN_GO(T, NS)                                                                                                     \
    do {                                                                                                                 \
        if (vec && NS > 0) {                                                                                             \
            SN_VEC(T, (NS > 0 ? NS : 1));                                                                                \
            break;                                                                                                       \
        }                                                                                                                \
        if (smem > 48 * 1024)                                                                                            \
            e = cudaFuncSetAttribute(stream_norm_kernel<T, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        if (e != cudaSuccess) RI_FAIL((int)e, "stream_norm: %s", cudaGetErrorString(e));                                 \
        ri_launch_pdl(stream_norm_kernel<T, NS>, dim3(n_rows), dim3(threads), smem, stream, resid, (const T*)delta, mix,  \
                      outw, read, rows, gain, (T*)out, streams, dim, eps, kind, write_back, (const T*)delta2, outw2,     \
                      (const T*)delta3, outw3, bias);                                                                    \
    } while (0)
#define SN_BY_STREAMS(T)                                                                                                 \
    switch (streams) {                                                                                                   \
        case 1: SN_GO(T, 1); break;                                                                                      \
        case 2: SN_GO(T, 2); break;                                                                                      \
        case 3: SN_GO(T, 3); break;                                                                                      \
        case 4: SN_GO(T, 4); break;                                                                                      \
        case 5: SN_GO(T, 5); break;                                                                                      \
        case 6: SN_GO(T, 6); break;                                                                                      \
        case 7: SN_GO(T, 7); break;                                                                                      \
        case 8: SN_GO(T, 8); break;                                                                                      \
        default: SN_GO(T, 0); break;                                                                                     \
    }
    if (dtype == RI_DTYPE_F32) SN_BY_STREAMS(float)
    else SN_BY_STREAMS(__nv_bfloat16)
#undef SN_BY_STREAMS
#undef SN_GO
#undef SN_VEC
    RI_CHECK_LAUNCH("stream_norm");
    return 0;
}

extern "C" int ri_stream_norm(float* resid, const void* delta, const float* mix, const float* outw, const float* read,
                              const int* rows, const float* gain, void* out, int n_rows, int streams, int dim, float eps,
                              int kind, int dtype, cudaStream_t stream) {
    return ri_stream_norm2(resid, delta, mix, outw, read, rows, gain, out, nullptr, nullptr, nullptr, nullptr, nullptr, n_rows, streams, dim,
                           eps, kind, dtype, stream);
}
