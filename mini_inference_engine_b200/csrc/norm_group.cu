// The norm of a model whose stream is normed AFTER each sum (post-norm), with RMS statistics per group:
//
//   v[r, :]   = alpha * res[r, :] + coef * (b0[r, :] + b1[r, :])
//   b_k[r, :] = d_k[r, :]                                               (inner weight absent)
//             = d_k[r, :] * rsqrt(mean(d_k[r, :]^2) + eps) * iw_k[:]    (inner weight given: a branch that is RMS-normed
//                                                                         over the whole row before it is added)
//   v is cut into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps); times gw[:]
//   res[r, :] = that (float32, in place);  out[r, :] = the same, rounded to the activation type (optional)
//
// Both d_k are optional: with none, alpha = 1 and groups = 1 this is a plain RMSNorm of the stream.  With `rows`
// the inputs are gathered (output row b from stream row rows[b]) and the stream is not written: the row
// selection in front of the output head.  One block per row; the row stays in shared memory; all statistics,
// sums and products are float32.
#include "common.cuh"
#include "range_check.cuh"

#define MIE_K_NORM_GROUP 9

template <typename TO>
__global__ void stream_norm_kernel(float* __restrict__ res, float alpha, const void* __restrict__ d0,
                                   const void* __restrict__ iw0, const void* __restrict__ d1,
                                   const void* __restrict__ iw1, int d_tag, int iw_tag, float coef,
                                   const void* __restrict__ gw, int gw_tag, int groups, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int n, int num_in_rows, int* report) {
    extern __shared__ float smem[];
    float* row = smem;                 // n
    float* gstat = smem + n;           // groups
    __shared__ float red[33];
    pdl_enter();
    const int b = blockIdx.x;
    const int64_t r = rows ? rows[b] : b;
    if (rows && range_row(r, num_in_rows) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_ROW, MIE_K_NORM_GROUP, b, (int)r);
        return;
    }
    float s0 = 1.f, s1 = 1.f;
    if (d0 && iw0) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = load_tagged(d0, r * n + i, d_tag); ss += v * v; }
        s0 = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    }
    if (d1 && iw1) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = load_tagged(d1, r * n + i, d_tag); ss += v * v; }
        s1 = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    }
    float* res_row = res + r * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float add = 0.f;
        if (d0) { float v = load_tagged(d0, r * n + i, d_tag); if (iw0) v = v * s0 * load_tagged(iw0, i, iw_tag); add += v; }
        if (d1) { float v = load_tagged(d1, r * n + i, d_tag); if (iw1) v = v * s1 * load_tagged(iw1, i, iw_tag); add += v; }
        row[i] = alpha * res_row[i] + coef * add;
    }
    __syncthreads();
    // a warp per group, in turn: the order of the sum does not depend on the batch
    const int gl = n / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int g = warp; g < groups; g += nw) {
        float ss = 0.f;
        for (int i = lane; i < gl; i += 32) { const float v = row[g * gl + i]; ss += v * v; }
        ss = warp_sum(ss);
        if (lane == 0) gstat[g] = 1.0f / sqrtf(ss / (float)gl + eps);
    }
    __syncthreads();
    TO* o_row = out ? out + (int64_t)b * n : nullptr;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = row[i] * gstat[i / gl] * load_tagged(gw, i, gw_tag);
        if (!rows) res_row[i] = v;
        if (o_row) o_row[i] = from_f32<TO>(v);
    }
}

// The same with 16-byte accesses, every input read once (branches stay in shared memory between their own
// statistics and the sum): float32 branches and weights, n % 4 == 0, n / groups % 4 == 0.
template <typename TO>
__global__ void stream_norm_vec4_kernel(float* __restrict__ res, float alpha, const float* __restrict__ d0,
                                        const float* __restrict__ iw0, const float* __restrict__ d1,
                                        const float* __restrict__ iw1, float coef, const float* __restrict__ gw, int groups,
                                        float eps, TO* __restrict__ out, const int* __restrict__ rows, int n, int num_in_rows,
                                        int* report) {
    extern __shared__ float4 smem4[];
    const int n4 = n >> 2;
    float4* row = smem4;                       // n4
    float4* b0 = row + n4;                     // n4 (used when d0 has a weight of its own)
    float4* b1 = b0 + n4;                      // n4
    float* gstat = reinterpret_cast<float*>(b1 + n4);
    __shared__ float red[33];
    pdl_enter();
    const int b = blockIdx.x;
    const int64_t r = rows ? rows[b] : b;
    if (rows && range_row(r, num_in_rows) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_ROW, MIE_K_NORM_GROUP, b, (int)r);
        return;
    }
    const float4* d0v = d0 ? reinterpret_cast<const float4*>(d0 + r * n) : nullptr;
    const float4* d1v = d1 ? reinterpret_cast<const float4*>(d1 + r * n) : nullptr;
    float s0 = 1.f, s1 = 1.f;
    if (d0v && iw0) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) { const float4 v = d0v[i]; b0[i] = v; ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
        s0 = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    }
    if (d1v && iw1) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) { const float4 v = d1v[i]; b1[i] = v; ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
        s1 = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    }
    float4* res_row = reinterpret_cast<float4*>(res + r * n);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {          // a thread reads back only what it stored itself
        float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
        if (d0v) {
            float4 v = iw0 ? b0[i] : d0v[i];
            if (iw0) { const float4 w = reinterpret_cast<const float4*>(iw0)[i]; v.x *= s0 * w.x; v.y *= s0 * w.y; v.z *= s0 * w.z; v.w *= s0 * w.w; }
            add = v;
        }
        if (d1v) {
            float4 v = iw1 ? b1[i] : d1v[i];
            if (iw1) { const float4 w = reinterpret_cast<const float4*>(iw1)[i]; v.x *= s1 * w.x; v.y *= s1 * w.y; v.z *= s1 * w.z; v.w *= s1 * w.w; }
            add.x += v.x; add.y += v.y; add.z += v.z; add.w += v.w;
        }
        const float4 x = res_row[i];
        row[i] = make_float4(alpha * x.x + coef * add.x, alpha * x.y + coef * add.y, alpha * x.z + coef * add.z, alpha * x.w + coef * add.w);
    }
    __syncthreads();
    const int gl4 = n4 / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int g = warp; g < groups; g += nw) {
        float ss = 0.f;
        for (int i = lane; i < gl4; i += 32) { const float4 v = row[g * gl4 + i]; ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
        ss = warp_sum(ss);
        if (lane == 0) gstat[g] = 1.0f / sqrtf(ss / (float)(gl4 * 4) + eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        const float st = gstat[i / gl4];
        const float4 w = reinterpret_cast<const float4*>(gw)[i], x = row[i];
        const float4 v = make_float4(x.x * st * w.x, x.y * st * w.y, x.z * st * w.z, x.w * st * w.w);
        if (!rows) res_row[i] = v;
        if (out) {
            TO* o = out + (int64_t)b * n + 4 * i;
            if constexpr (sizeof(TO) == 4) {
                *reinterpret_cast<float4*>(o) = v;
            } else {
                uint2 pk;
                *reinterpret_cast<__nv_bfloat162*>(&pk.x) = __floats2bfloat162_rn(v.x, v.y);
                *reinterpret_cast<__nv_bfloat162*>(&pk.y) = __floats2bfloat162_rn(v.z, v.w);
                *reinterpret_cast<uint2*>(o) = pk;
            }
        }
    }
}

extern "C" int mie_stream_norm(float* res, float alpha, const void* d0, const void* iw0, const void* d1, const void* iw1,
                               int d_tag, int iw_tag, float coef, const void* gw, int gw_tag, int groups, float eps,
                               void* out, int out_tag, const int* rows, int num_rows, int n, int num_in_rows,
                               cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (n <= 0 || groups <= 0 || n % groups || groups > 1024) return MIE_ERR_BAD_ARG;
    const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const size_t smem4 = (size_t)(3 * n + groups) * sizeof(float);
    if (n % 4 == 0 && (n / groups) % 4 == 0 && (d_tag == MIE_F32 || (!d0 && !d1)) && (iw_tag == MIE_F32 || (!iw0 && !iw1)) &&
        gw_tag == MIE_F32 && smem4 <= 200 * 1024 && aligned(res) && aligned(d0) && aligned(d1) && aligned(iw0) && aligned(iw1) &&
        aligned(gw) && aligned(out)) {
        if (out_tag == MIE_F32) {
            if (smem4 > 48 * 1024) cudaFuncSetAttribute(stream_norm_vec4_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4);
            return launch_kernel(stream_norm_vec4_kernel<float>, dim3(num_rows), dim3(threads), smem4, stream, res, alpha, (const float*)d0,
                                 (const float*)iw0, (const float*)d1, (const float*)iw1, coef, (const float*)gw, groups, eps, (float*)out,
                                 rows, n, num_in_rows, g_range_report);
        } else if (out_tag == MIE_BF16) {
            if (smem4 > 48 * 1024) cudaFuncSetAttribute(stream_norm_vec4_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4);
            return launch_kernel(stream_norm_vec4_kernel<bf16>, dim3(num_rows), dim3(threads), smem4, stream, res, alpha, (const float*)d0,
                                 (const float*)iw0, (const float*)d1, (const float*)iw1, coef, (const float*)gw, groups, eps, (bf16*)out,
                                 rows, n, num_in_rows, g_range_report);
        }
    }
    const size_t smem = (size_t)(n + groups) * sizeof(float);
    if (smem > 200 * 1024) return MIE_ERR_TOO_LARGE;
    if (out_tag == MIE_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(stream_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(stream_norm_kernel<float>, dim3(num_rows), dim3(threads), smem, stream, res, alpha, d0, iw0, d1, iw1,
                             d_tag, iw_tag, coef, gw, gw_tag, groups, eps, (float*)out, rows, n, num_in_rows, g_range_report);
    } else if (out_tag == MIE_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(stream_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(stream_norm_kernel<bf16>, dim3(num_rows), dim3(threads), smem, stream, res, alpha, d0, iw0, d1, iw1,
                             d_tag, iw_tag, coef, gw, gw_tag, groups, eps, (bf16*)out, rows, n, num_in_rows, g_range_report);
    }
    return MIE_ERR_BAD_ARG;
}
