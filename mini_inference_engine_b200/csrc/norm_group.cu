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

extern "C" int mie_stream_norm(float* res, float alpha, const void* d0, const void* iw0, const void* d1, const void* iw1,
                               int d_tag, int iw_tag, float coef, const void* gw, int gw_tag, int groups, float eps,
                               void* out, int out_tag, const int* rows, int num_rows, int n, int num_in_rows,
                               cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (n <= 0 || groups <= 0 || n % groups || groups > 1024) return MIE_ERR_BAD_ARG;
    const size_t smem = (size_t)(n + groups) * sizeof(float);
    if (smem > 200 * 1024) return MIE_ERR_TOO_LARGE;
    const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
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
