// Differential attention, the part after the two softmax maps: per token and query head h (of key/value group g = h / r,
// r query heads a group), with a1 and a2 the outputs of the head's two maps over the same values,
//
//   o   = a1 - lambda a2
//   o   = o * rsqrt(mean(o^2) + eps) * out_scale            (RMS over the head's Dv values, no weight)
//   out = o * sigmoid(gate[t, h])                            (one gate logit per head, if gate is given)
//
// The maps come from the paged attention kernels run over 2H query heads and 2G key heads: map m of head h = g r + i is
// their head (2g + m) r + i, so that their grouping rule "query head / r" finds key head 2g + m.  Rows of `maps` hold
// 2H heads of DP >= Dv entries, float32 (the attention kernels' float32 output: the subtraction then sees unrounded maps)
// or the activation type.  float32 arithmetic; a warp per (token, head).
#include "common.cuh"

template <typename TM, typename T>
__global__ void diff_combine_kernel(const TM* __restrict__ maps, const T* __restrict__ gate, int64_t gate_stride, T* __restrict__ out,
                                    int num_tokens, int H, int r, int Dv, int DP, float lambda, float eps, float out_scale) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)num_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const int g = h / r, i = h - g * r;
    const TM* a1 = maps + ((t * 2 * H) + (int64_t)(2 * g) * r + i) * DP;
    const TM* a2 = a1 + (int64_t)r * DP;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) {
        const float o = to_f32<TM>(a1[d]) - lambda * to_f32<TM>(a2[d]);
        ss += o * o;
    }
    float s = out_scale / sqrtf(warp_sum(ss) / (float)Dv + eps);
    if (gate) s /= 1.0f + expf(-to_f32<T>(gate[t * gate_stride + h]));
    for (int d = lane; d < Dv; d += 32)
        out[item * Dv + d] = from_f32<T>((to_f32<TM>(a1[d]) - lambda * to_f32<TM>(a2[d])) * s);
}

extern "C" int mie_diff_combine(const void* maps, int maps_tag, const void* gate, long long gate_stride, void* out, int tag, int num_tokens, int H,
                                int r, int Dv, int DP, float lambda, float eps, float out_scale, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (H <= 0 || r <= 0 || H % r || Dv <= 0 || DP < Dv) return MIE_ERR_BAD_ARG;
    const int warps = 4;
    const int64_t items = (int64_t)num_tokens * H;
    const int blocks = (int)((items + warps - 1) / warps);
    if (tag == MIE_BF16 && maps_tag == MIE_F32)
        return launch_kernel(diff_combine_kernel<float, bf16>, dim3(blocks), dim3(warps * 32), 0, stream, (const float*)maps, (const bf16*)gate,
                             (int64_t)gate_stride, (bf16*)out, num_tokens, H, r, Dv, DP, lambda, eps, out_scale);
    if (tag != maps_tag) return MIE_ERR_BAD_ARG;
    if (tag == MIE_F32)
        return launch_kernel(diff_combine_kernel<float, float>, dim3(blocks), dim3(warps * 32), 0, stream, (const float*)maps, (const float*)gate,
                             (int64_t)gate_stride, (float*)out, num_tokens, H, r, Dv, DP, lambda, eps, out_scale);
    else if (tag == MIE_BF16)
        return launch_kernel(diff_combine_kernel<bf16, bf16>, dim3(blocks), dim3(warps * 32), 0, stream, (const bf16*)maps, (const bf16*)gate,
                             (int64_t)gate_stride, (bf16*)out, num_tokens, H, r, Dv, DP, lambda, eps, out_scale);
    return MIE_ERR_BAD_ARG;
}
