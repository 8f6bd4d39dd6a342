// A routed mixture of experts: the router's choice, and the experts' activation for the form in which all experts are
// one wide feed-forward.
//
//   route      per token, from float32 router logits z [T, E]: the `top` experts with the largest logits (ties: the lower
//              index first), weights = softmax over the chosen logits only.  ids [T, top] int32, wts [T, top] float32.
//   dense_act  with up[t] = [expert 0: F | expert 1: F | ...] the up-projections of ALL experts (one product with the
//              experts' matrices stacked): act[t, e, :] = weight(t, e) f(up[t, e, :]) for a chosen expert, 0 for the others,
//              so that one product with the experts' down matrices side by side gives the weighted sum of the chosen
//              experts' outputs.  f: 0 relu(x)^2, 1 silu, 2 gelu (tanh form).
#include "common.cuh"

__global__ void moe_route_kernel(const float* __restrict__ z, int* __restrict__ ids, float* __restrict__ wts, int num_tokens, int E,
                                 int top) {
    pdl_enter();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= num_tokens) return;
    const float* zt = z + (int64_t)t * E;
    float prev_v = INFINITY;
    int prev_i = -1;
    float first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int bi = -1;
        for (int e = 0; e < E; ++e) {
            const float v = zt[e];
            const bool after_prev = v < prev_v || (v == prev_v && e > prev_i);      // not chosen yet
            if (after_prev && (bi < 0 || v > best)) { best = v; bi = e; }
        }
        if (bi < 0) { bi = 0; best = -INFINITY; }              // logits that are not numbers: keep the ids in range
        if (k == 0) first = best;
        const float p = expf(best - first);
        ids[(int64_t)t * top + k] = bi;
        wts[(int64_t)t * top + k] = p;
        sum += p;
        prev_v = best;
        prev_i = bi;
    }
    for (int k = 0; k < top; ++k) wts[(int64_t)t * top + k] /= sum;
}

__device__ __forceinline__ float expert_act(float x, int kind) {
    if (kind == 0) { const float r = fmaxf(x, 0.f); return r * r; }
    if (kind == 1) return x / (1.0f + expf(-x));
    return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

template <typename T>
__global__ void moe_dense_act_kernel(const T* __restrict__ up, const int* __restrict__ ids, const float* __restrict__ wts,
                                     T* __restrict__ act, int64_t total, int E, int F, int top, int kind) {
    pdl_enter();
    const int64_t EF = (int64_t)E * F;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / EF;
        const int e = (int)((idx - t * EF) / F);
        float w = 0.f;
        for (int k = 0; k < top; ++k)
            if (ids[t * top + k] == e) w = wts[t * top + k];
        act[idx] = from_f32<T>(w != 0.f ? w * expert_act(to_f32<T>(up[idx]), kind) : 0.f);
    }
}

extern "C" int mie_moe_route(const float* z, int* ids, float* wts, int num_tokens, int E, int top, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E) return MIE_ERR_BAD_ARG;
    const int threads = 64;
    return launch_kernel(moe_route_kernel, dim3((num_tokens + threads - 1) / threads), dim3(threads), 0, stream, z, ids, wts, num_tokens,
                         E, top);
}

extern "C" int mie_moe_dense_act(const void* up, const int* ids, const float* wts, void* act, int tag, int num_tokens, int E, int F,
                                 int top, int kind, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (E <= 0 || F <= 0 || top <= 0 || kind < 0 || kind > 2) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)num_tokens * E * F;
    const int threads = 256;
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > (int64_t)device_sm_count() * 16) blocks = (int64_t)device_sm_count() * 16;
    if (tag == MIE_F32)
        return launch_kernel(moe_dense_act_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)up, ids, wts,
                             (float*)act, total, E, F, top, kind);
    else if (tag == MIE_BF16)
        return launch_kernel(moe_dense_act_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)up, ids, wts,
                             (bf16*)act, total, E, F, top, kind);
    return MIE_ERR_BAD_ARG;
}
