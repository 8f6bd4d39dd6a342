// Latent attention: queries and keys/values that go through low-rank latents, with one rotated key part shared by all heads.
//
//   down[t] = [ dq: Rq | dkv: C + R | anything else ]        one product of the mixer's input (row stride `stride`)
//   cq = rms(dq) wq          (RMS over the Rq entries, eps inside the root)         -> the up-projection of the queries
//   c  = rms(dkv[:C]) wc                                                          -> the up-projections of keys and values
//   kr = rotate(dkv[C:])     (the shared key part; not normed)
//
// and, after the up-projections  qu[t] = [H x (D + R)],  kvu[t] = [k: H x D | v: H x Dv]:
//
//   q[h] = [ qu[h, :D] | rotate(qu[h, D:]) | 0 ]       -> q_out [T, H, DP]
//   k[h] = [ kvu.k[h]  | kr               | 0 ]       -> the cache slot of the token, head h
//   v[h] = [ kvu.v[h]  | 0 ]                           -> the cache slot
//
// so that the paged attention kernels, written for one head size DP >= max(D + R, Dv), serve it with H key/value heads.
// Rotation pairs entry 2i with 2i + 1 over the first `rot` entries of the rotated part; the angle is position x freq[i],
// computed here in float32 from the position (no table bounds the positions).  Norm statistics and the rotation are
// float32; outputs are rounded once to the activation type.  One block per token.
#include "common.cuh"
#include "range_check.cuh"

#define MIE_K_LATENT_KV 12

template <typename T>
__global__ void latent_norm_rope_kernel(const T* __restrict__ down, int64_t stride, const int* __restrict__ positions,
                                        const float* __restrict__ freq, const float* __restrict__ wq, const float* __restrict__ wc,
                                        float eps, T* __restrict__ cq, T* __restrict__ c, float* __restrict__ kr, int Rq, int C, int R,
                                        int rot) {
    __shared__ float red[33];
    pdl_enter();
    const int t = blockIdx.x;
    const T* dq = down + (int64_t)t * stride;
    const T* dkv = dq + Rq;
    float ss = 0.f;
    for (int i = threadIdx.x; i < Rq; i += blockDim.x) { const float x = to_f32<T>(dq[i]); ss += x * x; }
    const float sq = 1.0f / sqrtf(block_sum(ss, red) / (float)Rq + eps);
    ss = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) { const float x = to_f32<T>(dkv[i]); ss += x * x; }
    const float sc = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);
    for (int i = threadIdx.x; i < Rq; i += blockDim.x) cq[(int64_t)t * Rq + i] = from_f32<T>(to_f32<T>(dq[i]) * sq * wq[i]);
    for (int i = threadIdx.x; i < C; i += blockDim.x) c[(int64_t)t * C + i] = from_f32<T>(to_f32<T>(dkv[i]) * sc * wc[i]);
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        float v = to_f32<T>(dkv[C + i]);
        if (i < rot) {
            const float a = pos * freq[i >> 1];
            const float cs = cosf(a), sn = sinf(a);
            const float other = to_f32<T>(dkv[C + (i ^ 1)]);
            v = (i & 1) ? v * cs + other * sn : v * cs - other * sn;
        }
        kr[(int64_t)t * R + i] = v;
    }
}

template <typename T>
__global__ void latent_assemble_kernel(const T* __restrict__ qu, const T* __restrict__ kvu, const float* __restrict__ kr,
                                       const int* __restrict__ positions, const int* __restrict__ slots,
                                       const float* __restrict__ freq, T* __restrict__ q_out, T* __restrict__ k_cache,
                                       T* __restrict__ v_cache, int H, int D, int R, int Dv, int DP, int rot, int page_size,
                                       int64_t num_pages, int write_cache, int* report) {
    extern __shared__ float cs[];                 // cos [rot/2], sin [rot/2]
    pdl_enter();
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float a = pos * freq[i];
        cs[i] = cosf(a);
        cs[half + i] = sinf(a);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const T* q = qu + (int64_t)t * H * (D + R);
    T* qo = q_out + (int64_t)t * H * DP;
    for (int h = warp; h < H; h += nw) {
        const T* qh = q + h * (D + R);
        for (int d = lane; d < DP; d += 32) {
            float v = 0.f;
            if (d < D) v = to_f32<T>(qh[d]);
            else if (d < D + R) {
                const int i = d - D;
                v = to_f32<T>(qh[d]);
                if (i < rot) {
                    const float other = to_f32<T>(qh[D + (i ^ 1)]);
                    const float c = cs[i >> 1], s = cs[half + (i >> 1)];
                    v = (i & 1) ? v * c + other * s : v * c - other * s;
                }
            }
            qo[h * DP + d] = from_f32<T>(v);
        }
    }
    if (!write_cache) return;
    const int slot = slots[t];
    if (range_slot(slot, num_pages, page_size) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_SLOT, MIE_K_LATENT_KV, t, slot);
        return;
    }
    const int page = slot / page_size, off = slot - page * page_size;
    const T* kp = kvu + (int64_t)t * H * (D + Dv);
    const T* vp = kp + H * D;
    const float* krt = kr + (int64_t)t * R;
    for (int h = warp; h < H; h += nw) {
        const int64_t row = (((int64_t)page * H + h) * page_size + off) * DP;
        for (int d = lane; d < DP; d += 32) {
            k_cache[row + d] = d < D ? kp[h * D + d] : from_f32<T>(d < D + R ? krt[d - D] : 0.f);
            v_cache[row + d] = d < Dv ? vp[h * Dv + d] : from_f32<T>(0.f);
        }
    }
}

extern "C" int mie_latent_norm_rope(const void* down, int tag, long long stride, const int* positions, const float* freq,
                                    const float* wq, const float* wc, float eps, void* cq, void* c, float* kr, int num_tokens,
                                    int Rq, int C, int R, int rot, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (Rq <= 0 || C <= 0 || R < 0 || rot < 0 || rot > R || (rot & 1)) return MIE_ERR_BAD_ARG;
    const int threads = (Rq + C) >= 1024 ? 256 : 128;
    if (tag == MIE_F32)
        return launch_kernel(latent_norm_rope_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)down,
                             (int64_t)stride, positions, freq, wq, wc, eps, (float*)cq, (float*)c, kr, Rq, C, R, rot);
    else if (tag == MIE_BF16)
        return launch_kernel(latent_norm_rope_kernel<bf16>, dim3(num_tokens), dim3(threads), 0, stream, (const bf16*)down,
                             (int64_t)stride, positions, freq, wq, wc, eps, (bf16*)cq, (bf16*)c, kr, Rq, C, R, rot);
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_latent_assemble(const void* qu, const void* kvu, int tag, const float* kr, const int* positions, const int* slots,
                                   const float* freq, void* q_out, void* k_cache, void* v_cache, int num_tokens, int H, int D,
                                   int R, int Dv, int DP, int rot, int page_size, long long num_pages, int write_cache,
                                   cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (H <= 0 || D < 0 || R < 0 || Dv <= 0 || DP < D + R || DP < Dv || rot < 0 || rot > R || (rot & 1) || page_size <= 0)
        return MIE_ERR_BAD_ARG;
    const int threads = H * DP >= 2048 ? 256 : 128;
    if (tag == MIE_F32)
        return launch_kernel(latent_assemble_kernel<float>, dim3(num_tokens), dim3(threads), (size_t)rot * sizeof(float), stream,
                             (const float*)qu, (const float*)kvu, kr, positions, slots, freq, (float*)q_out, (float*)k_cache,
                             (float*)v_cache, H, D, R, Dv, DP, rot, page_size, (int64_t)num_pages, write_cache, g_range_report);
    else if (tag == MIE_BF16)
        return launch_kernel(latent_assemble_kernel<bf16>, dim3(num_tokens), dim3(threads), (size_t)rot * sizeof(float), stream,
                             (const bf16*)qu, (const bf16*)kvu, kr, positions, slots, freq, (bf16*)q_out, (bf16*)k_cache,
                             (bf16*)v_cache, H, D, R, Dv, DP, rot, page_size, (int64_t)num_pages, write_cache, g_range_report);
    return MIE_ERR_BAD_ARG;
}
