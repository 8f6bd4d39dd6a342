// Linear attention with a fixed decay per head and no softmax or denominator, as a recurrence over a
// float32 state per request and head (prompt portions and single tokens through the same kernel):
//
//   S_t = gamma_h * S_{t-1} + k_t v_t^T        S: [D, Dv],  S before a request's first token is zero
//   o_t = S_t^T q_t
//
// q and k are read from the fused projection [ q: H x D | k: H x D | v: H x Dv | ... ] and rotated here
// (rotate-half pairing over the first `rot` dims, angle = position * freq[i], float32), k is multiplied by
// `k_scale` after the rotation.  The state lives in `state[slot, h, c, d]` (value column c, key dimension d:
// transposed, so that the threads that share a column read neighbouring words).
//
// Work split: one block = one request, one head and a slice of value columns.  A column's state is held in the
// registers of P threads of one warp (thread p holds the key dimensions p, p + P, p + 2P, ...: up to RET_DPT of
// them), which add up their parts of o_t by shuffles.  Tokens are staged in shared memory RET_TT at a time.
// Everything is float32.
//
// The second kernel finishes the mixer's head stage: every head's o is divided by its root mean square (no
// weight) and multiplied by silu(g), g being another part of the fused projection.
#include "common.cuh"

#define RET_DPT 16      // key dimensions per thread
#define RET_TT 8        // tokens staged at a time

template <typename T>
__global__ void retention_scan_kernel(const T* __restrict__ qkv, int64_t stride, const int* __restrict__ row_q_start,
                                      const int* __restrict__ row_q_len, const int* __restrict__ row_ctx_len,
                                      const int* __restrict__ state_slots, const float* __restrict__ decay,
                                      const float* __restrict__ freq, float k_scale, float* __restrict__ state,
                                      float* __restrict__ out, int H, int D, int Dv, int rot, int P, int CW, int slices) {
    extern __shared__ float smem[];
    float* q_s = smem;                       // [RET_TT][D]
    float* k_s = q_s + RET_TT * D;           // [RET_TT][D]
    float* v_s = k_s + RET_TT * D;           // [RET_TT][CW]
    pdl_enter();
    const int r = blockIdx.y;
    const int h = blockIdx.x / slices, slice = blockIdx.x - h * slices;
    const int q_len = row_q_len[r], q_start = row_q_start[r], pos0 = row_ctx_len[r] - q_len;
    const int p = threadIdx.x % P, cl = threadIdx.x / P;
    const int c = slice * CW + cl;                                  // this thread's value column
    const bool col_ok = cl < CW && c < Dv;
    const float gamma = decay[h];
    const int half = rot >> 1;
    float* st = state + (((int64_t)state_slots[r] * H + h) * Dv + (col_ok ? c : 0)) * D;
    float S[RET_DPT];
#pragma unroll
    for (int j = 0; j < RET_DPT; ++j) {
        const int d = p + P * j;
        S[j] = (col_ok && d < D) ? st[d] : 0.f;
    }
    for (int t0 = 0; t0 < q_len; t0 += RET_TT) {
        const int nt = min(RET_TT, q_len - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * D; i += blockDim.x) {
            const int tt = i / D, d = i - tt * D;
            const T* src = qkv + (int64_t)(q_start + t0 + tt) * stride + h * D;
            float qo = to_f32<T>(src[d]), ko = to_f32<T>(src[H * D + d]);
            if (d < rot) {
                const int pd = d < half ? d + half : d - half;
                const float a = (float)(pos0 + t0 + tt) * freq[d < half ? d : d - half];
                const float cs = cosf(a), sn = sinf(a);
                const float qp = to_f32<T>(src[pd]), kp = to_f32<T>(src[H * D + pd]);
                qo = d < half ? qo * cs - qp * sn : qo * cs + qp * sn;
                ko = d < half ? ko * cs - kp * sn : ko * cs + kp * sn;
            }
            q_s[tt * D + d] = qo;
            k_s[tt * D + d] = ko * k_scale;
        }
        for (int i = threadIdx.x; i < nt * CW; i += blockDim.x) {
            const int tt = i / CW, cc = i - tt * CW;
            const int col = slice * CW + cc;
            v_s[tt * CW + cc] = col < Dv ? to_f32<T>(qkv[(int64_t)(q_start + t0 + tt) * stride + 2 * H * D + h * Dv + col]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vv = cl < CW ? v_s[tt * CW + cl] : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < RET_DPT; ++j) {
                const int d = p + P * j;
                if (d < D) {
                    S[j] = fmaf(gamma, S[j], k_s[tt * D + d] * vv);
                    acc = fmaf(S[j], q_s[tt * D + d], acc);
                }
            }
            for (int o = P >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (p == 0 && col_ok) out[(int64_t)(q_start + t0 + tt) * H * Dv + h * Dv + c] = acc;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int j = 0; j < RET_DPT; ++j) {
            const int d = p + P * j;
            if (d < D) st[d] = S[j];
        }
    }
}

// out[t, h, :] = o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * silu(g[t, h, :]); a warp per (token, head)
template <typename T>
__global__ void head_rms_gate_kernel(const float* __restrict__ o, const T* __restrict__ g, int64_t g_stride, T* __restrict__ out,
                                     int num_tokens, int H, int Dv, float eps) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)num_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const float* src = o + item * Dv;
    float ss = 0.f;
    for (int i = lane; i < Dv; i += 32) { const float v = src[i]; ss += v * v; }
    const float s = 1.0f / sqrtf(warp_sum(ss) / (float)Dv + eps);
    const T* gate = g + t * g_stride + h * Dv;
    for (int i = lane; i < Dv; i += 32) {
        const float z = to_f32<T>(gate[i]);
        out[item * Dv + i] = from_f32<T>(src[i] * s * (z / (1.0f + expf(-z))));
    }
}

extern "C" int mie_retention_scan(const void* qkv, int tag, long long stride, const int* row_q_start, const int* row_q_len,
                                  const int* row_ctx_len, const int* state_slots, const float* decay, const float* freq,
                                  float k_scale, float* state, float* out, int num_rows, int H, int D, int Dv, int rot,
                                  cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (H <= 0 || D <= 0 || Dv <= 0 || rot < 0 || rot > D || (rot & 1)) return MIE_ERR_BAD_ARG;
    int P = 1;
    while (P * RET_DPT < D) P <<= 1;
    if (P > 32) return MIE_ERR_TOO_LARGE;                      // key dimensions beyond 32 x RET_DPT
    int CW = 256 / P;
    if (CW > Dv) CW = Dv;
    const int slices = (Dv + CW - 1) / CW;
    const int threads = (CW * P + 31) / 32 * 32;
    const size_t smem = (size_t)RET_TT * (2 * D + CW) * sizeof(float);
    dim3 grid(H * slices, num_rows);
    if (tag == MIE_F32)
        return launch_kernel(retention_scan_kernel<float>, grid, dim3(threads), smem, stream, (const float*)qkv, (int64_t)stride,
                             row_q_start, row_q_len, row_ctx_len, state_slots, decay, freq, k_scale, state, out, H, D, Dv, rot, P, CW, slices);
    else if (tag == MIE_BF16)
        return launch_kernel(retention_scan_kernel<bf16>, grid, dim3(threads), smem, stream, (const bf16*)qkv, (int64_t)stride,
                             row_q_start, row_q_len, row_ctx_len, state_slots, decay, freq, k_scale, state, out, H, D, Dv, rot, P, CW, slices);
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_head_rms_gate(const float* o, const void* g, int tag, long long g_stride, void* out, int num_tokens, int H,
                                 int Dv, float eps, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (H <= 0 || Dv <= 0) return MIE_ERR_BAD_ARG;
    const int warps = 4;
    const int64_t items = (int64_t)num_tokens * H;
    const int blocks = (int)((items + warps - 1) / warps);
    if (tag == MIE_F32)
        return launch_kernel(head_rms_gate_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, o, (const float*)g,
                             (int64_t)g_stride, (float*)out, num_tokens, H, Dv, eps);
    else if (tag == MIE_BF16)
        return launch_kernel(head_rms_gate_kernel<bf16>, dim3(blocks), dim3(warps * 32), 0, stream, o, (const bf16*)g,
                             (int64_t)g_stride, (bf16*)out, num_tokens, H, Dv, eps);
    return MIE_ERR_BAD_ARG;
}
