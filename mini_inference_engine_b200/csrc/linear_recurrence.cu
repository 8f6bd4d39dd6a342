// The kernels of a gated linear recurrent unit with a short causal convolution in front of it:
//
//   u_t = cb + sum_j taps[:, j] * x_{t-(K-1)+j}            x before a request's first token is zero
//   r_t = sigmoid(Ra[b] u_t[b] + ra[b]),  i_t = sigmoid(Ri[b] u_t[b] + ri[b])     per block b of C / B channels
//   a_t = exp(-c * r_t * softplus(lam)),  s_t = a_t s_{t-1} + sqrt(1 - a_t^2) (i_t u_t),   s before the first token is zero
//   out_t = s_t * gelu_tanh(y_t)
//
// x and y are the two halves of one fused projection (activation type); everything from u on is float32.  Per
// request the unit keeps `state[slot]` = [K rows, C] float32: row 0 is s, rows 1 .. K-1 are the last K-1 inputs x
// of the convolution (oldest first).  Three launches:
//   conv      every (token, channel) on its own: inputs older than the portion come from the state
//   gates     a block of threads takes GATE_TT tokens of one channel block: u in shared memory, one output channel a
//             thread, both gate matrices in one pass; writes a_t and the gated input sqrt(1 - a_t^2) i_t u_t
//   scan      a request's tokens are cut into segments; every (segment, channel) thread first folds its segment
//             into (product of a, value from zero), the segments' starts follow from those in order, then each
//             segment is walked again from its start; the last one stores s, and the convolution's inputs move on
#include "common.cuh"

#define CONV_MAX_TAPS 16
#define GATE_TT 16

template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ x, int64_t x_stride, const int* __restrict__ token_row,
                                   const int* __restrict__ row_q_start, const int* __restrict__ state_slots,
                                   const void* __restrict__ taps, const void* __restrict__ bias, int w_tag,
                                   const float* __restrict__ state, float* __restrict__ u, int num_tokens, int C, int K) {
    pdl_enter();
    const int t = blockIdx.y;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= C || t >= num_tokens) return;
    const int r = token_row[t];
    const int lt = t - row_q_start[r];                       // index within the request's portion
    const float* hist = state + (int64_t)state_slots[r] * K * C + C;      // rows 1 .. K-1
    float acc = bias ? load_tagged(bias, ch, w_tag) : 0.f;
    for (int j = 0; j < K; ++j) {
        const int src = lt - (K - 1) + j;
        const float xv = src >= 0 ? to_f32<T>(x[(int64_t)(t - (K - 1) + j) * x_stride + ch])
                                  : hist[(int64_t)(src + K - 1) * C + ch];
        acc = fmaf(load_tagged(taps, (int64_t)ch * K + j, w_tag), xv, acc);
    }
    u[(int64_t)t * C + ch] = acc;
}

__global__ void recurrence_gates_kernel(const float* __restrict__ u, const void* __restrict__ wa, const void* __restrict__ ba,
                                        const void* __restrict__ wi, const void* __restrict__ bi, const void* __restrict__ lam,
                                        int w_tag, float c_exp, float* __restrict__ a_out, float* __restrict__ b_out,
                                        int num_tokens, int C, int bw) {
    extern __shared__ float u_s[];                           // [GATE_TT][bw]
    pdl_enter();
    const int blk = blockIdx.y;
    const int t0 = blockIdx.x * GATE_TT;
    const int nt = min(GATE_TT, num_tokens - t0);
    for (int i = threadIdx.x; i < GATE_TT * bw; i += blockDim.x) {
        const int tt = i / bw, k = i - tt * bw;
        u_s[i] = tt < nt ? u[(int64_t)(t0 + tt) * C + blk * bw + k] : 0.f;
    }
    __syncthreads();
    for (int o = threadIdx.x; o < bw; o += blockDim.x) {
        float ra[GATE_TT], ri[GATE_TT];
#pragma unroll
        for (int tt = 0; tt < GATE_TT; ++tt) { ra[tt] = 0.f; ri[tt] = 0.f; }
        const int64_t wrow = ((int64_t)blk * bw + o) * bw;
        for (int k = 0; k < bw; ++k) {
            const float a = load_tagged(wa, wrow + k, w_tag), b = load_tagged(wi, wrow + k, w_tag);
#pragma unroll
            for (int tt = 0; tt < GATE_TT; ++tt) {
                const float uv = u_s[tt * bw + k];
                ra[tt] = fmaf(a, uv, ra[tt]);
                ri[tt] = fmaf(b, uv, ri[tt]);
            }
        }
        const int ch = blk * bw + o;
        const float bra = load_tagged(ba, ch, w_tag), bri = load_tagged(bi, ch, w_tag);
        const float l = load_tagged(lam, ch, w_tag);
        const float sp = l > 20.f ? l : log1pf(expf(l));                  // softplus
#pragma unroll
        for (int tt = 0; tt < GATE_TT; ++tt) {
            if (tt < nt) {
                const float r = 1.0f / (1.0f + expf(-(ra[tt] + bra)));
                const float g = 1.0f / (1.0f + expf(-(ri[tt] + bri)));
                const float la = -c_exp * r * sp;
                const float a = expf(la);
                const float m = sqrtf(fmaxf(1.0f - a * a, 0.f));
                a_out[(int64_t)(t0 + tt) * C + ch] = a;
                b_out[(int64_t)(t0 + tt) * C + ch] = m * (g * u_s[tt * bw + o]);
            }
        }
    }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// blockDim = (32 channels, segments)
template <typename T>
__global__ void recurrence_scan_kernel(const float* __restrict__ a, const float* __restrict__ b, const T* __restrict__ y,
                                       int64_t y_stride, const T* __restrict__ x, int64_t x_stride,
                                       const int* __restrict__ row_q_start, const int* __restrict__ row_q_len,
                                       const int* __restrict__ state_slots, float* __restrict__ state, T* __restrict__ out,
                                       int C, int K) {
    extern __shared__ float seg_s[];                          // [2][segments][32]
    pdl_enter();
    const int r = blockIdx.y;
    const int ch = blockIdx.x * 32 + threadIdx.x;
    const int seg = threadIdx.y, nseg = blockDim.y;
    const int q_len = row_q_len[r], q_start = row_q_start[r];
    const int len = (q_len + nseg - 1) / nseg;
    const int lo = min(q_len, seg * len), hi = min(q_len, lo + len);
    const bool ok = ch < C;
    float* st = state + (int64_t)state_slots[r] * K * C;
    float* A_s = seg_s;
    float* B_s = seg_s + nseg * 32;
    float s = ok ? st[ch] : 0.f;                              // read before the barrier: the last segment overwrites it
    if (nseg > 1) {
        float A = 1.f, Bv = 0.f;
        if (ok)
            for (int t = lo; t < hi; ++t) {
                const int64_t i = (int64_t)(q_start + t) * C + ch;
                const float at = a[i];
                A *= at;
                Bv = fmaf(at, Bv, b[i]);
            }
        A_s[seg * 32 + threadIdx.x] = A;
        B_s[seg * 32 + threadIdx.x] = Bv;
        __syncthreads();
    }
    if (!ok) return;
    for (int k = 0; k < seg; ++k) s = fmaf(A_s[k * 32 + threadIdx.x], s, B_s[k * 32 + threadIdx.x]);
    for (int t = lo; t < hi; ++t) {
        const int64_t i = (int64_t)(q_start + t) * C + ch;
        s = fmaf(a[i], s, b[i]);
        out[i] = from_f32<T>(s * gelu_tanh_f(to_f32<T>(y[(int64_t)(q_start + t) * y_stride + ch])));
    }
    if (hi == q_len && lo < q_len) st[ch] = s;                // the segment that holds the last token
    if (seg == 0) {
        // the convolution's inputs move on: new row j holds the input at portion index q_len - (K-1) + j
        float keep[CONV_MAX_TAPS];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j < K - 1) {
                const int src = q_len - (K - 1) + j;
                keep[j] = src >= 0 ? to_f32<T>(x[(int64_t)(q_start + src) * x_stride + ch]) : st[(int64_t)(1 + src + K - 1) * C + ch];
            }
        }
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j < K - 1) st[(int64_t)(1 + j) * C + ch] = keep[j];
    }
}

extern "C" int mie_causal_conv(const void* x, int tag, long long x_stride, const int* token_row, const int* row_q_start,
                               const int* state_slots, const void* taps, const void* bias, int w_tag, const float* state,
                               float* u, int num_tokens, int C, int K, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (C <= 0 || K < 1 || K > CONV_MAX_TAPS) return MIE_ERR_BAD_ARG;
    const int threads = 128;
    dim3 grid((C + threads - 1) / threads, num_tokens);
    if (tag == MIE_F32)
        return launch_kernel(causal_conv_kernel<float>, grid, dim3(threads), 0, stream, (const float*)x, (int64_t)x_stride, token_row,
                             row_q_start, state_slots, taps, bias, w_tag, state, u, num_tokens, C, K);
    else if (tag == MIE_BF16)
        return launch_kernel(causal_conv_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)x, (int64_t)x_stride, token_row,
                             row_q_start, state_slots, taps, bias, w_tag, state, u, num_tokens, C, K);
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_recurrence_gates(const float* u, const void* wa, const void* ba, const void* wi, const void* bi,
                                    const void* lam, int w_tag, float c_exp, float* a_out, float* b_out, int num_tokens,
                                    int C, int blocks, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (C <= 0 || blocks <= 0 || C % blocks) return MIE_ERR_BAD_ARG;
    const int bw = C / blocks;
    const size_t smem = (size_t)GATE_TT * bw * sizeof(float);
    if (smem > 96 * 1024) return MIE_ERR_TOO_LARGE;
    if (smem > 48 * 1024) cudaFuncSetAttribute(recurrence_gates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int threads = bw >= 256 ? 256 : (bw + 31) / 32 * 32;
    dim3 grid((num_tokens + GATE_TT - 1) / GATE_TT, blocks);
    return launch_kernel(recurrence_gates_kernel, grid, dim3(threads), smem, stream, u, wa, ba, wi, bi, lam, w_tag, c_exp, a_out,
                         b_out, num_tokens, C, bw);
}

extern "C" int mie_recurrence_scan(const float* a, const float* b, const void* y, int tag, long long y_stride, const void* x,
                                   long long x_stride, const int* row_q_start, const int* row_q_len, const int* state_slots,
                                   float* state, void* out, int num_rows, int C, int K, int segments, cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (C <= 0 || K < 1 || K > CONV_MAX_TAPS || segments < 1 || segments > 32) return MIE_ERR_BAD_ARG;
    dim3 grid((C + 31) / 32, num_rows), block(32, segments);
    const size_t smem = (size_t)2 * segments * 32 * sizeof(float);
    if (tag == MIE_F32)
        return launch_kernel(recurrence_scan_kernel<float>, grid, block, smem, stream, a, b, (const float*)y, (int64_t)y_stride,
                             (const float*)x, (int64_t)x_stride, row_q_start, row_q_len, state_slots, state, (float*)out, C, K);
    else if (tag == MIE_BF16)
        return launch_kernel(recurrence_scan_kernel<bf16>, grid, block, smem, stream, a, b, (const bf16*)y, (int64_t)y_stride,
                             (const bf16*)x, (int64_t)x_stride, row_q_start, row_q_len, state_slots, state, (bf16*)out, C, K);
    return MIE_ERR_BAD_ARG;
}
