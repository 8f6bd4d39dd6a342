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
//   gates     both block-diagonal gate matrices in one tiled float32 product on CUDA cores (weights read as float32);
//             writes a_t and the gated input sqrt(1 - a_t^2) i_t u_t
//   scan      a request's tokens are cut into segments; every (segment, channel) thread first folds its segment
//             into (product of a, value from zero), the segments' starts follow from those in order, then each
//             segment is walked again from its start; the last one stores s, and the convolution's inputs move on
#include "common.cuh"

#define CONV_MAX_TAPS 8

#define CONV_TOKENS 8         // consecutive tokens a thread computes (their inputs overlap and come from the L1 cache)
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ x, int64_t x_stride, const int* __restrict__ token_row,
                                   const int* __restrict__ row_q_start, const int* __restrict__ state_slots,
                                   const float* __restrict__ taps, const float* __restrict__ bias,
                                   const float* __restrict__ state, float* __restrict__ u, int num_tokens, int C, int K) {
    pdl_enter();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= C) return;
    float w[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) w[j] = j < K ? taps[(int64_t)ch * K + j] : 0.f;
    const float cb = bias ? bias[ch] : 0.f;
#pragma unroll
    for (int n = 0; n < CONV_TOKENS; ++n) {
        const int t = blockIdx.y * CONV_TOKENS + n;
        if (t >= num_tokens) break;
        const int r = token_row[t];
        const int lt = t - row_q_start[r];                       // index within the request's portion
        const float* hist = state + (int64_t)state_slots[r] * K * C + C;      // rows 1 .. K-1
        float acc = cb;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j < K) {
                const int src = lt - (K - 1) + j;
                const float xv = src >= 0 ? to_f32<T>(x[(int64_t)(t - (K - 1) + j) * x_stride + ch])
                                          : hist[(int64_t)(src + K - 1) * C + ch];
                acc = fmaf(w[j], xv, acc);
            }
        }
        u[(int64_t)t * C + ch] = acc;
    }
}

// A tile of 64 IM tokens x 16 JN output channels of one channel block per thread block (16 x 16 threads, 4 IM tokens x
// JN outputs of both gate matrices a thread); u and both weight tiles go through shared memory GATE_TK input
// channels at a time, transposed so that a thread reads its four tokens (and, with JN = 4, its four channels) as one
// float4.  JN = 4 for prompt portions; JN = 1 for steps of few tokens, which then have four times as many blocks to
// stream the weights with.
#define GATE_TK 16
template <int JN, int IM>                 // JN outputs and 4 IM tokens a thread: a tile of 64 IM tokens x 16 JN outputs
__global__ void __launch_bounds__(256) recurrence_gates_kernel(
        const float* __restrict__ u, const float* __restrict__ wa, const float* __restrict__ ba, const float* __restrict__ wi,
        const float* __restrict__ bi, const float* __restrict__ lam, float c_exp, float* __restrict__ a_out,
        float* __restrict__ b_out, int num_tokens, int C, int bw, int n_tiles) {
    constexpr int TN = 16 * JN, GATE_TM = 64 * IM;
    __shared__ __align__(16) float u_s[GATE_TK][GATE_TM + 4];
    __shared__ __align__(16) float wa_s[GATE_TK][TN + 4];
    __shared__ __align__(16) float wi_s[GATE_TK][TN + 4];
    pdl_enter();
    const int blk = blockIdx.y / n_tiles, o0 = (blockIdx.y - blk * n_tiles) * TN;
    const int t0 = blockIdx.x * GATE_TM;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // tx: outputs JN tx .. JN tx + JN - 1, ty: tokens 4 IM ty .. 4 IM ty + 4 IM - 1
    float ra[4 * IM][JN], ri[4 * IM][JN];
#pragma unroll
    for (int i = 0; i < 4 * IM; ++i)
#pragma unroll
        for (int j = 0; j < JN; ++j) { ra[i][j] = 0.f; ri[i][j] = 0.f; }
    for (int k0 = 0; k0 < bw; k0 += GATE_TK) {
        __syncthreads();
        for (int i = threadIdx.x; i < GATE_TM * GATE_TK; i += 256) {
            const int row = i / GATE_TK, kk = i - row * GATE_TK;      // row: a token or an output channel
            const bool k_ok = k0 + kk < bw;
            u_s[kk][row] = (k_ok && t0 + row < num_tokens) ? u[(int64_t)(t0 + row) * C + blk * bw + k0 + kk] : 0.f;
            if (row < TN) {
                const bool w_ok = k_ok && o0 + row < bw;
                const int64_t w = ((int64_t)blk * bw + o0 + row) * bw + k0 + kk;
                wa_s[kk][row] = w_ok ? wa[w] : 0.f;
                wi_s[kk][row] = w_ok ? wi[w] : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GATE_TK; ++kk) {
            float uu[4 * IM];
#pragma unroll
            for (int m = 0; m < IM; ++m) {
                const float4 uv = *reinterpret_cast<const float4*>(&u_s[kk][4 * IM * ty + 4 * m]);
                uu[4 * m] = uv.x; uu[4 * m + 1] = uv.y; uu[4 * m + 2] = uv.z; uu[4 * m + 3] = uv.w;
            }
            float aa[JN], ii[JN];
#pragma unroll
            for (int j = 0; j < JN; ++j) { aa[j] = wa_s[kk][JN * tx + j]; ii[j] = wi_s[kk][JN * tx + j]; }
#pragma unroll
            for (int i = 0; i < 4 * IM; ++i)
#pragma unroll
                for (int j = 0; j < JN; ++j) {
                    ra[i][j] = fmaf(uu[i], aa[j], ra[i][j]);
                    ri[i][j] = fmaf(uu[i], ii[j], ri[i][j]);
                }
        }
    }
#pragma unroll
    for (int j = 0; j < JN; ++j) {
        const int o = o0 + JN * tx + j;
        if (o >= bw) continue;
        const int ch = blk * bw + o;
        const float bra = ba[ch], bri = bi[ch], l = lam[ch];
        const float sp = l > 20.f ? l : log1pf(expf(l));                  // softplus
#pragma unroll
        for (int i = 0; i < 4 * IM; ++i) {
            const int t = t0 + 4 * IM * ty + i;
            if (t >= num_tokens) continue;
            const float r = 1.0f / (1.0f + expf(-(ra[i][j] + bra)));
            const float g = 1.0f / (1.0f + expf(-(ri[i][j] + bri)));
            const float a = expf(-c_exp * r * sp);
            const float m = sqrtf(fmaxf(1.0f - a * a, 0.f));
            a_out[(int64_t)t * C + ch] = a;
            b_out[(int64_t)t * C + ch] = m * (g * u[(int64_t)t * C + ch]);
        }
    }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// blockDim = (channels, segments)
template <typename T>
__global__ void __launch_bounds__(1024) recurrence_scan_kernel(const float* __restrict__ a, const float* __restrict__ b, const T* __restrict__ y,
                                       int64_t y_stride, const T* __restrict__ x, int64_t x_stride,
                                       const int* __restrict__ row_q_start, const int* __restrict__ row_q_len,
                                       const int* __restrict__ state_slots, float* __restrict__ state, T* __restrict__ out,
                                       int C, int K) {
    extern __shared__ float seg_s[];                          // [2][segments][channels]
    pdl_enter();
    const int r = blockIdx.y;
    const int nch = blockDim.x;
    const int ch = blockIdx.x * nch + threadIdx.x;
    const int seg = threadIdx.y, nseg = blockDim.y;
    const int q_len = row_q_len[r], q_start = row_q_start[r];
    const int len = (q_len + nseg - 1) / nseg;
    const int lo = min(q_len, seg * len), hi = min(q_len, lo + len);
    const bool ok = ch < C;
    float* st = state + (int64_t)state_slots[r] * K * C;
    float* A_s = seg_s;
    float* B_s = seg_s + nseg * nch;
    float s = ok ? st[ch] : 0.f;                              // read before the barrier: the last segment overwrites it
    if (nseg > 1) {
        float A = 1.f, Bv = 0.f;
        if (ok)
            for (int t = lo; t < hi; t += 8) {                // eight tokens' loads in flight before the dependent chain
                float av[8], bv[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int64_t i = (int64_t)(q_start + t + k) * C + ch;
                    av[k] = t + k < hi ? a[i] : 1.f;
                    bv[k] = t + k < hi ? b[i] : 0.f;
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    A *= av[k];
                    Bv = fmaf(av[k], Bv, bv[k]);
                }
            }
        A_s[seg * nch + threadIdx.x] = A;
        B_s[seg * nch + threadIdx.x] = Bv;
        __syncthreads();
    }
    if (!ok) return;
    for (int k = 0; k < seg; ++k) s = fmaf(A_s[k * nch + threadIdx.x], s, B_s[k * nch + threadIdx.x]);
    for (int t = lo; t < hi; t += 8) {
        float av[8], bv[8], yv[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool in = t + k < hi;
            const int64_t i = (int64_t)(q_start + t + k) * C + ch;
            av[k] = in ? a[i] : 1.f;
            bv[k] = in ? b[i] : 0.f;
            yv[k] = in ? to_f32<T>(y[(int64_t)(q_start + t + k) * y_stride + ch]) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            s = fmaf(av[k], s, bv[k]);                          // past the end: a = 1, b = 0 leave s as it is
            if (t + k < hi) out[(int64_t)(q_start + t + k) * C + ch] = from_f32<T>(s * gelu_tanh_f(yv[k]));
        }
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
                               const int* state_slots, const float* taps, const float* bias, const float* state,
                               float* u, int num_tokens, int C, int K, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (C <= 0 || K < 1 || K > CONV_MAX_TAPS) return MIE_ERR_BAD_ARG;
    const int threads = 128;
    dim3 grid((C + threads - 1) / threads, (num_tokens + CONV_TOKENS - 1) / CONV_TOKENS);
    if (tag == MIE_F32)
        return launch_kernel(causal_conv_kernel<float>, grid, dim3(threads), 0, stream, (const float*)x, (int64_t)x_stride, token_row,
                             row_q_start, state_slots, taps, bias, state, u, num_tokens, C, K);
    else if (tag == MIE_BF16)
        return launch_kernel(causal_conv_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)x, (int64_t)x_stride, token_row,
                             row_q_start, state_slots, taps, bias, state, u, num_tokens, C, K);
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_recurrence_gates(const float* u, const float* wa, const float* ba, const float* wi, const float* bi,
                                    const float* lam, float c_exp, float* a_out, float* b_out, int num_tokens,
                                    int C, int blocks, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (C <= 0 || blocks <= 0 || C % blocks) return MIE_ERR_BAD_ARG;
    const int bw = C / blocks;
    const int token_tiles = (num_tokens + 63) / 64;
    if (token_tiles * ((bw + 63) / 64) * blocks >= 2 * device_sm_count()) {
        // 4 tokens x 4 outputs a thread; 8 x 4 (IM = 2) takes 107 registers and was measured slower: 229 against 183 us
        // at 2,048 tokens, 8 blocks of 256 channels
        const int n_tiles = (bw + 63) / 64;
        return launch_kernel(recurrence_gates_kernel<4, 1>, dim3(token_tiles, blocks * n_tiles), dim3(256), 0, stream, u, wa, ba, wi, bi,
                             lam, c_exp, a_out, b_out, num_tokens, C, bw, n_tiles);
    }
    const int n_tiles = (bw + 15) / 16;
    return launch_kernel(recurrence_gates_kernel<1, 1>, dim3(token_tiles, blocks * n_tiles), dim3(256), 0, stream, u, wa, ba, wi, bi,
                         lam, c_exp, a_out, b_out, num_tokens, C, bw, n_tiles);
}

extern "C" int mie_recurrence_scan(const float* a, const float* b, const void* y, int tag, long long y_stride, const void* x,
                                   long long x_stride, const int* row_q_start, const int* row_q_len, const int* state_slots,
                                   float* state, void* out, int num_rows, int C, int K, int segments, cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (C <= 0 || K < 1 || K > CONV_MAX_TAPS || segments < 1 || segments > 32) return MIE_ERR_BAD_ARG;
    const int nch = 32;      // 8 channels a block (four times the blocks) was measured slower: 66 against 49 us at 2,048 tokens x 2,048 channels
    dim3 grid((C + nch - 1) / nch, num_rows), block(nch, segments);
    const size_t smem = (size_t)2 * segments * nch * sizeof(float);
    if (tag == MIE_F32)
        return launch_kernel(recurrence_scan_kernel<float>, grid, block, smem, stream, a, b, (const float*)y, (int64_t)y_stride,
                             (const float*)x, (int64_t)x_stride, row_q_start, row_q_len, state_slots, state, (float*)out, C, K);
    else if (tag == MIE_BF16)
        return launch_kernel(recurrence_scan_kernel<bf16>, grid, block, smem, stream, a, b, (const bf16*)y, (int64_t)y_stride,
                             (const bf16*)x, (int64_t)x_stride, row_q_start, row_q_len, state_slots, state, (bf16*)out, C, K);
    return MIE_ERR_BAD_ARG;
}
