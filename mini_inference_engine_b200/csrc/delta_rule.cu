// The gated delta rule with one decay per head and key channel: a linear-attention mixer whose per-head state
// S [D, Dv] (float32) forgets per key channel, corrects what it holds under the new key, and is read by the query:
//
//   S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t        (in this order)
//
// Three kernels:
//   prepare    per token: the short causal convolution over time of q, k and v (inputs older than the step's portion come
//              from the request's convolution state), silu, q and k made unit vectors per head (q also scaled), beta =
//              sigmoid of its logit, g = exp(-exp(A_log[h]) softplus(a + dt_bias)) -- all float32;
//   conv_state the last K - 1 inputs of the convolution of every row move into its state slot (after prepare has read it);
//   scan       the recurrence, token by token per row, one block per (row, head, slice of value columns): a group of L
//              lanes owns one column of S (D / L entries each, in registers: 4, 8 or 16 by the key size), so S is read from memory once per step and
//              written once; the tokens' operands arrive through a ring in shared memory filled by asynchronous copies
//              two batches ahead.  The read-out uses S after the token's own write:
//              o = (g S)^T q + u (k . q), which needs one pass over the column for both sums.
//   head_norm_gate   o / rms(o) per head, times a weight shared by the heads, times sigmoid of a gate logit.
//
// State layouts: S [slot, H, Dv, D] float32 (a column of S contiguous); convolution [slot, K - 1, C] float32 with row i the
// input at K - 1 - i tokens before the next one.  Slot 0 is scratch.
#include "common.cuh"

#define DELTA_MAX_KEY 512    // the longest key: sixteen entries a lane, thirty-two lanes a column

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// The convolution's output for channel c (of C) at token t: taps [C, K], last tap on the token itself.
template <typename T>
__device__ __forceinline__ float conv_at(const T* __restrict__ x, int64_t stride, const float* __restrict__ taps,
                                         const float* __restrict__ st, int C, int K, int t, int local, int c) {
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
        const int back = K - 1 - j;                 // how many tokens before t
        const float xv = back <= local ? to_f32<T>(x[(int64_t)(t - back) * stride + c])
                                       : st[(int64_t)(K - 1 - (back - local)) * C + c];
        acc = fmaf(taps[(int64_t)c * K + j], xv, acc);
    }
    return acc / (1.0f + expf(-acc));
}

// proj[t] = [ q: G x D | k: G x D | v: H x Dv | beta logits: H | ... ] (activation type, row stride `stride`);
// low[t] = [ a: H x D | ... ] float32 (row stride low_stride).  One block per token, one warp per head of q, k or v.
template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ proj, int64_t stride, const float* __restrict__ low, int64_t low_stride,
                                     const float* __restrict__ taps, const float* __restrict__ conv_state,
                                     const int* __restrict__ token_row, const int* __restrict__ row_q_start,
                                     const int* __restrict__ state_slots, const float* __restrict__ a_log,
                                     const float* __restrict__ dt_bias, float* __restrict__ qn, float* __restrict__ kn,
                                     float* __restrict__ vn, float* __restrict__ beta, float* __restrict__ decay,
                                     float* __restrict__ kq, int H, int G, int D, int Dv, int K, float q_scale, float unit_eps) {
    pdl_enter();
    const int t = blockIdx.x;
    const int row = token_row[t];
    const int local = t - row_q_start[row];
    const int C = 2 * G * D + H * Dv;
    const float* st = conv_state + (int64_t)state_slots[row] * (K - 1) * C;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int unit = warp; unit < 2 * G + H; unit += nw) {
        const bool is_v = unit >= 2 * G;
        const int n = is_v ? Dv : D;
        const int c0 = is_v ? 2 * G * D + (unit - 2 * G) * Dv : unit * D;
        float* dst = is_v ? vn + (int64_t)t * H * Dv + (unit - 2 * G) * Dv
                          : (unit < G ? qn + (int64_t)t * G * D + unit * D : kn + (int64_t)t * G * D + (unit - G) * D);
        if (is_v) {
            for (int d = lane; d < n; d += 32) dst[d] = conv_at<T>(proj, stride, taps, st, C, K, t, local, c0 + d);
        } else if (n <= 256) {                                        // a head of up to 256 entries stays in registers between its two passes
            float y[8];
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                y[i] = d < n ? conv_at<T>(proj, stride, taps, st, C, K, t, local, c0 + d) : 0.f;
                ss = fmaf(y[i], y[i], ss);
            }
            const float s = (unit < G ? q_scale : 1.0f) / sqrtf(warp_sum(ss) + unit_eps);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                if (d < n) dst[d] = y[i] * s;
            }
        } else {
            float ss = 0.f;
            for (int d = lane; d < n; d += 32) {
                const float y = conv_at<T>(proj, stride, taps, st, C, K, t, local, c0 + d);
                dst[d] = y;
                ss += y * y;
            }
            const float s = (unit < G ? q_scale : 1.0f) / sqrtf(warp_sum(ss) + unit_eps);
            for (int d = lane; d < n; d += 32) dst[d] *= s;           // the lane's own entries
        }
    }
    const T* bl = proj + (int64_t)t * stride + C;
    for (int h = threadIdx.x; h < H; h += blockDim.x) beta[(int64_t)t * H + h] = 1.0f / (1.0f + expf(-to_f32<T>(bl[h])));
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
        const float rate = expf(a_log[i / D]);
        decay[(int64_t)t * H * D + i] = expf(-rate * softplus_f(low[(int64_t)t * low_stride + i] + dt_bias[i]));
    }
    __syncthreads();                                   // q and k of this token, written above by other warps of the block
    for (int g = warp; g < G; g += nw) {               // k . q per key head: the same for every value column of the recurrence
        float acc = 0.f;
        for (int d = lane; d < D; d += 32) acc = fmaf(qn[((int64_t)t * G + g) * D + d], kn[((int64_t)t * G + g) * D + d], acc);
        acc = warp_sum(acc);
        if (lane == 0) kq[(int64_t)t * G + g] = acc;
    }
}

// The convolution state of every row after the step: row i of the new state is the input at q_len - (K - 1) + i of the
// portion, or, where the portion is shorter than that reaches back, a row of the old state.  One thread per channel
// walks the rows upwards, so the move is safe in place.
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ x, int64_t stride, const int* __restrict__ row_q_start,
                                  const int* __restrict__ row_q_len, const int* __restrict__ state_slots,
                                  float* __restrict__ conv_state, int C, int K) {
    pdl_enter();
    const int row = blockIdx.y;
    const int slot = state_slots[row];
    const int q0 = row_q_start[row], n = row_q_len[row];
    float* st = conv_state + (int64_t)slot * (K - 1) * C;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < C; c += gridDim.x * blockDim.x) {
        for (int i = 0; i < K - 1; ++i) {
            const int li = n - (K - 1) + i;
            st[(int64_t)i * C + c] = li >= 0 ? to_f32<T>(x[(int64_t)(q0 + li) * stride + c]) : st[(int64_t)(i + n) * C + c];
        }
    }
}

// Four bytes from global to shared memory without passing through registers; groups of such copies complete in order.
__device__ __forceinline__ void cp_async4(float* dst_smem, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void cp_async16(float* dst_smem, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}

#define DELTA_BATCHES 3     // batches of tokens in the shared-memory ring: one computed, two on their way

// The recurrence is one dependent chain per token, so a token's operands must be at hand when its turn comes: the block
// copies k, q, the decays, its columns of v, beta and k . q for `tb` tokens at a time into a ring in shared memory
// (asynchronous copies, two batches ahead of the one being computed).  ring[slot] = [k: D | q: D | g: D | v: cols | beta | kq],
// padded to whole 16-byte pieces.  A lane holds R entries of its column: few, so that a column's sums are spread
// over many lanes and an SM holds many warps whose chains hide one another's latency.  VEC: D = L * R and D % 4 = 0, so the
// ring is filled and read 16 bytes at a time and nothing needs a bound check; otherwise everything goes entry by entry.
template <int R, bool VEC, int LT>
__global__ void delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vn,
                                  const float* __restrict__ beta, const float* __restrict__ decay, const float* __restrict__ kq,
                                  const int* __restrict__ row_q_start, const int* __restrict__ row_q_len,
                                  const int* __restrict__ state_slots, float* __restrict__ state, float* __restrict__ out, int H,
                                  int G, int D, int Dv, int L_rt, int cols, int tb, int slot_floats) {
    extern __shared__ __align__(16) float ring[];
    pdl_enter();
    const int L = LT > 0 ? LT : L_rt;                         // lanes a column: a constant where the launcher knows it (shifts, unrolled sums)
    const int row = blockIdx.x, h = blockIdx.y;
    const int l = threadIdx.x % L, cl = threadIdx.x / L, j0 = blockIdx.z * cols, j = j0 + cl;
    const bool active = cl < cols && j < Dv;                   // threads that only fill up the last warp own no column
    const int n = row_q_len[row], t0 = row_q_start[row];
    const int kh = h / (H / G);
    float* sp = state + (((int64_t)state_slots[row] * H + h) * Dv + (active ? j : 0)) * D;
    // register r of lane l holds row 4 (l + L (r / 4)) + r % 4: pieces of four consecutive rows, dealt out over the lanes,
    // so that the lanes of a column read consecutive 16-byte pieces of the ring (no bank conflicts)
    auto row_of = [&](int r) { return 4 * (l + L * (r >> 2)) + (r & 3); };
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = row_of(r);
        s[r] = (active && i < D) ? sp[i] : 0.f;
    }
    const int v_at = 3 * D + (cl < cols ? cl : 0);
    const float v_on = cl < cols ? 1.f : 0.f;
    const int batches = (n + tb - 1) / tb;
    auto issue = [&](int batch) {                              // every thread commits one group per call, also an empty one
        if (batch < batches) {
            float* base = ring + (size_t)(batch % DELTA_BATCHES) * tb * slot_floats;
            const int first = batch * tb, count = min(tb, n - first);
            const int64_t tf = t0 + first;
            if constexpr (VEC) {
                const int q4 = D >> 2;                         // 16-byte pieces of one operand
                for (int c = threadIdx.x; c < 3 * q4; c += blockDim.x) {
                    const int seg = c / q4, off = (c - seg * q4) * 4;
                    const float* src = seg == 0 ? kn + (tf * G + kh) * D : (seg == 1 ? qn + (tf * G + kh) * D : decay + (tf * H + h) * D);
                    const int64_t step = seg < 2 ? (int64_t)G * D : (int64_t)H * D;
                    float* dst = base + seg * D + off;
                    for (int tok = 0; tok < count; ++tok) cp_async16(dst + tok * slot_floats, src + off + tok * step);
                }
            } else {
                for (int c = threadIdx.x; c < 3 * D; c += blockDim.x) {
                    const int seg = c / D, off = c - seg * D;
                    const float* src = seg == 0 ? kn + (tf * G + kh) * D : (seg == 1 ? qn + (tf * G + kh) * D : decay + (tf * H + h) * D);
                    const int64_t step = seg < 2 ? (int64_t)G * D : (int64_t)H * D;
                    for (int tok = 0; tok < count; ++tok) cp_async4(base + tok * slot_floats + c, src + off + tok * step);
                }
            }
            for (int c = threadIdx.x; c < cols + 2; c += blockDim.x) {
                const float* src = c < cols ? vn + (tf * H + h) * Dv + min(j0 + c, Dv - 1) : (c == cols ? beta + tf * H + h : kq + tf * G + kh);
                const int64_t step = c < cols ? (int64_t)H * Dv : (c == cols ? H : G);
                for (int tok = 0; tok < count; ++tok) cp_async4(base + tok * slot_floats + 3 * D + c, src + tok * step);
            }
        }
        cp_async_commit();
    };
    issue(0);
    issue(1);
    for (int batch = 0; batch < batches; ++batch) {
        issue(batch + 2);                                      // into the slot whose batch was computed before the last barrier
        cp_async_wait_group<2>();                              // this thread's copies of `batch` have landed ...
        __syncthreads();                                       // ... and everybody else's
        const float* base = ring + (size_t)(batch % DELTA_BATCHES) * tb * slot_floats;
        const int first = batch * tb, count = min(tb, n - first);
#pragma unroll 4                                              // the next tokens' operands are read while a token's sums travel
        for (int tok = 0; tok < count; ++tok) {
            const float* op = base + tok * slot_floats;
            float k[R], q[R], g[R];
            if constexpr (VEC) {
#pragma unroll
                for (int r = 0; r < R; r += 4) {
                    const int i = 4 * (l + L * (r >> 2));
                    *reinterpret_cast<float4*>(k + r) = *reinterpret_cast<const float4*>(op + i);
                    *reinterpret_cast<float4*>(q + r) = *reinterpret_cast<const float4*>(op + D + i);
                    *reinterpret_cast<float4*>(g + r) = *reinterpret_cast<const float4*>(op + 2 * D + i);
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int i = row_of(r);
                    const bool ok = i < D;
                    k[r] = ok ? op[i] : 0.f;
                    q[r] = ok ? op[D + i] : 0.f;
                    g[r] = ok ? op[2 * D + i] : 0.f;
                }
            }
            float r1 = 0.f, r2 = 0.f, r1b = 0.f, r2b = 0.f;             // two chains each: half the dependent latency
#pragma unroll
            for (int r = 0; r < R; r += 2) {
                s[r] *= g[r];
                s[r + 1] *= g[r + 1];
                r1 = fmaf(s[r], k[r], r1);
                r1b = fmaf(s[r + 1], k[r + 1], r1b);
                r2 = fmaf(s[r], q[r], r2);
                r2b = fmaf(s[r + 1], q[r + 1], r2b);
            }
            r1 += r1b;
            r2 += r2b;
            if constexpr (LT > 0) {
#pragma unroll
                for (int o = LT >> 1; o > 0; o >>= 1) {
                    r1 += __shfl_xor_sync(0xffffffffu, r1, o);
                    r2 += __shfl_xor_sync(0xffffffffu, r2, o);
                }
            } else {
                for (int o = L >> 1; o > 0; o >>= 1) {
                    r1 += __shfl_xor_sync(0xffffffffu, r1, o);
                    r2 += __shfl_xor_sync(0xffffffffu, r2, o);
                }
            }
            const float u = op[3 * D + cols] * (v_on * op[v_at] - r1);
#pragma unroll
            for (int r = 0; r < R; ++r) s[r] = fmaf(k[r], u, s[r]);
            if (active && l == 0) out[((int64_t)(t0 + first + tok) * H + h) * Dv + j] = fmaf(u, op[3 * D + cols + 1], r2);
        }
        __syncthreads();                                       // the slot may be refilled
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = row_of(r);
            if (i < D) sp[i] = s[r];
        }
    }
}

// out[t, h, :] = o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * w[:] * sigmoid(gate[t, h, :]); a warp per (token, head).
// gate: float32 rows of stride gate_stride; w: float32 [Dv] or null.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, int64_t gate_stride,
                                      const float* __restrict__ w, T* __restrict__ out, int num_tokens, int H, int Dv, float eps) {
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
    const float* g = gate ? gate + t * gate_stride + (int64_t)h * Dv : nullptr;
    for (int i = lane; i < Dv; i += 32) {
        float v = src[i] * s;
        if (w) v *= w[i];
        if (g) v /= 1.0f + expf(-g[i]);
        out[item * Dv + i] = from_f32<T>(v);
    }
}

extern "C" int mie_delta_prepare(const void* proj, int tag, long long stride, const float* low, long long low_stride, const float* taps,
                                 const float* conv_state, const int* token_row, const int* row_q_start, const int* state_slots,
                                 const float* a_log, const float* dt_bias, float* qn, float* kn, float* vn, float* beta, float* decay,
                                 float* kq, int num_tokens, int H, int G, int D, int Dv, int K, float q_scale, float unit_eps,
                                 cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || Dv <= 0 || K < 1) return MIE_ERR_BAD_ARG;
    const int units = 2 * G + H;
    const int threads = units >= 8 ? 256 : (units >= 4 ? 128 : 64);
    if (tag == MIE_F32)
        return launch_kernel(delta_prepare_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)proj, (int64_t)stride,
                             low, (int64_t)low_stride, taps, conv_state, token_row, row_q_start, state_slots, a_log, dt_bias, qn, kn, vn,
                             beta, decay, kq, H, G, D, Dv, K, q_scale, unit_eps);
    else if (tag == MIE_BF16)
        return launch_kernel(delta_prepare_kernel<bf16>, dim3(num_tokens), dim3(threads), 0, stream, (const bf16*)proj, (int64_t)stride,
                             low, (int64_t)low_stride, taps, conv_state, token_row, row_q_start, state_slots, a_log, dt_bias, qn, kn, vn,
                             beta, decay, kq, H, G, D, Dv, K, q_scale, unit_eps);
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_conv_state_update(const void* x, int tag, long long stride, const int* row_q_start, const int* row_q_len,
                                     const int* state_slots, float* conv_state, int num_rows, int C, int K, cudaStream_t stream) {
    if (num_rows <= 0 || K <= 1) return 0;
    if (C <= 0) return MIE_ERR_BAD_ARG;
    const int threads = 128;
    const dim3 grid((C + threads - 1) / threads, num_rows);
    if (tag == MIE_F32)
        return launch_kernel(conv_state_kernel<float>, grid, dim3(threads), 0, stream, (const float*)x, (int64_t)stride, row_q_start,
                             row_q_len, state_slots, conv_state, C, K);
    else if (tag == MIE_BF16)
        return launch_kernel(conv_state_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)x, (int64_t)stride, row_q_start,
                             row_q_len, state_slots, conv_state, C, K);
    return MIE_ERR_BAD_ARG;
}

template <int R>
static int launch_scan(const float* qn, const float* kn, const float* vn, const float* beta, const float* decay, const float* kq,
                       const int* row_q_start, const int* row_q_len, const int* state_slots, float* state, float* out, int num_rows,
                       int H, int G, int D, int Dv, cudaStream_t stream) {
    int L = 1;
    while (L * R < D) L <<= 1;
    if (L > 32) return MIE_ERR_TOO_LARGE;
    int cols = 128 / L;                                        // value columns a block of 128 threads
    if (cols > Dv) cols = Dv;
    const int threads = (cols * L + 31) / 32 * 32;
    const dim3 grid(num_rows, H, (Dv + cols - 1) / cols);
    // tokens a batch of the ring: eight where three such batches stay within 48 KB, fewer for long keys
    const int slot_floats = (3 * D + cols + 2 + 3) / 4 * 4;
    const size_t slot_bytes = (size_t)slot_floats * sizeof(float);
    int tb = (int)(48 * 1024 / (DELTA_BATCHES * slot_bytes));
    if (tb > 8) tb = 8;
    if (tb < 1) tb = 1;
    const size_t smem = (size_t)DELTA_BATCHES * tb * slot_bytes;
    const bool vec = D == L * R && D % 4 == 0 &&
                     ((reinterpret_cast<uintptr_t>(qn) | reinterpret_cast<uintptr_t>(kn) | reinterpret_cast<uintptr_t>(decay)) & 15) == 0;
    // the vectorised kernel with the lanes a column as a constant for the common key sizes (64 and 128: 16 lanes), else at run time
    auto kernel = !vec ? delta_scan_kernel<R, false, 0> : (L == 16 ? delta_scan_kernel<R, true, 16> : delta_scan_kernel<R, true, 0>);
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_kernel(kernel, grid, dim3(threads), smem, stream, qn, kn, vn, beta, decay, kq, row_q_start, row_q_len,
                         state_slots, state, out, H, G, D, Dv, L, cols, tb, slot_floats);
}

extern "C" int mie_delta_scan(const float* qn, const float* kn, const float* vn, const float* beta, const float* decay, const float* kq,
                              const int* row_q_start, const int* row_q_len, const int* state_slots, float* state, float* out,
                              int num_rows, int H, int G, int D, int Dv, cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || Dv <= 0) return MIE_ERR_BAD_ARG;
    // entries of a column a lane: the fewest for which sixteen lanes hold a column (thirty-two for the longest keys)
    if (D <= 64) return launch_scan<4>(qn, kn, vn, beta, decay, kq, row_q_start, row_q_len, state_slots, state, out, num_rows, H, G, D, Dv, stream);
    if (D <= 128) return launch_scan<8>(qn, kn, vn, beta, decay, kq, row_q_start, row_q_len, state_slots, state, out, num_rows, H, G, D, Dv, stream);
    if (D <= DELTA_MAX_KEY) return launch_scan<16>(qn, kn, vn, beta, decay, kq, row_q_start, row_q_len, state_slots, state, out, num_rows, H, G, D, Dv, stream);
    return MIE_ERR_TOO_LARGE;
}

extern "C" int mie_head_norm_gate(const float* o, const float* gate, long long gate_stride, const float* w, void* out, int tag,
                                  int num_tokens, int H, int Dv, float eps, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (H <= 0 || Dv <= 0) return MIE_ERR_BAD_ARG;
    const int warps = 4;
    const int64_t items = (int64_t)num_tokens * H;
    const int blocks = (int)((items + warps - 1) / warps);
    if (tag == MIE_F32)
        return launch_kernel(head_norm_gate_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, o, gate, (int64_t)gate_stride, w,
                             (float*)out, num_tokens, H, Dv, eps);
    else if (tag == MIE_BF16)
        return launch_kernel(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(warps * 32), 0, stream, o, gate, (int64_t)gate_stride, w,
                             (bf16*)out, num_tokens, H, Dv, eps);
    return MIE_ERR_BAD_ARG;
}
