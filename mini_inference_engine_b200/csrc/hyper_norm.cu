// Hyper-connections and Dynamic Tanh, the read side and the write side of a sublayer in one pass over the streams.
//
// A model with hyper-connections carries S copies of the residual stream, res[t] = [x_0 | x_1 | ... | x_{S-1}], each
// of W float32 entries.  A sublayer reads one mixture of them and writes into all of them:
//
//   write (the sublayer BEFORE, whose output y is still pending):   x'_r = sum_s mix[s, r] x_s + outc[r] y
//   read  (the sublayer that runs next):                            u    = sum_r inc[r] x'_r
//   norm  (Dynamic Tanh: no statistics of the row):                 out  = tanh(alpha u) w + b
//
// All three per column, in float32: every stream entry is read once and (unless only some rows are gathered, in
// front of the output head) written once.  Without a pending output the write is skipped; with S = 1 and
// mix = outc = inc = 1 this is the ordinary "res += y; out = norm(res)" of a pre-norm layer.  `norm_kind` 0 is
// Dynamic Tanh, 1 hands on u itself (no norm).
#include "common.cuh"
#include "range_check.cuh"

#define HYPER_MAX_STREAMS 8
#define MIE_K_HYPER_NORM 11

struct HyperCoef {
    float mix[HYPER_MAX_STREAMS * HYPER_MAX_STREAMS];     // [from, to]
    float outc[HYPER_MAX_STREAMS];
    float inc[HYPER_MAX_STREAMS];
};

template <typename TY, typename TO, int V>
__global__ void hyper_norm_kernel(float* __restrict__ res, const TY* __restrict__ y, const float* __restrict__ mix,
                                  const float* __restrict__ outc, const float* __restrict__ inc,
                                  const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b,
                                  TO* __restrict__ out, const int* __restrict__ rows, int num_out, int W, int S,
                                  int num_rows, int norm_kind, int* report) {
    __shared__ HyperCoef c;
    pdl_enter();
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) c.mix[i] = mix ? mix[i] : ((i / S) == (i % S) ? 1.f : 0.f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        c.outc[i] = outc ? outc[i] : 1.f;
        c.inc[i] = inc ? inc[i] : 1.f;
    }
    __syncthreads();
    const float a = alpha ? alpha[0] : 1.f;
    const int WV = W / V;
    const int64_t total = (int64_t)num_out * WV;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = idx / WV;
        const int col = (int)(idx - o * WV) * V;
        int64_t t = o;
        if (rows) {
            t = rows[o];
            if (range_row(t, num_rows) != MIE_RANGE_OK) {
                range_report(report, MIE_RANGE_ROW, MIE_K_HYPER_NORM, (int)o, (int)t);
                continue;
            }
        }
        float* base = res + (t * S) * W + col;
        float x[HYPER_MAX_STREAMS][V];
#pragma unroll
        for (int s = 0; s < HYPER_MAX_STREAMS; ++s) {
            if (s < S) {
                if constexpr (V == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(base + (int64_t)s * W);
                    x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) x[s][i] = base[(int64_t)s * W + i];
                }
            }
        }
        float u[V];
#pragma unroll
        for (int i = 0; i < V; ++i) u[i] = 0.f;
        if (y) {
            float yv[V];
#pragma unroll
            for (int i = 0; i < V; ++i) yv[i] = to_f32<TY>(y[t * W + col + i]);
#pragma unroll
            for (int r = 0; r < HYPER_MAX_STREAMS; ++r) {
                if (r < S) {
                    float n[V];
#pragma unroll
                    for (int i = 0; i < V; ++i) n[i] = c.outc[r] * yv[i];
#pragma unroll
                    for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
                        if (s < S) {
#pragma unroll
                            for (int i = 0; i < V; ++i) n[i] = fmaf(c.mix[s * S + r], x[s][i], n[i]);
                        }
#pragma unroll
                    for (int i = 0; i < V; ++i) u[i] = fmaf(c.inc[r], n[i], u[i]);
                    if (!rows) {
                        if constexpr (V == 4) *reinterpret_cast<float4*>(base + (int64_t)r * W) = make_float4(n[0], n[1], n[2], n[3]);
                        else {
#pragma unroll
                            for (int i = 0; i < V; ++i) base[(int64_t)r * W + i] = n[i];
                        }
                    }
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
                if (s < S) {
#pragma unroll
                    for (int i = 0; i < V; ++i) u[i] = fmaf(c.inc[s], x[s][i], u[i]);
                }
        }
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float v = norm_kind == 0 ? fmaf(tanhf(a * u[i]), w[col + i], b[col + i]) : u[i];
            out[o * W + col + i] = from_f32<TO>(v);
        }
    }
}

template <typename TY, typename TO>
static int launch_hyper(float* res, const void* y, const float* mix, const float* outc, const float* inc, const float* alpha,
                        const float* w, const float* b, void* out, const int* rows, int num_out, int W, int S, int num_rows,
                        int norm_kind, cudaStream_t stream) {
    const bool vec = W % 4 == 0 && (reinterpret_cast<uintptr_t>(res) % 16 == 0);
    const int64_t total = (int64_t)num_out * (vec ? W / 4 : W);
    const int threads = 256;
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > (int64_t)device_sm_count() * 8) blocks = (int64_t)device_sm_count() * 8;
    if (vec)
        return launch_kernel(hyper_norm_kernel<TY, TO, 4>, dim3((int)blocks), dim3(threads), 0, stream, res, (const TY*)y, mix, outc,
                             inc, alpha, w, b, (TO*)out, rows, num_out, W, S, num_rows, norm_kind, g_range_report);
    return launch_kernel(hyper_norm_kernel<TY, TO, 1>, dim3((int)blocks), dim3(threads), 0, stream, res, (const TY*)y, mix, outc, inc,
                         alpha, w, b, (TO*)out, rows, num_out, W, S, num_rows, norm_kind, g_range_report);
}

// res: [num_rows, S, W] float32, updated in place when `y` is given and `rows` is not.  y: [num_rows, W] (type y_tag) or
// null.  mix [S, S], outc [S], inc [S], alpha [1], w [W], b [W]: float32 on the device; a null mix / outc / inc means
// identity / ones / ones.  out: [num_out, W] (type out_tag); with `rows`, output row o comes from stream row rows[o].
extern "C" int mie_hyper_norm(float* res, const void* y, int y_tag, const float* mix, const float* outc, const float* inc,
                              const float* alpha, const float* w, const float* b, void* out, int out_tag, const int* rows,
                              int num_out, int W, int S, int num_rows, int norm_kind, cudaStream_t stream) {
    if (num_out <= 0) return 0;
    if (W <= 0 || S < 1 || norm_kind < 0 || norm_kind > 1 || (norm_kind == 0 && (!w || !b))) return MIE_ERR_BAD_ARG;
    if (S > HYPER_MAX_STREAMS) return MIE_ERR_TOO_LARGE;
    if (!y) y_tag = MIE_F32;
    if (y_tag == MIE_F32 && out_tag == MIE_F32)
        return launch_hyper<float, float>(res, y, mix, outc, inc, alpha, w, b, out, rows, num_out, W, S, num_rows, norm_kind, stream);
    if (y_tag == MIE_F32 && out_tag == MIE_BF16)
        return launch_hyper<float, bf16>(res, y, mix, outc, inc, alpha, w, b, out, rows, num_out, W, S, num_rows, norm_kind, stream);
    if (y_tag == MIE_BF16 && out_tag == MIE_BF16)
        return launch_hyper<bf16, bf16>(res, y, mix, outc, inc, alpha, w, b, out, rows, num_out, W, S, num_rows, norm_kind, stream);
    if (y_tag == MIE_BF16 && out_tag == MIE_F32)
        return launch_hyper<bf16, float>(res, y, mix, outc, inc, alpha, w, b, out, rows, num_out, W, S, num_rows, norm_kind, stream);
    return MIE_ERR_BAD_ARG;
}
