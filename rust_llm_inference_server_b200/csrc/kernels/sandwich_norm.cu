// Norms of blocks that norm a sublayer's result before it joins the residual stream, and plain
// RMSNorms over activations inside a mixer.  All statistics, scales and sums are float32.
//
// post_norm_residual, one CTA a token:
//   y      = sub[t, :] (+ bias)                                   sublayer result, widened
//   resid += scale * (y / sqrt(mean(y^2) + eps) * w_post)         float32, in place
//   out    = resid / sqrt(mean(resid^2) + eps) * w_next           rounded once (only if w_next is given)
// so the addition and the norm in front of the next sublayer cost one pass over the row.
//
// act_norm, one CTA a token: out = x / sqrt(mean(x^2) + eps) * w (* sigmoid(gate)), x float32 or the
// activation type with a row stride of its own, gate in the activation type with a row stride.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 256;
constexpr int MAX_PER_THREAD = 32;   // widths up to THREADS * 32 are kept in registers

template <typename T>
__global__ __launch_bounds__(THREADS) void post_norm_residual_kernel(
    const T* __restrict__ sub, const float* __restrict__ bias, const float* __restrict__ w_post,
    const float* __restrict__ scale, float* __restrict__ resid, const float* __restrict__ w_next,
    T* __restrict__ out, int hidden, float eps_post, float eps_next) {
    pdl_wait_and_trigger();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * hidden;
    float v[MAX_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        v[i] = 0.f;
        if (c < hidden) {
            v[i] = to_f<T>(sub[base + c]) + (bias != nullptr ? bias[c] : 0.f);
            ss = fmaf(v[i], v[i], ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float r1 = 1.0f / sqrtf(ss / (float)hidden + eps_post);
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < hidden) {
            const float normed = v[i] * r1 * w_post[c];
            const float x = resid[base + c] + (scale != nullptr ? scale[c] * normed : normed);
            resid[base + c] = x;
            v[i] = x;
            ss2 = fmaf(x, x, ss2);
        }
    }
    if (w_next == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.0f / sqrtf(ss2 / (float)hidden + eps_next);
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < hidden) out[base + c] = from_f<T>(v[i] * r2 * w_next[c]);
    }
}

template <typename TIn, typename T>
__global__ __launch_bounds__(THREADS) void act_norm_kernel(
    const TIn* __restrict__ x, long long x_stride, const float* __restrict__ w,
    const T* __restrict__ gate, long long gate_stride, T* __restrict__ out, long long out_stride,
    int width, float eps) {
    pdl_wait_and_trigger();
    __shared__ float scratch[33];
    const TIn* xr = x + (size_t)blockIdx.x * x_stride;
    float v[MAX_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        v[i] = 0.f;
        if (c < width) {
            v[i] = to_f<TIn>(xr[c]);
            ss = fmaf(v[i], v[i], ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)width + eps);
    T* orow = out + (size_t)blockIdx.x * out_stride;
    const T* grow = gate != nullptr ? gate + (size_t)blockIdx.x * gate_stride : nullptr;
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < width) {
            float y = v[i] * r * w[c];
            if (grow != nullptr) y *= 1.0f / (1.0f + expf(-to_f<T>(grow[c])));
            orow[c] = from_f<T>(y);
        }
    }
}

// out = act(x + b): act 0 none, 1 the square of max(., 0).  Element-wise, float32 inside.
template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ x, const float* __restrict__ b, T* __restrict__ out,
                                long long n, int width, int act) {
    pdl_wait_and_trigger();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = to_f<T>(x[i]) + (b != nullptr ? b[i % width] : 0.f);
        if (act == 1) {
            v = fmaxf(v, 0.f);
            v = v * v;
        }
        out[i] = from_f<T>(v);
    }
}
}  // namespace

extern "C" int rlis_post_norm_residual(const void* sub, const float* bias, const float* w_post, const float* scale,
                                       float* resid, const float* w_next, void* out, int n_tokens, int hidden,
                                       float eps_post, float eps_next, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || hidden > THREADS * MAX_PER_THREAD) return RLIS_ERR_UNSUPPORTED;
    if (dtype == RLIS_F32)
        rlis_launch(post_norm_residual_kernel<float>, n_tokens, THREADS, 0, stream, (const float*)sub, bias, w_post,
                    scale, resid, w_next, (float*)out, hidden, eps_post, eps_next);
    else if (dtype == RLIS_BF16)
        rlis_launch(post_norm_residual_kernel<bf16>, n_tokens, THREADS, 0, stream, (const bf16*)sub, bias, w_post,
                    scale, resid, w_next, (bf16*)out, hidden, eps_post, eps_next);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

// x_f32 != 0: x is float32 whatever `dtype` (the activation type of gate and out) says.
extern "C" int rlis_act_norm(const void* x, long long x_stride, int x_f32, const float* w, const void* gate,
                             long long gate_stride, void* out, long long out_stride, int n_tokens, int width,
                             float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || width > THREADS * MAX_PER_THREAD) return RLIS_ERR_UNSUPPORTED;
    if (dtype == RLIS_F32)
        rlis_launch(act_norm_kernel<float, float>, n_tokens, THREADS, 0, stream, (const float*)x, x_stride, w,
                    (const float*)gate, gate_stride, (float*)out, out_stride, width, eps);
    else if (dtype == RLIS_BF16 && x_f32)
        rlis_launch(act_norm_kernel<float, bf16>, n_tokens, THREADS, 0, stream, (const float*)x, x_stride, w,
                    (const bf16*)gate, gate_stride, (bf16*)out, out_stride, width, eps);
    else if (dtype == RLIS_BF16)
        rlis_launch(act_norm_kernel<bf16, bf16>, n_tokens, THREADS, 0, stream, (const bf16*)x, x_stride, w,
                    (const bf16*)gate, gate_stride, (bf16*)out, out_stride, width, eps);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

extern "C" int rlis_bias_act(const void* x, const float* b, void* out, long long n_rows, int width, int act,
                             int dtype, cudaStream_t stream) {
    const long long n = n_rows * width;
    if (n <= 0) return 0;
    if (act < 0 || act > 1) return RLIS_ERR_UNSUPPORTED;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (dtype == RLIS_F32)
        rlis_launch(bias_act_kernel<float>, blocks, 256, 0, stream, (const float*)x, b, (float*)out, n, width, act);
    else if (dtype == RLIS_BF16)
        rlis_launch(bias_act_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)x, b, (bf16*)out, n, width, act);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}
