// Linear attention with a per-head decay, as a recurrence over a float32 state:
//
//   q, k = silu(.) [heads, d]; v = silu(.) [heads, dv]           (from one fused projection's rows)
//   S_t = decay_h * S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t        S [d, dv] per request and head
//
// The state of a request lives in its state slot between steps; a request whose first token is in
// this step starts from zero.  Columns of S evolve independently, so a CTA takes (request, head,
// 16 columns): 8 threads share a column, each holding d/8 of its entries in registers, and walk the
// request's tokens of this step in order.  Tokens are staged through shared memory 16 at a time.
// Everything after the projection is float32; the order of every sum depends on d only.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int COLS = 16, SLICES = 8, TOK = 16, MAX_E = 32;   // d up to 256

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

template <typename T>
__global__ __launch_bounds__(COLS * SLICES) void lightning_scan_kernel(
    const T* __restrict__ proj, long long stride, int q_off, int k_off, int v_off, float* __restrict__ out,
    float* __restrict__ state, const float* __restrict__ decay, const int* __restrict__ cu_seqlens,
    const int* __restrict__ ctx_lens, const int* __restrict__ state_slots, int nh, int d, int dv) {
    pdl_wait_and_trigger();
    extern __shared__ float sm[];
    float* qs = sm;                       // [TOK][d]
    float* ks = qs + TOK * d;             // [TOK][d]
    float* vs = ks + TOK * d;             // [TOK][COLS]
    float* os = vs + TOK * COLS;          // [TOK][COLS]
    const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int row0 = cu_seqlens[b], n = cu_seqlens[b + 1] - row0;
    const int slice = threadIdx.x % SLICES, col = threadIdx.x / SLICES;
    const bool live = c0 + col < dv;
    const bool fresh = ctx_lens[b] - n == 0;      // the request starts in this step
    const int slot = state_slots[b];
    float* S = state + ((size_t)slot * nh + h) * d * dv;
    const float g = decay[h];
    float s[MAX_E];
#pragma unroll
    for (int e = 0; e < MAX_E; ++e) {
        const int i = slice + SLICES * e;
        s[e] = (!fresh && live && i < d) ? S[(size_t)i * dv + c0 + col] : 0.f;
    }
    for (int t0 = 0; t0 < n; t0 += TOK) {
        const int nt = min(TOK, n - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * d; idx += blockDim.x) {
            const int tt = idx / d, i = idx - tt * d;
            const T* r = proj + (size_t)(row0 + t0 + tt) * stride + h * d + i;
            qs[tt * d + i] = silu_f(to_f<T>(r[q_off]));
            ks[tt * d + i] = silu_f(to_f<T>(r[k_off]));
        }
        for (int idx = threadIdx.x; idx < nt * COLS; idx += blockDim.x) {
            const int tt = idx / COLS, c = idx - tt * COLS;
            vs[idx] = c0 + c < dv ? silu_f(to_f<T>(proj[(size_t)(row0 + t0 + tt) * stride + v_off + h * dv + c0 + c])) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float v = vs[tt * COLS + col];
            const float* kr = ks + tt * d;
            const float* qr = qs + tt * d;
            float o = 0.f;
#pragma unroll
            for (int e = 0; e < MAX_E; ++e) {
                const int i = slice + SLICES * e;
                if (i < d) {
                    s[e] = fmaf(g, s[e], kr[i] * v);
                    o = fmaf(s[e], qr[i], o);
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (slice == 0) os[tt * COLS + col] = o;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * COLS; idx += blockDim.x) {
            const int tt = idx / COLS, c = idx - tt * COLS;
            if (c0 + c < dv) out[(size_t)(row0 + t0 + tt) * nh * dv + h * dv + c0 + c] = os[idx];
        }
    }
    if (live) {
#pragma unroll
        for (int e = 0; e < MAX_E; ++e) {
            const int i = slice + SLICES * e;
            if (i < d) S[(size_t)i * dv + c0 + col] = s[e];
        }
    }
}
}  // namespace

extern "C" int rlis_lightning_scan(const void* proj, long long stride, int q_off, int k_off, int v_off, float* out,
                                   float* state, const float* decay, const int* cu_seqlens, const int* ctx_lens,
                                   const int* state_slots, int n_seqs, int nh, int d, int dv, int dtype,
                                   cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (d <= 0 || d > SLICES * MAX_E || dv <= 0 || nh <= 0 || nh > 65535) return RLIS_ERR_UNSUPPORTED;
    dim3 grid(n_seqs, nh, (dv + COLS - 1) / COLS);
    if (grid.z > 65535) return RLIS_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(2 * TOK * d + 2 * TOK * COLS) * sizeof(float);
    if (dtype == RLIS_F32)
        rlis_launch(lightning_scan_kernel<float>, grid, COLS * SLICES, smem, stream, (const float*)proj, stride, q_off,
                    k_off, v_off, out, state, decay, cu_seqlens, ctx_lens, state_slots, nh, d, dv);
    else if (dtype == RLIS_BF16)
        rlis_launch(lightning_scan_kernel<bf16>, grid, COLS * SLICES, smem, stream, (const bf16*)proj, stride, q_off,
                    k_off, v_off, out, state, decay, cu_seqlens, ctx_lens, state_slots, nh, d, dv);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}
