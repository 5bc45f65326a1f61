// The routed feed-forward's two products on the tensor cores (bfloat16; moe.cu describes the layer and
// holds the float32 products).  A tile of 32 slots belongs to one expert (the sort pads every expert's
// run); a CTA of 4 warps forms 32 slots x 64 features of it with mma.sync m16n8k16 and float32 sums,
// operands by 16-byte asynchronous copies in steps of 32 along k, double-buffered.  The first product
// gathers its rows by token and forms gate and linear branch side by side, so the gating happens on the
// accumulators and neither branch reaches memory; the second reads the slots' rows and leaves float32.
#include "common.cuh"
#include "mma_utils.cuh"
#include <math.h>

namespace {
constexpr int TM = 32, TN = 64, TK = 32, SA = TK + 8;
constexpr int THREADS = 128;

template <bool GLU>
__global__ __launch_bounds__(THREADS) void moe_mma_kernel(
    const bf16* __restrict__ A, const bf16* __restrict__ Wg, const bf16* __restrict__ Wu, void* __restrict__ out_,
    const int* __restrict__ sorted_pair, const int* __restrict__ tile_expert, int top, int N, int K,
    float slope, float limit, float shift) {
    pdl_wait();
    const int e = tile_expert[blockIdx.y];
    if (e < 0) return;
    __shared__ __align__(16) bf16 As[2][TM * SA];
    __shared__ __align__(16) bf16 Gs[2][TN * SA];
    __shared__ __align__(16) bf16 Us[GLU ? 2 : 1][GLU ? TN * SA : 8];
    __shared__ int rows[TM];
    const int slot0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    if (threadIdx.x < TM) {
        const int pair = sorted_pair[slot0 + threadIdx.x];
        rows[threadIdx.x] = pair < 0 ? -1 : (GLU ? pair / top : slot0 + (int)threadIdx.x);
    }
    __syncthreads();
    const bf16* wg = Wg + (size_t)e * N * K;
    const bf16* wu = GLU ? Wu + (size_t)e * N * K : nullptr;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp & 1, wn = warp >> 1;                  // 2 x 2 warps: 16 rows x 32 features each
    const int g = lane >> 2, c = lane & 3;

    auto issue = [&](int k0, int st) {
        {   // 32 rows x 4 chunks of 8
            const int r = threadIdx.x >> 2, ch = threadIdx.x & 3;
            const int gr = rows[r], gk = k0 + ch * 8;
            const bool ok = gr >= 0 && gk < K;
            cp_async16(&As[st][r * SA + ch * 8], A + (ok ? (size_t)gr * K + gk : 0), ok);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = threadIdx.x + i * THREADS;
            const int r = idx >> 2, ch = idx & 3;
            const int gn = n0 + r, gk = k0 + ch * 8;
            const bool ok = gn < N && gk < K;
            const size_t off = ok ? (size_t)gn * K + gk : 0;
            cp_async16(&Gs[st][r * SA + ch * 8], wg + off, ok);
            if (GLU) cp_async16(&Us[st][r * SA + ch * 8], wu + off, ok);
        }
        cp_async_commit();
    };

    float accg[4][4], accu[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) accg[i][j] = accu[i][j] = 0.f;

    const int nk = (K + TK - 1) / TK;
    int st = 0;
    issue(0, 0);
    for (int kt = 0; kt < nk; ++kt) {
        if (kt + 1 < nk) {
            issue((kt + 1) * TK, st ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        uint32_t a[2][4];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
            ldmatrix_x4(a[kk], &As[st][(wm * 16 + (lane & 15)) * SA + kk * 16 + (lane >> 4) * 8]);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            uint32_t b[4];
            ldmatrix_x4(b, &Gs[st][(wn * 32 + nt * 8 + (lane & 7)) * SA + (lane >> 3) * 8]);
            mma_bf16_16816(accg[nt], a[0], b[0], b[1]);
            mma_bf16_16816(accg[nt], a[1], b[2], b[3]);
            if (GLU) {
                ldmatrix_x4(b, &Us[st][(wn * 32 + nt * 8 + (lane & 7)) * SA + (lane >> 3) * 8]);
                mma_bf16_16816(accu[nt], a[0], b[0], b[1]);
                mma_bf16_16816(accu[nt], a[1], b[2], b[3]);
            }
        }
        __syncthreads();
        st ^= 1;
    }
    pdl_trigger();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = wm * 16 + g + half * 8;
        if (rows[r] < 0) continue;
        const size_t orow = (size_t)(slot0 + r) * N;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int gn = n0 + wn * 32 + nt * 8 + 2 * c + j;
                if (gn >= N) continue;
                const float vg = accg[nt][half * 2 + j];
                if (GLU) {
                    const float gg = fminf(vg, limit);
                    const float uu = fminf(fmaxf(accu[nt][half * 2 + j], -limit), limit);
                    ((bf16*)out_)[orow + gn] = __float2bfloat16_rn(gg / (1.0f + expf(-slope * gg)) * (uu + shift));
                } else {
                    ((float*)out_)[orow + gn] = vg;
                }
            }
    }
}
}  // namespace

// The contract of rlis_moe_gemm (moe.cu) for bfloat16 operands whose k extent is a multiple of 8.
extern "C" int rlis_moe_gemm_mma(const void* A, const void* Wg, const void* Wu, void* out, const int* sorted_pair,
                                 const int* tile_expert, int max_tiles, int top, int N, int K, int glu, float slope,
                                 float limit, float shift, cudaStream_t stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (K % 8 != 0 || K <= 0) return RLIS_ERR_UNSUPPORTED;
    dim3 grid((N + TN - 1) / TN, max_tiles);
    if (grid.y > 65535) return RLIS_ERR_UNSUPPORTED;
    if (glu)
        rlis_launch(moe_mma_kernel<true>, grid, THREADS, 0, stream, (const bf16*)A, (const bf16*)Wg, (const bf16*)Wu, out,
                    sorted_pair, tile_expert, top, N, K, slope, limit, shift);
    else
        rlis_launch(moe_mma_kernel<false>, grid, THREADS, 0, stream, (const bf16*)A, (const bf16*)Wg, (const bf16*)Wu, out,
                    sorted_pair, tile_expert, top, N, K, slope, limit, shift);
    return RLIS_LAUNCH_CHECK();
}

extern "C" int rlis_moe_mma_tile_rows() { return TM; }
