// Attention over a cache of latents: every token keeps one row [latent | rotated key part] that all
// query heads share, and the keys and values of a head are linear maps of the latent.  With the
// key map folded into the query (qa = [W_uk^T q_plain | q_rot]) a head's score is qa . row and its
// value sum is taken over the latent part of the rows; the caller applies W_uv afterwards.
//
//   latent_kv_store : row = [ z[:r] / sqrt(mean(z[:r]^2) + eps) * w | rotate(z[r:]) ] -> paged cache
//                     (and, for the layer that projects both latents at once, the query latent's norm)
//   latent_q_rope   : qa[t, h, r:] = rotate(q[t, h, d:]), float32 (or bfloat16 for the tensor-core kernels)
//   attention_latent: softmax over keys 0..pos (or the last `window`), optionally with one more
//                     term exp(sink_h) in the denominator that has no value
//
// Rotation: rotate-half over the first `rot_dims` entries of the rotated part, angle = position *
// inv_freq[i] in float32, cos and sin multiplied by `mag`; the remaining entries pass unchanged.
// Scores, softmax and sums are float32; queries are float32; cache rows and the output are T.
// Keys are taken in blocks of 32 that start at multiples of 32, so a token's result does not
// depend on how the batch was cut.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;
constexpr int MAX_DV_REGS = 16;      // latent sizes up to 512

template <typename T>
__global__ __launch_bounds__(128) void latent_kv_store_kernel(
    const T* __restrict__ z, long long z_stride, const float* __restrict__ w, const float* __restrict__ inv_freq,
    const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ cache, int rank,
    int rot_width, int rot_dims, float mag, float eps, const T* __restrict__ zq, const float* __restrict__ wq,
    T* __restrict__ cq, int q_rank) {
    pdl_wait_and_trigger();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    if (zq != nullptr) {      // the query latent of the same projection's row: cq = rmsnorm(zq) * wq
        const T* qr = zq + (size_t)t * z_stride;
        float sq = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
            const float v = to_f<T>(qr[i]);
            sq = fmaf(v, v, sq);
        }
        sq = block_sum(sq, scratch);
        const float rq = 1.0f / sqrtf(sq / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq[(size_t)t * q_rank + i] = from_f<T>(to_f<T>(qr[i]) * rq * wq[i]);
    }
    const T* zr = z + (size_t)t * z_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_f<T>(zr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const int slot = slots[t];
    if (slot < 0) return;
    const float r = 1.0f / sqrtf(ss / (float)rank + eps);
    T* row = cache + (size_t)slot * (rank + rot_width);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) row[i] = from_f<T>(to_f<T>(zr[i]) * r * w[i]);
    const int half = rot_dims / 2;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < rot_width; i += blockDim.x) {
        float v = to_f<T>(zr[rank + i]);
        if (i < rot_dims) {
            const int j = i < half ? i : i - half;
            float s, c;
            sincosf(pos * inv_freq[j], &s, &c);
            s *= mag;
            c *= mag;
            const float a = to_f<T>(zr[rank + j]), b = to_f<T>(zr[rank + j + half]);
            v = i < half ? rope_first(a, b, c, s) : rope_second(a, b, c, s);
        }
        row[rank + i] = from_f<T>(v);
    }
}

template <typename T, typename TO>
__global__ void latent_q_rope_kernel(const T* __restrict__ q, TO* __restrict__ qa,
                                     const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                     int n_heads, int d_plain, int rot_width, int rot_dims, int rank, float mag,
                                     long long total) {
    pdl_wait_and_trigger();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int i = (int)(idx % rot_width);
    const long long th = idx / rot_width;                      // token * heads + head
    const int t = (int)(th / n_heads);
    const T* src = q + th * (d_plain + rot_width) + d_plain;
    float v = to_f<T>(src[i]);
    if (i < rot_dims) {
        const int half = rot_dims / 2;
        const int j = i < half ? i : i - half;
        float s, c;
        sincosf((float)positions[t] * inv_freq[j], &s, &c);
        s *= mag;
        c *= mag;
        const float a = to_f<T>(src[j]), b = to_f<T>(src[j + half]);
        v = i < half ? rope_first(a, b, c, s) : rope_second(a, b, c, s);
    }
    qa[th * (rank + rot_width) + rank + i] = from_f<TO>(v);
}

// One warp per (token, head).
template <typename T>
__global__ __launch_bounds__(WARPS * 32) void attention_latent_kernel(
    const float* __restrict__ qa, const T* __restrict__ cache, T* __restrict__ out,
    const float* __restrict__ sinks, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
    const int* __restrict__ block_tables, const int* __restrict__ token_rows, int max_blocks, int n_rows,
    int nh, int dk, int dv, int page_size, float scale, int window) {
    pdl_wait();
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gw = blockIdx.x * WARPS + warp;
    if (gw >= n_rows) return;  // no block-wide barrier below
    const int ti = gw / nh, h = gw - ti * nh;
    const int t = token_rows != nullptr ? token_rows[ti] : ti;
    const int pos = positions[t];
    const int* table = block_tables + (size_t)seq_of_token[t] * max_blocks;
    float* qs = qs_all + warp * dk;
    const float* qrow = qa + ((size_t)t * nh + h) * dk;
    for (int j = lane; j < dk; j += 32) qs[j] = qrow[j];
    __syncwarp();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    constexpr int VN = Vec16<T>::N;
    const bool vec = dk % VN == 0;
    // the extra term of the denominator is a key with score sink_h and no value
    float m = sinks != nullptr ? sinks[h] : -INFINITY;
    float l = sinks != nullptr ? 1.f : 0.f;
    float acc[MAX_DV_REGS];
#pragma unroll
    for (int i = 0; i < MAX_DV_REGS; ++i) acc[i] = 0.f;

    for (int kb = lo - (lo & 31); kb <= pos; kb += 32) {
        const int key = kb + lane;
        const bool valid = key >= lo && key <= pos;
        float s = -INFINITY;
        long long row_off = -1;
        if (valid) {
            const int page = table[key / page_size];
            if (page < 0) {
                s = NAN;  // a page the host did not map: make it visible, never read outside
            } else {
                row_off = ((long long)page * page_size + key % page_size) * dk;
                const T* krow = cache + row_off;
                float dot = 0.f;
                if (vec) {
                    for (int j = 0; j < dk; j += VN) {
                        float kv[VN];
                        load16<T>(krow + j, kv);
#pragma unroll
                        for (int u = 0; u < VN; ++u) dot = fmaf(qs[j + u], kv[u], dot);
                    }
                } else {
                    for (int j = 0; j < dk; ++j) dot = fmaf(qs[j], to_f<T>(krow[j]), dot);
                }
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_DV_REGS; ++i) acc[i] *= corr;
#pragma unroll 4
        for (int kk = 0; kk < 32; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const long long off = __shfl_sync(0xffffffffu, row_off, kk);
            const bool use = pk != 0.f && off >= 0;  // uniform over the warp
            const T* vrow = cache + (use ? off : 0);
#pragma unroll
            for (int i = 0; i < MAX_DV_REGS; ++i) {
                const int dim = lane + 32 * i;
                if (dim < dv) {
                    const float v = to_f<T>(vrow[dim]);
                    acc[i] = use ? fmaf(pk, v, acc[i]) : acc[i];
                }
            }
        }
        m = m_new;
    }
    T* orow = out + ((size_t)t * nh + h) * dv;
    const float inv_l = 1.0f / l;
#pragma unroll
    for (int i = 0; i < MAX_DV_REGS; ++i) {
        const int dim = lane + 32 * i;
        if (dim < dv) orow[dim] = from_f<T>(acc[i] * inv_l);
    }
    pdl_trigger();
}
}  // namespace

// zq != null: also cq[t, :] = rmsnorm(zq[t, :q_rank]) * wq (same eps), zq rows z_stride apart like z's.
extern "C" int rlis_latent_kv_store(const void* z, long long z_stride, const float* w, const float* inv_freq,
                                    const int* positions, const int* slots, void* cache, int n_tokens, int rank,
                                    int rot_width, int rot_dims, float mag, float eps, int dtype, const void* zq,
                                    const float* wq, void* cq, int q_rank, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || rot_width < 0 || rot_dims < 0 || rot_dims > rot_width || rot_dims % 2) return RLIS_ERR_UNSUPPORTED;
    if (dtype == RLIS_F32)
        rlis_launch(latent_kv_store_kernel<float>, n_tokens, 128, 0, stream, (const float*)z, z_stride, w, inv_freq,
                    positions, slots, (float*)cache, rank, rot_width, rot_dims, mag, eps, (const float*)zq, wq, (float*)cq,
                    q_rank);
    else if (dtype == RLIS_BF16)
        rlis_launch(latent_kv_store_kernel<bf16>, n_tokens, 128, 0, stream, (const bf16*)z, z_stride, w, inv_freq,
                    positions, slots, (bf16*)cache, rank, rot_width, rot_dims, mag, eps, (const bf16*)zq, wq, (bf16*)cq,
                    q_rank);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

// out_bf16 != 0: qa is bfloat16 (for the tensor-core attention kernels), else float32.
extern "C" int rlis_latent_q_rope(const void* q, void* qa, const float* inv_freq, const int* positions,
                                  int n_tokens, int n_heads, int d_plain, int rot_width, int rot_dims, int rank,
                                  float mag, int dtype, int out_bf16, cudaStream_t stream) {
    const long long total = (long long)n_tokens * n_heads * rot_width;
    if (total <= 0) return 0;
    if (rot_dims < 0 || rot_dims > rot_width || rot_dims % 2) return RLIS_ERR_UNSUPPORTED;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == RLIS_F32 && !out_bf16)
        rlis_launch(latent_q_rope_kernel<float, float>, blocks, 256, 0, stream, (const float*)q, (float*)qa, inv_freq,
                    positions, n_heads, d_plain, rot_width, rot_dims, rank, mag, total);
    else if (dtype == RLIS_BF16 && !out_bf16)
        rlis_launch(latent_q_rope_kernel<bf16, float>, blocks, 256, 0, stream, (const bf16*)q, (float*)qa, inv_freq,
                    positions, n_heads, d_plain, rot_width, rot_dims, rank, mag, total);
    else if (dtype == RLIS_BF16)
        rlis_launch(latent_q_rope_kernel<bf16, bf16>, blocks, 256, 0, stream, (const bf16*)q, (bf16*)qa, inv_freq,
                    positions, n_heads, d_plain, rot_width, rot_dims, rank, mag, total);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

extern "C" int rlis_attention_latent(const float* qa, const void* cache, void* out, const float* sinks,
                                     const int* seq_of_token, const int* positions, const int* block_tables,
                                     const int* token_rows, int max_blocks, int n_tokens, int nh, int dk, int dv,
                                     int page_size, float scale, int window, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dk <= 0 || dv <= 0 || dv > dk || dv > 32 * MAX_DV_REGS || dk > 2048 || nh <= 0) return RLIS_ERR_UNSUPPORTED;
    const long long n_rows = (long long)n_tokens * nh;
    if (n_rows > 0x7fffffffLL) return RLIS_ERR_UNSUPPORTED;
    const unsigned blocks = (unsigned)((n_rows + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * dk * sizeof(float);
    if (dtype == RLIS_F32)
        rlis_launch(attention_latent_kernel<float>, blocks, WARPS * 32, smem, stream, qa, (const float*)cache,
                    (float*)out, sinks, seq_of_token, positions, block_tables, token_rows, max_blocks, (int)n_rows,
                    nh, dk, dv, page_size, scale, window);
    else if (dtype == RLIS_BF16)
        rlis_launch(attention_latent_kernel<bf16>, blocks, WARPS * 32, smem, stream, qa, (const bf16*)cache,
                    (bf16*)out, sinks, seq_of_token, positions, block_tables, token_rows, max_blocks, (int)n_rows,
                    nh, dk, dv, page_size, scale, window);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}
