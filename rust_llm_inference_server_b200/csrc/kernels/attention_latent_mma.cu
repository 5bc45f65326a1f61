// Attention over a cache of latent rows on the tensor cores (bfloat16; mma.sync m16n8k16 with
// float32 sums), for prompt portions and for single decoded tokens.  The interface is that of
// attention_latent.cu: a row [latent | rotated key part] of DK entries a token, shared by all heads;
// score = scale * qa . row; values are the first DV entries of the same rows; an optional sink term
// exp(sink_h) in a head's softmax denominator.
//
// Keys come to shared memory by 16-byte asynchronous copies, double-buffered, rows padded by 8
// entries; a warp copies whole rows in runs of 512 contiguous bytes.
//   prompts: one head x 64 tokens a CTA of 8 warps, stages of 64 keys.  Two warps share 16 tokens:
//            each holds HALF of the value columns (its output sums are DV / 4 registers a thread) and
//            forms the scores of 32 of a stage's keys; the two exchange row maxima and the rounded
//            weights through shared memory (three barriers of 64 threads a stage).
//   decode : 16 heads of one token and one piece of its context a CTA of 4 warps, stages of 32 keys,
//            so that two CTAs fit an SM at the widest rows.  Warp w forms the scores of 8 of a stage's
//            keys and sums a QUARTER of the value columns over all 32; maxima and weights go through
//            shared memory.  Several pieces of a context are merged by a second small kernel.
// Queries arrive as bfloat16 (copied asynchronously) or as float32 (rounded once, into shared memory).
#include "common.cuh"
#include "mma_utils.cuh"
#include <math.h>

namespace {
constexpr int LF_BN_MAX = 64;             // the longest stage: pieces of a context are multiples of it
constexpr float LOG2E = 1.4426950408889634f;

// Barrier over the two warps of pair `p` (named barriers 1..4; 0 is __syncthreads).
__device__ __forceinline__ void pair_barrier(int p) { asm volatile("bar.sync %0, 64;" ::"r"(p + 1) : "memory"); }

struct LatentArgs {
    const void* qa;           // [T, nh, dk], float32 or (q_bf16) bfloat16
    const bf16* cache;        // [pages, 1, page, dk]
    bf16* out;                // [T, nh, dv]
    const float* sinks;       // [nh] or null
    const int* tiles;         // prompts: [n][2] (batch entry, first token of the tile)
    const int* cu_seqlens;
    const int* ctx_lens;
    const int* block_tables;
    const int* dec_rows;      // decode: token row and batch entry of every single token
    const int* dec_seqs;
    float* scratch;           // decode, several pieces: [n_dec][head tiles][pieces][16][dv + 2]
    int max_blocks, nh, dk, page_size, window, pieces, piece_keys;
    float scale;
    int q_bf16;
};

// Prompts: 64 query rows (tokens of one head) a CTA, four warp pairs, stages of 64 keys.
template <int DV>
__global__ __launch_bounds__(256) void latent_flash_kernel(const LatentArgs a) {
    pdl_wait();
    constexpr int LF_THREADS = 256;
    constexpr int LF_BN = 64;                    // keys a stage
    constexpr int NT = 4;                        // score tiles (8 keys each) a warp forms a stage
    constexpr int QR = 64;                       // query rows a CTA
    constexpr int NO = DV / 16;                  // output tiles (8 columns each) a warp owns: half of DV / 8
    const int dk = a.dk, stride = dk + 8, ksteps = dk / 16, cpr = dk / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);              // [QR][stride]
    bf16* kbuf = qs + QR * stride;                             // [2][64][stride]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int half = warp & 1, pair = warp >> 1;
    const int nh = a.nh;

    const int b = a.tiles[2 * blockIdx.y], t0 = a.tiles[2 * blockIdx.y + 1];
    const int q_start = a.cu_seqlens[b], q_len = a.cu_seqlens[b + 1] - q_start;
    const int q_row0 = q_start + t0;
    const int n_q_rows = min(64, q_len - t0);
    const int head0 = blockIdx.x;
    const int pos_base = a.ctx_lens[b] - q_len + t0;           // position of the tile's first token
    const int k_hi = pos_base + n_q_rows;                      // exclusive
    const int k_lo = a.window > 0 ? max(0, pos_base - a.window + 1) : 0;
    const int* table = a.block_tables + (size_t)b * a.max_blocks;

    // queries -> shared memory: bfloat16 ones by 16-byte asynchronous copies (they join the first stage's
    // group), float32 ones rounded once on the way; rows beyond the tile (or the heads) are zero
    if (a.q_bf16) {
        const bf16* qsrc = reinterpret_cast<const bf16*>(a.qa);
        for (int idx = threadIdx.x; idx < QR * cpr; idx += LF_THREADS) {
            const int r = idx / cpr, c16 = idx - r * cpr;
            const bool valid = r < n_q_rows;
            const size_t row = (size_t)(q_row0 + (valid ? r : 0)) * nh + head0;
            cp_async16(qs + r * stride + c16 * 8, qsrc + row * dk + c16 * 8, valid);
        }
    } else {
        const float* qsrc = reinterpret_cast<const float*>(a.qa);
        for (int idx = threadIdx.x; idx < QR * (dk / 2); idx += LF_THREADS) {
            const int r = idx / (dk / 2), j = (idx - r * (dk / 2)) * 2;
            float2 v = make_float2(0.f, 0.f);
            if (r < n_q_rows) v = *reinterpret_cast<const float2*>(qsrc + ((size_t)(q_row0 + r) * nh + head0) * dk + j);
            *reinterpret_cast<uint32_t*>(qs + r * stride + j) = pack_bf16(v.x, v.y);
        }
    }

    const int kt0 = k_lo / LF_BN, kt1 = k_hi > k_lo ? (k_hi + LF_BN - 1) / LF_BN : kt0;
    if (kt0 >= kt1) {      // no key at all: nothing will wait for the queries' copies
        cp_async_commit();
        cp_async_wait<0>();
    }
    const int page_size = a.page_size;
    // A warp copies 8 of a stage's keys: lanes 0..7 look the keys' pages up (one load each), the row
    // addresses go round by shuffle, and the 32 lanes copy a row in runs of 512 contiguous bytes.
    auto issue = [&](int kt, int stage) {
        const int key0 = kt * LF_BN + warp * 8;
        long long my_off = -1;
        if (lane < 8) {
            const int key = key0 + lane;
            if (key < k_hi && key >= k_lo) {
                const int pi = key / page_size;
                my_off = ((long long)table[pi] * page_size + (key - pi * page_size)) * dk;
            }
        }
        bf16* dst0 = kbuf + ((size_t)stage * LF_BN + warp * 8) * stride;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const long long off = __shfl_sync(0xffffffffu, my_off, k);
            const bool valid = off >= 0;
            const bf16* src = a.cache + (valid ? off : 0);
            bf16* dst = dst0 + k * stride;
            for (int c16 = lane; c16 < cpr; c16 += 32) cp_async16(dst + c16 * 8, src + c16 * 8, valid);
        }
        cp_async_commit();
    };

    // this lane's two rows (g and g + 8 of the warp's 16)
    const int row_base = pair * 16;
    const bool rv0 = row_base + g < n_q_rows, rv1 = row_base + g + 8 < n_q_rows;
    const int pos0 = pos_base + row_base + g, pos1 = pos0 + 8;
    const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int lo1 = a.window > 0 ? max(0, pos1 - a.window + 1) : 0;
    // the sink is one more key, with a score of its own and no value
    const bool has_sink = a.sinks != nullptr;
    float m_run[2], l_run[2];
    m_run[0] = has_sink && rv0 ? a.sinks[head0] * LOG2E : -INFINITY;
    m_run[1] = has_sink && rv1 ? a.sinks[head0] * LOG2E : -INFINITY;
    l_run[0] = has_sink && rv0 ? 1.f : 0.f;
    l_run[1] = has_sink && rv1 ? 1.f : 0.f;
    float oacc[NO][4];
#pragma unroll
    for (int n = 0; n < NO; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[n][e] = 0.f;
    const float scale_log2 = a.scale * LOG2E;
    const int key_off = half * 32;                           // the keys within a stage whose scores this warp forms
    // where the two warps of a pair exchange maxima and weights, 8 words a lane
    float* xch = reinterpret_cast<float*>(kbuf + (size_t)2 * LF_BN * stride);
    float* xw = xch + ((pair * 2 + half) * 32 + lane) * 8;
    const float* xo = xch + ((pair * 2 + (half ^ 1)) * 32 + lane) * 8;
    const int col0 = half * (DV / 2);                        // this warp's value columns

    int stage = 0;
    if (kt0 < kt1) issue(kt0, 0);
    for (int kt = kt0; kt < kt1; ++kt) {
        if (kt + 1 < kt1) {
            issue(kt + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* kst = kbuf + (size_t)stage * LF_BN * stride;
        const bf16* ks_ = kst + (size_t)key_off * stride;          // the keys whose scores this warp forms

        float sacc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[nt][e] = 0.f;
        for (int ks = 0; ks < ksteps; ++ks) {
            uint32_t qa[4];
            ldmatrix_x4(qa, qs + (row_base + ((lane >> 3) & 1) * 8 + (lane & 7)) * stride + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nt2 = 0; nt2 < NT / 2; ++nt2) {
                uint32_t kb[4];
                ldmatrix_x4(kb, ks_ + ((nt2 * 2 + (lane >> 4)) * 8 + (lane & 7)) * stride + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(sacc[2 * nt2], qa, kb[0], kb[1]);
                mma_bf16_16816(sacc[2 * nt2 + 1], qa, kb[2], kb[3]);
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
        const int key_base = kt * LF_BN + key_off;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key_base + nt * 8 + 2 * c + e;
                float s0 = sacc[nt][e] * scale_log2, s1 = sacc[nt][2 + e] * scale_log2;
                if (!(rv0 && key <= pos0 && key >= lo0 && key >= k_lo && key < k_hi)) s0 = -INFINITY;
                if (!(rv1 && key <= pos1 && key >= lo1 && key >= k_lo && key < k_hi)) s1 = -INFINITY;
                sacc[nt][e] = s0;
                sacc[nt][2 + e] = s1;
                mx0 = fmaxf(mx0, s0);
                mx1 = fmaxf(mx1, s1);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // the other warp of the pair has the maxima of the stage's other 32 keys
        xw[0] = mx0;
        xw[1] = mx1;
        pair_barrier(pair);
        mx0 = fmaxf(mx0, xo[0]);
        mx1 = fmaxf(mx1, xo[1]);
        pair_barrier(pair);
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float corr0 = exp2f(m_run[0] - ms0), corr1 = exp2f(m_run[1] - ms1);
        // weights, rounded to bfloat16 as the A operand of the value product: [16 keys][4 registers]
        uint32_t pown[NT / 2][4];
#pragma unroll
        for (int kk = 0; kk < NT / 2; ++kk) {
            pown[kk][0] = pack_bf16(exp2f(sacc[2 * kk][0] - ms0), exp2f(sacc[2 * kk][1] - ms0));
            pown[kk][1] = pack_bf16(exp2f(sacc[2 * kk][2] - ms1), exp2f(sacc[2 * kk][3] - ms1));
            pown[kk][2] = pack_bf16(exp2f(sacc[2 * kk + 1][0] - ms0), exp2f(sacc[2 * kk + 1][1] - ms0));
            pown[kk][3] = pack_bf16(exp2f(sacc[2 * kk + 1][2] - ms1), exp2f(sacc[2 * kk + 1][3] - ms1));
        }
        constexpr int PK = 4;                       // blocks of 16 keys in the value product
        uint32_t pall[PK][4];
        {
            uint32_t* xwu = reinterpret_cast<uint32_t*>(xw);
            const uint32_t* xou = reinterpret_cast<const uint32_t*>(xo);
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk)
#pragma unroll
                for (int e = 0; e < 4; ++e) xwu[kk * 4 + e] = pown[kk][e];
            pair_barrier(pair);
            uint32_t poth[NT / 2][4];
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk)
#pragma unroll
                for (int e = 0; e < 4; ++e) poth[kk][e] = xou[kk * 4 + e];
#pragma unroll
            for (int kk = 0; kk < PK; ++kk)          // blocks 0, 1 are the first warp's keys, 2, 3 the second's
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    pall[kk][e] = (kk >> 1) == half ? pown[kk % (NT / 2)][e] : poth[kk % (NT / 2)][e];
        }
        // the row sums are taken over the rounded weights, in key order, so that both warps of a pair
        // (and numerator and denominator) see the same numbers
        float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
        for (int kk = 0; kk < PK; ++kk) {
            const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pall[kk][0]));
            const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pall[kk][1]));
            const float2 a2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pall[kk][2]));
            const float2 a3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pall[kk][3]));
            ls0 += (a0.x + a0.y) + (a2.x + a2.y);
            ls1 += (a1.x + a1.y) + (a3.x + a3.y);
        }
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, 1);
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, 2);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, 1);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, 2);
        l_run[0] = l_run[0] * corr0 + ls0;
        l_run[1] = l_run[1] * corr1 + ls1;
        m_run[0] = mn0;
        m_run[1] = mn1;
#pragma unroll
        for (int n = 0; n < NO; ++n) {
            oacc[n][0] *= corr0;
            oacc[n][1] *= corr0;
            oacc[n][2] *= corr1;
            oacc[n][3] *= corr1;
        }
        const bf16* vs_ = kst;                      // the values of all 64 keys
#pragma unroll
        for (int kk = 0; kk < PK; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < NO / 2; ++n2) {
                uint32_t vb[4];
                const int mat = lane >> 3;
                ldmatrix_x4_trans(vb, vs_ + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * stride + col0 + (n2 * 2 + (mat >> 1)) * 8);
                mma_bf16_16816(oacc[2 * n2], pall[kk], vb[0], vb[1]);
                mma_bf16_16816(oacc[2 * n2 + 1], pall[kk], vb[2], vb[3]);
            }
        }
        __syncthreads();
        stage ^= 1;
    }

    const float inv0 = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
    const float inv1 = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
    if (rv0) {
        bf16* o = a.out + ((size_t)(q_row0 + row_base + g) * nh + head0) * DV + col0;
#pragma unroll
        for (int n = 0; n < NO; ++n)
            *reinterpret_cast<uint32_t*>(o + n * 8 + 2 * c) = pack_bf16(oacc[n][0] * inv0, oacc[n][1] * inv0);
    }
    if (rv1) {
        bf16* o = a.out + ((size_t)(q_row0 + row_base + g + 8) * nh + head0) * DV + col0;
#pragma unroll
        for (int n = 0; n < NO; ++n)
            *reinterpret_cast<uint32_t*>(o + n * 8 + 2 * c) = pack_bf16(oacc[n][2] * inv1, oacc[n][3] * inv1);
    }
    pdl_trigger();
}

// Two 8x8 b16 matrices; lanes 0..15 supply the row addresses (the others' are ignored but must be valid).
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(smem_u32(smem_row)));
}

// Decode: 16 heads of one token and one piece of its context a CTA of four warps; stages of 32 keys.
// Warp w forms the scores of keys 8 w .. 8 w + 7 of a stage (all 16 heads), the four exchange row maxima
// and the rounded weights through shared memory, and warp w sums the values' columns w DV/4 .. (w+1) DV/4
// over all 32 keys.  Every warp keeps the same running (max, sum); nothing is merged at the end.
template <int DV>
__global__ __launch_bounds__(128) void latent_decode_kernel(const LatentArgs a) {
    pdl_wait();
    constexpr int BN = 32, NO = DV / 32, PS = BN + 8;   // keys a stage; output tiles a warp; row pitch of the weights
    const int dk = a.dk, stride = dk + 8, ksteps = dk / 16, cpr = dk / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);              // [16][stride]
    bf16* kbuf = qs + 16 * stride;                             // [2][32][stride]
    bf16* pbuf = kbuf + 2 * BN * stride;                       // [16][PS] weights of a stage, bfloat16
    float* mxw = reinterpret_cast<float*>(pbuf + 16 * PS);     // [4 warps][16 rows] maxima

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int nh = a.nh;
    const int di = blockIdx.y;
    const int b = a.dec_seqs[di];
    const int q_row0 = a.dec_rows[di];
    const int head0 = blockIdx.x * 16;
    const int pos = a.ctx_lens[b] - 1;
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int k_lo = max(lo, (int)blockIdx.z * a.piece_keys);
    const int k_hi = min(pos + 1, (int)(blockIdx.z + 1) * a.piece_keys);
    const int* table = a.block_tables + (size_t)b * a.max_blocks;
    const int page_size = a.page_size;

    if (a.q_bf16) {
        const bf16* qsrc = reinterpret_cast<const bf16*>(a.qa);
        for (int idx = threadIdx.x; idx < 16 * cpr; idx += 128) {
            const int r = idx / cpr, c16 = idx - r * cpr;
            const bool valid = head0 + r < nh;
            cp_async16(qs + r * stride + c16 * 8, qsrc + ((size_t)q_row0 * nh + head0 + (valid ? r : 0)) * dk + c16 * 8, valid);
        }
    } else {
        const float* qsrc = reinterpret_cast<const float*>(a.qa);
        for (int idx = threadIdx.x; idx < 16 * (dk / 2); idx += 128) {
            const int r = idx / (dk / 2), j = (idx - r * (dk / 2)) * 2;
            float2 v = make_float2(0.f, 0.f);
            if (head0 + r < nh) v = *reinterpret_cast<const float2*>(qsrc + ((size_t)q_row0 * nh + head0 + r) * dk + j);
            *reinterpret_cast<uint32_t*>(qs + r * stride + j) = pack_bf16(v.x, v.y);
        }
    }
    const int kt0 = k_lo / BN, kt1 = k_hi > k_lo ? (k_hi + BN - 1) / BN : kt0;
    auto issue = [&](int kt, int stage) {      // a warp copies 8 keys' rows, in runs of 512 contiguous bytes
        const int key0 = kt * BN + warp * 8;
        long long my_off = -1;
        if (lane < 8) {
            const int key = key0 + lane;
            if (key < k_hi && key >= k_lo) {
                const int pi = key / page_size;
                my_off = ((long long)table[pi] * page_size + (key - pi * page_size)) * dk;
            }
        }
        bf16* dst0 = kbuf + ((size_t)stage * BN + warp * 8) * stride;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const long long off = __shfl_sync(0xffffffffu, my_off, k);
            const bool valid = off >= 0;
            const bf16* src = a.cache + (valid ? off : 0);
            for (int c16 = lane; c16 < cpr; c16 += 32) cp_async16(dst0 + k * stride + c16 * 8, src + c16 * 8, valid);
        }
        cp_async_commit();
    };

    const int h0 = head0 + g, h1 = h0 + 8;
    const bool rv0 = h0 < nh, rv1 = h1 < nh;
    // the sink is one more key with a score of its own and no value; it belongs to the first piece
    const bool has_sink = a.sinks != nullptr && blockIdx.z == 0;
    float m_run[2], l_run[2];
    m_run[0] = has_sink && rv0 ? a.sinks[h0] * LOG2E : -INFINITY;
    m_run[1] = has_sink && rv1 ? a.sinks[h1] * LOG2E : -INFINITY;
    l_run[0] = has_sink && rv0 ? 1.f : 0.f;
    l_run[1] = has_sink && rv1 ? 1.f : 0.f;
    float oacc[NO][4];
#pragma unroll
    for (int n = 0; n < NO; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[n][e] = 0.f;
    const float scale_log2 = a.scale * LOG2E;
    const int col0 = warp * (DV / 4);

    if (kt0 < kt1) issue(kt0, 0); else { cp_async_commit(); }
    int stage = 0;
    for (int kt = kt0; kt < kt1; ++kt) {
        cp_async_wait<0>();
        __syncthreads();                       // this stage has landed, and everybody is done with the other one
        if (kt + 1 < kt1) issue(kt + 1, stage ^ 1);
        const bf16* kst = kbuf + (size_t)stage * BN * stride;

        // scores of this warp's 8 keys, two chains of products
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
        const bf16* qrow = qs + (((lane >> 3) & 1) * 8 + (lane & 7)) * stride + (lane >> 4) * 8;
        const bf16* krow = kst + (warp * 8 + (lane & 7)) * stride + ((lane >> 3) & 1) * 8;
        int ks = 0;
        for (; ks + 1 < ksteps; ks += 2) {
            uint32_t qa0[4], qa1[4], b0, b1, b2, b3;
            ldmatrix_x4(qa0, qrow + ks * 16);
            ldmatrix_x2(b0, b1, krow + ks * 16);
            ldmatrix_x4(qa1, qrow + ks * 16 + 16);
            ldmatrix_x2(b2, b3, krow + ks * 16 + 16);
            mma_bf16_16816(sa, qa0, b0, b1);
            mma_bf16_16816(sb, qa1, b2, b3);
        }
        if (ks < ksteps) {
            uint32_t qa0[4], b0, b1;
            ldmatrix_x4(qa0, qrow + ks * 16);
            ldmatrix_x2(b0, b1, krow + ks * 16);
            mma_bf16_16816(sa, qa0, b0, b1);
        }
        float s[4];
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int key = kt * BN + warp * 8 + 2 * c + e;
            const bool seen = key <= pos && key >= k_lo && key < k_hi;
            s[e] = rv0 && seen ? (sa[e] + sb[e]) * scale_log2 : -INFINITY;
            s[2 + e] = rv1 && seen ? (sa[2 + e] + sb[2 + e]) * scale_log2 : -INFINITY;
            mx0 = fmaxf(mx0, s[e]);
            mx1 = fmaxf(mx1, s[2 + e]);
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if (c == 0) {
            mxw[warp * 16 + g] = mx0;
            mxw[warp * 16 + g + 8] = mx1;
        }
        __syncthreads();
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            mx0 = fmaxf(mx0, mxw[w * 16 + g]);
            mx1 = fmaxf(mx1, mxw[w * 16 + g + 8]);
        }
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float corr0 = exp2f(m_run[0] - ms0), corr1 = exp2f(m_run[1] - ms1);
        *reinterpret_cast<uint32_t*>(pbuf + g * PS + warp * 8 + 2 * c) = pack_bf16(exp2f(s[0] - ms0), exp2f(s[1] - ms0));
        *reinterpret_cast<uint32_t*>(pbuf + (g + 8) * PS + warp * 8 + 2 * c) = pack_bf16(exp2f(s[2] - ms1), exp2f(s[3] - ms1));
        __syncthreads();
        // all 32 keys' weights as the A operand; the row sums are taken over the rounded weights
        uint32_t pa[2][4];
        float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            ldmatrix_x4(pa[kk], pbuf + (((lane >> 3) & 1) * 8 + (lane & 7)) * PS + kk * 16 + (lane >> 4) * 8);
            const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pa[kk][0]));
            const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pa[kk][1]));
            const float2 a2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pa[kk][2]));
            const float2 a3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pa[kk][3]));
            ls0 += (a0.x + a0.y) + (a2.x + a2.y);
            ls1 += (a1.x + a1.y) + (a3.x + a3.y);
        }
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, 1);
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, 2);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, 1);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, 2);
        l_run[0] = l_run[0] * corr0 + ls0;
        l_run[1] = l_run[1] * corr1 + ls1;
        m_run[0] = mn0;
        m_run[1] = mn1;
#pragma unroll
        for (int n = 0; n < NO; ++n) {
            oacc[n][0] *= corr0;
            oacc[n][1] *= corr0;
            oacc[n][2] *= corr1;
            oacc[n][3] *= corr1;
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < NO / 2; ++n2) {
                uint32_t vb[4];
                const int mat = lane >> 3;
                ldmatrix_x4_trans(vb, kst + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * stride + col0 + (n2 * 2 + (mat >> 1)) * 8);
                mma_bf16_16816(oacc[2 * n2], pa[kk], vb[0], vb[1]);
                mma_bf16_16816(oacc[2 * n2 + 1], pa[kk], vb[2], vb[3]);
            }
        }
        stage ^= 1;
    }
    cp_async_wait<0>();

    if (a.pieces == 1) {
        const float inv0 = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
        if (rv0) {
            bf16* o = a.out + ((size_t)q_row0 * nh + h0) * DV + col0;
#pragma unroll
            for (int n = 0; n < NO; ++n)
                *reinterpret_cast<uint32_t*>(o + n * 8 + 2 * c) = pack_bf16(oacc[n][0] * inv0, oacc[n][1] * inv0);
        }
        if (rv1) {
            bf16* o = a.out + ((size_t)q_row0 * nh + h1) * DV + col0;
#pragma unroll
            for (int n = 0; n < NO; ++n)
                *reinterpret_cast<uint32_t*>(o + n * 8 + 2 * c) = pack_bf16(oacc[n][2] * inv1, oacc[n][3] * inv1);
        }
    } else {
        float* part = a.scratch + (((size_t)blockIdx.y * gridDim.x + blockIdx.x) * a.pieces + blockIdx.z) * 16 * (DV + 2);
        float* p0 = part + g * (DV + 2);
        float* p1 = part + (g + 8) * (DV + 2);
        if (warp == 0 && c == 0) {
            p0[DV] = m_run[0]; p0[DV + 1] = l_run[0];
            p1[DV] = m_run[1]; p1[DV + 1] = l_run[1];
        }
#pragma unroll
        for (int n = 0; n < NO; ++n) {
            const int col = col0 + n * 8 + 2 * c;
            *reinterpret_cast<float2*>(p0 + col) = make_float2(oacc[n][0], oacc[n][1]);
            *reinterpret_cast<float2*>(p1 + col) = make_float2(oacc[n][2], oacc[n][3]);
        }
    }
    pdl_trigger();
}

static size_t latent_decode_smem_bytes(int dk) {
    return (size_t)(16 + 2 * 32) * (dk + 8) * sizeof(bf16) + (size_t)16 * (32 + 8) * sizeof(bf16) + 4 * 16 * sizeof(float);
}

template <int DV>
int launch_latent_decode(const LatentArgs& a, dim3 grid, cudaStream_t stream) {
    const size_t smem = latent_decode_smem_bytes(a.dk);
    if (smem > 227 * 1024) return RLIS_ERR_UNSUPPORTED;
    static size_t allowed = 0;
    if (smem > allowed) {
        cudaFuncSetAttribute(latent_decode_kernel<DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        allowed = smem;
    }
    rlis_launch(latent_decode_kernel<DV>, grid, 128, smem, stream, a);
    return RLIS_LAUNCH_CHECK();
}

// One CTA a (decoded token, head): folds the pieces' (max, sum, output) into the output row.  The
// pieces' weights exp2(max_p - max) are worked out once, by one thread a piece.
template <int DV>
__global__ void latent_merge_kernel(const float* __restrict__ scratch, bf16* __restrict__ out,
                                    const int* __restrict__ dec_rows, int nh, int head_tiles, int pieces) {
    pdl_wait_and_trigger();
    extern __shared__ float wts[];                 // [pieces] weights, then [pieces] scratch
    __shared__ float red[33];
    const int di = blockIdx.y, h = blockIdx.x;
    const float* part = scratch + (((size_t)di * head_tiles + h / 16) * pieces) * 16 * (DV + 2) + (size_t)(h % 16) * (DV + 2);
    const size_t piece_stride = (size_t)16 * (DV + 2);
    float m = -INFINITY;
    for (int p = threadIdx.x; p < pieces; p += blockDim.x) {
        wts[pieces + p] = part[p * piece_stride + DV];
        m = fmaxf(m, wts[pieces + p]);
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = -INFINITY;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) m = fmaxf(m, red[w]);
    const float ms = m == -INFINITY ? 0.f : m;
    float l = 0.f;
    for (int p = threadIdx.x; p < pieces; p += blockDim.x) {
        const float w = exp2f(wts[pieces + p] - ms);
        wts[p] = w;
        l += part[p * piece_stride + DV + 1] * w;
    }
    l = block_sum(l, red);                         // (its barriers also publish the weights)
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    bf16* o = out + ((size_t)dec_rows[di] * nh + h) * DV;
    // two columns a thread at a time (rows of DV + 2 floats are 8-byte aligned), eight pieces' loads in flight
    for (int col = threadIdx.x * 2; col < DV; col += blockDim.x * 2) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
        for (int p = 0; p < pieces; ++p) {
            const float2 v = *reinterpret_cast<const float2*>(part + p * piece_stride + col);
            a0 = fmaf(v.x, wts[p], a0);
            a1 = fmaf(v.y, wts[p], a1);
        }
        *reinterpret_cast<uint32_t*>(o + col) = pack_bf16(a0 * inv, a1 * inv);
    }
}

static size_t latent_smem_bytes(int dk) {      // queries, two stages of keys, the pairs' exchange words
    return (size_t)(64 + 2 * 64) * (dk + 8) * sizeof(bf16) + (size_t)256 * 8 * sizeof(float);
}

template <int DV>
int launch_latent(const LatentArgs& a, dim3 grid, cudaStream_t stream) {
    const size_t smem = latent_smem_bytes(a.dk);
    if (smem > 227 * 1024) return RLIS_ERR_UNSUPPORTED;      // 232,448 bytes: the most a CTA can ask for
    static size_t allowed = 0;
    if (smem > allowed) {
        cudaFuncSetAttribute(latent_flash_kernel<DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        allowed = smem;
    }
    rlis_launch(latent_flash_kernel<DV>, grid, 256, smem, stream, a);
    return RLIS_LAUNCH_CHECK();
}
}  // namespace

// Whether the tensor-core kernels take these sizes: value widths of 64, 128, 256 or 512 and rows
// that are multiples of 16 entries and fit shared memory with two stages of keys.
extern "C" int rlis_attention_latent_mma_takes(int dk, int dv) {
    if (!(dv == 64 || dv == 128 || dv == 256 || dv == 512) || dk % 16 || dk < dv || dk <= 0) return 0;
    return latent_smem_bytes(dk) <= 227 * 1024 ? 1 : 0;
}

extern "C" int rlis_attention_latent_prefill(const void* qa, int q_bf16, const void* cache, void* out, const float* sinks,
                                             const int* tiles, int n_tiles, const int* cu_seqlens,
                                             const int* ctx_lens, const int* block_tables, int max_blocks, int nh,
                                             int dk, int dv, int page_size, float scale, int window,
                                             cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!rlis_attention_latent_mma_takes(dk, dv) || n_tiles > 65535 || nh <= 0) return RLIS_ERR_UNSUPPORTED;
    LatentArgs a = {qa, (const bf16*)cache, (bf16*)out, sinks, tiles, cu_seqlens, ctx_lens, block_tables, nullptr,
                    nullptr, nullptr, max_blocks, nh, dk, page_size, window, 1, 0, scale, q_bf16};
    dim3 grid(nh, n_tiles);
    switch (dv) {
        case 64: return launch_latent<64>(a, grid, stream);
        case 128: return launch_latent<128>(a, grid, stream);
        case 256: return launch_latent<256>(a, grid, stream);
        default: return launch_latent<512>(a, grid, stream);
    }
}

// pieces > 1: `scratch` holds n_dec * ceil(nh / 16) * pieces * 16 * (dv + 2) floats and the context
// is cut into pieces of `piece_keys` keys (a multiple of 64).
extern "C" int rlis_attention_latent_decode(const void* qa, int q_bf16, const void* cache, void* out, const float* sinks,
                                            float* scratch, const int* dec_rows, const int* dec_seqs,
                                            const int* ctx_lens, const int* block_tables, int max_blocks, int n_dec,
                                            int nh, int dk, int dv, int page_size, float scale, int window,
                                            int pieces, int piece_keys, cudaStream_t stream) {
    if (n_dec <= 0) return 0;
    if (!rlis_attention_latent_mma_takes(dk, dv) || n_dec > 65535 || nh <= 0 || pieces < 1 || pieces > 4096 ||
        (pieces > 1 && (scratch == nullptr || piece_keys <= 0 || piece_keys % LF_BN_MAX)))
        return RLIS_ERR_UNSUPPORTED;
    if (pieces == 1) piece_keys = 0x40000000;
    LatentArgs a = {qa, (const bf16*)cache, (bf16*)out, sinks, nullptr, nullptr, ctx_lens, block_tables, dec_rows,
                    dec_seqs, scratch, max_blocks, nh, dk, page_size, window, pieces, piece_keys, scale, q_bf16};
    const int head_tiles = (nh + 15) / 16;
    dim3 grid(head_tiles, n_dec, pieces);
    int rc;
    switch (dv) {
        case 64: rc = launch_latent_decode<64>(a, grid, stream); break;
        case 128: rc = launch_latent_decode<128>(a, grid, stream); break;
        case 256: rc = launch_latent_decode<256>(a, grid, stream); break;
        default: rc = launch_latent_decode<512>(a, grid, stream); break;
    }
    if (rc != 0 || pieces == 1) return rc;
    dim3 mgrid(nh, n_dec);
    switch (dv) {
        case 64: rlis_launch(latent_merge_kernel<64>, mgrid, 32, (size_t)2 * pieces * sizeof(float), stream, (const float*)scratch, (bf16*)out, dec_rows, nh, head_tiles, pieces); break;
        case 128: rlis_launch(latent_merge_kernel<128>, mgrid, 64, (size_t)2 * pieces * sizeof(float), stream, (const float*)scratch, (bf16*)out, dec_rows, nh, head_tiles, pieces); break;
        case 256: rlis_launch(latent_merge_kernel<256>, mgrid, 128, (size_t)2 * pieces * sizeof(float), stream, (const float*)scratch, (bf16*)out, dec_rows, nh, head_tiles, pieces); break;
        default: rlis_launch(latent_merge_kernel<512>, mgrid, 256, (size_t)2 * pieces * sizeof(float), stream, (const float*)scratch, (bf16*)out, dec_rows, nh, head_tiles, pieces); break;
    }
    return RLIS_LAUNCH_CHECK();
}
