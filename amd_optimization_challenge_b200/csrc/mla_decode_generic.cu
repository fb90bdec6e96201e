// Generic stage-1 MLA decode kernel: every head count / q_len / cache format, warp-level tensor
// cores (nvcuda::wmma, bf16) with the cache tile dequantised to bf16 in shared memory.
//
// It exists as the always-applicable path and as the on-GPU cross-check of the tcgen05 kernel.
// One CTA = one KV span (see mla_common.cuh) x 16 query rows; 64-token tiles:
//   gather rows (128-bit loads through the page table) -> bf16 tile [64][576]
//   S[16 x 64]   = Q[16 x 576] . K^T           (8 warps: 4 token blocks x 2 halves of the 576 dims)
//   online softmax in the exp2 domain, lazy re-centering (the accumulator is rescaled only when
//   a tile's maximum exceeds the reference maximum by more than 2^8)
//   O[16 x 512] += P[16 x 64] . V[64 x 512]    (8 warps x 64 output dims; V = first 512 dims of K)
// Role in the reference: the split-KV stage-1 kernels (mixed-mla/submission.py:122-250,
// mixed-mla/triton_fp8_decode.py:44-156, mixed-mla/versions/hip_mxfp4_v5/submission.py:214-656).
#include <mma.h>

#include "mla_common.cuh"

namespace b200mla {

using namespace nvcuda;

namespace generic {

constexpr int TILE = 64;
constexpr int ROWS = 16;
constexpr int THREADS = 256;
constexpr int KP = QK_DIM + 8;        // bf16 pitch of the K tile and of Q (584)
constexpr int PP = TILE + 8;          // bf16 pitch of P
constexpr float RECENTER = 8.0f;      // log2 units

struct Smem {
    __nv_bfloat16 kt[TILE * KP];
    __nv_bfloat16 qs[ROWS * KP];
    float s_part[2 * ROWS * TILE];    // two K-halves of S; reused as per-warp 16x16 scratch
    __nv_bfloat16 ps[ROWS * PP];
    float m[ROWS], l[ROWS], alpha[ROWS];
    unsigned int q_amax;               // block_q_scale's word
};

template <int KVFMT>
struct Chunks;                         // 16-byte chunks per token and loads per thread
template <> struct Chunks<KV_E4M3>   { static constexpr int per_tok = 36; };
template <> struct Chunks<KV_MXFP4>  { static constexpr int per_tok = 18; };
template <> struct Chunks<KV_HYBRID> { static constexpr int per_tok = 20; };   // 16 latent + 4 rope

template <int KVFMT>
struct TileRegs {
    static constexpr int N = (TILE * Chunks<KVFMT>::per_tok + THREADS - 1) / THREADS;
    uint4 v[N];
    uint8_t sc[N];
};

// Issue the global loads of one tile into registers (no dependence on shared memory).
template <int KVFMT>
__device__ __forceinline__ void load_tile(const MlaParams& p, int b, int seq_base, int page_base,
                                          int pos0, int pos_end, TileRegs<KVFMT>& r) {
    constexpr int CPT = Chunks<KVFMT>::per_tok;
#pragma unroll
    for (int i = 0; i < TileRegs<KVFMT>::N; ++i) {
        int cid = threadIdx.x + i * THREADS;
        int tok = cid / CPT, c = cid - tok * CPT;
        int pos = pos0 + tok;
        r.v[i] = make_uint4(0, 0, 0, 0);
        r.sc[i] = 127;
        if (tok < TILE && pos < pos_end) {
            const long long slot = clamp_slot(p, (int)slot_of(p, b, seq_base, page_base, pos));
            if (KVFMT == KV_E4M3) {
                r.v[i] = __ldg(reinterpret_cast<const uint4*>(p.kv_codes + slot * p.kv_codes_stride) + c);
            } else if (KVFMT == KV_MXFP4) {
                r.v[i] = __ldg(reinterpret_cast<const uint4*>(p.kv_codes + slot * p.kv_codes_stride) + c);
                r.sc[i] = __ldg(p.kv_bs + slot * p.kv_bs_stride + c);
            } else {
                if (c < 16) {
                    r.v[i] = __ldg(reinterpret_cast<const uint4*>(p.kv_codes + slot * p.kv_codes_stride) + c);
                    r.sc[i] = __ldg(p.kv_bs + slot * p.kv_bs_stride + c);
                } else {
                    r.v[i] = __ldg(reinterpret_cast<const uint4*>(p.kv_rope + slot * p.kv_rope_stride) + (c - 16));
                }
            }
        }
    }
}

__device__ __forceinline__ void store_fp8x16(__nv_bfloat16* dst, const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    __align__(16) __nv_bfloat162 o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float2 a = __half22float2(e4m3x2_to_half2((uint16_t)(w[j] & 0xffffu)));
        float2 c = __half22float2(e4m3x2_to_half2((uint16_t)(w[j] >> 16)));
        o[2 * j] = __floats2bfloat162_rn(a.x, a.y);
        o[2 * j + 1] = __floats2bfloat162_rn(c.x, c.y);
    }
    reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<uint4*>(o)[0];
    reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<uint4*>(o)[1];
}

__device__ __forceinline__ void store_fp4x32(__nv_bfloat16* dst, const uint4& v, uint8_t sc) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    const float s = e8m0_to_float(sc);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __align__(16) __nv_bfloat162 o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            uint32_t byte = (w[j] >> (8 * k)) & 0xffu;
            o[k] = __floats2bfloat162_rn(e2m1_to_float(byte & 0xfu) * s, e2m1_to_float(byte >> 4) * s);
        }
        reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<uint4*>(o)[0];
    }
}

// Dequantise the registers of one tile into the bf16 tile (exact for all three formats as long as
// the E8M0 exponent keeps e2m1 * 2^e inside bf16's normal range).
template <int KVFMT>
__device__ __forceinline__ void store_tile(Smem& s, const TileRegs<KVFMT>& r) {
    constexpr int CPT = Chunks<KVFMT>::per_tok;
#pragma unroll
    for (int i = 0; i < TileRegs<KVFMT>::N; ++i) {
        int cid = threadIdx.x + i * THREADS;
        int tok = cid / CPT, c = cid - tok * CPT;
        if (tok >= TILE) continue;
        __nv_bfloat16* row = s.kt + tok * KP;
        if (KVFMT == KV_E4M3) {
            store_fp8x16(row + c * 16, r.v[i]);
        } else if (KVFMT == KV_MXFP4) {
            store_fp4x32(row + c * 32, r.v[i], r.sc[i]);
        } else {
            if (c < 16) store_fp4x32(row + c * 32, r.v[i], r.sc[i]);
            else store_fp8x16(row + V_DIM + (c - 16) * 16, r.v[i]);
        }
    }
}

template <int KVFMT>
__global__ void __launch_bounds__(THREADS, 2) mla_decode_generic_kernel(const MlaParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>(smem_raw);
    int* prefix = reinterpret_cast<int*>(smem_raw + sizeof(Smem));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int w = blockIdx.x, G = p.num_ctas;
    const int row0 = blockIdx.y * ROWS;                 // first query row (of p.rows) of this CTA

    build_tile_prefix(p.kv_indptr, p.batch, TILE, prefix);
    const int TT = prefix[p.batch];
    if (w == 0 && blockIdx.y == 0)
        for (int i = tid; i <= p.batch; i += THREADS) p.tile_prefix[i] = prefix[i];
    if (TT == 0) return;
    const int t_begin = span_begin(prefix, p.batch, w, G), t_end = span_begin(prefix, p.batch, w + 1, G);
    if (t_begin >= t_end) return;
    if (blockIdx.y == 0) check_span_pages(p, prefix, t_begin, t_end, TILE, tid, THREADS);

    // scalar scales: scores get q_scale * kv_scale(e4m3 cache) * sm_scale * log2e, outputs kv_scale
    const float q_sc = p.q_format == Q_E4M3 ? block_q_scale(block_q_amax_begin(p.q_amax_parts, p.q_cast), p.q_scale, p.q_cast, &s.q_amax) : 1.0f;
    const float kv_sc = (KVFMT == KV_E4M3 || KVFMT == KV_HYBRID) ? __ldg(p.kv_scale) : 1.0f;
    const float score_scale = p.sm_scale * LOG2E * q_sc * (KVFMT == KV_E4M3 ? kv_sc : 1.0f);
    const float out_scale = KVFMT == KV_E4M3 ? kv_sc : 1.0f;
    const float rope_q_scale = KVFMT == KV_HYBRID ? kv_sc : 1.0f;   // rope scale folded into Q

    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[4];
    TileRegs<KVFMT> regs;

    int b = seq_of_tile(prefix, p.batch, t_begin);
    int t = t_begin;
    while (t < t_end) {
        while (prefix[b + 1] <= t) ++b;
        const int seq_t0 = prefix[b], seq_t1 = prefix[b + 1];
        const int my_t1 = min(t_end, seq_t1);
        const int seq_base = p.kv_indptr[b];
        const int seq_len = max(p.kv_indptr[b + 1] - seq_base, 0);
        const int page_base = p.kv_page_indptr ? p.kv_page_indptr[b] : seq_base;
        const int pos_off = p.kv_pos_offset ? p.kv_pos_offset[b] : 0;
        const int tot_len = p.kv_total_len ? p.kv_total_len[b] : seq_len;

        load_tile<KVFMT>(p, b, seq_base, page_base, (t - seq_t0) * TILE, seq_len, regs);

        // Q rows of this sequence -> bf16 smem
        for (int i = tid; i < ROWS * (QK_DIM / 8); i += THREADS) {
            int r = i / (QK_DIM / 8), c8 = (i - r * (QK_DIM / 8)) * 8;
            int rg = row0 + r;
            int j = rg / p.heads, h = rg - j * p.heads;
            long long off = (long long)(b * p.q_len + j) * p.q_row_stride + (long long)h * p.q_head_stride + c8;
            __align__(16) __nv_bfloat16 o[8];
            const float f = (c8 >= V_DIM) ? rope_q_scale : 1.0f;
            if (p.q_cast) {                      // bf16 in memory, used as the e4m3 value the reference's quantiser gives it
                uint4 raw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.q) + off));
                const uint2 codes = q_cast_e4m3x8(raw, q_sc);
                const uint8_t* in = reinterpret_cast<const uint8_t*>(&codes);
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16_rn(e4m3_to_float(in[k]) * f);
            } else if (p.q_format == Q_BF16) {
                uint4 raw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.q) + off));
                const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = f == 1.0f ? in[k] : __float2bfloat16_rn(__bfloat162float(in[k]) * f);
            } else {
                uint2 raw = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.q) + off));
                const uint8_t* in = reinterpret_cast<const uint8_t*>(&raw);
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16_rn(e4m3_to_float(in[k]) * f);
            }
            *reinterpret_cast<uint4*>(s.qs + r * KP + c8) = *reinterpret_cast<uint4*>(o);
        }
        if (tid < ROWS) { s.m[tid] = -INFINITY; s.l[tid] = 0.0f; }
#pragma unroll
        for (int n = 0; n < 4; ++n) wmma::fill_fragment(acc[n], 0.0f);

        for (int tt = t; tt < my_t1; ++tt) {
            const int pos0 = (tt - seq_t0) * TILE;
            __syncthreads();                            // previous tile fully consumed
            store_tile<KVFMT>(s, regs);
            __syncthreads();
            if (tt + 1 < my_t1) load_tile<KVFMT>(p, b, seq_base, page_base, pos0 + TILE, seq_len, regs);

            // ---- S = Q K^T: warp -> (token block nt, K half kh)
            {
                const int nt = warp & 3, kh = warp >> 2;
                wmma::fragment<wmma::accumulator, 16, 16, 16, float> sacc;
                wmma::fill_fragment(sacc, 0.0f);
#pragma unroll 6
                for (int ks = 0; ks < 18; ++ks) {
                    const int k0 = kh * 288 + ks * 16;
                    wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> bk;
                    wmma::load_matrix_sync(a, s.qs + k0, KP);
                    wmma::load_matrix_sync(bk, s.kt + nt * 16 * KP + k0, KP);
                    wmma::mma_sync(sacc, a, bk, sacc);
                }
                wmma::store_matrix_sync(s.s_part + kh * ROWS * TILE + nt * 16, sacc, TILE, wmma::mem_row_major);
            }
            __syncthreads();

            // ---- online softmax: 16 threads per row, 4 tokens each
            int rescale;
            {
                const int r = tid >> 4, sub = tid & 15;
                const int rg = row0 + r, j = rg / p.heads;
                const int limit = p.causal ? (tot_len - p.q_len + j) : 0x7fffffff;   // last visible position
                float sv[4];
                float mx = -INFINITY;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int tok = sub * 4 + k, pos = pos0 + tok;
                    float v = (s.s_part[r * TILE + tok] + s.s_part[ROWS * TILE + r * TILE + tok]) * score_scale;
                    const bool ok = pos < seq_len && (pos_off + pos) <= limit;
                    sv[k] = ok ? v : -INFINITY;
                    mx = fmaxf(mx, sv[k]);
                }
#pragma unroll
                for (int o = 8; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float m_old = s.m[r];
                float m_new = m_old, alpha = 1.0f;
                if (mx > m_old + RECENTER || (m_old == -INFINITY && mx > -INFINITY)) {
                    m_new = mx;
                    alpha = m_old == -INFINITY ? 0.0f : exp2f(m_old - m_new);
                }
                float sum = 0.0f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float pv = sv[k] == -INFINITY ? 0.0f : exp2f(sv[k] - m_new);
                    sum += pv;
                    s.ps[r * PP + sub * 4 + k] = __float2bfloat16_rn(pv);
                }
#pragma unroll
                for (int o = 8; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                rescale = alpha != 1.0f;
                __syncwarp();
                if (sub == 0) { s.m[r] = m_new; s.l[r] = s.l[r] * alpha + sum; s.alpha[r] = alpha; }
            }
            rescale = __syncthreads_or(rescale);

            // ---- rare: rescale the accumulator rows through a 16x16 scratch per warp
            if (rescale) {
                float* scr = s.s_part + warp * 256;
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    wmma::store_matrix_sync(scr, acc[n], 16, wmma::mem_row_major);
                    __syncwarp();
#pragma unroll
                    for (int e = lane; e < 256; e += 32) scr[e] *= s.alpha[e >> 4];
                    __syncwarp();
                    wmma::load_matrix_sync(acc[n], scr, 16, wmma::mem_row_major);
                    __syncwarp();
                }
            }

            // ---- O += P V: warp -> 64 output dims
#pragma unroll
            for (int ks = 0; ks < TILE / 16; ++ks) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
                wmma::load_matrix_sync(a, s.ps + ks * 16, PP);
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::row_major> bv;
                    wmma::load_matrix_sync(bv, s.kt + ks * 16 * KP + warp * 64 + n * 16, KP);
                    wmma::mma_sync(acc[n], a, bv, acc[n]);
                }
            }
        }

        // ---- finalise this (CTA, sequence) pair
        __syncthreads();
        const bool whole = (t == seq_t0) && (my_t1 == seq_t1);
        const int slot = w + b;
        {
            float* scr = s.s_part + warp * 256;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                wmma::store_matrix_sync(scr, acc[n], 16, wmma::mem_row_major);
                __syncwarp();
                for (int e = lane; e < 256; e += 32) {
                    const int r = e >> 4, c = e & 15;
                    const float l = s.l[r];
                    const float v = l > 0.0f ? scr[e] * (out_scale / l) : 0.0f;
                    const int d = warp * 64 + n * 16 + c;
                    const long long orow = (long long)b * p.rows + row0 + r;
                    if (whole) {
                        if (p.out) p.out[orow * V_DIM + d] = __float2bfloat16_rn(v);
                        if (p.out_o_f32) p.out_o_f32[orow * V_DIM + d] = v;
                    } else {
                        p.part_o[((long long)slot * p.rows + row0 + r) * V_DIM + d] = v;
                    }
                }
                __syncwarp();
            }
        }
        if (tid < ROWS) {
            const float l = s.l[tid];
            const float lse = l > 0.0f ? (s.m[tid] + log2f(l)) * LN2 : -INFINITY;
            if (whole) {
                if (p.out_lse) p.out_lse[(long long)b * p.rows + row0 + tid] = lse;
            } else {
                p.part_lse[(long long)slot * p.rows + row0 + tid] = lse;
            }
        }
        t = my_t1;
        __syncthreads();
    }
}

}  // namespace generic

size_t generic_smem_bytes(int batch) { return sizeof(generic::Smem) + (size_t)(batch + 1) * sizeof(int); }

cudaError_t launch_generic(const MlaParams& p, cudaStream_t stream) {
    const size_t smem = generic_smem_bytes(p.batch);
    dim3 grid(p.num_ctas, p.rows / generic::ROWS);
    cudaError_t e = cudaSuccess;
#define B200MLA_LAUNCH(FMT)                                                                          \
    e = cudaFuncSetAttribute(generic::mla_decode_generic_kernel<FMT>,                                 \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                 \
    if (e != cudaSuccess) return e;                                                                   \
    generic::mla_decode_generic_kernel<FMT><<<grid, generic::THREADS, smem, stream>>>(p);
    if (p.kv_format == KV_E4M3) { B200MLA_LAUNCH(KV_E4M3) }
    else if (p.kv_format == KV_MXFP4) { B200MLA_LAUNCH(KV_MXFP4) }
    else { B200MLA_LAUNCH(KV_HYBRID) }
#undef B200MLA_LAUNCH
    return cudaGetLastError();
}

}  // namespace b200mla
