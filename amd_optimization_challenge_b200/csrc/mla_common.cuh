// Shared device-side definitions for the MLA decode kernels: kernel parameter block, the
// KV-span schedule that every stage-1 CTA and the combine kernel derive from kv_indptr, and the
// byte-format decoders (e4m3fn, e2m1 + E8M0).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200mla {

constexpr int QK_DIM = 576;
constexpr int V_DIM = 512;
constexpr int ROPE_DIM = 64;
constexpr int MAX_BATCH = 8192;        // the per-CTA tile-prefix table lives in shared memory

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

enum { Q_BF16 = 0, Q_E4M3 = 1 };
constexpr int Q_AMAX_PARTS = 256;      // partial maxima handed over by the amax kernel when Q is cast on load
enum { KV_E4M3 = 0, KV_MXFP4 = 1, KV_HYBRID = 2 };
// Bits of the sticky status word at the head of the workspace (B200_MLA_STATUS_* in b200_mla.h).
enum { ST_OK = 0, ST_TIMEOUT = 1, ST_BAD_PAGE = 2 };

struct MlaParams {
    int batch, heads, q_len, rows;      // rows = q_len * heads (query rows per sequence)
    int q_format, kv_format, causal, page_size;
    float sm_scale;
    int num_ctas;                       // G: stage-1 CTAs along x (KV spans)
    int tile_tokens;                    // tokens per schedule tile (kernel specific)
    int rows_per_cta;                   // query rows handled by one CTA (grid.y = rows / rows_per_cta)

    const void* q; long long q_row_stride, q_head_stride; const float* q_scale;
    const uint8_t* kv_codes; long long kv_codes_stride;
    const uint8_t* kv_bs; long long kv_bs_stride;
    const uint8_t* kv_rope; long long kv_rope_stride;
    const float* kv_scale; long long num_slots;
    unsigned int last_slot;             // min(num_slots, 2^31) - 1: the row an out-of-range page id is redirected to
    long long total_kv_hint;            // > 0: the host's bound on kv_indptr[batch]; kv_indices holds at least that many tokens' ids
    const int* kv_indptr; const int* kv_indices; const int* kv_page_indptr;
    const int* kv_pos_offset; const int* kv_total_len;

    __nv_bfloat16* out; float* out_o_f32; float* out_lse;
    float* part_o;                      // [G + batch - 1][rows][512] normalised partial O
    float* part_lse;                    // [G + batch - 1][rows]      natural-log LSE
    int* tile_prefix;                   // [batch + 1] exclusive prefix of tiles per sequence
    uint8_t* q_split;                   // bf16 Q as two e4m3 planes [2][batch * rows][576] (tcgen05 kernels)
    float* q_split_scale;               // [batch][rows / rows_per_cta] factor that undoes the planes' scaling
    int* status;                        // sticky status word (bits ST_*), first word of the workspace
    int q_cast;                         // q is bf16 and is quantised to e4m3 (per-tensor, reference rule) as it is loaded;
    const unsigned int* q_amax_parts;   //   its scale comes from these Q_AMAX_PARTS partial maxima (bf16 bit patterns)
};

// ---------------------------------------------------------------------------------------------
// Schedule.  Sequence b owns tiles [P[b], P[b+1]) with ceil(len_b / tile_tokens) tiles.  The work is
// measured in units: one per tile plus SEQ_UNITS per sequence (its Q load, first-tile re-centering
// and epilogues cost a CTA about as much as two tiles; measured on config 1, the CTAs that hold a
// sequence boundary ran 10 % longer than the others under a plain tile split), so sequence b owns
// units [P[b] + K*b, P[b+1] + K*(b+1)), K = SEQ_UNITS, the first K being set-up units.  CTA w of G
// owns the units [w*TU/G, (w+1)*TU/G), TU = P[batch] + K*batch, i.e. the tiles those units stand
// for.  A (CTA, sequence) pair that does not cover the whole sequence writes a partial into slot
// w + b, which is unique because both coordinates are monotone along the chain of pairs.
// ---------------------------------------------------------------------------------------------
#ifndef B200MLA_SEQ_UNITS
#define B200MLA_SEQ_UNITS 2
#endif
constexpr int SEQ_UNITS = B200MLA_SEQ_UNITS;

__device__ __forceinline__ int total_units(int total_tiles, int batch) { return total_tiles + SEQ_UNITS * batch; }
// Sequence that owns unit u: the first b with P[b+1] + K*(b+1) > u.
__device__ __forceinline__ int seq_of_unit(const int* prefix, int batch, int u) {
    int lo = 0, hi = batch - 1;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid + 1] + SEQ_UNITS * (mid + 1) > u) hi = mid; else lo = mid + 1;
    }
    return lo;
}
// First tile of CTA w's span (w = G gives the total number of tiles).
// The 64-bit division is only taken where the product needs it (this runs in every CTA right after launch).
__device__ __forceinline__ int span_begin(const int* prefix, int batch, int w, int G) {
    if (w >= G) return prefix[batch];
    const int tu = total_units(prefix[batch], batch);
    const int u = ((unsigned long long)(unsigned)w * (unsigned)tu >> 32) == 0 ? (int)(((unsigned)w * (unsigned)tu) / (unsigned)G)
                                                                            : (int)(((long long)w * tu) / G);
    const int b = seq_of_unit(prefix, batch, u);
    return max(prefix[b], u - SEQ_UNITS * (b + 1));
}
// The same, also returning a sequence b_out <= the sequence of the returned tile (Walker::init_at starts from it,
// which saves the roles a binary search of their own at their start).
__device__ __forceinline__ int span_begin_seq(const int* prefix, int batch, int w, int G, int& b_out) {
    b_out = 0;
    if (w >= G) return prefix[batch];
    const int tu = total_units(prefix[batch], batch);
    const int u = ((unsigned long long)(unsigned)w * (unsigned)tu >> 32) == 0 ? (int)(((unsigned)w * (unsigned)tu) / (unsigned)G)
                                                                            : (int)(((long long)w * tu) / G);
    const int b = seq_of_unit(prefix, batch, u);
    b_out = b;
    return max(prefix[b], u - SEQ_UNITS * (b + 1));
}
// CTA whose span contains tile t of sequence b (unit t + K*(b+1)).
__device__ __forceinline__ int cta_of_tile(int t, int b, int units, int G) {
    return (int)((((long long)(t + SEQ_UNITS * (b + 1) + 1) * G + units - 1) / units) - 1);
}
// Does CTA w own any unit at all (G may exceed the number of units)?
__device__ __forceinline__ bool cta_has_units(int w, int units, int G) {
    return ((long long)w * units) / G < ((long long)(w + 1) * units) / G;
}

// Fills prefix[0..batch] (shared memory) with the exclusive prefix of tiles per sequence.
// All threads of the block must call it; ends with a __syncthreads().
__device__ inline void build_tile_prefix(const int* __restrict__ kv_indptr, int batch, int tile_tokens,
                                         int* prefix) {
    for (int b = threadIdx.x; b < batch; b += blockDim.x) {
        int len = kv_indptr[b + 1] - kv_indptr[b];
        prefix[b + 1] = len > 0 ? (len + tile_tokens - 1) / tile_tokens : 0;
    }
    if (threadIdx.x == 0) prefix[0] = 0;
    __syncthreads();
    if (threadIdx.x < 32) {
        int carry = 0;
        for (int base = 1; base <= batch; base += 32) {
            int i = base + threadIdx.x;
            int v = i <= batch ? prefix[i] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int n = __shfl_up_sync(0xffffffffu, v, o);
                if ((int)threadIdx.x >= o) v += n;
            }
            v += carry;
            if (i <= batch) prefix[i] = v;
            carry = __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
}

// First sequence b with prefix[b+1] > t (sequence containing global tile t).
__device__ __forceinline__ int seq_of_tile(const int* prefix, int batch, int t) {
    int lo = 0, hi = batch - 1;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (prefix[mid + 1] > t) hi = mid; else lo = mid + 1;
    }
    return lo;
}

// Cache slot of the token at position `pos` of sequence b, as the page table gives it (unchecked).
__device__ __forceinline__ long long slot_of(const MlaParams& p, int b, int seq_base, int page_base, int pos) {
    if (p.kv_indices == nullptr) return (long long)seq_base + pos;
    if (p.page_size == 1) return (long long)p.kv_indices[page_base + pos];
    int pg = pos / p.page_size;
    return (long long)p.kv_indices[page_base + pg] * p.page_size + (pos - pg * p.page_size);
}
// Row of the cache planes that is actually read for slot `s`: s itself inside [0, num_slots), else a row inside
// (negative values, the "no row" marker -1 included, map to the last row).  Nothing outside the planes is ever read;
// a key whose id needed the clamp reads as some other row, which check_span_pages reports as ST_BAD_PAGE.  The
// clamp is applied where a slot is turned into an address, not where it is loaded: the kernels load page ids one or
// two steps ahead of their use, and touching the value early would wait for that load (measured: 10-25 % of a call).
__device__ __forceinline__ unsigned int clamp_slot(const MlaParams& p, int s) { return min((unsigned int)s, p.last_slot); }

// Page ids of the tiles [t_begin, t_end) a stage-1 CTA owns: sets ST_BAD_PAGE if one of them names a page outside
// the cache planes (or, without a page table, if a token range reaches beyond them).  Called by `nthreads` threads
// (tid = 0 .. nthreads - 1) that have nothing else to do at the time; `tile` = tokens per tile.  Inlined: a call would
// make every thread of the kernel reserve a stack frame in local memory (measured: 19 MB of extra DRAM traffic per launch).
__device__ __forceinline__ void check_span_pages(const MlaParams& p, const int* prefix, int t_begin, int t_end, int tile,
                                              int tid, int nthreads) {
    bool bad = false;
    int b = seq_of_tile(prefix, p.batch, t_begin);
    for (int t = t_begin; t < t_end;) {
        while (prefix[b + 1] <= t) ++b;
        const int t1 = min(t_end, prefix[b + 1]);
        const int seq_base = p.kv_indptr[b], len = max(p.kv_indptr[b + 1] - seq_base, 0);
        const int pos0 = (t - prefix[b]) * tile, pos1 = min((t1 - prefix[b]) * tile, len);
        if (p.kv_indices != nullptr) {
            const int page_base = p.kv_page_indptr ? p.kv_page_indptr[b] : seq_base;
            const int e0 = pos0 / p.page_size, e1 = (pos1 + p.page_size - 1) / p.page_size;
            for (int e = e0 + tid; e < e1; e += nthreads) {
                const long long id = p.kv_indices[page_base + e];
                bad |= id < 0 || id * p.page_size >= p.num_slots;
            }
        } else if (tid == 0) {
            bad |= seq_base < 0 || (long long)seq_base + pos1 > p.num_slots;
        }
        t = t1;
    }
    if (bad) atomicOr(p.status, (int)ST_BAD_PAGE);
}

// Position of one role inside the CTA's span of global tiles [t_begin, t_end): which sequence the
// current tile belongs to, and that sequence's geometry.  Every role walks the span with its own copy.
struct Walker {
    int b, seq_t0, seq_t1;                  // sequence and its global tile range
    int seq_base, seq_len, page_base, pos_off, tot_len;
    int pair;                               // (CTA, sequence) pairs started so far, minus one
    __device__ __forceinline__ void init(const int* prefix, int batch, int t_begin) {
        b = seq_of_tile(prefix, batch, t_begin) - 1;
        seq_t0 = 0; seq_t1 = -1;
        seq_base = seq_len = page_base = pos_off = tot_len = 0;
        pair = -1;
    }
    // Start from a known sequence b0 <= the sequence of the first tile that will be sought.
    __device__ __forceinline__ void init_at(int b0) {
        b = b0 - 1;
        seq_t0 = 0; seq_t1 = -1;
        seq_base = seq_len = page_base = pos_off = tot_len = 0;
        pair = -1;
    }
    // Make the walker describe the sequence that owns global tile t (t only grows between calls).
    // Returns true when t is the first tile of a new (CTA, sequence) pair.
    __device__ __forceinline__ bool seek(const MlaParams& p, const int* prefix, int t) {
        if (t < seq_t1) return false;
        do { ++b; } while (prefix[b + 1] <= t);
        seq_t0 = prefix[b];
        seq_t1 = prefix[b + 1];
        seq_base = p.kv_indptr[b];
        seq_len = max(p.kv_indptr[b + 1] - seq_base, 0);
        page_base = p.kv_page_indptr ? p.kv_page_indptr[b] : seq_base;
        pos_off = p.kv_pos_offset ? p.kv_pos_offset[b] : 0;
        tot_len = p.kv_total_len ? p.kv_total_len[b] : seq_len;
        ++pair;
        return true;
    }
};

// ---------------------------------------------------------------------------------------------
// Per-tensor e4m3 quantisation of Q, arithmetic order of the reference's quantize_fp8
// (competitor_submissions/mi355x_reference/reference.py:65-80): every intermediate is a bf16 value.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float q_scale_from_amax_bits(unsigned int bits) {
    float amax = __bfloat162float(__ushort_as_bfloat16((unsigned short)bits));
    amax = __bfloat162float(__float2bfloat16_rn(fmaxf(amax, 1e-12f)));
    return __bfloat162float(__float2bfloat16_rn(amax / 448.0f));
}
// x / scale rounded to bf16, as a float: the reference divides two bf16 tensors, i.e. an IEEE fp32 division whose
// result is rounded to bf16.  Evaluated without a division: t = x * r with r = RN(1 / scale), one exact residual
// and one correction (Markstein) give the correctly rounded fp32 quotient; checked exhaustively on the CPU against
// x / scale for every finite bf16 x and every positive normal bf16 scale (identical after the bf16 rounding and the
// clamp to +-448).  The sign is taken from x, so that -0 stays -0.
__device__ __forceinline__ float q_quotient_bf16(float x, float scale, float rscale) {
    const float t = x * rscale;
    float y = fmaf(fmaf(-t, scale, x), rscale, t);
    if (!(fabsf(t) <= 3.0e38f)) y = t;                                        // infinite / NaN input
    y = copysignf(fabsf(y), x);
    return __bfloat162float(__float2bfloat16_rn(y));
}
__device__ __forceinline__ uint8_t q_cast_e4m3(__nv_bfloat16 x, float scale) {
    const float y = fminf(fmaxf(q_quotient_bf16(__bfloat162float(x), scale, __frcp_rn(scale)), -448.0f), 448.0f);
    return (uint8_t)__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
}
// eight bf16 values (one 16-byte vector) -> eight e4m3 bytes
__device__ __forceinline__ uint2 q_cast_e4m3x8(const uint4& v, float scale) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};             // by value: the vector stays in registers
    const float r = __frcp_rn(scale);
    uint32_t o[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float y[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t word = w[2 * h + (k >> 1)];
            const float x = __uint_as_float((k & 1) ? (word & 0xffff0000u) : (word << 16));   // bf16 -> fp32
            y[k] = q_quotient_bf16(x, scale, r);
        }
        // the conversion saturates to +-448, which is the reference's clamp
        uint16_t lo16, hi16;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo16) : "f"(y[0]), "f"(y[1]));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi16) : "f"(y[2]), "f"(y[3]));
        o[h] = (uint32_t)lo16 | ((uint32_t)hi16 << 16);
    }
    return make_uint2(o[0], o[1]);
}
// Scale of the e4m3 Q codes, the same value in every thread of the block.  All threads call it (it
// synchronises the block when the scale has to be reduced from the partial maxima); `word` is one
// 32-bit word of shared memory.
// block_q_amax_begin issues this thread's loads of the partial maxima (call it early, the result is
// only needed by block_q_scale); without a cast it returns 0 and touches nothing.
__device__ __forceinline__ unsigned int block_q_amax_begin(const unsigned int* amax_parts, int q_cast) {
    unsigned int m = 0;
    if (q_cast)
        for (int i = threadIdx.x; i < Q_AMAX_PARTS; i += blockDim.x) m = max(m, __ldg(amax_parts + i));
    return m;
}
__device__ inline float block_q_scale(unsigned int m, const float* q_scale, int q_cast, unsigned int* word) {
    if (!q_cast) return q_scale ? __ldg(q_scale) : 1.0f;
    if (threadIdx.x == 0) *word = 0u;
    __syncthreads();
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0 && m) atomicMax(word, m);
    __syncthreads();
    return q_scale_from_amax_bits(*word);
}

// ---------------------------------------------------------------------------------------------
// byte formats
// ---------------------------------------------------------------------------------------------

// two e4m3fn bytes (low 16 bits) -> two halves (exact)
__device__ __forceinline__ __half2 e4m3x2_to_half2(uint16_t v) {
    __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
    return *reinterpret_cast<__half2*>(&r);
}

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
    __half_raw r = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&r));
}

// E8M0 byte -> float 2^(b-127).  Byte 0 gives 2^-127 (a denormal), 255 is NaN in the format.
__device__ __forceinline__ float e8m0_to_float(uint8_t b) {
    if (b == 255) return __int_as_float(0x7fc00000);
    return b == 0 ? __int_as_float(0x00400000) : __int_as_float((int)b << 23);
}

// e2m1 code (4 bits, bit3 = sign) -> float
__device__ __forceinline__ float e2m1_to_float(uint32_t c) {
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
    uint32_t mag = c & 7u;
    float v = mag < 2u ? 0.5f * (float)mag
                       : __int_as_float((int)(((mag >> 1) + 126u) << 23) | (int)((mag & 1u) << 22));
    return (c & 8u) ? -v : v;
}

}  // namespace b200mla
