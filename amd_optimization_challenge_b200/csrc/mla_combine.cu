// Log-sum-exp combine kernels.
//
//  * combine_spans_kernel merges the partials that stage-1 CTAs wrote for sequences whose tiles
//    were spread over several KV spans (slot = cta + sequence, see mla_common.cuh), writes zeros
//    for empty sequences and leaves alone the sequences a single CTA finished by itself.
//  * combine_parts_kernel merges `parts` dense partial results [parts, rows, 512] + [parts, rows],
//    the form an all-gather of per-GPU shards produces.
//
// Math (natural-log LSE, normalised partial O):  M = max_i LSE_i,  w_i = exp(LSE_i - M),
// O = sum_i w_i O_i / sum_i w_i,  LSE = M + log(sum_i w_i); an empty part has LSE = -inf and weight 0.
// Role in the reference: _mla_mxfp4_reduce (mixed-mla/submission.py:257-294), aiter.mla_reduce_v1,
// stage 2 of competitor_submissions/dgavriloff_v114_hybrid_mxfp4k_fp8v.py:131-160.
#include "mla_common.cuh"

namespace b200mla {

namespace {

__device__ __forceinline__ void store_bf16x4(__nv_bfloat16* dst, float4 v) {
    __align__(8) __nv_bfloat162 o[2] = {__floats2bfloat162_rn(v.x, v.y), __floats2bfloat162_rn(v.z, v.w)};
    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<uint2*>(o);
}

__global__ void __launch_bounds__(128) combine_spans_kernel(const MlaParams p) {
    const int b = blockIdx.x, r = blockIdx.y, G = p.num_ctas;
    const int TT = p.tile_prefix[p.batch];
    const int t0 = p.tile_prefix[b], t1 = p.tile_prefix[b + 1];
    const long long orow = (long long)b * p.rows + r;
    const int d = threadIdx.x * 4;
    if (t1 <= t0) {                                       // empty key set: O = 0, LSE = -inf
        if (p.out) store_bf16x4(p.out + orow * V_DIM + d, make_float4(0.f, 0.f, 0.f, 0.f));
        if (p.out_o_f32) *reinterpret_cast<float4*>(p.out_o_f32 + orow * V_DIM + d) = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.out_lse && threadIdx.x == 0) p.out_lse[orow] = -INFINITY;
        return;
    }
    const int TU = total_units(TT, p.batch);              // schedule units: tiles plus the set-up units of every sequence
    const int w0 = cta_of_tile(t0, b, TU, G), w1 = cta_of_tile(t1 - 1, b, TU, G);
    if (w0 == w1) return;                                 // finished by a single stage-1 CTA
    // streaming merge, four partials per step so that their loads are in flight together;
    // CTAs without any unit (G > total units) wrote nothing and are skipped
    float M = -INFINITY, den = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int wb = w0; wb <= w1; wb += 4) {
        float l[4];
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int w = wb + u;
            // w0 and w1 hold the sequence's first and last tile; a CTA in between holds tiles of this sequence
            // only, unless it holds no unit at all
            const bool ok = w <= w1 && (w == w0 || w == w1 || cta_has_units(w, TU, G));
            const long long slot = (long long)(w + b) * p.rows + r;
            l[u] = ok ? p.part_lse[slot] : -INFINITY;
            v[u] = ok ? *reinterpret_cast<const float4*>(p.part_o + slot * V_DIM + d) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const float m_new = fmaxf(fmaxf(fmaxf(l[0], l[1]), fmaxf(l[2], l[3])), M);
        if (m_new > -INFINITY) {
            const float f = M > -INFINITY ? expf(M - m_new) : 0.f;
            acc.x *= f; acc.y *= f; acc.z *= f; acc.w *= f; den *= f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float wt = l[u] > -INFINITY ? expf(l[u] - m_new) : 0.f;
                acc.x += wt * v[u].x; acc.y += wt * v[u].y; acc.z += wt * v[u].z; acc.w += wt * v[u].w;
                den += wt;
            }
            M = m_new;
        }
    }
    if (den > 0.f) {
        const float inv = 1.0f / den;
        acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    }
    if (p.out) store_bf16x4(p.out + orow * V_DIM + d, acc);
    if (p.out_o_f32) *reinterpret_cast<float4*>(p.out_o_f32 + orow * V_DIM + d) = acc;
    if (p.out_lse && threadIdx.x == 0) p.out_lse[orow] = den > 0.f ? M + logf(den) : -INFINITY;
}

__global__ void __launch_bounds__(128) combine_parts_kernel(const float* __restrict__ o_parts,
                                                            const float* __restrict__ lse_parts, int parts,
                                                            long long rows, long long o_stride, long long lse_stride,
                                                            __nv_bfloat16* out, float* out_lse) {
    const long long r = blockIdx.x;
    const int d = threadIdx.x * 4;
    float M = -INFINITY;
    for (int i = 0; i < parts; ++i) M = fmaxf(M, lse_parts[i * lse_stride + r]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
    if (M > -INFINITY) {
        for (int i = 0; i < parts; ++i) {
            const float wt = expf(lse_parts[i * lse_stride + r] - M);
            const float4 v = *reinterpret_cast<const float4*>(o_parts + i * o_stride + r * V_DIM + d);
            acc.x += wt * v.x; acc.y += wt * v.y; acc.z += wt * v.z; acc.w += wt * v.w;
            den += wt;
        }
        const float inv = 1.0f / den;
        acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    }
    store_bf16x4(out + r * V_DIM + d, acc);
    if (out_lse && threadIdx.x == 0) out_lse[r] = den > 0.f ? M + logf(den) : -INFINITY;
}

}  // namespace

cudaError_t launch_combine_spans(const MlaParams& p, cudaStream_t stream) {
    dim3 grid(p.batch, p.rows);
    combine_spans_kernel<<<grid, 128, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_combine_parts(const float* o_parts, const float* lse_parts, int parts, long long rows,
                                 long long o_stride, long long lse_stride, __nv_bfloat16* out, float* out_lse,
                                 cudaStream_t stream) {
    combine_parts_kernel<<<(unsigned)rows, 128, 0, stream>>>(o_parts, lse_parts, parts, rows, o_stride, lse_stride, out, out_lse);
    return cudaGetLastError();
}

}  // namespace b200mla
