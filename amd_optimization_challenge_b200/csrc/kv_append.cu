// KV-cache append: bf16 latent rows [n, 576] -> rows of an FP8, MXFP4 or hybrid cache at given slots.
//
// The inverse of what the decode kernels read, with the arithmetic of the reference's quantisers so that a
// cache filled on the device holds the same bytes as one quantised by the reference on the host:
//   * e4m3 codes: x / scale rounded to bf16, clamped to +-448, cast (quantize_fp8,
//     competitor_submissions/mi355x_reference/reference.py:65-80).  The per-tensor scale is an input here:
//     rows appended later cannot change the scale of rows already in the cache.
//   * MXFP4: per block of 32 elements the E8M0 exponent floor(log2(amax rounded up at mantissa 1.75)) - 2 and
//     e2m1 codes rounded to nearest even (aiter's dynamic_mxfp4_quant as restated in
//     mxfp4-mm/submission_v3_self_contained.py:19-72; reference.py:88-113), two codes per byte, even element
//     in the low nibble.
//   * hybrid: dims 0..511 as MXFP4 (16 blocks), dims 512..575 as e4m3 with the per-tensor rope scale.
// One thread quantises one block of 32 elements (64 bytes in, 16 or 32 bytes out); HBM bound.
#include "mla_common.cuh"

namespace b200mla {

namespace {

struct AppendParams {
    const __nv_bfloat16* src; long long n; long long src_stride;   // elements between rows
    const int* slots; long long base_slot; long long num_slots;
    int kv_format;
    uint8_t* codes; long long codes_stride;
    uint8_t* bs; long long bs_stride;
    uint8_t* rope; long long rope_stride;
    const float* scale;
    int* bad;                                                       // set to 1 if a slot is outside [0, num_slots)
};

// 32 floats -> 16 bytes of e2m1 pairs and the block's E8M0 byte
__device__ __forceinline__ void quant_block_mxfp4(const float (&x)[32], uint4& codes, uint8_t& scale_byte) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[i]));
    // next power of two when the mantissa is >= 1.75, then two binades of headroom for the largest code (6 = 1.5 * 4)
    const unsigned int bits = ((unsigned int)__float_as_int(amax) + 0x200000u) & 0xFF800000u;
    const int e_field = (int)(bits >> 23);
    int e = e_field == 0 ? -127 : e_field - 127 - 2;
    e = max(-127, min(e, 127));
    scale_byte = (uint8_t)(e + 127);
    // 2^-e, also where it is a subnormal (e = 127)
    const float inv = e <= 126 ? __int_as_float((127 - e) << 23) : __int_as_float(0x00400000);
    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float q = x[i] * inv;
        const unsigned int qb = (unsigned int)__float_as_int(q);
        const unsigned int sign = (qb >> 28) & 0x8u;
        const unsigned int mb = qb & 0x7FFFFFFFu;
        const float mag = __int_as_float((int)mb);
        unsigned int code;
        if (mag >= 6.0f) code = 7u;
        else if (mag < 1.0f) code = (unsigned int)__float2int_rn(mag * 2.0f);      // 0, 0.5, 1.0: ties to even
        else {
            // [1, 6): re-bias the exponent 127 -> 1, keep one mantissa bit, round to nearest even
            const unsigned int odd = (mb >> 22) & 1u;
            code = ((mb - (126u << 23) + (1u << 21) - 1u + odd) >> 22) & 0xFFu;
        }
        w[i >> 3] |= (code | sign) << (4 * (i & 7));
    }
    codes = make_uint4(w[0], w[1], w[2], w[3]);
}

__global__ void __launch_bounds__(256) kv_append_kernel(const AppendParams p) {
    constexpr int BLOCKS_PER_ROW = QK_DIM / 32;                      // 18
    const long long total = p.n * BLOCKS_PER_ROW;
    const float scale = p.kv_format != KV_MXFP4 ? __ldg(p.scale) : 1.0f;
    for (long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (long long)gridDim.x * blockDim.x) {
        const long long row = id / BLOCKS_PER_ROW;
        const int blk = (int)(id - row * BLOCKS_PER_ROW);
        const long long slot = p.slots ? (long long)p.slots[row] : p.base_slot + row;
        if (slot < 0 || slot >= p.num_slots) { *p.bad = 1; continue; }          // never written
        const uint4* src = reinterpret_cast<const uint4*>(p.src + row * p.src_stride + blk * 32);
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __ldg(src + i);
        const bool as_e4m3 = p.kv_format == KV_E4M3 || (p.kv_format == KV_HYBRID && blk >= 16);
        if (as_e4m3) {
            uint2 o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] = q_cast_e4m3x8(v[i], scale);
            uint8_t* dst = p.kv_format == KV_E4M3 ? p.codes + slot * p.codes_stride + blk * 32
                                                  : p.rope + slot * p.rope_stride + (blk - 16) * 32;
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0].x, o[0].y, o[1].x, o[1].y);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[2].x, o[2].y, o[3].x, o[3].y);
        } else {
            float x[32];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    x[8 * i + k] = __bfloat162float(__ushort_as_bfloat16((unsigned short)(w[k >> 1] >> (16 * (k & 1)))));
            }
            uint4 codes;
            uint8_t sb;
            quant_block_mxfp4(x, codes, sb);
            *reinterpret_cast<uint4*>(p.codes + slot * p.codes_stride + blk * 16) = codes;
            p.bs[slot * p.bs_stride + blk] = sb;
        }
    }
}

}  // namespace

cudaError_t launch_kv_append(const void* src, long long n, long long src_stride, const int* slots, long long base_slot,
                             long long num_slots, int kv_format, void* codes, long long codes_stride, void* bs,
                             long long bs_stride, void* rope, long long rope_stride, const float* scale, int* bad,
                             cudaStream_t stream) {
    AppendParams p;
    p.src = (const __nv_bfloat16*)src; p.n = n; p.src_stride = src_stride;
    p.slots = slots; p.base_slot = base_slot; p.num_slots = num_slots; p.kv_format = kv_format;
    p.codes = (uint8_t*)codes; p.codes_stride = codes_stride;
    p.bs = (uint8_t*)bs; p.bs_stride = bs_stride;
    p.rope = (uint8_t*)rope; p.rope_stride = rope_stride;
    p.scale = scale; p.bad = bad;
    const long long total = n * (QK_DIM / 32);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    kv_append_kernel<<<(unsigned int)blocks, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace b200mla
