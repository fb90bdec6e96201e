// Dynamic per-tensor e4m3fn quantisation of a bf16 tensor (used for Q on the FP8-Q paths).
//
// Arithmetic order of the reference's quantize_fp8 (competitor_submissions/mi355x_reference/
// reference.py:65-80), which runs on a bf16 tensor so every intermediate is rounded to bf16:
//   amax  = max |x|, clamped below at 1e-12 (rounded to bf16)
//   scale = bf16(amax / 448)
//   y     = bf16(x / scale), clamped to +-448, cast to e4m3fn (round to nearest even)
// Two launches: an atomic-max reduction over the bf16 magnitudes, then the cast
// (same split as mixed-mla/fused_fp8_quant.py:27-82).
#include "mla_common.cuh"

namespace b200mla {

namespace {

__global__ void amax_kernel(const __nv_bfloat16* __restrict__ x, long long n, unsigned int* amax_bits) {
    unsigned int m = 0;
    const long long stride = (long long)gridDim.x * blockDim.x * 8;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
        if (i + 8 <= n) {
            uint4 v = __ldg(reinterpret_cast<const uint4*>(x + i));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                m = max(m, w[k] & 0x7fffu);
                m = max(m, (w[k] >> 16) & 0x7fffu);
            }
        } else {
            for (long long j = i; j < n; ++j) m = max(m, (unsigned)(__bfloat16_as_ushort(x[j]) & 0x7fffu));
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m) atomicMax(amax_bits, m);   // bf16 magnitudes order like their bit patterns
}

__device__ __forceinline__ float scale_from_amax_bits(unsigned int bits) {
    float amax = __bfloat162float(__ushort_as_bfloat16((unsigned short)bits));
    amax = __bfloat162float(__float2bfloat16_rn(fmaxf(amax, 1e-12f)));
    return __bfloat162float(__float2bfloat16_rn(amax / 448.0f));
}

__global__ void cast_kernel(const __nv_bfloat16* __restrict__ x, long long n, uint8_t* __restrict__ out,
                            float* scale_out, const unsigned int* amax_bits) {
    const float scale = scale_from_amax_bits(*amax_bits);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const long long stride = (long long)gridDim.x * blockDim.x * 8;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
        const int cnt = (int)min((long long)8, n - i);
        __align__(8) uint8_t o[8];
        for (int k = 0; k < cnt; ++k) {
            float y = __bfloat162float(x[i + k]) / scale;                       // IEEE division
            y = __bfloat162float(__float2bfloat16_rn(y));                        // bf16 rounding of the quotient
            y = fminf(fmaxf(y, -448.0f), 448.0f);
            o[k] = (uint8_t)__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
        }
        if (cnt == 8) *reinterpret_cast<uint2*>(out + i) = *reinterpret_cast<uint2*>(o);
        else for (int k = 0; k < cnt; ++k) out[i + k] = o[k];
    }
}

// Per-block maxima of the bf16 magnitudes, Q_AMAX_PARTS blocks, every block writes its word.
__global__ void __launch_bounds__(256) amax_parts_kernel(const __nv_bfloat16* __restrict__ x, long long n, unsigned int* parts) {
    __shared__ unsigned int red[8];
    unsigned int m = 0;
    const long long stride = (long long)gridDim.x * blockDim.x * 8;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
        if (i + 8 <= n) {
            uint4 v = __ldg(reinterpret_cast<const uint4*>(x + i));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                m = max(m, w[k] & 0x7fffu);
                m = max(m, (w[k] >> 16) & 0x7fffu);
            }
        } else {
            for (long long j = i; j < n; ++j) m = max(m, (unsigned)(__bfloat16_as_ushort(x[j]) & 0x7fffu));
        }
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 1; i < 8; ++i) m = max(m, red[i]);
        parts[blockIdx.x] = m;
    }
}

}  // namespace

cudaError_t launch_q_amax_parts(const __nv_bfloat16* x, long long n, unsigned int* parts, cudaStream_t stream) {
    amax_parts_kernel<<<Q_AMAX_PARTS, 256, 0, stream>>>(x, n, parts);
    return cudaGetLastError();
}

cudaError_t launch_quantize_fp8(const __nv_bfloat16* x, long long n, uint8_t* out, float* scale_out,
                                unsigned int* scratch, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(unsigned int), stream);
    if (e != cudaSuccess) return e;
    const int threads = 256;
    long long want = (n + threads * 8 - 1) / (threads * 8);
    const int blocks = (int)max((long long)1, min(want, (long long)1184));
    amax_kernel<<<blocks, threads, 0, stream>>>(x, n, scratch);
    cast_kernel<<<blocks, threads, 0, stream>>>(x, n, out, scale_out, scratch);
    return cudaGetLastError();
}

}  // namespace b200mla
