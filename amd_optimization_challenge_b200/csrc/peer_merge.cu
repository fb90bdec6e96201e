// Cross-GPU split-KV merge over peer memory: the exchange step and the log-sum-exp merge in ONE kernel.
//
// Every rank decodes its key range of every sequence into a normalised fp32 partial (O || LSE) that lives in an
// "exchange allocation" the other ranks have mapped (CUDA IPC).  Instead of an all-gather followed by a merge, the
// merge kernel of every rank
//   1. tells every peer "my partial of step e is complete" (one 4-byte release store per peer, system scope; the
//      partial was written by earlier kernels of the same stream),
//   2. waits, with a time limit, until every peer has said the same to it (acquire loads of its OWN flag words),
//   3. reads the peers' partials straight out of their memory with plain 16-byte loads over NVLink and merges them
//      row by row (math of combine_parts_kernel: M = max LSE_i, w_i = exp(LSE_i - M), O = sum w_i O_i / sum w_i).
// Nothing is copied twice and the link carries each partial once per reader.  The loads and stores are ordinary
// peer accesses to memory mapped with CUDA IPC; no switch-side reduction or broadcast object is bound to it.
//
// Exchange allocation of one rank:  [64 flag words | partial of even steps | partial of odd steps].  Flag word i is
// written by rank i only.  Two partial buffers are enough: a rank overwrites the buffer of step e-2 only after it
// passed the wait of step e-1, i.e. after every peer had started its merge of step e-1 and therefore (stream order)
// finished the merge of step e-2 that read that buffer.
//
// A peer that does not show up within the limit is reported (ST_TIMEOUT in the status word) and merged with weight
// 0; the kernel always returns.  The reference is single-GPU; what is merged is its split-KV reduce
// (mixed-mla/submission.py:257-294) across GPUs instead of across the splits of one GPU.
#include "mla_common.cuh"

namespace b200mla {

namespace {

constexpr int MAX_PEERS = 16;
constexpr int FLAG_BYTES = 256;

struct PeerMergeParams {
    const char* base[MAX_PEERS];           // every rank's exchange allocation as mapped here
    int world, rank;
    unsigned int epoch;
    unsigned long long limit_ns;
    long long rows;                        // batch * q_len * heads
    long long part_bytes;                  // bytes of one (O || LSE) partial, rounded up to 256
    __nv_bfloat16* out;
    int* status;
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <int W>
__global__ void __launch_bounds__(128) peer_merge_kernel(const PeerMergeParams p) {
    __shared__ unsigned int present[MAX_PEERS];
    const int tid = threadIdx.x;
    // 1. signal (one CTA), 2. wait (every CTA, one thread per peer)
    if (tid < W) {
        if (blockIdx.x == 0) {
            // release at system scope: the partial was written by earlier kernels of this stream (visible device-wide at
            // the kernel boundary); the release orders it before the flag for the peers as well
            st_release_sys(reinterpret_cast<unsigned int*>(const_cast<char*>(p.base[tid])) + p.rank, p.epoch);
        }
        const unsigned int* mine = reinterpret_cast<const unsigned int*>(p.base[p.rank]) + tid;
        unsigned int ok = tid == p.rank;
        if (!ok) {
            const unsigned long long t0 = global_ns();
            for (;;) {
                if ((int)(ld_acquire_sys(mine) - p.epoch) >= 0) { ok = 1u; break; }
                if (global_ns() - t0 > p.limit_ns) break;
                __nanosleep(64);
            }
            if (!ok) atomicOr(p.status, ST_TIMEOUT);
        }
        present[tid] = ok;
    }
    __syncthreads();
    // 3. merge the rows of this CTA
    const long long part_off = FLAG_BYTES + (long long)(p.epoch & 1u) * p.part_bytes;
    const long long lse_off = part_off + p.rows * V_DIM * 4;
    const int d = tid * 4;
    for (long long r = blockIdx.x; r < p.rows; r += gridDim.x) {
        float l[W];
        float4 v[W];
#pragma unroll
        for (int i = 0; i < W; ++i) {
            const bool ok = present[i] != 0u;
            l[i] = ok ? *reinterpret_cast<const float*>(p.base[i] + lse_off + r * 4) : -INFINITY;
            v[i] = ok ? *reinterpret_cast<const float4*>(p.base[i] + part_off + (r * V_DIM + d) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < W; ++i) M = fmaxf(M, l[i]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float den = 0.f;
        if (M > -INFINITY) {
#pragma unroll
            for (int i = 0; i < W; ++i) {
                const float wt = l[i] > -INFINITY ? expf(l[i] - M) : 0.f;
                acc.x += wt * v[i].x; acc.y += wt * v[i].y; acc.z += wt * v[i].z; acc.w += wt * v[i].w;
                den += wt;
            }
            const float inv = 1.0f / den;
            acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
        }
        __align__(8) __nv_bfloat162 o[2] = {__floats2bfloat162_rn(acc.x, acc.y), __floats2bfloat162_rn(acc.z, acc.w)};
        *reinterpret_cast<uint2*>(p.out + r * V_DIM + d) = *reinterpret_cast<uint2*>(o);
    }
}

}  // namespace

long long peer_part_bytes(long long rows) { return (rows * (V_DIM + 1) * 4 + 255) & ~255LL; }
long long peer_exchange_bytes(long long rows) { return FLAG_BYTES + 2 * peer_part_bytes(rows); }
long long peer_partial_offset(long long rows, unsigned int epoch) { return FLAG_BYTES + (long long)(epoch & 1u) * peer_part_bytes(rows); }

cudaError_t launch_peer_merge(const void* const* bases, int world, int rank, unsigned int epoch, unsigned long long limit_ns,
                              long long rows, void* out, int* status, cudaStream_t stream) {
    PeerMergeParams p;
    for (int i = 0; i < MAX_PEERS; ++i) p.base[i] = (const char*)bases[i < world ? i : 0];
    p.world = world; p.rank = rank; p.epoch = epoch; p.limit_ns = limit_ns;
    p.rows = rows; p.part_bytes = peer_part_bytes(rows);
    p.out = (__nv_bfloat16*)out; p.status = status;
    const unsigned int grid = (unsigned int)(rows < 148 * 8 ? rows : 148 * 8);
    switch (world) {
        case 1: peer_merge_kernel<1><<<grid, 128, 0, stream>>>(p); break;
        case 2: peer_merge_kernel<2><<<grid, 128, 0, stream>>>(p); break;
        case 4: peer_merge_kernel<4><<<grid, 128, 0, stream>>>(p); break;
        case 8: peer_merge_kernel<8><<<grid, 128, 0, stream>>>(p); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace b200mla
