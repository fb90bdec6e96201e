// PTX wrappers and descriptor helpers shared by the tcgen05 / TMEM decode kernels: mbarriers with
// bounded waits, cp.async, named barriers, TMEM allocation / load / store, tcgen05.mma issue and
// commit, shared-memory matrix descriptors and instruction descriptors (kind::f8f6f4).
#pragma once

#include "mla_common.cuh"

namespace b200mla {
namespace sm100 {

constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;   // ~1 s: far beyond any legitimate wait of this kernel

// ----------------------------------------------------------------------------------------------
// PTX wrappers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(20000u) : "memory");   // may sleep up to 20 us per try
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try_nb(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Wait for completion number `n` (0-based) of the barrier; n = -1 passes at once.
// The wait is bounded: when it expires the thread raises the CTA's abort flag and carries on, and
// every later wait of the CTA returns at once.  Control flow never depends on the outcome, so all
// threads still meet at the same barriers; the results of such a launch are garbage and the
// kernel reports ST_TIMEOUT through the status word.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, int n, volatile int* abort_flag) {
    const uint32_t parity = (uint32_t)n & 1u;
    if (mbar_try(bar, parity)) return;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try(bar, parity)) return;
        if ((it & 63u) == 0u) {
            if (*abort_flag) return;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) break;
        }
    }
    *abort_flag = 1;
}

// mbarrier arrival of the executing thread that also announces `bytes` of asynchronous (TMA) traffic to the phase.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Tiled 2-D TMA load of one box (as the tensor map defines it) whose first element is (x, y); x is in elements of
// the map (bytes here) and must be a multiple of 16 bytes.  Completion is counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// Tiled 2-D TMA gather of FOUR rows (y0..y3, any order, any distance) of the map's tensor, `box width` bytes each starting
// at byte x (a multiple of 16), into four consecutive rows at dst_smem; the map's box is {width, 1}.  The swizzle of the
// map is applied as for an ordinary tile.  Completion is counted in bytes (4 x width) on `bar`.  This GPU's memory only.
__device__ __forceinline__ void tma_gather4_2d(uint32_t dst_smem, const void* tmap, int x, int y0, int y1, int y2, int y3, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                 ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(smem_u32(bar)) : "memory");
}
// The same with an L2 eviction policy for the fetched lines (see l2_evict_first_policy).
__device__ __forceinline__ void tma_gather4_2d_hint(uint32_t dst_smem, const void* tmap, int x, int y0, int y1, int y2, int y3, uint64_t* bar,
                                                    uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4, %5, %6}], [%7], %8;"
                 ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
// Policy word for data that is read once (the cache rows): its lines are the first to leave L2, so the streaming
// megabytes do not push out what every launch needs again - the kernels' code, Q, the page table.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
// The barrier receives one arrival once all cp.async copies issued so far by this thread have landed.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Wait until at most PENDING of this thread's most recent cp.async groups are still in flight.
template <int PENDING>
__device__ __forceinline__ void cp_async_wait_pending() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ bool named_bar_or(int id, int n, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"(id), "r"(n), "r"((uint32_t)pred) : "memory");
    return r != 0;
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Warp-wide forms: every lane of a converged warp executes them and one elected lane (the same one every time for a
// full mask) issues the instruction.  The surrounding loop then runs warp-uniformly, which keeps the descriptor
// arithmetic off the issuing thread's critical path: 34 MMAs of a decode tile issue in ~1370 cycles this way against
// ~1950 from a single thread inside an `if (lane == 0)` region (measured, M = 128, N = 16 / 32).
__device__ __forceinline__ void umma_f8_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred P1, p;\n\t.reg .b32 r;\n\t"
        "elect.sync r|P1, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@P1 tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_elect(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .pred P1;\n\t.reg .b32 r;\n\t"
        "elect.sync r|P1, 0xffffffff;\n\t"
        "@P1 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t addr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(addr) : "memory");
}

// Shared-memory matrix descriptor (tcgen05): start address, leading / stride byte offsets (all
// in 16-byte units), descriptor version 1, swizzle mode in the top bits.
constexpr uint64_t SWIZZLE_NONE = 0, SWIZZLE_128B = 2, SWIZZLE_64B = 4;
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t swizzle) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (swizzle << 61);
}
// Same layout, start address moved by `bytes` (the address field never carries: smem < 256 KB).
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (uint64_t)(bytes >> 4); }
// Instruction descriptor, kind::f8f6f4: fp32 accumulate, e4m3 x e4m3.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Per-column reduction of v[NC] over the 128 threads of a softmax warpgroup (maximum or sum); the result is replicated
// in every thread.  `red` = float[4][32] in shared memory, `warp4` = warp index inside the group, `bar_id` = the
// group's named barrier.  (A form with fewer shuffle / shared-memory operations - redux.sync on an order-preserving
// integer image for the maxima, one storing lane per column, 16-byte reads - was measured 1.4 us slower per call on the
// FP8 kernel in a same-GPU comparison and dropped.)
template <int NC, bool IS_MAX>
__device__ __forceinline__ void reduce_cols_128(float (&v)[NC], float (*red)[32], int warp4, int lane, int bar_id) {
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        float x = v[c];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const float y = __shfl_xor_sync(0xffffffffu, x, o);
            x = IS_MAX ? fmaxf(x, y) : x + y;
        }
        if (lane == 0) red[warp4][c] = x;
    }
    named_bar_sync(bar_id, 128);
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        const float a0 = red[0][c], a1 = red[1][c], a2 = red[2][c], a3 = red[3][c];
        v[c] = IS_MAX ? fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)) : (a0 + a1) + (a2 + a3);
    }
    named_bar_sync(bar_id, 128);
}

// The same reduction in a fraction of the instructions, for code that runs once per sequence, where what counts is how
// many instruction lines the first pass has to fetch: the values go through a scratch area of NC/R x 128 floats
// (column-major: thread t of the group = row t), NC/R columns per round, R rounds; 128 / (NC/R) threads share a column,
// each folds a contiguous run of rows read as 16-byte vectors, a few shuffles finish the column, one lane per column
// publishes it in `red` (>= NC floats).  2R named barriers; the caller owns `scratch` for the duration.
// t = thread index inside the group.
template <int NC, bool IS_MAX, int R>
__device__ __forceinline__ void reduce_cols_128_scratch(float (&v)[NC], float* scratch, float* red, int t, int bar_id) {
    constexpr int H = NC / R, TPC = 128 / H;          // columns per round, threads per column (= rows per thread: H)
    static_assert(NC % R == 0 && H % 4 == 0 && H * TPC == 128 && TPC <= 32, "column split");
    const int col = t / TPC, seg = t % TPC;
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int c = 0; c < H; ++c) scratch[c * 128 + t] = v[r * H + c];
        named_bar_sync(bar_id, 128);
        const float4* src = reinterpret_cast<const float4*>(scratch + col * 128 + seg * H);
        float4 a = src[0];
#pragma unroll
        for (int i = 1; i < H / 4; ++i) {
            const float4 b = src[i];
            a.x = IS_MAX ? fmaxf(a.x, b.x) : a.x + b.x; a.y = IS_MAX ? fmaxf(a.y, b.y) : a.y + b.y;
            a.z = IS_MAX ? fmaxf(a.z, b.z) : a.z + b.z; a.w = IS_MAX ? fmaxf(a.w, b.w) : a.w + b.w;
        }
        float x = IS_MAX ? fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)) : (a.x + a.y) + (a.z + a.w);
#pragma unroll
        for (int o = TPC / 2; o >= 1; o >>= 1) {
            const float y = __shfl_xor_sync(0xffffffffu, x, o);
            x = IS_MAX ? fmaxf(x, y) : x + y;
        }
        if (seg == 0) red[r * H + col] = x;
        named_bar_sync(bar_id, 128);
    }
#pragma unroll
    for (int c = 0; c < NC; c += 4) {
        const float4 q = *reinterpret_cast<const float4*>(red + c);
        v[c] = q.x; v[c + 1] = q.y; v[c + 2] = q.z; v[c + 3] = q.w;
    }
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// pack four floats into four e4m3 bytes (round to nearest even, saturating)
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
    return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ float2 unpack_e4m3x2(uint16_t v) { return __half22float2(e4m3x2_to_half2(v)); }


}  // namespace sm100
}  // namespace b200mla
