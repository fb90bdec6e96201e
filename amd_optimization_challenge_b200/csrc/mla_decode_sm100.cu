// Stage-1 MLA decode on the 5th-generation tensor cores (tcgen05) with TMEM accumulators.
//
// Swap-AB formulation, so that the 128-row MMA dimension is filled by KV tokens and the small
// dimension (16..32 query rows) is the MMA N:
//     S^T[128 tok x N]   = K[128 tok x 576] . Q^T          A = K tile (K-major, 128B swizzle), B = Q
//     O^T[512 x 2N]     += V^T[512 x 128 tok] . P^T         A = the same tile read MN-major (V = first
//                                                           512 dims of K), B = P written by the
//                                                           softmax warps, 4 M-blocks of 128 dims
// Both contractions run as kind::f8f6f4 on e4m3 operands with fp32 accumulation in TMEM.  P is
// split into two e4m3 terms (P = hi + lo/16, the two halves of the 2N columns) so that the
// probabilities keep ~8 significant bits.
//
// The CTA walks its span of tiles (112 tokens at N = 16, three stages; 128 at N = 32, two stages) as one continuous
// stream: the gather, the MMA issue and the softmax each run their own loop over the tiles and meet only through
// mbarriers, also across the boundary between two sequences (Q is double buffered; only the first PV of the next
// sequence waits until the epilogue has read O out of TMEM).
//
// Roles:  warps 0-3  softmax / correction / epilogue (one TMEM lane = one token / one output dim per thread)
//         warp  4    tcgen05.mma issue (the whole warp runs the loop, one elected lane issues), TMEM allocation
//         warps 5..  gather of the cache rows (and of the Q rows of each sequence) straight into the swizzled UMMA
//                    layout, completion signalled on the stage's mbarrier:
//                      contiguous cache (no page table)  tiled TMA, five cp.async.bulk.tensor.2d copies per tile
//                      page table                        16-byte cp.async per row piece; the page ids reach shared
//                                                        memory by 4-byte cp.async three tiles ahead
// Movers measured on B200 for shuffled 576-byte rows, device-wide, one CTA per SM:
//         16-byte cp.async, 6 / 9 / 11 / 16 / 24 warps 3.9 / 4.3 / 4.1 / 5.4 / 5.2 TB/s, lands directly in operand layout
//         TMA tile::gather4 (4 rows x 128 B / instr)   1.3 - 2.9 TB/s, ~60 cycles per instruction
//         one cp.async.bulk per row, 4 issuing warps   5.3 TB/s, but row-major: needs ~80 KB of raw staging
//                                                      per SM beside the operand tiles plus a re-layout pass
// A tiled TMA box cannot fetch the rows of a page-size-1 table (they are not contiguous).
// Synchronisation is mbarrier based; every wait is bounded and on expiry sets a status word.
// Online softmax runs in the exp2 domain with lazy re-centering: the reference maximum is only
// raised (and O rescaled in TMEM) when a score exceeds it by more than 2^4.
//
// Role in the reference: the split-KV stage-1 kernels (mixed-mla/submission.py:122-250,
// mixed-mla/versions/hip_mxfp4_v5/submission.py:214-656).
#include <cuda.h>
#include <cstdlib>
#include <cstring>

#include "sm100_ptx.cuh"

namespace b200mla {
namespace sm100 {

constexpr int MMA_M = 128;                // rows of every MMA: tokens for QK, output dims for PV; S and P span MMA_M rows
constexpr int NS_MAX = 3;
constexpr int SLOT_RING = 8;              // tiles whose page ids can be in flight / in use at once
constexpr int SMEM_LIMIT = 232448;        // opt-in shared memory per CTA
constexpr float RECENTER = 4.0f;          // log2 units
constexpr float P_SCALE_LOG2 = 4.0f;      // probabilities are stored multiplied by 2^4

// ----------------------------------------------------------------------------------------------
// N = 16: three stages of 112-token tiles (63 KB each).  Every MMA still spans 128 rows: rows 112..127 of a QK
// operand are the first rows of whatever follows the panel (their scores are never read), and the phantom tokens
// 112..127 of a PV k-step are the head of the next panel of the same stage, multiplied by probabilities that are
// written as zeros.  The third stage is worth more than the 12.5 % of MMA rows it gives up: a stage is held from
// the start of its gather until PV of its tile, about two tile periods of tensor work plus the gather latency.
// N = 32: two stages of 128-token tiles (Q and P take the room of a third stage).
template <int N>
struct Layout {
    static constexpr int TILE = (N == 16) ? 112 : 128;           // tokens per tile
    static constexpr int NS = (N == 16) ? 3 : 2;                 // cache tile stages
    static constexpr int PANEL_BYTES = TILE * 128;               // dims 128j..128j+127, 128B swizzle
    static constexpr int ROPE_PANEL_BYTES = TILE * 64;           // dims 512..575: 64-byte rows, 64B swizzle
    static constexpr int STAGE_BYTES = 4 * PANEL_BYTES + ROPE_PANEL_BYTES;
    static constexpr int NPANEL = 5;                             // Q keeps five 128-byte-wide panels
        static constexpr int PRODUCER_WARPS = (N == 16) ? 9 : 2;     // N = 16: 288 = 8 x 36 threads, one 16-byte column and one row phase each; N = 32 needs the registers
    static constexpr int PRODUCERS = 32 * PRODUCER_WARPS;
    static constexpr int FIRST_PRODUCER = 160;
    static constexpr int THREADS = FIRST_PRODUCER + PRODUCERS;
    static constexpr int Q_PANEL_BYTES = N * 128;
    static constexpr int Q_BYTES = NPANEL * Q_PANEL_BYTES;        // one Q buffer (two of them: next sequence's Q loads early)
    static constexpr int P_CHUNKS = 2 * N / 16;                  // 16-column chunks of [hi | lo]
    static constexpr int P_BUF_BYTES = P_CHUNKS * MMA_M * 16;
    static constexpr int OFF_Q = NS * STAGE_BYTES;
    static constexpr int OFF_P = OFF_Q + 2 * Q_BYTES;
    static constexpr int OFF_MISC = OFF_P + 2 * P_BUF_BYTES;
    static constexpr int TMEM_S = 0;                              // two S buffers of N columns
    static constexpr int TMEM_O = 2 * N;                          // four O blocks of 2N columns
    static constexpr int TMEM_COLS = (10 * N <= 256) ? 256 : 512;
};

struct Misc {
    uint64_t kv_full[NS_MAX], kv_empty[NS_MAX], s_full[2], s_empty[2], p_full[2], p_empty[2];
    uint64_t q_full[2], q_empty[2], o_free;
    uint32_t tmem_base;
    int abort_flag;
    unsigned int q_amax;         // block_q_scale's word
    uint64_t slot_full[SLOT_RING];
    int slot[SLOT_RING][MMA_M];  // page ids of the tiles g .. g + NS, fetched by 4-byte cp.async
    __align__(16) float red[4][32];   // cross-warp exchange (max / sum), 32 = max N
};

template <int N, bool QCAST>
__global__ void __launch_bounds__(Layout<N>::THREADS, 1) mla_decode_sm100_kernel(const MlaParams p, int* status, const __grid_constant__ CUtensorMap tmap_lat,
                                                                                 const __grid_constant__ CUtensorMap tmap_rope, const int use_tma) {
    using L = Layout<N>;
    constexpr int PRODUCERS = L::PRODUCERS, THREADS = L::THREADS;
    constexpr int TILE = L::TILE, NS = L::NS, PANEL_BYTES = L::PANEL_BYTES, STAGE_BYTES = L::STAGE_BYTES;
    extern __shared__ __align__(1024) unsigned char smem[];
    Misc& ms = *reinterpret_cast<Misc*>(smem + L::OFF_MISC);
    int* prefix = reinterpret_cast<int*>(smem + L::OFF_MISC + sizeof(Misc));
    const uint32_t smem_base = smem_u32(smem);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int w = blockIdx.x, G = p.num_ctas;
    const int row0 = blockIdx.y * N;
    const unsigned int q_amax_local = block_q_amax_begin(p.q_amax_parts, QCAST);   // loads in flight during the prologue
    const float kv_sc = __ldg(p.kv_scale);       // issued here, first used by the softmax role: no role waits for it at its start

    // The page ids this CTA will walk lie near w/G of the table: pull that neighbourhood into L2 while kv_indptr is being
    // read and scanned, so that the first dependent page-table read is not a cold DRAM access.
    if (p.kv_indices != nullptr && p.total_kv_hint > 0 && p.total_kv_hint < (1LL << 31) && tid < 64) {
        const unsigned int n_ids = (unsigned int)p.total_kv_hint / (unsigned int)p.page_size, per = n_ids / (unsigned int)G;   // 32-bit: a few instructions
        const unsigned int lo = (w * per > 256u ? w * per - 256u : 0u) & ~31u, hi = min((w + 1) * per + 256u, n_ids);
        for (unsigned int i = lo + tid * 32; i < hi; i += 64 * 32)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.kv_indices + i));
    }
    if (tid == L::FIRST_PRODUCER && use_tma) {                 // the copy engine's descriptors: fetched while the schedule is computed
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_lat) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_rope) : "memory");
    }
    if (tid == 0) {
        for (int i = 0; i < NS; ++i) { mbar_init(&ms.kv_full[i], PRODUCERS); mbar_init(&ms.kv_empty[i], 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ms.s_full[i], 1); mbar_init(&ms.s_empty[i], 128);
            mbar_init(&ms.p_full[i], 128); mbar_init(&ms.p_empty[i], 1);
            mbar_init(&ms.q_full[i], PRODUCERS); mbar_init(&ms.q_empty[i], 1);
        }
        for (int i = 0; i < SLOT_RING; ++i) mbar_init(&ms.slot_full[i], PRODUCERS);
        mbar_init(&ms.o_free, 128);
        ms.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) { tmem_alloc(&ms.tmem_base, L::TMEM_COLS); tmem_relinquish(); }
    build_tile_prefix(p.kv_indptr, p.batch, TILE, prefix);       // ends with __syncthreads()
    tc_fence_after();
    const uint32_t tmem = ms.tmem_base;
    const int TT = prefix[p.batch];
    if (w == 0 && blockIdx.y == 0)
        for (int i = tid; i <= p.batch; i += THREADS) p.tile_prefix[i] = prefix[i];

    int b_begin = 0;
    const int t_begin = TT > 0 ? span_begin_seq(prefix, p.batch, w, G, b_begin) : 0, t_end = TT > 0 ? span_begin(prefix, p.batch, w + 1, G) : 0;
    const int n_total = t_end - t_begin;                          // tiles of this CTA; tile index g = 0..n_total-1

    const float q_sc = block_q_scale(q_amax_local, p.q_scale, QCAST, &ms.q_amax);
    volatile int* abort_flag = &ms.abort_flag;

    if (n_total > 0) {
        if (warp >= 5) {
            // =========================== gather ===========================
            // One stage = TILE tokens x 36 sixteen-byte columns.  Consecutive threads take consecutive
            // columns, so a warp instruction reads 512 contiguous bytes of (at most two) rows.
            const int pt = tid - L::FIRST_PRODUCER;
            Walker wk; wk.init_at(b_begin);
            Walker wn = wk;                                       // NS tiles ahead, for the page-table prefetch
            const bool paged = p.kv_indices != nullptr;
            // Page ids of tile g -> ring entry g % SLOT_RING by 4-byte cp.async, NS tiles before the tile's rows are
            // requested, completion on the entry's mbarrier (no registers held, no barrier among the gather threads).
            // An entry is rewritten SLOT_RING tiles later; a thread that prefetches for tile g + NS has passed the
            // kv_empty wait of tile g, so every other thread has at least issued tile g - NS and reads entries
            // g - NS + 1 .. g at most: no overlap with entry g + NS as long as SLOT_RING > 2 NS.
            static_assert(SLOT_RING > 2 * NS, "page-id ring");
            auto prefetch_ids = [&](int g) {
                if (!paged || use_tma == 2 || g >= n_total) return;     // the row gathers read their ids themselves
                wn.seek(p, prefix, t_begin + g);
                const int pos0 = (t_begin + g - wn.seq_t0) * TILE;
                for (int tok = pt; tok < TILE; tok += PRODUCERS) {
                    const int pos = pos0 + tok;
                    const bool ok = pos < wn.seq_len;
                    const int pg = p.page_size == 1 ? pos : pos / p.page_size;
                    cp_async4(smem_u32(&ms.slot[g % SLOT_RING][tok]), p.kv_indices + (ok ? wn.page_base + pg : 0), ok ? 4u : 0u);
                }
                cp_async_mbar_arrive_noinc(&ms.slot_full[g % SLOT_RING]);
            };
            // cache slot of token `tok` of tile g (wk describes its sequence), -1 past the end of the sequence
            auto slot_at = [&](int g, int pos0, int tok) -> int {
                const int pos = pos0 + tok;
                if (pos >= wk.seq_len) return -1;
                if (!paged) return wk.seq_base + pos;
                const int id = ms.slot[g % SLOT_RING][tok];
                return p.page_size == 1 ? id : id * p.page_size + (pos % p.page_size);
            };
            // Q of the (CTA, sequence) pair that has been loaded but not yet stored: sequence, pair index, tile at which to store
            constexpr int QV = (N * 72 + PRODUCERS - 1) / PRODUCERS;     // 16-byte bf16 vectors per thread
            constexpr bool Q_PRELOAD = QV <= 8;
            uint4 qv[Q_PRELOAD ? QV : 1];
            int q_b = 0, q_pair = 0;
            auto q_src = [&](int b, int i) {
                const int r = i / 72, v8 = i - r * 72;
                const int rg = row0 + r, j = rg / p.heads, h = rg - j * p.heads;
                return reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.q) +
                                                      (long long)(b * p.q_len + j) * p.q_row_stride + (long long)h * p.q_head_stride + v8 * 8);
            };
            // Q rows of sequence q_b -> swizzled K-major panels of Q buffer (q_pair & 1)
            auto flush_q = [&]() {
                const int qb = q_pair & 1;
                mbar_wait(&ms.q_empty[qb], q_pair / 2 - 1, abort_flag);
                const uint32_t q_addr = smem_base + L::OFF_Q + qb * L::Q_BYTES;
                if constexpr (QCAST) {
                    // bf16 rows, quantised here: eight values in, eight e4m3 bytes (half a 16-byte column) out
                    unsigned char* q_smem = smem + L::OFF_Q + qb * L::Q_BYTES;
                    auto put = [&](int i, const uint4& raw) {
                        const int r = i / 72, v8 = i - r * 72, c = v8 >> 1;
                        *reinterpret_cast<uint2*>(q_smem + (c >> 3) * L::Q_PANEL_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4) + (v8 & 1) * 8) =
                            q_cast_e4m3x8(raw, q_sc);
                    };
                    if constexpr (Q_PRELOAD) {
#pragma unroll
                        for (int k = 0; k < QV; ++k) {
                            const int i = pt + k * PRODUCERS;
                            if (i < N * 72) put(i, qv[Q_PRELOAD ? k : 0]);
                        }
                    } else {
                        for (int i0 = pt; i0 < N * 72; i0 += 8 * PRODUCERS) {     // eight loads in flight, then their conversion
                            uint4 raw[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u)
                                if (i0 + u * PRODUCERS < N * 72) raw[u] = __ldg(q_src(q_b, i0 + u * PRODUCERS));
#pragma unroll
                            for (int u = 0; u < 8; ++u)
                                if (i0 + u * PRODUCERS < N * 72) put(i0 + u * PRODUCERS, raw[u]);
                        }
                    }
                    fence_proxy_async();                      // the MMA reads Q through the async proxy
                    mbar_arrive(&ms.q_full[qb]);
                } else {
                    for (int i = pt; i < N * 36; i += PRODUCERS) {
                        const int r = i / 36, c = i - r * 36;
                        const int rg = row0 + r, j = rg / p.heads, h = rg - j * p.heads;
                        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.q) +
                                             (long long)(q_b * p.q_len + j) * p.q_row_stride + (long long)h * p.q_head_stride + c * 16;
                        cp_async16(q_addr + (c >> 3) * L::Q_PANEL_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4), src, 16u);
                    }
                    cp_async_mbar_arrive_noinc(&ms.q_full[qb]);
                }
            };
#pragma unroll 1
            for (int g = 0; g < NS; ++g) prefetch_ids(g);
            for (int g = 0; g < n_total; ++g) {
                const int st = g % NS;
                const bool first = wk.seek(p, prefix, t_begin + g);
                // Q rows of a new sequence.  A bf16 Q that is quantised on load is fetched into registers NOW, ahead of the
                // tile's copies (a load issued behind them returns only after the megabytes queued before it); it is converted
                // and stored right after them.  (Deferring the conversion until all stages are in flight was measured: 1.3 us
                // slower per call - three tiles requested at once make the first one land later.)
                if (first) {
                    q_b = wk.b; q_pair = wk.pair;
                    if constexpr (QCAST && Q_PRELOAD) {
#pragma unroll
                        for (int k = 0; k < QV; ++k) {
                            const int i = pt + k * PRODUCERS;
                            qv[Q_PRELOAD ? k : 0] = i < N * 72 ? __ldg(q_src(q_b, i)) : make_uint4(0u, 0u, 0u, 0u);
                        }
                    }
                }
                const int pos0 = (t_begin + g - wk.seq_t0) * TILE;
                // Row gathers by the TMA unit: the thread of group gi reads its four page ids (and the id of the tile's
                // first row, the stand-in for rows past the end) straight from the table, before the wait for the stage,
                // which hides their latency.  No ring, no barrier: nobody else needs these ids.
                constexpr int G4 = TILE / 4;
                constexpr int G4S = PRODUCERS / G4 >= 8 ? 8 : (PRODUCERS / G4 >= 4 ? 4 : (PRODUCERS / G4 >= 2 ? 2 : 1));
                static_assert(G4 * 4 == TILE && G4 * G4S <= PRODUCERS, "one thread per group of four rows");
                const int gi = pt / G4S;
                const bool g4_issuer = use_tma == 2 && pt % G4S == 0 && gi < G4;
                int r4[4] = {0, 0, 0, 0};
                if (g4_issuer) {
                    int id[5];
#pragma unroll
                    for (int k = 0; k < 5; ++k) {
                        const int pos = k < 4 ? pos0 + 4 * gi + k : pos0;
                        const int e = p.page_size == 1 ? pos : pos / p.page_size;
                        id[k] = pos < wk.seq_len ? __ldg(p.kv_indices + wk.page_base + e) : -1;
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int pos = id[k] < 0 ? pos0 : pos0 + 4 * gi + k;
                        const int pid = id[k] < 0 ? id[4] : id[k];
                        r4[k] = (int)clamp_slot(p, p.page_size == 1 ? pid : pid * p.page_size + pos % p.page_size);
                    }
                }
                if (paged && use_tma != 2) mbar_wait(&ms.slot_full[g % SLOT_RING], g / SLOT_RING, abort_flag);
                mbar_wait(&ms.kv_empty[st], g / NS - 1, abort_flag);
                const uint32_t stage_addr = smem_base + st * STAGE_BYTES;
                // Contiguous cache (no page table: token t of the batch lives in slot t) and a tile that lies wholly inside
                // its sequence: the tile is five tiled TMA copies (four 128-byte-wide panels, 128B swizzle, and the 64-byte
                // rope panel, 64B swizzle) issued by one thread and completed on the stage's mbarrier by byte count; the
                // other gather threads only arrive.  A tile that reaches past the end of its sequence takes the copy loop
                // below, which zero-fills the missing rows (TMA would bring whatever follows in memory, and zero
                // probabilities do not neutralise non-finite bytes).
                if (use_tma == 2) {
                    // Paged cache: the tile is TILE / 4 groups of four rows; one thread per group hands the four page
                    // ids to the TMA unit, which fetches the rows' five panels (four 128-byte-wide, one 64-byte) with the
                    // swizzle of the operand layout - 5 instructions per 4 rows instead of 144 16-byte copies.  A row past
                    // the end of the sequence names the tile's first row instead (real cache bytes, finite; its
                    // probabilities are zero).  Completion: bytes on the stage's mbarrier, announced per group.
                    if (g4_issuer) {
                        const int (&r)[4] = r4;
                        mbar_arrive_expect_tx(&ms.kv_full[st], 4u * QK_DIM);
                        const uint64_t pol = l2_evict_first_policy();
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            tma_gather4_2d_hint(stage_addr + j * PANEL_BYTES + gi * 512, &tmap_lat, 128 * j, r[0], r[1], r[2], r[3], &ms.kv_full[st], pol);
                        tma_gather4_2d_hint(stage_addr + 4 * PANEL_BYTES + gi * 256, &tmap_rope, 512, r[0], r[1], r[2], r[3], &ms.kv_full[st], pol);
                    } else {
                        mbar_arrive(&ms.kv_full[st]);
                    }
                } else if (use_tma == 1 && pos0 + TILE <= wk.seq_len) {
                    if (pt == 0) {
                        mbar_arrive_expect_tx(&ms.kv_full[st], (uint32_t)STAGE_BYTES);
                        const int row = wk.seq_base + pos0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) tma_load_2d(stage_addr + j * PANEL_BYTES, &tmap_lat, 128 * j, row, &ms.kv_full[st]);
                        tma_load_2d(stage_addr + 4 * PANEL_BYTES, &tmap_rope, 512, row, &ms.kv_full[st]);
                    } else {
                        mbar_arrive(&ms.kv_full[st]);
                    }
                } else {
                // Slots first, then the copies, for the whole tile at once: a shared-memory load that sits between copy
                // instructions waits behind them in the load/store unit, and the copies after it wait for the load
                // (measured in isolation: 4.1 TB/s with two batches per tile, 5.4 TB/s with one).
                if constexpr (PRODUCERS % 36 == 0 && (PRODUCERS / 36) == 8) {
                    // thread = (16-byte column c, row phase r): tokens r, r + 8, ...; the swizzle term of the destination
                    // depends on the token only through r, so source and destination advance by constants
                    constexpr int PER = TILE / 8;
                    const int c = pt % 36, r = pt / 36;
                    const uint32_t dst0 = c < 32 ? stage_addr + (c >> 3) * PANEL_BYTES + r * 128 + (((c & 7) ^ r) << 4)
                                                 : stage_addr + 4 * PANEL_BYTES + r * 64 + (((c - 32) ^ ((r >> 1) & 3)) << 4);
                    const uint32_t dstep = c < 32 ? 1024u : 512u;
                    const uint8_t* src0 = p.kv_codes + c * 16;
                    int sl[PER];
#pragma unroll
                    for (int i = 0; i < PER; ++i) sl[i] = slot_at(g, pos0, r + 8 * i);
#pragma unroll
                    for (int i = 0; i < PER; ++i)
                        cp_async16(dst0 + i * dstep, src0 + (long long)clamp_slot(p, sl[i]) * p.kv_codes_stride, sl[i] < 0 ? 0u : 16u);
                } else {
                    constexpr int PER_TILE = (TILE * 36 + PRODUCERS - 1) / PRODUCERS;
                    constexpr int BATCH = PER_TILE < 16 ? PER_TILE : 16;
                    for (int id0 = pt; id0 < TILE * 36; id0 += BATCH * PRODUCERS) {
                        int sl[BATCH];
#pragma unroll
                        for (int u = 0; u < BATCH; ++u) {
                            const int id = id0 + u * PRODUCERS;
                            sl[u] = id < TILE * 36 ? slot_at(g, pos0, id / 36) : -2;
                        }
#pragma unroll
                        for (int u = 0; u < BATCH; ++u) {
                            const int id = id0 + u * PRODUCERS;
                            if (sl[u] != -2) {
                                const int tok = id / 36, c = id - tok * 36;
                                const uint8_t* src = p.kv_codes + (long long)clamp_slot(p, sl[u]) * p.kv_codes_stride + c * 16;
                                const uint32_t dst = c < 32 ? stage_addr + (c >> 3) * PANEL_BYTES + tok * 128 + (((c & 7) ^ (tok & 7)) << 4)
                                                            : stage_addr + 4 * PANEL_BYTES + tok * 64 + (((c - 32) ^ ((tok >> 1) & 3)) << 4);
                                cp_async16(dst, src, sl[u] < 0 ? 0u : 16u);     // rows past the end of the sequence: zero fill
                            }
                        }
                    }
                }
                cp_async_mbar_arrive_noinc(&ms.kv_full[st]);   // asynchronous: the thread does not wait for its copies
                }
                prefetch_ids(g + NS);
                if (first) flush_q();       // Q rows of a new sequence go out right behind its first tile
            }
            // every tile has been requested and the last ones are still being multiplied: time to look over the page ids of
            // this CTA's span (reporting only, see clamp_slot) without delaying anything
            if (blockIdx.y == 0) check_span_pages(p, prefix, t_begin, t_end, TILE, pt, PRODUCERS);
            cp_async_wait_all();
        } else if (warp == 4) {
            // =========================== MMA issue (whole warp, one elected lane per instruction) ===========================
            {
                constexpr uint32_t IDESC_QK = make_idesc(MMA_M, N, false, false);
                constexpr uint32_t IDESC_PV = make_idesc(128, 2 * N, true, true);
                // descriptor bases; per-MMA descriptors differ only in the start address
                const uint64_t d_qk_a = make_desc(smem_base, 16, 1024, SWIZZLE_128B);                  // + stage
                const uint64_t d_qk_a_rope = make_desc(smem_base + 4 * PANEL_BYTES, 16, 512, SWIZZLE_64B);   // + stage
                const uint64_t d_qk_b = make_desc(smem_base + L::OFF_Q, 16, 1024, SWIZZLE_128B);       // + Q buffer
                const uint64_t d_pv_a = make_desc(smem_base, PANEL_BYTES, 1024, SWIZZLE_128B);         // + stage
                const uint64_t d_pv_b = make_desc(smem_base + L::OFF_P, 128, MMA_M * 16, SWIZZLE_NONE); // + buffer
                Walker wq, wv;                                    // the QK stream runs ahead of the PV stream
                wq.init_at(b_begin);
                wv = wq;
                // S^T[128 tok x N] = K . Q^T for tile g
                auto issue_qk = [&](int g) {
                    const int st = g % NS, sb = g & 1;
                    fence_proxy_async();       // stage and Q were written by cp.async (generic proxy); the MMA reads through the async proxy
                    tc_fence_after();
                    const uint64_t a0 = desc_advance(d_qk_a, st * STAGE_BYTES);
                    const uint64_t b0 = desc_advance(d_qk_b, (wq.pair & 1) * L::Q_BYTES);
                    // panel by panel, the loop over panels not unrolled: the issue code stays a few hundred bytes, which is
                    // what the first pass through it (instruction fetch from L2, on every CTA's critical path) pays for
#pragma unroll 1
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_f8_elect(tmem + L::TMEM_S + sb * N, desc_advance(a0, j * PANEL_BYTES + k * 32),
                                          desc_advance(b0, j * L::Q_PANEL_BYTES + k * 32), IDESC_QK, (j | k) ? 1u : 0u);
                    }
#pragma unroll
                    for (int k = 0; k < 2; ++k)
                        umma_f8_elect(tmem + L::TMEM_S + sb * N, desc_advance(d_qk_a_rope, st * STAGE_BYTES + k * 32),
                                      desc_advance(b0, 4 * L::Q_PANEL_BYTES + k * 32), IDESC_QK, 1u);
                    umma_commit_elect(&ms.s_full[sb]);
                    // last tile of this (CTA, sequence) pair: its Q buffer is free once these MMAs have run
                    if (t_begin + g + 1 == min(t_end, wq.seq_t1)) umma_commit_elect(&ms.q_empty[wq.pair & 1]);
                };
                // O^T += V^T P^T over the 128 tokens of tile g, four blocks of 128 dims
                auto issue_pv = [&](int g, bool first) {
                    const int st = g % NS, pb = g & 1;
                    tc_fence_after();
                    const uint64_t a0 = desc_advance(d_pv_a, st * STAGE_BYTES);
                    const uint64_t b0 = desc_advance(d_pv_b, pb * L::P_BUF_BYTES);
#pragma unroll 1
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            umma_f8_elect(tmem + L::TMEM_O + j * 2 * N, desc_advance(a0, j * PANEL_BYTES + kk * 32 * 128),
                                    desc_advance(b0, kk * 32 * 16), IDESC_PV, (first && kk == 0) ? 0u : 1u);
                        }
                    }
                    umma_commit_elect(&ms.kv_empty[st]);
                    umma_commit_elect(&ms.p_empty[pb]);
                };
                // Event driven: PV(g) as soon as P(g) is published (it frees the tile for the gather), else
                // QK of the next tile as soon as it has landed, its S buffer is free and its Q is in place.
                int nq = 0, nv = 0;
                bool q_first = wq.seek(p, prefix, t_begin), v_first = wv.seek(p, prefix, t_begin);
                long long t_idle = clock64();
                uint32_t spins = 0;
                while (nv < n_total) {
                    bool pv_ready = nv < nq && mbar_try_nb(&ms.p_full[nv & 1], (uint32_t)(nv / 2) & 1u);
                    // the first PV of a sequence overwrites O: the previous sequence's epilogue must have read it
                    if (pv_ready && v_first && wv.pair > 0) pv_ready = mbar_try_nb(&ms.o_free, (uint32_t)(wv.pair - 1) & 1u);
                    bool qk_ready = !pv_ready && nq < n_total &&
                                    mbar_try_nb(&ms.kv_full[nq % NS], (uint32_t)(nq / NS) & 1u) &&
                                    mbar_try_nb(&ms.s_empty[nq & 1], (uint32_t)(nq / 2 - 1) & 1u);
                    if (qk_ready && q_first) qk_ready = mbar_try_nb(&ms.q_full[wq.pair & 1], (uint32_t)(wq.pair / 2) & 1u);
                    // every lane takes the same decision: the elected-lane instructions below need a converged warp
                    pv_ready = __all_sync(0xffffffffu, pv_ready);
                    qk_ready = !pv_ready && __all_sync(0xffffffffu, qk_ready);
                    if (!pv_ready && !qk_ready && (++spins & 63u) == 0u) {
                        if (spins == 64u) t_idle = clock64();
                        const bool give_up = *abort_flag || clock64() - t_idle > WAIT_LIMIT_CYCLES;
                        if (__any_sync(0xffffffffu, give_up)) {
                            *abort_flag = 1;        // give up waiting; issue the rest regardless so that every commit still arrives
                            if (nq < n_total) qk_ready = true; else pv_ready = true;
                        }
                    }
                    __syncwarp();
                    if (pv_ready) {
                        issue_pv(nv, v_first);
                        ++nv; spins = 0;
                        if (nv < n_total) v_first = wv.seek(p, prefix, t_begin + nv);
                    } else if (qk_ready) {
                        issue_qk(nq);
                        ++nq; spins = 0;
                        if (nq < n_total) q_first = wq.seek(p, prefix, t_begin + nq);
                    }
                }
            }
        } else {
            // =========================== softmax / correction / epilogue (128 threads) ===========
            const float score_scale = p.sm_scale * LOG2E * q_sc * kv_sc;
            const float out_scale = kv_sc;
            const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
            Walker wk; wk.init_at(b_begin);
            // nm[c] = P_SCALE_LOG2 - (reference maximum of column c); +inf while the column has seen no key
            float nm[N], l_acc[N];
            // token position pos is visible to the rows of 16-column chunk q iff pos < lim[q]
            // (heads is a multiple of 16, so the query index j is constant inside a chunk)
            int lim[N / 16], lim_min = 0;
            for (int g = 0; g < n_total; ++g) {
                const int sb = g & 1;
                const bool first = wk.seek(p, prefix, t_begin + g);
                const bool last = t_begin + g + 1 == min(t_end, wk.seq_t1);
                const int pos_first = (t_begin + g - wk.seq_t0) * TILE;
                if (first) {
#pragma unroll
                    for (int c = 0; c < N; ++c) { nm[c] = INFINITY; l_acc[c] = 0.0f; }
                    lim_min = 0x7fffffff;
#pragma unroll
                    for (int q = 0; q < N / 16; ++q) {
                        const int j = (row0 + 16 * q) / p.heads;
                        const int causal_lim = p.causal ? (wk.tot_len - p.q_len + j + 1 - wk.pos_off) : 0x7fffffff;
                        lim[q] = min(wk.seq_len, causal_lim);
                        lim_min = min(lim_min, lim[q]);
                    }
                }
                mbar_wait(&ms.s_full[sb], g / 2, abort_flag);
                tc_fence_after();
                float s[N];
#pragma unroll
                for (int c0 = 0; c0 < N; c0 += 16) tmem_ld16(tmem + lane_base + L::TMEM_S + sb * N + c0, s + c0);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(&ms.s_empty[sb]);

                // x = log2-domain exponent of the stored probability: score*scale - m_ref + P_SCALE_LOG2
                const int pos = tid < TILE ? pos_first + tid : 0x7fffffff;           // lanes beyond the tile: always masked
                const bool masked_tile = TILE < MMA_M || pos_first + TILE > lim_min; // uniform
                float x[N];
#pragma unroll
                for (int c = 0; c < N; ++c) x[c] = fmaf(s[c], score_scale, nm[c]);
                if (masked_tile) {
#pragma unroll
                    for (int c = 0; c < N; ++c) if (pos >= lim[c / 16]) x[c] = -INFINITY;
                }
                float xm = x[0];
#pragma unroll
                for (int c = 1; c < N; ++c) xm = fmaxf(xm, x[c]);
                const bool recenter = named_bar_or(1, 128, xm > P_SCALE_LOG2 + RECENTER);
                uint8_t* pbuf = smem + L::OFF_P + sb * L::P_BUF_BYTES;
                if (recenter) {
                    // this tile's P buffer (free once PV(g-2) has completed) is the scratch area of the column reduction
                    mbar_wait(&ms.p_empty[sb], g / 2 - 1, abort_flag);
                    float mx[N];
#pragma unroll
                    for (int c = 0; c < N; ++c) mx[c] = (masked_tile && pos >= lim[c / 16]) ? -INFINITY : s[c] * score_scale;
                    reduce_cols_128_scratch<N, true, 2>(mx, reinterpret_cast<float*>(pbuf), &ms.red[0][0], tid, 1);
                    float f[N];
                    bool any = false;
#pragma unroll
                    for (int c = 0; c < N; ++c) {
                        const float m_old = P_SCALE_LOG2 - nm[c];                     // -inf for a fresh column
                        const float m_new = fmaxf(m_old, mx[c]);
                        f[c] = (m_new == m_old) ? 1.0f : (m_old == -INFINITY ? 0.0f : ex2(m_old - m_new));
                        any |= f[c] != 1.0f;
                        nm[c] = P_SCALE_LOG2 - m_new;
                        l_acc[c] *= f[c];
                        x[c] = (masked_tile && pos >= lim[c / 16]) ? -INFINITY : fmaf(s[c], score_scale, nm[c]);
                    }
                    if (!first && any) {
                        // O holds the sequence's earlier tiles once PV(g-1) has completed; nothing else touches it until P(g) is published
                        mbar_wait(&ms.p_empty[(g - 1) & 1], (g - 1) / 2, abort_flag);
                        tc_fence_after();
#pragma unroll 1
                        for (int jb = 0; jb < 4; ++jb) {                              // rare path: kept small, not unrolled
#pragma unroll
                            for (int c0 = 0; c0 < 2 * N; c0 += 16) {
                                float o[16];
                                const uint32_t addr = tmem + lane_base + L::TMEM_O + jb * 2 * N + c0;
                                tmem_ld16(addr, o);
                                tmem_wait_ld();
#pragma unroll
                                for (int c = 0; c < 16; ++c) o[c] *= f[(c0 + c) % N];
                                tmem_st16(addr, o);
                            }
                        }
                        tmem_wait_st();
                        tc_fence_before();
                    }
                }
                // P(g) may overwrite its buffer once PV(g-2) has completed
                mbar_wait(&ms.p_empty[sb], g / 2 - 1, abort_flag);
#pragma unroll
                for (int c0 = 0; c0 < N; c0 += 16) {
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        float pv[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int c = c0 + q4 * 4 + k;
                            pv[k] = ex2(x[c]);                                        // ex2(-inf) = 0 for masked keys
                            l_acc[c] += pv[k];
                        }
                        hi[q4] = pack_e4m3x4(pv[0], pv[1], pv[2], pv[3]);
                        const float2 h01 = unpack_e4m3x2((uint16_t)(hi[q4] & 0xffffu)), h23 = unpack_e4m3x2((uint16_t)(hi[q4] >> 16));
                        lo[q4] = pack_e4m3x4((pv[0] - h01.x) * 16.0f, (pv[1] - h01.y) * 16.0f,
                                             (pv[2] - h23.x) * 16.0f, (pv[3] - h23.y) * 16.0f);
                    }
                    *reinterpret_cast<uint4*>(pbuf + (c0 / 16) * (MMA_M * 16) + tid * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(pbuf + ((N + c0) / 16) * (MMA_M * 16) + tid * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
                fence_proxy_async();
                mbar_arrive(&ms.p_full[sb]);

                if (last) {
                    // ---- epilogue of this (CTA, sequence) pair: wait for its last PV, normalise, write out
                    mbar_wait(&ms.p_empty[sb], g / 2, abort_flag);
                    tc_fence_after();
                    reduce_cols_128_scratch<N, false, 2>(l_acc, reinterpret_cast<float*>(pbuf), &ms.red[0][0], tid, 1);   // PV(g) is done: P buffer free
                    const bool whole = (t_begin <= wk.seq_t0) && (wk.seq_t1 <= t_end);
                    const int slot = w + wk.b;
                    float inv[N];
#pragma unroll
                    for (int c = 0; c < N; ++c) inv[c] = l_acc[c] > 0.0f ? __fdividef(out_scale, l_acc[c]) : 0.0f;
                    // one output element per (row, dim): this thread owns dims tid, 128+tid, ... of every row
                    const long long orow0 = whole ? ((long long)wk.b * p.rows + row0) : ((long long)slot * p.rows + row0);
                    float* dst_f32 = whole ? p.out_o_f32 : p.part_o;
                    __nv_bfloat16* dst_bf16 = whole ? p.out : nullptr;
                    if (dst_f32) dst_f32 += orow0 * V_DIM + tid;
                    if (dst_bf16) dst_bf16 += orow0 * V_DIM + tid;
#pragma unroll 1
                    for (int jb = 0; jb < 4; ++jb) {                                  // once per sequence: code size before speed
#pragma unroll
                        for (int c0 = 0; c0 < N; c0 += 16) {
                            float ohi[16], olo[16];
                            tmem_ld16(tmem + lane_base + L::TMEM_O + jb * 2 * N + c0, ohi);
                            tmem_ld16(tmem + lane_base + L::TMEM_O + jb * 2 * N + N + c0, olo);
                            tmem_wait_ld();
#pragma unroll
                            for (int c = 0; c < 16; ++c) ohi[c] = fmaf(olo[c], 0.0625f, ohi[c]) * inv[c0 + c];
                            if (dst_bf16) {
#pragma unroll
                                for (int c = 0; c < 16; ++c) dst_bf16[(c0 + c) * V_DIM + jb * 128] = __float2bfloat16_rn(ohi[c]);
                            }
                            if (dst_f32) {
#pragma unroll
                                for (int c = 0; c < 16; ++c) dst_f32[(c0 + c) * V_DIM + jb * 128] = ohi[c];
                            }
                        }
                    }
                    // O has been read: the next sequence's first PV may overwrite it
                    tc_fence_before();
                    mbar_arrive(&ms.o_free);
                    if (tid < N) {
                        float lsum = 0.0f, nmc = 0.0f;
#pragma unroll
                        for (int c = 0; c < N; ++c) if (c == tid) { lsum = l_acc[c]; nmc = nm[c]; }
                        const float lse = lsum > 0.0f ? (log2f(lsum) - nmc) * LN2 : -INFINITY;
                        if (whole) { if (p.out_lse) p.out_lse[(long long)wk.b * p.rows + row0 + tid] = lse; }
                        else p.part_lse[(long long)slot * p.rows + row0 + tid] = lse;
                    }
                }
            }
        }
    }

    __syncthreads();
    if (tid == 0 && ms.abort_flag) atomicOr(status, (int)ST_TIMEOUT);
    if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem, L::TMEM_COLS); }
}

}  // namespace sm100

int sm100_rows_per_cta(const MlaParams& p) { return p.rows % 32 == 0 ? 32 : 16; }
int sm100_tile_tokens(const MlaParams& p) { return sm100_rows_per_cta(p) == 32 ? sm100::Layout<32>::TILE : sm100::Layout<16>::TILE; }

template <int N>
static size_t smem_need(int batch) {
    return (size_t)sm100::Layout<N>::OFF_MISC + sizeof(sm100::Misc) + (size_t)(batch + 1) * sizeof(int);
}

bool sm100_supported(const MlaParams& p) {
    if (p.kv_format != KV_E4M3 || p.q_format != Q_E4M3 || p.rows % 16 != 0) return false;
    // the tile-prefix table shares the tail of shared memory with the stages
    const size_t need = sm100_rows_per_cta(p) == 32 ? smem_need<32>(p.batch) : smem_need<16>(p.batch);
    return need <= (size_t)sm100::SMEM_LIMIT;
}

// Tensor map over the cache plane [num_slots rows x 576 bytes] with a box of `box_bytes` x `box_rows`; false if the
// driver entry point is missing or refuses the arguments (the caller then keeps the copy loop).
static bool make_cache_map(CUtensorMap* map, const MlaParams& p, int box_bytes, int box_rows, CUtensorMapSwizzle swizzle) {
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn encode = nullptr;
    static bool looked_up = false;
    if (!looked_up) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            encode = (encode_fn)fn;
        looked_up = true;
    }
    if (!encode) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)QK_DIM, (cuuint64_t)p.num_slots};
    const cuuint64_t strides[1] = {(cuuint64_t)p.kv_codes_stride};
    const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(p.kv_codes), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int N>
static cudaError_t launch_n(const MlaParams& p, int* status, cudaStream_t stream) {
    using L = sm100::Layout<N>;
    const size_t smem = smem_need<N>(p.batch);
    auto kernel = p.q_cast ? sm100::mla_decode_sm100_kernel<N, true> : sm100::mla_decode_sm100_kernel<N, false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    // contiguous cache: tiled TMA for the tiles (this GPU's own cache plane only; no multi-CTA delivery of any kind)
    // The maps depend on the plane's address, row count and stride only; the last few are kept per host thread, so a
    // serving loop that decodes from the same cache does not pay the two driver calls (~3 us) on every call.
    struct MapEntry { const void* base; long long slots, stride; int tile, ok; CUtensorMap lat, rope; };
    static thread_local MapEntry cache[4] = {};
    static thread_local int next = 0;
    CUtensorMap lat, rope;
    memset(&lat, 0, sizeof(lat));
    memset(&rope, 0, sizeof(rope));
    int use_tma = 0;
    const char* off = getenv("B200_MLA_DISABLE_TMA");                 // testing aid: "1" keeps every tile on the copy loop
    if (!(off && off[0] == '1') && ((uintptr_t)p.kv_codes & 15) == 0 && p.kv_codes_stride % 16 == 0 &&
        p.kv_codes_stride >= QK_DIM && p.num_slots > 0 && p.num_slots < (1LL << 31)) {
        // contiguous cache: boxes of a whole tile; page table: boxes of one row, fetched four at a time by row index
        const int box_rows = p.kv_indices == nullptr ? L::TILE : 1;
        MapEntry* hit = nullptr;
        for (MapEntry& m : cache)
            if (m.base == p.kv_codes && m.slots == p.num_slots && m.stride == p.kv_codes_stride && m.tile == box_rows) hit = &m;
        if (!hit) {
            hit = &cache[next];
            next = (next + 1) % 4;
            hit->base = p.kv_codes; hit->slots = p.num_slots; hit->stride = p.kv_codes_stride; hit->tile = box_rows;
            hit->ok = make_cache_map(&hit->lat, p, 128, box_rows, CU_TENSOR_MAP_SWIZZLE_128B) &&
                      make_cache_map(&hit->rope, p, 64, box_rows, CU_TENSOR_MAP_SWIZZLE_64B);
        }
        use_tma = hit->ok ? (p.kv_indices == nullptr ? 1 : 2) : 0;
        if (use_tma) { lat = hit->lat; rope = hit->rope; }
    }
    dim3 grid(p.num_ctas, p.rows / N);
    kernel<<<grid, L::THREADS, smem, stream>>>(p, status, lat, rope, use_tma);
    return cudaGetLastError();
}

cudaError_t launch_sm100(const MlaParams& p, int* status, cudaStream_t stream) {
    return p.rows_per_cta == 32 ? launch_n<32>(p, status, stream) : launch_n<16>(p, status, stream);
}

}  // namespace b200mla
