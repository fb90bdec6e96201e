// tcgen05 / TMEM stage-1 MLA decode for the cache / query formats that need a pass over the data
// before the tensor cores can take it: MXFP4 and hybrid caches (e2m1 codes + E8M0 block scales
// become e4m3 operands) and bf16 queries (split into two e4m3 terms).  Same swap-AB formulation,
// schedule, softmax and pipeline as mla_decode_sm100.cu (FP8 Q x FP8 KV), plus:
//
//  * "transform" warps.  For a block-scaled cache each transform warp fetches the raw codes and E8M0
//    bytes of 16 tokens at a time (a unit) into a landing buffer of its own, and turns every 32-code
//    block of a landed unit into 32 e4m3 bytes of the swizzled operand tile.  All blocks of a unit
//    share one exponent frame: byte value = e2m1 * 2^(scale - E_unit + 6) with E_unit the largest
//    E8M0 byte of the unit, which is exact in e4m3 for blocks up to 14 binades below the largest.
//    The softmax thread of a token applies 2^(E_unit - 133) to its scores and 2^(E_unit - E_run) to
//    its probabilities, E_run being the frame O is held in (O is rescaled in TMEM when a later tile
//    has a larger frame, like the softmax re-centering).
//  * bf16 Q: a small kernel ahead of this one writes every group of N query rows as Q = (hi + lo/16) / s
//    with hi, lo in e4m3 and s a power of two per group; the QK MMA then has 2N columns and the
//    softmax adds the two halves.  (No tensor-core kind mixes bf16 with fp8 / fp4 operands.)
//  * hybrid cache: the 64 rope dims are e4m3 with a per-tensor scale that is not a power of two,
//    so their QK k-steps accumulate into a second set of TMEM columns and the softmax adds
//    a_lat * S_lat + a_rope * S_rope.  The rope bytes go from HBM straight into the operand tile.
//
// Operand tile: four 128-byte-wide panels (dims 0..511, 128B swizzle; read K-major by QK and MN-major
// by PV) and one 64-byte-wide panel (dims 512..575, 64B swizzle; QK only).
// Roles: warps 0-3 softmax / epilogue, warp 4 MMA issue, then PW gather warps (the whole tile for an e4m3 cache;
// only Q and the hybrid rope bytes next to transform warps), then XW transform warps.
// Role in the reference: the MXFP4 split-KV stage-1 kernels (mixed-mla/submission.py:122-250,
// mixed-mla/versions/hip_mxfp4_v5/submission.py:214-656) and their block decode
// (mixed-mla/triton_mla_mxfp4.py:20-67).
#include "sm100_ptx.cuh"

namespace b200mla {
namespace sm100x {

using namespace sm100;

constexpr int TILE = 128;                 // tokens per tile = UMMA M
constexpr int UNIT_TOK = 16;              // tokens per raw unit
constexpr int NS = 2;                     // operand tile stages
constexpr int PANEL_BYTES = TILE * 128;
constexpr int ROPE_PANEL_BYTES = TILE * 64;
constexpr int STAGE_BYTES = 4 * PANEL_BYTES + ROPE_PANEL_BYTES;    // 72 KB
constexpr int SMEM_LIMIT = 232448;        // opt-in shared memory per CTA
constexpr float RECENTER = 4.0f;          // log2 units
constexpr float P_SCALE_LOG2 = 4.0f;      // probabilities are stored multiplied by 2^4
constexpr int E_BIAS = 127 + 6;           // operand bytes of a block-scaled unit are in units of 2^(E_unit - E_BIAS)

template <int N, int KVFMT, int QFMT>
struct Cfg {
    static constexpr bool QSPLIT = QFMT == Q_BF16;
    static constexpr bool XF = KVFMT != KV_E4M3;
    static constexpr bool ROPE_SEP = KVFMT == KV_HYBRID;
    static constexpr int NQ = N * (QSPLIT ? 2 : 1);               // Q rows in shared memory = columns of one S accumulator
    static constexpr int SC = NQ * (ROPE_SEP ? 2 : 1);            // S columns per buffer
    // with transform warps the gather role only moves Q and rope bytes; N = 32 runs 3 warps per scheduler either
    // way (registers are handed out per scheduler), so a hybrid cache's rope gather gets the two spare warps
    static constexpr int PW = XF ? 1 : (N == 16 ? 8 : 4);
    static constexpr int PRODUCERS = 32 * PW;
    // N = 64: two softmax warpgroups of 128 threads, each with 32 of the 64 query rows (warps w and w + 4 reach the same
    // TMEM lanes), so that a tile is gathered, converted and multiplied once for 64 rows with the softmax cost of 32.
    static constexpr int SMG = N == 64 ? 2 : 1;                   // softmax warpgroups
    static constexpr int NC = N / SMG;                            // query rows (S / O columns) per softmax thread
    static constexpr int SW = 4 * SMG;                            // softmax warps; warp SW issues the MMAs
    static constexpr int FIRST_PRODUCER = 32 * (SW + 1);
    // N = 64: P_hi and P_lo are two k-steps into the SAME O columns (O = 4 x N columns; with them side by side O alone
    // would fill the 512 TMEM columns), P_lo is then stored unscaled, and P is single buffered (shared memory).
    static constexpr bool MERGED = N == 64;
    static constexpr int OB = MERGED ? N : 2 * N;                 // TMEM columns of one O block
    static constexpr int P_BUFS = MERGED ? 1 : 2;
    static constexpr int NB = KVFMT == KV_MXFP4 ? 18 : 16;        // 32-code blocks per cache row
    static constexpr int RAW_ROW = NB * 16;                       // bytes of codes per row
    static constexpr int PITCH = RAW_ROW + 16;                    // row pitch in a landing buffer: eight rows hit eight bank groups
    static constexpr int OFF_UNIT_SCALES = UNIT_TOK * PITCH;      // 24 bytes per row: the aligned words around its E8M0 bytes
    static constexpr int UNIT_BYTES = OFF_UNIT_SCALES + UNIT_TOK * 24;
    static constexpr int Q_PANEL_BYTES = NQ * 128;
    static constexpr int Q_BYTES = NQ * QK_DIM;                   // four 128B-swizzled panels and one 64B-swizzled
    static constexpr int P_CHUNKS = 2 * N / 16;
    static constexpr int P_BUF_BYTES = P_CHUNKS * TILE * 16;
    static constexpr int MISC_RESERVE = 4096;                     // Misc + the tile prefix of ~700 sequences
    static constexpr int FIXED = NS * STAGE_BYTES + Q_BYTES + P_BUFS * P_BUF_BYTES + MISC_RESERVE;
    // Landing buffers of the transform warps: S per warp, private to it.  The 16-token units of the tile stream go to
    // the transform warps round robin, so any number of them works: as many as have a landing buffer, eight at most
    // (32 rows: five or six instead of four, 2.8 % on the 131072-key shape); four for 64 rows, where six were
    // measured 6 % slower (the two softmax warpgroups already fill the schedulers).
    static constexpr int RB_FIT = XF ? (SMEM_LIMIT - FIXED) / UNIT_BYTES : 0;
    static constexpr int XW_MAX = (N == 16 || (N == 32 && ROPE_SEP && !QSPLIT)) ? 8 : (N == 64 ? 4 : 6);
    static constexpr int XW = !XF ? 0 : (RB_FIT < XW_MAX ? RB_FIT : XW_MAX);
    static constexpr int XT = 32 * XW;
    static constexpr int THREADS = FIRST_PRODUCER + PRODUCERS + XT;
    static constexpr int S = !XF ? 0 : (RB_FIT >= 2 * XW ? 2 : 1);
    static constexpr int RB = XW * S;
    static constexpr int OFF_Q = NS * STAGE_BYTES;
    static constexpr int OFF_P = OFF_Q + Q_BYTES;
    static constexpr int OFF_RAW = OFF_P + P_BUFS * P_BUF_BYTES;
    static constexpr int OFF_MISC = OFF_RAW + RB * UNIT_BYTES;
    static constexpr int TMEM_O = 2 * SC;
    static constexpr int TMEM_NEED = 2 * SC + 4 * OB;
    static constexpr int TMEM_COLS = TMEM_NEED <= 128 ? 128 : (TMEM_NEED <= 256 ? 256 : 512);
    // rows of a stage handed back to the transform warps after each PV token step instead of after the whole PV:
    // worth 2-4 % for the pure MXFP4 cache; not for the hybrid one, whose rope gather waits for the whole stage anyway
    static constexpr bool ROWS_EARLY = XF && !ROPE_SEP;
    // a transform warp arrives once per unit it has stored (eight units per tile, whoever stores them)
    static constexpr int KV_FULL_COUNT = XF ? 32 * (TILE / UNIT_TOK) + (ROPE_SEP ? PRODUCERS : 0) : PRODUCERS;
    static_assert(TMEM_NEED <= 512, "TMEM columns");
    static_assert(N != 64 || !QSPLIT, "64 rows per CTA: e4m3 Q only");
    static_assert(!XF || (XW >= 1 && RB_FIT >= XW), "landing buffers");
    static_assert(THREADS <= 512 || N != 64, "the 64-row variant needs 128 registers per thread");
    static_assert((UNIT_TOK * NB) % 32 == 0 && UNIT_BYTES % 16 == 0, "unit layout");
};

struct Misc {
    uint64_t kv_full[NS], kv_empty[NS], s_full[2], s_empty[2], p_full[2], p_empty[2];
    uint64_t kv_rows_free[NS][4];   // tokens 32q..32q+31 of a stage have been read for the last time (PV k-step q done)
    uint64_t q_full, q_empty, o_free;
    uint32_t tmem_base;
    int abort_flag;
    unsigned int q_amax;         // block_q_scale's word
    int tile_exp[NS][TILE / UNIT_TOK];   // exponent frame of each 16-token unit of the tile in each operand stage
    int slot[NS][TILE];
    __align__(16) float red[2][4][32];   // softmax cross-warp exchange, per softmax warpgroup
    float nm[2][2][32];          // P_SCALE_LOG2 - reference maximum per query row: [warpgroup][double buffer][row]
};

// 2^e as a float; 0 below the normal range
__device__ __forceinline__ float pow2i(int e) {
    return e < -126 ? 0.0f : __int_as_float((min(e, 127) + 127) << 23);
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// 32 e2m1 codes (one uint4, even element in the low nibble) -> 32 e4m3 bytes, value = code * 2^k, k <= 6.
// Magnitudes: a byte permute through the 8-entry table of this block's k.  For k >= -5 every non-zero entry is a
// normal e4m3 number, i.e. the k = 0 bytes plus 8k; below that the table comes from the rounding conversion
// (entries that e4m3 cannot hold exactly are rounded or flushed).  Signs: a byte permute in sign-replication
// mode turns nibble bit 3 (of the code word and of the word shifted by 4) into 0xff / 0x00 bytes.
__device__ __forceinline__ void dequant_block(const uint4& v, int k, uint4& lo, uint4& hi) {
    uint32_t t0, t1;
    if (k >= -5) {
        t0 = 0x3C383000u + (uint32_t)(k * 0x08080800);           // 0, .5, 1, 1.5
        t1 = 0x4C484440u + (uint32_t)(k * 0x08080808);           // 2, 3, 4, 6
    } else {
        const float sc = pow2i(max(k, -40));
        t0 = pack_e4m3x4(0.0f, 0.5f * sc, sc, 1.5f * sc);
        t1 = pack_e4m3x4(2.0f * sc, 3.0f * sc, 4.0f * sc, 6.0f * sc);
    }
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t m = w[i] & 0x77777777u, w4 = w[i] << 4;
        o[2 * i] = prmt(t0, t1, m) | (prmt(w4, w[i], 0xD9C8u) & 0x80808080u);
        o[2 * i + 1] = prmt(t0, t1, m >> 16) | (prmt(w4, w[i], 0xFBEAu) & 0x80808080u);
    }
    lo = make_uint4(o[0], o[1], o[2], o[3]);
    hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// byte offset inside an operand stage of the 16-byte column c (0..35) of token tok
__device__ __forceinline__ uint32_t operand_offset(int tok, int c) {
    return c < 32 ? (uint32_t)((c >> 3) * PANEL_BYTES + tok * 128 + (((c & 7) ^ (tok & 7)) << 4))
                  : (uint32_t)(4 * PANEL_BYTES + tok * 64 + (((c - 32) ^ ((tok >> 1) & 3)) << 4));
}

template <int N, int KVFMT, int QFMT>
__global__ void __launch_bounds__(Cfg<N, KVFMT, QFMT>::THREADS, 1) mla_decode_sm100x_kernel(const MlaParams p, int* status) {
    using C = Cfg<N, KVFMT, QFMT>;
    constexpr int PRODUCERS = C::PRODUCERS, THREADS = C::THREADS, NQ = C::NQ;
    extern __shared__ __align__(1024) unsigned char smem[];
    Misc& ms = *reinterpret_cast<Misc*>(smem + C::OFF_MISC);
    int* prefix = reinterpret_cast<int*>(smem + C::OFF_MISC + sizeof(Misc));
    const uint32_t smem_base = smem_u32(smem);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int w = blockIdx.x, G = p.num_ctas;
    const int row0 = blockIdx.y * N;
    const unsigned int q_amax_local = block_q_amax_begin(p.q_amax_parts, QFMT == Q_E4M3 ? p.q_cast : 0);   // loads in flight during the prologue
    const float kv_tensor_scale = KVFMT != KV_MXFP4 ? __ldg(p.kv_scale) : 1.0f;   // issued here, first used by the softmax role

    if (tid == 0) {
        for (int i = 0; i < NS; ++i) {
            mbar_init(&ms.kv_full[i], C::KV_FULL_COUNT); mbar_init(&ms.kv_empty[i], 1);
            for (int q = 0; q < 4; ++q) mbar_init(&ms.kv_rows_free[i][q], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ms.s_full[i], 1); mbar_init(&ms.s_empty[i], 128 * C::SMG);
            mbar_init(&ms.p_full[i], 128 * C::SMG); mbar_init(&ms.p_empty[i], 1);
        }
        mbar_init(&ms.q_full, PRODUCERS); mbar_init(&ms.q_empty, 1);
        mbar_init(&ms.o_free, 128 * C::SMG);
        ms.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == C::SW) { tmem_alloc(&ms.tmem_base, C::TMEM_COLS); tmem_relinquish(); }
    build_tile_prefix(p.kv_indptr, p.batch, TILE, prefix);       // ends with __syncthreads()
    tc_fence_after();
    const uint32_t tmem = ms.tmem_base;
    const int TT = prefix[p.batch];
    if (w == 0 && blockIdx.y == 0)
        for (int i = tid; i <= p.batch; i += THREADS) p.tile_prefix[i] = prefix[i];

    const int t_begin = TT > 0 ? span_begin(prefix, p.batch, w, G) : 0, t_end = TT > 0 ? span_begin(prefix, p.batch, w + 1, G) : 0;
    const int n_total = t_end - t_begin;                          // tiles of this CTA; tile index g = 0..n_total-1
    const float q_tensor_scale = QFMT == Q_E4M3 ? block_q_scale(q_amax_local, p.q_scale, p.q_cast, &ms.q_amax) : 1.0f;
    volatile int* abort_flag = &ms.abort_flag;

    if (n_total > 0) {
        if (warp >= C::SW + 1 && warp < C::SW + 1 + C::PW) {
            // =========================== gather ===========================
            const int pt = tid - C::FIRST_PRODUCER;
            Walker wk; wk.init(prefix, p.batch, t_begin);
            Walker wn = wk;                                       // one tile ahead, for the page-table prefetch
            bool bad_page = false;
            constexpr int SLOTS_PER_THREAD = (TILE + PRODUCERS - 1) / PRODUCERS;
            int my_slot[SLOTS_PER_THREAD];
            auto slots_for = [&](int g) {
                if (g < n_total) wn.seek(p, prefix, t_begin + g);
#pragma unroll
                for (int k = 0; k < SLOTS_PER_THREAD; ++k) {
                    const int tok = pt + k * PRODUCERS;
                    const int pos = (t_begin + g - wn.seq_t0) * TILE + tok;
                    my_slot[k] = (g < n_total && tok < TILE && pos < wn.seq_len)
                                     ? (int)slot_of(p, wn.b, wn.seq_base, wn.page_base, pos) : -1;
                }
            };
            // Copies `ncols` 16-byte columns of the rows [tok0, tok0 + ntok) of the tile in stage st: column c of a
            // row comes from src_base + slot * stride + 16c and goes to dst_of(tok, c).  Consecutive threads take
            // consecutive columns.  Rows past the end of the sequence are zero filled.
            auto gather = [&](int st, int tok0, int ntok, int ncols, const uint8_t* src_base, long long stride, auto dst_of) {
                const int total = ntok * ncols;
                for (int id0 = pt; id0 < total; id0 += 16 * PRODUCERS) {   // batches of 16: slots first, then the copies
                    int sl[16];
#pragma unroll
                    for (int u = 0; u < 16; ++u) {
                        const int id = id0 + u * PRODUCERS;
                        sl[u] = id < total ? ms.slot[st][tok0 + id / ncols] : -2;
                    }
#pragma unroll
                    for (int u = 0; u < 16; ++u) {
                        const int id = id0 + u * PRODUCERS;
                        if (sl[u] != -2) {
                            const int tr = id / ncols, c = id - tr * ncols;
                            const uint8_t* src = src_base + (long long)clamp_slot(p, sl[u]) * stride + c * 16;
                            cp_async16(dst_of(tok0 + tr, c), src, sl[u] < 0 ? 0u : 16u);
                        }
                    }
                }
            };
            constexpr bool NEED_SLOTS = !C::XF || C::ROPE_SEP;        // does this role copy cache rows at all
            if (NEED_SLOTS) slots_for(0);
            for (int g = 0; g < n_total; ++g) {
                const int st = g % NS;
                const bool first = wk.seek(p, prefix, t_begin + g);
                if (NEED_SLOTS) {
                    // the gather threads are the only users of the slot table: the barrier pair orders the rewrite of
                    // stage st's entries after every thread's reads for tile g - NS
                    named_bar_sync(2, PRODUCERS);
#pragma unroll
                    for (int k = 0; k < SLOTS_PER_THREAD; ++k)
                        if (pt + k * PRODUCERS < TILE) {
                            ms.slot[st][pt + k * PRODUCERS] = my_slot[k];
                            // reporting (see clamp_slot): looked at here, where the id has arrived anyway, never at its load
                            bad_page |= my_slot[k] != -1 && (unsigned int)my_slot[k] > p.last_slot;      // -1: no row (past the end)
                        }
                    named_bar_sync(2, PRODUCERS);
                    slots_for(g + 1);
                }
                const uint32_t stage_addr = smem_base + st * STAGE_BYTES;
                if (!C::XF) {
                    mbar_wait(&ms.kv_empty[st], g / NS - 1, abort_flag);
                    gather(st, 0, TILE, 36, p.kv_codes, p.kv_codes_stride,
                           [&](int tok, int c) { return stage_addr + operand_offset(tok, c); });
                    cp_async_mbar_arrive_noinc(&ms.kv_full[st]);
                } else {
                    // the codes and E8M0 bytes are fetched by the transform warps themselves
                    if (C::ROPE_SEP) {                           // rope bytes are e4m3 already: straight into the rope panel
                        mbar_wait(&ms.kv_empty[st], g / NS - 1, abort_flag);
                        gather(st, 0, TILE, 4, p.kv_rope, p.kv_rope_stride,
                               [&](int tok, int c) { return stage_addr + operand_offset(tok, 32 + c); });
                        cp_async_mbar_arrive_noinc(&ms.kv_full[st]);
                    }
                }
                if (first) {
                    // Q rows of the new sequence -> swizzled K-major panels.  Issued after the tile so that the wait for
                    // the previous sequence's last QK does not hold the cache stream back.
                    mbar_wait(&ms.q_empty, wk.pair - 1, abort_flag);
                    const uint32_t q_addr = smem_base + C::OFF_Q;
                    const long long plane = (long long)p.batch * p.rows * QK_DIM;   // split Q: hi plane, then lo plane
                    if (!C::QSPLIT && p.q_cast) {
                        // bf16 rows, quantised here: eight values in, eight e4m3 bytes (half a 16-byte column) out
                        unsigned char* q_smem = smem + C::OFF_Q;
                        // eight loads in flight per thread, then their conversion (a few gather threads serve many rows)
                        for (int i0 = pt; i0 < N * 72; i0 += 8 * PRODUCERS) {
                            uint4 raw[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int i = i0 + u * PRODUCERS;
                                if (i < N * 72) {
                                    const int r = i / 72, v8 = i - r * 72;
                                    const int rg = row0 + r, j = rg / p.heads, h = rg - j * p.heads;
                                    raw[u] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.q) +
                                                   (long long)(wk.b * p.q_len + j) * p.q_row_stride + (long long)h * p.q_head_stride + v8 * 8));
                                }
                            }
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int i = i0 + u * PRODUCERS;
                                if (i < N * 72) {
                                    const int r = i / 72, v8 = i - r * 72, c = v8 >> 1;
                                    const int off = c < 32 ? (c >> 3) * C::Q_PANEL_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)
                                                           : 4 * C::Q_PANEL_BYTES + r * 64 + (((c - 32) ^ ((r >> 1) & 3)) << 4);
                                    *reinterpret_cast<uint2*>(q_smem + off + (v8 & 1) * 8) = q_cast_e4m3x8(raw[u], q_tensor_scale);
                                }
                            }
                        }
                        fence_proxy_async();                      // the MMA reads Q through the async proxy
                        mbar_arrive(&ms.q_full);
                    } else {
                    for (int i = pt; i < NQ * 36; i += PRODUCERS) {
                        const int r = i / 36, c = i - r * 36;
                        const uint8_t* src;
                        if (C::QSPLIT) {
                            const int rr = r % N;
                            src = p.q_split + (r / N) * plane + ((long long)wk.b * p.rows + row0 + rr) * QK_DIM + c * 16;
                        } else {
                            const int rg = row0 + r, j = rg / p.heads, h = rg - j * p.heads;
                            src = reinterpret_cast<const uint8_t*>(p.q) + (long long)(wk.b * p.q_len + j) * p.q_row_stride +
                                  (long long)h * p.q_head_stride + c * 16;
                        }
                        const uint32_t dst = c < 32 ? q_addr + (c >> 3) * C::Q_PANEL_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)
                                                    : q_addr + 4 * C::Q_PANEL_BYTES + r * 64 + (((c - 32) ^ ((r >> 1) & 3)) << 4);
                        cp_async16(dst, src, 16u);
                    }
                    cp_async_mbar_arrive_noinc(&ms.q_full);
                    }
                }
            }
            cp_async_wait_all();
            if (bad_page) atomicOr(p.status, (int)ST_BAD_PAGE);
        } else if (warp == C::SW) {
            // =========================== MMA issue (whole warp, one elected lane per instruction) ===========================
            {
                constexpr uint32_t IDESC_QK = make_idesc(TILE, NQ, false, false);
                constexpr uint32_t IDESC_PV = make_idesc(128, C::OB, true, true);
                // descriptor bases; per-MMA descriptors differ only in the start address
                const uint64_t d_qk_a = make_desc(smem_base, 16, 1024, SWIZZLE_128B);                              // + stage
                const uint64_t d_qk_a_rope = make_desc(smem_base + 4 * PANEL_BYTES, 16, 512, SWIZZLE_64B);         // + stage
                const uint64_t d_qk_b = make_desc(smem_base + C::OFF_Q, 16, 1024, SWIZZLE_128B);
                const uint64_t d_qk_b_rope = make_desc(smem_base + C::OFF_Q + 4 * C::Q_PANEL_BYTES, 16, 512, SWIZZLE_64B);
                const uint64_t d_pv_a = make_desc(smem_base, PANEL_BYTES, 1024, SWIZZLE_128B);                     // + stage
                const uint64_t d_pv_b = make_desc(smem_base + C::OFF_P, 128, TILE * 16, SWIZZLE_NONE);             // + buffer
                Walker wq, wv;                                    // the QK stream runs ahead of the PV stream
                wq.init(prefix, p.batch, t_begin);
                wv = wq;
                // S^T[128 tok x NQ] = K . Q^T for tile g; a hybrid cache keeps the rope dims in columns of their own.
                // QK_PARTS > 1 would issue it in pieces with PVs in between; measured slower (alternating the two MMA
                // shapes costs more than the PV gains), so it stays in one piece.
                constexpr int QK_PARTS = 1;
                static_assert(QK_PARTS == 1, "issue_qk issues the whole product");
                auto issue_qk = [&](int g, int part) {
                    const int st = g % NS, sb = g & 1;
                    if (part == 0) {
                        fence_proxy_async();   // cp.async wrote through the generic proxy; the MMA reads through the async proxy
                        tc_fence_after();
                    }
                    const uint32_t d_lat = tmem + sb * C::SC, d_rope = d_lat + (C::ROPE_SEP ? NQ : 0);
                    // panel by panel, the panel loop not unrolled: the issue code stays a few hundred bytes, which is what
                    // the first pass through it (instruction fetch, on every CTA's critical path) pays for
#pragma unroll 1
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_f8_elect(d_lat, desc_advance(d_qk_a, st * STAGE_BYTES + j * PANEL_BYTES + k * 32),
                                          desc_advance(d_qk_b, j * C::Q_PANEL_BYTES + k * 32), IDESC_QK, (j | k) ? 1u : 0u);
                    }
#pragma unroll
                    for (int k = 0; k < 2; ++k)
                        umma_f8_elect(d_rope, desc_advance(d_qk_a_rope, st * STAGE_BYTES + k * 32), desc_advance(d_qk_b_rope, k * 32),
                                      IDESC_QK, (!C::ROPE_SEP || k > 0) ? 1u : 0u);
                    if (part == QK_PARTS - 1) {
                        umma_commit_elect(&ms.s_full[sb]);
                        // last tile of this (CTA, sequence) pair: the Q buffer is free once these MMAs have run
                        if (t_begin + g + 1 == min(t_end, wq.seq_t1)) umma_commit_elect(&ms.q_empty);
                    }
                };
                // O^T += V^T P^T over the 128 tokens of tile g, four blocks of 128 dims
                auto issue_pv = [&](int g, bool first) {
                    const int st = g % NS, pb = g % C::P_BUFS;
                    tc_fence_after();
                    const uint64_t a0 = desc_advance(d_pv_a, st * STAGE_BYTES);
                    const uint64_t b0 = desc_advance(d_pv_b, pb * C::P_BUF_BYTES);
                    // token steps outside, dim blocks inside: after step kk nothing reads tokens 32kk..32kk+31 of the stage
                    // any more, and (ROWS_EARLY) the transform warps of those rows may write the tile after next.
                    // MERGED: the hi and the lo term of P are two k-steps into the same O columns (the lo chunks follow
                    // the hi chunks in the P buffer); otherwise they are the two halves of the MMA's 2N columns.
#pragma unroll 1
                    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                        for (int half = 0; half < (C::MERGED ? 2 : 1); ++half) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                umma_f8_elect(tmem + C::TMEM_O + j * C::OB, desc_advance(a0, j * PANEL_BYTES + kk * 32 * 128),
                                              desc_advance(b0, kk * 32 * 16 + half * (N / 16) * TILE * 16), IDESC_PV,
                                              (first && kk == 0 && half == 0) ? 0u : 1u);
                            }
                        }
                        if (C::ROWS_EARLY) umma_commit_elect(&ms.kv_rows_free[st][kk]);
                    }
                    umma_commit_elect(&ms.kv_empty[st]);
                    umma_commit_elect(&ms.p_empty[pb]);
                };
                // Event driven: PV(g) as soon as P(g) is published (it frees the tile for the next one), else
                // QK of the next tile as soon as it is in place, its S buffer is free and its Q has landed.
                int nq = 0, nv = 0, qk_part = 0;
                bool q_first = wq.seek(p, prefix, t_begin), v_first = wv.seek(p, prefix, t_begin);
                long long t_idle = clock64();
                uint32_t spins = 0;
                while (nv < n_total) {
                    bool pv_ready = nv < nq && mbar_try_nb(&ms.p_full[nv % C::P_BUFS], (uint32_t)(nv / C::P_BUFS) & 1u);
                    // the first PV of a sequence overwrites O: the previous sequence's epilogue must have read it
                    if (pv_ready && v_first && wv.pair > 0) pv_ready = mbar_try_nb(&ms.o_free, (uint32_t)(wv.pair - 1) & 1u);
                    bool qk_ready = !pv_ready && nq < n_total &&
                                    (qk_part > 0 ||
                                     (mbar_try_nb(&ms.kv_full[nq % NS], (uint32_t)(nq / NS) & 1u) &&
                                      mbar_try_nb(&ms.s_empty[nq & 1], (uint32_t)(nq / 2 - 1) & 1u) &&
                                      (!q_first || mbar_try_nb(&ms.q_full, (uint32_t)wq.pair & 1u))));
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
                        issue_qk(nq, qk_part);
                        spins = 0;
                        if (++qk_part == QK_PARTS) {
                            qk_part = 0;
                            ++nq;
                            if (nq < n_total) q_first = wq.seek(p, prefix, t_begin + nq);
                        }
                    }
                }
            }
        } else if (C::XF && warp >= C::SW + 1 + C::PW) {
            // =========================== transform (block-scaled caches) ===========================
            // The CTA's tiles are a stream of 16-token units (eight per tile); warp xw owns units xw, xw + XW, ... of
            // that stream (round robin, so XW need not divide eight) and S private landing buffers.  For each
            // unit it fetches the raw rows itself (16-byte cp.async of the codes, the aligned 8-byte words around the
            // E8M0 bytes; rows past the end of the sequence are zero filled), moves a landed unit into registers,
            // reuses the buffer for the unit S ahead at once, and then turns 32-code blocks into pairs of 16-byte
            // columns of the operand tile.  Lane = (row lane % 16, block parity lane / 16): a quarter warp stores the
            // same column of eight consecutive rows, which the swizzle spreads over all banks, and reads eight rows
            // whose padded pitch does the same.  Each unit has its own exponent frame: its largest E8M0 byte.
            constexpr int NBH = C::NB / 2;                                // blocks per lane per unit
            constexpr int UNITS = TILE / UNIT_TOK, XWN = C::XW > 0 ? C::XW : 1;   // units per tile; stride of this warp's units
            constexpr int S = C::S > 0 ? C::S : 1;
            constexpr int CODE_IT = UNIT_TOK * C::NB / 32, PER = CODE_IT + 2;   // copy instructions per lane per unit: codes, E8M0 words
            const int xw = warp - C::SW - 1 - C::PW;
            const int tok = lane & (UNIT_TOK - 1), par = lane >> 4;
            const int J = (n_total * UNITS - xw + XWN - 1) / XWN;         // units of this warp (xw < UNITS <= n_total * UNITS)
            Walker wn; wn.init(prefix, p.batch, t_begin);
            // cache slot of row `tok` of this warp's unit j; -1 past the end of the sequence or of the span
            auto fetch_slot = [&](int j) -> int {
                if (j >= J) return -1;
                const int u = xw + j * XWN, g = u / UNITS, k = u - g * UNITS;
                wn.seek(p, prefix, t_begin + g);
                const int pos = (t_begin + g - wn.seq_t0) * TILE + k * UNIT_TOK + tok;
                return pos < wn.seq_len ? (int)slot_of(p, wn.b, wn.seq_base, wn.page_base, pos) : -1;
            };
            // lane constants: where block par + 2i of row tok goes in unit 0 of an operand stage, and which
            // (row, 16-byte column) each copy instruction of this lane moves (consecutive lanes, consecutive columns)
            uint32_t st_off[NBH], cp_pk[CODE_IT];
#pragma unroll
            for (int i = 0; i < NBH; ++i) st_off[i] = operand_offset(tok, 2 * (par + 2 * i));
#pragma unroll
            for (int it = 0; it < CODE_IT; ++it) {
                const int id = lane + 32 * it, tr = id / C::NB, col = id - tr * C::NB;
                cp_pk[it] = (uint32_t)tr | ((uint32_t)(col * 16) << 4) | ((uint32_t)(tr * C::PITCH + col * 16) << 16);
            }
            // copy instruction `it` (0..PER-1) of one unit into landing buffer `buf`; row_slot = fetch_slot of that unit
            auto issue_part = [&](int buf, int row_slot, int it) {
                const uint32_t unit_addr = smem_base + C::OFF_RAW + (xw * S + buf) * C::UNIT_BYTES;
                if (it < CODE_IT) {
                    const uint32_t pk = cp_pk[it];
                    const int sl = __shfl_sync(0xffffffffu, row_slot, pk & 15u);
                    cp_async16(unit_addr + (pk >> 16), p.kv_codes + (long long)clamp_slot(p, sl) * p.kv_codes_stride + ((pk >> 4) & 0xfffu),
                               sl < 0 ? 0u : 16u);
                } else {
                    const int id = lane + 32 * (it - CODE_IT), tr = min(id / 3, UNIT_TOK - 1), wd = id - (id / 3) * 3;
                    const int sl = __shfl_sync(0xffffffffu, row_slot, tr);
                    const uintptr_t bs = reinterpret_cast<uintptr_t>(p.kv_bs + (long long)clamp_slot(p, sl) * p.kv_bs_stride);
                    const int nwords = ((int)(bs & 7) + C::NB + 7) >> 3;   // only words that overlap the row are read
                    if (id < UNIT_TOK * 3)
                        cp_async8(unit_addr + C::OFF_UNIT_SCALES + tr * 24 + wd * 8, reinterpret_cast<const void*>((bs & ~(uintptr_t)7) + wd * 8),
                                  (sl < 0 || wd >= nwords) ? 0u : 8u);
                }
            };
            bool bad_page = false;
            int held[S];                                                  // row slots of the units now in the buffers
            int nxt = fetch_slot(0);
#pragma unroll
            for (int d = 0; d < S; ++d) {
#pragma unroll
                for (int it = 0; it < PER; ++it) issue_part(d, nxt, it);
                cp_async_commit();
                held[d] = nxt;
                nxt = fetch_slot(d + 1);
            }
            int nxt2 = fetch_slot(S + 1);                                 // page-table entries are read two units ahead of their use
            for (int j = 0; j < J; ++j) {
                const int u = xw + j * XWN, g = u / UNITS, k = u - g * UNITS, st = g % NS, buf = j % S;
                cp_async_wait_pending<S - 1>();                           // this lane's copies of unit j have landed
                __syncwarp();                                             // ... and every other lane's
                const unsigned char* unit = smem + C::OFF_RAW + (xw * S + buf) * C::UNIT_BYTES;
                const int cur = S == 1 ? held[0] : (buf == 0 ? held[0] : held[S - 1]);
                // reporting (see clamp_slot): once per unit and row, on a value that has arrived anyway
                bad_page |= cur != -1 && (unsigned int)cur > p.last_slot;                     // -1: no row (past the end)
                // the unit moves into registers: blocks par, par + 2, ... of row tok with their E8M0 bytes (a zero-filled
                // row reads as codes 0, scale 0)
                const int o = (int)(reinterpret_cast<uintptr_t>(p.kv_bs + (long long)clamp_slot(p, cur) * p.kv_bs_stride) & 7);
                const unsigned char* sc_row = unit + C::OFF_UNIT_SCALES + tok * 24 + o + par;
                uint32_t sc[NBH], e = 0;
                uint4 v[NBH];
#pragma unroll
                for (int i = 0; i < NBH; ++i) {
                    sc[i] = sc_row[2 * i];
                    v[i] = *reinterpret_cast<const uint4*>(unit + tok * C::PITCH + (par + 2 * i) * 16);
                    e = max(e, sc[i]);
                }
                __syncwarp();                                             // the buffer has been read by every lane
                // the buffer goes back in flight at once: the copies of unit j + S (an empty group past the end)
#pragma unroll
                for (int it = 0; it < PER; ++it) issue_part(buf, nxt, it);
                cp_async_commit();
                if (S == 1 || buf == 0) held[0] = nxt; else held[S - 1] = nxt;
                nxt = nxt2;
                nxt2 = fetch_slot(j + S + 2);
                const int e_unit = (int)__reduce_max_sync(0xffffffffu, e);
                // The arithmetic needs no operand stage.  With 16 query rows per CTA it is done (and pinned in registers) before
                // the wait for the stage, so that only the stores are left between "stage free" and "tile ready"; for a hybrid
                // cache with 32 rows and for 64 rows the 64 registers of the converted unit do not fit beside the softmax role's (the
                // kernel spilled, and with nearly all of L1 configured as shared memory a spill is an L2 round trip): convert block by block.
                constexpr bool PIN = N == 16 || (N == 32 && !C::ROPE_SEP);
                uint4 ob[PIN ? 2 * NBH : 2];
                if (PIN) {
#pragma unroll
                    for (int i = 0; i < NBH; ++i) dequant_block(v[i], (int)sc[i] - e_unit + 6, ob[PIN ? 2 * i : 0], ob[PIN ? 2 * i + 1 : 1]);
#pragma unroll
                    for (int i = 0; i < (PIN ? 2 * NBH : 0); ++i) asm volatile("" : "+r"(ob[i].x), "+r"(ob[i].y), "+r"(ob[i].z), "+r"(ob[i].w));
                }
                // this unit's rows of the stage are free (the whole stage where the rows are not released one by one)
                if (C::ROWS_EARLY) mbar_wait(&ms.kv_rows_free[st][k / 2], g / NS - 1, abort_flag);
                else mbar_wait(&ms.kv_empty[st], g / NS - 1, abort_flag);
                if (lane == 0) ms.tile_exp[st][k] = e_unit;
                unsigned char* dst_lat = smem + st * STAGE_BYTES + k * (UNIT_TOK * 128);   // panels 0-3: 128-byte rows
                unsigned char* dst_rope = smem + st * STAGE_BYTES + k * (UNIT_TOK * 64);   // rope panel: 64-byte rows
#pragma unroll
                for (int i = 0; i < NBH; ++i) {
                    unsigned char* d = (2 * (2 * i) >= 32 ? dst_rope : dst_lat) + st_off[i];   // block par + 2i >= 16: rope dims
                    if (!PIN) dequant_block(v[i], (int)sc[i] - e_unit + 6, ob[0], ob[1]);
                    *reinterpret_cast<uint4*>(d) = ob[PIN ? 2 * i : 0];
                    *reinterpret_cast<uint4*>(reinterpret_cast<uintptr_t>(d) ^ 16) = ob[PIN ? 2 * i + 1 : 1];
                }
                fence_proxy_async();                                      // the MMA reads the tile through the async proxy
                mbar_arrive(&ms.kv_full[st]);                             // one arrival per lane and unit
            }
            cp_async_wait_all();
            if (bad_page && blockIdx.y == 0) atomicOr(p.status, (int)ST_BAD_PAGE);
        } else if (warp < C::SW) {
            // =========================== softmax / correction / epilogue (128 threads per warpgroup) ===========
            // warpgroup sg owns the query rows (S / O columns) [col0, col0 + NC); thread = token `tok` = TMEM lane
            constexpr int NC = C::NC;
            const int sg = warp >> 2, tok = tid & 127, col0 = sg * NC, bar_id = 1 + 2 * sg;
            const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
            Walker wk; wk.init(prefix, p.batch, t_begin);
            float qk_base = 0.0f;          // sm_scale * log2(e) * (scale of this sequence's Q bytes)
            int e_run = 0;                 // exponent frame of O (block-scaled caches)
            // nm[c] = P_SCALE_LOG2 - (reference maximum of column c); +inf while the column has seen no key.  The same
            // value in all 128 threads, so it lives in shared memory (read as a broadcast) rather than in NC registers per
            // thread; it changes only on the re-centering path, which writes the other half of a double buffer, then syncs.
            // (Only where the registers are needed - hybrid caches and 64 rows per CTA, whose kernels spilled otherwise; the
            // other variants keep the array in registers, which is 6 % faster on the long-context MXFP4 shape.)
            constexpr bool NM_SMEM = C::ROPE_SEP || N == 64;
            float l_acc[NC], nm_r[NM_SMEM ? 1 : NC] = {};
            int nm_cur = 0;
            auto nm = [&](int c) -> float { return NM_SMEM ? ms.nm[sg][nm_cur][c] : nm_r[NM_SMEM ? 0 : c]; };
            // token position pos is visible to the rows of 16-column chunk q iff pos < lim[q]
            // (heads is a multiple of 16, so the query index j is constant inside a chunk)
            int lim[NC / 16], lim_min = 0;
            for (int g = 0; g < n_total; ++g) {
                const int sb = g & 1, st = g % NS;
                const bool first = wk.seek(p, prefix, t_begin + g);
                const bool last = t_begin + g + 1 == min(t_end, wk.seq_t1);
                const int pos_first = (t_begin + g - wk.seq_t0) * TILE;
                if (first) {
#pragma unroll
                    for (int c = 0; c < NC; ++c) l_acc[c] = 0.0f;
                    if (NM_SMEM) {
                        named_bar_sync(bar_id, 128);              // every thread has read the previous sequence's maxima
                        if (tok < NC) ms.nm[sg][nm_cur][tok] = INFINITY;
                        named_bar_sync(bar_id, 128);
                    } else {
#pragma unroll
                        for (int c = 0; c < NC; ++c) nm_r[NM_SMEM ? 0 : c] = INFINITY;
                    }
                    lim_min = 0x7fffffff;
#pragma unroll
                    for (int q = 0; q < NC / 16; ++q) {
                        const int j = (row0 + col0 + 16 * q) / p.heads;
                        const int causal_lim = p.causal ? (wk.tot_len - p.q_len + j + 1 - wk.pos_off) : 0x7fffffff;
                        lim[q] = min(wk.seq_len, causal_lim);
                        lim_min = min(lim_min, lim[q]);
                    }
                    const float qs = C::QSPLIT ? __ldg(p.q_split_scale + (long long)wk.b * gridDim.y + blockIdx.y) : q_tensor_scale;
                    qk_base = p.sm_scale * LOG2E * qs;
                }
                mbar_wait(&ms.s_full[sb], g / 2, abort_flag);
                tc_fence_after();
                // exponent frames: e_unit of this thread's token, e_tile = the largest of the tile's units
                int e_unit = 0, e_tile = 0;
                if (C::XF) {
                    const volatile int* te = ms.tile_exp[st];
                    e_unit = te[tok / UNIT_TOK];
#pragma unroll
                    for (int i = 0; i < TILE / UNIT_TOK; ++i) e_tile = max(e_tile, te[i]);
                }
                const float a_lat = C::XF ? qk_base * pow2i(e_unit - E_BIAS) : qk_base * kv_tensor_scale;
                const float a_rope = qk_base * kv_tensor_scale;
                // score of (this thread's token, query row c) in log2 units, read from the S accumulators.  The scores are not
                // kept in registers beyond x: the rare re-centering path reads them again (the S buffer is handed back after it).
                const uint32_t s_addr = tmem + lane_base + sb * C::SC;
                auto load_scores = [&](float (&dst)[NC]) {
#pragma unroll
                    for (int c0 = 0; c0 < NC; c0 += 16) {
                        float v[16], vl[16], r[16], rl[16];
                        tmem_ld16(s_addr + col0 + c0, v);
                        if (C::QSPLIT) tmem_ld16(s_addr + N + col0 + c0, vl);
                        if (C::ROPE_SEP) {
                            tmem_ld16(s_addr + NQ + col0 + c0, r);
                            if (C::QSPLIT) tmem_ld16(s_addr + NQ + N + col0 + c0, rl);
                        }
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            float lat = v[c], rope = 0.0f;
                            if (C::QSPLIT) lat = fmaf(vl[c], 0.0625f, lat);
                            if (C::ROPE_SEP) { rope = r[c]; if (C::QSPLIT) rope = fmaf(rl[c], 0.0625f, rope); }
                            dst[c0 + c] = C::ROPE_SEP ? fmaf(rope, a_rope, lat * a_lat) : lat * a_lat;
                        }
                    }
                };

                // x = log2-domain exponent of the stored probability: score - m_ref + P_SCALE_LOG2
                const int pos = pos_first + tok;
                const bool masked_tile = pos_first + TILE > lim_min;                 // uniform
                float x[NC];
                load_scores(x);
#pragma unroll
                for (int c = 0; c < NC; ++c) x[c] += nm(c);
                if (masked_tile) {
#pragma unroll
                    for (int c = 0; c < NC; ++c) if (pos >= lim[c / 16]) x[c] = -INFINITY;
                }
                float xm = x[0];
#pragma unroll
                for (int c = 1; c < NC; ++c) xm = fmaxf(xm, x[c]);
                const bool recenter = named_bar_or(bar_id, 128, xm > P_SCALE_LOG2 + RECENTER);
                // a larger exponent frame than the one O is held in: O moves to the new frame
                float o_frame = 1.0f;
                if (C::XF) {
                    if (first) e_run = e_tile;
                    if (e_tile > e_run) { o_frame = pow2i(e_run - e_tile); e_run = e_tile; }
                }
                if (recenter || o_frame != 1.0f) {
                    float f[NC];
                    bool any = o_frame != 1.0f;
#pragma unroll
                    for (int c = 0; c < NC; ++c) f[c] = 1.0f;
                    if (recenter) {
                        // the warpgroup's hi chunks of this tile's P buffer (free once the PV that read it last has
                        // completed) are the scratch area of the column reduction
                        mbar_wait(&ms.p_empty[g % C::P_BUFS], g / C::P_BUFS - 1, abort_flag);
                        float* scratch = reinterpret_cast<float*>(smem + C::OFF_P + (g % C::P_BUFS) * C::P_BUF_BYTES + (col0 / 16) * (TILE * 16));
                        float sv[NC], mx[NC];
                        load_scores(sv);
#pragma unroll
                        for (int c = 0; c < NC; ++c) mx[c] = (masked_tile && pos >= lim[c / 16]) ? -INFINITY : sv[c];
                        reduce_cols_128_scratch<NC, true, 4>(mx, scratch, &ms.red[sg][0][0], tok, bar_id);
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            const float m_old = P_SCALE_LOG2 - nm(c);                 // -inf for a fresh column
                            const float m_new = fmaxf(m_old, mx[c]);
                            f[c] = (m_new == m_old) ? 1.0f : (m_old == -INFINITY ? 0.0f : ex2(m_old - m_new));
                            any |= f[c] != 1.0f;
                            const float nm_new = P_SCALE_LOG2 - m_new;
                            if (NM_SMEM) { if (tok == c) ms.nm[sg][nm_cur ^ 1][c] = nm_new; }
                            else nm_r[NM_SMEM ? 0 : c] = nm_new;
                            l_acc[c] *= f[c];
                            x[c] = (masked_tile && pos >= lim[c / 16]) ? -INFINITY : sv[c] + nm_new;
                        }
                        if (NM_SMEM) {
                            nm_cur ^= 1;
                            named_bar_sync(bar_id, 128);          // the new maxima are in place for every thread
                        }
                    }
                    if (!first && any) {
                        // O holds the sequence's earlier tiles once PV(g-1) has completed; nothing else touches it until P(g) is published
                        mbar_wait(&ms.p_empty[(g - 1) % C::P_BUFS], (g - 1) / C::P_BUFS, abort_flag);
                        tc_fence_after();
#pragma unroll 1
                        for (int jb = 0; jb < 4; ++jb) {                         // rare path: kept small, not unrolled
#pragma unroll
                            for (int h = 0; h < (C::MERGED ? 1 : 2); ++h) {      // side by side: the hi and the lo columns
#pragma unroll
                                for (int c0 = 0; c0 < NC; c0 += 16) {
                                    float o[16];
                                    const uint32_t addr = tmem + lane_base + C::TMEM_O + jb * C::OB + h * N + col0 + c0;
                                    tmem_ld16(addr, o);
                                    tmem_wait_ld();
#pragma unroll
                                    for (int c = 0; c < 16; ++c) o[c] *= f[c0 + c] * o_frame;
                                    tmem_st16(addr, o);
                                }
                            }
                        }
                        tmem_wait_st();
                        tc_fence_before();
                    }
                }
                tc_fence_before();
                mbar_arrive(&ms.s_empty[sb]);                     // the scores have been read for the last time
                // stored probability = p * 2^4 * 2^(e_unit - e_run): this token's V bytes are in the frame e_unit, O in e_run
                const float p_frame = C::XF ? pow2i(e_unit - e_run) : 1.0f;
                // P(g) may overwrite its buffer once the PV that read it last (tile g - P_BUFS) has completed
                const int pb = g % C::P_BUFS;
                mbar_wait(&ms.p_empty[pb], g / C::P_BUFS - 1, abort_flag);
                uint8_t* pbuf = smem + C::OFF_P + pb * C::P_BUF_BYTES;
                // MERGED: the lo term shares O's columns with the hi term, so it carries no factor of its own
                constexpr float LO_GAIN = C::MERGED ? 1.0f : 16.0f;
#pragma unroll
                for (int c0 = 0; c0 < NC; c0 += 16) {
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        float pv[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int c = c0 + q4 * 4 + k;
                            pv[k] = ex2(x[c]);                                        // ex2(-inf) = 0 for masked keys
                            l_acc[c] += pv[k];
                            if (C::XF) pv[k] *= p_frame;
                        }
                        hi[q4] = pack_e4m3x4(pv[0], pv[1], pv[2], pv[3]);
                        const float2 h01 = unpack_e4m3x2((uint16_t)(hi[q4] & 0xffffu)), h23 = unpack_e4m3x2((uint16_t)(hi[q4] >> 16));
                        lo[q4] = pack_e4m3x4((pv[0] - h01.x) * LO_GAIN, (pv[1] - h01.y) * LO_GAIN,
                                             (pv[2] - h23.x) * LO_GAIN, (pv[3] - h23.y) * LO_GAIN);
                    }
                    *reinterpret_cast<uint4*>(pbuf + ((col0 + c0) / 16) * (TILE * 16) + tok * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(pbuf + ((N + col0 + c0) / 16) * (TILE * 16) + tok * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
                fence_proxy_async();
                mbar_arrive(&ms.p_full[pb]);

                if (last) {
                    // ---- epilogue of this (CTA, sequence) pair: wait for its last PV, normalise, write out
                    mbar_wait(&ms.p_empty[pb], g / C::P_BUFS, abort_flag);
                    tc_fence_after();
                    reduce_cols_128_scratch<NC, false, 4>(l_acc, reinterpret_cast<float*>(pbuf + (col0 / 16) * (TILE * 16)), &ms.red[sg][0][0], tok,
                                                          bar_id);                   // PV(g) is done: the P buffer is free
                    const bool whole = (t_begin <= wk.seq_t0) && (wk.seq_t1 <= t_end);
                    const int slot = w + wk.b;
                    const float out_scale = C::XF ? pow2i(e_run - E_BIAS) : kv_tensor_scale;
                    float inv[NC];
#pragma unroll
                    for (int c = 0; c < NC; ++c) inv[c] = l_acc[c] > 0.0f ? __fdividef(out_scale, l_acc[c]) : 0.0f;
                    // one output element per (row, dim): this thread owns dims tok, 128 + tok, ... of its warpgroup's rows
                    const long long orow0 = (whole ? (long long)wk.b * p.rows : (long long)slot * p.rows) + row0 + col0;
                    float* dst_f32 = whole ? p.out_o_f32 : p.part_o;
                    __nv_bfloat16* dst_bf16 = whole ? p.out : nullptr;
                    if (dst_f32) dst_f32 += orow0 * V_DIM + tok;
                    if (dst_bf16) dst_bf16 += orow0 * V_DIM + tok;
#pragma unroll 1
                    for (int jb = 0; jb < 4; ++jb) {                             // once per sequence: code size before speed
#pragma unroll
                        for (int c0 = 0; c0 < NC; c0 += 16) {
                            float ohi[16], olo[16];
                            tmem_ld16(tmem + lane_base + C::TMEM_O + jb * C::OB + col0 + c0, ohi);
                            if (!C::MERGED) tmem_ld16(tmem + lane_base + C::TMEM_O + jb * C::OB + N + c0, olo);
                            tmem_wait_ld();
#pragma unroll
                            for (int c = 0; c < 16; ++c) ohi[c] = (C::MERGED ? ohi[c] : fmaf(olo[c], 0.0625f, ohi[c])) * inv[c0 + c];
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
                    if (tok < NC) {
                        float lsum = 0.0f, nmc = 0.0f;
#pragma unroll
                        for (int c = 0; c < NC; ++c) if (c == tok) { lsum = l_acc[c]; nmc = nm(c); }
                        const float lse = lsum > 0.0f ? (log2f(lsum) - nmc) * LN2 : -INFINITY;
                        if (whole) { if (p.out_lse) p.out_lse[(long long)wk.b * p.rows + row0 + col0 + tok] = lse; }
                        else p.part_lse[(long long)slot * p.rows + row0 + col0 + tok] = lse;
                    }
                }
            }
        }
    }

    __syncthreads();
    if (tid == 0 && ms.abort_flag) atomicOr(status, (int)ST_TIMEOUT);
    if (warp == C::SW) { tc_fence_after(); tmem_dealloc(tmem, C::TMEM_COLS); }
}

// bf16 Q -> two e4m3 planes.  Block (group, sequence) takes the N query rows [group*N, group*N + N) of one
// sequence, finds their largest magnitude, scales by the power of two s that puts it in [128, 256) and
// writes hi = e4m3(q*s), lo = e4m3((q*s - hi) * 16); 1/s goes to inv_scale[sequence][group].
// hi + lo/16 carries eight significant bits, as many as bf16 has.
template <int N>
__global__ void __launch_bounds__(256) q_split_kernel(const MlaParams p, uint8_t* planes, float* inv_scale) {
    constexpr int VECS = N * (QK_DIM / 8), PER = (VECS + 255) / 256;
    const int b = blockIdx.y, row0 = blockIdx.x * N, tid = threadIdx.x;
    __shared__ float red[8];
    uint4 v[PER];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int id = tid + i * 256;
        v[i] = make_uint4(0, 0, 0, 0);
        if (id < VECS) {
            const int r = id / (QK_DIM / 8), c8 = (id - r * (QK_DIM / 8)) * 8;
            const int rg = row0 + r, j = rg / p.heads, h = rg - j * p.heads;
            v[i] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.q) +
                         (long long)(b * p.q_len + j) * p.q_row_stride + (long long)h * p.q_head_stride + c8));
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(h2[k]);
                amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((tid & 31) == 0) red[tid >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
    // exponent of amax (clamped so that both s and 1/s stay normal); zero rows: s = 1
    int e = ((__float_as_int(amax) >> 23) & 0xff) - 127;
    e = amax > 0.0f ? max(-100, min(e, 100)) : 7;
    const float s = __int_as_float((7 - e + 127) << 23);
    if (tid == 0) inv_scale[(long long)b * gridDim.x + blockIdx.x] = __int_as_float((e - 7 + 127) << 23);
    const long long plane = (long long)p.batch * p.rows * QK_DIM;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int id = tid + i * 256;
        if (id < VECS) {
            const int r = id / (QK_DIM / 8), c8 = (id - r * (QK_DIM / 8)) * 8;
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
            float f[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 t = __bfloat1622float2(h2[k]); f[2 * k] = t.x * s; f[2 * k + 1] = t.y * s; }
            uint32_t hi[2], lo[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                hi[k] = sm100::pack_e4m3x4(f[4 * k], f[4 * k + 1], f[4 * k + 2], f[4 * k + 3]);
                const float2 h01 = sm100::unpack_e4m3x2((uint16_t)(hi[k] & 0xffffu)), h23 = sm100::unpack_e4m3x2((uint16_t)(hi[k] >> 16));
                lo[k] = sm100::pack_e4m3x4((f[4 * k] - h01.x) * 16.0f, (f[4 * k + 1] - h01.y) * 16.0f,
                                           (f[4 * k + 2] - h23.x) * 16.0f, (f[4 * k + 3] - h23.y) * 16.0f);
            }
            uint8_t* dst = planes + ((long long)b * p.rows + row0 + r) * QK_DIM + c8;
            *reinterpret_cast<uint2*>(dst) = make_uint2(hi[0], hi[1]);
            *reinterpret_cast<uint2*>(dst + plane) = make_uint2(lo[0], lo[1]);
        }
    }
}

}  // namespace sm100x

namespace {

template <int N, int KVFMT, int QFMT>
size_t smem_need(int batch) {
    return (size_t)sm100x::Cfg<N, KVFMT, QFMT>::OFF_MISC + sizeof(sm100x::Misc) + (size_t)(batch + 1) * sizeof(int);
}

template <int N, int KVFMT, int QFMT>
cudaError_t launch_cfg(const MlaParams& p, int* status, cudaStream_t stream, bool dry_run, bool* fits) {
    using C = sm100x::Cfg<N, KVFMT, QFMT>;
    const size_t smem = smem_need<N, KVFMT, QFMT>(p.batch);
    if (fits) *fits = smem <= (size_t)sm100x::SMEM_LIMIT;
    if (dry_run) return cudaSuccess;
    if (smem > (size_t)sm100x::SMEM_LIMIT) return cudaErrorInvalidConfiguration;
    if (QFMT == Q_BF16) {
        sm100x::q_split_kernel<N><<<dim3(p.rows / N, p.batch), 256, 0, stream>>>(p, p.q_split, p.q_split_scale);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    cudaError_t e = cudaFuncSetAttribute(sm100x::mla_decode_sm100x_kernel<N, KVFMT, QFMT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 grid(p.num_ctas, p.rows / N);
    sm100x::mla_decode_sm100x_kernel<N, KVFMT, QFMT><<<grid, C::THREADS, smem, stream>>>(p, status);
    return cudaGetLastError();
}

template <int N>
cudaError_t dispatch_formats(const MlaParams& p, int* status, cudaStream_t stream, bool dry_run, bool* fits) {
    if constexpr (N == 64) {                                      // 64 rows per CTA: e4m3 Q over a block-scaled cache
        if (p.q_format == Q_E4M3 && p.kv_format == KV_MXFP4) return launch_cfg<64, KV_MXFP4, Q_E4M3>(p, status, stream, dry_run, fits);
        if (p.q_format == Q_E4M3 && p.kv_format == KV_HYBRID) return launch_cfg<64, KV_HYBRID, Q_E4M3>(p, status, stream, dry_run, fits);
        if (fits) *fits = false;
        return cudaErrorInvalidValue;
    } else {
    if (p.q_format == Q_BF16) {
        if (p.kv_format == KV_E4M3) return launch_cfg<N, KV_E4M3, Q_BF16>(p, status, stream, dry_run, fits);
        if (p.kv_format == KV_MXFP4) return launch_cfg<N, KV_MXFP4, Q_BF16>(p, status, stream, dry_run, fits);
        return launch_cfg<N, KV_HYBRID, Q_BF16>(p, status, stream, dry_run, fits);
    }
    if (p.kv_format == KV_MXFP4) return launch_cfg<N, KV_MXFP4, Q_E4M3>(p, status, stream, dry_run, fits);
    if (p.kv_format == KV_HYBRID) return launch_cfg<N, KV_HYBRID, Q_E4M3>(p, status, stream, dry_run, fits);
    if (fits) *fits = false;                                      // e4m3 x e4m3 belongs to the plain tcgen05 kernel
    return cudaErrorInvalidValue;
    }
}

}  // namespace

// 64 query rows per CTA where the format pair has that variant (a tile is then gathered and converted once per 64
// rows), else 32 or 16.
int sm100x_rows_per_cta(const MlaParams& p) {
    // the widest variant whose shared-memory layout (it ends with the tile prefix of the batch) fits
    bool fits = false;
    if (p.rows % 64 == 0 && p.q_format == Q_E4M3 && p.kv_format != KV_E4M3) {
        dispatch_formats<64>(p, nullptr, nullptr, true, &fits);
        if (fits) return 64;
    }
    if (p.rows % 32 == 0) {
        dispatch_formats<32>(p, nullptr, nullptr, true, &fits);
        if (fits) return 32;
    }
    return 16;
}

// Every format pair except e4m3 Q x e4m3 cache; the tile-prefix table must fit beside the rings.
bool sm100x_supported(const MlaParams& p) {
    if (p.rows % 16 != 0 || (p.q_format == Q_E4M3 && p.kv_format == KV_E4M3)) return false;
    // the E8M0 rows are fetched as three aligned 8-byte words: they must start on an even address
    if (p.kv_format != KV_E4M3 && ((reinterpret_cast<uintptr_t>(p.kv_bs) | (uintptr_t)p.kv_bs_stride) & 1u)) return false;
    bool fits = false;
    const int n = sm100x_rows_per_cta(p);
    if (n == 64) dispatch_formats<64>(p, nullptr, nullptr, true, &fits);
    else if (n == 32) dispatch_formats<32>(p, nullptr, nullptr, true, &fits);
    else dispatch_formats<16>(p, nullptr, nullptr, true, &fits);
    return fits;
}

// bytes of the split-Q planes and of their per-group scales for a problem of this size
long long sm100x_q_split_bytes(int batch, int rows) { return 2LL * batch * rows * QK_DIM; }
long long sm100x_q_scale_bytes(int batch, int rows) { return (long long)batch * (rows / 16) * 4; }

cudaError_t launch_sm100x(const MlaParams& p, int* status, cudaStream_t stream) {
    if (p.rows_per_cta == 64) return dispatch_formats<64>(p, status, stream, false, nullptr);
    return p.rows_per_cta == 32 ? dispatch_formats<32>(p, status, stream, false, nullptr)
                                : dispatch_formats<16>(p, status, stream, false, nullptr);
}

}  // namespace b200mla
