/*
 * b200_mla.h - C ABI of the B200 (sm_100a) absorbed-MLA decode library (libb200mla.so).
 *
 * Plain pointers and sizes only; every pointer marked "device" must be valid on the CUDA device
 * that is current when the call is made, `stream` is a cudaStream_t passed as void*.
 * All entry points return 0 on success or a negative b200_mla_status; none of them synchronises
 * the stream or reads device memory on the host.
 *
 * Each entry point names the reference interface it replaces (paths relative to the reference
 * project root).
 */
#ifndef B200_MLA_H
#define B200_MLA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_MLA_QK_DIM 576   /* 512 latent + 64 rope (reference.py:40-46) */
#define B200_MLA_V_DIM 512    /* V = first 512 dims of the same cache row (task.py:20-23) */
#define B200_MLA_ROPE_DIM 64

typedef enum {
    B200_MLA_OK = 0,
    B200_MLA_ERR_INVALID_ARG = -1,      /* null pointer, bad stride / alignment, bad enum */
    B200_MLA_ERR_UNSUPPORTED = -2,      /* combination the kernels do not implement */
    B200_MLA_ERR_WORKSPACE = -3,        /* workspace too small */
    B200_MLA_ERR_CUDA = -4,             /* a CUDA runtime call failed; see b200_mla_last_error */
    B200_MLA_ERR_TOO_LARGE = -5         /* size beyond a documented limit */
} b200_mla_status;

/* B200_MLA_Q_BF16_CAST_E4M3: q is bf16 and is quantised to e4m3 with the reference's per-tensor rule while the
 * decode kernel loads it (same codes and scale as b200_mla_quantize_fp8 followed by B200_MLA_Q_E4M3, one launch
 * less); q_scale then points to the B200_MLA_Q_AMAX_PARTS partial maxima written by b200_mla_q_amax. */
typedef enum { B200_MLA_Q_BF16 = 0, B200_MLA_Q_E4M3 = 1, B200_MLA_Q_BF16_CAST_E4M3 = 2 } b200_mla_q_format;
#define B200_MLA_Q_AMAX_PARTS 256

typedef enum {
    B200_MLA_KV_E4M3 = 0,    /* [slots, 576] e4m3fn codes + fp32 per-tensor scale            */
    B200_MLA_KV_MXFP4 = 1,   /* [slots, 288] e2m1 x2 (even element in the low nibble)        */
                             /* + [slots, >=18] E8M0, one per 32 elements                    */
    B200_MLA_KV_HYBRID = 2   /* latent: [slots, 256] e2m1 x2 + [slots, 16] E8M0;             */
                             /* rope: [slots, 64] e4m3fn + fp32 per-tensor scale             */
} b200_mla_kv_format;

typedef enum {
    B200_MLA_IMPL_AUTO = 0,      /* tcgen05 kernel where it applies, else the generic one */
    B200_MLA_IMPL_GENERIC = 1,   /* warp-level tensor-core kernel, every shape */
    B200_MLA_IMPL_TCGEN05 = 2    /* tcgen05 / TMEM kernel; B200_MLA_ERR_UNSUPPORTED if it does not apply */
} b200_mla_impl;

/*
 * Arguments of one decode call.  The layout mirrors what the reference's native entry points
 * receive: aiter.mla_decode_stage1_asm_fwd(q, kv4d, qo_indptr, kv_indptr, kv_indices,
 * kv_last_page_lens, ..., sm_scale, logits, attn_lse, o, final_lse, q_scale, kv_scale)
 * (mixed-mla/versions/v34_direct_asm/submission.py:455-476) and the HIP extension
 * mla_mxfp4_v5_forward(Q_fp8, K_fp4, K_scale, V_fp8, kv_indptr, sm_scale, kv_scale, B, splits)
 * (mixed-mla/versions/hip_mxfp4_v5/submission.py:720-730).
 */
typedef struct {
    /* ---- problem ---- */
    int32_t batch;            /* sequences */
    int32_t heads;            /* query heads sharing the single latent KV head; multiple of 16 */
    int32_t q_len;            /* queries per sequence (1, or 2..8 for speculative decode) */
    int32_t q_format;         /* b200_mla_q_format */
    int32_t kv_format;        /* b200_mla_kv_format */
    int32_t causal;           /* non-zero: query j sees key position p iff p <= total_len - q_len + j */
    int32_t page_size;        /* tokens per page; kv_indices holds page ids. 1 for the reference layout */
    int32_t impl;             /* b200_mla_impl */
    float sm_scale;           /* softmax scale (reference: 1/sqrt(576), reference.py:46) */
    int32_t max_ctas;         /* cap on stage-1 CTAs per row group; 0 = fill the device (tuning / tests) */

    /* ---- Q: [batch*q_len, heads, 576] ---- */
    const void *q;            /* device; bf16 or e4m3fn */
    int64_t q_row_stride;     /* elements between consecutive query rows (heads*576 when dense) */
    int64_t q_head_stride;    /* elements between heads (576 when dense) */
    const float *q_scale;     /* device fp32[1] for B200_MLA_Q_E4M3; the partial maxima (uint32[B200_MLA_Q_AMAX_PARTS])
                               * of b200_mla_q_amax for B200_MLA_Q_BF16_CAST_E4M3; else NULL */

    /* ---- KV cache planes (device) ---- */
    const void *kv_codes;     /* e4m3: [slots,576]; mxfp4: [slots,288]; hybrid: latent [slots,256] */
    int64_t kv_codes_stride;  /* bytes between slots; multiple of 16.  e4m3 caches: a 16-byte aligned plane is fetched by the
                               * copy engine (TMA: tiled boxes without a page table, four-row gathers by page id with one);
                               * an unaligned one by 16-byte copies, with the same result */
    const void *kv_block_scales;   /* E8M0 bytes (mxfp4: >=18 per slot, hybrid: >=16); NULL for e4m3.  The tcgen05
                                    * kernels fetch a slot's bytes as the aligned 8-byte words around them: up to 7
                                    * bytes before the first and after the last row of the plane may be read
                                    * (never used), so the plane must not end flush against unmapped memory */
    int64_t kv_block_scales_stride;/* bytes between slots (the reference pads this plane, reference.py:125-148) */
    const void *kv_rope;      /* hybrid only: [slots,64] e4m3fn */
    int64_t kv_rope_stride;   /* bytes between slots; multiple of 16 */
    const float *kv_scale;    /* device fp32[1]: per-tensor scale of the e4m3 codes (e4m3: whole row, hybrid: rope) */
    int64_t num_slots;        /* rows in the cache planes, > 0.  Every slot the page table yields is clamped into
                               * [0, num_slots) on the device, so nothing outside the planes is ever read; a page id
                               * that needed the clamp sets B200_MLA_STATUS_BAD_PAGE and the outputs of that call
                               * are meaningless (the key read as some other row of the cache) */

    /* ---- page table ---- */
    const int32_t *kv_indptr;     /* device int32[batch+1], token offsets (task.py:14) */
    const int32_t *kv_indices;    /* device int32[...] page ids, or NULL: token t of the batch lives in slot t,
                                     exactly the arange the reference builds (reference.py:245) */
    const int32_t *kv_page_indptr;/* device int32[batch+1] offsets into kv_indices; NULL when page_size == 1
                                     (then kv_indptr is used) */
    int64_t total_kv_hint;        /* upper bound on kv_indptr[batch] known to the host (sizes the grid) */

    /* ---- sharded sequences (cross-GPU split-KV); NULL when the call sees whole sequences ---- */
    const int32_t *kv_pos_offset; /* device int32[batch]: position of the shard's first key in the sequence */
    const int32_t *kv_total_len;  /* device int32[batch]: full sequence length (for the causal mask) */

    /* ---- outputs (device) ---- */
    void *out;                /* bf16 [batch*q_len, heads, 512], dense; may be NULL if out_o_f32 is set */
    float *out_o_f32;         /* optional: normalised fp32 O [batch*q_len, heads, 512] (partial of a shard) */
    float *out_lse;           /* optional: fp32 natural-log LSE [batch*q_len, heads]; -inf for an empty key set */

    /* ---- scratch ---- */
    void *workspace;          /* device, 256-byte aligned.  Its first 256 bytes hold the sticky status word and must
                               * be zero before the first call that uses a fresh buffer (b200_mla_reset_status,
                               * or any memset); later calls leave them alone */
    int64_t workspace_bytes;  /* >= b200_mla_workspace_bytes() */
} b200_mla_decode_args;

/* Library / ABI version (major*1000 + minor). */
int32_t b200_mla_version(void);

/* Human-readable text for the last failing call on the calling thread. */
const char *b200_mla_last_error(void);

/*
 * Scratch size for one decode call on the current device.
 * Replaces aiter.get_mla_metadata_info_v1 (reference.py:174-182), which sizes the reference's six
 * work buffers, and the partial-buffer allocation of _get_mxfp4_buffers (mixed-mla/submission.py:301-318).
 */
int64_t b200_mla_workspace_bytes(int32_t batch, int32_t heads, int32_t q_len);

/*
 * Split-KV decode: stage 1 (partial attention per KV span) followed by the log-sum-exp combine,
 * both enqueued on `stream`.
 * Replaces mla_decode_fwd / mla_decode_stage1_asm_fwd + mla_reduce_v1
 * (mixed-mla/asm_dumps/aiter_mla.py:149-470), the Triton pair _mla_mxfp4_stage1 / _mla_mxfp4_reduce
 * (mixed-mla/submission.py:122-294) and the work-list builder get_mla_metadata_v1
 * (reference.py:184-200): the KV spans are derived on the device from kv_indptr.
 */
int32_t b200_mla_decode(const b200_mla_decode_args *args, void *stream);

/*
 * Log-sum-exp merge of `parts` normalised partial results, e.g. the per-GPU shards of a
 * split-KV sequence after an all-gather:
 *   o_parts   device fp32, part i at o_parts + i*o_part_stride, [rows, 512] dense inside a part
 *   lse_parts device fp32, part i at lse_parts + i*lse_part_stride, [rows]
 *   strides   in elements; 0 means dense ([parts, rows, 512] and [parts, rows]).  A fused
 *             all-gather buffer holding (O || LSE) per rank is merged in place with
 *             o_part_stride = lse_part_stride = rows*513 and lse_parts = o_parts + rows*512.
 *   out       device bf16 [rows, 512];  out_lse optional device fp32 [rows]
 * Replaces _mla_mxfp4_reduce (mixed-mla/submission.py:257-294), aiter.mla_reduce_v1
 * (mixed-mla/asm_dumps/aiter_mla.py:421-430) and the (O, LSE) form of
 * competitor_submissions/dgavriloff_v114_hybrid_mxfp4k_fp8v.py:131-160.
 */
int32_t b200_mla_combine(const float *o_parts, const float *lse_parts, int32_t parts, int64_t rows,
                         int64_t o_part_stride, int64_t lse_part_stride, void *out, float *out_lse, void *stream);

/*
 * Dynamic per-tensor e4m3fn quantisation of a dense bf16 tensor of n elements with the arithmetic
 * order of the reference's quantize_fp8 (reference.py:65-80; fused Triton form
 * mixed-mla/fused_fp8_quant.py:93-148): amax, scale = amax/448 and x/scale rounded to bf16, clamp,
 * cast.  `scale_out` (device fp32[1]) receives the scale; `scratch` is device, >= 4 bytes.
 */
int32_t b200_mla_quantize_fp8(const void *x_bf16, int64_t n, void *codes_out, float *scale_out,
                              void *scratch, void *stream);

/*
 * Append rows to a quantised cache: `n` bf16 latent rows [n, 576] -> the rows `slots[i]` (or base_slot + i when
 * slots is NULL) of an e4m3, MXFP4 or hybrid cache, with the reference quantisers' arithmetic, so that the bytes
 * equal what quantize_fp8 (reference.py:65-80, with the given per-tensor scale) and quantize_mxfp4
 * (reference.py:88-113; rounding rule mxfp4-mm/submission_v3_self_contained.py:19-72; fused Triton form
 * mixed-mla/versions/v22_small_config_opt/submission_triton_quant.py:88-187) produce for the same rows.
 * The per-tensor scale of an e4m3 cache / of a hybrid cache's rope dims is an input (device fp32[1]): rows added
 * later cannot change the scale of rows already stored.  A slot outside [0, num_slots) is not written and sets
 * *status (device int32, required with a slot list) to 1.
 */
typedef struct {
    const void *rows_bf16;    /* device bf16 [n, 576], 16-byte aligned */
    int64_t n;
    int64_t row_stride;       /* elements between rows (576 when dense; multiple of 8) */
    const int32_t *slots;     /* device int32[n] destination slots, or NULL */
    int64_t base_slot;        /* first destination slot when slots is NULL */
    int64_t num_slots;        /* rows in the cache planes */
    int32_t kv_format;        /* b200_mla_kv_format */
    int32_t reserved;
    void *kv_codes;           /* planes as in b200_mla_decode_args */
    int64_t kv_codes_stride;
    void *kv_block_scales;
    int64_t kv_block_scales_stride;
    void *kv_rope;
    int64_t kv_rope_stride;
    const float *kv_scale;    /* device fp32[1]; NULL for mxfp4 */
    int32_t *status;          /* device int32, may be NULL when slots is NULL */
} b200_mla_kv_append_args;
int32_t b200_mla_kv_append(const b200_mla_kv_append_args *args, void *stream);

/*
 * First half of that quantisation on its own (the amax of mixed-mla/fused_fp8_quant.py:27-53): the
 * largest bf16 magnitude of x, left as B200_MLA_Q_AMAX_PARTS per-block partial maxima (bf16 bit
 * patterns, uint32 each) in `parts_out`.  A decode call with q_format B200_MLA_Q_BF16_CAST_E4M3
 * takes them through q_scale and does the cast itself.  One launch, no memset, no atomics.
 */
int32_t b200_mla_q_amax(const void *x_bf16, int64_t n, uint32_t *parts_out, void *stream);

/*
 * Decode without any allocation on the caller's side (no counterpart in the reference, whose
 * wrappers allocate their partial buffers with torch on every path).
 *
 * For callers that cannot obtain device memory at call time: a serving loop whose memory pool is
 * frozen after start-up, code running under a framework that forbids allocator calls in its hot
 * section, or a plain C host that owns no allocator at all.  Same arguments and results as
 * b200_mla_decode, except that `workspace` / `workspace_bytes` are ignored: the split-KV partials,
 * the tile table and the status word live in a B200_MLA_STATIC_WORKSPACE_BYTES array that is part
 * of the library image on every GPU that loads it (held until the process exits).
 *   - A problem whose b200_mla_workspace_bytes() exceeds that size is refused with
 *     B200_MLA_ERR_TOO_LARGE; nothing is launched.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture.
 *   - The call itself performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *   - All calls on a device share the one array: calls that overlap on the GPU (two streams, two
 *     threads) race on the partials.  Contents persist from call to call; nothing in them has to
 *     be cleared by the caller (the status word starts at zero and is sticky).
 */
#define B200_MLA_STATIC_WORKSPACE_BYTES (16u << 20)
int32_t b200_mla_decode_static(const b200_mla_decode_args *args, void *stream);

/*
 * Device-side status of the decode calls that used `workspace` (no counterpart in the reference: AITER's kernels
 * report nothing, mixed-mla/submission.py:626-644 returns whatever they wrote).  The kernels OR bits into the first
 * word of the workspace and never clear them:
 *   B200_MLA_STATUS_TIMEOUT   a bounded device-side wait expired; the outputs of that call are not valid
 *   B200_MLA_STATUS_BAD_PAGE  kv_indptr / kv_indices named a slot outside [0, num_slots); nothing outside the cache
 *                             planes was read (the id was clamped), the outputs of that call are meaningless
 * b200_mla_read_status enqueues one 4-byte copy of the word into `out` (device, pinned or pageable host memory) on
 * `stream`; the caller decides whether and when to wait for it.  b200_mla_reset_status enqueues the zeroing of the
 * word (and of the rest of the 256-byte header); call it once on a fresh workspace.  workspace == NULL addresses
 * the built-in scratch of b200_mla_decode_static on the current device.
 */
#define B200_MLA_STATUS_TIMEOUT 1
#define B200_MLA_STATUS_BAD_PAGE 2
int32_t b200_mla_read_status(const void *workspace, int32_t *out, void *stream);
int32_t b200_mla_reset_status(void *workspace, void *stream);

/*
 * Profiling aid (no counterpart in the reference, whose harness times whole calls, eval.py:225-261):
 * while both events (cudaEvent_t) are non-NULL, every b200_mla_decode issued by the calling thread
 * records `start` before and `stop` after its stage-1 kernel on the call's stream.  Pass NULLs to
 * switch it off.
 */
int32_t b200_mla_set_stage1_events(void *start_event, void *stop_event);

/*
 * Cross-GPU split-KV over peer memory (one process per GPU on one NVLink / NVSwitch node).  The reference is
 * single-GPU; what is exchanged and merged here is the split-KV reduce of mixed-mla/submission.py:257-294 with the
 * splits living on different GPUs.  Rank r decodes its key range of every sequence with b200_mla_decode
 * (kv_pos_offset / kv_total_len, out_o_f32 / out_lse) straight into its exchange allocation; b200_mla_peer_merge then
 * signals the peers, waits for them with a time limit, reads their partials out of their memory with plain peer
 * loads and writes the merged bf16 rows - no collective call, no staging copy.
 *
 *   b200_mla_peer_exchange_bytes(rows)   size of one rank's exchange allocation; rows = batch * q_len * heads
 *   b200_mla_peer_alloc(rows, &base, handle)   cudaMalloc + zero + export: `handle` (B200_MLA_PEER_HANDLE_BYTES
 *                                        bytes) goes to the other ranks by any host channel
 *   b200_mla_peer_open(handle, &base)    map another rank's allocation into this process (CUDA IPC, peer access
 *                                        enabled on first use); b200_mla_peer_close unmaps it
 *   b200_mla_peer_partial_offset(rows, epoch)   byte offset, inside the allocation, of the (O [rows,512] fp32 ||
 *                                        LSE [rows] fp32) partial of step `epoch` (two buffers, chosen by epoch & 1)
 *   b200_mla_peer_merge(args, stream)    the fused signal + wait + merge kernel
 *
 * Protocol: all ranks call b200_mla_peer_merge once per decode step with the same `epoch`, which starts at 1 and
 * grows by 1 per step, after the kernels that wrote this step's partial on the same stream.  bases[i] is rank i's
 * allocation as mapped in the calling process (bases[rank] is its own).  A peer whose signal does not arrive
 * within wait_limit_ms (0 = 2000) is merged with weight 0 and B200_MLA_STATUS_TIMEOUT is set in the status word of
 * `workspace` (NULL = the built-in scratch); the kernel always returns.  world is 1, 2, 4 or 8.
 * Each rank runs on its own GPU: two ranks must never share one GPU (their kernels wait on one another).
 */
#define B200_MLA_PEER_HANDLE_BYTES 64
typedef struct {
    int32_t world;
    int32_t rank;
    uint32_t epoch;
    uint32_t wait_limit_ms;
    const void *const *bases; /* host array [world] of device pointers */
    int64_t rows;
    void *out;                /* device bf16 [rows, 512] */
    void *workspace;          /* holds the status word; NULL = built-in scratch */
} b200_mla_peer_merge_args;
int64_t b200_mla_peer_exchange_bytes(int64_t rows);
int64_t b200_mla_peer_partial_offset(int64_t rows, uint32_t epoch);
int32_t b200_mla_peer_alloc(int64_t rows, void **base, unsigned char *handle);
int32_t b200_mla_peer_open(const unsigned char *handle, void **base);
int32_t b200_mla_peer_close(void *base);
int32_t b200_mla_peer_free(void *base);
int32_t b200_mla_peer_merge(const b200_mla_peer_merge_args *args, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_MLA_H */
