/*
 * Scalar C restatement of absorbed-MLA decode over a quantised latent KV cache.
 *
 * TEST INFRASTRUCTURE ONLY: a second, independent opinion next to oracle/mla_oracle.py.  The
 * shipped library never links or loads this file.
 *
 * Follows the reference's own scalar kernel (one loop nest per (sequence, head): 576-wide dot
 * product, online softmax, 512-wide V accumulation, scalar scale applied to the scores and once
 * to the output): mixed-mla/versions/hip_phase1/submission.py:85-159, with
 *   - the OCP e4m3fn decoder (bias 7, max 448) in place of that file's AMD e4m3fnuz decoder
 *     (:52-74), as NVIDIA and gfx950 use e4m3fn (competitor_submissions/mi355x_reference/README.md:89);
 *   - the e2m1 / E8M0 decode of mixed-mla/triton_mla_mxfp4.py:20-31,:59;
 *   - the MXFP4 quantiser rule of mxfp4-mm/submission_v3_self_contained.py:19-72;
 *   - a page table (kv_indices) between kv_indptr and the cache rows, and a bottom-right causal
 *     mask for q_len > 1 (both absent from the reference; defined by this project).
 *
 * Build: make -C oracle   (gcc -O2 -shared -fPIC)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK_DIM 576
#define V_DIM 512
#define ROPE_DIM 64

enum { MO_KV_FP8 = 0, MO_KV_MXFP4 = 1, MO_KV_HYBRID = 2 };

float mo_e4m3fn_to_float(uint8_t b) {
    int e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0xF && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m / 8.0f, -6);
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return (b & 0x80) ? -v : v;
}

float mo_e2m1_to_float(uint8_t nib) {
    int e = (nib >> 1) & 3, m = nib & 1;
    float v = (e == 0) ? 0.5f * (float)m : ldexpf(1.0f + 0.5f * (float)m, e - 1);
    return (nib & 8) ? -v : v;
}

float mo_e8m0_to_float(uint8_t b) {
    if (b == 255) return NAN;
    return ldexpf(1.0f, (int)b - 127);
}

/* One block of 32 floats -> 16 packed bytes + one E8M0 byte. */
void mo_quantize_mxfp4_block(const float *x, uint8_t *packed16, uint8_t *scale) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) { float a = fabsf(x[i]); if (a > amax) amax = a; }
    uint32_t bits; memcpy(&bits, &amax, 4);
    bits = (uint32_t)(((uint64_t)bits + 0x200000u) & 0xFF800000u);
    int ef = (int)(bits >> 23);
    int ex = (ef == 0) ? -127 : ef - 127 - 2;
    if (ex < -127) ex = -127;
    if (ex > 127) ex = 127;
    *scale = (uint8_t)(ex + 127);
    uint8_t code[32];
    for (int i = 0; i < 32; i++) {
        float q = x[i] * ldexpf(1.0f, -ex);
        uint32_t qb; memcpy(&qb, &q, 4);
        uint8_t sign = (uint8_t)((qb >> 28) & 8);
        uint32_t mb = qb & 0x7FFFFFFFu;
        float mag; memcpy(&mag, &mb, 4);
        uint8_t c;
        if (mag >= 6.0f) c = 7;
        else if (mag < 1.0f) {
            volatile float t = mag + 4194304.0f;       /* 2^22: rounds to a multiple of 0.5, RNE */
            float tt = t; uint32_t tb; memcpy(&tb, &tt, 4);
            c = (uint8_t)(tb - 0x4A800000u);
        } else {
            uint32_t odd = (mb >> 22) & 1u;
            int64_t nb = (int64_t)mb - ((int64_t)126 << 23) + (1 << 21) - 1 + (int64_t)odd;
            c = (uint8_t)((nb >> 22) & 0xFF);
        }
        code[i] = c | sign;
    }
    for (int i = 0; i < 16; i++) packed16[i] = (uint8_t)(code[2 * i] | (code[2 * i + 1] << 4));
}

static void decode_row(int fmt, const uint8_t *kv0, const uint8_t *kv1, const uint8_t *kv2,
                       int64_t stride0, int64_t stride1, int64_t stride2,
                       float s0, float s2, int64_t slot, float *row) {
    if (fmt == MO_KV_FP8) {
        const uint8_t *p = kv0 + slot * stride0;
        for (int d = 0; d < QK_DIM; d++) row[d] = mo_e4m3fn_to_float(p[d]) * s0;
    } else if (fmt == MO_KV_MXFP4) {
        const uint8_t *p = kv0 + slot * stride0, *sc = kv1 + slot * stride1;
        for (int d = 0; d < QK_DIM; d++) {
            uint8_t byte = p[d >> 1];
            uint8_t nib = (d & 1) ? (byte >> 4) : (byte & 0xF);
            row[d] = mo_e2m1_to_float(nib) * mo_e8m0_to_float(sc[d >> 5]);
        }
    } else {
        const uint8_t *p = kv0 + slot * stride0, *sc = kv1 + slot * stride1, *r = kv2 + slot * stride2;
        for (int d = 0; d < V_DIM; d++) {
            uint8_t byte = p[d >> 1];
            uint8_t nib = (d & 1) ? (byte >> 4) : (byte & 0xF);
            row[d] = mo_e2m1_to_float(nib) * mo_e8m0_to_float(sc[d >> 5]);
        }
        for (int d = 0; d < ROPE_DIM; d++) row[V_DIM + d] = mo_e4m3fn_to_float(r[d]) * s2;
    }
}

/*
 * q        fp32 [batch*q_len, heads, 576] (already dequantised by the caller)
 * kv0/1/2  cache planes (fp8: codes | mxfp4: codes, e8m0 | hybrid: latent codes, latent e8m0, rope codes)
 * s0, s2   per-tensor scales (fp8 codes: s0; hybrid rope: s2)
 * out      fp32 [batch*q_len, heads, 512];  lse fp32 [batch*q_len, heads]
 * pos_offset/total_len (nullable) position of the first key of each sequence's range inside the
 *          full sequence and the full length, for the causal mask on a KV shard.
 */
int mo_mla_decode(const float *q, int fmt, const uint8_t *kv0, const uint8_t *kv1, const uint8_t *kv2,
                  int64_t stride0, int64_t stride1, int64_t stride2, float s0, float s2,
                  const int32_t *kv_indptr, const int32_t *kv_indices, int batch, int heads,
                  int q_len, int causal, const int32_t *pos_offset, const int32_t *total_len,
                  float sm_scale, float *out, float *lse) {
    float *row = (float *)malloc(sizeof(float) * QK_DIM);
    float *acc = (float *)malloc(sizeof(float) * V_DIM);
    if (!row || !acc) return -1;
    for (int b = 0; b < batch; b++) {
        int k0 = kv_indptr[b], k1 = kv_indptr[b + 1];
        int off = pos_offset ? pos_offset[b] : 0;
        int tot = total_len ? total_len[b] : (k1 - k0);
        for (int j = 0; j < q_len; j++) {
            for (int h = 0; h < heads; h++) {
                const float *qr = q + ((int64_t)(b * q_len + j) * heads + h) * QK_DIM;
                float mx = -INFINITY, sum = 0.0f;
                for (int v = 0; v < V_DIM; v++) acc[v] = 0.0f;
                for (int k = k0; k < k1; k++) {
                    int pos = off + (k - k0);
                    if (causal && q_len > 1 && pos > tot - q_len + j) continue;
                    int64_t slot = kv_indices ? kv_indices[k] : k;
                    decode_row(fmt, kv0, kv1, kv2, stride0, stride1, stride2, s0, s2, slot, row);
                    float sc = 0.0f;
                    for (int d = 0; d < QK_DIM; d++) sc += qr[d] * row[d];
                    sc *= sm_scale;
                    float nm = fmaxf(mx, sc);
                    float alpha = (mx == -INFINITY) ? 0.0f : expf(mx - nm);
                    float w = expf(sc - nm);
                    for (int v = 0; v < V_DIM; v++) acc[v] = acc[v] * alpha + w * row[v];
                    sum = sum * alpha + w;
                    mx = nm;
                }
                float *o = out + ((int64_t)(b * q_len + j) * heads + h) * V_DIM;
                float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
                for (int v = 0; v < V_DIM; v++) o[v] = acc[v] * inv;
                lse[(int64_t)(b * q_len + j) * heads + h] = sum > 0.0f ? mx + logf(sum) : -INFINITY;
            }
        }
    }
    free(row); free(acc);
    return 0;
}
