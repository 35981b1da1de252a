/*
 * cc_b200_seq.h -- C ABI of the position-addressed sequence kernels (libcc_b200_seq.so).
 *
 * These serve decoder designs that append every token to a slot cache in order (slot = position mod capacity:
 * a full cache while capacity >= sequence length, a ring for sliding-window layers) and need their attention
 * arithmetic in fp32: softmax with a sink term in the denominator, optional sliding window, unit-RMS q/k with a
 * position-dependent query gain, value mixing across layers, post-sum normalisation, a clamped gated feed-forward,
 * and a token + hashed-bigram + sinusoid embedding.
 *
 * Plain pointers and sizes only.  Every function returns 0 on success and a negative CC_ERR_* code (cc_b200.h
 * values) on failure; cc_seq_last_error() gives the message.  All pointers are DEVICE pointers owned by the caller.
 * Every call enqueues work on the caller's stream and never synchronises; positions are read from device memory,
 * so a decode step can be captured in a CUDA graph.
 */
#ifndef CC_B200_SEQ_H
#define CC_B200_SEQ_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CC_SEQ_ABI_VERSION 1

#define CC_SEQ_OK                     0
#define CC_SEQ_ERR_INVALID_ARG       -1
#define CC_SEQ_ERR_UNSUPPORTED_SHAPE -2
#define CC_SEQ_ERR_CUDA              -3

/* element types of activations, weights and cache rows */
#define CC_DT_F32   0
#define CC_DT_BF16  1

/* what the softmax denominator contains besides the keys */
#define CC_SINK_NONE     0
#define CC_SINK_LEARNED  1  /* exp(sink[h]), one fp32 logit per query head */
#define CC_SINK_ZERO     2  /* exp(0) = 1                                  */

/*
 * One attention layer's step over a chunk of T consecutive tokens whose first position is *input_pos.
 * Query i (position p = *input_pos + i) sees key position j when j <= p and (window == 0 or p - j < window).
 * Keys j >= *input_pos are rows of k_new / v_new; older keys are read from cache slot j mod L and count only if
 * pos[slot] == j (an empty, stale or overwritten slot is not a key).
 */
typedef struct CcSeqAttn {
    const float* q;            /* [T, H, Dk] fp32, already normalised and scaled by the query gain */
    const void* k_new;         /* [T, G, Dk] cache dtype */
    const void* v_new;         /* [T, G, Dv] cache dtype */
    void* k_cache;             /* [G, L, Dk] cache dtype */
    void* v_cache;             /* [G, L, Dv] cache dtype */
    int32_t* pos;              /* [L] position held by each slot, -1 = empty */
    uint8_t* mask;             /* [G, L] 1 = slot filled (may be NULL) */
    int32_t* cache_cts;        /* [1] number of filled slots (may be NULL) */
    const int32_t* input_pos;  /* [1] */
    void* y;                   /* [T, H, Dv] y dtype */
    const float* sink;         /* [H] fp32 for CC_SINK_LEARNED, else NULL */
    int32_t T, H, G, Dk, Dv, L;
    int32_t window;            /* 0 = every earlier key */
    int32_t sink_mode;
    int32_t cache_dtype, y_dtype;
    float scale;               /* multiplies q.k */
    int32_t append;            /* decode only (T == 1): also write the new row into its slot */
    void* workspace;           /* decode only: cc_seq_decode_workspace() bytes, zeroed once by the caller */
    uint64_t workspace_bytes;
} CcSeqAttn;

int cc_seq_abi_version(void);
const char* cc_seq_last_error(void);

/* x[t] = embed[tok[t]] * scale + bigram[row(t)] + sinusoid(pos(t)), fp32 [T, E] (and a copy in act dtype if x_act).
 * row(t) = (prev * mul_prev + tok * mul_cur) mod buckets with prev the token before (from *prev_token for t = 0),
 * row = buckets for position 0.  bigram may be NULL.  *prev_token is updated to tok[T-1].
 * inv_freq [ceil(E/2)] fp32: entry 2i = sin(p * inv_freq[i]), 2i+1 = cos(same). */
int cc_seq_embed(const int32_t* tokens, const int32_t* input_pos, int32_t* prev_token, const void* embed,
                 const void* bigram, const float* inv_freq, float* x, void* x_act, int32_t T, int32_t E, float scale,
                 int32_t buckets, int32_t mul_prev, int32_t mul_cur, int32_t table_dtype, int32_t act_dtype, void* stream);

/* Splits a fused projection row [H*Dk | G*Dk | G*Dv] (in_dtype, plus the fp32 bias row when given) per token: q and k heads divided by their root mean
 * square (when unit_norm), q multiplied by 1 + gain_coef * ln(floor((p + 1) / gain_every) + 1) (when gain_every > 0),
 * v <- (1 - *mix_lambda) v + *mix_lambda v_first (when v_first).  q_out fp32, k_out / v_out in out_dtype. */
int cc_seq_qkv_prepare(const void* qkv, int32_t in_dtype, const float* bias, const int32_t* input_pos,
                       const float* mix_lambda, const void* v_first, float* q_out, void* k_out, void* v_out,
                       int32_t out_dtype, int32_t T, int32_t H, int32_t G, int32_t Dk, int32_t Dv, float eps,
                       int32_t unit_norm, float gain_coef, int32_t gain_every, void* stream);

/* Attention of a chunk (any T >= 1) over cache + chunk; the cache is not written. */
int cc_seq_attention(const CcSeqAttn* a, void* stream);
/* T == 1: keys split over CTAs, partial results combined in split order by the last CTA of a head; with
 * a->append the new row is written to slot p mod L (k, v, pos, mask, cache_cts) by the same launch. */
int cc_seq_attention_decode(const CcSeqAttn* a, void* stream);
uint64_t cc_seq_decode_workspace(int32_t H, int32_t G, int32_t Dv, int32_t L, int32_t window);
/* Writes rows of k_new / v_new into slots (p mod L); of a chunk longer than L only the last L rows. */
int cc_seq_cache_append(const CcSeqAttn* a, void* stream);

/* x <- unit_rms(alpha * x + y) * (1 + w), fp32 [T, E] in place; y (y_dtype) may be NULL; a copy in act dtype goes to
 * x_act when given. */
int cc_seq_residual_norm(float* x, const void* y, int32_t y_dtype, const float* w, float alpha, float eps, void* x_act,
                         int32_t act_dtype, int32_t T, int32_t E, void* stream);

/* gu [T, 2F] = [gate | up] (io dtype): g = min(gate, limit), u = clamp(up, -limit, limit),
 * out [T, F] = g * sigmoid(slope * g) * (u + 1). */
int cc_seq_clamped_glu(const void* gu, void* out, int32_t io_dtype, int32_t out_dtype, float limit, float slope,
                       int32_t T, int32_t F, void* stream);

/*
 * One-token matrix-vector product out = epilogue(W xin) for the decode step, with the post-sum norm folded in:
 *   xin[k] = x[k]                                    (in_norm_w == NULL; x in x_dtype)
 *          = x[k] * rinv(x) * (1 + in_norm_w[k])      (x fp32 = a pre-norm sum; rinv = 1/sqrt(mean(x^2) + eps)),
 *            rounded to the weights' type, as the prompt path rounds its product inputs
 * epilogues (acc = W xin + bias in fp32):
 *   CC_GEMV_PLAIN     out[n] = acc                                             (fp32)
 *   CC_GEMV_RESIDUAL  out[n] = alpha * r[n] + acc, r = res or res * rinv(res) * (1 + res_norm_w)   (fp32 pre-norm sum)
 *   CC_GEMV_GLU       rows n and N + n of W: g = min(acc_n, limit), u = clamp(acc_{N+n}, +-limit),
 *                     out[n] = g * sigmoid(slope * g) * (u + 1)                 (out_dtype)
 * Every CTA recomputes the row statistics it needs (K and N floats from L2) instead of waiting for a norm kernel.
 */
#define CC_GEMV_PLAIN     0
#define CC_GEMV_RESIDUAL  1
#define CC_GEMV_GLU       2

typedef struct CcSeqGemv {
    const void* x;  int32_t x_dtype;
    const float* in_norm_w;
    const void* W;  int32_t w_dtype;      /* [N (2N for GLU), K] row-major */
    const float* bias;                    /* [N] or NULL (not with GLU) */
    const float* res;                     /* [N] fp32, RESIDUAL only */
    const float* res_norm_w;              /* [N] or NULL */
    float alpha, eps, limit, slope;
    int32_t mode;
    void* out;      int32_t out_dtype;
    int32_t N, K;
} CcSeqGemv;

int cc_seq_gemv(const CcSeqGemv* g, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CC_B200_SEQ_H */
