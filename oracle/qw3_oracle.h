/*
 * CPU oracle for the AWQ W4A16 decode path of the Qwen3-8B-shape decoder.
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, on the host, the arithmetic of the
 * reference's single translation unit (Inference.cu) so that the CUDA path can be checked
 * against it.  Nothing in the shipped library links, loads or calls it.
 *
 * PINNING: the reference ships no tests, no golden vectors and no CPU path, and its file does not compile as a
 * whole.  Its device kernels do: build_ref.py compiles them from the reference checkout into _ref/ and the GPU tests
 * run them beside this oracle.  Pinned that way: orc_dequant and orc_rope (bit for bit), orc_rmsnorm and orc_gelu
 * (up to the reference's fp32 summation order and the device's erff), orc_gemm_w4a16 (the reference's cublasGemmEx
 * call, same operands and leading dimensions, on the buffer its own dequantAwqKernel wrote: never more than the last
 * fp16 bit apart).  PARITY UNPINNED for the rest (the attention, whose reference kernel is broken and is never run,
 * and the token loop, which does not compile): anchored by a second, independent numpy restatement of the same rules
 * and by the committed fixtures under tests/golden/.
 *
 * Every function cites the reference lines (Inference.cu:N) whose arithmetic it follows.
 * All fp16 values cross this interface as raw uint16_t bit patterns.
 */
#ifndef QW3_ORACLE_H
#define QW3_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- seeded synthetic data (counter-based, order-independent) ------------------------ */

/* Tensor kinds used to key the random streams; tag = layer * 64 + kind. */
enum OrcKind {
    ORC_WQKV = 0, ORC_WQKV_SCALE = 1, ORC_WQKV_ZP = 2,
    ORC_WO = 3,   ORC_WO_SCALE = 4,   ORC_WO_ZP = 5,
    ORC_W1 = 6,   ORC_W1_SCALE = 7,   ORC_W1_ZP = 8,
    ORC_W2 = 9,   ORC_W2_SCALE = 10,  ORC_W2_ZP = 11,
    ORC_GAMMA = 12,
    ORC_EMB = 13, ORC_EMB_SCALE = 14, ORC_EMB_ZP = 15,
    ORC_UNEMB = 16, ORC_UNEMB_SCALE = 17, ORC_UNEMB_ZP = 18,
    ORC_ACT = 19, ORC_KV_K = 20, ORC_KV_V = 21, ORC_TOKENS = 22
};

uint64_t orc_mix64(uint64_t x);
uint64_t orc_stream_key(uint64_t seed, uint64_t tag);
/* n bytes, each holding two uniform 4-bit codes (low nibble first). */
void orc_gen_codes(uint64_t seed, uint64_t tag, int64_t n_bytes, uint8_t* out);
/* fp16( mean + std * N(0,1) ), or fp16(|..|) when take_abs != 0. */
void orc_gen_normal_f16(uint64_t seed, uint64_t tag, int64_t n, double mean, double std,
                        int take_abs, uint16_t* out);
/* fp16 of a uniform integer in [lo, hi]. */
void orc_gen_uniform_int_f16(uint64_t seed, uint64_t tag, int64_t n, int lo, int hi, uint16_t* out);
void orc_gen_tokens(uint64_t seed, uint64_t tag, int64_t n, int vocab, int32_t* out);

/* ---- operators ------------------------------------------------------------------------ */

/* Inference.cu:76-106 (dequantAwqKernel): out[r*cols+c] = hmul(hsub(half(q), zp[g]), scale[g]),
 * g = (c / group) mod n_groups_alloc.  The reference allocates rows/group entries and indexes
 * them by c/group; the wrap makes the out-of-range cases (w2, word_embedding) defined and is
 * the identity wherever the reference is in range. */
void orc_dequant(const uint8_t* packed, const uint16_t* scale, const uint16_t* zp,
                 int64_t n_groups_alloc, int64_t rows, int64_t cols, int group, uint16_t* out_f16);

/* Inference.cu:1052-1065 (and 1128,1176,1201,1260): the dequantised row-major buffer is handed
 * to cuBLAS as a column-major M x K matrix with lda = M, so
 *   y[i] = sum_j Wflat[i + j*M] * x[j],  Wflat = the dequantised buffer read as a flat array.
 * Products of fp16 operands are exact in fp32; they are accumulated in double (acc64 != 0) or
 * in float in j order (acc64 == 0).  y_f32 receives the unrounded sum, y_f16 the fp16 store the
 * reference performs (Inference.cu:1062).  n_rows_x > 1 gives the batched contraction:
 * x is [n_rows_x][K], outputs are [n_rows_x][M]. */
void orc_gemm_w4a16(const uint8_t* packed, const uint16_t* scale, const uint16_t* zp,
                    int64_t n_groups_alloc, int64_t M, int64_t K, int group,
                    const uint16_t* x_f16, int64_t n_rows_x, int acc64,
                    float* y_f32, uint16_t* y_f16);

/* Inference.cu:111-145 (rmsNormKernel): fp32 sum of squares (accumulated here in double, which
 * is within fp32 rounding of any summation order), scale = half(rsqrt(mean + eps)),
 * out = hmul(hmul(x, scale), gamma). */
void orc_rmsnorm(const uint16_t* x, const uint16_t* gamma, int64_t n, float eps, uint16_t* out);

/* Inference.cu:444-454: fp16 cos/sin tables [max_pos][head_dim/2], inv_freq = 1/powf(base, 2i/d). */
void orc_rope_tables(int max_pos, int head_dim, float base, uint16_t* cos_t, uint16_t* sin_t);
/* Inference.cu:150-177 (applyRotaryKernel): interleaved pairs, every product and sum in fp16. */
void orc_rope(uint16_t* qk, int heads, int head_dim, const uint16_t* cos_t, const uint16_t* sin_t, int pos);

/* Inference.cu:182-266 (attentionKernel), intended math with the shared-memory aliasing
 * repaired: per head, fp32 q.k / sqrt(d), max-subtracted softmax over positions 0..len-1,
 * fp32 sum of p*v, one rounding to fp16.  Caches are [heads][max_pos][head_dim]. */
void orc_attention(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                   int heads, int head_dim, int64_t max_pos, int64_t len, uint16_t* ctx);

/* Inference.cu:271-279 (geluKernel): 0.5*v*(1+erff(v*0.70710678f)) in fp32, stored as fp16. */
void orc_gelu(uint16_t* x, int64_t n);
/* Inference.cu:1149-1154: out = hadd(a, b). */
void orc_add(const uint16_t* a, const uint16_t* b, int64_t n, uint16_t* out);
/* Inference.cu:1278-1290: fp16 logits compared as float, strict '>', lowest index wins. */
int64_t orc_argmax_f16(const uint16_t* logits, int64_t n);
/* Inference.cu:1310-1315 (gather lambda): out[idx] = Wdq[tok + idx*vocab] for the embedding
 * stored as [hidden][vocab]; read straight from the packed stream. */
void orc_embed_gather(const uint8_t* packed, const uint16_t* scale, const uint16_t* zp,
                      int64_t n_groups_alloc, int64_t hidden, int64_t vocab, int group,
                      int64_t tok, uint16_t* out);

/* ---- whole model ---------------------------------------------------------------------- */

typedef struct OrcConfig {
    int32_t hidden;       /* Inference.cu:33  (4096)   */
    int32_t inter;        /* Inference.cu:34  (12288)  */
    int32_t heads;        /* Inference.cu:35  (32)     */
    int32_t head_dim;     /* Inference.cu:36  (128)    */
    int32_t layers;       /* Inference.cu:37  (36)     */
    int32_t vocab;        /* Inference.cu:38  (151936) */
    int32_t max_pos;      /* Inference.cu:39  (40960): KV rows and RoPE table rows kept */
    int32_t group;        /* Inference.cu:40  (128)    */
    float   eps;          /* Inference.cu:41  (1e-6)   */
    float   rope_base;    /* Inference.cu:449 (10000)  */
    int32_t sample_first; /* 0 = reference flow (Inference.cu:1355-1363): decode step 0 feeds the
                             last prompt token's final hidden state back into layer 0 */
} OrcConfig;

void orc_config_default(OrcConfig* c);

typedef struct OrcModel OrcModel;
OrcModel* orc_model_new(const OrcConfig* cfg);
void      orc_model_free(OrcModel* m);
/* Fill every weight from the seeded generator (same bytes orc_write_weight_dir writes). */
int orc_model_init_random(OrcModel* m, uint64_t seed);
/* Read the raw .bin set named as in Inference.cu:780-900.  Returns 0, or -1 on a missing/short file. */
int orc_model_load_dir(OrcModel* m, const char* dir);
int orc_write_weight_dir(const OrcConfig* cfg, uint64_t seed, const char* dir);
/* KV rows [0, upto) of every layer <- fp16 N(0,1) (seeded), as the one-layer config asks. */
void orc_model_fill_kv(OrcModel* m, uint64_t seed, int64_t upto);
/* Inference.cu:1029-1230 (runOneLayer) for one token at `pos`; hidden is updated in place.
 * Attention length is pos+1 in every layer (a token attends to itself and all earlier rows). */
void orc_model_layer(OrcModel* m, int layer, int64_t pos, uint16_t* hidden);
/* Inference.cu:1235-1292 (sampleNextToken): final norm with the last layer's gamma, unembed,
 * fp16 logits, argmax.  logits_f16 (vocab) may be NULL. */
int64_t orc_model_sample(OrcModel* m, const uint16_t* hidden, uint16_t* logits_f16);
/* Inference.cu:1297-1408 (generateResponse).  out_ids gets max_new ids.  last_logits_f16 (vocab,
 * may be NULL) receives the logits of the last decode step; margins (max_new floats, may be NULL)
 * the top-1 minus top-2 logit of each step. Returns 0 or -1 (sequence would exceed max_pos). */
int orc_model_generate(OrcModel* m, const int32_t* prompt, int32_t n_prompt, int32_t max_new,
                       int32_t* out_ids, uint16_t* last_logits_f16, float* margins);
/* The same flow with probes for the golden fixtures: per decode step the eight largest fp16 logits (top_idx,
 * top_val: [max_new][8], larger value first, lower index first among equals) and the hidden state after the layers
 * probe_layers[] at the positions probe_pos[] (probe_hidden: [n_probe_pos][n_probe_layers][hidden] fp16).  Any
 * output pointer may be NULL. */
int orc_model_generate_trace(OrcModel* m, const int32_t* prompt, int32_t n_prompt, int32_t max_new,
                             int32_t* out_ids, uint16_t* last_logits_f16, float* margins, int32_t* top_idx,
                             uint16_t* top_val, const int32_t* probe_layers, int32_t n_probe_layers,
                             const int32_t* probe_pos, int32_t n_probe_pos, uint16_t* probe_hidden);
/* Raw access for tests (pointers into the model; do not free). */
const uint8_t*  orc_model_packed(OrcModel* m, int layer, int kind);
const uint16_t* orc_model_f16(OrcModel* m, int layer, int kind);
uint16_t*       orc_model_kv(OrcModel* m, int layer, int which /*0=K,1=V*/);

int orc_num_threads(void);
void orc_set_num_threads(int n);   /* host threads of the parallel loops (timing the baseline at 1 thread) */

#ifdef __cplusplus
}
#endif
#endif
