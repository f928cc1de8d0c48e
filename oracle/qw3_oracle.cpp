// CPU oracle for the AWQ W4A16 decode path.  TEST INFRASTRUCTURE ONLY -- see qw3_oracle.h.
// PARITY UNPINNED: the reference has no golden vectors and does not build; this file is a
// restatement of Inference.cu's arithmetic, cross-checked by an independent numpy version.
//
// fp16 arithmetic is done as "one fp32 operation, then one rounding to fp16".  For +, -, * of
// two fp16 operands this equals the directly rounded fp16 result (fp32 carries 24 >= 2*11+2
// significand bits, so the double rounding is innocuous); it is how __hadd/__hsub/__hmul
// behave on the device.
#include "qw3_oracle.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__AVX2__) && defined(__F16C__)
#include <immintrin.h>
#define ORC_AVX2 1
#endif

namespace {

inline float h2f(uint16_t h) {
    _Float16 v;
    std::memcpy(&v, &h, 2);
    return (float)v;
}
inline uint16_t f2h(float f) {
    _Float16 v = (_Float16)f;  // round-to-nearest-even, subnormals kept
    uint16_t h;
    std::memcpy(&h, &v, 2);
    return h;
}
inline float rh(float f) { return h2f(f2h(f)); }  // round an fp32 value to the fp16 grid
inline float hadd_(float a, float b) { return rh(a + b); }
inline float hsub_(float a, float b) { return rh(a - b); }
inline float hmul_(float a, float b) { return rh(a * b); }
// fma.rn.f16: a * b + c with ONE rounding.  The product of two fp16 values and its sum with a third are exact in
// double; the double is taken to float with round-to-odd so that the final float -> half rounding is the correct
// rounding of the exact value.
inline float hfma_(float a, float b, float c) {
    const double e = (double)a * (double)b + (double)c;
    float f = (float)e;
    if ((double)f != e) {
        if (std::fabs((double)f) > std::fabs(e)) f = std::nextafterf(f, 0.0f);
        uint32_t u;
        std::memcpy(&u, &f, 4);
        u |= 1u;
        std::memcpy(&f, &u, 4);
    }
    return rh(f);
}

constexpr uint64_t GOLD = 0x9E3779B97F4A7C15ull;
inline uint64_t mix64(uint64_t x) {
    x += GOLD;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
inline uint64_t draw(uint64_t key, uint64_t k) { return mix64(key + k * GOLD); }
inline double u01(uint64_t r) { return ((double)(r >> 11) + 0.5) * (1.0 / 9007199254740992.0); }
inline double normal(uint64_t key, uint64_t k) {
    double u1 = u01(draw(key, 2 * k)), u2 = u01(draw(key, 2 * k + 1));
    return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586476925 * u2);
}

// One dequantised weight, Inference.cu:92-104.
inline float dq(int q, float z, float s) { return hmul_(hsub_((float)q, z), s); }

// 16-entry table of the dequantised values of one group.
inline void group_lut(float z, float s, float* lut) {
    for (int q = 0; q < 16; ++q) lut[q] = dq(q, z, s);
}

}  // namespace

extern "C" {

uint64_t orc_mix64(uint64_t x) { return mix64(x); }
uint64_t orc_stream_key(uint64_t seed, uint64_t tag) { return mix64(seed ^ mix64(tag ^ 0xA5A5A5A55A5A5A5Aull)); }

void orc_gen_codes(uint64_t seed, uint64_t tag, int64_t n_bytes, uint8_t* out) {
    const uint64_t key = orc_stream_key(seed, tag);
    const int64_t nw = (n_bytes + 7) / 8;
#pragma omp parallel for schedule(static)
    for (int64_t w = 0; w < nw; ++w) {
        uint64_t r = draw(key, (uint64_t)w);
        int64_t lim = n_bytes - w * 8 < 8 ? n_bytes - w * 8 : 8;
        for (int64_t b = 0; b < lim; ++b) out[w * 8 + b] = (uint8_t)(r >> (8 * b));
    }
}

void orc_gen_normal_f16(uint64_t seed, uint64_t tag, int64_t n, double mean, double std_, int take_abs, uint16_t* out) {
    const uint64_t key = orc_stream_key(seed, tag);
#pragma omp parallel for schedule(static)
    for (int64_t k = 0; k < n; ++k) {
        double v = normal(key, (uint64_t)k);
        if (take_abs) v = std::fabs(v);
        out[k] = f2h((float)(mean + std_ * v));
    }
}

void orc_gen_uniform_int_f16(uint64_t seed, uint64_t tag, int64_t n, int lo, int hi, uint16_t* out) {
    const uint64_t key = orc_stream_key(seed, tag);
    const uint64_t span = (uint64_t)(hi - lo + 1);
    for (int64_t k = 0; k < n; ++k) out[k] = f2h((float)(lo + (int)(draw(key, (uint64_t)k) % span)));
}

void orc_gen_tokens(uint64_t seed, uint64_t tag, int64_t n, int vocab, int32_t* out) {
    const uint64_t key = orc_stream_key(seed, tag);
    for (int64_t k = 0; k < n; ++k) out[k] = (int32_t)(draw(key, (uint64_t)k) % (uint64_t)vocab);
}

void orc_dequant(const uint8_t* packed, const uint16_t* scale, const uint16_t* zp, int64_t n_groups_alloc,
                 int64_t rows, int64_t cols, int group, uint16_t* out) {
    const int64_t pc = (cols + 1) / 2;  // Inference.cu:93
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t c = 0; c < cols; ++c) {
            int64_t g = (c / group) % n_groups_alloc;
            uint8_t b = packed[r * pc + (c >> 1)];
            int q = (c & 1) ? (b >> 4) & 15 : b & 15;
            out[r * cols + c] = f2h(dq(q, h2f(zp[g]), h2f(scale[g])));
        }
    }
}

// Group of flat element f = i + j*M:  c = f mod K,  g = (c / group) mod n_alloc.
static inline int64_t group_of(int64_t i, int64_t j, int64_t M, int64_t K, int group, int64_t n_alloc) {
    return (((i + j * M) % K) / group) % n_alloc;
}

// Plain scalar contraction (any shape).  acc64 == 0: float accumulator in j order.
static void gemm_scalar(const uint8_t* packed, const uint16_t* scale, const uint16_t* zp, int64_t n_alloc,
                        int64_t M, int64_t K, int group, const uint16_t* x, int64_t R, int acc64,
                        float* y32, uint16_t* y16) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t r = 0; r < R; ++r) {
        for (int64_t i = 0; i < M; ++i) {
            double ad = 0.0;
            float af = 0.0f;
            for (int64_t j = 0; j < K; ++j) {
                int64_t f = i + j * M;
                uint8_t b = packed[f >> 1];
                int q = (f & 1) ? (b >> 4) & 15 : b & 15;
                int64_t g = group_of(i, j, M, K, group, n_alloc);
                float w = dq(q, h2f(zp[g]), h2f(scale[g]));
                float p = w * h2f(x[r * K + j]);  // exact: 11 x 11 significand bits
                if (acc64) ad += (double)p; else af += p;
            }
            float v = acc64 ? (float)ad : af;
            if (y32) y32[r * M + i] = v;
            if (y16) y16[r * M + i] = f2h(v);
        }
    }
}

#ifdef ORC_AVX2
// Blocked AVX2 contraction for M, K multiples of 128 and group 128: for each block of 128
// outputs the group of (block, j) is ((ib + j*Mb) mod Kb) mod n_alloc, one 16-entry table each.
static void gemm_fast(const uint8_t* packed, const uint16_t* scale, const uint16_t* zp, int64_t n_alloc,
                      int64_t M, int64_t K, const uint16_t* x, int64_t R, float* y32, uint16_t* y16) {
    const int64_t Mb = M / 128, Kb = K / 128;
    std::vector<float> luts((size_t)n_alloc * 16);
    for (int64_t g = 0; g < n_alloc; ++g) group_lut(h2f(zp[g]), h2f(scale[g]), &luts[(size_t)g * 16]);
    std::vector<float> xf((size_t)R * K);
    for (int64_t t = 0; t < R * K; ++t) xf[t] = h2f(x[t]);
    const __m256i shifts = _mm256_setr_epi32(0, 4, 8, 12, 16, 20, 24, 28);
    const __m256i m15 = _mm256_set1_epi32(15), m7 = _mm256_set1_epi32(7);
    constexpr int JB = 256;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int64_t r = 0; r < R; ++r) {
        for (int64_t ib = 0; ib < Mb; ++ib) {
            double acc[128];
            for (int t = 0; t < 128; ++t) acc[t] = 0.0;
            const float* xr = &xf[(size_t)r * K];
            for (int64_t j0 = 0; j0 < K; j0 += JB) {
                const int64_t j1 = j0 + JB < K ? j0 + JB : K;
                for (int ic = 0; ic < 4; ++ic) {  // 32 outputs = 16 bytes per row
                    __m256d a[8];
                    for (int t = 0; t < 8; ++t) a[t] = _mm256_loadu_pd(&acc[ic * 32 + t * 4]);
                    for (int64_t j = j0; j < j1; ++j) {
                        const int64_t g = ((ib + j * Mb) % Kb) % n_alloc;
                        const __m256 lo = _mm256_loadu_ps(&luts[(size_t)g * 16]);
                        const __m256 hi = _mm256_loadu_ps(&luts[(size_t)g * 16 + 8]);
                        const __m256 xv = _mm256_set1_ps(xr[j]);
                        const uint8_t* p = packed + j * (M / 2) + ib * 64 + ic * 16;
                        for (int wd = 0; wd < 4; ++wd) {
                            uint32_t word;
                            std::memcpy(&word, p + wd * 4, 4);
                            __m256i idx = _mm256_and_si256(_mm256_srlv_epi32(_mm256_set1_epi32((int)word), shifts), m15);
                            __m256 wlo = _mm256_permutevar8x32_ps(lo, idx);
                            __m256 whi = _mm256_permutevar8x32_ps(hi, idx);
                            __m256 w = _mm256_blendv_ps(wlo, whi, _mm256_castsi256_ps(_mm256_cmpgt_epi32(idx, m7)));
                            __m256 pr = _mm256_mul_ps(w, xv);  // exact product
                            a[wd * 2] = _mm256_add_pd(a[wd * 2], _mm256_cvtps_pd(_mm256_castps256_ps128(pr)));
                            a[wd * 2 + 1] = _mm256_add_pd(a[wd * 2 + 1], _mm256_cvtps_pd(_mm256_extractf128_ps(pr, 1)));
                        }
                    }
                    for (int t = 0; t < 8; ++t) _mm256_storeu_pd(&acc[ic * 32 + t * 4], a[t]);
                }
            }
            for (int t = 0; t < 128; ++t) {
                float v = (float)acc[t];
                if (y32) y32[r * M + ib * 128 + t] = v;
                if (y16) y16[r * M + ib * 128 + t] = f2h(v);
            }
        }
    }
}
#endif

void orc_gemm_w4a16(const uint8_t* packed, const uint16_t* scale, const uint16_t* zp, int64_t n_alloc,
                    int64_t M, int64_t K, int group, const uint16_t* x, int64_t R, int acc64,
                    float* y32, uint16_t* y16) {
#ifdef ORC_AVX2
    if (acc64 && group == 128 && M % 128 == 0 && K % 128 == 0) {
        gemm_fast(packed, scale, zp, n_alloc, M, K, x, R, y32, y16);
        return;
    }
#endif
    gemm_scalar(packed, scale, zp, n_alloc, M, K, group, x, R, acc64, y32, y16);
}

void orc_rmsnorm(const uint16_t* x, const uint16_t* gamma, int64_t n, float eps, uint16_t* out) {
    double acc = 0.0;
    for (int64_t i = 0; i < n; ++i) {
        float v = h2f(x[i]);
        acc += (double)(v * v);  // v*v is exact in fp32
    }
    float mean_sq = (float)acc / (float)n;            // Inference.cu:136
    float denom = 1.0f / std::sqrt(mean_sq + eps);    // Inference.cu:137 (rsqrtf)
    float scale = rh(denom);                          // Inference.cu:138
    for (int64_t i = 0; i < n; ++i)                   // Inference.cu:142-143
        out[i] = f2h(hmul_(hmul_(h2f(x[i]), scale), h2f(gamma[i])));
}

void orc_rope_tables(int max_pos, int head_dim, float base, uint16_t* cos_t, uint16_t* sin_t) {
    const int half = head_dim / 2;
#pragma omp parallel for schedule(static)
    for (int pos = 0; pos < max_pos; ++pos) {
        for (int i = 0; i < half; ++i) {
            float inv_freq = 1.0f / powf(base, float(2 * i) / float(head_dim));
            float angle = float(pos) * inv_freq;
            cos_t[(int64_t)pos * half + i] = f2h(cosf(angle));
            sin_t[(int64_t)pos * half + i] = f2h(sinf(angle));
        }
    }
}

void orc_rope(uint16_t* qk, int heads, int head_dim, const uint16_t* cos_t, const uint16_t* sin_t, int pos) {
    const int half = head_dim / 2;
    for (int h = 0; h < heads; ++h) {
        for (int p = 0; p < half; ++p) {
            float x0 = h2f(qk[h * head_dim + 2 * p]), x1 = h2f(qk[h * head_dim + 2 * p + 1]);
            float c = h2f(cos_t[(int64_t)pos * half + p]), s = h2f(sin_t[(int64_t)pos * half + p]);
            // Inference.cu:172-173 as the reference's build executes them: __hmul / __hsub / __hadd emit mul.f16 /
            // sub.f16 / add.f16 without a rounding modifier, and the compiler contracts the first product of each
            // line into the add (one fma), keeping the second product rounded (checked against the compiled kernel)
            float t0 = hfma_(x0, c, -hmul_(x1, s));
            float t1 = hfma_(x0, s, hmul_(x1, c));
            qk[h * head_dim + 2 * p] = f2h(t0);
            qk[h * head_dim + 2 * p + 1] = f2h(t1);
        }
    }
}

void orc_attention(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, int heads, int head_dim,
                   int64_t max_pos, int64_t len, uint16_t* ctx) {
    const float scale = 1.0f / std::sqrt((float)head_dim);  // Inference.cu:218
#pragma omp parallel for schedule(static)
    for (int h = 0; h < heads; ++h) {
        std::vector<float> s((size_t)len);
        const uint16_t* kh = kc + (int64_t)h * max_pos * head_dim;
        const uint16_t* vh = vc + (int64_t)h * max_pos * head_dim;
        float mx = -INFINITY;
        for (int64_t k = 0; k < len; ++k) {
            double acc = 0.0;
            for (int i = 0; i < head_dim; ++i) acc += (double)(h2f(q[h * head_dim + i]) * h2f(kh[k * head_dim + i]));
            s[k] = (float)acc * scale;
            mx = std::fmax(mx, s[k]);
        }
        double sum = 0.0;
        for (int64_t k = 0; k < len; ++k) {
            s[k] = expf(s[k] - mx);
            sum += s[k];
        }
        for (int i = 0; i < head_dim; ++i) {
            double acc = 0.0;
            for (int64_t k = 0; k < len; ++k) acc += (double)s[k] * (double)h2f(vh[k * head_dim + i]);
            ctx[h * head_dim + i] = f2h((float)(acc / sum));
        }
    }
}

void orc_gelu(uint16_t* x, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        float v = h2f(x[i]);
        float y = 0.5f * v * (1.0f + erff(v * 0.70710678f));
        x[i] = f2h(y);
    }
}

void orc_add(const uint16_t* a, const uint16_t* b, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = f2h(hadd_(h2f(a[i]), h2f(b[i])));
}

int64_t orc_argmax_f16(const uint16_t* logits, int64_t n) {
    int64_t best = 0;
    float bv = h2f(logits[0]);
    for (int64_t i = 1; i < n; ++i) {
        float v = h2f(logits[i]);
        if (v > bv) { bv = v; best = i; }
    }
    return best;
}

void orc_embed_gather(const uint8_t* packed, const uint16_t* scale, const uint16_t* zp, int64_t n_alloc,
                      int64_t hidden, int64_t vocab, int group, int64_t tok, uint16_t* out) {
    const int64_t pc = (vocab + 1) / 2;
    const int64_t g = (tok / group) % n_alloc;
    const float z = h2f(zp[g]), s = h2f(scale[g]);
    for (int64_t idx = 0; idx < hidden; ++idx) {
        uint8_t b = packed[idx * pc + (tok >> 1)];
        int q = (tok & 1) ? (b >> 4) & 15 : b & 15;
        out[idx] = f2h(dq(q, z, s));
    }
}

void orc_config_default(OrcConfig* c) {
    c->hidden = 4096; c->inter = 12288; c->heads = 32; c->head_dim = 128; c->layers = 36;
    c->vocab = 151936; c->max_pos = 40960; c->group = 128; c->eps = 1e-6f; c->rope_base = 10000.0f;
    c->sample_first = 0;
}

struct OrcW4 {
    std::vector<uint8_t> packed;
    std::vector<uint16_t> scale, zp;
    int64_t out_dim = 0, in_dim = 0, n_alloc = 0;
};

struct OrcModel {
    OrcConfig cfg;
    std::vector<OrcW4> wqkv, wo, w1, w2;
    std::vector<std::vector<uint16_t>> gamma;
    OrcW4 emb, unemb;
    std::vector<std::vector<uint16_t>> kc, vc;
    std::vector<uint16_t> cos_t, sin_t;
};

static void w4_shape(OrcW4& w, int64_t out_dim, int64_t in_dim, int group) {
    w.out_dim = out_dim; w.in_dim = in_dim; w.n_alloc = out_dim / group;   // Inference.cu:619
    w.packed.resize((size_t)(out_dim * ((in_dim + 1) / 2)));               // Inference.cu:617-618
    w.scale.resize((size_t)w.n_alloc); w.zp.resize((size_t)w.n_alloc);
}

OrcModel* orc_model_new(const OrcConfig* cfg) {
    OrcModel* m = new OrcModel();
    m->cfg = *cfg;
    const int L = cfg->layers, H = cfg->hidden, I = cfg->inter, V = cfg->vocab, G = cfg->group;
    m->wqkv.resize(L); m->wo.resize(L); m->w1.resize(L); m->w2.resize(L); m->gamma.resize(L);
    m->kc.resize(L); m->vc.resize(L);
    for (int l = 0; l < L; ++l) {
        w4_shape(m->wqkv[l], 3 * H, H, G); w4_shape(m->wo[l], H, H, G);
        w4_shape(m->w1[l], I, H, G);       w4_shape(m->w2[l], H, I, G);
        m->gamma[l].assign((size_t)H, 0);
        size_t kv = (size_t)cfg->heads * cfg->max_pos * cfg->head_dim;
        m->kc[l].assign(kv, 0); m->vc[l].assign(kv, 0);                    // Inference.cu:431-437
    }
    w4_shape(m->emb, H, V, G); w4_shape(m->unemb, V, H, G);
    m->cos_t.resize((size_t)cfg->max_pos * cfg->head_dim / 2);
    m->sin_t.resize(m->cos_t.size());
    orc_rope_tables(cfg->max_pos, cfg->head_dim, cfg->rope_base, m->cos_t.data(), m->sin_t.data());
    return m;
}

void orc_model_free(OrcModel* m) { delete m; }

static void w4_random(OrcW4& w, uint64_t seed, int layer, int kind) {
    orc_gen_codes(seed, (uint64_t)layer * 64 + kind, (int64_t)w.packed.size(), w.packed.data());
    orc_gen_normal_f16(seed, (uint64_t)layer * 64 + kind + 1, w.n_alloc, 0.0, 0.02, 1, w.scale.data());
    orc_gen_uniform_int_f16(seed, (uint64_t)layer * 64 + kind + 2, w.n_alloc, 6, 9, w.zp.data());
}

int orc_model_init_random(OrcModel* m, uint64_t seed) {
    for (int l = 0; l < m->cfg.layers; ++l) {
        w4_random(m->wqkv[l], seed, l, ORC_WQKV); w4_random(m->wo[l], seed, l, ORC_WO);
        w4_random(m->w1[l], seed, l, ORC_W1);     w4_random(m->w2[l], seed, l, ORC_W2);
        orc_gen_normal_f16(seed, (uint64_t)l * 64 + ORC_GAMMA, m->cfg.hidden, 1.0, 0.02, 0, m->gamma[l].data());
    }
    w4_random(m->emb, seed, 0, ORC_EMB);
    w4_random(m->unemb, seed, 0, ORC_UNEMB);
    return 0;
}

static int read_file(const std::string& fn, void* dst, size_t bytes) {
    FILE* f = std::fopen(fn.c_str(), "rb");
    if (!f) return -1;
    size_t got = std::fread(dst, 1, bytes, f);   // excess bytes are ignored, Inference.cu:303-304
    std::fclose(f);
    return got == bytes ? 0 : -1;
}
static int write_file(const std::string& fn, const void* src, size_t bytes) {
    FILE* f = std::fopen(fn.c_str(), "wb");
    if (!f) return -1;
    size_t put = std::fwrite(src, 1, bytes, f);
    std::fclose(f);
    return put == bytes ? 0 : -1;
}

// File names: Inference.cu:780-900.
static void w4_names(const std::string& dir, int layer, int kind, std::string& p, std::string& s, std::string& z) {
    std::string L = dir + "/layer_" + std::to_string(layer) + "_";
    switch (kind) {
        case ORC_WQKV: p = L + "wqkv.bin"; s = L + "bqkv_scale.bin"; z = L + "bqkv_zp.bin"; break;
        case ORC_WO:   p = L + "wo.bin";   s = L + "wo_scale.bin";   z = L + "wo_zp.bin";   break;
        case ORC_W1:   p = L + "w1.bin";   s = L + "w1_scale.bin";   z = L + "w1_zp.bin";   break;
        case ORC_W2:   p = L + "w2.bin";   s = L + "w2_scale.bin";   z = L + "w2_zp.bin";   break;
        case ORC_EMB:  p = dir + "/word_embedding.bin"; s = dir + "/word_embed_scale.bin"; z = dir + "/word_embed_zp.bin"; break;
        default:       p = dir + "/unembed.bin"; s = dir + "/unembed_scale.bin"; z = dir + "/unembed_zp.bin"; break;
    }
}
static int w4_io(OrcW4& w, const std::string& dir, int layer, int kind, bool wr) {
    std::string p, s, z;
    w4_names(dir, layer, kind, p, s, z);
    if (wr)
        return write_file(p, w.packed.data(), w.packed.size()) | write_file(s, w.scale.data(), w.scale.size() * 2) |
               write_file(z, w.zp.data(), w.zp.size() * 2);
    return read_file(p, w.packed.data(), w.packed.size()) | read_file(s, w.scale.data(), w.scale.size() * 2) |
           read_file(z, w.zp.data(), w.zp.size() * 2);
}
static int model_io(OrcModel* m, const std::string& dir, bool wr) {
    int rc = 0;
    for (int l = 0; l < m->cfg.layers; ++l) {
        rc |= w4_io(m->wqkv[l], dir, l, ORC_WQKV, wr); rc |= w4_io(m->wo[l], dir, l, ORC_WO, wr);
        rc |= w4_io(m->w1[l], dir, l, ORC_W1, wr);     rc |= w4_io(m->w2[l], dir, l, ORC_W2, wr);
        std::string g = dir + "/rms_norm_gamma_" + std::to_string(l) + ".bin";
        rc |= wr ? write_file(g, m->gamma[l].data(), m->gamma[l].size() * 2)
                 : read_file(g, m->gamma[l].data(), m->gamma[l].size() * 2);
    }
    rc |= w4_io(m->emb, dir, 0, ORC_EMB, wr);
    rc |= w4_io(m->unemb, dir, 0, ORC_UNEMB, wr);
    return rc ? -1 : 0;
}

int orc_model_load_dir(OrcModel* m, const char* dir) { return model_io(m, dir, false); }

int orc_write_weight_dir(const OrcConfig* cfg, uint64_t seed, const char* dir) {
    // Streams one tensor at a time so that the full-size model never sits in memory twice.
    OrcConfig c = *cfg;
    const int H = c.hidden, I = c.inter, V = c.vocab, G = c.group;
    int rc = 0;
    for (int l = 0; l < c.layers; ++l) {
        OrcW4 w;
        w4_shape(w, 3 * H, H, G); w4_random(w, seed, l, ORC_WQKV); rc |= w4_io(w, dir, l, ORC_WQKV, true);
        w4_shape(w, H, H, G);     w4_random(w, seed, l, ORC_WO);   rc |= w4_io(w, dir, l, ORC_WO, true);
        w4_shape(w, I, H, G);     w4_random(w, seed, l, ORC_W1);   rc |= w4_io(w, dir, l, ORC_W1, true);
        w4_shape(w, H, I, G);     w4_random(w, seed, l, ORC_W2);   rc |= w4_io(w, dir, l, ORC_W2, true);
        std::vector<uint16_t> g((size_t)H);
        orc_gen_normal_f16(seed, (uint64_t)l * 64 + ORC_GAMMA, H, 1.0, 0.02, 0, g.data());
        rc |= write_file(std::string(dir) + "/rms_norm_gamma_" + std::to_string(l) + ".bin", g.data(), g.size() * 2);
    }
    OrcW4 e;
    w4_shape(e, H, V, G); w4_random(e, seed, 0, ORC_EMB);   rc |= w4_io(e, dir, 0, ORC_EMB, true);
    w4_shape(e, V, H, G); w4_random(e, seed, 0, ORC_UNEMB); rc |= w4_io(e, dir, 0, ORC_UNEMB, true);
    return rc ? -1 : 0;
}

void orc_model_fill_kv(OrcModel* m, uint64_t seed, int64_t upto) {
    const OrcConfig& c = m->cfg;
    std::vector<uint16_t> tmp((size_t)c.heads * upto * c.head_dim);
    for (int l = 0; l < c.layers; ++l) {
        for (int which = 0; which < 2; ++which) {
            orc_gen_normal_f16(seed, (uint64_t)l * 64 + (which ? ORC_KV_V : ORC_KV_K), (int64_t)tmp.size(), 0.0, 1.0, 0, tmp.data());
            std::vector<uint16_t>& dst = which ? m->vc[l] : m->kc[l];
            for (int h = 0; h < c.heads; ++h)  // generated as [heads][upto][head_dim]
                std::memcpy(&dst[(size_t)h * c.max_pos * c.head_dim], &tmp[(size_t)h * upto * c.head_dim],
                            (size_t)upto * c.head_dim * 2);
        }
    }
}

static void gemv(const OrcW4& w, const uint16_t* x, uint16_t* y, int group) {
    orc_gemm_w4a16(w.packed.data(), w.scale.data(), w.zp.data(), w.n_alloc, w.out_dim, w.in_dim, group, x, 1, 1, nullptr, y);
}

void orc_model_layer(OrcModel* m, int l, int64_t pos, uint16_t* hidden) {
    const OrcConfig& c = m->cfg;
    const int H = c.hidden, I = c.inter, D = c.head_dim, NH = c.heads;
    std::vector<uint16_t> normed(H), qkv(3 * (size_t)H), ctx(H), tmp(H), mlp(I);
    orc_rmsnorm(hidden, m->gamma[l].data(), H, c.eps, normed.data());            // Inference.cu:1040
    gemv(m->wqkv[l], normed.data(), qkv.data(), c.group);                        // Inference.cu:1052
    uint16_t *q = qkv.data(), *k = qkv.data() + H, *v = qkv.data() + 2 * H;      // Inference.cu:1070-1072
    orc_rope(q, NH, D, m->cos_t.data(), m->sin_t.data(), (int)pos);              // Inference.cu:1082
    orc_rope(k, NH, D, m->cos_t.data(), m->sin_t.data(), (int)pos);              // Inference.cu:1087
    for (int h = 0; h < NH; ++h) {                                               // Inference.cu:1094-1103
        std::memcpy(&m->kc[l][((size_t)h * c.max_pos + pos) * D], k + h * D, D * 2);
        std::memcpy(&m->vc[l][((size_t)h * c.max_pos + pos) * D], v + h * D, D * 2);
    }
    orc_attention(q, m->kc[l].data(), m->vc[l].data(), NH, D, c.max_pos, pos + 1, ctx.data());
    gemv(m->wo[l], ctx.data(), tmp.data(), c.group);                             // Inference.cu:1128
    orc_add(hidden, tmp.data(), H, hidden);                                      // Inference.cu:1155
    orc_rmsnorm(hidden, m->gamma[l].data(), H, c.eps, normed.data());            // Inference.cu:1163 (same gamma)
    gemv(m->w1[l], normed.data(), mlp.data(), c.group);                          // Inference.cu:1176
    orc_gelu(mlp.data(), I);                                                     // Inference.cu:1196
    gemv(m->w2[l], mlp.data(), tmp.data(), c.group);                             // Inference.cu:1201
    orc_add(hidden, tmp.data(), H, hidden);                                      // Inference.cu:1227
}

int64_t orc_model_sample(OrcModel* m, const uint16_t* hidden, uint16_t* logits_out) {
    const OrcConfig& c = m->cfg;
    std::vector<uint16_t> normed(c.hidden), logits(c.vocab);
    orc_rmsnorm(hidden, m->gamma[c.layers - 1].data(), c.hidden, c.eps, normed.data());  // Inference.cu:1247-1253
    gemv(m->unemb, normed.data(), logits.data(), c.group);                               // Inference.cu:1260
    if (logits_out) std::memcpy(logits_out, logits.data(), (size_t)c.vocab * 2);
    return orc_argmax_f16(logits.data(), c.vocab);                                        // Inference.cu:1282-1289
}

static float top2_margin(const uint16_t* logits, int64_t n) {
    float a = -INFINITY, b = -INFINITY;
    for (int64_t i = 0; i < n; ++i) {
        float v = h2f(logits[i]);
        if (v > a) { b = a; a = v; } else if (v > b) b = v;
    }
    return a - b;
}

// The eight largest logits of a step, first-max order (larger value first, lower index first among equals).
static void top8(const uint16_t* logits, int64_t n, int32_t* idx, uint16_t* val) {
    float bv[8];
    int64_t bi[8];
    int cnt = 0;
    for (int64_t i = 0; i < n; ++i) {
        const float v = h2f(logits[i]);
        if (cnt == 8 && !(v > bv[7])) continue;
        int p = cnt < 8 ? cnt : 7;
        while (p > 0 && v > bv[p - 1]) { bv[p] = bv[p - 1]; bi[p] = bi[p - 1]; --p; }
        bv[p] = v; bi[p] = i;
        if (cnt < 8) ++cnt;
    }
    for (int k = 0; k < 8; ++k) {
        idx[k] = k < cnt ? (int32_t)bi[k] : -1;
        val[k] = k < cnt ? logits[bi[k]] : 0;
    }
}

// generateResponse (Inference.cu:1297-1408) with optional probes: per decode step the top-1 minus top-2 margin and
// the eight largest logits; the hidden state after the layers named in probe_layers at the positions named in
// probe_pos (probe_hidden is [n_probe_pos][n_probe_layers][hidden]).
int orc_model_generate_trace(OrcModel* m, const int32_t* prompt, int32_t n_prompt, int32_t max_new,
                             int32_t* out_ids, uint16_t* last_logits, float* margins, int32_t* top_idx, uint16_t* top_val,
                             const int32_t* probe_layers, int32_t n_probe_layers, const int32_t* probe_pos,
                             int32_t n_probe_pos, uint16_t* probe_hidden) {
    const OrcConfig& c = m->cfg;
    if (n_prompt < 1 || max_new < 0 || (int64_t)n_prompt + max_new > c.max_pos) return -1;
    for (int32_t t = 0; t < n_prompt; ++t)
        if (prompt[t] < 0 || prompt[t] >= c.vocab) return -1;
    std::vector<uint16_t> hidden(c.hidden), logits(c.vocab);
    auto embed = [&](int64_t tok) {
        orc_embed_gather(m->emb.packed.data(), m->emb.scale.data(), m->emb.zp.data(), m->emb.n_alloc,
                         c.hidden, c.vocab, c.group, tok, hidden.data());
    };
    auto layers_at = [&](int64_t pos) {
        int pi = -1;
        for (int32_t k = 0; k < n_probe_pos; ++k)
            if (probe_pos[k] == pos) pi = k;
        for (int l = 0; l < c.layers; ++l) {
            orc_model_layer(m, l, pos, hidden.data());
            if (pi >= 0 && probe_hidden)
                for (int32_t k = 0; k < n_probe_layers; ++k)
                    if (probe_layers[k] == l)
                        std::memcpy(probe_hidden + ((size_t)pi * n_probe_layers + k) * c.hidden, hidden.data(), (size_t)c.hidden * 2);
        }
    };
    for (int32_t t = 0; t < n_prompt; ++t) {                 // Inference.cu:1304-1343
        embed(prompt[t]);
        layers_at(t);
    }
    int64_t pos = n_prompt;
    for (int32_t step = 0; step < max_new; ++step) {         // Inference.cu:1352-1405
        bool run_layers = true;
        if (c.sample_first) {
            // Opt-in repair: the prompt's own next token is sampled before any further layer pass.
            if (step == 0) run_layers = false; else embed(out_ids[step - 1]);
        } else if (step > 0) {
            embed(out_ids[step - 1]);                        // Inference.cu:1392-1398, 1357
        }                                                    // step 0: hidden carried over, Inference.cu:1357
        if (run_layers) {
            layers_at(pos);
            ++pos;
        }
        out_ids[step] = (int32_t)orc_model_sample(m, hidden.data(), logits.data());
        if (margins) margins[step] = top2_margin(logits.data(), c.vocab);
        if (top_idx && top_val) top8(logits.data(), c.vocab, top_idx + (size_t)step * 8, top_val + (size_t)step * 8);
    }
    if (last_logits && max_new > 0) std::memcpy(last_logits, logits.data(), (size_t)c.vocab * 2);
    return 0;
}

int orc_model_generate(OrcModel* m, const int32_t* prompt, int32_t n_prompt, int32_t max_new,
                       int32_t* out_ids, uint16_t* last_logits, float* margins) {
    return orc_model_generate_trace(m, prompt, n_prompt, max_new, out_ids, last_logits, margins, nullptr, nullptr,
                                    nullptr, 0, nullptr, 0, nullptr);
}

static OrcW4* pick(OrcModel* m, int layer, int kind) {
    switch (kind) {
        case ORC_WQKV: case ORC_WQKV_SCALE: case ORC_WQKV_ZP: return &m->wqkv[layer];
        case ORC_WO: case ORC_WO_SCALE: case ORC_WO_ZP: return &m->wo[layer];
        case ORC_W1: case ORC_W1_SCALE: case ORC_W1_ZP: return &m->w1[layer];
        case ORC_W2: case ORC_W2_SCALE: case ORC_W2_ZP: return &m->w2[layer];
        case ORC_EMB: case ORC_EMB_SCALE: case ORC_EMB_ZP: return &m->emb;
        case ORC_UNEMB: case ORC_UNEMB_SCALE: case ORC_UNEMB_ZP: return &m->unemb;
        default: return nullptr;
    }
}
const uint8_t* orc_model_packed(OrcModel* m, int layer, int kind) {
    OrcW4* w = pick(m, layer, kind);
    return w ? w->packed.data() : nullptr;
}
const uint16_t* orc_model_f16(OrcModel* m, int layer, int kind) {
    if (kind == ORC_GAMMA) return m->gamma[layer].data();
    OrcW4* w = pick(m, layer, kind);
    if (!w) return nullptr;
    int rel = kind % 3;  // kinds are laid out as (packed, scale, zp) triples starting at multiples of 3 ...
    if (kind >= ORC_EMB) rel = (kind - ORC_EMB) % 3;  // ... except after ORC_GAMMA
    return rel == 1 ? w->scale.data() : rel == 2 ? w->zp.data() : nullptr;
}
uint16_t* orc_model_kv(OrcModel* m, int layer, int which) { return which ? m->vc[layer].data() : m->kc[layer].data(); }

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"
