/*
 * CPU restatement of the TurboQuant hot path — see tq_oracle.h for scope and the
 * parity statement.  TEST INFRASTRUCTURE ONLY.  Build with -O2 -ffp-contract=off
 * (no -ffast-math): every fp32 operation below must round exactly once, in the
 * order written, because the reference's results are reproduced bit for bit.
 */
#include "tq_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---- fp16 helpers ---------------------------------------------------------- */

uint16_t tqo_f32_to_f16(float v) {
    _Float16 h = (_Float16)v;
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

float tqo_f16_to_f32(uint16_t b) {
    _Float16 h;
    memcpy(&h, &b, 2);
    return (float)h;
}

/* ---- codebook (src/codebook.cpp) --------------------------------------------- */

/* src/codebook.cpp:16-45 */
static const float k_c1[] = {-0.7978845608f, 0.7978845608f};
static const float k_c2[] = {-1.510232f, -0.4527800f, 0.4527800f, 1.510232f};
static const float k_c3[] = {-2.152176f, -1.344318f, -0.756130f, -0.245379f,
                             0.245379f,  0.756130f,  1.344318f,  2.152176f};
static const float k_c4[] = {-2.732590f, -2.069017f, -1.618046f, -1.256231f, -0.942340f, -0.656759f,
                             -0.388048f, -0.128395f, 0.128395f,  0.388048f,  0.656759f,  0.942340f,
                             1.256231f,  1.618046f,  2.069017f,  2.732590f};
static const float k_c5[] = {-3.255544f, -2.685239f, -2.311434f, -2.022174f, -1.780580f, -1.569614f, -1.379896f,
                             -1.205655f, -1.043046f, -0.889350f, -0.742542f, -0.601049f, -0.463598f, -0.329119f,
                             -0.196679f, -0.065429f, 0.065429f,  0.196679f,  0.329119f,  0.463598f,  0.601049f,
                             0.742542f,  0.889350f,  1.043046f,  1.205655f,  1.379896f,  1.569614f,  1.780580f,
                             2.022174f,  2.311434f,  2.685239f,  3.255544f};

void tqo_boundaries(const float* c, int n, float* b) {
    for (int i = 0; i + 1 < n; ++i) b[i] = (c[i] + c[i + 1]) * 0.5f; /* :49-57 */
}

int tqo_codebook(int bits, float* centroids, float* boundaries) {
    const float* src;
    switch (bits) { /* :71-85 */
        case 1: src = k_c1; break;
        case 2: src = k_c2; break;
        case 3: src = k_c3; break;
        case 4: src = k_c4; break;
        case 5: src = k_c5; break;
        default: return -1;
    }
    int n = 1 << bits;
    memcpy(centroids, src, (size_t)n * sizeof(float));
    if (boundaries) tqo_boundaries(centroids, n, boundaries);
    return 0;
}

/* std::lower_bound over the boundaries: number of boundaries strictly below v,
 * so v == boundary falls in the lower bin (src/codebook.cpp:295-297). */
static inline int bin_of(float v, const float* bounds, int n_bounds) {
    int lo = 0, len = n_bounds;
    while (len > 0) {
        int half = len >> 1;
        if (bounds[lo + half] < v) {
            lo += half + 1;
            len -= half + 1;
        } else {
            len = half;
        }
    }
    return lo;
}

void tqo_codebook_quantize(const float* values, long n, const float* boundaries, int n_centroids, uint8_t* out) {
    for (long i = 0; i < n; ++i) {
        int idx = bin_of(values[i], boundaries, n_centroids - 1);
        if (idx >= n_centroids) idx = n_centroids - 1;
        out[i] = (uint8_t)idx;
    }
}

int tqo_fit_codebook(const float* data, long n, int bits, int iterations, float* c, float* b) {
    if (tqo_codebook(bits, c, b)) return -1;
    int nc = 1 << bits;
    if (n <= 0) return 0; /* :270-273 */
    double* sum = (double*)malloc(sizeof(double) * nc);
    long* cnt = (long*)malloc(sizeof(long) * nc);
    for (int it = 0; it < iterations; ++it) { /* :107-136 */
        tqo_boundaries(c, nc, b);
        for (int i = 0; i < nc; ++i) { sum[i] = 0.0; cnt[i] = 0; }
        for (long i = 0; i < n; ++i) {
            int idx = bin_of(data[i], b, nc - 1);
            if (idx >= nc) idx = nc - 1;
            sum[idx] += (double)data[i];
            cnt[idx]++;
        }
        float max_shift = 0.0f;
        for (int i = 0; i < nc; ++i) {
            if (cnt[i] > 0) {
                float nv = (float)(sum[i] / (double)cnt[i]);
                float shift = fabsf(nv - c[i]);
                if (shift > max_shift) max_shift = shift;
                c[i] = nv;
            }
        }
        if (max_shift < 1e-6f) break;
    }
    tqo_boundaries(c, nc, b);
    free(sum);
    free(cnt);
    return 0;
}

/* ---- rotation (src/rotation.cpp) ----------------------------------------------- */

float tqo_sign(uint32_t seed, uint32_t i) {
    uint32_t h = seed * 2654435761u + i * 2246822519u; /* :35-39 */
    h ^= h >> 16;
    h *= 0x45d9f3bu;
    h ^= h >> 16;
    return (h & 1u) ? 1.0f : -1.0f;
}

static void fwht(float* d, int n) { /* :14-25 */
    for (int h = 1; h < n; h <<= 1)
        for (int i = 0; i < n; i += h << 1)
            for (int j = i; j < i + h; ++j) {
                float a = d[j], b = d[j + h];
                d[j] = a + b;
                d[j + h] = a - b;
            }
}

static void wht_rows(float* buf, int rows, int cols, uint32_t seed, int bs, int inverse) {
    const float inv_sqrt = 1.0f / sqrtf((float)bs); /* :301, :333 */
    float* signs = (float*)malloc(sizeof(float) * (size_t)bs);
    for (int j = 0; j < bs; ++j) signs[j] = tqo_sign(seed, (uint32_t)j);
    int nb = cols / bs;
    for (int r = 0; r < rows; ++r) {
        float* row = buf + (size_t)r * cols;
        for (int b = 0; b < nb; ++b) {
            float* blk = row + (size_t)b * bs;
            if (!inverse) { /* :309-315 */
                for (int j = 0; j < bs; ++j) blk[j] *= signs[j];
                fwht(blk, bs);
                for (int j = 0; j < bs; ++j) blk[j] *= inv_sqrt;
            } else { /* :341-346: the product inv_sqrt*sign is formed first */
                fwht(blk, bs);
                for (int j = 0; j < bs; ++j) blk[j] *= inv_sqrt * signs[j];
            }
        }
    }
    free(signs);
}

int tqo_wht(const float* in, int rows, int cols, uint32_t seed, uint32_t block, int inverse, float* out) {
    if (block == 0 || (block & (block - 1)) || cols % (int)block) return -1; /* :374 */
    if (out != in) memcpy(out, in, sizeof(float) * (size_t)rows * cols);
    wht_rows(out, rows, cols, seed, (int)block, inverse);
    return 0;
}

/* ---- weight quantiser (src/quantizer.cpp) --------------------------------------- */

uint32_t tqo_derive_seed(const float* w, size_t n, uint32_t salt) {
    uint32_t hash = 2166136261u ^ salt; /* :18 */
    const uint8_t* bytes = (const uint8_t*)w;
    size_t byte_count = n * sizeof(float);
    size_t stride = (byte_count > 4096) ? (byte_count / 4096) : 1; /* :22 */
    for (size_t i = 0; i < byte_count; i += stride) {
        hash ^= bytes[i];
        hash *= 16777619u;
    }
    return hash;
}

static void row_norms(const float* m, int rows, int cols, float* norms) {
    for (int r = 0; r < rows; ++r) {
        float acc = 0.0f; /* sequential fp32, the shim's definition of sum(axis=1) */
        const float* p = m + (size_t)r * cols;
        for (int j = 0; j < cols; ++j) {
            float sq = p[j] * p[j];
            acc += sq;
        }
        norms[r] = sqrtf(acc);
    }
}

static inline float lookup(const float* c, int n, int idx) { /* src/codebook.cpp:314-317 */
    if (idx >= n) idx = n - 1;
    return c[idx];
}

int tqo_quantize_weight(const float* w, int out, int in, const float* cb_p, int n_p, const float* cb_r, int n_r,
                        int primary_bits, int residual_bits, uint32_t block, int shared_rotation,
                        uint8_t* packed_primary, uint8_t* packed_residual, float* norms, uint32_t* seeds) {
    if (block == 0 || (block & (block - 1)) || in % (int)block || (in & 1)) return -1;
    const size_t total = (size_t)out * in;
    const float scale = sqrtf((float)in); /* :51-52 */
    const float inv_scale = 1.0f / scale;
    float* bp = (float*)malloc(sizeof(float) * (size_t)(n_p > 1 ? n_p - 1 : 1));
    float* br = (float*)malloc(sizeof(float) * (size_t)(n_r > 1 ? n_r - 1 : 1));
    tqo_boundaries(cb_p, n_p, bp);
    tqo_boundaries(cb_r, n_r, br);

    float* orig_norm = (float*)malloc(sizeof(float) * (size_t)out);
    float* scaled = (float*)malloc(sizeof(float) * total);
    float* tmp = (float*)malloc(sizeof(float) * total);
    uint8_t* idx_p = (uint8_t*)malloc(total);
    uint8_t* idx_r = (uint8_t*)calloc(total, 1);

    row_norms(w, out, in, orig_norm); /* :56-59 */
    for (int r = 0; r < out; ++r) {   /* :62-66 */
        float safe = orig_norm[r] > 1e-10f ? orig_norm[r] : 1e-10f;
        for (int j = 0; j < in; ++j) scaled[(size_t)r * in + j] = w[(size_t)r * in + j] / safe;
    }
    uint32_t seed_p = tqo_derive_seed(w, total, 0u); /* :69-70 */
    uint32_t seed_r = tqo_derive_seed(w, total, 1u);

    wht_rows(scaled, out, in, seed_p, (int)block, 0);      /* :74 */
    for (size_t i = 0; i < total; ++i) scaled[i] *= scale; /* :78 */
    tqo_codebook_quantize(scaled, (long)total, bp, n_p, idx_p); /* :83 */

    if (primary_bits <= 4) { /* :94-111, pack :33-39 */
        for (size_t i = 0; i < total; i += 2) packed_primary[i / 2] = (idx_p[i] & 0x0F) | ((idx_p[i + 1] & 0x0F) << 4);
    } else {
        memcpy(packed_primary, idx_p, total);
    }

    memset(packed_residual, 0, total / 2); /* :115, :157-160 */
    if (residual_bits > 0) {
        for (size_t i = 0; i < total; ++i) tmp[i] = scaled[i] - lookup(cb_p, n_p, idx_p[i]); /* :118-123 */
        if (!shared_rotation) { /* :131-145 */
            for (size_t i = 0; i < total; ++i) tmp[i] *= inv_scale;
            wht_rows(tmp, out, in, seed_p, (int)block, 1);
            wht_rows(tmp, out, in, seed_r, (int)block, 0);
            for (size_t i = 0; i < total; ++i) tmp[i] *= scale;
        }
        tqo_codebook_quantize(tmp, (long)total, br, n_r, idx_r); /* :148 */
        for (size_t i = 0; i < total; i += 2) packed_residual[i / 2] = (idx_r[i] & 0x0F) | ((idx_r[i + 1] & 0x0F) << 4);
        /* the reconstruction below re-reads the packed nibbles (:179-183), so mask like the pack did */
        for (size_t i = 0; i < total; ++i) idx_r[i] &= 0x0F;
    }

    /* norm correction, :162-248 */
    if (residual_bits > 0 && shared_rotation) { /* :173-200 */
        for (size_t i = 0; i < total; ++i) {
            float comb = lookup(cb_p, n_p, idx_p[i]) + lookup(cb_r, n_r, idx_r[i]);
            tmp[i] = comb * inv_scale;
        }
        wht_rows(tmp, out, in, seed_p, (int)block, 1);
    } else {
        for (size_t i = 0; i < total; ++i) tmp[i] = lookup(cb_p, n_p, idx_p[i]) * inv_scale; /* :203-206 */
        wht_rows(tmp, out, in, seed_p, (int)block, 1);
        if (residual_bits > 0) { /* :208-231 */
            for (size_t i = 0; i < total; ++i) scaled[i] = lookup(cb_r, n_r, idx_r[i]) * inv_scale;
            wht_rows(scaled, out, in, seed_r, (int)block, 1);
            for (size_t i = 0; i < total; ++i) tmp[i] = tmp[i] + scaled[i];
        }
    }
    row_norms(tmp, out, in, norms); /* :237-240 */
    for (int r = 0; r < out; ++r) { /* :243-248 */
        float safe = norms[r] > 1e-10f ? norms[r] : 1e-10f;
        norms[r] = orig_norm[r] / safe;
    }
    seeds[0] = seed_p; /* :255-258 */
    seeds[1] = (shared_rotation && residual_bits > 0) ? 0u : seed_r;
    seeds[2] = block;

    free(bp); free(br); free(orig_norm); free(scaled); free(tmp); free(idx_p); free(idx_r);
    return 0;
}

/* ---- weight dequantiser (src/dequantizer.cpp) ------------------------------------ */

int tqo_dequantize_weight(const uint8_t* pp, int out, int p_cols, const uint8_t* pr, int r_cols, const float* norms,
                          const uint32_t* seeds, const float* cb_p, int n_p, const float* cb_r, int n_r,
                          uint32_t block, float* result) {
    const int primary_5bit = (p_cols == r_cols * 2); /* :72-74 */
    const int in = primary_5bit ? p_cols : p_cols * 2;
    if (block == 0 || (block & (block - 1)) || in % (int)block) return -1;
    const size_t total = (size_t)out * in;
    const float inv_scale = 1.0f / sqrtf((float)in); /* :76 */
    const uint32_t seed_p = seeds[0], seed_r = seeds[1];

    int has_residual = 0; /* :118-128 */
    for (size_t i = 0, n = (size_t)out * r_cols; i < n; ++i)
        if (pr[i]) { has_residual = 1; break; }
    const int shared = (seed_r == 0 && has_residual); /* :133 */

    if (shared && !primary_5bit) { /* :136-184 */
        float lut[256];
        memset(lut, 0, sizeof lut);
        for (int r = 0; r < 16; ++r)
            for (int p = 0; p < n_p && p < 16; ++p) lut[(r << 4) | p] = cb_p[p] + lookup(cb_r, n_r, r);
        for (int row = 0; row < out; ++row)
            for (int k = 0; k < p_cols; ++k) {
                uint8_t pb = pp[(size_t)row * p_cols + k], rb = pr[(size_t)row * p_cols + k];
                float even = lut[(pb & 0x0F) | ((rb & 0x0F) << 4)];
                float odd = lut[((pb >> 4) & 0x0F) | (rb & 0xF0)];
                result[(size_t)row * in + 2 * k] = even * inv_scale;
                result[(size_t)row * in + 2 * k + 1] = odd * inv_scale;
            }
        wht_rows(result, out, in, seed_p, (int)block, 1);
    } else {
        for (size_t i = 0; i < total; ++i) { /* :83-106 */
            int idx = primary_5bit ? pp[i] : ((i & 1) ? (pp[i >> 1] >> 4) & 0x0F : pp[i >> 1] & 0x0F);
            result[i] = lookup(cb_p, n_p, idx);
        }
        if (shared) { /* 5-bit shared: :186-212 */
            for (size_t i = 0; i < total; ++i) {
                int ridx = (i & 1) ? (pr[i >> 1] >> 4) & 0x0F : pr[i >> 1] & 0x0F;
                float comb = result[i] + lookup(cb_r, n_r, ridx);
                result[i] = comb * inv_scale;
            }
            wht_rows(result, out, in, seed_p, (int)block, 1);
        } else { /* dual rotation or primary only: :214-246 */
            for (size_t i = 0; i < total; ++i) result[i] *= inv_scale;
            wht_rows(result, out, in, seed_p, (int)block, 1);
            if (has_residual) {
                float* res = (float*)malloc(sizeof(float) * total);
                for (size_t i = 0; i < total; ++i) {
                    int ridx = (i & 1) ? (pr[i >> 1] >> 4) & 0x0F : pr[i >> 1] & 0x0F;
                    res[i] = lookup(cb_r, n_r, ridx) * inv_scale;
                }
                wht_rows(res, out, in, seed_r, (int)block, 1);
                for (size_t i = 0; i < total; ++i) result[i] = result[i] + res[i];
                free(res);
            }
        }
    }
    for (int row = 0; row < out; ++row) /* :249-253 */
        for (int j = 0; j < in; ++j) result[(size_t)row * in + j] *= norms[row];
    return 0;
}

void tqo_linear_from_dequant(const float* w, int out, int in, const float* x, int batch, float* y) {
    float* xh = (float*)malloc(sizeof(float) * (size_t)in);
    for (int b = 0; b < batch; ++b) {
        for (int j = 0; j < in; ++j) xh[j] = tqo_f16_to_f32(tqo_f32_to_f16(x[(size_t)b * in + j]));
        for (int r = 0; r < out; ++r) {
            /* double accumulation: this is the yardstick, so keep its own error negligible */
            double acc = 0.0;
            const float* wr = w + (size_t)r * in;
            for (int j = 0; j < in; ++j) acc += (double)wr[j] * (double)xh[j];
            y[(size_t)b * out + r] = (float)acc;
        }
    }
    free(xh);
}

/* ---- KV cache (src/kv_cache.cpp) --------------------------------------------------- */

uint32_t tqo_kv_seed(uint32_t layer, uint32_t which) {
    uint32_t h = layer; /* :32-39 */
    h ^= which + 0x9e3779b9u + (h << 6) + (h >> 2);
    h = (h ^ (h >> 16)) * 0x45d9f3bu;
    h = (h ^ (h >> 16)) * 0x45d9f3bu;
    h ^= h >> 16;
    return h;
}

int tqo_kv_encode(const float* x, long n, int d, uint32_t wht_seed, uint32_t qjl_seed, uint32_t* words, float* norms,
                  uint32_t* qjl_words, float* qjl_norms) {
    if (d <= 0 || (d & (d - 1))) return -1;
    float c[8], b[7];
    tqo_codebook(3, c, b);
    const float scale = sqrtf((float)d); /* :72 */
    const int wph = (d + 9) / 10, qph = (d + 31) / 32;
    float* v = (float*)malloc(sizeof(float) * (size_t)d);
    uint8_t* idx = (uint8_t*)malloc((size_t)d);
    for (long i = 0; i < n; ++i) {
        const float* p = x + (size_t)i * d;
        float sum_sq = 0.0f; /* :84-88 */
        for (int j = 0; j < d; ++j) sum_sq += p[j] * p[j];
        float norm = sqrtf(sum_sq);
        norms[i] = norm;
        float inv_norm = (norm > 1e-10f) ? (1.0f / norm) : 0.0f; /* :93 */
        for (int j = 0; j < d; ++j) v[j] = p[j] * inv_norm;
        wht_rows(v, 1, d, wht_seed, d, 0);         /* :100-103 */
        for (int j = 0; j < d; ++j) v[j] *= scale; /* :107-110 */
        tqo_codebook_quantize(v, d, b, 8, idx);    /* :115 */
        if (qjl_words) {                           /* :215-258 */
            float rsq = 0.0f;
            uint32_t* qw = qjl_words + (size_t)i * qph;
            for (int w = 0; w < qph; ++w) qw[w] = 0;
            for (int j = 0; j < d; ++j) {
                float r = v[j] - c[idx[j]];
                rsq += r * r;
                uint32_t hash = qjl_seed * 2654435761u + (uint32_t)j * 2246822519u;
                float s = (hash >> 31) ? 1.0f : -1.0f;
                if (r * s > 0.0f) qw[j >> 5] |= 1u << (j & 31);
            }
            qjl_norms[i] = sqrtf(rsq);
        }
        uint32_t* ow = words + (size_t)i * wph; /* :119-128 */
        for (int w = 0; w < wph; ++w) {
            uint32_t word = 0;
            for (int k = 0; k < 10 && w * 10 + k < d; ++k) word |= ((uint32_t)idx[w * 10 + k] & 7u) << (k * 3);
            ow[w] = word;
        }
    }
    free(v);
    free(idx);
    return 0;
}

static void kv_decode_f32(const uint32_t* w, float norm, int d, uint32_t seed, const float* c, float* out) {
    const float inv_scale = 1.0f / sqrtf((float)d);                                  /* :302 */
    for (int j = 0; j < d; ++j) out[j] = c[(w[j / 10] >> ((j % 10) * 3)) & 7u];      /* :327-334 */
    for (int j = 0; j < d; ++j) out[j] *= inv_scale;                                 /* :337-339 */
    wht_rows(out, 1, d, seed, d, 1);                                                 /* :342-346 */
    for (int j = 0; j < d; ++j) out[j] = out[j] * norm;                              /* :349-356 */
}

int tqo_kv_decode_fp16(const uint32_t* words, const float* norms, long n, int d, uint32_t seed, uint16_t* out) {
    if (d <= 0 || (d & (d - 1))) return -1;
    float c[8];
    tqo_codebook(3, c, NULL);
    const int wph = (d + 9) / 10;
    float* v = (float*)malloc(sizeof(float) * (size_t)d);
    for (long i = 0; i < n; ++i) {
        kv_decode_f32(words + (size_t)i * wph, norms[i], d, seed, c, v);
        for (int j = 0; j < d; ++j) out[(size_t)i * d + j] = tqo_f32_to_f16(v[j]); /* :364 */
    }
    free(v);
    return 0;
}

int tqo_attention(const float* q, int q_heads, int kv_heads, int d, int tokens, int start, int end,
                  const uint32_t* k_words, const float* k_norms, const uint32_t* v_words, const float* v_norms,
                  const uint32_t* qjl_words, const float* qjl_norms, uint32_t k_seed, uint32_t v_seed,
                  uint32_t qjl_seed, int use_qjl, float* out) {
    if (start < 0 || end > tokens || start >= end || q_heads % kv_heads) return -1;
    float c[8];
    tqo_codebook(3, c, NULL);
    const int wph = (d + 9) / 10, qph = (d + 31) / 32, group = q_heads / kv_heads, n = end - start;
    const float scale = 1.0f / sqrtf((float)d); /* src/attention_dispatch.cpp:35 */
    const float inv_scale_d = 1.0f / sqrtf((float)d);
    const double gamma = sqrt(2.0 / (3.14159265358979323846 * (double)d));
    float* kv = (float*)malloc(sizeof(float) * (size_t)d);
    float* qrot = (float*)malloc(sizeof(float) * (size_t)d);
    double* s = (double*)malloc(sizeof(double) * (size_t)n);
    double* acc = (double*)malloc(sizeof(double) * (size_t)d);
    for (int h = 0; h < q_heads; ++h) {
        const int kh = h / group;
        float* qh = qrot; /* fp16-rounded query (src/attention_dispatch.cpp:70) */
        for (int j = 0; j < d; ++j) qh[j] = tqo_f16_to_f32(tqo_f32_to_f16(q[(size_t)h * d + j]));
        if (use_qjl) wht_rows(qh, 1, d, k_seed, d, 0); /* rotate the query once instead of every key */
        double m = -INFINITY;
        for (int t = 0; t < n; ++t) {
            size_t rec = (size_t)(start + t) * kv_heads + kh;
            double dot = 0.0;
            if (!use_qjl) {
                kv_decode_f32(k_words + rec * wph, k_norms[rec], d, k_seed, c, kv);
                for (int j = 0; j < d; ++j) dot += (double)qh[j] * (double)tqo_f16_to_f32(tqo_f32_to_f16(kv[j]));
            } else {
                const uint32_t* w = k_words + rec * wph;
                const uint32_t* qw = qjl_words + rec * qph;
                double main = 0.0, corr = 0.0;
                for (int j = 0; j < d; ++j) {
                    main += (double)qh[j] * (double)c[(w[j / 10] >> ((j % 10) * 3)) & 7u];
                    uint32_t hash = qjl_seed * 2654435761u + (uint32_t)j * 2246822519u;
                    double sj = (hash >> 31) ? 1.0 : -1.0;
                    double bit = ((qw[j >> 5] >> (j & 31)) & 1u) ? 1.0 : -1.0;
                    corr += (double)qh[j] * sj * bit;
                }
                dot = (double)k_norms[rec] * (double)inv_scale_d * (main + gamma * (double)qjl_norms[rec] * corr);
            }
            s[t] = dot * (double)scale;
            if (s[t] > m) m = s[t];
        }
        double z = 0.0;
        for (int j = 0; j < d; ++j) acc[j] = 0.0;
        for (int t = 0; t < n; ++t) {
            double p = exp(s[t] - m);
            z += p;
            size_t rec = (size_t)(start + t) * kv_heads + kh;
            kv_decode_f32(v_words + rec * wph, v_norms[rec], d, v_seed, c, kv);
            if (!use_qjl)
                for (int j = 0; j < d; ++j) acc[j] += p * (double)tqo_f16_to_f32(tqo_f32_to_f16(kv[j]));
            else
                for (int j = 0; j < d; ++j) acc[j] += p * (double)kv[j];
        }
        for (int j = 0; j < d; ++j) out[(size_t)h * d + j] = (float)(acc[j] / z);
    }
    free(kv); free(qrot); free(s); free(acc);
    return 0;
}
