/*
 * CPU oracle for the Co-Me hot path, plain C with OpenMP.  TEST INFRASTRUCTURE ONLY: it is the multi-threaded
 * checker and the timed CPU baseline of the benchmark; the product library never links or calls it.
 *
 * It restates the reference's PyTorch fallback path; each function names the reference lines it follows
 * (paths relative to the reference project root).  The numpy twin `come_oracle.py` is pinned against the
 * reference itself; the CPU tests require this file to agree with the numpy twin bit for bit.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC come_oracle.c -o libcome_oracle.so -lm
 * (no fast-math and no contraction: the float32 sums must round exactly like the restated algorithm).
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- float32 <-> 16-bit storage rounding (values are carried as float32) ------------------------------ */
static float round_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    memcpy(&x, &u, 4);
    return x;
}
static float round_f16(float x) { return (float)(_Float16)x; }
static float round_kind(float x, int kind) { return kind == 2 ? round_bf16(x) : kind == 1 ? round_f16(x) : x; }

/* ---- merge: co_me.py:152-222 (plan :177-183,199-201; data :185-222) -------------------------------------
 * src_of[r] gives, for merge-order row r of a frame (prefix rows first, then M groups of G rows), the index
 * of the source token inside the frame; src_of == NULL means the identity (the plain 1-D operator).
 * kind: 0 float32, 1 float16, 2 bfloat16 -- the merged mean is accumulated in float32 left to right, divided
 * by G, and rounded once to the storage precision. Returns P (rows written). */
int64_t orc_merge(const float *tokens, int64_t B, int64_t N, int64_t C, int64_t prefix, int64_t G, int64_t M,
                  const uint8_t *mask, const int64_t *src_of, int kind, float *out, int64_t *offsets,
                  int64_t *rev, float *weight) {
    offsets[0] = 0;
    for (int64_t b = 0; b < B; ++b) {
        int64_t k = 0;
        for (int64_t m = 0; m < M; ++m) k += mask[b * M + m] != 0;
        offsets[b + 1] = offsets[b] + prefix + (M - k) * G + k;
    }
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t b = 0; b < B; ++b) {
        const float *tb = tokens + b * N * C;
        int64_t dst = offsets[b];
        for (int64_t s = 0; s < prefix; ++s, ++dst) {
            int64_t src = src_of ? src_of[s] : s;
            memcpy(out + dst * C, tb + src * C, (size_t)C * sizeof(float));
            weight[dst] = 1.0f;
            rev[b * N + src] = dst;
        }
        for (int64_t m = 0; m < M; ++m) {
            if (mask[b * M + m]) {
                float *o = out + dst * C;
                for (int64_t c = 0; c < C; ++c) o[c] = 0.0f;
                for (int64_t g = 0; g < G; ++g) {
                    int64_t r = prefix + m * G + g;
                    int64_t src = src_of ? src_of[r] : r;
                    const float *t = tb + src * C;
                    for (int64_t c = 0; c < C; ++c) o[c] = o[c] + t[c];
                    rev[b * N + src] = dst;
                }
                for (int64_t c = 0; c < C; ++c) o[c] = round_kind(o[c] / (float)G, kind);
                weight[dst] = (float)G;
                dst += 1;
            } else {
                for (int64_t g = 0; g < G; ++g, ++dst) {
                    int64_t r = prefix + m * G + g;
                    int64_t src = src_of ? src_of[r] : r;
                    memcpy(out + dst * C, tb + src * C, (size_t)C * sizeof(float));
                    weight[dst] = 1.0f;
                    rev[b * N + src] = dst;
                }
            }
        }
    }
    return offsets[B];
}

/* Merge-order -> source-token map of a frame for gh x gw windows over the top-left floor(H/gh)*gh x
 * floor(W/gw)*gw region of an H x W grid behind `start` special tokens (co_me_2d.py:26-35,193-211; a grid
 * that the windows do not tile exactly keeps its uncovered patches, in row-major order, right behind the
 * specials as part of the never-merged prefix). Returns the prefix length; src_of has start + H*W entries. */
int64_t orc_layout2d(int64_t start, int64_t H, int64_t W, int64_t gh, int64_t gw, int64_t *src_of) {
    int64_t Hc = (H / gh) * gh, Wc = (W / gw) * gw, n = 0;
    for (int64_t s = 0; s < start; ++s) src_of[n++] = s;
    for (int64_t y = 0; y < H; ++y)
        for (int64_t x = 0; x < W; ++x)
            if (y >= Hc || x >= Wc) src_of[n++] = start + y * W + x;
    int64_t prefix = n;
    for (int64_t wy = 0; wy < Hc / gh; ++wy)
        for (int64_t wx = 0; wx < Wc / gw; ++wx)
            for (int64_t iy = 0; iy < gh; ++iy)
                for (int64_t ix = 0; ix < gw; ++ix) src_of[n++] = start + (wy * gh + iy) * W + wx * gw + ix;
    return prefix;
}

/* ---- unmerge: co_me.py:241-254 -------------------------------------------------------------------------- */
void orc_split(const float *merged, const int64_t *rev, int64_t total, int64_t C, float *out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total; ++i) memcpy(out + i * C, merged + rev[i] * C, (size_t)C * sizeof(float));
}

/* ---- window selection: co_me_2d.py:268-298, co_me.py:54-73 ----------------------------------------------- */
static int cmp_float(const void *a, const void *b) {
    float x = *(const float *)a, y = *(const float *)b;
    return (x > y) - (x < y);
}
/* torch.quantile(v.float(), q) with linear interpolation: rank = q*(n-1) in float32 and a fused lerp,
 * fma(w, b-a, a) below weight 0.5 and fma(w-1, b-a, b) from there on. `scratch` holds n floats. */
static float quantile_linear(const float *v, int64_t n, float q, float *scratch) {
    memcpy(scratch, v, (size_t)n * sizeof(float));
    qsort(scratch, (size_t)n, sizeof(float), cmp_float);
    float rank = q * (float)(n - 1);
    float lo = floorf(rank), hi = ceilf(rank), w = rank - lo;
    float a = scratch[(int64_t)lo], b = scratch[(int64_t)hi], d = b - a;
    if (w < 0.5f) return fmaf(w, d, a);
    return fmaf(w - 1.0f, d, b);
}
/* mode 0 = ranking (quantile), 1 = absolute threshold, 2 = absolute threshold on confidences z-normalised per batch
 * element: (x - mean) / (std + 1e-3), unbiased std, every tensor operation rounded to `kind`, mean and variance
 * accumulated in float64 (co_me_2d.py:274-281, co_me.py:54-59). scope 0 = quantile over all S*M windows of a batch
 * element, 1 = over the M windows of each frame. conf [B, S*H*W] float32 carrying `kind`-precision values.
 * In modes 1 and 2 the threshold is rounded to `kind` first (a tensor compared with a Python number). */
int orc_select(const float *conf_in, int64_t B, int64_t S, int64_t H, int64_t W, int64_t gh, int64_t gw,
               float thr, int mode, int scope, int kind, float *means_out, uint8_t *mask) {
    int64_t Hm = H / gh, Wm = W / gw, M = Hm * Wm, F = B * S;
    float *means = means_out ? means_out : (float *)malloc((size_t)(F * M) * sizeof(float));
    if (!means) return -1;
    const float *conf = conf_in;
    float *norm = NULL;
    if (mode == 2) {
        const int64_t n = S * H * W;
        norm = (float *)malloc((size_t)(B * n) * sizeof(float));
        if (!norm) return -1;
        for (int64_t b = 0; b < B; ++b) {
            const float *x = conf_in + b * n;
            double sum = 0.0, sq = 0.0;
            for (int64_t i = 0; i < n; ++i) sum += (double)x[i];
            const double mean64 = sum / (double)n;
            for (int64_t i = 0; i < n; ++i) sq += ((double)x[i] - mean64) * ((double)x[i] - mean64);
            const float mean = round_kind((float)mean64, kind);
            const float sd = round_kind((float)sqrt(n > 1 ? sq / (double)(n - 1) : NAN), kind);
            const float den = round_kind(sd + 1e-3f, kind);
            for (int64_t i = 0; i < n; ++i) norm[b * n + i] = round_kind(round_kind(x[i] - mean, kind) / den, kind);
        }
        conf = norm;
    }
#pragma omp parallel for schedule(static)
    for (int64_t f = 0; f < F; ++f)
        for (int64_t m = 0; m < M; ++m) {
            int64_t wy = m / Wm, wx = m % Wm;
            float acc = 0.0f;
            for (int64_t iy = 0; iy < gh; ++iy)
                for (int64_t ix = 0; ix < gw; ++ix)
                    acc = acc + conf[f * H * W + (wy * gh + iy) * W + wx * gw + ix];
            means[f * M + m] = round_kind(acc / (float)(gh * gw), kind);
        }
    if (mode == 1 || mode == 2) {
        const float thr_k = round_kind(thr, kind);
        for (int64_t i = 0; i < F * M; ++i) mask[i] = means[i] < thr_k;
    } else {
        int64_t groups = scope == 0 ? B : F, n = scope == 0 ? S * M : M;
        float *scratch = (float *)malloc((size_t)n * sizeof(float));
        if (!scratch) return -1;
        for (int64_t g = 0; g < groups; ++g) {
            float t = quantile_linear(means + g * n, n, thr, scratch);
            for (int64_t i = 0; i < n; ++i) mask[g * n + i] = means[g * n + i] < t;
        }
        free(scratch);
    }
    if (!means_out) free(means);
    free(norm);
    return 0;
}

/* ---- biased attention: test/auto_test/test_flex_attention_bias.py:26-36 ----------------------------------
 * out = softmax(q k^T * scale + bias[None, :]) v per packed segment and head, float32 throughout.
 * q, k, v: element (row, h, d) at ptr[row * row_stride + h * D + d]; out [P, H, D]; lse [H, P]; bias may be NULL.
 * Only query rows [q_lo, q_hi) of every segment are computed (q_hi < 0: to the segment end); the benchmark's
 * bounded CPU sample uses that, the tests always pass the whole range. */
void orc_attention(const float *q, const float *k, const float *v, int64_t row_stride, const float *bias,
                   const int32_t *cu, int64_t nseg, int64_t P, int64_t Hh, int64_t D, float scale, float *out,
                   float *lse, int64_t q_lo, int64_t q_hi) {
    for (int64_t s = 0; s < nseg; ++s)
        for (int64_t h = 0; h < Hh; ++h) {
            const int64_t a = cu[s], e = cu[s + 1];
            const int64_t i_lo = a + q_lo, i_hi = (q_hi >= 0 && a + q_hi < e) ? a + q_hi : e;
#pragma omp parallel
            {
                float *logit = (float *)malloc((size_t)(e > a ? e - a : 1) * sizeof(float));
#pragma omp for schedule(dynamic, 8)
                for (int64_t i = i_lo; i < i_hi; ++i) {
                    const float *qi = q + i * row_stride + h * D;
                    float mx = -INFINITY;
                    for (int64_t j = a; j < e; ++j) {
                        const float *kj = k + j * row_stride + h * D;
                        float dot = 0.0f;
                        for (int64_t d = 0; d < D; ++d) dot += qi[d] * kj[d];
                        float x = dot * scale + (bias ? bias[j] : 0.0f);
                        logit[j - a] = x;
                        if (x > mx) mx = x;
                    }
                    float l = 0.0f;
                    float *o = out + (i * Hh + h) * D;
                    for (int64_t d = 0; d < D; ++d) o[d] = 0.0f;
                    for (int64_t j = a; j < e; ++j) {
                        float p = expf(logit[j - a] - mx);
                        l += p;
                        const float *vj = v + j * row_stride + h * D;
                        for (int64_t d = 0; d < D; ++d) o[d] += p * vj[d];
                    }
                    for (int64_t d = 0; d < D; ++d) o[d] /= l;
                    lse[h * P + i] = mx + logf(l);
                }
                free(logit);
            }
        }
}

/* Number of OpenMP threads of the following calls (a launcher may have exported OMP_NUM_THREADS=1 for its workers). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
