/*
 * CPU oracle for the INT4-AWQ decode hot path.  TEST INFRASTRUCTURE ONLY; see
 * oracle.h for the contract and for the "parity unpinned" statement.
 *
 * Idiom follows the reference's only CPU kernel
 * (kuiper/source/op/kernel/cpu/add_kernel.cpp:5-26): free functions over raw
 * fp32 buffers with the preconditions checked on entry.  The reference uses
 * Armadillo's fvec operator+ there (add_kernel.cpp:22-25); that is restated
 * as a plain loop.
 */
#include "oracle.h"

#include <assert.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define ORC_CHECK(cond)                                                              \
    do {                                                                             \
        if (!(cond)) {                                                               \
            fprintf(stderr, "oracle check failed: %s (%s:%d)\n", #cond, __FILE__, __LINE__); \
            abort();                                                                 \
        }                                                                            \
    } while (0)

/* AWQ nibble order: nibble i of a word holds logical column 8*j + ORD[i] */
static const int ORD[8] = {0, 2, 4, 6, 1, 3, 5, 7};

/* ------------------------------------------------------------------ */
/* scalar conversions                                                  */
/* ------------------------------------------------------------------ */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

uint16_t orc_f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}
float orc_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

uint16_t orc_f32_to_f16(float f) {
    uint32_t u = f2u(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);          /* NaN */
    if (a >= 0x47800000u) {                                           /* >= 65536: inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (a < 0x38800000u) {                                            /* subnormal or zero */
        if (a < 0x33000000u) return (uint16_t)sign;                   /* < 2^-25 -> 0 */
        /* value = a_float; result mantissa = round(a_float * 2^24) */
        float af = u2f(a);
        float scaled = af * 16777216.0f; /* exact */
        uint32_t m = (uint32_t)lrintf(scaled); /* round-half-even under default mode */
        return (uint16_t)(sign | m);
    }
    uint32_t exp = (a >> 23) - 112u; /* rebias 127 -> 15 */
    uint32_t man = a & 0x7fffffu;
    uint32_t h = (exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++; /* carries into exponent correctly */
    return (uint16_t)(sign | h);
}
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return u2f(sign);
        float v = (float)man * (1.0f / 16777216.0f);
        return sign ? -v : v;
    }
    if (exp == 31) return u2f(sign | 0x7f800000u | (man << 13));
    return u2f(sign | ((exp + 112u) << 23) | (man << 13));
}
void orc_f32_to_bf16_n(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_f32_to_bf16(in[i]);
}
void orc_f32_to_f16_n(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_f32_to_f16(in[i]);
}
void orc_bf16_to_f32_n(const uint16_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_bf16_to_f32(in[i]);
}
/* number of OpenMP threads the oracle's loops use from now on (the timed CPU baseline sets this itself, because a
 * launcher may have exported OMP_NUM_THREADS=1); returns the value in effect */
#ifdef _OPENMP
#include <omp.h>
#endif
int orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}
static inline float round_act(float v, int mode) {
    if (mode == ORC_ROUND_FP16) return orc_f16_to_f32(orc_f32_to_f16(v));
    if (mode == ORC_ROUND_BF16) return orc_bf16_to_f32(orc_f32_to_bf16(v));
    return v;
}

/* Rounds the M rows of an operand [M, K] the way the matmul named by `mode` does.  ORC_ROUND_I16_BLOCK32 is a block
 * floating point: per 32 consecutive elements of a row, e is the largest exponent with |x * 2^e| < 2^14 for the
 * largest magnitude of the block (e <= 126; a zero block takes 126) and x' = rint(x * 2^e) * 2^-e, ties to even.
 * ORC_ROUND_ENGINE mirrors an engine created with act_mode 2: block floating point for a one-row pass, fp16 else. */
static int engine_mode(int mode, int M) {
    if (mode == ORC_ROUND_ENGINE) return M == 1 ? ORC_ROUND_I16_BLOCK32 : ORC_ROUND_FP16;
    return mode;
}
static void round_rows(const float* x, float* out, int M, int K, int mode) {
    mode = engine_mode(mode, M);
    if (mode != ORC_ROUND_I16_BLOCK32) {
        for (int64_t i = 0; i < (int64_t)M * K; i++) out[i] = round_act(x[i], mode);
        return;
    }
    for (int m = 0; m < M; m++) {
        for (int k0 = 0; k0 < K; k0 += 32) {
            const int n = K - k0 < 32 ? K - k0 : 32;
            const float* xb = x + (int64_t)m * K + k0;
            float* ob = out + (int64_t)m * K + k0;
            float amax = 0.0f;
            for (int i = 0; i < n; i++) {
                float a = fabsf(xb[i]);
                if (a > amax) amax = a;
            }
            uint32_t bits;
            memcpy(&bits, &amax, sizeof(bits));
            int ea = (int)((bits >> 23) & 0xffu) - 127; /* floor(log2 amax); -127 for zero and subnormals */
            int e = 13 - ea;
            if (e > 126) e = 126;
            const float scale = ldexpf(1.0f, e), inv = ldexpf(1.0f, -e);
            for (int i = 0; i < n; i++) ob[i] = rintf(xb[i] * scale) * inv;
        }
    }
}

/* ------------------------------------------------------------------ */
/* add                                                                 */
/* ------------------------------------------------------------------ */
void orc_add(const float* a, const float* b, float* out, int64_t n) {
    ORC_CHECK(a && b && out && n >= 0);
    for (int64_t i = 0; i < n; i++) out[i] = a[i] + b[i];
}

/* ------------------------------------------------------------------ */
/* AWQ pack / unpack / dequant / quantise                              */
/* ------------------------------------------------------------------ */
void orc_awq_pack(const uint8_t* q, int K, int N, int32_t* words) {
    ORC_CHECK(N % 8 == 0);
    int NW = N / 8;
    for (int k = 0; k < K; k++)
        for (int j = 0; j < NW; j++) {
            uint32_t w = 0;
            for (int i = 0; i < 8; i++) {
                uint32_t v = q[(int64_t)k * N + 8 * j + ORD[i]];
                ORC_CHECK(v < 16);
                w |= v << (4 * i);
            }
            words[(int64_t)k * NW + j] = (int32_t)w;
        }
}

void orc_awq_unpack(const int32_t* words, int K, int N, uint8_t* q) {
    ORC_CHECK(N % 8 == 0);
    int NW = N / 8;
#pragma omp parallel for schedule(static)
    for (int k = 0; k < K; k++)
        for (int j = 0; j < NW; j++) {
            uint32_t w = (uint32_t)words[(int64_t)k * NW + j];
            for (int i = 0; i < 8; i++) q[(int64_t)k * N + 8 * j + ORD[i]] = (uint8_t)((w >> (4 * i)) & 0xfu);
        }
}

static inline int nib(const int32_t* words, int NW, int row, int n) {
    /* logical column n lives in word n/8 at the nibble whose ORD entry is n%8 */
    static const int INV[8] = {0, 4, 1, 5, 2, 6, 3, 7};
    uint32_t w = (uint32_t)words[(int64_t)row * NW + (n >> 3)];
    return (int)((w >> (4 * INV[n & 7])) & 0xfu);
}

void orc_awq_dequant(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales_f16,
                     int K, int N, int group, float* W) {
    ORC_CHECK(N % 8 == 0 && group > 0 && K % group == 0);
    int NW = N / 8;
#pragma omp parallel for schedule(static)
    for (int k = 0; k < K; k++) {
        int g = k / group;
        for (int n = 0; n < N; n++) {
            int q = nib(qweight, NW, k, n);
            int z = nib(qzeros, NW, g, n);
            float s = orc_f16_to_f32(scales_f16[(int64_t)g * N + n]);
            W[(int64_t)k * N + n] = (float)(q - z) * s;
        }
    }
}

void orc_awq_quantize(const float* W, int K, int N, int group,
                      int32_t* qweight, int32_t* qzeros, uint16_t* scales_f16) {
    ORC_CHECK(N % 8 == 0 && group > 0 && K % group == 0);
    int G = K / group;
    uint8_t* q = (uint8_t*)malloc((size_t)K * N);
    uint8_t* z = (uint8_t*)malloc((size_t)G * N);
    ORC_CHECK(q && z);
#pragma omp parallel for schedule(static)
    for (int g = 0; g < G; g++)
        for (int n = 0; n < N; n++) {
            float mn = INFINITY, mx = -INFINITY;
            for (int k = g * group; k < (g + 1) * group; k++) {
                float v = W[(int64_t)k * N + n];
                if (v < mn) mn = v;
                if (v > mx) mx = v;
            }
            float sc = (mx - mn) / 15.0f;
            if (!(sc > 1e-8f)) sc = 1e-8f;
            uint16_t sh = orc_f32_to_f16(sc);
            if (sh == 0) sh = 1;
            float s = orc_f16_to_f32(sh);
            float zf = rintf(-mn / s);
            int zi = zf < 0 ? 0 : (zf > 15 ? 15 : (int)zf);
            scales_f16[(int64_t)g * N + n] = sh;
            z[(int64_t)g * N + n] = (uint8_t)zi;
            for (int k = g * group; k < (g + 1) * group; k++) {
                float r = rintf(W[(int64_t)k * N + n] / s) + (float)zi;
                int qi = r < 0 ? 0 : (r > 15 ? 15 : (int)r);
                q[(int64_t)k * N + n] = (uint8_t)qi;
            }
        }
    orc_awq_pack(q, K, N, qweight);
    orc_awq_pack(z, G, N, qzeros);
    free(q);
    free(z);
}

/* ------------------------------------------------------------------ */
/* matmuls                                                             */
/* ------------------------------------------------------------------ */
void orc_gemv_f32(const float* x, const float* W, float* y, int M, int K, int N,
                  int acc_double, int act_round) {
    ORC_CHECK(x && W && y && M > 0 && K > 0 && N > 0);
    float* xr = (float*)malloc((size_t)M * K * sizeof(float));
    ORC_CHECK(xr);
    round_rows(x, xr, M, K, act_round);
    /* column-blocked so W streams once per row of x and the accumulators stay in cache */
    enum { NB = 512 };
#pragma omp parallel for schedule(static)
    for (int n0 = 0; n0 < N; n0 += NB) {
        int nb = N - n0 < NB ? N - n0 : NB;
        for (int m = 0; m < M; m++) {
            if (acc_double) {
                double acc[NB];
                for (int j = 0; j < nb; j++) acc[j] = 0.0;
                for (int k = 0; k < K; k++) {
                    double xv = (double)xr[(int64_t)m * K + k];
                    const float* w = W + (int64_t)k * N + n0;
                    for (int j = 0; j < nb; j++) acc[j] += xv * (double)w[j];
                }
                for (int j = 0; j < nb; j++) y[(int64_t)m * N + n0 + j] = (float)acc[j];
            } else {
                float acc[NB];
                for (int j = 0; j < nb; j++) acc[j] = 0.0f;
                for (int k = 0; k < K; k++) {
                    float xv = xr[(int64_t)m * K + k];
                    const float* w = W + (int64_t)k * N + n0;
                    for (int j = 0; j < nb; j++) acc[j] += xv * w[j];
                }
                for (int j = 0; j < nb; j++) y[(int64_t)m * N + n0 + j] = acc[j];
            }
        }
    }
    free(xr);
}

void orc_awq_gemv(const float* x, const int32_t* qweight, const int32_t* qzeros,
                  const uint16_t* scales_f16, float* y, int M, int K, int N, int group,
                  int acc_double, int act_round) {
    ORC_CHECK(x && qweight && qzeros && scales_f16 && y);
    ORC_CHECK(N % 8 == 0 && group > 0 && K % group == 0 && M > 0);
    int NW = N / 8;
    float* xr = (float*)malloc((size_t)M * K * sizeof(float));
    ORC_CHECK(xr);
    round_rows(x, xr, M, K, act_round);
    /* one task per packed word column: 8 outputs; each weight is dequantised once and
       applied to all M rows */
#pragma omp parallel for schedule(static)
    for (int j = 0; j < NW; j++) {
        double* accd = (double*)calloc((size_t)M * 8, sizeof(double));
        float* accf = (float*)calloc((size_t)M * 8, sizeof(float));
        ORC_CHECK(accd && accf);
        for (int g = 0; g < K / group; g++) {
            uint32_t zw = (uint32_t)qzeros[(int64_t)g * NW + j];
            float s[8];
            int z[8];
            for (int i = 0; i < 8; i++) {
                z[i] = (int)((zw >> (4 * i)) & 0xfu);
                s[i] = orc_f16_to_f32(scales_f16[(int64_t)g * N + 8 * j + ORD[i]]);
            }
            for (int k = g * group; k < (g + 1) * group; k++) {
                uint32_t w = (uint32_t)qweight[(int64_t)k * NW + j];
                float wv[8];
                for (int i = 0; i < 8; i++) wv[i] = (float)((int)((w >> (4 * i)) & 0xfu) - z[i]) * s[i];
                for (int m = 0; m < M; m++) {
                    float xv = xr[(int64_t)m * K + k];
                    if (acc_double)
                        for (int i = 0; i < 8; i++) accd[m * 8 + i] += (double)xv * (double)wv[i];
                    else
                        for (int i = 0; i < 8; i++) accf[m * 8 + i] += xv * wv[i];
                }
            }
        }
        for (int m = 0; m < M; m++)
            for (int i = 0; i < 8; i++)
                y[(int64_t)m * N + 8 * j + ORD[i]] = acc_double ? (float)accd[m * 8 + i] : accf[m * 8 + i];
        free(accd);
        free(accf);
    }
    free(xr);
}

void orc_bf16_gemv(const float* x, const uint16_t* W_bf16, float* y, int M, int K, int N,
                   int acc_double) {
    ORC_CHECK(x && W_bf16 && y && M > 0 && K > 0 && N > 0);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const uint16_t* w = W_bf16 + (int64_t)n * K;
        for (int m = 0; m < M; m++) {
            const float* xv = x + (int64_t)m * K;
            if (acc_double) {
                double acc = 0.0;
                for (int k = 0; k < K; k++) acc += (double)xv[k] * (double)orc_bf16_to_f32(w[k]);
                y[(int64_t)m * N + n] = (float)acc;
            } else {
                float acc = 0.0f;
                for (int k = 0; k < K; k++) acc += xv[k] * orc_bf16_to_f32(w[k]);
                y[(int64_t)m * N + n] = acc;
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* norms, rotary, attention, activation                                */
/* ------------------------------------------------------------------ */
void orc_rmsnorm(const float* x, const uint16_t* w_bf16, float* y, int M, int H, float eps) {
    ORC_CHECK(x && w_bf16 && y && M > 0 && H > 0);
    for (int m = 0; m < M; m++) {
        const float* xr = x + (int64_t)m * H;
        double ss = 0.0;
        for (int i = 0; i < H; i++) ss += (double)xr[i] * (double)xr[i];
        float rstd = 1.0f / sqrtf((float)(ss / (double)H) + eps);
        for (int i = 0; i < H; i++) y[(int64_t)m * H + i] = (xr[i] * rstd) * orc_bf16_to_f32(w_bf16[i]);
    }
}

void orc_rope_tables(int max_pos, int D, double theta, float* cos_t, float* sin_t) {
    ORC_CHECK(D % 2 == 0);
    int half = D / 2;
    for (int p = 0; p < max_pos; p++)
        for (int i = 0; i < half; i++) {
            double inv = pow(theta, -2.0 * (double)i / (double)D);
            double a = (double)p * inv;
            cos_t[(int64_t)p * half + i] = (float)cos(a);
            sin_t[(int64_t)p * half + i] = (float)sin(a);
        }
}

static void head_norm_rope(const float* in, const uint16_t* w, const float* c, const float* s,
                           int D, float eps, float* out) {
    int half = D / 2;
    double ss = 0.0;
    for (int i = 0; i < D; i++) ss += (double)in[i] * (double)in[i];
    float rstd = 1.0f / sqrtf((float)(ss / (double)D) + eps);
    for (int i = 0; i < half; i++) {
        float a = (in[i] * rstd) * orc_bf16_to_f32(w[i]);
        float b = (in[i + half] * rstd) * orc_bf16_to_f32(w[i + half]);
        out[i] = a * c[i] - b * s[i];
        out[i + half] = b * c[i] + a * s[i];
    }
}

void orc_qknorm_rope_kvwrite(const float* qkv, const uint16_t* q_norm_w, const uint16_t* k_norm_w,
                             const float* cos_t, const float* sin_t, const int32_t* pos,
                             const int32_t* slot, int M, int Nq, int Nkv, int D, float eps,
                             int max_seq, float* q_out, uint16_t* kcache, uint16_t* vcache) {
    ORC_CHECK(D % 2 == 0 && D <= 512);
    int half = D / 2;
    int row = (Nq + 2 * Nkv) * D;
    for (int m = 0; m < M; m++) {
        int p = pos[m];
        ORC_CHECK(p >= 0 && p < max_seq);
        const float* c = cos_t + (int64_t)p * half;
        const float* s = sin_t + (int64_t)p * half;
        const float* r = qkv + (int64_t)m * row;
        for (int h = 0; h < Nq; h++)
            head_norm_rope(r + (int64_t)h * D, q_norm_w, c, s, D, eps, q_out + ((int64_t)m * Nq + h) * D);
        for (int h = 0; h < Nkv; h++) {
            float tmp[512];
            head_norm_rope(r + (int64_t)(Nq + h) * D, k_norm_w, c, s, D, eps, tmp);
            int64_t off = (((int64_t)slot[m] * Nkv + h) * max_seq + p) * D;
            const float* v = r + (int64_t)(Nq + Nkv + h) * D;
            for (int i = 0; i < D; i++) {
                kcache[off + i] = orc_f32_to_bf16(tmp[i]);
                vcache[off + i] = orc_f32_to_bf16(v[i]);
            }
        }
    }
}

void orc_attention(const float* q, const uint16_t* kcache, const uint16_t* vcache,
                   const int32_t* seq_len, const int32_t* slot, int M, int Nq, int Nkv, int D,
                   int max_seq, float* out) {
    ORC_CHECK(Nq % Nkv == 0);
    int rep = Nq / Nkv;
    double scale = 1.0 / sqrt((double)D);
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int m = 0; m < M; m++)
        for (int h = 0; h < Nq; h++) {
            int L = seq_len[m];
            int kvh = h / rep;
            const float* qv = q + ((int64_t)m * Nq + h) * D;
            const uint16_t* kb = kcache + ((int64_t)slot[m] * Nkv + kvh) * max_seq * D;
            const uint16_t* vb = vcache + ((int64_t)slot[m] * Nkv + kvh) * max_seq * D;
            float* o = out + ((int64_t)m * Nq + h) * D;
            if (L <= 0) {
                for (int i = 0; i < D; i++) o[i] = 0.0f;
                continue;
            }
            double* sc = (double*)malloc((size_t)L * sizeof(double));
            double* acc = (double*)calloc((size_t)D, sizeof(double));
            ORC_CHECK(sc && acc);
            double mx = -INFINITY;
            for (int j = 0; j < L; j++) {
                double d = 0.0;
                for (int i = 0; i < D; i++) d += (double)qv[i] * (double)orc_bf16_to_f32(kb[(int64_t)j * D + i]);
                sc[j] = d * scale;
                if (sc[j] > mx) mx = sc[j];
            }
            double den = 0.0;
            for (int j = 0; j < L; j++) {
                sc[j] = exp(sc[j] - mx);
                den += sc[j];
            }
            for (int j = 0; j < L; j++) {
                double p = sc[j];
                for (int i = 0; i < D; i++) acc[i] += p * (double)orc_bf16_to_f32(vb[(int64_t)j * D + i]);
            }
            for (int i = 0; i < D; i++) o[i] = (float)(acc[i] / den);
            free(sc);
            free(acc);
        }
}

void orc_swiglu(const float* gate, const float* up, float* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        float g = gate[i];
        out[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

void orc_embedding(const int32_t* tokens, const uint16_t* table_bf16, float* out, int M, int H) {
    for (int m = 0; m < M; m++)
        for (int i = 0; i < H; i++) out[(int64_t)m * H + i] = orc_bf16_to_f32(table_bf16[(int64_t)tokens[m] * H + i]);
}

void orc_argmax(const float* logits, int M, int V, int32_t* out) {
    for (int m = 0; m < M; m++) {
        const float* l = logits + (int64_t)m * V;
        int best = 0;
        for (int i = 1; i < V; i++)
            if (l[i] > l[best]) best = i;
        out[m] = best;
    }
}

/* ------------------------------------------------------------------ */
/* whole decoder                                                       */
/* ------------------------------------------------------------------ */
struct orc_model {
    orc_config cfg;
    const uint16_t *embed, *final_norm, *lm_head;
    orc_layer_weights* layers;
    uint16_t *kcache, *vcache; /* [L][max_batch][Nkv][max_seq][D] */
    float *cos_t, *sin_t;
};

orc_model* orc_model_create(const orc_config* cfg, const uint16_t* embed_bf16,
                            const uint16_t* final_norm_bf16, const uint16_t* lm_head_bf16,
                            const orc_layer_weights* layers) {
    orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
    ORC_CHECK(m);
    m->cfg = *cfg;
    m->embed = embed_bf16;
    m->final_norm = final_norm_bf16;
    m->lm_head = lm_head_bf16;
    m->layers = (orc_layer_weights*)malloc(sizeof(orc_layer_weights) * (size_t)cfg->n_layers);
    memcpy(m->layers, layers, sizeof(orc_layer_weights) * (size_t)cfg->n_layers);
    size_t cache = (size_t)cfg->n_layers * cfg->max_batch * cfg->n_kv_heads * cfg->max_seq * cfg->head_dim;
    m->kcache = (uint16_t*)calloc(cache, sizeof(uint16_t));
    m->vcache = (uint16_t*)calloc(cache, sizeof(uint16_t));
    m->cos_t = (float*)malloc(sizeof(float) * (size_t)cfg->max_seq * cfg->head_dim / 2);
    m->sin_t = (float*)malloc(sizeof(float) * (size_t)cfg->max_seq * cfg->head_dim / 2);
    ORC_CHECK(m->kcache && m->vcache && m->cos_t && m->sin_t);
    orc_rope_tables(cfg->max_seq, cfg->head_dim, cfg->rope_theta, m->cos_t, m->sin_t);
    return m;
}

void orc_model_destroy(orc_model* m) {
    if (!m) return;
    free(m->layers);
    free(m->kcache);
    free(m->vcache);
    free(m->cos_t);
    free(m->sin_t);
    free(m);
}

const uint16_t* orc_model_kcache(const orc_model* m) { return m->kcache; }
const uint16_t* orc_model_vcache(const orc_model* m) { return m->vcache; }

void orc_model_forward(orc_model* mdl, const int32_t* tokens, const int32_t* pos, const int32_t* slot,
                       int M, int acc_double, int logit_rows, float* logits, int32_t* next) {
    const orc_config* c = &mdl->cfg;
    int H = c->hidden, D = c->head_dim, Nq = c->n_q_heads, Nkv = c->n_kv_heads, I = c->inter;
    int QKV = (Nq + 2 * Nkv) * D;
    size_t layer_cache = (size_t)c->max_batch * Nkv * c->max_seq * D;
    float* h = (float*)malloc(sizeof(float) * (size_t)M * H);
    float* xn = (float*)malloc(sizeof(float) * (size_t)M * H);
    float* qkv = (float*)malloc(sizeof(float) * (size_t)M * QKV);
    float* q = (float*)malloc(sizeof(float) * (size_t)M * Nq * D);
    float* att = (float*)malloc(sizeof(float) * (size_t)M * Nq * D);
    float* proj = (float*)malloc(sizeof(float) * (size_t)M * H);
    float* gu = (float*)malloc(sizeof(float) * (size_t)M * 2 * I);
    float* act = (float*)malloc(sizeof(float) * (size_t)M * I);
    int32_t* seq = (int32_t*)malloc(sizeof(int32_t) * (size_t)M);
    ORC_CHECK(h && xn && qkv && q && att && proj && gu && act && seq);
    for (int m = 0; m < M; m++) {
        ORC_CHECK(tokens[m] >= 0 && tokens[m] < c->vocab);
        ORC_CHECK(slot[m] >= 0 && slot[m] < c->max_batch);
        seq[m] = pos[m] + 1; /* causal: a token sees positions 0..pos */
    }
    orc_embedding(tokens, mdl->embed, h, M, H);
    for (int l = 0; l < c->n_layers; l++) {
        const orc_layer_weights* w = &mdl->layers[l];
        uint16_t* kc = mdl->kcache + (size_t)l * layer_cache;
        uint16_t* vc = mdl->vcache + (size_t)l * layer_cache;
        orc_rmsnorm(h, w->input_norm, xn, M, H, c->eps);
        orc_awq_gemv(xn, w->qkv_qw, w->qkv_qz, w->qkv_s, qkv, M, H, QKV, c->group, acc_double, c->act_round);
        orc_qknorm_rope_kvwrite(qkv, w->q_norm, w->k_norm, mdl->cos_t, mdl->sin_t, pos, slot, M, Nq, Nkv, D,
                                c->eps, c->max_seq, q, kc, vc);
        orc_attention(q, kc, vc, seq, slot, M, Nq, Nkv, D, c->max_seq, att);
        orc_awq_gemv(att, w->o_qw, w->o_qz, w->o_s, proj, M, Nq * D, H, c->group, acc_double, c->act_round);
        orc_add(h, proj, h, (int64_t)M * H);
        orc_rmsnorm(h, w->post_norm, xn, M, H, c->eps);
        orc_awq_gemv(xn, w->gu_qw, w->gu_qz, w->gu_s, gu, M, H, 2 * I, c->group, acc_double, c->act_round);
        for (int m = 0; m < M; m++)
            orc_swiglu(gu + (size_t)m * 2 * I, gu + (size_t)m * 2 * I + I, act + (size_t)m * I, I);
        orc_awq_gemv(act, w->down_qw, w->down_qz, w->down_s, proj, M, I, H, c->group, acc_double, c->act_round);
        orc_add(h, proj, h, (int64_t)M * H);
    }
    if ((logits || next) && logit_rows > 0) {
        ORC_CHECK(logit_rows <= M);
        int r0 = M - logit_rows; /* logits for the last logit_rows rows only */
        float* lg = logits ? logits : (float*)malloc(sizeof(float) * (size_t)logit_rows * c->vocab);
        ORC_CHECK(lg);
        orc_rmsnorm(h + (size_t)r0 * H, mdl->final_norm, xn, logit_rows, H, c->eps);
        orc_bf16_gemv(xn, mdl->lm_head, lg, logit_rows, H, c->vocab, acc_double);
        if (next) orc_argmax(lg, logit_rows, c->vocab, next);
        if (!logits) free(lg);
    }
    free(h); free(xn); free(qkv); free(q); free(att); free(proj); free(gu); free(act); free(seq);
}
