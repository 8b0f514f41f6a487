/*
 * CPU oracle for the Anima DiT attention path of sonsegajp/kiln.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links, loads or calls this file;
 * it is the checker for the parity tests, the smoke check and the benchmark's CPU baseline.
 *
 * The reference has no CPU implementation of this path (its kernels are CUDA only), so every
 * function here restates the arithmetic of one reference kernel in plain C, citing the reference
 * file:line it follows (paths are relative to the reference project root):
 *
 *   ko_attention*     bench/tfa_test.cu:11-33  (ref_attn: two-pass fp32 attention with analytic npad)
 *                     engine/src/kernels.cu:809-826 (k_softmax_rows: the same npad rule in the engine)
 *   ko_rmsnorm        engine/src/kernels.cu:656-666 (k_rmsnorm_warp; weights are bf16 bit patterns)
 *   ko_rope_half      engine/src/kernels.cu:759-772 (k_rope_half, pairs (i, i+Dh/2))
 *   ko_cosmos_rope    engine/src/dit.cu:196-215     (cosmos_rope table for an image, T=1)
 *   ko_nag            engine/src/dit.cu:295-324     (k_nag: per-token L1 clamp over all channels)
 *   ko_torch_randn    engine/src/pipeline.cu:16-64  (torch-compatible CPU randn)
 *
 * Pinning: ko_torch_randn is pinned bit-for-bit against torch.randn on CPU; the attention,
 * RMSNorm, RoPE and NAG restatements are pinned against outputs of the reference's own kernels
 * compiled for sm_100a and run on a B200 (fixtures under tests/golden/, made by
 * tests/golden/make_ref_fixtures.py).
 *
 * Two accumulation modes: "f32" follows the reference's float arithmetic order exactly;
 * "f64" accumulates dot products, softmax sums and outputs in double and is the
 * "fp32 reference" that tolerance checks compare against.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define KO_D 128

int ko_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* size of the OpenMP team of the following calls (a launcher may export OMP_NUM_THREADS=1 to its ranks) */
void ko_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ---- 16-bit float helpers (round to nearest even), so Python and C agree on the rounded inputs ---- */
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float ko_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

uint16_t ko_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

uint16_t ko_f32_to_f16(float f) {
    uint32_t x = f32_bits(f), sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return (uint16_t)(sign | (x > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);               /* rounds to inf */
    if (x < 0x33000001u) return (uint16_t)sign;                            /* rounds to zero */
    int e = (int)(x >> 23) - 127;
    uint32_t m = (x & 0x7fffffu) | 0x800000u;
    int shift = e < -14 ? 13 + (-14 - e) : 13;                              /* subnormal halves shift more */
    uint32_t half_m = m >> shift, rem = m & ((1u << shift) - 1u), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half_m & 1u))) half_m++;
    uint32_t out = e < -14 ? half_m : (uint32_t)((e + 15) << 10) + (half_m - 0x400u);
    return (uint16_t)(sign | out);
}

float ko_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 0x3ffu;
    if (e == 31) return bits_f32(sign | 0x7f800000u | (m << 13));
    if (e == 0) {
        if (!m) return bits_f32(sign);
        float v = (float)m * (1.0f / 16777216.0f);  /* m * 2^-24 */
        return sign ? -v : v;
    }
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* round an fp32 array through a 16-bit type in place: kind 0 = fp16, 1 = bf16 */
void ko_round16(float* x, size_t n, int kind) {
    for (size_t i = 0; i < n; i++) x[i] = kind ? ko_bf16_to_f32(ko_f32_to_bf16(x[i])) : ko_f16_to_f32(ko_f32_to_f16(x[i]));
}

/* ---- torch-compatible CPU randn: MT19937, 24-bit uniforms, 16-wide Box-Muller (pipeline.cu:16-64) ---- */
typedef struct { uint32_t s[624]; int idx; } ko_mt;

static void mt_seed(ko_mt* g, uint64_t seed) {
    g->s[0] = (uint32_t)(seed & 0xffffffffu);
    for (int j = 1; j < 624; j++) g->s[j] = 1812433253u * (g->s[j - 1] ^ (g->s[j - 1] >> 30)) + (uint32_t)j;
    g->idx = 624;
}

static uint32_t mt_next(ko_mt* g) {
    if (g->idx >= 624) {
        for (int k = 0; k < 624; k++) {
            uint32_t y = (g->s[k] & 0x80000000u) | (g->s[(k + 1) % 624] & 0x7fffffffu);
            g->s[k] = g->s[(k + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
        }
        g->idx = 0;
    }
    uint32_t y = g->s[g->idx++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9d2c5680u;
    y ^= (y << 15) & 0xefc60000u;
    y ^= y >> 18;
    return y;
}

static float mt_uniform(ko_mt* g) { return (float)(mt_next(g) & 0xffffffu) * (1.0f / 16777216.0f); }

static void box_muller_16(float* d) {
    for (int j = 0; j < 8; j++) {
        float u1 = 1.f - d[j], u2 = d[j + 8];
        float radius = sqrtf(-2.f * logf(u1));
        float theta = 2.0f * 3.14159265358979323846f * u2;
        d[j] = radius * cosf(theta);
        d[j + 8] = radius * sinf(theta);
    }
}

/* n must be >= 16 (as torch's vectorised path requires); returns 0 on success */
int ko_torch_randn(uint64_t seed, size_t n, float* out) {
    if (n < 16) return -1;
    ko_mt g;
    mt_seed(&g, seed);
    for (size_t i = 0; i < n; i++) out[i] = mt_uniform(&g);
    for (size_t i = 0; i + 16 <= n; i += 16) box_muller_16(out + i);
    if (n % 16) {
        float* t = out + n - 16;
        for (int i = 0; i < 16; i++) t[i] = mt_uniform(&g);
        box_muller_16(t);
    }
    return 0;
}

/* ---- attention (bench/tfa_test.cu:11-33) ----
 * q [Tq, ldq], k/v [Tk, ld], out [Tq, ldo]; head h at columns [h*128, h*128+128).
 * npad all-zero keys join the softmax: running max starts at 0 and the denominator gets
 * npad*exp(-m); they add nothing to the numerator. */
void ko_attention_f32(float* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                      int Tq, int Tk, int H, int npad) {
    const float inv_sqrt_d = sqrtf(128.f);
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < Tq; t++)
        for (int h = 0; h < H; h++) {
            const float* qr = q + (size_t)t * ldq + h * KO_D;
            float m = npad ? 0.f : -INFINITY;
            for (int j = 0; j < Tk; j++) {
                const float* kr = k + (size_t)j * ldk + h * KO_D;
                float s = 0;
                for (int d = 0; d < KO_D; d++) s += qr[d] * kr[d];
                m = fmaxf(m, s / inv_sqrt_d);
            }
            float acc[KO_D] = {0}, l = npad * expf(-m);
            for (int j = 0; j < Tk; j++) {
                const float* kr = k + (size_t)j * ldk + h * KO_D;
                const float* vr = v + (size_t)j * ldv + h * KO_D;
                float s = 0;
                for (int d = 0; d < KO_D; d++) s += qr[d] * kr[d];
                float p = expf(s / inv_sqrt_d - m);
                l += p;
                for (int d = 0; d < KO_D; d++) acc[d] += p * vr[d];
            }
            float* o = out + (size_t)t * ldo + h * KO_D;
            for (int d = 0; d < KO_D; d++) o[d] = acc[d] / l;
        }
}

/* the same with double accumulation: the tolerance oracle */
void ko_attention_f64(float* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                      int Tq, int Tk, int H, int npad) {
    const double scale = 1.0 / sqrt(128.0);
#pragma omp parallel
    {
        double* sc = (double*)malloc(sizeof(double) * (size_t)(Tk > 0 ? Tk : 1));
#pragma omp for collapse(2) schedule(static)
        for (int t = 0; t < Tq; t++)
            for (int h = 0; h < H; h++) {
                const float* qr = q + (size_t)t * ldq + h * KO_D;
                double m = npad ? 0.0 : -INFINITY;
                for (int j = 0; j < Tk; j++) {
                    const float* kr = k + (size_t)j * ldk + h * KO_D;
                    double s = 0;
                    for (int d = 0; d < KO_D; d++) s += (double)qr[d] * (double)kr[d];
                    sc[j] = s * scale;
                    if (sc[j] > m) m = sc[j];
                }
                double acc[KO_D] = {0}, l = npad * exp(-m);
                for (int j = 0; j < Tk; j++) {
                    const float* vr = v + (size_t)j * ldv + h * KO_D;
                    double p = exp(sc[j] - m);
                    l += p;
                    for (int d = 0; d < KO_D; d++) acc[d] += p * (double)vr[d];
                }
                float* o = out + (size_t)t * ldo + h * KO_D;
                for (int d = 0; d < KO_D; d++) o[d] = (float)(acc[d] / l);
            }
        free(sc);
    }
}

/* ---- attention backward (train.cu:216-242 with k_softmax_pad, train.cu:103-121, and k_dsoftmax, train.cu:124-131) ----
 * q [Tq, ldq], k/v [Tk, ld], dout [Tq, ldo] -> dq [Tq, ldq'], dk, dv [Tk, ld']; head h at columns [h*128, +128). Per head:
 *   S = QK^T/sqrt(128); P = softmax over the Tk keys and npad zero keys of score 0; dP = dO V^T; dV = P^T dO;
 *   dS = P (dP - sum_j P dP) (padding keys have dP = 0 and drop out of the sum); dQ = dS K/sqrt(128); dK = dS^T Q/sqrt(128).
 * Everything in double (the reference runs fp32 cuBLAS SGEMMs). Key rows [j0, j1) of dk / dv only: dq rows are independent of
 * each other, so sampled query rows are exact with the full K/V; dk / dv need every query row, which the caller passes. */
void ko_attention_bwd(float* dq, int lddq, float* dk, int lddk, float* dv, int lddv, const float* q, int ldq, const float* k, int ldk,
                      const float* v, int ldv, const float* dout, int ldo, int Tq, int Tk, int H, int npad, int j0, int j1) {
    const double scale = 1.0 / sqrt(128.0);
    const int nj = j1 - j0;
    for (int h = 0; h < H; h++) {
        double* P = (double*)malloc(sizeof(double) * (size_t)Tq * (size_t)(Tk > 0 ? Tk : 1));
        double* dS = (double*)malloc(sizeof(double) * (size_t)Tq * (size_t)(Tk > 0 ? Tk : 1));
#pragma omp parallel for schedule(static)
        for (int t = 0; t < Tq; t++) {
            const float* qr = q + (size_t)t * ldq + h * KO_D;
            const float* gr = dout + (size_t)t * ldo + h * KO_D;
            double* pr = P + (size_t)t * Tk;
            double* dr = dS + (size_t)t * Tk;
            double m = npad ? 0.0 : -INFINITY;
            for (int j = 0; j < Tk; j++) {
                const float* kr = k + (size_t)j * ldk + h * KO_D;
                double s = 0;
                for (int d = 0; d < KO_D; d++) s += (double)qr[d] * (double)kr[d];
                pr[j] = s * scale;
                if (pr[j] > m) m = pr[j];
            }
            double l = npad * exp(-m);
            for (int j = 0; j < Tk; j++) { pr[j] = exp(pr[j] - m); l += pr[j]; }
            double dot = 0;
            for (int j = 0; j < Tk; j++) {
                const float* vr = v + (size_t)j * ldv + h * KO_D;
                double dp = 0;
                for (int d = 0; d < KO_D; d++) dp += (double)gr[d] * (double)vr[d];
                pr[j] /= l;
                dr[j] = dp;
                dot += pr[j] * dp;
            }
            double acc[KO_D] = {0};
            for (int j = 0; j < Tk; j++) {
                const float* kr = k + (size_t)j * ldk + h * KO_D;
                dr[j] = pr[j] * (dr[j] - dot);
                for (int d = 0; d < KO_D; d++) acc[d] += dr[j] * (double)kr[d];
            }
            if (dq) {
                float* o = dq + (size_t)t * lddq + h * KO_D;
                for (int d = 0; d < KO_D; d++) o[d] = (float)(acc[d] * scale);
            }
        }
#pragma omp parallel for schedule(static)
        for (int jj = 0; jj < nj; jj++) {
            const int j = j0 + jj;
            double ak[KO_D] = {0}, av[KO_D] = {0};
            for (int t = 0; t < Tq; t++) {
                const float* qr = q + (size_t)t * ldq + h * KO_D;
                const float* gr = dout + (size_t)t * ldo + h * KO_D;
                const double p = P[(size_t)t * Tk + j], ds = dS[(size_t)t * Tk + j];
                for (int d = 0; d < KO_D; d++) { av[d] += p * (double)gr[d]; ak[d] += ds * (double)qr[d]; }
            }
            if (dk) { float* o = dk + (size_t)jj * lddk + h * KO_D; for (int d = 0; d < KO_D; d++) o[d] = (float)(ak[d] * scale); }
            if (dv) { float* o = dv + (size_t)jj * lddv + h * KO_D; for (int d = 0; d < KO_D; d++) o[d] = (float)av[d]; }
        }
        free(P);
        free(dS);
    }
}

/* ---- RMSNorm over rows of `dim` (kernels.cu:656-666); w = bf16 bit patterns [dim] or NULL ---- */
void ko_rmsnorm(float* y, const float* x, const uint16_t* w, size_t rows, int dim, float eps) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++) {
        const float* xr = x + r * (size_t)dim;
        float* yr = y + r * (size_t)dim;
        /* the kernel sums lane-strided partials and then a butterfly; the order differs only in rounding */
        float part[32] = {0};
        for (int i = 0; i < dim; i++) part[i & 31] += xr[i] * xr[i];
        for (int o = 16; o > 0; o >>= 1)
            for (int i = 0; i < o; i++) part[i] += part[i + o];
        float rs = 1.0f / sqrtf(part[0] / (float)dim + eps);
        for (int i = 0; i < dim; i++) yr[i] = xr[i] * rs * (w ? ko_bf16_to_f32(w[i]) : 1.f);
    }
}

/* ---- rotate-half RoPE in place (kernels.cu:759-772); x [T, H, Dh] contiguous, tables [T, Dh/2] ---- */
void ko_rope_half(float* x, int T, int H, int Dh, const float* cos_t, const float* sin_t) {
    const int half = Dh / 2;
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < T; t++)
        for (int h = 0; h < H; h++) {
            float* p = x + ((size_t)t * H + h) * Dh;
            for (int i = 0; i < half; i++) {
                float c = cos_t[(size_t)t * half + i], s = sin_t[(size_t)t * half + i];
                float a = p[i], b = p[i + half];
                p[i] = a * c - b * s;
                p[i + half] = b * c + a * s;
            }
        }
}

/* ---- Cosmos 3D RoPE tables for an image (dit.cu:196-215); c, s are [Hp*Wp, 64] ---- */
void ko_cosmos_rope(float* c, float* s, int Hp, int Wp) {
    const int DH = 128;
    const int dim_h = DH / 6 * 2, dim_t = DH - 2 * dim_h; /* 42, 44 */
    double ntk = pow(4.0, (double)dim_h / (dim_h - 2));
    float h_theta = (float)(10000.0 * ntk);
    float hf[21];
    for (int j = 0; j < dim_h / 2; j++) hf[j] = 1.0f / powf(h_theta, (float)(2 * j) / (float)dim_h);
    int T = Hp * Wp, half = DH / 2;
    for (size_t i = 0; i < (size_t)T * half; i++) { c[i] = 1.f; s[i] = 0.f; }
    for (int t = 0; t < T; t++) {
        int y = t / Wp, x = t % Wp;
        for (int j = 0; j < dim_h / 2; j++) {
            float ah = (float)y * hf[j], aw = (float)x * hf[j];
            c[(size_t)t * half + dim_t / 2 + j] = cosf(ah);
            s[(size_t)t * half + dim_t / 2 + j] = sinf(ah);
            c[(size_t)t * half + dim_t / 2 + dim_h / 2 + j] = cosf(aw);
            s[(size_t)t * half + dim_t / 2 + dim_h / 2 + j] = sinf(aw);
        }
    }
}

/* ---- fp16-activation linear layer (tcgemm16.cuh:57-175 behind linear16, kernels.cu:559-609) ----
 * C = epi(A[M,K] . W[N,K]^T); A and W hold fp16-exact values as fp32. The products of fp16 values are exact in
 * fp32; they are summed in double here (the tensor-core kernels sum in fp32, and the reference's own kernel in fp16
 * within each 32-wide k tile: both differ from this only by summation rounding).
 * epi (tcgemm16.cuh:145-174): 0 C = acc; 1 C = fp16(acc); 2 C = fp16(gelu_erf(acc)); 3 C += gate[c] * acc. */
void ko_linear16(float* C, int ldc, const float* A, int lda, const float* W, int ldw, int M, int N, int K, int epi,
                 const float* gate) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int r = 0; r < M; r++)
        for (int c = 0; c < N; c++) {
            const float* a = A + (size_t)r * lda;
            const float* w = W + (size_t)c * ldw;
            double acc = 0;
            for (int k = 0; k < K; k++) acc += (double)a[k] * (double)w[k];
            float v = (float)acc;
            float* dst = C + (size_t)r * ldc + c;
            if (epi == 0) *dst = v;
            else if (epi == 1) *dst = ko_f16_to_f32(ko_f32_to_f16(v));
            else if (epi == 2) *dst = ko_f16_to_f32(ko_f32_to_f16(0.5f * v * (1.f + erff(v * 0.70710678118654752f))));
            else *dst += (gate ? gate[c] : 1.f) * v;
        }
}

/* ---- NAG combine in place on a (dit.cu:295-324): rows of `dim` (= all heads together) ----
 * g = s*p - (s-1)*n; ratio = |g|_1 / max(|p|_1, 1e-12); k = ratio > tau ? tau/ratio : 1;
 * a <- alpha*g*k + (1-alpha)*p.  acc64 != 0 sums the norms in double. */
void ko_nag(float* a, const float* an, int T, int dim, float s, float tau, float alpha, int acc64) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        float* p = a + (size_t)t * dim;
        const float* n = an + (size_t)t * dim;
        float ratio;
        if (acc64) {
            double lp = 0, lg = 0;
            for (int i = 0; i < dim; i++) {
                float g = p[i] * s - n[i] * (s - 1.f);
                lp += fabs((double)p[i]);
                lg += fabs((double)g);
            }
            ratio = (float)(lg / fmax(lp, 1e-12));
        } else {
            /* 256 strided partials, warp butterflies, then a serial sum over 8 warps, as the kernel does */
            float plp[256] = {0}, plg[256] = {0};
            for (int i = 0; i < dim; i++) {
                float g = p[i] * s - n[i] * (s - 1.f);
                plp[i & 255] += fabsf(p[i]);
                plg[i & 255] += fabsf(g);
            }
            float tp = 0.f, tg = 0.f;
            for (int w = 0; w < 8; w++) {
                float *a32 = plp + 32 * w, *b32 = plg + 32 * w;
                for (int o = 16; o > 0; o >>= 1)
                    for (int i = 0; i < o; i++) { a32[i] += a32[i + o]; b32[i] += b32[i + o]; }
                tp += a32[0];
                tg += b32[0];
            }
            ratio = tg / fmaxf(tp, 1e-12f);
        }
        float k = ratio > tau ? tau / ratio : 1.f;
        for (int i = 0; i < dim; i++) {
            float g = p[i] * s - n[i] * (s - 1.f);
            p[i] = alpha * g * k + (1.f - alpha) * p[i];
        }
    }
}
