/*
 * CPU oracle for the INT4 block-16 GEMV decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference engine's CUDA
 * kernels for the decode hot path so that the sm_100a kernels can be checked
 * against it.  It is never linked into, imported by, or called from the shipped
 * library; only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark use it.
 *
 * Parity status: the reference holds no golden vectors, known-answer tests or
 * fixtures for this path (its unit tests are skipped placeholders), and it has
 * no CPU implementation of the GEMV.  The oracle is pinned instead against the
 * reference's own CUDA kernels, rebuilt unchanged for sm_100a into
 * oracle/_ref/ and run on a B200 on the same seeded inputs; the outputs of that
 * run are committed as fixtures under tests/golden/ and re-checked on CPU.
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the reference project's root).
 *
 * Number formats
 *   nibble codec : byte = lo | hi << 4, lo = even-k element, value = nibble - 8
 *                  (src/kernels/gemv_int8.cu:472-479;
 *                   server/inference_server_int4_batched.cu:72-83)
 *   weights      : u8 [N][K/2], one scale per 16-element k-block [N][K/16]
 *   activations  : W4A4: u8 [M][K/2] + f32 [M][K/16]
 *                  W4A8: i8 [M][K]   + f32 [M][K/16]
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QB 16 /* quantization block (elements) */
#define PB 8  /* packed bytes per block        */

/* ------------------------------------------------------------------ helpers */

static inline int nib_lo(uint8_t b) { return (int)(b & 0x0F) - 8; }
static inline int nib_hi(uint8_t b) { return (int)((b >> 4) & 0x0F) - 8; }

/* IEEE binary16 -> binary32, all cases (subnormals, inf, nan). */
static inline float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even. */
static inline uint16_t float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t man = x & 0x7FFFFFu;
    if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - exp);
        uint32_t r = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1))) ++r;
        return (uint16_t)(sign | r);
    }
    uint32_t r = ((uint32_t)exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
    return (uint16_t)(sign | r);
}

void orc_half_to_float(const uint16_t* in, float* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = half_to_float(in[i]);
}
void orc_float_to_half(const float* in, uint16_t* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = float_to_half(in[i]);
}

/* ------------------------------------------------- activation quantization */

/* INT4 activation quantize, block 16.
 * Follows quantize_int4_kernel (src/kernels/gemv_int8.cu:1628-1666):
 *   absmax over the block; sc = absmax > 1e-10 ? absmax/7 : 1/7;
 *   q = clamp((int)roundf(v / sc), -8, 7); byte = (q0+8) | (q1+8) << 4.
 * in f32 [M][K] -> out u8 [M][K/2], sc f32 [M][K/16]. */
void orc_quantize_int4(const float* in, int K, int M, uint8_t* out, float* sc_out) {
    int nkb = K / QB;
    for (int m = 0; m < M; ++m)
        for (int kb = 0; kb < nkb; ++kb) {
            const float* v = in + (size_t)m * K + (size_t)kb * QB;
            float absmax = 0.f;
            for (int i = 0; i < QB; ++i) {
                float a = fabsf(v[i]);
                if (a > absmax) absmax = a;
            }
            float sc = (absmax > 1e-10f) ? (absmax / 7.f) : (1.f / 7.f);
            sc_out[(size_t)m * nkb + kb] = sc;
            for (int i = 0; i < PB; ++i) {
                int q0 = (int)roundf(v[2 * i] / sc);
                int q1 = (int)roundf(v[2 * i + 1] / sc);
                q0 = q0 < -8 ? -8 : (q0 > 7 ? 7 : q0);
                q1 = q1 < -8 ? -8 : (q1 > 7 ? 7 : q1);
                out[(size_t)m * (K / 2) + (size_t)kb * PB + i] =
                    (uint8_t)(((q0 + 8) & 0x0F) | (((q1 + 8) & 0x0F) << 4));
            }
        }
}

/* INT8 activation quantize, block 16.
 * Follows quantize_int8_kernel (src/kernels/gemv_int8.cu:718-748):
 *   sc = absmax/127; if (sc < 1e-10) sc = 1; q = clamp(roundf(v/sc), -127, 127).
 * in f32 [n] -> out i8 [n], sc f32 [n/16]. */
void orc_quantize_int8(const float* in, long n, int8_t* out, float* sc_out) {
    long nkb = n / QB;
    for (long kb = 0; kb < nkb; ++kb) {
        const float* v = in + kb * QB;
        float av = 0.f;
        for (int i = 0; i < QB; ++i) av = fmaxf(av, fabsf(v[i]));
        float sc = av / 127.0f;
        if (sc < 1e-10f) sc = 1.0f;
        sc_out[kb] = sc;
        for (int i = 0; i < QB; ++i) {
            float qf = roundf(v[i] / sc);
            qf = fminf(127.0f, fmaxf(-127.0f, qf));
            out[kb * QB + i] = (int8_t)(int)qf;
        }
    }
}

/* Fused-variant scale rule (src/kernels/fused_int4_ops.cu:155-242, 254-327):
 *   sc = fmaxf(absmax/7, 1e-9); q = clamp(roundf(v/sc), -7, 7) + 8.
 * Same layout as orc_quantize_int4 for one row. */
void orc_quantize_int4_fusedrule(const float* in, int K, uint8_t* out, float* sc_out) {
    int nkb = K / QB;
    for (int kb = 0; kb < nkb; ++kb) {
        const float* v = in + (size_t)kb * QB;
        float absmax = 0.f;
        for (int i = 0; i < QB; ++i) absmax = fmaxf(absmax, fabsf(v[i]));
        float sc = fmaxf(absmax / 7.0f, 1e-9f);
        sc_out[kb] = sc;
        for (int i = 0; i < PB; ++i) {
            float q0 = fminf(7.f, fmaxf(-7.f, roundf(v[2 * i] / sc)));
            float q1 = fminf(7.f, fmaxf(-7.f, roundf(v[2 * i + 1] / sc)));
            out[(size_t)kb * PB + i] = (uint8_t)((((int)q0 + 8) & 0x0F) | ((((int)q1 + 8) & 0x0F) << 4));
        }
    }
}

/* Weight quantizer of the reference's offline tools
 * (scripts/quantize_llama32_1b.py:57-75; better-inference/gguf.h:510-543):
 *   sc = absmax/7 (1.0 when the block is all zero); q = clip(round(w/sc), -7, 7);
 *   nibble = q + 8.  numpy's round is half-to-even, which rintf reproduces. */
void orc_quantize_weights_int4(const float* w, int K, int N, uint8_t* out, float* sc_out) {
    int nkb = K / QB;
    for (int n = 0; n < N; ++n)
        for (int kb = 0; kb < nkb; ++kb) {
            const float* v = w + (size_t)n * K + (size_t)kb * QB;
            float absmax = 0.f;
            for (int i = 0; i < QB; ++i) absmax = fmaxf(absmax, fabsf(v[i]));
            float sc = absmax / 7.0f;
            if (sc == 0.f) sc = 1.0f;
            sc_out[(size_t)n * nkb + kb] = sc;
            for (int i = 0; i < PB; ++i) {
                float q0 = fminf(7.f, fmaxf(-7.f, rintf(v[2 * i] / sc)));
                float q1 = fminf(7.f, fmaxf(-7.f, rintf(v[2 * i + 1] / sc)));
                out[(size_t)n * (K / 2) + (size_t)kb * PB + i] =
                    (uint8_t)((((int)q0 + 8) & 0x0F) | ((((int)q1 + 8) & 0x0F) << 4));
            }
        }
}

/* ------------------------------------------------------ per-block int dots */

static inline int32_t dot16_w4a4(const uint8_t* w, const uint8_t* x) {
    int32_t s = 0;
    for (int j = 0; j < PB; ++j) s += nib_lo(w[j]) * nib_lo(x[j]) + nib_hi(w[j]) * nib_hi(x[j]);
    return s;
}
static inline int32_t dot16_w4a8(const uint8_t* w, const int8_t* x) {
    int32_t s = 0;
    for (int j = 0; j < PB; ++j) s += nib_lo(w[j]) * (int)x[2 * j] + nib_hi(w[j]) * (int)x[2 * j + 1];
    return s;
}

/* Per-block integer dot products for one activation row: dots i32 [N][K/16].
 * The reference forms them in fp32 (gemv_int8.cu:955-962); the values are exact
 * integers there (|sum| <= 16*64), so int32 equality is well defined. */
void orc_block_dots_w4a4(const uint8_t* W, const uint8_t* x, int K, int N, int32_t* dots) {
    int nkb = K / QB;
    for (int n = 0; n < N; ++n)
        for (int kb = 0; kb < nkb; ++kb)
            dots[(size_t)n * nkb + kb] = dot16_w4a4(W + (size_t)n * (K / 2) + (size_t)kb * PB, x + (size_t)kb * PB);
}
void orc_block_dots_w4a8(const uint8_t* W, const int8_t* x, int K, int N, int32_t* dots) {
    int nkb = K / QB;
    for (int n = 0; n < N; ++n)
        for (int kb = 0; kb < nkb; ++kb)
            dots[(size_t)n * nkb + kb] = dot16_w4a8(W + (size_t)n * (K / 2) + (size_t)kb * PB, x + (size_t)kb * QB);
}

/* --------------------------------------------------------------- the GEMV */

/* Exact-order restatement of gemv_int4_batched_kernel<M>
 * (src/kernels/gemv_int8.cu:913-984): lane `tid` of a 32-lane warp walks
 * k-blocks tid, tid+32, ...; per block prod = w_sc * x_sc (one rounding) and
 * acc = fma(sum_f, prod, acc) (nvcc contracts `acc += sum_f * prod`); lanes are
 * then combined by the xor butterfly 16, 8, 4, 2, 1 and lane 0 is written.
 * W u8 [N][K/2], Wsc f32 [N][K/16], x u8 [M][K/2], xsc f32 [M][K/16] -> y f32 [M][N]. */
void orc_gemv_w4a4_exact(float* y, const uint8_t* x, const float* xsc, const uint8_t* W, const float* Wsc,
                         int K, int N, int M) {
    int nkb = K / QB;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            float lane[32];
            for (int l = 0; l < 32; ++l) {
                float acc = 0.f;
                for (int kb = l; kb < nkb; kb += 32) {
                    float sum_f = (float)dot16_w4a4(W + (size_t)n * (K / 2) + (size_t)kb * PB,
                                                    x + (size_t)m * (K / 2) + (size_t)kb * PB);
                    float prod = Wsc[(size_t)n * nkb + kb] * xsc[(size_t)m * nkb + kb];
                    acc = fmaf(sum_f, prod, acc);
                }
                lane[l] = acc;
            }
            for (int off = 16; off > 0; off >>= 1) {
                float nxt[32];
                for (int l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ off];
                memcpy(lane, nxt, sizeof(lane));
            }
            y[(size_t)m * N + n] = lane[0];
        }
    }
}

/* High-precision ground truth for the same computation: integer block dots,
 * double-precision scaling and summation in natural k order. */
void orc_gemv_w4a4_f64(double* y, const uint8_t* x, const float* xsc, const uint8_t* W, const float* Wsc,
                       int K, int N, int M) {
    int nkb = K / QB;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int m = 0; m < M; ++m) {
            double acc = 0.0;
            for (int kb = 0; kb < nkb; ++kb) {
                int32_t d = dot16_w4a4(W + (size_t)n * (K / 2) + (size_t)kb * PB,
                                       x + (size_t)m * (K / 2) + (size_t)kb * PB);
                acc += (double)d * ((double)Wsc[(size_t)n * nkb + kb] * (double)xsc[(size_t)m * nkb + kb]);
            }
            y[(size_t)m * N + n] = acc;
        }
}

/* W4A8 with fp16 weight scales: the same dequant-dot structure
 * (gemv_int8.cu:937-965) with int8 activations produced by quantize_int8
 * (gemv_int8.cu:718-748) and the weight scale stored as binary16. */
void orc_gemv_w4a8_f64(double* y, const int8_t* xq, const float* xsc, const uint8_t* W, const uint16_t* Wsc_h,
                       int K, int N, int M) {
    int nkb = K / QB;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int m = 0; m < M; ++m) {
            double acc = 0.0;
            for (int kb = 0; kb < nkb; ++kb) {
                int32_t d = dot16_w4a8(W + (size_t)n * (K / 2) + (size_t)kb * PB,
                                       xq + (size_t)m * K + (size_t)kb * QB);
                acc += (double)d * ((double)half_to_float(Wsc_h[(size_t)n * nkb + kb]) *
                                    (double)xsc[(size_t)m * nkb + kb]);
            }
            y[(size_t)m * N + n] = acc;
        }
}

/* Scalar fp32 dequant-dot, the form a host port of the reference kernel takes:
 * per block sum_f (exact) * (w_sc * x_sc), accumulated in fp32 in natural k
 * order.  This is the routine timed as the CPU baseline (threads = 0 means all
 * cores).  Returns the thread count used. */
int orc_gemv_w4a8_f32(float* y, const int8_t* xq, const float* xsc, const uint8_t* W, const uint16_t* Wsc_h,
                      int K, int N, int M, int threads) {
    int nkb = K / QB;
    int used = 1;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
    used = threads;
#pragma omp parallel for schedule(static) num_threads(threads)
#endif
    for (int n = 0; n < N; ++n)
        for (int m = 0; m < M; ++m) {
            float acc = 0.f;
            for (int kb = 0; kb < nkb; ++kb) {
                float sum_f = (float)dot16_w4a8(W + (size_t)n * (K / 2) + (size_t)kb * PB,
                                                xq + (size_t)m * K + (size_t)kb * QB);
                float prod = half_to_float(Wsc_h[(size_t)n * nkb + kb]) * xsc[(size_t)m * nkb + kb];
                acc = fmaf(sum_f, prod, acc);
            }
            y[(size_t)m * N + n] = acc;
        }
    return used;
}

int orc_gemv_w4a4_f32(float* y, const uint8_t* x, const float* xsc, const uint8_t* W, const float* Wsc,
                      int K, int N, int M, int threads) {
    int nkb = K / QB;
    int used = 1;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
    used = threads;
#pragma omp parallel for schedule(static) num_threads(threads)
#endif
    for (int n = 0; n < N; ++n)
        for (int m = 0; m < M; ++m) {
            float acc = 0.f;
            for (int kb = 0; kb < nkb; ++kb) {
                float sum_f = (float)dot16_w4a4(W + (size_t)n * (K / 2) + (size_t)kb * PB,
                                                x + (size_t)m * (K / 2) + (size_t)kb * PB);
                acc = fmaf(sum_f, Wsc[(size_t)n * nkb + kb] * xsc[(size_t)m * nkb + kb], acc);
            }
            y[(size_t)m * N + n] = acc;
        }
    return used;
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Row dequantisation, the host statement of the weight format
 * (server/inference_server_int4_batched.cu:72-83). */
void orc_dequant_row(float* out, long row, const uint8_t* W, const float* Wsc, int K) {
    int nkb = K / QB;
    for (int b = 0; b < nkb; ++b) {
        float sc = Wsc[(size_t)row * nkb + b];
        for (int i = 0; i < QB; ++i) {
            uint8_t byte = W[(size_t)row * (K / 2) + (size_t)b * PB + i / 2];
            int nib = (i & 1) ? ((byte >> 4) & 0x0F) : (byte & 0x0F);
            out[b * QB + i] = (float)(nib - 8) * sc;
        }
    }
}

/* ------------------------------------------------------ norm / elementwise */

/* RMSNorm: out = x * w * rsqrt(mean(x^2) + eps)  (src/kernels/norm.cu:44-89,
 * 114-155).  Double-precision reduction; all H elements participate (the
 * reference kernel silently drops elements >= 4096, a defect not restated). */
void orc_rmsnorm(float* out, const float* in, const float* w, int H, float eps, int M) {
    for (int m = 0; m < M; ++m) {
        const float* x = in + (size_t)m * H;
        double ss = 0.0;
        for (int i = 0; i < H; ++i) ss += (double)x[i] * (double)x[i];
        double rstd = 1.0 / sqrt(ss / (double)H + (double)eps);
        for (int i = 0; i < H; ++i) out[(size_t)m * H + i] = (float)((double)x[i] * (double)w[i] * rstd);
    }
}

/* Exact-order RMSNorm for H <= 4096 (norm.cu:44-89): thread t of 128 sums
 * elements 32t..32t+31 sequentially with fma, shfl_down tree 16..1 inside each
 * warp, then the 4 warp partials through the same tree; the final rsqrt is
 * taken as 1/sqrtf here (the device uses an approximate rsqrtf), so outputs
 * are compared with a 2-ulp allowance, not bitwise. */
void orc_rmsnorm_reforder(float* out, const float* in, const float* w, int H, float eps, int M) {
    for (int m = 0; m < M; ++m) {
        const float* x = in + (size_t)m * H;
        float part[128];
        for (int t = 0; t < 128; ++t) {
            float s = 0.f;
            int start = t * 32, end = start + 32 < H ? start + 32 : H;
            for (int i = start; i < end; ++i) s = fmaf(x[i], x[i], s);
            part[t] = s;
        }
        float wsum[4];
        for (int wp = 0; wp < 4; ++wp) {
            float v[32];
            memcpy(v, part + wp * 32, sizeof(v));
            for (int off = 16; off > 0; off >>= 1)
                for (int l = 0; l < 32; ++l) v[l] = v[l] + ((l + off < 32) ? v[l + off] : v[l]);
            wsum[wp] = v[0];
        }
        /* shfl_down tree over lanes 0..3 holding the warp partials, zeros above */
        float v[32] = {0};
        for (int i = 0; i < 4; ++i) v[i] = wsum[i];
        for (int off = 16; off > 0; off >>= 1)
            for (int l = 0; l < 32; ++l) v[l] = v[l] + ((l + off < 32) ? v[l + off] : v[l]);
        float rstd = 1.0f / sqrtf(v[0] / (float)H + eps);
        int lim = H < 4096 ? H : 4096;
        for (int i = 0; i < lim; ++i) out[(size_t)m * H + i] = x[i] * w[i] * rstd;
    }
}

/* SwiGLU: silu(g) * u with silu(x) = x / (1 + expf(-x))  (norm.cu:37-39,94-106). */
void orc_swiglu(float* out, const float* g, const float* u, long n) {
    for (long i = 0; i < n; ++i) out[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
}

/* The fused SwiGLU+quantize kernel writes the same function as
 * g * (1 / (1 + expf(-g))) * u  (src/kernels/fused_int4_ops.cu:270-277). */
void orc_swiglu_fusedform(float* out, const float* g, const float* u, long n) {
    for (long i = 0; i < n; ++i) out[i] = g[i] * (1.0f / (1.0f + expf(-g[i]))) * u[i];
}

/* Residual add (norm.cu:191-206). */
void orc_vector_add(float* out, const float* a, const float* b, long n) {
    for (long i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

/* Per-head RMSNorm then interleaved-pair RoPE, the two caller-side kernels of
 * the decode loop (server/inference_server_int4_batched.cu:49-70):
 *   d = d * rsqrt(mean(d^2) + eps) * w ;  theta = pos * 1e6^(-2i/hd),
 *   (x, y) = (x cos - y sin, x sin + y cos) on pairs (2i, 2i+1). */
void orc_head_norm(float* data, const float* w, int nh, int hd, float eps) {
    for (int h = 0; h < nh; ++h) {
        float* d = data + (size_t)h * hd;
        double s = 0.0;
        for (int i = 0; i < hd; ++i) s += (double)d[i] * d[i];
        float is = (float)(1.0 / sqrt(s / hd + (double)eps));
        for (int i = 0; i < hd; ++i) d[i] = d[i] * is * w[i];
    }
}
void orc_rope(float* data, int nh, int hd, int pos) {
    for (int h = 0; h < nh; ++h)
        for (int i = 0; i < hd / 2; ++i) {
            float* p = data + (size_t)h * hd + 2 * i;
            float theta = (float)pos * powf(1000000.0f, -2.0f * (float)i / (float)hd);
            float c = cosf(theta), s = sinf(theta), x = p[0], y = p[1];
            p[0] = x * c - y * s;
            p[1] = x * s + y * c;
        }
}

/* ---------------------------------------------------------------- KV cache */

/* update_kv_kernel (src/kernels/decode.cu:27-46): cache layout [head][max_seq][hd]. */
void orc_update_kv(float* kc, float* vc, const float* k_new, const float* v_new, int seq_pos, int nh, int hd,
                   int max_seq) {
    for (int h = 0; h < nh; ++h)
        for (int d = 0; d < hd; ++d) {
            size_t off = (size_t)h * max_seq * hd + (size_t)seq_pos * hd + d;
            kc[off] = k_new[h * hd + d];
            vc[off] = v_new[h * hd + d];
        }
}

/* GQA decode attention over an fp32 cache, the mathematics of
 * attn_batched_kernel (src/kernels/decode.cu:375-466): kv_head = head*nkv/nqh,
 * scores = q.K[t] / sqrt(hd) for t <= seq_pos, softmax with max subtraction,
 * out = sum p V / (sum p + 1e-9).  Sequential, race-free, in double. */
void orc_attention_decode_gqa(float* out, const float* Q, const float* Kc, const float* Vc, const int* seq_pos,
                              int per_seq_pos, int nqh, int nkv, int hd, int max_seq, int M,
                              size_t kv_batch_elems, size_t kv_layer_elems) {
    double scale = 1.0 / sqrt((double)hd);
#pragma omp parallel for schedule(static) collapse(2)
    for (int m = 0; m < M; ++m)
        for (int h = 0; h < nqh; ++h) {
            int kvh = h * nkv / nqh;
            int npos = (per_seq_pos ? seq_pos[m] : seq_pos[0]) + 1;
            const float* K = Kc + (size_t)m * kv_batch_elems + kv_layer_elems + (size_t)kvh * max_seq * hd;
            const float* V = Vc + (size_t)m * kv_batch_elems + kv_layer_elems + (size_t)kvh * max_seq * hd;
            const float* q = Q + ((size_t)m * nqh + h) * hd;
            double* sc = (double*)malloc(sizeof(double) * (size_t)npos);
            double mx = -1e300;
            for (int t = 0; t < npos; ++t) {
                double d = 0.0;
                for (int i = 0; i < hd; ++i) d += (double)q[i] * (double)K[(size_t)t * hd + i];
                sc[t] = d * scale;
                if (sc[t] > mx) mx = sc[t];
            }
            double sum = 0.0;
            for (int t = 0; t < npos; ++t) {
                sc[t] = exp(sc[t] - mx);
                sum += sc[t];
            }
            double inv = 1.0 / (sum + 1e-9);
            for (int i = 0; i < hd; ++i) {
                double o = 0.0;
                for (int t = 0; t < npos; ++t) o += sc[t] * (double)V[(size_t)t * hd + i];
                out[((size_t)m * nqh + h) * hd + i] = (float)(o * inv);
            }
            free(sc);
        }
}

/* Same mathematics over a binary16 cache laid out [M][nkv][max_seq][hd]. */
void orc_attention_decode_f16kv(float* out, const float* Q, const uint16_t* Kc, const uint16_t* Vc,
                                const int* seq_pos, int nqh, int nkv, int hd, int max_seq, int M) {
    double scale = 1.0 / sqrt((double)hd);
#pragma omp parallel for schedule(static) collapse(2)
    for (int m = 0; m < M; ++m)
        for (int h = 0; h < nqh; ++h) {
            int kvh = h * nkv / nqh;
            int npos = seq_pos[m] + 1;
            const uint16_t* K = Kc + ((size_t)m * nkv + kvh) * (size_t)max_seq * hd;
            const uint16_t* V = Vc + ((size_t)m * nkv + kvh) * (size_t)max_seq * hd;
            const float* q = Q + ((size_t)m * nqh + h) * hd;
            double* sc = (double*)malloc(sizeof(double) * (size_t)npos);
            double mx = -1e300;
            for (int t = 0; t < npos; ++t) {
                double d = 0.0;
                for (int i = 0; i < hd; ++i) d += (double)q[i] * (double)half_to_float(K[(size_t)t * hd + i]);
                sc[t] = d * scale;
                if (sc[t] > mx) mx = sc[t];
            }
            double sum = 0.0;
            for (int t = 0; t < npos; ++t) {
                sc[t] = exp(sc[t] - mx);
                sum += sc[t];
            }
            double inv = 1.0 / (sum + 1e-9);
            for (int i = 0; i < hd; ++i) {
                double o = 0.0;
                for (int t = 0; t < npos; ++t) o += sc[t] * (double)half_to_float(V[(size_t)t * hd + i]);
                out[((size_t)m * nqh + h) * hd + i] = (float)(o * inv);
            }
            free(sc);
        }
}

/* ----------------------------------------------------------------- sampling */

/* Greedy argmax (src/kernels/sample_gpu.cu:30-60).  Candidates start at
 * (-1e38, 0) and are replaced only on strict '>'; on an exact tie the lowest
 * index wins here. */
int orc_argmax(const float* logits, int vocab) {
    float bv = -1e38f;
    int bi = 0;
    for (int i = 0; i < vocab; ++i)
        if (logits[i] > bv) { bv = logits[i]; bi = i; }
    return bi;
}

/* Repetition penalty (src/kernels/decode.cu:694-731): for every id listed in
 * recent[], once: logit > 0 ? logit / p : logit * p.  No-op when p <= 1 or the
 * list is empty. */
void orc_repetition_penalty(float* logits, const int* recent, int num_recent, float penalty, int vocab) {
    if (penalty <= 1.0f || num_recent == 0) return;
    for (int v = 0; v < vocab; ++v)
        for (int i = 0; i < num_recent; ++i)
            if (recent[i] == v) {
                logits[v] = logits[v] > 0 ? logits[v] / penalty : logits[v] * penalty;
                break;
            }
}
