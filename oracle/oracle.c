/*
 * CPU oracle for the FP8 decode hot path.  TEST INFRASTRUCTURE ONLY: this file is
 * the checker the CUDA kernels are compared against (and the timed CPU baseline);
 * nothing in the product library links, loads or calls it.
 *
 * Every function restates, in plain C, the arithmetic of the reference project
 * (solidsf-inc/rvLLM v0.3.0); the file:line each one follows is cited beside it.
 * Paths are relative to the reference checkout.
 *
 * Parity pin: the encoder, RMSNorm, argmax and launcher known-answer vectors that the
 * reference's own tests hold (v3/crates/rvllm-core/src/fp8.rs:67-104,
 * v3/crates/rvllm-fused/src/reference.rs:341-405,
 * v3/crates/rvllm-invariants/tests/identity.rs:91-128, scripts/test_fp8_encode.py:10-31)
 * are replayed against this file by the CPU test-suite.  FP8 GEMM for M>1 has no
 * golden vector in the reference ("parity unpinned" for that one stage: the only
 * pin is the f64 host check of v3/crates/rvllm-bench/src/main.rs:832-843, which the
 * f64 mode below restates).
 *
 * Build: see Makefile (gcc -O3 -fopenmp -shared, no fast-math, no fp contraction).
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define FP8_MAX 448.0f

/* ------------------------------------------------------------------------- */
/* bit helpers                                                                */
/* ------------------------------------------------------------------------- */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* 16-bit storage types: dtype 0 = IEEE binary16 (what the reference uses,
 * kernels/fused_rmsnorm_fp8_quant.cu:56-57), 1 = bfloat16. */
float orc_h2f(uint16_t h, int dtype) {
    if (dtype == 1) return u2f((uint32_t)h << 16);
    uint32_t s = (uint32_t)(h >> 15) << 31;
    uint32_t e = (h >> 10) & 0x1f, m = h & 0x3ff;
    if (e == 0) {
        if (m == 0) return u2f(s);
        float v = (float)m * 5.9604644775390625e-8f; /* m * 2^-24 */
        return s ? -v : v;
    }
    if (e == 31) return u2f(s | 0x7f800000u | (m << 13));
    return u2f(s | ((e + 112u) << 23) | (m << 13));
}

/* round-to-nearest-even narrowing, as __float2half / __float2bfloat16 do */
uint16_t orc_f2h(float f, int dtype) {
    uint32_t u = f2u(f);
    if (dtype == 1) {
        if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
        uint32_t lsb = (u >> 16) & 1u;
        u += 0x7fffu + lsb;
        return (uint16_t)(u >> 16);
    }
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (a >= 0x47800000u) { /* >= 65536 -> inf (values in [65520,65536) round below) */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (a < 0x33000001u) return (uint16_t)sign; /* <= 2^-25 -> 0 (tie to even) */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    uint32_t shift, out;
    if (e < -14) {
        shift = (uint32_t)(13 + (-14 - e));
        out = 0;
    } else {
        shift = 13;
        out = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    out += q; /* mantissa carry propagates into the exponent, incl. to inf */
    return (uint16_t)(sign | out);
}

/* f16 narrowing that clamps to the largest finite value, as
 * v3/kernels/f32_to_f16_sat.cu:4-15 does after the reference GEMV. */
static inline uint16_t f2h_sat(float f, int dtype) {
    if (dtype == 0) {
        if (f > 65504.0f) f = 65504.0f;
        if (f < -65504.0f) f = -65504.0f;
    }
    return orc_f2h(f, dtype);
}

/* ------------------------------------------------------------------------- */
/* FP8 E4M3FN                                                                 */
/* ------------------------------------------------------------------------- */

/* v3/crates/rvllm-core/src/fp8.rs:12-65.  mode 0 = the Rust host encoder
 * (every zero result is the one +0 byte); mode 1 = what the CUDA kernels'
 * __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3) produces
 * (kernels/fused_rmsnorm_fp8_quant.cu:101): same rounding, but a negative
 * input that rounds to zero keeps its sign bit (0x80). */
uint8_t orc_e4m3_encode(float x, int mode) {
    if (x != x) return 0x7f;
    uint32_t bits = f2u(x);
    uint8_t sign = (bits >> 31) ? 0x80 : 0;
    uint8_t zero = mode ? sign : 0;
    bits &= 0x7fffffffu;
    float mag = u2f(bits);
    if (mag == 0.0f) return zero;
    if (mag > FP8_MAX) return sign | 0x7e;
    int exp32 = (int)((bits >> 23) & 0xff) - 127;
    uint32_t mant32 = bits & 0x7fffffu;
    int exp8 = exp32 + 7;
    if (exp8 <= 0) {
        int shift = 1 - exp8;
        uint32_t full = mant32 | (1u << 23);
        uint32_t rshift = (uint32_t)(20 + shift);
        if (rshift >= 32) return zero;
        uint32_t mantissa = full >> rshift;
        uint32_t round_bit = (full >> (rshift - 1)) & 1u;
        uint32_t sticky = (full & ((1u << (rshift - 1)) - 1u)) != 0;
        mantissa += round_bit & (sticky | (mantissa & 1u));
        if (mantissa >= 8) return sign | 0x08;
        if (mantissa == 0) return zero;
        return sign | (uint8_t)(mantissa & 7u);
    }
    uint32_t truncated = mant32 >> 20;
    uint32_t round_bit = (mant32 >> 19) & 1u;
    uint32_t sticky = (mant32 & 0x7ffffu) != 0;
    uint32_t mantissa = truncated + (round_bit & (sticky | (truncated & 1u)));
    if (mantissa >= 8) {
        exp8 += 1;
        if (exp8 > 15) return sign | 0x7e;
        return sign | (uint8_t)((exp8 & 0xf) << 3);
    }
    if (exp8 > 15) return sign | 0x7e;
    return sign | (uint8_t)((exp8 & 0xf) << 3) | (uint8_t)(mantissa & 7u);
}

/* v3/kernels/fp8_decode_v2.cu:41-56 (bit-math decode; 0x7f / 0xff are NaN) */
float orc_e4m3_decode(uint8_t x) {
    uint32_t s = (x >> 7) & 1u, e = (x >> 3) & 0xfu, m = x & 7u;
    if (e == 0) {
        if (m == 0) return 0.0f;
        float v = (float)m * 1.953125e-3f;
        return s ? -v : v;
    }
    if (e == 15 && m == 7) return u2f(0x7fc00000u);
    return u2f((s << 31) | ((e + 120u) << 23) | (m << 20));
}

void orc_e4m3_encode_n(const float *in, uint8_t *out, size_t n, int mode) {
    for (size_t i = 0; i < n; i++) out[i] = orc_e4m3_encode(in[i], mode);
}
void orc_e4m3_decode_n(const uint8_t *in, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = orc_e4m3_decode(in[i]);
}

static float g_lut[256];
static int g_lut_ready = 0;
static void lut_init(void) {
    if (g_lut_ready) return;
    for (int i = 0; i < 256; i++) g_lut[i] = orc_e4m3_decode((uint8_t)i);
    g_lut_ready = 1;
}

/* ------------------------------------------------------------------------- */
/* block reductions in the order the reference kernels perform them           */
/* ------------------------------------------------------------------------- */

/* kernels/fused_rmsnorm_fp8_quant.cu:11-36: per-thread strided partials, xor
 * butterfly inside each warp (offsets 16..1), warp totals parked in shared
 * memory, then warp 0 runs the same butterfly over lane<num_warps. */
static float block_sum_ref_order(const float *partial, int block_dim) {
    float warp_tot[32];
    int num_warps = (block_dim + 31) / 32;
    for (int w = 0; w < num_warps; w++) {
        float v[32];
        for (int l = 0; l < 32; l++) {
            int t = w * 32 + l;
            v[l] = t < block_dim ? partial[t] : 0.0f;
        }
        for (int off = 16; off > 0; off >>= 1) {
            float nv[32];
            for (int l = 0; l < 32; l++) nv[l] = v[l] + v[l ^ off];
            memcpy(v, nv, sizeof v);
        }
        warp_tot[w] = v[0];
    }
    float v[32];
    for (int l = 0; l < 32; l++) v[l] = l < num_warps ? warp_tot[l] : 0.0f;
    for (int off = 16; off > 0; off >>= 1) {
        float nv[32];
        for (int l = 0; l < 32; l++) nv[l] = v[l] + v[l ^ off];
        memcpy(v, nv, sizeof v);
    }
    return v[0];
}

/* Scale + encode of one row of f32 values.
 * mode 0: v3/crates/rvllm-fused/src/reference.rs:91-106 (amax clamped to 1e-12,
 *         scale = amax/448, encode(value / scale), Rust encoder).
 * mode 1: kernels/fused_rmsnorm_fp8_quant.cu:92-101 (scale = max(absmax/448, 1e-12),
 *         inv = 1/scale, encode(value * inv), CUDA encoder).
 * A non-finite value makes the row scale NaN in mode 1 when nan_on_invalid is set
 * (kernels/fused_silu_fp8_quant.cu:87,101). */
static void quant_row(const float *v, int n, uint8_t *out, float *scale_out, int mode,
                      int nan_on_invalid) {
    float amax = 0.0f;
    int invalid = 0;
    for (int i = 0; i < n; i++) {
        float a = fabsf(v[i]);
        if (!isfinite(v[i])) invalid = 1;
        amax = fmaxf(amax, a); /* fmaxf ignores NaN like the device fmaxf */
    }
    if (mode == 0) {
        amax = fmaxf(amax, 1e-12f);
        float scale = amax / FP8_MAX;
        *scale_out = scale;
        for (int i = 0; i < n; i++) out[i] = orc_e4m3_encode(v[i] / scale, 0);
    } else {
        float scale = fmaxf(amax / FP8_MAX, 1e-12f);
        if (nan_on_invalid && invalid) scale = u2f(0x7fffffffu); /* CUDART_NAN_F */
        *scale_out = scale;
        float inv = 1.0f / scale;
        for (int i = 0; i < n; i++) out[i] = orc_e4m3_encode(v[i] * inv, 1);
    }
}

/* ------------------------------------------------------------------------- */
/* stage 1: RMSNorm + per-token FP8 quantisation                              */
/* ------------------------------------------------------------------------- */

/* mode 0: rmsnorm_ref + quantize_fp8_per_token_ref,
 *         v3/crates/rvllm-fused/src/reference.rs:40-109 (sequential sum, 1/sqrt).
 * mode 1: fused_rmsnorm_fp8_quant_kernel, kernels/fused_rmsnorm_fp8_quant.cu:52-103,
 *         reduction order for a launch of block_dim threads.  The device rsqrtf is
 *         an approximation (2 ulp); 1/sqrtf stands in for it here, so scales may
 *         differ from the GPU's in the last place.
 * residual (may be NULL): fused_add_rmsnorm_fp8_quant_kernel :108-160 — writes the
 * rounded sum to residual_out, sums squares of the unrounded f32 sum, then
 * normalises the ROUNDED value (:129-131,143). */
int orc_rmsnorm_fp8_quant(uint8_t *out, float *scales, uint16_t *residual_out,
                          const uint16_t *in, const uint16_t *residual,
                          const uint16_t *gamma, float eps, int num_tokens, int hidden,
                          int dtype, int mode, int block_dim) {
    if (num_tokens <= 0 || hidden <= 0 || !out || !scales || !in || !gamma) return -1;
    if (block_dim <= 0 || block_dim > 1024) return -1;
    float *v = (float *)malloc(sizeof(float) * (size_t)hidden);
    float *x = (float *)malloc(sizeof(float) * (size_t)hidden);
    float partial[1024];
    for (int r = 0; r < num_tokens; r++) {
        const uint16_t *row = in + (size_t)r * hidden;
        float ss;
        if (mode == 0) {
            ss = 0.0f;
            for (int i = 0; i < hidden; i++) {
                float a = orc_h2f(row[i], dtype);
                if (residual) a += orc_h2f(residual[(size_t)r * hidden + i], dtype);
                x[i] = a;
                ss += a * a;
            }
            if (residual && residual_out)
                for (int i = 0; i < hidden; i++)
                    residual_out[(size_t)r * hidden + i] = orc_f2h(x[i], dtype);
        } else {
            for (int t = 0; t < block_dim; t++) partial[t] = 0.0f;
            for (int i = 0; i < hidden; i++) {
                float a = orc_h2f(row[i], dtype);
                if (residual) a += orc_h2f(residual[(size_t)r * hidden + i], dtype);
                partial[i % block_dim] = fmaf(a, a, partial[i % block_dim]); /* i ascending == thread-strided order; device code contracts to fma */
                if (residual) {
                    uint16_t h = orc_f2h(a, dtype);
                    if (residual_out) residual_out[(size_t)r * hidden + i] = h;
                    a = orc_h2f(h, dtype);
                }
                x[i] = a;
            }
            ss = block_sum_ref_order(partial, block_dim);
        }
        float rms;
        if (mode == 0) rms = 1.0f / sqrtf(ss / (float)hidden + eps);
        else rms = 1.0f / sqrtf(ss / (float)hidden + eps);
        for (int i = 0; i < hidden; i++) v[i] = x[i] * rms * orc_h2f(gamma[i], dtype);
        quant_row(v, hidden, out + (size_t)r * hidden, scales + r, mode, 0);
    }
    free(v);
    free(x);
    return 0;
}

/* f32-in / f32-out RMSNorm exactly as rmsnorm_ref (reference.rs:40-80), for the
 * hand-calculated known-answer test (reference.rs:341-350). */
int orc_rmsnorm_f32(const float *x, const float *gamma, float eps, int hidden, int rows,
                    float *out) {
    if (hidden <= 0 || rows <= 0 || !isfinite(eps)) return -1;
    for (int r = 0; r < rows; r++) {
        float ms = 0.0f;
        for (int i = 0; i < hidden; i++) {
            float a = x[(size_t)r * hidden + i];
            if (!isfinite(a)) return -1;
            ms += a * a;
            if (!isfinite(ms)) return -1;
        }
        ms /= (float)hidden;
        float den = ms + eps;
        if (!isfinite(den) || den <= 0.0f) return -1;
        float inv = 1.0f / sqrtf(den);
        for (int i = 0; i < hidden; i++) {
            float o = x[(size_t)r * hidden + i] * inv * gamma[i];
            if (!isfinite(o)) return -1;
            out[(size_t)r * hidden + i] = o;
        }
    }
    return 0;
}

/* quantize_fp8_per_token_kernel, kernels/fused_rmsnorm_fp8_quant.cu:166-200 (mode 1);
 * quantize_fp8_per_token_ref, reference.rs:82-109 (mode 0). */
int orc_quantize_fp8_per_token(uint8_t *out, float *scales, const uint16_t *in,
                               int num_tokens, int dim, int dtype, int mode) {
    if (num_tokens <= 0 || dim <= 0 || !out || !scales || !in) return -1;
    float *v = (float *)malloc(sizeof(float) * (size_t)dim);
    for (int r = 0; r < num_tokens; r++) {
        for (int i = 0; i < dim; i++) v[i] = orc_h2f(in[(size_t)r * dim + i], dtype);
        quant_row(v, dim, out + (size_t)r * dim, scales + r, mode, 0);
    }
    free(v);
    return 0;
}

/* Same on f32 input (the Rust reference is f32-in). */
int orc_quantize_fp8_per_token_f32(uint8_t *out, float *scales, const float *in,
                                   int num_tokens, int dim, int mode) {
    if (num_tokens <= 0 || dim <= 0) return -1;
    for (int r = 0; r < num_tokens; r++)
        quant_row(in + (size_t)r * dim, dim, out + (size_t)r * dim, scales + r, mode, 0);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* stage 2c: act(gate) * up + per-token FP8 quantisation                      */
/* ------------------------------------------------------------------------- */

/* act 0 = SiLU: kernels/fused_silu_fp8_quant.cu:42-120, reference.rs:137-166.
 * act 1 = GELU-tanh: v3/kernels/fused_gelu_mul_fp8_quant.cu:41-47,53-129,
 *         reference.rs:168-198.  Row layout [gate(0..I) | up(I..2I)]. */
static inline float act_f32(float g, int act) {
    if (act == 0) return g / (1.0f + expf(-g));
    float x3 = g * g * g; /* the device compiler contracts x + c*x3 into one fma */
    float inner = 0.7978845608f * fmaf(0.044715f, x3, g);
    return 0.5f * g * (1.0f + tanhf(inner));
}

int orc_act_mul_fp8_quant(uint8_t *out, float *scales, const uint16_t *gate_up,
                          int num_tokens, int inter, int act, int dtype, int mode) {
    if (num_tokens <= 0 || inter <= 0 || !out || !scales || !gate_up) return -1;
    float *v = (float *)malloc(sizeof(float) * (size_t)inter);
    for (int r = 0; r < num_tokens; r++) {
        const uint16_t *g = gate_up + (size_t)r * 2 * inter;
        const uint16_t *u = g + inter;
        for (int i = 0; i < inter; i++)
            v[i] = act_f32(orc_h2f(g[i], dtype), act) * orc_h2f(u[i], dtype);
        quant_row(v, inter, out + (size_t)r * inter, scales + r, mode, 1);
    }
    free(v);
    return 0;
}

/* f32 [T, 2I] input variant: the fused GEMM epilogue applies the activation to
 * unrounded accumulators; this is the same arithmetic on supplied f32 values. */
int orc_act_mul_fp8_quant_f32(uint8_t *out, float *scales, const float *gate_up,
                              int num_tokens, int inter, int act, int mode) {
    if (num_tokens <= 0 || inter <= 0) return -1;
    float *v = (float *)malloc(sizeof(float) * (size_t)inter);
    for (int r = 0; r < num_tokens; r++) {
        const float *g = gate_up + (size_t)r * 2 * inter;
        for (int i = 0; i < inter; i++) v[i] = act_f32(g[i], act) * g[inter + i];
        quant_row(v, inter, out + (size_t)r * inter, scales + r, mode, 1);
    }
    free(v);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* stage 2: per-row x per-output-channel scaled FP8 GEMM                       */
/* ------------------------------------------------------------------------- */

/* D[m,n] = cast( a_scale[m] * (w_scale[n] * acc) (+ residual[m,n]) ),
 * acc = sum_k dec(A[m,k]) * dec(W[n,k]); A [M,K] row-major, W [N,K] row-major.
 * Epilogue order: kernels/cutlass_fp8_gemm_channelscale.cu:41-62 and
 * kernels/cutlass_fp8_gemm_residual.cu:48-83.  acc64 = 1 accumulates in f64 like
 * the host check of v3/crates/rvllm-bench/src/main.rs:832-843; acc64 = 0 is the
 * fp32-accumulated reference the tolerance is stated against.
 * out_kind: 0 f16 (saturating), 1 bf16, 2 f32.  residual has the output's 16-bit type. */
int orc_fp8_gemm(void *out, const uint8_t *a, const uint8_t *w, const float *a_scale,
                 const float *w_scale, const void *residual, int M, int N, int K,
                 int out_kind, int acc64) {
    if (M <= 0 || N <= 0 || K <= 0 || !out || !a || !w || !a_scale || !w_scale) return -1;
    lut_init();
    float *af = (float *)malloc(sizeof(float) * (size_t)M * K);
    for (size_t i = 0; i < (size_t)M * K; i++) af[i] = g_lut[a[i]];
#pragma omp parallel
    {
        float *wf = (float *)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
        for (int n = 0; n < N; n++) {
            const uint8_t *wr = w + (size_t)n * K;
            for (int k = 0; k < K; k++) wf[k] = g_lut[wr[k]];
            for (int m = 0; m < M; m++) {
                const float *ar = af + (size_t)m * K;
                float accf;
                if (acc64) {
                    double acc = 0.0;
                    for (int k = 0; k < K; k++) acc += (double)ar[k] * (double)wf[k];
                    accf = (float)acc;
                } else {
                    /* fp32 accumulation in 8 interleaved lanes (lane j takes k = j mod 8), lanes
                     * added pairwise at the end: a fixed order that the compiler can keep in one
                     * vector register, so the timed CPU baseline is not a scalar strawman. */
                    float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    int k = 0;
                    for (; k + 8 <= K; k += 8)
                        for (int j = 0; j < 8; j++) lane[j] += ar[k + j] * wf[k + j];
                    for (; k < K; k++) lane[k & 7] += ar[k] * wf[k];
                    accf = ((lane[0] + lane[4]) + (lane[2] + lane[6])) + ((lane[1] + lane[5]) + (lane[3] + lane[7]));
                }
                float v = a_scale[m] * (w_scale[n] * accf);
                size_t o = (size_t)m * N + n;
                if (out_kind == 2) {
                    if (residual) v += ((const float *)residual)[o];
                    ((float *)out)[o] = v;
                } else {
                    if (residual) v += orc_h2f(((const uint16_t *)residual)[o], out_kind);
                    ((uint16_t *)out)[o] = f2h_sat(v, out_kind);
                }
            }
        }
        free(wf);
    }
    free(af);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* stage 3: FP8-KV paged GQA decode attention                                  */
/* ------------------------------------------------------------------------- */

/* Token -> cache slot, v3/kernels/fp8_decode_v2.cu:266-274,296:
 * page = t / block_size; sliding layers index the table as a ring
 * (page % max_blocks_per_seq); slot = phys * block_size + t % block_size.
 * Returns -1 when the physical block is outside [0, num_blocks_total). */
long long orc_resolve_slot(const int *block_tables, int seq, long long t, int block_size,
                           int max_blocks_per_seq, int num_blocks_total,
                           int window_size_left) {
    long long p = t / block_size;
    int table_page = window_size_left >= 0 ? (int)(p % max_blocks_per_seq) : (int)p;
    int phys = block_tables[(long long)seq * max_blocks_per_seq + table_page];
    if (phys < 0 || phys >= num_blocks_total) return -1;
    return (long long)phys * block_size + (t % block_size);
}

/* attended interval, fp8_decode_v2.cu:258-264 */
static void attend_interval(int ctx_len, int window_size_left, int *start, int *len) {
    *start = 0;
    *len = ctx_len;
    if (window_size_left >= 0 && *len > window_size_left + 1) {
        *len = window_size_left + 1;
        *start = ctx_len - *len;
    }
}

/* Fill `slots` (length batch * max_attend) with the resolved cache slot of every
 * attended token; used by the block-table index-echo test. */
int orc_attended_slots(long long *slots, int max_attend, const int *block_tables,
                       const int *context_lens, int batch, int block_size,
                       int max_blocks_per_seq, int num_blocks_total, int window_size_left) {
    for (int b = 0; b < batch; b++) {
        int start, len;
        attend_interval(context_lens[b], window_size_left, &start, &len);
        for (int i = 0; i < max_attend; i++) {
            slots[(size_t)b * max_attend + i] =
                i < len ? orc_resolve_slot(block_tables, b, (long long)start + i, block_size,
                                           max_blocks_per_seq, num_blocks_total,
                                           window_size_left)
                        : -2;
        }
    }
    return 0;
}

/* precise = 0: f32 step order of the scalar reference kernel
 *   paged_decode_fp8_kernel_reference, v3/kernels/fp8_decode_v2.cu:199-325
 *   (online softmax, m0 = -1e20, expf in place of the device __expf);
 * precise = 1: two-pass f64 softmax like reference_attention,
 *   v3/kernels/fa3_sm90_parity_bench.cu:252-325.
 * Guards (:229-236,271-274,306-311): ctx<0 or (no window and ctx > capacity) -> NaN row;
 * ctx==0 -> zeros; bad physical block or bad scale -> NaN row.
 * Output [batch, heads, head_dim] in the 16-bit type `dtype` (reference: f16). */
int orc_paged_decode_fp8(uint16_t *out, const uint8_t *q, const uint8_t *k_cache,
                         const uint8_t *v_cache, const int *block_tables,
                         const int *context_lens, const float *k_scale_cache,
                         const float *v_scale_cache, const float *q_scale_cache,
                         const float *q_descale, const float *k_descale,
                         const float *v_descale, float scale, int batch, int heads,
                         int kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                         int num_blocks_total, int window_size_left, int precise, int dtype) {
    if (batch <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || head_dim <= 0 ||
        block_size <= 0 || max_blocks_per_seq <= 0 || num_blocks_total <= 0 ||
        window_size_left < -1)
        return -1;
    if ((!q_scale_cache && !q_descale) || (!k_scale_cache && !k_descale) ||
        (!v_scale_cache && !v_descale))
        return -1;
    lut_init();
    const uint16_t nan16 = orc_f2h(u2f(0x7fc00000u), dtype);
    const long long capacity = (long long)block_size * max_blocks_per_seq;
    int work = batch * heads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int bh = 0; bh < work; bh++) {
        int b = bh / heads, h = bh % heads;
        int kvh = (int)((long long)h * kv_heads / heads);
        uint16_t *o = out + (size_t)bh * head_dim;
        int ctx = context_lens[b];
        if (ctx < 0 || (window_size_left < 0 && (long long)ctx > capacity)) {
            for (int d = 0; d < head_dim; d++) o[d] = nan16;
            continue;
        }
        if (ctx == 0) {
            for (int d = 0; d < head_dim; d++) o[d] = orc_f2h(0.0f, dtype);
            continue;
        }
        float q_ds = q_scale_cache ? q_scale_cache[(size_t)b * heads + h] : *q_descale;
        int start, len;
        attend_interval(ctx, window_size_left, &start, &len);
        int bad = 0;
        const uint8_t *qrow = q + (size_t)bh * head_dim;
        if (!precise) {
            float *qv = (float *)malloc(sizeof(float) * head_dim);
            float *acc = (float *)calloc(head_dim, sizeof(float));
            for (int d = 0; d < head_dim; d++) qv[d] = g_lut[qrow[d]] * q_ds;
            float m = -1e20f, l = 0.0f;
            for (int i = 0; i < len && !bad; i++) {
                long long slot = orc_resolve_slot(block_tables, b, (long long)start + i,
                                                  block_size, max_blocks_per_seq,
                                                  num_blocks_total, window_size_left);
                if (slot < 0) { bad = 1; break; }
                size_t sidx = (size_t)slot * kv_heads + kvh;
                float k_ds = k_scale_cache ? k_scale_cache[sidx] : *k_descale;
                float v_ds = v_scale_cache ? v_scale_cache[sidx] : *v_descale;
                const uint8_t *kr = k_cache + sidx * head_dim;
                const uint8_t *vr = v_cache + sidx * head_dim;
                float dot = 0.0f;
                for (int d = 0; d < head_dim; d++) dot += qv[d] * (g_lut[kr[d]] * k_ds);
                float qk = dot * scale;
                if (!isfinite(q_ds) || q_ds <= 0.0f || !isfinite(k_ds) || k_ds <= 0.0f ||
                    !isfinite(v_ds) || v_ds <= 0.0f || !isfinite(qk)) { bad = 1; break; }
                float m_new = fmaxf(m, qk);
                float e0 = expf(m - m_new), e1 = expf(qk - m_new);
                for (int d = 0; d < head_dim; d++)
                    acc[d] = acc[d] * e0 + e1 * (g_lut[vr[d]] * v_ds);
                l = l * e0 + e1;
                m = m_new;
            }
            for (int d = 0; d < head_dim; d++)
                o[d] = bad ? nan16 : orc_f2h(l > 0.0f ? acc[d] / l : acc[d], dtype);
            free(qv);
            free(acc);
        } else {
            double *s = (double *)malloc(sizeof(double) * (size_t)len);
            long long *slots = (long long *)malloc(sizeof(long long) * (size_t)len);
            double *acc = (double *)calloc(head_dim, sizeof(double));
            double mx = -INFINITY;
            for (int i = 0; i < len && !bad; i++) {
                long long slot = orc_resolve_slot(block_tables, b, (long long)start + i,
                                                  block_size, max_blocks_per_seq,
                                                  num_blocks_total, window_size_left);
                if (slot < 0) { bad = 1; break; }
                slots[i] = slot;
                size_t sidx = (size_t)slot * kv_heads + kvh;
                float k_ds = k_scale_cache ? k_scale_cache[sidx] : *k_descale;
                float v_ds = v_scale_cache ? v_scale_cache[sidx] : *v_descale;
                if (!isfinite(q_ds) || q_ds <= 0.0f || !isfinite(k_ds) || k_ds <= 0.0f ||
                    !isfinite(v_ds) || v_ds <= 0.0f) { bad = 1; break; }
                const uint8_t *kr = k_cache + sidx * head_dim;
                double dot = 0.0;
                for (int d = 0; d < head_dim; d++)
                    dot += (double)g_lut[qrow[d]] * (double)g_lut[kr[d]];
                s[i] = dot * (double)q_ds * (double)k_ds * (double)scale;
                if (!isfinite(s[i])) { bad = 1; break; }
                if (s[i] > mx) mx = s[i];
            }
            double lsum = 0.0;
            for (int i = 0; i < len && !bad; i++) {
                size_t sidx = (size_t)slots[i] * kv_heads + kvh;
                float v_ds = v_scale_cache ? v_scale_cache[sidx] : *v_descale;
                const uint8_t *vr = v_cache + sidx * head_dim;
                double p = exp(s[i] - mx);
                lsum += p;
                for (int d = 0; d < head_dim; d++)
                    acc[d] += p * (double)g_lut[vr[d]] * (double)v_ds;
            }
            for (int d = 0; d < head_dim; d++)
                o[d] = bad ? nan16 : orc_f2h((float)(lsum > 0.0 ? acc[d] / lsum : acc[d]), dtype);
            free(s);
            free(slots);
            free(acc);
        }
    }
    return 0;
}

/* Split-KV partials + log-sum-exp combine in the reference's order
 * (v3/kernels/fp8_decode_v2.cu:433-437,568-596,651-670): chunk_size =
 * ceil(attend_len / num_chunks), chunk c covers [start + c*chunk_size, ...),
 * partial (acc[HD], m, l) per chunk; combine walks chunks in order with
 * M = max(ma, mb), acc = acc_a*exp(ma-M) + acc_b*exp(mb-M).  Partials are returned
 * in `workspace` laid out [batch][heads][num_chunks][head_dim + 2] f32
 * (fp8_decode_v2.cu:26-31); untouched (empty) chunks keep m = -1e20, l = 0. */
int orc_paged_decode_fp8_split(uint16_t *out, float *workspace, const uint8_t *q,
                               const uint8_t *k_cache, const uint8_t *v_cache,
                               const int *block_tables, const int *context_lens,
                               const float *k_scale_cache, const float *v_scale_cache,
                               const float *q_scale_cache, float scale, int batch, int heads,
                               int kv_heads, int head_dim, int block_size,
                               int max_blocks_per_seq, int num_blocks_total,
                               int window_size_left, int num_chunks, int dtype) {
    if (num_chunks <= 0 || !k_scale_cache || !v_scale_cache || !q_scale_cache) return -1;
    lut_init();
    const int stride = head_dim + 2;
    for (int bh = 0; bh < batch * heads; bh++) {
        int b = bh / heads, h = bh % heads;
        int kvh = (int)((long long)h * kv_heads / heads);
        int ctx = context_lens[b];
        uint16_t *o = out + (size_t)bh * head_dim;
        float *ws = workspace + (size_t)bh * num_chunks * stride;
        for (int c = 0; c < num_chunks; c++) {
            for (int d = 0; d < head_dim; d++) ws[c * stride + d] = 0.0f;
            ws[c * stride + head_dim] = -1e20f;
            ws[c * stride + head_dim + 1] = 0.0f;
        }
        if (ctx <= 0) {
            for (int d = 0; d < head_dim; d++) o[d] = orc_f2h(0.0f, dtype);
            continue;
        }
        int start, len;
        attend_interval(ctx, window_size_left, &start, &len);
        int chunk = (len + num_chunks - 1) / num_chunks;
        float q_ds = q_scale_cache[(size_t)b * heads + h];
        for (int c = 0; c < num_chunks; c++) {
            int t0 = c * chunk, t1 = t0 + chunk < len ? t0 + chunk : len;
            float *acc = ws + c * stride;
            float m = -1e20f, l = 0.0f;
            for (int i = t0; i < t1; i++) {
                long long slot = orc_resolve_slot(block_tables, b, (long long)start + i,
                                                  block_size, max_blocks_per_seq,
                                                  num_blocks_total, window_size_left);
                if (slot < 0) return -2;
                size_t sidx = (size_t)slot * kv_heads + kvh;
                const uint8_t *kr = k_cache + sidx * head_dim;
                const uint8_t *vr = v_cache + sidx * head_dim;
                float dot = 0.0f;
                for (int d = 0; d < head_dim; d++)
                    dot = fmaf(g_lut[q[(size_t)bh * head_dim + d]] * q_ds, g_lut[kr[d]], dot);
                float qk = dot * (k_scale_cache[sidx] * scale);
                float m_new = fmaxf(m, qk);
                float e0 = expf(m - m_new), e1 = expf(qk - m_new);
                float ev = e1 * v_scale_cache[sidx];
                for (int d = 0; d < head_dim; d++) acc[d] = acc[d] * e0 + ev * g_lut[vr[d]];
                l = l * e0 + e1;
                m = m_new;
            }
            acc[head_dim] = m;
            acc[head_dim + 1] = l;
        }
        /* combine */
        float M = -1e20f, L = 0.0f;
        float *accum = (float *)calloc(head_dim, sizeof(float));
        for (int c = 0; c < num_chunks; c++) {
            if ((long long)c * chunk >= len) break;
            const float *p = ws + c * stride;
            float mb = p[head_dim], lb = p[head_dim + 1];
            float Mn = fmaxf(M, mb);
            float ea = expf(M - Mn), eb = expf(mb - Mn);
            for (int d = 0; d < head_dim; d++) accum[d] = accum[d] * ea + p[d] * eb;
            L = L * ea + lb * eb;
            M = Mn;
        }
        for (int d = 0; d < head_dim; d++)
            o[d] = orc_f2h(L > 0.0f ? accum[d] / L : accum[d], dtype);
        free(accum);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* stage 4: argmax                                                            */
/* ------------------------------------------------------------------------- */

/* mode 0: argmax_ref, v3/crates/rvllm-fused/src/reference.rs:200-225 (strict > scan
 *         from index 0; non-finite input is an error -> returns -1).
 * mode 1: argmax_kernel, kernels/argmax.cu:16-25,81-128 (NaN never wins, -inf may,
 *         ties -> lowest index, a row of only NaN -> -1). */
int orc_argmax_f32(const float *logits, int *out, int rows, int cols, int mode) {
    if (rows <= 0 || cols <= 0 || !logits || !out) return -1;
    for (int r = 0; r < rows; r++) {
        const float *row = logits + (size_t)r * cols;
        if (mode == 0) {
            int best = 0;
            for (int i = 0; i < cols; i++)
                if (!isfinite(row[i])) return -1;
            for (int i = 1; i < cols; i++)
                if (row[i] > row[best]) best = i;
            out[r] = best;
        } else {
            int best = -1;
            float bv = -INFINITY;
            for (int i = 0; i < cols; i++) {
                float v = row[i];
                if (v != v) continue;
                if (best < 0 || v > bv) { best = i; bv = v; }
            }
            out[r] = best;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* neighbours of the path: RoPE + KV-cache write, embedding gather             */
/* ------------------------------------------------------------------------- */

/* fused_rope_partial_fp8kv_kernel, v3/kernels/fused_rope_partial_fp8kv.cu:54-214:
 * half-split rotary pairing (lane i pairs with i + head_dim/2) over the first
 * rotary_dim/2 pairs, cos/sin tables [max_pos, rotary_dim/2] in the 16-bit type,
 * Q quantised per (token, head) with scale max(amax/448, 1e-12) into q_scale_cache,
 * K (post-RoPE) and V quantised per (slot, kv_head) into the paged caches
 * [slot, kv_head, head_dim] with scales at slot*kv_heads + head.  slot < 0 or
 * >= num_cache_slots skips the cache write.  CUDA encoder (mode 1). */
int orc_rope_fp8kv(const uint16_t *q_in, const uint16_t *k_in, const uint16_t *v_in,
                   int in_stride, uint8_t *q_fp8, uint8_t *k_cache, uint8_t *v_cache,
                   float *k_scale_cache, float *v_scale_cache, float *q_scale_cache,
                   const uint16_t *cos_t, const uint16_t *sin_t, const int *positions,
                   const int *slot_mapping, int num_tokens, int heads, int kv_heads,
                   int head_dim, int rotary_dim, int max_positions, int num_cache_slots,
                   int dtype) {
    if (num_tokens <= 0 || heads <= 0 || kv_heads < 0 || head_dim % 2 || rotary_dim % 2 ||
        rotary_dim > head_dim)
        return -1;
    int hh = head_dim / 2, hr = rotary_dim / 2;
    float *lo = (float *)malloc(sizeof(float) * hh), *hi = (float *)malloc(sizeof(float) * hh);
    for (int t = 0; t < num_tokens; t++) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_positions) continue;
        for (int pass = 0; pass < 2; pass++) {
            int nh = pass == 0 ? heads : kv_heads;
            const uint16_t *src = pass == 0 ? q_in : k_in;
            for (int h = 0; h < nh; h++) {
                const uint16_t *row = src + (size_t)t * in_stride + (size_t)h * head_dim;
                float amax = 0.0f;
                int invalid = 0; /* any non-finite post-RoPE value: NaN scale (fused_rope_partial_fp8kv.cu:133-137,178-198) */
                for (int i = 0; i < hh; i++) {
                    float a = orc_h2f(row[i], dtype), b = orc_h2f(row[i + hh], dtype);
                    if (i < hr) {
                        float c = orc_h2f(cos_t[(size_t)pos * hr + i], dtype);
                        float s = orc_h2f(sin_t[(size_t)pos * hr + i], dtype);
                        lo[i] = a * c - b * s;
                        hi[i] = a * s + b * c;
                    } else {
                        lo[i] = a;
                        hi[i] = b;
                    }
                    if (!isfinite(lo[i]) || !isfinite(hi[i])) invalid = 1;
                    else amax = fmaxf(amax, fmaxf(fabsf(lo[i]), fabsf(hi[i])));
                }
                float sc = invalid ? NAN : fmaxf(amax / FP8_MAX, 1e-12f), inv = 1.0f / sc;
                if (pass == 0) {
                    q_scale_cache[(size_t)t * heads + h] = sc;
                    uint8_t *o = q_fp8 + ((size_t)t * heads + h) * head_dim;
                    for (int i = 0; i < hh; i++) {
                        o[i] = orc_e4m3_encode(lo[i] * inv, 1);
                        o[i + hh] = orc_e4m3_encode(hi[i] * inv, 1);
                    }
                } else {
                    int slot = slot_mapping[t];
                    if (slot < 0 || slot >= num_cache_slots) continue;
                    size_t sidx = (size_t)slot * kv_heads + h;
                    k_scale_cache[sidx] = sc;
                    uint8_t *o = k_cache + sidx * head_dim;
                    for (int i = 0; i < hh; i++) {
                        o[i] = orc_e4m3_encode(lo[i] * inv, 1);
                        o[i + hh] = orc_e4m3_encode(hi[i] * inv, 1);
                    }
                    const uint16_t *vrow = v_in + (size_t)t * in_stride + (size_t)h * head_dim;
                    float vmax = 0.0f;
                    int vinvalid = 0; /* same rule for V (fused_rope_partial_fp8kv.cu:192-199) */
                    for (int i = 0; i < head_dim; i++) {
                        float x = orc_h2f(vrow[i], dtype);
                        if (!isfinite(x)) vinvalid = 1;
                        else vmax = fmaxf(vmax, fabsf(x));
                    }
                    float vs = vinvalid ? NAN : fmaxf(vmax / FP8_MAX, 1e-12f), vinv = 1.0f / vs;
                    v_scale_cache[sidx] = vs;
                    uint8_t *vo = v_cache + sidx * head_dim;
                    for (int i = 0; i < head_dim; i++)
                        vo[i] = orc_e4m3_encode(orc_h2f(vrow[i], dtype) * vinv, 1);
                }
            }
        }
    }
    free(lo);
    free(hi);
    return 0;
}

/* embedding_gather_ref, v3/crates/rvllm-fused/src/reference.rs:243-268 (16-bit rows) */
int orc_embedding_gather(uint16_t *out, const uint16_t *table, const int *token_ids,
                         int num_tokens, int hidden, int vocab) {
    for (int t = 0; t < num_tokens; t++) {
        int id = token_ids[t];
        if (id < 0 || id >= vocab) return -1;
        memcpy(out + (size_t)t * hidden, table + (size_t)id * hidden, (size_t)hidden * 2);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Gemma-4 decorations, soft cap, Llama-form RoPE                             */
/* ------------------------------------------------------------------------- */

/* fused_qkv_rmsnorm_kernel, v3/kernels/fused_qkv_rmsnorm.cu:28-130, for a launch of
 * block_dim threads: thread-strided sum of squares (:99-103, contracted to fma by the
 * device compiler), shuffle-down tree per warp (lane 0 holds the total; the pairing is
 * the xor butterfly's), the same tree over the warp totals, rsqrt(ss/head_dim + eps),
 * out = f16(x * rms [* gamma]) (:124-128).  qkv: packed rows [tokens][src_row_stride];
 * outputs compact [tokens][heads][head_dim].  1/sqrtf stands in for the device rsqrtf. */
int orc_qkv_rmsnorm(uint16_t *q_out, uint16_t *k_out, uint16_t *v_out, const uint16_t *qkv,
                    const uint16_t *q_gamma, const uint16_t *k_gamma, int num_tokens,
                    int num_heads, int num_kv_heads, int head_dim, float eps,
                    int src_row_stride, int dtype, int block_dim) {
    if (num_tokens <= 0 || num_heads <= 0 || num_kv_heads < 0 || head_dim <= 0 || !qkv || !q_out) return -1;
    if (block_dim < 32 || block_dim > 1024 || block_dim % 32) return -1;
    if (!(eps > 0.0f) || !isfinite(eps)) return -1;
    int total = num_heads + 2 * num_kv_heads;
    if ((long long)src_row_stride < (long long)total * head_dim) return -1;
    float partial[1024];
    for (int t = 0; t < num_tokens; t++)
        for (int hg = 0; hg < total; hg++) {
            const uint16_t *gamma = NULL;
            uint16_t *dst;
            long long src_off;
            if (hg < num_heads) {
                gamma = q_gamma;
                src_off = (long long)hg * head_dim;
                dst = q_out + ((size_t)t * num_heads + hg) * head_dim;
            } else if (hg < num_heads + num_kv_heads) {
                int hl = hg - num_heads;
                gamma = k_gamma;
                src_off = (long long)(num_heads + hl) * head_dim;
                dst = k_out + ((size_t)t * num_kv_heads + hl) * head_dim;
            } else {
                int hl = hg - num_heads - num_kv_heads;
                src_off = (long long)(num_heads + num_kv_heads + hl) * head_dim;
                dst = v_out + ((size_t)t * num_kv_heads + hl) * head_dim;
            }
            const uint16_t *src = qkv + (size_t)t * src_row_stride + src_off;
            for (int i = 0; i < block_dim; i++) partial[i] = 0.0f;
            for (int i = 0; i < head_dim; i++) {
                float a = orc_h2f(src[i], dtype);
                partial[i % block_dim] = fmaf(a, a, partial[i % block_dim]);
            }
            float ss = block_sum_ref_order(partial, block_dim);
            float rms = 1.0f / sqrtf(ss / (float)head_dim + eps);
            for (int i = 0; i < head_dim; i++) {
                float v = orc_h2f(src[i], dtype) * rms;
                if (gamma) v *= orc_h2f(gamma[i], dtype);
                dst[i] = orc_f2h(v, dtype);
            }
        }
    return 0;
}

/* fused_norm_add_residual_f16_kernel / _f16in_kernel,
 * v3/kernels/fused_norm_add_residual_f16.cu:8-58,67-116: x = gemm_out * channelscale
 * (f32 input) or the 16-bit GEMM output; thread-strided sum of squares, xor butterfly
 * per warp, warp totals added in warp order by thread 0 (:45-50); residual =
 * f16((residual + x * rms * gamma) * layer_scalar).  The device compiler contracts
 * residual + (x*rms)*gamma into one fma. */
int orc_norm_add_residual(uint16_t *residual, const float *gemm_f32, const uint16_t *gemm_16,
                          const float *channelscale, const uint16_t *gamma,
                          const uint16_t *layer_scalar, int num_tokens, int hidden, float eps,
                          int dtype, int block_dim) {
    if (num_tokens <= 0 || hidden <= 0 || !residual || !gamma || (!gemm_f32 && !gemm_16)) return -1;
    if (gemm_f32 && !channelscale) return -1;
    if (block_dim < 32 || block_dim > 1024 || block_dim % 32) return -1;
    if (!(eps > 0.0f) || !isfinite(eps)) return -1;
    float partial[1024];
    float *x = (float *)malloc(sizeof(float) * (size_t)hidden);
    float ls = layer_scalar ? orc_h2f(layer_scalar[0], dtype) : 1.0f;
    for (int t = 0; t < num_tokens; t++) {
        for (int i = 0; i < block_dim; i++) partial[i] = 0.0f;
        for (int i = 0; i < hidden; i++) {
            float a = gemm_f32 ? gemm_f32[(size_t)t * hidden + i] * channelscale[i]
                               : orc_h2f(gemm_16[(size_t)t * hidden + i], dtype);
            x[i] = a;
            partial[i % block_dim] = fmaf(a, a, partial[i % block_dim]);
        }
        int nw = (block_dim + 31) / 32;
        float total = 0.0f;
        for (int w = 0; w < nw; w++) {
            float v[32];
            for (int l = 0; l < 32; l++) v[l] = partial[w * 32 + l];
            for (int off = 16; off > 0; off >>= 1) {
                float nv[32];
                for (int l = 0; l < 32; l++) nv[l] = v[l] + v[l ^ off];
                memcpy(v, nv, sizeof v);
            }
            total += v[0];
        }
        float rms = 1.0f / sqrtf(total / (float)hidden + eps);
        uint16_t *res = residual + (size_t)t * hidden;
        for (int i = 0; i < hidden; i++) {
            float r = fmaf(x[i] * rms, orc_h2f(gamma[i], dtype), orc_h2f(res[i], dtype));
            res[i] = orc_f2h(r * ls, dtype);
        }
    }
    free(x);
    return 0;
}

/* residual_scale_f16_kernel, v3/kernels/residual_scale_f16.cu:13-27. */
int orc_residual_scale(uint16_t *residual, const uint16_t *scalar, size_t n, int dtype) {
    if (!residual || !scalar) return -1;
    float s = orc_h2f(scalar[0], dtype);
    for (size_t i = 0; i < n; i++) residual[i] = orc_f2h(orc_h2f(residual[i], dtype) * s, dtype);
    return 0;
}

/* logit_softcap_kernel, v3/kernels/logit_softcap.cu:12-31: cap * tanhf(x * (1/cap)). */
int orc_logit_softcap(uint16_t *logits, size_t n, float cap, int dtype) {
    if (!logits || !(cap > 0.0f) || !isfinite(cap)) return -1;
    float inv = 1.0f / cap;
    for (size_t i = 0; i < n; i++) logits[i] = orc_f2h(cap * tanhf(orc_h2f(logits[i], dtype) * inv), dtype);
    return 0;
}

/* fused_rope_cache_fp8kv_kernel, v3/kernels/fused_rope_cache_fp8kv.cu:20-101:
 * interleaved pairs (2t, 2t+1) over the whole head, cos/sin [max_positions][head_dim/2],
 * static scales; q' = (q0*c - q1*s, q0*s + q1*c) * (1/q_scale) (the device compiler
 * contracts a*b - c*d into fma(a, b, -(c*d)) and a*b + c*d into fma(a, b, c*d)); K
 * rotated and V unrotated into the paged cache times 1/kv_scale.  A bad position or
 * scale writes nothing; a slot outside the cache skips the cache write. */
int orc_rope_cache_fp8kv(const uint16_t *q_in, const uint16_t *k_in, const uint16_t *v_in,
                         long long q_stride, long long kv_stride, uint8_t *q_fp8, uint8_t *k_cache,
                         uint8_t *v_cache, const uint16_t *cos_t, const uint16_t *sin_t,
                         const int *positions, const int *slot_mapping, float q_scale,
                         float kv_scale, int num_tokens, int heads, int kv_heads, int head_dim,
                         int max_positions, int num_cache_slots, int dtype) {
    if (!q_in || !q_fp8 || !positions || num_tokens <= 0 || heads <= 0 || kv_heads < 0 ||
        head_dim <= 0 || head_dim % 2 || max_positions <= 0 || !cos_t || !sin_t) return -1;
    if (!isfinite(q_scale) || q_scale <= 0.0f) return 0;
    if (kv_heads > 0 && (!isfinite(kv_scale) || kv_scale <= 0.0f)) return 0;
    float q_inv = 1.0f / q_scale, kv_inv = kv_heads > 0 ? 1.0f / kv_scale : 0.0f;
    int half = head_dim / 2;
    for (int t = 0; t < num_tokens; t++) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_positions) continue;
        for (int p = 0; p < half; p++) {
            float c = orc_h2f(cos_t[(size_t)pos * half + p], dtype);
            float s = orc_h2f(sin_t[(size_t)pos * half + p], dtype);
            for (int h = 0; h < heads; h++) {
                const uint16_t *src = q_in + (size_t)t * q_stride + (size_t)h * head_dim + 2 * p;
                float a = orc_h2f(src[0], dtype), b = orc_h2f(src[1], dtype);
                uint8_t *o = q_fp8 + ((size_t)t * heads + h) * head_dim + 2 * p;
                o[0] = orc_e4m3_encode(fmaf(a, c, -(b * s)) * q_inv, 1);
                o[1] = orc_e4m3_encode(fmaf(a, s, b * c) * q_inv, 1);
            }
            int slot = kv_heads > 0 ? slot_mapping[t] : -1;
            if (slot < 0 || slot >= num_cache_slots) continue;
            for (int h = 0; h < kv_heads; h++) {
                size_t in_off = (size_t)t * kv_stride + (size_t)h * head_dim + 2 * p;
                float a = orc_h2f(k_in[in_off], dtype), b = orc_h2f(k_in[in_off + 1], dtype);
                size_t off = ((size_t)slot * kv_heads + h) * head_dim + 2 * p;
                k_cache[off] = orc_e4m3_encode(fmaf(a, c, -(b * s)) * kv_inv, 1);
                k_cache[off + 1] = orc_e4m3_encode(fmaf(a, s, b * c) * kv_inv, 1);
                v_cache[off] = orc_e4m3_encode(orc_h2f(v_in[in_off], dtype) * kv_inv, 1);
                v_cache[off + 1] = orc_e4m3_encode(orc_h2f(v_in[in_off + 1], dtype) * kv_inv, 1);
            }
        }
    }
    return 0;
}

/* fp8_gemv_blockwise_wpr_native_f16in_kernel, kernels/fp8_gemv.cu:811-891: out[m, n] =
 * f16(sum_k dec(W[n,k]) * scale[n/128][k/128] * x[m,k]) with the kernel's order: lane l of the
 * row's warp takes k = 8l + 256i, two accumulation chains (first four / last four of the
 * eight, each term (w*s)*x folded into the chain with one fma), chains added, shuffle-down
 * tree (lane 0's pairing is the xor butterfly's).  K a multiple of 8. */
int orc_fp8_gemv_blockscale(uint16_t *out, const uint8_t *w, const float *scale, const uint16_t *x,
                            int M, int N, int K, int dtype) {
    if (M <= 0 || N <= 0 || K <= 0 || (K & 7) || !out || !w || !scale || !x) return -1;
    lut_init();
    int ncb = (K + 127) / 128;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const float *srow = scale + (size_t)(n >> 7) * ncb;
        const uint8_t *wr = w + (size_t)n * K;
        for (int m = 0; m < M; m++) {
            const uint16_t *xr = x + (size_t)m * K;
            float lane_acc[32];
            for (int l = 0; l < 32; l++) {
                float a0 = 0.0f, a1 = 0.0f;
                for (int k = l * 8; k + 7 < K; k += 256) {
                    float s0 = srow[k >> 7], s4 = srow[(k + 4) >> 7];
                    for (int e = 0; e < 4; e++) a0 = fmaf(orc_e4m3_decode(wr[k + e]) * s0, orc_h2f(xr[k + e], dtype), a0);
                    for (int e = 4; e < 8; e++) a1 = fmaf(orc_e4m3_decode(wr[k + e]) * s4, orc_h2f(xr[k + e], dtype), a1);
                }
                lane_acc[l] = a0 + a1;
            }
            for (int off = 16; off > 0; off >>= 1)
                for (int l = 0; l + off < 32; l++)
                    if (l < off) lane_acc[l] = lane_acc[l] + lane_acc[l + off];
            out[(size_t)m * N + n] = orc_f2h(lane_acc[0], dtype);
        }
    }
    return 0;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Worker threads of the parallel loops from now on (a launcher may have exported OMP_NUM_THREADS=1). */
void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
