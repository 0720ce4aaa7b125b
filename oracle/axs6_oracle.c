/*
 * CPU oracle for the AXS-6 hot path (TEST INFRASTRUCTURE, never the product).
 *
 * A plain-C restatement of the reference's eager PyTorch algorithm, one scalar
 * loop per block, written for clarity.  Only the test-suite, the smoke check and
 * the CPU-baseline leg of the benchmark may call it; the CUDA library never does.
 * Parity is PINNED: tests/golden/ holds inputs and outputs produced by importing
 * the reference itself (generator: tests/golden/make_golden.py) and
 * tests/test_oracle_golden.py checks every function below against them.
 *
 * Each function names the reference file:line it follows (paths are relative to
 * the reference project root).
 *
 * Conventions: x is row-major (rows, cols) fp32; the last dim is cut into blocks
 * of B in {8,16,32} and zero-padded to nblk*B.  Planes are (rows, nblk, B).
 * `noise` (optional) holds U[0,1) draws in the padded (rows, nblk, B) layout and
 * switches the rounding to the reference's stochastic variant.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef int64_t i64;

/* Threads the parallel loops below use: n > 0 sets the count (a launcher may have exported
 * OMP_NUM_THREADS=1), the return value is the count in effect.  Used by the timed CPU baseline,
 * which states the number of cores it ran on. */
int orc_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* floor(log2(a)) as torch's fp32 CPU log2 returns it: the fp32 result of log2
 * behaves as the correctly rounded value, so an amax a few ulps below a power of
 * two rounds UP to the integer.  Restated as: round the double-precision log2 to
 * fp32, then floor.  (axs/unified/quantize_unified.py:173-175, :248-249;
 * axs/core.py:333-334; axs/unified/distributed.py:101-102) */
static int floor_log2_as_reference(float a)
{
    float l = (float)log2((double)a);
    return (int)floorf(l);
}

int orc_floor_log2(float a) { return floor_log2_as_reference(a); }

static float clamp_min_denorm(float a)
{
    /* tensor.clamp(min=1e-45): 1e-45 is the smallest fp32 denormal, 2^-149 */
    const float tiny = 1.401298464324817e-45f;
    return a < tiny ? tiny : a;
}

static float block_amax(const float *x, i64 n_valid, int B)
{
    float a = 0.0f;
    for (int i = 0; i < B; ++i) {
        float v = (i < n_valid) ? fabsf(x[i]) : 0.0f;
        if (v > a) a = v;
    }
    return a;
}

/* axs/unified/quantize_unified.py:121-204 (fused_fake_quantize).  y is (rows, cols),
 * fp32; casting to the input dtype is done by the caller. */
void orc_fq_nf5(const float *x, float *y, i64 rows, i64 cols, i64 ldx, i64 ldy, int B,
                const float *lut1024, const float *noise)
{
    i64 nblk = (cols + B - 1) / B;
#pragma omp parallel for schedule(static)
    for (i64 r = 0; r < rows; ++r) {
        for (i64 b = 0; b < nblk; ++b) {
            const float *xb = x + r * ldx + b * B;
            float *yb = y + r * ldy + b * B;
            i64 n_valid = cols - b * B; if (n_valid > B) n_valid = B;
            float amax = block_amax(xb, n_valid, B);                        /* :173 */
            float scale = exp2f((float)floor_log2_as_reference(clamp_min_denorm(amax)) + 1.0f); /* :174-175 */
            if (amax == 0.0f) scale = 1.0f;                                  /* :178-179 */
            for (i64 i = 0; i < n_valid; ++i) {
                float v = xb[i];
                float sgn = (v > 0.0f) ? 1.0f : ((v < 0.0f) ? -1.0f : 0.0f); /* :169 */
                float nrm = fabsf(v) / scale;                                /* :182 */
                if (nrm < 0.0f) nrm = 0.0f;
                if (nrm > 1.0f) nrm = 1.0f;
                int idx;
                if (noise) {                                                 /* :186-189 */
                    float u = noise[(r * nblk + b) * B + i];
                    float dither = (u - 0.5f) / 1023.0f;
                    float t = (nrm + dither) * 1023.0f;
                    idx = (int)t;
                } else {
                    float t = nrm * 1023.0f;                                 /* :191 */
                    idx = (int)t;
                }
                if (idx < 0) idx = 0;
                if (idx > 1023) idx = 1023;
                float rec = lut1024[idx];                                    /* :194 */
                yb[i] = (sgn * rec) * scale;                                 /* :197 */
            }
        }
    }
}

/* grid 1: axs/unified/quantize_unified.py:211-282 (quantize_unified), identical codes to
 *         axs/unified/distributed.py:70-120 (_pack_gradient);
 * grid 0: axs/core.py:294-369 (quantize, uniform grid). */
void orc_quantize(const float *x, i64 rows, i64 cols, i64 ldx, int B, int grid,
                  const uint8_t *rev1024, const float *noise,
                  uint8_t *se_out, uint8_t *sign_out, uint8_t *mag_out)
{
    i64 nblk = (cols + B - 1) / B;
#pragma omp parallel for schedule(static)
    for (i64 r = 0; r < rows; ++r) {
        for (i64 b = 0; b < nblk; ++b) {
            const float *xb = x + r * ldx + b * B;
            i64 n_valid = cols - b * B; if (n_valid > B) n_valid = B;
            float amax = block_amax(xb, n_valid, B);
            int raw = floor_log2_as_reference(clamp_min_denorm(amax)) + 1;   /* q_u:248-249, core:333-334 */
            int se = raw + 127;
            if (se < 0) se = 0;
            if (se > 255) se = 255;                                          /* q_u:250, core:335 */
            if (amax == 0.0f) se = 0;                                        /* q_u:251, core:338-339 */
            float scale = (grid == 1) ? exp2f((float)se - 127.0f)            /* q_u:253-255 */
                                      : powf(2.0f, (float)se - 127.0f);      /* core:342-347 */
            scale = clamp_min_denorm(scale);
            se_out[r * nblk + b] = (uint8_t)se;
            for (int i = 0; i < B; ++i) {
                float v = (i < n_valid) ? xb[i] : 0.0f;
                float nrm = fabsf(v) / scale;
                int mag;
                i64 o = (r * nblk + b) * B + i;
                if (grid == 1) {
                    if (nrm < 0.0f) nrm = 0.0f;
                    if (nrm > 1.0f) nrm = 1.0f;                              /* q_u:257 */
                    float t = noise ? (nrm + (noise[o] - 0.5f) / 1023.0f) * 1023.0f  /* q_u:263-265 */
                                    : nrm * 1023.0f;                         /* q_u:261 */
                    int idx = (int)t;
                    if (idx < 0) idx = 0;
                    if (idx > 1023) idx = 1023;
                    mag = rev1024[idx];                                      /* q_u:270-271 */
                } else {
                    float scaled = nrm * 31.0f;                              /* core:348-349 */
                    float m;
                    if (noise) {                                             /* core:351-355 */
                        float fl = floorf(scaled);
                        float frac = scaled - fl;
                        m = (noise[o] < frac) ? fl + 1.0f : fl;
                    } else {
                        m = nearbyintf(scaled);                              /* core:357, round-half-even */
                    }
                    if (m < 0.0f) m = 0.0f;
                    if (m > 31.0f) m = 31.0f;                                /* core:359 */
                    mag = (int)m;
                }
                mag_out[o] = (uint8_t)mag;
                sign_out[o] = (uint8_t)(v < 0.0f);                           /* q_u:273, core:360 */
            }
        }
    }
}

/* grid 1: axs/unified/quantize_unified.py:285-308 (dequantize_unified);
 * grid 0: axs/core.py:372-403 (dequantize).  y is (rows, cols) fp32. */
void orc_dequantize(const uint8_t *se, const uint8_t *sign, const uint8_t *mag,
                    i64 rows, i64 cols, i64 ldy, int B, int grid,
                    const float *codebook32, float *y)
{
    i64 nblk = (cols + B - 1) / B;
#pragma omp parallel for schedule(static)
    for (i64 r = 0; r < rows; ++r) {
        for (i64 b = 0; b < nblk; ++b) {
            float e = (float)se[r * nblk + b] - 127.0f;
            float scale = (grid == 1) ? exp2f(e) : powf(2.0f, e);           /* q_u:296-298, core:383-385 */
            i64 n_valid = cols - b * B; if (n_valid > B) n_valid = B;
            for (i64 i = 0; i < n_valid; ++i) {
                i64 o = (r * nblk + b) * B + i;
                float v = (grid == 1) ? codebook32[mag[o]] * scale          /* q_u:300-301 */
                                      : ((float)mag[o] / 31.0f) * scale;    /* core:388 */
                y[r * ldy + b * B + i] = sign[o] ? -v : v;                  /* q_u:302, core:389 */
            }
        }
    }
}

/* Payload shared by both byte layouts: the 6-bit codes (sign<<5)|mag of one block as a
 * little-endian bit stream (axs/core.py:103-116; axs/unified/distributed.py:165-189). */
static void pack_payload(const uint8_t *sign, const uint8_t *mag, int B, uint8_t *out)
{
    uint32_t acc = 0; int nb = 0; int o = 0;
    for (int i = 0; i < B; ++i) {
        uint32_t code = ((uint32_t)(sign[i] & 1) << 5) | (mag[i] & 31u);
        acc |= code << nb; nb += 6;
        while (nb >= 8) { out[o++] = (uint8_t)(acc & 0xFF); acc >>= 8; nb -= 8; }
    }
    if (nb > 0) out[o++] = (uint8_t)(acc & 0xFF);
}

static void unpack_payload(const uint8_t *in, int B, uint8_t *sign, uint8_t *mag)
{
    uint32_t acc = 0; int nb = 0; int p = 0;
    for (int i = 0; i < B; ++i) {
        while (nb < 6) { acc |= (uint32_t)in[p++] << nb; nb += 8; }
        uint32_t code = acc & 0x3F; acc >>= 6; nb -= 6;
        sign[i] = (uint8_t)((code >> 5) & 1);
        mag[i] = (uint8_t)(code & 31u);
    }
}

/* layout 1 ("wire", 1 + 3B/4 bytes per block): axs/unified/distributed.py:147-198
 * layout 2 ("spec", 2 + 3B/4 bytes per block, header = u16 LE (se<<2)|config, config 0):
 *          axs/core.py:97-118 and FORMAT_SPEC.md:29-48 */
void orc_pack_bytes(const uint8_t *se, const uint8_t *sign, const uint8_t *mag,
                    i64 nblocks, int B, int layout, uint8_t *out)
{
    int pay = B * 6 / 8, hdr = (layout == 2) ? 2 : 1, rec = hdr + pay;
#pragma omp parallel for schedule(static)
    for (i64 b = 0; b < nblocks; ++b) {
        uint8_t *o = out + b * rec;
        if (layout == 2) {
            uint32_t h = ((uint32_t)se[b] << 2) | 0u;
            o[0] = (uint8_t)(h & 0xFF); o[1] = (uint8_t)(h >> 8);
        } else {
            o[0] = se[b];
        }
        pack_payload(sign + b * B, mag + b * B, B, o + hdr);
    }
}

/* axs/unified/distributed.py:201-232 (_unpack_from_flat_buffer); axs/core.py:120-152 (from_bytes) */
void orc_unpack_bytes(const uint8_t *in, i64 nblocks, int B, int layout,
                      uint8_t *se, uint8_t *sign, uint8_t *mag)
{
    int pay = B * 6 / 8, hdr = (layout == 2) ? 2 : 1, rec = hdr + pay;
#pragma omp parallel for schedule(static)
    for (i64 b = 0; b < nblocks; ++b) {
        const uint8_t *p = in + b * rec;
        if (layout == 2) {
            uint32_t h = (uint32_t)p[0] | ((uint32_t)p[1] << 8);
            se[b] = (uint8_t)(h >> 2);
        } else {
            se[b] = p[0];
        }
        unpack_payload(p + hdr, B, sign + b * B, mag + b * B);
    }
}

/* fp32 <-> bf16 (round to nearest even), as torch's .to(torch.bfloat16) / .float() */
void orc_bf16_to_f32(const uint16_t *in, float *out, i64 n)
{
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; ++i) { uint32_t u = (uint32_t)in[i] << 16; memcpy(&out[i], &u, 4); }
}

void orc_f32_to_bf16(const float *in, uint16_t *out, i64 n)
{
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; ++i) {
        uint32_t u; memcpy(&u, &in[i], 4);
        if ((u & 0x7FFFFFFFu) > 0x7F800000u) { out[i] = (uint16_t)((u >> 16) | 0x40); continue; }
        uint32_t lsb = (u >> 16) & 1u;
        u += 0x7FFFu + lsb;
        out[i] = (uint16_t)(u >> 16);
    }
}

/* C[M,N] = A[M,K] * B[N,K]^T in fp32 with fp64 accumulation: the "fp32 matmul of the
 * dequantised operands" that the GEMM tolerance is stated against. */
void orc_gemm_nt(const float *A, const float *Bm, float *C, i64 M, i64 N, i64 K)
{
#pragma omp parallel for schedule(static)
    for (i64 m = 0; m < M; ++m)
        for (i64 n = 0; n < N; ++n) {
            double acc = 0.0;
            const float *a = A + m * K, *b = Bm + n * K;
            for (i64 k = 0; k < K; ++k) acc += (double)a[k] * (double)b[k];
            C[m * N + n] = (float)acc;
        }
}

/* Scan every positive finite fp32 value and report those whose floor(log2) above differs
 * from the true unbiased exponent (the "bumped" inputs).  Writes up to cap bit patterns,
 * returns the count.  Used once by the oracle's own test against the set recorded from
 * torch (tests/golden/log2_bump_set.npy). */
i64 orc_log2_bump_scan(uint32_t *out, i64 cap)
{
    i64 n = 0;
#pragma omp parallel for schedule(static)
    for (i64 b = 1; b < 0x7F800000LL; ++b) {
        uint32_t u = (uint32_t)b; float a; memcpy(&a, &u, 4);
        uint32_t ef = u >> 23, m = u & 0x7FFFFFu;
        int e_true = ef ? (int)ef - 127 : (31 - __builtin_clz(m)) - 149;
        if (floor_log2_as_reference(a) != e_true) {
#pragma omp critical
            { if (n < cap) out[n] = u; ++n; }
        }
    }
    return n;
}
