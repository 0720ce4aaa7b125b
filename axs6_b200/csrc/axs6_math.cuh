// Per-block and per-element arithmetic of the AXS-6 quantisers, shared by every kernel.
//
// All functions are plain scalar code that also compiles for the host (for unit checks of
// the arithmetic without a GPU); on the device each floating-point step uses the
// round-to-nearest intrinsics so that nothing is contracted into an FMA and denormals are
// kept.  The steps and their order follow the reference's eager PyTorch code:
//   NF5 fake-quantise   axs/unified/quantize_unified.py:168-197
//   NF5 codes           axs/unified/quantize_unified.py:244-273
//   uniform codes       axs/core.py:329-360
//   decode              axs/unified/quantize_unified.py:295-302, axs/core.py:383-389
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define AXS6_HD __host__ __device__ __forceinline__
#else
#define AXS6_HD inline
#include <math.h>
#endif

#if defined(__CUDA_ARCH__)
#define AXS6_MUL(a, b) __fmul_rn((a), (b))
#define AXS6_ADD(a, b) __fadd_rn((a), (b))
#define AXS6_SUB(a, b) __fsub_rn((a), (b))
#define AXS6_DIV(a, b) __fdiv_rn((a), (b))
#define AXS6_TRUNC_I(a) __float2int_rz(a)
#define AXS6_RINT(a) rintf(a)
#define AXS6_FLOOR(a) floorf(a)
#else
#define AXS6_MUL(a, b) ((a) * (b))
#define AXS6_ADD(a, b) ((a) + (b))
#define AXS6_SUB(a, b) ((a) - (b))
#define AXS6_DIV(a, b) ((a) / (b))
#define AXS6_TRUNC_I(a) ((int)(a))
#define AXS6_RINT(a) nearbyintf(a)
#define AXS6_FLOOR(a) floorf(a)
#endif

AXS6_HD float axs6_from_bits(uint32_t u)
{
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}

AXS6_HD uint32_t axs6_to_bits(float f)
{
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}

AXS6_HD int axs6_clz(uint32_t v)
{
#if defined(__CUDA_ARCH__)
    return __clz((int)v);
#else
    return v ? __builtin_clz(v) : 32;
#endif
}

// floor(log2(a)) exactly as the reference's fp32 `a.log2().floor()` returns it on the CPU
// (quantize_unified.py:175, :249; core.py:334).  That log2 behaves as the correctly rounded
// fp32 logarithm, so when a lies within a few ulps below a power of two 2^k the logarithm
// rounds up to the integer k and the floor is one more than the true exponent.  With
// a = 2^k (1 - D / 2^(t+1)) (t = position of a's leading mantissa bit, D = distance to the
// power of two in units of a's last place), log2(a) ~ k - D * log2(e) / 2^(t+1) rounds to k
// iff that offset is below half an ulp of the fp32 numbers next to k, which have exponent
// J = floor(log2(k - 1)) for k >= 2 and floor(log2(-k)) for k <= -1:
//     D <= floor(2^(J + t - 23) / log2(e))      -> thresholds {0,1,2,5,11,22,44,88}.
// Checked against torch for all 2^31 positive floats (tests/golden/log2_bump_set.npy).
// `abits`: bit pattern of a positive, non-zero, finite float.
AXS6_HD int axs6_ref_floor_log2(uint32_t abits)
{
    const uint32_t ef = abits >> 23;
    const uint32_t mant = abits & 0x7FFFFFu;
    int e, t;
    uint32_t dist;
    if (ef != 0) {
        e = (int)ef - 127;
        dist = 0x800000u - mant;
        if (dist > 44u) return e;            // common case: one compare
        t = 23;
    } else {
        t = 31 - axs6_clz(mant);
        e = t - 149;
        dist = (2u << t) - mant;
        if (dist > 88u) return e;
    }
    const int k = e + 1;
    int j;
    if (k >= 2) j = 31 - axs6_clz((uint32_t)(k - 1));
    else if (k <= -1) j = 31 - axs6_clz((uint32_t)(-k));
    else return e;
    const int s = j + t - 23;
    if (s < 0) return e;
    // floor(2^s / log2(e)) for s = 0..7, one byte each
    const uint64_t thr = 0x582C160B05020100ull;
    const uint32_t lim = (uint32_t)((thr >> (8 * s)) & 0xFFu);
    return e + (dist <= lim ? 1 : 0);
}

// 2^k as fp32 for k in [-149, 128]: denormal below -126, +inf at 128.
AXS6_HD float axs6_pow2(int k)
{
    if (k >= -126) return (k <= 127) ? axs6_from_bits((uint32_t)(k + 127) << 23) : axs6_from_bits(0x7F800000u);
    return (k >= -149) ? axs6_from_bits(1u << (k + 149)) : 0.0f;
}

struct Axs6Scale {
    float scale;  // block scale S = 2^k
    float inv;    // 1/S when `fast`, else unused
    int fast;     // k in [-116, 126]: S, 1/S, 1023/S and 31/S are all normal fp32 numbers
    int se;       // biased shared exponent byte (code paths)
};

// Why the fast path may fold the two roundings of trunc(RN(RN(|x| / S) * G)) (G = 1023 or 31)
// into ONE product RN(|x| * (G / S)): G / S is exact in fp32 (G has at most 10 significant bits,
// S is a power of two).  If |x| / S is representable the first rounding is the identity and both
// expressions round the same real number.  If it is not, |x| / S < 2^-126, so both products are
// below 2^-116 and truncate (or round) to index 0 alike.

// Scale of the fused fake-quantise: S = exp2(floor(log2(max(amax, 2^-149))) + 1), S = 1 for an
// all-zero block; no clamping of the exponent (quantize_unified.py:173-179).
AXS6_HD Axs6Scale axs6_scale_fq(uint32_t amax_bits)
{
    Axs6Scale s;
    s.se = 0;
    if (amax_bits == 0u) { s.scale = 1.0f; s.inv = 1.0f; s.fast = 1; return s; }
    const int k = axs6_ref_floor_log2(amax_bits) + 1;
    if (k >= -116 && k <= 126) {
        s.scale = axs6_from_bits((uint32_t)(k + 127) << 23);
        s.inv = axs6_from_bits((uint32_t)(127 - k) << 23);
        s.fast = 1;
    } else {
        s.scale = axs6_pow2(k);
        s.inv = 0.0f;
        s.fast = 0;
    }
    return s;
}

// Scale of the code paths: se = clamp(floor(log2(amax)) + 1 + 127, 0, 255), 0 for an all-zero
// block, S = 2^(se - 127) (quantize_unified.py:248-255, core.py:333-347).
AXS6_HD Axs6Scale axs6_scale_codes(uint32_t amax_bits)
{
    Axs6Scale s;
    if (amax_bits == 0u) {      // every code of the block is 0 whatever the scale
        s.se = 0; s.scale = axs6_pow2(-127); s.inv = 1.0f; s.fast = 1;
        return s;
    }
    int se = axs6_ref_floor_log2(amax_bits) + 1 + 127;
    se = se < 0 ? 0 : (se > 255 ? 255 : se);
    s.se = se;
    if (se >= 11 && se <= 253) {
        s.scale = axs6_from_bits((uint32_t)se << 23);
        s.inv = axs6_from_bits((uint32_t)(254 - se) << 23);
        s.fast = 1;
    } else {
        s.scale = axs6_pow2(se - 127);
        s.inv = 0.0f;
        s.fast = 0;
    }
    return s;
}

// Scale for decoding: 2^(se - 127) for any byte value.
AXS6_HD float axs6_scale_decode(uint32_t se) { return axs6_pow2((int)se - 127); }

// |x| / S, clamped to [0, 1].
AXS6_HD float axs6_normalise(float ax, const Axs6Scale &s)
{
    if (s.fast) return AXS6_MUL(ax, s.inv);   // exact power-of-two scaling, always <= 1
    float n = AXS6_DIV(ax, s.scale);
    n = n < 0.0f ? 0.0f : n;
    return n > 1.0f ? 1.0f : n;
}

// LUT index of a normalised magnitude: trunc(n * 1023), or with dither
// trunc((n + (u - 0.5) / 1023) * 1023), clamped to [0, 1023] (quantize_unified.py:186-191).
AXS6_HD int axs6_nf5_index(float n)
{
    int i = AXS6_TRUNC_I(AXS6_MUL(n, 1023.0f));
    i = i < 0 ? 0 : i;
    return i > 1023 ? 1023 : i;
}

AXS6_HD int axs6_nf5_index_dithered(float n, float u)
{
    const float d = AXS6_DIV(AXS6_SUB(u, 0.5f), 1023.0f);
    int i = AXS6_TRUNC_I(AXS6_MUL(AXS6_ADD(n, d), 1023.0f));
    i = i < 0 ? 0 : i;
    return i > 1023 ? 1023 : i;
}

// Fast-path forms (block scale in the `fast` range, see Axs6Scale): one product, no clamps --
// |x| < S guarantees an index below 1023 and a magnitude of at most 31.
AXS6_HD int axs6_nf5_index_fast(float ax, float g_over_s) { return AXS6_TRUNC_I(AXS6_MUL(ax, g_over_s)); }
#if defined(__CUDA_ARCH__)
AXS6_HD int axs6_uniform_mag_fast(float ax, float g_over_s) { return __float2int_rn(AXS6_MUL(ax, g_over_s)); }
#else
AXS6_HD int axs6_uniform_mag_fast(float ax, float g_over_s) { return (int)nearbyintf(AXS6_MUL(ax, g_over_s)); }
#endif

// Dithered index for draws that come from the library's own generator (no bit-level
// counterpart in the reference, whose draws come from torch's generator): the same dither of
// +-0.5 LUT steps, evaluated as ONE fused multiply-add trunc(|x| * (1023 / S) + (u - 0.5)).  The
// sum lies in (-0.5, 1023.5), so truncation already lands in [0, 1023].
#if defined(__CUDA_ARCH__)
AXS6_HD int axs6_nf5_index_dithered_fast(float ax, float g_over_s, float u)
{
    return __float2int_rz(__fmaf_rn(ax, g_over_s, AXS6_SUB(u, 0.5f)));
}
#else
AXS6_HD int axs6_nf5_index_dithered_fast(float ax, float g_over_s, float u)
{
    return (int)fmaf(ax, g_over_s, u - 0.5f);
}
#endif

// Uniform-grid magnitude: round-half-even of n * 31, or floor + (u < frac) (core.py:348-359).
AXS6_HD int axs6_uniform_mag(float n)
{
    float m = AXS6_RINT(AXS6_MUL(n, 31.0f));
    m = m < 0.0f ? 0.0f : m;
    m = m > 31.0f ? 31.0f : m;
    return (int)m;
}

AXS6_HD int axs6_uniform_mag_stochastic(float n, float u)
{
    const float t = AXS6_MUL(n, 31.0f);
    const float fl = AXS6_FLOOR(t);
    const float frac = AXS6_SUB(t, fl);
    float m = (u < frac) ? AXS6_ADD(fl, 1.0f) : fl;
    m = m < 0.0f ? 0.0f : m;
    m = m > 31.0f ? 31.0f : m;
    return (int)m;
}

// sign(x) * level * S with sign(+-0) = 0 (quantize_unified.py:169, :197): the magnitude is one
// RN product, the sign is copied from x, and an input zero yields +0.
AXS6_HD float axs6_fq_value(uint32_t xbits, float level, float scale)
{
    if ((xbits & 0x7FFFFFFFu) == 0u) return AXS6_MUL(AXS6_MUL(0.0f, level), scale);
    const float v = AXS6_MUL(level, scale);
    return axs6_from_bits(axs6_to_bits(v) | (xbits & 0x80000000u));
}

// Same for a finite scale, branch-free: |y| = level * S, sign of x, +0 for x = +-0.
AXS6_HD float axs6_fq_value_fast(float x, float level, float scale)
{
    const float v = AXS6_MUL(level, scale);
    const float y = axs6_from_bits(axs6_to_bits(v) | (axs6_to_bits(x) & 0x80000000u));
    return (x == 0.0f) ? 0.0f : y;
}

// where(sign, -v, v) with v = level * S (quantize_unified.py:300-302, core.py:388-389).
AXS6_HD float axs6_decode_value(uint32_t negative, float level, float scale)
{
    const float v = AXS6_MUL(level, scale);
    return axs6_from_bits(axs6_to_bits(v) ^ (negative << 31));
}

// Uniform-grid reconstruction level m / 31 (core.py:388).
AXS6_HD float axs6_uniform_level(int m) { return AXS6_DIV((float)m, 31.0f); }

// fp32 -> bf16 bits, round to nearest even (NaN kept quiet); bf16 bits -> fp32.
AXS6_HD uint16_t axs6_f32_to_bf16_bits(float f)
{
    uint32_t u = axs6_to_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

AXS6_HD float axs6_bf16_bits_to_f32(uint32_t b) { return axs6_from_bits(b << 16); }

// Philox4x32-10 (Salmon et al., SC'11): counter-based generator used for stochastic rounding.
struct Axs6Philox { uint32_t r[4]; };

AXS6_HD Axs6Philox axs6_philox(uint64_t counter, uint64_t key)
{
    uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0u, c3 = 0u;
    uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int i = 0; i < 10; ++i) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        const uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    Axs6Philox o;
    o.r[0] = c0; o.r[1] = c1; o.r[2] = c2; o.r[3] = c3;
    return o;
}

// The ten round keys for one 64-bit key, and the same generator taking them ready-made: kernels receive the
// struct by value, so the keys are constant-bank operands of the xors instead of twenty additions per block.
struct Axs6PhiloxKeys { uint32_t k0[10], k1[10]; };

AXS6_HD Axs6PhiloxKeys axs6_philox_keys(uint64_t key)
{
    Axs6PhiloxKeys ks;
    for (int i = 0; i < 10; ++i) {
        ks.k0[i] = (uint32_t)key + (uint32_t)i * 0x9E3779B9u;
        ks.k1[i] = (uint32_t)(key >> 32) + (uint32_t)i * 0xBB67AE85u;
    }
    return ks;
}

AXS6_HD Axs6Philox axs6_philox_keyed(uint64_t counter, const Axs6PhiloxKeys &ks)
{
    uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0u, c3 = 0u;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int i = 0; i < 10; ++i) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ ks.k0[i];
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ ks.k1[i];
        c1 = (uint32_t)p1; c3 = (uint32_t)p0; c0 = n0; c2 = n2;
    }
    Axs6Philox o;
    o.r[0] = c0; o.r[1] = c1; o.r[2] = c2; o.r[3] = c3;
    return o;
}

// 16 random bits -> the midpoints (h + 0.5) / 65536 of a 2^-16 grid on (0, 1): mean exactly 1/2.
AXS6_HD float axs6_u01_16(uint32_t h) { return ((float)h + 0.5f) * 1.52587890625e-5f; }
