// Pack (values -> 6-bit codes + shared exponent) and unpack kernels and their C entry points.
//
// Roofline: HBM bandwidth.  Algorithmic bytes per block of B values:
//   pack   B * sizeof(in)  +  record bytes (WIRE 1 + 3B/4, SPEC 2 + 3B/4)  or  1 + 2B (PLANES)
//   unpack the mirror image.
// Byte layouts: a CTA iteration owns 256*U consecutive chunks, i.e. a run of whole blocks
// whose records are contiguous in the output.  Threads drop their 6 payload bytes (8 codes)
// into a shared-memory image of that run, which is then moved with 128-bit accesses (the
// run's size is a multiple of 16 bytes for every block size and layout).
#include "async_copy.cuh"
#include "quant_device.cuh"

namespace axs6 {

ChunkGeom make_geom(int64_t rows, int64_t cols, int block);

struct CodecArgs {
    const void *x;       // pack: values in;   unpack: unused
    void *y;             // unpack: values out; pack: unused
    int64_t ld;          // leading dimension of x / y
    ChunkGeom g;
    uint32_t via_bf16;
    uint64_t seed, offset;
    Axs6PhiloxKeys keys;               // round keys of `seed`
    const unsigned long long *epoch;   // device counter added to `offset` (stochastic kernels only)
    const float *noise;
    float *err;              // error feedback (pack, fp32 in, planes out): residual added to x before, replaced after
    uint8_t *p0, *p1, *p2;   // planes (exp, sign, mag) or p0 = records
    int rec, hdr;            // record bytes and header bytes of the byte layout
    int lanes_log2;          // log2(block / 8): lanes that share one block
};

constexpr int kPlanes = 0, kBytes = 1;

// Split layout: position of block `blk` (row-major index over rows x nblk) in the exponent plane, which is stored by
// PAIRS of blocks: (ceil(nblk / 2), rows, 2) bytes.  The exponents that one GEMM operand tile needs (two consecutive
// blocks of 128 rows, or four blocks of 64 rows) are then contiguous runs that a bulk copy can fetch.
__device__ __forceinline__ int64_t split_exp_index(int64_t blk, int64_t nblk, int64_t rows)
{
    const int64_t row = blk / nblk, b = blk - row * nblk;
    return ((b >> 1) * rows + row) * 2 + (b & 1);
}
constexpr int kU = 2;                               // chunks per thread per iteration
constexpr int kStageBytes = kU * kThreads * 8;      // worst case: B = 8, 8-byte records

// 8 codes (6 bits each) of one chunk.
template <int GRID, int ROUND>
__device__ __forceinline__ void chunk_codes(const uint32_t (&v)[8], uint32_t (&code)[8], int &se,
                                            const uint8_t *rev, int lanes, const float (&u)[8])
{
    const uint32_t amax = group_max(chunk_amax_bits(v), lanes);
    const Axs6Scale s = axs6_scale_codes(amax);
    se = s.se;
    if (s.fast) {
        const float c = AXS6_MUL(s.inv, GRID == AXS6_GRID_NF5 ? 1023.0f : 31.0f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x = __uint_as_float(v[i]);
            int m;
            if (GRID == AXS6_GRID_NF5) {
                const int idx = (ROUND == kNearest) ? axs6_nf5_index_fast(fabsf(x), c)
                              : (ROUND == kPhilox) ? axs6_nf5_index_dithered_fast(fabsf(x), c, u[i])
                                                   : axs6_nf5_index_dithered(AXS6_MUL(fabsf(x), s.inv), u[i]);
                m = rev[idx];
            } else {
                m = (ROUND == kNearest) ? axs6_uniform_mag_fast(fabsf(x), c)
                                        : axs6_uniform_mag_stochastic(AXS6_MUL(fabsf(x), s.inv), u[i]);
            }
            code[i] = (uint32_t)m | (x < 0.0f ? 32u : 0u);          // x < 0 is false for -0.0
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t ab = v[i] & 0x7FFFFFFFu;
            const float n = axs6_normalise(__uint_as_float(ab), s);
            int m;
            if (GRID == AXS6_GRID_NF5) {
                const int idx = (ROUND == kNearest) ? axs6_nf5_index(n) : axs6_nf5_index_dithered(n, u[i]);
                m = rev[idx];
            } else {
                m = (ROUND == kNearest) ? axs6_uniform_mag(n) : axs6_uniform_mag_stochastic(n, u[i]);
            }
            const uint32_t neg = (ab != 0u) ? (v[i] >> 31) : 0u;
            code[i] = (neg << 5) | (uint32_t)m;
        }
    }
}

// kEf (fp32 input, planes out): error feedback in the same pass.  corrected = x + err (one fp32 addition), the codes
// are those of `corrected`, and err becomes corrected - reconstruction (the arithmetic of unpack_vec_kernel), as in
// quantize_with_error_feedback of the reference (axs/quantize.py:190-199) without its four extra passes over HBM.
template <typename Tin, int GRID, int ROUND, int LAYOUT, bool kEf = false>
__global__ void __launch_bounds__(kThreads) pack_vec_kernel(const CodecArgs a)
{
    __shared__ __align__(16) uint8_t rev[GRID == AXS6_GRID_NF5 ? 1024 : 16];
    __shared__ __align__(16) uint8_t stage[LAYOUT == kBytes ? kStageBytes : 16];
    __shared__ float lev[kEf ? 32 : 1];
    if (GRID == AXS6_GRID_NF5) build_reverse_lut(rev);
    if (kEf) build_levels<GRID>(lev);
    __syncthreads();
    pdl_wait();                    // nothing of the caller's memory is touched before this point

    const int lg = a.lanes_log2, lanes = 1 << lg;
    const uint64_t offset = (ROUND == kPhilox) ? a.offset + *a.epoch : 0ull;
    const int64_t total_blocks = a.g.total_chunks >> lg;
    const int64_t step = (int64_t)gridDim.x * kThreads * kU;
    const int j = threadIdx.x & (lanes - 1);
    const int lb_thread = (int)threadIdx.x >> lg;           // block of this thread inside a 256-chunk group
    const int blocks_per_group = kThreads >> lg;
    for (int64_t base = (int64_t)blockIdx.x * kThreads * kU; base < a.g.total_chunks; base += step) {
        if (base + step >= a.g.total_chunks) pdl_launch_dependents();      // last iteration of this CTA: the next kernel may move in
        uint32_t v[kU][8];
        bool act[kU];
        int64_t eo[kU];                                     // kEf: offset of the chunk's residuals, -1 = none
#pragma unroll
        for (int k = 0; k < kU; ++k) {
            const int64_t c = base + (int64_t)k * kThreads + threadIdx.x;
            act[k] = c < a.g.total_chunks;
            int64_t xo = c * kChunk;
            bool has = act[k];
            if (!a.g.flat) {
                const int64_t row = c / a.g.cpr;
                const int64_t col0 = (c - row * a.g.cpr) * kChunk;
                has = has && col0 < a.g.cols;
                xo = row * a.ld + col0;
            }
            eo[k] = has ? xo : -1;
            if (has) {
                ChunkIO<Tin>::load(a.x, xo, v[k], a.via_bf16 != 0u);
                if (kEf) {
                    const uint4 e0 = ld_stream16(a.err + xo), e1 = ld_stream16(a.err + xo + 4);
                    const uint32_t e[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        v[k][i] = __float_as_uint(AXS6_ADD(__uint_as_float(v[k][i]), __uint_as_float(e[i])));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[k][i] = 0u;
            }
        }
#pragma unroll
        for (int k = 0; k < kU; ++k) {
            const int64_t c = base + (int64_t)k * kThreads + threadIdx.x;
            float u[8];
            uint32_t code[8];
            int se;
            chunk_uniforms<ROUND>(u, c, act[k], a.keys, offset, a.noise);
            chunk_codes<GRID, ROUND>(v[k], code, se, rev, lanes, u);
            if (kEf && eo[k] >= 0) {
                const float scale = axs6_scale_decode((uint32_t)se);
                uint32_t r[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    r[i] = __float_as_uint(AXS6_SUB(__uint_as_float(v[k][i]), axs6_decode_value(code[i] >> 5, lev[code[i] & 31u], scale)));
                st_stream16(a.err + eo[k], make_uint4(r[0], r[1], r[2], r[3]));
                st_stream16(a.err + eo[k] + 4, make_uint4(r[4], r[5], r[6], r[7]));
            }
            if (LAYOUT == kPlanes) {
                if (act[k]) {
                    uint2 sg, mg;
                    sg.x = (code[0] >> 5) | ((code[1] >> 5) << 8) | ((code[2] >> 5) << 16) | ((code[3] >> 5) << 24);
                    sg.y = (code[4] >> 5) | ((code[5] >> 5) << 8) | ((code[6] >> 5) << 16) | ((code[7] >> 5) << 24);
                    mg.x = (code[0] & 31u) | ((code[1] & 31u) << 8) | ((code[2] & 31u) << 16) | ((code[3] & 31u) << 24);
                    mg.y = (code[4] & 31u) | ((code[5] & 31u) << 8) | ((code[6] & 31u) << 16) | ((code[7] & 31u) << 24);
                    st_stream8(a.p1 + c * kChunk, sg);
                    st_stream8(a.p2 + c * kChunk, mg);
                    if (j == 0) a.p0[c >> lg] = (uint8_t)se;
                }
            } else {
                const uint32_t lo = code[0] | (code[1] << 6) | (code[2] << 12) | (code[3] << 18) |
                                    (code[4] << 24) | (code[5] << 30);
                const uint32_t hi = (code[5] >> 2) | (code[6] << 4) | (code[7] << 10);
                const int lb = k * blocks_per_group + lb_thread;
                uint8_t *s = stage + lb * a.rec;
                if (j == 0) {
                    if (a.hdr == 1) {
                        s[0] = (uint8_t)se;
                    } else if (a.hdr == 2) {
                        s[0] = (uint8_t)((se << 2) & 0xFF);
                        s[1] = (uint8_t)(se >> 6);
                    } else if (act[k]) {
                        a.p1[split_exp_index(c >> lg, a.g.cpr >> lg, a.g.rows)] = (uint8_t)se;   // split layout: exponent plane
                    }
                }
                s += a.hdr + 6 * j;
                s[0] = (uint8_t)lo; s[1] = (uint8_t)(lo >> 8); s[2] = (uint8_t)(lo >> 16); s[3] = (uint8_t)(lo >> 24);
                s[4] = (uint8_t)hi; s[5] = (uint8_t)(hi >> 8);
            }
        }
        if (LAYOUT == kBytes) {
            __syncthreads();
            const int64_t blk0 = base >> lg;
            int nb = (kU * kThreads) >> lg;
            if ((int64_t)nb > total_blocks - blk0) nb = (int)(total_blocks - blk0);
            const int len = nb * a.rec;
            uint8_t *dst = a.p0 + blk0 * a.rec;                 // 16-byte aligned by construction
            const int nvec = len >> 4;
            for (int i = threadIdx.x; i < nvec; i += kThreads)
                st_stream16(dst + 16 * i, reinterpret_cast<const uint4 *>(stage)[i]);
            for (int i = (nvec << 4) + threadIdx.x; i < len; i += kThreads) dst[i] = stage[i];
            __syncthreads();
        }
    }
}

// One lane per value of the zero-padded row (any alignment).
template <typename Tin, int GRID, int ROUND, int LAYOUT>
__global__ void __launch_bounds__(kThreads) pack_generic_kernel(const CodecArgs a)
{
    __shared__ __align__(16) uint8_t rev[GRID == AXS6_GRID_NF5 ? 1024 : 16];
    if (GRID == AXS6_GRID_NF5) build_reverse_lut(rev);
    __syncthreads();
    pdl_wait();                    // nothing of the caller's memory is touched before this point

    const int lane = threadIdx.x & 31;
    const uint64_t offset = (ROUND == kPhilox) ? a.offset + *a.epoch : 0ull;
    const int B = a.g.block;
    const int64_t padded = a.g.cpr * kChunk;
    const int64_t nblk = padded / B;
    const int64_t tiles_per_row = (padded + 31) / 32;
    const int64_t tiles = a.g.rows * tiles_per_row;
    const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
    for (int64_t t = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); t < tiles; t += warps) {
        if (t + warps >= tiles) pdl_launch_dependents();
        const int64_t row = t / tiles_per_row;
        const int64_t pc = (t - row * tiles_per_row) * 32 + lane;
        const bool in_pad = pc < padded;
        const bool has = pc < a.g.cols;
        const uint32_t v = has ? ChunkIO<Tin>::load1(a.x, row * a.ld + pc, a.via_bf16 != 0u) : 0u;
        const uint32_t ab = v & 0x7FFFFFFFu;
        const uint32_t amax = group_max(ab, B);
        const Axs6Scale s = axs6_scale_codes(amax);
        const float n = axs6_normalise(__uint_as_float(ab), s);
        const float u = element_uniform<ROUND>(row * padded + pc, in_pad, a.keys, offset, a.noise);
        int m;
        if (GRID == AXS6_GRID_NF5) {
            const int idx = (ROUND == kNearest) ? axs6_nf5_index(n)
                          : (ROUND == kPhilox && s.fast) ? axs6_nf5_index_dithered_fast(__uint_as_float(ab), AXS6_MUL(s.inv, 1023.0f), u)
                                                         : axs6_nf5_index_dithered(n, u);
            m = rev[idx];
        } else {
            m = (ROUND == kNearest) ? axs6_uniform_mag(n) : axs6_uniform_mag_stochastic(n, u);
        }
        const uint32_t neg = (ab != 0u) ? (v >> 31) : 0u;
        const uint32_t code = (neg << 5) | (uint32_t)m;
        const uint32_t next = __shfl_down_sync(0xFFFFFFFFu, code, 1);
        const int i = (int)(pc % B);
        const int64_t blk = row * nblk + pc / B;
        if (!in_pad) continue;
        if (LAYOUT == kPlanes) {
            a.p1[row * padded + pc] = (uint8_t)neg;
            a.p2[row * padded + pc] = (uint8_t)m;
            if (i == 0) a.p0[blk] = (uint8_t)s.se;
        } else {
            uint8_t *r = a.p0 + blk * a.rec;
            if (i == 0) {
                if (a.hdr == 1) {
                    r[0] = (uint8_t)s.se;
                } else if (a.hdr == 2) {
                    r[0] = (uint8_t)((s.se << 2) & 0xFF);
                    r[1] = (uint8_t)(s.se >> 6);
                } else {
                    a.p1[split_exp_index(blk, nblk, a.g.rows)] = (uint8_t)s.se;
                }
            }
            const int q = i & 3;
            if (q != 3) {
                const uint32_t b = (q == 0) ? (code | (next << 6)) : (q == 1) ? ((code >> 2) | (next << 4))
                                                                              : ((code >> 4) | (next << 2));
                r[a.hdr + (i >> 2) * 3 + q] = (uint8_t)b;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------ unpack
template <typename Tout, int GRID, int LAYOUT>
__global__ void __launch_bounds__(kThreads) unpack_vec_kernel(const CodecArgs a)
{
    __shared__ float lev[32];
    __shared__ __align__(16) uint8_t stage[LAYOUT == kBytes ? kStageBytes : 16];
    build_levels<GRID>(lev);
    __syncthreads();
    pdl_wait();                    // nothing of the caller's memory is touched before this point

    const int lg = a.lanes_log2, lanes = 1 << lg;
    const int64_t total_blocks = a.g.total_chunks >> lg;
    const int64_t step = (int64_t)gridDim.x * kThreads * kU;
    const int j = threadIdx.x & (lanes - 1);
    const int lb_thread = (int)threadIdx.x >> lg;
    const int blocks_per_group = kThreads >> lg;
    for (int64_t base = (int64_t)blockIdx.x * kThreads * kU; base < a.g.total_chunks; base += step) {
        if (base + step >= a.g.total_chunks) pdl_launch_dependents();      // last iteration of this CTA: the next kernel may move in
        if (LAYOUT == kBytes) {
            const int64_t blk0 = base >> lg;
            int nb = (kU * kThreads) >> lg;
            if ((int64_t)nb > total_blocks - blk0) nb = (int)(total_blocks - blk0);
            const int len = nb * a.rec;
            const uint8_t *src = a.p0 + blk0 * a.rec;
            const int nvec = len >> 4;
            for (int i = threadIdx.x; i < nvec; i += kThreads)
                reinterpret_cast<uint4 *>(stage)[i] = ld_stream16(src + 16 * i);
            for (int i = (nvec << 4) + threadIdx.x; i < len; i += kThreads) stage[i] = src[i];
            __syncthreads();
        }
#pragma unroll
        for (int k = 0; k < kU; ++k) {
            const int64_t c = base + (int64_t)k * kThreads + threadIdx.x;
            bool act = c < a.g.total_chunks;
            int64_t yo = c * kChunk;
            if (!a.g.flat) {
                const int64_t row = c / a.g.cpr;
                const int64_t col0 = (c - row * a.g.cpr) * kChunk;
                act = act && col0 < a.g.cols;
                yo = row * a.ld + col0;
            }
            if (!act) continue;
            uint32_t se, neg[8], mag[8];
            if (LAYOUT == kPlanes) {
                se = a.p0[c >> lg];
                const uint2 sg = ld_stream8(a.p1 + c * kChunk), mg = ld_stream8(a.p2 + c * kChunk);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    neg[i] = (sg.x >> (8 * i)) & 1u; neg[4 + i] = (sg.y >> (8 * i)) & 1u;
                    mag[i] = (mg.x >> (8 * i)) & 31u; mag[4 + i] = (mg.y >> (8 * i)) & 31u;
                }
            } else {
                const int lb = k * blocks_per_group + lb_thread;
                const uint8_t *s = stage + lb * a.rec;
                se = (a.hdr == 1) ? (uint32_t)s[0] : (a.hdr == 2) ? (((uint32_t)s[0] | ((uint32_t)s[1] << 8)) >> 2) & 0xFFu
                                                                  : (uint32_t)a.p1[split_exp_index(c >> lg, a.g.cpr >> lg, a.g.rows)];
                s += a.hdr + 6 * j;
                const uint32_t lo = (uint32_t)s[0] | ((uint32_t)s[1] << 8) | ((uint32_t)s[2] << 16) | ((uint32_t)s[3] << 24);
                const uint32_t hi = (uint32_t)s[4] | ((uint32_t)s[5] << 8);
                uint32_t code[8];
                code[0] = lo & 63u; code[1] = (lo >> 6) & 63u; code[2] = (lo >> 12) & 63u; code[3] = (lo >> 18) & 63u;
                code[4] = (lo >> 24) & 63u; code[5] = ((lo >> 30) | (hi << 2)) & 63u;
                code[6] = (hi >> 4) & 63u; code[7] = (hi >> 10) & 63u;
#pragma unroll
                for (int i = 0; i < 8; ++i) { neg[i] = code[i] >> 5; mag[i] = code[i] & 31u; }
            }
            const float scale = axs6_scale_decode(se);
            float y[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = axs6_decode_value(neg[i], lev[mag[i]], scale);
            ChunkIO<Tout>::store(a.y, yo, y);
        }
        if (LAYOUT == kBytes) __syncthreads();
    }
}

template <typename Tout, int GRID, int LAYOUT>
__global__ void __launch_bounds__(kThreads) unpack_generic_kernel(const CodecArgs a)
{
    __shared__ float lev[32];
    build_levels<GRID>(lev);
    __syncthreads();
    pdl_wait();                    // nothing of the caller's memory is touched before this point

    const int B = a.g.block;
    const int64_t padded = a.g.cpr * kChunk;
    const int64_t nblk = padded / B;
    const int64_t total = a.g.rows * a.g.cols;
    const int64_t nthreads = (int64_t)gridDim.x * kThreads;
    for (int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x; e < total; e += nthreads) {
        if (e + nthreads >= total) pdl_launch_dependents();
        const int64_t row = e / a.g.cols;
        const int64_t pc = e - row * a.g.cols;
        const int i = (int)(pc % B);
        const int64_t blk = row * nblk + pc / B;
        uint32_t se, neg, mag;
        if (LAYOUT == kPlanes) {
            se = a.p0[blk];
            neg = a.p1[row * padded + pc] & 1u;
            mag = a.p2[row * padded + pc] & 31u;
        } else {
            const uint8_t *r = a.p0 + blk * a.rec;
            se = (a.hdr == 1) ? (uint32_t)r[0] : (a.hdr == 2) ? (((uint32_t)r[0] | ((uint32_t)r[1] << 8)) >> 2) & 0xFFu
                                                              : (uint32_t)a.p1[split_exp_index(blk, nblk, a.g.rows)];
            const int bit = 6 * i, k = bit >> 3, sh = bit & 7;
            uint32_t w = r[a.hdr + k];
            if (sh > 2) w |= (uint32_t)r[a.hdr + k + 1] << 8;
            const uint32_t code = (w >> sh) & 63u;
            neg = code >> 5;
            mag = code & 31u;
        }
        ChunkIO<Tout>::store1(a.y, row * a.ld + pc, axs6_decode_value(neg, lev[mag], axs6_scale_decode(se)));
    }
}

// ------------------------------------------------------------------------------------------ host
template <typename K>
static int launch_codec(K kernel, const CodecArgs &a, int64_t items_per_cta, int64_t items, cudaStream_t stream,
                        int max_per_sm = 0)
{
    const DeviceInfo &d = device_info();
    int per_sm = cached_occupancy(reinterpret_cast<const void *>(kernel), kThreads);
    if (per_sm < 1) return AXS6_ERR_LAUNCH;
    if (max_per_sm > 0 && per_sm > max_per_sm) per_sm = max_per_sm;
    int64_t ctas = (items + items_per_cta - 1) / items_per_cta;
    const int64_t cap = tune_value(1);
    if (cap > 0 && per_sm > cap) per_sm = (int)cap;
    const int64_t resident = (int64_t)d.sms * per_sm;
    if (ctas > resident) ctas = resident;
    if (ctas < 1) ctas = 1;
    const bool launched = launch_overlapped(false, kernel, (unsigned)ctas, kThreads, 0, stream, a) == cudaSuccess;
    count_launch();
    return launched ? check_launch() : AXS6_ERR_LAUNCH;
}

template <typename Tin, int GRID, int ROUND>
static int launch_pack(const CodecArgs &a, bool planes, bool vec, cudaStream_t st)
{
    const int64_t tiles = a.g.rows * ((a.g.cpr * kChunk + 31) / 32);
    if (vec) {
        if (planes) return launch_codec(pack_vec_kernel<Tin, GRID, ROUND, kPlanes>, a, (int64_t)kThreads * kU, a.g.total_chunks, st);
        return launch_codec(pack_vec_kernel<Tin, GRID, ROUND, kBytes>, a, (int64_t)kThreads * kU, a.g.total_chunks, st);
    }
    if (planes) return launch_codec(pack_generic_kernel<Tin, GRID, ROUND, kPlanes>, a, kThreads / 32, tiles, st);
    return launch_codec(pack_generic_kernel<Tin, GRID, ROUND, kBytes>, a, kThreads / 32, tiles, st);
}

template <typename Tin>
static int dispatch_pack(const CodecArgs &a, int grid, int round, bool planes, bool vec, cudaStream_t st)
{
#define AXS6_CASE(G, R) \
    if (grid == G && round == R) return launch_pack<Tin, G, R>(a, planes, vec, st);
    AXS6_CASE(AXS6_GRID_NF5, kNearest)
    AXS6_CASE(AXS6_GRID_NF5, kPhilox)
    AXS6_CASE(AXS6_GRID_NF5, kNoise)
    AXS6_CASE(AXS6_GRID_UNIFORM, kNearest)
    AXS6_CASE(AXS6_GRID_UNIFORM, kPhilox)
    AXS6_CASE(AXS6_GRID_UNIFORM, kNoise)
#undef AXS6_CASE
    return AXS6_ERR_ARG;
}

template <typename Tout, int GRID>
static int launch_unpack(const CodecArgs &a, bool planes, bool vec, cudaStream_t st)
{
    if (vec) {
        // planes -> fp32: 6.0 TB/s with 5 or 6 resident CTAs per SM, 4.5 with the 8 that fit (too many stores in
        // flight); planes -> bf16 is fastest with all 8
        if (planes) return launch_codec(unpack_vec_kernel<Tout, GRID, kPlanes>, a, (int64_t)kThreads * kU, a.g.total_chunks, st,
                                        sizeof(Tout) == 4 ? 6 : 0);
        return launch_codec(unpack_vec_kernel<Tout, GRID, kBytes>, a, (int64_t)kThreads * kU, a.g.total_chunks, st);
    }
    const int64_t total = a.g.rows * a.g.cols;
    if (planes) return launch_codec(unpack_generic_kernel<Tout, GRID, kPlanes>, a, kThreads, total, st);
    return launch_codec(unpack_generic_kernel<Tout, GRID, kBytes>, a, kThreads, total, st);
}

// ------------------------------------------------------------------------------------------ bf16 fast pack
// Specialised pack for the common case bf16 input, NF5 grid, nearest rounding, block 32, byte
// layouts, 16-byte aligned and contiguous: ONE THREAD PER BLOCK and integer arithmetic on the
// bf16 bit patterns.  About 10 instructions per value instead of 25 (the general kernel is bound
// by instruction issue, not by HBM).
//
// Why integers suffice: a bf16 value is (128 + m) * 2^(e - 134) with a 7-bit m.  For a block whose
// largest magnitude has exponent field E the scale is 2^(E - 126) (the top-of-binade exponent bump
// of the fp32 path cannot occur: the low 16 mantissa bits are zero), and
//     idx = trunc(|x| / S * 1023) = ((128 + m) * 1023) >> (8 + j),   j = E - e,
// exactly, because the fp32 product has only 18 significant bits.  idx = 0 for j >= 10.  So the
// 5-bit code depends on (j, m) only: key = ((E << 7) | 127) - |x|_bits = j * 128 + (127 - m) indexes a
// 1280-entry table; keys beyond it (small or zero values, denormals) give code 0.  Taken for
// E in [11, 252]; an all-zero block is a record of zeros; anything else (denormal-range or
// near-overflow block maxima) takes the per-value path of the general formulas.
constexpr int kFastBlocks = 256;         // blocks (threads) per CTA iteration
constexpr int kKeyLimit = 1280;

__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("max.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t min_u16x2(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("min.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// Codes of one block of 32 bf16 values (16 words of two) as the 192-bit payload and the exponent byte.
// `table` is the shared-memory key table built by build_key_table.
__device__ __forceinline__ void bf16_block_payload(const uint32_t (&w)[16], const uint8_t *table, uint32_t (&pay)[6], uint32_t &se)
{
    uint32_t mx = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) mx = max_u16x2(mx, w[i] & 0x7FFF7FFFu);
    const uint32_t amax16 = max(mx & 0xFFFFu, mx >> 16);
    const uint32_t ef = amax16 >> 7;
    if (amax16 == 0u || (ef >= 11u && ef <= 252u)) {
        se = amax16 ? ef + 1u : 0u;
        const uint32_t a1 = amax16 ? ((ef << 7) | 127u) : 0x7FFFu;
        const uint32_t a2 = a1 | (a1 << 16);
        const uint32_t lim2 = (uint32_t)kKeyLimit | ((uint32_t)kKeyLimit << 16);
#pragma unroll
        for (int gq = 0; gq < 8; ++gq) {                 // 4 values -> one 24-bit group
            const uint32_t wa = w[2 * gq], wc = w[2 * gq + 1];
            const uint32_t ma = wa & 0x7FFF7FFFu, mb = wc & 0x7FFF7FFFu;
            const uint32_t ka = min_u16x2(a2 - ma, lim2), kb = min_u16x2(a2 - mb, lim2);
            const uint32_t c0 = table[ka & 0xFFFFu], c1 = table[ka >> 16];
            const uint32_t c2 = table[kb & 0xFFFFu], c3 = table[kb >> 16];
            uint32_t g = c0 | (c1 << 6) | (c2 << 12) | (c3 << 18);
            // sign bits of the non-zero values: bit 15 / 31 of (w & (|w| + 0x7FFF)) per half
            const uint32_t ta = wa & (ma + 0x7FFF7FFFu), tb = wc & (mb + 0x7FFF7FFFu);
            // bytes 1, 3 of ta and 1, 3 of tb, each replicated from its top bit: 0x00 or 0xFF per value
            uint32_t r;
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(ta), "r"(tb), "r"(0xFDB9u));
            g |= (r & 0x00020820u) | ((r >> 8) & 0x00800000u);   // sign bits at 5, 11, 17 and 23
            // append the 24-bit group to the 192-bit payload
            if ((gq & 3) == 0) { pay[(gq >> 2) * 3] = g; }
            else if ((gq & 3) == 1) { pay[(gq >> 2) * 3] |= g << 24; pay[(gq >> 2) * 3 + 1] = g >> 8; }
            else if ((gq & 3) == 2) { pay[(gq >> 2) * 3 + 1] |= g << 16; pay[(gq >> 2) * 3 + 2] = g >> 16; }
            else { pay[(gq >> 2) * 3 + 2] |= g << 8; }
        }
    } else {
        // rare block (denormal-range or near-overflow maximum): the general fp32 formulas
        const Axs6Scale sc = axs6_scale_codes(amax16 << 16);
        se = (uint32_t)sc.se;
#pragma unroll
        for (int i = 0; i < 6; ++i) pay[i] = 0u;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const uint32_t bits = (i & 1) ? (w[i >> 1] & 0xFFFF0000u) : (w[i >> 1] << 16);
            const uint32_t ab = bits & 0x7FFFFFFFu;
            const int idx = axs6_nf5_index(axs6_normalise(__uint_as_float(ab), sc));
            const uint32_t code = (uint32_t)g_reverse[idx] | ((ab != 0u && (bits >> 31)) ? 32u : 0u);
            const int word = (6 * i) >> 5, off = (6 * i) & 31;
            pay[word] |= code << off;
            if (off > 26) pay[word + 1] |= code >> (32 - off);
        }
    }
}

__device__ __forceinline__ void build_key_table(uint8_t *table /*kKeyLimit + 16, 16-byte aligned*/, int tid, int nthreads)
{
    for (int i = tid; i < (kKeyLimit + 16) / 16; i += nthreads)
        reinterpret_cast<uint4 *>(table)[i] = reinterpret_cast<const uint4 *>(g_key_code)[i];
}

// The record of a block as seven 32-bit words of the output image, shifted so that its first byte lands
// on byte `sh` of the first word: sft = 8 * (sh + HDR).
template <int HDR>
__device__ __forceinline__ void record_words(const uint32_t (&pay)[6], uint32_t se, uint32_t sft, uint32_t (&W)[7])
{
    uint32_t prev = HDR == 1 ? (se << 24) : (((se << 2) & 0xFFFFu) << 16);
#pragma unroll
    for (int i = 0; i < 6; ++i) {
        W[i] = __funnelshift_lc(prev, pay[i], sft);
        prev = pay[i];
    }
    W[6] = __funnelshift_lc(prev, 0u, sft);
}

template <int HDR>
__global__ void __launch_bounds__(kFastBlocks) pack_bf16_nf5_b32_kernel(const uint16_t *__restrict__ x,
                                                                       uint8_t *__restrict__ out, int64_t nblocks)
{
    constexpr int REC = HDR + 24;
    __shared__ __align__(16) uint8_t table[kKeyLimit + 16];
    __shared__ __align__(16) uint8_t stage[2][kFastBlocks * REC];
    build_key_table(table, threadIdx.x, kFastBlocks);
    __syncthreads();

    int buf = 0;
    const int64_t groups = (nblocks + kFastBlocks - 1) / kFastBlocks;
    for (int64_t grp = blockIdx.x; grp < groups; grp += gridDim.x, buf ^= 1) {
        const int64_t b = grp * kFastBlocks + threadIdx.x;
        uint8_t *rec = &stage[buf][threadIdx.x * REC];
        if (b < nblocks) {
            uint32_t w[16];
            const uint16_t *src = x + b * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = ld_stream16(src + 8 * i);
                w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
            }
            uint32_t pay[6];
            uint32_t se;
            bf16_block_payload(w, table, pay, se);
            if (HDR == 1) {
                rec[0] = (uint8_t)se;
            } else {
                rec[0] = (uint8_t)((se << 2) & 0xFFu);
                rec[1] = (uint8_t)(se >> 6);
            }
#pragma unroll
            for (int i = 0; i < 6; ++i) {
                rec[HDR + 4 * i] = (uint8_t)pay[i];
                rec[HDR + 4 * i + 1] = (uint8_t)(pay[i] >> 8);
                rec[HDR + 4 * i + 2] = (uint8_t)(pay[i] >> 16);
                rec[HDR + 4 * i + 3] = (uint8_t)(pay[i] >> 24);
            }
        }
        __syncthreads();
        // move this iteration's records (contiguous, 16-byte aligned: 256 * REC is a multiple of 16)
        const int64_t blk0 = grp * kFastBlocks;
        int64_t nb = nblocks - blk0;
        if (nb > kFastBlocks) nb = kFastBlocks;
        const int len = (int)nb * REC;
        uint8_t *dst = out + blk0 * REC;
        const int nvec = len >> 4;
        for (int i = threadIdx.x; i < nvec; i += kFastBlocks)
            st_stream16(dst + 16 * i, reinterpret_cast<const uint4 *>(stage[buf])[i]);
        for (int i = (nvec << 4) + threadIdx.x; i < len; i += kFastBlocks) dst[i] = stage[buf][i];
        // the other buffer is written next; this one again only after the next __syncthreads
    }
}

static int launch_pack_fast(const void *x, void *out, int64_t nblocks, int hdr, cudaStream_t st)
{
    const DeviceInfo &d = device_info();
    const void *fn = hdr == 1 ? reinterpret_cast<const void *>(pack_bf16_nf5_b32_kernel<1>)
                              : reinterpret_cast<const void *>(pack_bf16_nf5_b32_kernel<2>);
    int per_sm = cached_occupancy(fn, kFastBlocks);
    if (per_sm < 1) return AXS6_ERR_LAUNCH;
    const int64_t cap = tune_value(1);
    if (cap > 0 && per_sm > cap) per_sm = (int)cap;
    int64_t ctas = (nblocks + kFastBlocks - 1) / kFastBlocks;
    if (ctas > (int64_t)d.sms * per_sm) ctas = (int64_t)d.sms * per_sm;
    if (ctas < 1) ctas = 1;
    if (hdr == 1)
        pack_bf16_nf5_b32_kernel<1><<<(unsigned)ctas, kFastBlocks, 0, st>>>(static_cast<const uint16_t *>(x), static_cast<uint8_t *>(out), nblocks);
    else
        pack_bf16_nf5_b32_kernel<2><<<(unsigned)ctas, kFastBlocks, 0, st>>>(static_cast<const uint16_t *>(x), static_cast<uint8_t *>(out), nblocks);
    count_launch();
    return check_launch();
}

// ------------------------------------------------------------------------------------------ bf16 pack, TMA-fed
// Same arithmetic as pack_bf16_nf5_b32_kernel, different data movement.  That kernel is bound by the
// SM's load/store data path (its wavefront counter sits at 81 % while DRAM is at 29 %): the per-thread
// 64-byte rows make every 128-bit global load a 16-wavefront access and the 25 byte-stores per record
// conflict in shared memory.  Here the TMA unit does both transfers, outside that data path:
//   in    a ring of 256-block tiles (16 KB each), loaded through a 2-D tensor map {32 values, nblocks}
//         with the 64-byte swizzle, so that the four 128-bit shared-memory reads of a thread (one
//         block = one 64-byte row) are free of bank conflicts;
//   out   the 256 records of an iteration are assembled as whole 32-bit words (funnel shifts; the
//         word a record shares with its successor is completed with one shuffle) and leave with ONE bulk
//         shared->global copy, double-buffered.
// Every mbarrier wait is bounded; a wait that gives up sets g_codec_status (read by axs6_codec_status)
// and the CTA leaves its loop.
namespace bulk {

using namespace acp;

constexpr int64_t kOverlapBlocks = 1ll << 21;     // launches of up to this many blocks ask for programmatic dependent launch
constexpr int kStages = 2;                        // with 4 CTAs per SM: 128 KB of loads in flight
constexpr int kStageBytes = kFastBlocks * 64;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kCtrlBytes = 1024;                  // mbarriers, in front of the 1024-aligned tiles

__device__ int g_codec_status;

template <int HDR>
constexpr int smem_bytes() { return 1024 + kCtrlBytes + kStages * kStageBytes + 2 * kFastBlocks * (HDR + 24); }   // dynamic part

template <int HDR>
__global__ void __launch_bounds__(kFastBlocks) pack_bf16_nf5_b32_bulk_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                                      uint8_t *__restrict__ out, int64_t nblocks)
{
    constexpr int REC = HDR + 24;
    constexpr int kOut = kFastBlocks * REC;
    extern __shared__ uint8_t raw[];
    uint8_t *base = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);   // stays a shared-space pointer
    uint8_t *in0 = base + kCtrlBytes;
    uint8_t *out0 = in0 + kStages * kStageBytes;
    __shared__ __align__(16) uint8_t table[kKeyLimit + 16];   // static: its address is an immediate of every lookup
    const uint32_t bar0 = smem_u32(base);
    const int tid = threadIdx.x;
    pdl_launch_dependents();                               // the next launch may take up residence now (it waits in pdl_wait)
    const int64_t groups = (nblocks + kFastBlocks - 1) / kFastBlocks;
    const int64_t nk = (int64_t)blockIdx.x < groups ? (groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    build_key_table(table, tid, kFastBlocks);              // module constants: may run while the previous kernel drains
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8 * s, 1);
        fence_barrier_init();
        fence_async_smem();
        pdl_wait();                                        // caller memory is read from here on
        for (int k = 0; k < kStages && k < nk; ++k) {
            mbar_expect_tx(bar0 + 8 * k, kStageBytes);
            tma_load_2d(smem_u32(in0 + k * kStageBytes), &xmap, bar0 + 8 * k, 0,
                        (int)(((int64_t)blockIdx.x + k * (int64_t)gridDim.x) * kFastBlocks));
        }
    }
    __syncthreads();
    pdl_wait();
    // this thread's block is row `tid` of a tile; 16-byte piece i of a row sits at piece i ^ ((row >> 1) & 3)
    uint32_t piece[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) piece[i] = (uint32_t)tid * 64u + (uint32_t)((i ^ ((tid >> 1) & 3)) << 4);
    // its record starts `sh` bytes into word `wb` of the output image
    const uint32_t wb = (uint32_t)(REC * tid) >> 2, sh = (uint32_t)(REC * tid) & 3u;
    const uint32_t sft = 8u * (sh + HDR);
    const bool owns_first = sh == 0u;                                   // else the predecessor writes that word
    const bool takes_next = ((uint32_t)(REC * (tid + 1)) & 3u) != 0u;    // the successor's head shares my last word

    int s = 0;
    uint32_t ph = 0;
    for (int64_t k = 0; k < nk; ++k) {
        const int64_t grp = (int64_t)blockIdx.x + k * (int64_t)gridDim.x;
        const int64_t b = grp * kFastBlocks + tid;
        uint8_t *ost = out0 + (k & 1) * kOut;
        const bool ok = mbar_wait_bounded(bar0 + 8 * s, ph, 1, &g_codec_status, kWaitLimit);
        uint32_t W[7];
#pragma unroll
        for (int i = 0; i < 7; ++i) W[i] = 0u;
        if (ok && b < nblocks) {
            uint32_t w[16];
            const uint8_t *tile = in0 + s * kStageBytes;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = *reinterpret_cast<const uint4 *>(tile + piece[i]);
                w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
            }
            uint32_t pay[6];
            uint32_t se;
            bf16_block_payload(w, table, pay, se);
            record_words<HDR>(pay, se, sft, W);
        }
        const uint32_t nxt = __shfl_down_sync(0xFFFFFFFFu, W[0], 1);
        if (takes_next) W[6] |= nxt;
        uint32_t *o32 = reinterpret_cast<uint32_t *>(ost) + wb;
        if (owns_first) o32[0] = W[0];
#pragma unroll
        for (int i = 1; i < 7; ++i) o32[i] = W[i];
        fence_async_smem();                    // my words are visible to the TMA unit after the barrier
        if (tid == 0) bulk_wait_read<0>();     // the previous iteration's store has left the other buffer
        if (__syncthreads_or(!ok)) {           // somebody's wait gave up: the whole CTA leaves, once the issuing
            if (tid == 0)                      // thread has waited for the tile loads that are still armed
                drain_ring(bar0, kStages, s, ph, (int)(nk - k < kStages ? nk - k : kStages), kWaitLimit);
            break;
        }
        const int64_t nb = nblocks - grp * kFastBlocks;
        if (nb >= kFastBlocks) {
            if (tid == 0) {
                bulk_store(out + grp * kOut, smem_u32(ost), kOut);
                bulk_commit();
            }
        } else {                               // the ragged last group: plain stores of nb records
            const int len = (int)nb * REC;
            uint8_t *dst = out + grp * kOut;
            const int nvec = len >> 4;
            for (int i = tid; i < nvec; i += kFastBlocks)
                st_stream16(dst + 16 * i, reinterpret_cast<const uint4 *>(ost)[i]);
            for (int i = (nvec << 4) + tid; i < len; i += kFastBlocks) dst[i] = ost[i];
        }
        if (tid == 0 && k + kStages < nk) {
            mbar_expect_tx(bar0 + 8 * s, kStageBytes);
            tma_load_2d(smem_u32(in0 + s * kStageBytes), &xmap, bar0 + 8 * s, 0,
                        (int)(((int64_t)blockIdx.x + (k + kStages) * (int64_t)gridDim.x) * kFastBlocks));
        }
        if (++s == kStages) { s = 0; ph ^= 1u; }
    }
    if (tid == 0) bulk_wait<0>();
}

// -> status, or 1 when this path does not apply (the caller then uses pack_bf16_nf5_b32_kernel)
static int launch_pack_bulk(const void *x, void *out, int64_t nblocks, int hdr, cudaStream_t st)
{
    if (nblocks >= (1ll << 31) - kFastBlocks) return 1;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return 1;
    CUtensorMap map;
    const cuuint64_t gdim[2] = {32, (cuuint64_t)nblocks};
    const cuuint64_t gstride[1] = {64};
    const cuuint32_t box[2] = {32, (cuuint32_t)kFastBlocks};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(x), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return 1;
    const DeviceInfo &d = device_info();
    int64_t ctas = (nblocks + kFastBlocks - 1) / kFastBlocks;
    const int64_t cap = tune_value(1);
    int per_sm = 4;                          // measured 4.9 TB/s; 3 per SM 4.8, 2 per SM 4.5 (3 stages do not help)
    if (cap > 0 && cap < per_sm) per_sm = (int)cap;
    if (ctas > (int64_t)d.sms * per_sm) ctas = (int64_t)d.sms * per_sm;
    if (ctas < 1) ctas = 1;
    uint8_t *o = static_cast<uint8_t *>(out);
    if (!ensure_dynamic_smem(reinterpret_cast<const void *>(&pack_bf16_nf5_b32_bulk_kernel<1>), smem_bytes<1>()) ||
        !ensure_dynamic_smem(reinterpret_cast<const void *>(&pack_bf16_nf5_b32_bulk_kernel<2>), smem_bytes<2>()))
        return AXS6_ERR_LAUNCH;
    const cudaError_t le = hdr == 1 ? launch_overlapped(nblocks <= kOverlapBlocks, pack_bf16_nf5_b32_bulk_kernel<1>, (unsigned)ctas, kFastBlocks, smem_bytes<1>(), st, map, o, nblocks)
                                    : launch_overlapped(nblocks <= kOverlapBlocks, pack_bf16_nf5_b32_bulk_kernel<2>, (unsigned)ctas, kFastBlocks, smem_bytes<2>(), st, map, o, nblocks);
    count_launch();
    return le == cudaSuccess ? check_launch() : AXS6_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------ fp32 pack, TMA-fed
// fp32 input, NF5 grid, nearest rounding, block 32, byte records: the data movement of the bf16 kernel
// above (tiles of 256 blocks x 128 bytes through a tensor map with the 128-byte swizzle, records out
// with one bulk copy), the arithmetic of the general kernel (axs6_scale_codes and the exact index
// formulas), one thread per block.
constexpr int kF32Tile = kFastBlocks * 128;

template <int HDR>
constexpr int pack_f32_smem_bytes() { return 1024 + kCtrlBytes + kStages * kF32Tile + 2 * kFastBlocks * (HDR + 24); }

template <int HDR>
__global__ void __launch_bounds__(kFastBlocks) pack_f32_nf5_b32_bulk_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                           uint8_t *__restrict__ out, int64_t nblocks)
{
    constexpr int REC = HDR + 24;
    constexpr int kOut = kFastBlocks * REC;
    extern __shared__ uint8_t raw[];
    __shared__ __align__(16) uint8_t rev[1024];
    uint8_t *base = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
    uint8_t *in0 = base + kCtrlBytes;
    uint8_t *out0 = in0 + kStages * kF32Tile;
    const uint32_t bar0 = smem_u32(base);
    const int tid = threadIdx.x;
    pdl_launch_dependents();                               // the next launch may take up residence now (it waits in pdl_wait)
    const int64_t groups = (nblocks + kFastBlocks - 1) / kFastBlocks;
    const int64_t nk = (int64_t)blockIdx.x < groups ? (groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    build_reverse_lut(rev);                                 // module constants: may run while the previous kernel drains
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8 * s, 1);
        fence_barrier_init();
        fence_async_smem();
        pdl_wait();                                        // caller memory is read from here on
        for (int k = 0; k < kStages && k < nk; ++k) {
            mbar_expect_tx(bar0 + 8 * k, kF32Tile);
            tma_load_2d(smem_u32(in0 + k * kF32Tile), &xmap, bar0 + 8 * k, 0,
                        (int)(((int64_t)blockIdx.x + k * (int64_t)gridDim.x) * kFastBlocks));
        }
    }
    __syncthreads();
    pdl_wait();
    uint32_t piece[8];                       // row tid, 16-byte piece i at piece i ^ (row & 7)
#pragma unroll
    for (int i = 0; i < 8; ++i) piece[i] = (uint32_t)tid * 128u + (uint32_t)((i ^ (tid & 7)) << 4);
    const uint32_t wb = (uint32_t)(REC * tid) >> 2, sh = (uint32_t)(REC * tid) & 3u;
    const uint32_t sft = 8u * (sh + HDR);
    const bool owns_first = sh == 0u;
    const bool takes_next = ((uint32_t)(REC * (tid + 1)) & 3u) != 0u;

    int s = 0;
    uint32_t ph = 0;
    for (int64_t k = 0; k < nk; ++k) {
        const int64_t grp = (int64_t)blockIdx.x + k * (int64_t)gridDim.x;
        const int64_t b = grp * kFastBlocks + tid;
        uint8_t *ost = out0 + (k & 1) * kOut;
        const bool ok = mbar_wait_bounded(bar0 + 8 * s, ph, 3, &g_codec_status, kWaitLimit);
        uint32_t W[7];
#pragma unroll
        for (int i = 0; i < 7; ++i) W[i] = 0u;
        if (ok && b < nblocks) {
            uint32_t v[32];
            const uint8_t *tile = in0 + s * kF32Tile;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 q = *reinterpret_cast<const uint4 *>(tile + piece[i]);
                v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
            }
            uint32_t amax = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i) amax = max(amax, v[i] & 0x7FFFFFFFu);
            const Axs6Scale sc = axs6_scale_codes(amax);
            uint32_t pay[6];
#pragma unroll
            for (int i = 0; i < 6; ++i) pay[i] = 0u;
            if (sc.fast) {
                const float c = AXS6_MUL(sc.inv, 1023.0f);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float x = __uint_as_float(v[i]);
                    const uint32_t code = (uint32_t)rev[axs6_nf5_index_fast(fabsf(x), c)] | (x < 0.0f ? 32u : 0u);
                    const int word = (6 * i) >> 5, off = (6 * i) & 31;
                    pay[word] |= code << off;
                    if (off > 26) pay[word + 1] |= code >> (32 - off);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const uint32_t ab = v[i] & 0x7FFFFFFFu;
                    const int idx = axs6_nf5_index(axs6_normalise(__uint_as_float(ab), sc));
                    const uint32_t code = (uint32_t)rev[idx] | ((ab != 0u && (v[i] >> 31)) ? 32u : 0u);
                    const int word = (6 * i) >> 5, off = (6 * i) & 31;
                    pay[word] |= code << off;
                    if (off > 26) pay[word + 1] |= code >> (32 - off);
                }
            }
            record_words<HDR>(pay, (uint32_t)sc.se, sft, W);
        }
        const uint32_t nxt = __shfl_down_sync(0xFFFFFFFFu, W[0], 1);
        if (takes_next) W[6] |= nxt;
        uint32_t *o32 = reinterpret_cast<uint32_t *>(ost) + wb;
        if (owns_first) o32[0] = W[0];
#pragma unroll
        for (int i = 1; i < 7; ++i) o32[i] = W[i];
        fence_async_smem();
        if (tid == 0) bulk_wait_read<0>();
        if (__syncthreads_or(!ok)) {
            if (tid == 0) drain_ring(bar0, kStages, s, ph, (int)(nk - k < kStages ? nk - k : kStages), kWaitLimit);
            break;
        }
        const int64_t nb = nblocks - grp * kFastBlocks;
        if (nb >= kFastBlocks) {
            if (tid == 0) {
                bulk_store(out + grp * kOut, smem_u32(ost), kOut);
                bulk_commit();
            }
        } else {
            const int len = (int)nb * REC;
            uint8_t *dst = out + grp * kOut;
            const int nvec = len >> 4;
            for (int i = tid; i < nvec; i += kFastBlocks)
                st_stream16(dst + 16 * i, reinterpret_cast<const uint4 *>(ost)[i]);
            for (int i = (nvec << 4) + tid; i < len; i += kFastBlocks) dst[i] = ost[i];
        }
        if (tid == 0 && k + kStages < nk) {
            mbar_expect_tx(bar0 + 8 * s, kF32Tile);
            tma_load_2d(smem_u32(in0 + s * kF32Tile), &xmap, bar0 + 8 * s, 0,
                        (int)(((int64_t)blockIdx.x + (k + kStages) * (int64_t)gridDim.x) * kFastBlocks));
        }
        if (++s == kStages) { s = 0; ph ^= 1u; }
    }
    if (tid == 0) bulk_wait<0>();
}

// -> status, or 1 when this path does not apply
static int launch_pack_f32_bulk(const void *x, void *out, int64_t nblocks, int hdr, cudaStream_t st)
{
    if (nblocks >= (1ll << 31) - kFastBlocks) return 1;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return 1;
    CUtensorMap map;
    const cuuint64_t gdim[2] = {32, (cuuint64_t)nblocks};
    const cuuint64_t gstride[1] = {128};
    const cuuint32_t box[2] = {32, (cuuint32_t)kFastBlocks};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(x), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return 1;
    const DeviceInfo &d = device_info();
    int64_t ctas = (nblocks + kFastBlocks - 1) / kFastBlocks;
    const int64_t cap = tune_value(1);
    int per_sm = 2;
    if (cap > 0 && cap < per_sm) per_sm = (int)cap;
    if (ctas > (int64_t)d.sms * per_sm) ctas = (int64_t)d.sms * per_sm;
    if (ctas < 1) ctas = 1;
    if (!ensure_dynamic_smem(reinterpret_cast<const void *>(&pack_f32_nf5_b32_bulk_kernel<1>), pack_f32_smem_bytes<1>()) ||
        !ensure_dynamic_smem(reinterpret_cast<const void *>(&pack_f32_nf5_b32_bulk_kernel<2>), pack_f32_smem_bytes<2>()))
        return AXS6_ERR_LAUNCH;
    uint8_t *o = static_cast<uint8_t *>(out);
    const cudaError_t le = hdr == 1 ? launch_overlapped(nblocks <= kOverlapBlocks, pack_f32_nf5_b32_bulk_kernel<1>, (unsigned)ctas, kFastBlocks, pack_f32_smem_bytes<1>(), st, map, o, nblocks)
                                    : launch_overlapped(nblocks <= kOverlapBlocks, pack_f32_nf5_b32_bulk_kernel<2>, (unsigned)ctas, kFastBlocks, pack_f32_smem_bytes<2>(), st, map, o, nblocks);
    count_launch();
    return le == cudaSuccess ? check_launch() : AXS6_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------ unpack, TMA-fed
// Records (NF5 grid, block 32, byte layouts) -> bf16 or fp32 values, one thread per block.  The 256
// records of an iteration arrive with one bulk copy; a thread reads its 25 or 26 bytes as seven words
// and funnel-shifts them into the exponent byte and the 192-bit payload.  A value is then ONE table
// lookup and one integer addition: the table holds, for each 6-bit code, the sign and the level's bit
// pattern with its exponent field lowered by 120, and adding (se - 7) to the exponent field multiplies
// by 2^(se - 127) exactly (taken for se in [8, 254], where every result is a normal number; other
// blocks use the fp32 product of the general kernel).  bf16 results are rounded once, in the table:
// rounding commutes with the power-of-two scale.  The output tile leaves through a tensor map with
// the swizzle that makes the 128-bit shared-memory stores of a thread conflict-free.
template <typename Tout>
struct UnpackOut;
template <>
struct UnpackOut<__nv_bfloat16> { static constexpr int kRowBytes = 64, kPieces = 4, kSwzMask = 3, kSwzShift = 1; };
template <>
struct UnpackOut<float> { static constexpr int kRowBytes = 128, kPieces = 8, kSwzMask = 7, kSwzShift = 0; };

template <typename Tout, int HDR>
constexpr int unpack_smem_bytes() { return 1024 + kCtrlBytes + 2 * kFastBlocks * UnpackOut<Tout>::kRowBytes + kStages * kFastBlocks * (HDR + 24); }

template <typename Tout, int HDR, bool kLane>
__global__ void __launch_bounds__(kFastBlocks) unpack_nf5_b32_bulk_kernel(const __grid_constant__ CUtensorMap ymap,
                                                                         const uint8_t *__restrict__ in, int64_t nblocks)
{
    constexpr bool kBf16 = sizeof(Tout) == 2;
    constexpr int REC = HDR + 24;
    constexpr int kIn = kFastBlocks * REC;
    constexpr int kTile = kFastBlocks * UnpackOut<Tout>::kRowBytes;
    constexpr int kPieces = UnpackOut<Tout>::kPieces;
    extern __shared__ uint8_t raw[];
    // code -> value bits (bf16: in the low half), one copy per lane: entry (code, lane) is word code * 32 + lane, so a
    // warp's 32 lookups always hit 32 different banks (with one shared copy the codes of a warp collide about three
    // deep, and the lookups, not DRAM, bounded the kernel)
    // (kLane: bf16 output of up to 64 Mi values, where it is worth 10 %; for larger launches, which are bound by
    // instruction issue, and for fp32 output the single shared copy is 2-4 % faster)
    constexpr int kCopies = kLane ? 32 : 1;
    constexpr int kCodeShift = kLane ? 7 : 2;       // byte offset of an entry = code << kCodeShift (+ lane * 4)
    __shared__ __align__(128) uint32_t tlo[64 * kCopies];
    __shared__ float lev[32];
    uint8_t *base = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
    uint8_t *tile0 = base + kCtrlBytes;             // 1024-aligned output tiles
    uint8_t *in0 = tile0 + 2 * kTile;
    const uint32_t bar0 = smem_u32(base);
    const int tid = threadIdx.x;
    pdl_launch_dependents();                               // the next launch may take up residence now (it waits in pdl_wait)
    const int64_t groups = (nblocks + kFastBlocks - 1) / kFastBlocks;
    const int64_t nk = (int64_t)blockIdx.x < groups ? (groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    for (int i = tid; i < 64 * kCopies; i += kFastBlocks) {
        const uint32_t code = (uint32_t)i / kCopies;
        const uint32_t bits = g_codebook_bits[code & 31u];
        const uint32_t sign = code >> 5;
        tlo[i] = kBf16 ? (((uint32_t)axs6_f32_to_bf16_bits(__uint_as_float(bits)) - (120u << 7)) | (sign << 15))
                       : ((bits - (120u << 23)) | (sign << 31));
    }
    if (tid < 32) lev[tid] = __uint_as_float(g_codebook_bits[tid]);
    const uint32_t lane4 = kLane ? ((uint32_t)tid & 31u) << 2 : 0u;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8 * s, 1);
        fence_barrier_init();
        fence_async_smem();
        pdl_wait();                                        // caller memory is read from here on
        // a group with fewer than 256 records (the last one) is fetched by the threads themselves
        for (int k = 0; k < kStages && k < nk; ++k) {
            const int64_t grp = (int64_t)blockIdx.x + k * (int64_t)gridDim.x;
            if (nblocks - grp * kFastBlocks >= kFastBlocks) {
                mbar_expect_tx(bar0 + 8 * k, kIn);
                bulk_load(smem_u32(in0 + k * kIn), in + grp * kIn, kIn, bar0 + 8 * k);
            }
        }
    }
    __syncthreads();
    pdl_wait();

    const uint32_t wb = (uint32_t)(REC * tid) >> 2, sh = (uint32_t)(REC * tid) & 3u;
    const uint32_t sft = 8u * (sh + HDR);
    uint32_t piece[kPieces];
#pragma unroll
    for (int i = 0; i < kPieces; ++i)
        piece[i] = (uint32_t)tid * UnpackOut<Tout>::kRowBytes +
                   (uint32_t)((i ^ ((tid >> UnpackOut<Tout>::kSwzShift) & UnpackOut<Tout>::kSwzMask)) << 4);

    int s = 0;
    uint32_t ph = 0;
    for (int64_t k = 0; k < nk; ++k) {
        const int64_t grp = (int64_t)blockIdx.x + k * (int64_t)gridDim.x;
        const int64_t b = grp * kFastBlocks + tid;
        const int64_t nb = nblocks - grp * kFastBlocks;
        uint8_t *tile = tile0 + (k & 1) * kTile;
        const uint8_t *stage = in0 + s * kIn;
        bool ok = true;
        if (nb >= kFastBlocks) {
            ok = mbar_wait_bounded(bar0 + 8 * s, ph, 2, &g_codec_status, kWaitLimit);
        } else {
            const int len = (int)nb * REC;
            const uint8_t *src = in + grp * kIn;
            uint8_t *dst = in0 + s * kIn;
            for (int i = tid; i < len; i += kFastBlocks) dst[i] = src[i];
            __syncthreads();
        }
        if (ok && b < nblocks) {
            const uint32_t *r32 = reinterpret_cast<const uint32_t *>(stage) + wb;
            uint32_t W[7];
#pragma unroll
            for (int i = 0; i < 7; ++i) W[i] = r32[i];
            uint32_t pay[6];
#pragma unroll
            for (int i = 0; i < 6; ++i) pay[i] = __funnelshift_rc(W[i], W[i + 1], sft);
            const uint32_t head = W[0] >> (8u * sh);
            const uint32_t se = HDR == 1 ? (head & 0xFFu) : ((head >> 2) & 0xFFu);
            uint32_t o[kBf16 ? 16 : 32];
            if (se >= 8u && se <= 254u) {
                const uint32_t kk = kBf16 ? (se - 7u) * 0x00800080u : (se - 7u) << 23;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    uint32_t a[2];                      // byte offsets of the table entries of values i and i + 1
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int bit = 6 * (i + e), word = bit >> 5, off = bit & 31;
                        uint32_t v;                     // the code at bits kCodeShift .. kCodeShift + 5
                        if (off < kCodeShift) v = pay[word] << (kCodeShift - off);
                        else if (off == kCodeShift) v = pay[word];
                        else if (off <= 26) v = pay[word] >> (off - kCodeShift);
                        else v = __funnelshift_r(pay[word], pay[word + 1], off - kCodeShift);
                        a[e] = (v & (0x3Fu << kCodeShift)) | lane4;
                    }
                    const uint32_t v0 = *reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(tlo) + a[0]);
                    const uint32_t v1 = *reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(tlo) + a[1]);
                    if (kBf16) {
                        o[i >> 1] = (v1 << 16) + v0 + kk;
                    } else {
                        o[i] = v0 + kk;
                        o[i + 1] = v1 + kk;
                    }
                }
            } else {
                // all-zero blocks (se = 0) and blocks at the ends of the exponent range: fp32 product
                const float scale = axs6_scale_decode(se);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int bit = 6 * i, word = bit >> 5, off = bit & 31;
                    const uint32_t code = (off <= 26 ? (pay[word] >> off) : __funnelshift_r(pay[word], pay[word + 1], off)) & 63u;
                    const float y = axs6_decode_value(code >> 5, lev[code & 31u], scale);
                    if (kBf16) {
                        const uint32_t h = axs6_f32_to_bf16_bits(y);
                        if (i & 1) o[i >> 1] |= h << 16; else o[i >> 1] = h;
                    } else {
                        o[i] = __float_as_uint(y);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kPieces; ++i)
                *reinterpret_cast<uint4 *>(tile + piece[i]) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
        fence_async_smem();
        if (tid == 0) bulk_wait_read<0>();     // the previous iteration's store has left the other tile
        if (__syncthreads_or(!ok)) {
            if (tid == 0) {                    // wait for the record loads still armed (whole groups only)
                int ahead = 0;
                for (int j = 0; j < kStages && k + j < nk; ++j)
                    if (nblocks - (grp + j * (int64_t)gridDim.x) * kFastBlocks >= kFastBlocks) ahead = j + 1;
                drain_ring(bar0, kStages, s, ph, ahead, kWaitLimit);
            }
            break;
        }
        if (tid == 0) {
            tma_store_2d(&ymap, smem_u32(tile), 0, (int)(grp * kFastBlocks));
            bulk_commit();
            if (k + kStages < nk) {
                const int64_t g2 = grp + kStages * (int64_t)gridDim.x;
                if (nblocks - g2 * kFastBlocks >= kFastBlocks) {
                    mbar_expect_tx(bar0 + 8 * s, kIn);
                    bulk_load(smem_u32(in0 + s * kIn), in + g2 * kIn, kIn, bar0 + 8 * s);
                }
            }
        }
        if (++s == kStages) { s = 0; ph ^= 1u; }
    }
    if (tid == 0) bulk_wait<0>();
}

// -> status, or 1 when this path does not apply (the caller then uses unpack_vec_kernel)
template <typename Tout>
static int launch_unpack_bulk(const void *in, void *y, int64_t nblocks, int hdr, cudaStream_t st)
{
    if (nblocks >= (1ll << 31) - kFastBlocks) return 1;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return 1;
    constexpr bool kBf16 = sizeof(Tout) == 2;
    CUtensorMap map;
    const cuuint64_t gdim[2] = {32, (cuuint64_t)nblocks};
    const cuuint64_t gstride[1] = {32 * sizeof(Tout)};
    const cuuint32_t box[2] = {32, (cuuint32_t)kFastBlocks};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, kBf16 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, y, gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, kBf16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return 1;
    const DeviceInfo &d = device_info();
    int64_t ctas = (nblocks + kFastBlocks - 1) / kFastBlocks;
    const int64_t cap = tune_value(1);
    int per_sm = kBf16 ? 4 : 2;
    if (cap > 0 && cap < per_sm) per_sm = (int)cap;
    if (ctas > (int64_t)d.sms * per_sm) ctas = (int64_t)d.sms * per_sm;
    if (ctas < 1) ctas = 1;
    const uint8_t *src = static_cast<const uint8_t *>(in);
    const bool overlap = nblocks <= kOverlapBlocks;
    cudaError_t le = cudaErrorUnknown;
    auto go = [&](auto kernel, int smem) {
        if (!ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), smem)) return;
        le = launch_overlapped(overlap, kernel, (unsigned)ctas, kFastBlocks, (size_t)smem, st, map, src, nblocks);
    };
    const bool lane = kBf16 && nblocks <= kOverlapBlocks;      // per-lane code table (see the kernel)
    if (hdr == 1) {
        if (lane) go(unpack_nf5_b32_bulk_kernel<Tout, 1, true>, unpack_smem_bytes<Tout, 1>());
        else go(unpack_nf5_b32_bulk_kernel<Tout, 1, false>, unpack_smem_bytes<Tout, 1>());
    } else {
        if (lane) go(unpack_nf5_b32_bulk_kernel<Tout, 2, true>, unpack_smem_bytes<Tout, 2>());
        else go(unpack_nf5_b32_bulk_kernel<Tout, 2, false>, unpack_smem_bytes<Tout, 2>());
    }
    count_launch();
    return le == cudaSuccess ? check_launch() : AXS6_ERR_LAUNCH;
}

}  // namespace bulk

static bool layout_ok(int layout)
{
    return layout == AXS6_LAYOUT_PLANES || layout == AXS6_LAYOUT_WIRE || layout == AXS6_LAYOUT_SPEC || layout == AXS6_LAYOUT_SPLIT;
}

}  // namespace axs6

// ------------------------------------------------------------------------------------------ planes <-> records
// One thread per block: planes (exponent, sign, magnitude bytes) to a byte record or back, no
// arithmetic on values.  The counterpart of _pack_to_flat_buffer / _unpack_from_flat_buffer
// (axs/unified/distributed.py:147-232) and of AXSBlock.to_bytes / from_bytes (axs/core.py:97-152)
// for callers that already hold an AXSTensor.
namespace axs6 {

__global__ void __launch_bounds__(256) planes_to_records_kernel(const uint8_t *se, const uint8_t *sg, const uint8_t *mg,
                                                               uint8_t *out, int64_t nblocks, int B, int hdr)
{
    const int rec = hdr + B * 3 / 4;
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (int64_t)gridDim.x * blockDim.x) {
        uint8_t *r = out + b * rec;
        const uint32_t e = se[b];
        if (hdr == 1) {
            r[0] = (uint8_t)e;
        } else {
            r[0] = (uint8_t)((e << 2) & 0xFFu);
            r[1] = (uint8_t)(e >> 6);
        }
        for (int g = 0; g < B / 4; ++g) {
            uint32_t v = 0;
            for (int i = 0; i < 4; ++i) {
                const int64_t o = b * B + 4 * g + i;
                v |= (((uint32_t)(sg[o] & 1u) << 5) | (uint32_t)(mg[o] & 31u)) << (6 * i);
            }
            r[hdr + 3 * g] = (uint8_t)v; r[hdr + 3 * g + 1] = (uint8_t)(v >> 8); r[hdr + 3 * g + 2] = (uint8_t)(v >> 16);
        }
    }
}

__global__ void __launch_bounds__(256) records_to_planes_kernel(const uint8_t *in, uint8_t *se, uint8_t *sg, uint8_t *mg,
                                                               int64_t nblocks, int B, int hdr)
{
    const int rec = hdr + B * 3 / 4;
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (int64_t)gridDim.x * blockDim.x) {
        const uint8_t *r = in + b * rec;
        se[b] = (hdr == 1) ? r[0] : (uint8_t)((((uint32_t)r[0] | ((uint32_t)r[1] << 8)) >> 2) & 0xFFu);
        for (int g = 0; g < B / 4; ++g) {
            const uint32_t v = (uint32_t)r[hdr + 3 * g] | ((uint32_t)r[hdr + 3 * g + 1] << 8) | ((uint32_t)r[hdr + 3 * g + 2] << 16);
            for (int i = 0; i < 4; ++i) {
                const uint32_t code = (v >> (6 * i)) & 63u;
                sg[b * B + 4 * g + i] = (uint8_t)(code >> 5);
                mg[b * B + 4 * g + i] = (uint8_t)(code & 31u);
            }
        }
    }
}

}  // namespace axs6

AXS6_API int axs6_repack(int to_records, int layout, int block, int64_t nblocks, void *exponents, void *signs,
                         void *magnitudes, void *records, axs6_stream_t stream)
{
    using namespace axs6;
    if (!valid_block(block) || (layout != AXS6_LAYOUT_WIRE && layout != AXS6_LAYOUT_SPEC) || nblocks < 0) return AXS6_ERR_ARG;
    if (nblocks == 0) return AXS6_OK;
    if (!exponents || !signs || !magnitudes || !records) return AXS6_ERR_ARG;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;
    int64_t ctas = (nblocks + 255) / 256;
    if (ctas > (int64_t)d.sms * 8) ctas = (int64_t)d.sms * 8;
    const int hdr = layout == AXS6_LAYOUT_SPEC ? 2 : 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (to_records)
        planes_to_records_kernel<<<(unsigned)ctas, 256, 0, st>>>(static_cast<const uint8_t *>(exponents), static_cast<const uint8_t *>(signs),
                                                                 static_cast<const uint8_t *>(magnitudes), static_cast<uint8_t *>(records), nblocks, block, hdr);
    else
        records_to_planes_kernel<<<(unsigned)ctas, 256, 0, st>>>(static_cast<const uint8_t *>(records), static_cast<uint8_t *>(exponents),
                                                                 static_cast<uint8_t *>(signs), static_cast<uint8_t *>(magnitudes), nblocks, block, hdr);
    count_launch();
    return check_launch();
}

AXS6_API int64_t axs6_record_bytes(int layout, int block)
{
    if (!axs6::valid_block(block)) return 0;
    if (layout == AXS6_LAYOUT_WIRE) return 1 + block * 3 / 4;
    if (layout == AXS6_LAYOUT_SPEC) return 2 + block * 3 / 4;
    if (layout == AXS6_LAYOUT_SPLIT) return block * 3 / 4;          // payload only; the exponent lives in its own plane
    return 0;
}

AXS6_API int axs6_pack_ef(const float *x, float *err, int64_t rows, int64_t cols, int64_t ld, int block, int grid,
                          int rounding, uint64_t seed, uint64_t offset, void *out_exp, void *out_sign, void *out_mag,
                          axs6_stream_t stream)
{
    using namespace axs6;
    if (!valid_block(block) || (grid != AXS6_GRID_NF5 && grid != AXS6_GRID_UNIFORM)) return AXS6_ERR_ARG;
    if (rounding != AXS6_ROUND_NEAREST && rounding != AXS6_ROUND_STOCHASTIC) return AXS6_ERR_ARG;
    if (rows < 0 || cols < 0 || ld < cols) return AXS6_ERR_ARG;
    if (rows == 0 || cols == 0) return AXS6_OK;
    if (!x || !err || !out_exp || !out_sign || !out_mag) return AXS6_ERR_ARG;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;
    if (!(aligned16(x) && aligned16(err) && cols % kChunk == 0 && ld % kChunk == 0 && aligned16(out_exp) && aligned16(out_sign) &&
          aligned16(out_mag)))
        return AXS6_ERR_UNSUPPORTED;      // the caller composes the steps from axs6_pack / axs6_unpack instead
    CodecArgs a;
    a.x = x; a.y = nullptr; a.ld = ld; a.err = err;
    a.g = make_geom(rows, cols, block);
    a.g.flat = (cols % block == 0 && ld == cols) ? 1 : 0;
    a.via_bf16 = 0u;
    a.seed = seed; a.offset = offset; a.noise = nullptr;
    a.keys = axs6_philox_keys(seed);
    a.epoch = philox_epoch_ptr();
    const bool stochastic = rounding == AXS6_ROUND_STOCHASTIC;
    if (stochastic && !a.epoch) return AXS6_ERR_DEVICE;
    a.p0 = static_cast<uint8_t *>(out_exp); a.p1 = static_cast<uint8_t *>(out_sign); a.p2 = static_cast<uint8_t *>(out_mag);
    a.rec = 0; a.hdr = 0;
    a.lanes_log2 = block == 32 ? 2 : (block == 16 ? 1 : 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t per_cta = (int64_t)kThreads * kU;
    if (grid == AXS6_GRID_UNIFORM)
        return stochastic ? launch_codec(pack_vec_kernel<float, AXS6_GRID_UNIFORM, kPhilox, kPlanes, true>, a, per_cta, a.g.total_chunks, st)
                          : launch_codec(pack_vec_kernel<float, AXS6_GRID_UNIFORM, kNearest, kPlanes, true>, a, per_cta, a.g.total_chunks, st);
    return stochastic ? launch_codec(pack_vec_kernel<float, AXS6_GRID_NF5, kPhilox, kPlanes, true>, a, per_cta, a.g.total_chunks, st)
                      : launch_codec(pack_vec_kernel<float, AXS6_GRID_NF5, kNearest, kPlanes, true>, a, per_cta, a.g.total_chunks, st);
}

AXS6_API int axs6_pack(const void *x, int in_dtype, int64_t rows, int64_t cols, int64_t ldx, int block, int grid,
                         int rounding, uint32_t flags, uint64_t seed, uint64_t offset, const float *noise,
                         int layout, void *out0, void *out1, void *out2, axs6_stream_t stream)
{
    using namespace axs6;
    if (!valid_dtype(in_dtype) || !valid_block(block) || !layout_ok(layout)) return AXS6_ERR_ARG;
    if (grid != AXS6_GRID_NF5 && grid != AXS6_GRID_UNIFORM) return AXS6_ERR_ARG;
    if (rounding != AXS6_ROUND_NEAREST && rounding != AXS6_ROUND_STOCHASTIC) return AXS6_ERR_ARG;
    if (rows < 0 || cols < 0 || ldx < cols) return AXS6_ERR_ARG;
    if (flags & ~AXS6_FLAG_INPUT_VIA_BF16) return AXS6_ERR_ARG;
    if (rows == 0 || cols == 0) return AXS6_OK;
    const bool planes = layout == AXS6_LAYOUT_PLANES;
    const bool split = layout == AXS6_LAYOUT_SPLIT;
    if (!x || !out0 || (planes && (!out1 || !out2)) || (split && !out1)) return AXS6_ERR_ARG;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;

    const int round = rounding == AXS6_ROUND_NEAREST ? kNearest : (noise ? kNoise : kPhilox);
    CodecArgs a;
    a.x = x; a.y = nullptr; a.ld = ldx; a.err = nullptr;
    a.g = make_geom(rows, cols, block);
    a.g.flat = (cols % block == 0 && ldx == cols) ? 1 : 0;
    a.via_bf16 = (flags & AXS6_FLAG_INPUT_VIA_BF16) ? 1u : 0u;
    a.seed = seed; a.offset = offset; a.noise = noise;
    a.keys = axs6_philox_keys(seed);
    a.epoch = philox_epoch_ptr();
    if (round == kPhilox && !a.epoch) return AXS6_ERR_DEVICE;
    a.p0 = static_cast<uint8_t *>(out0); a.p1 = static_cast<uint8_t *>(out1); a.p2 = static_cast<uint8_t *>(out2);
    a.rec = (int)axs6_record_bytes(layout, block);
    a.hdr = layout == AXS6_LAYOUT_SPEC ? 2 : (split ? 0 : 1);
    a.lanes_log2 = block == 32 ? 2 : (block == 16 ? 1 : 0);
    const bool vec = aligned16(x) && (cols % kChunk == 0) && (ldx % kChunk == 0) && aligned16(out0) &&
                     (!planes || (aligned16(out1) && aligned16(out2))) && (round != kNoise || aligned16(noise));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (split)          // general kernels only
        return in_dtype == AXS6_F32 ? dispatch_pack<float>(a, grid, round, planes, vec, st)
                                    : dispatch_pack<__nv_bfloat16>(a, grid, round, planes, vec, st);
    if (vec && !planes && a.g.flat && in_dtype == AXS6_F32 && !a.via_bf16 && grid == AXS6_GRID_NF5 && round == kNearest &&
        block == 32 && tune_value(2) != 1) {
        const int r = bulk::launch_pack_f32_bulk(x, out0, rows * (cols / 32), a.hdr, st);
        if (r != 1) return r;
    }
    if (vec && !planes && a.g.flat && in_dtype == AXS6_BF16 && grid == AXS6_GRID_NF5 && round == kNearest && block == 32 &&
        tune_value(2) != 1) {
        // tune key 2: 1 = general kernel, 2 = per-thread loads (no TMA); default = TMA-fed kernel
        if (tune_value(2) != 2) {
            const int r = bulk::launch_pack_bulk(x, out0, rows * (cols / 32), a.hdr, st);
            if (r != 1) return r;
        }
        return launch_pack_fast(x, out0, rows * (cols / 32), a.hdr, st);
    }
    return in_dtype == AXS6_F32 ? dispatch_pack<float>(a, grid, round, planes, vec, st)
                                : dispatch_pack<__nv_bfloat16>(a, grid, round, planes, vec, st);
}

AXS6_API int axs6_unpack(int layout, const void *in0, const void *in1, const void *in2, void *y, int out_dtype,
                           int64_t rows, int64_t cols, int64_t ldy, int block, int grid, axs6_stream_t stream)
{
    using namespace axs6;
    if (!valid_dtype(out_dtype) || !valid_block(block) || !layout_ok(layout)) return AXS6_ERR_ARG;
    if (grid != AXS6_GRID_NF5 && grid != AXS6_GRID_UNIFORM) return AXS6_ERR_ARG;
    if (rows < 0 || cols < 0 || ldy < cols) return AXS6_ERR_ARG;
    if (rows == 0 || cols == 0) return AXS6_OK;
    const bool planes = layout == AXS6_LAYOUT_PLANES;
    const bool split = layout == AXS6_LAYOUT_SPLIT;
    if (!y || !in0 || (planes && (!in1 || !in2)) || (split && !in1)) return AXS6_ERR_ARG;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;

    CodecArgs a;
    a.x = nullptr; a.y = y; a.ld = ldy; a.err = nullptr;
    a.g = make_geom(rows, cols, block);
    a.g.flat = (cols % block == 0 && ldy == cols) ? 1 : 0;
    a.via_bf16 = 0; a.seed = 0; a.offset = 0; a.noise = nullptr; a.epoch = nullptr;
    a.keys = axs6_philox_keys(0);
    a.p0 = const_cast<uint8_t *>(static_cast<const uint8_t *>(in0));
    a.p1 = const_cast<uint8_t *>(static_cast<const uint8_t *>(in1));
    a.p2 = const_cast<uint8_t *>(static_cast<const uint8_t *>(in2));
    a.rec = (int)axs6_record_bytes(layout, block);
    a.hdr = layout == AXS6_LAYOUT_SPEC ? 2 : (split ? 0 : 1);
    a.lanes_log2 = block == 32 ? 2 : (block == 16 ? 1 : 0);
    const bool vec = aligned16(y) && (cols % kChunk == 0) && (ldy % kChunk == 0) && aligned16(in0) &&
                     (!planes || (aligned16(in1) && aligned16(in2)));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // tune key 11: 1 = general kernel only
    if (vec && !planes && !split && a.g.flat && grid == AXS6_GRID_NF5 && block == 32 && tune_value(11) != 1) {
        const int r = out_dtype == AXS6_F32 ? bulk::launch_unpack_bulk<float>(in0, y, rows * (cols / 32), a.hdr, st)
                                            : bulk::launch_unpack_bulk<__nv_bfloat16>(in0, y, rows * (cols / 32), a.hdr, st);
        if (r != 1) return r;
    }
#define AXS6_CASE(T, G) return launch_unpack<T, G>(a, planes, vec, st)
    if (out_dtype == AXS6_F32) { if (grid == AXS6_GRID_NF5) AXS6_CASE(float, AXS6_GRID_NF5); AXS6_CASE(float, AXS6_GRID_UNIFORM); }
    if (grid == AXS6_GRID_NF5) AXS6_CASE(__nv_bfloat16, AXS6_GRID_NF5);
    AXS6_CASE(__nv_bfloat16, AXS6_GRID_UNIFORM);
#undef AXS6_CASE
}

namespace axs6 {
int exchange_status_fetch();     // exchange.cu
int fq_status_fetch();           // fq.cu
}

AXS6_API int axs6_codec_status(void)
{
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, axs6::bulk::g_codec_status, sizeof(int)) != cudaSuccess) return AXS6_ERR_DEVICE;
    // Only the word that is reported is cleared: a second failure recorded in another word stays for the next call.
    if (v != 0) {
        cudaMemcpyToSymbol(axs6::bulk::g_codec_status, &zero, sizeof(int));
        return v;
    }
    const int x = axs6::exchange_status_fetch();
    if (x != 0) return x < 0 ? x : 10 + x;
    const int q = axs6::fq_status_fetch();
    if (q != 0) return q < 0 ? q : 20 + q;
    return 0;
}
