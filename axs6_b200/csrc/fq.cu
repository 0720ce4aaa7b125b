// Fake-quantise kernels (NF5 and uniform grid) and their C entry points.
//
// One pass over HBM: every value is read once and written once.  Roofline: HBM bandwidth,
// algorithmic bytes per value = sizeof(in) + sizeof(out).
//   fq_vec_kernel      16-byte aligned tensors whose extents are multiples of 8 values: one
//                      thread owns 8 consecutive values (128-bit streaming loads/stores), the
//                      block amax is a 0..2-step xor shuffle, the NF5 reconstruction is one
//                      gather from a 4 KB shared-memory LUT.  Persistent grid sized from the
//                      occupancy of the instantiation, U independent chunks per thread in flight.
//   fq_generic_kernel  any pointer alignment / extent: one lane per value, coalesced scalar
//                      accesses, amax over B lanes.
#include "async_copy.cuh"
#include "quant_device.cuh"

namespace axs6 {

struct FqArgs {
    const void *x;
    void *y;
    int64_t ldx, ldy;
    ChunkGeom g;
    uint32_t via_bf16;
    uint32_t out_tf32;       // round fp32 results to the nearest TF32 value
    uint64_t seed, offset;
    Axs6PhiloxKeys keys;               // round keys of `seed`
    const unsigned long long *epoch;   // device counter added to `offset` (stochastic kernels only)
    const float *noise;
    const long long *row_index;        // gather: input row r is row row_index[r] of x (null: row r)
    long long table_rows;              // gather: rows of x; an index outside [0, table_rows) reads row 0 and sets the status word
};

// Nearest TF32 value (10-bit mantissa, ties away from zero), returned as fp32.
__device__ __forceinline__ float round_tf32(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

__device__ int g_gather_status;        // 1 = axs6_fq_gather met an index outside the table (that row read row 0 instead)

template <int GRID, int ROUND>
__device__ __forceinline__ void fq_chunk(const uint32_t (&v)[8], float (&y)[8], const float *tab,
                                         int lanes, const float (&u)[8])
{
    const uint32_t amax = group_max(chunk_amax_bits(v), lanes);
    if (GRID == AXS6_GRID_NF5) {
        const Axs6Scale s = axs6_scale_fq(amax);
        if (s.fast) {
            // block scale in the normal range (all but pathological blocks): two products,
            // one conversion and one LUT gather per value
            const float c = AXS6_MUL(s.inv, 1023.0f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float x = __uint_as_float(v[i]);
                const int idx = (ROUND == kNearest) ? axs6_nf5_index_fast(fabsf(x), c)
                              : (ROUND == kPhilox) ? axs6_nf5_index_dithered_fast(fabsf(x), c, u[i])
                                                   : axs6_nf5_index_dithered(AXS6_MUL(fabsf(x), s.inv), u[i]);
                y[i] = axs6_fq_value_fast(x, tab[idx], s.scale);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float n = axs6_normalise(__uint_as_float(v[i] & 0x7FFFFFFFu), s);
                const int idx = (ROUND == kNearest) ? axs6_nf5_index(n) : axs6_nf5_index_dithered(n, u[i]);
                y[i] = axs6_fq_value(v[i], tab[idx], s.scale);
            }
        }
    } else {
        const Axs6Scale s = axs6_scale_codes(amax);
        if (s.fast) {
            const float c = AXS6_MUL(s.inv, 31.0f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float x = __uint_as_float(v[i]);
                const int m = (ROUND == kNearest) ? axs6_uniform_mag_fast(fabsf(x), c)
                                                  : axs6_uniform_mag_stochastic(AXS6_MUL(fabsf(x), s.inv), u[i]);
                y[i] = axs6_decode_value(x < 0.0f ? 1u : 0u, tab[m], s.scale);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t ab = v[i] & 0x7FFFFFFFu;
                const float n = axs6_normalise(__uint_as_float(ab), s);
                const int m = (ROUND == kNearest) ? axs6_uniform_mag(n) : axs6_uniform_mag_stochastic(n, u[i]);
                y[i] = axs6_decode_value((ab != 0u) ? (v[i] >> 31) : 0u, tab[m], s.scale);
            }
        }
    }
}

template <typename Tin, typename Tout, int GRID, int ROUND, int U>
__global__ void __launch_bounds__(kThreads) fq_vec_kernel(const FqArgs a)
{
    __shared__ __align__(16) float tab[GRID == AXS6_GRID_NF5 ? 1024 : 32];
    if (GRID == AXS6_GRID_NF5) build_value_lut(tab); else build_levels<GRID>(tab);
    __syncthreads();
    pdl_wait();                    // nothing of the caller's memory is touched before this point

    const int lanes = a.g.block / kChunk;
    const uint64_t offset = (ROUND == kPhilox) ? a.offset + *a.epoch : 0ull;
    const int64_t step = (int64_t)gridDim.x * kThreads * U;
    for (int64_t base = (int64_t)blockIdx.x * kThreads * U; base < a.g.total_chunks; base += step) {
        if (base + step >= a.g.total_chunks) pdl_launch_dependents();      // last iteration of this CTA: the next kernel may move in
        uint32_t v[U][8];
        int64_t yo[U], cidx[U];
        bool act[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const int64_t c = base + (int64_t)k * kThreads + threadIdx.x;
            cidx[k] = c;
            act[k] = c < a.g.total_chunks;
            int64_t xo = c * kChunk;
            yo[k] = xo;
            if (!a.g.flat) {
                const int64_t row = c / a.g.cpr;
                const int64_t col0 = (c - row * a.g.cpr) * kChunk;
                act[k] = act[k] && col0 < a.g.cols;
                int64_t src = row;
                if (a.row_index && act[k]) {
                    src = a.row_index[row];
                    if (src < 0 || src >= a.table_rows) { src = 0; g_gather_status = 1; }
                }
                xo = src * a.ldx + col0;
                yo[k] = row * a.ldy + col0;
            }
            if (act[k]) {
                ChunkIO<Tin>::load(a.x, xo, v[k], a.via_bf16 != 0u);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[k][i] = 0u;
            }
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            float u[8], y[8];
            chunk_uniforms<ROUND>(u, cidx[k], act[k], a.keys, offset, a.noise);
            fq_chunk<GRID, ROUND>(v[k], y, tab, lanes, u);
            if (sizeof(Tout) == 4 && a.out_tf32) {
#pragma unroll
                for (int i = 0; i < 8; ++i) y[i] = round_tf32(y[i]);
            }
            if (act[k]) ChunkIO<Tout>::store(a.y, yo[k], y);
        }
    }
}

// One lane per value of the zero-padded row; a warp covers 32 consecutive padded columns.
template <typename Tin, typename Tout, int GRID, int ROUND>
__global__ void __launch_bounds__(kThreads) fq_generic_kernel(const FqArgs a)
{
    __shared__ __align__(16) float tab[GRID == AXS6_GRID_NF5 ? 1024 : 32];
    if (GRID == AXS6_GRID_NF5) build_value_lut(tab); else build_levels<GRID>(tab);
    __syncthreads();
    pdl_wait();

    const int lane = threadIdx.x & 31;
    const uint64_t offset = (ROUND == kPhilox) ? a.offset + *a.epoch : 0ull;
    const int64_t padded = a.g.cpr * kChunk;
    const int64_t tiles_per_row = (padded + 31) / 32;
    const int64_t tiles = a.g.rows * tiles_per_row;
    const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
    for (int64_t t = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); t < tiles; t += warps) {
        if (t + warps >= tiles) pdl_launch_dependents();
        const int64_t row = t / tiles_per_row;
        const int64_t pc = (t - row * tiles_per_row) * 32 + lane;
        const bool act = pc < a.g.cols;
        int64_t src = row;
        if (a.row_index && act) {
            src = a.row_index[row];
            if (src < 0 || src >= a.table_rows) { src = 0; g_gather_status = 1; }
        }
        const uint32_t v = act ? ChunkIO<Tin>::load1(a.x, src * a.ldx + pc, a.via_bf16 != 0u) : 0u;
        const uint32_t ab = v & 0x7FFFFFFFu;
        const uint32_t amax = group_max(ab, a.g.block);
        const float u = element_uniform<ROUND>(row * padded + pc, act, a.keys, offset, a.noise);
        float y;
        if (GRID == AXS6_GRID_NF5) {
            const Axs6Scale s = axs6_scale_fq(amax);
            const float n = axs6_normalise(__uint_as_float(ab), s);
            const int idx = (ROUND == kNearest) ? axs6_nf5_index(n)
                          : (ROUND == kPhilox && s.fast) ? axs6_nf5_index_dithered_fast(__uint_as_float(ab), AXS6_MUL(s.inv, 1023.0f), u)
                                                         : axs6_nf5_index_dithered(n, u);
            y = axs6_fq_value(v, tab[idx], s.scale);
        } else {
            const Axs6Scale s = axs6_scale_codes(amax);
            const float n = axs6_normalise(__uint_as_float(ab), s);
            const int m = (ROUND == kNearest) ? axs6_uniform_mag(n) : axs6_uniform_mag_stochastic(n, u);
            y = axs6_decode_value((ab != 0u) ? (v >> 31) : 0u, tab[m], s.scale);
        }
        if (sizeof(Tout) == 4 && a.out_tf32) y = round_tf32(y);
        if (act) ChunkIO<Tout>::store1(a.y, row * a.ldy + pc, y);
    }
}

// Launches of up to this many 8-value chunks (8 Mi values) ask for programmatic dependent launch: the small ones are
// bound by launch latency (1024 x 1024 fp32: 6.2 -> 4.8 us back to back; a 12-layer GPT step with 8192 x 1024
// activations: 25.2 -> 25.0 ms), while from 4096 x 4096 on the overlap costs 5-15 %.
constexpr int64_t kSmallLaunch = 1ll << 20;

// Persistent launch: at most `want_per_sm` CTAs per SM (0 = as many as fit).  Measured on B200:
// a streaming kernel is fastest with about 48 KB of loads in flight per SM; more resident
// CTAs than that lowers the achieved HBM bandwidth by up to 15 %.
template <typename K>
static int launch_persistent(K kernel, const FqArgs &a, int64_t work_items_per_cta, int64_t work_items,
                             int want_per_sm, cudaStream_t stream)
{
    const DeviceInfo &d = device_info();
    int per_sm = cached_occupancy(reinterpret_cast<const void *>(kernel), kThreads);
    if (per_sm < 1) return AXS6_ERR_LAUNCH;
    int64_t ctas = (work_items + work_items_per_cta - 1) / work_items_per_cta;
    const int64_t cap = tune_value(0) > 0 ? tune_value(0) : want_per_sm;
    if (cap > 0 && per_sm > cap) per_sm = (int)cap;
    const int64_t resident = (int64_t)d.sms * per_sm;
    if (ctas > resident) ctas = resident;
    if (ctas < 1) ctas = 1;
    const bool launched = launch_overlapped(work_items <= kSmallLaunch, kernel, (unsigned)ctas, kThreads, 0, stream, a) == cudaSuccess;
    count_launch();
    return launched ? check_launch() : AXS6_ERR_LAUNCH;
}

template <typename Tin, typename Tout, int GRID, int ROUND>
static int launch_fq(const FqArgs &a, bool vec, cudaStream_t stream)
{
    // Chunks per thread: two for fp32 input, one for bf16 input (that variant is bound by
    // instruction issue and wants warps rather than bytes per warp).  CTAs per SM: so that about
    // 96 KB of loads + stores are in flight per SM (3 CTAs for fp32 -> fp32, 4 for fp32 -> bf16,
    // every CTA that fits for bf16 input).
    constexpr int U = sizeof(Tin) == 4 ? 2 : 1;
    constexpr int kBytesPerCtaIter = (int)(sizeof(Tin) + sizeof(Tout)) * kChunk * kThreads * U;
    constexpr int kInFlight = (sizeof(Tin) == 4 ? 96 : 72) * 1024;      // measured optimum per SM
    constexpr int kWant = (kInFlight + kBytesPerCtaIter / 2) / kBytesPerCtaIter;
    if (vec)
        return launch_persistent(fq_vec_kernel<Tin, Tout, GRID, ROUND, U>, a, (int64_t)kThreads * U,
                                 a.g.total_chunks, kWant, stream);
    const int64_t tiles = a.g.rows * ((a.g.cpr * kChunk + 31) / 32);
    return launch_persistent(fq_generic_kernel<Tin, Tout, GRID, ROUND>, a, kThreads / 32, tiles, 0, stream);
}

template <typename Tin, typename Tout>
static int dispatch_fq(const FqArgs &a, int grid, int round, bool vec, cudaStream_t stream)
{
#define AXS6_CASE(G, R) \
    if (grid == G && round == R) return launch_fq<Tin, Tout, G, R>(a, vec, stream);
    AXS6_CASE(AXS6_GRID_NF5, kNearest)
    AXS6_CASE(AXS6_GRID_NF5, kPhilox)
    AXS6_CASE(AXS6_GRID_NF5, kNoise)
    AXS6_CASE(AXS6_GRID_UNIFORM, kNearest)
    AXS6_CASE(AXS6_GRID_UNIFORM, kPhilox)
    AXS6_CASE(AXS6_GRID_UNIFORM, kNoise)
#undef AXS6_CASE
    return AXS6_ERR_ARG;
}

ChunkGeom make_geom(int64_t rows, int64_t cols, int block)
{
    ChunkGeom g;
    g.rows = rows;
    g.cols = cols;
    g.block = block;
    const int64_t nblk = (cols + block - 1) / block;
    g.cpr = nblk * block / kChunk;
    g.total_chunks = rows * g.cpr;
    g.flat = 0;
    return g;
}

// ------------------------------------------------------------------------------------------ bf16 -> bf16, TMA-fed
// bf16 in, bf16 out, NF5 grid, block 32, contiguous and 16-byte aligned, nearest rounding or stochastic
// rounding with the library's own draws (the noise-supplied form stays with the general kernel): one thread per
// block, tiles of 256 blocks moved by the TMA unit in both directions and quantised IN PLACE in shared
// memory (a 3-slot ring: one slot being loaded, one computed, one stored).  The arithmetic is integer
// arithmetic on the bf16 bit patterns.  With E the exponent field of the block maximum the scale is
// S = 2^(E - 126) (the top-of-binade exponent bump of the fp32 path cannot occur: the low 16 mantissa
// bits are zero) and for a value (128 + m) * 2^(e - 134)
//     idx = trunc(|x| / S * 1023) = ((128 + m) * 1023) >> (8 + j),   j = E - e,   exactly,
// so the reconstruction level depends on key = ((E << 7) | 127) - |x|_bits only.  The table holds, per key,
// the level rounded to bf16 (rounding commutes with the power-of-two scale) with its exponent field lowered
// by 120; adding (E - 6) to the exponent field multiplies by S.  Taken for E in [11, 252] and for all-zero
// blocks; other blocks (denormal-range or near-overflow maxima) use the fp32 formulas of the general kernel.
namespace fqb {

using namespace acp;

constexpr int kBlocksB = 256;
constexpr int kSlots = 3;
constexpr int kSlotBytes = kBlocksB * 64;
constexpr int kKeyLim = 1280;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kSmemBytes = 1024 + 1024 + kSlots * kSlotBytes;

__device__ int g_fq_status;

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

// ROUND = kNearest: the integer path described above.  ROUND = kPhilox (stochastic rounding with the
// library's own draws; the round keys arrive as a kernel constant): the arithmetic of fq_vec_kernel, value by value -- same Philox block per 8 values,
// same fused multiply-add for the dithered index, same products -- so both kernels give the same bits.
template <int ROUND>
__global__ void __launch_bounds__(kBlocksB) fq_bf16_nf5_b32_bulk_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                       const __grid_constant__ CUtensorMap ymap, int64_t nblocks,
                                                                       uint64_t seed, uint64_t offset0,
                                                                       const unsigned long long *epoch,
                                                                       const __grid_constant__ Axs6PhiloxKeys keys)
{
    extern __shared__ uint8_t raw[];
    __shared__ __align__(16) uint16_t table[ROUND == kNearest ? kKeyLim + 8 : 8];   // key -> level bits (bf16), exponent field - 120
    __shared__ __align__(16) uint16_t lvl[ROUND == kNearest ? 8 : 1024];   // LUT index -> the same
    uint8_t *base = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
    uint8_t *slot0 = base + 1024;
    const uint32_t bar0 = smem_u32(base);
    const int tid = threadIdx.x;
    const int64_t groups = (nblocks + kBlocksB - 1) / kBlocksB;
    const int64_t nk = (int64_t)blockIdx.x < groups ? (groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    if (ROUND == kNearest) {
        for (int i = tid; i < (kKeyLim + 8) / 8; i += kBlocksB)
            reinterpret_cast<uint4 *>(table)[i] = reinterpret_cast<const uint4 *>(g_key_level_bf16)[i];
    } else {
        for (int i = tid; i < 1024 / 8; i += kBlocksB)
            reinterpret_cast<uint4 *>(lvl)[i] = reinterpret_cast<const uint4 *>(g_lut_level_bf16)[i];
    }
    if (tid == 0) {
        for (int s = 0; s < kSlots; ++s) mbar_init(bar0 + 8 * s, 1);
        fence_barrier_init();
        fence_async_smem();
        pdl_wait();                                            // the first loads of caller memory come after this
        for (int k = 0; k < 2 && k < nk; ++k) {                // two tiles ahead; the third slot is the one being stored
            mbar_expect_tx(bar0 + 8 * k, kSlotBytes);
            tma_load_2d(smem_u32(slot0 + k * kSlotBytes), &xmap, bar0 + 8 * k, 0,
                        (int)(((int64_t)blockIdx.x + k * (int64_t)gridDim.x) * kBlocksB));
        }
    }
    __syncthreads();
    pdl_wait();
    const uint64_t offset = ROUND == kPhilox ? offset0 + *epoch : 0ull;

    uint32_t piece[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) piece[i] = (uint32_t)tid * 64u + (uint32_t)((i ^ ((tid >> 1) & 3)) << 4);

    int s = 0;
    uint32_t ph = 0;
    for (int64_t k = 0; k < nk; ++k) {
        if (k + 1 == nk) pdl_launch_dependents();                             // last tile of this CTA: the next kernel may move in
        const int64_t grp = (int64_t)blockIdx.x + k * (int64_t)gridDim.x;
        const int64_t b = grp * kBlocksB + tid;
        uint8_t *slot = slot0 + s * kSlotBytes;
        const bool ok = mbar_wait_bounded(bar0 + 8 * s, ph, 1, &g_fq_status, kWaitLimit);
        if (ok && b < nblocks) {
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = *reinterpret_cast<const uint4 *>(slot + piece[i]);
                w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
            }
            uint32_t mx = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) mx = max_u16x2(mx, w[i] & 0x7FFF7FFFu);
            const uint32_t amax16 = max(mx & 0xFFFFu, mx >> 16);
            const uint32_t ef = amax16 >> 7;
            if (ROUND == kPhilox && amax16 != 0u && ef >= 11u && ef <= 252u) {
                // the dithered index exactly as fq_vec_kernel forms it, trunc(fma(|x|, 1023 / S, u - 0.5)) with
                // u - 0.5 = fma(h, 2^-16, 2^-17 - 0.5) (exact); the value through the bf16 level table
                const float c = AXS6_MUL(__uint_as_float((253u - ef) << 23), 1023.0f);
                const uint32_t kk = (ef - 6u) * 0x00800080u;
#pragma unroll
                for (int q = 0; q < 4; ++q) {                      // chunks of 8 values: one Philox block each
                    const Axs6Philox rnd = axs6_philox_keyed(offset + (uint64_t)(b * 4 + q), keys);
#pragma unroll
                    for (int pi = 0; pi < 4; ++pi) {
                        const uint32_t wi = w[4 * q + pi];
                        const float d0 = __fmaf_rn((float)(rnd.r[pi] & 0xFFFFu), 1.52587890625e-5f, -0.49999237060546875f);
                        const float d1 = __fmaf_rn((float)(rnd.r[pi] >> 16), 1.52587890625e-5f, -0.49999237060546875f);
                        const int i0 = __float2int_rz(__fmaf_rn(fabsf(__uint_as_float(wi << 16)), c, d0));
                        const int i1 = __float2int_rz(__fmaf_rn(fabsf(__uint_as_float(wi & 0xFFFF0000u)), c, d1));
                        const uint32_t val = ((uint32_t)lvl[i1] * 65536u + (uint32_t)lvl[i0]) + kk;
                        const uint32_t t = (wi & 0x7FFF7FFFu) + 0x7FFF7FFFu;
                        uint32_t nz;
                        asm("prmt.b32 %0, %1, %1, %2;" : "=r"(nz) : "r"(t), "r"(0xBB99u));
                        w[4 * q + pi] = (val | (wi & 0x80008000u)) & nz;
                    }
                }
            } else if (ROUND == kPhilox && amax16 != 0u) {
                // rare block: the fp32 formulas of the general kernel
                const Axs6Scale sc = axs6_scale_fq(amax16 << 16);
                const float c = AXS6_MUL(sc.inv, 1023.0f);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float u[8];
                    chunk_uniforms<kPhilox>(u, b * 4 + q, true, keys, offset, nullptr);
#pragma unroll
                    for (int pi = 0; pi < 4; ++pi) {
                        uint32_t o = 0;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t wi = w[4 * q + pi];
                            const uint32_t bits = h ? (wi & 0xFFFF0000u) : (wi << 16);
                            const float x = __uint_as_float(bits);
                            float y;
                            if (sc.fast) {
                                const float level = __uint_as_float(g_codebook_bits[g_reverse[axs6_nf5_index_dithered_fast(fabsf(x), c, u[2 * pi + h])]]);
                                y = axs6_fq_value_fast(x, level, sc.scale);
                            } else {
                                const float n = axs6_normalise(__uint_as_float(bits & 0x7FFFFFFFu), sc);
                                y = axs6_fq_value(bits, __uint_as_float(g_codebook_bits[g_reverse[axs6_nf5_index_dithered(n, u[2 * pi + h])]]), sc.scale);
                            }
                            o |= (uint32_t)axs6_f32_to_bf16_bits(y) << (16 * h);
                        }
                        w[4 * q + pi] = o;
                    }
                }
            } else if (amax16 == 0u || (ef >= 11u && ef <= 252u)) {
                const uint32_t a1 = amax16 ? ((ef << 7) | 127u) : 0x7FFFu;
                const uint32_t a2 = a1 | (a1 << 16);
                const uint32_t lim2 = (uint32_t)kKeyLim | ((uint32_t)kKeyLim << 16);
                const uint32_t kk = amax16 ? (ef - 6u) * 0x00800080u : 0u;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t wi = w[i];
                    const uint32_t ma = wi & 0x7FFF7FFFu;
                    const uint32_t k2 = min_u16x2(a2 - ma, lim2) << 1;            // byte offsets of the two table entries
                    const uint32_t lo = *reinterpret_cast<const uint16_t *>(reinterpret_cast<const uint8_t *>(table) + (k2 & 0xFFFFu));
                    const uint32_t hi = *reinterpret_cast<const uint16_t *>(reinterpret_cast<const uint8_t *>(table) + (k2 >> 16));
                    const uint32_t val = (hi * 65536u + lo) + kk;
                    // halves that hold +-0 become +0: bit 15 / 31 of t says "non-zero", spread over its half
                    const uint32_t t = ma + 0x7FFF7FFFu;
                    uint32_t nz;
                    asm("prmt.b32 %0, %1, %1, %2;" : "=r"(nz) : "r"(t), "r"(0xBB99u));
                    w[i] = (val | (wi & 0x80008000u)) & nz;
                }
            } else {
                const Axs6Scale sc = axs6_scale_fq(amax16 << 16);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    uint32_t o = 0;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t bits = h ? (w[i] & 0xFFFF0000u) : (w[i] << 16);
                        const float n = axs6_normalise(__uint_as_float(bits & 0x7FFFFFFFu), sc);
                        const int idx = axs6_nf5_index(n);
                        const float y = axs6_fq_value(bits, __uint_as_float(g_codebook_bits[g_reverse[idx]]), sc.scale);
                        o |= (uint32_t)axs6_f32_to_bf16_bits(y) << (16 * h);
                    }
                    w[i] = o;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4 *>(slot + piece[i]) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
        fence_async_smem();
        if (__syncthreads_or(!ok)) {
            // somebody's wait gave up: the whole CTA leaves, after the issuing thread has waited for the (at most two)
            // tile loads that are still armed
            if (tid == 0) drain_ring(bar0, kSlots, s, ph, (int)(nk - k < 2 ? nk - k : 2), kWaitLimit);
            break;
        }
        if (tid == 0) {
            tma_store_2d(&ymap, smem_u32(slot), 0, (int)(grp * kBlocksB));
            bulk_commit();
            if (k + 2 < nk) {
                // the slot of the previous iteration: its store has finished reading once at most one store
                // (the one just committed) is pending
                bulk_wait_read<1>();
                const int s2 = s == 0 ? kSlots - 1 : s - 1;
                mbar_expect_tx(bar0 + 8 * s2, kSlotBytes);
                tma_load_2d(smem_u32(slot0 + s2 * kSlotBytes), &xmap, bar0 + 8 * s2, 0,
                            (int)(((int64_t)blockIdx.x + (k + 2) * (int64_t)gridDim.x) * kBlocksB));
            }
        }
        if (++s == kSlots) { s = 0; ph ^= 1u; }
    }
    if (tid == 0) bulk_wait<0>();
}

// -> status, or 1 when this path does not apply
static int launch(const void *x, void *y, int64_t nblocks, int round, uint64_t seed, uint64_t offset,
                  const unsigned long long *epoch, cudaStream_t st)
{
    if (nblocks >= (1ll << 31) - kBlocksB) return 1;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return 1;
    CUtensorMap xm, ym;
    const cuuint64_t gdim[2] = {32, (cuuint64_t)nblocks};
    const cuuint64_t gstride[1] = {64};
    const cuuint32_t box[2] = {32, (cuuint32_t)kBlocksB};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&xm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(x), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
        enc(&ym, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, y, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return 1;
    const DeviceInfo &d = device_info();
    int64_t ctas = (nblocks + kBlocksB - 1) / kBlocksB;
    const int64_t cap = tune_value(0);
    int per_sm = 3;                          // 32768 x 8192: 6.47 TB/s with 3 CTAs per SM, 5.96 with 4, 5.79 with 2
    if (cap > 0 && cap < per_sm) per_sm = (int)cap;
    if (ctas > (int64_t)d.sms * per_sm) ctas = (int64_t)d.sms * per_sm;
    if (ctas < 1) ctas = 1;
    if (!ensure_dynamic_smem(reinterpret_cast<const void *>(&fq_bf16_nf5_b32_bulk_kernel<kNearest>), kSmemBytes) ||
        !ensure_dynamic_smem(reinterpret_cast<const void *>(&fq_bf16_nf5_b32_bulk_kernel<kPhilox>), kSmemBytes))
        return AXS6_ERR_LAUNCH;
    const Axs6PhiloxKeys keys = axs6_philox_keys(seed);
    cudaError_t le;
    if (round == kNearest) le = launch_overlapped(nblocks * 4 <= kSmallLaunch, fq_bf16_nf5_b32_bulk_kernel<kNearest>, (unsigned)ctas, kBlocksB, kSmemBytes, st, xm, ym, nblocks, 0ull, 0ull, (const unsigned long long *)nullptr, keys);
    else                   le = launch_overlapped(nblocks * 4 <= kSmallLaunch, fq_bf16_nf5_b32_bulk_kernel<kPhilox>, (unsigned)ctas, kBlocksB, kSmemBytes, st, xm, ym, nblocks, seed, offset, epoch, keys);
    count_launch();
    return le == cudaSuccess ? check_launch() : AXS6_ERR_LAUNCH;
}

}  // namespace fqb

// Status word of the TMA-fed fake-quantise kernel, cleared when non-zero (read by axs6_codec_status).
int fq_status_fetch()
{
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, fqb::g_fq_status, sizeof(int)) != cudaSuccess) return AXS6_ERR_DEVICE;
    if (v != 0) cudaMemcpyToSymbol(fqb::g_fq_status, &zero, sizeof(int));
    return v;
}

static int fq_entry(const void *x, void *y, int in_dtype, int out_dtype, int64_t rows, int64_t cols,
                    int64_t ldx, int64_t ldy, int block, int grid, int round, uint32_t flags,
                    uint64_t seed, uint64_t offset, const float *noise, cudaStream_t stream,
                    const long long *row_index = nullptr, int64_t table_rows = 0)
{
    if (!valid_dtype(in_dtype) || !valid_dtype(out_dtype) || !valid_block(block)) return AXS6_ERR_ARG;
    if (grid != AXS6_GRID_NF5 && grid != AXS6_GRID_UNIFORM) return AXS6_ERR_ARG;
    if (rows < 0 || cols < 0 || ldx < cols || ldy < cols) return AXS6_ERR_ARG;
    if (flags & ~(AXS6_FLAG_INPUT_VIA_BF16 | AXS6_FLAG_OUTPUT_TF32)) return AXS6_ERR_ARG;
    if (rows == 0 || cols == 0) return AXS6_OK;
    if (!x || !y) return AXS6_ERR_ARG;
    if (round == kNoise && !noise) return AXS6_ERR_ARG;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;

    FqArgs a;
    a.x = x; a.y = y; a.ldx = ldx; a.ldy = ldy;
    a.g = make_geom(rows, cols, block);
    a.g.flat = (cols % block == 0 && ldx == cols && ldy == cols && !row_index) ? 1 : 0;
    a.row_index = row_index; a.table_rows = table_rows;
    a.via_bf16 = (flags & AXS6_FLAG_INPUT_VIA_BF16) ? 1u : 0u;
    a.out_tf32 = (flags & AXS6_FLAG_OUTPUT_TF32) ? 1u : 0u;
    a.seed = seed; a.offset = offset; a.noise = noise;
    a.keys = axs6_philox_keys(seed);
    a.epoch = philox_epoch_ptr();
    if (round == kPhilox && !a.epoch) return AXS6_ERR_DEVICE;
    const bool vec = aligned16(x) && aligned16(y) && (cols % kChunk == 0) && (ldx % kChunk == 0) &&
                     (ldy % kChunk == 0) && (round != kNoise || aligned16(noise));
    // tune key 12: 1 = general kernel only
    if (vec && a.g.flat && in_dtype == AXS6_BF16 && out_dtype == AXS6_BF16 && grid == AXS6_GRID_NF5 &&
        (round == kNearest || round == kPhilox) && block == 32 && tune_value(12) != 1) {
        const int r = fqb::launch(x, y, rows * (cols / 32), round, seed, offset, a.epoch, stream);
        if (r != 1) return r;
    }
    if (in_dtype == AXS6_F32 && out_dtype == AXS6_F32) return dispatch_fq<float, float>(a, grid, round, vec, stream);
    if (in_dtype == AXS6_F32 && out_dtype == AXS6_BF16) return dispatch_fq<float, __nv_bfloat16>(a, grid, round, vec, stream);
    if (in_dtype == AXS6_BF16 && out_dtype == AXS6_F32) return dispatch_fq<__nv_bfloat16, float>(a, grid, round, vec, stream);
    return dispatch_fq<__nv_bfloat16, __nv_bfloat16>(a, grid, round, vec, stream);
}

}  // namespace axs6

AXS6_API int axs6_fq(const void *x, void *y, int in_dtype, int out_dtype, int64_t rows, int64_t cols,
                       int64_t ldx, int64_t ldy, int block, int grid, int rounding, uint32_t flags,
                       uint64_t seed, uint64_t offset, axs6_stream_t stream)
{
    if (rounding != AXS6_ROUND_NEAREST && rounding != AXS6_ROUND_STOCHASTIC) return AXS6_ERR_ARG;
    return axs6::fq_entry(x, y, in_dtype, out_dtype, rows, cols, ldx, ldy, block, grid,
                          rounding == AXS6_ROUND_NEAREST ? axs6::kNearest : axs6::kPhilox, flags, seed, offset,
                          nullptr, static_cast<cudaStream_t>(stream));
}

AXS6_API int axs6_fq_gather(const void *table, int64_t table_rows, const long long *row_index, void *y, int in_dtype,
                            int out_dtype, int64_t rows, int64_t cols, int64_t ld_table, int64_t ldy, int block, int grid,
                            int rounding, uint64_t seed, uint64_t offset, axs6_stream_t stream)
{
    if (rounding != AXS6_ROUND_NEAREST && rounding != AXS6_ROUND_STOCHASTIC) return AXS6_ERR_ARG;
    if (!row_index || table_rows <= 0) return AXS6_ERR_ARG;
    return axs6::fq_entry(table, y, in_dtype, out_dtype, rows, cols, ld_table, ldy, block, grid,
                          rounding == AXS6_ROUND_NEAREST ? axs6::kNearest : axs6::kPhilox, 0, seed, offset,
                          nullptr, static_cast<cudaStream_t>(stream), row_index, table_rows);
}

AXS6_API int axs6_fq_gather_status(void)
{
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, axs6::g_gather_status, sizeof(int)) != cudaSuccess) return AXS6_ERR_DEVICE;
    if (v != 0) cudaMemcpyToSymbol(axs6::g_gather_status, &zero, sizeof(int));
    return v;
}

AXS6_API int axs6_fq_with_noise(const void *x, void *y, int in_dtype, int out_dtype, int64_t rows,
                                  int64_t cols, int64_t ldx, int64_t ldy, int block, int grid, uint32_t flags,
                                  const float *noise, axs6_stream_t stream)
{
    return axs6::fq_entry(x, y, in_dtype, out_dtype, rows, cols, ldx, ldy, block, grid, axs6::kNoise, flags,
                          0, 0, noise, static_cast<cudaStream_t>(stream));
}
