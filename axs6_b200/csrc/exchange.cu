// Fused "unpack every rank's records and average": the receiving side of the compressed gradient
// exchange.  After the all-gather of the ranks' packed buckets a rank holds nsrc record buffers of the
// same tensor; instead of nsrc unpack passes and nsrc - 1 additions over fp32 tensors (12 bytes of HBM
// traffic per value and source) this kernel reads every record once and writes the result once:
//     y = (unpack(src 0) + unpack(src 1) + ... ) / divisor        summed in fp32, in source order,
// which is bit for bit what the unfused sequence computes.
//
// Roofline: HBM.  Algorithmic bytes per block of B values: nsrc * record bytes + B * sizeof(out).
//
//   unpack_sum_bulk_kernel     NF5 grid, block 32, byte records, contiguous 16-byte aligned output:
//                              8 consumer warps (one thread per block) + 1 producer warp.  The producer
//                              streams (group of 256 records, source) pairs through a 4-stage ring with
//                              one bulk copy each; consumers decode as the TMA-fed unpack kernel does
//                              (one table lookup + one integer add per value), accumulate 32 floats in
//                              registers, and the finished tile leaves through a tensor map.
//   unpack_sum_generic_kernel  everything else: one thread per value.
// Every mbarrier wait is bounded; a wait that gives up sets the status word that axs6_codec_status reads.
#include "async_copy.cuh"
#include "quant_device.cuh"

namespace axs6 {
namespace exchange {

using namespace acp;

constexpr int kBlocks = 256;                 // blocks (consumer threads) per group
constexpr int kThreadsX = kBlocks + 32;      // + the producer warp
constexpr int kStagesX = 4;
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ int g_exchange_status;

template <typename Tout>
struct Out;
template <>
struct Out<__nv_bfloat16> { static constexpr int kRowBytes = 64, kPieces = 4, kSwzMask = 3, kSwzShift = 1; };
template <>
struct Out<float> { static constexpr int kRowBytes = 128, kPieces = 8, kSwzMask = 7, kSwzShift = 0; };

template <typename Tout, int HDR>
constexpr int smem_bytes() { return 1024 + 1024 + 2 * kBlocks * Out<Tout>::kRowBytes + kStagesX * kBlocks * (HDR + 24); }

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kBlocks) : "memory"); }

// One record (seven words starting at the word that holds its first byte, `sft` = 8 * (byte offset in
// that word + header bytes)) added to, or for the first source stored into, the 32 accumulators.
template <int HDR, bool kFirst>
__device__ __forceinline__ void accumulate_record(const uint32_t (&W)[7], uint32_t head, uint32_t sft,
                                                  const uint32_t *table, uint32_t lane4, const float *lev, float (&acc)[32])
{
    uint32_t pay[6];
#pragma unroll
    for (int i = 0; i < 6; ++i) pay[i] = __funnelshift_rc(W[i], W[i + 1], sft);
    const uint32_t se = HDR == 1 ? (head & 0xFFu) : ((head >> 2) & 0xFFu);
    if (se >= 8u && se <= 254u) {
        const uint32_t kk = (se - 7u) << 23;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int bit = 6 * i, word = bit >> 5, off = bit & 31;
            uint32_t v;                                 // the code at bits 7..12
            if (off < 7) v = pay[word] << (7 - off);
            else if (off == 7) v = pay[word];
            else if (off <= 26) v = pay[word] >> (off - 7);
            else v = __funnelshift_r(pay[word], pay[word + 1], off - 7);
            const float val = __uint_as_float(*reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(table) + ((v & 0x1F80u) | lane4)) + kk);
            acc[i] = kFirst ? val : AXS6_ADD(acc[i], val);
        }
    } else {
        const float scale = axs6_scale_decode(se);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int bit = 6 * i, word = bit >> 5, off = bit & 31;
            const uint32_t code = (off <= 26 ? (pay[word] >> off) : __funnelshift_r(pay[word], pay[word + 1], off)) & 63u;
            const float val = axs6_decode_value(code >> 5, lev[code & 31u], scale);
            acc[i] = kFirst ? val : AXS6_ADD(acc[i], val);
        }
    }
}

template <typename Tout, int HDR>
__global__ void __launch_bounds__(kThreadsX) unpack_sum_bulk_kernel(const __grid_constant__ CUtensorMap ymap,
                                                                   const uint8_t *__restrict__ in, int64_t nsrc,
                                                                   int64_t src_stride, int64_t nblocks, float divisor,
                                                                   uint32_t wait_limit, int producer_muted)
{
    constexpr bool kBf16 = sizeof(Tout) == 2;
    constexpr int REC = HDR + 24;
    constexpr int kIn = kBlocks * REC;
    constexpr int kTile = kBlocks * Out<Tout>::kRowBytes;
    constexpr int kPieces = Out<Tout>::kPieces;
    extern __shared__ uint8_t raw[];
    // code -> sign and level bits, exponent field lowered by 120; one copy per lane (entry (code, lane) is word
    // code * 32 + lane), so that the 32 lookups of a warp always fall into 32 different banks
    __shared__ __align__(128) uint32_t table[64 * 32];
    __shared__ float lev[32];
    __shared__ int gave_up[2];                       // by parity of the group: some consumer's wait ran out
    uint8_t *base = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
    uint8_t *tile0 = base + 1024;
    uint8_t *in0 = tile0 + 2 * kTile;
    const uint32_t full0 = smem_u32(base), empty0 = full0 + 8 * kStagesX;
    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int s = 0; s < kStagesX; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, kBlocks / 32); }
        gave_up[0] = gave_up[1] = 0;
        fence_barrier_init();
        fence_async_smem();
    }
    for (int i = tid; i < 64 * 32; i += kThreadsX) {
        const uint32_t code = (uint32_t)i >> 5;
        table[i] = (g_codebook_bits[code & 31u] - (120u << 23)) | ((code >> 5) << 31);
    }
    if (tid < 32) lev[tid] = __uint_as_float(g_codebook_bits[tid]);
    __syncthreads();

    const int64_t groups = (nblocks + kBlocks - 1) / kBlocks;
    const int64_t nk = (int64_t)blockIdx.x < groups ? (groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (tid >= kBlocks) {
        // ---------------------------------------------------------------- producer warp (one lane)
        if (tid == kBlocks && !producer_muted) {
            int s = 0;
            uint32_t ph = 0;
            long long armed = 0;                                   // loads issued so far
            bool ok = true;
            for (int64_t k = 0; k < nk && ok; ++k) {
                const int64_t grp = (int64_t)blockIdx.x + k * (int64_t)gridDim.x;
                if (nblocks - grp * kBlocks < kBlocks) break;      // the ragged last group is read by the consumers
                for (int64_t r = 0; r < nsrc; ++r) {
                    if (!mbar_wait_bounded(empty0 + 8 * s, ph ^ 1u, 2, &g_exchange_status, wait_limit)) { ok = false; break; }
                    mbar_expect_tx(full0 + 8 * s, kIn);
                    bulk_load(smem_u32(in0 + s * kIn), in + r * src_stride + grp * kIn, kIn, full0 + 8 * s);
                    ++armed;
                    if (++s == kStagesX) { s = 0; ph ^= 1u; }
                }
            }
            // This thread leaves last: the shared memory of the CTA stays allocated until it does, so it waits
            // (bounded) until every load it issued has landed.  After a normal run the consumers have already seen
            // all of them and the waits return at once.
            for (long long back = 0; back < kStagesX && back < armed; ++back) {
                const long long idx = armed - 1 - back;
                mbar_wait_quiet(full0 + 8 * (uint32_t)(idx % kStagesX), (uint32_t)((idx / kStagesX) & 1), wait_limit);
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumers: one thread per block
    const uint32_t wb = (uint32_t)(REC * tid) >> 2, sh = (uint32_t)(REC * tid) & 3u;
    const uint32_t sft = 8u * (sh + HDR);
    const uint32_t lane4 = ((uint32_t)tid & 31u) << 2;
    uint32_t piece[kPieces];
#pragma unroll
    for (int i = 0; i < kPieces; ++i)
        piece[i] = (uint32_t)tid * Out<Tout>::kRowBytes + (uint32_t)((i ^ ((tid >> Out<Tout>::kSwzShift) & Out<Tout>::kSwzMask)) << 4);

    int s = 0;
    uint32_t ph = 0;
    for (int64_t k = 0; k < nk; ++k) {
        const int64_t grp = (int64_t)blockIdx.x + k * (int64_t)gridDim.x;
        const int64_t b = grp * kBlocks + tid;
        const bool whole = nblocks - grp * kBlocks >= kBlocks;
        uint8_t *tile = tile0 + (k & 1) * kTile;
        float acc[32];
        bool ok = true;
        for (int64_t r = 0; r < nsrc; ++r) {
            uint32_t W[7];
            uint32_t sft_r = sft, head_shift = 8u * sh;
            if (whole) {
                if (ok) ok = mbar_wait_bounded(full0 + 8 * s, ph, 1, &g_exchange_status, wait_limit);
                const uint32_t *r32 = reinterpret_cast<const uint32_t *>(in0 + s * kIn) + wb;
#pragma unroll
                for (int i = 0; i < 7; ++i) W[i] = r32[i];
                __syncwarp();
                if ((tid & 31) == 0) mbar_arrive(empty0 + 8 * s);          // this warp has read its records
                if (++s == kStagesX) { s = 0; ph ^= 1u; }
            } else {
#pragma unroll
                for (int i = 0; i < 7; ++i) W[i] = 0u;
                if (b < nblocks) {
                    const uint8_t *rec = in + r * src_stride + b * REC;
#pragma unroll
                    for (int i = 0; i < REC; ++i) W[i >> 2] |= (uint32_t)rec[i] << (8 * (i & 3));
                }
                sft_r = 8u * HDR;
                head_shift = 0u;
            }
            if (ok && b < nblocks) {
                if (r == 0) accumulate_record<HDR, true>(W, W[0] >> head_shift, sft_r, table, lane4, lev, acc);
                else        accumulate_record<HDR, false>(W, W[0] >> head_shift, sft_r, table, lane4, lev, acc);
            }
        }
        if (ok && b < nblocks) {
            uint32_t o[kBf16 ? 16 : 32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float y = AXS6_DIV(acc[i], divisor);
                if (kBf16) {
                    const uint32_t h = axs6_f32_to_bf16_bits(y);
                    if (i & 1) o[i >> 1] |= h << 16; else o[i >> 1] = h;
                } else {
                    o[i] = __float_as_uint(y);
                }
            }
#pragma unroll
            for (int i = 0; i < kPieces; ++i)
                *reinterpret_cast<uint4 *>(tile + piece[i]) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
        if (!ok) gave_up[k & 1] = 1;
        fence_async_smem();
        if (tid == 0) bulk_wait_read<0>();        // the previous group's store has left the other tile
        consumer_barrier();
        if (*reinterpret_cast<volatile int *>(&gave_up[k & 1])) break;
        if (tid == 0) {
            tma_store_2d(&ymap, smem_u32(tile), 0, (int)(grp * kBlocks));
            bulk_commit();
        }
    }
    if (tid == 0) bulk_wait<0>();
}

// One thread per value: any grid, block size, layout of y.
template <typename Tout, int GRID>
__global__ void __launch_bounds__(256) unpack_sum_generic_kernel(const uint8_t *__restrict__ in, int64_t nsrc, int64_t src_stride,
                                                                Tout *__restrict__ y, int64_t rows, int64_t cols, int64_t ldy,
                                                                int B, int hdr, float divisor)
{
    __shared__ float lev[32];
    build_levels<GRID>(lev);
    __syncthreads();
    const int rec = hdr + B * 3 / 4;
    const int64_t nblk = (cols + B - 1) / B;
    const int64_t total = rows * cols;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = e / cols, pc = e - row * cols;
        const int i = (int)(pc % B);
        const int64_t blk = row * nblk + pc / B;
        float acc = 0.0f;
        for (int64_t r = 0; r < nsrc; ++r) {
            const uint8_t *p = in + r * src_stride + blk * rec;
            const uint32_t se = (hdr == 1) ? (uint32_t)p[0] : (((uint32_t)p[0] | ((uint32_t)p[1] << 8)) >> 2) & 0xFFu;
            const int bit = 6 * i, k = bit >> 3, sh = bit & 7;
            uint32_t w = p[hdr + k];
            if (sh > 2) w |= (uint32_t)p[hdr + k + 1] << 8;
            const uint32_t code = (w >> sh) & 63u;
            const float v = axs6_decode_value(code >> 5, lev[code & 31u], axs6_scale_decode(se));
            acc = r == 0 ? v : AXS6_ADD(acc, v);
        }
        ChunkIO<Tout>::store1(y, row * ldy + pc, AXS6_DIV(acc, divisor));
    }
}

template <typename Tout>
static int launch_bulk(const uint8_t *in, int64_t nsrc, int64_t src_stride, void *y, int64_t nblocks, int hdr, float divisor,
                       cudaStream_t st)
{
    if (nblocks >= (1ll << 31) - kBlocks) return 1;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return 1;
    constexpr bool kBf16 = sizeof(Tout) == 2;
    CUtensorMap map;
    const cuuint64_t gdim[2] = {32, (cuuint64_t)nblocks};
    const cuuint64_t gstride[1] = {32 * sizeof(Tout)};
    const cuuint32_t box[2] = {32, (cuuint32_t)kBlocks};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, kBf16 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, y, gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, kBf16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return 1;
    const DeviceInfo &d = device_info();
    int64_t ctas = (nblocks + kBlocks - 1) / kBlocks;
    const int64_t cap = tune_value(1);
    int per_sm = 2;
    if (cap > 0 && cap < per_sm) per_sm = (int)cap;
    if (ctas > (int64_t)d.sms * per_sm) ctas = (int64_t)d.sms * per_sm;
    if (ctas < 1) ctas = 1;
    if (!ensure_dynamic_smem(reinterpret_cast<const void *>(&unpack_sum_bulk_kernel<Tout, 1>), smem_bytes<Tout, 1>()) ||
        !ensure_dynamic_smem(reinterpret_cast<const void *>(&unpack_sum_bulk_kernel<Tout, 2>), smem_bytes<Tout, 2>()))
        return AXS6_ERR_LAUNCH;
    // tune key 13: poll limit of the waits (0 = built-in); tune key 14 = 1: the producer issues no load at all, so the
    // consumers' first wait runs out with nothing in flight (exists so that the give-up path can be exercised safely)
    const uint32_t limit = tune_value(13) > 0 ? (uint32_t)tune_value(13) : kWaitLimit;
    const int muted = tune_value(14) == 1 ? 1 : 0;
    if (hdr == 1) unpack_sum_bulk_kernel<Tout, 1><<<(unsigned)ctas, kThreadsX, smem_bytes<Tout, 1>(), st>>>(map, in, nsrc, src_stride, nblocks, divisor, limit, muted);
    else          unpack_sum_bulk_kernel<Tout, 2><<<(unsigned)ctas, kThreadsX, smem_bytes<Tout, 2>(), st>>>(map, in, nsrc, src_stride, nblocks, divisor, limit, muted);
    count_launch();
    return check_launch();
}

template <typename Tout>
static int launch_generic(const uint8_t *in, int64_t nsrc, int64_t src_stride, void *y, int64_t rows, int64_t cols, int64_t ldy,
                          int block, int grid, int hdr, float divisor, cudaStream_t st)
{
    const DeviceInfo &d = device_info();
    int64_t ctas = (rows * cols + 255) / 256;
    if (ctas > (int64_t)d.sms * 8) ctas = (int64_t)d.sms * 8;
    if (grid == AXS6_GRID_NF5)
        unpack_sum_generic_kernel<Tout, AXS6_GRID_NF5><<<(unsigned)ctas, 256, 0, st>>>(in, nsrc, src_stride, static_cast<Tout *>(y), rows, cols, ldy, block, hdr, divisor);
    else
        unpack_sum_generic_kernel<Tout, AXS6_GRID_UNIFORM><<<(unsigned)ctas, 256, 0, st>>>(in, nsrc, src_stride, static_cast<Tout *>(y), rows, cols, ldy, block, hdr, divisor);
    count_launch();
    return check_launch();
}

}  // namespace exchange

// Status word of the kernels of this file, cleared when non-zero (read by axs6_codec_status).
int exchange_status_fetch()
{
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, exchange::g_exchange_status, sizeof(int)) != cudaSuccess) return AXS6_ERR_DEVICE;
    if (v != 0) cudaMemcpyToSymbol(exchange::g_exchange_status, &zero, sizeof(int));
    return v;
}

}  // namespace axs6

AXS6_API int axs6_unpack_sum(int layout, const void *records, int64_t nsrc, int64_t src_stride, void *y, int out_dtype,
                             int64_t rows, int64_t cols, int64_t ldy, int block, int grid, float divisor,
                             axs6_stream_t stream)
{
    using namespace axs6;
    if (!valid_dtype(out_dtype) || !valid_block(block)) return AXS6_ERR_ARG;
    if (layout != AXS6_LAYOUT_WIRE && layout != AXS6_LAYOUT_SPEC) return AXS6_ERR_ARG;
    if (grid != AXS6_GRID_NF5 && grid != AXS6_GRID_UNIFORM) return AXS6_ERR_ARG;
    if (rows < 0 || cols < 0 || ldy < cols || nsrc < 1 || !(divisor != 0.0f)) return AXS6_ERR_ARG;
    if (rows == 0 || cols == 0) return AXS6_OK;
    if (!records || !y) return AXS6_ERR_ARG;
    const int hdr = layout == AXS6_LAYOUT_SPEC ? 2 : 1;
    const int64_t need = rows * ((cols + block - 1) / block) * (hdr + block * 3 / 4);
    if (nsrc > 1 && src_stride < need) return AXS6_ERR_ARG;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t *in = static_cast<const uint8_t *>(records);
    // tune key 11: 1 = one-thread-per-value kernel only
    if (grid == AXS6_GRID_NF5 && block == 32 && cols % 32 == 0 && ldy == cols && aligned16(y) && aligned16(records) &&
        src_stride % 16 == 0 && tune_value(11) != 1) {
        const int r = out_dtype == AXS6_F32 ? exchange::launch_bulk<float>(in, nsrc, src_stride, y, rows * (cols / 32), hdr, divisor, st)
                                            : exchange::launch_bulk<__nv_bfloat16>(in, nsrc, src_stride, y, rows * (cols / 32), hdr, divisor, st);
        if (r != 1) return r;
    }
    return out_dtype == AXS6_F32 ? exchange::launch_generic<float>(in, nsrc, src_stride, y, rows, cols, ldy, block, grid, hdr, divisor, st)
                                 : exchange::launch_generic<__nv_bfloat16>(in, nsrc, src_stride, y, rows, cols, ldy, block, grid, hdr, divisor, st);
}
