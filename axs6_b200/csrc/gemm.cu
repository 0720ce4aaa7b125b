// bf16 x bf16 -> fp32-accumulate GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), fed
// by TMA, for the three products of the AXS-6 Linear:
//     forward   Y  = Xq  Wq^T      A = Xq (M x K, K-major)        B = Wq (N x K, K-major)
//     dX        dX = Gq  Wq        A = Gq (M x N, K-major)        B = Wq (N x K, MN-major)
//     dW        dW = Gq^T Xq       A = Gq (M x N, MN-major)       B = Xq (M x K, MN-major)
// "K-major" = the contraction index is the contiguous one in global memory; "MN-major" = the
// output index is contiguous.  Both are consumed in place: the shared-memory matrix descriptors
// and the a_major / b_major bits of the instruction descriptor select the layout, so no operand
// is ever transposed in HBM.
//
// The same kernel is instantiated for fp32 operands consumed as TF32 (kind::tf32: the tensor
// core reads 10 mantissa bits), used by the fp32 Linear paths where bf16 operands would miss the
// 1e-3 accuracy bar.  Tile geometry in BYTES is identical (rows of 128 B, K step of 32 B), so
// a k-block is 64 bf16 or 32 fp32 values.
//
// Roofline: tensor pipe; 2*M*N*K flops per launch.
//
// One persistent CTA per SM, 192 threads:
//   warp 0      TMA producer (one lane): 4-stage ring of {A 128x64, B 256x64} bf16 tiles, 128-byte
//               swizzle, one mbarrier per stage armed with the stage's byte count
//   warp 1      allocates TMEM (512 columns = two 128x256 fp32 accumulators); one lane issues
//               tcgen05.mma (cta_group::1, M128 N256 K16) and commits stage-free / tile-done barriers
//   warps 2..5  epilogue: tcgen05.ld of the finished accumulator (each warp its 32 TMEM lanes),
//               bias add, conversion, 16-byte global stores; overlaps the next tile's main loop
//               through the second accumulator.
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiting role records an error
// code in g_gemm_status and all roles leave their loops, TMEM is freed and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <string.h>

#include "async_copy.cuh"
#include "common.cuh"

namespace axs6 {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreadsGemm = 192;
constexpr int kTmemCols = 512;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ int g_gemm_status;   // 0 = ok; otherwise the code of the first wait that gave up

struct Params {
    int M, N, K;              // C is M x N, contraction length K
    int a_mn, b_mn;           // operand is MN-major
    void *c;
    long long ldc;
    int c_bf16;               // output dtype: 1 bf16, 0 fp32
    const float *bias;        // length N or null
    int bias_bf16;            // round each bias value to bf16 before adding (F.linear with a bf16 bias)
    int tiles_m, tiles_n;
    uint32_t a_lbo, a_sbo, a_kstep, b_lbo, b_sbo, b_kstep;   // descriptor strides (bytes)
    int bk;                   // values per k-block: 64 (bf16) or 32 (tf32)
    int splits;               // split-K factor (>= 2: fp32 output accumulated with red.add into a zero-filled C)
    int tail_begin;           // 2-CTA kernel: tiles from this one on are computed as two K halves (0 = none)
    uint32_t mn_box_bytes;    // bytes of one MN-major TMA box: 128 B x bk rows
    int dynamic;              // CTA-pair kernel: one cluster per work unit, units taken over through cluster launch control
    int a_mn4, b_mn4;         // CTA-pair kernel: the MN-major operand arrives as ONE 4-D box per stage (see make_mn4_map)
    int c_tma;                // CTA-pair kernel: output leaves through shared memory and tensor maps (aligned C): 1 bf16, 2 fp32
    float *ws;                // split-K workspace (null: partials are added into C with red.add): partial `part` of the
    long long ws_stride;      // product is stored at ws + part * ws_stride as an (M, ws_ld) fp32 matrix and a second
    int ws_ld;                // kernel adds the partials in index order, which makes the sum reproducible
};

// ------------------------------------------------------------------------------------- PTX helpers
using acp::smem_u32;
using acp::mbar_init;
using acp::mbar_expect_tx;
using acp::mbar_arrive;
using acp::tma_load_2d;

// Bounded wait.  Returns false if it gave up (status set) or if another role already failed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code)
{
    return acp::mbar_wait_bounded(bar, parity, code, &g_gemm_status, kSpinLimit);
}

// On the way out of a kernel in which a wait gave up: tile loads and products that were already issued may still be
// running, and their barriers live partly in the other CTA of the pair, so they cannot all be waited for one by one.
// Every thread lingers for a fifth of a millisecond instead (loads and products complete within microseconds) before
// shared and tensor memory are released.  Costs nothing on the normal path (one read of the status word).
__device__ __forceinline__ void linger_if_failed()
{
    if (*(volatile int *)&g_gemm_status != 0)
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <bool kTf32>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    if (kTf32)
        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                     " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                     ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                     " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                     ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// Shared-memory matrix descriptor: start address, leading / stride byte offsets (all >> 4),
// descriptor version 1 (sm_100), 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo)
{
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}

// Instruction descriptor of tcgen05.mma: D fp32 (bit 4), A and B format at bits 7 and 10
// (kind::f16: 1 = bf16; kind::tf32: 2 = tf32), optional MN-major operands (bits 15, 16),
// N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t instr_desc(int a_mn, int b_mn, uint32_t fmt)
{
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

#define AXS6_TMEM_LD32(taddr, r)                                                                                      \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                            \
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26," \
                 "%27,%28,%29,%30,%31}, [%32];"                                                                        \
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),     \
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),            \
                   "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),          \
                   "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),          \
                   "=r"(r[29]), "=r"(r[30]), "=r"(r[31])                                                               \
                 : "r"(taddr))

// Drains one 128 x 256 fp32 accumulator: this thread owns TMEM lane (= output row) `row` and walks
// the 256 columns in chunks of 32 (tcgen05.ld 32x32b.x32), adds the bias, converts and stores.
__device__ __forceinline__ void epilogue_tile(const Params &p, uint32_t taddr, int row, int n0, bool vec_ok,
                                              bool accumulate = false, bool add_bias = true, int part = 0)
{
    const bool to_ws = accumulate && p.ws != nullptr;
    if (to_ws) add_bias = false;                       // the reducing kernel adds the bias
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        AXS6_TMEM_LD32(taddr + (uint32_t)(c * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            if (p.bias && add_bias) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col0 + i < p.N) {
                        const float bv = __ldg(p.bias + col0 + i);
                        v[i] += p.bias_bf16 ? __bfloat162float(__float2bfloat16_rn(bv)) : bv;
                    }
            }
            const bool full = col0 + 32 <= p.N;
            if (p.c_bf16) {
                __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(p.c) + (long long)row * p.ldc + col0;
                if (full && vec_ok) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
                            w[j] = *reinterpret_cast<const uint32_t *>(&h);
                        }
                        *reinterpret_cast<uint4 *>(dst + 8 * i) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                } else {
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < p.N) dst[i] = __float2bfloat16_rn(v[i]);
                }
            } else if (to_ws) {
                // split-K partial kept apart: plain stores into this part's slice of the workspace
                float *dst = p.ws + (long long)part * p.ws_stride + (long long)row * p.ws_ld + col0;
                if (full) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<float4 *>(dst + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                } else {
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < p.N) dst[i] = v[i];
                }
            } else if (accumulate) {
                // split-K partial: add into the zero-initialised fp32 output.  With two partials the
                // result does not depend on their order (0 + a + b == 0 + b + a exactly).
                float *dst = reinterpret_cast<float *>(p.c) + (long long)row * p.ldc + col0;
                if (full && vec_ok) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * i), "f"(v[4 * i]),
                                     "f"(v[4 * i + 1]), "f"(v[4 * i + 2]), "f"(v[4 * i + 3]) : "memory");
                } else {
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < p.N) atomicAdd(dst + i, v[i]);
                }
            } else {
                float *dst = reinterpret_cast<float *>(p.c) + (long long)row * p.ldc + col0;
                if (full && vec_ok) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<float4 *>(dst + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                } else {
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < p.N) dst[i] = v[i];
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------- kernel
template <bool kTf32>
__global__ void __launch_bounds__(kThreadsGemm, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = base + kStages * kStageBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };
    const uint32_t tmem_slot = bar0 + 8u * (2 * kStages + 4);
    uint8_t *smem_gen = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(smem_gen + kStages * kStageBytes + 8 * (2 * kStages + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int splits = p.splits;
    const int num_tiles = p.tiles_m * p.tiles_n * splits;  // work units: (tile, K range)
    const int total_kb = (p.K + p.bk - 1) / p.bk;
    auto kb_begin = [&](int t) { return (int)(((long long)(t % splits) * total_kb) / splits); };
    auto kb_end = [&](int t) { return (int)(((long long)(t % splits + 1) * total_kb) / splits); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    pdl_wait();                                          // barriers, tensor memory and descriptors are set up; caller memory from here on

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int tile = t / splits;
                const int m0 = (tile / p.tiles_n) * BM, n0 = (tile % p.tiles_n) * BN;
                for (int kb = kb_begin(t); kb < kb_end(t); ++kb) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, 1)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), kStageBytes);
                    const uint32_t sa = base + s * kStageBytes, sb = sa + kABytes;
                    const int k0 = kb * p.bk;
                    if (!p.a_mn) {
                        tma_load_2d(sa, &map_a, full_bar(s), k0, m0);                  // box {64 k, 128 rows}
                    } else {
                        const int per_box = p.bk;                                      // output indices per 128-byte row (= 128 / element size)
                        for (int j = 0; j < BM / per_box; ++j)                         // boxes {128 B of m, bk rows of k}
                            tma_load_2d(sa + j * p.mn_box_bytes, &map_a, full_bar(s), m0 + per_box * j, k0);
                    }
                    if (!p.b_mn) {
                        tma_load_2d(sb, &map_b, full_bar(s), k0, n0);                  // box {64 k, 256 rows}
                    } else {
                        const int per_box = p.bk;
                        for (int j = 0; j < BN / per_box; ++j)
                            tma_load_2d(sb + j * p.mn_box_bytes, &map_b, full_bar(s), n0 + per_box * j, k0);
                    }
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = instr_desc(p.a_mn, p.b_mn, kTf32 ? 2u : 1u);
            int s = 0, acc = 0;
            uint32_t ph = 0, aph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                if (!mbar_wait(tempty_bar(acc), aph ^ 1u, 2)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                const int kb0 = kb_begin(t);
                for (int kb = kb0; kb < kb_end(t); ++kb) {
                    if (!mbar_wait(full_bar(s), ph, 3)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + s * kStageBytes, sb = sa + kABytes;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {                  // four 32-byte K steps per 128-byte row
                        const uint64_t ad = smem_desc(sa + k * p.a_kstep, p.a_lbo, p.a_sbo);
                        const uint64_t bd = smem_desc(sb + k * p.b_kstep, p.b_lbo, p.b_sbo);
                        tc_mma<kTf32>(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(empty_bar(s));            // stage reusable once these MMAs have read it
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                tc_commit(tfull_bar(acc));              // accumulator complete
                acc ^= 1;
                if (acc == 0) aph ^= 1u;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;                         // TMEM lane quarter this warp may read
        int acc = 0;
        uint32_t aph = 0;
        bool ok = true;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0) && (p.ldc % 8 == 0);
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const int tile = t / splits;
            const int m0 = (tile / p.tiles_n) * BM, n0 = (tile % p.tiles_n) * BN;
            if (!mbar_wait(tfull_bar(acc), aph, 4)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
            epilogue_tile(p, taddr, row, n0, vec_ok, splits > 1, (t % splits) == 0, t % splits);
            tc_fence_before();
            mbar_arrive(tempty_bar(acc));
            acc ^= 1;
            if (acc == 0) aph ^= 1u;
        }
    }

    linger_if_failed();
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------- 2-CTA kernel
// Pairs of CTAs (cluster of 2, on neighbouring SMs) share one 256 x 256 output tile with
// tcgen05.mma.cta_group::2: each CTA stages ITS 128 rows of A and ITS 128-wide half of B (32 KB per
// k-block instead of 48 KB), the leader CTA (cluster rank 0) issues M256 N256 K16 instructions
// that read both CTAs' shared memory and write 128 accumulator rows into each CTA's TMEM.
// Less shared-memory traffic per flop and a 6-deep ring in the same amount of shared memory.
//   * every TMA load of either CTA (each CTA fetches its own tiles) reports its bytes to the LEADER's stage
//     barrier, which the leader arms with the bytes of both CTAs;
//   * "stage free" and "accumulator ready" are committed by the leader to its own barrier and,
//     with a second tcgen05.commit, to the peer's barrier at the same offset;
//   * "accumulator drained" arrives on the leader's barrier from the epilogue warps of both CTAs.
// Seven warps per CTA: TMA producer, MMA issuer (leader only), four epilogue warps (tensor memory -> registers ->
// swizzled pieces in shared memory -> tensor-map stores), and a scheduler warp that is idle with the default static
// schedule (unit u of cluster c is c + u * clusters) and hands out work units with the dynamic one (see clc_try_cancel).
// All waits are bounded as in the 1-CTA kernel.
struct Pair {
    static constexpr int TN = 256;                             // tile width
    static constexpr int kStages = 6;
    static constexpr int kABytes = 128 * BK * 2;               // this CTA's 128 rows of A
    static constexpr int kBBytes = (TN / 2) * BK * 2;          // this CTA's half of the TN output columns of B
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kOutBytes = 4 * 2 * 4096;             // epilogue staging: per epilogue warp two 32 x 64 bf16 pieces
    static constexpr int kSmemBytes = kStages * kStageBytes + kOutBytes + 1024 + 512;
    static constexpr int kThreads = 224;                       // producer, MMA issuer, 4 epilogue warps, tile scheduler
    static constexpr int kUnitSlots = 4;                       // work units handed out ahead of their use (dynamic schedule)
};

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Cluster launch control: a running cluster asks the hardware for the launch of a cluster of this grid that has not
// started yet; if there is one, that cluster never starts and its first CTA's index comes back (16 bytes written to
// shared memory, counted on an mbarrier), so the asking cluster does that work unit itself.  With a grid of one
// cluster per unit this is a persistent kernel whose units go to whichever cluster is free: a cluster that starts late
// or shares its SMs with another kernel (a collective on another stream) simply takes fewer units.
__device__ __forceinline__ void clc_try_cancel(uint32_t resp, uint32_t bar)
{
    asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
                 ::"r"(resp), "r"(bar) : "memory");
}
// blockIdx.x of the first CTA of the cluster whose launch was taken over, or -1 when none was left
__device__ __forceinline__ int clc_result(uint32_t resp)
{
    uint32_t x, ok;
    asm volatile("{\n\t"
                 ".reg .pred p;\n\t"
                 ".reg .b128 r;\n\t"
                 "ld.shared.b128 r, [%2];\n\t"
                 "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, r;\n\t"
                 "selp.u32 %1, 1, 0, p;\n\t"
                 "mov.u32 %0, 0;\n\t"
                 "@p clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %0, r;\n\t"
                 "}"
                 : "=r"(x), "=r"(ok) : "r"(resp) : "memory");
    return ok ? (int)x : -1;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v)
{
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// Bounded wait whose acquire covers writes made from the other CTA of the cluster before its (cluster-scope) arrive.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int code)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (i > 64) {
            __nanosleep(40);
            if ((i & 255u) == 0u && *(volatile int *)&g_gemm_status != 0) return false;
        }
    }
    atomicCAS(&g_gemm_status, 0, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tc_commit2(uint32_t bar_cluster)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}
// The 64-bit shared-memory descriptor as two words.  Only the 14-bit start-address field of the low word changes from
// one MMA to the next (stage and K step), so the issuing thread keeps the words of stage 0 / K step 0 in registers and
// ADDS (byte offset >> 4) to the low word: one integer add per operand per MMA instead of rebuilding the descriptor.
// (Shared memory ends below 256 KB, so the sum never carries out of the field.)
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo) { return ((addr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16); }
__device__ __forceinline__ uint32_t desc_hi(uint32_t sbo) { return (sbo >> 4) | (1u << 14) | (2u << 29); }
template <bool kTf32 = false>
__device__ __forceinline__ void tc_mma2_words(uint32_t tmem_d, uint32_t alo, uint32_t ahi, uint32_t blo, uint32_t bhi,
                                              uint32_t idesc, uint32_t accumulate)
{
    if (kTf32)
        asm volatile("{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %6, 0;\n mov.b64 da, {%1, %2};\n mov.b64 db, {%3, %4};\n"
                     " tcgen05.mma.cta_group::2.kind::tf32 [%0], da, db, %5, p;\n}"
                     ::"r"(tmem_d), "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %6, 0;\n mov.b64 da, {%1, %2};\n mov.b64 db, {%3, %4};\n"
                     " tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n}"
                     ::"r"(tmem_d), "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_mma2(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// Drains one 128 x 256 fp32 accumulator to a bf16 C through shared memory and the TMA unit: this warp owns 32 rows;
// per 64 columns each thread converts its row's 64 values, writes them as eight 16-byte pieces into a 128-byte-swizzled
// 32 x 128 B piece (two pieces per warp, alternating), and one lane hands the piece to a tensor-map store, which writes
// whole 128-byte lines and drops rows and columns outside C.  (The direct path stores 16 bytes per thread and row: 32
// half-used sectors per instruction.)  Returns after the last tensor-memory read; the stores finish asynchronously.
__device__ __forceinline__ void epilogue_tile_tma(const Params &p, const CUtensorMap *map_c, uint32_t taddr, uint32_t stag,
                                                  int m_row0, int n0, int lane, uint32_t &piece)
{
#pragma unroll 1
    for (int cc = 0; cc < 4; ++cc) {
        const int col0 = n0 + cc * 64;
        if (col0 >= p.N || m_row0 >= p.M) break;                 // nothing of this piece lies inside C
        uint32_t r0[32], r1[32];
        AXS6_TMEM_LD32(taddr + (uint32_t)(cc * 64), r0);
        AXS6_TMEM_LD32(taddr + (uint32_t)(cc * 64 + 32), r1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        uint32_t w[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            float v0 = __uint_as_float(r0[i]), v1 = __uint_as_float(r0[i + 1]);
            float u0 = __uint_as_float(r1[i]), u1 = __uint_as_float(r1[i + 1]);
            if (p.bias) {
                float b0 = col0 + i < p.N ? __ldg(p.bias + col0 + i) : 0.0f, b1 = col0 + i + 1 < p.N ? __ldg(p.bias + col0 + i + 1) : 0.0f;
                float c0 = col0 + 32 + i < p.N ? __ldg(p.bias + col0 + 32 + i) : 0.0f;
                float c1 = col0 + 33 + i < p.N ? __ldg(p.bias + col0 + 33 + i) : 0.0f;
                if (p.bias_bf16) {
                    b0 = __bfloat162float(__float2bfloat16_rn(b0)); b1 = __bfloat162float(__float2bfloat16_rn(b1));
                    c0 = __bfloat162float(__float2bfloat16_rn(c0)); c1 = __bfloat162float(__float2bfloat16_rn(c1));
                }
                v0 += b0; v1 += b1; u0 += c0; u1 += c1;
            }
            const __nv_bfloat162 h0 = __floats2bfloat162_rn(v0, v1), h1 = __floats2bfloat162_rn(u0, u1);
            w[i >> 1] = *reinterpret_cast<const uint32_t *>(&h0);
            w[16 + (i >> 1)] = *reinterpret_cast<const uint32_t *>(&h1);
        }
        const uint32_t buf = stag + (piece & 1u) * 4096u;
        // the store issued two pieces ago read this buffer: it must have finished reading before it is overwritten
        if (lane == 0) acp::bulk_wait_read<1>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t addr = buf + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * j]), "r"(w[4 * j + 1]), "r"(w[4 * j + 2]),
                         "r"(w[4 * j + 3]) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            acp::tma_store_2d(map_c, buf, col0, m_row0);
            acp::bulk_commit();
        }
        ++piece;
    }
}

// The same for an fp32 C: a piece is 32 rows x 32 columns (128 B per row).  `how`: 0 store into C, 1 add into the
// zero-filled C (a partial product of a split contraction; the adds are done by the memory system, and with two
// addends per element their order does not matter), 2 store into slice `part` of the split-K workspace (3-D map).
__device__ __forceinline__ void epilogue_tile_tma_f32(const Params &p, const CUtensorMap *map, uint32_t taddr, uint32_t stag,
                                                      int m_row0, int n0, int lane, uint32_t &piece, int how, int part,
                                                      bool add_bias)
{
#pragma unroll 1
    for (int cc = 0; cc < 8; ++cc) {
        const int col0 = n0 + cc * 32;
        if (col0 >= p.N || m_row0 >= p.M) break;
        uint32_t w[32];
        AXS6_TMEM_LD32(taddr + (uint32_t)(cc * 32), w);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (p.bias && add_bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float bv = col0 + i < p.N ? __ldg(p.bias + col0 + i) : 0.0f;
                w[i] = __float_as_uint(__uint_as_float(w[i]) + (p.bias_bf16 ? __bfloat162float(__float2bfloat16_rn(bv)) : bv));
            }
        }
        const uint32_t buf = stag + (piece & 1u) * 4096u;
        if (lane == 0) acp::bulk_wait_read<1>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t addr = buf + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * j]), "r"(w[4 * j + 1]), "r"(w[4 * j + 2]),
                         "r"(w[4 * j + 3]) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            if (how == 0) acp::tma_store_2d(map, buf, col0, m_row0);
            else if (how == 1) acp::tma_reduce_add_2d(map, buf, col0, m_row0);
            else acp::tma_store_3d(map, buf, col0, m_row0, part);
            acp::bulk_commit();
        }
        ++piece;
    }
}

template <bool kTf32>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Pair::kThreads, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_ws, const Params p)
{
    constexpr int TN = Pair::TN;
    constexpr int kBK = kTf32 ? 32 : 64;                // values per k-block (128 bytes per row either way)
    constexpr int kStages2 = Pair::kStages, kA2Bytes = Pair::kABytes, kStage2Bytes = Pair::kStageBytes;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t stag0 = base + kStages2 * kStage2Bytes;             // epilogue staging (1024-aligned)
    const uint32_t bar0 = stag0 + Pair::kOutBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages2 + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages2 + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages2 + 2 + a); };
    const uint32_t tmem_slot = bar0 + 8u * (2 * kStages2 + 4);
    // dynamic schedule: a ring of kUnitSlots unit numbers, each with a "published" barrier (in both CTAs) and a "read by
    // every role of both CTAs" barrier (the leader's is the one used); one barrier and 16 bytes for the launch-control answer
    constexpr int kSlots = Pair::kUnitSlots;
    const uint32_t sched0 = bar0 + 8u * (2 * kStages2 + 5);
    auto sfull_bar = [&](int i) { return sched0 + 8u * i; };
    auto sempty_bar = [&](int i) { return sched0 + 8u * (kSlots + i); };
    const uint32_t clc_bar = sched0 + 8u * (2 * kSlots);
    const uint32_t clc_resp = (clc_bar + 8u + 15u) & ~15u;
    const uint32_t unit_slot0 = clc_resp + 16u;
    uint8_t *smem_gen = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(smem_gen + kStages2 * kStage2Bytes + Pair::kOutBytes + 8 * (2 * kStages2 + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 = leader
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    const int tiles_m = (p.M + 255) / 256, tiles_n = (p.N + TN - 1) / TN;
    // Work units.  With splits == 1 and no tail (p.tail_begin == 0) every tile is one unit.  Tiles from tail_begin on (the
    // ones that would otherwise form a last, partly filled wave) are two units each, one per half of the
    // contraction, accumulated into the zero-filled output with red.add; with two addends the sum does not
    // depend on their order.  p.splits > 1 splits every tile instead.
    const int splits = p.splits;
    const int total_kb = (p.K + kBK - 1) / kBK;
    const int all_tiles = tiles_m * tiles_n;
    const int tail_begin = splits > 1 ? 0 : ((p.tail_begin <= 0 || p.tail_begin > all_tiles) ? all_tiles : p.tail_begin);
    const int tail_parts = splits > 1 ? splits : 2;
    const int num_tiles = tail_begin + (all_tiles - tail_begin) * tail_parts;
    auto unit_tile = [&](int t) { return t < tail_begin ? t : tail_begin + (t - tail_begin) / tail_parts; };
    auto unit_part = [&](int t) { return t < tail_begin ? 0 : (t - tail_begin) % tail_parts; };
    auto unit_split = [&](int t) { return t >= tail_begin; };
    auto kb_begin = [&](int t) { return unit_split(t) ? (int)(((long long)unit_part(t) * total_kb) / tail_parts) : 0; };
    auto kb_end = [&](int t) { return unit_split(t) ? (int)(((long long)(unit_part(t) + 1) * total_kb) / tail_parts) : total_kb; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        // accumulator drained: one arrival per epilogue warp of both CTAs (on the leader's barrier)
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
        // a unit number is read by the producer and the 4 epilogue warps of each CTA and by the MMA issuer of the
        // leader; every reader arrives on its OWN CTA's "read" barrier (a CTA-scope arrive: a cluster-scope release
        // in the thread that issues the MMAs waits for the products in flight), and the peer's forwarding thread
        // passes the peer's five on to the leader's barrier as one arrival: 6 + 1 there, 5 in the peer
        for (int i = 0; i < kSlots; ++i) { mbar_init(sfull_bar(i), 1); mbar_init(sempty_bar(i), cluster_ctarank() == 0 ? 7 : 5); }
        mbar_init(clc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // both CTAs' barriers exist before any remote signal
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    pdl_wait();                                          // barriers, tensor memory and descriptors are set up; caller memory from here on

    // The next work unit of this cluster, for one thread of a role; false = no more (or a wait gave up).
    // Static schedule: units cluster_id, cluster_id + num_clusters, ...  Dynamic: the numbers the scheduler publishes.
    auto next_unit = [&](int &t, int &slot, uint32_t &sph, bool &first) -> bool {
        if (!p.dynamic) {
            t = first ? cluster_id : t + num_clusters;
            first = false;
            return t < num_tiles;
        }
        // in the peer CTA the number was stored by the leader's scheduler thread through the cluster's shared window
        if (!(rank == 0 ? mbar_wait(sfull_bar(slot), sph, 10) : mbar_wait_cluster(sfull_bar(slot), sph, 10))) return false;
        asm volatile("ld.shared.s32 %0, [%1];" : "=r"(t) : "r"(unit_slot0 + 4u * (uint32_t)slot) : "memory");
        mbar_arrive(sempty_bar(slot));
        if (++slot == kSlots) { slot = 0; sph ^= 1u; }
        return t >= 0;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true, first = true;
            int t = 0, uslot = 0;
            uint32_t uph = 0;
            while (ok && next_unit(t, uslot, uph, first)) {
                const int tile = unit_tile(t);
                const int m0 = (tile / tiles_n) * 256 + (int)rank * 128;
                const int n0 = (tile % tiles_n) * TN + (int)rank * (TN / 2);
                for (int kb = kb_begin(t); kb < kb_end(t); ++kb) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, 1)) { ok = false; break; }
                    const uint32_t lead_full = map_to_cta(full_bar(s), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * kStage2Bytes);
                    const uint32_t sa = base + s * kStage2Bytes, sb = sa + kA2Bytes;
                    const int k0 = kb * kBK;
                    if (!p.a_mn) {
                        tma_load_2d_pair(sa, &map_a, lead_full, k0, m0);
                    } else if (p.a_mn4) {
                        tma_load_4d_pair(sa, &map_a, lead_full, 0, 0, m0 >> 6, k0 >> 3);
                    } else {
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * 8192, &map_a, lead_full, m0 + 64 * j, k0);
                    }
                    if (!p.b_mn) {
                        tma_load_2d_pair(sb, &map_b, lead_full, k0, n0);
                    } else if (p.b_mn4) {
                        tma_load_4d_pair(sb, &map_b, lead_full, 0, 0, n0 >> 6, k0 >> 3);
                    } else {
                        for (int j = 0; j < TN / 128; ++j) tma_load_2d_pair(sb + j * 8192, &map_b, lead_full, n0 + 64 * j, k0);
                    }
                    if (++s == kStages2) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            // M = 256 (>> 4 = 16) over the pair, N = TN
            constexpr uint32_t fmt = kTf32 ? 2u : 1u;   // operand format within the instruction kind: bf16 / tf32
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) |
                                   ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int s = 0, acc = 0;
            uint32_t ph = 0, aph = 0;
            bool ok = true;
            // descriptor words of stage 0, K step 0; per stage / K step only the low words move (see desc_lo)
            const uint32_t a_lo0 = desc_lo(base, p.a_lbo), b_lo0 = desc_lo(base + kA2Bytes, p.b_lbo);
            const uint32_t a_hi = desc_hi(p.a_sbo), b_hi = desc_hi(p.b_sbo);
            const uint32_t a_kinc = p.a_kstep >> 4, b_kinc = p.b_kstep >> 4;
            const uint32_t peer_empty0 = map_to_cta(empty_bar(0), 1);
            bool first = true;
            int t = 0, uslot = 0;
            uint32_t uph = 0;
            while (ok && next_unit(t, uslot, uph, first)) {
                if (!mbar_wait(tempty_bar(acc), aph ^ 1u, 2)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * TN);
                const int kb0 = kb_begin(t), kb1 = kb_end(t);
                uint32_t fresh = 0u;                                // 0 for the first product of the tile (overwrites the accumulator)
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(full_bar(s), ph, 3)) { ok = false; break; }
                    const uint32_t soff = (uint32_t)(s * kStage2Bytes) >> 4;
                    uint32_t alo = a_lo0 + soff, blo = b_lo0 + soff;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        tc_mma2_words<kTf32>(d_tmem, alo, a_hi, blo, b_hi, idesc, fresh);
                        fresh = 1u;
                        alo += a_kinc; blo += b_kinc;
                    }
                    tc_commit2(empty_bar(s));                       // frees the stage here ...
                    tc_commit2(peer_empty0 + 8u * (uint32_t)s);     // ... and in the peer
                    if (++s == kStages2) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                tc_commit2(tfull_bar(acc));
                tc_commit2(map_to_cta(tfull_bar(acc), 1));
                acc ^= 1;
                if (acc == 0) aph ^= 1u;
            }
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------------ unit scheduler (leader CTA, dynamic schedule)
        if (lane == 0 && rank == 1 && p.dynamic) {
            // peer: once its five readers have read a slot, tell the leader's scheduler (one cluster-scope arrival)
            int slot = 0;
            uint32_t ph = 0;
            for (;;) {
                int t;
                if (!mbar_wait_cluster(sfull_bar(slot), ph, 11)) break;
                asm volatile("ld.shared.s32 %0, [%1];" : "=r"(t) : "r"(unit_slot0 + 4u * (uint32_t)slot) : "memory");
                if (!mbar_wait(sempty_bar(slot), ph, 12)) break;
                mbar_arrive_cluster(map_to_cta(sempty_bar(slot), 0));
                if (t < 0) break;
                if (++slot == kSlots) { slot = 0; ph ^= 1u; }
            }
        }
        if (lane == 0 && rank == 0 && p.dynamic) {
            int slot = 0, cur = cluster_id;              // the cluster's own unit first
            uint32_t eph = 0, cph = 0;
            for (;;) {
                if (!mbar_wait(sempty_bar(slot), eph ^ 1u, 8)) break;
                const uint32_t sa = unit_slot0 + 4u * (uint32_t)slot;
                asm volatile("st.shared.s32 [%0], %1;" ::"r"(sa), "r"(cur) : "memory");
                st_cluster_u32(map_to_cta(sa, 1), (uint32_t)cur);
                mbar_arrive_cluster(map_to_cta(sfull_bar(slot), 0));
                mbar_arrive_cluster(map_to_cta(sfull_bar(slot), 1));
                if (++slot == kSlots) { slot = 0; eph ^= 1u; }
                if (cur < 0) break;                      // the end mark has been published
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(clc_bar, 16);
                clc_try_cancel(clc_resp, clc_bar);
                if (!mbar_wait(clc_bar, cph, 9)) break;
                cph ^= 1u;
                const int x = clc_result(clc_resp);
                cur = x < 0 ? -1 : (x >> 1);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int q = warp & 3;
        int acc = 0;
        uint32_t aph = 0, piece = 0;
        bool ok = true;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0) && (p.ldc % 8 == 0);
        bool first = true;
        int t = 0, uslot = 0;
        uint32_t uph = 0;
        while (ok) {
            int more = 0;
            if (lane == 0) more = next_unit(t, uslot, uph, first) ? 1 : 0;
            more = __shfl_sync(0xFFFFFFFFu, more, 0);
            t = __shfl_sync(0xFFFFFFFFu, t, 0);
            if (!more) break;
            const int tile = unit_tile(t);
            const int m0 = (tile / tiles_n) * 256 + (int)rank * 128, n0 = (tile % tiles_n) * TN;
            if (!mbar_wait(tfull_bar(acc), aph, 4)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * TN);
            if (p.c_tma == 1) {
                epilogue_tile_tma(p, &map_c, taddr, stag0 + (uint32_t)q * 8192u, m0 + q * 32, n0, lane, piece);
            } else if (p.c_tma == 2) {
                const bool acc_unit = unit_split(t), to_ws = acc_unit && p.ws != nullptr;
                epilogue_tile_tma_f32(p, to_ws ? &map_ws : &map_c, taddr, stag0 + (uint32_t)q * 8192u, m0 + q * 32, n0, lane, piece,
                                      to_ws ? 2 : (acc_unit ? 1 : 0), unit_part(t), !to_ws && unit_part(t) == 0);
            } else {
                epilogue_tile(p, taddr, row, n0, vec_ok, unit_split(t), unit_part(t) == 0, unit_part(t));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
            acc ^= 1;
            if (acc == 0) aph ^= 1u;
        }
        if (p.c_tma && lane == 0) acp::bulk_wait<0>();          // every tensor-map store of this warp has completed
    }

    linger_if_failed();
    pdl_launch_dependents();                             // this CTA has no more work to start: the next kernel may set up
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // the peer's shared memory and barriers stay alive until both are done
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------- 2-CTA kernel, 256 x 512 tiles
// Per k-block a pair of the kernel above fetches 64 KB (A 256 x 64 + B 256 x 64) for one 256 x 256 x 64 product.
// This variant gives a pair a 256 x 512 tile: the A tile of a k-block feeds TWO
// products (output columns 0..255 and 256..511), so a pair fetches 96 KB per two products = 48 KB per 256 x 256 x 64,
// a quarter less.  Price: the two 256-column accumulators fill tensor memory (512 columns), so there is no second
// accumulator set for the next tile; instead each accumulator has its own "ready" / "drained" barriers and its own
// group of four epilogue warps, the leader issues a k-block's products in the order accumulator 0, accumulator 1, and
// the first products of the next tile start as soon as accumulator 0 has been drained.
// Stage = A (128 rows) 16 KB + two B halves (128 columns each) 32 KB = 48 KB, 4 stages.  10 warps: producer, MMA
// issuer, epilogue group 0 (warps 2..5), epilogue group 1 (warps 6..9).  No split-K here (the launcher takes this
// kernel only when every tile is computed whole).
struct PairW {
    static constexpr int TN = 512;
    static constexpr int kStages = 4;
    static constexpr int kABytes = 128 * BK * 2;
    static constexpr int kBHalf = 128 * BK * 2;                // this CTA's 128 columns of one 256-column product
    static constexpr int kStageBytes = kABytes + 2 * kBHalf;   // 48 KB
    static constexpr int kThreads = 320;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairW::kThreads, 1)
gemm2w_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p)
{
    constexpr int S = PairW::kStages, kA = PairW::kABytes, kBH = PairW::kBHalf, kStage = PairW::kStageBytes, TN = PairW::TN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = base + S * kStage;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * S + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * S + 2 + a); };
    const uint32_t tmem_slot = bar0 + 8u * (2 * S + 4);
    uint8_t *smem_gen = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(smem_gen + S * kStage + 8 * (2 * S + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    const int tiles_m = (p.M + 255) / 256, tiles_n = (p.N + TN - 1) / TN;
    const int num_tiles = tiles_m * tiles_n;
    const int total_kb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    pdl_wait();                                          // barriers, tensor memory and descriptors are set up; caller memory from here on

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
                const int m0 = (t / tiles_n) * 256 + (int)rank * 128;
                const int nbase = (t % tiles_n) * TN + (int)rank * 128;      // product h uses columns nbase + 256 h .. + 127
                for (int kb = 0; kb < total_kb; ++kb) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, 1)) { ok = false; break; }
                    const uint32_t lead_full = map_to_cta(full_bar(s), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * kStage);
                    const uint32_t sa = base + s * kStage, sb = sa + kA;
                    const int k0 = kb * BK;
                    if (!p.a_mn) {
                        tma_load_2d_pair(sa, &map_a, lead_full, k0, m0);
                    } else {
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * 8192, &map_a, lead_full, m0 + 64 * j, k0);
                    }
                    for (int h = 0; h < 2; ++h) {
                        const int n0 = nbase + 256 * h;
                        if (!p.b_mn) {
                            tma_load_2d_pair(sb + h * kBH, &map_b, lead_full, k0, n0);
                        } else {
                            for (int j = 0; j < 2; ++j) tma_load_2d_pair(sb + h * kBH + j * 8192, &map_b, lead_full, n0 + 64 * j, k0);
                        }
                    }
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) |
                                   ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int s = 0;
            uint32_t ph = 0, aph = 0;
            bool ok = true;
            const uint32_t a_lo0 = desc_lo(base, p.a_lbo), b_lo0 = desc_lo(base + kA, p.b_lbo);
            const uint32_t a_hi = desc_hi(p.a_sbo), b_hi = desc_hi(p.b_sbo);
            const uint32_t a_kinc = p.a_kstep >> 4, b_kinc = p.b_kstep >> 4;
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
                for (int kb = 0; kb < total_kb && ok; ++kb) {
                    if (!mbar_wait(full_bar(s), ph, 3)) { ok = false; break; }
                    const uint32_t soff = (uint32_t)(s * kStage) >> 4;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        // the first products of a tile into accumulator h wait until the epilogue has drained it
                        if (kb == 0) {
                            if (!mbar_wait(tempty_bar(h), aph ^ 1u, 2)) { ok = false; break; }
                            tc_fence_after();
                        }
                        uint32_t alo = a_lo0 + soff, blo = b_lo0 + soff + (uint32_t)(h * kBH >> 4);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            tc_mma2_words(tmem_base + (uint32_t)(h * 256), alo, a_hi, blo, b_hi, idesc, (kb | k) != 0 ? 1u : 0u);
                            alo += a_kinc; blo += b_kinc;
                        }
                        if (kb == total_kb - 1) {              // accumulator h is complete with these products
                            tc_commit2(tfull_bar(h));
                            tc_commit2(map_to_cta(tfull_bar(h), 1));
                        }
                    }
                    if (!ok) break;
                    tc_commit2(empty_bar(s));
                    tc_commit2(map_to_cta(empty_bar(s), 1));
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                aph ^= 1u;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: group h = (warp - 2) / 4 drains accumulator h
        const int h = (warp - 2) >> 2;
        const int q = warp & 3;                          // TMEM lane quarter this warp may read
        uint32_t aph = 0;
        bool ok = true;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0) && (p.ldc % 8 == 0);
        for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
            const int m0 = (t / tiles_n) * 256 + (int)rank * 128, n0 = (t % tiles_n) * TN + 256 * h;
            if (!mbar_wait(tfull_bar(h), aph, 4)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * 256);
            epilogue_tile(p, taddr, row, n0, vec_ok, false, true);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(h), 0));
            aph ^= 1u;
        }
    }

    linger_if_failed();
    pdl_launch_dependents();                             // this CTA has no more work to start: the next kernel may set up
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

#include "gemm_packed_kernel.cuh"

// c (M, N) = sum over parts of ws[part] (+ bias), partials added in index order: the second half of a split-K
// product whose partials were kept apart, so that the result does not depend on the order in which CTAs finished.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ ws, int parts, long long ws_stride, int ws_ld,
                                                            float *__restrict__ c, long long ldc, const float *__restrict__ bias,
                                                            int bias_bf16, int M, int N)
{
    pdl_wait();
    const int chunks = ws_ld / 4;
    const long long total = (long long)M * chunks;
    const bool vec = ((reinterpret_cast<uintptr_t>(c) & 15u) == 0) && (ldc % 4 == 0);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / chunks), col = (int)(i - (long long)row * chunks) * 4;
        float4 acc = *reinterpret_cast<const float4 *>(ws + (long long)row * ws_ld + col);
        for (int s = 1; s < parts; ++s) {
            const float4 v = *reinterpret_cast<const float4 *>(ws + s * ws_stride + (long long)row * ws_ld + col);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        float o[4] = {acc.x, acc.y, acc.z, acc.w};
        if (bias) {
            for (int j = 0; j < 4; ++j)
                if (col + j < N) {
                    const float bv = bias[col + j];
                    o[j] += bias_bf16 ? __bfloat162float(__float2bfloat16_rn(bv)) : bv;
                }
        }
        float *dst = c + (long long)row * ldc + col;
        if (vec && col + 4 <= N) {
            *reinterpret_cast<float4 *>(dst) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
            for (int j = 0; j < 4; ++j)
                if (col + j < N) dst[j] = o[j];
        }
    }
}

// ------------------------------------------------------------------------------------- host
using acp::EncodeTiledFn;
using acp::encode_fn;

// 2-D tensor map over rows of `inner` contiguous values (`esize` bytes each, `ld` values apart):
// box = {128 bytes, box_rows}, 128-byte swizzle, out-of-bounds reads give zeros.
static bool make_map(CUtensorMap *map, const void *ptr, int esize, uint64_t inner, uint64_t rows, uint64_t ld,
                     uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t gdim[2] = {inner, rows};
    const cuuint64_t gstride[1] = {ld * (uint64_t)esize};
    const cuuint32_t box[2] = {(cuuint32_t)(128 / esize), box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
              const_cast<void *>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}



// MN-major bf16 operand (`k_rows` rows of `mn` contiguous values, `ld` values apart) for the CTA-pair kernel, as a 4-D
// view whose box is a whole 128 x 64 stage tile: dim 0 = 64 values (one 128-byte swizzle row), dim 1 = 8 consecutive
// k-rows, dim 2 = 64-value chunk along MN, dim 3 = group of 8 k-rows; box {64, 8, 2, 8}.  In shared memory the 1 KB
// swizzle atoms then lie [k-group][MN chunk]: the two chunks that one MMA reads for a k-group are adjacent (descriptor
// strides: 1 KB between MN chunks, 2 KB between k-groups, 4 KB per K step of 16) and the tile arrives with ONE copy
// instead of two.  Needs mn % 64 == 0 and k_rows % 8 == 0 so that coordinates past the edges fall outside the view
// (zero fill) instead of wrapping into the next row.
static bool make_mn4_map(CUtensorMap *map, const void *ptr, uint64_t mn, uint64_t k_rows, uint64_t ld)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn || mn % 64 != 0 || k_rows % 8 != 0) return false;
    const cuuint64_t gdim[4] = {64, 8, mn / 64, k_rows / 8};
    const cuuint64_t gstride[3] = {ld * 2, 128, 8 * ld * 2};
    const cuuint32_t box[4] = {64, 8, 2, 8};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMap tmp;
    if (fn(&tmp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(ptr), gdim, gstride, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;                                   // the caller keeps its 2-D map
    *map = tmp;
    return true;
}

// SMs the GEMM may use: all of them, minus the reserve of tune key 8 (left to a collective on another stream).
static int64_t usable_sms(const DeviceInfo &d)
{
    const int64_t r = tune_value(8);
    return d.sms - (r > 0 && r < d.sms - 2 ? r : 0);
}

// 2-D tensor map over a plane of payload bytes: rows of `pitch` bytes, box = {box_bytes, box_rows}, no swizzle,
// bytes outside the plane read as zero.
static bool make_byte_map(CUtensorMap *map, const void *ptr, uint64_t pitch, uint64_t rows, uint32_t box_bytes, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t gdim[2] = {pitch, rows};
    const cuuint64_t gstride[1] = {pitch};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), gdim, gstride, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// C = op(A) op(B) where an operand with a non-null exponent plane is held as AXS-6 codes in the split layout
// (blocks of 32 along its contiguous dimension) and decoded to bf16 inside the kernel.
static int launch_gemm_packed(const void *a, const void *a_exps, int64_t lda, const void *b, const void *b_exps, int64_t ldb,
                              void *c, const float *bias, int64_t M, int64_t N, int64_t K, int64_t ldc, int a_mn, int b_mn,
                              int c_dtype, int bias_via_bf16, cudaStream_t stream)
{
    if (M < 0 || N < 0 || K < 0 || (a_mn & ~1) || (b_mn & ~1) || !valid_dtype(c_dtype)) return AXS6_ERR_ARG;
    if (M == 0 || N == 0) return AXS6_OK;
    if (!a || !b || !c || K == 0 || ldc < N) return AXS6_ERR_ARG;
    if (!a_exps && !b_exps) return AXS6_ERR_ARG;                 // nothing packed: axs6_gemm_bf16 is the entry point
    if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return AXS6_ERR_UNSUPPORTED;
    if (!aligned16(a) || !aligned16(b) || (a_exps && !aligned16(a_exps)) || (b_exps && !aligned16(b_exps))) return AXS6_ERR_ALIGN;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;
    // stored shape of each operand: (rows, cols) with cols contiguous
    const int64_t a_rows = a_mn ? K : M, a_cols = a_mn ? M : K;
    const int64_t b_rows = b_mn ? K : N, b_cols = b_mn ? N : K;
    CUtensorMap ma, mb;
    PackedParams q;
    q.a_exps = static_cast<const uint8_t *>(a_exps); q.b_exps = static_cast<const uint8_t *>(b_exps);
    q.a_nblk = (int)(a_cols / 32); q.b_nblk = (int)(b_cols / 32);
    q.a_rows = (int)a_rows; q.b_rows = (int)b_rows;
    q.gather_arrivals = tune_value(9) == 1 ? 0 : 1;
    bool ok = true;
    if (a_exps) {
        if (a_cols % 64 || a_rows % 8) return AXS6_ERR_UNSUPPORTED;   // payload rows and exponent runs must be 16-byte multiples
        ok = ok && make_byte_map(&ma, a, (uint64_t)a_cols * 3 / 4, (uint64_t)a_rows, a_mn ? 96 : 48, a_mn ? 64 : 128);
    } else {
        if (lda < a_cols) return AXS6_ERR_ARG;
        if ((lda * 2) % 16) return AXS6_ERR_ALIGN;
        ok = ok && (a_mn ? make_map(&ma, a, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BK)
                         : make_map(&ma, a, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 128));
    }
    if (b_exps) {
        if (b_cols % 64 || b_rows % 8) return AXS6_ERR_UNSUPPORTED;
        ok = ok && make_byte_map(&mb, b, (uint64_t)b_cols * 3 / 4, (uint64_t)b_rows, b_mn ? 96 : 48, b_mn ? 64 : 128);
    } else {
        if (ldb < b_cols) return AXS6_ERR_ARG;
        if ((ldb * 2) % 16) return AXS6_ERR_ALIGN;
        ok = ok && (b_mn ? make_map(&mb, b, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, BK)
                         : make_map(&mb, b, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 128));
    }
    if (!ok) return AXS6_ERR_DEVICE;

    Params p = {};
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.a_mn = a_mn; p.b_mn = b_mn;
    p.c = c; p.ldc = ldc; p.c_bf16 = (c_dtype == AXS6_BF16) ? 1 : 0;
    p.bias = bias; p.bias_bf16 = bias_via_bf16;
    p.tiles_m = (int)((M + BM - 1) / BM); p.tiles_n = (int)((N + BN - 1) / BN);
    p.bk = BK; p.mn_box_bytes = 128u * BK; p.splits = 1; p.tail_begin = 0;
    p.ws = nullptr; p.ws_stride = 0; p.ws_ld = 0;
    p.c_tma = 0;

    p.a_lbo = a_mn ? p.mn_box_bytes : 0u; p.a_sbo = 1024u; p.a_kstep = a_mn ? 16u * 128u : 32u;
    p.b_lbo = b_mn ? p.mn_box_bytes : 0u; p.b_sbo = 1024u; p.b_kstep = b_mn ? 16u * 128u : 32u;

    const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
    const int64_t usable = usable_sms(d);
    const int clusters = (int)(pair_tiles < usable / 2 ? pair_tiles : usable / 2);
    const void *kern = a_exps && b_exps ? reinterpret_cast<const void *>(&gemm2q_kernel<true, true>)
                       : a_exps        ? reinterpret_cast<const void *>(&gemm2q_kernel<true, false>)
                                       : reinterpret_cast<const void *>(&gemm2q_kernel<false, true>);
    if (!ensure_dynamic_smem(kern, PairQ::kSmemBytes)) return AXS6_ERR_LAUNCH;
    if (a_exps && b_exps) gemm2q_kernel<true, true><<<2 * clusters, kThreadsPacked, PairQ::kSmemBytes, stream>>>(ma, mb, p, q);
    else if (a_exps)      gemm2q_kernel<true, false><<<2 * clusters, kThreadsPacked, PairQ::kSmemBytes, stream>>>(ma, mb, p, q);
    else                  gemm2q_kernel<false, true><<<2 * clusters, kThreadsPacked, PairQ::kSmemBytes, stream>>>(ma, mb, p, q);
    count_launch();
    return check_launch();
}

// Split-K plan for a problem with few output tiles and a long contraction (fp32 output): how many K ranges per tile
// so that most SMs get a work unit.  `cap` bounds the number of partials.
static int64_t plan_pair_splits(const DeviceInfo &d, int64_t M, int64_t N, int64_t K, int64_t cap, int64_t bk)
{
    const int64_t pair_tiles = ((M + 255) / 256) * ((N + Pair::TN - 1) / Pair::TN);
    if (pair_tiles >= d.sms / 2) return 1;
    const int64_t total_kb = (K + bk - 1) / bk;
    int64_t splits = (d.sms / 2) / pair_tiles;
    if (splits > total_kb / 16) splits = total_kb / 16;
    if (splits > cap) splits = cap;
    return splits < 1 ? 1 : splits;
}

static int64_t ws_ld_of(int64_t N) { return (N + 3) / 4 * 4; }

template <bool kTf32>
static int launch_gemm(const void *a, const void *b, void *c, const float *bias, int64_t M, int64_t N, int64_t K,
                       int64_t lda, int64_t ldb, int64_t ldc, int a_mn, int b_mn, int c_dtype, int bias_via_bf16,
                       cudaStream_t stream, void *ws = nullptr, int64_t ws_bytes = 0)
{
    constexpr int esize = kTf32 ? 4 : 2;
    constexpr int bk = 128 / esize;                     // values per k-block
    if (M < 0 || N < 0 || K < 0 || (a_mn & ~1) || (b_mn & ~1) || !valid_dtype(c_dtype)) return AXS6_ERR_ARG;
    if (M == 0 || N == 0) return AXS6_OK;
    if (!a || !b || !c || K == 0) return AXS6_ERR_ARG;
    if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return AXS6_ERR_UNSUPPORTED;
    if (lda < (a_mn ? M : K) || ldb < (b_mn ? N : K) || ldc < N) return AXS6_ERR_ARG;
    if (!aligned16(a) || !aligned16(b) || (lda * esize) % 16 || (ldb * esize) % 16) return AXS6_ERR_ALIGN;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;

    // Split policy (fp32 output only; partial products are added into the zero-filled output with red.add).
    // Built-in: at most TWO partials per output element, whose sum does not depend on their order, so every
    // result is bit-reproducible.  Tune key 3: 1 = never split, 2 = two-way split of every tile of the CTA-pair
    // kernel, 3 = allow up to 8 (pairs) / 16 (single CTA) partials, added in no fixed order (last bits can
    // differ from run to run).
    const int64_t split_mode = tune_value(3);
    const int64_t max_pair_splits = split_mode == 3 ? 8 : 2, max_cta_splits = split_mode == 3 ? 16 : 2;
    const bool may_split = c_dtype == AXS6_F32 && split_mode != 1;

    // bf16: CTA pairs on 256 x 256 tiles (tune key 7: 1 forces the single-CTA kernel, 2 forces pairs).
    // Fewer pair tiles than clusters: pairs still win over the single-CTA kernel when at least a quarter of the
    // clusters get a tile (a pair reads a third fewer bytes per flop from L2, and the single-CTA kernel on
    // 4096 x 1024 x 8192 was bound by that feed), or when the contraction can be split so that more clusters
    // get a unit (weight gradients of small layers).
    const int64_t pair_tiles = ((M + 255) / 256) * ((N + Pair::TN - 1) / Pair::TN);
    const int64_t mode = tune_value(7);
    int64_t pair_splits = 1;
    bool use_ws = false;
    if (may_split) {
        pair_splits = plan_pair_splits(d, M, N, K, max_pair_splits, bk);
        // With a workspace the partials are kept apart and added in a fixed order by a second kernel: more than two
        // partials without giving up reproducibility.
        if (ws && aligned16(ws) && split_mode != 2) {
            const int64_t want = plan_pair_splits(d, M, N, K, 8, bk);
            if (want > 2 && ws_bytes >= want * M * ws_ld_of(N) * 4) { pair_splits = want; use_ws = true; }
        }
    }
    // (the TF32 instruction takes K-major operands only, and so does its CTA-pair instantiation)
    const bool pairs = !(kTf32 && (a_mn || b_mn)) && mode != 1 && (mode == 2 || mode == 3 || pair_tiles * pair_splits >= d.sms / 4);

    CUtensorMap ma, mb;
    const bool oka = a_mn ? make_map(&ma, a, esize, (uint64_t)M, (uint64_t)K, (uint64_t)lda, bk)
                          : make_map(&ma, a, esize, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BM);
    const bool okb = b_mn ? make_map(&mb, b, esize, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, bk)
                          : make_map(&mb, b, esize, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, pairs ? Pair::TN / 2 : BN);
    if (!oka || !okb) return AXS6_ERR_DEVICE;

    Params p = {};
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.a_mn = a_mn; p.b_mn = b_mn;
    p.c = c; p.ldc = ldc; p.c_bf16 = (c_dtype == AXS6_BF16) ? 1 : 0;
    p.bias = bias;
    p.bias_bf16 = bias_via_bf16;
    p.tiles_m = (int)((M + BM - 1) / BM);
    p.tiles_n = (int)((N + BN - 1) / BN);
    p.bk = bk;
    p.mn_box_bytes = 128u * bk;
    p.splits = 1;
    p.tail_begin = 0;
    p.ws = nullptr; p.ws_stride = 0; p.ws_ld = 0;
    p.c_tma = 0;
    p.a_mn4 = p.b_mn4 = 0;
    // K-major, 128-byte swizzle: 8-row groups are 1024 B apart, one MMA K step is 32 B.
    // MN-major: 128-byte chunks of the output index are one TMA box (bk k-rows x 128 B) apart,
    // groups of 8 k-rows 1024 B apart, one MMA K step (32 B / esize rows) is that many rows x 128 B.
    const uint32_t mn_kstep = (32u / esize) * 128u;
    p.a_lbo = a_mn ? p.mn_box_bytes : 0u; p.a_sbo = 1024u; p.a_kstep = a_mn ? mn_kstep : 32u;
    p.b_lbo = b_mn ? p.mn_box_bytes : 0u; p.b_sbo = 1024u; p.b_kstep = b_mn ? mn_kstep : 32u;

    if (pairs) {
        if (may_split && split_mode == 2 && K >= 16 * bk) p.splits = 2;
        if (pair_splits > 1) p.splits = (int)pair_splits;
        // 256 x 512 tiles (a quarter less operand feed per flop): taken when no split is planned and the wider tiles fill
        // their waves of clusters about as well as the 256 x 256 ones (tune key 7: 3 forces them, 2 forbids them)
        {
            const int64_t usable_c = usable_sms(d) / 2;
            const int64_t wide_tiles = ((M + 255) / 256) * ((N + PairW::TN - 1) / PairW::TN);
            auto fill = [&](int64_t tiles) { return (double)tiles / (double)(((tiles + usable_c - 1) / usable_c) * usable_c); };
            // work per tile differs by 2: compare time = waves x tile time
            const double t_narrow = (double)((pair_tiles + usable_c - 1) / usable_c) * 1.0;
            const double t_wide = (double)((wide_tiles + usable_c - 1) / usable_c) * 2.0 * 0.85;     // 0.85: measured gain per flop
            // measured: the wide tile pays only for long contractions (16384 x 4096 x 4096 equal; dW with K = 16384 +4 %,
            // K = 32000 +8 %; K = 1024 is 30 % slower because its two accumulators are drained one tile at a time)
            bool wide = !kTf32 && p.splits == 1 && mode != 2 && wide_tiles >= usable_c && t_wide <= t_narrow && N > 256 && K >= 8192;
            if (p.splits == 1 && may_split && K >= 32 * bk && pair_tiles > usable_c) {
                const int64_t rem = pair_tiles % usable_c;
                if (rem > 0 && 2 * rem <= usable_c) wide = wide && fill(wide_tiles) >= 0.9;      // the tail split would help the narrow kernel
            }
            if (mode == 3 && p.splits == 1 && N > 256 && !kTf32) wide = true;
            if (wide) {
                if (!ensure_dynamic_smem(reinterpret_cast<const void *>(&gemm2w_kernel), PairW::kSmemBytes)) return AXS6_ERR_LAUNCH;
                const int clusters = (int)(wide_tiles < usable_c ? wide_tiles : usable_c);
                if (launch_overlapped(true, gemm2w_kernel, 2 * clusters, PairW::kThreads, PairW::kSmemBytes, stream, ma, mb, p) != cudaSuccess) return AXS6_ERR_LAUNCH;
                count_launch();
                return check_launch();
            }
        }
        if (!ensure_dynamic_smem(reinterpret_cast<const void *>(&gemm2_kernel<kTf32>), Pair::kSmemBytes)) return AXS6_ERR_LAUNCH;
        if (!kTf32 && tune_value(4) != 1) {
            if (a_mn && make_mn4_map(&ma, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda)) {
                p.a_mn4 = 1; p.a_lbo = 1024u; p.a_sbo = 2048u; p.a_kstep = 4096u;
            }
            if (b_mn && make_mn4_map(&mb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb)) {
                p.b_mn4 = 1; p.b_lbo = 1024u; p.b_sbo = 2048u; p.b_kstep = 4096u;
            }
        }
        const int64_t units = pair_tiles * p.splits;
        const int64_t usable = usable_sms(d);
        const int clusters = (int)(units < usable / 2 ? units : usable / 2);
        // Tail split (long contraction): when the last wave of tiles would be at most half full, its tiles are
        // computed as two K halves each, so that wave takes half the time.  Weight gradient 4096 x 4096 x 16384:
        // 256 tiles on 74 clusters, 3 full waves + 34 tiles -> 68 half units: 3.5 waves instead of 4.  The rows
        // that hold those tiles are zero-filled first.
        if (p.splits == 1 && may_split && K >= 32 * bk && pair_tiles > clusters) {
            const int64_t rem = pair_tiles % clusters;
            if (rem > 0 && 2 * rem <= clusters) {
                p.tail_begin = (int)(pair_tiles - rem);
                const int64_t tiles_n2 = (N + Pair::TN - 1) / Pair::TN;
                const int64_t row0 = (p.tail_begin / tiles_n2) * 256;
                if (cudaMemset2DAsync(static_cast<float *>(c) + row0 * ldc, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)(M - row0),
                                      stream) != cudaSuccess)
                    return AXS6_ERR_LAUNCH;
            }
        }
        if (use_ws && p.splits > 2) {
            p.ws = static_cast<float *>(ws); p.ws_ld = (int)ws_ld_of(N); p.ws_stride = (long long)M * p.ws_ld;
        } else if (p.splits > 1 &&
                   cudaMemset2DAsync(c, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, stream) != cudaSuccess) {
            return AXS6_ERR_LAUNCH;
        }
        // One cluster per work unit and units taken over through cluster launch control (tune key 6 = 1), unless SMs
        // are to be left free (tune key 8), which only a fixed number of clusters can do
        const int64_t dyn_units = p.tail_begin > 0 ? p.tail_begin + (pair_tiles - p.tail_begin) * 2 : pair_tiles * p.splits;
        p.dynamic = (tune_value(6) == 1 && usable == d.sms && dyn_units > clusters && 2 * dyn_units < (1ll << 30)) ? 1 : 0;
        // Output into an aligned C (and an aligned split-K workspace): the epilogue stores through shared memory and
        // tensor maps
        CUtensorMap mc, mw;
        memset(&mc, 0, sizeof(mc));
        memset(&mw, 0, sizeof(mw));
        p.c_tma = 0;
        if (aligned16(c) && tune_value(5) != 1) {
            EncodeTiledFn fn = encode_fn();
            const cuuint32_t estr[3] = {1, 1, 1};
            if (c_dtype == AXS6_BF16 && ldc % 8 == 0) {
                const cuuint64_t gdim[2] = {(cuuint64_t)N, (cuuint64_t)M};
                const cuuint64_t gstride[1] = {(cuuint64_t)ldc * 2};
                const cuuint32_t box[2] = {64, 32};
                if (fn && fn(&mc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
                    p.c_tma = 1;
            } else if (c_dtype == AXS6_F32 && ldc % 4 == 0 && (!p.ws || (aligned16(p.ws) && p.ws_ld % 4 == 0 && p.ws_stride % 4 == 0))) {
                const cuuint64_t gdim[2] = {(cuuint64_t)N, (cuuint64_t)M};
                const cuuint64_t gstride[1] = {(cuuint64_t)ldc * 4};
                const cuuint32_t box[2] = {32, 32};
                bool ok = fn && fn(&mc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, c, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
                if (ok && p.ws) {
                    const cuuint64_t wdim[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)p.splits};
                    const cuuint64_t wstride[2] = {(cuuint64_t)p.ws_ld * 4, (cuuint64_t)p.ws_stride * 4};
                    const cuuint32_t wbox[3] = {32, 32, 1};
                    ok = fn(&mw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, p.ws, wdim, wstride, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
                }
                if (ok) p.c_tma = 2;
            }
        }
        if (launch_overlapped(true, gemm2_kernel<kTf32>, (unsigned)(p.dynamic ? 2 * dyn_units : 2 * clusters), Pair::kThreads, Pair::kSmemBytes, stream, ma, mb, mc, mw, p) != cudaSuccess) return AXS6_ERR_LAUNCH;
        count_launch();
        if (p.ws) {
            const long long chunks = (long long)M * (p.ws_ld / 4);
            int64_t ctas = (chunks + 255) / 256;
            if (ctas > (int64_t)d.sms * 8) ctas = (int64_t)d.sms * 8;
            if (launch_overlapped(true, splitk_reduce_kernel, (unsigned)ctas, 256, 0, stream, (const float *)p.ws, p.splits, p.ws_stride,
                                  p.ws_ld, static_cast<float *>(c), (long long)ldc, bias, bias_via_bf16, (int)M, (int)N) != cudaSuccess)
                return AXS6_ERR_LAUNCH;
            count_launch();
        }
        return check_launch();
    }

    if (!ensure_dynamic_smem(reinterpret_cast<const void *>(&gemm_kernel<kTf32>), kSmemBytes)) return AXS6_ERR_LAUNCH;
    // Few output tiles but a long contraction (the weight gradient of a small layer): split K so that more SMs
    // get a work unit.
    if (may_split) {
        const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
        int64_t want = d.sms / tiles;
        const int64_t max_by_k = K / (8 * bk);
        if (want > max_by_k) want = max_by_k;
        if (want > max_cta_splits) want = max_cta_splits;
        if (want >= 2) p.splits = (int)want;
    }
    int ctas = p.tiles_m * p.tiles_n * p.splits;
    if (ctas > usable_sms(d)) ctas = (int)usable_sms(d);
    if (p.splits > 1 &&
        cudaMemset2DAsync(c, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, stream) != cudaSuccess)
        return AXS6_ERR_LAUNCH;
    if (launch_overlapped(true, gemm_kernel<kTf32>, ctas, kThreadsGemm, kSmemBytes, stream, ma, mb, p) != cudaSuccess) return AXS6_ERR_LAUNCH;
    count_launch();
    return check_launch();
}

}  // namespace gemm

int gemm_launch(bool tf32, const void *a, const void *b, void *c, const float *bias, int64_t M, int64_t N, int64_t K,
                int64_t lda, int64_t ldb, int64_t ldc, int a_mn, int b_mn, int c_dtype, int bias_via_bf16,
                cudaStream_t stream)
{
    if (tf32) {
        if (a_mn || b_mn) return AXS6_ERR_UNSUPPORTED;
        return gemm::launch_gemm<true>(a, b, c, bias, M, N, K, lda, ldb, ldc, 0, 0, c_dtype, bias_via_bf16, stream);
    }
    return gemm::launch_gemm<false>(a, b, c, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, c_dtype, bias_via_bf16, stream);
}

int gemm_packed_launch(const void *a, const void *a_exps, int64_t lda, const void *b, const void *b_exps, int64_t ldb, void *c,
                       const float *bias, int64_t M, int64_t N, int64_t K, int64_t ldc, int a_mn, int b_mn, int c_dtype,
                       int bias_via_bf16, cudaStream_t stream)
{
    return gemm::launch_gemm_packed(a, a_exps, lda, b, b_exps, ldb, c, bias, M, N, K, ldc, a_mn, b_mn, c_dtype, bias_via_bf16, stream);
}

}  // namespace axs6

AXS6_API int axs6_gemm_packed(const void *a, const void *a_exps, int64_t lda, const void *b, const void *b_exps, int64_t ldb,
                              void *c, const float *bias, int64_t M, int64_t N, int64_t K, int64_t ldc, int a_mn, int b_mn,
                              int c_dtype, axs6_stream_t stream)
{
    return axs6::gemm::launch_gemm_packed(a, a_exps, lda, b, b_exps, ldb, c, bias, M, N, K, ldc, a_mn, b_mn, c_dtype, 0,
                                          static_cast<cudaStream_t>(stream));
}

// C[M,N] (+ bias[N]) = op(A) * op(B) with bf16 operands and fp32 accumulation.
//   a_mn = 0: A is (M, K) row-major with leading dimension lda;  a_mn = 1: A is (K, M) row-major.
//   b_mn = 0: B is (N, K) row-major with leading dimension ldb;  b_mn = 1: B is (K, N) row-major.
AXS6_API int axs6_gemm_bf16(const void *a, const void *b, void *c, const float *bias, int64_t M, int64_t N, int64_t K,
                            int64_t lda, int64_t ldb, int64_t ldc, int a_mn, int b_mn, int c_dtype,
                            axs6_stream_t stream)
{
    return axs6::gemm::launch_gemm<false>(a, b, c, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, c_dtype, 0,
                                          static_cast<cudaStream_t>(stream));
}

// The same with a caller-owned workspace for split-K partials (see axs6_gemm_workspace_bytes).
AXS6_API int axs6_gemm_bf16_ws(const void *a, const void *b, void *c, const float *bias, int64_t M, int64_t N, int64_t K,
                               int64_t lda, int64_t ldb, int64_t ldc, int a_mn, int b_mn, int c_dtype, void *ws,
                               int64_t ws_bytes, axs6_stream_t stream)
{
    return axs6::gemm::launch_gemm<false>(a, b, c, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, c_dtype, 0,
                                          static_cast<cudaStream_t>(stream), ws, ws_bytes);
}

AXS6_API int64_t axs6_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int c_dtype)
{
    using namespace axs6;
    if (M <= 0 || N <= 0 || K <= 0 || c_dtype != AXS6_F32) return 0;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return 0;
    const int64_t want = gemm::plan_pair_splits(d, M, N, K, 8, gemm::BK);
    return want > 2 ? want * M * gemm::ws_ld_of(N) * 4 : 0;
}

// Same with fp32 operands consumed as TF32 by the tensor cores (the low 13 mantissa bits of each
// operand value are ignored; pre-round the operands to TF32 for round-to-nearest behaviour).
AXS6_API int axs6_gemm_tf32(const void *a, const void *b, void *c, const float *bias, int64_t M, int64_t N, int64_t K,
                            int64_t lda, int64_t ldb, int64_t ldc, int a_mn, int b_mn, int c_dtype,
                            axs6_stream_t stream)
{
    if (a_mn || b_mn) return AXS6_ERR_UNSUPPORTED;      // kind::tf32 gives zeros for MN-major operands on sm_100
    return axs6::gemm::launch_gemm<true>(a, b, c, bias, M, N, K, lda, ldb, ldc, 0, 0, c_dtype, 0,
                                         static_cast<cudaStream_t>(stream));
}

// Reads (and clears) the device-side status word of the GEMM kernels: 0 = every wait completed,
// otherwise the code of the first bounded wait that gave up (1 producer/stage-free, 2 MMA/accumulator-free,
// 3 MMA/stage-full, 4 epilogue/accumulator-full).  Synchronises the device.
AXS6_API int axs6_gemm_status(void)
{
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, axs6::gemm::g_gemm_status, sizeof(int)) != cudaSuccess) return AXS6_ERR_DEVICE;
    if (v != 0) cudaMemcpyToSymbol(axs6::gemm::g_gemm_status, &zero, sizeof(int));
    return v;
}
