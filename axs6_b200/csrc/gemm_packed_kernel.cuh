// Decode-on-load variant of the CTA-pair GEMM: one or both operands arrive as AXS-6 codes (NF5 grid,
// blocks of 32 along the operand's contiguous dimension, split layout: a plane of 24-byte payloads and a
// plane of exponent bytes) and are turned into bf16 tiles in shared memory by decode warps, so the
// quantised operand never exists in HBM as bf16.  This is the data flow of the reference's fused kernel
// (axs/unified/triton_kernels.py:151-282: the quantised tile is produced inside the K loop), with the
// tensor-core contraction on tcgen05 / TMEM.
//
// Included by gemm.cu inside namespace axs6::gemm.
//
// CTA pair on a 256 x 256 tile as in gemm2_kernel; 22 warps per CTA:
//   warp 0       producer: per k-block, TMA-loads this CTA's tile of every bf16 operand straight into the
//                MMA stage (bytes counted on the leader's "full" barrier), and for every packed operand the
//                payload tile (128 rows x 48 B, or 64 k-rows x 96 B for an MN-major operand) plus its 256
//                exponent bytes (one or two contiguous runs of the pair-major exponent plane, bulk copies) into a
//                raw stage (bytes counted on this CTA's "raw full" barrier)
//   warp 1       MMA issuer (leader CTA), unchanged
//   warps 2..5   epilogue, unchanged
//   warps 6..21  decode: thread t owns half-block t (16 values) of the 512 half-blocks of a packed operand tile:
//                reads its 12 payload bytes and its exponent byte from the raw stage, looks two 6-bit codes at a
//                time up in a 4096-entry table (two bf16 levels with the exponent field lowered by 120, signs
//                included), adds the block exponent to both exponent fields with one integer add, and writes
//                two 16-byte pieces to the 128-byte-swizzled position the UMMA descriptor expects; then
//                fence.proxy.async and one arrival per warp on the leader's "full" barrier and on the own
//                "raw empty" barrier.  One lane of each warp polls the barriers.
// A bf16 value is (level bits - 120 << 7) + (se - 7 << 7): exact, because the power-of-two block scale
// only moves the exponent field (blocks with se < 8 or se = 255, where that field would leave its range,
// use the fp32 product and one rounding instead; all-zero blocks have se = 0).
// Positions outside the operand (rows >= extent, blocks beyond the last) are written as zeros.
//
// Every wait is bounded; on giving up a role records a code (5 decode/raw tile, 6 decode/stage free,
// 7 producer/raw stage free) and all roles leave, as in the other kernels.

constexpr int kDecodeWarps = 16;
constexpr int kDecodeGroups = 4;                               // groups of decode warps; group g decodes k-blocks g, g + 4, ...
constexpr int kGroupWarps = kDecodeWarps / kDecodeGroups;      // 4 warps = 128 threads, 4 half-blocks per thread and operand
constexpr int kThreadsPacked = (6 + kDecodeWarps) * 32;       // 704

struct PackedParams {
    const uint8_t *a_exps, *b_exps;     // exponent planes, pair-major (null: operand is bf16)
    int a_nblk, b_nblk;                 // blocks per row of the stored operand matrix
    int a_rows, b_rows;                 // rows of the stored operand matrix (K-major: M or N; MN-major: K)
    int gather_arrivals;                // 1: the last decode warp of a CTA to finish a stage signals the leader for all 16
};

struct PairQ {
    static constexpr int kStages = 5;                              // decoded (MMA) stages
    static constexpr int kRawStages = 4;                           // payload + exponent stages: one per decode group (see the decode warps)
    static constexpr int kABytes = 128 * BK * 2, kBBytes = 128 * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;          // 32 KB
    static constexpr int kRawOp = 128 * 48;                        // payload tile of one operand: 6 KB
    static constexpr int kExpOp = 256;                             // its 256 exponent bytes
    static constexpr int kRawBytes = 2 * (kRawOp + kExpOp);
    static constexpr int kSmemBytes = 1024 /*alignment slack*/ + kStages * kStageBytes + kRawStages * kRawBytes + 512;   // dynamic part
};

__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// All-zero blocks (exponent 0) and blocks at the ends of the exponent range: fp32 product, one rounding.  Rare, and kept
// out of line (loads and stores included) so that the decode loop stays small enough for the instruction cache.
__device__ __noinline__ void decode_half_block_slow(uint32_t raw, uint32_t se, uint32_t dst0, uint32_t dst1)
{
    uint32_t w[3], o[8];
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[0]) : "r"(raw));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[1]) : "r"(raw + 4u));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[2]) : "r"(raw + 8u));
    const float scale = axs6_scale_decode(se);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int bit = 6 * i, word = bit >> 5, off = bit & 31;
        const uint32_t code = (off <= 26 ? (w[word] >> off) : __funnelshift_r(w[word], w[word + 1 < 3 ? word + 1 : 2], off)) & 63u;
        const float y = axs6_decode_value(code >> 5, __uint_as_float(g_codebook_bits[code & 31u]), scale);
        const uint32_t h = axs6_f32_to_bf16_bits(y);
        if (i & 1) o[i >> 1] |= h << 16; else o[i >> 1] = h;
    }
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst0), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst1), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
}

// Decodes half a block: 16 codes = 12 payload bytes at shared address `raw` (4-byte aligned), exponent `se`, into
// 16 bf16 values = 8 words.  `lut` is the code table in static shared memory with one copy per lane: entry
// (code, lane) is word code * 32 + lane, so the 32 lookups of a warp always hit 32 different banks (`lane4` = lane * 4).
__device__ __forceinline__ void decode_half_block(uint32_t raw, uint32_t se, const uint32_t *lut, uint32_t lane4, uint32_t (&o)[8])
{
    uint32_t w[3];
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[0]) : "r"(raw));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[1]) : "r"(raw + 4u));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[2]) : "r"(raw + 8u));
    const uint32_t kk = (se - 7u) * 0x00800080u;                  // the caller has checked 8 <= se <= 254
#pragma unroll
    for (int pr = 0; pr < 8; ++pr) {
        uint32_t v[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            // byte offset of the entry of value 2 pr + e: its code moved to bits 7..12, plus this lane's word
            const int bit = 6 * (2 * pr + e), word = bit >> 5, off = bit & 31;
            uint32_t x;
            if (off < 7) x = w[word] << (7 - off);
            else if (off == 7) x = w[word];
            else if (off <= 26) x = w[word] >> (off - 7);
            else x = __funnelshift_r(w[word], w[word + 1 < 3 ? word + 1 : 2], off - 7);
            v[e] = *reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(lut) + ((x & (0x3Fu << 7)) | lane4));
        }
        o[pr] = (v[1] << 16) + v[0] + kk;
    }
}

template <bool QA, bool QB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsPacked, 1)
gemm2q_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p,
              const PackedParams q)
{
    constexpr int S = PairQ::kStages, R = PairQ::kRawStages, kA2 = PairQ::kABytes, kStage = PairQ::kStageBytes, kRaw = PairQ::kRawBytes;
    constexpr int TN = 256;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(128) uint32_t lut[64 * 32];                         // code -> bf16 bits, one copy per lane (8 KB, static)
    __shared__ uint32_t stage_done[PairQ::kStages];                          // decode warps of this CTA finished with a stage (running count)
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;             // MMA stages (1024-aligned)
    const uint32_t raw0 = base + S * kStage;                                 // raw stages: [A payload | B payload | A exps | B exps]
    const uint32_t bar0 = raw0 + R * kRaw;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
    auto rfull_bar = [&](int s) { return bar0 + 8u * (2 * S + s); };
    auto rempty_bar = [&](int s) { return bar0 + 8u * (2 * S + R + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * S + 2 * R + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * S + 2 * R + 2 + a); };
    const uint32_t tmem_slot = bar0 + 8u * (2 * S + 2 * R + 4);
    uint8_t *smem_gen = smem_raw + (base - smem_u32(smem_raw));              // generic pointer to the 1024-aligned base
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(smem_gen + (tmem_slot - base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    const int tiles_m = (p.M + 255) / 256, tiles_n = (p.N + TN - 1) / TN;
    const int num_tiles = tiles_m * tiles_n;
    const int total_kb = (p.K + BK - 1) / BK;
    constexpr int kPacked = (QA ? 1 : 0) + (QB ? 1 : 0);
    constexpr bool kAnyTma = !QA || !QB;                                     // some operand goes straight to the MMA stage

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            // full: (leader's expect_tx arrival if a bf16 operand is loaded) + one arrival per CTA (or per warp of the
            // group that decoded the stage, both CTAs)
            mbar_init(full_bar(s), (kAnyTma ? 1 : 0) + (q.gather_arrivals ? 2 : 2 * kGroupWarps));
            mbar_init(empty_bar(s), 1);
            stage_done[s] = 0u;
        }
        for (int s = 0; s < R; ++s) {
            mbar_init(rfull_bar(s), 1);
            mbar_init(rempty_bar(s), kGroupWarps);
        }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    {
        uint32_t *tl = lut;
        for (int i = threadIdx.x; i < 64 * 32; i += kThreadsPacked) {
            const int c = i >> 5;
            const uint32_t bits = g_codebook_bits[c & 31];
            tl[i] = ((uint32_t)axs6_f32_to_bf16_bits(__uint_as_float(bits)) - (120u << 7)) | ((uint32_t)(c >> 5) << 15);
        }
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

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            int s = 0, rs = 0;
            uint32_t ph = 0, rph = 0;
            bool ok = true;
            int armed = 0;                                   // raw loads issued so far (for the drain at the end)
            // exponent bytes of one operand tile: K-major = 256 contiguous bytes (pair kb, rows o0 .. o0 + 127);
            // MN-major = two runs of 128 bytes (pairs o0 / 64 and o0 / 64 + 1, rows k0 .. k0 + 63).  Returns the bytes
            // requested (runs are clipped to the rows that exist).
            auto load_exps = [&](const uint8_t *exps, int nblk, int rows, bool mn, int o0, int kb, uint32_t dst, uint32_t bar) -> uint32_t {
                const int npair = (nblk + 1) >> 1;
                uint32_t bytes = 0;
                if (!mn) {
                    const int n = rows - o0 < 128 ? rows - o0 : 128;
                    if (n > 0 && kb < npair) {
                        bytes = (uint32_t)n * 2u;
                        acp::bulk_load(dst, exps + ((long long)kb * rows + o0) * 2, bytes, bar);
                    }
                } else {
                    const int k0 = kb * BK;
                    const int n = rows - k0 < 64 ? rows - k0 : 64;
                    for (int i = 0; i < 2; ++i) {
                        const int pr = (o0 >> 6) + i;
                        if (n > 0 && pr < npair) {
                            acp::bulk_load(dst + 128u * i, exps + ((long long)pr * rows + k0) * 2, (uint32_t)n * 2u, bar);
                            bytes += (uint32_t)n * 2u;
                        }
                    }
                }
                return bytes;
            };
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
                const int m0 = (t / tiles_n) * 256 + (int)rank * 128;
                const int n0 = (t % tiles_n) * TN + (int)rank * 128;
                for (int kb = 0; kb < total_kb; ++kb) {
                    const int k0 = kb * BK;
                    const uint32_t sa = base + s * kStage, sb = sa + kA2;
                    if (kAnyTma) {
                        if (!mbar_wait(empty_bar(s), ph ^ 1u, 1)) { ok = false; break; }
                        const uint32_t lead_full = map_to_cta(full_bar(s), 0);
                        if (rank == 0) mbar_expect_tx(full_bar(s), 2 * ((QA ? 0 : kA2) + (QB ? 0 : PairQ::kBBytes)));
                        if (!QA) {
                            if (!p.a_mn) tma_load_2d_pair(sa, &map_a, lead_full, k0, m0);
                            else for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * 8192, &map_a, lead_full, m0 + 64 * j, k0);
                        }
                        if (!QB) {
                            if (!p.b_mn) tma_load_2d_pair(sb, &map_b, lead_full, k0, n0);
                            else for (int j = 0; j < 2; ++j) tma_load_2d_pair(sb + j * 8192, &map_b, lead_full, n0 + 64 * j, k0);
                        }
                    }
                    if (kPacked) {
                        if (!mbar_wait(rempty_bar(rs), rph ^ 1u, 7)) { ok = false; break; }
                        const uint32_t ra = raw0 + rs * kRaw, rb = ra + PairQ::kRawOp;
                        const uint32_t ea = ra + 2 * PairQ::kRawOp, eb = ea + PairQ::kExpOp;
                        const uint32_t rfull = rfull_bar(rs);
                        if (++rs == R) { rs = 0; rph ^= 1u; }
                        // the exponent runs first: their byte count is known only after clipping, and the barrier is armed
                        // with the total before any copy can complete the phase (a copy that lands early only makes the
                        // pending count negative for a moment)
                        uint32_t bytes = kPacked * PairQ::kRawOp;
                        if (QA) bytes += load_exps(q.a_exps, q.a_nblk, q.a_rows, p.a_mn, m0, kb, ea, rfull);
                        if (QB) bytes += load_exps(q.b_exps, q.b_nblk, q.b_rows, p.b_mn, n0, kb, eb, rfull);
                        mbar_expect_tx(rfull, bytes);
                        // payload bytes: 3/4 byte per value along the contiguous dimension
                        if (QA) {
                            if (!p.a_mn) tma_load_2d(ra, &map_a, rfull, k0 * 3 / 4, m0);      // box {48 B, 128 rows}
                            else tma_load_2d(ra, &map_a, rfull, m0 * 3 / 4, k0);               // box {96 B, 64 k-rows}
                        }
                        if (QB) {
                            if (!p.b_mn) tma_load_2d(rb, &map_b, rfull, k0 * 3 / 4, n0);
                            else tma_load_2d(rb, &map_b, rfull, n0 * 3 / 4, k0);
                        }
                        ++armed;
                    }
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
            // never leave while a raw load may still be landing: wait (bounded) for the last phase armed on every stage
            if (kPacked && !ok) {
                for (int back = 0; back < R && back < armed; ++back) {
                    const int idx = armed - 1 - back;
                    acp::mbar_wait_quiet(rfull_bar(idx % R), (uint32_t)((idx / R) & 1), kSpinLimit);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) |
                                   ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int s = 0, acc = 0;
            uint32_t ph = 0, aph = 0;
            bool ok = true;
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
                if (!mbar_wait(tempty_bar(acc), aph ^ 1u, 2)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * TN);
                for (int kb = 0; kb < total_kb; ++kb) {
                    if (!mbar_wait(full_bar(s), ph, 3)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + s * kStage, sb = sa + kA2;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t ad = smem_desc(sa + k * p.a_kstep, p.a_lbo, p.a_sbo);
                        const uint64_t bd = smem_desc(sb + k * p.b_kstep, p.b_lbo, p.b_sbo);
                        tc_mma2(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit2(empty_bar(s));
                    tc_commit2(map_to_cta(empty_bar(s), 1));
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                tc_commit2(tfull_bar(acc));
                tc_commit2(map_to_cta(tfull_bar(acc), 1));
                acc ^= 1;
                if (acc == 0) aph ^= 1u;
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int qd = warp & 3;
        int acc = 0;
        uint32_t aph = 0;
        bool ok = true;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0) && (p.ldc % 8 == 0);
        for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
            const int m0 = (t / tiles_n) * 256 + (int)rank * 128, n0 = (t % tiles_n) * TN;
            if (!mbar_wait(tfull_bar(acc), aph, 4)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + qd * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(qd * 32) << 16) + (uint32_t)(acc * TN);
            epilogue_tile(p, taddr, row, n0, vec_ok, false, true);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
            acc ^= 1;
            if (acc == 0) aph ^= 1u;
        }
    } else if (kPacked) {
        // ------------------------------------------------------------------ decode (warps 6..21, both CTAs)
        // A packed operand tile is 512 half-blocks of 16 values (block = hb >> 1 in row-major order of the raw tile,
        // half = hb & 1).  The sixteen warps work as four groups: group g decodes the k-blocks g, g + 4, ... of the
        // cluster's sequence, so that up to four stages are being filled at the same time and a warp pays its waits,
        // fence and arrivals once per four half-blocks per operand.  Thread gt of a group owns half-blocks gt + 128 j.
        // A parity wait tells two neighbouring phases of a barrier apart and no more, so a group must never wait
        // for a phase while the one before it is still open: with one raw stage per group the fill it waits for
        // follows the fill it has just consumed, and with at least as many decoded stages as groups the stage it
        // wants back was handed to the tensor core before the stage it got back one turn earlier.
        static_assert(PairQ::kRawStages == kDecodeGroups && PairQ::kStages >= kDecodeGroups, "stage counts against the decode groups");
        static_assert(kGroupWarps * 32 * 4 == 512, "four half-blocks per thread and operand");
        const int dt = threadIdx.x - 6 * 32;
        const int grp = dt >> 7, gt = dt & 127;
        const uint32_t lane4 = (uint32_t)lane << 2;
        struct Geo { uint32_t raw, exp, dst0; int row, col; };
        auto geo = [&](bool mn, int hb) -> Geo {
            Geo g;
            const int blk = hb >> 1, half = hb & 1;
            g.raw = (uint32_t)hb * 12u;
            if (!mn) {               // tile row r = blk >> 1 (output index), j = blk & 1 of the two contraction blocks
                const uint32_t r = (uint32_t)blk >> 1, j = (uint32_t)blk & 1u;
                g.exp = (uint32_t)blk;
                const uint32_t p0 = 4u * j + 2u * (uint32_t)half;
                g.dst0 = r * 128u + (((p0) ^ (r & 7u)) << 4);
                g.row = (int)r; g.col = (int)j;
            } else {                 // k-row r = blk >> 2, b = blk & 3 of the four output blocks
                const uint32_t r = (uint32_t)blk >> 2, b = (uint32_t)blk & 3u;
                g.exp = (b >> 1) * 128u + r * 2u + (b & 1u);
                const uint32_t p0 = 4u * (b & 1u) + 2u * (uint32_t)half;
                g.dst0 = (b >> 1) * 8192u + r * 128u + (((p0) ^ (r & 7u)) << 4);
                g.row = (int)r; g.col = (int)b;
            }
            return g;                // the second 16-byte chunk of the half-block sits at dst0 ^ 16 (p0 is even)
        };
        // is this thread's block inside the operand?  K-major: row o0 + row < rows, block 2 kb + col < nblk;
        // MN-major: k-row kb * 64 + row < rows, block o0 / 32 + col < nblk
        auto inside = [&](const Geo &g, bool mn, int rows, int nblk, int o0, int kb) -> bool {
            return mn ? (kb * BK + g.row < rows && (o0 >> 5) + g.col < nblk) : (o0 + g.row < rows && 2 * kb + g.col < nblk);
        };
        auto put = [&](uint32_t stage_half, const Geo &g, bool valid, uint32_t raw_op, uint32_t exp_op) {
            uint32_t o[8];
            const uint32_t d0 = stage_half + g.dst0, d1 = stage_half + (g.dst0 ^ 16u);
            if (valid) {
                uint32_t se;
                asm volatile("ld.shared.u8 %0, [%1];" : "=r"(se) : "r"(exp_op + g.exp));
                if (se < 8u || se > 254u) {
                    decode_half_block_slow(raw_op + g.raw, se, d0, d1);
                    return;
                }
                decode_half_block(raw_op + g.raw, se, lut, lane4, o);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = 0u;
            }
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(d0), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(d1), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
        };
        int s = 0, rs = 0, turn = 0;
        uint32_t ph = 0, rph = 0;
        bool ok = true;
        for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
            const int m0 = (t / tiles_n) * 256 + (int)rank * 128;
            const int n0 = (t % tiles_n) * TN + (int)rank * 128;
            for (int kb = 0; kb < total_kb; ++kb) {
                if (turn == grp) {
                    // one lane polls, the warp follows
                    int go = 1;
                    if (lane == 0) go = (mbar_wait(rfull_bar(rs), rph, 5) && mbar_wait(empty_bar(s), ph ^ 1u, 6)) ? 1 : 0;
                    go = __shfl_sync(0xFFFFFFFFu, go, 0);
                    if (!go) { ok = false; break; }
                    const uint32_t sa = base + s * kStage, sb = sa + kA2;
                    const uint32_t ra = raw0 + rs * kRaw, rb = ra + PairQ::kRawOp;
                    const uint32_t ea = ra + 2 * PairQ::kRawOp, eb = ea + PairQ::kExpOp;
#pragma unroll 1
                    for (int j = 0; j < 512 / (kGroupWarps * 32); ++j) {
                        const int hb = gt + kGroupWarps * 32 * j;
                        if (QA) { const Geo g = geo(p.a_mn, hb); put(sa, g, inside(g, p.a_mn, q.a_rows, q.a_nblk, m0, kb), ra, ea); }
                        if (QB) { const Geo g = geo(p.b_mn, hb); put(sb, g, inside(g, p.b_mn, q.b_rows, q.b_nblk, n0, kb), rb, eb); }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // decoded tile visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) {
                        // A cluster-scope release per warp and k-block is what the decode warps stalled on most.  With
                        // gathered arrivals the warps of the group count themselves in shared memory (CTA scope) and only
                        // the one that completes the group releases to the leader's barrier; the count runs on, a stage
                        // is not decoded again before the tensor core has read it.
                        bool signal = true;
                        if (q.gather_arrivals) {
                            uint32_t before;
                            asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], 1;"
                                         : "=r"(before) : "r"(smem_u32(&stage_done[s])) : "memory");
                            signal = (before % kGroupWarps) == kGroupWarps - 1;
                        }
                        if (signal) mbar_arrive_release_cluster(map_to_cta(full_bar(s), 0));
                        mbar_arrive(rempty_bar(rs));
                    }
                }
                if (++turn == kDecodeGroups) turn = 0;
                if (++s == S) { s = 0; ph ^= 1u; }
                if (++rs == R) { rs = 0; rph ^= 1u; }
            }
        }
    }

    linger_if_failed();
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}
