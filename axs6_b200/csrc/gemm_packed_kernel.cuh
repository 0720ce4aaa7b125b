// Decode-on-load variant of the CTA-pair GEMM: one or both operands arrive as AXS-6 codes (NF5 grid,
// blocks of 32 along the operand's contiguous dimension, split layout: a plane of 24-byte payloads and a
// plane of exponent bytes) and are turned into bf16 tiles in shared memory by decode warps, so the
// quantised operand never exists in HBM as bf16.  This is the data flow of the reference's fused kernel
// (axs/unified/triton_kernels.py:151-282: the quantised tile is produced inside the K loop), with the
// tensor-core contraction on tcgen05 / TMEM.
//
// Included by gemm.cu inside namespace axs6::gemm.
//
// CTA pair on a 256 x 256 tile as in gemm2_kernel; 14 warps per CTA:
//   warp 0       producer: per k-block, TMA-loads this CTA's tile of every bf16 operand straight into the
//                MMA stage (bytes counted on the leader's "full" barrier), and the payload tile of every packed
//                operand (128 rows x 48 B, or 64 k-rows x 96 B for an MN-major operand) into a raw stage
//                (bytes counted on this CTA's "raw full" barrier)
//   warp 1       MMA issuer (leader CTA), unchanged
//   warps 2..5   epilogue, unchanged
//   warps 6..13  decode: thread t owns block t of the 256 blocks of a packed operand tile: reads its 24-byte
//                payload from the raw stage and its exponent byte from global memory (fetched one k-block
//                ahead), looks every 6-bit code up in a per-lane copy of the 64-entry table (bf16 level with
//                the exponent field lowered by 120, sign included; bank-conflict free), adds the block
//                exponent to the exponent fields of two values at a time, and writes four 16-byte pieces to
//                the 128-byte-swizzled position the UMMA descriptor expects; then fence.proxy.async and one
//                arrival per warp on the leader's "full" barrier and on the own "raw empty" barrier.
// A bf16 value is (level bits - 120 << 7) + (se - 7 << 7): exact, because the power-of-two block scale
// only moves the exponent field (blocks with se < 8 or se = 255, where that field would leave its range,
// use the fp32 product and one rounding instead; all-zero blocks have se = 0).
// Positions outside the operand (rows >= extent, blocks beyond the last) are written as zeros.
//
// Every wait is bounded; on giving up a role records a code (5 decode/raw tile, 6 decode/stage free,
// 7 producer/raw stage free) and all roles leave, as in the other kernels.

constexpr int kThreadsPacked = 448;
constexpr int kDecodeWarps = 8;

struct PackedParams {
    const uint8_t *a_exps, *b_exps;     // exponent planes (null: operand is bf16)
    int a_nblk, b_nblk;                 // blocks per row of the exponent plane
    int a_rows, b_rows;                 // rows of the stored operand matrix (K-major: M or N; MN-major: K)
};

struct PairQ {
    static constexpr int kStages = 4;
    static constexpr int kABytes = 128 * BK * 2, kBBytes = 128 * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;          // 32 KB
    static constexpr int kRawOp = 128 * 48;                        // payload tile of one operand: 6 KB
    static constexpr int kRawBytes = 2 * kRawOp;
    static constexpr int kLutBytes = 2 * 64 * 32 * 4;              // two per-lane tables of 8 KB
    static constexpr int kSmemBytes = 8192 /*alignment slack for the tables*/ + kLutBytes + kStages * (kStageBytes + kRawBytes) + 512;
};

__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Decodes one block (24-byte payload at shared address `raw`, exponent `se`) into 32 bf16 values = 16 words.
// `lut_lo` / `lut_hi` are this lane's table bases (value in the low / high half of the word).
__device__ __forceinline__ void decode_block(uint32_t raw, uint32_t se, uint32_t lut_lo, uint32_t lut_hi, uint32_t (&o)[16])
{
    uint32_t pay[6];
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(pay[0]), "=r"(pay[1]) : "r"(raw));
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(pay[2]), "=r"(pay[3]) : "r"(raw + 8u));
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(pay[4]), "=r"(pay[5]) : "r"(raw + 16u));
    if (se >= 8u && se <= 254u) {
        const uint32_t kk = (se - 7u) * 0x00800080u;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            uint32_t v[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                // table offset of code c is c * 128 (32 lanes x 4 bytes per entry)
                const int bit = 6 * (i + e), word = bit >> 5, off = bit & 31;
                uint32_t x;
                if (off < 7) x = pay[word] << (7 - off);
                else if (off <= 26) x = pay[word] >> (off - 7);
                else x = __funnelshift_r(pay[word], pay[word + 1], off - 7);
                const uint32_t addr = (x & 0x1F80u) | (e ? lut_hi : lut_lo);
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v[e]) : "r"(addr));
            }
            o[i >> 1] = v[0] + v[1] + kk;
        }
    } else {
        const float scale = axs6_scale_decode(se);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int bit = 6 * i, word = bit >> 5, off = bit & 31;
            const uint32_t code = (off <= 26 ? (pay[word] >> off) : __funnelshift_r(pay[word], pay[word + 1], off)) & 63u;
            const float y = axs6_decode_value(code >> 5, __uint_as_float(g_codebook_bits[code & 31u]), scale);
            const uint32_t h = axs6_f32_to_bf16_bits(y);
            if (i & 1) o[i >> 1] |= h << 16; else o[i >> 1] = h;
        }
    }
}

template <bool QA, bool QB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsPacked, 1)
gemm2q_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p,
              const PackedParams q)
{
    constexpr int S = PairQ::kStages, kA2 = PairQ::kABytes, kStage = PairQ::kStageBytes, kRaw = PairQ::kRawBytes;
    constexpr int TN = 256;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t lut = (smem_u32(smem_raw) + 8191u) & ~8191u;              // tables: 8 KB aligned (address bits OR-ed in)
    const uint32_t base = lut + PairQ::kLutBytes;                            // MMA stages (1024-aligned)
    const uint32_t raw0 = base + S * kStage;                                 // raw stages
    const uint32_t bar0 = raw0 + S * kRaw;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
    auto rfull_bar = [&](int s) { return bar0 + 8u * (2 * S + s); };
    auto rempty_bar = [&](int s) { return bar0 + 8u * (3 * S + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (4 * S + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (4 * S + 2 + a); };
    const uint32_t tmem_slot = bar0 + 8u * (4 * S + 4);
    uint8_t *smem_gen = smem_raw + (lut - smem_u32(smem_raw));               // generic pointer to the tables
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(smem_gen + (tmem_slot - lut));

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
            // full: (leader's expect_tx arrival if a bf16 operand is loaded) + one arrival per decode warp, packed operand and CTA
            mbar_init(full_bar(s), (kAnyTma ? 1 : 0) + 2 * kDecodeWarps * kPacked);
            mbar_init(empty_bar(s), 1);
            mbar_init(rfull_bar(s), 1);
            mbar_init(rempty_bar(s), kDecodeWarps * kPacked);
        }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // per-lane copies of the 64-entry code table: entry c of lane l at (c * 32 + l) * 4
    {
        uint32_t *tl = reinterpret_cast<uint32_t *>(smem_gen);
        uint32_t *th = tl + 64 * 32;
        for (int i = threadIdx.x; i < 64 * 32; i += kThreadsPacked) {
            const int c = i >> 5;
            const uint32_t bits = g_codebook_bits[c & 31];
            const uint32_t v = ((uint32_t)axs6_f32_to_bf16_bits(__uint_as_float(bits)) - (120u << 7)) | ((uint32_t)(c >> 5) << 15);
            tl[i] = v;
            th[i] = v << 16;
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
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int armed = 0;                                   // raw loads issued so far (for the drain at the end)
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
                        if (!mbar_wait(rempty_bar(s), ph ^ 1u, 7)) { ok = false; break; }
                        mbar_expect_tx(rfull_bar(s), kPacked * PairQ::kRawOp);
                        const uint32_t ra = raw0 + s * kRaw, rb = ra + PairQ::kRawOp;
                        // payload bytes: 3/4 byte per value along the contiguous dimension
                        if (QA) {
                            if (!p.a_mn) tma_load_2d(ra, &map_a, rfull_bar(s), k0 * 3 / 4, m0);      // box {48 B, 128 rows}
                            else tma_load_2d(ra, &map_a, rfull_bar(s), m0 * 3 / 4, k0);               // box {96 B, 64 k-rows}
                        }
                        if (QB) {
                            if (!p.b_mn) tma_load_2d(rb, &map_b, rfull_bar(s), k0 * 3 / 4, n0);
                            else tma_load_2d(rb, &map_b, rfull_bar(s), n0 * 3 / 4, k0);
                        }
                        ++armed;
                    }
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
            // never leave while a raw load may still be landing: wait (bounded) for the last phase armed on every stage
            if (kPacked && !ok) {
                for (int back = 0; back < S && back < armed; ++back) {
                    const int idx = armed - 1 - back;
                    mbar_wait(rfull_bar(idx % S), (uint32_t)((idx / S) & 1), 7);
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
        // ------------------------------------------------------------------ decode (warps 6..13, both CTAs)
        const int dt = threadIdx.x - 6 * 32;                 // 0..255: block of the operand tile
        const uint32_t lut_lo = lut + 4u * lane, lut_hi = lut_lo + 64u * 32u * 4u;
        // geometry of this thread's block inside a tile, per operand layout
        //   K-major:  tile row r = dt >> 1 (output index), block j = dt & 1 of the 64 contraction values
        //   MN-major: k-row r = dt >> 2, block b = dt & 3 of the 128 output values
        auto dst_off = [&](bool mn) -> uint32_t {            // byte offset of piece 0's row inside the operand's stage half
            return mn ? (uint32_t)((dt & 3) >> 1) * 8192u + (uint32_t)(dt >> 2) * 128u : (uint32_t)(dt >> 1) * 128u;
        };
        auto piece0 = [&](bool mn) -> uint32_t { return mn ? 4u * ((uint32_t)dt & 1u) : 4u * ((uint32_t)dt & 1u); };
        auto swz = [&](bool mn) -> uint32_t { return mn ? ((uint32_t)(dt >> 2) & 7u) : ((uint32_t)(dt >> 1) & 7u); };
        auto raw_off = [&](bool mn) -> uint32_t { return (uint32_t)dt * 24u; };    // both layouts: block dt of the tile in row-major order
        const uint32_t a_dst = dst_off(p.a_mn), a_p0 = piece0(p.a_mn), a_sw = swz(p.a_mn);
        const uint32_t b_dst = dst_off(p.b_mn), b_p0 = piece0(p.b_mn), b_sw = swz(p.b_mn);
        // exponent of this thread's block for (tile origin o0 along the output index, k-block kb); 0x100 = outside
        auto fetch = [&](const uint8_t *exps, int nblk, int rows, bool mn, int o0, int kb) -> uint32_t {
            int row, blk;
            if (!mn) { row = o0 + (dt >> 1); blk = 2 * kb + (dt & 1); }
            else { row = kb * BK + (dt >> 2); blk = (o0 >> 5) + (dt & 3); }
            if (row >= rows || blk >= nblk) return 0x100u;
            return (uint32_t)__ldg(exps + (long long)row * nblk + blk);
        };
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        uint32_t ea = 0x100u, eb = 0x100u;
        bool have = false;
        for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
            const int m0 = (t / tiles_n) * 256 + (int)rank * 128;
            const int n0 = (t % tiles_n) * TN + (int)rank * 128;
            if (!have) {
                if (QA) ea = fetch(q.a_exps, q.a_nblk, q.a_rows, p.a_mn, m0, 0);
                if (QB) eb = fetch(q.b_exps, q.b_nblk, q.b_rows, p.b_mn, n0, 0);
                have = true;
            }
            for (int kb = 0; kb < total_kb; ++kb) {
                // exponents of the next k-block (or of the next tile's first one), in flight while this one is decoded
                uint32_t na = 0x100u, nb = 0x100u;
                {
                    int nt = t, nkb = kb + 1;
                    if (nkb == total_kb) { nt = t + num_clusters; nkb = 0; }
                    if (nt < num_tiles) {
                        const int nm0 = (nt / tiles_n) * 256 + (int)rank * 128;
                        const int nn0 = (nt % tiles_n) * TN + (int)rank * 128;
                        if (QA) na = fetch(q.a_exps, q.a_nblk, q.a_rows, p.a_mn, nm0, nkb);
                        if (QB) nb = fetch(q.b_exps, q.b_nblk, q.b_rows, p.b_mn, nn0, nkb);
                    }
                }
                if (!mbar_wait(rfull_bar(s), ph, 5)) { ok = false; break; }
                if (!mbar_wait(empty_bar(s), ph ^ 1u, 6)) { ok = false; break; }
                const uint32_t sa = base + s * kStage, sb = sa + kA2;
                const uint32_t ra = raw0 + s * kRaw, rb = ra + PairQ::kRawOp;
                if (QA) {
                    uint32_t o[16];
                    if (ea < 0x100u) decode_block(ra + raw_off(p.a_mn), ea, lut_lo, lut_hi, o);
                    else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = 0u;
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t addr = sa + a_dst + (((a_p0 + i) ^ a_sw) << 4);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[4 * i]), "r"(o[4 * i + 1]),
                                     "r"(o[4 * i + 2]), "r"(o[4 * i + 3]) : "memory");
                    }
                }
                if (QB) {
                    uint32_t o[16];
                    if (eb < 0x100u) decode_block(rb + raw_off(p.b_mn), eb, lut_lo, lut_hi, o);
                    else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = 0u;
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t addr = sb + b_dst + (((b_p0 + i) ^ b_sw) << 4);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[4 * i]), "r"(o[4 * i + 1]),
                                     "r"(o[4 * i + 2]), "r"(o[4 * i + 3]) : "memory");
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // decoded tile visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) {
                    const uint32_t lead_full = map_to_cta(full_bar(s), 0);
#pragma unroll
                    for (int i = 0; i < kPacked; ++i) {
                        mbar_arrive_release_cluster(lead_full);
                        mbar_arrive(rempty_bar(s));
                    }
                }
                ea = na; eb = nb;
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}
