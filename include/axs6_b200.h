/*
 * axs6_b200 -- C ABI of the B200 (sm_100a) implementation of the AXS-6 hot path.
 *
 * Every entry point takes plain device pointers and sizes, validates its arguments on
 * the host before any launch, enqueues its work on the given CUDA stream and returns
 * without synchronising.  Return value: AXS6_OK (0) or a negative AXS6_ERR_* code;
 * axs6_strerror() gives the text.  The library never allocates device memory: every
 * buffer, workspace included, belongs to the caller.  There is no CPU path: on a
 * device that is not compute capability 10.x the calls return AXS6_ERR_DEVICE.
 *
 * Tensors are row-major 2-D views (rows, cols) with a leading dimension in ELEMENTS.
 * The last dimension is cut into blocks of `block` (8, 16 or 32) values that share one
 * 8-bit exponent; a ragged last block behaves as if zero-padded, exactly like the
 * reference's F.pad.  "Reference" citations below are paths in the bwiemz/axs-6 tree.
 */
#ifndef AXS6_B200_H
#define AXS6_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *axs6_stream_t; /* a cudaStream_t */

enum { AXS6_F32 = 0, AXS6_BF16 = 1 };
enum { AXS6_GRID_UNIFORM = 0, /* V1: 31 equal steps          (axs/core.py)                    */
       AXS6_GRID_NF5 = 1 };   /* 32 half-normal levels via the 1024-entry LUT (axs/unified)   */
enum { AXS6_ROUND_NEAREST = 0, AXS6_ROUND_STOCHASTIC = 1 };
enum { AXS6_LAYOUT_PLANES = 0, /* AXSTensor planes: u8 exponent (rows,nblk), u8 sign and u8
                                  magnitude (rows,nblk,block)      (axs/core.py:160-182)      */
       AXS6_LAYOUT_WIRE = 1,   /* per block: 1 exponent byte + 6-bit codes, 25 B for block 32
                                  (axs/unified/distributed.py:147-198)                        */
       AXS6_LAYOUT_SPEC = 2,   /* per block: u16 LE (exponent<<2 | config 0) + 6-bit codes,
                                  26 B for block 32 (axs/core.py:97-118, FORMAT_SPEC.md:29-48) */
       AXS6_LAYOUT_SPLIT = 3 };/* the bytes of a WIRE record in two planes: payloads (rows, nblk, 3*block/4)
                                  and exponents u8 stored by pairs of blocks, (ceil(nblk/2), rows, 2): the
                                  exponent of block b of row r is byte ((b/2)*rows + r)*2 + b%2.  Rows of the
                                  payload plane start 16-byte aligned when cols is a multiple of 64 and the
                                  exponents of an operand tile are contiguous runs, which is what lets the
                                  TMA unit fetch tiles of packed codes for axs6_gemm_packed.  (No counterpart
                                  in the reference; same 25 bytes per block of 32.)                         */

/* flags */
#define AXS6_FLAG_INPUT_VIA_BF16 1u /* round an fp32 input to bf16 before quantising: the
                                       `weight.to(bfloat16)` of the mixed-precision Linear
                                       (axs/unified/mixed_precision.py:96-100) fused in    */

#define AXS6_FLAG_OUTPUT_TF32 2u     /* round an fp32 result to the nearest TF32 value (10-bit
                                       mantissa) so that a kind::tf32 GEMM reads it exactly     */

#define AXS6_LINEAR_QUANTIZE_INPUT 1u /* fake-quantise the activations (else only cast to bf16) */
#define AXS6_LINEAR_QUANTIZE_GRAD 2u  /* fake-quantise the upstream gradient, stochastic rounding */
#define AXS6_LINEAR_COMPUTE_TF32 4u   /* fp32 graph: operands fake-quantised in fp32 (no bf16 cast),
                                         rounded to TF32, products on the TF32 tensor cores; work
                                         buffers are fp32 (workspace codes 4, 5, 6)              */
#define AXS6_LINEAR_BIAS_VIA_BF16 16u  /* forward: add bf16(bias) instead of bias, as F.linear does with
                                         `bias.to(bfloat16)` (mixed_precision.py:108)                 */
#define AXS6_LINEAR_BIAS_FROM_QUANTIZED 8u /* db sums the QUANTISED gradient, as the fp32 reference
                                         functions do (functional_unified.py:151, :161-165)      */

#define AXS6_LINEAR_REUSE_WQ 32u       /* backward: `wq` already holds FQ(bf16(w)) -- the buffer the forward call of the
                                         same step filled, with the weight unchanged since -- so it is not
                                         recomputed (bit-identical by construction; the reference recomputes only
                                         to save memory, mixed_precision.py:130); `w` may then be NULL      */
#define AXS6_LINEAR_REUSE_GQ 64u       /* backward: `gq` already holds the quantised gradient, written by an earlier
                                         axs6_linear_bwd call on the same g (lets a caller ask for dw first, start
                                         its all-reduce, and then ask for dx / db without a second rounding pass) */

#define AXS6_LINEAR_OPERANDS_PACKED 128u /* quantise on load: xq / wq / gq hold 6-bit codes (payload plane, then the exponent
                                         plane at the next 256-byte boundary; workspace codes 8, 9, 10) instead of bf16,
                                         and the GEMMs decode them in shared memory (axs6_gemm_packed).  Needs
                                         AXS6_LINEAR_QUANTIZE_INPUT / _GRAD, NF5, block 32, K and N multiples of 64, M a
                                         multiple of 8 (AXS6_ERR_UNSUPPORTED otherwise).  The saved activation shrinks from 2 to
                                         0.78 bytes per value.  Equal to the bf16 path except where an operand holds
                                         an exact zero, which codes cannot express (see axs6_gemm_packed)        */

#define AXS6_LINEAR_SPLITK_WORKSPACE 256u /* backward, bf16 graph: `tf32_scratch` holds axs6_linear_workspace_bytes(11, M, N, K)
                                         bytes in which the weight-gradient product keeps split-K partials apart; they
                                         are added in a fixed order, so dw is bit-reproducible with more than two
                                         partials (small layers with long contractions) */

#define AXS6_LINEAR_FP32_ACCURACY 512u  /* forward, with AXS6_LINEAR_COMPUTE_TF32: the product of the fp32 fake-quantised
                                         operands to fp32 accuracy (about 2^-21 relative) instead of TF32 accuracy
                                         (2^-11): each operand is split into two TF32 parts and three TF32 products are
                                         accumulated in one GEMM over the tripled contraction.  What the reference's
                                         fused kernel computes (`input_precision="ieee"`, triton_kernels.py:262) and its
                                         tests hold it to (tests/test_triton_fused_linear.py:33-35: 1e-3 absolute).
                                         xq / wq are workspace codes 12 / 13; xq starts with the fp32 quantised
                                         activations, which is what backward reads                              */

#define AXS6_OK 0
#define AXS6_ERR_ARG (-1)         /* null pointer, negative size, bad enum, bad block size  */
#define AXS6_ERR_ALIGN (-2)       /* pointer or leading dimension violates a stated alignment */
#define AXS6_ERR_DEVICE (-3)      /* current device is not sm_100 / CUDA runtime error         */
#define AXS6_ERR_LAUNCH (-4)      /* kernel launch failed                                       */
#define AXS6_ERR_WORKSPACE (-5)   /* workspace missing or too small                             */
#define AXS6_ERR_UNSUPPORTED (-6) /* valid request this build does not implement               */
#define AXS6_ERR_TOO_LARGE (-7)   /* size beyond the fixed capacity of a *_static entry point   */

const char *axs6_strerror(int status);

/* what: 0 = 1 if the current device can run the kernels (cc 10.x) else 0, 1 = SM count,
 * 2 = ABI version, 3 = number of kernels launched by this process so far, 4 = the last CUDA error code
 * a launch of this library returned (0 = none; a debugging aid for AXS6_ERR_LAUNCH). */
int64_t axs6_query(int what);

/* Performance knobs for experiments and tests (process-wide, never needed for correct results;
 * value 0 restores the built-in choice):
 *   key 0   cap on resident CTAs per SM of the fake-quantise kernels
 *   key 1   the same for the pack / unpack kernels
 *   key 2   record pack of bf16 / fp32 input: 1 = general kernel only, 2 = bf16 kernel with per-thread
 *           loads instead of the TMA-fed one
 *   key 3   GEMM K splits of fp32 outputs.  Built-in (0): at most two partial products per output element,
 *           whose sum does not depend on their order, so every result is bit-reproducible.  1 = never
 *           split, 2 = two-way split of every tile in the CTA-pair kernel, 3 = allow up to 8 / 16 partials
 *           for problems with few tiles: faster weight gradients of small layers, but the partials are added
 *           in no fixed order and the last bits can differ from run to run
 *   key 4   1 = MN-major operands of the CTA-pair GEMM arrive as two 2-D boxes per stage (64-value chunks one after the
 *           other) instead of one 4-D box (the two chunks of a group of 8 k-rows side by side)
 *   key 5   1 = the CTA-pair GEMM writes bf16 outputs with per-thread stores instead of staging each tile
 *           in shared memory for a TMA store
 *   key 6   1 = the CTA-pair GEMM is launched with one cluster per work unit and running clusters take over the units of
 *           clusters that have not started (cluster launch control) instead of a fixed assignment of units to 74
 *           clusters: same results; measured 1-2 % slower alone, better only next to a kernel that holds SMs
 *   key 7   GEMM kernel: 1 single-CTA, 2 CTA pairs on 256 x 256 tiles, 3 CTA pairs on 256 x 512 tiles
 *   key 8   SMs the GEMM leaves free (for a collective on another stream)
 *   key 9   1 = every decode warp of the quantise-on-load GEMM signals the leader CTA's stage barrier itself (32 cluster-scope
 *           arrivals per k-block) instead of the last warp of each CTA doing it for all sixteen (2 per k-block)
 *   key 11  1 = general unpack / unpack-and-sum kernels only (no TMA-fed kernel)
 *   key 12  1 = general fake-quantise kernel only (no TMA-fed bf16 kernel)
 *   key 13  poll limit of the bounded waits inside axs6_unpack_sum's fast kernel (default 2^22 polls)
 *   key 14  1 = the producer warp of that kernel issues no load at all, so that the consumers' first wait runs
 *           out with nothing in flight and the kernel returns with status 11: exists only so that a test can
 *           walk the give-up path without faulting or hanging the GPU
 *   key 15  1 = no kernel is launched with the programmatic-dependent-launch attribute (each kernel then
 *           starts only after the one before it on the stream has finished) */
int axs6_tune(int key, int64_t value);

/* Every stochastic kernel adds a per-device, device-resident epoch to its Philox counter offset.
 * This call enqueues epoch += delta (or epoch = 0 with reset != 0) on `stream`.  It exists for
 * CUDA-graph replay: the host-side (seed, offset) arguments are frozen into a captured graph, so a
 * captured training step starts with axs6_philox_advance(large delta) and thereby draws fresh
 * numbers on every replay.  Without any call the epoch is 0 and nothing changes.  (No
 * counterpart in the reference, which draws a new seed on the host for every launch.) */
int axs6_philox_advance(uint64_t delta, int reset, axs6_stream_t stream);

/* Reads the current device's epoch into *epoch (synchronises the device: meant for checkpoints, which store it next
 * to the host-side offset and restore it with axs6_philox_advance(0, 1, s) followed by axs6_philox_advance(value, 0, s)). */
int axs6_philox_epoch(uint64_t *epoch);

/* Fake-quantise: y = dequantise(quantise(x)) in one pass.
 * Replaces fused_fake_quantize (axs/unified/quantize_unified.py:121-204), the Triton
 * launcher triton_fused_fake_quantize (axs/unified/triton_kernels.py:295-370) and, with
 * grid = AXS6_GRID_UNIFORM, dequantize(quantize(x)) of axs/core.py:294-403 as used by
 * axs/nn/functional.py:46-53.  Nearest rounding is bit-exact with the reference's eager
 * CPU result.  Stochastic rounding draws one 16-bit uniform per element from Philox4x32-10 keyed
 * by `seed`: counter = `offset` + padded element index / 8, eight draws per 128-bit block.
 * Any alignment is accepted; 16-byte aligned pointers with cols and both leading
 * dimensions multiples of 8 elements take the vectorised path. */
int axs6_fq(const void *x, void *y, int in_dtype, int out_dtype,
            int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
            int block, int grid, int rounding, uint32_t flags,
            uint64_t seed, uint64_t offset, axs6_stream_t stream);

/* Quantise with error feedback in one pass (reference: quantize_with_error_feedback, axs/quantize.py:149-200, which
 * adds the residual, quantises, dequantises and subtracts as four tensor operations): corrected = x + err (fp32),
 * planes <- codes of corrected, err <- corrected - reconstruction.  fp32 x and err with the same leading dimension,
 * AXSTensor planes out; needs 16-byte aligned pointers and cols, ld multiples of 8 (AXS6_ERR_UNSUPPORTED otherwise:
 * compose axs6_pack / axs6_unpack instead).  Bit-identical to the four-step form. */
int axs6_pack_ef(const float *x, float *err, int64_t rows, int64_t cols, int64_t ld, int block, int grid, int rounding,
                 uint64_t seed, uint64_t offset, void *out_exp, void *out_sign, void *out_mag, axs6_stream_t stream);

/* Fake-quantise of gathered rows in one pass: y[r, :] = FQ(table[row_index[r], :]) for r < rows.  Replaces the
 * gather followed by a fake-quantise of the reference's embedding (axs/unified/modules_unified.py:181-185:
 * F.embedding, then fake_quantize_unified on the looked-up rows) without writing the raw rows to HBM in between.
 * `row_index`: `rows` int64 values on the device.  An index outside [0, table_rows) does not fault: that row is
 * read from row 0 instead and axs6_fq_gather_status() returns 1 once (and clears the flag). */
int axs6_fq_gather(const void *table, int64_t table_rows, const long long *row_index, void *y, int in_dtype, int out_dtype,
                   int64_t rows, int64_t cols, int64_t ld_table, int64_t ldy, int block, int grid, int rounding,
                   uint64_t seed, uint64_t offset, axs6_stream_t stream);
int axs6_fq_gather_status(void);

/* Same arithmetic with the uniform draws supplied by the caller: `noise` holds fp32
 * U[0,1) in the zero-padded (rows, nblk, block) layout, as torch.rand_like produces it in
 * the reference (quantize_unified.py:186-189, core.py:351-355).  Makes the stochastic
 * path bit-comparable. */
int axs6_fq_with_noise(const void *x, void *y, int in_dtype, int out_dtype,
                       int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                       int block, int grid, uint32_t flags,
                       const float *noise, axs6_stream_t stream);

/* Quantise to codes.  Replaces quantize_unified (axs/unified/quantize_unified.py:211-282),
 * quantize (axs/core.py:294-369), _pack_gradient + _pack_to_flat_buffer
 * (axs/unified/distributed.py:70-198) and AXSBlock.to_bytes (axs/core.py:97-118).
 * layout PLANES: out0 = exponents u8 (rows*nblk), out1 = signs u8 (rows*nblk*block),
 *                out2 = magnitudes u8 (rows*nblk*block).
 * layout WIRE/SPEC: out0 = rows*nblk records of (1|2) + block*3/4 bytes; out1/out2 unused.
 * layout SPLIT: out0 = rows*nblk payloads of block*3/4 bytes, out1 = ceil(nblk/2)*rows*2 exponent bytes.
 * `noise` (may be NULL) as in axs6_fq_with_noise; if NULL and rounding is stochastic the
 * Philox stream (seed, offset) is used. */
int axs6_pack(const void *x, int in_dtype, int64_t rows, int64_t cols, int64_t ldx,
              int block, int grid, int rounding, uint32_t flags,
              uint64_t seed, uint64_t offset, const float *noise,
              int layout, void *out0, void *out1, void *out2, axs6_stream_t stream);

/* Codes back to values.  Replaces dequantize_unified (axs/unified/quantize_unified.py:285-308),
 * dequantize (axs/core.py:372-403), _unpack_from_flat_buffer + _unpack_gradient
 * (axs/unified/distributed.py:123-144, :201-232) and AXSBlock.from_bytes (axs/core.py:120-152).
 * The fp32 result is bit-exact; out_dtype BF16 rounds it to nearest-even. */
int axs6_unpack(int layout, const void *in0, const void *in1, const void *in2,
                void *y, int out_dtype, int64_t rows, int64_t cols, int64_t ldy,
                int block, int grid, axs6_stream_t stream);

/* Planes <-> byte records without touching values: to_records = 1 packs (exponents, signs,
 * magnitudes) of `nblocks` blocks into WIRE or SPEC records, to_records = 0 unpacks them.
 * Replaces _pack_to_flat_buffer / _unpack_from_flat_buffer (axs/unified/distributed.py:147-232)
 * and AXSBlock.to_bytes / from_bytes (axs/core.py:97-152) for data already held as planes. */
int axs6_repack(int to_records, int layout, int block, int64_t nblocks,
                void *exponents, void *signs, void *magnitudes, void *records, axs6_stream_t stream);

/* Bytes per block record of a byte layout (0 for PLANES or bad arguments). */
int64_t axs6_record_bytes(int layout, int block);

/* C[M,N] (+ bias[N]) = op(A) * op(B): bf16 operands, fp32 accumulation in tensor memory
 * (tcgen05), C stored as fp32 or bf16.  This is the GEMM under F.linear / torch.matmul / `@` in
 * the reference's Linear functions (axs/unified/mixed_precision.py:108, :139, :145;
 * axs/unified/functional_unified.py:123, :155-160; axs/nn/functional.py:121, :144-145), applied
 * to operands that are already fake-quantised.
 *   a_mn = 0: A is (M, K) row-major, leading dimension lda;  a_mn = 1: A is (K, M) row-major.
 *   b_mn = 0: B is (N, K) row-major, leading dimension ldb;  b_mn = 1: B is (K, N) row-major.
 * So forward = (0,0) with A = x_q, B = w_q;  dX = (0,1) with A = g_q, B = w_q;
 * dW = (1,1) with A = g_q, B = x_q (contraction over the rows of both).
 * A and B must be 16-byte aligned with leading dimensions multiples of 8 elements
 * (AXS6_ERR_ALIGN otherwise); C may have any alignment. */
int axs6_gemm_bf16(const void *a, const void *b, void *c, const float *bias,
                   int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                   int a_mn, int b_mn, int c_dtype, axs6_stream_t stream);

/* axs6_gemm_bf16 with a caller-owned workspace.  A product with few output tiles and a long contraction (fp32
 * output: the weight gradient of a small layer) is split along K so that most SMs get work.  Without a workspace at
 * most two partial products are formed and added into C in either order (bit-reproducible).  With `ws` of
 * axs6_gemm_workspace_bytes(M, N, K, c_dtype) bytes (16-byte aligned) up to eight partials are kept apart in it and
 * added in index order by a second kernel: as reproducible, and faster on such shapes.  A workspace that is null or
 * too small is ignored.  (No counterpart in the reference: torch.matmul owns its workspace.) */
int axs6_gemm_bf16_ws(const void *a, const void *b, void *c, const float *bias,
                      int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                      int a_mn, int b_mn, int c_dtype, void *ws, int64_t ws_bytes, axs6_stream_t stream);

/* Bytes of workspace from which axs6_gemm_bf16_ws can profit for this product on the current device (0: none). */
int64_t axs6_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int c_dtype);

/* The same product with one or both operands held as AXS-6 codes and decoded to bf16 inside the kernel
 * ("quantise on load"): the data flow of the reference's fused linear kernel, which produces the quantised
 * tile inside its K loop (axs/unified/triton_kernels.py:151-282), so that no quantised operand is written to
 * HBM as bf16.  An operand with a non-null exponent plane (`a_exps` / `b_exps`) is packed: its pointer is the
 * payload plane of AXS6_LAYOUT_SPLIT (NF5 grid, block 32, blocks along the operand's contiguous dimension,
 * as written by axs6_pack for the stored matrix: (M,K) or (K,M) for A, (N,K) or (K,N) for B) and its
 * leading dimension is ignored; its contiguous extent must be a multiple of 64 and its row count a multiple
 * of 8 (AXS6_ERR_UNSUPPORTED otherwise), both planes 16-byte aligned.  An operand with a null exponent plane is bf16 as in axs6_gemm_bf16.  At least one operand
 * must be packed.  The decoded values are bit-identical to axs6_unpack(..., AXS6_BF16) of the same codes;
 * note that codes cannot express an exact zero (axs/unified/quantize_unified.py:273, :300-302: a zero
 * input packs to the smallest level), which is where this differs from fake-quantising the operand. */
int axs6_gemm_packed(const void *a, const void *a_exps, int64_t lda, const void *b, const void *b_exps, int64_t ldb,
                     void *c, const float *bias, int64_t M, int64_t N, int64_t K, int64_t ldc,
                     int a_mn, int b_mn, int c_dtype, axs6_stream_t stream);

/* Same product with fp32 operands that the tensor cores consume as TF32 (kind::tf32): 10 mantissa
 * bits of every operand value are used, the rest is ignored.  For the fp32 Linear paths
 * (axs/unified/functional_unified.py:123, :155-160; axs/nn/functional.py:121, :144-145;
 * axs/unified/backend.py:540-618), where bf16 operands would exceed the 1e-3 error bar.  Operands
 * 16-byte aligned, leading dimensions multiples of 4 elements.  AXS6_FLAG_OUTPUT_TF32 of
 * axs6_fq produces operands already rounded to nearest TF32.  Only K-major operands
 * (a_mn = b_mn = 0): the TF32 instruction does not take MN-major ones (AXS6_ERR_UNSUPPORTED);
 * axs6_transpose_f32 makes the copy. */
int axs6_gemm_tf32(const void *a, const void *b, void *c, const float *bias,
                   int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                   int a_mn, int b_mn, int c_dtype, axs6_stream_t stream);

/* out (cols, rows) = in (rows, cols) transposed, fp32.  Plumbing for the TF32 products, which
 * need K-major operands (replaces the `.t().contiguous()` of
 * axs/unified/functional_unified.py:157-158). */
int axs6_transpose_f32(const float *in, float *out, int64_t rows, int64_t cols,
                       int64_t ldin, int64_t ldout, axs6_stream_t stream);

/* Device-side status of the GEMM kernels since the last call of this function: 0 = every
 * wait inside the kernels completed; n > 0 = a bounded wait gave up (1 TMA producer waiting
 * for a free stage, 2 MMA issuer waiting for a free accumulator, 3 MMA issuer waiting for a
 * loaded stage, 4 epilogue waiting for a finished accumulator; axs6_gemm_packed also 5 decode warps waiting
 * for a payload tile, 6 decode warps waiting for a free stage, 7 producer waiting for a free payload stage)
 * and the result is invalid.
 * Synchronises the device and clears the status. */
int axs6_gemm_status(void);

/* The same for the pack / unpack kernels that are fed by the TMA unit (NF5 grid, nearest rounding,
 * block 32, byte layouts) and for axs6_unpack_sum: 0 = every wait completed; 1..3 = a pack (1 bf16,
 * 3 fp32) or unpack (2) kernel gave up waiting for a loaded tile, 11 / 12 = a consumer / the producer
 * of axs6_unpack_sum gave up, 21 = the TMA-fed bf16 fake-quantise kernel gave up; the output of that
 * launch is incomplete.  Synchronises the device and
 * clears the status.  No counterpart in the reference. */
int axs6_codec_status(void);

/* y = (unpack(records) + unpack(records + src_stride) + ... nsrc terms) / divisor, summed in fp32 in
 * source order; every source holds the byte records (AXS6_LAYOUT_WIRE or AXS6_LAYOUT_SPEC) of the same
 * rows x cols tensor.  The receiving side of the compressed gradient exchange in ONE pass: it replaces
 * the loop "unpack each rank's buffer, add, divide by the world size" that follows the all-gather
 * (axs/unified/distributed.py:308-367 is the reference's packed hook; its arithmetic on the packed
 * bytes is not reproduced, the result here is the mean of the ranks' reconstructions).
 * src_stride in bytes (a multiple of 16 for the fast kernel); divisor != 0. */
int axs6_unpack_sum(int layout, const void *records, int64_t nsrc, int64_t src_stride, void *y,
                    int out_dtype, int64_t rows, int64_t cols, int64_t ldy, int block, int grid,
                    float divisor, axs6_stream_t stream);

/* AXS-6 Linear with bf16 tensor-core compute: the graph of _AXSLinearBF16Function
 * (axs/unified/mixed_precision.py:86-155), also reached through accelerated_linear /
 * triton_fused_linear (axs/unified/backend.py:540-618, axs/unified/triton_kernels.py:385-482).
 *
 * Forward:  xq = FQ(bf16(x)) (or bf16(x) without AXS6_LINEAR_QUANTIZE_INPUT), wq = FQ(bf16(w)),
 *           y (M,N) = xq wq^T + bias, fp32 accumulation, y stored as y_dtype.
 * With AXS6_LINEAR_COMPUTE_TF32 the same call runs the fp32 graph of _AXSLinearUnifiedFunction
 * (axs/unified/functional_unified.py:89-170) and, with grid = AXS6_GRID_UNIFORM, of
 * _AXSLinearFunction (axs/nn/functional.py:93-148): no bf16 cast, TF32 products.
 * x is (M,K), w is (N,K); bias (fp32, length N) may be NULL.  xq and wq are caller-owned bf16
 * buffers of axs6_linear_workspace_bytes(0 | 1, M, N, K) bytes, 16-byte aligned, row length
 * round_up(K, 8); xq must be kept for the backward call (the reference saves input_q). */
int axs6_linear_fwd(const void *x, int x_dtype, int64_t ldx, const void *w, int w_dtype, int64_t ldw,
                    const float *bias, void *y, int y_dtype, int64_t ldy,
                    int64_t M, int64_t N, int64_t K, int block, int grid, uint32_t flags,
                    void *xq, void *wq, axs6_stream_t stream);

/* Backward:  gq = FQ_stochastic(bf16(g)) (or bf16(g) without AXS6_LINEAR_QUANTIZE_GRAD,
 *            mixed_precision.py:133-136), dw (N,K) = gq^T xq in fp32 (:145), wq = FQ(bf16(w)) (recomputed, :130,
 *            unless AXS6_LINEAR_REUSE_WQ), dx (M,K) = gq wq stored as dx_dtype (:139), db (N) = column sums of
 *            the un-quantised g in fp32 (:150), enqueued in this order.  Any of dx, dw, db may be NULL (not needed).
 * `noise` (may be NULL): U[0,1) draws for the gradient in the padded (M, nblk, block) layout,
 * instead of the Philox stream (seed, offset).  Workspaces: gq = what 2, wq = what 1,
 * db_partial = what 3 of axs6_linear_workspace_bytes (db_partial only if db is given);
 * tf32_scratch = what 7, only for AXS6_LINEAR_COMPUTE_TF32 (transposed operand copies), else NULL. */
int axs6_linear_bwd(const void *g, int g_dtype, int64_t ldg, const void *xq,
                    const void *w, int w_dtype, int64_t ldw,
                    void *dx, int dx_dtype, int64_t lddx, float *dw, int64_t lddw, float *db,
                    int64_t M, int64_t N, int64_t K, int block, int grid, uint32_t flags,
                    uint64_t seed, uint64_t offset, const float *noise,
                    void *gq, void *wq, float *db_partial, void *tf32_scratch, axs6_stream_t stream);

/* Bias gradient: db[n] = sum over rows of g[row, n], accumulated in fp32 in a fixed order
 * (deterministic).  Replaces grad_output.float().sum(dim=...) of the Linear backward
 * (axs/unified/mixed_precision.py:149-153, axs/unified/functional_unified.py:161-165,
 * axs/nn/functional.py:146).  db_partial: caller-owned scratch of
 * axs6_linear_workspace_bytes(3, 0, cols, 0) bytes that holds the per-row-range partial sums. */
int axs6_bias_grad(const void *g, int g_dtype, int64_t ldg, int64_t rows, int64_t cols,
                   float *db, float *db_partial, axs6_stream_t stream);

/* Bias gradient for callers that cannot hand over a scratch buffer.  (No counterpart in the
 * reference: its bias gradient is a torch reduction that allocates freely.)
 * Same result as axs6_bias_grad, bit for bit, but the partial sums go to a fixed 2 MiB array
 * inside the library instead of `db_partial`, and the call performs no cudaMalloc / cudaFree
 * and uses no allocating library routine.  Meant for hosts that own no device allocator at
 * the point of the call: a plugin behind cgo / JNI / ctypes that is given input and output
 * pointers only, or a serving process whose memory plan was fixed at start-up and which has
 * handed all remaining HBM to its own pool, where a late cudaMalloc fails or stalls every
 * stream with its implicit synchronisation.
 *   - cols <= 16384, otherwise AXS6_ERR_TOO_LARGE; any number of rows.
 *   - The first call on each device looks up the array's device address (that device must be
 *     current, as for every call); make that first call before any stream capture begins.
 *   - All calls on a device share the one array.  It keeps the previous call's contents, which
 *     is harmless because each call overwrites every entry it later reads; but two calls whose
 *     kernels overlap on the GPU (different streams, no ordering) race on it and give garbage.
 *     Order them on one stream or with events.
 *   - The array stays resident on every GPU that loads the library until the process exits. */
int axs6_bias_grad_static(const void *g, int g_dtype, int64_t ldg, int64_t rows, int64_t cols,
                          float *db, axs6_stream_t stream);

/* Bytes of a caller-owned work buffer: what 0 = xq, 1 = wq, 2 = gq (bf16 compute), 3 = db_partial,
 * 4 = xq, 5 = wq, 6 = gq of the AXS6_LINEAR_COMPUTE_TF32 graph (fp32), 7 = its tf32_scratch,
 * 12 = xq, 13 = wq of AXS6_LINEAR_FP32_ACCURACY,
 * 8 = xq, 9 = wq, 10 = gq of AXS6_LINEAR_OPERANDS_PACKED (codes), 11 = split-K partials of dw for
 * AXS6_LINEAR_SPLITK_WORKSPACE (0 when the product would not be split further). */
int64_t axs6_linear_workspace_bytes(int what, int64_t M, int64_t N, int64_t K);

#ifdef __cplusplus
}
#endif
#endif /* AXS6_B200_H */
