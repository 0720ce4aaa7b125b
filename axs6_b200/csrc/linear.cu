// AXS-6 Linear forward and backward as sequences of library kernels on one stream:
// fake-quantise the operands to bf16 (one HBM pass each), then the tcgen05 GEMMs.
//
//   forward   xq = FQ(bf16(x))  wq = FQ(bf16(w))  y = xq wq^T + bias
//   backward  gq = FQ_stochastic(bf16(g))  dw = gq^T xq (fp32)  wq = FQ(bf16(w)) (or the forward's, reused)
//             dx = gq wq  db = column sums of the un-quantised g (fp32)
// This is the graph of _AXSLinearBF16Function (axs/unified/mixed_precision.py:86-155).  xq is
// materialised because backward needs it (the reference saves input_q); gq is materialised
// because dx and dw must see the same stochastic rounding (the reference quantises once).
// Also here: the cast kernel for operands that are not quantised and the column-sum kernels.
#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"

namespace axs6 {

// ------------------------------------------------------------------------------ cast to bf16
// y(bf16) = x (fp32 or bf16), row-major with leading dimensions; 8 values per thread when
// aligned, scalar otherwise.
template <typename Tin>
__global__ void __launch_bounds__(256) cast_bf16_kernel(const Tin *x, __nv_bfloat16 *y, int64_t rows, int64_t cols,
                                                        int64_t ldx, int64_t ldy, int vec)
{
    if (vec) {
        const int64_t cpr = cols / 8, total = rows * cpr;
        for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < total; c += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = c / cpr, col = (c - r * cpr) * 8;
            uint4 out;
            if (sizeof(Tin) == 4) {
                const float4 a = *reinterpret_cast<const float4 *>(x + r * ldx + col);
                const float4 b = *reinterpret_cast<const float4 *>(x + r * ldx + col + 4);
                __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x, a.y), h1 = __floats2bfloat162_rn(a.z, a.w);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(b.x, b.y), h3 = __floats2bfloat162_rn(b.z, b.w);
                out = make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                                 *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
            } else {
                out = *reinterpret_cast<const uint4 *>(x + r * ldx + col);
            }
            *reinterpret_cast<uint4 *>(y + r * ldy + col) = out;
        }
    } else {
        const int64_t total = rows * cols;
        for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = e / cols, col = e - r * cols;
            y[r * ldy + col] = __float2bfloat16_rn((float)x[r * ldx + col]);
        }
    }
}

static int cast_to_bf16(const void *x, int dtype, void *y, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                        cudaStream_t st)
{
    const DeviceInfo &d = device_info();
    const int vec = aligned16(x) && aligned16(y) && cols % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0;
    int64_t items = vec ? rows * cols / 8 : rows * cols;
    int64_t ctas = (items + 255) / 256;
    if (ctas > (int64_t)d.sms * 8) ctas = (int64_t)d.sms * 8;
    if (ctas < 1) ctas = 1;
    if (dtype == AXS6_F32)
        cast_bf16_kernel<float><<<(unsigned)ctas, 256, 0, st>>>(static_cast<const float *>(x), static_cast<__nv_bfloat16 *>(y), rows, cols, ldx, ldy, vec);
    else
        cast_bf16_kernel<__nv_bfloat16><<<(unsigned)ctas, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), static_cast<__nv_bfloat16 *>(y), rows, cols, ldx, ldy, vec);
    count_launch();
    return check_launch();
}

// y(fp32, rounded to the nearest TF32 value) = x (fp32 or bf16): the operand copy of the TF32
// Linear for tensors that are not quantised.
template <typename Tin>
__global__ void __launch_bounds__(256) cast_tf32_kernel(const Tin *x, float *y, int64_t rows, int64_t cols,
                                                        int64_t ldx, int64_t ldy, int round)
{
    const int64_t total = rows * cols;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = e / cols, col = e - r * cols;
        const float v = (float)x[r * ldx + col];
        uint32_t t = __float_as_uint(v);
        if (round) asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(v));
        y[r * ldy + col] = __uint_as_float(t);
    }
}

static int cast_to_tf32(const void *x, int dtype, void *y, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                        cudaStream_t st, int round = 1)
{
    const DeviceInfo &d = device_info();
    int64_t ctas = (rows * cols + 255) / 256;
    if (ctas > (int64_t)d.sms * 8) ctas = (int64_t)d.sms * 8;
    if (ctas < 1) ctas = 1;
    if (dtype == AXS6_F32)
        cast_tf32_kernel<float><<<(unsigned)ctas, 256, 0, st>>>(static_cast<const float *>(x), static_cast<float *>(y), rows, cols, ldx, ldy, round);
    else
        cast_tf32_kernel<__nv_bfloat16><<<(unsigned)ctas, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), static_cast<float *>(y), rows, cols, ldx, ldy, round);
    count_launch();
    return check_launch();
}

// ------------------------------------------------------------------------------ fp32 as two TF32 parts
// out (rows, 3 * ld) = three column blocks built from x = hi + lo, hi = the nearest TF32 value, lo = the nearest
// TF32 value of the remainder:  which = 0 (left operand)  [hi | hi | lo],  which = 1 (right operand)  [hi | lo | hi].
// The product of a left and a right operand over the tripled contraction is hi*hi + hi*lo + lo*hi: the fp32 product
// to about 2^-21 instead of the 2^-11 of a single TF32 product.  Columns >= cols of each block are zero.
__global__ void __launch_bounds__(256) split_tf32_kernel(const float *x, float *out, int64_t rows, int64_t cols, int64_t ldx,
                                                         int64_t ld, int which)
{
    const int64_t total = rows * ld;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = e / ld, c = e - r * ld;
        const float v = c < cols ? x[r * ldx + c] : 0.0f;
        uint32_t hb, lb;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(v));
        const float hi = __uint_as_float(hb);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(v - hi));
        const float lo = __uint_as_float(lb);
        float *o = out + r * 3 * ld + c;
        o[0] = hi;
        o[ld] = which ? lo : hi;
        o[2 * ld] = which ? hi : lo;
    }
}

static int split_tf32(const float *x, float *out, int64_t rows, int64_t cols, int64_t ldx, int64_t ld, int which, cudaStream_t st)
{
    const DeviceInfo &d = device_info();
    int64_t ctas = (rows * ld + 255) / 256;
    if (ctas > (int64_t)d.sms * 8) ctas = (int64_t)d.sms * 8;
    if (ctas < 1) ctas = 1;
    split_tf32_kernel<<<(unsigned)ctas, 256, 0, st>>>(x, out, rows, cols, ldx, ld, which);
    count_launch();
    return check_launch();
}

// ------------------------------------------------------------------------------ fp32 transpose
// out (cols, rows) = in (rows, cols)^T through 32 x 33 shared-memory tiles.  The TF32 tensor-core
// instruction takes K-major operands only, so the two backward products of the fp32 graph read
// transposed copies of their operands.
__global__ void __launch_bounds__(256) transpose_f32_kernel(const float *in, float *out, int64_t rows, int64_t cols,
                                                            int64_t ldin, int64_t ldout, int round_tf32)
{
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;       // 32 x 8
    const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    for (int i = ty; i < 32; i += 8) {
        const int64_t r = r0 + i, c = c0 + tx;
        float v = (r < rows && c < cols) ? in[r * ldin + c] : 0.0f;
        if (round_tf32) {                // the TF32 tensor core would truncate: round to nearest here instead
            uint32_t t;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(v));
            v = __uint_as_float(t);
        }
        tile[i][tx] = v;
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const int64_t c = c0 + i, r = r0 + tx;
        if (c < cols && r < rows) out[c * ldout + r] = tile[tx][i];
    }
}

static int transpose_f32(const float *in, float *out, int64_t rows, int64_t cols, int64_t ldin, int64_t ldout, cudaStream_t st,
                         int round_tf32 = 0)
{
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
    if (grid.y > 65535u) return AXS6_ERR_UNSUPPORTED;
    transpose_f32_kernel<<<grid, 256, 0, st>>>(in, out, rows, cols, ldin, ldout, round_tf32);
    count_launch();
    return check_launch();
}

// ------------------------------------------------------------------------------ column sums
// out[n] = sum over rows of g[row, n] in fp32, deterministic: phase 1 writes kSplits partial
// sums per column (each over a contiguous row range, rows visited in order), phase 2 adds them.
constexpr int kSplits = 32;

template <typename T>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const T *g, float *partial, int64_t rows, int64_t cols, int64_t ld)
{
    // CTA: 64 columns x (256/64 = 4 row lanes); grid (ceil(cols/64), kSplits)
    __shared__ float red[4][64];
    pdl_launch_dependents();                          // the second phase may set up; it waits for this grid before it reads
    const int cx = threadIdx.x & 63, ry = threadIdx.x >> 6;
    const int64_t col = (int64_t)blockIdx.x * 64 + cx;
    const int64_t per = (rows + kSplits - 1) / kSplits;
    const int64_t r0 = (int64_t)blockIdx.y * per;
    const int64_t r1 = r0 + per < rows ? r0 + per : rows;
    float acc = 0.0f;
    if (col < cols)
        for (int64_t r = r0 + ry; r < r1; r += 4) acc += (float)g[r * ld + col];
    red[ry][cx] = acc;
    __syncthreads();
    if (ry == 0 && col < cols)
        partial[(int64_t)blockIdx.y * cols + col] = (red[0][cx] + red[1][cx]) + (red[2][cx] + red[3][cx]);
}

// Same partial sums with 16-byte loads (aligned tensors whose column count is a multiple of 8 values for
// bf16 / 4 for fp32): CTA = 32 column chunks x 8 row lanes, each thread keeps one chunk's running sums.
// The order of additions per column is: rows r0 + lane, r0 + lane + 8, ... within a lane, then lanes 0..7.
template <typename T>
__global__ void __launch_bounds__(256) colsum_partial_vec_kernel(const T *g, float *partial, int64_t rows, int64_t cols, int64_t ld)
{
    constexpr int V = 16 / (int)sizeof(T);            // values per 16-byte chunk
    __shared__ float red[8][32 * V + 1];
    pdl_launch_dependents();
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int64_t col0 = ((int64_t)blockIdx.x * 32 + cx) * V;
    const int64_t per = (rows + kSplits - 1) / kSplits;
    const int64_t r0 = (int64_t)blockIdx.y * per;
    const int64_t r1 = r0 + per < rows ? r0 + per : rows;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.0f;
    if (col0 < cols) {
        for (int64_t r = r0 + ry; r < r1; r += 8) {
            const uint4 v = *reinterpret_cast<const uint4 *>(g + r * ld + col0);
            if (sizeof(T) == 4) {
                acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
                acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
            } else {
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[(2 * i) % V] += __uint_as_float(w[i] << 16);
                    acc[(2 * i + 1) % V] += __uint_as_float(w[i] & 0xFFFF0000u);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) red[ry][cx * V + i] = acc[i];
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * V; i += 256) {
        const int64_t col = (int64_t)blockIdx.x * 32 * V + i;
        if (col < cols) {
            float s = 0.0f;
#pragma unroll
            for (int l = 0; l < 8; ++l) s += red[l][i];
            partial[(int64_t)blockIdx.y * cols + col] = s;
        }
    }
}

__global__ void __launch_bounds__(256) colsum_final_kernel(const float *partial, float *out, int64_t cols)
{
    const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_wait();                                       // phase 1 has finished and its partial sums are visible
    if (col >= cols) return;
    float acc = 0.0f;
    for (int s = 0; s < kSplits; ++s) acc += partial[(int64_t)s * cols + col];
    out[col] = acc;
}

static int column_sums(const void *g, int dtype, float *out, float *partial, int64_t rows, int64_t cols, int64_t ld,
                       cudaStream_t st)
{
    const int V = dtype == AXS6_F32 ? 4 : 8;
    if (aligned16(g) && cols % V == 0 && ld % V == 0) {
        dim3 grid((unsigned)((cols + 32 * V - 1) / (32 * V)), kSplits);
        if (dtype == AXS6_F32)
            colsum_partial_vec_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float *>(g), partial, rows, cols, ld);
        else
            colsum_partial_vec_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(g), partial, rows, cols, ld);
    } else {
        dim3 grid((unsigned)((cols + 63) / 64), kSplits);
        if (dtype == AXS6_F32)
            colsum_partial_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float *>(g), partial, rows, cols, ld);
        else
            colsum_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(g), partial, rows, cols, ld);
    }
    if (launch_overlapped(true, colsum_final_kernel, (unsigned)((cols + 255) / 256), 256, 0, st, (const float *)partial, out, cols) != cudaSuccess)
        return AXS6_ERR_LAUNCH;
    count_launch(2);
    return check_launch();
}

static int64_t round_up8(int64_t v) { return (v + 7) / 8 * 8; }
// A (rows, cols) operand held as codes: the payload plane (rows * cols/32 * 24 bytes, rounded up to 256) followed by
// the exponent plane (stored by pairs of blocks: ceil(nblk / 2) * rows * 2 bytes).
static int64_t packed_exps_offset(int64_t rows, int64_t cols) { return (rows * ((cols + 31) / 32) * 24 + 255) / 256 * 256; }
static int64_t packed_bytes(int64_t rows, int64_t cols)
{
    return packed_exps_offset(rows, cols) + ((((cols + 31) / 32) + 1) / 2) * rows * 2;
}
static int pack_operand(const void *x, int dtype, int64_t rows, int64_t cols, int64_t ld, int rounding, uint64_t seed,
                        uint64_t offset, const float *noise, void *ws, axs6_stream_t stream)
{
    return axs6_pack(x, dtype, rows, cols, ld, 32, AXS6_GRID_NF5, rounding, AXS6_FLAG_INPUT_VIA_BF16, seed, offset, noise,
                     AXS6_LAYOUT_SPLIT, ws, static_cast<uint8_t *>(ws) + packed_exps_offset(rows, cols), nullptr, stream);
}
static const void *exps_of(const void *ws, int64_t rows, int64_t cols)
{
    return static_cast<const uint8_t *>(ws) + packed_exps_offset(rows, cols);
}
static int64_t round_up4(int64_t v) { return (v + 3) / 4 * 4; }

}  // namespace axs6

AXS6_API int axs6_bias_grad(const void *g, int g_dtype, int64_t ldg, int64_t rows, int64_t cols, float *db,
                            float *db_partial, axs6_stream_t stream)
{
    using namespace axs6;
    if (!valid_dtype(g_dtype) || rows < 0 || cols < 0 || ldg < cols) return AXS6_ERR_ARG;
    if (cols == 0) return AXS6_OK;
    if (!g || !db) return AXS6_ERR_ARG;
    if (!db_partial) return AXS6_ERR_WORKSPACE;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;
    return column_sums(g, g_dtype, db, db_partial, rows, cols, ldg, static_cast<cudaStream_t>(stream));
}

AXS6_API int64_t axs6_linear_workspace_bytes(int what, int64_t M, int64_t N, int64_t K)
{
    using namespace axs6;
    if (M < 0 || N < 0 || K < 0) return -1;
    switch (what) {
    case 0: return M * round_up8(K) * 2;            // xq: bf16 (M, round_up(K, 8))
    case 1: return N * round_up8(K) * 2;            // wq: bf16 (N, round_up(K, 8))
    case 2: return M * round_up8(N) * 2;            // gq: bf16 (M, round_up(N, 8))
    case 3: return (int64_t)kSplits * N * 4;        // column-sum partials
    case 4: return M * round_up4(K) * 4;            // xq of the TF32 path: fp32 (M, round_up(K, 4))
    case 5: return N * round_up4(K) * 4;            // wq, TF32 path
    case 6: return M * round_up4(N) * 4;            // gq, TF32 path
    case 7: return (K * round_up4(N) + N * round_up4(M) + K * round_up4(M)) * 4;   // transposes, TF32 backward
    case 8: return packed_bytes(M, K);              // xq as codes (AXS6_LINEAR_OPERANDS_PACKED)
    case 9: return packed_bytes(N, K);              // wq as codes
    case 10: return packed_bytes(M, N);             // gq as codes
    case 12: return M * round_up4(K) * 16;          // xq of AXS6_LINEAR_FP32_ACCURACY: fp32 (M, ld) + its three-part split (M, 3 ld)
    case 13: return N * round_up4(K) * 16;          // wq, the same
    case 11: return axs6_gemm_workspace_bytes(N, K, M, AXS6_F32);   // split-K partials of dw (0: none useful)
    default: return -1;
    }
}

AXS6_API int axs6_linear_fwd(const void *x, int x_dtype, int64_t ldx, const void *w, int w_dtype, int64_t ldw,
                             const float *bias, void *y, int y_dtype, int64_t ldy, int64_t M, int64_t N, int64_t K,
                             int block, int grid, uint32_t flags, void *xq, void *wq, axs6_stream_t stream)
{
    using namespace axs6;
    if (!valid_dtype(x_dtype) || !valid_dtype(w_dtype) || !valid_dtype(y_dtype) || !valid_block(block)) return AXS6_ERR_ARG;
    if (grid != AXS6_GRID_NF5 && grid != AXS6_GRID_UNIFORM) return AXS6_ERR_ARG;
    if (M < 0 || N < 0 || K < 0 || ldx < K || ldw < K || ldy < N) return AXS6_ERR_ARG;
    if (flags & ~(AXS6_LINEAR_QUANTIZE_INPUT | AXS6_LINEAR_COMPUTE_TF32 | AXS6_LINEAR_BIAS_VIA_BF16 | AXS6_LINEAR_OPERANDS_PACKED |
                  AXS6_LINEAR_FP32_ACCURACY))
        return AXS6_ERR_ARG;
    if ((flags & AXS6_LINEAR_FP32_ACCURACY) && !(flags & AXS6_LINEAR_COMPUTE_TF32)) return AXS6_ERR_ARG;
    if (M == 0 || N == 0) return AXS6_OK;
    if (!x || !w || !y || !xq || !wq || K == 0) return AXS6_ERR_ARG;
    if (!aligned16(xq) || !aligned16(wq)) return AXS6_ERR_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (flags & AXS6_LINEAR_OPERANDS_PACKED) {
        // quantise on load: both operands go to HBM as 6-bit codes (0.78 bytes per value) and are decoded to bf16
        // inside the GEMM; xq (codes) is what backward keeps
        if ((flags & AXS6_LINEAR_COMPUTE_TF32) || !(flags & AXS6_LINEAR_QUANTIZE_INPUT) || block != 32 || grid != AXS6_GRID_NF5 ||
            K % 64 || N % 64 || M % 8)
            return AXS6_ERR_UNSUPPORTED;
        int rcp = pack_operand(w, w_dtype, N, K, ldw, AXS6_ROUND_NEAREST, 0, 0, nullptr, wq, stream);
        if (rcp) return rcp;
        rcp = pack_operand(x, x_dtype, M, K, ldx, AXS6_ROUND_NEAREST, 0, 0, nullptr, xq, stream);
        if (rcp) return rcp;
        return gemm_packed_launch(xq, exps_of(xq, M, K), 0, wq, exps_of(wq, N, K), 0, y, bias, M, N, K, ldy, 0, 0, y_dtype,
                                  (flags & AXS6_LINEAR_BIAS_VIA_BF16) ? 1 : 0, st);
    }
    if (flags & AXS6_LINEAR_COMPUTE_TF32) {
        // fp32 graph (axs/unified/functional_unified.py:107-131, axs/nn/functional.py:101-129): operands
        // fake-quantised in fp32, rounded to TF32, product on the TF32 tensor cores
        const int64_t ld4 = round_up4(K);
        if (flags & AXS6_LINEAR_FP32_ACCURACY) {
            // fp32 accuracy on the TF32 tensor cores: the fake-quantised operands stay full fp32 (xq keeps them for
            // backward), each is split into two TF32 parts, and one product over the tripled contraction adds
            // hi*hi + hi*lo + lo*hi (axs/unified/triton_kernels.py:262 asks its dot product for "ieee" precision)
            float *xf = static_cast<float *>(xq), *wf = static_cast<float *>(wq);
            float *xs = xf + M * ld4, *ws = wf + N * ld4;
            int rc3 = axs6_fq(w, wf, w_dtype, AXS6_F32, N, K, ldw, ld4, block, grid, AXS6_ROUND_NEAREST, 0, 0, 0, stream);
            if (rc3) return rc3;
            rc3 = (flags & AXS6_LINEAR_QUANTIZE_INPUT)
                      ? axs6_fq(x, xf, x_dtype, AXS6_F32, M, K, ldx, ld4, block, grid, AXS6_ROUND_NEAREST, 0, 0, 0, stream)
                      : cast_to_tf32(x, x_dtype, xf, M, K, ldx, ld4, st, 0);
            if (rc3) return rc3;
            rc3 = split_tf32(xf, xs, M, K, ld4, ld4, 0, st);
            if (rc3) return rc3;
            rc3 = split_tf32(wf, ws, N, K, ld4, ld4, 1, st);
            if (rc3) return rc3;
            return axs6_gemm_tf32(xs, ws, y, bias, M, N, 3 * ld4, 3 * ld4, 3 * ld4, ldy, 0, 0, y_dtype, stream);
        }
        int rc4 = axs6_fq(w, wq, w_dtype, AXS6_F32, N, K, ldw, ld4, block, grid, AXS6_ROUND_NEAREST,
                          AXS6_FLAG_OUTPUT_TF32, 0, 0, stream);
        if (rc4) return rc4;
        if (flags & AXS6_LINEAR_QUANTIZE_INPUT)
            rc4 = axs6_fq(x, xq, x_dtype, AXS6_F32, M, K, ldx, ld4, block, grid, AXS6_ROUND_NEAREST,
                          AXS6_FLAG_OUTPUT_TF32, 0, 0, stream);
        else
            rc4 = cast_to_tf32(x, x_dtype, xq, M, K, ldx, ld4, st);
        if (rc4) return rc4;
        return axs6_gemm_tf32(xq, wq, y, bias, M, N, K, ld4, ld4, ldy, 0, 0, y_dtype, stream);
    }
    const int64_t ldq = round_up8(K);
    int rc = axs6_fq(w, wq, w_dtype, AXS6_BF16, N, K, ldw, ldq, block, grid, AXS6_ROUND_NEAREST,
                     AXS6_FLAG_INPUT_VIA_BF16, 0, 0, stream);
    if (rc) return rc;
    if (flags & AXS6_LINEAR_QUANTIZE_INPUT)
        rc = axs6_fq(x, xq, x_dtype, AXS6_BF16, M, K, ldx, ldq, block, grid, AXS6_ROUND_NEAREST,
                     AXS6_FLAG_INPUT_VIA_BF16, 0, 0, stream);
    else
        rc = cast_to_bf16(x, x_dtype, xq, M, K, ldx, ldq, st);
    if (rc) return rc;
    return gemm_launch(false, xq, wq, y, bias, M, N, K, ldq, ldq, ldy, 0, 0, y_dtype,
                       (flags & AXS6_LINEAR_BIAS_VIA_BF16) ? 1 : 0, st);
}

AXS6_API int axs6_linear_bwd(const void *g, int g_dtype, int64_t ldg, const void *xq, const void *w, int w_dtype,
                             int64_t ldw, void *dx, int dx_dtype, int64_t lddx, float *dw, int64_t lddw, float *db,
                             int64_t M, int64_t N, int64_t K, int block, int grid, uint32_t flags, uint64_t seed,
                             uint64_t offset, const float *noise, void *gq, void *wq, float *db_partial,
                             void *tf32_scratch, axs6_stream_t stream)
{
    using namespace axs6;
    if (!valid_dtype(g_dtype) || !valid_dtype(w_dtype) || !valid_block(block)) return AXS6_ERR_ARG;
    if (grid != AXS6_GRID_NF5 && grid != AXS6_GRID_UNIFORM) return AXS6_ERR_ARG;
    if (M < 0 || N < 0 || K < 0 || ldg < N) return AXS6_ERR_ARG;
    if (flags & ~(AXS6_LINEAR_QUANTIZE_GRAD | AXS6_LINEAR_COMPUTE_TF32 | AXS6_LINEAR_BIAS_FROM_QUANTIZED |
                  AXS6_LINEAR_REUSE_WQ | AXS6_LINEAR_REUSE_GQ | AXS6_LINEAR_OPERANDS_PACKED | AXS6_LINEAR_SPLITK_WORKSPACE))
        return AXS6_ERR_ARG;
    if ((flags & AXS6_LINEAR_SPLITK_WORKSPACE) && ((flags & AXS6_LINEAR_COMPUTE_TF32) || !tf32_scratch)) return AXS6_ERR_WORKSPACE;
    if ((flags & AXS6_LINEAR_COMPUTE_TF32) && (flags & (AXS6_LINEAR_REUSE_WQ | AXS6_LINEAR_REUSE_GQ))) return AXS6_ERR_UNSUPPORTED;
    if (M == 0 || N == 0 || K == 0) return AXS6_OK;
    if (!g || !gq) return AXS6_ERR_ARG;
    if (dx && (!wq || !valid_dtype(dx_dtype) || lddx < K)) return AXS6_ERR_ARG;
    if (dx && !(flags & AXS6_LINEAR_REUSE_WQ) && (!w || ldw < K)) return AXS6_ERR_ARG;
    if (dw && (!xq || lddw < K)) return AXS6_ERR_ARG;
    if (db && !db_partial) return AXS6_ERR_WORKSPACE;
    if (!aligned16(gq) || (wq && !aligned16(wq)) || (xq && !aligned16(xq))) return AXS6_ERR_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    if (flags & AXS6_LINEAR_COMPUTE_TF32) {
        // fp32 graph (axs/unified/functional_unified.py:134-170, axs/nn/functional.py:131-148)
        const int64_t ld4 = round_up4(K), ldg4 = round_up4(N);
        if (flags & AXS6_LINEAR_QUANTIZE_GRAD) {
            rc = noise ? axs6_fq_with_noise(g, gq, g_dtype, AXS6_F32, M, N, ldg, ldg4, block, grid,
                                            AXS6_FLAG_OUTPUT_TF32, noise, stream)
                       : axs6_fq(g, gq, g_dtype, AXS6_F32, M, N, ldg, ldg4, block, grid, AXS6_ROUND_STOCHASTIC,
                                 AXS6_FLAG_OUTPUT_TF32, seed, offset, stream);
        } else {
            rc = cast_to_tf32(g, g_dtype, gq, M, N, ldg, ldg4, st);
        }
        if (rc) return rc;
        if ((dx || dw) && !tf32_scratch) return AXS6_ERR_WORKSPACE;
        const int64_t ldn4 = round_up4(N), ldm4 = round_up4(M);
        float *wqT = static_cast<float *>(tf32_scratch);          // (K, N)
        float *gqT = wqT + K * ldn4;                               // (N, M)
        float *xqT = gqT + N * ldm4;                               // (K, M)
        if (dx) {
            rc = axs6_fq(w, wq, w_dtype, AXS6_F32, N, K, ldw, ld4, block, grid, AXS6_ROUND_NEAREST,
                         AXS6_FLAG_OUTPUT_TF32, 0, 0, stream);
            if (rc) return rc;
            rc = transpose_f32(static_cast<const float *>(wq), wqT, N, K, ld4, ldn4, st, 1);
            if (rc) return rc;
            // dx (M, K) = gq (M, N) * wq (N, K) = gq * (wq^T)^T with both operands K-major
            rc = axs6_gemm_tf32(gq, wqT, dx, nullptr, M, K, N, ldg4, ldn4, lddx, 0, 0, dx_dtype, stream);
            if (rc) return rc;
        }
        if (dw) {
            rc = transpose_f32(static_cast<const float *>(gq), gqT, M, N, ldg4, ldm4, st, 1);
            if (rc) return rc;
            // xq may hold full-precision fp32 (forward with AXS6_LINEAR_FP32_ACCURACY): rounded to TF32 on the way
            rc = transpose_f32(static_cast<const float *>(xq), xqT, M, K, ld4, ldm4, st, 1);
            if (rc) return rc;
            // dw (N, K) = gq^T (N, M) * xq (M, K)
            rc = axs6_gemm_tf32(gqT, xqT, dw, nullptr, N, K, M, ldm4, ldm4, lddw, 0, 0, AXS6_F32, stream);
            if (rc) return rc;
        }
        if (db) {
            // the quantised gradient's sums where the graph asks for them; without gradient quantisation gq is only the
            // TF32-rounded copy of g for the products, and the sums are taken from g itself
            const bool from_gq = (flags & AXS6_LINEAR_BIAS_FROM_QUANTIZED) && (flags & AXS6_LINEAR_QUANTIZE_GRAD);
            rc = from_gq ? axs6_bias_grad(gq, AXS6_F32, ldg4, M, N, db, db_partial, stream)
                         : axs6_bias_grad(g, g_dtype, ldg, M, N, db, db_partial, stream);
            if (rc) return rc;
        }
        return AXS6_OK;
    }
    if (flags & AXS6_LINEAR_OPERANDS_PACKED) {
        if ((flags & (AXS6_LINEAR_COMPUTE_TF32 | AXS6_LINEAR_BIAS_FROM_QUANTIZED)) || !(flags & AXS6_LINEAR_QUANTIZE_GRAD) ||
            block != 32 || grid != AXS6_GRID_NF5 || K % 64 || N % 64 || M % 8)
            return AXS6_ERR_UNSUPPORTED;
        if (!(flags & AXS6_LINEAR_REUSE_GQ)) {
            rc = pack_operand(g, g_dtype, M, N, ldg, AXS6_ROUND_STOCHASTIC, seed, offset, noise, gq, stream);
            if (rc) return rc;
        }
        if (dw) {       // dw (N, K) = gq^T xq: both operands stored (contraction, output), blocks along the output index
            rc = gemm_packed_launch(gq, exps_of(gq, M, N), 0, xq, exps_of(xq, M, K), 0, dw, nullptr, N, K, M, lddw, 1, 1,
                                    AXS6_F32, 0, st);
            if (rc) return rc;
        }
        if (dx) {
            if (!(flags & AXS6_LINEAR_REUSE_WQ)) {
                rc = pack_operand(w, w_dtype, N, K, ldw, AXS6_ROUND_NEAREST, 0, 0, nullptr, wq, stream);
                if (rc) return rc;
            }
            rc = gemm_packed_launch(gq, exps_of(gq, M, N), 0, wq, exps_of(wq, N, K), 0, dx, nullptr, M, K, N, lddx, 0, 1,
                                    dx_dtype, 0, st);
            if (rc) return rc;
        }
        if (db) {
            rc = axs6_bias_grad(g, g_dtype, ldg, M, N, db, db_partial, stream);
            if (rc) return rc;
        }
        return AXS6_OK;
    }
    const int64_t ldq = round_up8(K), ldgq = round_up8(N);
    if (flags & AXS6_LINEAR_REUSE_GQ) {
        rc = AXS6_OK;            // gq holds the quantised gradient of an earlier call on the same g
    } else if (flags & AXS6_LINEAR_QUANTIZE_GRAD) {
        rc = noise ? axs6_fq_with_noise(g, gq, g_dtype, AXS6_BF16, M, N, ldg, ldgq, block, grid,
                                        AXS6_FLAG_INPUT_VIA_BF16, noise, stream)
                   : axs6_fq(g, gq, g_dtype, AXS6_BF16, M, N, ldg, ldgq, block, grid, AXS6_ROUND_STOCHASTIC,
                             AXS6_FLAG_INPUT_VIA_BF16, seed, offset, stream);
    } else {
        rc = cast_to_bf16(g, g_dtype, gq, M, N, ldg, ldgq, st);
    }
    if (rc) return rc;
    // The weight gradient comes first: it is the product a data-parallel caller hands to its all-reduce, which
    // can then run under the input-gradient product (call once with dw only, start the collective, call again
    // with dx / db and AXS6_LINEAR_REUSE_GQ).
    if (dw) {
        // dw (N, K) = gq^T (N, M) * xq (M, K): contraction over M; both operands (contraction, output) row-major
        rc = (flags & AXS6_LINEAR_SPLITK_WORKSPACE)
                 ? axs6_gemm_bf16_ws(gq, xq, dw, nullptr, N, K, M, ldgq, ldq, lddw, 1, 1, AXS6_F32, tf32_scratch,
                                     axs6_gemm_workspace_bytes(N, K, M, AXS6_F32), stream)
                 : axs6_gemm_bf16(gq, xq, dw, nullptr, N, K, M, ldgq, ldq, lddw, 1, 1, AXS6_F32, stream);
        if (rc) return rc;
    }
    if (dx) {
        if (!(flags & AXS6_LINEAR_REUSE_WQ)) {
            rc = axs6_fq(w, wq, w_dtype, AXS6_BF16, N, K, ldw, ldq, block, grid, AXS6_ROUND_NEAREST,
                         AXS6_FLAG_INPUT_VIA_BF16, 0, 0, stream);
            if (rc) return rc;
        }
        // dx (M, K) = gq (M, N) * wq (N, K): contraction over N; wq is (contraction, output) row-major
        rc = axs6_gemm_bf16(gq, wq, dx, nullptr, M, K, N, ldgq, ldq, lddx, 0, 1, dx_dtype, stream);
        if (rc) return rc;
    }
    if (db) {
        rc = (flags & AXS6_LINEAR_BIAS_FROM_QUANTIZED) ? axs6_bias_grad(gq, AXS6_BF16, ldgq, M, N, db, db_partial, stream)
                                                       : axs6_bias_grad(g, g_dtype, ldg, M, N, db, db_partial, stream);
        if (rc) return rc;
    }
    return AXS6_OK;
}

// ------------------------------------------------------------------------------ bias gradient, no allocation
// Scratch for axs6_bias_grad_static: the per-row-range partial sums live in this fixed array
// instead of a caller-supplied buffer.  It is part of the module image, so every GPU that loads
// the library carries these 2 MiB until the process exits.
namespace axs6 {
constexpr int64_t kStaticMaxCols = 16384;
static __device__ __align__(256) float g_bias_grad_scratch[kSplits * kStaticMaxCols];
}  // namespace axs6

AXS6_API int axs6_bias_grad_static(const void *g, int g_dtype, int64_t ldg, int64_t rows, int64_t cols, float *db,
                                   axs6_stream_t stream)
{
    using namespace axs6;
    if (!valid_dtype(g_dtype) || rows < 0 || cols < 0 || ldg < cols) return AXS6_ERR_ARG;
    if (cols > kStaticMaxCols) return AXS6_ERR_TOO_LARGE;
    if (cols == 0) return AXS6_OK;
    if (!g || !db) return AXS6_ERR_ARG;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;

    // In host code the array's name is only a handle; the address the kernels need comes from
    // cudaGetSymbolAddress, looked up once per device while that device is current.
    static float *scratch_of_device[64];
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return AXS6_ERR_DEVICE;
    float *scratch;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!scratch_of_device[dev]) {
            void *ptr = nullptr;
            if (cudaGetSymbolAddress(&ptr, g_bias_grad_scratch) != cudaSuccess || !ptr) return AXS6_ERR_DEVICE;
            scratch_of_device[dev] = static_cast<float *>(ptr);
        }
        scratch = scratch_of_device[dev];
    }
    // Nothing has to start at zero: the first kernel writes every partial sum of the `cols`
    // columns before the second one reads them, so whatever the previous call left is overwritten.
    return column_sums(g, g_dtype, db, scratch, rows, cols, ldg, static_cast<cudaStream_t>(stream));
}

AXS6_API int axs6_transpose_f32(const float *in, float *out, int64_t rows, int64_t cols, int64_t ldin, int64_t ldout,
                                axs6_stream_t stream)
{
    using namespace axs6;
    if (rows < 0 || cols < 0 || ldin < cols || ldout < rows) return AXS6_ERR_ARG;
    if (rows == 0 || cols == 0) return AXS6_OK;
    if (!in || !out) return AXS6_ERR_ARG;
    const DeviceInfo &d = device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;
    return transpose_f32(in, out, rows, cols, ldin, ldout, static_cast<cudaStream_t>(stream));
}
