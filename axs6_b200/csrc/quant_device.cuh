// Device-side building blocks of the fake-quantise and codec kernels.
//
// Work decomposition of the vectorised kernels: the zero-padded tensor (rows, nblk*B) is cut
// into "chunks" of 8 consecutive values; one thread owns one chunk (one or two 128-bit
// loads), so a block of B values is owned by B/8 neighbouring lanes and its amax is a
// 0..2-step xor-shuffle.  Chunk c always starts at padded element index 8*c.
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace axs6 {

constexpr int kThreads = 256;      // threads per CTA of every elementwise kernel
constexpr int kChunk = 8;          // values per thread-chunk

enum Rounding { kNearest = 0, kPhilox = 1, kNoise = 2 };

struct ChunkGeom {
    int64_t rows, cols;      // logical extent
    int64_t cpr;             // chunks per zero-padded row = nblk * B / 8
    int64_t total_chunks;    // rows * cpr
    int block;               // B
    int flat;                // cols % B == 0 and all leading dimensions == cols
};

// ---- streaming 128-bit / 64-bit global accesses (data is touched exactly once) --------------
__device__ __forceinline__ uint4 ld_stream16(const void *p)
{
    uint4 v;
#ifndef AXS6_LD_HINT
#define AXS6_LD_HINT ".cs"
#endif
#ifndef AXS6_ST_HINT
#define AXS6_ST_HINT ".cs"
#endif
    asm volatile("ld.global" AXS6_LD_HINT ".v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream16(void *p, uint4 v)
{
    asm volatile("st.global" AXS6_ST_HINT ".v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint2 ld_stream8(const void *p)
{
    uint2 v;
    asm volatile("ld.global.cs.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream8(void *p, uint2 v)
{
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" :: "l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// ---- chunk load: 8 values -> fp32 bit patterns ----------------------------------------------
template <typename T> struct ChunkIO;

template <> struct ChunkIO<float> {
    static __device__ __forceinline__ void load(const void *base, int64_t elem, uint32_t (&v)[8], bool via_bf16)
    {
        const float *p = reinterpret_cast<const float *>(base) + elem;
        const uint4 a = ld_stream16(p), b = ld_stream16(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        if (via_bf16) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = (uint32_t)axs6_f32_to_bf16_bits(axs6_from_bits(v[i])) << 16;
        }
    }
    static __device__ __forceinline__ void store(void *base, int64_t elem, const float (&y)[8])
    {
        float *p = reinterpret_cast<float *>(base) + elem;
        st_stream16(p, make_uint4(__float_as_uint(y[0]), __float_as_uint(y[1]), __float_as_uint(y[2]), __float_as_uint(y[3])));
        st_stream16(p + 4, make_uint4(__float_as_uint(y[4]), __float_as_uint(y[5]), __float_as_uint(y[6]), __float_as_uint(y[7])));
    }
    static __device__ __forceinline__ uint32_t load1(const void *base, int64_t elem, bool via_bf16)
    {
        uint32_t u = __float_as_uint(reinterpret_cast<const float *>(base)[elem]);
        if (via_bf16) u = (uint32_t)axs6_f32_to_bf16_bits(axs6_from_bits(u)) << 16;
        return u;
    }
    static __device__ __forceinline__ void store1(void *base, int64_t elem, float y)
    {
        reinterpret_cast<float *>(base)[elem] = y;
    }
};

template <> struct ChunkIO<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const void *base, int64_t elem, uint32_t (&v)[8], bool)
    {
        const uint16_t *p = reinterpret_cast<const uint16_t *>(base) + elem;
        const uint4 a = ld_stream16(p);
        v[0] = a.x << 16; v[1] = a.x & 0xFFFF0000u; v[2] = a.y << 16; v[3] = a.y & 0xFFFF0000u;
        v[4] = a.z << 16; v[5] = a.z & 0xFFFF0000u; v[6] = a.w << 16; v[7] = a.w & 0xFFFF0000u;
    }
    static __device__ __forceinline__ void store(void *base, int64_t elem, const float (&y)[8])
    {
        uint16_t *p = reinterpret_cast<uint16_t *>(base) + elem;
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {   // one cvt.rn.bf16x2.f32 per pair (round to nearest even)
            const __nv_bfloat162 h = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        st_stream16(p, make_uint4(w[0], w[1], w[2], w[3]));
    }
    static __device__ __forceinline__ uint32_t load1(const void *base, int64_t elem, bool)
    {
        return (uint32_t)reinterpret_cast<const uint16_t *>(base)[elem] << 16;
    }
    static __device__ __forceinline__ void store1(void *base, int64_t elem, float y)
    {
        reinterpret_cast<uint16_t *>(base)[elem] = axs6_f32_to_bf16_bits(y);
    }
};

// ---- amax of a block spread over `lanes` neighbouring lanes ----------------------------------
// Works on |x| bit patterns: for non-negative floats the integer order is the float order.
__device__ __forceinline__ uint32_t chunk_amax_bits(const uint32_t (&v)[8])
{
    float m = 0.0f;                      // one FMNMX with |.| operand modifier per value
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(__uint_as_float(v[i])));
    return __float_as_uint(m);
}

__device__ __forceinline__ uint32_t group_max(uint32_t m, int lanes)
{
    // lanes in {1, 2, 4, 8, 16, 32}; uniform across the warp
    for (int d = 1; d < lanes; d <<= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, d));
    return m;
}

// ---- uniform draws for one chunk ---------------------------------------------------------------
template <int ROUND>
__device__ __forceinline__ void chunk_uniforms(float (&u)[8], int64_t chunk, bool active,
                                               const Axs6PhiloxKeys &keys, uint64_t offset, const float *noise)
{
    if (ROUND == kPhilox) {
        // one Philox4x32-10 block per chunk: eight 16-bit draws
        const Axs6Philox a = axs6_philox_keyed(offset + (uint64_t)chunk, keys);
#pragma unroll
        for (int i = 0; i < 4; ++i) { u[2 * i] = axs6_u01_16(a.r[i] & 0xFFFFu); u[2 * i + 1] = axs6_u01_16(a.r[i] >> 16); }
    } else if (ROUND == kNoise) {
        if (active) {
            const float4 a = *reinterpret_cast<const float4 *>(noise + chunk * 8);
            const float4 b = *reinterpret_cast<const float4 *>(noise + chunk * 8 + 4);
            u[0] = a.x; u[1] = a.y; u[2] = a.z; u[3] = a.w; u[4] = b.x; u[5] = b.y; u[6] = b.z; u[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) u[i] = 0.0f;
        }
    }
}

// Uniform draw for one padded element index (generic kernels).
template <int ROUND>
__device__ __forceinline__ float element_uniform(int64_t padded_index, bool active,
                                                 const Axs6PhiloxKeys &keys, uint64_t offset, const float *noise)
{
    if (ROUND == kPhilox) {
        const Axs6Philox a = axs6_philox_keyed(offset + (uint64_t)(padded_index >> 3), keys);
        const uint32_t w = a.r[(padded_index & 7) >> 1];
        return axs6_u01_16((padded_index & 1) ? (w >> 16) : (w & 0xFFFFu));
    }
    if (ROUND == kNoise) return active ? noise[padded_index] : 0.0f;
    return 0.0f;
}

// ---- shared-memory tables ----------------------------------------------------------------------
// NF5: the 1024-entry value LUT, rebuilt as codebook[reverse[i]] (bit-identical to the
// reference's FUSED_NF5_LUT).  One gather per element instead of two.
__device__ __forceinline__ void build_value_lut(float *lut /*1024, 16-byte aligned*/)
{
    for (int i = threadIdx.x; i < 256; i += blockDim.x)
        reinterpret_cast<uint4 *>(lut)[i] = reinterpret_cast<const uint4 *>(g_value_lut_bits)[i];
}
__device__ __forceinline__ void build_reverse_lut(uint8_t *rev /*1024*/)
{
    for (int i = threadIdx.x; i < 256; i += blockDim.x)
        reinterpret_cast<uint32_t *>(rev)[i] = reinterpret_cast<const uint32_t *>(g_reverse)[i];
}
// Reconstruction levels by code: NF5 codebook, or m / 31 for the uniform grid.
template <int GRID>
__device__ __forceinline__ void build_levels(float *lev /*32*/)
{
    if (threadIdx.x < 32)
        lev[threadIdx.x] = (GRID == AXS6_GRID_NF5) ? __uint_as_float(g_codebook_bits[threadIdx.x])
                                                    : axs6_uniform_level((int)threadIdx.x);
}

}  // namespace axs6
