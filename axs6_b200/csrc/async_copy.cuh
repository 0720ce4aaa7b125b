// PTX wrappers shared by the kernels that move tiles with the TMA unit: mbarrier primitives, the
// 2-D tensor-map load, bulk shared->global stores, and the host-side tensor-map encoder (looked up
// through the runtime, so the library does not link against libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace axs6 {
namespace acp {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Poll `bar` for `parity` at most `limit` times; false = gave up.  `status` is a device-global word
// shared by all roles of a kernel: a non-zero value (somebody else gave up) ends the wait early,
// and a wait that runs out stores `code` there if it is still zero.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int code, int *status, uint32_t limit)
{
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (i > 64) {
            __nanosleep(40);
            if ((i & 255u) == 0u && *(volatile int *)status != 0) return false;
        }
    }
    atomicCAS(status, 0, code);
    return false;
}

// Poll `bar` for `parity` at most `limit` times, whatever the status word says.  Used on the way out of a kernel
// that gave up: the thread that issued asynchronous loads waits for the ones still in flight, so that none can
// land after the CTA has released its shared memory.
__device__ __forceinline__ bool mbar_wait_quiet(uint32_t bar, uint32_t parity, uint32_t limit)
{
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (i > 64) __nanosleep(40);
    }
    return false;
}
// The same for `ahead` consecutive stages of a ring of `stages` barriers (8 bytes apart from `bar0`) starting at
// position (s, ph).
__device__ __forceinline__ void drain_ring(uint32_t bar0, int stages, int s, uint32_t ph, int ahead, uint32_t limit)
{
    for (int j = 0; j < ahead; ++j) {
        int sj = s + j;
        uint32_t pj = ph;
        if (sj >= stages) { sj -= stages; pj ^= 1u; }
        mbar_wait_quiet(bar0 + 8u * (uint32_t)sj, pj, limit);
    }
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Orders this thread's ordinary shared-memory accesses before later accesses by the TMA unit.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

// Tile of shared memory -> global memory through a 2-D tensor map (rows outside the tensor are dropped).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
}

// The same tile added (fp32) to what global memory holds: one atomic add per element, done by the memory system.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, uint32_t src, int c0, int c1)
{
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// Contiguous global -> shared copy by the TMA unit, counted on `bar`; addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t sdst, const void *gsrc, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(sdst), "l"(gsrc), "r"(bytes), "r"(bar) : "memory");
}

// Contiguous shared -> global copy by the TMA unit; both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_store(void *gdst, uint32_t ssrc, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(ssrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All but the newest `N` committed groups of this thread have finished READING shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

}  // namespace acp
}  // namespace axs6
