// Host-side plumbing shared by the translation units: status codes, device checks,
// launch bookkeeping, and the device tables.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/axs6_b200.h"
#include "axs6_math.cuh"
#include "axs6_tables.cuh"

#define AXS6_API extern "C" __attribute__((visibility("default")))

namespace axs6 {

// Per-device facts, looked up once per device.
struct DeviceInfo {
    int valid;     // 0 on a CUDA error while looking the device up
    int ok;        // compute capability 10.x
    int sms;       // multiprocessor count
};

const DeviceInfo &device_info();      // for the current device
void count_launch(int n = 1);         // bookkeeping behind axs6_query(3)
int64_t tune_value(int key);          // axs6_tune() knobs (0 = default)
// cudaOccupancyMaxActiveBlocksPerMultiprocessor, remembered per (kernel, device); 0 on error
int cached_occupancy(const void *kernel, int threads);
// cudaFuncSetAttribute(kernel, max dynamic shared memory, bytes), done once per (kernel, device) under a
// lock, so concurrent first calls from several host threads are safe.  false on error.
bool ensure_dynamic_smem(const void *kernel, int bytes);
// Device address of this device's Philox epoch counter (added to every stochastic kernel's offset; see
// axs6_philox_advance).  nullptr on error.
const unsigned long long *philox_epoch_ptr();
// GEMM with the options the exported entry points do not expose (defined in gemm.cu)
int gemm_launch(bool tf32, const void *a, const void *b, void *c, const float *bias, int64_t M, int64_t N, int64_t K,
                int64_t lda, int64_t ldb, int64_t ldc, int a_mn, int b_mn, int c_dtype, int bias_via_bf16,
                cudaStream_t stream);

int gemm_packed_launch(const void *a, const void *a_exps, int64_t lda, const void *b, const void *b_exps, int64_t ldb, void *c,
                       const float *bias, int64_t M, int64_t N, int64_t K, int64_t ldc, int a_mn, int b_mn, int c_dtype,
                       int bias_via_bf16, cudaStream_t stream);

void note_cuda_error(cudaError_t e);      // remembers the last CUDA error a launch returned (axs6_query(4))

// Programmatic dependent launch.  A kernel launched with launch_overlapped(true, ...) may become resident while the
// kernel before it on the stream is still running: its CTAs run their prologue (barrier initialisation, tables
// copied from the module image into shared memory) and then block in pdl_wait() until that earlier kernel has
// completed and its writes are visible.  Everything that reads or writes caller memory comes after pdl_wait(), so
// the result is the same as with an ordinary launch; what is saved is the launch gap and the prologue between
// back-to-back kernels.  Measured on B200: worth 10-20 % for the TMA-fed pack / unpack kernels at 20-30 us per launch
// (8192 x 4096), but the fake-quantise kernels lose 10 % at 32768 x 8192 (the CTAs of the next launch, released all at
// once, stream in lockstep), so only short launches of the TMA-fed codec kernels ask for it.  Without the launch
// attribute the two device calls do nothing.  Tune key 15 = 1 turns the attribute off everywhere.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(bool overlap, void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem,
                                     cudaStream_t stream, Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (overlap && tune_value(15) != 1) ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    note_cuda_error(e);
    return e;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int check_launch()
{
    const cudaError_t e = cudaGetLastError();
    note_cuda_error(e);
    return e == cudaSuccess ? AXS6_OK : AXS6_ERR_LAUNCH;
}

inline bool valid_block(int b) { return b == 8 || b == 16 || b == 32; }
inline bool valid_dtype(int d) { return d == AXS6_F32 || d == AXS6_BF16; }

// Codebook levels (fp32 bits) and LUT-index -> code table, baked into each module image.
static __device__ __align__(16) const uint32_t g_codebook_bits[32] = AXS6_CODEBOOK_BITS_INIT;
static __device__ __align__(16) const uint8_t g_reverse[1024] = AXS6_REVERSE_INIT;
// derived tables (see gen_tables.py): kernels copy them into shared memory with 16-byte loads
static __device__ __align__(16) const uint32_t g_value_lut_bits[1024] = AXS6_VALUE_LUT_BITS_INIT;
static __device__ __align__(16) const uint8_t g_key_code[1296] = AXS6_KEY_CODE_INIT;
static __device__ __align__(16) const uint16_t g_key_level_bf16[1288] = AXS6_KEY_LEVEL_BF16_INIT;
static __device__ __align__(16) const uint16_t g_lut_level_bf16[1024] = AXS6_LUT_LEVEL_BF16_INIT;

}  // namespace axs6
