// Status text, device query and launch bookkeeping of the C ABI.
#include <atomic>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace axs6 {

static std::atomic<long long> g_launches{0};

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static std::atomic<long long> g_tune[16];
static std::atomic<int> g_last_cuda_error{0};
void note_cuda_error(cudaError_t e) { if (e != cudaSuccess) g_last_cuda_error.store((int)e, std::memory_order_relaxed); }

int64_t tune_value(int key) { return (key >= 0 && key < 16) ? g_tune[key].load(std::memory_order_relaxed) : 0; }

int cached_occupancy(const void *kernel, int threads)
{
    static std::map<std::pair<const void *, int>, int> cache;
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find({kernel, dev});
    if (it != cache.end()) return it->second;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess) per_sm = 0;
    cache[{kernel, dev}] = per_sm;
    return per_sm;
}

bool ensure_dynamic_smem(const void *kernel, int bytes)
{
    static std::map<std::pair<const void *, int>, int> done;
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    std::lock_guard<std::mutex> lock(mu);
    auto it = done.find({kernel, dev});
    if (it != done.end() && it->second >= bytes) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    done[{kernel, dev}] = bytes;
    return true;
}

// ---- Philox epoch: a device-resident addend to the counter offset of every stochastic kernel -------
__device__ unsigned long long g_philox_epoch;

__global__ void philox_epoch_kernel(unsigned long long delta, int reset)
{
    g_philox_epoch = reset ? 0ull : g_philox_epoch + delta;
}

const unsigned long long *philox_epoch_ptr()
{
    static const unsigned long long *table[64];
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!table[dev]) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_philox_epoch) != cudaSuccess) return nullptr;
        table[dev] = static_cast<const unsigned long long *>(ptr);
    }
    return table[dev];
}

const DeviceInfo &device_info()
{
    static DeviceInfo table[64];
    static std::mutex mu;
    static const DeviceInfo bad = {0, 0, 0};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return bad;
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo &d = table[dev];
    if (!d.valid) {
        int major = 0, sms = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return bad;
        d.ok = (major == 10) ? 1 : 0;
        d.sms = sms;
        d.valid = 1;
    }
    return d;
}

}  // namespace axs6

AXS6_API const char *axs6_strerror(int status)
{
    switch (status) {
    case AXS6_OK: return "ok";
    case AXS6_ERR_ARG: return "invalid argument (null pointer, negative extent, bad enum or block size)";
    case AXS6_ERR_ALIGN: return "pointer or leading dimension violates the required alignment";
    case AXS6_ERR_DEVICE: return "current CUDA device is not compute capability 10.x (B200) or is unusable";
    case AXS6_ERR_LAUNCH: return "kernel launch failed";
    case AXS6_ERR_WORKSPACE: return "workspace missing or too small";
    case AXS6_ERR_UNSUPPORTED: return "request not supported by this build";
    case AXS6_ERR_TOO_LARGE: return "size exceeds the fixed capacity of an entry point that allocates nothing";
    default: return "unknown status";
    }
}

AXS6_API int64_t axs6_query(int what)
{
    switch (what) {
    case 0: { const axs6::DeviceInfo &d = axs6::device_info(); return d.valid && d.ok; }
    case 1: { const axs6::DeviceInfo &d = axs6::device_info(); return d.valid ? d.sms : 0; }
    case 2: return 1;
    case 3: return axs6::g_launches.load(std::memory_order_relaxed);
    case 4: return axs6::g_last_cuda_error.load(std::memory_order_relaxed);
    default: return -1;
    }
}

AXS6_API int axs6_tune(int key, int64_t value)
{
    if (key < 0 || key >= 16) return AXS6_ERR_ARG;
    axs6::g_tune[key].store(value, std::memory_order_relaxed);
    return AXS6_OK;
}

AXS6_API int axs6_philox_epoch(uint64_t *epoch)
{
    if (!epoch) return AXS6_ERR_ARG;
    const axs6::DeviceInfo &d = axs6::device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;
    unsigned long long v = 0;
    if (cudaMemcpyFromSymbol(&v, axs6::g_philox_epoch, sizeof(v)) != cudaSuccess) return AXS6_ERR_DEVICE;
    *epoch = v;
    return AXS6_OK;
}

AXS6_API int axs6_philox_advance(uint64_t delta, int reset, axs6_stream_t stream)
{
    const axs6::DeviceInfo &d = axs6::device_info();
    if (!d.valid || !d.ok) return AXS6_ERR_DEVICE;
    if (!axs6::philox_epoch_ptr()) return AXS6_ERR_DEVICE;
    axs6::philox_epoch_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(delta, reset);
    axs6::count_launch();
    return axs6::check_launch();
}
