// Column sums without any allocation.
//
// sb200_gemm_batched computes the bias gradient (column sums of op(B)) through
// partial sums in a scratch buffer that the context obtains with cudaMalloc.
// Some callers must not trigger an allocation: code that runs underneath
// another allocator which believes it owns the device's free memory (Sapphire's
// own ResourceManager pools, a framework's caching allocator), where a foreign
// cudaMalloc can fail or force that allocator to give memory back; and code on
// a latency path, because cudaMalloc / cudaFree synchronise the whole device.
// For them this file offers the same two kernels with the scratch living in a
// fixed array inside the library image.
#include <mutex>

#include "common.cuh"

namespace sb200 {
// gemm_simt.cu
int colsum_slices(int sm_count, int64_t K, int64_t N);
int launch_colsum_with_scratch(sb200_ctx* ctx, const float* B, int transB, int64_t K, int64_t N,
                               int64_t ldb, float* out, float scale, float* scratch, int slices,
                               cudaStream_t stream);
}  // namespace sb200

namespace {

constexpr int64_t NOALLOC_MAX_N = SB200_COLSUM_NOALLOC_MAX_N;   // columns
constexpr int NOALLOC_MAX_SLICES = 64;                           // k slices
constexpr int MAX_DEVICES = 64;

// slices x columns partial sums: 64 x 16384 floats = 4 MiB on every GPU that
// loads the library, held until the process exits
static __device__ __align__(256) float g_colsum_scratch[NOALLOC_MAX_SLICES * NOALLOC_MAX_N];

struct DeviceSetup {
    bool done = false;
    float* scratch = nullptr;     // device address of g_colsum_scratch on this device
    int sm_count = 0;
};
DeviceSetup g_setup[MAX_DEVICES];
std::mutex g_setup_mutex;

// The array's name is only a host-side handle; the address kernels can use
// comes from cudaGetSymbolAddress, once per device, with that device current.
int setup_current_device(DeviceSetup** out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        return SB200_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    DeviceSetup& s = g_setup[dev];
    if (!s.done) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_colsum_scratch) != cudaSuccess || !ptr)
            return SB200_ERR_CUDA;
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            sms <= 0)
            return SB200_ERR_CUDA;
        s.scratch = static_cast<float*>(ptr);
        s.sm_count = sms;
        s.done = true;
    }
    *out = &s;
    return SB200_OK;
}

}  // namespace

extern "C" int sb200_colsum_noalloc(const float* B, int transB, int64_t K, int64_t N, int64_t ldb,
                                    float* out, float scale, sb200_stream stream_)
{
    if (K < 0 || N < 0)
        return SB200_ERR_INVALID_ARG;
    if (N == 0)
        return SB200_OK;
    if (!out || (K > 0 && !B) || ldb < (transB ? K : N))
        return SB200_ERR_INVALID_ARG;
    if (N > NOALLOC_MAX_N)
        return SB200_ERR_TOO_LARGE;           // more columns than the fixed scratch holds
    DeviceSetup* s = nullptr;
    const int rc = setup_current_device(&s);
    if (rc)
        return rc;
    int slices = sb200::colsum_slices(s->sm_count, K, N);
    if (slices > NOALLOC_MAX_SLICES)
        slices = NOALLOC_MAX_SLICES;
    // every (slice, column) cell below `slices` x N is overwritten by the first
    // kernel before the second reads it, so nothing has to be cleared
    return sb200::launch_colsum_with_scratch(nullptr, B, transB != 0, K, N, ldb, out, scale,
                                             s->scratch, slices, static_cast<cudaStream_t>(stream_));
}
