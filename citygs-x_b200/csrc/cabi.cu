// Status handling and the small host-only entry points of the C ABI.
#include <string.h>
#include "cgx_common.cuh"

namespace cgx {

static thread_local char g_cuda_error[256] = "";
static unsigned long long g_launches = 0;  // kernels launched by this library in this process



void set_cuda_error(cudaError_t e)
{
    strncpy(g_cuda_error, cudaGetErrorString(e), sizeof(g_cuda_error) - 1);
    g_cuda_error[sizeof(g_cuda_error) - 1] = 0;
}

void set_error_text(const char* text)
{
    strncpy(g_cuda_error, text, sizeof(g_cuda_error) - 1);
    g_cuda_error[sizeof(g_cuda_error) - 1] = 0;
}

// Launch errors only (no synchronisation): configuration problems surface here, execution faults
// surface at the caller's next synchronising call.
int check_launch(int launched)
{
    __atomic_fetch_add(&g_launches, (unsigned long long)launched, __ATOMIC_RELAXED);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_cuda_error(e);
        return CGX_ECUDA;
    }
    return CGX_OK;
}

}  // namespace cgx

extern "C" const char* cgx_strerror(int status)
{
    switch (status) {
    case CGX_OK: return "ok";
    case CGX_EINVAL: return "invalid argument (shape, null or misaligned pointer)";
    case CGX_ENOMEM: return "workspace or capacity too small";
    case CGX_ETIMEDOUT: return "a bounded device-side wait gave up";
    case CGX_ECUDA: return "CUDA runtime error";
    default: return "unknown status";
    }
}

extern "C" const char* cgx_last_cuda_error(void) { return cgx::g_cuda_error; }

extern "C" unsigned long long cgx_launch_count(void) { return __atomic_load_n(&cgx::g_launches, __ATOMIC_RELAXED); }

extern "C" const char* cgx_version(void) { return "cgx_raster 0.1 (sm_100a)"; }

extern "C" int cgx_block_xy(int* block_x, int* block_y, int* one_dim_block)
{
    if (!block_x || !block_y || !one_dim_block) return CGX_EINVAL;
    *block_x = CGX_BLOCK_X;
    *block_y = CGX_BLOCK_Y;
    *one_dim_block = CGX_BLOCK_SIZE;
    return CGX_OK;
}

namespace cgx {
int fetch_render_status(int* out);  // render.cu
int fetch_peer_status(int* out);    // peer.cu
int fetch_sort_status(int* out);    // binning.cu
int fetch_render_status_async(int* out_pinned, cudaStream_t st);
int fetch_peer_status_async(int* out_pinned, cudaStream_t st);
int fetch_sort_status_async(int* out_pinned, cudaStream_t st);
}  // namespace cgx

namespace cgx {
__global__ void post_words_kernel(const uint32_t* __restrict__ src, volatile uint32_t* dst, int n)
{
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
    __threadfence_system();
}

int post_words(const void* src_dev, void* dst_host_pinned, int n_words, cudaStream_t st)
{
    if (n_words < 0 || (n_words && (!src_dev || !dst_host_pinned))) return CGX_EINVAL;
    if (((uintptr_t)src_dev | (uintptr_t)dst_host_pinned) & 3u) return CGX_EINVAL;
    if (n_words == 0) return CGX_OK;
    void* mapped = nullptr;     // fails for pageable memory: the caller must pass page-locked memory
    cudaError_t e = cudaHostGetDevicePointer(&mapped, dst_host_pinned, 0);
    if (e != cudaSuccess || !mapped) { (void)cudaGetLastError(); return CGX_EINVAL; }
    post_words_kernel<<<1, 128, 0, st>>>((const uint32_t*)src_dev, (volatile uint32_t*)mapped, n_words);
    return check_launch();
}
}  // namespace cgx

extern "C" int cgx_post_words(const void* src_device, void* dst_host_pinned, int n_words32, void* stream)
{
    return cgx::post_words(src_device, dst_host_pinned, n_words32, (cudaStream_t)stream);
}

extern "C" int cgx_device_status_async(int* status_pinned_host4, void* stream)
{
    if (!status_pinned_host4) return CGX_EINVAL;
    int st = cgx::fetch_render_status_async(status_pinned_host4, (cudaStream_t)stream);
    if (st == CGX_OK) st = cgx::fetch_peer_status_async(status_pinned_host4 + 1, (cudaStream_t)stream);
    if (st == CGX_OK) st = cgx::fetch_sort_status_async(status_pinned_host4 + 2, (cudaStream_t)stream);
    status_pinned_host4[3] = 0;
    return st;
}

extern "C" int cgx_device_status(int* status_host, void* stream)
{
    if (!status_host) return CGX_EINVAL;
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) { cgx::set_cuda_error(e); return CGX_ECUDA; }
    int a = 0, b = 0, c = 0;
    int st = cgx::fetch_render_status(&a);
    if (st == CGX_OK) st = cgx::fetch_peer_status(&b);
    if (st == CGX_OK) st = cgx::fetch_sort_status(&c);
    if (st != CGX_OK) return st;
    *status_host = a ? a : (b ? b : c);
    return CGX_OK;
}
