// Stream-ordered barrier between the ranks of one NVLink/NVSwitch domain, over flag words that every rank has
// mapped from every peer (symmetric memory).  Used to order the direct peer stores of the Gaussian exchange
// against their readers.  Epochs only grow, so the flags never need resetting; every wait is bounded.
#include "cgx_common.cuh"

namespace cgx {

__device__ int g_peer_status = 0;  // CGX_ETIMEDOUT when a barrier wait gave up

constexpr int PEER_MAX = 32;
constexpr unsigned long long PEER_WAIT_LIMIT_CYCLES = 1ull << 32;  // ~2 s at B200 clocks

struct PeerFlags {
    uint32_t* p[PEER_MAX];  // p[r] = flag array (>= PEER_MAX words) living in rank r's memory
};

__global__ void __launch_bounds__(PEER_MAX)
peer_barrier_kernel(PeerFlags flags, int ws, int rank, uint32_t epoch, unsigned long long limit_cycles)
{
    const int t = threadIdx.x;
    if (t >= ws) return;
    __threadfence_system();
    // tell rank t that this rank has reached `epoch` ...
    uint32_t* remote = flags.p[t] + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    // ... and wait until rank t has told us the same
    const uint32_t* mine = flags.p[rank] + t;
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)(v - epoch) >= 0) break;
        if ((unsigned long long)(clock64() - t0) > limit_cycles) {
            atomicExch(&g_peer_status, CGX_ETIMEDOUT);
            break;
        }
    }
    __threadfence_system();
}

int fetch_peer_status_async(int* out_pinned, cudaStream_t st)
{
    void* word = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&word, g_peer_status);
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    return post_words(word, out_pinned, 1, st);
}

int fetch_peer_status(int* out)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, g_peer_status, sizeof(int));
    if (e != cudaSuccess) { set_cuda_error(e); return CGX_ECUDA; }
    if (*out != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int));
    }
    return CGX_OK;
}

}  // namespace cgx

extern "C" int cgx_peer_barrier_limited(int ws, int rank, uint32_t* const* flag_ptrs, uint32_t epoch,
                                        unsigned long long wait_limit_cycles, void* stream)
{
    if (wait_limit_cycles == 0) wait_limit_cycles = cgx::PEER_WAIT_LIMIT_CYCLES;
    if (ws <= 0 || ws > cgx::PEER_MAX || rank < 0 || rank >= ws || !flag_ptrs) return CGX_EINVAL;
    cgx::PeerFlags f;
    for (int r = 0; r < cgx::PEER_MAX; r++) {
        f.p[r] = r < ws ? flag_ptrs[r] : nullptr;
        if (r < ws && (!f.p[r] || ((uintptr_t)f.p[r] & 3))) return CGX_EINVAL;
    }
    cgx::peer_barrier_kernel<<<1, cgx::PEER_MAX, 0, (cudaStream_t)stream>>>(f, ws, rank, epoch, wait_limit_cycles);
    return cgx::check_launch();
}

extern "C" int cgx_peer_barrier(int ws, int rank, uint32_t* const* flag_ptrs, uint32_t epoch, void* stream)
{
    return cgx_peer_barrier_limited(ws, rank, flag_ptrs, epoch, 0ull, stream);
}
